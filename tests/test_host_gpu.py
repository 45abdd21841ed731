"""GPU: the host-buffer entry point (chunked copy / compute / copy-back pipeline)
gives the same result as the device-resident op."""
import numpy as np
import pytest
import torch

from gpu_util import TOL_ABS_16BIT, to_np

pytestmark = pytest.mark.gpu


def test_host_pipeline_matches_device_op(oracle):
    from tinytorch_b200 import op
    from tinytorch_b200.host import HostAttention, sdpAttentionHost
    B, Hq, Hkv, S, D = 5, 4, 2, 300, 128   # 5 sequences in 4 chunks: ragged chunking
    g = torch.Generator().manual_seed(5)
    hq = torch.randn((B, Hq, S, D), generator=g).to(torch.bfloat16).pin_memory()
    hk = torch.randn((B, Hkv, S, D), generator=g).to(torch.bfloat16).pin_memory()
    hv = torch.randn((B, Hkv, S, D), generator=g).to(torch.bfloat16).pin_memory()
    want, _ = op.sdpAttentionFwd(hq.cuda(), hk.cuda(), hv.cuda(), isCausal=True)
    got = sdpAttentionHost(hq, hk, hv, isCausal=True)
    assert torch.equal(got, want.cpu())
    wo, _ = oracle.fwd(hq[:1].float().numpy(), hk[:1].float().numpy(), hv[:1].float().numpy(), causal=True)
    assert np.abs(to_np(got[:1]) - wo).max() <= TOL_ABS_16BIT
    # reusable pipeline, two calls in a row, with per-sequence lengths
    lens = torch.tensor([300, 17, 128, 129, 1], dtype=torch.int32, device="cuda")
    pipe = HostAttention(hq.shape, hk.shape, torch.bfloat16, chunks=3)
    out = torch.empty(hq.shape, dtype=torch.bfloat16).pin_memory()
    for _ in range(2):
        out.zero_()
        pipe(hq, hk, hv, out, isCausal=False, kvLens=lens)
        torch.cuda.synchronize()
        want, _ = op.sdpAttentionFwd(hq.cuda(), hk.cuda(), hv.cuda(), isCausal=False, kvLens=lens)
        assert torch.equal(out, want.cpu())
