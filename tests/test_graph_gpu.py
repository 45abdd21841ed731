"""The entry points enqueue work on the caller's stream and never synchronise or call cudaMalloc themselves, so a
token loop can be captured into a CUDA graph and replayed (the workspace comes from the caller here; the allocator
hook is not touched during capture)."""
import numpy as np
import pytest
import torch

from gpu_util import TOL_ABS_16BIT, make, to_np

pytestmark = pytest.mark.gpu


def _capture(fn):
    # one eager call first: it creates the tensor-map encoder and sets kernel attributes outside the capture
    fn()
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(s):
        fn()  # warm-up on the side stream
        s.synchronize()
        with torch.cuda.graph(g, stream=s):
            out = fn()
    torch.cuda.current_stream().wait_stream(s)
    return g, out


@pytest.mark.parametrize("Hq,Hkv", [(8, 8), (8, 2)])  # scan kernel / tensor-core kernel (work counter memset inside)
def test_decode_replays_from_a_cuda_graph(oracle, Hq, Hkv):
    from tinytorch_b200 import _capi, op
    B, cap, D = 3, 2048, 128
    q, _ = make((B, Hq, 1, D), torch.bfloat16, 701)
    k, kn = make((B, Hkv, cap, D), torch.bfloat16, 702)
    v, vn = make((B, Hkv, cap, D), torch.bfloat16, 703)
    lens = torch.tensor([2048, 700, 1], dtype=torch.int32, device="cuda")
    need = op.workspaceBytes(_capi.KIND_DECODE, torch.bfloat16, B, Hq, Hkv, 1, cap, D)
    ws = torch.empty(max(need, 256), dtype=torch.uint8, device="cuda")
    g, (o, _) = _capture(lambda: op.sdpAttentionDecode(q, k, v, lens, workspace=ws))
    # new inputs in the captured buffers, then replay
    q2, q2n = make((B, Hq, 1, D), torch.bfloat16, 704)
    q.copy_(q2)
    lens.copy_(torch.tensor([5, 2048, 1024], dtype=torch.int32))
    g.replay()
    torch.cuda.synchronize()
    wo, _ = oracle.fwd(q2n, kn, vn, kv_lens=np.array([5, 2048, 1024], dtype=np.int32))
    assert np.abs(to_np(o) - wo).max() <= TOL_ABS_16BIT


def test_block_operators_and_prefill_replay_from_a_cuda_graph(oracle):
    from oracle.loader import FusedOracle
    from tinytorch_b200 import fused, op
    forc = FusedOracle()
    x, xn = make((64, 256), torch.bfloat16, 711)
    w, wn = make((384, 256), torch.bfloat16, 712, std=0.1)
    b, bn = make((384,), torch.bfloat16, 713)
    B, H, S, D = 1, 3, 64, 128     # the projection's output is read as q, k, v of three heads

    def step():
        y = fused._linear_raw(x, w, b)                   # [64, 384] -> three heads of 128
        qkv = y.view(1, S, H, D).permute(0, 2, 1, 3).contiguous()
        o, _ = op.sdpAttentionFwd(qkv, qkv, qkv, isCausal=True, needLse=False)
        return fused.siluMul(o.reshape(H * S, D)), y

    g, (z, y) = _capture(step)
    x2, x2n = make((64, 256), torch.bfloat16, 714)
    x.copy_(x2)
    g.replay()
    torch.cuda.synchronize()
    want_y = forc.linear(x2n, wn, bn)
    assert np.abs(to_np(y) - want_y).max() <= TOL_ABS_16BIT * max(1.0, np.abs(want_y).max())
    yy = to_np(y).reshape(1, S, H, D).transpose(0, 2, 1, 3)
    wo, _ = oracle.fwd(yy, yy, yy, causal=True)
    want_z = forc.silu_mul(torch.from_numpy(wo).bfloat16().float().numpy().reshape(H * S, D))
    assert np.abs(to_np(z) - want_z).max() <= 4 * TOL_ABS_16BIT * max(1.0, np.abs(want_z).max())


def test_forward_and_backward_replay_from_a_cuda_graph(oracle):
    # the backward's three kernels (delta pre-pass, tensor-core kernel, conversion) are chained by programmatic
    # dependent launches: the capture keeps those edges, and a replay with new data gives the new gradients
    from tinytorch_b200 import op
    B, H, S, D = 1, 2, 256, 64
    q, qn = make((B, H, S, D), torch.float16, 721)
    k, kn = make((B, H, S, D), torch.float16, 722)
    v, vn = make((B, H, S, D), torch.float16, 723)
    do, _ = make((B, H, S, D), torch.float16, 724)

    def step():
        o, lse = op.sdpAttentionFwd(q, k, v, isCausal=True)
        return op.sdpAttentionBwd(do, q, k, v, o, lse, isCausal=True)

    g, (dq, dk, dv) = _capture(step)
    do2, do2n = make((B, H, S, D), torch.float16, 725)
    do.copy_(do2)
    g.replay()
    torch.cuda.synchronize()
    wq, wk, wv = oracle.bwd(qn, kn, vn, do2n, causal=True)
    for got, want in ((dq, wq), (dk, wk), (dv, wv)):
        assert np.abs(to_np(got) - want).max() <= TOL_ABS_16BIT
