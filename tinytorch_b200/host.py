"""Attention on HOST buffers: the call a caller with tensors in (pinned) host
memory makes.  Inputs are copied to the device, the fused kernels run, the result
is copied back - split into batch chunks on three streams so that the
host-to-device copy of chunk i+1, the kernels of chunk i and the device-to-host
copy of chunk i-1 overlap.  PCIe, not the kernel, bounds this path; the
pipeline's job is to keep the link busy in both directions.
"""
import torch

from . import op


class HostAttention:
    """Reusable pipeline for one problem shape (device staging buffers are allocated once)."""

    def __init__(self, q_shape, kv_shape, dtype, device=None, chunks=4, decode=False):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        B = q_shape[0]
        self.chunks = max(1, min(chunks, B))
        self.bounds = [(B * c // self.chunks, B * (c + 1) // self.chunks) for c in range(self.chunks)]
        mb = max(e - b for b, e in self.bounds)
        self.decode = decode
        mk = lambda shp: torch.empty((mb,) + tuple(shp[1:]), dtype=dtype, device=self.device)
        # two staging slots: one being filled while the other is being computed on
        self.dq = [mk(q_shape) for _ in range(2)]
        self.dk = [mk(kv_shape) for _ in range(2)]
        self.dv = [mk(kv_shape) for _ in range(2)]
        self.s_in = torch.cuda.Stream(self.device)
        self.s_run = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)

    def __call__(self, hq, hk, hv, ho, isCausal=False, scale=None, kvLens=None):
        """hq/hk/hv/ho: pinned host tensors [B,H,S,D]; kvLens: device int32 [B] or None."""
        cur = torch.cuda.current_stream(self.device)
        self.s_in.wait_stream(cur)
        self.s_run.wait_stream(cur)
        self.s_out.wait_stream(cur)
        ran = [None, None]  # event: kernels that read staging slot s have finished
        for c, (b0, b1) in enumerate(self.bounds):
            s, n = c & 1, b1 - b0
            with torch.cuda.stream(self.s_in):
                if ran[s] is not None:
                    self.s_in.wait_event(ran[s])
                self.dq[s][:n].copy_(hq[b0:b1], non_blocking=True)
                self.dk[s][:n].copy_(hk[b0:b1], non_blocking=True)
                self.dv[s][:n].copy_(hv[b0:b1], non_blocking=True)
                loaded = torch.cuda.Event()
                loaded.record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(loaded)
                lens = kvLens[b0:b1] if kvLens is not None else None
                if self.decode:
                    o, _ = op.sdpAttentionDecode(self.dq[s][:n], self.dk[s][:n], self.dv[s][:n], lens, scale)
                else:
                    o, _ = op.sdpAttentionFwd(self.dq[s][:n], self.dk[s][:n], self.dv[s][:n], isCausal, scale, lens,
                                              needLse=False)
                ran[s] = torch.cuda.Event()
                ran[s].record(self.s_run)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(ran[s])
                o.record_stream(self.s_out)
                ho[b0:b1].copy_(o, non_blocking=True)
        cur.wait_stream(self.s_out)
        cur.wait_stream(self.s_run)
        return ho


def sdpAttentionHost(hq, hk, hv, isCausal=False, scale=None, kvLens=None, chunks=4, out=None):
    """One-shot convenience wrapper around HostAttention (forward, no autograd)."""
    if out is None:
        out = torch.empty(hq.shape, dtype=hq.dtype).pin_memory()
    pipe = HostAttention(hq.shape, hk.shape, hq.dtype, chunks=chunks, decode=False)
    pipe(hq, hk, hv, out, isCausal, scale, kvLens)
    torch.cuda.current_stream().synchronize()
    return out
