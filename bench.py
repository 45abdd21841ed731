#!/usr/bin/env python
"""Benchmark of the fused attention path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

A "step" is one pass of the hot path over one batch of seeded synthetic input.
The default workload is the causal bf16 prefill forward at B=4, H=32, S=4096,
D=128 (metric: causal-adjusted attention TFLOP/s); the same run also measures the
bf16 decode workload (B=64, H=32, D=128, cache 8192, lengths U[1024, 8192]) in
HBM GB/s and reports it under "decode".  With N > 1 (one process per GPU under
torchrun) every rank runs the same per-GPU workload on its own batch shard, no
collective on the data path (weak scaling); the time is the max over ranks.

--impl reference times the reference's own CPU implementation (oracle/_ref, built
from the unmodified reference sources; else the plain-C oracle) on bounded samples
of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: dict(kind, dtype, B, Hq, Hkv, L, S, D, causal)
    "prefill": dict(kind="fwd", dtype="bf16", B=4, Hq=32, Hkv=32, L=4096, S=4096, D=128, causal=True, std=1.0),
    "gqa": dict(kind="fwd", dtype="f16", B=8, Hq=32, Hkv=8, L=2048, S=2048, D=128, causal=True, std=0.5),
    "train": dict(kind="fwdbwd", dtype="f16", B=8, Hq=16, Hkv=16, L=2048, S=2048, D=64, causal=True, std=1.0),
    "cfg1": dict(kind="fwdbwd", dtype="f32", B=2, Hq=4, Hkv=4, L=128, S=128, D=64, causal=True, std=1.0),
    "decode": dict(kind="decode", dtype="bf16", B=64, Hq=32, Hkv=32, L=1, S=8192, D=128, causal=False, std=1.0),
    # reduced copies of the two headline workloads, sized for an ncu capture (inputs still larger than L2)
    "prefill_ncu": dict(kind="fwd", dtype="bf16", B=2, Hq=32, Hkv=32, L=4096, S=4096, D=128, causal=True, std=1.0),
    # the fused decode step: rotary embedding + cache append + attention (same bytes, one more row per sequence)
    "decode_append": dict(kind="decode", dtype="bf16", B=64, Hq=32, Hkv=32, L=1, S=8192, D=128, causal=False, std=1.0,
                          append=True),
    # the reference's two fused transformer-block operators (HBM bound): 32768 tokens x hidden 8192,
    # and a gated MLP of width 14336 over 16384 tokens
    "rmsnorm": dict(kind="fused", opname="fusedAddRmsNorm", dtype="bf16", rows=32768, dim=8192),
    "silumul": dict(kind="fused", opname="siluMul", dtype="bf16", rows=16384, dim=14336),
    # reduced copies for profiler captures (a few hundred MB, still larger than L2)
    "rmsnorm_ncu": dict(kind="fused", opname="fusedAddRmsNorm", dtype="bf16", rows=8192, dim=8192),
    "silumul_ncu": dict(kind="fused", opname="siluMul", dtype="bf16", rows=4096, dim=14336),
    "decode_append_ncu": dict(kind="decode", dtype="bf16", B=16, Hq=32, Hkv=32, L=1, S=8192, D=128, causal=False, std=1.0,
                              append=True),
    # the QKV projection in front of attention: 16384 tokens, hidden 4096 -> 3 x 4096 (tensor bound)
    "linear": dict(kind="fused", opname="linear", dtype="bf16", rows=16384, dim=4096, n_out=12288),
    "linear_ncu": dict(kind="fused", opname="linear", dtype="bf16", rows=4096, dim=4096, n_out=4096),
    # grouped-query decode (4 query heads per kv head): the tensor-core decode kernel
    "decode_gqa": dict(kind="decode", dtype="bf16", B=256, Hq=32, Hkv=8, L=1, S=8192, D=128, causal=False, std=1.0),
    "decode_gqa_ncu": dict(kind="decode", dtype="bf16", B=64, Hq=32, Hkv=8, L=1, S=8192, D=128, causal=False, std=1.0),
    "train128_ncu": dict(kind="fwdbwd", dtype="bf16", B=1, Hq=16, Hkv=16, L=4096, S=4096, D=128, causal=True, std=1.0),
    # a token loop of 32 layers at a small batch, eager and replayed from a CUDA graph (launch-bound)
    "decode_loop": dict(kind="loop", dtype="bf16", B=8, Hq=32, Hkv=8, S=4096, D=128, layers=32),
    "decode_ncu": dict(kind="decode", dtype="bf16", B=16, Hq=32, Hkv=32, L=1, S=8192, D=128, causal=False, std=1.0),
}
ESIZE = {"f32": 4, "f16": 2, "bf16": 2}


def fwd_flops(w):
    """4*B*Hq*L*S*D, halved under the causal mask (L == S)."""
    f = 4.0 * w["B"] * w["Hq"] * w["L"] * w["S"] * w["D"]
    return f / 2 if w["causal"] else f


def step_flops(w):
    return fwd_flops(w) * (3.5 if w["kind"] == "fwdbwd" else 1.0)


def decode_bytes(w, lens):
    """K and V rows below each sequence's length, plus q and O."""
    es = ESIZE[w["dtype"]]
    return float(int(lens.sum()) * w["Hkv"] * w["D"] * 2 * es + 2 * w["B"] * w["Hq"] * w["D"] * es)


def fwd_bytes(w):
    """Q, K, V read once, O and the fp32 LSE written once."""
    es = ESIZE[w["dtype"]]
    q = w["B"] * w["Hq"] * w["L"] * w["D"]
    kv = w["B"] * w["Hkv"] * w["S"] * w["D"]
    return float((2 * q + 2 * kv) * es + 4 * w["B"] * w["Hq"] * w["L"])


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one launch over the algorithmic bytes of the same
# launch, from one ncu capture of a reduced case of each kernel; traffic grows in proportion to the units a launch
# processes, so the figure reported for a full launch is this ratio times the launch's algorithmic bytes.
NCU_TRAFFIC_RATIO = {
    "fwd_tc_kernel": (254.1 / 269.5, "profiles/fwd_tc_kernel_prefill_bf16_S4096_D128.md"),
    "bwd_tc64_kernel": (296.3 / 270.5, "profiles/bwd_tc64_kernel_train_fp16_S2048_D64.md"),
    "decode_kernel": (1218.2 / 1213.0, "profiles/decode_kernel_bf16_cap8192_D128.md"),
    "decode_tc_kernel": (1271.9 / 1248.0, "profiles/decode_tc_kernel_bf16_gqa4_cap8192_D128.md"),
    "linear_tc_kernel": (87.4 / 100.7, "profiles/linear_tc_kernel_bf16_4096x4096x4096.md"),
    "add_rms_norm_kernel": (478.5 / 536.9, "profiles/add_rms_norm_kernel_bf16_8192x8192.md"),
    "silu_mul_kernel": (309.3 / 352.3, "profiles/silu_mul_rows_kernel_bf16_4096x28672.md"),
}


def traffic_of(kernel, algorithmic_bytes):
    """(bytes per launch, source) scaled from the kernel's ncu capture, or (None, None) without one."""
    if kernel not in NCU_TRAFFIC_RATIO or algorithmic_bytes is None:
        return None, None
    ratio, src = NCU_TRAFFIC_RATIO[kernel]
    return ratio * algorithmic_bytes, "ncu capture of a reduced case scaled by algorithmic bytes (%s)" % src


def nominal_peaks():
    """Datasheet figures: dense bf16 / fp16 tensor throughput and HBM3e bandwidth (the 8 TB/s quoted for the target)."""
    return dict(tflops=2250.0, gbs=8000.0)


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return dict(tflops=float(d["bf16_tflops"]), gbs=float(d["hbm_gbs"]),
                    tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                    source="measured (MEASURED_PEAKS.json, burst)")
    return dict(tflops=1590.0, gbs=6650.0, tflops_sustained=1400.0, source="fallback (earlier measurement on this pool)")


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.idx), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = dict(sm_mhz=None, sm_max_mhz=None, reasons=[], samples=0)
        if self.proc is None:
            return out
        time.sleep(0.25)
        self.proc.terminate()  # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1])), mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out.update(sm_mhz=float(np.median(sm)), sm_max_mhz=float(max(mx)), reasons=sorted(reasons), samples=len(sm))
        return out


# ------------------------------------------------------------------ CPU side --
def cpu_reference_runner():
    """(callable fwd(q,k,v,causal,kv_lens) , callable grad(...), kind, threads usable)."""
    from oracle.loader import Oracle, Reference
    if Reference.available():
        r = Reference()
        return r, "reference"
    return Oracle(threads=os.cpu_count() or 1), "port"


def cpu_sample(w, runner, kind, n_units, threads, seed=99):
    """Times `n_units` independent (batch, head) units of workload `w` on the host.

    The reference's CPU path is single-threaded; independent units run on
    `threads` host threads (the ctypes calls release the GIL).
    Returns (seconds, work) with work in FLOPs (or bytes for decode).
    """
    import concurrent.futures as cf
    rng = np.random.default_rng(seed)
    L, S, D = w["L"], w["S"], w["D"]
    g = w["Hq"] // w["Hkv"]
    units = []
    for _ in range(n_units):
        q = (rng.standard_normal((1, g, L, D), dtype=np.float32) * np.float32(w["std"]))
        k, v = ((rng.standard_normal((1, 1, S, D), dtype=np.float32) * np.float32(w["std"])) for _ in range(2))
        units.append((q, k, v))
    lens = rng.integers(1024, 8193, size=n_units).astype(np.int32) if w["kind"] == "decode" else None

    def one(i):
        q, k, v = units[i]
        if kind == "reference":
            if g > 1:  # the reference's GQA route: repeatInterleave, then attention
                k, v = runner.repeat_interleave(k, g), runner.repeat_interleave(v, g)
            if w["kind"] == "decode":
                runner.fwd(q, k, v, kv_lens=lens[i:i + 1])
            elif w["kind"] == "fwdbwd":
                runner.grad(q, k, v, q, causal=w["causal"])
            else:
                runner.fwd(q, k, v, causal=w["causal"])
        else:
            kw = dict(causal=w["causal"], kv_lens=lens[i:i + 1] if lens is not None else None)
            runner.fwd(q, k, v, **kw)
            if w["kind"] == "fwdbwd":
                runner.bwd(q, k, v, q, **kw)

    if kind == "port":
        runner.set_threads(1)
    t0 = time.perf_counter()
    if threads <= 1:
        for i in range(n_units):
            one(i)
    else:
        with cf.ThreadPoolExecutor(max_workers=threads) as ex:
            list(ex.map(one, range(n_units)))
    dt = time.perf_counter() - t0
    if w["kind"] == "decode":
        work = float(int(lens.sum()) * D * 2 * ESIZE[w["dtype"]])
    else:
        unit = dict(w, B=1, Hq=g, Hkv=1)
        work = step_flops(unit) * n_units
    return dt, work


def run_reference_arm(args, w, wname):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    runner, kind = cpu_reference_runner()
    threads = os.cpu_count() or 1
    # one step = `threads` units (one per host thread), sized to a few seconds
    n_units = max(1, min(threads, 32))
    for _ in range(min(args.warmup, 1)):
        cpu_sample(w, runner, kind, max(1, n_units // 4), threads)
    tot_t, tot_w = 0.0, 0.0
    for s in range(args.steps):
        dt, work = cpu_sample(w, runner, kind, n_units, threads, seed=100 + s)
        tot_t += dt
        tot_w += work
    decode = w["kind"] == "decode"
    value = tot_w / tot_t / (1e9 if decode else 1e12)
    unit = "GB/s" if decode else "TFLOP/s"
    sample = "%d independent (batch, kv-head) units of %s per step (of %d in the full workload)" % (
        n_units, wname, w["B"] * w["Hkv"])
    line = {
        "impl": "reference", "metric": metric_name(w), "value": value, "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": tot_t / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_of(w, wname),
        "cpu_baseline": {"value": value, "unit": unit, "cores": min(threads, n_units), "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def gpu_reference(w):
    """The reference's own CUDA composition of the same attention (cuBLAS batched gemm + its generic kernels,
    src/Function/FuncNNLayer.h:231-266) on this GPU, through oracle/_ref/shim_driver (the unmodified reference
    sources compiled with USE_CUDA).  Its large-row softmax launch needs B*H*L <= 65535 per call
    (src/Operation/OpNNLayerCuda.cuh:375), so one chunk of (batch, head) slices is timed and the whole
    configuration is that time x the number of chunks."""
    drv = os.path.join(ROOT, "oracle", "_ref", "shim_driver")
    if not os.path.exists(drv):
        return {"unavailable": "oracle/_ref/shim_driver not built (needs the reference tree at build time)"}
    per_chunk = max(1, 65535 // w["L"])
    n_slices = w["B"] * w["Hq"]
    n = min(per_chunk, n_slices)
    rng = np.random.default_rng(77)
    tmp = tempfile.mkdtemp()
    try:
        paths = []
        for name, S in (("q", w["L"]), ("k", w["S"]), ("v", w["S"])):
            pth = os.path.join(tmp, name + ".bin")
            (rng.standard_normal((n, 1, S, w["D"]), dtype=np.float32) * np.float32(w["std"])).tofile(pth)
            paths.append(pth)
        cmd = [drv, "fwd", w["dtype"], str(n), "1", "1", str(w["L"]), str(w["S"]), str(w["D"]), "1" if w["causal"] else "0",
               "ref", str(n), "0"] + paths + [os.path.join(tmp, "o.bin")]
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
        ms = None
        for tok in r.stdout.split():
            if tok.startswith("ms="):
                ms = float(tok[3:])
        if r.returncode != 0 or ms is None:
            return {"unavailable": "shim_driver failed: %s" % (r.stderr.strip()[-200:] or r.stdout.strip()[-200:])}
        chunks = -(-n_slices // n)
        unit = dict(w, B=n, Hq=1, Hkv=1)
        return {"value": step_flops(unit) / (ms / 1e3) / 1e12, "unit": "TFLOP/s", "ms_per_chunk": ms,
                "slices_per_chunk": n, "chunks": chunks, "extrapolated": True,
                "ms_whole_config": ms * n_slices / n,
                "what": "function::sdpAttention of the reference on CUDA tensors, %s" % w["dtype"]}
    except Exception as e:  # a baseline must not take the benchmark down
        return {"unavailable": "%s: %s" % (type(e).__name__, e)}
    finally:
        for f in os.listdir(tmp):
            os.unlink(os.path.join(tmp, f))
        os.rmdir(tmp)


def metric_name(w):
    return "decode HBM GB/s" if w["kind"] == "decode" else "attention TFLOP/s (causal-adj)"


def config_of(w, wname):
    return {"workload": "%s: %s %s B=%d Hq=%d Hkv=%d L=%d S=%d D=%d causal=%s" % (
        wname, w["kind"], w["dtype"], w["B"], w["Hq"], w["Hkv"], w["L"], w["S"], w["D"], w["causal"]),
        "l2": "inputs larger than L2 (no flush)" if w["kind"] != "fwdbwd" or w["B"] > 2 else "fits L2",
        "sharding": "batch x head units per rank, no collective"}


# ------------------------------------------------------------------ GPU side --
def run_ours(args, w, wname):
    import torch
    import torch.distributed as dist
    from tinytorch_b200 import op

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the attention ops have no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    TDT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
    peaks = measured_peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        """Device time of `steps` calls of fn: CUDA events on the launching stream, max over ranks."""
        for _ in range(warmup):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / 1e3

    def build_inputs(wl, seed):
        g = torch.Generator(device=dev).manual_seed(seed + rank)
        mk = lambda *s: (torch.randn(s, generator=g, device=dev) * wl["std"]).to(TDT[wl["dtype"]])
        q = mk(wl["B"], wl["Hq"], wl["L"], wl["D"])
        k = mk(wl["B"], wl["Hkv"], wl["S"], wl["D"])
        v = mk(wl["B"], wl["Hkv"], wl["S"], wl["D"])
        return q, k, v

    def measure(wl, name, steps, warmup, with_e2e):
        tdt = TDT[wl["dtype"]]  # each configuration in its own dtype
        q, k, v = build_inputs(wl, 1234)
        res = {}
        if wl["kind"] == "decode":
            lens_np = np.random.default_rng(1234 + rank).integers(1024, wl["S"] + 1, size=wl["B"]).astype(np.int32)
            if wl.get("append"):
                lens_np = np.minimum(lens_np, wl["S"] - 1)  # room for the step's row
            lens = torch.from_numpy(lens_np).to(dev)
            if wl.get("append"):
                kn, vn = k[:, :, :1].contiguous(), v[:, :, :1].contiguous()
                cos, sin = op.ropeTables(wl["S"], wl["D"], device=dev)
                fn = lambda: op.sdpAttentionDecodeAppend(q, kn, vn, k, v, lens, cos, sin)
                work = decode_bytes(wl, lens_np + 1)
            else:
                fn = lambda: op.sdpAttentionDecode(q, k, v, lens)
                work = decode_bytes(wl, lens_np)
            launches = 2
        elif wl["kind"] == "fwdbwd":
            do = torch.randn_like(q)
            def fn():
                o, lse = op.sdpAttentionFwd(q, k, v, isCausal=wl["causal"])
                op.sdpAttentionBwd(do, q, k, v, o, lse, isCausal=wl["causal"])
            work = step_flops(wl)
            launches = 4
        else:
            fn = lambda: op.sdpAttentionFwd(q, k, v, isCausal=wl["causal"])
            work = step_flops(wl)
            launches = 1
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        sec = timed(fn, steps, warmup)
        clocks = sampler.stop() if rank == 0 else {}
        sustained = None
        if rank == 0 and world == 1:
            # The timed region is a few milliseconds, shorter than the sampler's period and than the time the
            # board takes to settle under its power limit.  One more second of the same launches, back to back
            # and timed with CUDA events, shows what the kernel sustains and the clocks it settles at.
            probe = ClockSampler(local)
            probe.start()
            p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            n_probe = 0
            t_end = time.time() + 1.0
            p0.record()
            while time.time() < t_end:
                for _ in range(20):
                    fn()
                n_probe += 20
                if n_probe % 200 == 0:
                    torch.cuda.synchronize()  # bounds the launch queue; the device stays busy for a second
            p1.record()
            torch.cuda.synchronize()
            probe_sec = p0.elapsed_time(p1) / 1e3
            clocks["sustained_probe"] = probe.stop()
            sustained = {"steps": n_probe, "seconds": probe_sec, "clocks": clocks["sustained_probe"]}
        decode = wl["kind"] == "decode"
        div = 1e9 if decode else 1e12
        per_gpu = work * steps / sec / div
        res.update(value=per_gpu * world, ms_per_step=sec / steps * 1e3, clocks=clocks, launches=launches * steps,
                   per_gpu=per_gpu, work=work)
        peak = peaks["gbs"] if decode else peaks["tflops"]
        if sustained:
            sv = work * sustained["steps"] / sustained["seconds"] / div
            speak = peak if decode else peaks["tflops_sustained"]
            sustained.update(value=sv, unit="GB/s" if decode else "TFLOP/s", peak=speak, frac=sv / speak,
                             peak_source="copy rate (MEASURED_PEAKS.json)" if decode
                             else "bf16 matmul back to back for seconds (MEASURED_PEAKS.json, bf16_tflops_sustained)")
            res["sustained"] = sustained
        train = wl["kind"] == "fwdbwd"
        # the kernel that takes most of the step's device time (profiles/launch_list_bench_default.md)
        kern = (("decode_tc_kernel" if wl["Hq"] != wl["Hkv"] else "decode_kernel") if decode
                else ("fwd_simt_kernel" if wl["dtype"] == "f32" else
                      (("bwd_tc64_kernel" if wl["D"] == 64 else "bwd_tc_kernel") if train else "fwd_tc_kernel")))
        # algorithmic bytes of that kernel's launch (backward: Q, K, V, dO read, dK, dV and the fp32 dQ written)
        alg_bytes = work if decode else (fwd_bytes(wl) if wl["kind"] == "fwd" else (
            float((4 * wl["B"] * wl["Hq"] * wl["L"] * wl["D"] + 2 * wl["B"] * wl["Hkv"] * wl["S"] * wl["D"]) * ESIZE[wl["dtype"]]
                  + 4 * wl["B"] * wl["Hq"] * wl["L"] * (wl["D"] + 2)) if wl["dtype"] != "f32" else None))
        traffic, traffic_src = traffic_of(kern, alg_bytes)
        nominal = nominal_peaks()["gbs" if decode else "tflops"]
        res["roofline"] = {"bound": "hbm" if decode else "tensor", "achieved": per_gpu, "peak": peak,
                           "unit": "GB/s" if decode else "TFLOP/s", "frac": per_gpu / peak, "traffic": traffic,
                           "traffic_source": traffic_src, "algorithmic_bytes": alg_bytes,
                           "peak_source": peaks["source"], "frac_nominal": per_gpu / nominal, "kernel": kern}
        if with_e2e:
            # public API with HOST buffers: pinned inputs -> device, op, result -> pinned host, every step
            hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
            ho = torch.empty(q.shape, dtype=tdt).pin_memory()
            train = wl["kind"] == "fwdbwd"
            if train:
                # fwd + bwd on host buffers: inputs and dO in, O and the three gradients out
                dq_, dk_, dv_ = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
                hdo = do.cpu().pin_memory()
                ddo_ = torch.empty_like(q)
                hg = [torch.empty(t.shape, dtype=tdt).pin_memory() for t in (q, k, v)]
                def e2e_step():
                    dq_.copy_(hq, non_blocking=True), dk_.copy_(hk, non_blocking=True), dv_.copy_(hv, non_blocking=True)
                    ddo_.copy_(hdo, non_blocking=True)
                    o, lse = op.sdpAttentionFwd(dq_, dk_, dv_, isCausal=wl["causal"])
                    for h_, g_ in zip(hg, op.sdpAttentionBwd(ddo_, dq_, dk_, dv_, o, lse, isCausal=wl["causal"])):
                        h_.copy_(g_, non_blocking=True)
                    ho.copy_(o, non_blocking=True)
            else:
                # the public host-buffer call: chunked over the batch, copies and kernels overlapped
                from tinytorch_b200.host import HostAttention
                pipe = HostAttention(q.shape, k.shape, tdt, device=dev, chunks=4, decode=decode)
                def e2e_step():
                    pipe(hq, hk, hv, ho, isCausal=wl["causal"], kvLens=lens if decode else None)
            es = max(2, min(steps, 5))
            sec2 = timed(e2e_step, es, 1)
            h2d = sum(t.numel() * t.element_size() for t in ((hq, hk, hv, hdo) if train else (hq, hk, hv)))
            d2h = ho.numel() * ho.element_size() + (sum(t.numel() * t.element_size() for t in hg) if train else 0)
            # What the host link alone allows: the same pinned buffers copied in and out, no kernel.  With N ranks
            # on one host the copies of all ranks share its PCIe root ports and memory bandwidth.
            dsts = [torch.empty_like(t, device=dev) for t in ((hq, hk, hv, hdo) if train else (hq, hk, hv))]
            outs = ([ho] + hg) if train else [ho]
            dos = [torch.empty_like(t, device=dev) for t in outs]
            cp_in, cp_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
            def copy_only():
                cur = torch.cuda.current_stream(dev)
                cp_in.wait_stream(cur), cp_out.wait_stream(cur)
                with torch.cuda.stream(cp_in):
                    for d_, h_ in zip(dsts, (hq, hk, hv, hdo) if train else (hq, hk, hv)):
                        d_.copy_(h_, non_blocking=True)
                with torch.cuda.stream(cp_out):
                    for h_, d_ in zip(outs, dos):
                        h_.copy_(d_, non_blocking=True)
                cur.wait_stream(cp_in), cur.wait_stream(cp_out)
            sec3 = timed(copy_only, es, 1)
            res["e2e"] = {"value": work * es / sec2 / div * world, "unit": "GB/s" if decode else "TFLOP/s",
                          "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                          "ms_per_step": sec2 / es * 1e3,
                          "copy_only_ms_per_step": sec3 / es * 1e3,
                          "host_link_gbs": (h2d + d2h) * world * es / sec3 / 1e9,
                          "frac_of_copy_ceiling": sec3 / sec2}
        return res

    def strong(wl, name, steps, warmup):
        """The named configuration partitioned over the ranks: each rank holds only its contiguous range of
        (batch, kv-head) units (tinytorch_b200.shard.unit_range), runs the same kernels on it, and the value is
        the whole configuration's work over the slowest rank's time.  Then the optional all-gather of O."""
        from tinytorch_b200 import shard
        n_units = wl["B"] * wl["Hkv"]
        g = wl["Hq"] // wl["Hkv"]
        decode = wl["kind"] == "decode"
        ranges = None
        if decode:
            # lengths belong to sequences; every unit of a sequence carries its sequence's length.  Units are
            # split by work (valid cache rows), not by count: equal counts of config 4's units differ by up to
            # 36 % in rows at 8 ranks, and the slowest rank is the time
            lens_b = np.random.default_rng(1234).integers(1024, wl["S"] + 1, size=wl["B"]).astype(np.int32)
            lens_all = np.repeat(lens_b, wl["Hkv"])
            ranges = shard.balanced_ranges(lens_all.tolist(), world)
            u0, u1 = ranges[rank]
        else:
            u0, u1 = shard.unit_range(n_units, rank, world)
        sw = dict(wl, B=u1 - u0, Hq=g, Hkv=1)  # a unit is one kv head with its g query heads: a batch entry of its own
        q, k, v = build_inputs(sw, 4321)
        if decode:
            lens_u = lens_all[u0:u1].copy()
            lens = torch.from_numpy(lens_u).to(dev)
            fn = lambda: op.sdpAttentionDecode(q, k, v, lens)
            total = decode_bytes(wl, lens_b)
        else:
            fn = lambda: op.sdpAttentionFwd(q, k, v, isCausal=wl["causal"])
            total = step_flops(wl)
        sec = timed(fn, steps, warmup)
        # all-gather of the rank's O block on a side stream, handed over by events
        # (reference: src/Distributed/BackendNCCL.cpp:49-62, src/Distributed/BackendNCCL.h:167-189)
        o = fn()[0]
        o_view = o.reshape(1, (u1 - u0) * g, wl["L"], wl["D"])
        side = torch.cuda.Stream(dev)
        def gather():
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                out = shard.all_gather_output(o_view, n_units, world, group_size=g, ranges=ranges)
            torch.cuda.current_stream(dev).wait_stream(side)
            return out
        gsec = timed(gather, 3, 1)
        div = 1e9 if decode else 1e12
        return {"value": total * steps / sec / div, "unit": "GB/s" if decode else "TFLOP/s",
                "ms_per_step": sec / steps * 1e3,
                "units_per_rank": ([e - b for b, e in ranges] if ranges else [n_units // world, -(-n_units // world)]),
                "partition": "contiguous unit ranges of equal work (valid cache rows)" if ranges
                else "contiguous unit ranges of equal size",
                "allgather_ms": gsec / 3 * 1e3, "allgather_bytes": wl["B"] * wl["Hq"] * wl["L"] * wl["D"] * ESIZE[wl["dtype"]],
                "scaling": "strong", "config": config_of(wl, name)}

    main = measure(w, wname, args.steps, args.warmup, with_e2e=not args.no_e2e)
    extra, others = None, {}
    strong_keys = {}
    if wname == "prefill" and world > 1 and not args.no_decode:
        strong_keys["prefill"] = strong(w, wname, args.steps, args.warmup)
        strong_keys["decode"] = strong(WORKLOADS["decode"], "decode", max(5, args.steps), max(3, args.warmup))
    if wname == "prefill" and not args.no_decode:
        extra = measure(WORKLOADS["decode"], "decode", max(5, args.steps), max(3, args.warmup), with_e2e=False)
        # the other configurations of the benchmark table, device-resident inputs only
        others = {n: measure(WORKLOADS[n], n, max(5, args.steps), max(3, args.warmup), with_e2e=False)
                  for n in ("gqa", "train")}

    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu:
            runner, kind = cpu_reference_runner()
            # bounded sample: a few units of the same workload on one core (the reference is single-threaded)
            n = {"prefill": 6, "gqa": 4, "train": 6, "cfg1": 8, "decode": 16, "decode_ncu": 16}.get(wname, 4)
            dt, work = cpu_sample(w, runner, kind, n, 1)
            dec = w["kind"] == "decode"
            cpu = {"value": work / dt / (1e9 if dec else 1e12), "unit": "GB/s" if dec else "TFLOP/s", "cores": 1,
                   "kind": kind, "sample": "%d of %d (batch, kv-head) units of %s, %.1f s" % (
                       n, w["B"] * w["Hkv"], wname, dt)}
        decode = w["kind"] == "decode"
        line = {
            "metric": metric_name(w), "value": main["value"], "unit": "GB/s" if decode else "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": main["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": w["dtype"],
            "data": "synthetic", "config": config_of(w, wname), "clocks": main["clocks"],
            "e2e": main.get("e2e"), "gpu_launches": main["launches"], "roofline": main["roofline"],
            "cpu_baseline": cpu,
        }
        if main.get("sustained"):
            line["sustained"] = main["sustained"]
        if world == 1 and wname == "prefill" and not args.no_decode and not args.no_cpu:
            line["gpu_reference"] = gpu_reference(w)
        for n, r in others.items():
            line[n] = {"metric": metric_name(WORKLOADS[n]), "value": r["value"], "unit": "TFLOP/s",
                       "ms_per_step": r["ms_per_step"], "roofline": r["roofline"],
                       "config": config_of(WORKLOADS[n], n), "clocks": r["clocks"]}
            if r.get("sustained"):
                line[n]["sustained"] = r["sustained"]
        if strong_keys:
            line["strong"] = strong_keys
        # last, so that a record that keeps only the end of the line keeps the decode figures
        if extra:
            line["decode"] = {"metric": "decode HBM GB/s", "value": extra["value"], "unit": "GB/s",
                              "ms_per_step": extra["ms_per_step"], "roofline": extra["roofline"],
                              "config": config_of(WORKLOADS["decode"], "decode"), "clocks": extra["clocks"]}
            if extra.get("sustained"):
                line["decode"]["sustained"] = extra["sustained"]
            if strong_keys:
                line["decode"]["strong_value"] = strong_keys["decode"]["value"]
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_fused(args, w, wname):
    """fusedAddRmsNorm / siluMul: GB/s over the algorithmic bytes (every tensor crosses HBM once)."""
    import torch
    import torch.distributed as dist
    from tinytorch_b200 import fused as F

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the fused ops have no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    rows, dim, es = w["rows"], w["dim"], ESIZE[w["dtype"]]
    tdt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[w["dtype"]]
    g = torch.Generator(device=dev).manual_seed(4321 + rank)
    rms = w["opname"] == "fusedAddRmsNorm"
    lin = w["opname"] == "linear"
    if lin:
        x = (torch.randn((rows, dim), generator=g, device=dev) * 0.5).to(tdt)
        wt = (torch.randn((w["n_out"], dim), generator=g, device=dev) * 0.05).to(tdt)
        bs = torch.randn((w["n_out"],), generator=g, device=dev).to(tdt)
        fn = lambda: F._linear_raw(x, wt, bs)
        nbytes = 2.0 * rows * dim * w["n_out"]  # FLOPs for this operator
        h2d, d2h = rows * dim * es, rows * w["n_out"] * es
    elif rms:
        a = torch.randn((rows, dim), generator=g, device=dev).to(tdt)
        b = torch.randn((rows, dim), generator=g, device=dev).to(tdt)
        wt = torch.ones(dim, device=dev, dtype=tdt)
        fn = lambda: F.fusedAddRmsNorm(a, b, wt, 1e-5)
        nbytes = float(4 * rows * dim * es + dim * es)  # read input, residual; write both; weight once
        h2d, d2h = 2 * rows * dim * es, 2 * rows * dim * es
    else:
        x = torch.randn((rows, 2 * dim), generator=g, device=dev).to(tdt)
        fn = lambda: F.siluMul(x)
        nbytes = float(3 * rows * dim * es)
        h2d, d2h = 2 * rows * dim * es, rows * dim * es

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(f, steps, warmup):
        for _ in range(warmup):
            f()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            f()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / 1e3

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    sec = timed(fn, args.steps, args.warmup)
    clocks = sampler.stop() if rank == 0 else None
    div, unit = (1e12, "TFLOP/s") if lin else (1e9, "GB/s")
    per_gpu = nbytes * args.steps / sec / div
    peaks = measured_peaks()
    peak = peaks["tflops"] if lin else peaks["gbs"]
    fused_kernel = "linear_tc_kernel" if lin else ("add_rms_norm_kernel" if rms else "silu_mul_kernel")
    fused_alg = float((rows * dim + w["n_out"] * dim + rows * w["n_out"]) * ESIZE[w["dtype"]]) if lin else nbytes
    fused_traffic = traffic_of(fused_kernel, fused_alg)
    line = {
        "metric": "projection TFLOP/s" if lin else w["opname"] + " HBM GB/s", "value": per_gpu * world, "unit": unit,
        "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic (seeded normal)",
        "config": {"workload": "%s rows=%d dim=%d %s" % (w["opname"], rows, dim, w["dtype"]),
                   "l2": "tensors larger than L2 (no flush)", "sharding": "rows per rank, no collective"},
        "roofline": {"bound": "tensor" if lin else "hbm", "achieved": per_gpu, "peak": peak, "unit": unit,
                     "frac": per_gpu / peak, "traffic": fused_traffic[0], "traffic_source": fused_traffic[1],
                     "peak_source": peaks["source"],
                     "frac_nominal": per_gpu / nominal_peaks()["tflops" if lin else "gbs"], "kernel": fused_kernel},
        "clocks": clocks, "gpu_launches": args.steps,
    }
    if not args.no_e2e:
        # host buffers: pinned H2D of the inputs, the kernel, D2H of what the op produces
        if lin:
            hx = torch.empty((rows, dim), dtype=tdt).pin_memory()
            hy = torch.empty((rows, w["n_out"]), dtype=tdt).pin_memory()
            def e2e():
                x.copy_(hx, non_blocking=True)
                hy.copy_(F._linear_raw(x, wt, bs), non_blocking=True)
        elif rms:
            ha, hb = (torch.empty((rows, dim), dtype=tdt).pin_memory() for _ in range(2))
            def e2e():
                a.copy_(ha, non_blocking=True), b.copy_(hb, non_blocking=True)
                F.fusedAddRmsNorm(a, b, wt, 1e-5)
                ha.copy_(a, non_blocking=True), hb.copy_(b, non_blocking=True)
        else:
            hx, ho = torch.empty((rows, 2 * dim), dtype=tdt).pin_memory(), torch.empty((rows, dim), dtype=tdt).pin_memory()
            def e2e():
                x.copy_(hx, non_blocking=True)
                ho.copy_(F.siluMul(x), non_blocking=True)
        n2 = max(3, args.steps // 4)
        sec2 = timed(e2e, n2, 2)
        line["e2e"] = {"value": nbytes * n2 / sec2 / div * world, "unit": unit, "h2d_bytes_per_step": h2d,
                       "d2h_bytes_per_step": d2h}
    if rank == 0 and not args.no_cpu:
        line["cpu_baseline"] = fused_cpu_sample(w)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def fused_cpu_sample(w, budget_rows=None):
    """The reference's own CPU code (oracle/_ref) or the C port on a bounded slice of the rows, one core."""
    from oracle.loader import FusedOracle, Reference
    ref = Reference() if Reference.available() else FusedOracle()
    kind = "reference" if Reference.available() else "port"
    rows = budget_rows or max(1, min(w["rows"], (1 << 28) // (w["dim"] * 4 * 4)))  # ~256 MB of fp32 traffic
    rng = np.random.default_rng(9)
    es = ESIZE[w["dtype"]]
    if w["opname"] == "linear":
        rows = budget_rows or 8  # 8 rows x 4096 x 12288 = 0.8 GFLOP of the reference's scalar gemm
        x = rng.standard_normal((rows, w["dim"]), dtype=np.float32)
        wt = rng.standard_normal((w["n_out"], w["dim"]), dtype=np.float32)
        bs = rng.standard_normal(w["n_out"], dtype=np.float32)
        t0 = time.perf_counter()
        ref.linear(x, wt, bs)
        dt = time.perf_counter() - t0
        return {"value": 2.0 * rows * w["dim"] * w["n_out"] / dt / 1e12, "unit": "TFLOP/s", "cores": 1, "kind": kind,
                "sample": "%d of %d rows, fp32 on the host" % (rows, w["rows"])}
    if w["opname"] == "fusedAddRmsNorm":
        a, b = (rng.standard_normal((rows, w["dim"]), dtype=np.float32) for _ in range(2))
        wt = np.ones(w["dim"], dtype=np.float32)
        t0 = time.perf_counter()
        ref.fused_add_rms_norm(a, b, wt, 1e-5)
        dt = time.perf_counter() - t0
        nbytes = 4 * rows * w["dim"] * es
    else:
        x = rng.standard_normal((rows, 2 * w["dim"]), dtype=np.float32)
        t0 = time.perf_counter()
        ref.silu_mul(x)
        dt = time.perf_counter() - t0
        nbytes = 3 * rows * w["dim"] * es
    return {"value": nbytes / dt / 1e9, "unit": "GB/s", "cores": 1, "kind": kind,
            "sample": "%d of %d rows, fp32 on the host, bytes counted at the workload's dtype" % (rows, w["rows"])}


def run_fused_reference_arm(args, w, wname):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals = []
    for _ in range(args.warmup + args.steps):
        vals.append(fused_cpu_sample(w, budget_rows=4 if w["opname"] == "linear" else max(1, (1 << 26) // (w["dim"] * 4 * 4))))
    vals = vals[args.warmup:]
    v = float(np.mean([x["value"] for x in vals]))
    cb = dict(vals[0], value=v)
    print(json.dumps({
        "impl": "reference", "metric": "projection TFLOP/s" if w["opname"] == "linear" else w["opname"] + " HBM GB/s",
        "value": v, "unit": vals[0]["unit"],
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": None, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic (seeded normal)",
        "config": {"workload": "%s rows=%d dim=%d (bounded sample per step)" % (w["opname"], w["rows"], w["dim"])},
        "cpu_baseline": cb, "e2e": {"value": v, "unit": vals[0]["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def run_loop(args, w, wname):
    """32 layers x (rotary embedding + cache append + grouped-query attention) for one token, per step:
    eager launches against one CUDA-graph replay.  Value: layer-steps per second through the graph."""
    import torch
    from tinytorch_b200 import _capi, op

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    B, Hq, Hkv, S, D, L = w["B"], w["Hq"], w["Hkv"], w["S"], w["D"], w["layers"]
    g = torch.Generator(device=dev).manual_seed(99)
    mk = lambda *s: torch.randn(s, generator=g, device=dev).to(torch.bfloat16)
    caches = [(mk(B, Hkv, S, D), mk(B, Hkv, S, D)) for _ in range(L)]
    q, kn, vn = mk(B, Hq, 1, D), mk(B, Hkv, 1, D), mk(B, Hkv, 1, D)
    lens = torch.full((B,), S // 2, dtype=torch.int32, device=dev)
    cos, sin = op.ropeTables(S, D, device=dev)

    def step():
        out = q
        for kc, vc in caches:
            out, _, _ = op.sdpAttentionDecodeAppend(out, kn, vn, kc, vc, lens, cos, sin)
        return out

    def timed(fn, n):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 1e3 / n

    t_eager = timed(step, args.steps)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        step()
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            step()
    torch.cuda.current_stream().wait_stream(side)
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    t_graph = timed(graph.replay, args.steps)
    clocks = sampler.stop()
    nbytes = float(L * B * (S // 2 + 1) * Hkv * D * 2 * 2)
    print(json.dumps({
        "metric": "decode layer-steps/s (CUDA graph)", "value": L / t_graph, "unit": "layer-steps/s", "n_gpus": 1,
        "steps": args.steps, "warmup": 3, "ms_per_step": t_graph * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic (seeded normal)",
        "config": {"workload": "token loop: %d layers, B=%d Hq=%d Hkv=%d cache %d (half full) D=%d, rotary + append + attention"
                               % (L, B, Hq, Hkv, S, D)},
        "eager": {"value": L / t_eager, "unit": "layer-steps/s", "ms_per_step": t_eager * 1e3},
        "roofline": {"bound": "hbm", "achieved": nbytes / t_graph / 1e9, "peak": measured_peaks()["gbs"], "unit": "GB/s",
                     "frac": nbytes / t_graph / 1e9 / measured_peaks()["gbs"], "traffic": None,
                     "peak_source": measured_peaks()["source"], "kernel": "decode_tc_kernel"},
        "clocks": clocks, "gpu_launches": 4 * L * args.steps,
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="prefill", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-decode", action="store_true", help="skip the secondary measurements (decode, GQA prefill, training step)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    if w["kind"] == "loop":
        run_loop(args, w, args.workload)
    elif w["kind"] == "fused":
        (run_fused_reference_arm if args.impl == "reference" else run_fused)(args, w, args.workload)
    elif args.impl == "reference":
        run_reference_arm(args, w, args.workload)
    else:
        run_ours(args, w, args.workload)


if __name__ == "__main__":
    main()
