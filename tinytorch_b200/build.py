"""Compile the CUDA sources under csrc/ into lib/libtt_attn.so (sm_100a only).

nvcc cross-compiles without a GPU.  Object files are rebuilt only when a source
or header is newer.  Run as ``python -m tinytorch_b200.build``.
"""
import concurrent.futures as cf
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "lib")
LIB = os.path.join(OUT, "libtt_attn.so")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers_mtime():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs.append(os.path.join(HERE, "..", "include", "tt_attn.h"))
    hs.append(os.path.join(HERE, "..", "include", "tt_fused.h"))
    return max(os.path.getmtime(h) for h in hs)


def _compile(src, verbose, out_dir=None, defines=()):
    obj = os.path.join(out_dir or OUT, src[:-3] + ".o")
    spath = os.path.join(CSRC, src)
    if os.path.exists(obj) and os.path.getmtime(obj) > max(os.path.getmtime(spath), _headers_mtime()):
        return obj
    cmd = [NVCC] + FLAGS + ["-D" + d for d in defines] + (["-Xptxas", "-v"] if verbose else []) + ["-c", spath, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, r.stdout, r.stderr))
    if verbose:
        sys.stderr.write(r.stderr)
    return obj


def build(verbose=False, force=False, out_dir=None, defines=()):
    """Build into `out_dir` (default lib/).  `defines` are extra -D macros, used to
    build tuning variants side by side; load one with TT_ATTN_LIB=<path>."""
    out = out_dir or OUT
    lib = os.path.join(out, "libtt_attn.so")
    os.makedirs(out, exist_ok=True)
    if force:
        for f in os.listdir(out):
            if f.endswith((".o", ".so")):
                os.remove(os.path.join(out, f))
    with cf.ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose, out, defines), _sources()))
    if os.path.exists(lib) and os.path.getmtime(lib) > max(os.path.getmtime(o) for o in objs):
        return lib
    LIB = lib
    # cudart is linked statically (nvcc default), so the library loads on a
    # machine without a driver; the driver's tensor-map encoder is looked up at
    # run time through cudaGetDriverEntryPoint.
    cmd = [NVCC, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n%s\n%s" % (r.stdout, r.stderr))
    return LIB


if __name__ == "__main__":
    defs = [a[2:] for a in sys.argv[1:] if a.startswith("-D")]
    outs = [a[6:] for a in sys.argv[1:] if a.startswith("--out=")]
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv, out_dir=outs[0] if outs else None, defines=defs))
