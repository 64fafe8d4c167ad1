"""Build libferro_b200.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

Usage: python -m ferro_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  The library lands in ferro_b200/lib/ and is
loaded by ferro_b200._lib through ctypes; nothing is installed elsewhere.
"""
import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(HERE, "..", "include")
OUT_DIR = os.path.join(HERE, "lib")
OBJ_DIR = os.path.join(OUT_DIR, "obj")
LIB = os.path.join(OUT_DIR, "libferro_b200.so")

SOURCES = ["api.cu", "elementwise.cu", "chain.cu", "chain_interp_tile.cu", "chain_interp_seg.cu", "chain_static.cu",
           "reduce.cu", "softmax.cu", "layer_norm.cu", "optim.cu", "mlp.cu", "ddp.cu", "rng.cu", "views.cu", "index_ops.cu", "wire.cu", "host_pipe.cu", "dlpack.cu"]

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr", "-I", INCLUDE]
# -fmad=false where results must equal ferro's CPU path bit for bit: that path
# rounds every multiply and add separately (Rust never contracts), and its
# optimizer and exact-kind tests compare bitwise.  The row kernels (softmax,
# LayerNorm, reductions) are held to a relative tolerance instead and are
# bound by instruction issue as much as by HBM, so they keep the fused
# multiply-add.
NO_FMAD = {"index_ops.cu", "elementwise.cu", "chain.cu", "chain_interp_tile.cu", "chain_interp_seg.cu", "chain_static.cu", "optim.cu",
           "mlp.cu"}


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _includes(path, seen=None):
    """Files `path` pulls in through #include "...", transitively (quoted includes only)."""
    seen = set() if seen is None else seen
    with open(path) as f:
        for line in f:
            line = line.strip()
            if not line.startswith('#include "'):
                continue
            dep = os.path.normpath(os.path.join(os.path.dirname(path), line.split('"')[1]))
            if dep not in seen and os.path.exists(dep):
                seen.add(dep)
                _includes(dep, seen)
    return seen


def build(force=False, verbose=False):
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = _nvcc()
    jobs = []
    objs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
        objs.append(o)
        if force or _stale(o, [s, os.path.abspath(__file__), *_includes(s)]):
            cmd = [nvcc, *NVCC_FLAGS, *(["-fmad=false"] if src in NO_FMAD else []), "-c", s, "-o", o]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for cmd, r in ex.map(run, jobs):
            if verbose or r.returncode != 0:
                sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {cmd[-3]}")
    if force or jobs or _stale(LIB, objs):
        cmd = [nvcc, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
               "-cudart", "shared", "-ldl", "-lpthread"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
