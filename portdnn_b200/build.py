"""Builds libportdnn_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

Each source is compiled to its own object (in parallel, only when it or a header changed) and
the objects are linked into the shared library.

Usage: python -m portdnn_b200.build [--force] [--verbose]
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "_obj")
LIB = os.path.join(HERE, "libportdnn_b200.so")
SOURCES = ["c_api.cu", "hbm_kernels.cu", "direct_conv.cu", "tc_gemm.cu", "winograd.cu", "norm_kernels.cu",
           "layout_kernels.cu", "collective.cu"]
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
         "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall"]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _headers():
    return [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))] + \
        [os.path.join(HERE, "..", "include", "portdnn_b200.h")]


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def needs_build():
    return _stale(LIB, [os.path.join(CSRC, s) for s in SOURCES] + _headers())


def _run(cmd, verbose):
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed: %s" % " ".join(cmd))


def build(force=False, verbose=False):
    if not force and not needs_build():
        return LIB
    os.makedirs(OBJ, exist_ok=True)
    nvcc, headers = _nvcc(), _headers()
    jobs = []
    for src in SOURCES:
        path, obj = os.path.join(CSRC, src), os.path.join(OBJ, src[:-3] + ".o")
        if force or _stale(obj, [path] + headers):
            jobs.append([nvcc] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", path, "-o", obj])
    with ThreadPoolExecutor(max_workers=max(1, min(len(jobs), os.cpu_count() or 1))) as pool:
        list(pool.map(lambda c: _run(c, verbose), jobs))
    objs = [os.path.join(OBJ, s[:-3] + ".o") for s in SOURCES]
    _run([nvcc, "-shared", "-cudart", "shared", "-Xcompiler", "-fPIC"] + objs + ["-ldl", "-o", LIB], verbose)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(LIB)
