"""Builds the test-only CUDA helpers of this directory (none of them is part of the library)."""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")


def build(name="wait_timeout"):
    src, lib = os.path.join(HERE, name + ".cu"), os.path.join(HERE, "lib%s.so" % name)
    deps = [src, os.path.join(ROOT, "portdnn_b200", "csrc", "umma.cuh")]
    if os.path.exists(lib) and all(os.path.getmtime(lib) >= os.path.getmtime(d) for d in deps):
        return lib
    cmd = [NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O2", "-std=c++17", "-Xcompiler", "-fPIC",
           "-shared", "-cudart", "shared", src, "-o", lib]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError(res.stdout)
    return lib


if __name__ == "__main__":
    print(build())
