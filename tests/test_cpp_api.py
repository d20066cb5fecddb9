"""The C++ mirror of portDNN's API (include/portdnn/**): it must compile as plain C++17 against
the C ABI, and on a GPU the reference-style test program tests/cpp/api_test.cc must pass."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "api_test.cc")
EXE = os.path.join(ROOT, "tests", "cpp", "api_test")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _build():
    from portdnn_b200 import build
    build.build()
    deps = [SRC, os.path.join(ROOT, "include", "portdnn_b200.h")]
    for d, _, files in os.walk(os.path.join(ROOT, "include", "portdnn")):
        deps += [os.path.join(d, f) for f in files]
    if os.path.exists(EXE) and all(os.path.getmtime(EXE) >= os.path.getmtime(d) for d in deps):
        return
    cmd = ["g++", "-std=c++17", "-Wall", "-I" + os.path.join(ROOT, "include"), "-I" + os.path.join(CUDA, "include"), SRC,
           "-L" + os.path.join(ROOT, "portdnn_b200"), "-lportdnn_b200", "-L" + os.path.join(CUDA, "lib64"), "-lcudart",
           "-Wl,-rpath," + os.path.join(ROOT, "portdnn_b200"), "-Wl,-rpath," + os.path.join(CUDA, "lib64"), "-o", EXE]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert res.returncode == 0, res.stdout


def test_headers_compile_and_link():
    _build()
    assert os.path.exists(EXE)


@pytest.mark.gpu
def test_reference_style_program_passes():
    _build()
    res = subprocess.run([EXE], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    assert res.returncode == 0, res.stdout
    assert "all checks passed" in res.stdout
