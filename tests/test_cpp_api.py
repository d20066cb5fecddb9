"""The C++ mirror of portDNN's API (include/portdnn/**): it must compile as plain C++17 against
the C ABI, and on a GPU the reference-style test program tests/cpp/api_test.cc must pass."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")
# api_test: every operator through the sycldnn:: templates; network_test: the layer / network
# wrappers of include/tools/ on a VGG-style and a ResNet-style stack; compat_batchnorm_test: the
# cuDNN-style batchnorm wrappers of include/portdnn/compat/batchnorm.hpp; compat_conv_test: the cuDNN-style
# convolution / pooling calls on the cases of the reference's test/compat/*.cc.
PROGRAMS = ["api_test", "network_test", "compat_batchnorm_test", "compat_conv_test", "event_dependency_test"]


def _paths(name):
    return os.path.join(ROOT, "tests", "cpp", name + ".cc"), os.path.join(ROOT, "tests", "cpp", name)


def _build(name):
    from portdnn_b200 import build
    build.build()
    src, exe = _paths(name)
    deps = [src, os.path.join(ROOT, "include", "portdnn_b200.h"), os.path.join(ROOT, "tests", "cpp", "compat_kat.inc")]
    for sub in ("portdnn", "tools"):
        for d, _, files in os.walk(os.path.join(ROOT, "include", sub)):
            deps += [os.path.join(d, f) for f in files]
    if os.path.exists(exe) and all(os.path.getmtime(exe) >= os.path.getmtime(d) for d in deps):
        return exe
    cmd = ["g++", "-std=c++17", "-Wall", "-I" + os.path.join(ROOT, "include"), "-I" + os.path.join(CUDA, "include"), src,
           "-L" + os.path.join(ROOT, "portdnn_b200"), "-lportdnn_b200", "-L" + os.path.join(CUDA, "lib64"), "-lcudart",
           "-Wl,-rpath," + os.path.join(ROOT, "portdnn_b200"), "-Wl,-rpath," + os.path.join(CUDA, "lib64"), "-o", exe]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert res.returncode == 0, res.stdout
    return exe


@pytest.mark.parametrize("name", PROGRAMS)
def test_headers_compile_and_link(name):
    assert os.path.exists(_build(name))


@pytest.mark.gpu
@pytest.mark.parametrize("name", PROGRAMS)
def test_reference_style_program_passes(name):
    exe = _build(name)
    res = subprocess.run([exe], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    assert res.returncode == 0, res.stdout
    assert "all checks passed" in res.stdout
