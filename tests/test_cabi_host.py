"""CPU-side checks of the C ABI: the library loads, exports every symbol the header declares,
validates parameters like the reference, and refuses to compute without a GPU."""
import ctypes
import os
import re

import pytest

import portdnn_b200 as pd

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L():
    from portdnn_b200 import build
    build.build()
    return pd.lib()


def test_every_declared_symbol_is_exported(L):
    hdr = open(os.path.join(ROOT, "include", "portdnn_b200.h")).read()
    names = sorted(set(re.findall(r"\b(pdnn_\w+)\s*\(", hdr)))
    assert len(names) >= 15
    for n in names:
        assert hasattr(L, n), n


def test_param_structs_match_header_layout():
    assert ctypes.sizeof(pd.Conv2DParams) == 19 * 4
    assert ctypes.sizeof(pd.DepthwiseConv2DParams) == 13 * 4
    assert ctypes.sizeof(pd.PoolingParams) == 13 * 4


def test_validate_params_like_reference(L):
    # include/portdnn/internal/conv2d/launch.h:42-97,169-197
    ok = pd.conv_params(1, 8, 8, 4, 4, 3, 1)
    assert pd.conv2d_validate(pd.FORWARD, ok, pd.ALGO_DIRECT) == pd.StatusCode.OK
    for field, val in (("batch", 0), ("channels", 0), ("features", -1), ("in_rows", 0), ("out_cols", 0),
                       ("window_rows", 0), ("stride_cols", 0), ("pad_rows", -1), ("dilation_rows", 2)):
        p = pd.conv_params(1, 8, 8, 4, 4, 3, 1)
        setattr(p, field, val)
        assert pd.conv2d_validate(pd.FORWARD, p, pd.ALGO_DIRECT) == pd.StatusCode.InvalidParameter, field
    p = pd.conv_params(1, 8, 8, 4, 4, 3, 1)
    p.input_format, p.filter_format = 0, 1          # NHWC with FCHW
    assert pd.conv2d_validate(pd.FORWARD, p, pd.ALGO_DIRECT) == pd.StatusCode.InvalidParameter
    p = pd.conv_params(1, 8, 8, 4, 4, 3, 1, groups=2)
    assert pd.conv2d_validate(pd.INPUT_BACKPROP, p, pd.ALGO_IM2COL) == pd.StatusCode.InvalidParameter
    assert pd.conv2d_validate(pd.FORWARD, p, pd.ALGO_DIRECT) == pd.StatusCode.InvalidAlgorithm
    assert pd.conv2d_validate(pd.FORWARD, p, pd.ALGO_IM2COL) == pd.StatusCode.OK
    p = pd.conv_params(1, 8, 8, 4, 4, 3, 1)
    assert pd.conv2d_validate(pd.FORWARD, p, 0) == pd.StatusCode.InvalidAlgorithm   # NotSupported
    assert pd.conv2d_validate(pd.FORWARD, p, pd.ALGO_MATMUL) == pd.StatusCode.InvalidParameter  # 3x3 is no matmul
    p.input_format, p.filter_format = 1, 1          # NCHW: Direct only
    assert pd.conv2d_validate(pd.FORWARD, p, pd.ALGO_TILED) == pd.StatusCode.InvalidAlgorithm


def test_algorithm_tags_report_the_reference_status(L):
    """Which (algorithm, window, stride, pass) combinations the reference's launchers refuse, and how:
    src/conv2d/tiled/launch_tiled.cc:164-273 (InvalidAlgorithm), include/portdnn/internal/conv2d/winograd/launch.h:298-396
    (InvalidAlgorithm), include/portdnn/conv2d/implementation/matmul.h:95-104 (InvalidParameter)."""
    OK, IA, IP = pd.StatusCode.OK, pd.StatusCode.InvalidAlgorithm, pd.StatusCode.InvalidParameter
    cases = [
        # window, stride, pass, algorithm, expected
        (3, 1, pd.FORWARD, pd.ALGO_TILED, OK), (3, 2, pd.INPUT_BACKPROP, pd.ALGO_TILED, OK), (5, 1, pd.FORWARD, pd.ALGO_TILED, OK),
        (5, 2, pd.FORWARD, pd.ALGO_TILED, IA), (7, 1, pd.FORWARD, pd.ALGO_TILED, IA), (3, 1, pd.FILTER_BACKPROP, pd.ALGO_TILED, IA),
        (3, 1, pd.FORWARD, pd.ALGO_WINOGRAD, OK), (3, 1, pd.FILTER_BACKPROP, pd.ALGO_WINOGRAD_LARGE, OK),
        (5, 1, pd.FORWARD, pd.ALGO_WINOGRAD, IA), (1, 1, pd.FORWARD, pd.ALGO_WINOGRAD_LARGE, IA),
        (1, 1, pd.FORWARD, pd.ALGO_MATMUL, OK), (1, 2, pd.FORWARD, pd.ALGO_MATMUL, IP), (3, 1, pd.INPUT_BACKPROP, pd.ALGO_MATMUL, IP),
        (7, 2, pd.FILTER_BACKPROP, pd.ALGO_IM2COL, OK), (11, 4, pd.FORWARD, pd.ALGO_DIRECT, OK),
    ]
    for window, stride, pass_, algo, want in cases:
        p = pd.conv_params(2, 16, 16, 8, 8, window, stride)
        assert pd.conv2d_validate(pass_, p, algo) == want, (window, stride, pass_, algo)
    p = pd.conv_params(2, 16, 16, 8, 8, 3, 1)
    p.window_cols = 1   # 3x1: Winograd only
    assert pd.conv2d_validate(pd.FORWARD, p, pd.ALGO_WINOGRAD) == OK
    assert pd.conv2d_validate(pd.FORWARD, p, pd.ALGO_WINOGRAD_LARGE) == IA
    assert pd.conv2d_validate(pd.FORWARD, p, pd.ALGO_TILED) == IA


def test_padding_helper_matches_oracle(orc):
    for inp in (1, 2, 5, 7, 14, 56, 224):
        for window in (1, 3, 5, 7, 11):
            for stride in (1, 2, 4):
                for same in (True, False):
                    out, pad = orc.padding(inp, window, stride, same)
                    assert pd.calculate_padding(inp, window, stride, same) == (pad, out)


def test_workspace_size_direct_is_zero(L):
    p = pd.conv_params(4, 16, 16, 8, 8, 3, 1)
    assert pd.conv2d_workspace_size(pd.FORWARD, pd.F32, p, pd.ALGO_DIRECT) == (0, 0)
    req, rec = pd.conv2d_workspace_size(pd.FORWARD, pd.F16, p, pd.ALGO_IM2COL)
    assert req == 0   # implicit GEMM reads the tensors in place


def test_compute_fails_loudly_without_gpu(L):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    p = pd.conv_params(1, 4, 4, 8, 8, 3, 1)
    buf = (ctypes.c_float * 4096)()
    st = L.pdnn_conv2d(0, 0, buf, buf, buf, ctypes.byref(p), pd.ALGO_DIRECT, None, ctypes.c_size_t(0), None)
    assert st == pd.StatusCode.AllocationProblem
    assert b"CUDA" in L.pdnn_last_error()
    st = L.pdnn_matmul(0, 0, 0, buf, buf, buf, 1, 8, 8, 8, ctypes.c_float(0), None)
    assert st == pd.StatusCode.AllocationProblem
