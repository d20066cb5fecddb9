"""Winograd F(2x2,3x3) (Algorithm::Winograd / WinogradLarge with a workspace) against the CPU
oracle, through the C ABI: forward and input backprop of 3x3 stride-1 layers.

The transforms add rounding steps the direct algorithms do not have; the bars are nevertheless
the same as for the implicit GEMM (fp32 through 3xTF32 products <= 1e-4, fp16 / bf16 <= 2e-2,
relative to the largest reference value).  Each case also checks, by the launch counter, that
the three transforms and the batched matmul really ran.
"""
import numpy as np
import pytest
import torch

import portdnn_b200 as pd
from conftest import rel_err
from gpu_util import TORCH_DTYPES, assert_no_device_error, rounded, to_dev, to_host

pytestmark = pytest.mark.gpu

WINO_TOL = {"f32": 1e-4, "f16": 2e-2, "bf16": 2e-2}

SHAPES = [
    # n, h, w, c, k, same, pad
    (1, 56, 56, 256, 256, True, None),   # the single VGG-style layer
    (2, 28, 28, 128, 128, True, None),
    (3, 15, 13, 24, 40, True, None),     # odd output extents: partial 2x2 tiles
    (2, 9, 11, 16, 8, False, None),      # VALID
    (1, 7, 7, 512, 512, True, None),
    (2, 10, 10, 8, 8, None, 2),          # "full" padding
]


def _case(orc, dtype, n, h, w, c, k, same, pad, seed=11):
    rng = np.random.default_rng(seed)
    p = pd.conv_params(n, h, w, c, k, 3, 1, bool(same), pad)
    po = orc.conv_params(n, h, w, c, k, 3, 1, bool(same), pad)
    x = rounded(rng.uniform(-1, 1, n * h * w * c).astype(np.float32), dtype)
    wt = rounded((rng.uniform(-1, 1, 9 * c * k) * np.sqrt(1.0 / (9 * c))).astype(np.float32), dtype)
    dy = rounded(rng.standard_normal(n * p.out_rows * p.out_cols * k).astype(np.float32), dtype)
    return p, po, x, wt, dy


def _workspace(pass_, dtype, p, algo):
    _, rec = pd.conv2d_workspace_size(pass_, {"f32": pd.F32, "f16": pd.F16, "bf16": pd.BF16}[dtype], p, algo)
    assert rec > 0
    return torch.empty(rec, dtype=TORCH_DTYPES[dtype], device="cuda")


@pytest.mark.parametrize("algo", [pd.ALGO_WINOGRAD, pd.ALGO_WINOGRAD_LARGE])
@pytest.mark.parametrize("dtype", ["f16", "bf16", "f32"])
@pytest.mark.parametrize("shape", SHAPES)
def test_winograd_forward(orc, dtype, shape, algo):
    p, po, x, wt, _ = _case(orc, dtype, *shape)
    ws = _workspace(pd.FORWARD, dtype, p, algo)
    before = pd.launch_count()
    y = to_host(pd.conv2d(pd.FORWARD, to_dev(x, dtype), to_dev(wt, dtype), p, algorithm=algo, workspace=ws))
    assert pd.launch_count() - before >= 4, "the Winograd pipeline (3 transforms + matmul) did not run"
    assert_no_device_error()
    assert rel_err(y, orc.conv2d(orc.FORWARD, x, wt, po)) <= WINO_TOL[dtype]


@pytest.mark.parametrize("dtype", ["f16", "f32"])
@pytest.mark.parametrize("shape", SHAPES)
def test_winograd_input_backprop(orc, dtype, shape):
    p, po, _, wt, dy = _case(orc, dtype, *shape)
    ws = _workspace(pd.INPUT_BACKPROP, dtype, p, pd.ALGO_WINOGRAD)
    before = pd.launch_count()
    dx = to_host(pd.conv2d(pd.INPUT_BACKPROP, to_dev(dy, dtype), to_dev(wt, dtype), p, algorithm=pd.ALGO_WINOGRAD,
                           workspace=ws))
    assert pd.launch_count() - before >= 4
    assert_no_device_error()
    assert rel_err(dx, orc.conv2d(orc.INPUT_BACKPROP, dy, wt, po)) <= WINO_TOL[dtype]


def test_winograd_fused_epilogue(orc):
    dtype = "f16"
    p, po, x, wt, _ = _case(orc, dtype, 2, 28, 28, 64, 64, True, None)
    rng = np.random.default_rng(5)
    bias = rounded(rng.standard_normal(64).astype(np.float32), dtype)
    ref = np.maximum(orc.conv2d(orc.FORWARD, x, wt, po) + np.tile(bias, 2 * 28 * 28), 0)
    ws = _workspace(pd.FORWARD, dtype, p, pd.ALGO_WINOGRAD)
    y = to_host(pd.conv2d(pd.FORWARD, to_dev(x, dtype), to_dev(wt, dtype), p, algorithm=pd.ALGO_WINOGRAD, workspace=ws,
                          bias=to_dev(bias, dtype), activation=pd.ACT_RELU))
    assert rel_err(y, ref) <= WINO_TOL[dtype]


def test_winograd_tag_without_workspace_runs_implicit_gemm(orc):
    """No scratch: the layer still runs (one implicit-GEMM launch) and matches the oracle."""
    dtype = "f16"
    p, po, x, wt, _ = _case(orc, dtype, 2, 14, 14, 64, 64, True, None)
    before = pd.launch_count()
    y = to_host(pd.conv2d(pd.FORWARD, to_dev(x, dtype), to_dev(wt, dtype), p, algorithm=pd.ALGO_WINOGRAD_LARGE))
    assert pd.launch_count() - before == 1
    assert rel_err(y, orc.conv2d(orc.FORWARD, x, wt, po)) <= 2e-2
