"""HBM-bound operators (pooling, depthwise, pointwise, bias, blend) against the CPU oracle on
seeded inputs, through the C ABI, in fp32 / fp16 / bf16, at the workload's layer shapes
(reduced batch) and at ragged shapes."""
import numpy as np
import pytest
import torch

import portdnn_b200 as pd
from conftest import rel_err
from gpu_util import TOL, rounded, to_dev, to_host

pytestmark = pytest.mark.gpu

POOL_SHAPES = [
    # n, h, w, c, window, stride, same
    (2, 112, 112, 64, 3, 2, True),    # ResNet stem pool (pad_low 0, pad_high 1)
    (2, 56, 56, 128, 2, 2, False),    # VGG stage pool
    (3, 7, 7, 2048, 7, 1, False),     # ResNet global average pool
    (2, 13, 9, 5, 3, 1, True),        # ragged: scalar path
    (1, 10, 11, 12, 5, 2, True),
    (2, 15, 13, 16, 3, 2, True),      # 3x3/2 gather kernel: odd extents, padding on both sides
    (3, 9, 12, 8, 3, 2, False),       # ... VALID
    (1, 3, 3, 32, 3, 2, True),        # ... a single window row
]


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("shape", POOL_SHAPES)
def test_max_pool_forward_and_grad_bit_exact(orc, dtype, shape):
    n, h, w, c, win, st, same = shape
    rng = np.random.default_rng(7)
    # few distinct values -> many ties, so the first-maximum rule is exercised
    x = rounded(rng.integers(-4, 5, size=n * h * w * c).astype(np.float32) * 0.5, dtype)
    p, po = pd.pool_params(n, h, w, c, win, st, same), orc.pool_params(n, h, w, c, win, st, same)
    y = pd.pooling(pd.POOL_MAX, 0, to_dev(x, dtype), p)
    y_ref = orc.pool_forward(orc.POOL_MAX, x, po)
    assert np.array_equal(to_host(y), y_ref)
    dy = rounded(rng.integers(1, 4, size=y_ref.size).astype(np.float32), dtype)
    dx = pd.pooling_max_grad(pd.POOL_MAX, to_dev(x, dtype), y, to_dev(dy, dtype), p)
    dx_ref = orc.pool_max_grad(orc.POOL_MAX, x, y_ref, dy, po)
    assert np.array_equal(to_host(dx), rounded(dx_ref, dtype))


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("shape", POOL_SHAPES)
def test_max_pool_grad_with_relu_gradient(orc, dtype, shape):
    """pdnn_pooling_max_grad_relu = max-pool gradient followed by pointwise Relu Gradient on the pooled
    tensor (src/pointwise/kernels.h:205-233), for a ReLU output with many exact zeros."""
    n, h, w, c, win, st, same = shape
    rng = np.random.default_rng(17)
    x = rounded(np.maximum(rng.integers(-4, 5, size=n * h * w * c), 0).astype(np.float32) * 0.5, dtype)
    p, po = pd.pool_params(n, h, w, c, win, st, same), orc.pool_params(n, h, w, c, win, st, same)
    y_ref = orc.pool_forward(orc.POOL_MAX, x, po)
    dy = rounded(rng.integers(1, 4, size=y_ref.size).astype(np.float32), dtype)
    dx = pd.pooling_max_grad(pd.POOL_MAX, to_dev(x, dtype), to_dev(y_ref, dtype), to_dev(dy, dtype), p, relu_input=True)
    ref = orc.pointwise_grad(0, x, orc.pool_max_grad(orc.POOL_MAX, x, y_ref, dy, po))
    assert np.array_equal(to_host(dx), rounded(ref, dtype))


def test_max_pool_random_values_and_nan(orc):
    n, h, w, c, win, st = 2, 17, 19, 8, 3, 2
    rng = np.random.default_rng(8)
    x = rng.standard_normal(n * h * w * c).astype(np.float32)
    x[::37] = np.nan
    p, po = pd.pool_params(n, h, w, c, win, st), orc.pool_params(n, h, w, c, win, st)
    for op in (pd.POOL_MAX, pd.POOL_MAX_WITH_NAN):
        y = to_host(pd.pooling(op, 0, to_dev(x, "f32"), p))
        y_ref = orc.pool_forward(op, x, po)
        assert np.array_equal(np.isnan(y), np.isnan(y_ref))
        assert np.array_equal(y[~np.isnan(y)], y_ref[~np.isnan(y_ref)])
        dy = rng.standard_normal(y_ref.size).astype(np.float32)
        dx = to_host(pd.pooling_max_grad(op, to_dev(x, "f32"), to_dev(y_ref, "f32"), to_dev(dy, "f32"), p))
        dx_ref = orc.pool_max_grad(op, x, y_ref, dy, po)
        np.testing.assert_allclose(dx, dx_ref, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("stride", [1, 2])
def test_max_pool_grad_3x3_ties_nan_and_signed_zeros(orc, dtype, stride):
    """The 3x3 winner map (strip kernel) with ties, NaNs and signed zeros, both operators."""
    n, h, w, c, win = 2, 19, 21, 16, 3
    rng = np.random.default_rng(18)
    x = rounded(rng.integers(-2, 3, size=n * h * w * c).astype(np.float32) * 0.5, dtype)
    x[::41] = np.nan
    x[7::29] = -0.0
    p, po = pd.pool_params(n, h, w, c, win, stride, True), orc.pool_params(n, h, w, c, win, stride, True)
    for op in (pd.POOL_MAX, pd.POOL_MAX_WITH_NAN):
        y = to_host(pd.pooling(op, 0, to_dev(x, dtype), p))
        y_ref = orc.pool_forward(op, x, po)
        assert np.array_equal(np.isnan(y), np.isnan(y_ref))
        assert np.array_equal(y[~np.isnan(y)], y_ref[~np.isnan(y_ref)])
        dy = rounded(rng.integers(1, 4, size=y_ref.size).astype(np.float32), dtype)
        dx = to_host(pd.pooling_max_grad(op, to_dev(x, dtype), to_dev(y_ref, dtype), to_dev(dy, dtype), p))
        dx_ref = orc.pool_max_grad(op, x, y_ref, dy, po)
        assert np.array_equal(dx, rounded(dx_ref, dtype)), (op, np.abs(dx - dx_ref).max())


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("shape", POOL_SHAPES)
def test_avg_pool_forward_and_grad(orc, dtype, shape):
    n, h, w, c, win, st, same = shape
    rng = np.random.default_rng(9)
    x = rounded(rng.standard_normal(n * h * w * c).astype(np.float32), dtype)
    p, po = pd.pool_params(n, h, w, c, win, st, same), orc.pool_params(n, h, w, c, win, st, same)
    y = to_host(pd.pooling(pd.POOL_AVERAGE, 0, to_dev(x, dtype), p))
    y_ref = orc.pool_forward(orc.POOL_AVERAGE, x, po)
    if dtype == "f32":
        assert np.array_equal(y, y_ref)  # same summation order and one division
    else:
        assert rel_err(y, y_ref) <= TOL[dtype]
    dy = rounded(rng.standard_normal(y_ref.size).astype(np.float32), dtype)
    dx = to_host(pd.pooling(pd.POOL_AVERAGE, 1, to_dev(dy, dtype), p))
    dx_ref = orc.pool_avg_grad(dy, po)
    assert rel_err(dx, dx_ref) <= (1e-6 if dtype == "f32" else TOL[dtype])


DW_SHAPES = [
    # n, h, w, c, mult, window, stride  (MobileNet-v2 layers at batch 2 + ragged)
    (2, 112, 112, 32, 1, 3, 1), (2, 112, 112, 96, 1, 3, 2), (2, 56, 56, 144, 1, 3, 2), (2, 14, 14, 576, 1, 3, 1),
    (2, 7, 7, 960, 1, 3, 1), (2, 9, 11, 6, 2, 3, 2), (1, 12, 12, 5, 1, 5, 1), (3, 8, 8, 8, 4, 3, 1),
    (2, 15, 13, 16, 1, 3, 2), (3, 28, 30, 8, 1, 3, 2), (1, 5, 4, 32, 1, 3, 2),   # stride-2 gather kernel, odd extents
]


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("shape", DW_SHAPES)
def test_depthwise_three_passes(orc, dtype, shape):
    n, h, w, c, m, win, st = shape
    rng = np.random.default_rng(11)
    p, po = pd.depthwise_params(n, h, w, c, m, win, st), orc.depthwise_params(n, h, w, c, m, win, st)
    x = rounded(rng.standard_normal(n * h * w * c).astype(np.float32), dtype)
    fil = rounded(rng.standard_normal(win * win * c * m).astype(np.float32) * np.sqrt(2.0 / (win * win)), dtype)
    dy = rounded(rng.standard_normal(n * p.out_rows * p.out_cols * c * m).astype(np.float32), dtype)
    tol = 1e-5 if dtype == "f32" else TOL[dtype]
    y = to_host(pd.depthwise_conv2d(pd.FORWARD, to_dev(x, dtype), to_dev(fil, dtype), p))
    assert rel_err(y, orc.depthwise_conv2d(orc.FORWARD, x, fil, po)) <= tol
    dx = to_host(pd.depthwise_conv2d(pd.INPUT_BACKPROP, to_dev(dy, dtype), to_dev(fil, dtype), p))
    assert rel_err(dx, orc.depthwise_conv2d(orc.INPUT_BACKPROP, dy, fil, po)) <= tol
    dw = to_host(pd.depthwise_conv2d(pd.FILTER_BACKPROP, to_dev(x, dtype), to_dev(dy, dtype), p))
    assert rel_err(dw, orc.depthwise_conv2d(orc.FILTER_BACKPROP, x, dy, po)) <= tol


def test_depthwise_filter_backprop_with_caller_workspace(orc):
    n, h, w, c, m, win, st = 4, 28, 28, 192, 1, 3, 1
    rng = np.random.default_rng(12)
    p, po = pd.depthwise_params(n, h, w, c, m, win, st), orc.depthwise_params(n, h, w, c, m, win, st)
    x = rng.standard_normal(n * h * w * c).astype(np.float32)
    dy = rng.standard_normal(n * p.out_rows * p.out_cols * c).astype(np.float32)
    need = pd.api.depthwise_workspace_bytes(pd.FILTER_BACKPROP, pd.F32, p)
    assert need > 0
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    dw = to_host(pd.depthwise_conv2d(pd.FILTER_BACKPROP, to_dev(x, "f32"), to_dev(dy, "f32"), p, workspace=ws))
    assert rel_err(dw, orc.depthwise_conv2d(orc.FILTER_BACKPROP, x, dy, po)) <= 1e-5


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("n", [1, 8, 9, 10, 4096, 100003])
def test_pointwise_exp_log_floor_sqrt(orc, dtype, n):
    """The reference's other pointwise operators (test/pointwise/{log,sqrt,floor}_*.cc shapes plus
    larger ones), forward and gradient, against the oracle; Floor is bit-exact and has no gradient."""
    rng = np.random.default_rng(17)
    pos = rounded(rng.uniform(0.25, 4.0, n).astype(np.float32), dtype)   # log / sqrt want positive input
    x = rounded(rng.uniform(-3.0, 3.0, n).astype(np.float32), dtype)
    err = rounded(rng.standard_normal(n).astype(np.float32), dtype)
    pd_, xd, ed = to_dev(pos, dtype), to_dev(x, dtype), to_dev(err, dtype)
    tol = 1e-6 if dtype == "f32" else TOL[dtype]
    assert np.array_equal(to_host(pd.pointwise(pd.PW_FLOOR, xd)), orc.pointwise_forward(orc.FLOOR, x))
    assert rel_err(to_host(pd.pointwise(pd.PW_EXP, xd)), orc.pointwise_forward(orc.EXP, x)) <= tol
    assert rel_err(to_host(pd.pointwise(pd.PW_LOG, pd_)), orc.pointwise_forward(orc.LOG, pos)) <= tol
    assert rel_err(to_host(pd.pointwise(pd.PW_SQRT, pd_)), orc.pointwise_forward(orc.SQRT, pos)) <= tol
    for op_gpu, op_orc, v, vd in ((pd.PW_EXP, orc.EXP, x, xd), (pd.PW_LOG, orc.LOG, pos, pd_),
                                  (pd.PW_SQRT, orc.SQRT, pos, pd_)):
        assert rel_err(to_host(pd.pointwise_grad(op_gpu, vd, ed)), orc.pointwise_grad(op_orc, v, err)) <= tol
    with pytest.raises(pd.PortDNNError):
        pd.pointwise_grad(pd.PW_FLOOR, xd, ed)
    with pytest.raises(pd.PortDNNError):
        pd.pointwise(7, xd)


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("n", [1, 7, 4096, 100003, 1 << 20])
def test_pointwise_bias_blend(orc, dtype, n):
    rng = np.random.default_rng(13)
    x = rounded(rng.standard_normal(n).astype(np.float32) * 2, dtype)
    err = rounded(rng.standard_normal(n).astype(np.float32), dtype)
    xd, ed = to_dev(x, dtype), to_dev(err, dtype)
    tol = 1e-6 if dtype == "f32" else TOL[dtype]
    assert np.array_equal(to_host(pd.pointwise(pd.ACT_RELU, xd)), orc.pointwise_forward(orc.RELU, x))
    assert rel_err(to_host(pd.pointwise(pd.ACT_TANH, xd)), orc.pointwise_forward(orc.TANH, x)) <= tol
    assert np.array_equal(to_host(pd.pointwise_grad(pd.ACT_RELU, xd, ed)), orc.pointwise_grad(orc.RELU, x, err))
    assert rel_err(to_host(pd.pointwise_grad(pd.ACT_TANH, xd, ed)), orc.pointwise_grad(orc.TANH, x, err)) <= tol
    for ch in (1, 7, 64):
        if n % ch:
            continue
        b = rounded(rng.standard_normal(ch).astype(np.float32), dtype)
        got = to_host(pd.bias_add(xd, to_dev(b, dtype), ch))
        assert np.array_equal(got, rounded(orc.bias_add(x, b, ch), dtype))
        got = to_host(pd.bias_add(xd, to_dev(b, dtype), ch, activation=pd.ACT_RELU))
        assert np.array_equal(got, np.maximum(rounded(orc.bias_add(x, b, ch), dtype), 0))
    got = to_host(pd.scale_blend(xd, 0.5, ed, 2.0))
    assert rel_err(got, 0.5 * x + 2.0 * err) <= tol
    assert np.array_equal(to_host(pd.scale_blend(xd, 2.0)), rounded(2.0 * x, dtype))
