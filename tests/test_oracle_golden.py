"""The CPU oracle against the reference's known-answer vectors (committed subset) and
against an independent implementation (torch on CPU, float64)."""
import numpy as np
import pytest

from conftest import ulp_diff


def _replay(orc, family, table, data):
    bad = []
    for row in table:
        op, pd, window, stride, n, h, w, c, feat, same = [int(v) for v in row[:10]]
        max_val = float(row[10])
        off, ln = int(row[11]), int(row[12])
        exp = data[off:off + ln]
        if family == "conv2d":
            p = orc.conv_params(n, h, w, c, feat, window, stride, bool(same))
            n_in, n_fil, _ = orc.conv_sizes(pd, p)
            got = orc.conv2d(pd, orc.iota(n_in, max_val), orc.iota(n_fil, max_val), p)
            tol = 10  # test/conv2d/convolution_fixture.h:152
        elif family == "depthwise_conv2d":
            p = orc.depthwise_params(n, h, w, c, feat, window, stride, bool(same))
            n_in, n_fil, _ = orc.depthwise_sizes(pd, p)
            got = orc.depthwise_conv2d(pd, orc.iota(n_in, max_val), orc.iota(n_fil, max_val), p)
            tol = 10
        else:
            p = orc.pool_params(n, h, w, c, window, stride, bool(same))
            x = orc.iota(n * h * w * c, max_val)
            if pd == 0:
                got = orc.pool_forward(op, x, p)
                tol = 8 if op == orc.POOL_AVERAGE else 0  # test/pooling/pooling_fixture.h:107-134
            elif op == orc.POOL_AVERAGE:
                got = orc.pool_avg_grad(orc.iota(n * p.out_rows * p.out_cols * c, max_val), p)
                tol = 8
            else:
                y = orc.pool_forward(orc.POOL_MAX, x, p)  # test/pooling/pooling_fixture.h:172-176
                got = orc.pool_max_grad(op, x, y, orc.iota(y.size, max_val), p)
                tol = 0  # EXPECT_EQ, test/pooling/pooling_fixture.h:212-215
        if got.size != exp.size or ulp_diff(got, exp).max(initial=0) > tol:
            bad.append(row[:11].tolist())
    return bad


@pytest.mark.parametrize("family", ["conv2d", "depthwise_conv2d", "pooling"])
def test_oracle_matches_reference_vectors(orc, golden, family):
    table, data = golden(family)
    assert table.shape[0] > 500
    assert _replay(orc, family, table, data) == []


def test_padding_matches_reference_table(orc):
    # SAME / VALID cases worked out from include/portdnn/helpers/padding.h:46-66
    assert orc.padding(56, 3, 1, True) == (56, 1)
    assert orc.padding(56, 3, 2, True) == (28, 0)     # need 1 -> low 0, high 1
    assert orc.padding(112, 3, 2, True) == (56, 0)
    assert orc.padding(224, 7, 2, True) == (112, 2)   # need 5 -> low 2, high 3
    assert orc.padding(224, 7, 2, False) == (109, 0)
    assert orc.padding(230, 7, 2, False) == (112, 0)  # the reference's ResNet stem entry
    assert orc.padding(4, 1, 2, True) == (2, 0)       # negative need truncates to 0
    assert orc.padding(2, 3, 1, False) == (0, 0)


def _torch_conv(x, w, p, dtype):
    import torch
    import torch.nn.functional as F
    xt = torch.from_numpy(x.reshape(p.batch, p.in_rows, p.in_cols, p.channels)).to(dtype).permute(0, 3, 1, 2)
    wt = torch.from_numpy(w.reshape(p.window_rows, p.window_cols, p.channels, p.features)).to(dtype).permute(3, 2, 0, 1)
    need_r = max((p.out_rows - 1) * p.stride_rows + p.window_rows - p.in_rows, 0)
    need_c = max((p.out_cols - 1) * p.stride_cols + p.window_cols - p.in_cols, 0)
    xt = F.pad(xt, (p.pad_cols, need_c - p.pad_cols, p.pad_rows, need_r - p.pad_rows))
    y = F.conv2d(xt, wt, stride=(p.stride_rows, p.stride_cols))
    return y[:, :, :p.out_rows, :p.out_cols]


@pytest.mark.parametrize("shape", [(2, 9, 11, 5, 7, 3, 1, True), (2, 12, 10, 4, 6, 3, 2, True),
                                   (1, 14, 14, 3, 8, 7, 2, True), (3, 8, 8, 6, 5, 1, 2, False),
                                   (2, 10, 9, 4, 4, 5, 1, False)])
def test_oracle_conv_against_torch_float64(orc, shape):
    import torch
    n, h, w, c, k, win, st, same = shape
    rng = np.random.default_rng(1)
    p = orc.conv_params(n, h, w, c, k, win, st, same)
    x = rng.standard_normal(n * h * w * c).astype(np.float32)
    wt = rng.standard_normal(win * win * c * k).astype(np.float32)
    y = orc.conv2d(orc.FORWARD, x, wt, p)
    ref = _torch_conv(x, wt, p, torch.float64).permute(0, 2, 3, 1).contiguous().numpy().ravel()
    np.testing.assert_allclose(y, ref, rtol=1e-5, atol=1e-5)
    # the two backprop passes against autograd
    xt = torch.from_numpy(x.reshape(n, h, w, c)).double().requires_grad_(True)
    wtt = torch.from_numpy(wt.reshape(win, win, c, k)).double().requires_grad_(True)
    import torch.nn.functional as F
    need_r = max((p.out_rows - 1) * st + win - h, 0)
    need_c = max((p.out_cols - 1) * st + win - w, 0)
    xp = F.pad(xt.permute(0, 3, 1, 2), (p.pad_cols, need_c - p.pad_cols, p.pad_rows, need_r - p.pad_rows))
    yt = F.conv2d(xp, wtt.permute(3, 2, 0, 1), stride=st)[:, :, :p.out_rows, :p.out_cols]
    dy = rng.standard_normal(yt.shape).astype(np.float32)
    yt.backward(torch.from_numpy(dy).double())
    dy_nhwc = np.ascontiguousarray(dy.transpose(0, 2, 3, 1)).ravel()
    dx = orc.conv2d(orc.INPUT_BACKPROP, dy_nhwc, wt, p)
    dw = orc.conv2d(orc.FILTER_BACKPROP, x, dy_nhwc, p)
    np.testing.assert_allclose(dx, xt.grad.numpy().ravel(), rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(dw, wtt.grad.numpy().ravel(), rtol=1e-5, atol=1e-4)


def test_oracle_pool_nan_rules(orc):
    # src/pooling/operators_impl.h:27-65: Max never takes a NaN, MaxWithNan keeps it.
    p = orc.pool_params(1, 2, 2, 1, 2, 2, False)
    x = np.array([1.0, np.nan, 3.0, 2.0], dtype=np.float32)
    assert orc.pool_forward(orc.POOL_MAX, x, p)[0] == 3.0
    assert np.isnan(orc.pool_forward(orc.POOL_MAX_WITH_NAN, x, p)[0])


def test_oracle_maxgrad_first_maximum_wins(orc):
    # ties: the first maximum in row-major window order receives the gradient
    # (src/pooling/kernels.h:197-240)
    p = orc.pool_params(1, 2, 2, 1, 2, 2, False)
    x = np.array([5.0, 5.0, 5.0, 1.0], dtype=np.float32)
    y = orc.pool_forward(orc.POOL_MAX, x, p)
    dx = orc.pool_max_grad(orc.POOL_MAX, x, y, np.array([7.0], dtype=np.float32), p)
    assert dx.tolist() == [7.0, 0.0, 0.0, 0.0]


def test_oracle_matmul_and_pointwise(orc):
    rng = np.random.default_rng(3)
    a = rng.standard_normal((2, 5, 7)).astype(np.float32)
    b = rng.standard_normal((2, 7, 3)).astype(np.float32)
    ref = np.einsum("bmk,bkn->bmn", a.astype(np.float64), b.astype(np.float64))
    got = orc.matmul(False, False, a, b, 2, 5, 7, 3)
    np.testing.assert_allclose(got, ref.ravel(), rtol=1e-6)
    got_t = orc.matmul(True, True, np.ascontiguousarray(a.transpose(0, 2, 1)), np.ascontiguousarray(b.transpose(0, 2, 1)),
                       2, 5, 7, 3, beta=2.0, out=np.ones(30, dtype=np.float32))
    np.testing.assert_allclose(got_t, ref.ravel() + 2.0, rtol=1e-5)
    x = np.array([-1.0, 0.0, 2.0], dtype=np.float32)
    assert orc.pointwise_forward(orc.RELU, x).tolist() == [0.0, 0.0, 2.0]
    assert orc.pointwise_grad(orc.RELU, x, np.array([3.0, 3.0, 3.0], np.float32)).tolist() == [0.0, 0.0, 3.0]
    np.testing.assert_allclose(orc.pointwise_grad(orc.TANH, x, np.ones(3, np.float32)), 1 - x * x)
    # test/pointwise/{log,sqrt}_grad.cc feed the ramp 1..n as both tensors: log' = (1/v)*v = 1 and
    # sqrt' = (0.5/v)*v = 0.5 on every shape; floor_forward.cc, log_forward.cc, sqrt_forward.cc
    for n in (1, 8, 9, 10):
        r = np.arange(1, n + 1, dtype=np.float32)
        np.testing.assert_allclose(orc.pointwise_grad(orc.LOG, r, r), np.ones(n), rtol=1e-6)
        np.testing.assert_allclose(orc.pointwise_grad(orc.SQRT, r, r), np.full(n, 0.5), rtol=1e-6)
        np.testing.assert_allclose(orc.pointwise_forward(orc.LOG, r), np.log(r.astype(np.float64)), rtol=1e-6, atol=1e-7)
        np.testing.assert_allclose(orc.pointwise_forward(orc.SQRT, r), np.sqrt(r.astype(np.float64)), rtol=1e-6)
        assert orc.pointwise_forward(orc.FLOOR, r - 0.5).tolist() == np.floor(r - 0.5).tolist()
    np.testing.assert_allclose(orc.pointwise_grad(orc.EXP, x, np.ones(3, np.float32)), np.exp(x.astype(np.float64)) + 1, rtol=1e-6)
