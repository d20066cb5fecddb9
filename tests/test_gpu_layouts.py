"""Transposition and the NCHW / FCHW forms of convolution and pooling, through the C ABI.

The reference runs its convolution and pooling known-answer tests a second time with
layout::NCHW: the fixture transposes the NHWC inputs on the host, runs the operator, transposes
the result back and compares with the same expected values (test/conv2d/convolution_fixture.h:94-144).
The tests here do that with a slice of those known-answer cases, and compare larger seeded
shapes with the NHWC path.  Transposition itself is checked against numpy, bit for bit.
"""
import numpy as np
import pytest
import torch

import portdnn_b200 as pd
from conftest import rel_err, ulp_diff
from gpu_util import TOL, rounded, to_dev, to_host

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dims,perm", [
    ((3, 5, 7, 4), (0, 3, 1, 2)), ((3, 4, 5, 7), (0, 2, 3, 1)), ((64, 56, 56, 24), (0, 3, 1, 2)),
    ((3, 3, 16, 40), (3, 2, 0, 1)), ((40, 16, 3, 3), (2, 3, 1, 0)), ((33, 65), (1, 0)), ((7, 33, 65), (0, 2, 1)),
    ((2, 3, 4, 5), (3, 1, 0, 2)), ((2, 3, 4, 5, 6), (4, 0, 2, 1, 3)), ((5, 1, 7), (2, 1, 0)), ((6, 5), (0, 1)),
    ((2, 3, 2, 3, 2, 3), (5, 4, 3, 2, 1, 0))])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.int8, torch.float64])
def test_transpose_against_numpy(dims, perm, dtype):
    n = int(np.prod(dims))
    x = torch.arange(n, device="cuda").remainder(251).to(dtype)
    got = pd.transpose(x, dims, perm).cpu().numpy()
    want = np.ascontiguousarray(x.cpu().numpy().reshape(dims).transpose(perm)).ravel()
    assert np.array_equal(got, want)


def test_transpose_rejects_bad_permutations():
    x = torch.zeros(24, device="cuda")
    for dims, perm in (((2, 3, 4), (0, 1, 1)), ((2, 3, 4), (0, 1, 3)), ((2, 3, 4, 1, 1, 1, 1), (0, 1, 2, 3, 4, 5, 6))):
        with pytest.raises(pd.PortDNNError) as e:
            pd.transpose(x, dims, perm)
        assert e.value.status == pd.StatusCode.InvalidParameter


def _nchw(a, n, h, w, c):
    return np.ascontiguousarray(a.reshape(n, h, w, c).transpose(0, 3, 1, 2)).ravel()


def _nhwc(a, n, c, h, w):
    return np.ascontiguousarray(a.reshape(n, c, h, w).transpose(0, 2, 3, 1)).ravel()


def _fchw(a, r, s, c, k):
    return np.ascontiguousarray(a.reshape(r, s, c, k).transpose(3, 2, 0, 1)).ravel()


def _run_nchw(pass_, a, b, p, dtype):
    """The pass on NCHW / FCHW tensors built from NHWC / HWCF host arrays; the result comes back NHWC / HWCF."""
    n, c, k = p.batch, p.channels, p.features
    q = pd.Conv2DParams.from_buffer_copy(p)
    q.input_format, q.filter_format = 1, 1
    x_like = lambda t: _nchw(t, n, p.in_rows, p.in_cols, c)
    y_like = lambda t: _nchw(t, n, p.out_rows, p.out_cols, k)
    w_like = lambda t: _fchw(t, p.window_rows, p.window_cols, c, k)
    if pass_ == pd.FORWARD:
        out = pd.conv2d(pass_, to_dev(x_like(a), dtype), to_dev(w_like(b), dtype), q, algorithm=pd.ALGO_DIRECT)
        return _nhwc(to_host(out), n, k, p.out_rows, p.out_cols)
    if pass_ == pd.INPUT_BACKPROP:
        out = pd.conv2d(pass_, to_dev(y_like(a), dtype), to_dev(w_like(b), dtype), q, algorithm=pd.ALGO_DIRECT)
        return _nhwc(to_host(out), n, c, p.in_rows, p.in_cols)
    out = pd.conv2d(pass_, to_dev(x_like(a), dtype), to_dev(y_like(b), dtype), q, algorithm=pd.ALGO_DIRECT)
    return np.ascontiguousarray(to_host(out).reshape(k, c, p.window_rows, p.window_cols).transpose(2, 3, 1, 0)).ravel()


def test_nchw_convolution_replays_reference_vectors(golden, orc):
    table, data = golden("conv2d")
    checked = 0
    for row in table[::40]:
        _, pass_, window, stride, n, h, w, c, feat, same = [int(v) for v in row[:10]]
        max_val, off, ne = float(row[10]), int(row[11]), int(row[12])
        p = pd.conv_params(n, h, w, c, feat, window, stride, bool(same))
        po = orc.conv_params(n, h, w, c, feat, window, stride, bool(same))
        n_in, n_fil, _ = orc.conv_sizes(pass_, po)
        a, b = orc.iota(n_in, max_val), orc.iota(n_fil, max_val)
        got = _run_nchw(pass_, a, b, p, "f32")
        assert ulp_diff(got, data[off:off + ne].astype(np.float32)).max() <= 10, tuple(row[:9])
        checked += 1
    assert checked >= 20


@pytest.mark.parametrize("dtype", ["f16", "f32"])
@pytest.mark.parametrize("shape", [(2, 28, 28, 64, 128, 3, 1), (3, 14, 14, 256, 64, 1, 1), (2, 15, 13, 24, 40, 3, 2)])
def test_nchw_convolution_matches_the_oracle(orc, dtype, shape):
    n, h, w, c, k, win, st = shape
    rng = np.random.default_rng(7)
    p, po = pd.conv_params(n, h, w, c, k, win, st), orc.conv_params(n, h, w, c, k, win, st)
    x = rounded(rng.uniform(-1, 1, n * h * w * c).astype(np.float32), dtype)
    wt = rounded((rng.uniform(-1, 1, win * win * c * k) / np.sqrt(win * win * c)).astype(np.float32), dtype)
    dy = rounded(rng.standard_normal(n * p.out_rows * p.out_cols * k).astype(np.float32), dtype)
    for pass_, a, b in ((pd.FORWARD, x, wt), (pd.INPUT_BACKPROP, dy, wt), (pd.FILTER_BACKPROP, x, dy)):
        assert rel_err(_run_nchw(pass_, a, b, p, dtype), orc.conv2d(pass_, a, b, po)) <= TOL[dtype], pass_


def test_nchw_pooling_matches_nhwc(orc):
    n, h, w, c = 3, 13, 17, 24
    rng = np.random.default_rng(3)
    x = rng.standard_normal(n * h * w * c).astype(np.float32)
    for op, win, st in ((pd.POOL_MAX, 3, 2), (pd.POOL_AVERAGE, 2, 2), (pd.POOL_MAX_WITH_NAN, 5, 1)):
        p, po = pd.pool_params(n, h, w, c, win, st), orc.pool_params(n, h, w, c, win, st)
        q = pd.PoolingParams.from_buffer_copy(p)
        q.input_format = 1
        y = pd.pooling(op, 0, to_dev(_nchw(x, n, h, w, c), "f32"), q)
        want = orc.pool_forward(op, x, po)
        assert np.array_equal(_nhwc(to_host(y), n, c, p.out_rows, p.out_cols), want)
        if op != pd.POOL_AVERAGE:
            dy = rng.standard_normal(want.size).astype(np.float32)
            dx = pd.pooling_max_grad(op, to_dev(_nchw(x, n, h, w, c), "f32"), y,
                                     to_dev(_nchw(dy, n, p.out_rows, p.out_cols, c), "f32"), q)
            assert np.array_equal(_nhwc(to_host(dx), n, c, h, w), orc.pool_max_grad(op, x, want, dy, po))
