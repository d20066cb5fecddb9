"""Replay of the reference's remaining known-answer tests for the convolution path, on the CPU
oracle (always) and on the GPU through the C ABI (-m gpu): the matmul suites, the hand-written
convolution tests (1x1 inputs, simple convolutions, pointer offsets), pointwise forward /
gradient, bias add, max pooling with NaNs and pooling with pointer offsets.  Fixtures come from
tests/golden/make_golden_misc.py; tolerances are the reference fixtures' own (10 ULP for matmul,
convolution, pointwise forward and bias, test/helpers/float_comparison.h; 1e-5 absolute for
pointwise gradients, test/pointwise/pointwise_fixture.h:79; float equality and NaN-ness for the
NaN pooling tests, test/pooling/max_pooling_with_nan.cc:74-82).

Pointer offsets: the reference's fixtures place the tensors `offset` elements into larger
allocations and check that the elements in front of the output are left alone; here the same
is done with slices of larger device tensors, which also exercises unaligned base pointers.
"""
import json
import os

import numpy as np
import pytest

from conftest import ulp_diff

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
MISC = json.load(open(os.path.join(ROOT, "tests", "golden", "misc_kat.json")))
_MM = np.load(os.path.join(ROOT, "tests", "golden", "matmul_kat.npz"))
FIELDS = ["channels", "features", "batch", "in_rows", "in_cols", "window_rows", "window_cols", "stride_rows", "stride_cols",
          "out_rows", "out_cols", "pad_rows", "pad_cols", "dilation_rows", "dilation_cols"]


def iota(n, max_val):
    """test/gen/iota_initialised_data.h:45-79: 1, 2, ..., max_val, 1, 2, ... (max_val < 1: 1..n)."""
    idx = np.arange(n, dtype=np.float64)
    return (idx + 1 if max_val < 1 else idx % int(max_val) + 1).astype(np.float32)


def signed_iota(n):
    """test/gen/iota_initialised_data.h:89-97: -ceil(n/2), ..., n - 1 - ceil(n/2)."""
    d = (n + 1) // 2
    return (np.arange(n) - d).astype(np.float32)


def nanarr(v):
    return np.asarray([np.nan if x is None else x for x in v], dtype=np.float32)


def matmul_cases():
    table, data, pos = _MM["table"], _MM["data"], 0
    for row in table:
        tl, tr, b, m, k, n = [int(v) for v in row[:6]]
        beta, max_val = float(row[6]), float(row[7])
        offs, ne = [int(v) for v in row[8:11]], int(row[11])
        yield tl, tr, b, m, k, n, beta, max_val, offs, data[pos:pos + ne].astype(np.float32)
        pos += ne


class OracleRunner:
    """The operators on the CPU oracle; tensors are numpy arrays."""

    def __init__(self, orc):
        self.orc = orc

    def matmul(self, tl, tr, a, b, batches, m, k, n, beta, out):
        return self.orc.matmul(bool(tl), bool(tr), a, b, batches, m, k, n, beta=beta, out=out)

    def conv(self, pass_, a, b, vals):
        p = self.orc.ConvParams(*vals, 1, 0, 0, 0)
        return self.orc.conv2d(pass_, a, b, p)

    def pointwise(self, op, x):
        return self.orc.pointwise_forward(op, x)

    def pointwise_grad(self, op, fwd, err):
        return self.orc.pointwise_grad(op, fwd, err)

    def bias(self, x, b, channels):
        return self.orc.bias_add(x, b, channels)

    def pool_params(self, shape, window, stride, same):
        n, h, w, c = shape
        return self.orc.pool_params(n, h, w, c, window, stride, same)

    def pool_forward(self, op, x, p, off=(0, 0)):
        return self.orc.pool_forward(op, x, p)

    def pool_max_grad(self, op, x, dy, p, offs=(0, 0, 0, 0)):
        y = self.orc.pool_forward(op, x, p)
        return self.orc.pool_max_grad(op, x, y, dy, p)

    def pool_avg_grad(self, dy, p, offs=(0, 0)):
        return self.orc.pool_avg_grad(dy, p)


class GpuRunner:
    """The same through the C ABI; every tensor is placed `offset` elements into a larger device
    tensor whose leading elements must stay untouched (they hold a sentinel)."""

    def __init__(self):
        import torch

        import portdnn_b200 as pd
        self.torch, self.pd = torch, pd

    def dev(self, a, off=0):
        t = self.torch.full((off + a.size,), -77.0, dtype=self.torch.float32, device="cuda")
        t[off:] = self.torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()
        return t

    def back(self, t, off=0):
        assert bool((t[:off] == -77.0).all()), "the elements in front of the output were written"
        return t[off:].cpu().numpy()

    def matmul(self, tl, tr, a, b, batches, m, k, n, beta, out, offs=(0, 0, 0)):
        ta, tb, to = self.dev(a, offs[0]), self.dev(b, offs[1]), self.dev(out, offs[2])
        self.pd.matmul(ta[offs[0]:], tb[offs[1]:], batches, m, k, n, bool(tl), bool(tr), beta=beta, out=to[offs[2]:])
        return self.back(to, offs[2])

    def conv(self, pass_, a, b, vals, offs=(0, 0, 0), n_out=0):
        pd = self.pd
        p = pd.Conv2DParams(*vals, 1, 0, 0, 0)
        ta, tb = self.dev(a, offs[0]), self.dev(b, offs[1])
        to = self.dev(np.zeros(n_out, np.float32), offs[2])
        for algo in (pd.ALGO_DIRECT, pd.ALGO_IM2COL):
            pd.conv2d(pass_, ta[offs[0]:], tb[offs[1]:], p, algorithm=algo, out=to[offs[2]:])
            res = self.back(to, offs[2])
            yield res

    def pointwise(self, op, x):
        return self.pd.pointwise(op, self.dev(x)).cpu().numpy()

    def pointwise_grad(self, op, fwd, err):
        return self.pd.pointwise_grad(op, self.dev(fwd), self.dev(err)).cpu().numpy()

    def bias(self, x, b, channels):
        return self.pd.bias_add(self.dev(x), self.dev(b), channels).cpu().numpy()

    def pool_params(self, shape, window, stride, same):
        n, h, w, c = shape
        return self.pd.pool_params(n, h, w, c, window, stride, same)

    def pool_forward(self, op, x, p, off=(0, 0)):
        tx = self.dev(x, off[0])
        ty = self.dev(np.zeros(p.batch * p.out_rows * p.out_cols * p.channels, np.float32), off[1])
        self.pd.pooling(op, 0, tx[off[0]:], p, out=ty[off[1]:])
        return self.back(ty, off[1])

    def pool_max_grad(self, op, x, dy, p, offs=(0, 0, 0, 0)):
        tx, tdy = self.dev(x, offs[0]), self.dev(dy, offs[2])
        ty = self.dev(np.zeros(dy.size, np.float32), offs[1])
        tdx = self.dev(np.zeros(x.size, np.float32), offs[3])
        self.pd.pooling(op, 0, tx[offs[0]:], p, out=ty[offs[1]:])
        self.pd.pooling_max_grad(op, tx[offs[0]:], ty[offs[1]:], tdy[offs[2]:], p, out=tdx[offs[3]:])
        return self.back(tdx, offs[3])

    def pool_avg_grad(self, dy, p, offs=(0, 0)):
        tdy = self.dev(dy, offs[0])
        tdx = self.dev(np.zeros(p.batch * p.in_rows * p.in_cols * p.channels, np.float32), offs[1])
        self.pd.pooling(self.pd.POOL_AVERAGE, 1, tdy[offs[0]:], p, out=tdx[offs[1]:])
        return self.back(tdx, offs[1])


def replay_matmul(run, on_gpu):
    n_cases = 0
    for tl, tr, b, m, k, n, beta, max_val, offs, exp in matmul_cases():
        lhs, rhs = iota(b * m * k + offs[0], max_val), iota(b * k * n + offs[1], max_val)
        out = iota(b * m * n + offs[2], max_val)
        if on_gpu:
            got = run.matmul(tl, tr, lhs[offs[0]:], rhs[offs[1]:], b, m, k, n, beta, out[offs[2]:], offs)
        else:
            got = run.matmul(tl, tr, lhs[offs[0]:], rhs[offs[1]:], b, m, k, n, beta, out[offs[2]:])
        assert ulp_diff(got, exp[offs[2]:]).max() <= 10, (tl, tr, b, m, k, n, beta)
        n_cases += 1
    assert n_cases == 434


def replay_conv(run, orc, on_gpu):
    for c in MISC["conv2d"]:
        vals = c["params"]
        po = orc.ConvParams(*vals, 1, 0, 0, 0)
        n_in, n_fil, n_out = orc.conv_sizes(c["conv_type"], po)
        a, b, exp = iota(n_in, c["max_val"]), iota(n_fil, c["max_val"]), np.asarray(c["exp"], np.float32)
        assert exp.size == n_out, c["name"]
        results = run.conv(c["conv_type"], a, b, vals, c["offsets"], n_out) if on_gpu else [run.conv(c["conv_type"], a, b, vals)]
        for got in results:
            assert ulp_diff(got, exp).max() <= 10, c["name"]


def replay_pointwise(run):
    for c in MISC["pointwise"]:
        x = signed_iota(c["signed_n"]) if c["signed_n"] else iota(c["plain_n"], c["plain_n"])
        exp = nanarr(c["exp"])
        if not c["grad"]:
            assert ulp_diff(run.pointwise(c["op"], x), exp).max() <= 10, c["name"]
        else:
            # the gradient's first tensor is the forward OUTPUT, except for Log, which takes the
            # forward input (test/pointwise/pointwise_fixture.h:113-122)
            first = x if c["op"] == 4 else run.pointwise(c["op"], x)
            assert np.abs(run.pointwise_grad(c["op"], first, x) - exp).max() <= 1e-5, c["name"]


def replay_bias(run):
    for c in MISC["bias"]:
        n, h, w, ch = c["shape"]
        x = iota(n * h * w * ch, c["max_val"])
        b = iota(ch, ch)  # test/bias/bias_fixture.h:47-48
        assert ulp_diff(run.bias(x, b, ch), np.asarray(c["exp"], np.float32)).max() <= 10, c["name"]


def replay_pooling(run, on_gpu):
    for c in MISC["pooling"]:
        p = run.pool_params(c["shape"], c["window"], c["stride"], c["same"])
        n_in = int(np.prod(c["shape"]))
        n_out = p.batch * p.out_rows * p.out_cols * p.channels
        exp = nanarr(c["exp"])
        offs = (list(c.get("offsets", [])) + [0, 0, 0, 0])[:4 if c["kind"] == "max_grad" else 2]
        if c["name"].startswith("nan."):
            x = nanarr(c["input"])
            got = run.pool_forward(c["op"], x, p) if c["kind"] == "forward" else run.pool_max_grad(c["op"], x, nanarr(c["errors"]), p)
        elif c["kind"] == "forward":
            got = run.pool_forward(c["op"], iota(n_in, c["max_val"]), p, offs if on_gpu else (0, 0))
        elif c["kind"] == "avg_grad":
            got = run.pool_avg_grad(iota(n_out, c["max_val"]), p, offs if on_gpu else (0, 0))
        else:
            got = run.pool_max_grad(c["op"], iota(n_in, c["max_val"]), iota(n_out, c["max_val"]), p, offs if on_gpu else (0, 0, 0, 0))
        assert np.array_equal(np.isnan(got), np.isnan(exp)), c["name"]
        ok = ~np.isnan(exp)
        assert ulp_diff(got[ok], exp[ok]).max(initial=0) <= 4, c["name"]  # EXPECT_FLOAT_EQ is 4 ULP


# ---- CPU: the oracle against the reference's vectors ------------------------------------------------
def test_oracle_matmul_kats(orc):
    replay_matmul(OracleRunner(orc), False)


def test_oracle_handwritten_conv_kats(orc):
    replay_conv(OracleRunner(orc), orc, False)


def test_oracle_pointwise_bias_pooling_kats(orc):
    run = OracleRunner(orc)
    replay_pointwise(run)
    replay_bias(run)
    replay_pooling(run, False)


# ---- GPU: the CUDA kernels through the C ABI --------------------------------------------------------
@pytest.mark.gpu
def test_gpu_matmul_kats():
    replay_matmul(GpuRunner(), True)


@pytest.mark.gpu
def test_gpu_handwritten_conv_kats(orc):
    replay_conv(GpuRunner(), orc, True)


@pytest.mark.gpu
def test_gpu_pointwise_bias_pooling_kats():
    run = GpuRunner()
    replay_pointwise(run)
    replay_bias(run)
    replay_pooling(run, True)
