"""The CUDA kernels against the reference's own known-answer vectors (committed subset of its
generated gtest cases), through the C ABI, in fp32.  Shapes are tiny (C, K <= 4), so conv runs
on the direct kernel; tolerances are the reference's."""
import numpy as np
import pytest
import torch

import portdnn_b200 as pd
from conftest import ulp_diff
from gpu_util import to_dev, to_host

pytestmark = pytest.mark.gpu


def _mismatches(orc, family, table, data, algorithm):
    bad = []
    for row in table:
        op, pdir, window, stride, n, h, w, c, feat, same = [int(v) for v in row[:10]]
        max_val = float(row[10])
        off, ln = int(row[11]), int(row[12])
        exp = data[off:off + ln]
        if family == "conv2d":
            p = pd.conv_params(n, h, w, c, feat, window, stride, bool(same))
            n_in, n_fil, _ = pd.api.conv_sizes(pdir, p)
            got = pd.conv2d(pdir, to_dev(orc.iota(n_in, max_val), "f32"), to_dev(orc.iota(n_fil, max_val), "f32"), p,
                            algorithm=algorithm)
            tol = 10
        elif family == "depthwise_conv2d":
            p = pd.depthwise_params(n, h, w, c, feat, window, stride, bool(same))
            po = orc.depthwise_params(n, h, w, c, feat, window, stride, bool(same))
            n_in, n_fil, _ = orc.depthwise_sizes(pdir, po)
            got = pd.depthwise_conv2d(pdir, to_dev(orc.iota(n_in, max_val), "f32"),
                                      to_dev(orc.iota(n_fil, max_val), "f32"), p)
            tol = 10
        else:
            p = pd.pool_params(n, h, w, c, window, stride, bool(same))
            x = to_dev(orc.iota(n * h * w * c, max_val), "f32")
            if pdir == 0:
                got = pd.pooling(op, 0, x, p)
                tol = 8 if op == pd.POOL_AVERAGE else 0
            elif op == pd.POOL_AVERAGE:
                got = pd.pooling(op, 1, to_dev(orc.iota(n * p.out_rows * p.out_cols * c, max_val), "f32"), p)
                tol = 8
            else:
                y = pd.pooling(pd.POOL_MAX, 0, x, p)
                got = pd.pooling_max_grad(op, x, y, to_dev(orc.iota(y.numel(), max_val), "f32"), p)
                tol = 0
        got = to_host(got)
        if got.size != exp.size or ulp_diff(got, exp).max(initial=0) > tol:
            bad.append(row[:11].tolist())
    return bad


@pytest.mark.parametrize("family", ["conv2d", "depthwise_conv2d", "pooling"])
def test_reference_vectors_on_gpu(orc, golden, family):
    table, data = golden(family)
    assert _mismatches(orc, family, table, data, pd.ALGO_DIRECT) == []


def test_reference_vectors_default_routing(orc, golden):
    # Any algorithm tag must give the same answers: shapes the tensor-core engine cannot
    # take are handed to the direct kernel.
    table, data = golden("conv2d")
    assert _mismatches(orc, "conv2d", table[::7], data, pd.ALGO_IM2COL) == []
