"""Softmax and batchnorm on the GPU, through the C ABI: the reference's 324 known-answer cases
(fp32, the fixtures' tolerances) and seeded random tensors against the oracle in fp32 / fp16 / bf16."""
import numpy as np
import pytest
import torch

import norm_cases
import portdnn_b200 as pd
from conftest import rel_err
from gpu_util import TOL, rounded, to_dev, to_host

pytestmark = pytest.mark.gpu


class _Gpu:
    """The four operators with the oracle's calling convention, on fp32 device tensors."""

    @staticmethod
    def _dims(n, c):
        return 1, 1, n // c, c

    def softmax_forward(self, x, c):
        b, h, w, _ = self._dims(x.size, c)
        return to_host(pd.softmax(to_dev(x, "f32"), b, h, w, c))

    def softmax_grad(self, y, dy, c):
        b, h, w, _ = self._dims(y.size, c)
        return to_host(pd.softmax(to_dev(y, "f32"), b, h, w, c, gradient=to_dev(dy, "f32")))

    def batchnorm_forward(self, x, beta, gamma, mean, var, c, eps, momentum, training):
        b, h, w, _ = self._dims(x.size, c)
        p = pd.batchnorm_params(b, h, w, c, training, eps, momentum)
        out, rm, rv = pd.batchnorm_forward(*(to_dev(t, "f32") for t in (x, beta, gamma, mean, var)), p)
        return to_host(out), (to_host(rm) if rm is not None else None), (to_host(rv) if rv is not None else None)

    def batchnorm_grad(self, x, dy, gamma, pm, pv, c, eps, training):
        b, h, w, _ = self._dims(x.size, c)
        p = pd.batchnorm_params(b, h, w, c, training, eps, 0.9)
        dx, bg, gg = pd.batchnorm_gradient(to_dev(x, "f32"), to_dev(dy, "f32"), to_dev(gamma, "f32"), p,
                                           pop_mean=to_dev(pm, "f32"), pop_variance=to_dev(pv, "f32"))
        return to_host(dx), to_host(bg), to_host(gg)


def test_reference_known_answers():
    failures = []
    gpu = _Gpu()
    for case in norm_cases.load_cases():
        for what, ok, err in norm_cases.run_case(case, gpu):
            if not ok:
                failures.append((case["op"], case["name"], what, err))
    assert not failures, failures[:10]


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("shape", [(4, 1, 1, 1000), (2, 7, 5, 33), (3, 4, 4, 8)])
def test_softmax_against_oracle(orc, dtype, shape):
    n, h, w, c = shape
    rng = np.random.default_rng(3)
    x = rounded(rng.standard_normal(n * h * w * c).astype(np.float32) * 3, dtype)
    y = to_host(pd.softmax(to_dev(x, dtype), n, h, w, c))
    ref = orc.softmax_forward(x, c)
    assert rel_err(y, ref) <= TOL[dtype]
    dy = rounded(rng.standard_normal(x.size).astype(np.float32), dtype)
    yr = rounded(ref, dtype)
    dx = to_host(pd.softmax(to_dev(yr, dtype), n, h, w, c, gradient=to_dev(dy, dtype)))
    assert rel_err(dx, orc.softmax_grad(yr, dy, c)) <= TOL[dtype]


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("training", [False, True])
@pytest.mark.parametrize("shape", [(8, 14, 14, 256), (3, 9, 7, 24), (2, 5, 5, 3)])
def test_batchnorm_against_oracle(orc, dtype, training, shape):
    n, h, w, c = shape
    rng = np.random.default_rng(4)
    x = rounded(rng.standard_normal(n * h * w * c).astype(np.float32) * 2 + 0.5, dtype)
    dy = rounded(rng.standard_normal(x.size).astype(np.float32), dtype)
    beta, gamma, mean = (rounded(rng.standard_normal(c).astype(np.float32), dtype) for _ in range(3))
    var = rounded(rng.uniform(0.5, 2.0, c).astype(np.float32), dtype)
    p = pd.batchnorm_params(n, h, w, c, training, 1e-3, 0.9)
    out, rm, rv = pd.batchnorm_forward(*(to_dev(t, dtype) for t in (x, beta, gamma, mean, var)), p)
    ref, rrm, rrv = orc.batchnorm_forward(x, beta, gamma, mean, var, c, 1e-3, 0.9, training)
    assert rel_err(to_host(out), ref) <= TOL[dtype]
    if training:
        assert rel_err(to_host(rm), rrm) <= TOL[dtype]
        assert rel_err(to_host(rv), rrv) <= TOL[dtype]
    dx, bg, gg = pd.batchnorm_gradient(to_dev(x, dtype), to_dev(dy, dtype), to_dev(gamma, dtype), p,
                                       pop_mean=to_dev(mean, dtype), pop_variance=to_dev(var, dtype))
    rdx, rbg, rgg = orc.batchnorm_grad(x, dy, gamma, mean, var, c, 1e-3, training)
    assert rel_err(to_host(dx), rdx) <= TOL[dtype]
    assert rel_err(to_host(bg), rbg) <= TOL[dtype]
    assert rel_err(to_host(gg), rgg) <= TOL[dtype]


def test_validation_errors():
    x = torch.zeros(0, device="cuda")
    with pytest.raises(pd.PortDNNError) as e:
        pd.softmax(x, 1, 0, 1, 8)  # rows must be positive (include/portdnn/softmax/launch.h:40-50)
    assert e.value.status == pd.StatusCode.InvalidParameter
