"""Shared driver for the softmax / batchnorm known-answer cases of tests/golden/norm_kat.npz: builds
every case's inputs (ramps, test/gen/iota_initialised_data.h:45-79) and checks an implementation's
outputs with the reference fixtures' tolerances (test/softmax/softmax_fixture.h:117,
test/batchnorm/batchnorm_fixture.h:100-118: 10 ULP, or an absolute epsilon where one is given)."""
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def load_cases():
    return list(np.load(os.path.join(HERE, "golden", "norm_kat.npz"), allow_pickle=True)["cases"])


def iota(size, max_val):
    a = np.arange(size, dtype=np.float64)
    if max_val >= 1:
        a = a % int(max_val)
    return (a + 1).astype(np.float32)


def close(got, exp, ulps=10, eps=0.0):
    got = np.asarray(got, dtype=np.float32).ravel()
    exp = np.asarray(exp, dtype=np.float32).ravel()
    assert got.shape == exp.shape, (got.shape, exp.shape)
    gi = got.view(np.int32).astype(np.int64)
    ei = exp.view(np.int32).astype(np.int64)
    gi = np.where(gi < 0, -(gi & 0x7FFFFFFF), gi)
    ei = np.where(ei < 0, -(ei & 0x7FFFFFFF), ei)
    ok = (np.abs(gi - ei) <= ulps) | (np.abs(got.astype(np.float64) - exp.astype(np.float64)) <= eps)
    return bool(ok.all()), float(np.max(np.abs(got.astype(np.float64) - exp.astype(np.float64)))) if got.size else 0.0


def run_case(case, impl):
    """impl: object with softmax_forward(x, C), softmax_grad(y, dy, C), batchnorm_forward(x, beta, gamma,
    mean, var, C, eps, momentum, training) -> (out, rm, rv), batchnorm_grad(x, dy, gamma, pm, pv, C, eps,
    training) -> (dx, dbeta, dgamma).  Returns a list of (what, ok, max abs error)."""
    n, h, w, c = case["shape"]
    size = n * h * w * c
    op = case["op"]
    res = []
    if op.startswith("softmax"):
        x = iota(size, case["max_input_val"])
        y = impl.softmax_forward(x, c)
        if op == "softmax_forward":
            res.append(("out",) + close(y, case["exp_out"], 10, 1e-7))
        else:
            dx = impl.softmax_grad(y, x, c)
            res.append(("grad",) + close(dx, case["exp_out"], 10, 2e-4))
        return res
    training = bool(case["is_training"])
    x = iota(size, case["max_input_val"])
    gamma = iota(c, case["max_gamma_val"])
    if op.startswith("batchnorm_forward"):
        beta = iota(c, case["max_beta_val"])
        mean = iota(c, case["max_input_mean_val"])
        var = iota(c, case["max_input_var_val"])
        out, rm, rv = impl.batchnorm_forward(x, beta, gamma, mean, var, c, case["epsilon"], case["momentum"], training)
        res.append(("out",) + close(out, case["exp_out"], 10, 2e-5))
        if training:
            res.append(("running_mean",) + close(rm, case["exp_running_mean"], 10, 1e-5))
            res.append(("running_var",) + close(rv, case["exp_running_var"], 10, 1e-5))
        return res
    dy = iota(size, case["max_gradient_val"])
    pm = iota(c, case["max_pop_mean_val"])
    pv = iota(c, case["max_pop_var_val"])
    dx, dbeta, dgamma = impl.batchnorm_grad(x, dy, gamma, pm, pv, c, case["epsilon"], training)
    # test/batchnorm/batchnorm_fixture.h:271-287: the gradients cancel to ~0 on the ramps
    res.append(("grad",) + close(dx, case["exp_grad"], 30, 1e-2))
    res.append(("beta_grad",) + close(dbeta, case["beta_grad"], 10, 1e-5))
    res.append(("gamma_grad",) + close(dgamma, case["gamma_grad"], 30, 1e-2))
    return res
