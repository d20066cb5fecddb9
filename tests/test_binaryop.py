"""Binary operators with broadcasting: the oracle and the CUDA path (through the C ABI) on the 52
known-answer cases of the reference's test/binaryop/binaryop_{add,sub,mul,div}.cc
(tests/golden/binaryop_kat.npz, made by tests/golden/make_golden_binaryop.py), on larger seeded
shapes against the oracle, and the shapes the reference rejects."""
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
CASES = list(np.load(os.path.join(HERE, "golden", "binaryop_kat.npz"), allow_pickle=True)["cases"])
IDS = ["%s-%s" % (c["op"], c["name"]) for c in CASES]
OPS = ["add", "sub", "mul", "div"]


def ramp(n, wrap):
    """1, 2, ..., wrap, 1, ...: the reference's iota_initialised_data (test/gen/iota_initialised_data.h:45-79)."""
    return (np.arange(n) % int(wrap) + 1).astype(np.float32)


def _operands(case):
    return (ramp(int(np.prod(case["lhs_dims"])), case["max_input_val"]),
            ramp(int(np.prod(case["rhs_dims"])), case["max_input_val"]))


@pytest.mark.parametrize("case", CASES, ids=IDS)
def test_oracle_matches_reference_vectors(orc, case):
    lhs, rhs = _operands(case)
    out = orc.binaryop(OPS.index(case["op"]), lhs, case["lhs_dims"], rhs, case["rhs_dims"])
    # the fixture compares within 10 ULP (test/binaryop/fixture.h:69-72)
    np.testing.assert_allclose(out, case["exp_out"], rtol=10 * 2.0 ** -23)


def test_oracle_rejects_what_the_reference_rejects(orc):
    one = np.ones(6, np.float32)
    with pytest.raises(ValueError):
        orc.binaryop(0, one, [2, 3], one, [3, 2])        # extents that cannot be broadcast
    with pytest.raises(ValueError):
        orc.binaryop(0, one, [1, 1, 1, 2, 3], one, [6])  # more than four extents


@pytest.mark.gpu
@pytest.mark.parametrize("case", CASES, ids=IDS)
def test_gpu_matches_reference_vectors(case):
    import portdnn_b200 as pd
    from gpu_util import to_dev, to_host
    lhs, rhs = _operands(case)
    out = to_host(pd.binaryop(OPS.index(case["op"]), to_dev(lhs, "f32"), case["lhs_dims"], to_dev(rhs, "f32"),
                              case["rhs_dims"]))
    np.testing.assert_allclose(out, case["exp_out"], rtol=10 * 2.0 ** -23)


SHAPES = [
    ([64, 56, 56, 64], [64, 56, 56, 64]),     # equal shapes: one extent after merging
    ([64 * 56 * 56, 256], [1, 256]),          # the bias form
    ([32, 28, 28, 128], [32, 1, 1, 128]),     # per-image, per-channel (squeeze-excite scale)
    ([32, 28, 28, 128], [1]),                 # scalar right side
    ([], [7, 9, 11]),                         # scalar left side, odd sizes
    ([5, 1, 33], [1, 17, 1]),                 # both sides broadcast, innermost not a packet
    ([3, 1, 16], [2, 1, 7, 1]),
    ([12, 40, 1], [12, 1, 24]),               # innermost extent broadcast on the left
]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("op", [0, 1, 2, 3])
@pytest.mark.parametrize("shape", SHAPES, ids=[str(s) for s in SHAPES])
def test_gpu_matches_oracle(orc, shape, op, dtype):
    import portdnn_b200 as pd
    from conftest import rel_err
    from gpu_util import rounded, to_dev, to_host
    rng = np.random.default_rng(23)
    ld, rd = shape
    lhs = rounded(rng.uniform(0.5, 2.0, int(np.prod(ld))).astype(np.float32), dtype)
    rhs = rounded(rng.uniform(0.5, 2.0, int(np.prod(rd))).astype(np.float32), dtype)
    ref = orc.binaryop(op, lhs, ld, rhs, rd)
    out = to_host(pd.binaryop(op, to_dev(lhs, dtype), ld, to_dev(rhs, dtype), rd))
    if dtype == "f32":
        np.testing.assert_array_equal(out, ref)   # one IEEE operation per element
    else:
        assert rel_err(out, ref) <= 2.0 ** -8


@pytest.mark.gpu
def test_gpu_rejects_bad_shapes():
    import torch
    import portdnn_b200 as pd
    x = torch.ones(6, device="cuda")
    for ld, rd in (([2, 3], [3, 2]), ([1, 1, 1, 2, 3], [6]), ([0, 6], [6])):
        with pytest.raises(pd.PortDNNError) as e:
            pd.binaryop(pd.BINARY_ADD, x, ld, x, rd)
        assert e.value.status == pd.StatusCode.InvalidParameter
    with pytest.raises(pd.PortDNNError):
        pd.binaryop(4, x, [6], x, [6])
