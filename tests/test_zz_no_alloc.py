"""The allocation-free entry point, pdnn_depthwise_filter_backprop_noalloc, against the regular
depthwise filter backprop (pdnn_depthwise_conv2d), both through the C ABI.

Some callers cannot let a library allocate device memory while they run (a server with a fixed
memory plan, a framework that owns the device heap).  For them this entry point keeps its
partial sums in a fixed array inside the library.  The test calls it twice in a row, on
different shapes, so that the second call runs over whatever the first one left in that array;
each result must equal the regular entry point's, within the tolerance the depthwise parity
tests use (1e-5 relative for fp32, 2e-2 for fp16).  The file name sorts last so that a run that
stops at the first failure has already been through every other test.
"""
import numpy as np
import pytest
import torch

import portdnn_b200 as pd
from portdnn_b200 import api

pytestmark = pytest.mark.gpu


def _case(dtype, n, h, w, c, m, win, st, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    p = pd.depthwise_params(n, h, w, c, m, win, st)
    x = torch.randn(n * h * w * c, device="cuda", generator=g).to(dtype)
    dy = torch.randn(n * p.out_rows * p.out_cols * c * m, device="cuda", generator=g).to(dtype)
    return p, x, dy


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.float16, 2e-2)])
def test_noalloc_matches_regular_entry_point_twice_in_a_row(dtype, tol):
    shapes = [(4, 28, 28, 192, 1, 3, 1, 1), (3, 15, 17, 24, 2, 5, 2, 2)]
    for n, h, w, c, m, win, st, seed in shapes:
        p, x, dy = _case(dtype, n, h, w, c, m, win, st, seed)
        ref = pd.depthwise_conv2d(pd.FILTER_BACKPROP, x, dy, p).float()
        out = torch.full((win * win * c * m,), 7.0, dtype=dtype, device="cuda")  # caller-owned output
        api.depthwise_filter_backprop_noalloc(x, dy, p, out)
        torch.cuda.synchronize()
        err = ((out.float() - ref).abs().max() / ref.abs().max()).item()
        assert err <= tol, (n, h, w, c, m, win, st, err)


def test_noalloc_rejects_what_does_not_fit():
    # a filter gradient larger than the fixed scratch: R*S*C*mult*4 bytes > the array
    limit = api.noalloc_scratch_bytes()
    c = limit // (4 * 9) + 64
    p = pd.depthwise_params(1, 3, 3, c, 1, 3, 1)
    x = torch.zeros(9 * c, device="cuda")
    dy = torch.zeros(9 * c, device="cuda")
    out = torch.zeros(9 * c, device="cuda")
    with pytest.raises(pd.PortDNNError) as e:
        api.depthwise_filter_backprop_noalloc(x, dy, p, out)
    assert e.value.status == pd.StatusCode.InsufficientWorkspace
