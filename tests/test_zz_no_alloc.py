"""The allocation-free entry point, pdnn_depthwise_filter_backprop_noalloc, against the regular
depthwise filter backprop (pdnn_depthwise_conv2d), both through the C ABI.

Some callers cannot let a library allocate device memory while they run (a server with a fixed
memory plan, a framework that owns the device heap).  For them this entry point keeps its
partial sums in a fixed array inside the library.  The test calls it twice in a row, on
different shapes, so that the second call runs over whatever the first one left in that array;
each result must equal the regular entry point's, and the CPU oracle's, within the tolerance the
depthwise parity tests use (1e-5 relative for fp32, 2e-2 for fp16).  A further test checks what the
entry point promises: the device's free memory and the stream-ordered allocator's pool are the
same before and after a call.  The file name sorts last so that a run that stops at the first
failure has already been through every other test.
"""
import ctypes

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
def test_noalloc_matches_regular_entry_point_and_oracle_twice_in_a_row(orc, dtype, tol):
    # the second shape has a channel multiplier (scalar path); the third, fp16 only, has a filter
    # gradient so large that fewer pixel slices fit into the fixed array than the regular path uses
    shapes = [(4, 28, 28, 192, 1, 3, 1, 1), (3, 15, 17, 24, 2, 5, 2, 2)]
    if dtype == torch.float16:
        shapes.append((4, 35, 35, 16384, 1, 3, 1, 3))
    for n, h, w, c, m, win, st, seed in shapes:
        p, x, dy = _case(dtype, n, h, w, c, m, win, st, seed)
        ref = pd.depthwise_conv2d(pd.FILTER_BACKPROP, x, dy, p).float()
        out = torch.full((win * win * c * m,), 7.0, dtype=dtype, device="cuda")  # caller-owned output
        api.depthwise_filter_backprop_noalloc(x, dy, p, out)
        torch.cuda.synchronize()
        err = ((out.float() - ref).abs().max() / ref.abs().max()).item()
        assert err <= tol, (n, h, w, c, m, win, st, err)
        if c <= 1024:  # the oracle is a scalar loop: keep it to the small shapes
            po = orc.depthwise_params(n, h, w, c, m, win, st)
            want = orc.depthwise_conv2d(orc.FILTER_BACKPROP, x.float().cpu().numpy(), dy.float().cpu().numpy(), po)
            got = out.float().cpu().numpy()
            assert np.abs(got - want).max() <= tol * max(np.abs(want).max(), 1e-30) * (1 if dtype == torch.float16 else 10)


def test_noalloc_call_allocates_nothing():
    """Free device memory and the default memory pool's reserved / used bytes do not move across a call."""
    rt = ctypes.CDLL("libcudart.so.12")
    pool = ctypes.c_void_p()
    assert rt.cudaDeviceGetDefaultMemPool(ctypes.byref(pool), torch.cuda.current_device()) == 0

    def pool_bytes():
        vals = []
        for attr in (5, 7):  # cudaMemPoolAttrReservedMemCurrent, cudaMemPoolAttrUsedMemCurrent
            v = ctypes.c_uint64(0)
            assert rt.cudaMemPoolGetAttribute(pool, attr, ctypes.byref(v)) == 0
            vals.append(v.value)
        return vals

    p, x, dy = _case(torch.float16, 4, 28, 28, 192, 1, 3, 1, 9)
    out = torch.empty(9 * 192, dtype=torch.float16, device="cuda")
    api.depthwise_filter_backprop_noalloc(x, dy, p, out)   # the first call on the device does the one-time set-up
    torch.cuda.synchronize()
    free0, pool0 = torch.cuda.mem_get_info()[0], pool_bytes()
    api.depthwise_filter_backprop_noalloc(x, dy, p, out)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0
    assert pool_bytes() == pool0


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
