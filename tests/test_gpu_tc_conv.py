"""The tcgen05 implicit-GEMM engine (conv2d forward / input backprop / filter backprop and the
matmul backend) against the CPU oracle on seeded inputs, through the C ABI.

Parity bars (relative error = max |diff| / max |ref| on identical, already-rounded inputs):
fp32 via 3xTF32 <= 1e-4, fp16 / bf16 <= 2e-2.
"""
import numpy as np
import pytest
import torch

import portdnn_b200 as pd
from conftest import rel_err
from gpu_util import TOL, assert_no_device_error, rounded, to_dev, to_host

pytestmark = pytest.mark.gpu


def _conv_case(orc, dtype, n, h, w, c, k, win, st, same=True, pad=None, seed=0):
    rng = np.random.default_rng(seed)
    p = pd.conv_params(n, h, w, c, k, win, st, same, pad)
    po = orc.conv_params(n, h, w, c, k, win, st, same, pad)
    x = rounded(rng.uniform(-1, 1, n * h * w * c).astype(np.float32), dtype)
    wt = rounded((rng.uniform(-1, 1, win * win * c * k) * np.sqrt(1.0 / (win * win * c))).astype(np.float32), dtype)
    dy = rounded(rng.standard_normal(n * p.out_rows * p.out_cols * k).astype(np.float32), dtype)
    return p, po, x, wt, dy


FWD_SHAPES = [
    # n, h, w, c, k, window, stride, same, pad
    (1, 56, 56, 256, 256, 3, 1, True, None),   # the single VGG-style layer
    (2, 56, 56, 64, 64, 3, 1, True, None),     # ResNet stage-1 3x3
    (2, 56, 56, 64, 256, 1, 1, True, None),    # 1x1 expand
    (2, 56, 56, 128, 128, 3, 2, True, None),   # stride-2 3x3 (pad_low 0, pad_high 1)
    (2, 56, 56, 256, 512, 1, 2, True, None),   # stride-2 projection
    (3, 14, 14, 256, 256, 3, 1, True, None),
    (5, 7, 7, 512, 512, 3, 1, True, None),
    (2, 32, 32, 8, 64, 7, 2, None, 3),         # stem-like 7x7/2 with explicit pad 3
    (2, 15, 13, 24, 40, 3, 1, True, None),     # ragged rows, column tail
    (3, 9, 9, 16, 16, 5, 2, False, None),      # VALID
    (2, 10, 12, 72, 96, 1, 1, True, None),     # MobileNet-like widths
    # the kernel's operand-staging variants
    (2, 56, 56, 64, 64, 3, 1, False, None),    # halo mode (resident filter, 8x16 tiles), VALID: ragged 54x54 output
    (1, 24, 40, 32, 64, 3, 1, True, None),     # halo mode, tile wider than tall, partial channel block
    (2, 16, 16, 16, 32, 5, 1, True, None),     # halo mode with a 5x5 window
    (3, 14, 14, 256, 1024, 1, 1, True, None),  # one resident filter column tile per CTA (8 column tiles)
    (3, 14, 14, 256, 256, 3, 1, True, None),   # pair mode, 256-column tiles
    (5, 7, 7, 512, 1024, 3, 1, True, None),    # pair mode, several column tiles, odd number of row tiles
    (2, 14, 14, 1024, 2048, 1, 2, True, None), # pair mode on a stride-2 projection
    (2, 28, 28, 512, 128, 1, 1, True, None),   # whole filter resident (128 KB)
]


@pytest.mark.parametrize("dtype", ["f16", "bf16", "f32"])
@pytest.mark.parametrize("shape", FWD_SHAPES)
def test_forward_against_oracle(orc, dtype, shape):
    n, h, w, c, k, win, st, same, pad = shape
    p, po, x, wt, _ = _conv_case(orc, dtype, n, h, w, c, k, win, st, bool(same), pad)
    y = to_host(pd.conv2d(pd.FORWARD, to_dev(x, dtype), to_dev(wt, dtype), p, algorithm=pd.ALGO_IM2COL))
    assert_no_device_error()
    assert rel_err(y, orc.conv2d(orc.FORWARD, x, wt, po)) <= TOL[dtype]


@pytest.mark.parametrize("dtype", ["f16", "f32"])
def test_forward_fhwc_filter(orc, dtype):
    n, h, w, c, k, win, st = 2, 20, 20, 64, 48, 3, 1
    p, po, x, wt, _ = _conv_case(orc, dtype, n, h, w, c, k, win, st)
    p.filter_format = 2
    w_fhwc = np.ascontiguousarray(wt.reshape(win, win, c, k).transpose(3, 0, 1, 2))
    y = to_host(pd.conv2d(pd.FORWARD, to_dev(x, dtype), to_dev(w_fhwc, dtype), p, algorithm=pd.ALGO_IM2COL))
    assert_no_device_error()
    assert rel_err(y, orc.conv2d(orc.FORWARD, x, wt, po)) <= TOL[dtype]


@pytest.mark.parametrize("dtype", ["f16", "f32"])
def test_forward_fused_epilogue(orc, dtype):
    n, h, w, c, k, win, st = 2, 28, 28, 128, 128, 3, 1
    p, po, x, wt, _ = _conv_case(orc, dtype, n, h, w, c, k, win, st)
    rng = np.random.default_rng(5)
    bias = rounded(rng.standard_normal(k).astype(np.float32), dtype)
    prev = rounded(rng.standard_normal(n * h * w * k).astype(np.float32), dtype)
    conv = orc.conv2d(orc.FORWARD, x, wt, po)
    ref = np.maximum(0.5 * conv + np.tile(bias, n * h * w), 0) + 0.25 * prev
    out = to_dev(prev, dtype)
    pd.conv2d(pd.FORWARD, to_dev(x, dtype), to_dev(wt, dtype), p, algorithm=pd.ALGO_IM2COL, out=out,
              bias=to_dev(bias, dtype), activation=pd.ACT_RELU, alpha=0.5, beta=0.25)
    assert_no_device_error()
    assert rel_err(to_host(out), ref) <= TOL[dtype]


@pytest.mark.parametrize("dtype", ["f16", "f32"])
@pytest.mark.parametrize("shape", [(2, 28, 28, 512, 128, 1, 1), (3, 14, 14, 256, 256, 3, 1), (2, 56, 56, 128, 128, 3, 2),
                                   (2, 56, 56, 64, 256, 1, 1)])
def test_constant_filter_changes_nothing_but_the_schedule(orc, dtype, shape):
    """constant_filter only moves the fetch of filter and bias ahead of the wait for the preceding kernel
    (resident-filter plans of the forward pass and the input backprop): the results are bit for bit the same."""
    n, h, w, c, k, win, st = shape
    p, po, x, wt, dy = _conv_case(orc, dtype, n, h, w, c, k, win, st)
    bias = to_dev(rounded(np.random.default_rng(2).standard_normal(k).astype(np.float32), dtype), dtype)
    xd, wd, dyd = to_dev(x, dtype), to_dev(wt, dtype), to_dev(dy, dtype)
    plain = pd.conv2d(pd.FORWARD, xd, wd, p, bias=bias, activation=pd.ACT_RELU)
    early = pd.conv2d(pd.FORWARD, xd, wd, p, bias=bias, activation=pd.ACT_RELU, constant_filter=True)
    assert torch.equal(plain, early)
    plain = pd.conv2d(pd.INPUT_BACKPROP, dyd, wd, p)
    early = pd.conv2d(pd.INPUT_BACKPROP, dyd, wd, p, constant_filter=True)
    assert torch.equal(plain, early)
    assert_no_device_error()
    assert rel_err(to_host(early), orc.conv2d(orc.INPUT_BACKPROP, dy, wt, po)) <= TOL[dtype]


GROUPED_SHAPES = [
    # n, h, w, c, k, window, stride, groups
    (2, 14, 14, 64, 128, 3, 1, 2),
    (3, 28, 28, 128, 128, 3, 2, 4),   # stride 2: one tensor map per input parity and group
    (2, 9, 11, 96, 48, 1, 1, 3),      # 16 features per group: partial column tiles
    (1, 16, 16, 256, 256, 3, 1, 32),  # ResNeXt-like: 8 channels per group
]


@pytest.mark.parametrize("dtype", ["f16", "f32"])
@pytest.mark.parametrize("fhwc", [False, True])
@pytest.mark.parametrize("shape", GROUPED_SHAPES)
def test_grouped_forward_on_tensor_cores(orc, dtype, fhwc, shape):
    """STRIDED groups with at least 8 channels and features per group: one implicit GEMM per group on
    channel slices (as many launches as groups), against the oracle's grouped convolution; bias and
    ReLU go through the same slices."""
    n, h, w, c, k, win, st, groups = shape
    rng = np.random.default_rng(11)
    p = pd.conv_params(n, h, w, c, k, win, st, groups=groups, filter_format=2 if fhwc else 0)
    po = orc.conv_params(n, h, w, c, k, win, st, groups=groups)
    cg = c // groups
    x = rounded(rng.uniform(-1, 1, n * h * w * c).astype(np.float32), dtype)
    wt = rounded((rng.uniform(-1, 1, win * win * cg * k) * np.sqrt(1.0 / (win * win * cg))).astype(np.float32), dtype)
    bias = rounded(rng.standard_normal(k).astype(np.float32), dtype)
    ref = np.maximum(orc.conv2d(orc.FORWARD, x, wt, po).reshape(-1, k) + bias, 0).ravel()
    w_dev = wt
    if fhwc:  # [K][R][S][C/G]: a group's filters are a contiguous run of rows
        w_dev = np.ascontiguousarray(wt.reshape(win * win * cg, k).T)
    before = pd.launch_count()
    y = to_host(pd.conv2d(pd.FORWARD, to_dev(x, dtype), to_dev(w_dev, dtype), p, algorithm=pd.ALGO_IM2COL,
                          bias=to_dev(bias, dtype), activation=pd.ACT_RELU))
    launches = pd.launch_count() - before
    assert_no_device_error()
    assert rel_err(y, ref) <= TOL[dtype]
    # 16-bit: four groups share a launch where their kernel has a multi-GEMM form (else one launch per group);
    # fp32: one launch per group, plus a filter-splitting launch per group where the filter slice is contiguous (FHWC)
    assert launches in ((-(-groups // 4), groups) if dtype == "f16" else (groups, 2 * groups)), launches
    if dtype == "f16" and not fhwc:
        assert launches == -(-groups // 4), launches


# Shapes large enough for the plans that need the whole device busy: clusters of two CTAs on 256 x 256
# tiles (long reduction, features a multiple of 256, at least 74 pairs of row tiles).
CTA_PAIR_SHAPES = [
    (128, 14, 14, 512, 512, 3, 1, True, None),
    (128, 14, 14, 2048, 512, 1, 1, True, None),
    (256, 28, 28, 256, 256, 3, 2, True, None),   # stride 2: one tensor map per input parity
    (131, 7, 7, 512, 512, 3, 1, True, None),     # an odd number of row tiles: the last pair is half empty
]


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("shape", CTA_PAIR_SHAPES)
def test_forward_cta_pair_plan_against_direct_kernel_and_oracle(orc, dtype, shape):
    """Forward layers that run on clusters of two CTAs (tcgen05 cta_group::2): the whole output against
    the CUDA-core direct kernel, and the first and last images against the oracle, with bias + ReLU."""
    n, h, w, c, k, win, st, same, pad = shape
    p, po, x, wt, _ = _conv_case(orc, dtype, n, h, w, c, k, win, st, bool(same), pad)
    rng = np.random.default_rng(3)
    b = rounded(rng.standard_normal(k).astype(np.float32) * 0.1, dtype)
    xd, wd, bd = to_dev(x, dtype), to_dev(wt, dtype), to_dev(b, dtype)
    y = pd.conv2d(pd.FORWARD, xd, wd, p, algorithm=pd.ALGO_IM2COL, bias=bd, activation=pd.ACT_RELU)
    assert_no_device_error()
    slow = pd.conv2d(pd.FORWARD, xd, wd, p, algorithm=pd.ALGO_DIRECT).float()
    slow = torch.relu((slow.view(-1, k) + bd.float()[None, :])).view(-1)
    err = ((y.float() - slow).abs().max() / slow.abs().max()).item()
    assert err <= TOL[dtype], err
    per_in, per_out = h * w * c, p.out_rows * p.out_cols * k
    p1 = orc.conv_params(1, h, w, c, k, win, st, bool(same), pad)
    for img in (0, n - 1):
        ref = orc.conv2d(orc.FORWARD, x[img * per_in:(img + 1) * per_in], wt, p1)
        ref = np.maximum(rounded(ref, dtype).reshape(-1, k) + b[None, :], 0).ravel()
        assert rel_err(to_host(y[img * per_out:(img + 1) * per_out]), ref) <= TOL[dtype], img


BWD_SHAPES = [
    (2, 28, 28, 128, 128, 3, 1, True, None),
    (2, 28, 28, 64, 256, 1, 1, True, None),
    (2, 28, 28, 128, 128, 3, 2, True, None),
    (2, 28, 28, 256, 512, 1, 2, True, None),
    (3, 7, 7, 512, 512, 3, 1, True, None),
    (2, 15, 13, 24, 40, 3, 1, True, None),
    (2, 17, 17, 16, 32, 5, 2, False, None),
    (2, 56, 56, 64, 64, 3, 1, False, None),    # input backprop in halo mode, VALID (ragged rows)
    (1, 24, 40, 32, 64, 3, 1, True, None),     # halo mode, wide tiles
    (2, 16, 16, 16, 32, 5, 1, True, None),     # halo mode, 5x5 window
    (2, 56, 56, 64, 256, 1, 1, True, None),    # 1x1: a single filter-gradient tile, many pixel splits
]


@pytest.mark.parametrize("dtype", ["f16", "bf16", "f32"])
@pytest.mark.parametrize("shape", BWD_SHAPES)
def test_input_backprop_against_oracle(orc, dtype, shape):
    n, h, w, c, k, win, st, same, pad = shape
    p, po, _, wt, dy = _conv_case(orc, dtype, n, h, w, c, k, win, st, bool(same), pad)
    dx = to_host(pd.conv2d(pd.INPUT_BACKPROP, to_dev(dy, dtype), to_dev(wt, dtype), p, algorithm=pd.ALGO_IM2COL))
    assert_no_device_error()
    assert rel_err(dx, orc.conv2d(orc.INPUT_BACKPROP, dy, wt, po)) <= TOL[dtype]


@pytest.mark.parametrize("dtype", ["f16", "bf16", "f32"])
@pytest.mark.parametrize("shape", BWD_SHAPES)
def test_filter_backprop_against_oracle(orc, dtype, shape):
    n, h, w, c, k, win, st, same, pad = shape
    p, po, x, _, dy = _conv_case(orc, dtype, n, h, w, c, k, win, st, bool(same), pad)
    dw = to_host(pd.conv2d(pd.FILTER_BACKPROP, to_dev(x, dtype), to_dev(dy, dtype), p, algorithm=pd.ALGO_IM2COL))
    assert_no_device_error()
    assert rel_err(dw, orc.conv2d(orc.FILTER_BACKPROP, x, dy, po)) <= TOL[dtype]


@pytest.mark.parametrize("dtype", ["f16", "bf16", "f32"])
@pytest.mark.parametrize("shape", [(2, 32, 32, 3, 64, 7, 2, None, 3), (2, 24, 24, 3, 64, 3, 1, True, None),
                                   (3, 17, 19, 3, 32, 5, 2, True, None), (2, 20, 20, 1, 16, 3, 1, False, None),
                                   # one plain copy per tile (rows of 32, 64 and 128 pixel pairs)
                                   (2, 56, 52, 3, 64, 7, 2, None, 3), (1, 112, 112, 3, 32, 7, 2, None, 3),
                                   (1, 224, 224, 3, 64, 7, 2, None, 3), (2, 54, 54, 4, 16, 5, 2, True, None),
                                   (2, 57, 57, 2, 24, 3, 2, False, None)])
def test_stem_forward_and_filter_backprop_few_channels(orc, dtype, shape):
    """Network stems (C < 8): the packed-row tensor-core path, forward and filter gradient."""
    n, h, w, c, k, win, st, same, pad = shape
    p, po, x, wt, dy = _conv_case(orc, dtype, n, h, w, c, k, win, st, bool(same), pad)
    y = to_host(pd.conv2d(pd.FORWARD, to_dev(x, dtype), to_dev(wt, dtype), p, algorithm=pd.ALGO_IM2COL))
    assert_no_device_error()
    assert rel_err(y, orc.conv2d(orc.FORWARD, x, wt, po)) <= TOL[dtype]
    dw = to_host(pd.conv2d(pd.FILTER_BACKPROP, to_dev(x, dtype), to_dev(dy, dtype), p, algorithm=pd.ALGO_IM2COL))
    assert_no_device_error()
    assert rel_err(dw, orc.conv2d(orc.FILTER_BACKPROP, x, dy, po)) <= TOL[dtype]


def test_filter_backprop_with_caller_workspace(orc):
    n, h, w, c, k, win, st = 8, 28, 28, 64, 64, 3, 1
    p, po, x, _, dy = _conv_case(orc, "f16", n, h, w, c, k, win, st)
    _, rec = pd.conv2d_workspace_size(pd.FILTER_BACKPROP, pd.F16, p, pd.ALGO_IM2COL)
    assert rec > 0
    ws = torch.empty(rec, dtype=torch.float16, device="cuda")
    dw = to_host(pd.conv2d(pd.FILTER_BACKPROP, to_dev(x, "f16"), to_dev(dy, "f16"), p, algorithm=pd.ALGO_IM2COL,
                           workspace=ws))
    assert_no_device_error()
    assert rel_err(dw, orc.conv2d(orc.FILTER_BACKPROP, x, dy, po)) <= TOL["f16"]


@pytest.mark.parametrize("dtype", ["f16", "bf16", "f32"])
@pytest.mark.parametrize("tl", [False, True])
@pytest.mark.parametrize("tr", [False, True])
@pytest.mark.parametrize("dims", [(1, 256, 192, 128, 0.0), (2, 200, 136, 72, 0.0), (3, 128, 64, 64, 1.0)])
def test_matmul_against_oracle(orc, dtype, tl, tr, dims):
    batches, m, k, n, beta = dims
    rng = np.random.default_rng(21)
    a = rounded(rng.uniform(-1, 1, batches * m * k).astype(np.float32), dtype)
    b = rounded(rng.uniform(-1, 1, batches * k * n).astype(np.float32), dtype)
    c0 = rounded(rng.uniform(-1, 1, batches * m * n).astype(np.float32), dtype)
    out = to_dev(c0, dtype)
    pd.matmul(to_dev(a, dtype), to_dev(b, dtype), batches, m, k, n, tl, tr, beta=beta, out=out)
    assert_no_device_error()
    ref = orc.matmul(tl, tr, a, b, batches, m, k, n, beta=beta, out=c0)
    assert rel_err(to_host(out), ref) <= TOL[dtype]


def test_matmul_odd_sizes_take_the_simt_kernel(orc):
    batches, m, k, n = 2, 13, 7, 5
    rng = np.random.default_rng(22)
    a = rng.standard_normal(batches * m * k).astype(np.float32)
    b = rng.standard_normal(batches * k * n).astype(np.float32)
    got = to_host(pd.matmul(to_dev(a, "f32"), to_dev(b, "f32"), batches, m, k, n))
    assert rel_err(got, orc.matmul(False, False, a, b, batches, m, k, n)) <= 1e-5


@pytest.mark.parametrize("shape", [(64, 56, 56, 64, 64, 3, 1), (64, 56, 56, 256, 128, 1, 2), (32, 28, 28, 128, 128, 3, 2)])
def test_full_size_layers_tensor_core_vs_direct_kernel(shape):
    """At sizes the CPU oracle cannot finish quickly: the tensor-core engine against the direct
    CUDA kernel (itself checked against the oracle and the reference vectors), all three passes,
    plus linearity of the forward pass."""
    n, h, w, c, k, win, st = shape
    g = torch.Generator(device="cuda").manual_seed(3)
    p = pd.conv_params(n, h, w, c, k, win, st)
    x = (torch.rand(n * h * w * c, device="cuda", generator=g) * 2 - 1).half()
    wt = ((torch.rand(win * win * c * k, device="cuda", generator=g) * 2 - 1) * (1.0 / (win * win * c)) ** 0.5).half()
    dy = torch.randn(n * p.out_rows * p.out_cols * k, device="cuda", generator=g).half()
    for pass_, a, b in ((pd.FORWARD, x, wt), (pd.INPUT_BACKPROP, dy, wt), (pd.FILTER_BACKPROP, x, dy)):
        fast = pd.conv2d(pass_, a, b, p, algorithm=pd.ALGO_IM2COL).float()
        slow = pd.conv2d(pass_, a, b, p, algorithm=pd.ALGO_DIRECT).float()
        assert_no_device_error()
        err = (fast - slow).abs().max().item() / slow.abs().max().item()
        assert err <= 2e-2, (pass_, err)
    y1 = pd.conv2d(pd.FORWARD, x, wt, p).float()
    y2 = pd.conv2d(pd.FORWARD, (x.float() * 0.5).half(), wt, p).float()
    assert ((y1 * 0.5 - y2).abs().max() / y1.abs().max()).item() <= 2e-3


@pytest.mark.parametrize("dtype", ["f16", "bf16", "f32"])
@pytest.mark.parametrize("shape", BWD_SHAPES + [(2, 20, 20, 24, 40, 3, 2, True, None), (3, 9, 9, 5, 7, 3, 1, True, None)])
def test_fused_backprop_forms_against_oracle(orc, dtype, shape):
    """PdnnBackpropFusion: the input backprop with the ReLU-gradient mask of the preceding layer
    applied on the way out, and the filter backprop written as fp32, against the oracle chain
    input backprop -> pointwise Relu Gradient (src/pointwise/kernels.h:205-233) and its fp32
    filter gradient.  The last shape takes the direct kernel (channels not a multiple of 8)."""
    n, h, w, c, k, win, st, same, pad = shape
    p, po, x, wt, dy = _conv_case(orc, dtype, n, h, w, c, k, win, st, bool(same), pad)
    rng = np.random.default_rng(31)
    # forward output of the preceding layer: about half of it zero, as a ReLU leaves it
    y_prev = rounded(np.maximum(rng.standard_normal(n * h * w * c), 0).astype(np.float32), dtype)
    dx = to_host(pd.conv2d(pd.INPUT_BACKPROP, to_dev(dy, dtype), to_dev(wt, dtype), p, algorithm=pd.ALGO_IM2COL,
                           relu_forward_output=to_dev(y_prev, dtype)))
    assert_no_device_error()
    ref = orc.pointwise_grad(0, y_prev, orc.conv2d(orc.INPUT_BACKPROP, dy, wt, po))
    assert rel_err(dx, ref) <= TOL[dtype]
    assert not np.any(dx[y_prev <= 0] != 0)
    dw = pd.conv2d(pd.FILTER_BACKPROP, to_dev(x, dtype), to_dev(dy, dtype), p, algorithm=pd.ALGO_IM2COL,
                   output_f32=dtype != "f32")
    assert dw.dtype == torch.float32
    assert_no_device_error()
    assert rel_err(to_host(dw), orc.conv2d(orc.FILTER_BACKPROP, x, dy, po)) <= TOL[dtype]


@pytest.mark.parametrize("dtype", ["f16", "bf16", "f32"])
@pytest.mark.parametrize("masked", [True, False, "premasked"])
@pytest.mark.parametrize("shape", BWD_SHAPES + [(2, 20, 20, 24, 40, 3, 2, True, None), (3, 9, 9, 5, 7, 3, 1, True, None),
                                                (4, 28, 28, 128, 256, 1, 2, True, None), (2, 14, 14, 512, 256, 1, 1, True, None)])
def test_accumulating_input_backprop_against_oracle(orc, dtype, masked, shape):
    """PdnnBackpropFusion::accumulate: dx already holds the gradient from another reader of the tensor;
    the call adds its own and (optionally) masks the sum, against the oracle chain input backprop ->
    add -> pointwise Relu Gradient.  Pixels outside every parity class of a strided layer keep
    (masked) what was there."""
    n, h, w, c, k, win, st, same, pad = shape
    p, po, x, wt, dy = _conv_case(orc, dtype, n, h, w, c, k, win, st, bool(same), pad)
    rng = np.random.default_rng(77)
    y_prev = rounded(np.maximum(rng.standard_normal(n * h * w * c), 0).astype(np.float32), dtype)
    before = rounded(rng.standard_normal(n * h * w * c).astype(np.float32), dtype)
    if masked == "premasked":  # accumulate = 2: dx already carries the mask, untouched positions may be skipped
        before = orc.pointwise_grad(0, y_prev, before)
    dx = to_dev(before, dtype)
    pd.conv2d(pd.INPUT_BACKPROP, to_dev(dy, dtype), to_dev(wt, dtype), p, algorithm=pd.ALGO_IM2COL, out=dx,
              relu_forward_output=to_dev(y_prev, dtype) if masked else None, accumulate=2 if masked == "premasked" else True)
    assert_no_device_error()
    ref = before + orc.conv2d(orc.INPUT_BACKPROP, dy, wt, po)
    if masked:
        ref = orc.pointwise_grad(0, y_prev, ref)
    got = to_host(dx)
    assert rel_err(got, ref) <= TOL[dtype]
    if masked:
        assert not np.any(got[y_prev <= 0] != 0)


@pytest.mark.parametrize("dtype", ["f16", "bf16", "f32"])
@pytest.mark.parametrize("f32_out", [True, False])
@pytest.mark.parametrize("shape", BWD_SHAPES + [(2, 32, 32, 3, 64, 7, 2, None, 3), (3, 9, 9, 5, 7, 3, 1, True, None)])
def test_accumulating_filter_backprop_against_oracle(orc, dtype, f32_out, shape):
    """PdnnBackpropFusion::accumulate for the filter backprop: dW += gradient, twice in a row onto a
    non-zero start (fp32 gradients: the pixel splits add their tiles by TMA reduction; otherwise the
    split reduction adds)."""
    if dtype == "f32" and f32_out:
        pytest.skip("fp32 tensors always have fp32 gradients")
    n, h, w, c, k, win, st, same, pad = shape
    p, po, x, wt, dy = _conv_case(orc, dtype, n, h, w, c, k, win, st, same if same is None else bool(same), pad)
    rng = np.random.default_rng(91)
    out_kind = "f32" if (f32_out or dtype == "f32") else dtype
    before = rounded(rng.standard_normal(wt.size).astype(np.float32), out_kind)
    dw = to_dev(before, out_kind)
    for _ in range(2):
        pd.conv2d(pd.FILTER_BACKPROP, to_dev(x, dtype), to_dev(dy, dtype), p, algorithm=pd.ALGO_IM2COL, out=dw,
                  output_f32=f32_out, accumulate=True)
    assert_no_device_error()
    grad = orc.conv2d(orc.FILTER_BACKPROP, x, dy, po)
    # the 16-bit accumulator rounds after each addition; compare against the same chain
    ref = rounded(rounded(before + grad, out_kind) + grad, out_kind) if out_kind != "f32" else before + 2 * grad
    assert rel_err(to_host(dw), ref) <= 2 * TOL[dtype]


def _pack_bits(mask):
    """numpy bool array -> the library's bitmask bytes (bit i % 8 of byte i / 8)."""
    return np.packbits(mask.astype(np.uint8), bitorder="little")


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("shape", [(2, 28, 28, 128, 128, 3, 1, True, None), (2, 28, 28, 64, 256, 1, 1, True, None),
                                   (2, 15, 13, 24, 40, 3, 1, True, None), (2, 28, 28, 256, 512, 1, 2, True, None),
                                   (128, 14, 14, 512, 512, 3, 1, True, None), (2, 32, 32, 3, 64, 7, 2, None, 3)])
def test_forward_writes_the_relu_bitmask(orc, dtype, shape):
    """PdnnConvEpilogue::relu_bitmask: bit i is set exactly where output element i is positive, whichever kernel
    ran (packed epilogue of the tensor-core kernels, the CTA-pair kernel, or the pass over the output)."""
    n, h, w, c, k, win, st, same, pad = shape
    p, po, x, wt, _ = _conv_case(orc, dtype, n, h, w, c, k, win, st, same if same is None else bool(same), pad)
    rng = np.random.default_rng(5)
    b = rounded(rng.standard_normal(k).astype(np.float32) * 0.1, dtype)
    n_out = n * p.out_rows * p.out_cols * k
    bits = torch.full((n_out // 8,), 0xAA, dtype=torch.uint8, device="cuda")
    y = pd.conv2d(pd.FORWARD, to_dev(x, dtype), to_dev(wt, dtype), p, algorithm=pd.ALGO_IM2COL, bias=to_dev(b, dtype),
                  activation=pd.ACT_RELU, relu_bitmask=bits)
    assert_no_device_error()
    assert np.array_equal(bits.cpu().numpy(), _pack_bits(to_host(y) > 0))


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("accumulate", [0, 1, 2])
@pytest.mark.parametrize("shape", BWD_SHAPES + [(2, 20, 20, 24, 40, 3, 2, True, None), (4, 28, 28, 128, 256, 1, 2, True, None),
                                                (2, 14, 14, 512, 256, 1, 1, True, None)])
def test_input_backprop_with_the_relu_bitmask_equals_the_tensor_form(orc, dtype, accumulate, shape):
    """PdnnBackpropFusion::relu_bitmask gives bit for bit what relu_forward_output gives."""
    n, h, w, c, k, win, st, same, pad = shape
    p, po, x, wt, dy = _conv_case(orc, dtype, n, h, w, c, k, win, st, bool(same), pad)
    if c % 8:
        pytest.skip("the bitmask needs a multiple of 8 channels")
    rng = np.random.default_rng(41)
    y_prev = rounded(np.maximum(rng.standard_normal(n * h * w * c), 0).astype(np.float32), dtype)
    before = orc.pointwise_grad(0, y_prev, rounded(rng.standard_normal(n * h * w * c).astype(np.float32), dtype))
    bits = torch.from_numpy(_pack_bits(y_prev > 0)).cuda()
    results = []
    for kw in ({"relu_forward_output": to_dev(y_prev, dtype)}, {"relu_bitmask": bits}):
        dx = to_dev(before, dtype)
        pd.conv2d(pd.INPUT_BACKPROP, to_dev(dy, dtype), to_dev(wt, dtype), p, algorithm=pd.ALGO_IM2COL, out=dx,
                  accumulate=accumulate, **kw)
        assert_no_device_error()
        results.append(to_host(dx))
    assert np.array_equal(results[0], results[1])
    assert not np.any(results[1][y_prev <= 0] != 0)


def test_fused_backprop_stem_filter_gradient_fp32(orc):
    n, h, w, c, k, win, st = 2, 32, 32, 3, 64, 7, 2
    p, po, x, _, dy = _conv_case(orc, "f16", n, h, w, c, k, win, st, None, 3)
    dw = pd.conv2d(pd.FILTER_BACKPROP, to_dev(x, "f16"), to_dev(dy, "f16"), p, algorithm=pd.ALGO_IM2COL, output_f32=True)
    assert dw.dtype == torch.float32
    assert rel_err(to_host(dw), orc.conv2d(orc.FILTER_BACKPROP, x, dy, po)) <= TOL["f16"]
