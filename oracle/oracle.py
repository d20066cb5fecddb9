"""ctypes front end of the CPU oracle (oracle/portdnn_oracle.c).

TEST INFRASTRUCTURE ONLY.  Imported by tests/, by __graft_entry__.smoke() and by the
CPU arm of bench.py; the product package never imports it.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

FORWARD, INPUT_BACKPROP, FILTER_BACKPROP = 0, 1, 2
POOL_MAX, POOL_MAX_WITH_NAN, POOL_AVERAGE = 0, 1, 2
ADD, SUB, MUL, DIV = 0, 1, 2, 3
RELU, TANH = 0, 1
EXP, LOG, FLOOR, SQRT = 3, 4, 5, 6


class ConvParams(ctypes.Structure):
    """Same field order as sycldnn::conv2d::Conv2DParams (include/portdnn/conv2d/params.h:32-112)."""
    _fields_ = [(n, ctypes.c_int) for n in (
        "channels", "features", "batch", "in_rows", "in_cols", "window_rows", "window_cols",
        "stride_rows", "stride_cols", "out_rows", "out_cols", "pad_rows", "pad_cols",
        "dilation_rows", "dilation_cols", "groups", "input_format", "filter_format", "group_format")]


class DepthwiseParams(ctypes.Structure):
    """Same field order as DepthwiseConv2DParams (include/portdnn/depthwise_conv2d/params.h:33-94)."""
    _fields_ = [(n, ctypes.c_int) for n in (
        "channels", "channel_multiplier", "batch", "in_rows", "in_cols", "window_rows", "window_cols",
        "stride_rows", "stride_cols", "out_rows", "out_cols", "pad_rows", "pad_cols")]


class PoolParams(ctypes.Structure):
    """Same field order as PoolingParams (include/portdnn/pooling/params.h:30-73)."""
    _fields_ = [(n, ctypes.c_int) for n in (
        "in_rows", "in_cols", "out_rows", "out_cols", "window_rows", "window_cols", "stride_rows",
        "stride_cols", "batch", "channels", "pad_rows", "pad_cols", "input_format")]


def build(force=False):
    so = os.path.join(_HERE, "liboracle.so")
    src = os.path.join(_HERE, "portdnn_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "liboracle.so"], stdout=subprocess.DEVNULL)
    return so


def lib():
    global _LIB
    if _LIB is None:
        _LIB = ctypes.CDLL(build())
        _LIB.orc_padding.restype = ctypes.c_int
    return _LIB


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def padding(inp, window, stride, same):
    pad = ctypes.c_int(0)
    out = lib().orc_padding(int(inp), int(window), int(stride), int(bool(same)), ctypes.byref(pad))
    return out, pad.value


def conv_params(batch, in_rows, in_cols, channels, features, window, stride, same=True, pad=None,
                window_cols=None, stride_cols=None, groups=1, group_format=0):
    """Build params the way the reference's tests do (helpers::add_padding_to,
    include/portdnn/helpers/padding.h:76-88); ``pad`` overrides with an explicit low-side pad
    and out = (in + 2*pad - window)/stride + 1 like the compat API
    (include/portdnn/compat/convolution.hpp:411-415)."""
    wc = window if window_cols is None else window_cols
    sc = stride if stride_cols is None else stride_cols
    if pad is None:
        orow, prow = padding(in_rows, window, stride, same)
        ocol, pcol = padding(in_cols, wc, sc, same)
    else:
        prow = pcol = pad
        orow = (in_rows + 2 * pad - window) // stride + 1
        ocol = (in_cols + 2 * pad - wc) // sc + 1
    return ConvParams(channels, features, batch, in_rows, in_cols, window, wc, stride, sc, orow, ocol,
                      prow, pcol, 1, 1, groups, 0, 0, group_format)


def depthwise_params(batch, in_rows, in_cols, channels, mult, window, stride, same=True):
    orow, prow = padding(in_rows, window, stride, same)
    ocol, pcol = padding(in_cols, window, stride, same)
    return DepthwiseParams(channels, mult, batch, in_rows, in_cols, window, window, stride, stride,
                           orow, ocol, prow, pcol)


def pool_params(batch, in_rows, in_cols, channels, window, stride, same=True):
    orow, prow = padding(in_rows, window, stride, same)
    ocol, pcol = padding(in_cols, window, stride, same)
    return PoolParams(in_rows, in_cols, orow, ocol, window, window, stride, stride, batch, channels,
                      prow, pcol, 0)


def conv_sizes(pass_, p):
    """Element counts of the (input, filter, output) argument slots, conv2d/sizes.h:52-179."""
    x = p.batch * p.in_rows * p.in_cols * p.channels
    w = p.window_rows * p.window_cols * (p.channels // max(p.groups, 1)) * p.features
    y = p.batch * p.out_rows * p.out_cols * p.features
    return {FORWARD: (x, w, y), INPUT_BACKPROP: (y, w, x), FILTER_BACKPROP: (x, y, w)}[pass_]


def conv2d(pass_, inp, fil, p):
    n_in, n_fil, n_out = conv_sizes(pass_, p)
    inp, pi = _f(inp)
    fil, pf = _f(fil)
    assert inp.size == n_in and fil.size == n_fil, (inp.size, n_in, fil.size, n_fil)
    out = np.empty(n_out, dtype=np.float32)
    rc = lib().orc_conv2d(pass_, pi, pf, out.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), ctypes.byref(p))
    if rc != 0:
        raise ValueError("oracle: unsupported conv2d parameters")
    return out


def conv2d_forward_f32(x, w, p):
    x, px = _f(x)
    w, pw = _f(w)
    out = np.empty(p.batch * p.out_rows * p.out_cols * p.features, dtype=np.float32)
    lib().orc_conv2d_forward_f32(px, pw, out.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), ctypes.byref(p))
    return out


def depthwise_sizes(pass_, p):
    x = p.batch * p.in_rows * p.in_cols * p.channels
    w = p.window_rows * p.window_cols * p.channels * p.channel_multiplier
    y = p.batch * p.out_rows * p.out_cols * p.channels * p.channel_multiplier
    return {FORWARD: (x, w, y), INPUT_BACKPROP: (y, w, x), FILTER_BACKPROP: (x, y, w)}[pass_]


def depthwise_conv2d(pass_, inp, fil, p):
    n_in, n_fil, n_out = depthwise_sizes(pass_, p)
    inp, pi = _f(inp)
    fil, pf = _f(fil)
    assert inp.size == n_in and fil.size == n_fil
    out = np.empty(n_out, dtype=np.float32)
    lib().orc_depthwise_conv2d(pass_, pi, pf, out.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), ctypes.byref(p))
    return out


def pool_forward(op, x, p):
    x, px = _f(x)
    out = np.empty(p.batch * p.out_rows * p.out_cols * p.channels, dtype=np.float32)
    lib().orc_pool_forward(op, px, out.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), ctypes.byref(p))
    return out


def pool_max_grad(op, x, y, dy, p):
    x, px = _f(x)
    y, py = _f(y)
    dy, pdy = _f(dy)
    out = np.empty(x.size, dtype=np.float32)
    lib().orc_pool_max_grad(op, px, py, pdy, out.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), ctypes.byref(p))
    return out


def pool_avg_grad(dy, p):
    dy, pdy = _f(dy)
    out = np.empty(p.batch * p.in_rows * p.in_cols * p.channels, dtype=np.float32)
    lib().orc_pool_avg_grad(pdy, out.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), ctypes.byref(p))
    return out


def pointwise_forward(op, x):
    x, px = _f(x)
    out = np.empty_like(x)
    lib().orc_pointwise_forward(op, px, out.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), ctypes.c_size_t(x.size))
    return out


def pointwise_grad(op, fwd, err):
    fwd, pf = _f(fwd)
    err, pe = _f(err)
    out = np.empty_like(fwd)
    lib().orc_pointwise_grad(op, pf, pe, out.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), ctypes.c_size_t(fwd.size))
    return out


def binaryop(op, lhs, lhs_dims, rhs, rhs_dims):
    """lhs (op) rhs with numpy-style broadcasting of at most four extents; raises ValueError for
    shapes the reference rejects."""
    lhs, pl = _f(lhs)
    rhs, pr = _f(rhs)
    ld = (ctypes.c_int * max(len(lhs_dims), 1))(*lhs_dims)
    rd = (ctypes.c_int * max(len(rhs_dims), 1))(*rhs_dims)
    if len(lhs_dims) > 4 or len(rhs_dims) > 4:
        raise ValueError("binaryop: more than four extents")
    pad = lambda d: [1] * (4 - len(d)) + list(d)
    out = np.empty(int(np.prod([max(a, b) for a, b in zip(pad(lhs_dims), pad(rhs_dims))])), dtype=np.float32)
    if lib().orc_binaryop(op, pl, ld, len(lhs_dims), pr, rd, len(rhs_dims),
                          out.ctypes.data_as(ctypes.POINTER(ctypes.c_float))) != 0:
        raise ValueError("binaryop: shapes %s and %s cannot be broadcast" % (list(lhs_dims), list(rhs_dims)))
    return out


def bias_add(x, bias, channels):
    x, px = _f(x)
    bias, pb = _f(bias)
    out = np.empty_like(x)
    lib().orc_bias_add(px, pb, out.ctypes.data_as(ctypes.POINTER(ctypes.c_float)),
                       ctypes.c_size_t(x.size // channels), int(channels))
    return out


def matmul(tl, tr, lhs, rhs, batches, m, k, n, beta=0.0, out=None):
    lhs, pl = _f(lhs)
    rhs, pr = _f(rhs)
    res = np.zeros(batches * m * n, dtype=np.float32) if out is None else np.array(out, dtype=np.float32).ravel()
    lib().orc_matmul(int(tl), int(tr), pl, pr, res.ctypes.data_as(ctypes.POINTER(ctypes.c_float)),
                     int(batches), int(m), int(k), int(n), ctypes.c_float(beta))
    return res


def _out(n):
    a = np.empty(n, dtype=np.float32)
    return a, a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def softmax_forward(x, channels):
    x, px = _f(x)
    y, py = _out(x.size)
    lib().orc_softmax_forward(px, py, ctypes.c_size_t(x.size // channels), int(channels))
    return y


def softmax_grad(y, dy, channels):
    y, py = _f(y)
    dy, pdy = _f(dy)
    dx, pdx = _out(y.size)
    lib().orc_softmax_grad(py, pdy, pdx, ctypes.c_size_t(y.size // channels), int(channels))
    return dx


def batchnorm_forward(x, beta, gamma, mean, var, channels, eps=1e-3, momentum=0.9, training=False):
    """-> (output, running_mean, running_variance); the last two are None unless training."""
    x, px = _f(x)
    beta, pb = _f(beta)
    gamma, pg = _f(gamma)
    mean, pm = _f(mean)
    var, pv = _f(var)
    out, po = _out(x.size)
    rm, prm = _out(channels)
    rv, prv = _out(channels)
    lib().orc_batchnorm_forward(px, pb, pg, pm, pv, po, prm, prv, ctypes.c_size_t(x.size // channels), int(channels),
                                ctypes.c_float(eps), ctypes.c_float(momentum), int(bool(training)))
    return (out, rm, rv) if training else (out, None, None)


def batchnorm_grad(x, dy, gamma, pop_mean, pop_var, channels, eps=1e-3, training=False):
    """-> (input gradient, beta gradient, gamma gradient)."""
    x, px = _f(x)
    dy, pdy = _f(dy)
    gamma, pg = _f(gamma)
    pop_mean, pm = _f(pop_mean if pop_mean is not None else np.zeros(channels))
    pop_var, pv = _f(pop_var if pop_var is not None else np.ones(channels))
    out, po = _out(x.size)
    bg, pbg = _out(channels)
    gg, pgg = _out(channels)
    lib().orc_batchnorm_grad(px, pdy, pg, pm, pv, pbg, pgg, po, ctypes.c_size_t(x.size // channels), int(channels),
                             ctypes.c_float(eps), int(bool(training)))
    return out, bg, gg


def iota(size, max_val):
    """1, 2, ..., max_val, 1, 2, ... ; max_val < 1 means no wrap
    (reference test/gen/iota_initialised_data.h:45-79)."""
    a = np.arange(size, dtype=np.float64)
    if max_val >= 1:
        a = a % int(max_val)
    return (a + 1).astype(np.float32)
