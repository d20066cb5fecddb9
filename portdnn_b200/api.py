"""ctypes front end of libportdnn_b200.so working on torch CUDA tensors.

Function names and argument meaning follow the reference's launch functions
(include/portdnn/<op>/launch.h); the parameter structs have the reference's field order.
torch is used for device memory and streams only.
"""
import ctypes
import enum
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

FORWARD, INPUT_BACKPROP, FILTER_BACKPROP = 0, 1, 2
F32, F16, BF16 = 0, 1, 2
ALGO_DIRECT, ALGO_TILED, ALGO_IM2COL, ALGO_WINOGRAD, ALGO_WINOGRAD_LARGE, ALGO_MATMUL = 1, 2, 3, 4, 5, 6
POOL_MAX, POOL_MAX_WITH_NAN, POOL_AVERAGE = 0, 1, 2
ACT_NONE, ACT_RELU, ACT_TANH, ACT_RELU6 = -1, 0, 1, 2
BINARY_ADD, BINARY_SUB, BINARY_MUL, BINARY_DIV = 0, 1, 2, 3
PW_EXP, PW_LOG, PW_FLOOR, PW_SQRT = 3, 4, 5, 6  # the other sycldnn::pointwise operators (pointwise() only)


class StatusCode(enum.IntEnum):
    """sycldnn::StatusCode, include/portdnn/status.h:31-44."""
    OK = 0
    InvalidAlgorithm = 1
    IndexExceeded = 2
    InsufficientWorkspace = 3
    AllocationProblem = 4
    InvalidParameter = 5


class PortDNNError(RuntimeError):
    def __init__(self, status, message):
        super().__init__("%s: %s" % (StatusCode(status).name, message))
        self.status = StatusCode(status)


def _ints(*names):
    return [(n, ctypes.c_int) for n in names]


class Conv2DParams(ctypes.Structure):
    """sycldnn::conv2d::Conv2DParams, include/portdnn/conv2d/params.h:32-112."""
    _fields_ = _ints("channels", "features", "batch", "in_rows", "in_cols", "window_rows", "window_cols",
                     "stride_rows", "stride_cols", "out_rows", "out_cols", "pad_rows", "pad_cols",
                     "dilation_rows", "dilation_cols", "groups", "input_format", "filter_format", "group_format")


class DepthwiseConv2DParams(ctypes.Structure):
    """sycldnn::depthwise_conv2d::DepthwiseConv2DParams, include/portdnn/depthwise_conv2d/params.h:33-94."""
    _fields_ = _ints("channels", "channel_multiplier", "batch", "in_rows", "in_cols", "window_rows", "window_cols",
                     "stride_rows", "stride_cols", "out_rows", "out_cols", "pad_rows", "pad_cols")


class PoolingParams(ctypes.Structure):
    """sycldnn::pooling::PoolingParams, include/portdnn/pooling/params.h:30-73."""
    _fields_ = _ints("in_rows", "in_cols", "out_rows", "out_cols", "window_rows", "window_cols", "stride_rows",
                     "stride_cols", "batch", "channels", "pad_rows", "pad_cols", "input_format")


class SoftmaxParams(ctypes.Structure):
    """sycldnn::softmax::SoftmaxParams, include/portdnn/softmax/params.h:27-54."""
    _fields_ = _ints("channels", "batch", "rows", "cols", "input_format")


class BatchNormParams(ctypes.Structure):
    """sycldnn::batchnorm::BatchNormParams, include/portdnn/batchnorm/params.h:32-72."""
    _fields_ = _ints("batch", "rows", "cols", "channels", "is_training") + \
        [("epsilon", ctypes.c_float), ("momentum", ctypes.c_float), ("input_format", ctypes.c_int)]


class _BackpropFusion(ctypes.Structure):
    _fields_ = [("relu_forward_output", ctypes.c_void_p), ("output_f32", ctypes.c_int), ("accumulate", ctypes.c_int),
                ("relu_bitmask", ctypes.c_void_p), ("constant_filter", ctypes.c_int)]


class _Epilogue(ctypes.Structure):
    _fields_ = [("bias", ctypes.c_void_p), ("activation", ctypes.c_int), ("alpha", ctypes.c_float),
                ("beta", ctypes.c_float), ("relu_bitmask", ctypes.c_void_p), ("constant_filter", ctypes.c_int)]


def library_path():
    return os.path.join(_HERE, "libportdnn_b200.so")


def lib():
    """Loads the CUDA library; raises if it has not been built (there is no fallback)."""
    global _LIB
    if _LIB is None:
        path = library_path()
        if not os.path.exists(path):
            raise ImportError("%s is missing: build it with `python -m portdnn_b200.build`" % path)
        L = ctypes.CDLL(path)
        L.pdnn_last_error.restype = ctypes.c_char_p
        L.pdnn_launch_count.restype = ctypes.c_ulonglong
        L.pdnn_depthwise_workspace_bytes.restype = ctypes.c_size_t
        L.pdnn_noalloc_scratch_bytes.restype = ctypes.c_size_t
        _LIB = L
    return _LIB


def _check(status):
    if status != 0:
        raise PortDNNError(status, lib().pdnn_last_error().decode())


def calculate_padding(inp, window, stride, same):
    """helpers::calculate_padding, include/portdnn/helpers/padding.h:46-66 -> (pad_low, out)."""
    if same:
        out = -(-inp // stride)
        need = (out - 1) * stride + window - inp
        return int(need / 2), out  # C integer division truncates toward zero
    num = inp - window + 1
    out = -(-num // stride) if num >= 0 else int(num / stride)
    return 0, out


def conv_params(batch, in_rows, in_cols, channels, features, window, stride, same=True, pad=None, groups=1,
                filter_format=0, group_format=0):
    """Params as helpers::add_padding_to builds them (include/portdnn/helpers/padding.h:76-88); an explicit
    ``pad`` gives the compat API's symmetric form (include/portdnn/compat/convolution.hpp:411-415)."""
    if pad is None:
        prow, orow = calculate_padding(in_rows, window, stride, same)
        pcol, ocol = calculate_padding(in_cols, window, stride, same)
    else:
        prow = pcol = pad
        orow = (in_rows + 2 * pad - window) // stride + 1
        ocol = (in_cols + 2 * pad - window) // stride + 1
    return Conv2DParams(channels, features, batch, in_rows, in_cols, window, window, stride, stride, orow, ocol,
                        prow, pcol, 1, 1, groups, 0, filter_format, group_format)


def depthwise_params(batch, in_rows, in_cols, channels, mult, window, stride, same=True):
    prow, orow = calculate_padding(in_rows, window, stride, same)
    pcol, ocol = calculate_padding(in_cols, window, stride, same)
    return DepthwiseConv2DParams(channels, mult, batch, in_rows, in_cols, window, window, stride, stride, orow, ocol,
                                 prow, pcol)


def pool_params(batch, in_rows, in_cols, channels, window, stride, same=True):
    prow, orow = calculate_padding(in_rows, window, stride, same)
    pcol, ocol = calculate_padding(in_cols, window, stride, same)
    return PoolingParams(in_rows, in_cols, orow, ocol, window, window, stride, stride, batch, channels, prow, pcol, 0)


def _torch():
    import torch
    return torch


def _dtype_code(t):
    torch = _torch()
    return {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}[t.dtype]


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


def _stream():
    return ctypes.c_void_p(_torch().cuda.current_stream().cuda_stream)


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise ValueError("tensors must be contiguous CUDA tensors")


def conv_sizes(pass_, p):
    """(input, filter, output) element counts of the argument slots, include/portdnn/conv2d/sizes.h:52-179."""
    x = p.batch * p.in_rows * p.in_cols * p.channels
    w = p.window_rows * p.window_cols * (p.channels // max(p.groups, 1)) * p.features
    y = p.batch * p.out_rows * p.out_cols * p.features
    return {FORWARD: (x, w, y), INPUT_BACKPROP: (y, w, x), FILTER_BACKPROP: (x, y, w)}[pass_]


def conv2d_validate(pass_, params, algorithm):
    return StatusCode(lib().pdnn_conv2d_validate(pass_, ctypes.byref(params), algorithm))


def conv2d_workspace_size(pass_, dtype, params, algorithm):
    """conv2d::query_workspace_size, include/portdnn/conv2d/workspace_size.h:158-163 -> (required, recommended) elements."""
    req, rec = ctypes.c_size_t(0), ctypes.c_size_t(0)
    _check(lib().pdnn_conv2d_workspace_size(pass_, dtype, ctypes.byref(params), algorithm, ctypes.byref(req),
                                            ctypes.byref(rec)))
    return req.value, rec.value


def conv2d(pass_, inp, fil, params, algorithm=ALGO_IM2COL, out=None, workspace=None, bias=None, activation=ACT_NONE,
           alpha=1.0, beta=0.0, relu_forward_output=None, output_f32=False, accumulate=False, relu_bitmask=None,
           constant_filter=False):
    """conv2d::launch<T, ConvType>(input, filter, output, params, selector, backend, workspace, size)
    (include/portdnn/conv2d/launch.h:59-72) with the selector's answer passed as ``algorithm``.
    Slots: Forward (x, w) -> y; InputBackprop (dy, w) -> dx; FilterBackprop (x, dy) -> dW.
    bias / activation / alpha / beta select the fused forward epilogue; relu_forward_output and accumulate
    (InputBackprop: dx += ..., then the mask; FilterBackprop: dW += ...) and output_f32 (FilterBackprop) the fused backprop forms of
    PdnnBackpropFusion.  relu_bitmask: a uint8 tensor of one bit per element (numel / 8 bytes) - written by
    the forward pass beside its output, read by the input backprop in place of relu_forward_output.
    constant_filter (Forward, InputBackprop): filter and bias were not written by the kernel that precedes this
    call in the stream, so the kernel may fetch them while that kernel is still finishing."""
    torch = _torch()
    _require_cuda(inp, fil, out, workspace, bias)
    n_in, n_fil, n_out = conv_sizes(pass_, params)
    if inp.numel() != n_in or fil.numel() != n_fil:
        raise ValueError("tensor sizes do not match the parameters: %d/%d, %d/%d" % (inp.numel(), n_in, fil.numel(), n_fil))
    _require_cuda(relu_bitmask)
    if relu_bitmask is not None:
        if pass_ == FILTER_BACKPROP:
            raise ValueError("relu_bitmask belongs to the forward pass (output) and the input backprop (input)")
        n_bits = n_out  # forward: the output's mask; input backprop: the mask of dx
        if relu_bitmask.dtype != torch.uint8 or relu_bitmask.numel() * 8 != n_bits:
            raise ValueError("relu_bitmask must be a uint8 tensor of one bit per element")
    backprop_fused = (relu_forward_output is not None or output_f32 or accumulate or
                      (relu_bitmask is not None and pass_ != FORWARD) or (constant_filter and pass_ == INPUT_BACKPROP))
    if backprop_fused and (pass_ == FORWARD or (relu_forward_output is not None and pass_ != INPUT_BACKPROP) or
                           (output_f32 and pass_ != FILTER_BACKPROP)):
        raise ValueError("relu_forward_output belongs to the input backprop, output_f32 to the filter backprop")
    if accumulate and out is None:
        raise ValueError("accumulate needs the tensor to add to as out")
    _require_cuda(relu_forward_output)
    if out is None:
        out = torch.empty(n_out, dtype=torch.float32 if output_f32 else inp.dtype, device=inp.device)
    if out.numel() != n_out or out.dtype != (torch.float32 if output_f32 else inp.dtype):
        raise ValueError("output tensor does not match the parameters")
    ws_elems = workspace.numel() * workspace.element_size() // inp.element_size() if workspace is not None else 0
    if backprop_fused:
        if relu_forward_output is not None and relu_forward_output.numel() != n_out:
            raise ValueError("relu_forward_output must have the shape of the input gradient")
        fus = _BackpropFusion(relu_forward_output.data_ptr() if relu_forward_output is not None else None, int(output_f32),
                              int(accumulate),  # accumulate: False / True, or 2 (dx already carries the mask)
                              relu_bitmask.data_ptr() if relu_bitmask is not None else None, int(bool(constant_filter)))
        _check(lib().pdnn_conv2d_backprop_fused(pass_, _dtype_code(inp), _ptr(inp), _ptr(fil), _ptr(out),
                                                ctypes.byref(params), algorithm, ctypes.byref(fus), _ptr(workspace),
                                                ctypes.c_size_t(ws_elems), _stream()))
        return out
    fused = (bias is not None or activation != ACT_NONE or alpha != 1.0 or beta != 0.0 or relu_bitmask is not None or
             (constant_filter and pass_ == FORWARD))
    if fused:
        if pass_ != FORWARD:
            raise ValueError("the fused epilogue exists for the forward pass only")
        epi = _Epilogue(bias.data_ptr() if bias is not None else None, activation, alpha, beta,
                        relu_bitmask.data_ptr() if relu_bitmask is not None else None, int(bool(constant_filter)))
        st = lib().pdnn_conv2d_fused(_dtype_code(inp), _ptr(inp), _ptr(fil), _ptr(out), ctypes.byref(params), algorithm,
                                     ctypes.byref(epi), _ptr(workspace), ctypes.c_size_t(ws_elems), _stream())
    else:
        st = lib().pdnn_conv2d(pass_, _dtype_code(inp), _ptr(inp), _ptr(fil), _ptr(out), ctypes.byref(params), algorithm,
                               _ptr(workspace), ctypes.c_size_t(ws_elems), _stream())
    _check(st)
    return out


def depthwise_conv2d(pass_, inp, fil, params, out=None, workspace=None):
    """depthwise_conv2d::launch<T, ConvType> (include/portdnn/depthwise_conv2d/launch.h:54-91)."""
    torch = _torch()
    _require_cuda(inp, fil, out, workspace)
    p = params
    x = p.batch * p.in_rows * p.in_cols * p.channels
    w = p.window_rows * p.window_cols * p.channels * p.channel_multiplier
    y = p.batch * p.out_rows * p.out_cols * p.channels * p.channel_multiplier
    n_in, n_fil, n_out = {FORWARD: (x, w, y), INPUT_BACKPROP: (y, w, x), FILTER_BACKPROP: (x, y, w)}[pass_]
    if inp.numel() != n_in or fil.numel() != n_fil:
        raise ValueError("tensor sizes do not match the parameters")
    if out is None:
        out = torch.empty(n_out, dtype=inp.dtype, device=inp.device)
    ws_bytes = workspace.numel() * workspace.element_size() if workspace is not None else 0
    _check(lib().pdnn_depthwise_conv2d(pass_, _dtype_code(inp), _ptr(inp), _ptr(fil), _ptr(out), ctypes.byref(p),
                                       _ptr(workspace), ctypes.c_size_t(ws_bytes), _stream()))
    return out


def depthwise_filter_backprop_noalloc(inp, output_grad, params, out):
    """pdnn_depthwise_filter_backprop_noalloc: (x, dy) -> dW into the caller's ``out`` without any
    device allocation inside the library (the partial sums use the library's fixed scratch array).
    No counterpart in the reference."""
    _require_cuda(inp, output_grad, out)
    _check(lib().pdnn_depthwise_filter_backprop_noalloc(_dtype_code(inp), _ptr(inp), _ptr(output_grad), _ptr(out),
                                                        ctypes.byref(params), _stream()))
    return out


def noalloc_scratch_bytes():
    return int(lib().pdnn_noalloc_scratch_bytes())


def depthwise_workspace_bytes(pass_, dtype, params):
    return lib().pdnn_depthwise_workspace_bytes(pass_, dtype, ctypes.byref(params))


def pooling(op, direction, inp, params, out=None):
    """pooling::launch<T, Op, Direction>, two-pointer form (include/portdnn/pooling/launch.h:112-180):
    direction 0 = Forward (x -> y); direction 1 = Backpropagate, Average only (dy -> dx)."""
    torch = _torch()
    _require_cuda(inp, out)
    p = params
    n_out = (p.batch * p.out_rows * p.out_cols if direction == 0 else p.batch * p.in_rows * p.in_cols) * p.channels
    if out is None:
        out = torch.empty(n_out, dtype=inp.dtype, device=inp.device)
    _check(lib().pdnn_pooling(op, direction, _dtype_code(inp), _ptr(inp), _ptr(out), ctypes.byref(p), _stream()))
    return out


def pooling_max_grad(op, input_data, output_data, input_backprop, params, out=None, relu_input=False):
    """pooling::launch<T, Max|MaxWithNan, Backpropagate>, four-pointer form
    (include/portdnn/pooling/launch.h:182-257): (x, y, dy) -> dx.  relu_input: x is a ReLU's output and
    dx is to be the gradient with respect to that ReLU's input (pdnn_pooling_max_grad_relu)."""
    torch = _torch()
    _require_cuda(input_data, output_data, input_backprop, out)
    if out is None:
        out = torch.empty(input_data.numel(), dtype=input_data.dtype, device=input_data.device)
    fn = lib().pdnn_pooling_max_grad_relu if relu_input else lib().pdnn_pooling_max_grad
    _check(fn(op, _dtype_code(input_data), _ptr(input_data), _ptr(output_data),
                                       _ptr(input_backprop), _ptr(out), ctypes.byref(params), _stream()))
    return out


def pointwise(op, inp, out=None):
    """pointwise::launch<T, Op, Forward> (include/portdnn/pointwise/launch.h:61-100)."""
    torch = _torch()
    _require_cuda(inp, out)
    if out is None:
        out = torch.empty_like(inp)
    _check(lib().pdnn_pointwise(op, _dtype_code(inp), _ptr(inp), _ptr(out), ctypes.c_size_t(inp.numel()), _stream()))
    return out


def pointwise_grad(op, output_forward, input_backprop, out=None):
    """pointwise::launch<T, Op, Gradient> (include/portdnn/pointwise/launch.h:133-179)."""
    torch = _torch()
    _require_cuda(output_forward, input_backprop, out)
    if out is None:
        out = torch.empty_like(output_forward)
    _check(lib().pdnn_pointwise_grad(op, _dtype_code(output_forward), _ptr(output_forward), _ptr(input_backprop),
                                     _ptr(out), ctypes.c_size_t(output_forward.numel()), _stream()))
    return out


def bias_add(inp, bias, channels, activation=ACT_NONE, out=None):
    """binaryop::launch<T, Add> with lhs_dims={rows, C}, rhs_dims={1, C} (test/bias/bias_fixture.h:78-85)."""
    torch = _torch()
    _require_cuda(inp, bias, out)
    if out is None:
        out = torch.empty_like(inp)
    _check(lib().pdnn_bias_add(_dtype_code(inp), _ptr(inp), _ptr(bias), _ptr(out),
                               ctypes.c_size_t(inp.numel() // channels), int(channels), int(activation), _stream()))
    return out


def binaryop(op, lhs, lhs_dims, rhs, rhs_dims, out=None):
    """binaryop::launch<T, Op> (include/portdnn/binaryop/launch.h:58-97): lhs (op) rhs with numpy-style
    broadcasting of at most four extents per operand; `op` is one of BINARY_ADD / SUB / MUL / DIV."""
    torch = _torch()
    _require_cuda(lhs, rhs, out)
    lhs_dims, rhs_dims = [int(d) for d in lhs_dims], [int(d) for d in rhs_dims]
    if out is None:
        n = max(len(lhs_dims), len(rhs_dims))
        pad = lambda d: [1] * (n - len(d)) + d
        numel = 1
        for x, y in zip(pad(lhs_dims), pad(rhs_dims)):
            numel *= max(x, y, 0)
        out = torch.empty(numel, dtype=lhs.dtype, device=lhs.device)
    ld = (ctypes.c_int * max(len(lhs_dims), 1))(*lhs_dims)
    rd = (ctypes.c_int * max(len(rhs_dims), 1))(*rhs_dims)
    _check(lib().pdnn_binaryop(int(op), _dtype_code(lhs), _ptr(lhs), ld, len(lhs_dims), _ptr(rhs), rd, len(rhs_dims),
                               _ptr(out), _stream()))
    return out


def scale_blend(a, alpha, b=None, beta=0.0, out=None):
    """out = alpha*a + beta*b, the compat layer's blend (include/portdnn/compat/scaling.hpp:202-281)."""
    torch = _torch()
    _require_cuda(a, b, out)
    if out is None:
        out = torch.empty_like(a)
    _check(lib().pdnn_scale_blend(_dtype_code(a), _ptr(a), ctypes.c_float(alpha), _ptr(b), ctypes.c_float(beta),
                                  _ptr(out), ctypes.c_size_t(a.numel()), _stream()))
    return out


def matmul(lhs, rhs, batches, m, k, n, transpose_lhs=False, transpose_rhs=False, beta=0.0, out=None):
    """matmul::launch<T, TransposeLHS, TransposeRHS> (include/portdnn/matmul/launch.h:37-90):
    out[b] = beta*out[b] + op(lhs[b]) @ op(rhs[b]), row-major, strided batches."""
    torch = _torch()
    _require_cuda(lhs, rhs, out)
    if lhs.numel() != batches * m * k or rhs.numel() != batches * k * n:
        raise ValueError("tensor sizes do not match the parameters")
    if out is None:
        if beta != 0.0:
            raise ValueError("beta != 0 needs an output tensor to accumulate into")
        out = torch.empty(batches * m * n, dtype=lhs.dtype, device=lhs.device)
    _check(lib().pdnn_matmul(_dtype_code(lhs), int(transpose_lhs), int(transpose_rhs), _ptr(lhs), _ptr(rhs), _ptr(out),
                             int(batches), int(m), int(k), int(n), ctypes.c_float(beta), _stream()))
    return out


def transpose(inp, dims, permutation, out=None):
    """transpose::launch<T> (include/portdnn/transpose/launch.h:66-111): output extent d is dims[permutation[d]]."""
    torch = _torch()
    _require_cuda(inp, out)
    dims, permutation = [int(d) for d in dims], [int(d) for d in permutation]
    n = 1
    for d in dims:
        n *= d
    if inp.numel() != n or len(dims) != len(permutation):
        raise ValueError("tensor size does not match the dimensions")
    if out is None:
        out = torch.empty_like(inp)
    cd, cp = (ctypes.c_int * len(dims))(*dims), (ctypes.c_int * len(dims))(*permutation)
    _check(lib().pdnn_transpose(inp.element_size(), _ptr(inp), _ptr(out), cd, len(dims), cp, _stream()))
    return out


def softmax(inp, batch, rows, cols, channels, gradient=None, out=None):
    """softmax::launch<T, Forward> (gradient None) or <T, Gradient> (inp = the forward output, gradient = dy),
    include/portdnn/softmax/launch.h:64-165."""
    torch = _torch()
    _require_cuda(inp, gradient, out)
    if inp.numel() != batch * rows * cols * channels:
        raise ValueError("tensor size does not match the parameters")
    if out is None:
        out = torch.empty_like(inp)
    p = SoftmaxParams(channels, batch, rows, cols, 0)
    _check(lib().pdnn_softmax(0 if gradient is None else 1, _dtype_code(inp), _ptr(inp), _ptr(gradient), _ptr(out),
                              ctypes.byref(p), _stream()))
    return out


def batchnorm_params(batch, rows, cols, channels, training, epsilon=1e-3, momentum=0.9):
    return BatchNormParams(batch, rows, cols, channels, int(bool(training)), epsilon, momentum, 0)


def batchnorm_forward(inp, beta, gamma, mean, variance, params, out=None):
    """batchnorm::launch<T, Backend, Forward> (include/portdnn/batchnorm/launch.h:222-330)
    -> (output, running_mean, running_variance); the last two are None for frozen parameters."""
    torch = _torch()
    _require_cuda(inp, beta, gamma, mean, variance, out)
    if out is None:
        out = torch.empty_like(inp)
    rm = rv = None
    if params.is_training:
        rm, rv = torch.empty_like(mean), torch.empty_like(variance)
    _check(lib().pdnn_batchnorm_forward(_dtype_code(inp), _ptr(inp), _ptr(beta), _ptr(gamma), _ptr(mean), _ptr(variance),
                                        _ptr(rm), _ptr(rv), _ptr(out), ctypes.byref(params), _stream()))
    return out, rm, rv


def batchnorm_gradient(inp, gradient, gamma, params, pop_mean=None, pop_variance=None, out=None):
    """batchnorm::launch<T, Backend, Gradient> (include/portdnn/batchnorm/launch.h:332-444)
    -> (input gradient, beta gradient, gamma gradient)."""
    torch = _torch()
    _require_cuda(inp, gradient, gamma, pop_mean, pop_variance, out)
    if out is None:
        out = torch.empty_like(inp)
    bg, gg = torch.empty_like(gamma), torch.empty_like(gamma)
    _check(lib().pdnn_batchnorm_gradient(_dtype_code(inp), _ptr(inp), _ptr(gradient), _ptr(gamma), _ptr(pop_mean),
                                         _ptr(pop_variance), _ptr(bg), _ptr(gg), _ptr(out), ctypes.byref(params),
                                         _stream()))
    return out, bg, gg


def device_error_record(clear=True):
    """The tensor-core kernels' error record (4 words, word 0 == 0: no error). Synchronises."""
    words = (ctypes.c_uint * 4)()
    _check(lib().pdnn_device_error_record(words, int(clear)))
    return list(words)


def launch_count():
    return int(lib().pdnn_launch_count())
