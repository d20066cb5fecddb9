"""B200-native implementation of portDNN's conv2d hot path.

The product is ``libportdnn_b200.so`` (hand-written sm_100a CUDA behind the C ABI of
``include/portdnn_b200.h``) plus the C++ headers under ``include/portdnn/`` that rebuild
portDNN's ``sycldnn::`` API on top of it.  This package is the Python front end used by
the tests and the benchmark: thin ctypes calls on torch CUDA tensors, named after the
reference's operators.  There is no CPU path: without the built library, or without a
B200, every call raises.
"""
from .api import (  # noqa: F401
    FORWARD, INPUT_BACKPROP, FILTER_BACKPROP,
    F32, F16, BF16,
    ALGO_DIRECT, ALGO_TILED, ALGO_IM2COL, ALGO_WINOGRAD, ALGO_WINOGRAD_LARGE, ALGO_MATMUL,
    POOL_MAX, POOL_MAX_WITH_NAN, POOL_AVERAGE,
    ACT_NONE, ACT_RELU, ACT_TANH, ACT_RELU6,
    PW_EXP, PW_LOG, PW_FLOOR, PW_SQRT, BINARY_ADD, BINARY_SUB, BINARY_MUL, BINARY_DIV,
    StatusCode, PortDNNError,
    Conv2DParams, DepthwiseConv2DParams, PoolingParams, SoftmaxParams, BatchNormParams,
    conv_params, depthwise_params, pool_params, calculate_padding,
    conv2d, conv2d_workspace_size, conv2d_validate, depthwise_conv2d, pooling, pooling_max_grad,
    pointwise, pointwise_grad, bias_add, binaryop, scale_blend, matmul, transpose,
    softmax, batchnorm_params, batchnorm_forward, batchnorm_gradient,
    device_error_record, launch_count, lib, library_path,
)
