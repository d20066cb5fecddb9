// extern "C" entry points declared in include/portdnn_b200.h.
#include "common.cuh"
#include "tc_gemm.cuh"

#include <mutex>

namespace pdnn {

std::atomic<unsigned long long> g_launches{0};

char* last_error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

bool& bitmask_written_flag() {
  static thread_local bool written = false;
  return written;
}

int current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return dev;
}

// SM count of the CURRENT device (-1 if it is not an sm_100 part), looked up once per device.
int device_sm_count() {
  static std::mutex mu;
  static int table[kMaxDevices];
  static bool known[kMaxDevices] = {};
  const int dev = current_device();
  if (dev < 0 || dev >= kMaxDevices) return -1;
  std::lock_guard<std::mutex> lock(mu);
  if (!known[dev]) {
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) {
      cudaGetLastError();
      return -1;
    }
    table[dev] = prop.major >= 10 ? prop.multiProcessorCount : -1;  // the kernels are sm_100a only
    // Scratch that a call takes from the stream-ordered allocator goes back to the device's
    // default pool; keep it there instead of returning it to the driver at the next
    // synchronisation, or every such call pays for a fresh allocation.
    cudaMemPool_t pool;
    if (table[dev] > 0 && cudaDeviceGetDefaultMemPool(&pool, dev) == cudaSuccess) {
      unsigned long long keep = 1ull << 32;  // up to 4 GiB cached
      cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
    }
    cudaGetLastError();
    known[dev] = true;
  }
  return table[dev];
}

namespace {

// conv2d::validate_params + the checks of sublaunch (include/portdnn/internal/conv2d/launch.h:42-97,169-197).
int validate_conv(int pass, const PdnnConv2DParams* p, int algorithm) {
  if (p == nullptr) return fail(PDNN_INVALID_PARAMETER, "conv2d: null params");
  if (pass < 0 || pass > 2) return fail(PDNN_INVALID_PARAMETER, "conv2d: bad pass %d", pass);
#define PDNN_REQUIRE(cond, msg) \
  if (!(cond)) return fail(PDNN_INVALID_PARAMETER, "conv2d: %s", msg)
  PDNN_REQUIRE(p->batch > 0, "The number of batches must be positive.");
  PDNN_REQUIRE(p->channels > 0, "The number of channels must be positive.");
  PDNN_REQUIRE(p->features > 0, "The number of features must be positive.");
  PDNN_REQUIRE(p->in_rows > 0, "The number of input rows must be positive.");
  PDNN_REQUIRE(p->in_cols > 0, "The number of input columns must be positive.");
  PDNN_REQUIRE(p->out_rows > 0, "The number of output rows must be positive.");
  PDNN_REQUIRE(p->out_cols > 0, "The number of output columns must be positive.");
  PDNN_REQUIRE(p->window_rows > 0, "The number of window rows must be positive.");
  PDNN_REQUIRE(p->window_cols > 0, "The number of window columns must be positive.");
  PDNN_REQUIRE(p->stride_rows > 0, "The stride in the row direction must be positive.");
  PDNN_REQUIRE(p->stride_cols > 0, "The stride in the column direction must be positive.");
  PDNN_REQUIRE(p->pad_rows >= 0, "The padding in the row direction must be non-negative.");
  PDNN_REQUIRE(p->pad_cols >= 0, "The padding in the column direction must be non-negative.");
  PDNN_REQUIRE(p->groups > 0, "The number of groups must be positive.");
  PDNN_REQUIRE(p->channels % p->groups == 0, "Channels must be divisible by groups.");
  PDNN_REQUIRE(p->features % p->groups == 0, "Features must be divisible by groups.");
  PDNN_REQUIRE(p->dilation_rows == 1 && p->dilation_cols == 1, "Only dilation 1 is supported.");
  PDNN_REQUIRE(p->input_format != 0 || p->filter_format == 0 || p->filter_format == 2, "Unsupported layout combination.");
  PDNN_REQUIRE(p->input_format != 1 || p->filter_format == 1, "Unsupported layout combination.");
  PDNN_REQUIRE(p->input_format == 0 || p->input_format == 1, "Unknown input format.");
  PDNN_REQUIRE(p->groups != 1 || p->group_format == 0, "Interleaved is unsupported when group size is one.");
  PDNN_REQUIRE(p->group_format != 1 || p->filter_format == 0, "Unsupported group and filter format combination.");
  PDNN_REQUIRE(p->groups == 1 || pass == PDNN_FORWARD, "Grouped convolution is only supported for the forward pass.");
#undef PDNN_REQUIRE
  if (algorithm <= PDNN_ALGO_NOT_SUPPORTED || algorithm > PDNN_ALGO_MATMUL)
    return fail(PDNN_INVALID_ALGORITHM, "conv2d: algorithm %d is not runnable", algorithm);
  if (p->input_format == 1 && algorithm != PDNN_ALGO_DIRECT)
    return fail(PDNN_INVALID_ALGORITHM, "conv2d: NCHW is only supported by the direct algorithm");
  if (p->groups > 1 && algorithm != PDNN_ALGO_IM2COL)
    return fail(PDNN_INVALID_ALGORITHM, "conv2d: grouped convolution is only supported by the im2col algorithm");
  // Per-algorithm applicability, with the status codes of the reference's launchers.
  const bool square = p->window_rows == p->window_cols && p->stride_rows == p->stride_cols;
  if (algorithm == PDNN_ALGO_MATMUL &&
      !(p->window_rows == 1 && p->window_cols == 1 && p->stride_rows == 1 && p->stride_cols == 1))
    // include/portdnn/conv2d/implementation/matmul.h:95-104 (SNN_VALIDATE_PARAM)
    return fail(PDNN_INVALID_PARAMETER, "conv2d: Matmul can only be used for 1x1 NHWC convolutions with stride 1.");
  if (algorithm == PDNN_ALGO_TILED) {
    // src/conv2d/tiled/launch_tiled.cc:164-273: no filter backprop; forward and input backprop for
    // square windows 1 and 3 with stride 1 or 2 and window 5 with stride 1
    const int w = p->window_rows, st = p->stride_rows;
    const bool listed = square && ((w == 1 || w == 3) ? (st == 1 || st == 2) : (w == 5 && st == 1));
    if (pass == PDNN_FILTER_BACKPROP || !listed)
      return fail(PDNN_INVALID_ALGORITHM, "conv2d: the tiled algorithm does not cover this window / stride / pass");
  }
  if (algorithm == PDNN_ALGO_WINOGRAD || algorithm == PDNN_ALGO_WINOGRAD_LARGE) {
    // include/portdnn/internal/conv2d/winograd/launch.h:298-396: 3x3 (both tags), 3x1 and 1x3 (Winograd only)
    const bool w33 = p->window_rows == 3 && p->window_cols == 3;
    const bool w31 = (p->window_rows == 3 && p->window_cols == 1) || (p->window_rows == 1 && p->window_cols == 3);
    if (!(w33 || (algorithm == PDNN_ALGO_WINOGRAD && w31)))
      return fail(PDNN_INVALID_ALGORITHM, "conv2d: the Winograd algorithms need a 3x3 (or 3x1 / 1x3) window");
  }
  return PDNN_OK;
}

template <typename T>
__global__ void __launch_bounds__(256) widen_to_f32_kernel(const T* __restrict__ in, float* __restrict__ out, size_t n,
                                                           bool accumulate) {
  for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (size_t)gridDim.x * 256)
    out[i] = (accumulate ? out[i] : 0.f) + to_f32(in[i]);
}

// The direct kernel with the fused backprop forms applied afterwards (shapes the tensor-core engine
// does not take): the ReLU-gradient mask as a pointwise pass in place, an fp32 filter gradient
// through a temporary in the tensors' own type.
int run_direct_backprop(int pass, int dtype, const void* in, const void* fil, void* out, const PdnnConv2DParams& p,
                        const PdnnBackpropFusion* fusion, cudaStream_t s) {
  const size_t es = dtype_size(dtype);
  if (pass == PDNN_FILTER_BACKPROP && fusion != nullptr && fusion->accumulate && !(fusion->output_f32 && dtype != PDNN_F32)) {
    // dW += gradient in the tensors' own type: the gradient into a temporary, then one blend
    const size_t n = (size_t)p.window_rows * p.window_cols * (p.channels / p.groups) * p.features;
    void* tmp = nullptr;
    if (cudaMallocAsync(&tmp, n * es, s) != cudaSuccess) {
      cudaGetLastError();
      return fail(PDNN_ALLOCATION_PROBLEM, "conv2d: cannot allocate %zu bytes for the filter gradient", n * es);
    }
    int st = launch_direct_conv(pass, dtype, in, fil, tmp, p, nullptr, s);
    if (st == PDNN_OK) st = launch_scale_blend(dtype, tmp, 1.f, out, 1.f, out, n, s);
    cudaFreeAsync(tmp, s);
    return st;
  }
  if (pass == PDNN_FILTER_BACKPROP && fusion != nullptr && fusion->output_f32 && dtype != PDNN_F32) {
    const size_t n = (size_t)p.window_rows * p.window_cols * (p.channels / p.groups) * p.features;
    void* tmp = nullptr;
    if (cudaMallocAsync(&tmp, n * es, s) != cudaSuccess) {
      cudaGetLastError();
      return fail(PDNN_ALLOCATION_PROBLEM, "conv2d: cannot allocate %zu bytes for the filter gradient", n * es);
    }
    int st = launch_direct_conv(pass, dtype, in, fil, tmp, p, nullptr, s);
    if (st == PDNN_OK) {
      const unsigned grid = grid_for(n, 256, device_sm_count());
      if (dtype == PDNN_F16) widen_to_f32_kernel<__half><<<grid, 256, 0, s>>>(static_cast<const __half*>(tmp), static_cast<float*>(out), n, fusion->accumulate != 0);
      else widen_to_f32_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(tmp), static_cast<float*>(out), n, fusion->accumulate != 0);
      st = check_launch("filter gradient widening");
    }
    cudaFreeAsync(tmp, s);
    return st;
  }
  const size_t n_dx = (size_t)p.batch * p.in_rows * p.in_cols * p.channels;
  int st;
  if (pass == PDNN_INPUT_BACKPROP && fusion != nullptr && fusion->accumulate) {
    void* tmp = nullptr;
    if (cudaMallocAsync(&tmp, n_dx * es, s) != cudaSuccess) {
      cudaGetLastError();
      return fail(PDNN_ALLOCATION_PROBLEM, "conv2d: cannot allocate %zu bytes for the input gradient", n_dx * es);
    }
    st = launch_direct_conv(pass, dtype, in, fil, tmp, p, nullptr, s);
    if (st == PDNN_OK) st = launch_scale_blend(dtype, tmp, 1.f, out, 1.f, out, n_dx, s);
    cudaFreeAsync(tmp, s);
  } else {
    st = launch_direct_conv(pass, dtype, in, fil, out, p, nullptr, s);
  }
  if (st != PDNN_OK || pass != PDNN_INPUT_BACKPROP || fusion == nullptr) return st;
  if (fusion->relu_bitmask != nullptr) return launch_relu_grad_bits(dtype, fusion->relu_bitmask, out, n_dx, s);
  if (fusion->relu_forward_output == nullptr) return st;
  return launch_pointwise_grad(PDNN_ACT_RELU, dtype, fusion->relu_forward_output, out, out, n_dx, s);
}

int dispatch_conv(int pass, int dtype, const void* in, const void* fil, void* out, const PdnnConv2DParams* p, int algorithm,
                  const PdnnConvEpilogue* epi, const PdnnBackpropFusion* fusion, void* ws, size_t ws_elems, cudaStream_t s);

int run_conv(int pass, int dtype, const void* in, const void* fil, void* out, const PdnnConv2DParams* p, int algorithm,
             const PdnnConvEpilogue* epi, const PdnnBackpropFusion* fusion, void* ws, size_t ws_elems, void* stream) {
  int st = validate_conv(pass, p, algorithm);
  if (st != PDNN_OK) return st;
  if (dtype < PDNN_F32 || dtype > PDNN_BF16) return fail(PDNN_INVALID_PARAMETER, "conv2d: unknown dtype %d", dtype);
  if (in == nullptr || fil == nullptr || out == nullptr) return fail(PDNN_INVALID_PARAMETER, "conv2d: null tensor");
  if (device_sm_count() <= 0) return fail(PDNN_ALLOCATION_PROBLEM, "conv2d: no sm_100 CUDA device");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (p->input_format == 1) {
    // NCHW tensors with an FCHW filter (the only pairing validate_conv lets through): the NHWC
    // kernels between two transposes.  The reference's NCHW path is its direct kernel
    // (src/conv2d/direct/kernels_nchw.h:28,157,300), which computes the same sums.
    if (fusion != nullptr && (fusion->relu_forward_output != nullptr || fusion->relu_bitmask != nullptr || fusion->accumulate))
      return fail(PDNN_INVALID_PARAMETER, "conv2d: the fused input-backprop forms need NHWC tensors");
    if (epi != nullptr && epi->relu_bitmask != nullptr)
      return fail(PDNN_INVALID_PARAMETER, "conv2d: a ReLU bitmask needs NHWC tensors");
    const bool read_out = epi != nullptr && epi->beta != 0.f;
    return conv2d_nchw(pass, dtype, in, fil, out, *p, read_out, s,
                       [&](const void* a, const void* b, void* c, const PdnnConv2DParams& q) {
                         return dispatch_conv(pass, dtype, a, b, c, &q, PDNN_ALGO_TILED, epi, fusion, nullptr, 0, s);
                       });
  }
  return dispatch_conv(pass, dtype, in, fil, out, p, algorithm, epi, fusion, ws, ws_elems, s);
}

int dispatch_conv(int pass, int dtype, const void* in, const void* fil, void* out, const PdnnConv2DParams* p, int algorithm,
                  const PdnnConvEpilogue* epi, const PdnnBackpropFusion* fusion, void* ws, size_t ws_elems, cudaStream_t s) {
  // The Winograd tags run F(2x2,3x3) when the caller brought the scratch it needs; without it the
  // implicit-GEMM kernel, which needs none, runs the layer instead of reporting
  // InsufficientWorkspace (include/portdnn/internal/conv2d/winograd/launch.h:280).
  if ((algorithm == PDNN_ALGO_WINOGRAD || algorithm == PDNN_ALGO_WINOGRAD_LARGE) && fusion == nullptr &&
      winograd_applicable(pass, dtype, *p) && ws != nullptr && ws_elems >= winograd_workspace_elems(pass, dtype, *p) &&
      aligned16(ws) && aligned16(in) && aligned16(fil) && aligned16(out))
    return launch_winograd(pass, dtype, in, fil, out, *p, epi, ws, ws_elems, s);
  if (pass == PDNN_FORWARD && p->groups > 1 && tc_grouped_conv_supported(dtype, in, fil, out, *p) &&
      (epi == nullptr || epi->relu_bitmask == nullptr))
    return tc_grouped_conv_forward(dtype, in, fil, out, *p, epi, s);
  if (algorithm != PDNN_ALGO_DIRECT && tc_conv_supported(pass, dtype, in, fil, out, *p)) {
    const int st2 = tc_conv2d(pass, dtype, in, fil, out, *p, epi, fusion, ws, ws_elems, s);
    if (st2 != kNeedsDirect) return st2;
  }
  if (pass != PDNN_FORWARD) return run_direct_backprop(pass, dtype, in, fil, out, *p, fusion, s);
  return launch_direct_conv(pass, dtype, in, fil, out, *p, epi, s);
}

}  // namespace
}  // namespace pdnn

using namespace pdnn;

extern "C" {

int pdnn_conv2d(int pass, int dtype, const void* input, const void* filter, void* output,
                const PdnnConv2DParams* params, int algorithm, void* workspace, size_t workspace_elems, void* stream) {
  return run_conv(pass, dtype, input, filter, output, params, algorithm, nullptr, nullptr, workspace, workspace_elems,
                  stream);
}

int pdnn_conv2d_backprop_fused(int pass, int dtype, const void* input, const void* filter, void* output,
                               const PdnnConv2DParams* params, int algorithm, const PdnnBackpropFusion* fusion,
                               void* workspace, size_t workspace_elems, void* stream) {
  if (pass != PDNN_INPUT_BACKPROP && pass != PDNN_FILTER_BACKPROP)
    return fail(PDNN_INVALID_PARAMETER, "conv2d: the fused backprop forms exist for the two backprop passes only");
  if (fusion != nullptr && pass == PDNN_FILTER_BACKPROP && (fusion->relu_forward_output != nullptr || fusion->relu_bitmask != nullptr))
    return fail(PDNN_INVALID_PARAMETER, "conv2d: relu_forward_output / relu_bitmask belong to the input backprop");
  if (fusion != nullptr && fusion->relu_bitmask != nullptr &&
      (fusion->relu_forward_output != nullptr || params == nullptr || params->channels % 8 != 0 || dtype == PDNN_F32))
    return fail(PDNN_INVALID_PARAMETER,
                "conv2d: relu_bitmask stands in for relu_forward_output (16-bit tensors, a multiple of 8 channels)");
  if (fusion != nullptr && pass == PDNN_INPUT_BACKPROP && fusion->output_f32)
    return fail(PDNN_INVALID_PARAMETER, "conv2d: output_f32 belongs to the filter backprop");
  return run_conv(pass, dtype, input, filter, output, params, algorithm, nullptr, fusion, workspace, workspace_elems,
                  stream);
}

int pdnn_conv2d_fused(int dtype, const void* input, const void* filter, void* output, const PdnnConv2DParams* params,
                      int algorithm, const PdnnConvEpilogue* epilogue, void* workspace, size_t workspace_elems,
                      void* stream) {
  if (epilogue != nullptr && (epilogue->activation < PDNN_ACT_NONE || epilogue->activation > PDNN_ACT_RELU6))
    return fail(PDNN_INVALID_PARAMETER, "conv2d: unknown activation %d", epilogue->activation);
  const bool want_bits = epilogue != nullptr && epilogue->relu_bitmask != nullptr;
  if (want_bits && params != nullptr && (params->features % 8 != 0 || params->input_format != 0))
    return fail(PDNN_INVALID_PARAMETER, "conv2d: a ReLU bitmask needs NHWC tensors and a multiple of 8 features");
  bitmask_written_flag() = false;
  const int st = run_conv(PDNN_FORWARD, dtype, input, filter, output, params, algorithm, epilogue, nullptr, workspace,
                          workspace_elems, stream);
  if (st != PDNN_OK || !want_bits || bitmask_written_flag()) return st;
  // the kernel that ran has no bitmask form: one pass over the output
  return launch_relu_bitmask(dtype, output, epilogue->relu_bitmask,
                             (size_t)params->batch * params->out_rows * params->out_cols * params->features,
                             static_cast<cudaStream_t>(stream));
}

int pdnn_conv2d_validate(int pass, const PdnnConv2DParams* params, int algorithm) {
  return validate_conv(pass, params, algorithm);
}

int pdnn_conv2d_workspace_size(int pass, int dtype, const PdnnConv2DParams* params, int algorithm,
                               size_t* required_elems, size_t* recommended_elems) {
  if (required_elems) *required_elems = 0;
  if (recommended_elems) *recommended_elems = 0;
  int st = validate_conv(pass, params, algorithm);
  if (st != PDNN_OK) return st;
  if (algorithm == PDNN_ALGO_DIRECT) return PDNN_OK;
  // The implicit-GEMM kernels read the tensors in place; only the filter backprop's split
  // reduction wants scratch, and it can do without (it then allocates for the call).
  size_t elems = tc_conv_workspace_elems(pass, dtype, *params);
  // Winograd: 16 * (C*K + tiles*C + tiles*K), include/portdnn/conv2d/workspace_size.h:53-73.  It is
  // reported as recommended, not required: without it the layer still runs (on the implicit GEMM).
  if ((algorithm == PDNN_ALGO_WINOGRAD || algorithm == PDNN_ALGO_WINOGRAD_LARGE) &&
      winograd_applicable(pass, dtype, *params)) {
    const size_t w = winograd_workspace_elems(pass, dtype, *params);
    if (w > elems) elems = w;
  }
  if (recommended_elems) *recommended_elems = elems;
  return PDNN_OK;
}

int pdnn_depthwise_conv2d(int pass, int dtype, const void* input, const void* filter, void* output,
                          const PdnnDepthwiseConv2DParams* params, void* workspace, size_t workspace_bytes,
                          void* stream) {
  if (params == nullptr || input == nullptr || filter == nullptr || output == nullptr)
    return fail(PDNN_INVALID_PARAMETER, "depthwise: null argument");
  return launch_depthwise(pass, dtype, input, filter, output, *params, workspace, workspace_bytes,
                          static_cast<cudaStream_t>(stream));
}

int pdnn_depthwise_filter_backprop_noalloc(int dtype, const void* input, const void* output_grad, void* filter_grad,
                                           const PdnnDepthwiseConv2DParams* params, void* stream) {
  if (params == nullptr || input == nullptr || output_grad == nullptr || filter_grad == nullptr)
    return fail(PDNN_INVALID_PARAMETER, "depthwise: null argument");
  return launch_depthwise_filter_backprop_static(dtype, input, output_grad, filter_grad, *params,
                                                 static_cast<cudaStream_t>(stream));
}

size_t pdnn_noalloc_scratch_bytes(void) { return static_scratch_bytes(); }

size_t pdnn_depthwise_workspace_bytes(int pass, int dtype, const PdnnDepthwiseConv2DParams* params) {
  if (params == nullptr) return 0;
  return depthwise_workspace_bytes(pass, dtype, *params);
}

int pdnn_pooling(int op, int direction, int dtype, const void* input, void* output, const PdnnPoolingParams* params,
                 void* stream) {
  if (params == nullptr || input == nullptr || output == nullptr) return fail(PDNN_INVALID_PARAMETER, "pooling: null argument");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (params->input_format == 1) {  // NCHW (the reference has it for the forward pass, src/pooling/kernels.h:418-482)
    if (dtype < PDNN_F32 || dtype > PDNN_BF16) return fail(PDNN_INVALID_PARAMETER, "pooling: unknown dtype %d", dtype);
    const size_t in_px = (size_t)params->in_rows * params->in_cols, out_px = (size_t)params->out_rows * params->out_cols;
    const void* ins[1] = {input};
    const size_t rows[1] = {direction == 0 ? in_px : out_px};
    return pooling_nchw(dtype, ins, rows, 1, output, direction == 0 ? out_px : in_px, *params, s,
                        [&](const void* const* t, void* o, const PdnnPoolingParams& q) {
                          return launch_pooling(op, direction, dtype, t[0], o, q, s);
                        });
  }
  return launch_pooling(op, direction, dtype, input, output, *params, s);
}

namespace {
int run_pooling_max_grad(int op, int dtype, const void* input_data, const void* output_data, const void* input_backprop,
                         void* output_backprop, const PdnnPoolingParams* params, bool relu_input, void* stream) {
  if (params == nullptr || input_data == nullptr || output_data == nullptr || input_backprop == nullptr ||
      output_backprop == nullptr)
    return fail(PDNN_INVALID_PARAMETER, "pooling: null argument");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (params->input_format == 1) {
    if (dtype < PDNN_F32 || dtype > PDNN_BF16) return fail(PDNN_INVALID_PARAMETER, "pooling: unknown dtype %d", dtype);
    const size_t in_px = (size_t)params->in_rows * params->in_cols, out_px = (size_t)params->out_rows * params->out_cols;
    const void* ins[3] = {input_data, output_data, input_backprop};
    const size_t rows[3] = {in_px, out_px, out_px};
    return pooling_nchw(dtype, ins, rows, 3, output_backprop, in_px, *params, s,
                        [&](const void* const* t, void* o, const PdnnPoolingParams& q) {
                          return launch_pooling_max_grad(op, dtype, t[0], t[1], t[2], o, q, relu_input, s);
                        });
  }
  return launch_pooling_max_grad(op, dtype, input_data, output_data, input_backprop, output_backprop, *params, relu_input, s);
}
}  // namespace

int pdnn_pooling_max_grad(int op, int dtype, const void* input_data, const void* output_data,
                          const void* input_backprop, void* output_backprop, const PdnnPoolingParams* params,
                          void* stream) {
  return run_pooling_max_grad(op, dtype, input_data, output_data, input_backprop, output_backprop, params, false, stream);
}

int pdnn_pooling_max_grad_relu(int op, int dtype, const void* input_data, const void* output_data,
                               const void* input_backprop, void* output_backprop, const PdnnPoolingParams* params,
                               void* stream) {
  return run_pooling_max_grad(op, dtype, input_data, output_data, input_backprop, output_backprop, params, true, stream);
}

int pdnn_softmax(int direction, int dtype, const void* input, const void* gradient, void* output,
                 const PdnnSoftmaxParams* params, void* stream) {
  if (params == nullptr) return fail(PDNN_INVALID_PARAMETER, "softmax: null params");
  if (direction != 0 && direction != 1) return fail(PDNN_INVALID_PARAMETER, "softmax: direction must be 0 or 1");
  return launch_softmax(direction, dtype, input, gradient, output, *params, static_cast<cudaStream_t>(stream));
}

int pdnn_batchnorm_forward(int dtype, const void* input, const void* beta, const void* gamma, const void* mean,
                           const void* variance, void* running_mean, void* running_variance, void* output,
                           const PdnnBatchNormParams* params, void* stream) {
  if (params == nullptr) return fail(PDNN_INVALID_PARAMETER, "batchnorm: null params");
  return launch_batchnorm_forward(dtype, input, beta, gamma, mean, variance, running_mean, running_variance, output,
                                  *params, static_cast<cudaStream_t>(stream));
}

int pdnn_batchnorm_gradient(int dtype, const void* input, const void* gradient, const void* gamma,
                            const void* pop_mean, const void* pop_variance, void* beta_grad, void* gamma_grad,
                            void* output, const PdnnBatchNormParams* params, void* stream) {
  if (params == nullptr) return fail(PDNN_INVALID_PARAMETER, "batchnorm: null params");
  return launch_batchnorm_gradient(dtype, input, gradient, gamma, pop_mean, pop_variance, beta_grad, gamma_grad,
                                   output, *params, static_cast<cudaStream_t>(stream));
}

int pdnn_pointwise(int op, int dtype, const void* input, void* output, size_t n_items, void* stream) {
  if (n_items != 0 && (input == nullptr || output == nullptr)) return fail(PDNN_INVALID_PARAMETER, "pointwise: null tensor");
  return launch_pointwise(op, dtype, input, output, n_items, static_cast<cudaStream_t>(stream));
}

int pdnn_pointwise_grad(int op, int dtype, const void* output_forward, const void* input_backprop,
                        void* output_backprop, size_t n_items, void* stream) {
  if (n_items != 0 && (output_forward == nullptr || input_backprop == nullptr || output_backprop == nullptr))
    return fail(PDNN_INVALID_PARAMETER, "pointwise: null tensor");
  return launch_pointwise_grad(op, dtype, output_forward, input_backprop, output_backprop, n_items,
                               static_cast<cudaStream_t>(stream));
}

int pdnn_bias_add(int dtype, const void* input, const void* bias, void* output, size_t rows, int channels,
                  int activation, void* stream) {
  if (rows != 0 && (input == nullptr || bias == nullptr || output == nullptr))
    return fail(PDNN_INVALID_PARAMETER, "bias: null tensor");
  return launch_bias_add(dtype, input, bias, output, rows, channels, activation, static_cast<cudaStream_t>(stream));
}

int pdnn_binaryop(int op, int dtype, const void* lhs, const int* lhs_dims, int n_lhs_dims, const void* rhs,
                  const int* rhs_dims, int n_rhs_dims, void* output, void* stream) {
  if ((n_lhs_dims > 0 && lhs_dims == nullptr) || (n_rhs_dims > 0 && rhs_dims == nullptr))
    return fail(PDNN_INVALID_PARAMETER, "binaryop: null extents");
  return launch_binaryop(op, dtype, lhs, lhs_dims, n_lhs_dims, rhs, rhs_dims, n_rhs_dims, output,
                         static_cast<cudaStream_t>(stream));
}

int pdnn_scale_blend(int dtype, const void* a, float alpha, const void* b, float beta, void* out, size_t n_items,
                     void* stream) {
  if (n_items != 0 && (a == nullptr || out == nullptr || (beta != 0.f && b == nullptr)))
    return fail(PDNN_INVALID_PARAMETER, "blend: null tensor");
  return launch_scale_blend(dtype, a, alpha, b, beta, out, n_items, static_cast<cudaStream_t>(stream));
}

int pdnn_transpose(int elem_bytes, const void* input, void* output, const int* dims, int n_dims, const int* permutation,
                   void* stream) {
  if (input == nullptr || output == nullptr || dims == nullptr || permutation == nullptr)
    return fail(PDNN_INVALID_PARAMETER, "transpose: null argument");
  return launch_transpose(elem_bytes, input, output, dims, n_dims, permutation, static_cast<cudaStream_t>(stream));
}

int pdnn_matmul(int dtype, int transpose_lhs, int transpose_rhs, const void* lhs, const void* rhs, void* output,
                int batches, int m, int k, int n, float beta, void* stream) {
  if (batches <= 0 || m <= 0 || k <= 0 || n <= 0) return fail(PDNN_INVALID_PARAMETER, "matmul: sizes must be positive");
  if (lhs == nullptr || rhs == nullptr || output == nullptr) return fail(PDNN_INVALID_PARAMETER, "matmul: null tensor");
  if (dtype < PDNN_F32 || dtype > PDNN_BF16) return fail(PDNN_INVALID_PARAMETER, "matmul: unknown dtype %d", dtype);
  if (device_sm_count() <= 0) return fail(PDNN_ALLOCATION_PROBLEM, "matmul: no sm_100 CUDA device");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int tl = transpose_lhs != 0, tr = transpose_rhs != 0;
  if (tc_matmul_supported(dtype, tl, tr, lhs, rhs, output, batches, m, k, n))
    return tc_matmul(dtype, tl, tr, lhs, rhs, output, batches, m, k, n, beta, s);
  return simt_matmul(dtype, tl, tr, lhs, rhs, output, batches, m, k, n, beta, s);
}

int pdnn_device_error_record(unsigned words[4], int clear) {
  if (words == nullptr) return fail(PDNN_INVALID_PARAMETER, "null output");
  if (device_sm_count() <= 0) return fail(PDNN_ALLOCATION_PROBLEM, "no sm_100 CUDA device");
  return tc_read_error_record(words, clear);
}

const char* pdnn_last_error(void) { return last_error_buffer(); }

unsigned long long pdnn_launch_count(void) { return g_launches.load(); }

}  // extern "C"
