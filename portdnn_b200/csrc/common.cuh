// Shared host/device helpers for the sm_100a kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <functional>

#include "../../include/portdnn_b200.h"

namespace pdnn {

// ---- error text + launch counter (host) -----------------------------------------------------
char* last_error_buffer();                       // thread-local, 512 bytes
extern std::atomic<unsigned long long> g_launches;

inline int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buffer(), 512, fmt, ap);
  va_end(ap);
  return status;
}

inline void count_launch(int n = 1) { g_launches.fetch_add((unsigned long long)n, std::memory_order_relaxed); }

// Maps the error state after a launch to a status code.
inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(PDNN_ALLOCATION_PROBLEM, "%s: %s", what, cudaGetErrorString(e));
  count_launch();
  return PDNN_OK;
}

inline size_t dtype_size(int dtype) { return dtype == PDNN_F32 ? 4 : 2; }

// ---- element conversion (device) ------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// A 16-byte packet of elements: 4 floats or 8 halves/bfloat16s.
template <typename T>
struct Vec16 {
  static constexpr int N = 16 / sizeof(T);
  uint4 raw;
  __device__ __forceinline__ T get(int i) const { return reinterpret_cast<const T*>(&raw)[i]; }
  __device__ __forceinline__ void set(int i, T v) { reinterpret_cast<T*>(&raw)[i] = v; }
};

template <typename T>
__device__ __forceinline__ Vec16<T> load16(const T* p) {
  Vec16<T> v;
  v.raw = __ldg(reinterpret_cast<const uint4*>(p));
  return v;
}
template <typename T>
__device__ __forceinline__ void store16(T* p, const Vec16<T>& v) {
  *reinterpret_cast<uint4*>(p) = v.raw;
}

__device__ __forceinline__ float apply_activation(float v, int act) {
  switch (act) {
    case PDNN_ACT_RELU: return fmaxf(v, 0.f);
    case PDNN_ACT_TANH: return tanhf(v);
    case PDNN_ACT_RELU6: return fminf(fmaxf(v, 0.f), 6.f);
    default: return v;
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Grid for a grid-stride loop over `items`: enough CTAs to fill the device a few times over.
inline unsigned grid_for(size_t items, int block, int sm_count) {
  size_t need = (items + block - 1) / block;
  size_t cap = (size_t)sm_count * 32;
  if (need < 1) need = 1;
  return (unsigned)(need < cap ? need : cap);
}

// Per-device state is kept in small tables indexed by the CUDA device ordinal.
constexpr int kMaxDevices = 64;
int current_device();    // ordinal of the current device, -1 on error
int device_sm_count();   // SM count of the current device; -1 if it is not an sm_100 part

// ---- operator launchers implemented in the .cu files ------------------------------------------
int launch_pooling(int op, int direction, int dtype, const void* in, void* out, const PdnnPoolingParams& p,
                   cudaStream_t s);
int launch_pooling_max_grad(int op, int dtype, const void* x, const void* y, const void* dy, void* dx,
                            const PdnnPoolingParams& p, bool relu_input, cudaStream_t s);
int launch_depthwise(int pass, int dtype, const void* in, const void* fil, void* out,
                     const PdnnDepthwiseConv2DParams& p, void* ws, size_t ws_bytes, cudaStream_t s);
size_t depthwise_workspace_bytes(int pass, int dtype, const PdnnDepthwiseConv2DParams& p);
int launch_depthwise_filter_backprop_static(int dtype, const void* in, const void* dy, void* dw,
                                            const PdnnDepthwiseConv2DParams& p, cudaStream_t s);
size_t static_scratch_bytes();
int launch_pointwise(int op, int dtype, const void* in, void* out, size_t n, cudaStream_t s);
int launch_pointwise_grad(int op, int dtype, const void* fwd, const void* err, void* out, size_t n, cudaStream_t s);
int launch_bias_add(int dtype, const void* in, const void* bias, void* out, size_t rows, int channels, int act,
                    cudaStream_t s);
int launch_binaryop(int op, int dtype, const void* lhs, const int* lhs_dims, int n_lhs, const void* rhs,
                    const int* rhs_dims, int n_rhs, void* out, cudaStream_t s);
int launch_relu_bitmask(int dtype, const void* y, void* bits, size_t n, cudaStream_t s);
int launch_relu_grad_bits(int dtype, const void* bits, void* dx, size_t n, cudaStream_t s);
// Set by the tensor-core launch when its epilogue wrote the bitmask the caller asked for (thread-local).
bool& bitmask_written_flag();
int launch_scale_blend(int dtype, const void* a, float alpha, const void* b, float beta, void* out, size_t n,
                       cudaStream_t s);
int launch_direct_conv(int pass, int dtype, const void* in, const void* fil, void* out, const PdnnConv2DParams& p,
                       const PdnnConvEpilogue* epi, cudaStream_t s);

// Transposition and the NCHW forms built on it (layout_kernels.cu).  elem_bytes is 1, 2, 4 or 8;
// out[i_perm[0]][i_perm[1]]... = in[i_0][i_1]... with output extent d = dims[perm[d]].
int launch_transpose(int elem_bytes, const void* in, void* out, const int* dims, int n_dims, const int* perm,
                     cudaStream_t s);
// Runs `run` on NHWC / HWCF copies of the NCHW / FCHW tensors of a convolution pass and brings the
// result back; read_out: the previous contents of `out` are needed (a beta blend).
using ConvRunner = std::function<int(const void* in, const void* fil, void* out, const PdnnConv2DParams& nhwc_params)>;
int conv2d_nchw(int pass, int dtype, const void* in, const void* fil, void* out, const PdnnConv2DParams& p, bool read_out,
                cudaStream_t s, const ConvRunner& run);
// The same for pooling: n_inputs tensors of input_rows[i] spatial positions per (image, channel).
using PoolRunner = std::function<int(const void* const* nhwc_inputs, void* nhwc_out, const PdnnPoolingParams& nhwc_params)>;
int pooling_nchw(int dtype, const void* const* inputs, const size_t* input_rows, int n_inputs, void* out, size_t out_rows,
                 const PdnnPoolingParams& p, cudaStream_t s, const PoolRunner& run);

// softmax and batchnorm (norm_kernels.cu)
int launch_softmax(int direction, int dtype, const void* input, const void* gradient, void* output,
                   const PdnnSoftmaxParams& p, cudaStream_t s);
int launch_batchnorm_forward(int dtype, const void* input, const void* beta, const void* gamma, const void* mean,
                             const void* variance, void* running_mean, void* running_variance, void* output,
                             const PdnnBatchNormParams& p, cudaStream_t s);
int launch_batchnorm_gradient(int dtype, const void* input, const void* gradient, const void* gamma,
                              const void* pop_mean, const void* pop_variance, void* beta_grad, void* gamma_grad,
                              void* output, const PdnnBatchNormParams& p, cudaStream_t s);

// Winograd F(2x2,3x3) (winograd.cu): forward and input backprop of 3x3 stride-1 layers.
bool winograd_applicable(int pass, int dtype, const PdnnConv2DParams& p);
size_t winograd_workspace_elems(int pass, int dtype, const PdnnConv2DParams& p);
int launch_winograd(int pass, int dtype, const void* in, const void* fil, void* out, const PdnnConv2DParams& p,
                    const PdnnConvEpilogue* epi, void* ws, size_t ws_elems, cudaStream_t s);

}  // namespace pdnn
