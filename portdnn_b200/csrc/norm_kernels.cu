// Softmax and batchnorm (NHWC): the operators the reference's network wrappers need beside the
// convolution path (tools/layer.h:128-205, 284-310).  HBM-bound; arithmetic in fp32, one rounding on
// store.  The reference composes both from reduce / binaryop / pointwise launches
// (include/portdnn/internal/softmax/launch_internal.h:45-275,
// include/portdnn/internal/batchnorm/launch_internal.h:95-640); here each is one to three kernels.
#include "common.cuh"

namespace pdnn {
namespace {

constexpr int kBlock = 256;

template <typename F>
int dispatch(int dtype, F&& f) {
  switch (dtype) {
    case PDNN_F32: return f(float{});
    case PDNN_F16: return f(__half{});
    case PDNN_BF16: return f(__nv_bfloat16{});
  }
  return fail(PDNN_INVALID_PARAMETER, "unknown dtype %d", dtype);
}

__device__ __forceinline__ float warp_max(float v) {
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}

// V consecutive elements as floats (one 16-byte access when V > 1).
template <typename T, int V>
__device__ __forceinline__ void load_v(const T* p, float (&v)[V]) {
  if constexpr (V == 1) {
    v[0] = to_f32(__ldg(p));
  } else {
    const Vec16<T> pk = load16(p);
#pragma unroll
    for (int i = 0; i < V; ++i) v[i] = to_f32(pk.get(i));
  }
}
template <typename T, int V>
__device__ __forceinline__ void store_v(T* p, const float (&v)[V]) {
  if constexpr (V == 1) {
    p[0] = from_f32<T>(v[0]);
  } else {
    Vec16<T> pk;
#pragma unroll
    for (int i = 0; i < V; ++i) pk.set(i, from_f32<T>(v[i]));
    store16(p, pk);
  }
}

// One warp per pixel, packets of V channels, at most R packets per lane (C <= 32 * R * V): the
// pixel is read once and stays in registers through the three steps.
template <typename T, int V, int R>
__global__ void __launch_bounds__(kBlock) softmax_forward_vec_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                                     size_t rows, int C) {
  const int lane = threadIdx.x & 31, packets = C / V;
  const size_t warps = (size_t)gridDim.x * (kBlock / 32);
  for (size_t row = (size_t)blockIdx.x * (kBlock / 32) + (threadIdx.x >> 5); row < rows; row += warps) {
    const T* xr = x + row * C;
    float v[R][V];
    float m = -INFINITY;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int pk = lane + 32 * r;
      if (pk < packets) {
        load_v<T, V>(xr + pk * V, v[r]);
#pragma unroll
        for (int k = 0; k < V; ++k) m = fmaxf(m, v[r][k]);
      }
    }
    m = warp_max(m);
    float sum = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r)
      if (lane + 32 * r < packets) {
#pragma unroll
        for (int k = 0; k < V; ++k) {
          v[r][k] = expf(v[r][k] - m);
          sum += v[r][k];
        }
      }
    sum = warp_sum(sum);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int pk = lane + 32 * r;
      if (pk < packets) {
#pragma unroll
        for (int k = 0; k < V; ++k) v[r][k] = v[r][k] / sum;
        store_v<T, V>(y + row * C + pk * V, v[r]);
      }
    }
  }
}

// One warp per pixel: y = exp(x - max) / sum exp(x - max) over the pixel's C channels.
template <typename T>
__global__ void __launch_bounds__(kBlock) softmax_forward_kernel(const T* __restrict__ x, T* __restrict__ y, size_t rows,
                                                                 int C) {
  const int lane = threadIdx.x & 31;
  const size_t warps = (size_t)gridDim.x * (kBlock / 32);
  for (size_t row = (size_t)blockIdx.x * (kBlock / 32) + (threadIdx.x >> 5); row < rows; row += warps) {
    const T* xr = x + row * C;
    T* yr = y + row * C;
    float m = -INFINITY;
    for (int c = lane; c < C; c += 32) m = fmaxf(m, to_f32(xr[c]));
    m = warp_max(m);
    float sum = 0.f;
    for (int c = lane; c < C; c += 32) sum += expf(to_f32(xr[c]) - m);
    sum = warp_sum(sum);
    for (int c = lane; c < C; c += 32) yr[c] = from_f32<T>(expf(to_f32(xr[c]) - m) / sum);
  }
}

// dx = (dy - sum_c(dy * y)) * y, y = the forward output.
template <typename T>
__global__ void __launch_bounds__(kBlock) softmax_grad_kernel(const T* __restrict__ y, const T* __restrict__ dy,
                                                              T* __restrict__ dx, size_t rows, int C) {
  const int lane = threadIdx.x & 31;
  const size_t warps = (size_t)gridDim.x * (kBlock / 32);
  for (size_t row = (size_t)blockIdx.x * (kBlock / 32) + (threadIdx.x >> 5); row < rows; row += warps) {
    const T* yr = y + row * C;
    const T* gr = dy + row * C;
    float sum = 0.f;
    for (int c = lane; c < C; c += 32) sum += to_f32(gr[c]) * to_f32(yr[c]);
    sum = warp_sum(sum);
    for (int c = lane; c < C; c += 32) dx[row * C + c] = from_f32<T>((to_f32(gr[c]) - sum) * to_f32(yr[c]));
  }
}

// The elementwise steps on packets of V channels (C % V == 0, 16-byte aligned tensors): n counts
// packets.  The per-channel operands are read as packets too (they stay in L1).
template <typename T, int V>
__global__ void __launch_bounds__(kBlock)
    batchnorm_apply_vec_kernel(const T* __restrict__ x, const T* __restrict__ beta, const T* __restrict__ gamma,
                               const T* __restrict__ mean, const T* __restrict__ var, T* __restrict__ out, size_t n,
                               int C, float eps) {
  const size_t cvecs = (size_t)(C / V);
  const size_t step = (size_t)gridDim.x * kBlock;
  size_t i = (size_t)blockIdx.x * kBlock + threadIdx.x;
  if (step % cvecs == 0) {
    // every packet of this thread belongs to the same channels (the host sizes the grid for
    // this): the per-channel operands and the square root are taken once
    if (i >= n) return;
    const int c = (int)(i % cvecs) * V;
    float b[V], g[V], m[V], sd[V];
    load_v<T, V>(beta + c, b);
    load_v<T, V>(gamma + c, g);
    load_v<T, V>(mean + c, m);
    load_v<T, V>(var + c, sd);
    // 1 / sqrt(var + eps) once per channel: the division per element would make the kernel
    // instruction-bound; the product differs from the quotient by at most one ulp of fp32
#pragma unroll
    for (int k = 0; k < V; ++k) sd[k] = 1.f / sqrtf(sd[k] + eps);
    for (; i < n; i += step) {
      float xv[V], o[V];
      load_v<T, V>(x + i * V, xv);
#pragma unroll
      for (int k = 0; k < V; ++k) o[k] = (xv[k] - m[k]) * sd[k] * g[k] + b[k];
      store_v<T, V>(out + i * V, o);
    }
    return;
  }
  for (; i < n; i += step) {
    const int c = (int)(i % cvecs) * V;
    float xv[V], b[V], g[V], m[V], v[V], o[V];
    load_v<T, V>(x + i * V, xv);
    load_v<T, V>(beta + c, b);
    load_v<T, V>(gamma + c, g);
    load_v<T, V>(mean + c, m);
    load_v<T, V>(var + c, v);
#pragma unroll
    for (int k = 0; k < V; ++k) o[k] = (xv[k] - m[k]) / sqrtf(v[k] + eps) * g[k] + b[k];
    store_v<T, V>(out + i * V, o);
  }
}

template <typename T, int V>
__global__ void __launch_bounds__(kBlock)
    batchnorm_grad_training_vec_kernel(const T* __restrict__ x, const T* __restrict__ dy, const T* __restrict__ gamma,
                                       const float* __restrict__ stats0, const float* __restrict__ stats1,
                                       T* __restrict__ out, size_t n, int C, float rows, float eps) {
  const size_t cvecs = (size_t)(C / V);
  const size_t step = (size_t)gridDim.x * kBlock;
  size_t i = (size_t)blockIdx.x * kBlock + threadIdx.x;
  if (step % cvecs == 0) {  // the thread's channels never change: per-channel terms taken once
    if (i >= n) return;
    const int c = (int)(i % cvecs) * V;
    float g[V], mx[V], mdy[V], kk[V], sd[V];
    load_v<T, V>(gamma + c, g);
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const float v = stats1[c + k] + eps;
      sd[k] = sqrtf(v);
      kk[k] = stats1[C + c + k] / rows / v;
      mx[k] = stats0[c + k];
      mdy[k] = stats0[C + c + k];
    }
    for (; i < n; i += step) {
      float xv[V], gv[V], o[V];
      load_v<T, V>(x + i * V, xv);
      load_v<T, V>(dy + i * V, gv);
#pragma unroll
      for (int k = 0; k < V; ++k) o[k] = ((gv[k] - mdy[k]) - (xv[k] - mx[k]) * kk[k]) * g[k] / sd[k];
      store_v<T, V>(out + i * V, o);
    }
    return;
  }
  for (; i < n; i += step) {
    const int c = (int)(i % cvecs) * V;
    float xv[V], gv[V], g[V], o[V];
    load_v<T, V>(x + i * V, xv);
    load_v<T, V>(dy + i * V, gv);
    load_v<T, V>(gamma + c, g);
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const float v = stats1[c + k] + eps, sd = sqrtf(v);
      const float kk = stats1[C + c + k] / rows / v;
      o[k] = ((gv[k] - stats0[C + c + k]) - (xv[k] - stats0[c + k]) * kk) * g[k] / sd;
    }
    store_v<T, V>(out + i * V, o);
  }
}

template <typename T, int V>
__global__ void __launch_bounds__(kBlock)
    batchnorm_grad_frozen_vec_kernel(const T* __restrict__ dy, const T* __restrict__ gamma,
                                     const T* __restrict__ pop_var, T* __restrict__ out, size_t n, int C, float eps) {
  const size_t cvecs = (size_t)(C / V);
  const size_t step = (size_t)gridDim.x * kBlock;
  size_t i = (size_t)blockIdx.x * kBlock + threadIdx.x;
  if (step % cvecs == 0) {  // the thread's channels never change: scale taken once
    if (i >= n) return;
    const int c = (int)(i % cvecs) * V;
    float g[V], v[V];
    load_v<T, V>(gamma + c, g);
    load_v<T, V>(pop_var + c, v);
#pragma unroll
    for (int k = 0; k < V; ++k) g[k] = g[k] / sqrtf(v[k] + eps);
    for (; i < n; i += step) {
      float gv[V], o[V];
      load_v<T, V>(dy + i * V, gv);
#pragma unroll
      for (int k = 0; k < V; ++k) o[k] = gv[k] * g[k];
      store_v<T, V>(out + i * V, o);
    }
    return;
  }
  for (; i < n; i += step) {
    const int c = (int)(i % cvecs) * V;
    float gv[V], g[V], v[V], o[V];
    load_v<T, V>(dy + i * V, gv);
    load_v<T, V>(gamma + c, g);
    load_v<T, V>(pop_var + c, v);
#pragma unroll
    for (int k = 0; k < V; ++k) o[k] = gv[k] * (g[k] / sqrtf(v[k] + eps));
    store_v<T, V>(out + i * V, o);
  }
}

// The sums kernel on packets: lane tx of the block owns V channels; 32 lanes x 8 row lanes.
template <typename T, int V, int MODE>
__global__ void __launch_bounds__(kBlock)
    batchnorm_sums_vec_kernel(const T* __restrict__ x, const T* __restrict__ dy, const float* __restrict__ shift,
                              const float* __restrict__ scale, float* __restrict__ partial, size_t rows, int C,
                              size_t rows_per_slice) {
  __shared__ float red[2][8][32][V];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c = (blockIdx.y * 32 + tx) * V;
  const size_t begin = (size_t)blockIdx.x * rows_per_slice;
  const size_t end = begin + rows_per_slice < rows ? begin + rows_per_slice : rows;
  float a[V], b[V], sh[V], sc[V];
#pragma unroll
  for (int k = 0; k < V; ++k) a[k] = b[k] = 0.f, sh[k] = 0.f, sc[k] = 1.f;
  if (c < C) {
#pragma unroll
    for (int k = 0; k < V; ++k) {
      if (MODE != 0) sh[k] = shift[c + k];
      if (MODE == 2) sc[k] = scale[c + k];
    }
    for (size_t r = begin + ty; r < end; r += 8) {
      float xv[V], gv[V];
      load_v<T, V>(x + r * C + c, xv);
      if (dy != nullptr) {
        load_v<T, V>(dy + r * C + c, gv);
      } else {
#pragma unroll
        for (int k = 0; k < V; ++k) gv[k] = 0.f;
      }
#pragma unroll
      for (int k = 0; k < V; ++k) {
        if (MODE == 0) {
          a[k] += xv[k];
          b[k] += gv[k];
        } else if (MODE == 1) {
          const float d = xv[k] - sh[k];
          a[k] += d * d;
          b[k] += gv[k] * d;
        } else {
          a[k] += gv[k];
          b[k] += (xv[k] - sh[k]) * gv[k] / sc[k];
        }
      }
    }
  }
#pragma unroll
  for (int k = 0; k < V; ++k) {
    red[0][ty][tx][k] = a[k];
    red[1][ty][tx][k] = b[k];
  }
  __syncthreads();
  if (ty < 2 && c < C) {
#pragma unroll
    for (int k = 0; k < V; ++k) {
      float sum = 0.f;
#pragma unroll
      for (int l = 0; l < 8; ++l) sum += red[ty][l][tx][k];
      partial[((size_t)blockIdx.x * 2 + ty) * C + c + k] = sum;
    }
  }
}

// out = (x - mean[c]) / sqrt(var[c] + eps) * gamma[c] + beta[c]
template <typename T>
__global__ void __launch_bounds__(kBlock)
    batchnorm_apply_kernel(const T* __restrict__ x, const T* __restrict__ beta, const T* __restrict__ gamma,
                           const T* __restrict__ mean, const T* __restrict__ var, T* __restrict__ out, size_t n, int C,
                           float eps) {
  for (size_t i = (size_t)blockIdx.x * kBlock + threadIdx.x; i < n; i += (size_t)gridDim.x * kBlock) {
    const int c = (int)(i % C);
    const float v = (to_f32(x[i]) - to_f32(mean[c])) / sqrtf(to_f32(var[c]) + eps) * to_f32(gamma[c]) + to_f32(beta[c]);
    out[i] = from_f32<T>(v);
  }
}

// Per-channel sums over the rows of one slice: partial[slice][0][c], partial[slice][1][c].
//   MODE 0: sum x,                 sum dy
//   MODE 1: sum (x - shift)^2,     sum dy * (x - shift)         shift = per-channel float
//   MODE 2: sum dy,                sum (x - shift) * dy / scale shift, scale = per-channel float
// dy may be NULL (its sums are then zero).  Block: 32 channel lanes x 8 row lanes.
template <typename T, int MODE>
__global__ void __launch_bounds__(kBlock)
    batchnorm_sums_kernel(const T* __restrict__ x, const T* __restrict__ dy, const float* __restrict__ shift,
                          const float* __restrict__ scale, float* __restrict__ partial, size_t rows, int C,
                          size_t rows_per_slice) {
  __shared__ float red[2][8][32];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c = blockIdx.y * 32 + tx;
  const size_t begin = (size_t)blockIdx.x * rows_per_slice;
  const size_t end = begin + rows_per_slice < rows ? begin + rows_per_slice : rows;
  float a = 0.f, b = 0.f;
  if (c < C) {
    const float sh = MODE == 0 ? 0.f : shift[c];
    const float sc = MODE == 2 ? scale[c] : 1.f;
    for (size_t r = begin + ty; r < end; r += 8) {
      const float xv = to_f32(x[r * C + c]);
      const float gv = dy != nullptr ? to_f32(dy[r * C + c]) : 0.f;
      if (MODE == 0) {
        a += xv;
        b += gv;
      } else if (MODE == 1) {
        const float d = xv - sh;
        a += d * d;
        b += gv * d;
      } else {
        a += gv;
        b += (xv - sh) * gv / sc;
      }
    }
  }
  red[0][ty][tx] = a;
  red[1][ty][tx] = b;
  __syncthreads();
  if (ty < 2 && c < C) {
    float sum = 0.f;
#pragma unroll
    for (int l = 0; l < 8; ++l) sum += red[ty][l][tx];
    partial[((size_t)blockIdx.x * 2 + ty) * C + c] = sum;
  }
}

// totals[k][c] = sum over slices of partial[slice][k][c], optionally divided by `divide_by`.
__global__ void __launch_bounds__(kBlock)
    batchnorm_totals_kernel(const float* __restrict__ partial, float* __restrict__ totals, int slices, int C,
                            float divide0, float divide1) {
  const int i = blockIdx.x * kBlock + threadIdx.x;
  if (i >= 2 * C) return;
  const int k = i / C, c = i % C;
  float sum = 0.f;
  for (int s = 0; s < slices; ++s) sum += partial[((size_t)s * 2 + k) * C + c];
  totals[i] = sum / (k == 0 ? divide0 : divide1);
}

// Training forward, last step: running = batch * (1 - m) + given * m.
template <typename T>
__global__ void __launch_bounds__(kBlock)
    batchnorm_running_kernel(const float* __restrict__ batch_mean, const float* __restrict__ batch_var,
                             const T* __restrict__ mean, const T* __restrict__ var, T* __restrict__ run_mean,
                             T* __restrict__ run_var, int C, float momentum) {
  const int c = blockIdx.x * kBlock + threadIdx.x;
  if (c >= C) return;
  run_mean[c] = from_f32<T>(batch_mean[c] * (1.f - momentum) + to_f32(mean[c]) * momentum);
  run_var[c] = from_f32<T>(batch_var[c] * (1.f - momentum) + to_f32(var[c]) * momentum);
}

// Training gradient, elementwise step.  stats0 = [mean x | mean dy], stats1 = [var | sum dy * xc].
template <typename T>
__global__ void __launch_bounds__(kBlock)
    batchnorm_grad_training_kernel(const T* __restrict__ x, const T* __restrict__ dy, const T* __restrict__ gamma,
                                   const float* __restrict__ stats0, const float* __restrict__ stats1,
                                   T* __restrict__ out, size_t n, int C, float rows, float eps) {
  for (size_t i = (size_t)blockIdx.x * kBlock + threadIdx.x; i < n; i += (size_t)gridDim.x * kBlock) {
    const int c = (int)(i % C);
    const float v = stats1[c] + eps, sd = sqrtf(v);
    const float k = stats1[C + c] / rows / v;
    const float d = to_f32(x[i]) - stats0[c];
    out[i] = from_f32<T>(((to_f32(dy[i]) - stats0[C + c]) - d * k) * to_f32(gamma[c]) / sd);
  }
}

// Per-channel results of the gradients.  Training: beta_grad = mean dy * rows, gamma_grad =
// sum(dy * xc) / sqrt(var + eps).  Frozen: the two sums as they are.
template <typename T>
__global__ void __launch_bounds__(kBlock)
    batchnorm_param_grads_kernel(const float* __restrict__ stats0, const float* __restrict__ stats1,
                                 T* __restrict__ beta_grad, T* __restrict__ gamma_grad, int C, float rows, float eps,
                                 int training) {
  const int c = blockIdx.x * kBlock + threadIdx.x;
  if (c >= C) return;
  if (training) {
    beta_grad[c] = from_f32<T>(stats0[C + c] * rows);
    gamma_grad[c] = from_f32<T>(stats1[C + c] / sqrtf(stats1[c] + eps));
  } else {
    beta_grad[c] = from_f32<T>(stats0[c]);
    gamma_grad[c] = from_f32<T>(stats0[C + c]);
  }
}

// Frozen gradient, elementwise step: out = dy * gamma / sqrt(pop_var + eps).
template <typename T>
__global__ void __launch_bounds__(kBlock)
    batchnorm_grad_frozen_kernel(const T* __restrict__ dy, const T* __restrict__ gamma, const T* __restrict__ pop_var,
                                 T* __restrict__ out, size_t n, int C, float eps) {
  for (size_t i = (size_t)blockIdx.x * kBlock + threadIdx.x; i < n; i += (size_t)gridDim.x * kBlock) {
    const int c = (int)(i % C);
    out[i] = from_f32<T>(to_f32(dy[i]) * (to_f32(gamma[c]) / sqrtf(to_f32(pop_var[c]) + eps)));
  }
}

// Channel vectors of T as float (shift / scale operands of the sums kernel).
template <typename T>
__global__ void __launch_bounds__(kBlock)
    batchnorm_prepare_frozen_kernel(const T* __restrict__ pop_mean, const T* __restrict__ pop_var,
                                    float* __restrict__ shift, float* __restrict__ scale, int C, float eps) {
  const int c = blockIdx.x * kBlock + threadIdx.x;
  if (c >= C) return;
  shift[c] = to_f32(pop_mean[c]);
  scale[c] = sqrtf(to_f32(pop_var[c]) + eps);
}

// Row slices of the per-channel reductions: enough blocks to fill the device a few times over
// (a block covers `block_channels` channels), at least 64 rows per slice.
int slices_for(size_t rows, int C, int sms, int block_channels) {
  const size_t ctiles = (size_t)(C + block_channels - 1) / block_channels;
  size_t want = ((size_t)sms * 8 + ctiles - 1) / ctiles;
  const size_t cap = (rows + 63) / 64;
  if (want > cap) want = cap;
  if (want < 1) want = 1;
  if (want > 4096) want = 4096;
  return (int)want;
}

// Grid of an elementwise packet kernel whose threads should keep their channels: the number of
// threads is made a multiple of the packets per pixel when that costs little.
unsigned channel_stable_grid(size_t packets, int cvecs, int sms) {
  unsigned grid = grid_for(packets, kBlock, sms);
  // threads = grid * kBlock must be a multiple of cvecs: grid a multiple of cvecs / gcd(cvecs, kBlock)
  int a = cvecs, b = kBlock;
  while (b != 0) {
    const int t = a % b;
    a = b;
    b = t;
  }
  const unsigned unit = (unsigned)(cvecs / a);
  if (unit > 1 && grid > 4 * unit) grid -= grid % unit;
  return grid;
}

bool params_ok(int batch, int rows, int cols, int channels) { return batch > 0 && rows > 0 && cols > 0 && channels > 0; }

// Scratch of one call: [partial: slices * 2 * C][stats0: 2C][stats1: 2C][shift: C][scale: C] floats.
struct Scratch {
  float *partial, *stats0, *stats1, *shift, *scale;
  void* base;
};

int get_scratch(Scratch* sc, int slices, int C, cudaStream_t s) {
  const size_t floats = (size_t)slices * 2 * C + 6 * (size_t)C;
  if (cudaMallocAsync(&sc->base, floats * sizeof(float), s) != cudaSuccess) {
    cudaGetLastError();
    return fail(PDNN_ALLOCATION_PROBLEM, "batchnorm: cannot allocate %zu bytes of scratch", floats * sizeof(float));
  }
  sc->partial = static_cast<float*>(sc->base);
  sc->stats0 = sc->partial + (size_t)slices * 2 * C;
  sc->stats1 = sc->stats0 + 2 * C;
  sc->shift = sc->stats1 + 2 * C;
  sc->scale = sc->shift + C;
  return PDNN_OK;
}

}  // namespace

int launch_softmax(int direction, int dtype, const void* input, const void* gradient, void* output,
                   const PdnnSoftmaxParams& p, cudaStream_t s) {
  // validate_params, include/portdnn/softmax/launch.h:40-50
  if (!params_ok(p.batch, p.rows, p.cols, p.channels))
    return fail(PDNN_INVALID_PARAMETER, "softmax: batch, rows, cols and channels must be positive");
  if (p.input_format != 0) return fail(PDNN_INVALID_PARAMETER, "softmax: only NHWC is implemented");
  if (input == nullptr || output == nullptr || (direction == 1 && gradient == nullptr))
    return fail(PDNN_INVALID_PARAMETER, "softmax: null tensor");
  const int sms = device_sm_count();
  if (sms <= 0) return fail(PDNN_ALLOCATION_PROBLEM, "no CUDA device");
  const size_t rows = (size_t)p.batch * p.rows * p.cols;
  const unsigned grid = grid_for(rows * 32, kBlock, sms);
  return dispatch(dtype, [&](auto tag) {
    using T = decltype(tag);
    constexpr int VN = Vec16<T>::N;
    const bool vec = p.channels % VN == 0 && aligned16(input) && aligned16(output);
    if (direction == 0 && vec && p.channels <= 32 * VN)
      softmax_forward_vec_kernel<T, VN, 1><<<grid, kBlock, 0, s>>>(static_cast<const T*>(input),
                                                                  static_cast<T*>(output), rows, p.channels);
    else if (direction == 0 && vec && p.channels <= 128 * VN)
      softmax_forward_vec_kernel<T, VN, 4><<<grid, kBlock, 0, s>>>(static_cast<const T*>(input),
                                                                  static_cast<T*>(output), rows, p.channels);
    else if (direction == 0)
      softmax_forward_kernel<T><<<grid, kBlock, 0, s>>>(static_cast<const T*>(input), static_cast<T*>(output), rows,
                                                        p.channels);
    else
      softmax_grad_kernel<T><<<grid, kBlock, 0, s>>>(static_cast<const T*>(input), static_cast<const T*>(gradient),
                                                     static_cast<T*>(output), rows, p.channels);
    return check_launch(direction == 0 ? "softmax forward" : "softmax gradient");
  });
}

int launch_batchnorm_forward(int dtype, const void* input, const void* beta, const void* gamma, const void* mean,
                             const void* variance, void* running_mean, void* running_variance, void* output,
                             const PdnnBatchNormParams& p, cudaStream_t s) {
  if (!params_ok(p.batch, p.rows, p.cols, p.channels))
    return fail(PDNN_INVALID_PARAMETER, "batchnorm: batch, rows, cols and channels must be positive");
  if (p.input_format != 0) return fail(PDNN_INVALID_PARAMETER, "batchnorm: only NHWC is implemented");
  if (!(p.epsilon > 0.f)) return fail(PDNN_INVALID_PARAMETER, "batchnorm: epsilon must be positive");
  if (input == nullptr || beta == nullptr || gamma == nullptr || mean == nullptr || variance == nullptr ||
      output == nullptr || (p.is_training && (running_mean == nullptr || running_variance == nullptr)))
    return fail(PDNN_INVALID_PARAMETER, "batchnorm: null tensor");
  const int sms = device_sm_count();
  if (sms <= 0) return fail(PDNN_ALLOCATION_PROBLEM, "no CUDA device");
  const size_t rows = (size_t)p.batch * p.rows * p.cols, n = rows * p.channels;
  const int C = p.channels;
  return dispatch(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    constexpr int VN = Vec16<T>::N;
    const bool vec = C % VN == 0 && aligned16(input) && aligned16(output) && aligned16(beta) && aligned16(gamma) &&
                     aligned16(mean) && aligned16(variance);
    if (vec)
      batchnorm_apply_vec_kernel<T, VN><<<channel_stable_grid(n / VN, C / VN, sms), kBlock, 0, s>>>(
          static_cast<const T*>(input), static_cast<const T*>(beta), static_cast<const T*>(gamma),
          static_cast<const T*>(mean), static_cast<const T*>(variance), static_cast<T*>(output), n / VN, C, p.epsilon);
    else
      batchnorm_apply_kernel<T><<<grid_for(n, kBlock, sms), kBlock, 0, s>>>(
          static_cast<const T*>(input), static_cast<const T*>(beta), static_cast<const T*>(gamma),
          static_cast<const T*>(mean), static_cast<const T*>(variance), static_cast<T*>(output), n, C, p.epsilon);
    int st = check_launch("batchnorm forward");
    if (st != PDNN_OK || !p.is_training) return st;
    // batch mean, then the biased batch variance around it, then the running statistics
    const int slices = slices_for(rows, C, sms, vec ? 32 * VN : 32);
    const size_t per_slice = (rows + slices - 1) / slices;
    Scratch sc;
    st = get_scratch(&sc, slices, C, s);
    if (st != PDNN_OK) return st;
    const dim3 grid(slices, (C + 31) / 32), vgrid(slices, (C / VN + 31) / 32);
    const unsigned cgrid = (2 * C + kBlock - 1) / kBlock;
    if (vec)
      batchnorm_sums_vec_kernel<T, VN, 0><<<vgrid, kBlock, 0, s>>>(static_cast<const T*>(input), nullptr, nullptr,
                                                                  nullptr, sc.partial, rows, C, per_slice);
    else
      batchnorm_sums_kernel<T, 0><<<grid, kBlock, 0, s>>>(static_cast<const T*>(input), nullptr, nullptr, nullptr,
                                                         sc.partial, rows, C, per_slice);
    batchnorm_totals_kernel<<<cgrid, kBlock, 0, s>>>(sc.partial, sc.stats0, slices, C, (float)rows, (float)rows);
    if (vec)
      batchnorm_sums_vec_kernel<T, VN, 1><<<vgrid, kBlock, 0, s>>>(static_cast<const T*>(input), nullptr, sc.stats0,
                                                                  nullptr, sc.partial, rows, C, per_slice);
    else
      batchnorm_sums_kernel<T, 1><<<grid, kBlock, 0, s>>>(static_cast<const T*>(input), nullptr, sc.stats0, nullptr,
                                                         sc.partial, rows, C, per_slice);
    batchnorm_totals_kernel<<<cgrid, kBlock, 0, s>>>(sc.partial, sc.stats1, slices, C, (float)rows, 1.f);
    batchnorm_running_kernel<T><<<(C + kBlock - 1) / kBlock, kBlock, 0, s>>>(
        sc.stats0, sc.stats1, static_cast<const T*>(mean), static_cast<const T*>(variance),
        static_cast<T*>(running_mean), static_cast<T*>(running_variance), C, p.momentum);
    st = check_launch("batchnorm forward (batch statistics)");
    count_launch(4);
    cudaFreeAsync(sc.base, s);
    return st;
  });
}

int launch_batchnorm_gradient(int dtype, const void* input, const void* gradient, const void* gamma,
                              const void* pop_mean, const void* pop_variance, void* beta_grad, void* gamma_grad,
                              void* output, const PdnnBatchNormParams& p, cudaStream_t s) {
  if (!params_ok(p.batch, p.rows, p.cols, p.channels))
    return fail(PDNN_INVALID_PARAMETER, "batchnorm: batch, rows, cols and channels must be positive");
  if (p.input_format != 0) return fail(PDNN_INVALID_PARAMETER, "batchnorm: only NHWC is implemented");
  if (!(p.epsilon > 0.f)) return fail(PDNN_INVALID_PARAMETER, "batchnorm: epsilon must be positive");
  if (input == nullptr || gradient == nullptr || gamma == nullptr || beta_grad == nullptr || gamma_grad == nullptr ||
      output == nullptr || (!p.is_training && (pop_mean == nullptr || pop_variance == nullptr)))
    return fail(PDNN_INVALID_PARAMETER, "batchnorm gradient: null tensor");
  const int sms = device_sm_count();
  if (sms <= 0) return fail(PDNN_ALLOCATION_PROBLEM, "no CUDA device");
  const size_t rows = (size_t)p.batch * p.rows * p.cols, n = rows * p.channels;
  const int C = p.channels;
  return dispatch(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    constexpr int VN = Vec16<T>::N;
    const bool vec = C % VN == 0 && aligned16(input) && aligned16(gradient) && aligned16(output) && aligned16(gamma) &&
                     (p.is_training || aligned16(pop_variance));
    const int slices = slices_for(rows, C, sms, vec ? 32 * VN : 32);
    const size_t per_slice = (rows + slices - 1) / slices;
    Scratch sc;
    int st = get_scratch(&sc, slices, C, s);
    if (st != PDNN_OK) return st;
    const dim3 grid(slices, (C + 31) / 32), vgrid(slices, (C / VN + 31) / 32);
    const unsigned cgrid = (2 * C + kBlock - 1) / kBlock, c1grid = (C + kBlock - 1) / kBlock;
    const T *x = static_cast<const T*>(input), *dy = static_cast<const T*>(gradient), *g = static_cast<const T*>(gamma);
    if (p.is_training) {
      if (vec) batchnorm_sums_vec_kernel<T, VN, 0><<<vgrid, kBlock, 0, s>>>(x, dy, nullptr, nullptr, sc.partial, rows, C, per_slice);
      else batchnorm_sums_kernel<T, 0><<<grid, kBlock, 0, s>>>(x, dy, nullptr, nullptr, sc.partial, rows, C, per_slice);
      batchnorm_totals_kernel<<<cgrid, kBlock, 0, s>>>(sc.partial, sc.stats0, slices, C, (float)rows, (float)rows);
      if (vec) batchnorm_sums_vec_kernel<T, VN, 1><<<vgrid, kBlock, 0, s>>>(x, dy, sc.stats0, nullptr, sc.partial, rows, C, per_slice);
      else batchnorm_sums_kernel<T, 1><<<grid, kBlock, 0, s>>>(x, dy, sc.stats0, nullptr, sc.partial, rows, C, per_slice);
      batchnorm_totals_kernel<<<cgrid, kBlock, 0, s>>>(sc.partial, sc.stats1, slices, C, (float)rows, 1.f);
      if (vec)
        batchnorm_grad_training_vec_kernel<T, VN><<<channel_stable_grid(n / VN, C / VN, sms), kBlock, 0, s>>>(
            x, dy, g, sc.stats0, sc.stats1, static_cast<T*>(output), n / VN, C, (float)rows, p.epsilon);
      else
        batchnorm_grad_training_kernel<T><<<grid_for(n, kBlock, sms), kBlock, 0, s>>>(
            x, dy, g, sc.stats0, sc.stats1, static_cast<T*>(output), n, C, (float)rows, p.epsilon);
      count_launch(4);
    } else {
      batchnorm_prepare_frozen_kernel<T><<<c1grid, kBlock, 0, s>>>(static_cast<const T*>(pop_mean),
                                                                 static_cast<const T*>(pop_variance), sc.shift, sc.scale,
                                                                 C, p.epsilon);
      if (vec) batchnorm_sums_vec_kernel<T, VN, 2><<<vgrid, kBlock, 0, s>>>(x, dy, sc.shift, sc.scale, sc.partial, rows, C, per_slice);
      else batchnorm_sums_kernel<T, 2><<<grid, kBlock, 0, s>>>(x, dy, sc.shift, sc.scale, sc.partial, rows, C, per_slice);
      batchnorm_totals_kernel<<<cgrid, kBlock, 0, s>>>(sc.partial, sc.stats0, slices, C, 1.f, 1.f);
      if (vec)
        batchnorm_grad_frozen_vec_kernel<T, VN><<<channel_stable_grid(n / VN, C / VN, sms), kBlock, 0, s>>>(
            dy, g, static_cast<const T*>(pop_variance), static_cast<T*>(output), n / VN, C, p.epsilon);
      else
        batchnorm_grad_frozen_kernel<T><<<grid_for(n, kBlock, sms), kBlock, 0, s>>>(
            dy, g, static_cast<const T*>(pop_variance), static_cast<T*>(output), n, C, p.epsilon);
      count_launch(3);
    }
    batchnorm_param_grads_kernel<T><<<c1grid, kBlock, 0, s>>>(sc.stats0, sc.stats1, static_cast<T*>(beta_grad),
                                                             static_cast<T*>(gamma_grad), C, (float)rows, p.epsilon,
                                                             p.is_training);
    st = check_launch("batchnorm gradient");
    cudaFreeAsync(sc.base, s);
    return st;
  });
}

}  // namespace pdnn
