// General direct convolution on CUDA cores: one thread per output element, fp32 accumulation.
// It takes every shape conv2d::launch accepts in NHWC (any channel/feature count, any window and
// stride, grouped forward, HWCF or FHWC filters) and is what Algorithm::Direct runs; the
// tensor-core kernels hand it the shapes they cannot tile.
//
// Definitions follow portDNN's direct kernels: src/conv2d/direct/kernels_nhwc.h:62-130 (forward),
// :206-278 (input backprop), :356-420 (filter backprop).
#include "common.cuh"

namespace pdnn {
namespace {

constexpr int kBlock = 256;

struct FilterIndex {
  int R, S, Cg, K, fhwc;
  __device__ __forceinline__ size_t operator()(int r, int s, int c, int k) const {
    return fhwc ? (((size_t)k * R + r) * S + s) * Cg + c : (((size_t)r * S + s) * Cg + c) * K + k;
  }
};

struct Epilogue {
  const void* bias;
  int act;
  float alpha, beta;
};

template <typename T>
__global__ void __launch_bounds__(kBlock)
    direct_forward_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y, PdnnConv2DParams p,
                          Epilogue e, size_t n_items) {
  const int G = p.groups, Cg = p.channels / G, Kg = p.features / G;
  const FilterIndex fi{p.window_rows, p.window_cols, Cg, p.features, p.filter_format == 2};
  for (size_t idx = (size_t)blockIdx.x * kBlock + threadIdx.x; idx < n_items; idx += (size_t)gridDim.x * kBlock) {
    const int k = (int)(idx % p.features);
    size_t t = idx / p.features;
    const int ow = (int)(t % p.out_cols);
    t /= p.out_cols;
    const int oh = (int)(t % p.out_rows);
    const int n = (int)(t / p.out_rows);
    // STRIDED groups: a group's channels and features are contiguous; INTERLEAVED: the group is the
    // fastest index of both axes (include/portdnn/batch_format.h:33-47)
    const bool interleaved = p.group_format == 1;
    const int g = interleaved ? k % G : k / Kg;
    const int c_first = interleaved ? g : g * Cg, c_step = interleaved ? G : 1;
    float acc = 0.f;
    for (int r = 0; r < p.window_rows; ++r) {
      const int ih = oh * p.stride_rows - p.pad_rows + r;
      if (ih < 0 || ih >= p.in_rows) continue;
      for (int s = 0; s < p.window_cols; ++s) {
        const int iw = ow * p.stride_cols - p.pad_cols + s;
        if (iw < 0 || iw >= p.in_cols) continue;
        const T* xp = x + (((size_t)n * p.in_rows + ih) * p.in_cols + iw) * p.channels + c_first;
        for (int c = 0; c < Cg; ++c) acc = fmaf(to_f32(__ldg(xp + c * c_step)), to_f32(__ldg(w + fi(r, s, c, k))), acc);
      }
    }
    float v = e.alpha * acc;
    if (e.bias != nullptr) v = to_f32(from_f32<T>(v)) + to_f32(static_cast<const T*>(e.bias)[k]);
    if (e.act != PDNN_ACT_NONE) v = apply_activation(to_f32(from_f32<T>(v)), e.act);
    if (e.beta != 0.f) v = to_f32(from_f32<T>(v)) + to_f32(from_f32<T>(e.beta * to_f32(y[idx])));
    y[idx] = from_f32<T>(v);
  }
}

template <typename T>
__global__ void __launch_bounds__(kBlock)
    direct_input_backprop_kernel(const T* __restrict__ dy, const T* __restrict__ w, T* __restrict__ dx,
                                 PdnnConv2DParams p, size_t n_items) {
  const FilterIndex fi{p.window_rows, p.window_cols, p.channels, p.features, p.filter_format == 2};
  for (size_t idx = (size_t)blockIdx.x * kBlock + threadIdx.x; idx < n_items; idx += (size_t)gridDim.x * kBlock) {
    const int c = (int)(idx % p.channels);
    size_t t = idx / p.channels;
    const int wi = (int)(t % p.in_cols);
    t /= p.in_cols;
    const int h = (int)(t % p.in_rows);
    const int n = (int)(t / p.in_rows);
    float acc = 0.f;
    for (int r = 0; r < p.window_rows; ++r) {
      const int th = h + p.pad_rows - r;
      if (th < 0 || th % p.stride_rows) continue;
      const int oh = th / p.stride_rows;
      if (oh >= p.out_rows) continue;
      for (int s = 0; s < p.window_cols; ++s) {
        const int tw = wi + p.pad_cols - s;
        if (tw < 0 || tw % p.stride_cols) continue;
        const int ow = tw / p.stride_cols;
        if (ow >= p.out_cols) continue;
        const T* dp = dy + (((size_t)n * p.out_rows + oh) * p.out_cols + ow) * p.features;
        for (int k = 0; k < p.features; ++k) acc = fmaf(to_f32(__ldg(dp + k)), to_f32(__ldg(w + fi(r, s, c, k))), acc);
      }
    }
    dx[idx] = from_f32<T>(acc);
  }
}

// One warp per filter-gradient element group: threadIdx.x walks features (coalesced dy reads),
// the block's 8 warps split the pixel range and are summed through shared memory.
template <typename T>
__global__ void __launch_bounds__(kBlock)
    direct_filter_backprop_kernel(const T* __restrict__ x, const T* __restrict__ dy, T* __restrict__ dw,
                                  PdnnConv2DParams p) {
  __shared__ float red[8][32];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int k = blockIdx.x * 32 + lane;
  const int c = blockIdx.y;
  const int tap = blockIdx.z, r = tap / p.window_cols, s = tap % p.window_cols;
  float acc = 0.f;
  if (k < p.features) {
    const long long pixels = (long long)p.batch * p.out_rows * p.out_cols;
    for (long long pix = wid; pix < pixels; pix += 8) {
      const int ow = (int)(pix % p.out_cols);
      const long long t = pix / p.out_cols;
      const int oh = (int)(t % p.out_rows);
      const int n = (int)(t / p.out_rows);
      const int ih = oh * p.stride_rows - p.pad_rows + r, iw = ow * p.stride_cols - p.pad_cols + s;
      if (ih < 0 || ih >= p.in_rows || iw < 0 || iw >= p.in_cols) continue;
      acc = fmaf(to_f32(__ldg(x + (((size_t)n * p.in_rows + ih) * p.in_cols + iw) * p.channels + c)),
                 to_f32(__ldg(dy + (size_t)pix * p.features + k)), acc);
    }
  }
  red[wid][lane] = acc;
  __syncthreads();
  if (wid == 0 && k < p.features) {
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) sum += red[i][lane];
    const FilterIndex fi{p.window_rows, p.window_cols, p.channels, p.features, p.filter_format == 2};
    dw[fi(r, s, c, k)] = from_f32<T>(sum);
  }
}

}  // namespace

int launch_direct_conv(int pass, int dtype, const void* in, const void* fil, void* out, const PdnnConv2DParams& p,
                       const PdnnConvEpilogue* epi, cudaStream_t s) {
  if (p.input_format != 0) return fail(PDNN_INVALID_ALGORITHM, "direct conv: NCHW is not implemented");
  if (p.filter_format == 1) return fail(PDNN_INVALID_PARAMETER, "direct conv: FCHW filters need NCHW tensors");
  const int sms = device_sm_count();
  if (sms <= 0) return fail(PDNN_ALLOCATION_PROBLEM, "no CUDA device");
  Epilogue e{nullptr, PDNN_ACT_NONE, 1.f, 0.f};
  if (epi != nullptr) e = Epilogue{epi->bias, epi->activation, epi->alpha, epi->beta};
  auto run = [&](auto tag) -> int {
    using T = decltype(tag);
    if (pass == PDNN_FORWARD) {
      const size_t items = (size_t)p.batch * p.out_rows * p.out_cols * p.features;
      direct_forward_kernel<T><<<grid_for(items, kBlock, sms), kBlock, 0, s>>>(
          static_cast<const T*>(in), static_cast<const T*>(fil), static_cast<T*>(out), p, e, items);
    } else if (pass == PDNN_INPUT_BACKPROP) {
      const size_t items = (size_t)p.batch * p.in_rows * p.in_cols * p.channels;
      direct_input_backprop_kernel<T><<<grid_for(items, kBlock, sms), kBlock, 0, s>>>(
          static_cast<const T*>(in), static_cast<const T*>(fil), static_cast<T*>(out), p, items);
    } else {
      dim3 grid((p.features + 31) / 32, p.channels, p.window_rows * p.window_cols);
      if (grid.y > 65535u || grid.z > 65535u) return fail(PDNN_INDEX_EXCEEDED, "direct filter backprop: grid too large");
      direct_filter_backprop_kernel<T><<<grid, kBlock, 0, s>>>(static_cast<const T*>(in), static_cast<const T*>(fil),
                                                              static_cast<T*>(out), p);
    }
    return check_launch("direct conv2d");
  };
  switch (dtype) {
    case PDNN_F32: return run(float{});
    case PDNN_F16: return run(__half{});
    case PDNN_BF16: return run(__nv_bfloat16{});
  }
  return fail(PDNN_INVALID_PARAMETER, "unknown dtype %d", dtype);
}

}  // namespace pdnn
