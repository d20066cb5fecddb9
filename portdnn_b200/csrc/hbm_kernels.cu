// HBM-bound operators for NHWC tensors: pooling, depthwise convolution, pointwise
// activations, bias add and the alpha/beta blend.  One thread owns a 16-byte packet of
// channels (8 halves or 4 floats) of one pixel, so that a warp reads and writes whole
// 512-byte lines along the channel axis; shapes whose channel count is not a multiple of
// the packet fall back to one element per thread.  Arithmetic is done in fp32 and rounded
// once on store.
//
// Semantics follow portDNN: src/pooling/kernels.h, src/pooling/operators_impl.h,
// src/depthwise_conv2d/kernels.h, src/pointwise/kernels.h, src/binaryop/kernels.h.
#include "common.cuh"

#include <cfloat>
#include <mutex>
#include <type_traits>

namespace pdnn {

namespace {

constexpr int kBlock = 256;

template <typename T>
__device__ __forceinline__ float lowest_of();
template <>
__device__ __forceinline__ float lowest_of<float>() { return -FLT_MAX; }
template <>
__device__ __forceinline__ float lowest_of<__half>() { return -65504.f; }
template <>
__device__ __forceinline__ float lowest_of<__nv_bfloat16>() { return -3.3895313892515355e38f; }

// V elements starting at p: one 16-byte load when V > 1.
template <typename T, int V>
__device__ __forceinline__ void load_vec(const T* p, float (&v)[V]) {
  if constexpr (V == 1) {
    v[0] = to_f32(__ldg(p));
  } else {
    Vec16<T> pk = load16(p);
#pragma unroll
    for (int i = 0; i < V; ++i) v[i] = to_f32(pk.get(i));
  }
}
template <typename T, int V>
__device__ __forceinline__ void store_vec(T* p, const float (&v)[V]) {
  if constexpr (V == 1) {
    p[0] = from_f32<T>(v[0]);
  } else {
    Vec16<T> pk;
#pragma unroll
    for (int i = 0; i < V; ++i) pk.set(i, from_f32<T>(v[i]));
    store16(p, pk);
  }
}

// ------------------------------------------------------------------------------------------
// Pooling forward.  Window clamped to the image; Average divides by the valid count
// (src/pooling/kernels.h:61-101).  Max keeps v only if v > max starting from lowest(), so a
// NaN never wins; MaxWithNan takes a NaN and then keeps it (src/pooling/operators_impl.h:27-65).
// ------------------------------------------------------------------------------------------
template <typename T, int OP, int V, typename Index>
__global__ void __launch_bounds__(kBlock) pool_forward_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                              PdnnPoolingParams p, Index n_items) {
  const Index cvecs = (Index)(p.channels / V);
  for (Index idx = (Index)blockIdx.x * kBlock + threadIdx.x; idx < n_items; idx += (Index)gridDim.x * kBlock) {
    const Index cv = idx % cvecs;
    Index t = idx / cvecs;
    const int ow = (int)(t % (Index)p.out_cols);
    t /= (Index)p.out_cols;
    const int oh = (int)(t % (Index)p.out_rows);
    const int n = (int)(t / (Index)p.out_rows);
    int r0 = oh * p.stride_rows - p.pad_rows, c0 = ow * p.stride_cols - p.pad_cols;
    const int r1 = min(r0 + p.window_rows, p.in_rows), c1 = min(c0 + p.window_cols, p.in_cols);
    r0 = max(r0, 0);
    c0 = max(c0, 0);
    float acc[V];
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] = (OP == PDNN_POOL_AVERAGE) ? 0.f : lowest_of<T>();
    const T* xn = x + (size_t)n * p.in_rows * p.in_cols * p.channels + (size_t)cv * V;
    for (int r = r0; r < r1; ++r) {
      for (int c = c0; c < c1; ++c) {
        float v[V];
        load_vec<T, V>(xn + ((size_t)r * p.in_cols + c) * p.channels, v);
#pragma unroll
        for (int i = 0; i < V; ++i) {
          if (OP == PDNN_POOL_MAX) {
            if (v[i] > acc[i]) acc[i] = v[i];
          } else if (OP == PDNN_POOL_MAX_WITH_NAN) {
            if (isnan(v[i]) || v[i] > acc[i]) acc[i] = v[i];
          } else {
            acc[i] += v[i];
          }
        }
      }
    }
    if (OP == PDNN_POOL_AVERAGE) {
      const float tally = (float)((r1 - r0) * (c1 - c0));
#pragma unroll
      for (int i = 0; i < V; ++i) acc[i] = acc[i] / tally;
    }
    store_vec<T, V>(y + (size_t)idx * V, acc);
  }
}

template <int OP>
__device__ __forceinline__ bool pool_equal(float a, float b) {
  // src/pooling/operators_impl.h:89-108
  if (OP == PDNN_POOL_MAX_WITH_NAN) return a == b || (isnan(a) && isnan(b));
  return a == b;
}

// ------------------------------------------------------------------------------------------
// Max-pool gradient (src/pooling/kernels.h:142-243): dx[i] collects dy[o] from every output o
// whose clamped window holds i, if x[i] == y[o] and no earlier element of that window
// (row-major) equals y[o].  The scan for an earlier maximum only runs for lanes that matched.
// ------------------------------------------------------------------------------------------
template <typename T, int OP, int V, typename Index>
__global__ void __launch_bounds__(kBlock)
    pool_max_grad_kernel(const T* __restrict__ x, const T* __restrict__ y, const T* __restrict__ dy,
                         T* __restrict__ dx, PdnnPoolingParams p, Index n_items) {
  const Index cvecs = (Index)(p.channels / V);
  for (Index idx = (Index)blockIdx.x * kBlock + threadIdx.x; idx < n_items; idx += (Index)gridDim.x * kBlock) {
    const Index cv = idx % cvecs;
    Index t = idx / cvecs;
    const int w = (int)(t % (Index)p.in_cols);
    t /= (Index)p.in_cols;
    const int h = (int)(t % (Index)p.in_rows);
    const int n = (int)(t / (Index)p.in_rows);
    float xv[V], grad[V];
    load_vec<T, V>(x + (size_t)idx * V, xv);
#pragma unroll
    for (int i = 0; i < V; ++i) grad[i] = 0.f;
    const int hp = h + p.pad_rows, wp = w + p.pad_cols;
    const int oh_lo = hp < p.window_rows ? 0 : (hp - p.window_rows) / p.stride_rows + 1;
    const int oh_hi = min(hp / p.stride_rows + 1, p.out_rows);
    const int ow_lo = wp < p.window_cols ? 0 : (wp - p.window_cols) / p.stride_cols + 1;
    const int ow_hi = min(wp / p.stride_cols + 1, p.out_cols);
    const T* xn = x + (size_t)n * p.in_rows * p.in_cols * p.channels + (size_t)cv * V;
    const size_t out_n = (size_t)n * p.out_rows * p.out_cols * p.channels + (size_t)cv * V;
    for (int oh = oh_lo; oh < oh_hi; ++oh) {
      int r0 = oh * p.stride_rows - p.pad_rows;
      const int r1 = min(r0 + p.window_rows, p.in_rows);
      r0 = max(r0, 0);
      for (int ow = ow_lo; ow < ow_hi; ++ow) {
        int c0 = ow * p.stride_cols - p.pad_cols;
        const int c1 = min(c0 + p.window_cols, p.in_cols);
        c0 = max(c0, 0);
        const size_t o = out_n + ((size_t)oh * p.out_cols + ow) * p.channels;
        float yv[V];
        load_vec<T, V>(y + o, yv);
        bool hit[V];
        bool any = false;
#pragma unroll
        for (int i = 0; i < V; ++i) {
          hit[i] = pool_equal<OP>(xv[i], yv[i]);
          any |= hit[i];
        }
        if (!any) continue;
        bool scanning = true;
        for (int r = r0; r < r1 && scanning; ++r) {
          for (int c = c0; c < c1; ++c) {
            if (r == h && c == w) {
              scanning = false;
              break;
            }
            float ev[V];
            load_vec<T, V>(xn + ((size_t)r * p.in_cols + c) * p.channels, ev);
#pragma unroll
            for (int i = 0; i < V; ++i)
              if (pool_equal<OP>(ev[i], yv[i])) hit[i] = false;
          }
        }
        float dv[V];
        load_vec<T, V>(dy + o, dv);
#pragma unroll
        for (int i = 0; i < V; ++i)
          if (hit[i]) grad[i] += dv[i];
      }
    }
    store_vec<T, V>(dx + (size_t)idx * V, grad);
  }
}

// Max-pool gradient when the windows tile the input exactly (stride == window, no padding,
// in == out * stride: the 2x2/2 pools of VGG).  Every input element belongs to exactly one window,
// so one thread per output packet reads its window once, finds per channel the first element equal
// to y (the same rule as above) and writes dy there and zero elsewhere: x, y and dy are read once
// and dx is written once.
template <typename T, int OP, int V, typename Index>
__global__ void __launch_bounds__(kBlock)
    pool_max_grad_tiled_kernel(const T* __restrict__ x, const T* __restrict__ y, const T* __restrict__ dy,
                               T* __restrict__ dx, PdnnPoolingParams p, Index n_items) {
  const Index cvecs = (Index)(p.channels / V);
  for (Index idx = (Index)blockIdx.x * kBlock + threadIdx.x; idx < n_items; idx += (Index)gridDim.x * kBlock) {
    const Index cv = idx % cvecs;
    Index t = idx / cvecs;
    const int ow = (int)(t % (Index)p.out_cols);
    t /= (Index)p.out_cols;
    const int oh = (int)(t % (Index)p.out_rows);
    const int n = (int)(t / (Index)p.out_rows);
    float yv[V], dv[V];
    load_vec<T, V>(y + (size_t)idx * V, yv);
    load_vec<T, V>(dy + (size_t)idx * V, dv);
    bool open[V];  // no element of the window has matched yet
#pragma unroll
    for (int i = 0; i < V; ++i) open[i] = true;
    const size_t base = ((size_t)n * p.in_rows + (size_t)oh * p.stride_rows) * p.in_cols + (size_t)ow * p.stride_cols;
    for (int r = 0; r < p.window_rows; ++r)
      for (int c = 0; c < p.window_cols; ++c) {
        const size_t off = ((base + (size_t)r * p.in_cols + c) * p.channels) + (size_t)cv * V;
        float xv[V], g[V];
        load_vec<T, V>(x + off, xv);
#pragma unroll
        for (int i = 0; i < V; ++i) {
          const bool hit = open[i] && pool_equal<OP>(xv[i], yv[i]);
          g[i] = hit ? dv[i] : 0.f;
          open[i] = open[i] && !hit;
        }
        store_vec<T, V>(dx + off, g);
      }
  }
}

// V bytes (V = 4 or 8, address a multiple of V) <-> V words, through registers only.
template <int V>
__device__ __forceinline__ void store_bytes(unsigned char* p, const unsigned (&v)[V]) {
  static_assert(V == 4 || V == 8, "packet of 4 or 8 channels");
  const unsigned lo = v[0] | (v[1] << 8) | (v[2] << 16) | (v[3] << 24);
  if constexpr (V == 8) {
    const unsigned hi = v[4] | (v[5] << 8) | (v[6] << 16) | (v[7] << 24);
    *reinterpret_cast<uint2*>(p) = make_uint2(lo, hi);
  } else {
    *reinterpret_cast<unsigned*>(p) = lo;
  }
}
template <int V>
__device__ __forceinline__ void load_bytes(const unsigned char* p, unsigned (&v)[V]) {
  static_assert(V == 4 || V == 8, "packet of 4 or 8 channels");
  unsigned lo, hi = 0u;
  if constexpr (V == 8) {
    const uint2 raw = __ldg(reinterpret_cast<const uint2*>(p));
    lo = raw.x;
    hi = raw.y;
  } else {
    lo = __ldg(reinterpret_cast<const unsigned*>(p));
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = (lo >> (8 * i)) & 0xFFu;
  if constexpr (V == 8) {
#pragma unroll
    for (int i = 0; i < 4; ++i) v[4 + i] = (hi >> (8 * i)) & 0xFFu;
  }
}

// Max-pool gradient for overlapping windows, in two passes.  Pass 1 (one thread per output packet)
// records for every output element which element of its window is the first maximum, as
// 1 + row * window_cols + col in unclamped window coordinates (0: none).  Pass 2 (one thread per
// input packet) visits the windows that hold the element, in the same order as
// pool_max_grad_kernel, and adds dy where the recorded winner is this element.  The scan for an
// earlier maximum, which pool_max_grad_kernel repeats for every (input, window) pair, is done once
// per window.
template <typename T, int OP, int V, typename Index>
__global__ void __launch_bounds__(kBlock)
    pool_winner_kernel(const T* __restrict__ x, const T* __restrict__ y, unsigned char* __restrict__ winner,
                       PdnnPoolingParams p, Index n_items) {
  const Index cvecs = (Index)(p.channels / V);
  for (Index idx = (Index)blockIdx.x * kBlock + threadIdx.x; idx < n_items; idx += (Index)gridDim.x * kBlock) {
    const Index cv = idx % cvecs;
    Index t = idx / cvecs;
    const int ow = (int)(t % (Index)p.out_cols);
    t /= (Index)p.out_cols;
    const int oh = (int)(t % (Index)p.out_rows);
    const int n = (int)(t / (Index)p.out_rows);
    const int ur = oh * p.stride_rows - p.pad_rows, uc = ow * p.stride_cols - p.pad_cols;  // unclamped origin
    const int r0 = max(ur, 0), c0 = max(uc, 0);
    const int r1 = min(ur + p.window_rows, p.in_rows), c1 = min(uc + p.window_cols, p.in_cols);
    float yv[V];
    load_vec<T, V>(y + (size_t)idx * V, yv);
    unsigned win[V];
#pragma unroll
    for (int i = 0; i < V; ++i) win[i] = 0u;
    const T* xn = x + (size_t)n * p.in_rows * p.in_cols * p.channels + (size_t)cv * V;
    if (p.window_rows == 3 && p.window_cols == 3) {
      // 3x3: a row of three loads at a time, unconditional (clamped coordinates, masked match)
#pragma unroll
      for (int r = 0; r < 3; ++r) {
        const int ir = ur + r;
        const bool row_ok = ir >= r0 && ir < r1;
        const T* xr = xn + (size_t)min(max(ir, 0), p.in_rows - 1) * p.in_cols * p.channels;
        float xv[3][V];
#pragma unroll
        for (int c = 0; c < 3; ++c) load_vec<T, V>(xr + (size_t)min(max(uc + c, 0), p.in_cols - 1) * p.channels, xv[c]);
#pragma unroll
        for (int c = 0; c < 3; ++c) {
          const bool ok = row_ok && uc + c >= c0 && uc + c < c1;
          const unsigned id = (unsigned)(1 + r * 3 + c);
#pragma unroll
          for (int i = 0; i < V; ++i)
            if (ok && win[i] == 0u && pool_equal<OP>(xv[c][i], yv[i])) win[i] = id;
        }
      }
    } else {
      for (int r = r0; r < r1; ++r)
        for (int c = c0; c < c1; ++c) {
          float xv[V];
          load_vec<T, V>(xn + ((size_t)r * p.in_cols + c) * p.channels, xv);
          const unsigned id = (unsigned)(1 + (r - ur) * p.window_cols + (c - uc));
#pragma unroll
          for (int i = 0; i < V; ++i)
            if (win[i] == 0u && pool_equal<OP>(xv[i], yv[i])) win[i] = id;
        }
    }
    store_bytes<V>(winner + (size_t)idx * V, win);
  }
}

template <typename T, int V, typename Index>
__global__ void __launch_bounds__(kBlock)
    pool_max_grad_from_winner_kernel(const unsigned char* __restrict__ winner, const T* __restrict__ dy,
                                     T* __restrict__ dx, PdnnPoolingParams p, Index n_items) {
  const Index cvecs = (Index)(p.channels / V);
  for (Index idx = (Index)blockIdx.x * kBlock + threadIdx.x; idx < n_items; idx += (Index)gridDim.x * kBlock) {
    const Index cv = idx % cvecs;
    Index t = idx / cvecs;
    const int w = (int)(t % (Index)p.in_cols);
    t /= (Index)p.in_cols;
    const int h = (int)(t % (Index)p.in_rows);
    const int n = (int)(t / (Index)p.in_rows);
    float grad[V];
#pragma unroll
    for (int i = 0; i < V; ++i) grad[i] = 0.f;
    const int hp = h + p.pad_rows, wp = w + p.pad_cols;
    const int oh_lo = hp < p.window_rows ? 0 : (hp - p.window_rows) / p.stride_rows + 1;
    const int oh_hi = min(hp / p.stride_rows + 1, p.out_rows);
    const int ow_lo = wp < p.window_cols ? 0 : (wp - p.window_cols) / p.stride_cols + 1;
    const int ow_hi = min(wp / p.stride_cols + 1, p.out_cols);
    const size_t out_n = (size_t)n * p.out_rows * p.out_cols * p.channels + (size_t)cv * V;
    if (oh_hi - oh_lo <= 2 && ow_hi - ow_lo <= 2) {
      // At most 2 x 2 windows hold the element (window <= 2 * stride): all four winner words and
      // all four dy packets are requested at once, with clamped coordinates and a mask, instead
      // of one dependent pair of loads after another.
      unsigned win[4][V];
      float dv[4][V];
      bool ok[4];
      unsigned me[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int oh = oh_lo + (k >> 1), ow = ow_lo + (k & 1);
        ok[k] = oh < oh_hi && ow < ow_hi;
        const int ohc = min(oh, p.out_rows - 1), owc = min(ow, p.out_cols - 1);
        const size_t o = out_n + ((size_t)ohc * p.out_cols + owc) * p.channels;
        me[k] = (unsigned)(1 + (hp - oh * p.stride_rows) * p.window_cols + (wp - ow * p.stride_cols));
        load_bytes<V>(winner + o, win[k]);
        load_vec<T, V>(dy + o, dv[k]);
      }
#pragma unroll
      for (int k = 0; k < 4; ++k)  // k = 2 * row + column: the same order as the loops below
#pragma unroll
        for (int i = 0; i < V; ++i)
          if (ok[k] && win[k][i] == me[k]) grad[i] += dv[k][i];
      store_vec<T, V>(dx + (size_t)idx * V, grad);
      continue;
    }
    for (int oh = oh_lo; oh < oh_hi; ++oh)
      for (int ow = ow_lo; ow < ow_hi; ++ow) {
        const size_t o = out_n + ((size_t)oh * p.out_cols + ow) * p.channels;
        const unsigned me = (unsigned)(1 + (hp - oh * p.stride_rows) * p.window_cols + (wp - ow * p.stride_cols));
        unsigned win[V];
        load_bytes<V>(winner + o, win);
        bool any = false;
#pragma unroll
        for (int i = 0; i < V; ++i) any |= win[i] == me;
        if (!any) continue;
        float dv[V];
        load_vec<T, V>(dy + o, dv);
#pragma unroll
        for (int i = 0; i < V; ++i)
          if (win[i] == me) grad[i] += dv[i];
      }
    store_vec<T, V>(dx + (size_t)idx * V, grad);
  }
}

// The gather for 3x3 windows with stride 2, walking the windows instead of the input pixels.  With
// m = (h + pad) / 2 the input rows 2m - pad and 2m + 1 - pad lie in windows {m - 1, m} (as their
// rows 2 and 0) and {m} (row 1); columns likewise.  A thread owns a packet of channels at one
// window column k and walks `rows` values of m: per step it loads the winner ids and dy of windows
// (m, k-1) and (m, k), keeps those of row m - 1, and writes the 2x2 block of dx pixels.  Sums run
// in the order (m-1,k-1), (m-1,k), (m,k-1), (m,k), the order of the general gather above.
struct PoolS2Geometry {
  int H, W, Ho, Wo, C, pad_r, pad_c, N;
  int M, K, rows, strips;
};

template <typename T, int V>
__global__ void __launch_bounds__(kBlock)
    pool_max_grad_s2_kernel(const unsigned char* __restrict__ winner, const T* __restrict__ dy, T* __restrict__ dx,
                            PoolS2Geometry g, unsigned n_items) {
  const unsigned cvecs = (unsigned)(g.C / V);
  for (unsigned idx = blockIdx.x * kBlock + threadIdx.x; idx < n_items; idx += gridDim.x * kBlock) {
    const unsigned cv = idx % cvecs;
    unsigned t = idx / cvecs;
    const int k = (int)(t % (unsigned)g.K);
    t /= (unsigned)g.K;
    const int strip = (int)(t % (unsigned)g.strips), n = (int)(t / (unsigned)g.strips);
    const size_t c = (size_t)cv * V;
    const size_t out_n = (size_t)n * g.Ho * g.Wo * g.C + c;
    T* dxn = dx + (size_t)n * g.H * g.W * g.C + c;
    const bool k_ok = k < g.Wo, k1_ok = k >= 1 && k - 1 < g.Wo;
    // a = window (m, k), b = window (m, k - 1); id 0 (matches nothing) outside the output
    auto load_row = [&](int m, unsigned (&wa)[V], float (&da)[V], unsigned (&wb)[V], float (&db)[V]) {
#pragma unroll
      for (int i = 0; i < V; ++i) {
        wa[i] = wb[i] = 0u;
        da[i] = db[i] = 0.f;
      }
      if (m < 0 || m >= g.Ho) return;
      const size_t row = out_n + (size_t)m * g.Wo * g.C;
      if (k_ok) {
        load_bytes<V>(winner + row + (size_t)k * g.C, wa);
        load_vec<T, V>(dy + row + (size_t)k * g.C, da);
      }
      if (k1_ok) {
        load_bytes<V>(winner + row + (size_t)(k - 1) * g.C, wb);
        load_vec<T, V>(dy + row + (size_t)(k - 1) * g.C, db);
      }
    };
    const int m0 = strip * g.rows, m1 = min(m0 + g.rows, g.M);
    unsigned pwa[V], pwb[V], cwa[V], cwb[V];
    float pda[V], pdb[V], cda[V], cdb[V];
    load_row(m0 - 1, pwa, pda, pwb, pdb);
    const int w0 = 2 * k - g.pad_c, w1 = w0 + 1;
    const bool w0_ok = w0 >= 0 && w0 < g.W, w1_ok = w1 >= 0 && w1 < g.W;
    for (int m = m0; m < m1; ++m) {
      load_row(m, cwa, cda, cwb, cdb);
      const int h0 = 2 * m - g.pad_r, h1 = h0 + 1;
      float o[V];
      if (h0 >= 0 && h0 < g.H) {
        T* orow = dxn + (size_t)h0 * g.W * g.C;
        if (w0_ok) {  // row 2 / 0, column 2 / 0 of the four windows
#pragma unroll
          for (int i = 0; i < V; ++i) {
            float v = 0.f;
            if (pwb[i] == 9u) v += pdb[i];
            if (pwa[i] == 7u) v += pda[i];
            if (cwb[i] == 3u) v += cdb[i];
            if (cwa[i] == 1u) v += cda[i];
            o[i] = v;
          }
          store_vec<T, V>(orow + (size_t)w0 * g.C, o);
        }
        if (w1_ok) {  // column 1 of windows (m - 1, k) and (m, k)
#pragma unroll
          for (int i = 0; i < V; ++i) {
            float v = 0.f;
            if (pwa[i] == 8u) v += pda[i];
            if (cwa[i] == 2u) v += cda[i];
            o[i] = v;
          }
          store_vec<T, V>(orow + (size_t)w1 * g.C, o);
        }
      }
      if (h1 >= 0 && h1 < g.H) {
        T* orow = dxn + (size_t)h1 * g.W * g.C;
        if (w0_ok) {  // row 1 of windows (m, k - 1) and (m, k)
#pragma unroll
          for (int i = 0; i < V; ++i) {
            float v = 0.f;
            if (cwb[i] == 6u) v += cdb[i];
            if (cwa[i] == 4u) v += cda[i];
            o[i] = v;
          }
          store_vec<T, V>(orow + (size_t)w0 * g.C, o);
        }
        if (w1_ok) {  // the centre of window (m, k)
#pragma unroll
          for (int i = 0; i < V; ++i) o[i] = cwa[i] == 5u ? cda[i] : 0.f;
          store_vec<T, V>(orow + (size_t)w1 * g.C, o);
        }
      }
#pragma unroll
      for (int i = 0; i < V; ++i) {
        pwa[i] = cwa[i];
        pwb[i] = cwb[i];
        pda[i] = cda[i];
        pdb[i] = cdb[i];
      }
    }
  }
}

// Average-pool gradient (src/pooling/kernels.h:312-366): dx[i] = sum_o dy[o] / valid(o).
template <typename T, int V, typename Index>
__global__ void __launch_bounds__(kBlock)
    pool_avg_grad_kernel(const T* __restrict__ dy, T* __restrict__ dx, PdnnPoolingParams p, Index n_items) {
  const Index cvecs = (Index)(p.channels / V);
  for (Index idx = (Index)blockIdx.x * kBlock + threadIdx.x; idx < n_items; idx += (Index)gridDim.x * kBlock) {
    const Index cv = idx % cvecs;
    Index t = idx / cvecs;
    const int w = (int)(t % (Index)p.in_cols);
    t /= (Index)p.in_cols;
    const int h = (int)(t % (Index)p.in_rows);
    const int n = (int)(t / (Index)p.in_rows);
    float grad[V];
#pragma unroll
    for (int i = 0; i < V; ++i) grad[i] = 0.f;
    const int hp = h + p.pad_rows, wp = w + p.pad_cols;
    const int oh_lo = hp < p.window_rows ? 0 : (hp - p.window_rows) / p.stride_rows + 1;
    const int oh_hi = min(hp / p.stride_rows + 1, p.out_rows);
    const int ow_lo = wp < p.window_cols ? 0 : (wp - p.window_cols) / p.stride_cols + 1;
    const int ow_hi = min(wp / p.stride_cols + 1, p.out_cols);
    const size_t out_n = (size_t)n * p.out_rows * p.out_cols * p.channels + (size_t)cv * V;
    for (int oh = oh_lo; oh < oh_hi; ++oh) {
      int r0 = oh * p.stride_rows - p.pad_rows;
      const int r1 = min(r0 + p.window_rows, p.in_rows);
      r0 = max(r0, 0);
      for (int ow = ow_lo; ow < ow_hi; ++ow) {
        int c0 = ow * p.stride_cols - p.pad_cols;
        const int c1 = min(c0 + p.window_cols, p.in_cols);
        c0 = max(c0, 0);
        const float cnt = (float)((r1 - r0) * (c1 - c0));
        float dv[V];
        load_vec<T, V>(dy + out_n + ((size_t)oh * p.out_cols + ow) * p.channels, dv);
#pragma unroll
        for (int i = 0; i < V; ++i) grad[i] += dv[i] / cnt;
      }
    }
    store_vec<T, V>(dx + (size_t)idx * V, grad);
  }
}

// The same when one window covers the whole image (global pooling): every pixel of an image
// receives dy / (rows * cols); one division by a runtime value per thread instead of the window walk.
template <typename T, int V>
__global__ void __launch_bounds__(kBlock)
    pool_avg_grad_global_kernel(const T* __restrict__ dy, T* __restrict__ dx, unsigned cvecs, unsigned per_image,
                                float count, unsigned n_items) {
  for (unsigned idx = blockIdx.x * kBlock + threadIdx.x; idx < n_items; idx += gridDim.x * kBlock) {
    const unsigned n = idx / per_image, cv = idx % cvecs;  // per_image is a multiple of cvecs
    float dv[V];
    load_vec<T, V>(dy + ((size_t)n * cvecs + cv) * V, dv);
#pragma unroll
    for (int i = 0; i < V; ++i) dv[i] = dv[i] / count;  // the division of the general kernel, for equal results
    store_vec<T, V>(dx + (size_t)idx * V, dv);
  }
}

// ------------------------------------------------------------------------------------------
// Depthwise convolution.  Filter [R][S][C][mult], output channel c*mult+m
// (src/depthwise_conv2d/kernels.h:58-125).  The packet form needs mult == 1.
// ------------------------------------------------------------------------------------------
template <typename T, int V, typename Index>
__global__ void __launch_bounds__(kBlock)
    depthwise_forward_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y,
                             PdnnDepthwiseConv2DParams p, Index n_items) {
  const int F = p.channels * p.channel_multiplier;
  const Index fvecs = (Index)(F / V);
  for (Index idx = (Index)blockIdx.x * kBlock + threadIdx.x; idx < n_items; idx += (Index)gridDim.x * kBlock) {
    const int f = (int)(idx % fvecs) * V;
    Index t = idx / fvecs;
    const int ow = (int)(t % (Index)p.out_cols);
    t /= (Index)p.out_cols;
    const int oh = (int)(t % (Index)p.out_rows);
    const int n = (int)(t / (Index)p.out_rows);
    const int c = (V == 1) ? f / p.channel_multiplier : f;
    float acc[V];
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] = 0.f;
    const T* xn = x + (size_t)n * p.in_rows * p.in_cols * p.channels + c;
    const int ih0 = oh * p.stride_rows - p.pad_rows, iw0 = ow * p.stride_cols - p.pad_cols;
    for (int r = 0; r < p.window_rows; ++r) {
      const int ih = ih0 + r;
      if (ih < 0 || ih >= p.in_rows) continue;
      for (int s = 0; s < p.window_cols; ++s) {
        const int iw = iw0 + s;
        if (iw < 0 || iw >= p.in_cols) continue;
        float xv[V], wv[V];
        load_vec<T, V>(xn + ((size_t)ih * p.in_cols + iw) * p.channels, xv);
        load_vec<T, V>(w + ((size_t)r * p.window_cols + s) * F + f, wv);
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] = fmaf(xv[i], wv[i], acc[i]);
      }
    }
    store_vec<T, V>(y + (size_t)idx * V, acc);
  }
}

// Input backprop (src/depthwise_conv2d/kernels.h:154-225): dx[n,h,w,c] = sum over taps (r,s)
// with (h+pad-r) divisible by the stride, and over the multiplier, of dy * w.
template <typename T, int V, typename Index>
__global__ void __launch_bounds__(kBlock)
    depthwise_input_backprop_kernel(const T* __restrict__ dy, const T* __restrict__ w, T* __restrict__ dx,
                                    PdnnDepthwiseConv2DParams p, Index n_items) {
  const int M = p.channel_multiplier, F = p.channels * M;
  const Index cvecs = (Index)(p.channels / V);
  for (Index idx = (Index)blockIdx.x * kBlock + threadIdx.x; idx < n_items; idx += (Index)gridDim.x * kBlock) {
    const int c = (int)(idx % cvecs) * V;
    Index t = idx / cvecs;
    const int wi = (int)(t % (Index)p.in_cols);
    t /= (Index)p.in_cols;
    const int h = (int)(t % (Index)p.in_rows);
    const int n = (int)(t / (Index)p.in_rows);
    float acc[V];
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] = 0.f;
    const T* dyn = dy + (size_t)n * p.out_rows * p.out_cols * F + (size_t)c * M;
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
        const T* dp = dyn + ((size_t)oh * p.out_cols + ow) * F;
        const T* wp = w + ((size_t)r * p.window_cols + s) * F + (size_t)c * M;
        if constexpr (V == 1) {
          for (int m = 0; m < M; ++m) acc[0] = fmaf(to_f32(__ldg(dp + m)), to_f32(__ldg(wp + m)), acc[0]);
        } else {
          float dv[V], wv[V];
          load_vec<T, V>(dp, dv);
          load_vec<T, V>(wp, wv);
#pragma unroll
          for (int i = 0; i < V; ++i) acc[i] = fmaf(dv[i], wv[i], acc[i]);
        }
      }
    }
    store_vec<T, V>(dx + (size_t)idx * V, acc);
  }
}

// Input backprop of a 3x3 window with stride 2, multiplier 1, as a gather over dy that visits every
// dy pixel once per thread column instead of testing nine taps per dx pixel.  With m = (h + pad) / 2
// the two dx rows 2m - pad and 2m + 1 - pad read dy rows {m, m - 1} (filter rows 0 and 2) and {m}
// (filter row 1); columns likewise.  A thread owns one packet of channels at one k and walks `rows`
// values of m downwards: it loads dy[m][k-1], dy[m][k], keeps the two packets of row m - 1 from the
// previous step, and writes the four dx pixels of the 2x2 block:
//   dx(2m,   2k)   = d[m][k] w00 + d[m][k-1] w02 + d[m-1][k] w20 + d[m-1][k-1] w22
//   dx(2m,   2k+1) = d[m][k] w01 + d[m-1][k] w21
//   dx(2m+1, 2k)   = d[m][k] w10 + d[m][k-1] w12
//   dx(2m+1, 2k+1) = d[m][k] w11                                   (coordinates before "- pad")
struct IbpS2Geometry {
  int H, W, Ho, Wo, C, pad_r, pad_c, N;
  int M, K;     // values of m and k that touch a dx pixel
  int rows;     // m values per thread
  int strips;   // ceil(M / rows)
};

template <typename T, int V>
__global__ void __launch_bounds__(kBlock) depthwise_ibp_s2_kernel(const T* __restrict__ dy, const T* __restrict__ w,
                                                                  T* __restrict__ dx, IbpS2Geometry g, unsigned n_items) {
  const unsigned cvecs = (unsigned)(g.C / V);
  for (unsigned idx = blockIdx.x * kBlock + threadIdx.x; idx < n_items; idx += gridDim.x * kBlock) {
    const unsigned cv = idx % cvecs;
    unsigned t = idx / cvecs;
    const int k = (int)(t % (unsigned)g.K);
    t /= (unsigned)g.K;
    const int strip = (int)(t % (unsigned)g.strips), n = (int)(t / (unsigned)g.strips);
    const int c = (int)cv * V;
    float wf[9][V];
#pragma unroll
    for (int i = 0; i < 9; ++i) load_vec<T, V>(w + (size_t)i * g.C + c, wf[i]);
    const T* dyn = dy + (size_t)n * g.Ho * g.Wo * g.C + c;
    T* dxn = dx + (size_t)n * g.H * g.W * g.C + c;
    const bool k_ok = k < g.Wo, k1_ok = k >= 1 && k - 1 < g.Wo;
    auto load_row = [&](int m, float (&a)[V], float (&b)[V]) {  // a = dy[m][k], b = dy[m][k-1]; zeros outside dy
#pragma unroll
      for (int i = 0; i < V; ++i) a[i] = b[i] = 0.f;
      if (m < 0 || m >= g.Ho) return;
      const T* row = dyn + (size_t)m * g.Wo * g.C;
      if (k_ok) load_vec<T, V>(row + (size_t)k * g.C, a);
      if (k1_ok) load_vec<T, V>(row + (size_t)(k - 1) * g.C, b);
    };
    const int m0 = strip * g.rows, m1 = min(m0 + g.rows, g.M);
    float pk[V], pk1[V], ck[V], ck1[V];
    load_row(m0 - 1, pk, pk1);
    const int w0 = 2 * k - g.pad_c, w1 = w0 + 1;
    const bool w0_ok = w0 >= 0 && w0 < g.W, w1_ok = w1 >= 0 && w1 < g.W;
    for (int m = m0; m < m1; ++m) {
      load_row(m, ck, ck1);
      const int h0 = 2 * m - g.pad_r, h1 = h0 + 1;
      float o[V];
      if (h0 >= 0 && h0 < g.H) {
        T* orow = dxn + (size_t)h0 * g.W * g.C;
        if (w0_ok) {
#pragma unroll
          for (int i = 0; i < V; ++i)
            o[i] = fmaf(ck[i], wf[0][i], fmaf(ck1[i], wf[2][i], fmaf(pk[i], wf[6][i], pk1[i] * wf[8][i])));
          store_vec<T, V>(orow + (size_t)w0 * g.C, o);
        }
        if (w1_ok) {
#pragma unroll
          for (int i = 0; i < V; ++i) o[i] = fmaf(ck[i], wf[1][i], pk[i] * wf[7][i]);
          store_vec<T, V>(orow + (size_t)w1 * g.C, o);
        }
      }
      if (h1 >= 0 && h1 < g.H) {
        T* orow = dxn + (size_t)h1 * g.W * g.C;
        if (w0_ok) {
#pragma unroll
          for (int i = 0; i < V; ++i) o[i] = fmaf(ck[i], wf[3][i], ck1[i] * wf[5][i]);
          store_vec<T, V>(orow + (size_t)w0 * g.C, o);
        }
        if (w1_ok) {
#pragma unroll
          for (int i = 0; i < V; ++i) o[i] = ck[i] * wf[4][i];
          store_vec<T, V>(orow + (size_t)w1 * g.C, o);
        }
      }
#pragma unroll
      for (int i = 0; i < V; ++i) {
        pk[i] = ck[i];
        pk1[i] = ck1[i];
      }
    }
  }
}

// Filter backprop, stage 1 (src/depthwise_conv2d/kernels.h:259-360 computes the same sum with
// a work-group reduction): dW[r,s,f] = sum_{n,oh,ow} x[n,oh*st-pad+r,ow*st-pad+s,c] * dy[n,oh,ow,f].
// blockIdx.x = slice of the N*Ho*Wo pixels, blockIdx.y = tap, blockIdx.z = tile of 32*V features.
// threadIdx.x walks feature packets (coalesced), threadIdx.y walks pixels; the 8 pixel lanes are
// summed through shared memory and the block writes partial[slice][tap][f] in fp32.
constexpr int kFbpLanesF = 32, kFbpLanesP = 8;

template <typename T, int V>
__global__ void __launch_bounds__(kFbpLanesF* kFbpLanesP)
    depthwise_filter_backprop_partial_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                                             float* __restrict__ partial, PdnnDepthwiseConv2DParams p,
                                             long long pixels_per_slice) {
  __shared__ float red[kFbpLanesP][kFbpLanesF][V];
  const int M = p.channel_multiplier, F = p.channels * M;
  const int tap = blockIdx.y, r = tap / p.window_cols, s = tap % p.window_cols;
  const int f = (blockIdx.z * kFbpLanesF + threadIdx.x) * V;
  const long long pixels = (long long)p.batch * p.out_rows * p.out_cols;
  const long long begin = (long long)blockIdx.x * pixels_per_slice;
  const long long end = begin + pixels_per_slice < pixels ? begin + pixels_per_slice : pixels;
  float acc[V];
#pragma unroll
  for (int i = 0; i < V; ++i) acc[i] = 0.f;
  if (f < F) {
    const int c = (V == 1) ? f / M : f;
    for (long long pix = begin + threadIdx.y; pix < end; pix += kFbpLanesP) {
      const int ow = (int)(pix % p.out_cols);
      const long long t = pix / p.out_cols;
      const int oh = (int)(t % p.out_rows);
      const int n = (int)(t / p.out_rows);
      const int ih = oh * p.stride_rows - p.pad_rows + r, iw = ow * p.stride_cols - p.pad_cols + s;
      if (ih < 0 || ih >= p.in_rows || iw < 0 || iw >= p.in_cols) continue;
      float xv[V], dv[V];
      load_vec<T, V>(x + (((size_t)n * p.in_rows + ih) * p.in_cols + iw) * p.channels + c, xv);
      load_vec<T, V>(dy + (size_t)pix * F + f, dv);
#pragma unroll
      for (int i = 0; i < V; ++i) acc[i] = fmaf(xv[i], dv[i], acc[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < V; ++i) red[threadIdx.y][threadIdx.x][i] = acc[i];
  __syncthreads();
  if (threadIdx.y == 0 && f < F) {
#pragma unroll
    for (int i = 0; i < V; ++i) {
      float sum = 0.f;
#pragma unroll
      for (int l = 0; l < kFbpLanesP; ++l) sum += red[l][threadIdx.x][i];
      partial[((size_t)blockIdx.x * gridDim.y + tap) * F + f + i] = sum;
    }
  }
}

// The same for a 3x3 window and one packet of channels per thread, all nine taps in one block:
// dy is read once and the nine x packets of a pixel come from the same few cache lines, instead
// of both tensors being streamed once per tap.  partial[slice][tap][f] as above.
template <typename T, int V>
__global__ void __launch_bounds__(kFbpLanesF* kFbpLanesP)
    depthwise_filter_backprop_partial9_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                                              float* __restrict__ partial, PdnnDepthwiseConv2DParams p,
                                              long long pixels_per_slice) {
  __shared__ float red[kFbpLanesP * kFbpLanesF][V];  // [pixel lane][channel lane], blockDim.y x blockDim.x
  const int F = p.channels;  // channel multiplier 1
  const int lanes_f = blockDim.x, lanes_p = blockDim.y;
  const int f = (blockIdx.z * lanes_f + threadIdx.x) * V;
  const long long pixels = (long long)p.batch * p.out_rows * p.out_cols;
  const long long begin = (long long)blockIdx.x * pixels_per_slice;
  const long long end = begin + pixels_per_slice < pixels ? begin + pixels_per_slice : pixels;
  float acc[9][V];
#pragma unroll
  for (int t = 0; t < 9; ++t)
#pragma unroll
    for (int i = 0; i < V; ++i) acc[t][i] = 0.f;
  if (f < F) {
    // pixel coordinates advance with the loop instead of being decoded every time
    long long pix = begin + threadIdx.y;
    int ow = (int)(pix % p.out_cols);
    long long tt = pix / p.out_cols;
    int oh = (int)(tt % p.out_rows);
    int n = (int)(tt / p.out_rows);
    for (; pix < end; pix += lanes_p) {
      float dv[V];
      load_vec<T, V>(dy + (size_t)pix * F + f, dv);
      const int ih0 = oh * p.stride_rows - p.pad_rows, iw0 = ow * p.stride_cols - p.pad_cols;
      const T* xn = x + (size_t)n * p.in_rows * p.in_cols * p.channels + f;
      // Loads are made unconditional (coordinates clamped into the image, the product masked)
      // and issued a row at a time, so that they overlap instead of each waiting behind a branch.
#pragma unroll
      for (int r = 0; r < 3; ++r) {
        const int ih = ih0 + r;
        const bool row_ok = ih >= 0 && ih < p.in_rows;
        const T* xr = xn + (size_t)min(max(ih, 0), p.in_rows - 1) * p.in_cols * p.channels;
        float xv[3][V];
#pragma unroll
        for (int c = 0; c < 3; ++c) load_vec<T, V>(xr + (size_t)min(max(iw0 + c, 0), p.in_cols - 1) * p.channels, xv[c]);
#pragma unroll
        for (int c = 0; c < 3; ++c) {
          const bool ok = row_ok && iw0 + c >= 0 && iw0 + c < p.in_cols;
#pragma unroll
          for (int i = 0; i < V; ++i) acc[r * 3 + c][i] = fmaf(ok ? xv[c][i] : 0.f, dv[i], acc[r * 3 + c][i]);
        }
      }
      ow += lanes_p;
      while (ow >= p.out_cols) {
        ow -= p.out_cols;
        if (++oh == p.out_rows) {
          oh = 0;
          ++n;
        }
      }
    }
  }
  // Reduction over the block's pixel lanes: first across the pixel lanes that share a warp
  // (a warp is lanes_f channel lanes x 32 / lanes_f pixel lanes) by shuffles, then across the
  // eight warps through shared memory.
  const int tid = threadIdx.y * lanes_f + threadIdx.x, warp = tid >> 5, lane = tid & 31;
#pragma unroll
  for (int t = 0; t < 9; ++t) {
#pragma unroll
    for (int i = 0; i < V; ++i) {
      float v = acc[t][i];
      for (int off = lanes_f; off < 32; off <<= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
      acc[t][i] = v;
    }
    if (lane < lanes_f) {
#pragma unroll
      for (int i = 0; i < V; ++i) red[warp * 32 + lane][i] = acc[t][i];
    }
    __syncthreads();
    if (warp == 0 && lane < lanes_f && f < F) {
#pragma unroll
      for (int i = 0; i < V; ++i) {
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < kFbpLanesF * kFbpLanesP / 32; ++w) sum += red[w * 32 + lane][i];
        partial[((size_t)blockIdx.x * 9 + t) * F + f + i] = sum;
      }
    }
    __syncthreads();
  }
}

// The 3x3 filter gradient with one 32-bit word of channels per lane (two 16-bit channels or one
// fp32 channel): a warp covers 128 contiguous bytes of a pixel, walks whole output rows and keeps
// the 9 x (1 or 2) sums of its channels in registers across all its rows.  Few registers, so the SM
// holds enough warps to cover the load latency (the packet form above keeps 72 sums per thread and
// runs at one block per SM), and every load instruction of a warp is one full line.  The 3x3 window
// of x slides along the row.  partial[slice][tap][f] as above; a
// block is eight warps of one channel group, slice = blockIdx.x.
template <typename T>
struct WordOf;
template <>
struct WordOf<float> {
  static constexpr int E = 1;
  static __device__ __forceinline__ void unpack(unsigned w, float (&v)[1]) { v[0] = __uint_as_float(w); }
  // acc += a * b, element by element, on packed words
  static __device__ __forceinline__ void fma(float (&acc)[1], unsigned a, unsigned b) {
    acc[0] = fmaf(__uint_as_float(a), __uint_as_float(b), acc[0]);
  }
};
template <>
struct WordOf<__half> {
  static constexpr int E = 2;
  static __device__ __forceinline__ void unpack(unsigned w, float (&v)[2]) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
    v[0] = f.x;
    v[1] = f.y;
  }
  // The mixed-precision multiply-add takes the 16-bit operands as they are (the product of two halves
  // is exact in fp32, so the result equals convert-then-fmaf): no conversions, and the window stays
  // packed, one register per word.  Measured against unpacking on arrival (two conversions per word,
  // fp32 window): 0.113 -> 0.098 ms on 56x56x144; the packed fp32 multiply-add (two lanes per
  // instruction on an unpacked window) was slower than either.
  static __device__ __forceinline__ void fma(float (&acc)[2], unsigned a, unsigned b) {
    asm("{\n\t.reg .b16 al, ah, bl, bh;\n\t"
        "mov.b32 {al, ah}, %2;\n\tmov.b32 {bl, bh}, %3;\n\t"
        "fma.rn.f32.f16 %0, al, bl, %0;\n\tfma.rn.f32.f16 %1, ah, bh, %1;\n\t}"
        : "+f"(acc[0]), "+f"(acc[1])
        : "r"(a), "r"(b));
  }
};
template <>
struct WordOf<__nv_bfloat16> {
  static constexpr int E = 2;
  static __device__ __forceinline__ void unpack(unsigned w, float (&v)[2]) {
    v[0] = __uint_as_float(w << 16);
    v[1] = __uint_as_float(w & 0xFFFF0000u);
  }
  static __device__ __forceinline__ void fma(float (&acc)[2], unsigned a, unsigned b) {
    asm("{\n\t.reg .b16 al, ah, bl, bh;\n\t"
        "mov.b32 {al, ah}, %2;\n\tmov.b32 {bl, bh}, %3;\n\t"
        "fma.rn.f32.bf16 %0, al, bl, %0;\n\tfma.rn.f32.bf16 %1, ah, bh, %1;\n\t}"
        : "+f"(acc[0]), "+f"(acc[1])
        : "r"(a), "r"(b));
  }
};

constexpr int kFbpRowsWarps = 8, kFbpRowsBlocks = 3;  // 80 registers per thread, 24 warps per SM
template <typename T, int ST>
__global__ void __launch_bounds__(kFbpRowsWarps * 32, kFbpRowsBlocks)
    depthwise_filter_backprop_rows_kernel(const T* __restrict__ x, const T* __restrict__ dy, float* __restrict__ partial,
                                          PdnnDepthwiseConv2DParams p, int segs, int seg_cols, int per_full, int per_tail) {
  constexpr int E = WordOf<T>::E;
  // U output columns per trip: their ST * U new input columns and U dy words are requested together
  // (a warp has to keep a dozen lines in flight to cover the latency), the CARRY columns the next
  // trip's first window shares with this one stay in registers.
  constexpr int U = ST == 1 ? 4 : 2, CARRY = 3 - ST, NEW = U * ST;
  __shared__ float red[kFbpRowsWarps][9 * E][32];
  const int F = p.channels, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned wstride = (unsigned)(F / E);  // 32-bit words per pixel
  // The last block of words may be narrow (72 words per pixel leave 8): up to 16 words wide it takes
  // several rows side by side, rows_here of them, lane = row * words_here + word; otherwise idle lanes
  // repeat the last word.
  // The grid is one row of blocks: per_full blocks for each full block of 32 words, per_tail for the last
  // block of words (which has less to do when it packs rows); block bx of nbx works on word block by and
  // writes slice bx of the partial sums.
  const int groups = ((int)wstride + 31) / 32;
  const int by = min((int)blockIdx.x / per_full, groups - 1), bx = (int)blockIdx.x - by * per_full;
  const int nbx = by == groups - 1 ? per_tail : per_full;
  const int first_word = by * 32, words_here = min(32, (int)wstride - first_word);
  const int rows_here = words_here <= 16 ? 32 / words_here : 1;
  const int sub = rows_here > 1 ? lane / words_here : 0;
  const unsigned lw = (unsigned)(first_word + (rows_here > 1 ? lane % words_here : min(lane, words_here - 1)));
  // 32-bit word indices from the tensors' bases (the host only takes this path below 2^32 words)
  const unsigned* __restrict__ xw = reinterpret_cast<const unsigned*>(x);
  const unsigned* __restrict__ dw = reinterpret_cast<const unsigned*>(dy);
  float acc[9][E];
#pragma unroll
  for (int t = 0; t < 9; ++t)
#pragma unroll
    for (int e = 0; e < E; ++e) acc[t][e] = 0.f;
  // A unit of work is one segment (seg_cols columns, a multiple of U) of one output row: whole rows
  // are too coarse to spread evenly over a wave of warps (6.05 rows per warp cost as much as 7).
  const unsigned all_rows = (unsigned)(p.batch * p.out_rows);
  const unsigned units = ((all_rows + (unsigned)rows_here - 1u) / (unsigned)rows_here) * (unsigned)segs;
  for (unsigned u = (unsigned)bx * (unsigned)kFbpRowsWarps + (unsigned)warp; u < units; u += (unsigned)nbx * (unsigned)kFbpRowsWarps) {
    const int seg = (int)(u % (unsigned)segs);
    const unsigned want_row = (u / (unsigned)segs) * (unsigned)rows_here + (unsigned)sub;
    // a lane without a row (beyond the last one, or beyond the rows a warp packs) walks the last row and adds zeros
    const bool dead = sub >= rows_here || want_row >= all_rows;
    const unsigned row = min(want_row, all_rows - 1u);
    const int oh = (int)(row % (unsigned)p.out_rows), n = (int)(row / (unsigned)p.out_rows);
    const int ow_begin = seg * seg_cols, ow_end = min(ow_begin + seg_cols, p.out_cols);
    const int ih0 = oh * ST - p.pad_rows;
    const bool rows_inside = !dead && ih0 >= 0 && ih0 + 2 < p.in_rows;
    unsigned xrow[3];  // word index of column 0 of the three input rows (clamped into the image)
    bool rok[3];
#pragma unroll
    for (int r = 0; r < 3; ++r) {
      const int ih = ih0 + r;
      rok[r] = ih >= 0 && ih < p.in_rows;
      xrow[r] = (unsigned)((n * p.in_rows + min(max(ih, 0), p.in_rows - 1)) * p.in_cols) * wstride + lw;
    }
    const unsigned drow = (unsigned)((n * p.out_rows + oh) * p.out_cols) * wstride + lw;
    // The window stays packed (one register per pixel and row); words from outside the tensors are
    // requested at a clamped index and replaced by zero.
    unsigned win[CARRY + NEW][3];
    auto fetch_col = [&](int iw, unsigned (&col)[3]) {
      const unsigned off = (unsigned)min(max(iw, 0), p.in_cols - 1) * wstride;
#pragma unroll
      for (int r = 0; r < 3; ++r) col[r] = __ldg(xw + xrow[r] + off);
    };
    auto zero_outside = [&](int iw, unsigned (&col)[3]) {
      const bool cok = iw >= 0 && iw < p.in_cols;
#pragma unroll
      for (int r = 0; r < 3; ++r)
        if (!(cok && rok[r])) col[r] = 0u;
    };
#pragma unroll
    for (int k = 0; k < CARRY; ++k) {
      fetch_col(ow_begin * ST - p.pad_cols + k, win[k]);
      zero_outside(ow_begin * ST - p.pad_cols + k, win[k]);
    }
    // The words of a trip are requested one trip ahead, so that their latency passes behind the
    // previous trip's arithmetic (16 requests per lane in flight).
    unsigned nx[NEW][3], nd[U];
    auto interior = [&](int ow) {
      const int iw_new = ow * ST - p.pad_cols + CARRY;
      return rows_inside && iw_new >= 0 && iw_new + NEW <= p.in_cols && ow + U <= p.out_cols;
    };
    auto fetch = [&](int ow) {
      const int iw_new = ow * ST - p.pad_cols + CARRY;
      if (interior(ow)) {  // no clamps, one index addition per load
        unsigned off = (unsigned)iw_new * wstride;
#pragma unroll
        for (int j = 0; j < NEW; ++j, off += wstride)
#pragma unroll
          for (int r = 0; r < 3; ++r) nx[j][r] = __ldg(xw + xrow[r] + off);
        unsigned doff = drow + (unsigned)ow * wstride;
#pragma unroll
        for (int uu = 0; uu < U; ++uu, doff += wstride) nd[uu] = __ldg(dw + doff);
      } else {
#pragma unroll
        for (int j = 0; j < NEW; ++j) fetch_col(iw_new + j, nx[j]);
#pragma unroll
        for (int uu = 0; uu < U; ++uu) nd[uu] = __ldg(dw + drow + (unsigned)min(ow + uu, p.out_cols - 1) * wstride);
      }
    };
    fetch(ow_begin);
    for (int ow = ow_begin; ow < ow_end; ow += U) {
      const int iw_new = ow * ST - p.pad_cols + CARRY;
      unsigned dv[U];
#pragma unroll
      for (int j = 0; j < NEW; ++j)
#pragma unroll
        for (int r = 0; r < 3; ++r) win[CARRY + j][r] = nx[j][r];
#pragma unroll
      for (int uu = 0; uu < U; ++uu) dv[uu] = nd[uu];
      if (!interior(ow)) {
#pragma unroll
        for (int j = 0; j < NEW; ++j) zero_outside(iw_new + j, win[CARRY + j]);
#pragma unroll
        for (int uu = 0; uu < U; ++uu)
          if (dead || ow + uu >= p.out_cols) dv[uu] = 0u;
      }
      if (ow + U < ow_end) fetch(ow + U);
#pragma unroll
      for (int uu = 0; uu < U; ++uu)
#pragma unroll
        for (int r = 0; r < 3; ++r)
#pragma unroll
          for (int c3 = 0; c3 < 3; ++c3) WordOf<T>::fma(acc[r * 3 + c3], win[uu * ST + c3][r], dv[uu]);
#pragma unroll
      for (int k = 0; k < CARRY; ++k)
#pragma unroll
        for (int r = 0; r < 3; ++r) win[k][r] = win[NEW + k][r];
    }
  }
#pragma unroll
  for (int t = 0; t < 9; ++t)
#pragma unroll
    for (int e = 0; e < E; ++e) red[warp][t * E + e][lane] = acc[t][e];
  __syncthreads();
  for (int i = threadIdx.x; i < 9 * E * words_here; i += kFbpRowsWarps * 32) {
    const int wd = i % words_here, te = i / words_here, t = te / E, e = te % E;
    const int ch = (first_word + wd) * E + e;
    float sum = 0.f;
    for (int r = 0; r < rows_here; ++r)
#pragma unroll
      for (int w = 0; w < kFbpRowsWarps; ++w) sum += red[w][te][r * words_here + wd];
    partial[((size_t)bx * 9 + t) * F + ch] = sum;
    // the slices that only the full word blocks fill hold zeros for these channels
    for (int slice = bx + nbx; slice < per_full; slice += nbx) partial[((size_t)slice * 9 + t) * F + ch] = 0.f;
  }
}

// Stage 2: dW[i] = sum over slices of partial[slice][i], in slice order (deterministic).
template <typename T>
__global__ void __launch_bounds__(kBlock)
    reduce_slices_kernel(const float* __restrict__ partial, T* __restrict__ out, int slices, size_t n) {
  for (size_t i = (size_t)blockIdx.x * kBlock + threadIdx.x; i < n; i += (size_t)gridDim.x * kBlock) {
    float sum = 0.f;
    for (int sl = 0; sl < slices; ++sl) sum += partial[(size_t)sl * n + i];
    out[i] = from_f32<T>(sum);
  }
}

// ------------------------------------------------------------------------------------------
// Pointwise, bias, blend
// ------------------------------------------------------------------------------------------
// src/pointwise/kernels.h:47-137: the activations plus exp, log, floor and sqrt.
__device__ __forceinline__ float pointwise_forward_value(float v, int op) {
  switch (op) {
    case PDNN_PW_EXP: return expf(v);
    case PDNN_PW_LOG: return logf(v);
    case PDNN_PW_FLOOR: return floorf(v);
    case PDNN_PW_SQRT: return sqrtf(v);
    default: return apply_activation(v, op);
  }
}
// v is the forward output, e the incoming gradient (src/pointwise/kernels.h:53-137, 205-233); the
// exp case is the reference's formula as it stands (exp(v) + e, kernels.h:94-101).
__device__ __forceinline__ float pointwise_grad_value(float v, float e, int op) {
  switch (op) {
    case PDNN_ACT_RELU: return v > 0.f ? e : 0.f;
    case PDNN_ACT_TANH: return (1.f - v * v) * e;
    case PDNN_PW_EXP: return expf(v) + e;
    case PDNN_PW_LOG: return (1.f / v) * e;
    case PDNN_PW_SQRT: return (0.5f / v) * e;
    default: return (v > 0.f && v < 6.f) ? e : 0.f;  // ReLU6
  }
}

template <typename T, int V, int MODE>  // MODE 0: forward, 1: gradient
__global__ void __launch_bounds__(kBlock)
    pointwise_kernel(int op, const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, size_t n_packets) {
  for (size_t i = (size_t)blockIdx.x * kBlock + threadIdx.x; i < n_packets; i += (size_t)gridDim.x * kBlock) {
    float av[V], res[V];
    load_vec<T, V>(a + i * V, av);
    if (MODE == 0) {
#pragma unroll
      for (int j = 0; j < V; ++j) res[j] = pointwise_forward_value(av[j], op);
    } else {
      float bv[V];
      load_vec<T, V>(b + i * V, bv);
#pragma unroll
      for (int j = 0; j < V; ++j) res[j] = pointwise_grad_value(av[j], bv[j], op);
    }
    store_vec<T, V>(out + i * V, res);
  }
}

template <typename T, int V>
__global__ void __launch_bounds__(kBlock) bias_add_kernel(const T* __restrict__ in, const T* __restrict__ bias,
                                                          T* __restrict__ out, size_t n_packets, int cvecs, int act) {
  for (size_t i = (size_t)blockIdx.x * kBlock + threadIdx.x; i < n_packets; i += (size_t)gridDim.x * kBlock) {
    float v[V], b[V];
    load_vec<T, V>(in + i * V, v);
    load_vec<T, V>(bias + (i % cvecs) * V, b);
#pragma unroll
    for (int j = 0; j < V; ++j) v[j] = apply_activation(to_f32(from_f32<T>(v[j] + b[j])), act);  // sum rounded to T first, as two passes would
    store_vec<T, V>(out + i * V, v);
  }
}

template <typename T, int V>
__global__ void __launch_bounds__(kBlock) scale_blend_kernel(const T* __restrict__ a, float alpha, const T* __restrict__ b,
                                                             float beta, T* __restrict__ out, size_t n_packets) {
  for (size_t i = (size_t)blockIdx.x * kBlock + threadIdx.x; i < n_packets; i += (size_t)gridDim.x * kBlock) {
    float av[V], res[V];
    load_vec<T, V>(a + i * V, av);
    if (b != nullptr) {
      float bv[V];
      load_vec<T, V>(b + i * V, bv);
      // Rounded separately, like the reference's Mul, Mul, Add passes
      // (include/portdnn/compat/scaling.hpp:202-259).
#pragma unroll
      for (int j = 0; j < V; ++j)
        res[j] = __fadd_rn(to_f32(from_f32<T>(__fmul_rn(alpha, av[j]))), to_f32(from_f32<T>(__fmul_rn(beta, bv[j]))));
    } else {
#pragma unroll
      for (int j = 0; j < V; ++j) res[j] = __fmul_rn(alpha, av[j]);
    }
    store_vec<T, V>(out + i * V, res);
  }
}

// ------------------------------------------------------------------------------------------
// 3x3 windows, register-tiled: the overlapping-window operators above issue nine input loads per
// output packet and are bound by L1 wavefronts long before HBM.  Here a thread owns one channel
// packet and a strip of four output columns, walks down the output rows and keeps the three
// input rows it needs in registers (one new row per step at stride 1, two at stride 2), so each
// input packet is loaded once per strip instead of up to nine times.  Arithmetic is done on the
// packet in its own type: half2 FMAs / maxima for fp16 (the reference also accumulates in the
// tensor type), plain fp32 for float.
// ------------------------------------------------------------------------------------------
template <typename T>
struct Packet;
template <>
struct Packet<__half> {
  __half2 v[4];
  static __device__ __forceinline__ Packet load(const __half* p) {
    const uint4 r = __ldg(reinterpret_cast<const uint4*>(p));
    Packet o;
    o.v[0] = *reinterpret_cast<const __half2*>(&r.x);
    o.v[1] = *reinterpret_cast<const __half2*>(&r.y);
    o.v[2] = *reinterpret_cast<const __half2*>(&r.z);
    o.v[3] = *reinterpret_cast<const __half2*>(&r.w);
    return o;
  }
  static __device__ __forceinline__ Packet from_raw(const uint4& r) {
    Packet o;
    o.v[0] = *reinterpret_cast<const __half2*>(&r.x);
    o.v[1] = *reinterpret_cast<const __half2*>(&r.y);
    o.v[2] = *reinterpret_cast<const __half2*>(&r.z);
    o.v[3] = *reinterpret_cast<const __half2*>(&r.w);
    return o;
  }
  static __device__ __forceinline__ Packet splat(float f) {
    Packet o;
#pragma unroll
    for (int i = 0; i < 4; ++i) o.v[i] = __float2half2_rn(f);
    return o;
  }
  __device__ __forceinline__ void fma(const Packet& a, const Packet& b) {
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = __hfma2(a.v[i], b.v[i], v[i]);
  }
  __device__ __forceinline__ void max_ignore_nan(const Packet& a) {
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = __hmax2(v[i], a.v[i]);
  }
  __device__ __forceinline__ void max_keep_nan(const Packet& a) {
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = __hmax2_nan(v[i], a.v[i]);
  }
  // Winner bookkeeping of the max-pool gradient: wherever this packet equals `m` (or both are NaN,
  // keep_nan), the two 16-bit lanes of win[i] take `id`.  Visiting the window backwards leaves the
  // first match.
  __device__ __forceinline__ void mark_equal(const Packet& m, unsigned id, bool keep_nan, unsigned (&win)[4]) const {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      unsigned mask = __heq2_mask(v[i], m.v[i]);
      if (keep_nan) mask |= __hneu2_mask(v[i], v[i]) & __hneu2_mask(m.v[i], m.v[i]);
      win[i] = (win[i] & ~mask) | ((id * 0x00010001u) & mask);
    }
  }
  // Clears the winner wherever the maximum `m` is not positive (the ReLU gradient of the pooled tensor).
  static __device__ __forceinline__ void keep_positive(const Packet& m, unsigned (&win)[4]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) win[i] &= __hgt2_mask(m.v[i], splat(0.f).v[0]);
  }
  static __device__ __forceinline__ void store_winners(unsigned char* p, const unsigned (&win)[4]) {
    *reinterpret_cast<uint2*>(p) = make_uint2(__byte_perm(win[0], win[1], 0x6420), __byte_perm(win[2], win[3], 0x6420));
  }
  __device__ __forceinline__ void store(__half* p) const {
    uint4 r;
    r.x = *reinterpret_cast<const uint32_t*>(&v[0]);
    r.y = *reinterpret_cast<const uint32_t*>(&v[1]);
    r.z = *reinterpret_cast<const uint32_t*>(&v[2]);
    r.w = *reinterpret_cast<const uint32_t*>(&v[3]);
    *reinterpret_cast<uint4*>(p) = r;
  }
};
template <>
struct Packet<__nv_bfloat16> {  // maxima only: bf16 products would lose too much in a packed sum
  __nv_bfloat162 v[4];
  static __device__ __forceinline__ Packet load(const __nv_bfloat16* p) {
    const uint4 r = __ldg(reinterpret_cast<const uint4*>(p));
    Packet o;
    o.v[0] = *reinterpret_cast<const __nv_bfloat162*>(&r.x);
    o.v[1] = *reinterpret_cast<const __nv_bfloat162*>(&r.y);
    o.v[2] = *reinterpret_cast<const __nv_bfloat162*>(&r.z);
    o.v[3] = *reinterpret_cast<const __nv_bfloat162*>(&r.w);
    return o;
  }
  static __device__ __forceinline__ Packet splat(float f) {
    Packet o;
#pragma unroll
    for (int i = 0; i < 4; ++i) o.v[i] = __float2bfloat162_rn(f);
    return o;
  }
  __device__ __forceinline__ void max_ignore_nan(const Packet& a) {
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = __hmax2(v[i], a.v[i]);
  }
  __device__ __forceinline__ void max_keep_nan(const Packet& a) {
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = __hmax2_nan(v[i], a.v[i]);
  }
  // Winner bookkeeping of the max-pool gradient: wherever this packet equals `m` (or both are NaN,
  // keep_nan), the two 16-bit lanes of win[i] take `id`.  Visiting the window backwards leaves the
  // first match.
  __device__ __forceinline__ void mark_equal(const Packet& m, unsigned id, bool keep_nan, unsigned (&win)[4]) const {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      unsigned mask = __heq2_mask(v[i], m.v[i]);
      if (keep_nan) mask |= __hneu2_mask(v[i], v[i]) & __hneu2_mask(m.v[i], m.v[i]);
      win[i] = (win[i] & ~mask) | ((id * 0x00010001u) & mask);
    }
  }
  // Clears the winner wherever the maximum `m` is not positive (the ReLU gradient of the pooled tensor).
  static __device__ __forceinline__ void keep_positive(const Packet& m, unsigned (&win)[4]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) win[i] &= __hgt2_mask(m.v[i], splat(0.f).v[0]);
  }
  static __device__ __forceinline__ void store_winners(unsigned char* p, const unsigned (&win)[4]) {
    *reinterpret_cast<uint2*>(p) = make_uint2(__byte_perm(win[0], win[1], 0x6420), __byte_perm(win[2], win[3], 0x6420));
  }
  __device__ __forceinline__ void store(__nv_bfloat16* p) const {
    uint4 r;
    r.x = *reinterpret_cast<const uint32_t*>(&v[0]);
    r.y = *reinterpret_cast<const uint32_t*>(&v[1]);
    r.z = *reinterpret_cast<const uint32_t*>(&v[2]);
    r.w = *reinterpret_cast<const uint32_t*>(&v[3]);
    *reinterpret_cast<uint4*>(p) = r;
  }
};
template <>
struct Packet<float> {
  float v[4];
  static __device__ __forceinline__ Packet load(const float* p) {
    const float4 r = __ldg(reinterpret_cast<const float4*>(p));
    Packet o;
    o.v[0] = r.x;
    o.v[1] = r.y;
    o.v[2] = r.z;
    o.v[3] = r.w;
    return o;
  }
  static __device__ __forceinline__ Packet from_raw(const uint4& r) {
    Packet o;
    o.v[0] = __uint_as_float(r.x);
    o.v[1] = __uint_as_float(r.y);
    o.v[2] = __uint_as_float(r.z);
    o.v[3] = __uint_as_float(r.w);
    return o;
  }
  static __device__ __forceinline__ Packet splat(float f) {
    Packet o;
#pragma unroll
    for (int i = 0; i < 4; ++i) o.v[i] = f;
    return o;
  }
  __device__ __forceinline__ void fma(const Packet& a, const Packet& b) {
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = fmaf(a.v[i], b.v[i], v[i]);
  }
  __device__ __forceinline__ void max_ignore_nan(const Packet& a) {
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = a.v[i] > v[i] ? a.v[i] : v[i];
  }
  __device__ __forceinline__ void max_keep_nan(const Packet& a) {
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = (isnan(a.v[i]) || a.v[i] > v[i]) ? a.v[i] : v[i];
  }
  __device__ __forceinline__ void mark_equal(const Packet& m, unsigned id, bool keep_nan, unsigned (&win)[4]) const {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (v[i] == m.v[i] || (keep_nan && isnan(v[i]) && isnan(m.v[i]))) win[i] = id;
  }
  static __device__ __forceinline__ void keep_positive(const Packet& m, unsigned (&win)[4]) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (!(m.v[i] > 0.f)) win[i] = 0u;
  }
  static __device__ __forceinline__ void store_winners(unsigned char* p, const unsigned (&win)[4]) {
    *reinterpret_cast<unsigned*>(p) = win[0] | (win[1] << 8) | (win[2] << 16) | (win[3] << 24);
  }
  __device__ __forceinline__ void store(float* p) const {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};

// Output columns per thread: four at stride 1 (six input columns feed four windows); two at stride
// 2, where neighbouring windows share only one input column and the registers are better spent on
// more threads in flight (measured: 3x3/2 max pool 0.103 -> 0.090 ms, stride-2 depthwise 8% faster).
template <int ST>
struct StripWidth {
  static constexpr int value = ST == 2 ? 2 : 4;
};
constexpr int kStripBlock = 128;

struct StripGeometry {
  int in_rows, in_cols, out_rows, out_cols, channels, pad_rows, pad_cols, batch;
  int rows_per_thread, wgroups, hchunks;
  int flip;  // MODE 0: read the filter mirrored in both window axes (stride-1 input backprop)
  int positive_only;  // MODE 3 / 4: a window whose maximum is not positive has no winner
};

// MODE 0: depthwise 3x3 (needs Packet::fma); MODE 1: max ignoring NaN; MODE 2: max keeping NaN;
// MODE 3 / 4: as 1 / 2, but instead of the maximum the kernel writes, one byte per element, which
// element of the window is the first to equal it (1 + row * 3 + col, the winner map of the max-pool
// gradient); y then points at bytes.
template <typename T, int ST, int MODE>
__global__ void __launch_bounds__(kStripBlock)
    window3_strip_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y, StripGeometry g,
                         size_t n_threads) {
  using P = Packet<T>;
  constexpr int V = 16 / sizeof(T);
  constexpr int kStripW = StripWidth<ST>::value;
  constexpr int NIN = (kStripW - 1) * ST + 3;
  const size_t idx = (size_t)blockIdx.x * kStripBlock + threadIdx.x;
  if (idx >= n_threads) return;
  const int cvecs = g.channels / V;
  const int cv = (int)(idx % cvecs);
  size_t t = idx / cvecs;
  const int wg = (int)(t % g.wgroups);
  t /= g.wgroups;
  const int hc = (int)(t % g.hchunks);
  const int n = (int)(t / g.hchunks);
  const int c = cv * V;
  const int ow0 = wg * kStripW, iw0 = ow0 * ST - g.pad_cols;
  const int oh_begin = hc * g.rows_per_thread, oh_end = min(oh_begin + g.rows_per_thread, g.out_rows);
  const T* xn = x + (size_t)n * g.in_rows * g.in_cols * g.channels + c;
  T* yn = y + (size_t)n * g.out_rows * g.out_cols * g.channels + c;
  const float fill = MODE == 0 ? 0.f : lowest_of<T>();

  P wt[MODE == 0 ? 3 : 1][3];
  if constexpr (MODE == 0) {
#pragma unroll
    for (int r = 0; r < 3; ++r)
#pragma unroll
      for (int s2 = 0; s2 < 3; ++s2)
        wt[r][s2] = P::load(w + (size_t)(g.flip ? (2 - r) * 3 + (2 - s2) : r * 3 + s2) * g.channels + c);
  }
  auto load_row = [&](P (&row)[NIN], int ih) {
    const bool row_ok = ih >= 0 && ih < g.in_rows;
    const T* xr = xn + (size_t)ih * g.in_cols * g.channels;
#pragma unroll
    for (int j = 0; j < NIN; ++j) {
      const int iw = iw0 + j;
      row[j] = (row_ok && iw >= 0 && iw < g.in_cols) ? P::load(xr + (size_t)iw * g.channels) : P::splat(fill);
    }
  };
  P ra[NIN], rb[NIN], rc[NIN];
  int ih0 = oh_begin * ST - g.pad_rows;
  load_row(ra, ih0);
  load_row(rb, ih0 + 1);
  load_row(rc, ih0 + 2);
  for (int oh = oh_begin; oh < oh_end; ++oh) {
    // stride 1: the one new row of the next step is requested before this step's arithmetic, so
    // that its latency hides behind it
    P rn[ST == 1 ? NIN : 1];
    if (ST == 1 && oh + 1 < oh_end) load_row(reinterpret_cast<P(&)[NIN]>(rn), ih0 + 3);
#pragma unroll
    for (int o = 0; o < kStripW; ++o) {
      P acc = P::splat(fill);
#pragma unroll
      for (int s2 = 0; s2 < 3; ++s2) {
        if constexpr (MODE == 0) {
          acc.fma(ra[o * ST + s2], wt[0][s2]);
          acc.fma(rb[o * ST + s2], wt[1][s2]);
          acc.fma(rc[o * ST + s2], wt[2][s2]);
        } else if constexpr (MODE == 1 || MODE == 3) {
          acc.max_ignore_nan(ra[o * ST + s2]);
          acc.max_ignore_nan(rb[o * ST + s2]);
          acc.max_ignore_nan(rc[o * ST + s2]);
        } else {
          acc.max_keep_nan(ra[o * ST + s2]);
          acc.max_keep_nan(rb[o * ST + s2]);
          acc.max_keep_nan(rc[o * ST + s2]);
        }
      }
      if constexpr (MODE >= 3) {
        // the window backwards, so that the first element equal to the maximum is the one that stays;
        // elements outside the image never win
        unsigned win[4] = {0u, 0u, 0u, 0u};
#pragma unroll
        for (int r = 2; r >= 0; --r) {
          const int ih = ih0 + r;
          if (ih < 0 || ih >= g.in_rows) continue;
#pragma unroll
          for (int s2 = 2; s2 >= 0; --s2) {
            const int iw = iw0 + o * ST + s2;
            if (iw < 0 || iw >= g.in_cols) continue;
            const P& e = r == 0 ? ra[o * ST + s2] : r == 1 ? rb[o * ST + s2] : rc[o * ST + s2];
            e.mark_equal(acc, (unsigned)(1 + r * 3 + s2), MODE == 4, win);
          }
        }
        if (g.positive_only) P::keep_positive(acc, win);
        if (ow0 + o < g.out_cols)
          P::store_winners(reinterpret_cast<unsigned char*>(y) +
                               (((size_t)n * g.out_rows + oh) * g.out_cols + ow0 + o) * g.channels + c, win);
      } else {
        if (ow0 + o < g.out_cols) acc.store(yn + ((size_t)oh * g.out_cols + ow0 + o) * g.channels);
      }
    }
    if (oh + 1 < oh_end) {
      ih0 += ST;
      if (ST == 1) {
#pragma unroll
        for (int j = 0; j < NIN; ++j) {
          ra[j] = rb[j];
          rb[j] = rc[j];
          rc[j] = rn[j];
        }
      } else {
#pragma unroll
        for (int j = 0; j < NIN; ++j) ra[j] = rc[j];
        load_row(rb, ih0 + 1);
        load_row(rc, ih0 + 2);
      }
    }
  }
}

// Depthwise 3x3 as the strip walk above (MODE 0), with the rows a thread will need PF steps from now
// already on their way: every step's new rows are requested by cp.async into shared-memory slots
// of the thread's own (PF + 1 groups of ST rows; nobody else reads them, so no barrier), and only
// cp.async.wait_group stands between the request and the copy into registers.  The strip kernel
// keeps its requests in registers, which limits a thread to one row in flight and an SM to about
// 36 KB; the copies here cost no registers while they fly.  (The nine filter packets stay in
// registers: fetched from shared memory tap by tap the kernel was a quarter slower at stride 1.)
// Measured on MobileNet-v2 at batch 128 (fp16, graph replay): 112x112x32 0.064 -> 0.043 ms, 112x112x96/2
// 0.074 -> 0.067 ms, 56x56x144 0.068 -> 0.046 ms, the 17 layers 0.46 -> 0.36 ms.
template <typename T, int ST, int PF>
__global__ void __launch_bounds__(kStripBlock, 3)
    depthwise3_async_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y, StripGeometry g,
                            size_t n_threads) {
  using P = Packet<T>;
  constexpr int V = 16 / sizeof(T);
  constexpr int kStripW = StripWidth<ST>::value;
  constexpr int NIN = (kStripW - 1) * ST + 3;
  constexpr int GROUP = ST * NIN;  // packets one step brings in
  constexpr int SLOTS = PF + 1;
  constexpr uint32_t kPacketPitch = kStripBlock * 16;  // bytes between two packets of one thread
  extern __shared__ uint4 dw_async_smem[];
  // Launched with programmatic stream serialization: the blocks are placed while the preceding kernel of the
  // stream is finishing and wait here for its results; the next kernel may be placed as soon as the last of
  // these blocks has started.  (Both are no-ops under an ordinary launch.)
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const size_t idx = (size_t)blockIdx.x * kStripBlock + threadIdx.x;
  if (idx >= n_threads) return;
  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(dw_async_smem) + threadIdx.x * 16u;
  const int cvecs = g.channels / V;
  const int cv = (int)(idx % cvecs);
  size_t t = idx / cvecs;
  const int wg = (int)(t % g.wgroups);
  t /= g.wgroups;
  const int hc = (int)(t % g.hchunks);
  const int n = (int)(t / g.hchunks);
  const int c = cv * V;
  const int ow0 = wg * kStripW, iw0 = ow0 * ST - g.pad_cols;
  const int oh_begin = hc * g.rows_per_thread, oh_end = min(oh_begin + g.rows_per_thread, g.out_rows);
  const int nsteps = oh_end - oh_begin;
  const T* xn = x + (size_t)n * g.in_rows * g.in_cols * g.channels + c;
  T* yn = y + (size_t)n * g.out_rows * g.out_cols * g.channels + c;
  const int ih_first = oh_begin * ST - g.pad_rows;

  auto lds = [](uint32_t addr) {
    uint4 r;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(addr));
    return P::from_raw(r);
  };
  P wt[3][3];
#pragma unroll
  for (int r = 0; r < 3; ++r)
#pragma unroll
    for (int s2 = 0; s2 < 3; ++s2)
      wt[r][s2] = P::load(w + (size_t)(g.flip ? (2 - r) * 3 + (2 - s2) : r * 3 + s2) * g.channels + c);
  // requests the rows step k (>= 1) adds to the window; always one commit, so that the groups count steps
  auto request = [&](int k) {
    if (k < nsteps) {
      const uint32_t slot = ring + (uint32_t)((k % SLOTS) * GROUP) * kPacketPitch;
#pragma unroll
      for (int i = 0; i < ST; ++i) {
        const int ih = ih_first + 3 + (k - 1) * ST + i;
        const bool row_ok = ih >= 0 && ih < g.in_rows;
        const T* xr = xn + (size_t)(row_ok ? ih : 0) * g.in_cols * g.channels;
#pragma unroll
        for (int j = 0; j < NIN; ++j) {
          const int iw = iw0 + j;
          const bool ok = row_ok && iw >= 0 && iw < g.in_cols;
          // outside the image: zero bytes are read and the packet is filled with zeros
          asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(slot + (uint32_t)(i * NIN + j) * kPacketPitch),
                       "l"(ok ? xr + (size_t)iw * g.channels : xn), "r"(ok ? 16 : 0)
                       : "memory");
        }
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  auto load_row = [&](P (&row)[NIN], int ih) {
    const bool row_ok = ih >= 0 && ih < g.in_rows;
    const T* xr = xn + (size_t)ih * g.in_cols * g.channels;
#pragma unroll
    for (int j = 0; j < NIN; ++j) {
      const int iw = iw0 + j;
      row[j] = (row_ok && iw >= 0 && iw < g.in_cols) ? P::load(xr + (size_t)iw * g.channels) : P::splat(0.f);
    }
  };
  P ra[NIN], rb[NIN], rc[NIN];
  load_row(ra, ih_first);
  load_row(rb, ih_first + 1);
  load_row(rc, ih_first + 2);
#pragma unroll
  for (int k = 1; k <= PF; ++k) request(k);
  // One step: the window is rows r0, r1, r2; afterwards the rows the next step adds replace the ones
  // it no longer needs, in place (the callers rotate the roles instead of moving 18 packets).
  auto step = [&](int k, P (&r0)[NIN], P (&r1)[NIN], P (&r2)[NIN]) {
    const int oh = oh_begin + k;
    P acc[kStripW];
#pragma unroll
    for (int o = 0; o < kStripW; ++o) acc[o] = P::splat(0.f);
#pragma unroll
    for (int s2 = 0; s2 < 3; ++s2) {
#pragma unroll
      for (int o = 0; o < kStripW; ++o) {
        acc[o].fma(r0[o * ST + s2], wt[0][s2]);
        acc[o].fma(r1[o * ST + s2], wt[1][s2]);
        acc[o].fma(r2[o * ST + s2], wt[2][s2]);
      }
    }
#pragma unroll
    for (int o = 0; o < kStripW; ++o)
      if (ow0 + o < g.out_cols) acc[o].store(yn + ((size_t)oh * g.out_cols + ow0 + o) * g.channels);
    // The slot of step k (copied to registers one step ago and consumed just now) takes step
    // k + PF + 1; then everything but the newest PF groups has landed, step k + 1 among it.
    request(k + PF + 1);
    asm volatile("cp.async.wait_group %0;" ::"n"(PF) : "memory");
    if (k + 1 < nsteps) {
      const uint32_t slot = ring + (uint32_t)(((k + 1) % SLOTS) * GROUP) * kPacketPitch;
#pragma unroll
      for (int j = 0; j < NIN; ++j) {
        r0[j] = lds(slot + (uint32_t)j * kPacketPitch);                           // stride 1: the next window is r1, r2, r0
        if constexpr (ST == 2) r1[j] = lds(slot + (uint32_t)(NIN + j) * kPacketPitch);  // stride 2: r2, r0, r1
      }
    }
  };
#pragma unroll 1
  for (int k = 0; k < nsteps; k += 3) {
    step(k, ra, rb, rc);
    if constexpr (ST == 1) {
      if (k + 1 < nsteps) step(k + 1, rb, rc, ra);
      if (k + 2 < nsteps) step(k + 2, rc, ra, rb);
    } else {
      if (k + 1 < nsteps) step(k + 1, rc, ra, rb);
      if (k + 2 < nsteps) step(k + 2, rb, rc, ra);
    }
  }
}

template <typename T, int ST, int PF>
bool launch_depthwise3_async(const T* x, const T* w, T* y, const StripGeometry& g, size_t n_threads, unsigned blocks,
                             cudaStream_t s) {
  constexpr int NIN = (StripWidth<ST>::value - 1) * ST + 3;
  constexpr size_t kSmem = (size_t)((PF + 1) * ST * NIN) * kStripBlock * 16;
  auto kernel = depthwise3_async_kernel<T, ST, PF>;
  static bool attr_set[kMaxDevices] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= kMaxDevices) return false;
  if (!attr_set[dev]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem) != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(blocks);
  cfg.blockDim = dim3(kStripBlock);
  cfg.dynamicSmemBytes = kSmem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kernel, x, w, y, g, n_threads) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return true;
}

// Chooses how many output rows a thread walks: as many as possible while the launch still has
// enough threads to fill the device.
template <typename T, int MODE>
int launch_window3_strip(const T* x, const T* w, T* y, int stride, StripGeometry g, int sms, cudaStream_t s) {
  constexpr int V = 16 / sizeof(T);
  const int strip_w = stride == 1 ? StripWidth<1>::value : StripWidth<2>::value;
  g.wgroups = (g.out_cols + strip_w - 1) / strip_w;
  const size_t per_row_chunk = (size_t)g.batch * g.wgroups * (g.channels / V);
  int rows = 16;
  if constexpr (MODE == 0) {
    // the prefetching kernel: two waves of its 384 threads per SM, walks of at most 16 rows
    const size_t want = (size_t)sms * 768;
    const int chunks = (int)std::min<size_t>((want + per_row_chunk - 1) / per_row_chunk, (size_t)g.out_rows);
    rows = std::min(16, (g.out_rows + chunks - 1) / chunks);
  } else {
    const size_t want = (size_t)sms * 1024;
    while (rows > 1 && per_row_chunk * ((g.out_rows + rows - 1) / rows) < want) rows >>= 1;
  }
  g.rows_per_thread = rows;
  g.hchunks = (g.out_rows + rows - 1) / rows;
  const size_t n_threads = per_row_chunk * g.hchunks;
  const size_t blocks = (n_threads + kStripBlock - 1) / kStripBlock;
  if (blocks > 0x7FFFFFFFull) return -1;
  if constexpr (MODE == 0) {
    // (falls through to the strip kernel if the shared-memory attribute cannot be set)
    if (stride == 1 ? launch_depthwise3_async<T, 1, 2>(x, w, y, g, n_threads, (unsigned)blocks, s)
                    : launch_depthwise3_async<T, 2, 1>(x, w, y, g, n_threads, (unsigned)blocks, s))
      return 0;
  }
  if (stride == 1)
    window3_strip_kernel<T, 1, MODE><<<(unsigned)blocks, kStripBlock, 0, s>>>(x, w, y, g, n_threads);
  else
    window3_strip_kernel<T, 2, MODE><<<(unsigned)blocks, kStripBlock, 0, s>>>(x, w, y, g, n_threads);
  return 0;
}

// ---- dispatch helpers -------------------------------------------------------------------------
template <typename F>
int dispatch_dtype(int dtype, F&& f) {
  switch (dtype) {
    case PDNN_F32: return f(float{});
    case PDNN_F16: return f(__half{});
    case PDNN_BF16: return f(__nv_bfloat16{});
  }
  return fail(PDNN_INVALID_PARAMETER, "unknown dtype %d", dtype);
}

bool pool_params_ok(const PdnnPoolingParams& p) {
  // pooling::validate_params, include/portdnn/pooling/launch.h:56-88
  return p.batch > 0 && p.channels > 0 && p.in_rows > 0 && p.in_cols > 0 && p.out_rows > 0 && p.out_cols > 0 &&
         p.window_rows > 0 && p.window_cols > 0 && p.stride_rows > 0 && p.stride_cols > 0 && p.pad_rows >= 0 &&
         p.pad_cols >= 0;
}

}  // namespace

int launch_pooling(int op, int direction, int dtype, const void* in, void* out, const PdnnPoolingParams& p,
                   cudaStream_t s) {
  if (!pool_params_ok(p)) return fail(PDNN_INVALID_PARAMETER, "pooling: non-positive size or negative padding");
  if (p.input_format != 0) return fail(PDNN_INVALID_PARAMETER, "pooling: only NHWC is implemented");
  if (op < 0 || op > 2 || direction < 0 || direction > 1) return fail(PDNN_INVALID_PARAMETER, "pooling: bad op/direction");
  if (direction == 1 && op != PDNN_POOL_AVERAGE)
    return fail(PDNN_INVALID_PARAMETER, "pooling: the max gradient takes four tensors (pdnn_pooling_max_grad)");
  const int sms = device_sm_count();
  if (sms <= 0) return fail(PDNN_ALLOCATION_PROBLEM, "no CUDA device");
  return dispatch_dtype(dtype, [&](auto tag) {
    using T = decltype(tag);
    constexpr int VN = Vec16<T>::N;
    const bool vec = (p.channels % VN == 0) && aligned16(in) && aligned16(out);
    if (direction == 0 && op != PDNN_POOL_AVERAGE && vec && p.window_rows == 3 && p.window_cols == 3 &&
        p.stride_rows == p.stride_cols && (p.stride_rows == 1 || p.stride_rows == 2)) {
      const StripGeometry g{p.in_rows, p.in_cols, p.out_rows, p.out_cols, p.channels, p.pad_rows, p.pad_cols, p.batch, 0, 0, 0};
      const int r = op == PDNN_POOL_MAX
                        ? launch_window3_strip<T, 1>(static_cast<const T*>(in), nullptr, static_cast<T*>(out), p.stride_rows, g, sms, s)
                        : launch_window3_strip<T, 2>(static_cast<const T*>(in), nullptr, static_cast<T*>(out), p.stride_rows, g, sms, s);
      if (r == 0) return check_launch("pooling (3x3 strips)");
    }
    const size_t pixels = direction == 0 ? (size_t)p.batch * p.out_rows * p.out_cols
                                         : (size_t)p.batch * p.in_rows * p.in_cols;
    const size_t items = pixels * (p.channels / (vec ? VN : 1));
    if (direction == 1 && vec && p.out_rows == 1 && p.out_cols == 1 && p.pad_rows == 0 && p.pad_cols == 0 &&
        p.window_rows == p.in_rows && p.window_cols == p.in_cols && items < 0xFFFF0000ull) {
      const unsigned cvecs = (unsigned)(p.channels / VN);
      pool_avg_grad_global_kernel<T, VN><<<grid_for(items, kBlock, sms), kBlock, 0, s>>>(
          static_cast<const T*>(in), static_cast<T*>(out), cvecs, (unsigned)(p.in_rows * p.in_cols) * cvecs,
          (float)(p.in_rows * p.in_cols), (unsigned)items);
      return check_launch("pooling average gradient (global)");
    }
    const unsigned grid = grid_for(items, kBlock, sms);
    const bool wide = items >= 0xFFFFFFFFull - (size_t)grid * kBlock;
    auto go = [&](auto vtag, auto itag) {
      constexpr int V = decltype(vtag)::value;
      using Index = decltype(itag);
      const T* x = static_cast<const T*>(in);
      T* y = static_cast<T*>(out);
      if (direction == 1) {
        pool_avg_grad_kernel<T, V, Index><<<grid, kBlock, 0, s>>>(x, y, p, (Index)items);
      } else if (op == PDNN_POOL_MAX) {
        pool_forward_kernel<T, PDNN_POOL_MAX, V, Index><<<grid, kBlock, 0, s>>>(x, y, p, (Index)items);
      } else if (op == PDNN_POOL_MAX_WITH_NAN) {
        pool_forward_kernel<T, PDNN_POOL_MAX_WITH_NAN, V, Index><<<grid, kBlock, 0, s>>>(x, y, p, (Index)items);
      } else {
        pool_forward_kernel<T, PDNN_POOL_AVERAGE, V, Index><<<grid, kBlock, 0, s>>>(x, y, p, (Index)items);
      }
    };
    if (vec) {
      if (wide) go(std::integral_constant<int, VN>{}, (unsigned long long)0);
      else go(std::integral_constant<int, VN>{}, (unsigned)0);
    } else {
      if (wide) go(std::integral_constant<int, 1>{}, (unsigned long long)0);
      else go(std::integral_constant<int, 1>{}, (unsigned)0);
    }
    return check_launch("pooling");
  });
}

namespace {
int pooling_max_grad_impl(int op, int dtype, const void* x, const void* y, const void* dy, void* dx,
                          const PdnnPoolingParams& p, bool positive_only, bool* positive_applied, cudaStream_t s);
}

// relu_input: x is the output of a ReLU and dx is to be the gradient with respect to that ReLU's
// input: elements that are not positive receive nothing.  Where the winner map comes from the strip
// kernel this costs nothing (a window whose maximum is not positive has no winner); elsewhere a
// ReLU-gradient pass follows.
int launch_pooling_max_grad(int op, int dtype, const void* x, const void* y, const void* dy, void* dx,
                            const PdnnPoolingParams& p, bool relu_input, cudaStream_t s) {
  bool applied = false;
  int st = pooling_max_grad_impl(op, dtype, x, y, dy, dx, p, relu_input, &applied, s);
  if (st == PDNN_OK && relu_input && !applied)
    st = launch_pointwise_grad(PDNN_ACT_RELU, dtype, x, dx, dx, (size_t)p.batch * p.in_rows * p.in_cols * p.channels, s);
  return st;
}

namespace {
int pooling_max_grad_impl(int op, int dtype, const void* x, const void* y, const void* dy, void* dx,
                          const PdnnPoolingParams& p, bool positive_only, bool* positive_applied, cudaStream_t s) {
  if (!pool_params_ok(p)) return fail(PDNN_INVALID_PARAMETER, "pooling: non-positive size or negative padding");
  if (p.input_format != 0) return fail(PDNN_INVALID_PARAMETER, "pooling: only NHWC is implemented");
  if (op != PDNN_POOL_MAX && op != PDNN_POOL_MAX_WITH_NAN) return fail(PDNN_INVALID_PARAMETER, "max gradient: bad op");
  const int sms = device_sm_count();
  if (sms <= 0) return fail(PDNN_ALLOCATION_PROBLEM, "no CUDA device");
  return dispatch_dtype(dtype, [&](auto tag) {
    using T = decltype(tag);
    constexpr int VN = Vec16<T>::N;
    const bool vec = (p.channels % VN == 0) && aligned16(x) && aligned16(y) && aligned16(dy) && aligned16(dx);
    const size_t out_items = (size_t)p.batch * p.out_rows * p.out_cols * (p.channels / VN);
    const size_t in_items = (size_t)p.batch * p.in_rows * p.in_cols * (p.channels / VN);
    const bool small = in_items < 0xFFFFFFFFull - (size_t)sms * 32 * kBlock;
    const T *xt = static_cast<const T*>(x), *yt = static_cast<const T*>(y), *dyt = static_cast<const T*>(dy);
    T* dxt = static_cast<T*>(dx);
    if (vec && small && p.pad_rows == 0 && p.pad_cols == 0 && p.stride_rows == p.window_rows &&
        p.stride_cols == p.window_cols && p.in_rows == p.out_rows * p.stride_rows &&
        p.in_cols == p.out_cols * p.stride_cols) {
      // the windows tile the input: one pass
      const unsigned g1 = grid_for(out_items, kBlock, sms);
      if (op == PDNN_POOL_MAX)
        pool_max_grad_tiled_kernel<T, PDNN_POOL_MAX, VN, unsigned><<<g1, kBlock, 0, s>>>(xt, yt, dyt, dxt, p, (unsigned)out_items);
      else
        pool_max_grad_tiled_kernel<T, PDNN_POOL_MAX_WITH_NAN, VN, unsigned><<<g1, kBlock, 0, s>>>(xt, yt, dyt, dxt, p, (unsigned)out_items);
      return check_launch("pooling max gradient (tiling windows)");
    }
    if (vec && small && p.window_rows * p.window_cols < 255) {
      // overlapping windows: winners first, then a gather; the winner map comes from the
      // stream-ordered allocator
      unsigned char* winner = nullptr;
      const size_t bytes = out_items * VN;
      if (cudaMallocAsync(reinterpret_cast<void**>(&winner), bytes, s) == cudaSuccess) {
        const unsigned g1 = grid_for(out_items, kBlock, sms), g2 = grid_for(in_items, kBlock, sms);
        bool winners_done = false;
        if (p.window_rows == 3 && p.window_cols == 3 && p.stride_rows == p.stride_cols &&
            (p.stride_rows == 1 || p.stride_rows == 2)) {
          // the forward pool's strip walk, writing the winner map instead of the maxima
          const StripGeometry sg{p.in_rows, p.in_cols, p.out_rows, p.out_cols, p.channels, p.pad_rows, p.pad_cols, p.batch, 0, 0, 0,
                                 0, positive_only ? 1 : 0};
          T* wmap = reinterpret_cast<T*>(winner);
          winners_done = (op == PDNN_POOL_MAX ? launch_window3_strip<T, 3>(xt, nullptr, wmap, p.stride_rows, sg, sms, s)
                                              : launch_window3_strip<T, 4>(xt, nullptr, wmap, p.stride_rows, sg, sms, s)) == 0;
        }
        if (winners_done) {
          *positive_applied = positive_only;
        } else if (op == PDNN_POOL_MAX)
          pool_winner_kernel<T, PDNN_POOL_MAX, VN, unsigned><<<g1, kBlock, 0, s>>>(xt, yt, winner, p, (unsigned)out_items);
        else
          pool_winner_kernel<T, PDNN_POOL_MAX_WITH_NAN, VN, unsigned><<<g1, kBlock, 0, s>>>(xt, yt, winner, p, (unsigned)out_items);
        int st = check_launch("pooling max gradient (winners)");
        if (st == PDNN_OK && p.window_rows == 3 && p.window_cols == 3 && p.stride_rows == 2 && p.stride_cols == 2) {
          PoolS2Geometry g{p.in_rows, p.in_cols, p.out_rows, p.out_cols, p.channels, p.pad_rows, p.pad_cols, p.batch,
                           (p.in_rows - 1 + p.pad_rows) / 2 + 1, (p.in_cols - 1 + p.pad_cols) / 2 + 1, 0, 0};
          const size_t columns = (size_t)p.batch * g.K * (p.channels / VN);
          g.rows = g.M;
          while (g.rows > 4 && columns * ((g.M + g.rows - 1) / g.rows) < (size_t)sms * 2048) g.rows = (g.rows + 1) / 2;
          g.strips = (g.M + g.rows - 1) / g.rows;
          const size_t n_items = columns * g.strips;
          pool_max_grad_s2_kernel<T, VN><<<grid_for(n_items, kBlock, sms), kBlock, 0, s>>>(winner, dyt, dxt, g,
                                                                                         (unsigned)n_items);
          st = check_launch("pooling max gradient (3x3 / 2 gather)");
        } else if (st == PDNN_OK) {
          pool_max_grad_from_winner_kernel<T, VN, unsigned><<<g2, kBlock, 0, s>>>(winner, dyt, dxt, p, (unsigned)in_items);
          st = check_launch("pooling max gradient (gather)");
        }
        cudaFreeAsync(winner, s);
        return st;
      }
      cudaGetLastError();  // no scratch: fall through to the single-pass kernel
    }
    const size_t items = (size_t)p.batch * p.in_rows * p.in_cols * (p.channels / (vec ? VN : 1));
    const unsigned grid = grid_for(items, kBlock, sms);
    const bool wide = items >= 0xFFFFFFFFull - (size_t)grid * kBlock;
    auto go = [&](auto vtag, auto itag) {
      constexpr int V = decltype(vtag)::value;
      using Index = decltype(itag);
      if (op == PDNN_POOL_MAX)
        pool_max_grad_kernel<T, PDNN_POOL_MAX, V, Index><<<grid, kBlock, 0, s>>>(
            static_cast<const T*>(x), static_cast<const T*>(y), static_cast<const T*>(dy), static_cast<T*>(dx), p,
            (Index)items);
      else
        pool_max_grad_kernel<T, PDNN_POOL_MAX_WITH_NAN, V, Index><<<grid, kBlock, 0, s>>>(
            static_cast<const T*>(x), static_cast<const T*>(y), static_cast<const T*>(dy), static_cast<T*>(dx), p,
            (Index)items);
    };
    if (vec) {
      if (wide) go(std::integral_constant<int, VN>{}, (unsigned long long)0);
      else go(std::integral_constant<int, VN>{}, (unsigned)0);
    } else {
      if (wide) go(std::integral_constant<int, 1>{}, (unsigned long long)0);
      else go(std::integral_constant<int, 1>{}, (unsigned)0);
    }
    return check_launch("pooling max gradient");
  });
}
}  // namespace

namespace {
bool depthwise_params_ok(const PdnnDepthwiseConv2DParams& p) {
  return p.batch > 0 && p.channels > 0 && p.channel_multiplier > 0 && p.in_rows > 0 && p.in_cols > 0 &&
         p.out_rows > 0 && p.out_cols > 0 && p.window_rows > 0 && p.window_cols > 0 && p.stride_rows > 0 &&
         p.stride_cols > 0 && p.pad_rows >= 0 && p.pad_cols >= 0;
}

// Number of pixel slices of the filter-backprop reduction: enough blocks to fill the device,
// at least 256 pixels per slice.
// The all-taps kernel runs 3x3 windows with whole channel packets.
bool fbp_all_taps(const PdnnDepthwiseConv2DParams& p, int V) {
  return V > 1 && p.window_rows == 3 && p.window_cols == 3 && p.channel_multiplier == 1;
}

// Channel lanes per block of the all-taps kernel: 4, 8, 16 or 32 (the block always has 256
// threads), whichever wastes the fewest lanes on the last channel tile; ties go to the wider one.
int fbp_channel_lanes(int packets) {
  int best = 32;
  double best_eff = 0;
  for (int lanes = 32; lanes >= 4; lanes >>= 1) {
    const int tiles = (packets + lanes - 1) / lanes;
    const double eff = (double)packets / (tiles * lanes);
    if (eff > best_eff + 1e-9) {
      best_eff = eff;
      best = lanes;
    }
  }
  return best;
}

int fbp_slices(const PdnnDepthwiseConv2DParams& p, int V, int sms) {
  const long long pixels = (long long)p.batch * p.out_rows * p.out_cols;
  const int F = p.channels * p.channel_multiplier;
  const bool all_taps = fbp_all_taps(p, V);
  const int lanes = all_taps ? fbp_channel_lanes(F / V) : kFbpLanesF;
  const int ftiles = (F + lanes * V - 1) / (lanes * V);
  const long long other = all_taps ? ftiles : (long long)p.window_rows * p.window_cols * ftiles;
  long long want = ((long long)sms * 8 + other - 1) / other;
  const long long cap = (pixels + 255) / 256;
  if (want > cap) want = cap;
  if (want < 1) want = 1;
  if (want > 1024) want = 1024;
  return (int)want;
}

// Stage 1 of the depthwise filter backprop: partial[slice][tap][f].  Returns the number of slices written.
template <typename T>
int launch_fbp_partials(bool vec, const T* in, const T* dy, float* partial, const PdnnDepthwiseConv2DParams& p,
                         int slices, cudaStream_t s) {
  constexpr int VN = Vec16<T>::N;
  const int V = vec ? VN : 1, F = p.channels * p.channel_multiplier;
  const long long pixels = (long long)p.batch * p.out_rows * p.out_cols;
  const long long per_slice = (pixels + slices - 1) / slices;
  constexpr int E = 4 / (int)sizeof(T);
  const unsigned long long x_words = (unsigned long long)p.batch * p.in_rows * p.in_cols * (F / E);
  if (p.window_rows == 3 && p.window_cols == 3 && p.channel_multiplier == 1 && F % E == 0 && aligned16(in) && aligned16(dy) &&
      p.stride_rows == p.stride_cols && (p.stride_rows == 1 || p.stride_rows == 2) && x_words < 0xFFFFFFFFull) {
    // whole output rows per warp, one 32-bit word of channels per lane
    const long long units = (long long)p.batch * p.out_rows;
    const int groups = (F / E + 31) / 32;
    // one wave of blocks, as long as the scratch holds that many slices
    const int sms = device_sm_count();
    int per_sm = 0;
    const cudaError_t oe = p.stride_rows == 1
        ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, depthwise_filter_backprop_rows_kernel<T, 1>, kFbpRowsWarps * 32, 0)
        : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, depthwise_filter_backprop_rows_kernel<T, 2>, kFbpRowsWarps * 32, 0);
    if (oe != cudaSuccess || per_sm < 1) {
      cudaGetLastError();
      per_sm = 2;
    }
    // the last block of words packs several rows per warp when it is narrow, and gets that much less of the wave
    const int tail_words = F / E - 32 * (groups - 1), tail_rows = tail_words <= 16 ? 32 / tail_words : 1;
    const long long wave = std::max<long long>(1, (long long)(per_sm * sms / (groups - 1 + 1.0 / tail_rows)));
    const unsigned gx = (unsigned)std::min<long long>(std::min<long long>(slices, wave), (units + kFbpRowsWarps - 1) / kFbpRowsWarps);
    const unsigned g_tail = std::max(1u, (gx + (unsigned)tail_rows - 1u) / (unsigned)tail_rows);
    dim3 grid(gx * (unsigned)(groups - 1) + g_tail);
    // rows are cut into up to four segments until a warp has a dozen units to walk
    const int trip = p.stride_rows == 1 ? 4 : 2;  // the kernel's U
    int segs = 1;
    while (segs < 4 && units * segs < (long long)gx * kFbpRowsWarps * 12 && (p.out_cols + 2 * segs - 1) / (2 * segs) >= 2 * trip) segs *= 2;
    const int seg_cols = ((p.out_cols + segs - 1) / segs + trip - 1) / trip * trip;
    segs = (p.out_cols + seg_cols - 1) / seg_cols;
    if (p.stride_rows == 1) depthwise_filter_backprop_rows_kernel<T, 1><<<grid, kFbpRowsWarps * 32, 0, s>>>(in, dy, partial, p, segs, seg_cols, (int)gx, (int)g_tail);
    else depthwise_filter_backprop_rows_kernel<T, 2><<<grid, kFbpRowsWarps * 32, 0, s>>>(in, dy, partial, p, segs, seg_cols, (int)gx, (int)g_tail);
    return (int)gx;
  }
  if (fbp_all_taps(p, V)) {
    const int lanes = fbp_channel_lanes(F / V);
    dim3 block(lanes, kFbpLanesF * kFbpLanesP / lanes);
    dim3 grid(slices, 1, (F + lanes * V - 1) / (lanes * V));
    depthwise_filter_backprop_partial9_kernel<T, VN><<<grid, block, 0, s>>>(in, dy, partial, p, per_slice);
    return slices;
  }
  dim3 block(kFbpLanesF, kFbpLanesP);
  dim3 grid(slices, p.window_rows * p.window_cols, (F + kFbpLanesF * V - 1) / (kFbpLanesF * V));
  if (vec) depthwise_filter_backprop_partial_kernel<T, VN><<<grid, block, 0, s>>>(in, dy, partial, p, per_slice);
  else depthwise_filter_backprop_partial_kernel<T, 1><<<grid, block, 0, s>>>(in, dy, partial, p, per_slice);
  return slices;
}

}  // namespace

size_t depthwise_workspace_bytes(int pass, int dtype, const PdnnDepthwiseConv2DParams& p) {
  if (pass != PDNN_FILTER_BACKPROP || !depthwise_params_ok(p)) return 0;
  int sms = device_sm_count();
  if (sms <= 0) sms = 148;
  const int VN = 16 / (int)dtype_size(dtype);
  // sized for the scalar form, which never uses fewer slices than the packet form
  const int slices = fbp_slices(p, 1, sms) > fbp_slices(p, VN, sms) ? fbp_slices(p, 1, sms) : fbp_slices(p, VN, sms);
  return (size_t)slices * p.window_rows * p.window_cols * p.channels * p.channel_multiplier * sizeof(float);
}

int launch_depthwise(int pass, int dtype, const void* in, const void* fil, void* out,
                     const PdnnDepthwiseConv2DParams& p, void* ws, size_t ws_bytes, cudaStream_t s) {
  if (!depthwise_params_ok(p)) return fail(PDNN_INVALID_PARAMETER, "depthwise: non-positive size or negative padding");
  if (pass < 0 || pass > 2) return fail(PDNN_INVALID_PARAMETER, "depthwise: bad pass");
  const int sms = device_sm_count();
  if (sms <= 0) return fail(PDNN_ALLOCATION_PROBLEM, "no CUDA device");
  return dispatch_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    constexpr int VN = Vec16<T>::N;
    const int F = p.channels * p.channel_multiplier;
    // the reference vectorises only for multiplier 1 too (src/depthwise_conv2d/launch.cc:41-121)
    const bool vec = p.channel_multiplier == 1 && (p.channels % VN == 0) && aligned16(in) && aligned16(fil) && aligned16(out);
    if (pass == PDNN_FILTER_BACKPROP) {
      const int V = vec ? VN : 1;
      const int slices = fbp_slices(p, V, sms);
      const size_t n_out = (size_t)p.window_rows * p.window_cols * F;
      const size_t need = (size_t)slices * n_out * sizeof(float);
      float* partial = static_cast<float*>(ws);
      bool own = false;
      if (partial == nullptr || ws_bytes < need) {
        if (cudaMallocAsync(reinterpret_cast<void**>(&partial), need, s) != cudaSuccess) {
          cudaGetLastError();
          return fail(PDNN_ALLOCATION_PROBLEM, "depthwise filter backprop: cannot allocate %zu bytes of scratch", need);
        }
        own = true;
      }
      const int written = launch_fbp_partials<T>(vec, static_cast<const T*>(in), static_cast<const T*>(fil), partial, p, slices, s);
      int st = check_launch("depthwise filter backprop (partial sums)");
      if (st == PDNN_OK) {
        reduce_slices_kernel<T><<<grid_for(n_out, kBlock, sms), kBlock, 0, s>>>(partial, static_cast<T*>(out), written, n_out);
        st = check_launch("depthwise filter backprop (slice reduction)");
      }
      if (own) cudaFreeAsync(partial, s);
      return st;
    }
    if constexpr (!std::is_same<T, __nv_bfloat16>::value) {
      if (pass == PDNN_FORWARD && vec && p.window_rows == 3 && p.window_cols == 3 && p.stride_rows == p.stride_cols &&
          (p.stride_rows == 1 || p.stride_rows == 2)) {
        const StripGeometry g{p.in_rows, p.in_cols, p.out_rows, p.out_cols, p.channels, p.pad_rows, p.pad_cols, p.batch, 0, 0, 0, 0};
        if (launch_window3_strip<T, 0>(static_cast<const T*>(in), static_cast<const T*>(fil), static_cast<T*>(out),
                                       p.stride_rows, g, sms, s) == 0)
          return check_launch("depthwise conv2d (3x3 strips)");
      }
      // Stride-1 input backprop is the forward operator on dy with the filter mirrored and the
      // padding complemented: dx[h][w] = sum dy[h + pad - r][w + pad - s] * w[r][s].
      if (pass == PDNN_INPUT_BACKPROP && vec && p.channel_multiplier == 1 && p.window_rows == 3 && p.window_cols == 3 &&
          p.stride_rows == 1 && p.stride_cols == 1 && p.pad_rows <= 2 && p.pad_cols <= 2) {
        const StripGeometry g{p.out_rows, p.out_cols, p.in_rows, p.in_cols, p.channels, 2 - p.pad_rows, 2 - p.pad_cols,
                              p.batch, 0, 0, 0, 1};
        if (launch_window3_strip<T, 0>(static_cast<const T*>(in), static_cast<const T*>(fil), static_cast<T*>(out), 1, g,
                                       sms, s) == 0)
          return check_launch("depthwise input backprop (3x3 strips)");
      }
    }
    if (pass == PDNN_INPUT_BACKPROP && vec && p.window_rows == 3 && p.window_cols == 3 && p.stride_rows == 2 &&
        p.stride_cols == 2) {
      IbpS2Geometry g{p.in_rows, p.in_cols, p.out_rows, p.out_cols, p.channels, p.pad_rows, p.pad_cols, p.batch,
                      (p.in_rows - 1 + p.pad_rows) / 2 + 1, (p.in_cols - 1 + p.pad_cols) / 2 + 1, 0, 0};
      // enough threads to fill the device a few times over, otherwise strips as long as possible
      const size_t columns = (size_t)p.batch * g.K * (p.channels / VN);
      g.rows = g.M;
      while (g.rows > 4 && columns * ((g.M + g.rows - 1) / g.rows) < (size_t)sms * 2048) g.rows = (g.rows + 1) / 2;
      g.strips = (g.M + g.rows - 1) / g.rows;
      const size_t n_items = columns * g.strips;
      if (n_items < 0xFFFF0000ull) {
        depthwise_ibp_s2_kernel<T, VN><<<grid_for(n_items, kBlock, sms), kBlock, 0, s>>>(
            static_cast<const T*>(in), static_cast<const T*>(fil), static_cast<T*>(out), g, (unsigned)n_items);
        return check_launch("depthwise input backprop (3x3, stride 2)");
      }
    }
    const size_t pixels = pass == PDNN_FORWARD ? (size_t)p.batch * p.out_rows * p.out_cols
                                               : (size_t)p.batch * p.in_rows * p.in_cols;
    const size_t items = pixels * ((pass == PDNN_FORWARD ? F : p.channels) / (vec ? VN : 1));
    const unsigned grid = grid_for(items, kBlock, sms);
    const bool wide = items >= 0xFFFFFFFFull - (size_t)grid * kBlock;
    auto go = [&](auto vtag, auto itag) {
      constexpr int V = decltype(vtag)::value;
      using Index = decltype(itag);
      if (pass == PDNN_FORWARD)
        depthwise_forward_kernel<T, V, Index><<<grid, kBlock, 0, s>>>(
            static_cast<const T*>(in), static_cast<const T*>(fil), static_cast<T*>(out), p, (Index)items);
      else
        depthwise_input_backprop_kernel<T, V, Index><<<grid, kBlock, 0, s>>>(
            static_cast<const T*>(in), static_cast<const T*>(fil), static_cast<T*>(out), p, (Index)items);
    };
    if (vec) {
      if (wide) go(std::integral_constant<int, VN>{}, (unsigned long long)0);
      else go(std::integral_constant<int, VN>{}, (unsigned)0);
    } else {
      if (wide) go(std::integral_constant<int, 1>{}, (unsigned long long)0);
      else go(std::integral_constant<int, 1>{}, (unsigned)0);
    }
    return check_launch("depthwise conv2d");
  });
}

int launch_pointwise(int op, int dtype, const void* in, void* out, size_t n, cudaStream_t s) {
  if (op < 0 || op > PDNN_PW_SQRT) return fail(PDNN_INVALID_PARAMETER, "pointwise: bad op");
  if (n == 0) return PDNN_OK;
  const int sms = device_sm_count();
  if (sms <= 0) return fail(PDNN_ALLOCATION_PROBLEM, "no CUDA device");
  return dispatch_dtype(dtype, [&](auto tag) {
    using T = decltype(tag);
    constexpr int VN = Vec16<T>::N;
    // the reference picks the widest vector that divides n (src/pointwise/launch_pointwise_forward.cc:32-70)
    if (n % VN == 0 && aligned16(in) && aligned16(out))
      pointwise_kernel<T, VN, 0><<<grid_for(n / VN, kBlock, sms), kBlock, 0, s>>>(
          op, static_cast<const T*>(in), nullptr, static_cast<T*>(out), n / VN);
    else
      pointwise_kernel<T, 1, 0><<<grid_for(n, kBlock, sms), kBlock, 0, s>>>(op, static_cast<const T*>(in), nullptr,
                                                                            static_cast<T*>(out), n);
    return check_launch("pointwise");
  });
}

int launch_pointwise_grad(int op, int dtype, const void* fwd, const void* err, void* out, size_t n, cudaStream_t s) {
  if (op < 0 || op > PDNN_PW_SQRT || op == PDNN_PW_FLOOR)
    return fail(PDNN_INVALID_PARAMETER, "pointwise: op %d has no gradient", op);
  if (n == 0) return PDNN_OK;
  const int sms = device_sm_count();
  if (sms <= 0) return fail(PDNN_ALLOCATION_PROBLEM, "no CUDA device");
  return dispatch_dtype(dtype, [&](auto tag) {
    using T = decltype(tag);
    constexpr int VN = Vec16<T>::N;
    if (n % VN == 0 && aligned16(fwd) && aligned16(err) && aligned16(out))
      pointwise_kernel<T, VN, 1><<<grid_for(n / VN, kBlock, sms), kBlock, 0, s>>>(
          op, static_cast<const T*>(fwd), static_cast<const T*>(err), static_cast<T*>(out), n / VN);
    else
      pointwise_kernel<T, 1, 1><<<grid_for(n, kBlock, sms), kBlock, 0, s>>>(
          op, static_cast<const T*>(fwd), static_cast<const T*>(err), static_cast<T*>(out), n);
    return check_launch("pointwise gradient");
  });
}

int launch_bias_add(int dtype, const void* in, const void* bias, void* out, size_t rows, int channels, int act,
                    cudaStream_t s) {
  if (channels <= 0) return fail(PDNN_INVALID_PARAMETER, "bias: channels must be positive");
  if (act < PDNN_ACT_NONE || act > PDNN_ACT_RELU6) return fail(PDNN_INVALID_PARAMETER, "bias: unknown activation %d", act);
  if (rows == 0) return PDNN_OK;
  const int sms = device_sm_count();
  if (sms <= 0) return fail(PDNN_ALLOCATION_PROBLEM, "no CUDA device");
  return dispatch_dtype(dtype, [&](auto tag) {
    using T = decltype(tag);
    constexpr int VN = Vec16<T>::N;
    const size_t n = rows * (size_t)channels;
    if (channels % VN == 0 && aligned16(in) && aligned16(bias) && aligned16(out))
      bias_add_kernel<T, VN><<<grid_for(n / VN, kBlock, sms), kBlock, 0, s>>>(
          static_cast<const T*>(in), static_cast<const T*>(bias), static_cast<T*>(out), n / VN, channels / VN, act);
    else
      bias_add_kernel<T, 1><<<grid_for(n, kBlock, sms), kBlock, 0, s>>>(
          static_cast<const T*>(in), static_cast<const T*>(bias), static_cast<T*>(out), n, channels, act);
    return check_launch("bias add");
  });
}

int launch_scale_blend(int dtype, const void* a, float alpha, const void* b, float beta, void* out, size_t n,
                       cudaStream_t s) {
  if (n == 0) return PDNN_OK;
  const int sms = device_sm_count();
  if (sms <= 0) return fail(PDNN_ALLOCATION_PROBLEM, "no CUDA device");
  if (beta == 0.f) b = nullptr;
  return dispatch_dtype(dtype, [&](auto tag) {
    using T = decltype(tag);
    constexpr int VN = Vec16<T>::N;
    if (n % VN == 0 && aligned16(a) && aligned16(out) && (b == nullptr || aligned16(b)))
      scale_blend_kernel<T, VN><<<grid_for(n / VN, kBlock, sms), kBlock, 0, s>>>(
          static_cast<const T*>(a), alpha, static_cast<const T*>(b), beta, static_cast<T*>(out), n / VN);
    else
      scale_blend_kernel<T, 1><<<grid_for(n, kBlock, sms), kBlock, 0, s>>>(
          static_cast<const T*>(a), alpha, static_cast<const T*>(b), beta, static_cast<T*>(out), n);
    return check_launch("scale blend");
  });
}

// ------------------------------------------------------------------------------------------
// Binary operators with broadcasting
// ------------------------------------------------------------------------------------------
// out = lhs (op) rhs over an output of at most four extents; an operand's stride is 0 along the
// extents it is broadcast over (include/portdnn/internal/binaryop/launch.h:34-115,
// src/binaryop/kernels.h).  A thread owns V consecutive elements of the innermost extent: an
// operand that runs along it is read as one packet, one that is broadcast along it as one scalar.
struct BinaryGeometry {
  unsigned od[4];       // output extents, outermost first
  unsigned ls[4], rs[4];  // element strides of the operands
};

template <typename T, int V>
__global__ void __launch_bounds__(kBlock) binaryop_kernel(int op, const T* __restrict__ lhs, const T* __restrict__ rhs,
                                                          T* __restrict__ out, BinaryGeometry g, size_t n_packets) {
  const unsigned inner_packets = g.od[3] / V;
  for (size_t i = (size_t)blockIdx.x * kBlock + threadIdx.x; i < n_packets; i += (size_t)gridDim.x * kBlock) {
    // the output has fewer than 2^32 elements (checked by the host): 32-bit divisions
    const unsigned p = (unsigned)i;
    unsigned t = p / inner_packets;
    const unsigned d3 = (p - t * inner_packets) * V;
    unsigned q = t / g.od[2];
    const unsigned d2 = t - q * g.od[2];
    const unsigned d0 = q / g.od[1], d1 = q - d0 * g.od[1];
    const size_t li = (size_t)d0 * g.ls[0] + (size_t)d1 * g.ls[1] + (size_t)d2 * g.ls[2] + (size_t)d3 * g.ls[3];
    const size_t ri = (size_t)d0 * g.rs[0] + (size_t)d1 * g.rs[1] + (size_t)d2 * g.rs[2] + (size_t)d3 * g.rs[3];
    float a[V], b[V], res[V];
    if (V == 1 || g.ls[3] != 0) {
      load_vec<T, V>(lhs + li, a);
    } else {
      const float v = to_f32(lhs[li]);
#pragma unroll
      for (int j = 0; j < V; ++j) a[j] = v;
    }
    if (V == 1 || g.rs[3] != 0) {
      load_vec<T, V>(rhs + ri, b);
    } else {
      const float v = to_f32(rhs[ri]);
#pragma unroll
      for (int j = 0; j < V; ++j) b[j] = v;
    }
#pragma unroll
    for (int j = 0; j < V; ++j)
      res[j] = op == PDNN_BINARY_ADD ? a[j] + b[j] : op == PDNN_BINARY_SUB ? a[j] - b[j]
               : op == PDNN_BINARY_MUL ? a[j] * b[j] : a[j] / b[j];
    store_vec<T, V>(out + i * V, res);
  }
}

int launch_binaryop(int op, int dtype, const void* lhs, const int* lhs_dims, int n_lhs, const void* rhs,
                    const int* rhs_dims, int n_rhs, void* out, cudaStream_t s) {
  if (op < PDNN_BINARY_ADD || op > PDNN_BINARY_DIV) return fail(PDNN_INVALID_PARAMETER, "binaryop: unknown operator %d", op);
  if (n_lhs < 0 || n_lhs > 4 || n_rhs < 0 || n_rhs > 4)
    return fail(PDNN_INVALID_PARAMETER, "binaryop: an operand has more than four extents");
  long long ld[4] = {1, 1, 1, 1}, rd[4] = {1, 1, 1, 1}, od[4];
  for (int i = 0; i < n_lhs; ++i) ld[4 - n_lhs + i] = lhs_dims[i];
  for (int i = 0; i < n_rhs; ++i) rd[4 - n_rhs + i] = rhs_dims[i];
  long long total = 1;
  for (int i = 0; i < 4; ++i) {
    if (ld[i] <= 0 || rd[i] <= 0) return fail(PDNN_INVALID_PARAMETER, "binaryop: operand size cannot be zero");
    if (ld[i] != rd[i] && ld[i] != 1 && rd[i] != 1)
      return fail(PDNN_INVALID_PARAMETER, "binaryop: extents %lld and %lld cannot be broadcast", ld[i], rd[i]);
    od[i] = std::max(ld[i], rd[i]);
    total *= od[i];
    if (total > 0xFFFFFFFFll) return fail(PDNN_INDEX_EXCEEDED, "binaryop: more than 2^32 output elements");
  }
  if (lhs == nullptr || rhs == nullptr || out == nullptr) return fail(PDNN_INVALID_PARAMETER, "binaryop: null tensor");
  // Merge neighbouring extents that both operands walk the same way (both run, or both stay): equal
  // shapes collapse to one extent, the bias form to [rows, C].
  long long cd[4], cl[4], cr[4];
  int k = 0;
  for (int i = 0; i < 4; ++i) {
    if (od[i] == 1) continue;
    const bool lb = ld[i] == 1, rb = rd[i] == 1;
    if (k > 0 && lb == (cl[k - 1] == 1) && rb == (cr[k - 1] == 1)) {
      cd[k - 1] *= od[i];
      cl[k - 1] *= ld[i];
      cr[k - 1] *= rd[i];
    } else {
      cd[k] = od[i];
      cl[k] = ld[i];
      cr[k] = rd[i];
      ++k;
    }
  }
  BinaryGeometry g;
  long long lstride = 1, rstride = 1;
  for (int i = 3, j = k - 1; i >= 0; --i, --j) {
    if (j >= 0) {
      g.od[i] = (unsigned)cd[j];
      g.ls[i] = cl[j] == 1 ? 0u : (unsigned)lstride;
      g.rs[i] = cr[j] == 1 ? 0u : (unsigned)rstride;
      lstride *= cl[j];
      rstride *= cr[j];
    } else {
      g.od[i] = 1u;
      g.ls[i] = g.rs[i] = 0u;
    }
  }
  const int sms = device_sm_count();
  if (sms <= 0) return fail(PDNN_ALLOCATION_PROBLEM, "no CUDA device");
  return dispatch_dtype(dtype, [&](auto tag) {
    using T = decltype(tag);
    constexpr int VN = Vec16<T>::N;
    // packets need the innermost extent to be whole packets; every outer stride of an operand
    // that runs along it is then a multiple of the packet too
    const bool vec = g.od[3] % VN == 0 && aligned16(lhs) && aligned16(rhs) && aligned16(out);
    const size_t n = (size_t)total;
    if (vec)
      binaryop_kernel<T, VN><<<grid_for(n / VN, kBlock, sms), kBlock, 0, s>>>(
          op, static_cast<const T*>(lhs), static_cast<const T*>(rhs), static_cast<T*>(out), g, n / VN);
    else
      binaryop_kernel<T, 1><<<grid_for(n, kBlock, sms), kBlock, 0, s>>>(
          op, static_cast<const T*>(lhs), static_cast<const T*>(rhs), static_cast<T*>(out), g, n);
    return check_launch("binaryop");
  });
}

// ------------------------------------------------------------------------------------------
// Depthwise filter backprop for callers that must not allocate
// ------------------------------------------------------------------------------------------
// Some hosts of this library run where a device allocation is off the table: inside a framework
// that hands every byte of device memory to its own arena up front, in a real-time serving loop
// that forbids allocator calls after start-up, or under a memory budget that is fixed before the
// first request.  launch_depthwise() needs scratch for the per-slice partial sums of its filter
// backprop and takes it from the caller or from cudaMallocAsync; this variant instead keeps the
// partial sums in the fixed array below, which every device that loads the library holds from
// load until the process exits.
constexpr size_t kStaticScratchBytes = 8u << 20;  // 8 MiB of fp32 partial sums
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {
std::mutex g_static_scratch_mutex;
float* g_static_scratch_ptr[kMaxDevices] = {};

// The array's name is only a host-side handle: the address the kernels need has to be asked for,
// once per device and with that device current.  The kernels run on the device the stream belongs
// to, so a stream of another device than the current one is refused (its launch would fail anyway)
// rather than handed the current device's copy of the array.
int static_scratch_for_current_device(float** out, cudaStream_t s) {
  const int dev = current_device();
  if (dev < 0 || dev >= kMaxDevices) return fail(PDNN_ALLOCATION_PROBLEM, "static scratch: no usable current device");
  if (s != nullptr && s != cudaStreamLegacy && s != cudaStreamPerThread) {
    int stream_dev = dev;
    if (cudaStreamGetDevice(s, &stream_dev) != cudaSuccess) {
      cudaGetLastError();
      return fail(PDNN_INVALID_PARAMETER, "static scratch: not a valid stream");
    }
    if (stream_dev != dev)
      return fail(PDNN_INVALID_PARAMETER, "static scratch: the stream belongs to device %d but device %d is current",
                  stream_dev, dev);
  }
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return fail(PDNN_ALLOCATION_PROBLEM, "static scratch: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    }
    g_static_scratch_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_static_scratch_ptr[dev];
  return PDNN_OK;
}
}  // namespace

size_t static_scratch_bytes() { return kStaticScratchBytes; }

int launch_depthwise_filter_backprop_static(int dtype, const void* in, const void* dy, void* dw,
                                            const PdnnDepthwiseConv2DParams& p, cudaStream_t s) {
  if (!depthwise_params_ok(p)) return fail(PDNN_INVALID_PARAMETER, "depthwise: non-positive size or negative padding");
  const int sms = device_sm_count();
  if (sms <= 0) return fail(PDNN_ALLOCATION_PROBLEM, "no CUDA device");
  const int F = p.channels * p.channel_multiplier;
  const size_t n_out = (size_t)p.window_rows * p.window_cols * F;
  if (n_out * sizeof(float) > kStaticScratchBytes)
    return fail(PDNN_INSUFFICIENT_WORKSPACE,
                "depthwise filter backprop without allocation: the filter gradient has %zu elements, the fixed "
                "scratch holds at most %zu",
                n_out, kStaticScratchBytes / sizeof(float));
  float* partial = nullptr;
  const int st0 = static_scratch_for_current_device(&partial, s);
  if (st0 != PDNN_OK) return st0;
  return dispatch_dtype(dtype, [&](auto tag) -> int {
    using T = decltype(tag);
    constexpr int VN = Vec16<T>::N;
    const bool vec = p.channel_multiplier == 1 && (p.channels % VN == 0) && aligned16(in) && aligned16(dy) && aligned16(dw);
    const int V = vec ? VN : 1;
    // as many pixel slices as the general path would use, but no more than the array holds
    int slices = fbp_slices(p, V, sms);
    const size_t fit = kStaticScratchBytes / (n_out * sizeof(float));
    if ((size_t)slices > fit) slices = (int)fit;
    // Stage 1 writes every partial[slice][tap][f] it later reads, so the array's old contents
    // never leak into a result and nothing has to be cleared first.
    const int written = launch_fbp_partials<T>(vec, static_cast<const T*>(in), static_cast<const T*>(dy), partial, p, slices, s);
    int st = check_launch("depthwise filter backprop, fixed scratch (partial sums)");
    if (st != PDNN_OK) return st;
    reduce_slices_kernel<T><<<grid_for(n_out, kBlock, sms), kBlock, 0, s>>>(partial, static_cast<T*>(dw), written, n_out);
    return check_launch("depthwise filter backprop, fixed scratch (slice reduction)");
  });
}

// ------------------------------------------------------------------------------------------
// One-bit-per-element ReLU masks (bit e of byte i / 8 for element i: "positive"), the general forms
// beside the tensor-core epilogues that write and read them: from a tensor, and applied to a gradient.
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kBlock) relu_bitmask_kernel(const T* __restrict__ y, unsigned char* __restrict__ bits,
                                                              size_t n_bytes) {
  for (size_t i = (size_t)blockIdx.x * kBlock + threadIdx.x; i < n_bytes; i += (size_t)gridDim.x * kBlock) {
    unsigned b = 0u;
#pragma unroll
    for (int e = 0; e < 8; ++e) b |= (to_f32(y[i * 8 + e]) > 0.f ? 1u : 0u) << e;
    bits[i] = (unsigned char)b;
  }
}
template <typename T>
__global__ void __launch_bounds__(kBlock) relu_grad_bits_kernel(const unsigned char* __restrict__ bits, T* __restrict__ dx,
                                                                size_t n_bytes) {
  for (size_t i = (size_t)blockIdx.x * kBlock + threadIdx.x; i < n_bytes; i += (size_t)gridDim.x * kBlock) {
    const unsigned b = bits[i];
#pragma unroll
    for (int e = 0; e < 8; ++e)
      if (!((b >> e) & 1u)) dx[i * 8 + e] = from_f32<T>(0.f);
  }
}

int launch_relu_bitmask(int dtype, const void* y, void* bits, size_t n, cudaStream_t s) {
  if (n % 8) return fail(PDNN_INVALID_PARAMETER, "relu bitmask: the element count must be a multiple of 8");
  const int sms = device_sm_count();
  return dispatch_dtype(dtype, [&](auto tag) {
    using T = decltype(tag);
    relu_bitmask_kernel<T><<<grid_for(n / 8, kBlock, sms), kBlock, 0, s>>>(static_cast<const T*>(y),
                                                                          static_cast<unsigned char*>(bits), n / 8);
    return check_launch("relu bitmask");
  });
}

int launch_relu_grad_bits(int dtype, const void* bits, void* dx, size_t n, cudaStream_t s) {
  if (n % 8) return fail(PDNN_INVALID_PARAMETER, "relu bitmask: the element count must be a multiple of 8");
  const int sms = device_sm_count();
  return dispatch_dtype(dtype, [&](auto tag) {
    using T = decltype(tag);
    relu_grad_bits_kernel<T><<<grid_for(n / 8, kBlock, sms), kBlock, 0, s>>>(static_cast<const unsigned char*>(bits),
                                                                            static_cast<T*>(dx), n / 8);
    return check_launch("relu gradient from a bitmask");
  });
}

}  // namespace pdnn
