// Winograd F(2x2, 3x3) convolution for Algorithm::Winograd / WinogradLarge: forward and input
// backprop of 3x3, stride-1 convolutions.
//
//   V[xi][tile][c] = (B^T d B)[xi]      input transform of each 4x4 patch d (stride 2 between tiles)
//   U[xi][c][k]    = (G g G^T)[xi]      filter transform
//   M[xi]          = V[xi] * U[xi]      16 independent [tiles x C] x [C x K] products on the
//                                       tcgen05 engine (one batched pdnn matmul)
//   Y tile (2x2)   = A^T M A            output transform, with bias / activation applied on the way
//
// The structure (three transforms around a batched matmul, scratch carved from the caller's
// workspace as [U | V | M]) is the reference's, include/portdnn/internal/conv2d/winograd/launch.h:68-264,
// with its matrices for F(2x2,3x3), src/conv2d/winograd/kernels/tiles_impl.h:70-198.  Input backprop
// is the forward algorithm on dy with the filter mirrored and its channel/feature axes swapped
// (include/portdnn/internal/conv2d/winograd/kernel_params.h:46-55).  The transforms are separate
// HBM passes; on this hardware the implicit-GEMM kernel is the faster way to run the same layer,
// so the default selector does not pick this path.
#include "common.cuh"
#include "tc_gemm.cuh"

namespace pdnn {
namespace {

constexpr int kBlock = 256;

struct WinoGeometry {
  int batch, in_rows, in_cols, channels, features, out_rows, out_cols, pad_rows, pad_cols;
  int tile_rows, tile_cols;  // ceil(out/2)
  long long tiles;           // batch * tile_rows * tile_cols
};

// One thread: one tile, one channel.  Adjacent threads take adjacent channels.
template <typename T>
__global__ void __launch_bounds__(kBlock)
    wino_input_transform_kernel(const T* __restrict__ x, T* __restrict__ v, WinoGeometry g, size_t n_items) {
  for (size_t idx = (size_t)blockIdx.x * kBlock + threadIdx.x; idx < n_items; idx += (size_t)gridDim.x * kBlock) {
    const int c = (int)(idx % g.channels);
    const long long tile = (long long)(idx / g.channels);
    const int tc = (int)(tile % g.tile_cols);
    const int tr = (int)((tile / g.tile_cols) % g.tile_rows);
    const int n = (int)(tile / ((long long)g.tile_cols * g.tile_rows));
    const int h0 = 2 * tr - g.pad_rows, w0 = 2 * tc - g.pad_cols;
    float d[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int h = h0 + i, w = w0 + j;
        d[i][j] = (h >= 0 && h < g.in_rows && w >= 0 && w < g.in_cols)
                      ? to_f32(__ldg(x + (((size_t)n * g.in_rows + h) * g.in_cols + w) * g.channels + c))
                      : 0.f;
      }
    // t = B^T d, rows: [d0-d2, d1+d2, d2-d1, d1-d3]
    float t[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      t[0][j] = d[0][j] - d[2][j];
      t[1][j] = d[1][j] + d[2][j];
      t[2][j] = d[2][j] - d[1][j];
      t[3][j] = d[1][j] - d[3][j];
    }
    // V = t B, columns likewise
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float o0 = t[i][0] - t[i][2], o1 = t[i][1] + t[i][2], o2 = t[i][2] - t[i][1], o3 = t[i][1] - t[i][3];
      const size_t base = ((size_t)(i * 4) * g.tiles + tile) * g.channels + c;
      const size_t step = (size_t)g.tiles * g.channels;
      v[base] = from_f32<T>(o0);
      v[base + step] = from_f32<T>(o1);
      v[base + 2 * step] = from_f32<T>(o2);
      v[base + 3 * step] = from_f32<T>(o3);
    }
  }
}

// One thread: one (c, k) pair of the GEMM's [C x K] operand.  For the input backprop the GEMM
// reduces over features and produces channels, and the filter is read mirrored.
template <typename T>
__global__ void __launch_bounds__(kBlock)
    wino_filter_transform_kernel(const T* __restrict__ w, T* __restrict__ u, int C, int K, int backprop) {
  const int red = backprop ? K : C, cols = backprop ? C : K;  // GEMM reduction / output extents
  const size_t n_items = (size_t)red * cols;
  for (size_t idx = (size_t)blockIdx.x * kBlock + threadIdx.x; idx < n_items; idx += (size_t)gridDim.x * kBlock) {
    const int col = (int)(idx % cols), r0 = (int)(idx / cols);
    const int c = backprop ? col : r0, k = backprop ? r0 : col;
    float gm[3][3];
#pragma unroll
    for (int r = 0; r < 3; ++r)
#pragma unroll
      for (int s = 0; s < 3; ++s) {
        const int rr = backprop ? 2 - r : r, ss = backprop ? 2 - s : s;
        gm[r][s] = to_f32(__ldg(w + (((size_t)rr * 3 + ss) * C + c) * K + k));
      }
    // t = G g  (4x3), G = [[1,0,0],[.5,.5,.5],[.5,-.5,.5],[0,0,1]]
    float t[4][3];
#pragma unroll
    for (int s = 0; s < 3; ++s) {
      t[0][s] = gm[0][s];
      t[1][s] = 0.5f * (gm[0][s] + gm[1][s] + gm[2][s]);
      t[2][s] = 0.5f * (gm[0][s] - gm[1][s] + gm[2][s]);
      t[3][s] = gm[2][s];
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float o0 = t[i][0], o1 = 0.5f * (t[i][0] + t[i][1] + t[i][2]), o2 = 0.5f * (t[i][0] - t[i][1] + t[i][2]),
                  o3 = t[i][2];
      const size_t base = (size_t)(i * 4) * n_items + idx, step = n_items;
      u[base] = from_f32<T>(o0);
      u[base + step] = from_f32<T>(o1);
      u[base + 2 * step] = from_f32<T>(o2);
      u[base + 3 * step] = from_f32<T>(o3);
    }
  }
}

// One thread: one tile, one output column (feature, or channel for the backprop).
// M is fp32 whatever T is: rounding the sixteen products to 16 bits before they are combined (with
// cancellation) would cost the 16-bit types about a factor of two in accuracy.
template <typename T>
__global__ void __launch_bounds__(kBlock)
    wino_output_transform_kernel(const float* __restrict__ m, T* __restrict__ y, const T* __restrict__ bias, int act,
                                 float alpha, float beta, WinoGeometry g, int cols, size_t n_items) {
  for (size_t idx = (size_t)blockIdx.x * kBlock + threadIdx.x; idx < n_items; idx += (size_t)gridDim.x * kBlock) {
    const int k = (int)(idx % cols);
    const long long tile = (long long)(idx / cols);
    const int tc = (int)(tile % g.tile_cols);
    const int tr = (int)((tile / g.tile_cols) % g.tile_rows);
    const int n = (int)(tile / ((long long)g.tile_cols * g.tile_rows));
    float mm[4][4];
    const size_t step = (size_t)g.tiles * cols;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) mm[i][j] = __ldg(m + (size_t)(i * 4 + j) * step + (size_t)tile * cols + k);
    // t = A^T m (2x4), A^T = [[1,1,1,0],[0,1,-1,-1]]
    float t[2][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      t[0][j] = mm[0][j] + mm[1][j] + mm[2][j];
      t[1][j] = mm[1][j] - mm[2][j] - mm[3][j];
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float o[2] = {t[i][0] + t[i][1] + t[i][2], t[i][1] - t[i][2] - t[i][3]};
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int oh = 2 * tr + i, ow = 2 * tc + j;
        if (oh >= g.out_rows || ow >= g.out_cols) continue;
        const size_t off = (((size_t)n * g.out_rows + oh) * g.out_cols + ow) * cols + k;
        float v = alpha * o[j];
        if (bias != nullptr) v += to_f32(bias[k]);
        v = apply_activation(v, act);
        if (beta != 0.f) v += beta * to_f32(y[off]);
        y[off] = from_f32<T>(v);
      }
    }
  }
}

WinoGeometry geometry(int pass, const PdnnConv2DParams& p) {
  WinoGeometry g;
  const bool bp = pass == PDNN_INPUT_BACKPROP;
  // the backprop convolves dy (out-sized, K channels) into dx (in-sized, C channels) with pad' = 2 - pad
  g.batch = p.batch;
  g.in_rows = bp ? p.out_rows : p.in_rows;
  g.in_cols = bp ? p.out_cols : p.in_cols;
  g.channels = bp ? p.features : p.channels;
  g.features = bp ? p.channels : p.features;
  g.out_rows = bp ? p.in_rows : p.out_rows;
  g.out_cols = bp ? p.in_cols : p.out_cols;
  g.pad_rows = bp ? 2 - p.pad_rows : p.pad_rows;
  g.pad_cols = bp ? 2 - p.pad_cols : p.pad_cols;
  g.tile_rows = (g.out_rows + 1) / 2;
  g.tile_cols = (g.out_cols + 1) / 2;
  g.tiles = (long long)g.batch * g.tile_rows * g.tile_cols;
  return g;
}

}  // namespace

bool winograd_applicable(int pass, int dtype, const PdnnConv2DParams& p) {
  const int align = dtype == PDNN_F32 ? 4 : 8;
  return (pass == PDNN_FORWARD || pass == PDNN_INPUT_BACKPROP) && p.window_rows == 3 && p.window_cols == 3 &&
         p.stride_rows == 1 && p.stride_cols == 1 && p.groups == 1 && p.input_format == 0 && p.filter_format == 0 &&
         p.channels % align == 0 && p.features % align == 0 && p.pad_rows <= 2 && p.pad_cols <= 2;
}

// Elements (of dtype) of scratch: 16 * (C*K + tiles*C + tiles*K), the reference's formula for
// A = B = 4 (include/portdnn/conv2d/workspace_size.h:53-73), with the last term counted twice for
// 16-bit types because the products M are kept in fp32.
size_t winograd_workspace_elems(int pass, int dtype, const PdnnConv2DParams& p) {
  const WinoGeometry g = geometry(pass, p);
  const size_t align = 64;  // keep every sub-buffer 16-byte aligned
  auto up = [&](size_t n) { return (n + align - 1) / align * align; };
  return up(16 * (size_t)g.channels * g.features) + up(16 * (size_t)g.tiles * g.channels) +
         up(16 * (size_t)g.tiles * g.features) * (sizeof(float) / dtype_size(dtype));
}

int launch_winograd(int pass, int dtype, const void* in, const void* fil, void* out, const PdnnConv2DParams& p,
                    const PdnnConvEpilogue* epi, void* ws, size_t ws_elems, cudaStream_t s) {
  if (ws == nullptr || ws_elems == 0)
    return fail(PDNN_INSUFFICIENT_WORKSPACE, "winograd: a workspace is required (query pdnn_conv2d_workspace_size)");
  if (ws_elems < winograd_workspace_elems(pass, dtype, p) || !aligned16(ws))
    return fail(PDNN_INSUFFICIENT_WORKSPACE, "winograd: workspace of %zu elements, %zu needed", ws_elems,
                winograd_workspace_elems(pass, dtype, p));
  const int sms = device_sm_count();
  if (sms <= 0) return fail(PDNN_ALLOCATION_PROBLEM, "no CUDA device");
  const WinoGeometry g = geometry(pass, p);
  if (g.tiles > 0x7FFFFFFFll) return fail(PDNN_INDEX_EXCEEDED, "winograd: too many tiles");
  const size_t es = dtype_size(dtype);
  auto up = [&](size_t n) { return (n + 63) / 64 * 64; };
  char* u = static_cast<char*>(ws);
  char* v = u + up(16 * (size_t)g.channels * g.features) * es;
  char* m = v + up(16 * (size_t)g.tiles * g.channels) * es;
  const size_t n_in = (size_t)g.tiles * g.channels, n_fil = (size_t)g.channels * g.features,
               n_out = (size_t)g.tiles * g.features;
  const void* bias = epi ? epi->bias : nullptr;
  const int act = epi ? epi->activation : PDNN_ACT_NONE;
  const float alpha = epi ? epi->alpha : 1.f, beta = epi ? epi->beta : 0.f;
  auto run = [&](auto tag) -> int {
    using T = decltype(tag);
    wino_filter_transform_kernel<T><<<grid_for(n_fil, kBlock, sms), kBlock, 0, s>>>(
        static_cast<const T*>(fil), reinterpret_cast<T*>(u), p.channels, p.features, pass == PDNN_INPUT_BACKPROP);
    int st = check_launch("winograd filter transform");
    if (st != PDNN_OK) return st;
    wino_input_transform_kernel<T><<<grid_for(n_in, kBlock, sms), kBlock, 0, s>>>(static_cast<const T*>(in),
                                                                                 reinterpret_cast<T*>(v), g, n_in);
    st = check_launch("winograd input transform");
    if (st != PDNN_OK) return st;
    // 16 products [tiles x C] x [C x K]
    if (tc_matmul_supported(dtype, 0, 0, v, u, m, 16, (int)g.tiles, g.channels, g.features))
      st = tc_matmul(dtype, 0, 0, v, u, m, 16, (int)g.tiles, g.channels, g.features, 0.f, s, /*out_f32=*/true);
    else
      st = simt_matmul(dtype, 0, 0, v, u, m, 16, (int)g.tiles, g.channels, g.features, 0.f, s, /*out_f32=*/true);
    if (st != PDNN_OK) return st;
    wino_output_transform_kernel<T><<<grid_for(n_out, kBlock, sms), kBlock, 0, s>>>(
        reinterpret_cast<const float*>(m), static_cast<T*>(out), static_cast<const T*>(bias), act, alpha, beta, g,
        g.features, n_out);
    return check_launch("winograd output transform");
  };
  switch (dtype) {
    case PDNN_F32: return run(float{});
    case PDNN_F16: return run(__half{});
    case PDNN_BF16: return run(__nv_bfloat16{});
  }
  return fail(PDNN_INVALID_PARAMETER, "unknown dtype %d", dtype);
}

}  // namespace pdnn
