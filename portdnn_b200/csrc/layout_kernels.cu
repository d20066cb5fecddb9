// Tensor transposition (portDNN's transpose::launch, include/portdnn/transpose/launch.h:66-233,
// src/transpose/kernels.h) and, built on it, the NCHW / FCHW forms of convolution and pooling.
//
// The reference moves elements as raw words of the element's size (it casts every type to an
// unsigned integer of that width, include/portdnn/internal/transpose/launch.h:47-83); so does this
// file.  A permutation whose effect is "batches of a 2-D transpose" - NHWC <-> NCHW, HWCF <-> FCHW
// with merged extents, any swap of two groups of neighbouring extents - goes through a 32 x 32
// shared-memory tile so that both the reads and the writes are coalesced; everything else takes a
// kernel that decomposes the output index.
//
// NCHW convolution and pooling run the NHWC kernels between two such transposes, in scratch taken
// from the stream-ordered allocator for the call.  The reference has dedicated NCHW direct kernels
// (src/conv2d/direct/kernels_nchw.h) whose results these match.
#include "common.cuh"
#include "tc_gemm.cuh"

namespace pdnn {
namespace {

constexpr int kMaxDims = 6;

struct PermuteArgs {
  int n_dims;
  int out_dims[kMaxDims];         // extents of the output, outermost first
  long long in_strides[kMaxDims]; // stride in the INPUT of the extent that output dimension d walks
};

template <typename W>
__global__ void __launch_bounds__(256) permute_kernel(const W* __restrict__ in, W* __restrict__ out, PermuteArgs a, size_t n) {
  for (size_t idx = (size_t)blockIdx.x * 256 + threadIdx.x; idx < n; idx += (size_t)gridDim.x * 256) {
    size_t rest = idx;
    long long src = 0;
#pragma unroll
    for (int d = kMaxDims - 1; d >= 0; --d) {
      if (d < a.n_dims) {
        const int i = (int)(rest % (size_t)a.out_dims[d]);
        rest /= (size_t)a.out_dims[d];
        src += (long long)i * a.in_strides[d];
      }
    }
    out[idx] = in[src];
  }
}

// out[b][c][r] = in[b][r][c] for b < batches, r < rows, c < cols.
template <typename W>
__global__ void __launch_bounds__(256) transpose_tiles_kernel(const W* __restrict__ in, W* __restrict__ out, int rows,
                                                              int cols, long long tiles_per_batch, int tiles_c,
                                                              long long total_tiles) {
  __shared__ W tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8 threads
  for (long long t = blockIdx.x; t < total_tiles; t += gridDim.x) {
    const long long b = t / tiles_per_batch;
    const int rem = (int)(t - b * tiles_per_batch);
    const int r0 = (rem / tiles_c) * 32, c0 = (rem % tiles_c) * 32;
    const W* src = in + (size_t)b * rows * cols;
    W* dst = out + (size_t)b * rows * cols;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int r = r0 + ty + 8 * k, c = c0 + tx;
      if (r < rows && c < cols) tile[ty + 8 * k][tx] = src[(size_t)r * cols + c];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int c = c0 + ty + 8 * k, r = r0 + tx;
      if (r < rows && c < cols) dst[(size_t)c * rows + r] = tile[tx][ty + 8 * k];
    }
    __syncthreads();
  }
}

template <typename W>
int run_transpose(const void* in, void* out, const int* dims, int n_dims, const int* perm, cudaStream_t s) {
  const int sms = device_sm_count();
  if (sms <= 0) return fail(PDNN_ALLOCATION_PROBLEM, "transpose: no sm_100 CUDA device");
  size_t n = 1;
  for (int d = 0; d < n_dims; ++d) n *= (size_t)dims[d];
  if (n == 0) return PDNN_OK;
  // drop extents of one, then merge input extents that stay neighbours in the output
  int dd[kMaxDims], pp[kMaxDims], m = 0;
  {
    int keep[kMaxDims], rank[kMaxDims], k = 0;
    for (int d = 0; d < n_dims; ++d) keep[d] = dims[d] != 1 ? k++ : -1;
    for (int d = 0; d < n_dims; ++d)
      if (keep[d] >= 0) dd[keep[d]] = dims[d];
    for (int d = 0; d < n_dims; ++d)
      if (keep[perm[d]] >= 0) pp[m++] = keep[perm[d]];
    (void)rank;
  }
  // merge runs: output positions j, j+1 that read input dims q, q+1
  int od[kMaxDims], src_dim[kMaxDims], groups = 0;
  long long in_stride[kMaxDims];
  {
    long long st[kMaxDims];
    long long acc = 1;
    for (int d = m - 1; d >= 0; --d) {
      st[d] = acc;
      acc *= dd[d];
    }
    for (int j = 0; j < m; ++j) {
      if (groups > 0 && pp[j] == pp[j - 1] + 1) {
        od[groups - 1] *= dd[pp[j]];
        in_stride[groups - 1] = st[pp[j]];
      } else {
        od[groups] = dd[pp[j]];
        in_stride[groups] = st[pp[j]];
        src_dim[groups] = pp[j];
        ++groups;
      }
    }
  }
  if (groups <= 1) {  // nothing moves
    if (in != out && cudaMemcpyAsync(out, in, n * sizeof(W), cudaMemcpyDeviceToDevice, s) != cudaSuccess) {
      cudaGetLastError();
      return fail(PDNN_ALLOCATION_PROBLEM, "transpose: copy failed");
    }
    return PDNN_OK;
  }
  // [batch][A][B] -> [batch][B][A]: two or three groups where the last two swap
  const bool swap2 = groups == 2 && src_dim[0] > src_dim[1];
  const bool swap3 = groups == 3 && src_dim[0] < src_dim[2] && src_dim[2] < src_dim[1];
  if (swap2 || swap3) {
    const long long batches = swap3 ? od[0] : 1;
    const int cols = swap3 ? od[1] : od[0], rows = swap3 ? od[2] : od[1];  // input is [rows][cols]
    const int tiles_c = (cols + 31) / 32, tiles_r = (rows + 31) / 32;
    const long long per_batch = (long long)tiles_c * tiles_r, total = per_batch * batches;
    const unsigned grid = (unsigned)std::min<long long>(total, (long long)sms * 16);
    transpose_tiles_kernel<W><<<grid, 256, 0, s>>>(static_cast<const W*>(in), static_cast<W*>(out), rows, cols, per_batch,
                                                   tiles_c, total);
    return check_launch("transpose (tiles)");
  }
  PermuteArgs a;
  a.n_dims = groups;
  for (int g = 0; g < groups; ++g) {
    a.out_dims[g] = od[g];
    a.in_strides[g] = in_stride[g];
  }
  permute_kernel<W><<<grid_for(n, 256, sms), 256, 0, s>>>(static_cast<const W*>(in), static_cast<W*>(out), a, n);
  return check_launch("transpose (general)");
}

// Scratch from the stream-ordered allocator, released when it goes out of scope.
struct AsyncScratch {
  void* p = nullptr;
  cudaStream_t s;
  explicit AsyncScratch(cudaStream_t stream) : s(stream) {}
  bool get(size_t bytes) {
    if (cudaMallocAsync(&p, bytes > 0 ? bytes : 16, s) != cudaSuccess) {
      cudaGetLastError();
      p = nullptr;
      return false;
    }
    return true;
  }
  ~AsyncScratch() {
    if (p != nullptr) cudaFreeAsync(p, s);
  }
};

}  // namespace

int launch_transpose(int elem_bytes, const void* in, void* out, const int* dims, int n_dims, const int* perm,
                     cudaStream_t s) {
  if (n_dims < 1 || n_dims > kMaxDims) return fail(PDNN_INVALID_PARAMETER, "transpose: 1 to %d dimensions are supported", kMaxDims);
  bool seen[kMaxDims] = {};
  for (int d = 0; d < n_dims; ++d) {
    if (dims[d] <= 0) return fail(PDNN_INVALID_PARAMETER, "transpose: extents must be positive");
    if (perm[d] < 0 || perm[d] >= n_dims || seen[perm[d]])
      return fail(PDNN_INVALID_PARAMETER, "transpose: not a permutation of the dimensions");
    seen[perm[d]] = true;
  }
  if (in == out) return fail(PDNN_INVALID_PARAMETER, "transpose: cannot work in place");
  switch (elem_bytes) {
    case 1: return run_transpose<uint8_t>(in, out, dims, n_dims, perm, s);
    case 2: return run_transpose<uint16_t>(in, out, dims, n_dims, perm, s);
    case 4: return run_transpose<uint32_t>(in, out, dims, n_dims, perm, s);
    case 8: return run_transpose<uint64_t>(in, out, dims, n_dims, perm, s);
  }
  return fail(PDNN_INVALID_PARAMETER, "transpose: element size %d", elem_bytes);
}

// conv2d with input_format NCHW and filter_format FCHW: `run` is handed the NHWC / HWCF tensors.
int conv2d_nchw(int pass, int dtype, const void* in, const void* fil, void* out, const PdnnConv2DParams& p, bool read_out,
                cudaStream_t s, const ConvRunner& run) {
  const int es = (int)dtype_size(dtype);
  const int x_dims[4] = {p.batch, p.channels, p.in_rows, p.in_cols};      // NCHW
  const int y_dims[4] = {p.batch, p.features, p.out_rows, p.out_cols};    // NCHW
  const int w_dims[4] = {p.features, p.channels / p.groups, p.window_rows, p.window_cols};  // FCHW
  const int to_nhwc[4] = {0, 2, 3, 1}, to_hwcf[4] = {2, 3, 1, 0};
  const size_t n_x = (size_t)x_dims[0] * x_dims[1] * x_dims[2] * x_dims[3];
  const size_t n_y = (size_t)y_dims[0] * y_dims[1] * y_dims[2] * y_dims[3];
  const size_t n_w = (size_t)w_dims[0] * w_dims[1] * w_dims[2] * w_dims[3];
  // argument slots: Forward (x, w) -> y; InputBackprop (dy, w) -> dx; FilterBackprop (x, dy) -> dW
  const int* in_dims = pass == PDNN_INPUT_BACKPROP ? y_dims : x_dims;
  const size_t n_in = pass == PDNN_INPUT_BACKPROP ? n_y : n_x;
  const bool fil_is_tensor = pass == PDNN_FILTER_BACKPROP;
  const size_t n_fil = fil_is_tensor ? n_y : n_w;
  const size_t n_out = pass == PDNN_FORWARD ? n_y : pass == PDNN_INPUT_BACKPROP ? n_x : n_w;
  AsyncScratch a(s), b(s), c(s);
  if (!a.get(n_in * es) || !b.get(n_fil * es) || !c.get(n_out * es))
    return fail(PDNN_ALLOCATION_PROBLEM, "conv2d (NCHW): cannot allocate the NHWC copies");
  int st = launch_transpose(es, in, a.p, in_dims, 4, to_nhwc, s);
  if (st == PDNN_OK) st = launch_transpose(es, fil, b.p, fil_is_tensor ? y_dims : w_dims, 4, fil_is_tensor ? to_nhwc : to_hwcf, s);
  if (st != PDNN_OK) return st;
  // NHWC / HWCF extents of the output, for the way back
  const int y_nhwc[4] = {p.batch, p.out_rows, p.out_cols, p.features}, x_nhwc[4] = {p.batch, p.in_rows, p.in_cols, p.channels};
  const int w_hwcf[4] = {p.window_rows, p.window_cols, p.channels / p.groups, p.features};
  const int to_nchw[4] = {0, 3, 1, 2}, to_fchw[4] = {3, 2, 0, 1};
  const int* out_nhwc = pass == PDNN_FORWARD ? y_nhwc : pass == PDNN_INPUT_BACKPROP ? x_nhwc : w_hwcf;
  if (read_out) {  // a blend reads the previous output
    const int* out_dims = pass == PDNN_FORWARD ? y_dims : pass == PDNN_INPUT_BACKPROP ? x_dims : w_dims;
    st = launch_transpose(es, out, c.p, out_dims, 4, pass == PDNN_FILTER_BACKPROP ? to_hwcf : to_nhwc, s);
    if (st != PDNN_OK) return st;
  }
  PdnnConv2DParams q = p;
  q.input_format = 0;
  q.filter_format = 0;
  st = run(a.p, b.p, c.p, q);
  if (st != PDNN_OK) return st;
  return launch_transpose(es, c.p, out, out_nhwc, 4, pass == PDNN_FILTER_BACKPROP ? to_fchw : to_nchw, s);
}

// Pooling with input_format NCHW: every tensor of the call is transposed to NHWC and back.
int pooling_nchw(int dtype, const void* const* inputs, const size_t* input_rows, int n_inputs, void* out, size_t out_rows,
                 const PdnnPoolingParams& p, cudaStream_t s, const PoolRunner& run) {
  // a tensor of `rows` spatial positions per (batch, channel): NCHW [N][C][rows] <-> NHWC [N][rows][C]
  const int es = (int)dtype_size(dtype);
  AsyncScratch tmp[3] = {AsyncScratch(s), AsyncScratch(s), AsyncScratch(s)};
  AsyncScratch res(s);
  const void* nhwc[3] = {nullptr, nullptr, nullptr};
  if (n_inputs > 3) return fail(PDNN_INVALID_PARAMETER, "pooling (NCHW): too many tensors");
  for (int i = 0; i < n_inputs; ++i) {
    const int dims[3] = {p.batch, p.channels, (int)input_rows[i]}, perm[3] = {0, 2, 1};
    if (!tmp[i].get((size_t)p.batch * p.channels * input_rows[i] * es))
      return fail(PDNN_ALLOCATION_PROBLEM, "pooling (NCHW): cannot allocate the NHWC copies");
    const int st = launch_transpose(es, inputs[i], tmp[i].p, dims, 3, perm, s);
    if (st != PDNN_OK) return st;
    nhwc[i] = tmp[i].p;
  }
  if (!res.get((size_t)p.batch * p.channels * out_rows * es))
    return fail(PDNN_ALLOCATION_PROBLEM, "pooling (NCHW): cannot allocate the NHWC result");
  PdnnPoolingParams q = p;
  q.input_format = 0;
  const int st = run(nhwc, res.p, q);
  if (st != PDNN_OK) return st;
  const int dims[3] = {p.batch, (int)out_rows, p.channels}, perm[3] = {0, 2, 1};
  return launch_transpose(es, res.p, out, dims, 3, perm, s);
}

}  // namespace pdnn
