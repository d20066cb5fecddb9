// Implicit-GEMM engine on the Blackwell tensor cores: one persistent, warp-specialised kernel
// serves conv2d forward / input backprop / filter backprop and the (batched) matmul.
//
//   D[128 x BN] (fp32, in TMEM) = sum over reduction steps of A_step[128 x 64] * B_step[64 x BN]
//
// Each step's operands are fetched by TMA straight from the NHWC activation tensor and the filter
// (no im2col buffer): a 128-row A tile is a box of output pixels (tw x th x tn) shifted by the
// filter tap, with TMA's out-of-bounds zero fill standing in for the padding.  Stride-2
// convolutions read through one tensor map per input parity, so every load is a dense box.
// Operands land in shared memory in the 128-byte swizzled layout that tcgen05.mma consumes; the
// accumulators live in tensor memory (two buffers, so the epilogue of one tile overlaps the
// main loop of the next) and are written to global memory by four epilogue warps with bias,
// activation and alpha/beta applied on the way.
//
// fp32 tensors are multiplied as three TF32 products (hi*hi + hi*lo + lo*hi): four extra warps
// split each landed stage into its high and low parts in shared memory before the MMA warp
// consumes it.
//
// Warp roles (192 threads; 320 with the split): warp 0 TMA producer, warp 1 MMA issuer and TMEM
// owner, warps 2-5 epilogue, warps 6-9 hi/lo split.
#include "tc_gemm.cuh"
#include "umma.cuh"

#include <algorithm>
#include <cstring>
#include <mutex>
#include <vector>

namespace pdnn {

using namespace umma;

namespace {

constexpr int kMaxTaps = 64;
constexpr int kTileM = 128;
constexpr int kABytes = kTileM * 128;  // one A stage: 128 rows of 128 bytes
constexpr int kMaxStages = 8;
constexpr int kSmemBudget = 227 * 1024;
constexpr int kBarsPerGroup = 3 * kMaxStages + 4;  // full, empty, ready per stage; accumulator full / empty x 2
constexpr int kBarBlockBytes = 512;                // barriers of two groups, the resident-B barrier, TMEM slot, abort flag

__device__ unsigned g_error_record[4];

// One reduction step of a forward-style GEMM: which input map, at which pixel offset, against which
// filter tap.  In halo mode an entry stands for `cnt` taps that differ only by one input row each
// (dh, dh + 1, ...; filter taps b_tap, b_tap + b_step, ...): their A tiles are overlapping row
// ranges of ONE copy of th + cnt - 1 input rows.
struct TapEntry {
  short dw, dh, a_map, b_tap, cnt, b_step;
};

enum BMode { B_MN_3 = 0, B_K_3 = 1, B_K_FHWC = 2, B_MN_FHWC = 3, B_MN_4 = 4, B_K_4 = 5, B_MN_3X = 6 };

struct alignas(64) GemmArgs {
  CUtensorMap a_map[4];
  CUtensorMap b_map;
  CUtensorMap out_map;  // used when tma_store != 0
  TapEntry taps[kMaxTaps];
  int a_mn;          // 0: A rows are output pixels (K-major); 1: A rows are reduction steps (MN-major)
  int b_mode;        // BMode
  int epr;           // elements per 128-byte row: 64 (16-bit) or 32 (fp32)
  int n_tiles, bn;   // column tiles and their width
  int tiles_w, tiles_h, tiles_n;  // row-tile grid
  int tw, th, tn;    // a_mn == 0: pixel box of a row tile; a_mn == 1: pixel box of a reduction slab
  int etw, eth, etn; // pixel box of a row tile as the epilogue sees it
  int num_taps;
  int b_presplit;    // fp32 (3xTF32): the lo part of B arrives by TMA too (b_map_lo); only A is split in the kernel
  int cta_pair;      // 1: run by umma_gemm_pair2_kernel (clusters of two CTAs, 256 x 256 tiles)
  int tap_pack;      // a_mn == 1: taps per tile (2: the second 64 rows of the A tile are the next tap's channels)
  int cblocks;       // a_mn == 0: reduction blocks per tap
  int slabs_w, slabs_h, slabs_n, splits, slabs_per_split, split_is_batch;  // a_mn == 1
  int b_batch_mul;
  int stages, tmem_cols;
  unsigned idesc;
  unsigned a_lbo, a_sbo, a_kadv, b_lbo, b_sbo, b_kadv;  // bytes
  unsigned a_layout, b_layout;  // descriptor swizzle codes
  int a_boxes, b_boxes;
  unsigned a_box_bytes, b_box_bytes;
  // epilogue
  void* out;
  const void* bias;
  int out_dtype, act;
  float alpha, beta;
  int ext_w, ext_h, ext_n, ext_cols;
  long long stride_w, stride_h, stride_n, split_stride, tap_stride;  // elements
  int vec_ok;  // rows are 16-byte aligned: packed stores allowed
  int tma_store;  // 1: the epilogue stages 128-byte column blocks in shared memory and stores them by TMA
  int cpb;        // output columns per 128-byte block: 64 (16-bit) or 32 (fp32)
  int nsw;        // staging slices per epilogue warp (1, 2 or 4)
  int groups;     // pipelines per CTA (1 or 2; always 1 for the fp32 variant)
  int acc_bufs;   // accumulator buffers per group (1 or 2)
  int acc_stride; // TMEM columns between accumulator buffers
  int bias_smem_bytes;  // size of the CTA's bias copy (fast epilogue only), a multiple of 128
  int epi_fast;   // 1: 16-bit output, alpha 1, bias/ReLU done on packed pairs (see epilogue_tile_tma_fast)
  // 1: the whole B operand (every column tile, every reduction step) is copied into shared memory
  // once per CTA and stays there; pipeline stages then carry A tiles only.  2: the same for the one
  // column tile the CTA works on (the grid is then a multiple of n_tiles, so that the tiles
  // blockIdx.x, blockIdx.x + gridDim.x, ... all share their column tile).
  int b_res;
  unsigned b_res_bytes;
  // 1: halo mode (needs b_res, tn == 1, tw % 8 == 0): a stage holds th + cnt - 1 input rows of tw
  // pixels and feeds the MMAs of cnt taps; halo_stage_bytes is the stage size.
  int halo;
  unsigned halo_stage_bytes;
  int res_taps;  // filter taps per column tile in the resident copy (halo mode: the sum of cnt)
  // 1: pair mode.  The two pipelines of a CTA work on two neighbouring row tiles of the SAME column
  // tile and share one ring: a stage holds both A tiles and one B tile, loaded by one producer,
  // and is released when both issuers have read it.  The tile grid in tiles_w / tiles_h / tiles_n
  // counts PAIRS along dimension pair_dim (1: w, 2: h, 3: n).  Halves the B bytes an SM pulls
  // from L2 per MMA, which is what bounds long reductions over wide filters.
  int pair, pair_dim;
  int bias_tile_only;  // 1: the CTA keeps one column tile's bias slice (the grid is a multiple of n_tiles)
  // Geometry of a reduction step: bytes per A row (128, or 64 for the narrow few-channel stem
  // layout), MMAs per step (row bytes / 32) and bytes of one step's B tile (bn * row bytes).
  int a_row_bytes, kmmas;
  unsigned b_step_bytes;
  // Fast epilogue only: the forward output of the layer whose ReLU the result is the gradient of,
  // laid out exactly like `out` (stride_w / stride_h / stride_n).  Where it is not positive the
  // result is replaced by zero: pointwise::launch<Relu, Gradient> applied on the way out.
  const void* relu_mask;
  CUtensorMap mask_map;  // the mask tensor with the geometry of out_map (set when relu_mask is)
  CUtensorMap b_map_lo;  // b_presplit: the lo parts of B, same geometry as b_map
  // One bit per output element, bit e of byte (element offset / 8): "the element is positive".
  // bitmask_out (packed forward epilogue): written beside the output, for a later input backprop;
  // mask_bits (mask epilogue): the ReLU mask in that form, read instead of the mask tensor.
  void* bitmask_out;
  const void* mask_bits;
  int mask_slots;        // 4 KB mask slots per epilogue warp: 2 where shared memory allows, else 1
  // 1: the filter (the resident B copy) and the bias are known not to be written by the kernel that
  // precedes this one in the stream: they are fetched before the wait for that kernel
  int early_b;
  int accumulate;  // packed 16-bit epilogues, no bias: the block already in the output is added (before the mask)
  int reduce_add;  // staged fp32 epilogue of the filter backprop: every pixel split adds its tile to the output
  int mask_smem_bytes;  // the barriers of the epilogue warps' mask slots (the slots themselves follow the staging slices)
  // Time limit of one barrier wait; a wait that lasts longer means a lost arrival, and the CTA
  // gives up (see umma::mbar_wait).
  unsigned long long wait_limit_ns;
};

struct TileCoord {
  int w0, h0, n0, nf0, nt, tap, split;  // nt: column-tile index, nf0 = nt * bn
  long long out_off;
  int ks_begin, ks_end;
};

// Walks the tiles first, first + step, ... of one pipeline without a division per tile: the tile
// index is kept as four mixed-radix digits (column tile, row-tile column, row-tile row or tap, the
// rest) and the step is added digit by digit.  A lone thread pays several hundred cycles for the
// six divisions a direct decode needs, which is a visible gap between two short tiles.
struct TileWalker {
  int r0, r1, r2;      // radices of digits 0..2; digit 3 is unbounded
  int d0, d1, d2, d3;  // digits of the current tile
  int s0, s1, s2, s3;  // digits of the step

  __device__ __forceinline__ void init(const GemmArgs& a, int first, int step) {
    r0 = a.n_tiles;
    r1 = a.tiles_w;
    r2 = a.a_mn ? (a.num_taps + a.tap_pack - 1) / a.tap_pack : a.tiles_h;
    d0 = first % r0, first /= r0;
    d1 = first % r1, first /= r1;
    d2 = first % r2, d3 = first / r2;
    s0 = step % r0, step /= r0;
    s1 = step % r1, step /= r1;
    s2 = step % r2, s3 = step / r2;
  }
  __device__ __forceinline__ void advance() {
    d0 += s0;
    int c = d0 >= r0 ? 1 : 0;
    d0 -= c ? r0 : 0;
    d1 += s1 + c;
    c = d1 >= r1 ? 1 : 0;
    d1 -= c ? r1 : 0;
    d2 += s2 + c;
    c = d2 >= r2 ? 1 : 0;
    d2 -= c ? r2 : 0;
    d3 += s3 + c;
  }
  __device__ __forceinline__ TileCoord coord(const GemmArgs& a) const {
    TileCoord t;
    t.nt = d0;
    t.nf0 = d0 * a.bn;
    if (!a.a_mn) {
      // in pair mode the paired dimension's digit counts pairs of tiles
      t.w0 = (a.pair_dim == 1 ? 2 * d1 : d1) * a.tw;
      t.h0 = (a.pair_dim == 2 ? 2 * d2 : d2) * a.th;
      t.n0 = (a.pair_dim == 3 ? 2 * d3 : d3) * a.tn;
      t.tap = 0;
      t.split = 0;
      t.out_off = 0;
      t.ks_begin = 0;
      t.ks_end = a.num_taps * a.cblocks;
    } else {
      t.tap = d2 * a.tap_pack;
      t.split = d3;
      t.w0 = d1 * kTileM;
      t.h0 = a.tap_pack > 1 ? t.tap : 0;  // packed taps: the tap is the second digit of a row's position
      t.n0 = 0;
      t.out_off = (long long)t.split * a.split_stride + (a.tap_pack > 1 ? 0ll : (long long)t.tap * a.tap_stride);
      const int total = a.slabs_w * a.slabs_h * a.slabs_n;
      t.ks_begin = a.split_is_batch ? 0 : t.split * a.slabs_per_split;
      t.ks_end = min(t.ks_begin + a.slabs_per_split, total);
    }
    return t;
  }
};

template <typename OutT, int N>
__device__ __forceinline__ void store_chunk(const GemmArgs& a, const uint32_t (&acc)[N], bool zero, OutT* row_ptr,
                                            const OutT* bias, int col0, bool row_valid) {
  // row_ptr points at column 0 of this row; col0 is the first column of the chunk.
  constexpr int P = 16 / sizeof(OutT);  // elements per 16-byte packet
#pragma unroll
  for (int g = 0; g < N / P; ++g) {
    const int c = col0 + g * P;
    if (!row_valid || c >= a.ext_cols) continue;
    float v[P];
#pragma unroll
    for (int i = 0; i < P; ++i) v[i] = zero ? 0.f : a.alpha * __uint_as_float(acc[g * P + i]);
    const bool full = a.vec_ok && (c + P <= a.ext_cols);
    if (bias != nullptr) {
#pragma unroll
      for (int i = 0; i < P; ++i)
        if (c + i < a.ext_cols) v[i] += to_f32(__ldg(bias + c + i));
    }
    if (a.act != PDNN_ACT_NONE) {
#pragma unroll
      for (int i = 0; i < P; ++i) v[i] = apply_activation(v[i], a.act);
    }
    if (full) {
      if (a.beta != 0.f) {
        Vec16<OutT> old;
        old.raw = *reinterpret_cast<const uint4*>(row_ptr + c);
#pragma unroll
        for (int i = 0; i < P; ++i) v[i] += a.beta * to_f32(old.get(i));
      }
      Vec16<OutT> pk;
#pragma unroll
      for (int i = 0; i < P; ++i) pk.set(i, from_f32<OutT>(v[i]));
      *reinterpret_cast<uint4*>(row_ptr + c) = pk.raw;
    } else {
#pragma unroll
      for (int i = 0; i < P; ++i) {
        if (c + i < a.ext_cols) {
          float r = v[i];
          if (a.beta != 0.f) r += a.beta * to_f32(row_ptr[c + i]);
          row_ptr[c + i] = from_f32<OutT>(r);
        }
      }
    }
  }
}

template <typename OutT>
__device__ __forceinline__ void epilogue_tile(const GemmArgs& a, const TileCoord& t, uint32_t tmem_acc, int row,
                                              bool zero) {
  const int lw = row % a.etw, lh = (row / a.etw) % a.eth, ln = row / (a.etw * a.eth);
  const int w = t.w0 + lw, h = t.h0 + lh, n = t.n0 + ln;
  const bool row_valid = (w < a.ext_w) && (h < a.ext_h) && (n < a.ext_n);
  OutT* row_ptr = static_cast<OutT*>(a.out) + t.out_off + (long long)n * a.stride_n + (long long)h * a.stride_h +
                  (long long)w * a.stride_w;
  const OutT* bias = static_cast<const OutT*>(a.bias);
  int c0 = 0;
  for (; c0 + 32 <= a.bn; c0 += 32) {
    uint32_t acc[32];
    if (!zero) {
      tmem_ld_32x32(tmem_acc + (uint32_t)c0, acc);
      tmem_wait_ld();
    }
    store_chunk<OutT, 32>(a, acc, zero, row_ptr, bias, t.nf0 + c0, row_valid);
  }
  if (c0 < a.bn) {  // bn is a multiple of 16
    uint32_t acc[16];
    if (!zero) {
      tmem_ld_32x16(tmem_acc + (uint32_t)c0, acc);
      tmem_wait_ld();
    }
    store_chunk<OutT, 16>(a, acc, zero, row_ptr, bias, t.nf0 + c0, row_valid);
  }
}

// Epilogue through shared memory.  Each of the 128 epilogue threads owns one accumulator row and
// each epilogue warp works on its own: per 128-byte column block (64 16-bit or 32 fp32 outputs)
// the warp converts its 32 rows, writes them to a 4 KB staging slice in the 128-byte swizzled
// layout (16-byte chunk j of row r lands at chunk j ^ (r % 8), which spreads the warp's stores
// over all banks) and its lane 0 issues a TMA store of that 32-row block.  32 consecutive rows of
// a row tile are themselves a box of pixels because every tile extent is a power of two.  The
// tensor map clips rows and columns outside the tensor.  A warp cycles through `nsw` slices and
// only waits for the store that last read the slice it is about to overwrite, so several stores
// per warp are in flight and no warp waits for another.
struct WarpStore {
  uint8_t* buf;       // this warp's slices
  uint32_t buf_addr;  // the same, as a shared-space address
  int nsw;            // number of slices (2 or 4)
  int qw, qh, qn;     // position of the warp's rows inside the row tile
};

__device__ __forceinline__ void wait_slice_free(const WarpStore& ws, int lane) {
  if (lane == 0) {
    if (ws.nsw == 4) bulk_wait_group_read<3>();
    else if (ws.nsw == 2) bulk_wait_group_read<1>();
    else bulk_wait_group_read<0>();
  }
  __syncwarp();
}

__device__ __forceinline__ void issue_slice_store(const GemmArgs& a, const TileCoord& t, const WarpStore& ws,
                                                  uint32_t slot, int col, int lane) {
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0) {
    const int c2 = (a.a_mn ? t.tap : t.h0) + ws.qh, c3 = (a.a_mn ? (a.reduce_add ? 0 : t.split) : t.n0) + ws.qn;
    if (a.a_mn && c2 >= a.num_taps) {  // packed taps, odd count: the last tile's second half has no tap
    } else if (a.reduce_add) tma_reduce_add_4d(&a.out_map, ws.buf_addr + slot * 4096u, col, t.w0 + ws.qw, c2, c3);
    else tma_store_4d(&a.out_map, ws.buf_addr + slot * 4096u, col, t.w0 + ws.qw, c2, c3);
    bulk_commit_group();
  }
}

template <typename OutT>
__device__ __forceinline__ void epilogue_tile_tma(const GemmArgs& a, const TileCoord& t, uint32_t tmem_acc, int lane,
                                                  bool zero, const WarpStore& ws, uint32_t& store_count) {
  constexpr int CPB = 128 / sizeof(OutT);  // columns per block
  constexpr int P = 16 / sizeof(OutT);     // columns per 16-byte chunk
  const OutT* bias = static_cast<const OutT*>(a.bias);
  for (int c0 = 0; c0 < a.bn; c0 += CPB, ++store_count) {
    const uint32_t slot = store_count & (uint32_t)(ws.nsw - 1);
    wait_slice_free(ws, lane);
    uint8_t* row_ptr = ws.buf + slot * 4096u + (size_t)lane * 128;
#pragma unroll
    for (int half = 0; half < CPB / 32; ++half) {
      uint32_t acc[32];
      if (!zero) {
        tmem_ld_32x32(tmem_acc + (uint32_t)(c0 + half * 32), acc);
        tmem_wait_ld();
      }
      const int colbase = t.nf0 + c0 + half * 32;
#pragma unroll
      for (int g = 0; g < 32 / P; ++g) {
        float v[P];
#pragma unroll
        for (int i = 0; i < P; ++i) v[i] = zero ? 0.f : a.alpha * __uint_as_float(acc[g * P + i]);
        if (bias != nullptr) {
#pragma unroll
          for (int i = 0; i < P; ++i) {
            const int c = colbase + g * P + i;
            if (c < a.ext_cols) v[i] += to_f32(__ldg(bias + c));
          }
        }
        if (a.act != PDNN_ACT_NONE) {
#pragma unroll
          for (int i = 0; i < P; ++i) v[i] = apply_activation(v[i], a.act);
        }
        Vec16<OutT> pk;
#pragma unroll
        for (int i = 0; i < P; ++i) pk.set(i, from_f32<OutT>(v[i]));
        const int chunk = half * (32 / P) + g;  // 0..7 within the 128-byte row
        *reinterpret_cast<uint4*>(row_ptr + ((chunk ^ (lane & 7)) << 4)) = pk.raw;
      }
    }
    issue_slice_store(a, t, ws, slot, t.nf0 + c0, lane);
  }
}

// Packed-pair arithmetic for the 16-bit fast epilogue.
template <typename OutT>
struct Pair;
template <>
struct Pair<__half> {
  using type = __half2;
  static __device__ __forceinline__ type pack(float a, float b) { return __floats2half2_rn(a, b); }
  static __device__ __forceinline__ type splat(float v) { return __float2half2_rn(v); }
};
template <>
struct Pair<__nv_bfloat16> {
  using type = __nv_bfloat162;
  static __device__ __forceinline__ type pack(float a, float b) { return __floats2bfloat162_rn(a, b); }
  static __device__ __forceinline__ type splat(float v) { return __float2bfloat162_rn(v); }
};

template <typename P2>
__device__ __forceinline__ uint32_t pair_bits(P2 v) {
  return *reinterpret_cast<uint32_t*>(&v);
}
template <typename P2>
__device__ __forceinline__ P2 bits_pair(uint32_t v) {
  return *reinterpret_cast<P2*>(&v);
}

// Shared-memory load of 16 bytes.  Volatile so that it is issued where it is written: the bias
// loads of a column block are batched ahead of the wait for the accumulators, and their latencies
// overlap instead of each load sitting directly in front of its first use (a lone warp stalls on
// every one of them: eight round trips cost more than the arithmetic of the block).
__device__ __forceinline__ uint4 ld_global_v4(const void* ptr) {
  uint4 v;
  asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr));
  return v;
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// Converts 32 accumulator columns of one row (four 16-byte chunks, numbered from chunk_base) and
// writes them into the row's 128 bytes of the staging slice.  `bv` holds the bias of those 32
// columns (zeros without a bias), `mk` (MASK only) the keep masks of those columns.
template <typename OutT, bool MASK, bool BITS = false>
__device__ __forceinline__ uint32_t fast_convert_store(const uint32_t (&acc)[32], bool zero, bool has_bias, const uint4* bv,
                                                       int act, uint8_t* row_ptr, int row, int chunk_base, const uint4* mk) {
  constexpr bool want_bits = BITS && !MASK;
  using P2 = typename Pair<OutT>::type;
  const P2 zero2 = Pair<OutT>::splat(0.f), six2 = Pair<OutT>::splat(6.f);
  uint32_t bits = 0u;  // want_bits: bit c = column c of these 32 is positive (a positive 16-bit float is a positive integer)
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    const uint32_t bw[4] = {bv[g].x, bv[g].y, bv[g].z, bv[g].w};
    uint32_t o[4];
    [[maybe_unused]] uint32_t pos[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      P2 v = zero ? zero2
                  : Pair<OutT>::pack(__uint_as_float(acc[g * 8 + 2 * i]), __uint_as_float(acc[g * 8 + 2 * i + 1]));
      if (has_bias) v = __hadd2(v, bits_pair<P2>(bw[i]));  // the bias, or what the output held before
      if (!MASK) {  // the gradient form has no activation
        if (act != PDNN_ACT_NONE) v = __hmax2(v, zero2);
        if (act == PDNN_ACT_RELU6) v = __hmin2(v, six2);
      }
      o[i] = pair_bits(v);
      if constexpr (want_bits) pos[i] = __hgt2_mask(v, zero2);  // 0xFFFF per positive half
    }
    if constexpr (want_bits) {
      // one distinct bit per element, then the two halves folded: elements 2i (low halves) and 2i + 1
      const uint32_t c = (pos[0] & 0x00020001u) | (pos[1] & 0x00080004u) | (pos[2] & 0x00200010u) | (pos[3] & 0x00800040u);
      bits |= ((c | (c >> 16)) & 0xFFu) << (g * 8);
    }
    if (MASK) {  // mk: 0xFFFF in every halfword whose mask element is positive
      o[0] &= mk[g].x;
      o[1] &= mk[g].y;
      o[2] &= mk[g].z;
      o[3] &= mk[g].w;
    }
    *reinterpret_cast<uint4*>(row_ptr + (((chunk_base + g) ^ (row & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
  }
  return bits;
}

// Element offset of the lane's row of the tile in the output tensor (row = q32 + lane), or -1 if the row
// lies outside the tensor.
__device__ __forceinline__ long long row_element_offset(const GemmArgs& a, const TileCoord& t, int q32, int lane) {
  const int sh_w = __ffs(a.etw) - 1, sh_h = __ffs(a.eth) - 1, row = q32 + lane;
  const int w = t.w0 + (row & (a.etw - 1)), h = t.h0 + ((row >> sh_w) & (a.eth - 1)), n = t.n0 + (row >> (sh_w + sh_h));
  if (!(w < a.ext_w && h < a.ext_h && n < a.ext_n)) return -1;
  return (long long)n * a.stride_n + (long long)h * a.stride_h + (long long)w * a.stride_w;
}

// 64 mask bits of a row -> keep masks of the eight 16-byte chunks (0xFFFF per kept halfword).
__device__ __forceinline__ void expand_mask_bits(uint2 bits, uint4 (&mk)[8]) {
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    const uint32_t b = ((g < 4 ? bits.x : bits.y) >> (8 * (g & 3))) & 0xFFu;
    uint32_t m[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      // a one-bit field read as a signed number is 0 or all ones
      const int lo = ((int)(b << (31 - 2 * i))) >> 31, hi = ((int)(b << (30 - 2 * i))) >> 31;
      m[i] = __byte_perm((uint32_t)lo, (uint32_t)hi, 0x5410);
    }
    mk[g] = make_uint4(m[0], m[1], m[2], m[3]);
  }
}

// The ReLU mask of a 32-row x 64-column block (16-bit elements) comes into the warp's mask slot in
// shared memory by TMA, through a tensor map with the geometry and swizzle of the output map, so a
// lane finds its row's 128 bytes where it will put its own results in the staging slice.  A positive
// 16-bit float is a positive 16-bit integer, so "mask > 0" is one packed integer compare per pair
// (NaNs do not occur in a ReLU output).  Requests run one or two blocks ahead of the block being
// worked on (as many as the warp has slots), across tile boundaries: a slot is requested again as
// soon as its words have been taken out.
struct MaskSlot {
  uint32_t addr;       // shared-memory address of the warp's first 4 KB slot
  uint32_t bar;        // mbarrier of the first slot (one per slot, 8 bytes apart)
  uint32_t nslots;     // 1 or 2: how many blocks ahead the requests run
  uint32_t issued, consumed;
  // the block the next request is for: the warp's blocks in the order it will work on them
  TileWalker walker;
  int tile, c0, tile_step, total_tiles, sub_w, sub_h, sub_n;
};

// Requests the mask of the next block that has none yet (if any is left).
__device__ __forceinline__ void request_mask_block(const GemmArgs& a, const WarpStore& ws, MaskSlot& ms) {
  if (ms.tile >= ms.total_tiles) return;
  const TileCoord t = ms.walker.coord(a);
  const uint32_t slot = ms.issued % ms.nslots;
  if (elect_one()) {
    mbar_arrive_expect_tx(ms.bar + 8u * slot, 4096u);
    tma_load_4d(ms.addr + slot * 4096u, &a.mask_map, ms.bar + 8u * slot, t.nf0 + ms.c0, t.w0 + ms.sub_w + ws.qw,
                t.h0 + ms.sub_h + ws.qh, t.n0 + ms.sub_n + ws.qn);
  }
  ++ms.issued;
  ms.c0 += 64;
  if (ms.c0 >= a.bn) {
    ms.c0 = 0;
    ms.tile += ms.tile_step;
    ms.walker.advance();
  }
}

// The common case of the staged epilogue, kept short because a lone warp per scheduler is
// latency-bound: 16-bit output, alpha == 1, optional bias, activation none / ReLU / ReLU6.  The
// accumulators are rounded to the output type first and bias and activation are applied to
// packed pairs in that type - the arithmetic of separate convolution, bias-add and activation
// passes.  MASK: the result is additionally zeroed wherever a.relu_mask is not positive.  BITS: the
// sign bits of the result are written to a.bitmask_out.  (Both are compile-time forms: as run-time
// branches of one instantiation they cost the plain forward epilogue 7 % of the ResNet-50 step.)
template <typename OutT, bool MASK, bool BITS = false, bool MBITS = false>
__device__ __forceinline__ bool epilogue_tile_tma_fast(const GemmArgs& a, const TileCoord& t, uint32_t tmem_acc,
                                                       int lane, bool zero, const WarpStore& ws,
                                                       uint32_t& store_count, uint32_t bias_s, int q32, MaskSlot& ms,
                                                       volatile int* abort_flag) {
  const int act = a.act;
  static_assert(!(MASK && BITS) && (MASK || !MBITS), "one form per instantiation");
  constexpr bool bit_mask = MBITS;  // the mask arrives as one bit per element (a.mask_bits), not as a tensor
  constexpr bool emit_bits = BITS;
  long long row_off = -1;
  if constexpr (MASK || BITS) {
    if (a.accumulate != 0 || bit_mask || emit_bits) row_off = row_element_offset(a, t, q32, lane);
  }
  // mask bits of the lane's row for every 64-column block of the tile, requested up front
  [[maybe_unused]] uint2 pre[MBITS ? 4 : 1];
  if constexpr (MBITS) {
#pragma unroll
    for (int b = 0; b < 4; ++b) pre[b] = make_uint2(0u, 0u);
    if (row_off >= 0) {
#pragma unroll
      for (int b = 0; b < 4; ++b)
        if (b * 64 < a.bn && t.nf0 + b * 64 < a.ext_cols)
          pre[b] = __ldg(reinterpret_cast<const uint2*>(static_cast<const uint8_t*>(a.mask_bits) + ((row_off + t.nf0 + b * 64) >> 3)));
    }
  }
#pragma unroll 1
  for (int c0 = 0; c0 < a.bn; c0 += 64, ++store_count) {
    const uint32_t slot = store_count & (uint32_t)(ws.nsw - 1);
    uint32_t acc0[32], acc1[32];
    if (!zero) {  // issued before waiting for the staging slice
      tmem_ld_32x32(tmem_acc + (uint32_t)c0, acc0);
      tmem_ld_32x32(tmem_acc + (uint32_t)(c0 + 32), acc1);
    }
    // the block's bias, all eight loads in flight at once (and before the waits below)
    uint4 bv[8];
    const bool add_prev = a.accumulate != 0, has_bias = add_prev || (!MASK && bias_s != 0u);
    if (add_prev) {
      // accumulating form: the lane's own row of the block that is in the output already (128 bytes)
      const long long off = (MASK || BITS) ? row_off : row_element_offset(a, t, q32, lane);
      const uint16_t* prev = off >= 0 ? static_cast<const uint16_t*>(a.out) + off + t.nf0 + c0 : nullptr;
#pragma unroll
      for (int g = 0; g < 8; ++g)
        bv[g] = (prev != nullptr && t.nf0 + c0 + g * 8 < a.ext_cols) ? ld_global_v4(prev + g * 8) : make_uint4(0u, 0u, 0u, 0u);
    } else {
#pragma unroll
      for (int g = 0; g < 8; ++g)
        bv[g] = has_bias ? ld_shared_v4(bias_s + (uint32_t)(t.nf0 + c0 + g * 8) * 2u) : make_uint4(0u, 0u, 0u, 0u);
    }
    uint4 mk[MASK ? 8 : 1];
    if constexpr (MASK) {
     if constexpr (MBITS) {
      const int blk = c0 >> 6;
      expand_mask_bits(blk == 0 ? pre[0] : blk == 1 ? pre[1] : blk == 2 ? pre[2] : pre[3], mk);
     } else {
      // this block's mask was requested earlier: take the lane's row out of the slot as keep masks,
      // then let the next request reuse the slot
      const uint32_t mslot = ms.consumed % ms.nslots;
      if (!mbar_wait(ms.bar + 8u * mslot, (ms.consumed / ms.nslots) & 1u, abort_flag, g_error_record, a.wait_limit_ns, 0x700u))
        return false;
      const uint32_t row_addr = ms.addr + mslot * 4096u + (uint32_t)lane * 128u;
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        const uint4 m = ld_shared_v4(row_addr + (uint32_t)((g ^ (lane & 7)) << 4));
        using P2 = typename Pair<OutT>::type;
        const P2 zero2 = Pair<OutT>::splat(0.f);
        mk[g] = make_uint4(__hgt2_mask(bits_pair<P2>(m.x), zero2), __hgt2_mask(bits_pair<P2>(m.y), zero2),
                           __hgt2_mask(bits_pair<P2>(m.z), zero2), __hgt2_mask(bits_pair<P2>(m.w), zero2));
      }
      __syncwarp();  // every lane holds its masks: the slot may be overwritten
      ++ms.consumed;
      request_mask_block(a, ws, ms);
     }
    }
    wait_slice_free(ws, lane);
    if (!zero) tmem_wait_ld();
    uint8_t* row_ptr = ws.buf + slot * 4096u + (size_t)lane * 128;
    const uint32_t lo_bits = fast_convert_store<OutT, MASK, BITS>(acc0, zero, has_bias, bv, act, row_ptr, lane, 0, mk);
    const uint32_t hi_bits = fast_convert_store<OutT, MASK, BITS>(acc1, zero, has_bias, bv + 4, act, row_ptr, lane, 4, MASK ? mk + 4 : mk);
    if constexpr (emit_bits) {
      if (row_off >= 0 && t.nf0 + c0 < a.ext_cols)
        *reinterpret_cast<uint2*>(static_cast<uint8_t*>(a.bitmask_out) + ((row_off + t.nf0 + c0) >> 3)) = make_uint2(lo_bits, hi_bits);
    }
    issue_slice_store(a, t, ws, slot, t.nf0 + c0, lane);
  }
  return true;
}

// EPI selects the epilogue compiled into the instantiation: 0 = direct stores from registers,
// 1 = staged TMA store with fp32 arithmetic, 2 = staged TMA store with packed 16-bit arithmetic,
// 3 = as 2 with the ReLU-gradient mask (GemmArgs::relu_mask), 4 = as 2 writing the sign bits of the
// result (GemmArgs::bitmask_out), 5 = as 3 with the mask as one bit per element (GemmArgs::mask_bits).
// One epilogue per instantiation keeps each kernel's register allocation tight.
//
// A CTA runs up to two independent pipelines ("groups") side by side, each with its own TMA
// producer warp, MMA issuer warp, four epilogue warps, ring of stages, accumulators in TMEM and
// staging slices; group g takes every second tile of the CTA.  One thread can issue a
// tcgen05.mma only every ~130 cycles once the barrier wait, the commit and the loop around four
// MMAs are counted, which is two to three times the time the tensor pipe needs for a 128 x 64 or
// 128 x 128 MMA; two issuers keep the pipe busy, and two epilogue teams halve the time a tile's
// accumulator waits to be drained.  The resident B tiles, the bias copy and the TMEM allocation
// are shared.  The fp32 (3xTF32) variant runs one group plus the four hi/lo split warps.
//
// The role loops carry `#pragma unroll 1`: left alone the compiler unrolls them fourfold, the
// kernel grows from 59 to 80 KB, and the instruction-cache hit rate drops (92% measured on the
// stem layer); the single-thread roles then stall several hundred cycles at loop back-edges.  The
// compact kernel is about 1% faster over the ResNet-50 stack.
//
//   warp 6g + 0      producer of group g
//   warp 6g + 1      MMA issuer of group g (warp 1 also owns the TMEM allocation)
//   warps 6g + 2..5  epilogue of group g (warp % 4 selects the TMEM lane quarter)
//   SPLIT: warps 6..9 are the hi/lo split warps of the only group
// The body of the kernel for CTA `cta` of `n_ctas` that work on the GEMM `a` (the whole grid, or the share
// of it that umma_gemm_multi_kernel gives to one of its GEMMs).
template <bool SPLIT, int EPI, typename OutT>
__device__ __forceinline__ void umma_gemm_body(const GemmArgs& a, const int cta, const int n_ctas) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;  // swizzled tiles need 1024-byte alignment
  uint8_t* smem = smem_raw + (base - raw_addr);

  constexpr int kMaxGroups = SPLIT ? 1 : 2;
  const int groups = SPLIT ? 1 : a.groups;
  // The warp index is broadcast from lane 0 so that the compiler can prove it, and everything derived
  // from it (group, role, ring addresses, descriptor words), uniform across the warp: tcgen05.mma and
  // the TMA copies take their operands from uniform registers, and values it cannot prove uniform
  // cost a register-file round trip per operand per instruction on the one thread everything waits
  // for.
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  const int grp = SPLIT ? 0 : warp / 6;
  const int role = SPLIT ? warp : warp - grp * 6;  // 0 producer, 1 issuer, 2..5 epilogue, 6..9 split (SPLIT)

  const uint32_t b_bytes = a.b_step_bytes;
  const uint32_t part_bytes = kABytes + b_bytes;              // one A tile + one B tile
  const bool b_res = !SPLIT && a.b_res != 0;
  const uint32_t res_bytes = b_res ? a.b_res_bytes : 0u;      // resident B tiles come first
  const bool halo = !SPLIT && a.halo != 0;
  const bool pair = !SPLIT && a.pair != 0;
  const uint32_t stage_bytes = SPLIT  ? 2u * part_bytes
                               : pair ? part_bytes + (uint32_t)kABytes
                               : halo ? a.halo_stage_bytes
                                      : (b_res ? (uint32_t)kABytes : part_bytes);
  const int S = a.stages;                                     // stages per group
  const uint32_t ring_bytes = (uint32_t)S * stage_bytes;
  const int rings = pair ? 1 : groups;                        // pair mode: one ring for both groups
  const uint32_t ring_base = base + res_bytes + (pair ? 0u : (uint32_t)grp * ring_bytes);  // this group's ring
  uint8_t* ring_mem = smem + res_bytes + (pair ? 0u : (size_t)grp * ring_bytes);
  // staging slices for the TMA-store epilogue (per group: 4 warps x nsw slices), then the barrier
  // block, then the bias copy
  const uint32_t group_staging = a.tma_store ? ((uint32_t)a.nsw + (EPI == 3 ? (uint32_t)a.mask_slots : 0u)) * 4u * 4096u : 0u;
  const uint32_t staging_off = res_bytes + (uint32_t)rings * ring_bytes;
  const uint32_t bar_off = staging_off + (uint32_t)groups * group_staging;
  uint8_t* bar_mem = smem + bar_off;
  const uint32_t bar_base = base + bar_off;
  auto gbar = [&](int g, int i) { return bar_base + 8u * (uint32_t)(g * kBarsPerGroup + i); };
  const int ring_grp = pair ? 0 : grp;  // whose stage barriers this warp uses
  auto full_bar = [&](int s) { return gbar(ring_grp, s); };
  auto empty_bar = [&](int s) { return gbar(ring_grp, kMaxStages + s); };
  auto ready_bar = [&](int s) { return gbar(grp, 2 * kMaxStages + s); };
  auto acc_full_bar = [&](int b) { return gbar(grp, 3 * kMaxStages + b); };
  auto acc_empty_bar = [&](int b) { return gbar(grp, 3 * kMaxStages + 2 + b); };
  const uint32_t bres_bar = bar_base + 8u * (uint32_t)(2 * kBarsPerGroup);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_mem + 8 * (2 * kBarsPerGroup + 1));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_mem + 8 * (2 * kBarsPerGroup + 1) + 4);
  // with bias_tile_only the copy starts at the CTA's column tile; the address is biased so that
  // indexing by absolute column still works
  const int bias_col0 = a.bias_tile_only ? (cta % a.n_tiles) * a.bn : 0;
  const uint32_t bias_s =
      (EPI >= 2 && a.bias != nullptr) ? bar_base + kBarBlockBytes - (uint32_t)bias_col0 * 2u : 0u;

  // One barrier per thread (a single thread initialising all of them costs about a microsecond of
  // every launch): full, empty and ready per stage, accumulator full / empty per buffer, per group.
  if ((int)threadIdx.x < kMaxGroups * kBarsPerGroup) {
    const int g = (int)threadIdx.x / kBarsPerGroup, j = (int)threadIdx.x % kBarsPerGroup;
    const uint32_t count = j < kMaxStages                ? 1u
                           : j < 2 * kMaxStages          ? (pair ? 2u : 1u)  // pair mode: both issuers release a stage
                           : j < 3 * kMaxStages          ? 4u
                           : j < 3 * kMaxStages + 2      ? 1u
                                                         : 4u;
    mbar_init(gbar(g, j), count);
    fence_barrier_init();
  } else if ((int)threadIdx.x == kMaxGroups * kBarsPerGroup) {
    mbar_init(bres_bar, 1);
    *abort_flag = 0;
    fence_barrier_init();
  } else if (EPI == 3 && (int)threadIdx.x < kMaxGroups * kBarsPerGroup + 17) {
    // one barrier per mask slot of the epilogue warps, after the bias copy
    const int i = (int)threadIdx.x - kMaxGroups * kBarsPerGroup - 1;
    mbar_init(bar_base + (uint32_t)kBarBlockBytes + (uint32_t)a.bias_smem_bytes + 8u * (uint32_t)i, 1);
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), (uint32_t)a.tmem_cols);
    tmem_relinquish();
  }
  // Under programmatic dependent launch everything above overlaps the tail of the previous kernel
  // in the stream; nothing before this point reads or writes global memory.  From here on the
  // kernel touches tensors that kernel may have written (or may still be reading), so it waits
  // for it.  The next kernel may be scheduled as soon as SMs free up: this grid is a single wave,
  // so nothing of it is still waiting for an SM.
  const int total_tiles = a.a_mn ? a.n_tiles * a.tiles_w * ((a.num_taps + a.tap_pack - 1) / a.tap_pack) * a.splits
                                 : a.n_tiles * a.tiles_w * a.tiles_h * a.tiles_n;
  // one B tile of a forward-style GEMM (a_mn == 0): reduction block kc of tap btap, columns from nf0
  auto load_b_from = [&](const CUtensorMap* bmap, uint32_t sb, uint32_t fb, int kc, int nf0, int btap) {
    const int epr = a.epr;
    switch (a.b_mode) {
      case B_MN_3X: warp_tma_load_4d(sb, bmap, fb, 0, kc, nf0 / epr, btap); break;
      case B_MN_3:
#pragma unroll 1
        for (int j = 0; j < a.b_boxes; ++j)
          warp_tma_load_4d(sb + (uint32_t)j * a.b_box_bytes, bmap, fb, nf0 + j * epr, kc, btap, 0);
        break;
      case B_K_3: warp_tma_load_4d(sb, bmap, fb, kc, nf0, btap, 0); break;
      case B_K_FHWC: warp_tma_load_4d(sb, bmap, fb, kc, btap, nf0, 0); break;
      default:  // B_MN_FHWC
#pragma unroll 1
        for (int j = 0; j < a.b_boxes; ++j)
          warp_tma_load_4d(sb + (uint32_t)j * a.b_box_bytes, bmap, fb, nf0 + j * epr, btap, kc, 0);
        break;
    }
  };
  // the whole B operand of the CTA's column tiles into the resident area (called by one warp)
  auto load_resident_b = [&] {
    warp_arrive_expect_tx(bres_bar, res_bytes);
    uint32_t dst = base;
    const int nt_begin = a.b_res == 2 ? cta % a.n_tiles : 0;
    const int nt_end = a.b_res == 2 ? nt_begin + 1 : a.n_tiles;
#pragma unroll 1
    for (int nt = nt_begin; nt < nt_end; ++nt)
#pragma unroll 1
      for (int tap = 0; tap < a.num_taps; ++tap) {
        const TapEntry e = a.taps[tap];
        const int cnt = halo ? e.cnt : 1;
#pragma unroll 1
        for (int g = 0; g < cnt; ++g)
#pragma unroll 1
          for (int cb = 0, kc = 0; cb < a.cblocks; ++cb, kc += a.epr, dst += b_bytes)
            load_b_from(&a.b_map, dst, bres_bar, kc, nt * a.bn, e.b_tap + g * e.b_step);
      }
  };
  auto copy_bias = [&] {
    if (EPI >= 2 && a.bias != nullptr) {
      // the CTA's copy of the bias vector, zero beyond the last column
      const OutT* bias = static_cast<const OutT*>(a.bias);
      uint4* dst = reinterpret_cast<uint4*>(bar_mem + kBarBlockBytes);
      const int chunks = a.bias_smem_bytes >> 4;
      for (int i = threadIdx.x; i < chunks; i += blockDim.x) {
        const int col = bias_col0 + i * 8;
        dst[i] = (col + 8 <= a.ext_cols) ? __ldg(reinterpret_cast<const uint4*>(bias + col)) : make_uint4(0u, 0u, 0u, 0u);
      }
    }
  };
  const bool early_b = !SPLIT && a.early_b != 0;
  if (early_b) {
    __syncthreads();  // the barrier of the resident copy is initialised
    if (warp == 0 && b_res && cta < total_tiles) load_resident_b();
    copy_bias();
  }
  grid_dependency_wait();
  grid_launch_dependents();
  if (!early_b) copy_bias();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // accumulator buffer b of group g starts at column (g * acc_bufs + b) * acc_stride
  const uint32_t acc_bufs = (uint32_t)a.acc_bufs, acc_stride = (uint32_t)a.acc_stride;
  const uint32_t grp_tmem = tmem_base + (uint32_t)grp * acc_bufs * acc_stride;

  // pair mode: both groups walk the same tiles (each takes one row tile of the pair)
  const int first_tile = cta + (pair ? 0 : grp * n_ctas);
  const int tile_step = (pair ? 1 : groups) * n_ctas;
  const bool active = grp < groups;
  // offset of this group's row tile inside the pair
  const int sub_w = pair && a.pair_dim == 1 ? grp * a.tw : 0, sub_h = pair && a.pair_dim == 2 ? grp * a.th : 0,
            sub_n = pair && a.pair_dim == 3 ? grp * a.tn : 0;

  if (!active) {
    // a group that is switched off has nothing to do
  } else if (role == 0) {
    // ------------------------------- TMA producer ------------------------------------------
    // One thread; the loop body is kept to a wait, an expect_tx and the copies, with all
    // coordinates advanced incrementally: a lone thread issues an instruction every few cycles
    // at best, so every division or table lookup per step would show up as pipeline bubbles.
    // The whole warp walks the tiles and waits on the barriers (every value stays warp-uniform); the
    // warp_* wrappers elect the one lane that issues each copy.
    if (!(pair && grp != 0)) {  // pair mode: group 0's producer fills the shared ring
      if (lane == 0) {
        for (int i = 0; i < 4; ++i) prefetch_tensormap(&a.a_map[i]);
        prefetch_tensormap(&a.b_map);
      }
      const int epr = a.epr, b_mode = a.b_mode, b_boxes = a.b_boxes, a_boxes = a.a_boxes, cblocks = a.cblocks;
      const bool presplit = SPLIT && a.b_presplit != 0;
      const uint32_t a_box_bytes = a.a_box_bytes, b_box_bytes = a.b_box_bytes,
                     tx_bytes = pair ? 2u * kABytes + b_bytes
                                     : (b_res ? (uint32_t)kABytes : kABytes + (presplit ? 2u * b_bytes : b_bytes));
      // pair mode: where the second row tile of the pair starts, relative to the first
      const int pair_dw = a.pair_dim == 1 ? a.tw : 0, pair_dh = a.pair_dim == 2 ? a.th : 0,
                pair_dn = a.pair_dim == 3 ? a.tn : 0;
      const CUtensorMap* bmap = &a.b_map;
      auto load_b = [&](uint32_t sb, uint32_t fb, int kc, int nf0, int btap) { load_b_from(bmap, sb, fb, kc, nf0, btap); };
      if (b_res && !early_b && grp == 0 && cta < total_tiles) load_resident_b();
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      auto next_stage = [&] {
        if (++s == S) {
          s = 0;
          ph ^= 1u;
        }
      };
      TileWalker walker;
      walker.init(a, first_tile, tile_step);
#pragma unroll 1
      for (int tile = first_tile; tile < total_tiles && ok; tile += tile_step, walker.advance()) {
        const TileCoord t = walker.coord(a);
        if (!a.a_mn) {
#pragma unroll 1
          for (int tap = 0; tap < a.num_taps && ok; ++tap) {
            const TapEntry e = a.taps[tap];
            const CUtensorMap* amap = &a.a_map[e.a_map];
            const int aw = t.w0 + e.dw, ah = t.h0 + e.dh;
            const int btap = e.b_tap + t.n0 * a.b_batch_mul;
            const uint32_t tx = halo ? (uint32_t)(a.th + e.cnt - 1) * (uint32_t)(a.tw * a.a_row_bytes) : tx_bytes;
#pragma unroll 1
            for (int cb = 0, kc = 0; cb < cblocks; ++cb, kc += epr) {
              if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, g_error_record, a.wait_limit_ns, 0x100u + (unsigned)s)) {
                ok = false;
                break;
              }
              {
                const uint32_t fb = full_bar(s);
                warp_arrive_expect_tx(fb, tx);
                const uint32_t sa = ring_base + (uint32_t)s * stage_bytes;
                warp_tma_load_4d(sa, amap, fb, kc, aw, ah, t.n0);
                if (pair) {
                  warp_tma_load_4d(sa + kABytes, amap, fb, kc, aw + pair_dw, ah + pair_dh, t.n0 + pair_dn);
                  load_b(sa + 2u * kABytes, fb, kc, t.nf0, btap);
                } else if (!b_res) {
                  load_b(sa + kABytes, fb, kc, t.nf0, btap);
                  if (presplit) load_b_from(&a.b_map_lo, sa + part_bytes + kABytes, fb, kc, t.nf0, btap);
                }
              }
              next_stage();
            }
          }
        } else {
          const TapEntry e = a.taps[t.tap];
          const CUtensorMap* amap = &a.a_map[e.a_map];
          // packed taps: the second box holds the same channels as seen by the next tap (none: a box
          // beyond the last channel, which TMA fills with zeros)
          const bool packed = a.tap_pack > 1, second = packed && t.tap + 1 < a.num_taps;
          const TapEntry e2 = a.taps[second ? t.tap + 1 : t.tap];
          const CUtensorMap* amap2 = &a.a_map[e2.a_map];
          const int c2nd = second ? t.w0 : 0x40000000;
          const int batch = a.split_is_batch ? t.split : 0;
          // slab coordinates of ks_begin, then advanced like an odometer
          int iw = t.ks_begin % a.slabs_w, ih = (t.ks_begin / a.slabs_w) % a.slabs_h,
              in = t.ks_begin / (a.slabs_w * a.slabs_h);
#pragma unroll 1
          for (int ks = t.ks_begin; ks < t.ks_end; ++ks) {
            if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, g_error_record, a.wait_limit_ns, 0x100u + (unsigned)s)) {
              ok = false;
              break;
            }
            {
              const uint32_t fb = full_bar(s);
              warp_arrive_expect_tx(fb, tx_bytes);
              const uint32_t sa = ring_base + (uint32_t)s * stage_bytes;
              const uint32_t sb = sa + kABytes;
              const int kw = iw * a.tw, kh = ih * a.th, kn = in * a.tn + batch;
              if (packed) {
                warp_tma_load_4d(sa, amap, fb, t.w0, kw + e.dw, kh + e.dh, kn);
                warp_tma_load_4d(sa + a_box_bytes, amap2, fb, c2nd, kw + e2.dw, kh + e2.dh, kn);
              } else {
#pragma unroll 1
                for (int j = 0; j < a_boxes; ++j)
                  warp_tma_load_4d(sa + (uint32_t)j * a_box_bytes, amap, fb, t.w0 + j * epr, kw + e.dw, kh + e.dh, kn);
              }
              if (b_mode == B_MN_4) {
#pragma unroll 1
                for (int j = 0; j < b_boxes; ++j)
                  warp_tma_load_4d(sb + (uint32_t)j * b_box_bytes, bmap, fb, t.nf0 + j * epr, kw, kh, kn);
              } else {  // B_K_4
                warp_tma_load_4d(sb, bmap, fb, kw, t.nf0, 0, kn);
              }
            }
            if (++iw == a.slabs_w) {
              iw = 0;
              if (++ih == a.slabs_h) {
                ih = 0;
                ++in;
              }
            }
            next_stage();
          }
        }
      }
    }
  } else if (role == 1) {
    // ------------------------------- MMA issuer ---------------------------------------------
    {
      // The whole warp runs the loops on warp-uniform values; warp_mma_* / warp_commit elect the one
      // lane that issues each instruction.
      // Descriptor words that do not change: everything but the 14-bit start address.
      const uint64_t a_desc0 = make_smem_desc(0, a.a_lbo, a.a_sbo, a.a_layout);
      const uint64_t b_desc0 = make_smem_desc(0, a.b_lbo, a.b_sbo, a.b_layout);
      const uint32_t a_kadv = a.a_kadv >> 4, b_kadv = a.b_kadv >> 4, idesc = a.idesc;
      const uint32_t lo_off = part_bytes >> 4;
      int s = 0;
      uint32_t ph = 0;
      uint32_t buf = 0, aph = 0;  // accumulator buffer of this tile and the parity of its barriers
      bool ok = true;
      if (b_res && first_tile < total_tiles) ok = mbar_wait(bres_bar, 0u, abort_flag, g_error_record, a.wait_limit_ns, 0x600u);
      // Loop constants of the forward-style main loop, all in units of 16 bytes (the unit of a
      // descriptor's address field).
      struct {
        uint32_t a_lo0, a_hi, b_lo0, b_hi;  // descriptor words without a start address
        uint32_t ring16, stage16;           // this group's ring and the size of a stage
        uint32_t my_a16, my_b16;            // this group's A tile and the B tile inside a stage
        uint32_t halo_row16;                // halo mode: one tile row further down
        uint32_t b_tap16, b_bytes16;        // resident B: next tap of the entry, next reduction block
        uint32_t res16_base, res_tile16;    // resident B: first tile, tiles of one column tile
        uint32_t cnts;                      // taps per entry, 4 bits each (1 outside halo mode)
        int num_taps, cblocks;
        bool four;
      } fw;
      fw.a_lo0 = (uint32_t)a_desc0;
      fw.a_hi = (uint32_t)(a_desc0 >> 32);
      fw.b_lo0 = (uint32_t)b_desc0;
      fw.b_hi = (uint32_t)(b_desc0 >> 32);
      fw.ring16 = ring_base >> 4;
      fw.stage16 = stage_bytes >> 4;
      fw.my_a16 = pair ? ((uint32_t)grp * kABytes) >> 4 : 0u;
      fw.my_b16 = (pair ? 2u * kABytes : (uint32_t)kABytes) >> 4;
      fw.halo_row16 = (uint32_t)(a.tw * a.a_row_bytes) >> 4;
      fw.b_bytes16 = b_bytes >> 4;
      fw.b_tap16 = (uint32_t)a.cblocks * (b_bytes >> 4);
      fw.res16_base = base >> 4;
      fw.res_tile16 = (uint32_t)(a.res_taps * a.cblocks) * (b_bytes >> 4);
      fw.num_taps = a.num_taps;
      fw.cblocks = a.cblocks;
      fw.four = a.kmmas == 4;
      fw.cnts = 0u;  // halo mode has at most 8 entries of at most 15 taps (checked by the host)
      if (halo)
        for (int i = 0; i < a.num_taps && i < 8; ++i) fw.cnts |= (uint32_t)(a.taps[i].cnt & 15) << (4 * i);
      uint32_t sa16 = fw.ring16;  // start of the current stage
      TileWalker walker;
      walker.init(a, first_tile, tile_step);
#pragma unroll 1
      for (int tile = first_tile; tile < total_tiles && ok; tile += tile_step, walker.advance()) {
        const TileCoord t = walker.coord(a);
        if (!mbar_wait(acc_empty_bar((int)buf), aph ^ 1u, abort_flag, g_error_record, a.wait_limit_ns, 0x200u + buf)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = grp_tmem + buf * acc_stride;
        uint32_t accumulate = 0u;
        if (!SPLIT && !a.a_mn) {
          // Forward-style GEMM: one stage per (tap entry, reduction block); in halo mode a stage
          // feeds the MMAs of all cnt taps of its entry.  Everything in this loop is kept to
          // 32-bit additions on values prepared outside it: the lone issuing thread is what bounds
          // tiles of 64 or 128 columns, and it needs the tile's nt only (the walker's digit 0).
          uint32_t res16 = fw.res16_base + (a.b_res == 1 ? (uint32_t)walker.d0 * fw.res_tile16 : 0u);
#pragma unroll 1
          for (int tap = 0; tap < fw.num_taps && ok; ++tap) {
            const int cnt = halo ? (int)((fw.cnts >> (4 * tap)) & 15u) : 1;
#pragma unroll 1
            for (int cb = 0; cb < fw.cblocks; ++cb) {
              if (!mbar_wait(full_bar(s), ph, abort_flag, g_error_record, a.wait_limit_ns, 0x300u + (unsigned)s)) {
                ok = false;
                break;
              }
              // no tcgen05 fence here: the stage was written by TMA and is read by the MMA, both in
              // the async proxy, and the mbarrier's complete_tx orders them
              // start addresses stay below 2^18, so adding to the low descriptor word never carries
              // into the neighbouring field
              uint32_t a_lo = fw.a_lo0 + sa16 + fw.my_a16;
              uint32_t b_lo = b_res ? fw.b_lo0 + res16 + (uint32_t)cb * fw.b_bytes16 : fw.b_lo0 + sa16 + fw.my_b16;
              if (fw.four) {  // 128-byte rows: four 32-byte reduction slices per tap
#pragma unroll 1
                for (int g = 0; g < cnt; ++g) {
                  const uint64_t da = ((uint64_t)fw.a_hi << 32) | a_lo, db = ((uint64_t)fw.b_hi << 32) | b_lo;
                  warp_mma_f16(d_tmem, da, db, idesc, accumulate);
                  warp_mma_f16(d_tmem, da + a_kadv, db + b_kadv, idesc, 1u);
                  warp_mma_f16(d_tmem, da + 2 * a_kadv, db + 2 * b_kadv, idesc, 1u);
                  warp_mma_f16(d_tmem, da + 3 * a_kadv, db + 3 * b_kadv, idesc, 1u);
                  accumulate = 1u;
                  a_lo += fw.halo_row16;
                  b_lo += fw.b_tap16;
                }
              } else {  // 64-byte rows (narrow stem): two slices per tap, two taps per trip
                int g = 0;
#pragma unroll 1
                for (; g + 1 < cnt; g += 2) {
                  const uint64_t da = ((uint64_t)fw.a_hi << 32) | a_lo, db = ((uint64_t)fw.b_hi << 32) | b_lo;
                  const uint64_t da2 = da + fw.halo_row16, db2 = db + fw.b_tap16;
                  warp_mma_f16(d_tmem, da, db, idesc, accumulate);
                  warp_mma_f16(d_tmem, da + a_kadv, db + b_kadv, idesc, 1u);
                  warp_mma_f16(d_tmem, da2, db2, idesc, 1u);
                  warp_mma_f16(d_tmem, da2 + a_kadv, db2 + b_kadv, idesc, 1u);
                  accumulate = 1u;
                  a_lo += 2 * fw.halo_row16;
                  b_lo += 2 * fw.b_tap16;
                }
                if (g < cnt) {
                  const uint64_t da = ((uint64_t)fw.a_hi << 32) | a_lo, db = ((uint64_t)fw.b_hi << 32) | b_lo;
                  warp_mma_f16(d_tmem, da, db, idesc, accumulate);
                  warp_mma_f16(d_tmem, da + a_kadv, db + b_kadv, idesc, 1u);
                  accumulate = 1u;
                }
              }
              warp_commit(empty_bar(s));  // frees the stage once these MMAs have read it
              sa16 += fw.stage16;
              if (++s == S) {
                s = 0;
                ph ^= 1u;
                sa16 = fw.ring16;
              }
            }
            res16 += (uint32_t)cnt * fw.b_tap16;
          }
        } else {
#pragma unroll 1
          for (int ks = t.ks_begin; ks < t.ks_end; ++ks) {
            if (!mbar_wait(SPLIT ? ready_bar(s) : full_bar(s), ph, abort_flag, g_error_record, a.wait_limit_ns, 0x300u + (unsigned)s)) {
              ok = false;
              break;
            }
            tc_fence_after_sync();
            const uint32_t sa = ring_base + (uint32_t)s * stage_bytes;
            uint64_t da = a_desc0 + (uint64_t)(sa >> 4);
            uint64_t db = b_desc0 + (uint64_t)((sa + kABytes) >> 4);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              if (SPLIT) {
                warp_mma_tf32(d_tmem, da + lo_off, db, idesc, accumulate);
                warp_mma_tf32(d_tmem, da, db + lo_off, idesc, 1u);
                warp_mma_tf32(d_tmem, da, db, idesc, 1u);
              } else {
                warp_mma_f16(d_tmem, da, db, idesc, accumulate);
              }
              accumulate = 1u;
              da += a_kadv;
              db += b_kadv;
            }
            warp_commit(empty_bar(s));  // frees the stage once these MMAs have read it
            if (++s == S) {
              s = 0;
              ph ^= 1u;
            }
          }
        }
        if (!ok) break;
        if (t.ks_end > t.ks_begin) warp_commit(acc_full_bar((int)buf));
        else if (elect_one()) mbar_arrive(acc_full_bar((int)buf));  // nothing to accumulate: the epilogue writes zeros
        if (++buf == acc_bufs) {
          buf = 0;
          aph ^= 1u;
        }
      }
    }
  } else if (role < 6) {
    // ------------------------------- epilogue ------------------------------------------------
    const int q = warp & 3;  // TMEM lanes [32q, 32q+32) are the ones this warp may read
    [[maybe_unused]] const int row = q * 32 + lane;
    uint32_t store_count = 0;
    const int wslot = role - 2;  // 0..3: which staging slices of the group this warp owns
    WarpStore ws;
    ws.nsw = a.nsw;
    const uint32_t warp_slices = (uint32_t)a.nsw + (EPI == 3 ? (uint32_t)a.mask_slots : 0u);  // the last ones are the mask slots
    const uint32_t my_staging = staging_off + (uint32_t)grp * group_staging + (uint32_t)wslot * warp_slices * 4096u;
    ws.buf = smem + my_staging;
    ws.buf_addr = base + my_staging;
    [[maybe_unused]] MaskSlot mask_slot;
    mask_slot.addr = base + my_staging + (uint32_t)a.nsw * 4096u;
    mask_slot.bar = bar_base + (uint32_t)kBarBlockBytes + (uint32_t)a.bias_smem_bytes + 16u * (uint32_t)(grp * 4 + wslot);
    mask_slot.nslots = (uint32_t)a.mask_slots;
    mask_slot.issued = mask_slot.consumed = 0;
    ws.qw = (q * 32) % a.etw;
    ws.qh = ((q * 32) / a.etw) % a.eth;
    ws.qn = (q * 32) / (a.etw * a.eth);
    uint32_t buf = 0, aph = 0;
    TileWalker walker;
    walker.init(a, first_tile, tile_step);
    if constexpr (EPI == 3) {
      mask_slot.walker = walker;
      mask_slot.tile = first_tile;
      mask_slot.c0 = 0;
      mask_slot.tile_step = tile_step;
      mask_slot.total_tiles = total_tiles;
      mask_slot.sub_w = sub_w;
      mask_slot.sub_h = sub_h;
      mask_slot.sub_n = sub_n;
      for (uint32_t i = 0; i < mask_slot.nslots; ++i) request_mask_block(a, ws, mask_slot);
    }
#pragma unroll 1
    for (int tile = first_tile; tile < total_tiles; tile += tile_step, walker.advance()) {
      TileCoord t = walker.coord(a);
      t.w0 += sub_w;
      t.h0 += sub_h;
      t.n0 += sub_n;
      if (!mbar_wait(acc_full_bar((int)buf), aph, abort_flag, g_error_record, a.wait_limit_ns, 0x400u + buf)) break;
      tc_fence_after_sync();
      const uint32_t tmem_acc = grp_tmem + ((uint32_t)(q * 32) << 16) + buf * acc_stride;
      const bool zero = !(t.ks_end > t.ks_begin);
      if constexpr (EPI >= 2) {
        if (!epilogue_tile_tma_fast<OutT, EPI == 3 || EPI == 5, EPI == 4, EPI == 5>(a, t, tmem_acc, lane, zero, ws, store_count, bias_s, q * 32, mask_slot,
                                                    abort_flag))
          break;
      } else if constexpr (EPI == 1) {
        epilogue_tile_tma<OutT>(a, t, tmem_acc, lane, zero, ws, store_count);
      } else {
        epilogue_tile<OutT>(a, t, tmem_acc, row, zero);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty_bar((int)buf));
      if (++buf == acc_bufs) {
        buf = 0;
        aph ^= 1u;
      }
    }
    // the staging tiles must not be released while a store is still reading them
    if (EPI != 0 && lane == 0) bulk_wait_group<0>();
  } else if (SPLIT) {
    // ------------------------------- hi/lo split (fp32 as 3xTF32) ----------------------------
    // hi is the 19 leading bits of an fp32 word, which is all the tensor core reads of it, so the
    // landed tile serves as the hi part as it is; lo = x - hi is exact in fp32 and is written to the
    // second part of the stage.  Element positions do not change, so the swizzle is irrelevant here.
    const int tid = threadIdx.x - 6 * 32;  // 0..127
    const int chunks = (int)((a.b_presplit ? (uint32_t)kABytes : part_bytes) >> 4);  // A comes first in a part
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    TileWalker walker;
    walker.init(a, first_tile, tile_step);
#pragma unroll 1
    for (int tile = first_tile; tile < total_tiles && ok; tile += tile_step, walker.advance()) {
      const TileCoord t = walker.coord(a);
#pragma unroll 1
      for (int ks = t.ks_begin; ks < t.ks_end; ++ks) {
        if (!mbar_wait(full_bar(s), ph, abort_flag, g_error_record, a.wait_limit_ns, 0x500u + (unsigned)s)) {
          ok = false;
          break;
        }
        uint4* hi = reinterpret_cast<uint4*>(ring_mem + (size_t)s * stage_bytes);
        uint4* lo = reinterpret_cast<uint4*>(ring_mem + (size_t)s * stage_bytes + part_bytes);
        for (int c = tid; c < chunks; c += 128) {
          uint4 v = hi[c], h, l;
          h.x = v.x & 0xFFFFE000u;
          h.y = v.y & 0xFFFFE000u;
          h.z = v.z & 0xFFFFE000u;
          h.w = v.w & 0xFFFFE000u;
          l.x = __float_as_uint(__uint_as_float(v.x) - __uint_as_float(h.x));
          l.y = __float_as_uint(__uint_as_float(v.y) - __uint_as_float(h.y));
          l.z = __float_as_uint(__uint_as_float(v.z) - __uint_as_float(h.z));
          l.w = __float_as_uint(__uint_as_float(v.w) - __uint_as_float(h.w));
          lo[c] = l;  // the hi part stays as it is: the tensor core reads the 19 leading bits of an fp32 word only
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(ready_bar(s));
        if (++s == S) {
          s = 0;
          ph ^= 1u;
        }
      }
    }
  }

  // ------------------------------- teardown ---------------------------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    // Loads already issued may still be landing in shared memory: give them time before the
    // CTA's shared memory is released.
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) {
    }
    __syncthreads();
  }
  if (warp == 1) tmem_dealloc(tmem_base, (uint32_t)a.tmem_cols);
}

template <bool SPLIT, int EPI, typename OutT>
__global__ void __launch_bounds__(SPLIT ? 320 : 384, 1) umma_gemm_kernel(const __grid_constant__ GemmArgs args) {
  umma_gemm_body<SPLIT, EPI, OutT>(args, (int)blockIdx.x, (int)gridDim.x);
}

// Several independent GEMMs in one launch, each on its own share of the grid: the parity classes of
// a strided input backprop (up to four GEMMs over disjoint pixels of dx).  As separate launches each
// class pays its own ramp and tail on a quarter of the work; side by side they finish together.
// CTAs first_cta[i] .. first_cta[i + 1] - 1 work on GEMM i.
constexpr int kMaxMulti = 4;
struct alignas(64) GemmArgsMulti {
  GemmArgs gemm[kMaxMulti];
  int count;
  int first_cta[kMaxMulti + 1];
};

template <int EPI, typename OutT>
__global__ void __launch_bounds__(384, 1) umma_gemm_multi_kernel(const __grid_constant__ GemmArgsMulti args) {
  int which = 0;
  while (which + 1 < args.count && (int)blockIdx.x >= args.first_cta[which + 1]) ++which;
  const int cta = (int)blockIdx.x - args.first_cta[which], n_ctas = args.first_cta[which + 1] - args.first_cta[which];
  // One copy of the body per GEMM: with a run-time index the fields of the arguments stop being
  // constant-bank operands and become loads, which the single-thread roles and the short epilogues
  // of the body cannot afford (measured: twice the time on the 56x56 layer).
  switch (which) {
    case 0: umma_gemm_body<false, EPI, OutT>(args.gemm[0], cta, n_ctas); break;
    case 1: umma_gemm_body<false, EPI, OutT>(args.gemm[1], cta, n_ctas); break;
    case 2: umma_gemm_body<false, EPI, OutT>(args.gemm[2], cta, n_ctas); break;
    default: umma_gemm_body<false, EPI, OutT>(args.gemm[3], cta, n_ctas); break;
  }
}

// ------------------------------------------------------------------------------------------------
// CTA-pair variant (tcgen05 cta_group::2) of the forward-style GEMM with a long reduction and 256
// output columns per tile.  A cluster of two CTAs works on a tile of 256 rows (two neighbouring row
// tiles, as in pair mode) x 256 columns: each CTA loads its own 128 rows of A and 128 of the 256
// columns of B per stage, the CTA of rank 0 issues MMAs of 256 x 256 x 16 that read both shared
// memories, and each CTA finds its 128 rows of the accumulator in its own tensor memory (two
// buffers of 256 columns, so the epilogue overlaps the next tile).  Per MMA an SM reads 4 KB of A and
// 4 KB of B from shared memory for 128 cycles of math, against 12 KB for a 128 x 256 tile of one CTA.
//   warp 0  producer (both CTAs: own A rows, own half of B; the bytes of both count on rank 0's barrier)
//   warp 1  MMA issuer (rank 0 only; warp 1 of both CTAs owns the TMEM allocation)
//   warps 2..5  epilogue of the CTA's own 128 rows (packed 16-bit epilogue with TMA stores)
// Barriers live at the same offsets in both CTAs: full[s] is used in rank 0 only; empty[s] and
// acc_full[b] are signalled in both CTAs by the issuer's commits; acc_empty[b] of rank 0 collects the
// eight epilogue warps of the pair.
template <typename OutT, bool BITS>
__global__ void __launch_bounds__(192, 1) umma_gemm_pair2_kernel(const __grid_constant__ GemmArgs args) {
  extern __shared__ uint8_t smem_raw[];
  const GemmArgs& a = args;
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const int warp = __shfl_sync(0xFFFFFFFFu, (int)(threadIdx.x >> 5), 0), lane = (int)(threadIdx.x & 31);
  const uint32_t rank = cluster_cta_rank();
  const bool leader = rank == 0;
  const int S = a.stages;
  constexpr uint32_t kStage = 2u * kABytes;  // A tile 16 KB + half of the B tile 16 KB
  const uint32_t staging_off = (uint32_t)S * kStage;
  const uint32_t bar_off = staging_off + (uint32_t)a.nsw * 4u * 4096u;
  uint8_t* bar_mem = smem + bar_off;
  const uint32_t bar_base = base + bar_off;
  auto full_bar = [&](int s) { return bar_base + 8u * (uint32_t)s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (uint32_t)(kMaxStages + s); };
  auto acc_full_bar = [&](int b) { return bar_base + 8u * (uint32_t)(2 * kMaxStages + b); };
  auto acc_empty_bar = [&](int b) { return bar_base + 8u * (uint32_t)(2 * kMaxStages + 2 + b); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_mem + 8 * (2 * kMaxStages + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_mem + 8 * (2 * kMaxStages + 4) + 4);
  const uint32_t bias_s = a.bias != nullptr ? bar_base + (uint32_t)kBarBlockBytes : 0u;

  if ((int)threadIdx.x < 2 * kMaxStages + 4) {  // one barrier per thread
    const int j = (int)threadIdx.x;
    mbar_init(bar_base + 8u * (uint32_t)j, j >= 2 * kMaxStages + 2 ? 8u : 1u);
    if (j == 0) *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&a.a_map[0]);
    prefetch_tensormap(&a.b_map);
    prefetch_tensormap(&a.out_map);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), 512u);
    tmem_relinquish_pair();
  }
  // the peer's barriers are initialised before anything of this CTA signals them
  tc_fence_before_sync();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  grid_dependency_wait();
  grid_launch_dependents();
  if (a.bias != nullptr) {
    const OutT* bias = static_cast<const OutT*>(a.bias);
    uint4* dst = reinterpret_cast<uint4*>(bar_mem + kBarBlockBytes);
    const int chunks = a.bias_smem_bytes >> 4;
    for (int i = threadIdx.x; i < chunks; i += blockDim.x) {
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (i * 8 + 8 <= a.ext_cols) v = __ldg(reinterpret_cast<const uint4*>(bias) + i);
      dst[i] = v;
    }
  }
  __syncthreads();

  const int total_tiles = a.n_tiles * a.tiles_w * a.tiles_h * a.tiles_n;  // tiles of 256 rows
  const int first_tile = (int)(blockIdx.x >> 1), tile_step = (int)(gridDim.x >> 1);
  // this CTA's 128 rows inside the 256-row tile
  const int sub_w = a.pair_dim == 1 ? (int)rank * a.tw : 0, sub_h = a.pair_dim == 2 ? (int)rank * a.th : 0,
            sub_n = a.pair_dim == 3 ? (int)rank * a.tn : 0;

  if (warp == 0) {
    // ------------------------------- producer ------------------------------------------------
    const int epr = a.epr, cblocks = a.cblocks;
    const CUtensorMap* bmap = &a.b_map;
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    TileWalker walker;
    walker.init(a, first_tile, tile_step);
#pragma unroll 1
    for (int tile = first_tile; tile < total_tiles && ok; tile += tile_step, walker.advance()) {
      const TileCoord t = walker.coord(a);
      const int nf0 = t.nf0 + (int)rank * 128;  // this CTA's half of the tile's columns
#pragma unroll 1
      for (int tap = 0; tap < a.num_taps && ok; ++tap) {
        const TapEntry e = a.taps[tap];
        const CUtensorMap* amap = &a.a_map[e.a_map];
        const int aw = t.w0 + sub_w + e.dw, ah = t.h0 + sub_h + e.dh, an = t.n0 + sub_n;
#pragma unroll 1
        for (int cb = 0, kc = 0; cb < cblocks; ++cb, kc += epr) {
          if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, g_error_record, a.wait_limit_ns, 0x900u + (unsigned)s)) {
            ok = false;
            break;
          }
          const uint32_t fb = full_bar(s);
          if (leader) warp_arrive_expect_tx(fb, 2u * kStage);  // the bytes of both CTAs
          const uint32_t sa = base + (uint32_t)s * kStage;
          warp_tma_load_4d_pair(sa, amap, fb, kc, aw, ah, an);
          warp_tma_load_4d_pair(sa + kABytes, bmap, fb, 0, kc, nf0 / epr, e.b_tap);  // two 64-column blocks
          if (++s == S) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (rank 0) --------------------------------------
    if (leader) {
      const uint64_t a_desc0 = make_smem_desc(0, a.a_lbo, a.a_sbo, a.a_layout);
      const uint64_t b_desc0 = make_smem_desc(0, a.b_lbo, a.b_sbo, a.b_layout);
      const uint32_t a_kadv = a.a_kadv >> 4, b_kadv = a.b_kadv >> 4, idesc = a.idesc;
      const int steps = a.num_taps * a.cblocks;
      int s = 0;
      uint32_t ph = 0, buf = 0, aph = 0;
      bool ok = true;
#pragma unroll 1
      for (int tile = first_tile; tile < total_tiles && ok; tile += tile_step) {
        if (!mbar_wait(acc_empty_bar((int)buf), aph ^ 1u, abort_flag, g_error_record, a.wait_limit_ns, 0xA00u + buf)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * 256u;
        uint32_t accumulate = 0u;
#pragma unroll 1
        for (int ks = 0; ks < steps; ++ks) {
          if (!mbar_wait(full_bar(s), ph, abort_flag, g_error_record, a.wait_limit_ns, 0xB00u + (unsigned)s)) {
            ok = false;
            break;
          }
          const uint32_t sa = (base + (uint32_t)s * kStage) & 0x3FFFFu;  // offset inside the CTA's shared memory
          const uint64_t da = a_desc0 + (uint64_t)(sa >> 4), db = b_desc0 + (uint64_t)((sa + kABytes) >> 4);
          warp_mma_f16_pair(d_tmem, da, db, idesc, accumulate);
          warp_mma_f16_pair(d_tmem, da + a_kadv, db + b_kadv, idesc, 1u);
          warp_mma_f16_pair(d_tmem, da + 2 * a_kadv, db + 2 * b_kadv, idesc, 1u);
          warp_mma_f16_pair(d_tmem, da + 3 * a_kadv, db + 3 * b_kadv, idesc, 1u);
          accumulate = 1u;
          warp_commit_pair(empty_bar(s), cluster_map_shared(empty_bar(s), 1u));  // both CTAs may refill the stage
          if (++s == S) {
            s = 0;
            ph ^= 1u;
          }
        }
        if (!ok) break;
        warp_commit_pair(acc_full_bar((int)buf), cluster_map_shared(acc_full_bar((int)buf), 1u));
        if (++buf == 2u) {
          buf = 0;
          aph ^= 1u;
        }
      }
    }
  } else {
    // ------------------------------- epilogue (own 128 rows) ----------------------------------
    const int q = warp & 3;  // TMEM lanes [32q, 32q+32)
    const int wslot = warp - 2;
    uint32_t store_count = 0;
    WarpStore ws;
    ws.nsw = a.nsw;
    const uint32_t my_staging = staging_off + (uint32_t)wslot * (uint32_t)a.nsw * 4096u;
    ws.buf = smem + my_staging;
    ws.buf_addr = base + my_staging;
    ws.qw = (q * 32) % a.etw;
    ws.qh = ((q * 32) / a.etw) % a.eth;
    ws.qn = (q * 32) / (a.etw * a.eth);
    MaskSlot unused_mask;
    uint32_t buf = 0, aph = 0;
    TileWalker walker;
    walker.init(a, first_tile, tile_step);
#pragma unroll 1
    for (int tile = first_tile; tile < total_tiles; tile += tile_step, walker.advance()) {
      TileCoord t = walker.coord(a);
      t.w0 += sub_w;
      t.h0 += sub_h;
      t.n0 += sub_n;
      if (!mbar_wait(acc_full_bar((int)buf), aph, abort_flag, g_error_record, a.wait_limit_ns, 0xC00u + buf)) break;
      tc_fence_after_sync();
      const uint32_t tmem_acc = tmem_base + ((uint32_t)(q * 32) << 16) + buf * 256u;
      if (!epilogue_tile_tma_fast<OutT, false, BITS>(a, t, tmem_acc, lane, false, ws, store_count, bias_s, q * 32, unused_mask,
                                               abort_flag))
        break;
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty_bar((int)buf) & kPeerBitMask);  // rank 0 collects both CTAs
      if (++buf == 2u) {
        buf = 0;
        aph ^= 1u;
      }
    }
    if (lane == 0) bulk_wait_group<0>();
  }

  // ------------------------------- teardown ---------------------------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) {
    }
    __syncthreads();
  }
  // neither CTA leaves (and frees its shared and tensor memory) while the other may still use them
  cluster_sync_all();
  if (warp == 1) tmem_dealloc_pair(tmem_base, 512u);
}

// ================================================================================================
// Host side: tensor maps and launch plans
// ================================================================================================

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    else
      cudaGetLastError();
  });
  return fn;
}

// 4-D tiled map with a 128-byte swizzle and zero fill outside the tensor.  dims[0] is the
// contiguous dimension; strides_bytes[i] is the stride of dims[i+1].  A 32-bit operand that the
// MMA reads MN-major must be swizzled in 32-byte units (the only MN-major layout tcgen05 accepts
// for tf32); everything else uses the ordinary 16-byte-unit pattern.
bool make_map(CUtensorMap* map, int dtype, bool mn_major, const void* base, const uint64_t dims[4],
              const uint64_t strides_bytes[3], const uint32_t box[4], bool rows64 = false) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) {
    fail(PDNN_ALLOCATION_PROBLEM, "cuTensorMapEncodeTiled is unavailable");
    return false;
  }
  CUtensorMapDataType dt = dtype == PDNN_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                          : dtype == PDNN_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                              : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  cuuint64_t d[4], st[3];
  cuuint32_t b[4], es[4] = {1, 1, 1, 1};
  for (int i = 0; i < 4; ++i) {
    d[i] = dims[i];
    b[i] = box[i];
  }
  for (int i = 0; i < 3; ++i) st[i] = strides_bytes[i];
  // rows64: the box is 64 bytes wide and lands as 64-byte rows swizzled in 16-byte units
  const CUtensorMapSwizzle sw = rows64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                : (dtype == PDNN_F32 && mn_major) ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                                                                  : CU_TENSOR_MAP_SWIZZLE_128B;
  CUresult r = fn(map, dt, 4, const_cast<void*>(base), d, st, b, es, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fail(PDNN_INVALID_PARAMETER,
         "cuTensorMapEncodeTiled failed (%d): dims %llu %llu %llu %llu strides %llu %llu %llu box %u %u %u %u", (int)r,
         (unsigned long long)d[0], (unsigned long long)d[1], (unsigned long long)d[2], (unsigned long long)d[3],
         (unsigned long long)st[0], (unsigned long long)st[1], (unsigned long long)st[2], b[0], b[1], b[2], b[3]);
    return false;
  }
  return true;
}

int floor_div(int a, int b) { return (a >= 0) ? a / b : -((-a + b - 1) / b); }
int pos_mod(int a, int b) { return a - floor_div(a, b) * b; }
int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Splits `total` (a power of two) rows into a box tw x th x tn of powers of two that wastes the
// fewest rows when tiled over [W, H, N]; ties go to the widest box.
void choose_box(int total, int W, int H, int N, int* tw, int* th, int* tn) {
  double best = -1;
  for (int w = total; w >= 1; w >>= 1)
    for (int h = total / w; h >= 1; h >>= 1) {
      const int n = total / (w * h);
      if (w > 256 || h > 256 || n > 256) continue;
      const double covered = (double)ceil_div(W, w) * w * (double)ceil_div(H, h) * h * (double)ceil_div(N, n) * n;
      const double eff = ((double)W * H * N) / covered;
      if (eff > best + 1e-9) {
        best = eff;
        *tw = w;
        *th = h;
        *tn = n;
      }
    }
}

constexpr size_t kMaxResidentB = 128 * 1024;

constexpr int kPlanAgain = -2;  // internal: the halo plan does not fit, plan the layer without it

// Row-tile box for halo mode: one image (tn == 1), tw a multiple of 8 so that a shift by one tile
// row is a whole number of 1024-byte swizzle groups.  `rows` is the number of taps that share a
// copy.  Picks the box that loads the fewest bytes per useful output pixel; returns false if every
// candidate wastes more than 15% of its rows.
bool choose_box_halo(int W, int H, int rows, int* tw, int* th) {
  double best = 1e30;
  for (int w = 8; w <= kTileM; w <<= 1) {
    const int h = kTileM / w;
    const double eff = ((double)W / (ceil_div(W, w) * w)) * ((double)H / (ceil_div(H, h) * h));
    if (eff < 0.85) continue;
    const double cost = (double)(h + rows - 1) / h / eff;
    if (cost < best - 1e-9) {
      best = cost;
      *tw = w;
      *th = h;
    }
  }
  return best < 1e29;
}

// Tiles with a short reduction spend most of their time in the epilogue: column tiles of at most
// 128 leave room for two accumulator buffers per pipeline, so that the next tile's MMAs overlap it.
bool want_narrow(int ksteps, int cols) { return ksteps <= 4 || cols <= 128; }

int pick_bn(long long row_tiles, int cols, int unit, int max_bn, int sms, int ksteps = 1 << 30) {
  if (want_narrow(ksteps, cols)) max_bn = std::min(max_bn, 128);
  sms *= 2;  // two pipelines per CTA work on two tiles at a time
  // cost ~ waves * (bn + fixed overhead); unit: granularity the B loader needs
  int best_bn = unit;
  double best = 1e30;
  for (int bn = unit; bn <= max_bn; bn += unit) {
    if (bn != 16 && bn != 32 && bn != 48 && bn % 64 != 0) continue;
    if (cols >= 64 && bn % 64 != 0) continue;  // whole 128-byte output blocks for the TMA-store epilogue
    const long long tiles = row_tiles * ceil_div(cols, bn);
    const double waves = (double)((tiles + sms - 1) / sms);
    const double cost = waves * (bn + 40.0);
    if (cost < best - 1e-9) {
      best = cost;
      best_bn = bn;
    }
    if (bn >= ((cols + unit - 1) / unit) * unit) break;
  }
  return best_bn;
}

int next_pow2(int v) {
  int p = 32;
  while (p < v) p <<= 1;
  return p;
}

void set_operand_layout(GemmArgs& g, int dtype, int b_mn) {
  const bool f32 = dtype == PDNN_F32;
  g.epr = f32 ? 32 : 64;
  const unsigned kstep_bytes_k = 32;                     // one UMMA K step inside a 128-byte row
  const unsigned kstep_bytes_mn = (f32 ? 8u : 16u) * 128u;  // UMMA K rows of 128 bytes
  const unsigned rows = (unsigned)g.epr;                 // reduction rows per stage for MN-major operands
  // MN-major fp32: 32-byte swizzle units, pattern repeats every 4 rows of 128 bytes.
  const unsigned mn_sbo = f32 ? 512u : 1024u, mn_layout = f32 ? 1u : 2u;
  g.a_layout = g.a_mn ? mn_layout : 2u;
  g.b_layout = b_mn ? mn_layout : 2u;
  if (g.a_mn) {
    g.a_lbo = rows * 128u;
    g.a_sbo = mn_sbo;
    g.a_kadv = kstep_bytes_mn;
    g.a_boxes = kTileM / g.epr;
    g.a_box_bytes = rows * 128u;
  } else {
    g.a_lbo = 16u;
    g.a_sbo = 1024u;
    g.a_kadv = kstep_bytes_k;
    g.a_boxes = 1;
    g.a_box_bytes = kABytes;
  }
  if (b_mn) {
    g.b_lbo = rows * 128u;
    g.b_sbo = mn_sbo;
    g.b_kadv = kstep_bytes_mn;
    g.b_boxes = g.bn / g.epr;
    g.b_box_bytes = rows * 128u;
  } else {
    g.b_lbo = 16u;
    g.b_sbo = 1024u;
    g.b_kadv = kstep_bytes_k;
    g.b_boxes = 1;
    g.b_box_bytes = (unsigned)g.bn * 128u;
  }
  g.a_row_bytes = 128;
  g.kmmas = 4;
  g.b_step_bytes = (unsigned)g.bn * 128u;
  g.idesc = make_idesc(dtype == PDNN_F32 ? 2 : (dtype == PDNN_BF16 ? 1 : 0), g.a_mn, b_mn, g.bn);
  g.tmem_cols = next_pow2(2 * g.bn);
}

// Chooses the store path of the epilogue and sizes the pipeline; call once the output fields of
// `g` are set.  out_dims / out_strides describe the output as a 4-D tensor whose dimension 0 is
// the column (feature) axis and whose other dimensions are the ones the row-tile box spans.
bool setup_store(GemmArgs& g, int compute_dtype, const uint64_t out_dims[4], const uint64_t out_strides[3]) {
  g.cpb = 128 / (int)dtype_size(g.out_dtype);
  g.tma_store = 0;
  if (g.beta == 0.f && g.bn % g.cpb == 0 && aligned16(g.out)) {
    // one store covers the 32 rows of one epilogue warp: a sub-box of the row tile
    const int sw = std::min(g.etw, 32), sh = std::min(g.eth, 32 / sw), sn = 32 / (sw * sh);
    const uint32_t box[4] = {(uint32_t)g.cpb, (uint32_t)sw, (uint32_t)sh, (uint32_t)sn};
    if (!make_map(&g.out_map, g.out_dtype, false, g.out, out_dims, out_strides, box)) return false;
    g.tma_store = 1;
    g.epi_fast = (g.out_dtype != PDNN_F32 && g.alpha == 1.f && g.ext_cols % 8 == 0 &&
                  (g.act == PDNN_ACT_NONE || g.act == PDNN_ACT_RELU || g.act == PDNN_ACT_RELU6) &&
                  (g.bias == nullptr || aligned16(g.bias)))
                     ? 1
                     : 0;
    // the mask tensor is read through a map with the geometry of the output map
    if (g.epi_fast && g.relu_mask != nullptr && g.mask_bits == nullptr &&
        !make_map(&g.mask_map, g.out_dtype, false, g.relu_mask, out_dims, out_strides, box))
      g.relu_mask = nullptr;
  }
  // the one-bit-per-element forms work on whole 64-column blocks of the packed epilogue
  if (!(g.epi_fast && g.ext_cols % 64 == 0)) {
    g.bitmask_out = nullptr;
    if (g.mask_bits != nullptr) g.relu_mask = g.mask_bits = nullptr;
  }
  const bool split = compute_dtype == PDNN_F32;
  // Two pipelines per CTA, except for 256-column tiles outside pair mode with a reduction of 8 steps or
  // more: their MMAs take 128 cycles each, which one issuer sustains, and a single pipeline leaves
  // TMEM for a second accumulator buffer, so that the epilogue overlaps the next tile.
  {
    const int steps = g.a_mn ? g.slabs_per_split : g.num_taps * g.cblocks * (g.halo ? 3 : 1);
    const int dflt = (!g.a_mn && !g.pair && g.bn == 256 && steps >= 8) ? 1 : 2;
    g.groups = split ? 1 : dflt;
  }
  g.acc_stride = std::max(32, next_pow2(g.bn));
  g.acc_bufs = g.groups * 2 * g.acc_stride <= 512 ? 2 : 1;
  g.tmem_cols = next_pow2(g.groups * g.acc_bufs * g.acc_stride);
  g.bias_smem_bytes = 0;
  g.bias_tile_only = 0;
  if (!g.epi_fast) g.relu_mask = nullptr;  // only the fast epilogue applies the mask; the caller checks
  g.mask_smem_bytes = g.relu_mask != nullptr ? 128 : 0;  // the mask slots' barriers; the slots count as staging
  if (g.pair && !g.cta_pair && (split || g.groups != 2 || !g.tma_store)) return false;  // the caller plans again without pairing
  if (g.epi_fast && g.bias != nullptr) {
    const int padded = ceil_div(g.n_tiles * g.bn, 64) * 64;
    if (g.pair && !g.cta_pair && g.n_tiles <= 16) {
      g.bias_tile_only = 1;  // every byte counts towards a third stage
      g.bias_smem_bytes = ceil_div(g.bn, 64) * 128;
    } else if (padded * 2 > 8192) {
      g.epi_fast = 0;  // the general staged epilogue reads the bias from global memory
    } else {
      g.bias_smem_bytes = padded * 2;
    }
  }
  unsigned stage = (kABytes + (unsigned)g.bn * 128u) * (split ? 2u : 1u);
  int ksteps = g.a_mn ? g.slabs_per_split : g.num_taps * g.cblocks;
  if (!g.halo) g.res_taps = g.num_taps;
  else ksteps = g.res_taps * g.cblocks;
  g.b_res = 0;
  g.b_res_bytes = 0;
  const int fixed = 1024 + kBarBlockBytes + g.bias_smem_bytes + g.mask_smem_bytes;
  g.mask_slots = (g.relu_mask != nullptr && g.mask_bits == nullptr) ? 1 : 0;
  auto staging = [&](int nsw) { return g.tma_store ? g.groups * 4 * (nsw + g.mask_slots) * 4096 : 0; };
  // A small filter (all taps, all column tiles) is kept in shared memory for the whole kernel:
  // the filter tiles are the part of the L2 -> SM traffic that never changes.
  if (g.cta_pair) {
    // one pipeline per CTA: a stage is the CTA's A tile and its half of the B tile
    if (split || !g.tma_store || !g.epi_fast || g.relu_mask != nullptr || g.bn != 256) return false;
    g.groups = 1;
    g.acc_bufs = 2;
    g.acc_stride = 256;
    g.tmem_cols = 512;
    const int avail = kSmemBudget - fixed, stage2 = 2 * kABytes;
    auto stages_with = [&](int nsw) { return (avail - 4 * nsw * 4096) / stage2; };
    g.nsw = stages_with(2) >= 6 ? 2 : 1;
    g.stages = std::min(kMaxStages, stages_with(g.nsw));
    return g.stages >= 4;
  }
  if (g.pair) {
    stage = 2u * kABytes + (unsigned)g.bn * 128u;
    const int avail = kSmemBudget - fixed;
    auto stages_with = [&](int nsw) { return (avail - staging(nsw)) / (int)stage; };
    g.nsw = stages_with(2) >= 4 ? 2 : 1;
    if (g.mask_slots == 1) {  // a second mask slot per warp where four stages remain
      g.mask_slots = 2;
      if (stages_with(g.nsw) < 4) g.mask_slots = 1;
    }
    g.stages = std::min(kMaxStages, stages_with(g.nsw));
    return g.stages >= 2;
  }
  if (!g.a_mn && !split && g.tma_store && g.b_batch_mul == 0) {
    const size_t res_tile = (size_t)ksteps * g.b_step_bytes, res_all = res_tile * g.n_tiles;
    const int a_stage = g.halo ? (int)g.halo_stage_bytes : kABytes;
    auto fits = [&](size_t res) {
      return res <= kMaxResidentB && res % 1024 == 0 &&
             (kSmemBudget - fixed - (int)res - staging(1)) / (g.groups * a_stage) >= (g.halo ? 2 : 3);
    };
    if (fits(res_all)) {
      g.b_res = 1;
      g.b_res_bytes = (unsigned)res_all;
      stage = (unsigned)a_stage;
    } else if (!g.halo && g.n_tiles <= 16 && fits(res_tile)) {
      g.b_res = 2;  // one column tile per CTA
      g.b_res_bytes = (unsigned)res_tile;
      stage = (unsigned)a_stage;
    }
  }
  if (g.halo && !g.b_res) return false;  // the caller plans the layer again without the halo
  // Staging slices per epilogue warp: a second slice lets a warp convert one 128-byte column
  // block while the store of the previous one still reads its slice; it is given up when the
  // load rings would otherwise be shallower than three stages.
  const int avail = kSmemBudget - fixed - (int)g.b_res_bytes;
  auto stages_with = [&](int nsw) { return (avail - staging(nsw)) / (g.groups * (int)stage); };
  g.nsw = stages_with(2) >= 3 ? 2 : 1;
  if (g.mask_slots == 1) {  // a second mask slot per warp where four stages remain
    g.mask_slots = 2;
    if (stages_with(g.nsw) < 4) g.mask_slots = 1;
  }
  g.stages = std::min(kMaxStages, stages_with(g.nsw));
  if (g.stages < 2 && g.groups == 2) {  // very wide stages: one pipeline with a deeper ring
    g.groups = 1;
    g.acc_bufs = 2 * g.acc_stride <= 512 ? 2 : 1;
    g.tmem_cols = next_pow2(g.acc_bufs * g.acc_stride);
    g.nsw = stages_with(2) >= 3 ? 2 : 1;
    g.stages = std::min(kMaxStages, stages_with(g.nsw));
  }
  return g.stages >= 1;
}

using GemmKernel = void (*)(const GemmArgs);
using GemmKernelMulti = void (*)(const GemmArgsMulti);

// Kernel instantiation for (split, epilogue kind, output dtype); nullptr for combinations that
// are never launched (the split kernel only produces fp32; packed arithmetic is 16-bit only).
GemmKernel select_kernel(bool split, int epi, int out_dtype) {
  if (split) {
    if (out_dtype != PDNN_F32) return nullptr;
    return epi == 1 ? umma_gemm_kernel<true, 1, float> : epi == 0 ? umma_gemm_kernel<true, 0, float> : nullptr;
  }
  switch (out_dtype) {
    case PDNN_F16:
      return epi == 5 ? umma_gemm_kernel<false, 5, __half>
             : epi == 4 ? umma_gemm_kernel<false, 4, __half>
             : epi == 3 ? umma_gemm_kernel<false, 3, __half>
             : epi == 2 ? umma_gemm_kernel<false, 2, __half>
                      : epi == 1 ? umma_gemm_kernel<false, 1, __half> : umma_gemm_kernel<false, 0, __half>;
    case PDNN_BF16:
      return epi == 5 ? umma_gemm_kernel<false, 5, __nv_bfloat16>
             : epi == 4 ? umma_gemm_kernel<false, 4, __nv_bfloat16>
             : epi == 3 ? umma_gemm_kernel<false, 3, __nv_bfloat16>
             : epi == 2 ? umma_gemm_kernel<false, 2, __nv_bfloat16>
                      : epi == 1 ? umma_gemm_kernel<false, 1, __nv_bfloat16> : umma_gemm_kernel<false, 0, __nv_bfloat16>;
    default:
      return epi == 1 ? umma_gemm_kernel<false, 1, float> : epi == 0 ? umma_gemm_kernel<false, 0, float> : nullptr;
  }
}

// Launch of the CTA-pair kernel: clusters of two CTAs, one cluster per pair of SMs.
int launch_gemm_pair2(const GemmArgs& g, long long total_pairs, cudaStream_t s) {
  const bool bits = g.bitmask_out != nullptr;
  GemmKernel kernel = g.out_dtype == PDNN_F16 ? (bits ? umma_gemm_pair2_kernel<__half, true> : umma_gemm_pair2_kernel<__half, false>)
                                              : (bits ? umma_gemm_pair2_kernel<__nv_bfloat16, true>
                                                      : umma_gemm_pair2_kernel<__nv_bfloat16, false>);
  const size_t smem = 1024 + (size_t)g.stages * 2 * kABytes + (size_t)g.nsw * 4 * 4096 + kBarBlockBytes + (size_t)g.bias_smem_bytes;
  if (smem > (size_t)kSmemBudget) return fail(PDNN_INVALID_PARAMETER, "tensor-core gemm: plan needs %zu bytes of shared memory", smem);
  {
    static std::mutex mu;
    static bool opted_in[kMaxDevices] = {};
    const int dev = current_device();
    if (dev < 0 || dev >= kMaxDevices) return fail(PDNN_ALLOCATION_PROBLEM, "tensor-core gemm: no usable current device");
    std::lock_guard<std::mutex> lock(mu);
    if (!opted_in[dev]) {
      bool ok = true;
      for (GemmKernel k : {GemmKernel(umma_gemm_pair2_kernel<__half, false>), GemmKernel(umma_gemm_pair2_kernel<__half, true>),
                           GemmKernel(umma_gemm_pair2_kernel<__nv_bfloat16, false>),
                           GemmKernel(umma_gemm_pair2_kernel<__nv_bfloat16, true>)})
        ok = ok && cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget) == cudaSuccess;
      if (!ok) {
        cudaGetLastError();
        return fail(PDNN_ALLOCATION_PROBLEM, "cannot opt in to %d bytes of shared memory", kSmemBudget);
      }
      opted_in[dev] = true;
    }
  }
  const int sms = device_sm_count();
  unsigned grid = (unsigned)std::min<long long>(2 * total_pairs, (long long)sms);
  grid -= grid % 2u;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  GemmArgs args = g;
  args.tap_pack = 1;
  args.wait_limit_ns = kWaitLimitNs;
  const cudaError_t le = cudaLaunchKernelEx(&cfg, kernel, args);
  if (le != cudaSuccess) {
    cudaGetLastError();
    return fail(PDNN_ALLOCATION_PROBLEM, "tensor-core gemm (CTA pairs): launch failed: %s", cudaGetErrorString(le));
  }
  if (g.bitmask_out != nullptr) bitmask_written_flag() = true;
  return check_launch("tensor-core gemm (CTA pairs)");
}

int launch_gemm(const GemmArgs& g, int dtype, cudaStream_t s) {
  const bool split = dtype == PDNN_F32;
  const int tap_pack = std::max(g.tap_pack, 1);
  const long long total = g.a_mn ? (long long)g.n_tiles * g.tiles_w * ((g.num_taps + tap_pack - 1) / tap_pack) * g.splits
                                 : (long long)g.n_tiles * g.tiles_w * g.tiles_h * g.tiles_n;
  if (total <= 0) return PDNN_OK;
  if (total > 0x7FFFFFFFll) return fail(PDNN_INDEX_EXCEEDED, "tensor-core gemm: too many tiles");
  if (g.cta_pair) return launch_gemm_pair2(g, total, s);
  const unsigned stage = g.pair   ? 2u * kABytes + (unsigned)g.bn * 128u
                         : g.halo ? g.halo_stage_bytes
                                  : g.b_res ? (unsigned)kABytes : (kABytes + (unsigned)g.bn * 128u) * (split ? 2u : 1u);
  const int rings = g.pair ? 1 : g.groups;
  // At least 120 KB, so that two CTAs never share an SM: the second one would wait for TMEM
  // columns the first one holds.
  size_t smem = 1024 + (size_t)g.b_res_bytes + (size_t)rings * g.stages * stage +
                (g.tma_store ? (size_t)g.groups * (g.nsw + g.mask_slots) * 4 * 4096 : 0) + kBarBlockBytes +
                (size_t)g.bias_smem_bytes + (size_t)g.mask_smem_bytes;
  smem = std::max<size_t>(smem, 120 * 1024);
  if (smem > (size_t)kSmemBudget) return fail(PDNN_INVALID_PARAMETER, "tensor-core gemm: plan needs %zu bytes of shared memory", smem);
  // The opt-in to large dynamic shared memory is a per-device attribute of each kernel: it is made
  // once for every device this process launches on, with that device current.
  {
    static std::mutex mu;
    static bool opted_in[kMaxDevices] = {};
    const int dev = current_device();
    if (dev < 0 || dev >= kMaxDevices) return fail(PDNN_ALLOCATION_PROBLEM, "tensor-core gemm: no usable current device");
    std::lock_guard<std::mutex> lock(mu);
    if (!opted_in[dev]) {
      for (int sp = 0; sp < 2; ++sp)
        for (int epi = 0; epi < 6; ++epi)
          for (int dt = 0; dt < 3; ++dt) {
            GemmKernel k = select_kernel(sp != 0, epi, dt);
            if (k != nullptr && cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget) != cudaSuccess) {
              cudaGetLastError();
              return fail(PDNN_ALLOCATION_PROBLEM, "cannot opt in to %d bytes of shared memory", kSmemBudget);
            }
          }
      opted_in[dev] = true;
    }
  }
  const int epi = g.epi_fast ? (g.mask_bits != nullptr ? 5 : g.relu_mask != nullptr ? 3 : g.bitmask_out != nullptr ? 4 : 2)
                             : (g.tma_store ? 1 : 0);
  GemmKernel kernel = select_kernel(split, epi, g.out_dtype);
  if (kernel == nullptr) return fail(PDNN_INVALID_PARAMETER, "tensor-core gemm: no kernel for this output type");
  const int sms = device_sm_count();
  unsigned grid = (unsigned)std::min<long long>(total, (long long)sms);
  if (g.b_res == 2 || g.bias_tile_only) {
    // every CTA stays on one column tile: tiles advance by a multiple of n_tiles
    if (grid < (unsigned)g.n_tiles) return fail(PDNN_INVALID_PARAMETER, "tensor-core gemm: grid smaller than the column tiles");
    grid -= grid % (unsigned)g.n_tiles;
  }
  // Programmatic dependent launch: the kernel's set-up may overlap the tail of the previous kernel
  // in the stream (the kernel waits for that kernel before it touches any tensor it wrote).
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(split ? 320 : 384);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  GemmArgs args = g;
  args.tap_pack = tap_pack;
  args.wait_limit_ns = kWaitLimitNs;
  const cudaError_t le = cudaLaunchKernelEx(&cfg, kernel, args);
  if (le != cudaSuccess) {
    cudaGetLastError();
    return fail(PDNN_ALLOCATION_PROBLEM, "tensor-core gemm: launch failed: %s", cudaGetErrorString(le));
  }
  if (g.bitmask_out != nullptr) bitmask_written_flag() = true;
  return check_launch("tensor-core gemm");
}

// The packed-epilogue kernels that exist as multi-GEMM instantiations: plain, tensor mask, bit mask.
GemmKernelMulti select_multi_kernel(int epi, int out_dtype) {
  if (out_dtype == PDNN_F16)
    return epi == 2 ? umma_gemm_multi_kernel<2, __half>
           : epi == 3 ? umma_gemm_multi_kernel<3, __half> : epi == 5 ? umma_gemm_multi_kernel<5, __half> : nullptr;
  if (out_dtype == PDNN_BF16)
    return epi == 2 ? umma_gemm_multi_kernel<2, __nv_bfloat16>
           : epi == 3 ? umma_gemm_multi_kernel<3, __nv_bfloat16> : epi == 5 ? umma_gemm_multi_kernel<5, __nv_bfloat16> : nullptr;
  return nullptr;
}

int gemm_epilogue_kind(const GemmArgs& g) {
  return g.epi_fast ? (g.mask_bits != nullptr ? 5 : g.relu_mask != nullptr ? 3 : g.bitmask_out != nullptr ? 4 : 2)
                    : (g.tma_store ? 1 : 0);
}

size_t gemm_smem_bytes(const GemmArgs& g, bool split) {
  const unsigned stage = g.pair   ? 2u * kABytes + (unsigned)g.bn * 128u
                         : g.halo ? g.halo_stage_bytes
                                  : g.b_res ? (unsigned)kABytes : (kABytes + (unsigned)g.bn * 128u) * (split ? 2u : 1u);
  const int rings = g.pair ? 1 : g.groups;
  const size_t smem = 1024 + (size_t)g.b_res_bytes + (size_t)rings * g.stages * stage +
                      (g.tma_store ? (size_t)g.groups * (g.nsw + g.mask_slots) * 4 * 4096 : 0) + kBarBlockBytes +
                      (size_t)g.bias_smem_bytes + (size_t)g.mask_smem_bytes;
  // At least 120 KB, so that two CTAs never share an SM: the second one would wait for TMEM
  // columns the first one holds.
  return std::max<size_t>(smem, 120 * 1024);
}

long long gemm_total_tiles(const GemmArgs& g) {
  const int tap_pack = std::max(g.tap_pack, 1);
  return g.a_mn ? (long long)g.n_tiles * g.tiles_w * ((g.num_taps + tap_pack - 1) / tap_pack) * g.splits
                : (long long)g.n_tiles * g.tiles_w * g.tiles_h * g.tiles_n;
}

// True if these GEMMs can share one launch: 16-bit packed epilogue of one kind, one pipeline layout
// (no CTA pairs, no fp32 split), every GEMM with work, and enough SMs to give each its column tiles.
bool multi_launchable(const GemmArgs* list, int count, int sms) {
  if (count < 2 || count > kMaxMulti) return false;
  const int epi = gemm_epilogue_kind(list[0]);
  if (select_multi_kernel(epi, list[0].out_dtype) == nullptr) return false;
  int min_ctas = 0;
  for (int i = 0; i < count; ++i) {
    const GemmArgs& g = list[i];
    if (gemm_epilogue_kind(g) != epi || g.out_dtype != list[0].out_dtype || g.cta_pair || g.a_mn) return false;
    // a GEMM without reduction steps only writes zeros: side by side it would take SMs from the ones that
    // compute and finish no sooner (measured on a strided 1x1 layer: 0.31 against 0.21 ms)
    if (g.num_taps < 1) return false;
    const long long total = gemm_total_tiles(g);
    if (total <= 0 || total > 0x7FFFFFFFll) return false;
    if (gemm_smem_bytes(g, false) > (size_t)kSmemBudget) return false;
    min_ctas += (g.b_res == 2 || g.bias_tile_only) ? g.n_tiles : 1;
  }
  return min_ctas <= sms;
}

int launch_gemm_multi(const GemmArgs* list, int count, cudaStream_t s) {
  const int sms = device_sm_count();
  const int epi = gemm_epilogue_kind(list[0]);
  GemmKernelMulti kernel = select_multi_kernel(epi, list[0].out_dtype);
  {
    static std::mutex mu;
    static bool opted_in[kMaxDevices] = {};
    const int dev = current_device();
    if (dev < 0 || dev >= kMaxDevices) return fail(PDNN_ALLOCATION_PROBLEM, "tensor-core gemm: no usable current device");
    std::lock_guard<std::mutex> lock(mu);
    if (!opted_in[dev]) {
      for (int e : {2, 3, 5})
        for (int dt : {PDNN_F16, PDNN_BF16})
          if (cudaFuncSetAttribute(select_multi_kernel(e, dt), cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget) != cudaSuccess) {
            cudaGetLastError();
            return fail(PDNN_ALLOCATION_PROBLEM, "cannot opt in to %d bytes of shared memory", kSmemBudget);
          }
      opted_in[dev] = true;
    }
  }
  // Shares of the SMs in proportion to the time each GEMM needs (tiles x cost of a tile),
  // every GEMM at least one CTA (or one per column tile where its CTAs stay on one column tile).
  static thread_local GemmArgsMulti m;  // (8 KB: kept off the stack)
  m.count = count;
  size_t smem = 0;
  double work[kMaxMulti], all_work = 0;
  int floor_ctas[kMaxMulti], share[kMaxMulti], given = 0;
  for (int i = 0; i < count; ++i) {
    m.gemm[i] = list[i];
    m.gemm[i].tap_pack = std::max(list[i].tap_pack, 1);
    m.gemm[i].wait_limit_ns = kWaitLimitNs;
    smem = std::max(smem, gemm_smem_bytes(list[i], false));
    // a tile costs its reduction steps, but never less than its epilogue and its bytes: about four steps' worth
    work[i] = (double)gemm_total_tiles(list[i]) * std::max(4, list[i].num_taps * list[i].cblocks);
    all_work += work[i];
    floor_ctas[i] = (list[i].b_res == 2 || list[i].bias_tile_only) ? list[i].n_tiles : 1;
  }
  for (int i = 0; i < count; ++i) {
    const long long total = gemm_total_tiles(list[i]);
    int want = (int)std::min<long long>(total, std::max<long long>(floor_ctas[i], (long long)(sms * work[i] / all_work)));
    want = std::max(want, floor_ctas[i]);
    if (floor_ctas[i] > 1) want -= want % floor_ctas[i];
    share[i] = want;
    given += want;
  }
  // rounding may leave SMs over or ask for too many: take from / give to the largest share
  while (given > sms) {
    int big = 0;
    for (int i = 1; i < count; ++i)
      if (share[i] - floor_ctas[i] > share[big] - floor_ctas[big]) big = i;
    const int step = floor_ctas[big] > 1 ? floor_ctas[big] : 1;
    if (share[big] - step < floor_ctas[big]) return kPlanAgain;  // (the caller launches the GEMMs one by one)
    share[big] -= step;
    given -= step;
  }
  // ... and SMs that the rounding left over go to the GEMM with the most work per CTA
  while (given < sms) {
    int best = -1;
    for (int i = 0; i < count; ++i) {
      const int step = floor_ctas[i] > 1 ? floor_ctas[i] : 1;
      if (given + step > sms || share[i] + step > gemm_total_tiles(list[i])) continue;
      if (best < 0 || work[i] / share[i] > work[best] / share[best]) best = i;
    }
    if (best < 0) break;
    const int step = floor_ctas[best] > 1 ? floor_ctas[best] : 1;
    share[best] += step;
    given += step;
  }
  m.first_cta[0] = 0;
  for (int i = 0; i < count; ++i) m.first_cta[i + 1] = m.first_cta[i] + share[i];
  for (int i = count + 1; i <= kMaxMulti; ++i) m.first_cta[i] = m.first_cta[count];
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)m.first_cta[count]);
  cfg.blockDim = dim3(384);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t le = cudaLaunchKernelEx(&cfg, kernel, m);
  if (le != cudaSuccess) {
    cudaGetLastError();
    return fail(PDNN_ALLOCATION_PROBLEM, "tensor-core gemm: launch failed: %s", cudaGetErrorString(le));
  }
  return check_launch("tensor-core gemm (several GEMMs)");
}

void set_epilogue(GemmArgs& g, const PdnnConvEpilogue* epi) {
  g.bitmask_out = nullptr;
  g.bias = nullptr;
  g.act = PDNN_ACT_NONE;
  g.alpha = 1.f;
  g.beta = 0.f;
  if (epi != nullptr) {
    g.bias = epi->bias;
    g.act = epi->activation;
    g.alpha = epi->alpha;
    g.beta = epi->beta;
    g.bitmask_out = epi->relu_bitmask;
  }
}

bool conv_common_ok(int dtype, const PdnnConv2DParams& p) {
  const int align = dtype == PDNN_F32 ? 4 : 8;
  if (p.input_format != 0 || p.groups != 1) return false;
  if (p.filter_format != 0 && p.filter_format != 2) return false;
  if (p.channels % align || p.features % align) return false;
  if (p.stride_rows < 1 || p.stride_rows > 2 || p.stride_cols < 1 || p.stride_cols > 2) return false;
  if (p.window_rows * p.window_cols > kMaxTaps) return false;
  if (p.in_cols > 32767 || p.in_rows > 32767) return false;
  return true;
}

// One tensor map per input parity of x ([C, W', H', N] view of the pixels with h % sr == ph,
// w % sc == pw).  Returns false if a parity class is empty.
// Leading dimensions, in elements, of tensors that are channel slices of wider ones (one group of a
// grouped convolution): between two pixels of x, two rows of the HWCF filter matrix, two pixels of y.
// Zero stands for the dense value (channels, features, features).
struct ConvLd {
  int x, w, y;
};

bool make_parity_maps(GemmArgs& g, int dtype, bool mn_major, const void* x, const PdnnConv2DParams& p,
                      const uint32_t box[4], int x_ld = 0) {
  const size_t es = dtype_size(dtype);
  const uint64_t ld = x_ld > 0 ? (uint64_t)x_ld : (uint64_t)p.channels;
  for (int ph = 0; ph < p.stride_rows; ++ph)
    for (int pw = 0; pw < p.stride_cols; ++pw) {
      const int Hq = ceil_div(p.in_rows - ph, p.stride_rows), Wq = ceil_div(p.in_cols - pw, p.stride_cols);
      if (Hq <= 0 || Wq <= 0) return false;
      const uint64_t dims[4] = {(uint64_t)p.channels, (uint64_t)Wq, (uint64_t)Hq, (uint64_t)p.batch};
      const uint64_t st[3] = {(uint64_t)p.stride_cols * ld * es, (uint64_t)p.stride_rows * p.in_cols * ld * es,
                              (uint64_t)p.in_rows * p.in_cols * ld * es};
      const char* base = static_cast<const char*>(x) + ((size_t)ph * p.in_cols + pw) * ld * es;
      if (!make_map(&g.a_map[ph * p.stride_cols + pw], dtype, mn_major, base, dims, st, box)) return false;
    }
  for (int i = p.stride_rows * p.stride_cols; i < 4; ++i) g.a_map[i] = g.a_map[0];
  return true;
}

// Output side of a forward convolution: y is [N, Ho, Wo, K].
// plan_out (may be null): the finished plan is stored there instead of being launched.
int finish_forward(GemmArgs& g, int dtype, void* y, const PdnnConv2DParams& p, const PdnnConvEpilogue* epi,
                   cudaStream_t s, int y_ld = 0, GemmArgs* plan_out = nullptr) {
  const size_t es = dtype_size(dtype);
  const long long ld = y_ld > 0 ? y_ld : p.features;
  set_epilogue(g, epi);
  g.out = y;
  g.out_dtype = dtype;
  g.ext_w = p.out_cols;
  g.ext_h = p.out_rows;
  g.ext_n = p.batch;
  g.ext_cols = p.features;
  g.stride_w = ld;
  g.stride_h = (long long)p.out_cols * ld;
  g.stride_n = (long long)p.out_rows * p.out_cols * ld;
  g.vec_ok = 1;
  const uint64_t od[4] = {(uint64_t)p.features, (uint64_t)p.out_cols, (uint64_t)p.out_rows, (uint64_t)p.batch};
  const uint64_t os[3] = {(uint64_t)ld * es, (uint64_t)p.out_cols * ld * es, (uint64_t)p.out_rows * p.out_cols * ld * es};
  if (!setup_store(g, dtype, od, os)) return (g.halo || g.pair) ? kPlanAgain : PDNN_INVALID_PARAMETER;
  if (plan_out != nullptr) {
    *plan_out = g;
    return PDNN_OK;
  }
  return launch_gemm(g, dtype, s);
}

// ---- forward convolution for very few input channels (network stems) ---------------------------
// With C < 8 (16-bit) or C < 4 (fp32) a pixel is narrower than the 16-byte unit TMA needs, and a
// 64-element reduction step per tap would be mostly padding.  Instead the input is first copied
// into a zero-padded tensor with CP = 8 (4) channels per pixel and explicit spatial padding; one
// 128-byte row then holds 8 consecutive pixels, i.e. a whole filter row (S <= 8) of one output
// pixel, and the tensor map walks output pixels with a stride of stride_cols pixels, so rows
// overlap.  The reduction runs over filter rows: R steps of 64 (32) elements.  The filter is
// repacked the same way ([R][8][CP][K], zeros in the padding).
// One thread per packed pixel; the grid is (row segments, padded rows, images), so no thread divides.
template <typename T>
__global__ void __launch_bounds__(256) pack_small_c_input_kernel(const T* __restrict__ x, uint4* __restrict__ xp, int N,
                                                                int H, int W, int C, int Hp, int Wp, int pad_top,
                                                                int pad_left) {
  constexpr int CP = 16 / sizeof(T);
  const int wp = (int)(blockIdx.x * 256u + threadIdx.x), hp = (int)blockIdx.y, n = (int)blockIdx.z;
  if (wp >= Wp) return;
  const int h = hp - pad_top, w = wp - pad_left;
  Vec16<T> pk;
  pk.raw = make_uint4(0u, 0u, 0u, 0u);
  if (h >= 0 && h < H && w >= 0 && w < W) {
    const T* src = x + (((size_t)n * H + h) * W + w) * C;
    for (int c = 0; c < C && c < CP; ++c) pk.set(c, src[c]);
  }
  xp[((size_t)n * Hp + hp) * Wp + wp] = pk.raw;
}

// The same with 4 channels of 16 bits per pixel (8 bytes): half the bytes for a 3-channel image.
__global__ void __launch_bounds__(256) pack_small_c_input_narrow_kernel(const unsigned short* __restrict__ x,
                                                                       uint2* __restrict__ xp, int N, int H, int W,
                                                                       int C, int Hp, int Wp, int pad_top,
                                                                       int pad_left) {
  const int wp = (int)(blockIdx.x * 256u + threadIdx.x), hp = (int)blockIdx.y, n = (int)blockIdx.z;
  if (wp >= Wp) return;
  const int h = hp - pad_top, w = wp - pad_left;
  unsigned v[4] = {0u, 0u, 0u, 0u};
  if (h >= 0 && h < H && w >= 0 && w < W) {
    const unsigned short* src = x + (((size_t)n * H + h) * W + w) * C;
    for (int c = 0; c < C && c < 4; ++c) v[c] = src[c];
  }
  xp[((size_t)n * Hp + hp) * Wp + wp] = make_uint2(v[0] | (v[1] << 16), v[2] | (v[3] << 16));
}

// Filter [R][S][C][K] -> [R][8][CP][K], zeros for s >= S and c >= C.
template <typename T>
__global__ void __launch_bounds__(256) pack_small_c_filter_kernel(const T* __restrict__ w, T* __restrict__ wp, int R,
                                                                 int S, int C, int K, int CP) {
  const size_t total = (size_t)R * 8 * CP * K;
  for (size_t idx = (size_t)blockIdx.x * 256 + threadIdx.x; idx < total; idx += (size_t)gridDim.x * 256) {
    const int k = (int)(idx % K);
    size_t t = idx / K;
    const int c = (int)(t % CP);
    t /= CP;
    const int sidx = (int)(t % 8);
    const int r = (int)(t / 8);
    wp[idx] = (sidx < S && c < C) ? w[(((size_t)r * S + sidx) * C + c) * K + k] : from_f32<T>(0.f);
  }
}

bool small_c_applicable(int dtype, const PdnnConv2DParams& p) {
  const int cp = 16 / (int)dtype_size(dtype);
  return p.input_format == 0 && p.filter_format == 0 && p.groups == 1 && p.channels < cp && p.window_cols <= 8 &&
         p.window_rows <= kMaxTaps && p.stride_rows <= 4 && p.stride_cols <= 4 && p.features % cp == 0 &&
         p.batch <= 65535 && (p.out_rows - 1) * p.stride_rows + p.window_rows <= 65535;  // the repack's grid
}

struct SmallCPlan {
  int Hp, Wp;
  size_t xp_bytes, wp_bytes;
};

SmallCPlan plan_small_c(int dtype, const PdnnConv2DParams& p) {
  SmallCPlan sp;
  const size_t es = dtype_size(dtype);
  sp.Hp = (p.out_rows - 1) * p.stride_rows + p.window_rows;
  sp.Wp = (p.out_cols - 1) * p.stride_cols + 8;
  sp.xp_bytes = (((size_t)p.batch * sp.Hp * sp.Wp * 16) + 255) / 256 * 256;
  sp.wp_bytes = (((size_t)p.window_rows * 8 * (16 / es) * p.features * es) + 255) / 256 * 256;
  return sp;
}

// Returns PDNN_OK, an error, or -1 if the tensor maps could not be encoded (the caller then uses
// the direct kernel).
int conv_forward_small_c(int dtype, const void* x, const void* w, void* y, const PdnnConv2DParams& p,
                         const PdnnConvEpilogue* epi, void* ws, size_t ws_elems, cudaStream_t s, bool try_halo = true) {
  const size_t es = dtype_size(dtype);
  const int sms = device_sm_count();
  const int epr = dtype == PDNN_F32 ? 32 : 64;
  const SmallCPlan sp = plan_small_c(dtype, p);
  const size_t need = sp.xp_bytes + sp.wp_bytes;
  char* scratch = static_cast<char*>(ws);
  bool own = false;
  if (scratch == nullptr || ws_elems * es < need || ((uintptr_t)scratch & 255u)) {
    if (cudaMallocAsync(reinterpret_cast<void**>(&scratch), need, s) != cudaSuccess) {
      cudaGetLastError();
      return fail(PDNN_ALLOCATION_PROBLEM, "conv2d: cannot allocate %zu bytes of scratch for the packed input", need);
    }
    own = true;
  }
  char* xp = scratch;
  char* wpk = scratch + sp.xp_bytes;
  auto release = [&] {
    if (own) cudaFreeAsync(scratch, s);
  };

  GemmArgs g;
  std::memset(&g, 0, sizeof(g));
  g.a_mn = 0;
  // Filter rows of the same input-row parity read overlapping input rows: in halo mode each
  // parity class is one reduction step over one copy.
  const int rows_per_class = ceil_div(p.window_rows, p.stride_rows);
  int hw = 0, hh = 0;
  const bool halo = try_halo && dtype != PDNN_F32 && rows_per_class >= 2 && rows_per_class <= 15 &&
                    p.stride_rows <= 8 && p.window_rows >= p.stride_rows && choose_box_halo(p.out_cols, p.out_rows, rows_per_class, &hw, &hh);
  if (halo) {
    g.tw = hw;
    g.th = hh;
    g.tn = 1;
  } else {
    choose_box(kTileM, p.out_cols, p.out_rows, p.batch, &g.tw, &g.th, &g.tn);
  }
  g.etw = g.tw;
  g.eth = g.th;
  g.etn = g.tn;
  g.tiles_w = ceil_div(p.out_cols, g.tw);
  g.tiles_h = ceil_div(p.out_rows, g.th);
  g.tiles_n = ceil_div(p.batch, g.tn);
  g.bn = pick_bn((long long)g.tiles_w * g.tiles_h * g.tiles_n, p.features, epr, dtype == PDNN_F32 ? 128 : 256, sms);
  g.n_tiles = ceil_div(p.features, g.bn);
  set_operand_layout(g, dtype, 1);
  // Narrow layout (16-bit, at most 4 channels, even column stride, halo mode): 4 channels per pixel,
  // so a filter row of 8 pixels is 64 bytes and a reduction step is two MMAs instead of four, with
  // half the bytes to pack, load and multiply.  The tiles are 64-byte rows with the 64-byte
  // swizzle; a pixel step of stride_cols * 8 bytes is still a multiple of TMA's 16 bytes.
  const bool narrow = halo && p.channels <= 4 && p.stride_cols % 2 == 0 &&
                      (size_t)p.batch * sp.Hp * (sp.Wp + 1) < 0x7FFFFFFFull;
  const int pix_bytes = narrow ? 8 : 16;
  const int krows = narrow ? 32 : epr;            // reduction elements per step
  const int Wp = narrow ? (sp.Wp + 1) / 2 * 2 : sp.Wp;  // narrow: rows stay 16-byte aligned
  if (narrow) {
    g.a_row_bytes = 64;
    g.kmmas = 2;
    g.a_sbo = 512;   // 8 rows of 64 bytes
    g.a_layout = 4;  // 64-byte swizzle
    g.b_lbo = (unsigned)krows * 128u;
    g.b_box_bytes = (unsigned)krows * 128u;
    g.b_step_bytes = (unsigned)g.bn * 64u;
  }
  const size_t row_pitch = (size_t)Wp * pix_bytes;
  for (int q = 0; q < p.stride_rows; ++q) {
    const int Hq = ceil_div(sp.Hp - q, p.stride_rows);
    const uint64_t dims[4] = {(uint64_t)krows, (uint64_t)p.out_cols, (uint64_t)std::max(Hq, 1), (uint64_t)p.batch};
    const uint64_t st[3] = {(uint64_t)p.stride_cols * pix_bytes, (uint64_t)p.stride_rows * row_pitch,
                            (uint64_t)sp.Hp * row_pitch};
    // filter rows q, q + stride, ... read this parity class
    const int cnt = (p.window_rows - q + p.stride_rows - 1) / p.stride_rows;
    const uint32_t box[4] = {(uint32_t)krows, (uint32_t)g.tw, (uint32_t)(halo ? g.th + cnt - 1 : g.th), (uint32_t)g.tn};
    if (!make_map(&g.a_map[q], dtype, false, xp + (size_t)q * row_pitch, dims, st, box, narrow)) {
      release();
      return -1;
    }
  }
  for (int q = p.stride_rows; q < 4; ++q) g.a_map[q] = g.a_map[0];
  if (halo) {
    g.halo = 1;
    g.res_taps = p.window_rows;
    unsigned widest = 0;
    for (int q = 0; q < p.stride_rows; ++q) {
      const int cnt = (p.window_rows - q + p.stride_rows - 1) / p.stride_rows;
      g.taps[q] = TapEntry{0, 0, (short)q, (short)q, (short)cnt, (short)p.stride_rows};
      widest = std::max(widest, (unsigned)(g.tw * (g.th + cnt - 1) * g.a_row_bytes));
    }
    g.num_taps = p.stride_rows;
    g.halo_stage_bytes = (widest + 1023u) & ~1023u;
  } else {
    for (int r = 0; r < p.window_rows; ++r)
      g.taps[r] = TapEntry{0, (short)(r / p.stride_rows), (short)(r % p.stride_rows), (short)r, 1, 0};
    g.num_taps = p.window_rows;
  }
  g.cblocks = 1;
  {
    g.b_mode = B_MN_3;
    const uint64_t dims[4] = {(uint64_t)p.features, (uint64_t)krows, (uint64_t)p.window_rows, 1};
    const uint64_t st[3] = {(uint64_t)p.features * es, (uint64_t)krows * p.features * es,
                            (uint64_t)p.window_rows * krows * p.features * es};
    const uint32_t box[4] = {(uint32_t)epr, (uint32_t)krows, 1, 1};
    if (!make_map(&g.b_map, dtype, true, wpk, dims, st, box)) {
      release();
      return -1;
    }
  }
  const size_t n_fil = (size_t)p.window_rows * krows * p.features;
  if (dtype == PDNN_F32) {
    pack_small_c_input_kernel<float><<<dim3((unsigned)ceil_div(sp.Wp, 256), (unsigned)sp.Hp, (unsigned)p.batch), 256, 0, s>>>(
        static_cast<const float*>(x), reinterpret_cast<uint4*>(xp), p.batch, p.in_rows, p.in_cols, p.channels, sp.Hp,
        sp.Wp, p.pad_rows, p.pad_cols);
    pack_small_c_filter_kernel<float><<<grid_for(n_fil, 256, sms), 256, 0, s>>>(
        static_cast<const float*>(w), reinterpret_cast<float*>(wpk), p.window_rows, p.window_cols, p.channels, p.features, 4);
  } else {
    // fp16 and bf16 are both moved as 16-bit words
    if (narrow)
      pack_small_c_input_narrow_kernel<<<dim3((unsigned)ceil_div(Wp, 256), (unsigned)sp.Hp, (unsigned)p.batch), 256, 0, s>>>(
          static_cast<const unsigned short*>(x), reinterpret_cast<uint2*>(xp), p.batch, p.in_rows, p.in_cols, p.channels,
          sp.Hp, Wp, p.pad_rows, p.pad_cols);
    else
      pack_small_c_input_kernel<__half><<<dim3((unsigned)ceil_div(sp.Wp, 256), (unsigned)sp.Hp, (unsigned)p.batch), 256, 0, s>>>(
          static_cast<const __half*>(x), reinterpret_cast<uint4*>(xp), p.batch, p.in_rows, p.in_cols, p.channels, sp.Hp,
          sp.Wp, p.pad_rows, p.pad_cols);
    pack_small_c_filter_kernel<__half><<<grid_for(n_fil, 256, sms), 256, 0, s>>>(
        static_cast<const __half*>(w), reinterpret_cast<__half*>(wpk), p.window_rows, p.window_cols, p.channels, p.features,
        narrow ? 4 : 8);
  }
  int st = check_launch("conv2d small-channel packing");
  count_launch();
  if (st == PDNN_OK) st = finish_forward(g, dtype, y, p, epi, s);
  release();
  if (st == kPlanAgain) return conv_forward_small_c(dtype, x, w, y, p, epi, ws, ws_elems, s, false);
  return st;
}

// The lo part of a 3xTF32 operand: the tensor core reads the 19 leading bits of an fp32 word (hi, which
// therefore needs no copy); lo = x - hi is exact in fp32.
__global__ void __launch_bounds__(256) split_lo_kernel(const float* __restrict__ x, float* __restrict__ lo, size_t n) {
  for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (size_t)gridDim.x * 256) {
    const float v = x[i];
    lo[i] = v - __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
  }
}

int conv_forward(int dtype, const void* x, const void* w, void* y, const PdnnConv2DParams& p,
                 const PdnnConvEpilogue* epi, cudaStream_t s, bool try_halo = true, bool try_cta_pair = true,
                 const ConvLd* ld = nullptr, GemmArgs* plan_out = nullptr) {
  if (plan_out != nullptr && dtype == PDNN_F32) return PDNN_INVALID_PARAMETER;  // (the fp32 plan owns scratch)
  const int x_ld = ld != nullptr ? ld->x : 0, y_ld = ld != nullptr ? ld->y : 0;
  const uint64_t w_ld = ld != nullptr && ld->w > 0 ? (uint64_t)ld->w : (uint64_t)p.features;
  GemmArgs g;
  std::memset(&g, 0, sizeof(g));
  const size_t es = dtype_size(dtype);
  const int sms = device_sm_count();
  g.a_mn = 0;
  const bool hwcf = p.filter_format == 0;
  const int epr = dtype == PDNN_F32 ? 32 : 64;
  // Stride-1 windows of two or more rows: the taps of one window column read overlapping input
  // rows, so each column becomes one reduction step over one copy (halo mode), provided the whole
  // filter can stay in shared memory.
  int hw = 0, hh = 0;
  const bool halo = try_halo && dtype != PDNN_F32 && p.stride_rows == 1 && p.stride_cols == 1 &&
                    p.window_rows >= 2 && p.window_rows <= 15 && p.window_cols <= 8 &&
                    (size_t)p.window_rows * p.window_cols * ceil_div(p.channels, epr) * 128u *
                            (size_t)(ceil_div(p.features, 64) * 64) <= kMaxResidentB &&
                    choose_box_halo(p.out_cols, p.out_rows, p.window_rows, &hw, &hh);
  if (halo) {
    g.tw = hw;
    g.th = hh;
    g.tn = 1;
  } else {
    choose_box(kTileM, p.out_cols, p.out_rows, p.batch, &g.tw, &g.th, &g.tn);
  }
  g.etw = g.tw;
  g.eth = g.th;
  g.etn = g.tn;
  g.tiles_w = ceil_div(p.out_cols, g.tw);
  g.tiles_h = ceil_div(p.out_rows, g.th);
  g.tiles_n = ceil_div(p.batch, g.tn);
  const long long row_tiles = (long long)g.tiles_w * g.tiles_h * g.tiles_n;
  const int ksteps_all = p.window_rows * p.window_cols * ceil_div(p.channels, epr);
  // Long reductions over filters too large to keep in shared memory are bound by the bytes that
  // pass through an SM's shared memory per MMA (the operand reads of the tensor core and the TMA
  // fills share its 128 bytes per cycle): the two pipelines then share one B tile per stage (pair
  // mode).  Measured on ResNet-50 shapes it pays from 16 reduction steps on for filters of 128
  // features and from 32 on for wider ones (which
  // do better as single 256-column tiles on one double-buffered pipeline until then), provided the
  // pairs still fill the device: a grid of fewer pair tiles than SMs leaves SMs idle that single
  // tiles would use.
  const int pair_bn_auto = (p.features % 256 == 0 && p.features >= 512) ? 256 : 128;
  const bool pair_auto = ksteps_all >= (p.features >= 256 ? 32 : 16) &&
                         (row_tiles / 2) * ceil_div(p.features, pair_bn_auto) >= sms;
  const bool pairing = try_halo && !halo && dtype != PDNN_F32 && hwcf && p.features % 128 == 0 && pair_auto &&
                       row_tiles >= 2 && (!epi || epi->beta == 0.f);
  // Pairs of row tiles with 256 columns go to clusters of two CTAs (umma_gemm_pair2_kernel) when the
  // epilogue is the plain packed one: half the B operand reads per SM, double-buffered accumulators.
  // Measured on the ResNet-50 shapes: 3x3 layers gain 10-18 % (256 at 14x14: 0.0558 -> 0.0496 ms); 1x1
  // layers, whose tiles are short, lose 6-10 % against two pipelines per CTA and stay there.
  const bool cta_pair = try_cta_pair && pairing && p.features % 256 == 0 && sms % 2 == 0 &&
                        p.window_rows * p.window_cols > 1 && (row_tiles / 2) * (p.features / 256) >= sms / 2;
  if (pairing) {
    g.pair = 1;
    g.cta_pair = cta_pair ? 1 : 0;
    // 128-column tiles leave room for two accumulator buffers per pipeline; narrow filters use them
    g.bn = cta_pair ? 256 : pair_bn_auto;
    if (g.tiles_w % 2 == 0) {
      g.pair_dim = 1;
      g.tiles_w /= 2;
    } else if (g.tiles_h % 2 == 0) {
      g.pair_dim = 2;
      g.tiles_h /= 2;
    } else {
      g.pair_dim = 3;  // an odd count leaves the last pair half empty: loads read zeros, stores are clipped
      g.tiles_n = ceil_div(g.tiles_n, 2);
    }
  } else {
    g.bn = pick_bn(row_tiles, p.features, hwcf ? epr : 16, dtype == PDNN_F32 ? 128 : 256, sms, ksteps_all);
    // A single tap with a long reduction into exactly 256 features: one 256-column tile per row tile
    // reads the input once instead of twice and runs as one double-buffered pipeline (measured 12%
    // faster than two 128-column pipelines on 14x14x1024 -> 256).
    if (dtype != PDNN_F32 && !halo && p.window_rows * p.window_cols == 1 &&
        ksteps_all >= 16 && p.features == 256 && row_tiles >= 2 * sms)
      g.bn = 256;
    // One or two reduction steps over pixels narrower than 64 bytes (MobileNet-v2's 24 -> 144 expansions):
    // with two column tiles the input tile is fetched twice, and fetching such short rows is what the layer
    // spends its time on; one wide tile reads it once (measured 0.053 -> 0.035 ms on 56x56x24 -> 144; layers
    // with 32 and more channels do not care, 64 -> 256 is 2% better with two tiles).
    if (dtype != PDNN_F32 && !halo && ksteps_all <= 2 && p.features > 128 && p.features <= 256 && p.channels * es < 64)
      g.bn = ceil_div(p.features, 64) * 64;
  }
  g.n_tiles = ceil_div(p.features, g.bn);
  set_operand_layout(g, dtype, hwcf ? 1 : 0);
  if (g.cta_pair)  // MMAs of 256 rows (128 per CTA) x 256 columns
    g.idesc = make_idesc(dtype == PDNN_BF16 ? 1 : 0, 0, 1, 256, 256);
  const uint32_t abox[4] = {(uint32_t)epr, (uint32_t)g.tw, (uint32_t)(halo ? g.th + p.window_rows - 1 : g.th),
                            (uint32_t)g.tn};
  g.early_b = (epi != nullptr && epi->constant_filter != 0 && dtype != PDNN_F32) ? 1 : 0;
  if (!make_parity_maps(g, dtype, false, x, p, abox, x_ld)) return PDNN_INVALID_PARAMETER;
  // taps
  int nt = 0;
  if (halo) {
    g.halo = 1;
    g.res_taps = p.window_rows * p.window_cols;
    g.halo_stage_bytes = ((unsigned)(g.tw * (g.th + p.window_rows - 1) * 128) + 1023u) & ~1023u;
    for (int c = 0; c < p.window_cols; ++c)  // window column c: rows 0 .. R-1 of the filter, taps c, c + S, ...
      g.taps[nt++] = TapEntry{(short)(c - p.pad_cols), (short)(-p.pad_rows), 0, (short)c, (short)p.window_rows,
                              (short)p.window_cols};
  } else {
    for (int r = 0; r < p.window_rows; ++r)
      for (int c = 0; c < p.window_cols; ++c) {
        const int hh = r - p.pad_rows, ww = c - p.pad_cols;
        TapEntry e;
        e.dh = (short)floor_div(hh, p.stride_rows);
        e.dw = (short)floor_div(ww, p.stride_cols);
        e.a_map = (short)(pos_mod(hh, p.stride_rows) * p.stride_cols + pos_mod(ww, p.stride_cols));
        e.b_tap = (short)(r * p.window_cols + c);
        e.cnt = 1;
        e.b_step = 0;
        g.taps[nt++] = e;
      }
  }
  g.num_taps = nt;
  g.cblocks = ceil_div(p.channels, epr);
  const uint64_t taps = (uint64_t)p.window_rows * p.window_cols;
  // fp32 (3xTF32) with enough work to pay for one extra pass over the filter: the lo part of the filter
  // is computed once, ahead of the GEMM, and arrives by TMA like the filter itself (whose words serve as
  // the hi part); the kernel's split warps then only have the A tiles to split.
  const size_t filter_elems = (size_t)taps * p.channels * p.features;
  float* w_split = nullptr;
  if (dtype == PDNN_F32 && (size_t)p.batch * p.out_rows * p.out_cols >= 2048 && aligned16(w) &&
      (!hwcf || w_ld == (uint64_t)p.features)) {  // (a column slice of a wider filter is not one contiguous run)
    if (cudaMallocAsync(reinterpret_cast<void**>(&w_split), filter_elems * sizeof(float), s) == cudaSuccess) {
      split_lo_kernel<<<grid_for(filter_elems, 256, sms), 256, 0, s>>>(static_cast<const float*>(w), w_split, filter_elems);
      count_launch();
      g.b_presplit = 1;
    } else {
      cudaGetLastError();
      w_split = nullptr;
    }
  }
  auto make_b_map = [&](CUtensorMap* map, const void* base) {
    if (hwcf && p.features % epr == 0) {
      // All 128-byte column blocks of the tile in one copy: the block index is a tensor dimension
      // of its own (stride 128 bytes), placed after the reduction rows so that the blocks land
      // one after another in shared memory.
      g.b_mode = B_MN_3X;
      const uint64_t dims[4] = {(uint64_t)epr, (uint64_t)p.channels, (uint64_t)(p.features / epr), taps};
      const uint64_t st[3] = {w_ld * es, 128, (uint64_t)p.channels * w_ld * es};
      // (a CTA pair: each CTA copies its own half of the tile's columns)
      const uint32_t box[4] = {(uint32_t)epr, (uint32_t)epr, (uint32_t)((g.cta_pair ? g.bn / 2 : g.bn) / epr), 1};
      return make_map(map, dtype, true, base, dims, st, box);
    }
    if (hwcf) {
      g.b_mode = B_MN_3;
      const uint64_t dims[4] = {(uint64_t)p.features, (uint64_t)p.channels, taps, 1};
      const uint64_t st[3] = {w_ld * es, (uint64_t)p.channels * w_ld * es, taps * p.channels * w_ld * es};
      const uint32_t box[4] = {(uint32_t)epr, (uint32_t)epr, 1, 1};
      return make_map(map, dtype, true, base, dims, st, box);
    }
    g.b_mode = B_K_FHWC;
    const uint64_t dims[4] = {(uint64_t)p.channels, taps, (uint64_t)p.features, 1};
    const uint64_t st[3] = {(uint64_t)p.channels * es, taps * p.channels * es, taps * p.channels * p.features * es};
    const uint32_t box[4] = {(uint32_t)epr, 1, (uint32_t)g.bn, 1};
    return make_map(map, dtype, false, base, dims, st, box);
  };
  const bool maps_ok = make_b_map(&g.b_map, w) && (w_split == nullptr || make_b_map(&g.b_map_lo, w_split));
  if (!maps_ok) {
    if (w_split != nullptr) cudaFreeAsync(w_split, s);
    return PDNN_INVALID_PARAMETER;
  }
  const int status = finish_forward(g, dtype, y, p, epi, s, y_ld, plan_out);
  if (w_split != nullptr) cudaFreeAsync(w_split, s);
  if (status == kPlanAgain)  // first without the CTA pairs, then without halo / pair mode
    return g.cta_pair ? conv_forward(dtype, x, w, y, p, epi, s, try_halo, false, ld, plan_out)
                      : conv_forward(dtype, x, w, y, p, epi, s, false, false, ld, plan_out);
  return status;
}

// relu_mask (may be null): the forward output of the layer that produced the tensor dx is the gradient
// of; dx is zeroed wherever it is not positive (in the epilogue where the fast epilogue runs, else
// by a pointwise pass afterwards).
// accumulate: 0 dx = result; 1 dx += result (the mask then applies to the sum); 2 as 1 where dx already
// carries the same mask, so that positions this convolution does not reach (parity classes without a
// tap) are left as they are.
int conv_input_backprop(int dtype, const void* dy, const void* w, void* dx, const PdnnConv2DParams& p,
                        const void* relu_mask, const void* mask_bits, int accumulate, bool constant_filter, cudaStream_t s,
                        bool try_halo = true) {
  bool mask_pending = false;  // some parity class could not apply the mask in its epilogue
  const size_t es = dtype_size(dtype);
  const int sms = device_sm_count();
  const bool hwcf = p.filter_format == 0;
  const int epr = dtype == PDNN_F32 ? 32 : 64;
  // fp32: the lo part of the filter computed ahead of the GEMMs, as in the forward pass
  const size_t filter_elems = (size_t)p.window_rows * p.window_cols * p.channels * p.features;
  float* w_split = nullptr;
  if (dtype == PDNN_F32 && (size_t)p.batch * p.in_rows * p.in_cols >= 2048 && aligned16(w) &&
      cudaMallocAsync(reinterpret_cast<void**>(&w_split), filter_elems * sizeof(float), s) == cudaSuccess) {
    split_lo_kernel<<<grid_for(filter_elems, 256, sms), 256, 0, s>>>(static_cast<const float*>(w), w_split, filter_elems);
    count_launch();
  } else if (dtype == PDNN_F32) {
    cudaGetLastError();
    w_split = nullptr;
  }
  struct Release {
    float* ptr;
    cudaStream_t s;
    ~Release() {
      if (ptr != nullptr) cudaFreeAsync(ptr, s);
    }
  } release{w_split, s};

  // dx is produced one output parity class at a time: positions h = sr*i + qh, w = sc*j + qw only
  // receive taps with r = (qh + pad) mod sr, s = (qw + pad) mod sc, and within a class the
  // relation between i and the dy row is a plain shift.
  std::vector<GemmArgs> planned_classes;
  for (int qh = 0; qh < p.stride_rows; ++qh)
    for (int qw = 0; qw < p.stride_cols; ++qw) {
      const int Hq = ceil_div(p.in_rows - qh, p.stride_rows), Wq = ceil_div(p.in_cols - qw, p.stride_cols);
      if (Hq <= 0 || Wq <= 0) continue;
      GemmArgs g;
      std::memset(&g, 0, sizeof(g));
      g.a_mn = 0;
      g.early_b = (constant_filter && dtype != PDNN_F32) ? 1 : 0;
      // Stride 1: the taps of one window column read overlapping rows of dy, as in the forward
      // pass (halo mode), if the whole filter can stay in shared memory.
      int hw = 0, hh = 0;
      const bool halo = try_halo && dtype != PDNN_F32 && p.stride_rows == 1 && p.stride_cols == 1 &&
                        p.window_rows >= 2 && p.window_rows <= 15 && p.window_cols <= 8 &&
                        (size_t)p.window_rows * p.window_cols * ceil_div(p.features, epr) * 128u *
                                (size_t)(ceil_div(p.channels, 64) * 64) <= kMaxResidentB &&
                        choose_box_halo(Wq, Hq, p.window_rows, &hw, &hh);
      if (halo) {
        g.tw = hw;
        g.th = hh;
        g.tn = 1;
      } else {
        choose_box(kTileM, Wq, Hq, p.batch, &g.tw, &g.th, &g.tn);
      }
      g.etw = g.tw;
      g.eth = g.th;
      g.etn = g.tn;
      g.tiles_w = ceil_div(Wq, g.tw);
      g.tiles_h = ceil_div(Hq, g.th);
      g.tiles_n = ceil_div(p.batch, g.tn);
      const long long row_tiles = (long long)g.tiles_w * g.tiles_h * g.tiles_n;
      // Reduction steps of this parity class: the taps that reach it, times the feature blocks.
      int class_taps = 0;
      for (int r = 0; r < p.window_rows; ++r)
        for (int c = 0; c < p.window_cols; ++c)
          if (pos_mod(qh + p.pad_rows - r, p.stride_rows) == 0 && pos_mod(qw + p.pad_cols - c, p.stride_cols) == 0) ++class_taps;
      if (class_taps == 0 && accumulate == 2) continue;  // nothing to add, and what is there is masked already
      const int ksteps_all = class_taps * ceil_div(p.features, epr);
      // Pair mode as in the forward pass (two row tiles share the filter tile of a stage); the output
      // columns are the channels here.
      // 128-column tiles throughout (the epilogue of this pass is the longer one when it applies the
      // ReLU mask, and two accumulator buffers hide it), pairs from 16 reduction steps on.
      const int pair_bn_auto = 128;
      const bool pair_auto = ksteps_all >= 16 && (row_tiles / 2) * ceil_div(p.channels, pair_bn_auto) >= sms;
      const bool pairing = try_halo && !halo && dtype != PDNN_F32 && hwcf && p.channels % 128 == 0 && row_tiles >= 2 &&
                           pair_auto;
      if (pairing) {
        g.pair = 1;
        g.bn = pair_bn_auto;
        if (g.tiles_w % 2 == 0) {
          g.pair_dim = 1;
          g.tiles_w /= 2;
        } else if (g.tiles_h % 2 == 0) {
          g.pair_dim = 2;
          g.tiles_h /= 2;
        } else {
          g.pair_dim = 3;
          g.tiles_n = ceil_div(g.tiles_n, 2);
        }
      } else {
        g.bn = pick_bn(row_tiles, p.channels, hwcf ? 16 : epr, 128, sms, ksteps_all);
      }
      g.n_tiles = ceil_div(p.channels, g.bn);
      set_operand_layout(g, dtype, hwcf ? 0 : 1);
      {
        const uint64_t dims[4] = {(uint64_t)p.features, (uint64_t)p.out_cols, (uint64_t)p.out_rows, (uint64_t)p.batch};
        const uint64_t st[3] = {(uint64_t)p.features * es, (uint64_t)p.out_cols * p.features * es,
                                (uint64_t)p.out_rows * p.out_cols * p.features * es};
        const uint32_t box[4] = {(uint32_t)epr, (uint32_t)g.tw, (uint32_t)(halo ? g.th + p.window_rows - 1 : g.th),
                                 (uint32_t)g.tn};
        if (!make_map(&g.a_map[0], dtype, false, dy, dims, st, box)) return PDNN_INVALID_PARAMETER;
        for (int i = 1; i < 4; ++i) g.a_map[i] = g.a_map[0];
      }
      int nt = 0;
      if (halo) {
        // window column c: filter rows R-1 .. 0 read dy rows pad - (R-1) .. pad, in that order
        g.halo = 1;
        g.res_taps = p.window_rows * p.window_cols;
        g.halo_stage_bytes = ((unsigned)(g.tw * (g.th + p.window_rows - 1) * 128) + 1023u) & ~1023u;
        for (int c = 0; c < p.window_cols; ++c)
          g.taps[nt++] = TapEntry{(short)(p.pad_cols - c), (short)(p.pad_rows - (p.window_rows - 1)), 0,
                                  (short)((p.window_rows - 1) * p.window_cols + c), (short)p.window_rows,
                                  (short)(-p.window_cols)};
      }
      for (int r = 0; r < p.window_rows && !halo; ++r) {
        const int th = qh + p.pad_rows - r;
        if (pos_mod(th, p.stride_rows) != 0) continue;
        for (int c = 0; c < p.window_cols; ++c) {
          const int tw = qw + p.pad_cols - c;
          if (pos_mod(tw, p.stride_cols) != 0) continue;
          TapEntry e;
          e.dh = (short)floor_div(th, p.stride_rows);
          e.dw = (short)floor_div(tw, p.stride_cols);
          e.a_map = 0;
          e.b_tap = (short)(r * p.window_cols + c);
          e.cnt = 1;
          e.b_step = 0;
          g.taps[nt++] = e;
        }
      }
      g.num_taps = nt;
      g.cblocks = ceil_div(p.features, epr);
      const uint64_t taps = (uint64_t)p.window_rows * p.window_cols;
      if (hwcf) {
        g.b_mode = B_K_3;
        const uint64_t dims[4] = {(uint64_t)p.features, (uint64_t)p.channels, taps, 1};
        const uint64_t st[3] = {(uint64_t)p.features * es, (uint64_t)p.channels * p.features * es,
                                taps * p.channels * p.features * es};
        const uint32_t box[4] = {(uint32_t)epr, (uint32_t)g.bn, 1, 1};
        if (!make_map(&g.b_map, dtype, false, w, dims, st, box)) return PDNN_INVALID_PARAMETER;
        if (w_split != nullptr && !make_map(&g.b_map_lo, dtype, false, w_split, dims, st, box))
          return PDNN_INVALID_PARAMETER;
      } else {
        g.b_mode = B_MN_FHWC;
        const uint64_t dims[4] = {(uint64_t)p.channels, taps, (uint64_t)p.features, 1};
        const uint64_t st[3] = {(uint64_t)p.channels * es, taps * p.channels * es, taps * p.channels * p.features * es};
        const uint32_t box[4] = {(uint32_t)epr, 1, (uint32_t)epr, 1};
        if (!make_map(&g.b_map, dtype, true, w, dims, st, box)) return PDNN_INVALID_PARAMETER;
        if (w_split != nullptr && !make_map(&g.b_map_lo, dtype, true, w_split, dims, st, box))
          return PDNN_INVALID_PARAMETER;
      }
      g.b_presplit = w_split != nullptr ? 1 : 0;
      set_epilogue(g, nullptr);
      g.relu_mask = (relu_mask != nullptr && !mask_pending && aligned16(relu_mask))
                        ? static_cast<const char*>(relu_mask) + ((size_t)qh * p.in_cols + qw) * p.channels * es
                        : nullptr;
      if (mask_bits != nullptr && !mask_pending && p.channels % 64 == 0 && ((uintptr_t)mask_bits & 7u) == 0) {
        // the mask as one bit per element: the class's first pixel starts ((qh * W + qw) * C) / 8 bytes in
        g.mask_bits = static_cast<const char*>(mask_bits) + ((size_t)qh * p.in_cols + qw) * p.channels / 8;
        g.relu_mask = g.mask_bits;  // "a mask is applied in the epilogue"
      }
      g.out = static_cast<char*>(dx) + ((size_t)qh * p.in_cols + qw) * p.channels * es;
      g.out_dtype = dtype;
      g.ext_w = Wq;
      g.ext_h = Hq;
      g.ext_n = p.batch;
      g.ext_cols = p.channels;
      g.stride_w = (long long)p.stride_cols * p.channels;
      g.stride_h = (long long)p.stride_rows * p.in_cols * p.channels;
      g.stride_n = (long long)p.in_rows * p.in_cols * p.channels;
      g.vec_ok = 1;
      {
        const uint64_t od[4] = {(uint64_t)p.channels, (uint64_t)Wq, (uint64_t)Hq, (uint64_t)p.batch};
        const uint64_t os[3] = {(uint64_t)p.stride_cols * p.channels * es,
                                (uint64_t)p.stride_rows * p.in_cols * p.channels * es,
                                (uint64_t)p.in_rows * p.in_cols * p.channels * es};
        // Accumulating form (dx += ...): inside the packed 16-bit epilogue when that runs, else through
        // the general epilogue's beta.
        g.accumulate = accumulate ? 1 : 0;
        bool planned = setup_store(g, dtype, od, os);
        if (planned && accumulate && !g.epi_fast) {
          g.accumulate = 0;
          g.beta = 1.f;
          planned = setup_store(g, dtype, od, os);
        }
        if (!planned) {
          if (g.halo || g.pair) return conv_input_backprop(dtype, dy, w, dx, p, relu_mask, mask_bits, accumulate, constant_filter, s, false);  // plan again without the halo / pairing
          return PDNN_INVALID_PARAMETER;
        }
      }
      if ((relu_mask != nullptr || mask_bits != nullptr) && g.relu_mask == nullptr) {
        // An earlier class may already have masked its pixels; masking them again changes nothing.
        mask_pending = true;
      }
      planned_classes.push_back(g);
    }
  // The classes of a strided layer write disjoint pixels of dx: side by side in one launch where
  // their kernels agree, else one launch each.
  int together = kPlanAgain;
  if (multi_launchable(planned_classes.data(), (int)planned_classes.size(), sms))
    together = launch_gemm_multi(planned_classes.data(), (int)planned_classes.size(), s);
  if (together == kPlanAgain) {
    for (const GemmArgs& g : planned_classes) {
      const int st_ = launch_gemm(g, dtype, s);
      if (st_ != PDNN_OK) return st_;
    }
  } else if (together != PDNN_OK) {
    return together;
  }
  if (mask_pending && mask_bits != nullptr)
    return launch_relu_grad_bits(dtype, mask_bits, dx, (size_t)p.batch * p.in_rows * p.in_cols * p.channels, s);
  if (mask_pending)
    return launch_pointwise_grad(PDNN_ACT_RELU, dtype, relu_mask, dx, dx,
                                 (size_t)p.batch * p.in_rows * p.in_cols * p.channels, s);
  return PDNN_OK;
}

struct FbpPlan {
  int tw, th, tn, slabs_w, slabs_h, slabs_n, splits, slabs_per_split, m_tiles, n_tiles, bn, tap_pack;
};

FbpPlan plan_filter_backprop(int dtype, const PdnnConv2DParams& p, int sms) {
  FbpPlan f;
  const int epr = dtype == PDNN_F32 ? 32 : 64;
  choose_box(epr, p.out_cols, p.out_rows, p.batch, &f.tw, &f.th, &f.tn);
  f.slabs_w = ceil_div(p.out_cols, f.tw);
  f.slabs_h = ceil_div(p.out_rows, f.th);
  f.slabs_n = ceil_div(p.batch, f.tn);
  f.m_tiles = ceil_div(p.channels, kTileM);
  const int max_bn = dtype == PDNN_F32 ? 128 : 256;
  // 128-column tiles: two accumulator buffers per pipeline, so the fp32 epilogue of one tile overlaps the
  // reduction of the next (measured over the ResNet-50 layers: 9% less time than 256-column tiles)
  f.bn = std::min(std::min(max_bn, 128), ceil_div(p.features, epr) * epr);
  f.n_tiles = ceil_div(p.features, f.bn);
  // At most 64 channels and several taps: a tile holds two taps, the second 64 accumulator rows being
  // the same channels as the next tap sees them, instead of rows that no channel uses.
  f.tap_pack = (dtype != PDNN_F32 && p.channels <= 64 && p.window_rows * p.window_cols >= 2) ? 2 : 1;
  const long long out_tiles = (long long)f.m_tiles * f.n_tiles * ceil_div(p.window_rows * p.window_cols, f.tap_pack);
  const long long total_slabs = (long long)f.slabs_w * f.slabs_h * f.slabs_n;
  long long want = std::max<long long>(1, (2ll * sms) / out_tiles);
  want = std::min<long long>(want, std::max<long long>(1, total_slabs / 8));  // at least 8 slabs per split
  want = std::min<long long>(want, 512);
  f.slabs_per_split = (int)((total_slabs + want - 1) / want);
  f.splits = (int)((total_slabs + f.slabs_per_split - 1) / f.slabs_per_split);
  return f;
}

template <typename T>
__global__ void __launch_bounds__(256) reduce_splits_kernel(const float* __restrict__ partial, T* __restrict__ out,
                                                            int splits, size_t n, bool accumulate) {
  for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (size_t)gridDim.x * 256) {
    float sum = accumulate ? to_f32(out[i]) : 0.f;
    for (int sp = 0; sp < splits; ++sp) sum += partial[(size_t)sp * n + i];
    out[i] = from_f32<T>(sum);
  }
}

// ---- filter backprop for very few input channels (network stems) ---------------------------------
// Mirror image of conv_forward_small_c: with the input packed to CP channels per pixel and
// padded, the gradient of filter row r is one GEMM  dWp[r][64][K] = Xr^T * dy, where a row of
// Xr is the 128-byte packed run of 8 pixels x CP channels that output pixel reads for filter
// row r.  The 64 rows of the result are exactly [s (8)][c (CP)], i.e. the packed filter layout;
// the final kernel sums the pixel splits and drops the padding entries.
template <typename T, typename OutT = T>
__global__ void __launch_bounds__(256)
    unpack_small_c_filter_grad_kernel(const float* __restrict__ partial, OutT* __restrict__ dw, int splits, int R, int S,
                                      int C, int K, int rows_per_tap, bool accumulate) {
  constexpr int CP = 16 / sizeof(T);
  const size_t total = (size_t)R * S * C * K;
  const size_t split_stride = (size_t)R * rows_per_tap * K;
  for (size_t idx = (size_t)blockIdx.x * 256 + threadIdx.x; idx < total; idx += (size_t)gridDim.x * 256) {
    const int k = (int)(idx % K);
    size_t t = idx / K;
    const int c = (int)(t % C);
    t /= C;
    const int sidx = (int)(t % S);
    const int r = (int)(t / S);
    const size_t src = ((size_t)r * rows_per_tap + (size_t)sidx * CP + c) * K + k;
    float sum = accumulate ? to_f32(dw[idx]) : 0.f;
    for (int sp = 0; sp < splits; ++sp) sum += partial[(size_t)sp * split_stride + src];
    dw[idx] = from_f32<OutT>(sum);
  }
}

struct SmallCFbpPlan {
  FbpPlan f;
  SmallCPlan sp;
  size_t partial_bytes;
};

SmallCFbpPlan plan_small_c_fbp(int dtype, const PdnnConv2DParams& p, int sms) {
  SmallCFbpPlan q;
  const int epr = dtype == PDNN_F32 ? 32 : 64;
  q.sp = plan_small_c(dtype, p);
  FbpPlan& f = q.f;
  choose_box(epr, p.out_cols, p.out_rows, p.batch, &f.tw, &f.th, &f.tn);
  f.slabs_w = ceil_div(p.out_cols, f.tw);
  f.slabs_h = ceil_div(p.out_rows, f.th);
  f.slabs_n = ceil_div(p.batch, f.tn);
  f.m_tiles = 1;
  f.tap_pack = (dtype != PDNN_F32 && p.window_rows >= 2) ? 2 : 1;  // 64 packed rows per filter row: two per tile
  f.bn = std::min(dtype == PDNN_F32 ? 128 : 256, ceil_div(p.features, epr) * epr);
  f.n_tiles = ceil_div(p.features, f.bn);
  const long long out_tiles = (long long)f.n_tiles * ceil_div(p.window_rows, f.tap_pack);
  const long long total_slabs = (long long)f.slabs_w * f.slabs_h * f.slabs_n;
  long long want = std::max<long long>(1, (2ll * sms) / out_tiles);
  want = std::min<long long>(want, std::max<long long>(1, total_slabs / 8));
  want = std::min<long long>(want, 512);
  f.slabs_per_split = (int)((total_slabs + want - 1) / want);
  f.splits = (int)((total_slabs + f.slabs_per_split - 1) / f.slabs_per_split);
  q.partial_bytes = (((size_t)f.splits * p.window_rows * epr * p.features * sizeof(float)) + 255) / 256 * 256;
  return q;
}

// Returns PDNN_OK, an error, or -1 if a tensor map could not be encoded (the caller falls back to
// the direct kernel).
int conv_filter_backprop_small_c(int dtype, const void* x, const void* dy, void* dw, const PdnnConv2DParams& p,
                                 bool out_f32, bool accumulate, void* ws, size_t ws_elems, cudaStream_t s) {
  const size_t es = dtype_size(dtype);
  const int sms = device_sm_count();
  const int epr = dtype == PDNN_F32 ? 32 : 64;
  const SmallCFbpPlan q = plan_small_c_fbp(dtype, p, sms);
  const FbpPlan& f = q.f;
  const size_t need = q.sp.xp_bytes + q.partial_bytes;
  char* scratch = static_cast<char*>(ws);
  bool own = false;
  if (scratch == nullptr || ws_elems * es < need || ((uintptr_t)scratch & 255u)) {
    if (cudaMallocAsync(reinterpret_cast<void**>(&scratch), need, s) != cudaSuccess) {
      cudaGetLastError();
      return fail(PDNN_ALLOCATION_PROBLEM, "conv2d: cannot allocate %zu bytes of scratch for the packed input", need);
    }
    own = true;
  }
  char* xp = scratch;
  float* partial = reinterpret_cast<float*>(scratch + q.sp.xp_bytes);
  auto release = [&] {
    if (own) cudaFreeAsync(scratch, s);
  };
  GemmArgs g;
  std::memset(&g, 0, sizeof(g));
  g.a_mn = 1;
  g.tw = f.tw;
  g.th = f.th;
  g.tn = f.tn;
  g.etw = kTileM;
  g.eth = g.etn = 1;
  g.tiles_w = 1;
  g.tiles_h = g.tiles_n = 1;
  g.bn = f.bn;
  g.n_tiles = f.n_tiles;
  g.slabs_w = f.slabs_w;
  g.slabs_h = f.slabs_h;
  g.slabs_n = f.slabs_n;
  g.splits = f.splits;
  g.slabs_per_split = f.slabs_per_split;
  set_operand_layout(g, dtype, 1);
  const size_t row_pitch = (size_t)q.sp.Wp * 16;
  const uint32_t box[4] = {(uint32_t)epr, (uint32_t)f.tw, (uint32_t)f.th, (uint32_t)f.tn};
  for (int r = 0; r < p.stride_rows; ++r) {
    const int Hq = ceil_div(q.sp.Hp - r, p.stride_rows);
    const uint64_t dims[4] = {(uint64_t)epr, (uint64_t)p.out_cols, (uint64_t)std::max(Hq, 1), (uint64_t)p.batch};
    const uint64_t st[3] = {(uint64_t)p.stride_cols * 16, (uint64_t)p.stride_rows * row_pitch,
                            (uint64_t)q.sp.Hp * row_pitch};
    if (!make_map(&g.a_map[r], dtype, true, xp + (size_t)r * row_pitch, dims, st, box)) {
      release();
      return -1;
    }
  }
  for (int r = p.stride_rows; r < 4; ++r) g.a_map[r] = g.a_map[0];
  {
    g.b_mode = B_MN_4;
    const uint64_t dims[4] = {(uint64_t)p.features, (uint64_t)p.out_cols, (uint64_t)p.out_rows, (uint64_t)p.batch};
    const uint64_t st[3] = {(uint64_t)p.features * es, (uint64_t)p.out_cols * p.features * es,
                            (uint64_t)p.out_rows * p.out_cols * p.features * es};
    if (!make_map(&g.b_map, dtype, true, dy, dims, st, box)) {
      release();
      return -1;
    }
  }
  for (int r = 0; r < p.window_rows; ++r)
    g.taps[r] = TapEntry{0, (short)(r / p.stride_rows), (short)(r % p.stride_rows), 0};
  g.num_taps = p.window_rows;
  set_epilogue(g, nullptr);
  g.out = partial;
  g.out_dtype = PDNN_F32;
  g.ext_w = epr;  // the rows of a tap's result that exist: [s][c] of the packed filter
  g.ext_h = g.ext_n = 1;
  g.ext_cols = p.features;
  g.stride_w = p.features;
  g.tap_stride = (long long)epr * p.features;
  g.split_stride = (long long)p.window_rows * epr * p.features;
  g.tap_pack = f.tap_pack;
  if (f.tap_pack == 2) {  // two filter rows per tile: 2 x 64 accumulator rows
    g.etw = 64;
    g.eth = 2;
    g.ext_h = p.window_rows;
    g.stride_h = g.tap_stride;
  }
  g.vec_ok = 1;
  {
    const uint64_t od[4] = {(uint64_t)p.features, (uint64_t)epr, (uint64_t)p.window_rows, (uint64_t)f.splits};
    const uint64_t os[3] = {(uint64_t)p.features * 4, (uint64_t)epr * p.features * 4,
                            (uint64_t)p.window_rows * epr * p.features * 4};
    if (!setup_store(g, dtype, od, os)) {
      release();
      return -1;
    }
  }
  if (dtype == PDNN_F32)
    pack_small_c_input_kernel<float><<<dim3((unsigned)ceil_div(q.sp.Wp, 256), (unsigned)q.sp.Hp, (unsigned)p.batch), 256, 0, s>>>(
        static_cast<const float*>(x), reinterpret_cast<uint4*>(xp), p.batch, p.in_rows, p.in_cols, p.channels, q.sp.Hp,
        q.sp.Wp, p.pad_rows, p.pad_cols);
  else
    pack_small_c_input_kernel<__half><<<dim3((unsigned)ceil_div(q.sp.Wp, 256), (unsigned)q.sp.Hp, (unsigned)p.batch), 256, 0, s>>>(
        static_cast<const __half*>(x), reinterpret_cast<uint4*>(xp), p.batch, p.in_rows, p.in_cols, p.channels,
        q.sp.Hp, q.sp.Wp, p.pad_rows, p.pad_cols);
  int st = check_launch("conv2d small-channel packing");
  if (st == PDNN_OK) st = launch_gemm(g, dtype, s);
  if (st == PDNN_OK) {
    const size_t n_out = (size_t)p.window_rows * p.window_cols * p.channels * p.features;
    const unsigned grid = grid_for(n_out, 256, sms);
    if (dtype == PDNN_F32)
      unpack_small_c_filter_grad_kernel<float><<<grid, 256, 0, s>>>(partial, static_cast<float*>(dw), f.splits,
                                                                    p.window_rows, p.window_cols, p.channels, p.features, epr, accumulate);
    else if (out_f32)  // 16-bit tensors (8 channels per packed pixel), fp32 gradient
      unpack_small_c_filter_grad_kernel<__half, float><<<grid, 256, 0, s>>>(
          partial, static_cast<float*>(dw), f.splits, p.window_rows, p.window_cols, p.channels, p.features, epr, accumulate);
    else if (dtype == PDNN_F16)
      unpack_small_c_filter_grad_kernel<__half><<<grid, 256, 0, s>>>(partial, static_cast<__half*>(dw), f.splits,
                                                                     p.window_rows, p.window_cols, p.channels, p.features, epr, accumulate);
    else
      unpack_small_c_filter_grad_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(
          partial, static_cast<__nv_bfloat16*>(dw), f.splits, p.window_rows, p.window_cols, p.channels, p.features, epr, accumulate);
    st = check_launch("conv2d small-channel filter gradient unpack");
  }
  release();
  return st;
}

// out_f32: dW is written as fp32 whatever the tensors' type (the split reduction, or the epilogue
// when there is one split, produces it directly).
// accumulate: dW += the gradient.  With fp32 gradients every pixel split adds its tiles to dW by TMA
// reduction (no partial sums, no second kernel; the order of the float additions is then not fixed);
// otherwise the split reduction adds to what dW held.
int conv_filter_backprop(int dtype, const void* x, const void* dy, void* dw, const PdnnConv2DParams& p, bool out_f32,
                         bool accumulate, void* ws, size_t ws_elems, cudaStream_t s, bool try_reduce = true) {
  const size_t es = dtype_size(dtype);
  const int sms = device_sm_count();
  const int epr = dtype == PDNN_F32 ? 32 : 64;
  const FbpPlan f = plan_filter_backprop(dtype, p, sms);
  GemmArgs g;
  std::memset(&g, 0, sizeof(g));
  g.a_mn = 1;
  g.tw = f.tw;
  g.th = f.th;
  g.tn = f.tn;
  g.etw = kTileM;
  g.eth = 1;
  g.etn = 1;
  g.tiles_w = f.m_tiles;
  g.tiles_h = g.tiles_n = 1;
  g.bn = f.bn;
  g.n_tiles = f.n_tiles;
  g.slabs_w = f.slabs_w;
  g.slabs_h = f.slabs_h;
  g.slabs_n = f.slabs_n;
  g.splits = f.splits;
  g.slabs_per_split = f.slabs_per_split;
  g.split_is_batch = 0;
  set_operand_layout(g, dtype, 1);
  const uint32_t box[4] = {(uint32_t)epr, (uint32_t)f.tw, (uint32_t)f.th, (uint32_t)f.tn};
  if (!make_parity_maps(g, dtype, true, x, p, box)) return PDNN_INVALID_PARAMETER;
  {
    g.b_mode = B_MN_4;
    const uint64_t dims[4] = {(uint64_t)p.features, (uint64_t)p.out_cols, (uint64_t)p.out_rows, (uint64_t)p.batch};
    const uint64_t st[3] = {(uint64_t)p.features * es, (uint64_t)p.out_cols * p.features * es,
                            (uint64_t)p.out_rows * p.out_cols * p.features * es};
    if (!make_map(&g.b_map, dtype, true, dy, dims, st, box)) return PDNN_INVALID_PARAMETER;
  }
  int nt = 0;
  for (int r = 0; r < p.window_rows; ++r)
    for (int c = 0; c < p.window_cols; ++c) {
      const int hh = r - p.pad_rows, ww = c - p.pad_cols;
      TapEntry e;
      e.dh = (short)floor_div(hh, p.stride_rows);
      e.dw = (short)floor_div(ww, p.stride_cols);
      e.a_map = (short)(pos_mod(hh, p.stride_rows) * p.stride_cols + pos_mod(ww, p.stride_cols));
      e.b_tap = 0;
      g.taps[nt++] = e;
    }
  g.num_taps = nt;
  set_epilogue(g, nullptr);
  const size_t n_out = (size_t)nt * p.channels * p.features;
  float* partial = nullptr;
  bool own = false;
  const bool reduce = try_reduce && accumulate && (out_f32 || dtype == PDNN_F32) && aligned16(dw);
  const bool use_partial = !reduce && (f.splits > 1 || accumulate);
  if (use_partial) {
    const size_t need_bytes = (size_t)f.splits * n_out * sizeof(float);
    if (ws != nullptr && ws_elems * es >= need_bytes && aligned16(ws)) {
      partial = static_cast<float*>(ws);
    } else {
      if (cudaMallocAsync(reinterpret_cast<void**>(&partial), need_bytes, s) != cudaSuccess) {
        cudaGetLastError();
        return fail(PDNN_ALLOCATION_PROBLEM, "filter backprop: cannot allocate %zu bytes of scratch", need_bytes);
      }
      own = true;
    }
    g.out = partial;
    g.out_dtype = PDNN_F32;
  } else {
    g.out = dw;
    g.out_dtype = (out_f32 || reduce) ? PDNN_F32 : dtype;
    g.reduce_add = reduce ? 1 : 0;
  }
  g.ext_w = p.channels;
  g.ext_h = g.ext_n = 1;
  g.ext_cols = p.features;
  g.stride_w = p.features;
  g.stride_h = g.stride_n = 0;
  g.split_stride = (long long)n_out;
  g.tap_stride = (long long)p.channels * p.features;
  g.tap_pack = f.tap_pack;
  if (f.tap_pack == 2) {  // rows 64..127 of a tile are channels 0..63 of the next tap
    g.etw = 64;
    g.eth = 2;
    g.ext_h = nt;
    g.stride_h = g.tap_stride;
  }
  g.vec_ok = 1;
  {
    const uint64_t eo = dtype_size(g.out_dtype);
    const uint64_t od[4] = {(uint64_t)p.features, (uint64_t)p.channels, (uint64_t)nt, (uint64_t)(reduce ? 1 : f.splits)};
    const uint64_t os[3] = {(uint64_t)p.features * eo, (uint64_t)p.channels * p.features * eo, (uint64_t)n_out * eo};
    if (!setup_store(g, dtype, od, os)) {
      if (own) cudaFreeAsync(partial, s);
      return PDNN_INVALID_PARAMETER;
    }
    // only the staged TMA epilogue can add; anything else goes through partial sums
    if (reduce && !g.tma_store) return conv_filter_backprop(dtype, x, dy, dw, p, out_f32, accumulate, ws, ws_elems, s, false);
  }
  int st = launch_gemm(g, dtype, s);
  if (st == PDNN_OK && use_partial) {
    const unsigned grid = grid_for(n_out, 256, sms);
    if (dtype == PDNN_F32 || out_f32) reduce_splits_kernel<float><<<grid, 256, 0, s>>>(partial, static_cast<float*>(dw), f.splits, n_out, accumulate);
    else if (dtype == PDNN_F16) reduce_splits_kernel<__half><<<grid, 256, 0, s>>>(partial, static_cast<__half*>(dw), f.splits, n_out, accumulate);
    else reduce_splits_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(partial, static_cast<__nv_bfloat16*>(dw), f.splits, n_out, accumulate);
    st = check_launch("filter backprop split reduction");
  }
  if (own) cudaFreeAsync(partial, s);
  return st;
}

// ---- SIMT matmul ---------------------------------------------------------------------------------
template <typename T, typename OutT = T>
__global__ void __launch_bounds__(256) simt_matmul_kernel(const T* __restrict__ lhs, const T* __restrict__ rhs,
                                                          OutT* __restrict__ out, int tl, int tr, int batches, int m, int k,
                                                          int n, float beta) {
  const size_t total = (size_t)batches * m * n;
  for (size_t idx = (size_t)blockIdx.x * 256 + threadIdx.x; idx < total; idx += (size_t)gridDim.x * 256) {
    const int j = (int)(idx % n);
    const int i = (int)((idx / n) % m);
    const int b = (int)(idx / ((size_t)m * n));
    const T* A = lhs + (size_t)b * m * k;
    const T* B = rhs + (size_t)b * k * n;
    float acc = 0.f;
    for (int l = 0; l < k; ++l) {
      const float av = to_f32(tl ? A[(size_t)l * m + i] : A[(size_t)i * k + l]);
      const float bv = to_f32(tr ? B[(size_t)j * k + l] : B[(size_t)l * n + j]);
      acc = fmaf(av, bv, acc);
    }
    if (beta != 0.f) acc += beta * to_f32(out[idx]);
    out[idx] = from_f32<OutT>(acc);
  }
}

}  // namespace

// ================================================================================================
// Public (library-internal) interface
// ================================================================================================

bool tc_conv_supported(int pass, int dtype, const void* in, const void* fil, const void* out,
                       const PdnnConv2DParams& p) {
  if (encode_fn() == nullptr) return false;
  if (pass == PDNN_FORWARD && small_c_applicable(dtype, p)) return aligned16(out);
  if (pass == PDNN_FILTER_BACKPROP && small_c_applicable(dtype, p)) return aligned16(fil);
  if (!conv_common_ok(dtype, p)) return false;
  if (!aligned16(in) || !aligned16(fil) || !aligned16(out)) return false;
  for (int ph = 0; ph < p.stride_rows; ++ph)
    for (int pw = 0; pw < p.stride_cols; ++pw)
      if (p.in_rows - ph <= 0 || p.in_cols - pw <= 0) return false;
  if (pass == PDNN_FILTER_BACKPROP && p.filter_format != 0) return false;
  return true;
}

// Grouped forward convolution (STRIDED groups: group g reads channels [g*C/G, (g+1)*C/G) and writes
// features [g*K/G, (g+1)*K/G), include/portdnn/internal/conv2d/im2col.h:90-137) as one implicit GEMM
// per group on channel slices of the tensors: the tensor maps take the slices' leading dimensions,
// nothing is copied or transposed.
bool tc_grouped_conv_supported(int dtype, const void* in, const void* fil, const void* out, const PdnnConv2DParams& p) {
  if (encode_fn() == nullptr || p.groups <= 1 || p.group_format != 0) return false;
  if (p.channels % p.groups || p.features % p.groups) return false;
  PdnnConv2DParams q = p;
  q.channels = p.channels / p.groups;
  q.features = p.features / p.groups;
  q.groups = 1;
  if (!conv_common_ok(dtype, q) || small_c_applicable(dtype, q)) return false;
  if (!aligned16(in) || !aligned16(fil) || !aligned16(out)) return false;
  for (int ph = 0; ph < p.stride_rows; ++ph)
    for (int pw = 0; pw < p.stride_cols; ++pw)
      if (p.in_rows - ph <= 0 || p.in_cols - pw <= 0) return false;
  return true;
}

int tc_grouped_conv_forward(int dtype, const void* in, const void* fil, void* out, const PdnnConv2DParams& p,
                            const PdnnConvEpilogue* epi, cudaStream_t s) {
  const size_t es = dtype_size(dtype);
  PdnnConv2DParams q = p;
  q.channels = p.channels / p.groups;
  q.features = p.features / p.groups;
  q.groups = 1;
  const bool hwcf = p.filter_format == 0;
  const ConvLd ld{p.channels, hwcf ? p.features : 0, p.features};
  const size_t fhwc_group = (size_t)q.features * p.window_rows * p.window_cols * q.channels;
  // 16-bit: the groups are planned first and launched four at a time, side by side (umma_gemm_multi_kernel):
  // a group is a small GEMM that rarely fills the device on its own.
  const int sms = device_sm_count();
  GemmArgs plans[kMaxMulti];
  int planned = 0;
  auto flush = [&]() -> int {
    int st = kPlanAgain;
    if (multi_launchable(plans, planned, sms)) st = launch_gemm_multi(plans, planned, s);
    if (st == kPlanAgain) {
      st = PDNN_OK;
      for (int i = 0; i < planned && st == PDNN_OK; ++i) st = launch_gemm(plans[i], dtype, s);
    }
    planned = 0;
    return st;
  };
  for (int g = 0; g < p.groups; ++g) {
    PdnnConvEpilogue e;
    if (epi != nullptr) {
      e = *epi;
      if (e.bias != nullptr) e.bias = static_cast<const char*>(e.bias) + (size_t)g * q.features * es;
    }
    const char* xg = static_cast<const char*>(in) + (size_t)g * q.channels * es;
    const char* wg = static_cast<const char*>(fil) + (hwcf ? (size_t)g * q.features : (size_t)g * fhwc_group) * es;
    char* yg = static_cast<char*>(out) + (size_t)g * q.features * es;
    const bool plan_only = dtype != PDNN_F32;
    const int st = conv_forward(dtype, xg, wg, yg, q, epi != nullptr ? &e : nullptr, s, true, true, &ld,
                                plan_only ? &plans[planned] : nullptr);
    if (st != PDNN_OK) return st;
    if (plan_only && ++planned == kMaxMulti) {
      const int fs = flush();
      if (fs != PDNN_OK) return fs;
    }
  }
  return planned > 0 ? flush() : PDNN_OK;
}

size_t tc_conv_workspace_elems(int pass, int dtype, const PdnnConv2DParams& p) {
  if (pass == PDNN_FORWARD && small_c_applicable(dtype, p)) {
    const SmallCPlan sp = plan_small_c(dtype, p);
    return (sp.xp_bytes + sp.wp_bytes) / dtype_size(dtype);
  }
  if (pass == PDNN_FILTER_BACKPROP && small_c_applicable(dtype, p)) {
    int sms = device_sm_count();
    if (sms <= 0) sms = 148;
    const SmallCFbpPlan q = plan_small_c_fbp(dtype, p, sms);
    return (q.sp.xp_bytes + q.partial_bytes) / dtype_size(dtype);
  }
  if (pass != PDNN_FILTER_BACKPROP || !conv_common_ok(dtype, p) || p.filter_format != 0) return 0;
  int sms = device_sm_count();
  if (sms <= 0) sms = 148;
  const FbpPlan f = plan_filter_backprop(dtype, p, sms);
  if (f.splits <= 1) return 0;
  const size_t bytes = (size_t)f.splits * p.window_rows * p.window_cols * p.channels * p.features * sizeof(float);
  return (bytes + dtype_size(dtype) - 1) / dtype_size(dtype);
}

int tc_conv2d(int pass, int dtype, const void* in, const void* fil, void* out, const PdnnConv2DParams& p,
              const PdnnConvEpilogue* epi, const PdnnBackpropFusion* fusion, void* ws, size_t ws_elems, cudaStream_t s) {
  const void* relu_mask = fusion != nullptr ? fusion->relu_forward_output : nullptr;
  const bool out_f32 = fusion != nullptr && fusion->output_f32 != 0 && dtype != PDNN_F32;
  const int accumulate = fusion != nullptr ? fusion->accumulate : 0;
  switch (pass) {
    case PDNN_FORWARD:
      if (small_c_applicable(dtype, p)) {
        const int st = conv_forward_small_c(dtype, in, fil, out, p, epi, ws, ws_elems, s);
        return st == -1 ? kNeedsDirect : st;
      }
      return conv_forward(dtype, in, fil, out, p, epi, s);
    case PDNN_INPUT_BACKPROP:
      return conv_input_backprop(dtype, in, fil, out, p, relu_mask, fusion != nullptr ? fusion->relu_bitmask : nullptr,
                                 accumulate, fusion != nullptr && fusion->constant_filter != 0, s);
    case PDNN_FILTER_BACKPROP:
      if (small_c_applicable(dtype, p)) {
        const int st = conv_filter_backprop_small_c(dtype, in, fil, out, p, out_f32, accumulate != 0, ws, ws_elems, s);
        return st == -1 ? kNeedsDirect : st;
      }
      return conv_filter_backprop(dtype, in, fil, out, p, out_f32, accumulate != 0, ws, ws_elems, s);
  }
  return fail(PDNN_INVALID_PARAMETER, "bad pass %d", pass);
}

bool tc_matmul_supported(int dtype, int tl, int tr, const void* lhs, const void* rhs, const void* out, int batches,
                         int m, int k, int n) {
  const int align = dtype == PDNN_F32 ? 4 : 8;
  if (!aligned16(lhs) || !aligned16(rhs) || !aligned16(out)) return false;
  if (encode_fn() == nullptr) return false;
  if ((tl ? m : k) % align) return false;  // lhs row pitch
  if ((tr ? k : n) % align) return false;  // rhs row pitch
  if (n % align) return false;             // output row pitch
  // batch strides must be multiples of 16 bytes too
  if (batches > 1 && (((size_t)m * k) % align || ((size_t)k * n) % align || ((size_t)m * n) % align)) return false;
  return m > 0 && k > 0 && n > 0 && batches > 0;
}

int tc_matmul(int dtype, int tl, int tr, const void* lhs, const void* rhs, void* out, int batches, int m, int k, int n,
              float beta, cudaStream_t s, bool out_f32) {
  const size_t es = dtype_size(dtype);
  const int sms = device_sm_count();
  const int epr = dtype == PDNN_F32 ? 32 : 64;
  GemmArgs g;
  std::memset(&g, 0, sizeof(g));
  g.a_mn = tl ? 1 : 0;
  const int m_tiles = ceil_div(m, kTileM);
  const int b_mn = tr ? 0 : 1;
  g.bn = pick_bn((long long)m_tiles * batches, n, b_mn ? epr : 16, dtype == PDNN_F32 ? 128 : 256, sms, ceil_div(k, epr));
  g.n_tiles = ceil_div(n, g.bn);
  set_operand_layout(g, dtype, b_mn);
  g.taps[0] = TapEntry{0, 0, 0, 0};
  g.num_taps = 1;
  g.etw = kTileM;
  g.eth = g.etn = 1;
  if (!tl) {
    g.tw = kTileM;
    g.th = g.tn = 1;
    g.tiles_w = m_tiles;
    g.tiles_h = 1;
    g.tiles_n = batches;
    g.cblocks = ceil_div(k, epr);
    g.b_batch_mul = 1;
    const uint64_t dims[4] = {(uint64_t)k, (uint64_t)m, 1, (uint64_t)batches};
    const uint64_t st[3] = {(uint64_t)k * es, (uint64_t)m * k * es, (uint64_t)m * k * es};
    const uint32_t box[4] = {(uint32_t)epr, (uint32_t)kTileM, 1, 1};
    if (!make_map(&g.a_map[0], dtype, false, lhs, dims, st, box)) return PDNN_INVALID_PARAMETER;
    if (b_mn) {
      g.b_mode = B_MN_3;
      const uint64_t bd[4] = {(uint64_t)n, (uint64_t)k, (uint64_t)batches, 1};
      const uint64_t bs[3] = {(uint64_t)n * es, (uint64_t)k * n * es, (uint64_t)batches * k * n * es};
      const uint32_t bb[4] = {(uint32_t)epr, (uint32_t)epr, 1, 1};
      if (!make_map(&g.b_map, dtype, true, rhs, bd, bs, bb)) return PDNN_INVALID_PARAMETER;
    } else {
      g.b_mode = B_K_3;
      const uint64_t bd[4] = {(uint64_t)k, (uint64_t)n, (uint64_t)batches, 1};
      const uint64_t bs[3] = {(uint64_t)k * es, (uint64_t)k * n * es, (uint64_t)batches * k * n * es};
      const uint32_t bb[4] = {(uint32_t)epr, (uint32_t)g.bn, 1, 1};
      if (!make_map(&g.b_map, dtype, false, rhs, bd, bs, bb)) return PDNN_INVALID_PARAMETER;
    }
    g.ext_w = m;
    g.ext_h = 1;
    g.ext_n = batches;
    g.stride_w = n;
    g.stride_h = 0;
    g.stride_n = (long long)m * n;
  } else {
    g.tw = epr;
    g.th = g.tn = 1;
    g.tiles_w = m_tiles;
    g.tiles_h = g.tiles_n = 1;
    g.slabs_w = ceil_div(k, epr);
    g.slabs_h = g.slabs_n = 1;
    g.splits = batches;
    g.slabs_per_split = g.slabs_w;
    g.split_is_batch = 1;
    const uint64_t dims[4] = {(uint64_t)m, (uint64_t)k, 1, (uint64_t)batches};
    const uint64_t st[3] = {(uint64_t)m * es, (uint64_t)m * k * es, (uint64_t)m * k * es};
    const uint32_t box[4] = {(uint32_t)epr, (uint32_t)epr, 1, 1};
    if (!make_map(&g.a_map[0], dtype, true, lhs, dims, st, box)) return PDNN_INVALID_PARAMETER;
    if (b_mn) {
      g.b_mode = B_MN_4;
      const uint64_t bd[4] = {(uint64_t)n, (uint64_t)k, 1, (uint64_t)batches};
      const uint64_t bs[3] = {(uint64_t)n * es, (uint64_t)k * n * es, (uint64_t)k * n * es};
      const uint32_t bb[4] = {(uint32_t)epr, (uint32_t)epr, 1, 1};
      if (!make_map(&g.b_map, dtype, true, rhs, bd, bs, bb)) return PDNN_INVALID_PARAMETER;
    } else {
      g.b_mode = B_K_4;
      const uint64_t bd[4] = {(uint64_t)k, (uint64_t)n, 1, (uint64_t)batches};
      const uint64_t bs[3] = {(uint64_t)k * es, (uint64_t)k * n * es, (uint64_t)k * n * es};
      const uint32_t bb[4] = {(uint32_t)epr, (uint32_t)g.bn, 1, 1};
      if (!make_map(&g.b_map, dtype, false, rhs, bd, bs, bb)) return PDNN_INVALID_PARAMETER;
    }
    g.ext_w = m;
    g.ext_h = g.ext_n = 1;
    g.stride_w = n;
    g.split_stride = (long long)m * n;
    g.tap_stride = 0;
  }
  for (int i = 1; i < 4; ++i) g.a_map[i] = g.a_map[0];
  set_epilogue(g, nullptr);
  g.beta = beta;
  g.out = out;
  g.out_dtype = out_f32 ? PDNN_F32 : dtype;
  g.ext_cols = n;
  g.vec_ok = 1;
  {
    const uint64_t eo = dtype_size(g.out_dtype);
    const uint64_t od[4] = {(uint64_t)n, (uint64_t)m, 1, (uint64_t)batches};
    const uint64_t os[3] = {(uint64_t)n * eo, (uint64_t)m * n * eo, (uint64_t)m * n * eo};
    if (!setup_store(g, dtype, od, os)) return PDNN_INVALID_PARAMETER;
  }
  return launch_gemm(g, dtype, s);
}

int simt_matmul(int dtype, int tl, int tr, const void* lhs, const void* rhs, void* out, int batches, int m, int k, int n,
                float beta, cudaStream_t s, bool out_f32) {
  const int sms = device_sm_count();
  if (sms <= 0) return fail(PDNN_ALLOCATION_PROBLEM, "no CUDA device");
  const size_t total = (size_t)batches * m * n;
  const unsigned grid = grid_for(total, 256, sms);
  if (dtype == PDNN_F32)
    simt_matmul_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(lhs), static_cast<const float*>(rhs),
                                                    static_cast<float*>(out), tl, tr, batches, m, k, n, beta);
  else if (out_f32 && dtype == PDNN_F16)
    simt_matmul_kernel<__half, float><<<grid, 256, 0, s>>>(static_cast<const __half*>(lhs), static_cast<const __half*>(rhs),
                                                            static_cast<float*>(out), tl, tr, batches, m, k, n, beta);
  else if (out_f32 && dtype == PDNN_BF16)
    simt_matmul_kernel<__nv_bfloat16, float><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(lhs),
                                                                   static_cast<const __nv_bfloat16*>(rhs),
                                                                   static_cast<float*>(out), tl, tr, batches, m, k, n, beta);
  else if (dtype == PDNN_F16)
    simt_matmul_kernel<__half><<<grid, 256, 0, s>>>(static_cast<const __half*>(lhs), static_cast<const __half*>(rhs),
                                                     static_cast<__half*>(out), tl, tr, batches, m, k, n, beta);
  else if (dtype == PDNN_BF16)
    simt_matmul_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(lhs),
                                                            static_cast<const __nv_bfloat16*>(rhs),
                                                            static_cast<__nv_bfloat16*>(out), tl, tr, batches, m, k, n, beta);
  else
    return fail(PDNN_INVALID_PARAMETER, "unknown dtype %d", dtype);
  return check_launch("simt matmul");
}

int tc_read_error_record(unsigned out[4], int clear) {
  if (cudaMemcpyFromSymbol(out, g_error_record, sizeof(unsigned) * 4) != cudaSuccess) {
    cudaGetLastError();
    return fail(PDNN_ALLOCATION_PROBLEM, "cannot read the device error record");
  }
  if (clear) {
    const unsigned zero[4] = {0, 0, 0, 0};
    cudaMemcpyToSymbol(g_error_record, zero, sizeof(zero));
  }
  return PDNN_OK;
}



}  // namespace pdnn
