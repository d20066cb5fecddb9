// Thin inline-PTX layer for the Blackwell (sm_100a) asynchronous pipeline: mbarriers with
// bounded waits, TMA tile loads, tcgen05 MMA / TMEM management.  Every wait gives up after a
// time limit, records where, and lets the kernel unwind (free TMEM, return) instead of
// spinning forever.
#pragma once

#include <cuda.h>  // CUtensorMap (type only; the encoder is fetched through the runtime)

#include <cstdint>

namespace pdnn {
namespace umma {

// ---- device error record ----------------------------------------------------------------------
// word 0: code (0 = none), word 1: blockIdx.x, word 2: role/location, word 3: extra.
enum : unsigned { kErrWaitTimeout = 1, kErrBadConfig = 2 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// ---- mbarrier ----------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Default time limit of a single wait.  A stage of this pipeline completes in microseconds; a
// wait that lasts a second means a lost arrival.
constexpr uint64_t kWaitLimitNs = 1000ull * 1000ull * 1000ull;

// Waits for the phase with the given parity, for at most limit_ns.  Returns false if the CTA is
// aborting or the limit ran out (in which case it raises the abort flag and fills the error
// record).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          unsigned* error_record, uint64_t limit_ns, unsigned where) {
  uint64_t t0 = 0;
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 63u) == 0) {
      if (*abort_flag) return false;
      const uint64_t now = global_timer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > limit_ns) {
        *abort_flag = 1;
        if (atomicCAS(error_record, 0u, (unsigned)kErrWaitTimeout) == 0u) {
          error_record[1] = blockIdx.x;
          error_record[2] = where;
          error_record[3] = parity;
        }
        return false;
      }
    }
  }
}

// True in exactly one lane of the (fully active) warp.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(pred));
  return pred != 0;
}

// ---- TMA -----------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_4d(uint32_t smem_dst, const CUtensorMap* map, uint32_t bar, int c0, int c1,
                                            int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// Tile store shared -> global through a tensor map; rows/columns outside the tensor are clipped.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t smem_src, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(map),
               "r"(smem_src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
// The same tile added to global memory element by element (fp32 tensor map: atomic float adds).
__device__ __forceinline__ void tma_reduce_add_4d(const CUtensorMap* map, uint32_t smem_src, int c0, int c1, int c2, int c3) {
  asm volatile("cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(map),
               "r"(smem_src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until at most N of this thread's bulk groups still have to READ their shared-memory source.
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// Waits until at most N of this thread's bulk groups are still in flight at all.
template <int N>
__device__ __forceinline__ void bulk_wait_group() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// Barrier among `count` threads (a multiple of 32) that all name the same id (1..15).
__device__ __forceinline__ void named_barrier_sync(uint32_t id, uint32_t count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
// Makes generic-proxy writes to shared memory visible to the async proxy (TMA / tcgen05 reads).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- programmatic dependent launch -------------------------------------------------------------
// A kernel launched with programmatic stream serialisation may start while its predecessor in the
// stream is still running.  grid_dependency_wait() blocks until the predecessor has completed and
// its writes are visible (a no-op for an ordinary launch); grid_launch_dependents() tells the
// runtime that the successor may be scheduled as soon as resources free up.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- TMEM ----------------------------------------------------------------------------------------
// Warp-wide. Writes the base address of `columns` (power of two, >= 32) TMEM columns to *smem_slot.
__device__ __forceinline__ void tmem_alloc(uint32_t smem_slot, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot), "r"(columns)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// 32 lanes x 32 consecutive fp32 columns: thread t of the warp receives lane (base lane + t).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// ---- tcgen05.mma ---------------------------------------------------------------------------------
// D[tmem] (+)= A[smem desc] * B[smem desc]; issued by ONE thread.  accumulate == 0 overwrites D.
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
      "}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The mbarrier receives one arrival once every tcgen05 operation issued so far by this thread
// has completed.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// ---- whole-warp forms ------------------------------------------------------------------------------
// Called by all 32 lanes of a warp with warp-uniform arguments; one elected lane issues the
// instruction.  Keeping the surrounding loop convergent lets the compiler hold descriptors, barrier
// addresses and coordinates in uniform registers, which is where these instructions read them.
__device__ __forceinline__ void warp_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  if (elect_one()) mma_f16(d_tmem, a_desc, b_desc, idesc, accumulate);
}
__device__ __forceinline__ void warp_mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              uint32_t accumulate) {
  if (elect_one()) mma_tf32(d_tmem, a_desc, b_desc, idesc, accumulate);
}
__device__ __forceinline__ void warp_commit(uint32_t bar) {
  if (elect_one()) mma_commit(bar);
}
__device__ __forceinline__ void warp_tma_load_4d(uint32_t smem_dst, const CUtensorMap* map, uint32_t bar, int c0, int c1,
                                                 int c2, int c3) {
  if (elect_one()) tma_load_4d(smem_dst, map, bar, c0, c1, c2, c3);
}
__device__ __forceinline__ void warp_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  if (elect_one()) mbar_arrive_expect_tx(bar, bytes);
}

// ---- CTA pairs (cta_group::2) --------------------------------------------------------------------
// Two CTAs of a cluster work on one 256-row tile: each holds its own 128 rows of A and half of the
// columns of B in its shared memory and receives its 128 rows of the accumulator in its tensor
// memory; the MMAs are issued by the CTA of rank 0 only, and read both shared memories.  A shared
// memory address of the same offset in the CTA of rank 0 is the own address with bit 24 cleared.
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The address of `addr` (an own shared-memory address) in the CTA of rank `rank` of the cluster.
__device__ __forceinline__ uint32_t cluster_map_shared(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_slot, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot), "r"(columns)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t base, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}
// TMA load into the own shared memory whose bytes are counted by the barrier of the CTA of rank 0.
__device__ __forceinline__ void tma_load_4d_pair(uint32_t smem_dst, const CUtensorMap* map, uint32_t bar, int c0, int c1,
                                                 int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_dst), "l"(map), "r"(bar & kPeerBitMask), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void mma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the barrier at `cluster_addr` (any CTA of the cluster) once all MMAs issued so far are done.
__device__ __forceinline__ void mma_commit_pair(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void warp_mma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                  uint32_t accumulate) {
  if (elect_one()) mma_f16_pair(d_tmem, a_desc, b_desc, idesc, accumulate);
}
// Both CTAs of the pair learn that the MMAs issued so far are done.
__device__ __forceinline__ void warp_commit_pair(uint32_t bar, uint32_t peer_bar) {
  if (elect_one()) {
    mma_commit_pair(bar);
    mma_commit_pair(peer_bar);
  }
}
__device__ __forceinline__ void warp_tma_load_4d_pair(uint32_t smem_dst, const CUtensorMap* map, uint32_t bar, int c0,
                                                      int c1, int c2, int c3) {
  if (elect_one()) tma_load_4d_pair(smem_dst, map, bar, c0, c1, c2, c3);
}

// ---- descriptors ---------------------------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle.  Addresses and offsets are in bytes here and
// stored in units of 16 bytes; bits [46,48) = 1 marks the sm_100 format, bits [61,64) hold the
// swizzle code: 2 = 128-byte rows swizzled in 16-byte units, 1 = 128-byte rows swizzled in
// 32-byte units (the MN-major layout of 32-bit operands).  For a K-major operand `sbo` is the
// distance between groups of 8 rows (1024 for dense 128-byte rows) and `lbo` is unused; for an
// MN-major operand `lbo` is the distance between 128-byte column blocks and `sbo` the distance
// between groups of 8 k-rows (4 k-rows for code 1).
__host__ __device__ inline uint64_t make_smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo, uint32_t layout = 2) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFFu);
  d |= (uint64_t)((lbo >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)(layout & 7u) << 61;
  return d;
}

// Instruction descriptor for kind::f16 / kind::tf32 with fp32 accumulation, M = 128 (256 for a CTA pair).
// format: 0 = f16, 1 = bf16, 2 = tf32.  *_mn: operand is MN-major (1) or K-major (0).
__host__ __device__ inline uint32_t make_idesc(int format, int a_mn, int b_mn, int n, int m = 128) {
  uint32_t d = 0;
  d |= 1u << 4;                         // D format: f32
  d |= (uint32_t)(format & 7) << 7;     // A format
  d |= (uint32_t)(format & 7) << 10;    // B format
  d |= (uint32_t)(a_mn & 1) << 15;
  d |= (uint32_t)(b_mn & 1) << 16;
  d |= (uint32_t)((n >> 3) & 0x3F) << 17;
  d |= (uint32_t)((m >> 4) & 0x1F) << 24;
  return d;
}

}  // namespace umma
}  // namespace pdnn
