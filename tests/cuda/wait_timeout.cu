// Test-only kernel, not part of libportdnn_b200.so: one CTA waits on an mbarrier that nobody
// ever arrives at, using the library's own bounded wait (portdnn_b200/csrc/umma.cuh).  The wait
// must give up after the limit it is handed, fill the error record and let the kernel return,
// which leaves the CUDA context usable.  This is the failure-detection path of the tensor-core
// kernels (every role loop leaves through the same `return false`), exercised without a fault.
#include <cuda_runtime.h>

#include "../../portdnn_b200/csrc/umma.cuh"

using namespace pdnn::umma;

__global__ void wait_runs_out_kernel(unsigned* record, unsigned long long limit_ns, unsigned long long* elapsed_ns) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned long long t0 = global_timer_ns();
    // phase 0 of a freshly initialised barrier never completes: nothing arrives
    const bool ok = mbar_wait(smem_u32(&bar), 0u, &abort_flag, record, limit_ns, 0x700u);
    *elapsed_ns = global_timer_ns() - t0;
    if (ok) record[0] = 0xBADu;  // the wait must not report success
  }
  __syncthreads();
  // a second role that only polls the abort flag, as the other warps of the real kernel do
  if (threadIdx.x == 32 && abort_flag == 0) record[3] = 0xBADu;
}

// Launches the kernel on the default stream and returns the record and the time the wait took.
// Returns the cudaError_t of the first failing call (0 = success).
extern "C" int pdnn_test_wait_runs_out(unsigned long long limit_ns, unsigned record_out[4],
                                       unsigned long long* elapsed_ns_out) {
  unsigned* record = nullptr;
  unsigned long long* elapsed = nullptr;
  cudaError_t e = cudaMalloc(&record, 4 * sizeof(unsigned));
  if (e != cudaSuccess) return (int)e;
  e = cudaMalloc(&elapsed, sizeof(unsigned long long));
  if (e != cudaSuccess) return (int)e;
  cudaMemset(record, 0, 4 * sizeof(unsigned));
  cudaMemset(elapsed, 0, sizeof(unsigned long long));
  wait_runs_out_kernel<<<1, 64>>>(record, limit_ns, elapsed);
  e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpy(record_out, record, 4 * sizeof(unsigned), cudaMemcpyDeviceToHost);
  if (e == cudaSuccess) e = cudaMemcpy(elapsed_ns_out, elapsed, sizeof(unsigned long long), cudaMemcpyDeviceToHost);
  cudaFree(record);
  cudaFree(elapsed);
  return (int)e;
}
