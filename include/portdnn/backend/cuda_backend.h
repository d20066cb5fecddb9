// The one backend of this implementation: device pointers and a CUDA stream.  It fills the role
// of portDNN's USM backend (include/portdnn/backend/snn_usm_backend.h:40-163) and satisfies the
// backend contract of include/portdnn/backend/backend_interface.h:30-153: pointer_type<T> and
// internal_pointer_type<T> are plain T*, allocate/deallocate are stream-ordered, matmul and
// batch_matmul run on the tcgen05 engine (pdnn_matmul).
#ifndef PORTDNN_B200_BACKEND_CUDA_BACKEND_H_
#define PORTDNN_B200_BACKEND_CUDA_BACKEND_H_
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime_api.h>

#include <cstddef>
#include <stdexcept>
#include <type_traits>

#include "portdnn/data_format.h"
#include "portdnn/status.h"
#include "portdnn_b200.h"

namespace sycldnn {
namespace backend {

/** PdnnDataType of an element type. */
template <typename T>
struct dtype_of;
template <>
struct dtype_of<float> { static constexpr int value = PDNN_F32; };
template <>
struct dtype_of<__half> { static constexpr int value = PDNN_F16; };
template <>
struct dtype_of<__nv_bfloat16> { static constexpr int value = PDNN_BF16; };

class CUDABackend {
 public:
  template <typename T>
  using pointer_type = T*;
  template <typename T>
  using internal_pointer_type = T*;

  explicit CUDABackend(cudaStream_t stream = nullptr) : stream_(stream) {}

  static char const* name() { return "CUDABackend"; }
  /** The stream plays the part of the reference's sycl::queue. */
  cudaStream_t get_queue() const { return stream_; }

  template <typename T>
  T* allocate(size_t n_elems) {
    if (n_elems == 0) return nullptr;
    void* p = nullptr;
    if (cudaMallocAsync(&p, n_elems * sizeof(T), stream_) != cudaSuccess) throw std::bad_alloc();
    return static_cast<T*>(p);
  }
  template <typename T>
  void deallocate(T* ptr) {
    if (ptr != nullptr) cudaFreeAsync(const_cast<std::remove_const_t<T>*>(ptr), stream_);
  }
  template <typename T>
  T* to_internal_pointer(T* ptr) { return ptr; }
  template <typename T>
  void release_internal_pointer(T*) {}
  /** Pointers are their own memory objects here (the reference wraps them in USMMemObject). */
  template <typename T>
  T* get_mem_object(T* ptr, size_t) { return ptr; }
  template <typename T>
  T* get_mem_object_internal(T* ptr, size_t) { return ptr; }

  /** output = beta*output + op(lhs)*op(rhs), row-major; lhs is [m x k], rhs [k x n]. */
  template <bool TransposeLHS, bool TransposeRHS, typename T, typename Index>
  Event matmul(T const* lhs, T const* rhs, T* output, T beta, Index m, Index k, Index n) {
    check(pdnn_matmul(dtype_of<T>::value, TransposeLHS, TransposeRHS, lhs, rhs, output, 1, int(m), int(k), int(n),
                      float(beta), stream_));
    return Event{stream_};
  }
  /** Strided batches, output overwritten (beta = 0), as the reference's batch_matmul. */
  template <bool TransposeLHS, bool TransposeRHS, typename T, typename Index>
  Event batch_matmul(T const* lhs, T const* rhs, T* output, Index n_batches, Index m, Index k, Index n,
                     BatchFormat batch_type = BatchFormat::STRIDED) {
    if (batch_type != BatchFormat::STRIDED) throw std::runtime_error("CUDABackend: interleaved batches are not supported");
    check(pdnn_matmul(dtype_of<T>::value, TransposeLHS, TransposeRHS, lhs, rhs, output, int(n_batches), int(m), int(k),
                      int(n), 0.f, stream_));
    return Event{stream_};
  }

 private:
  static void check(int st) {
    if (st != PDNN_OK) throw std::runtime_error(pdnn_last_error());
  }
  cudaStream_t stream_;
};

template <typename Backend>
struct is_usm_backend : std::true_type {};
template <typename Backend>
struct supports_interleaved_matmul : std::false_type {};

}  // namespace backend
}  // namespace sycldnn
#endif
