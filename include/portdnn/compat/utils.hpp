// cuDNN-style handle and tensor descriptors, after portDNN's include/portdnn/compat/utils.hpp:51-400.
// The handle owns a CUDABackend on a CUDA stream where the reference owns an SNNUSMBackend on an
// in-order SYCL queue.
#ifndef PORTDNN_B200_COMPAT_UTILS_HPP_
#define PORTDNN_B200_COMPAT_UTILS_HPP_
#include <memory>
#include <vector>

#include "portdnn/backend/cuda_backend.h"
#include "portdnn/conv2d/params.h"
#include "portdnn/status.h"

namespace sycldnn {
namespace compat {

enum class SNNDataType { SNN_FLOAT = 0, SNN_DOUBLE, SNN_HALF };
enum class NanPropagation { NOT_PROPAGATE_NAN = 0, PROPAGATE_NAN };

/** One entry of the algorithm search results. */
struct convolutionFwdAlgoPerf_t {
  conv2d::Algorithm algo;
  StatusCode status;
  float time;
};

class SNNHandle {
 public:
  using Backend = backend::CUDABackend;
  SNNHandle() : backend_(new Backend(nullptr)) {}
  Backend& getBackend() { return *backend_; }
  cudaStream_t getQueue() const { return backend_->get_queue(); }
  void setStream(cudaStream_t stream) { backend_.reset(new Backend(stream)); }

 private:
  std::unique_ptr<Backend> backend_;
};

/** Creates the handle on the legacy default stream (the reference builds an in-order queue). */
inline StatusCode SNNCreate(SNNHandle& handle) {
  handle.setStream(nullptr);
  return StatusCode::OK;
}
/** queueSet of the reference, with the stream standing in for the queue. */
inline StatusCode queueSet(SNNHandle& handle, cudaStream_t stream) {
  handle.setStream(stream);
  return StatusCode::OK;
}

/** 4-d tensor descriptor.  The four extents are always given in n, c, h, w order whatever the
 * layout, like the reference (utils.hpp:210-342); the reported data type is always SNN_FLOAT. */
class TensorDescriptor {
 public:
  StatusCode set4d(DataFormat format, int n, int c, int h, int w) {
    if (n <= 0 || c <= 0 || h <= 0 || w <= 0) return StatusCode::InvalidParameter;
    format_ = format;
    n_ = n;
    c_ = c;
    h_ = h;
    w_ = w;
    return StatusCode::OK;
  }
  StatusCode get4dDescriptorDims(int* n, int* c, int* h, int* w) const {
    *n = n_;
    *c = c_;
    *h = h_;
    *w = w_;
    return StatusCode::OK;
  }
  DataFormat getFormat() const { return format_; }
  size_t getSize() const { return size_t(n_) * c_ * h_ * w_; }
  int n() const { return n_; }
  int c() const { return c_; }
  int h() const { return h_; }
  int w() const { return w_; }

 private:
  DataFormat format_ = DataFormat::NCHW;
  int n_ = 0, c_ = 0, h_ = 0, w_ = 0;
};

inline StatusCode setTensor4dDescriptor(TensorDescriptor& desc, DataFormat format, SNNDataType, int n, int c, int h,
                                        int w) {
  return desc.set4d(format, n, c, h, w);
}
inline StatusCode getTensor4dDescriptor(TensorDescriptor const& desc, SNNDataType* dataType, int* n, int* c, int* h,
                                        int* w, int* nStride, int* cStride, int* hStride, int* wStride) {
  *dataType = SNNDataType::SNN_FLOAT;
  desc.get4dDescriptorDims(n, c, h, w);
  if (desc.getFormat() == DataFormat::NHWC) {
    *cStride = 1;
    *wStride = *c;
    *hStride = *w * *c;
    *nStride = *h * *w * *c;
  } else {
    *wStride = 1;
    *hStride = *w;
    *cStride = *h * *w;
    *nStride = *c * *h * *w;
  }
  return StatusCode::OK;
}

namespace internal {
/** y = alpha*result + beta*y_prev around an operator that overwrites its output
 * (include/portdnn/compat/scaling.hpp:37-287): alpha == 0 skips the operator; result and previous
 * contents are blended in one pass.  `run(dst)` must queue the operator writing `dst`. */
template <typename T, typename Run>
SNNStatus scaled_launch(backend::CUDABackend& be, T alpha, T beta, T* y, size_t n, Run&& run) {
  auto near = [](T a, T b) { return (a > b ? a - b : b - a) < T(1e-9); };
  cudaStream_t s = be.get_queue();
  const int dt = backend::dtype_of<T>::value;
  if (near(alpha, T(0))) {
    if (near(beta, T(0))) {
      cudaMemsetAsync(y, 0, n * sizeof(T), s);
      return SNNStatus{Event{s}, StatusCode::OK};
    }
    return SNNStatus{Event{s}, StatusCode(pdnn_scale_blend(dt, y, float(beta), nullptr, 0.f, y, n, s))};
  }
  if (near(alpha, T(1)) && near(beta, T(0))) return run(y);
  T* tmp = be.allocate<T>(n);
  SNNStatus st = run(tmp);
  if (st.status == StatusCode::OK)
    st.status = StatusCode(pdnn_scale_blend(dt, tmp, float(alpha), y, float(beta), y, n, s));
  be.deallocate(tmp);
  return st;
}
}  // namespace internal

}  // namespace compat
}  // namespace sycldnn
#endif
