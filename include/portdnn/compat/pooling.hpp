// cuDNN-style pooling forward, after portDNN's include/portdnn/compat/pooling.hpp:31-239.  As in
// the reference only POOLING_MAX_DETERMINISTIC and POOLING_AVERAGE_COUNT_EXCLUDE_PADDING are
// accepted (pooling.hpp:111-115).
#ifndef PORTDNN_B200_COMPAT_POOLING_HPP_
#define PORTDNN_B200_COMPAT_POOLING_HPP_
#include "portdnn/compat/utils.hpp"
#include "portdnn/pooling/launch.h"

namespace sycldnn {
namespace compat {

enum class PoolingMode {
  POOLING_MAX = 0,
  POOLING_AVERAGE_COUNT_INCLUDE_PADDING,
  POOLING_AVERAGE_COUNT_EXCLUDE_PADDING,
  POOLING_MAX_DETERMINISTIC
};

class PoolingDescriptor {
 public:
  StatusCode set2d(int window_h, int window_w, int pad_h, int pad_w, int stride_h, int stride_w, PoolingMode mode,
                   NanPropagation nan_opt) {
    if (window_h <= 0 || window_w <= 0 || pad_h < 0 || pad_w < 0 || stride_h <= 0 || stride_w <= 0)
      return StatusCode::InvalidParameter;
    if (mode == PoolingMode::POOLING_MAX || mode == PoolingMode::POOLING_AVERAGE_COUNT_INCLUDE_PADDING)
      return StatusCode::InvalidParameter;
    window_h_ = window_h;
    window_w_ = window_w;
    pad_h_ = pad_h;
    pad_w_ = pad_w;
    stride_h_ = stride_h;
    stride_w_ = stride_w;
    mode_ = mode;
    nan_ = nan_opt;
    return StatusCode::OK;
  }
  PoolingMode getMode() const { return mode_; }
  NanPropagation getMaxPoolNanOpt() const { return nan_; }
  int window_h_ = 1, window_w_ = 1, pad_h_ = 0, pad_w_ = 0, stride_h_ = 1, stride_w_ = 1;

 private:
  PoolingMode mode_ = PoolingMode::POOLING_MAX_DETERMINISTIC;
  NanPropagation nan_ = NanPropagation::NOT_PROPAGATE_NAN;
};

inline StatusCode setPooling2dDescriptor(PoolingDescriptor& desc, PoolingMode mode, NanPropagation nan_opt, int window_h,
                                         int window_w, int pad_h, int pad_w, int stride_h, int stride_w) {
  return desc.set2d(window_h, window_w, pad_h, pad_w, stride_h, stride_w, mode, nan_opt);
}

/** y = alpha * pool(x) + beta * y. */
template <typename ValueT>
SNNStatus poolingForward(SNNHandle& handle, PoolingDescriptor const& poolDesc, const ValueT* alpha,
                         TensorDescriptor const& xDesc, const void* x, const ValueT* beta,
                         TensorDescriptor const& yDesc, void* y) {
  pooling::PoolingParams p{};
  p.in_rows = xDesc.h();
  p.in_cols = xDesc.w();
  p.out_rows = yDesc.h();
  p.out_cols = yDesc.w();
  p.window_rows = poolDesc.window_h_;
  p.window_cols = poolDesc.window_w_;
  p.stride_rows = poolDesc.stride_h_;
  p.stride_cols = poolDesc.stride_w_;
  p.batch = xDesc.n();
  p.channels = xDesc.c();
  p.pad_rows = poolDesc.pad_h_;
  p.pad_cols = poolDesc.pad_w_;
  p.input_format = xDesc.getFormat();
  auto& be = handle.getBackend();
  return internal::scaled_launch<ValueT>(be, *alpha, *beta, static_cast<ValueT*>(y), yDesc.getSize(), [&](ValueT* dst) {
    const ValueT* in = static_cast<const ValueT*>(x);
    if (poolDesc.getMode() != PoolingMode::POOLING_MAX_DETERMINISTIC)
      return pooling::launch<ValueT, pooling::Average, pooling::Forward>(in, dst, p, be);
    if (poolDesc.getMaxPoolNanOpt() == NanPropagation::NOT_PROPAGATE_NAN)
      return pooling::launch<ValueT, pooling::Max, pooling::Forward>(in, dst, p, be);
    return pooling::launch<ValueT, pooling::MaxWithNan, pooling::Forward>(in, dst, p, be);
  });
}

}  // namespace compat
}  // namespace sycldnn
#endif
