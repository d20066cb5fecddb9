// cuDNN-style wrappers of batch normalisation, after portDNN's include/portdnn/compat/batchnorm.hpp
// (modes :17-22, descriptor checks :34-80, inference :121-150, training :179-249, backward
// :279-346).  Argument meaning follows the reference, including two things a cuDNN user would not
// expect: `bnScale` is handed to the operator as its additive term (beta) and `bnBias` as its
// multiplicative term (gamma) in the forward calls (the reference's own test feeds them that way,
// test/compat/batchnorm_compat.cc:159-173), and the training call normalises with the running
// statistics it is given, then overwrites them with the blended ones.
#ifndef PORTDNN_B200_COMPAT_BATCHNORM_HPP_
#define PORTDNN_B200_COMPAT_BATCHNORM_HPP_
#include "portdnn/batchnorm/launch.h"
#include "portdnn/compat/utils.hpp"

namespace sycldnn {
namespace compat {

enum BatchNormMode {
  BATCHNORM_PER_ACTIVATION,  // scale and bias are 1xCxHxW: not supported, as in the reference
  BATCHNORM_SPATIAL,         // scale and bias are 1xCx1x1
  BATCHNORM_SPATIAL_PERSISTENT
};

namespace internal {
inline SNNStatus validateBatchnormParams(const TensorDescriptor& xDesc, const TensorDescriptor& yDesc,
                                         const TensorDescriptor& bnDesc, BatchNormMode mode) {
  const bool spatial = mode == BATCHNORM_SPATIAL || mode == BATCHNORM_SPATIAL_PERSISTENT;
  const bool same_shape = xDesc.n() == yDesc.n() && xDesc.c() == yDesc.c() && xDesc.h() == yDesc.h() &&
                          xDesc.w() == yDesc.w() && xDesc.getFormat() == yDesc.getFormat();
  const bool per_channel = bnDesc.n() == 1 && bnDesc.c() == xDesc.c() && bnDesc.h() == 1 && bnDesc.w() == 1;
  return (spatial && same_shape && per_channel) ? StatusCode::OK : StatusCode::InvalidParameter;
}

inline batchnorm::BatchNormParams descToSnnBatchnormParams(const TensorDescriptor& xDesc, bool is_training,
                                                           float epsilon) {
  batchnorm::BatchNormParams p{};
  p.batch = xDesc.n();
  p.rows = xDesc.h();
  p.cols = xDesc.w();
  p.channels = xDesc.c();
  p.is_training = is_training;
  p.epsilon = epsilon;
  p.input_format = xDesc.getFormat();
  return p;
}
}  // namespace internal

/** y = alpha * batchnorm(x; estimatedMean, estimatedVariance) + beta * y. */
template <typename ValueT>
SNNStatus batchNormalizationForwardInference(SNNHandle& handle, BatchNormMode mode, const ValueT* alpha,
                                             const ValueT* beta, const TensorDescriptor& xDesc, const void* x,
                                             const TensorDescriptor& yDesc, void* y, const TensorDescriptor& bnDesc,
                                             const void* bnScale, const void* bnBias, const void* estimatedMean,
                                             const void* estimatedVariance, double epsilon) {
  SNNStatus v = internal::validateBatchnormParams(xDesc, yDesc, bnDesc, mode);
  if (v.status != StatusCode::OK) return v;
  using Backend = SNNHandle::Backend;
  const batchnorm::BatchNormParams p = internal::descToSnnBatchnormParams(xDesc, false, float(epsilon));
  Backend& be = handle.getBackend();
  return internal::scaled_launch<ValueT>(be, *alpha, *beta, static_cast<ValueT*>(y), yDesc.getSize(), [&](ValueT* dst) {
    return batchnorm::launch<ValueT, Backend, batchnorm::Forward>(
        static_cast<const ValueT*>(x), static_cast<const ValueT*>(bnScale), static_cast<const ValueT*>(bnBias),
        static_cast<const ValueT*>(estimatedMean), static_cast<const ValueT*>(estimatedVariance), nullptr, nullptr,
        dst, p, be);
  });
}

/** Training forward: y = alpha * batchnorm(x; running statistics as given) + beta * y, and
 * running = batch * exponentialAverageFactor + running * (1 - exponentialAverageFactor), with the
 * biased batch variance.  resultSaveMean / resultSaveInvVariance, when given, receive the same
 * blended statistics (the reference stores them there first and copies them to the running
 * tensors).  With alpha == 0 the statistics are still updated and y becomes beta * y (the
 * reference in that corner scales the fresh result by beta instead, an artefact of the order of
 * its scaling passes). */
template <typename ValueT>
SNNStatus batchNormalizationForwardTraining(SNNHandle& handle, BatchNormMode mode, const ValueT* alpha,
                                            const ValueT* beta, const TensorDescriptor& xDesc, const void* x,
                                            const TensorDescriptor& yDesc, void* y, const TensorDescriptor& bnDesc,
                                            const void* bnScale, const void* bnBias, double exponentialAverageFactor,
                                            void* resultRunningMean, void* resultRunningVariance, double epsilon,
                                            void* resultSaveMean, void* resultSaveInvVariance) {
  SNNStatus v = internal::validateBatchnormParams(xDesc, yDesc, bnDesc, mode);
  if (v.status != StatusCode::OK) return v;
  if (!resultSaveMean != !resultSaveInvVariance) return StatusCode::InvalidParameter;  // both or neither
  using Backend = SNNHandle::Backend;
  Backend& be = handle.getBackend();
  cudaStream_t s = be.get_queue();
  batchnorm::BatchNormParams p = internal::descToSnnBatchnormParams(xDesc, true, float(epsilon));
  p.momentum = float(1.0 - exponentialAverageFactor);
  const size_t c = size_t(p.channels), n = yDesc.getSize();
  ValueT* new_mean = static_cast<ValueT*>(resultSaveMean);
  ValueT* new_var = static_cast<ValueT*>(resultSaveInvVariance);
  ValueT* stats_tmp = nullptr;
  if (new_mean == nullptr) {
    stats_tmp = be.template allocate<ValueT>(2 * c);
    new_mean = stats_tmp;
    new_var = stats_tmp + c;
  }
  auto near = [](ValueT a, ValueT b) { return (a > b ? a - b : b - a) < ValueT(1e-9); };
  const bool plain = near(*alpha, ValueT(1)) && near(*beta, ValueT(0));
  ValueT* dst = plain ? static_cast<ValueT*>(y) : be.template allocate<ValueT>(n);
  SNNStatus st = batchnorm::launch<ValueT, Backend, batchnorm::Forward>(
      static_cast<const ValueT*>(x), static_cast<const ValueT*>(bnScale), static_cast<const ValueT*>(bnBias),
      static_cast<const ValueT*>(resultRunningMean), static_cast<const ValueT*>(resultRunningVariance), new_mean,
      new_var, dst, p, be);
  if (st.status == StatusCode::OK) {
    cudaMemcpyAsync(resultRunningMean, new_mean, c * sizeof(ValueT), cudaMemcpyDeviceToDevice, s);
    cudaMemcpyAsync(resultRunningVariance, new_var, c * sizeof(ValueT), cudaMemcpyDeviceToDevice, s);
    if (!plain)
      st.status = StatusCode(pdnn_scale_blend(backend::dtype_of<ValueT>::value, dst, float(*alpha), y, float(*beta), y,
                                              n, s));
  }
  if (!plain) be.deallocate(dst);
  if (stats_tmp != nullptr) be.deallocate(stats_tmp);
  return SNNStatus{Event{s}, st.status};
}

/** Backward with batch statistics: dx = alphaDataDiff * d/dx + betaDataDiff * dx, and both
 * parameter gradients blended with alphaParamDiff / betaParamDiff.  `bnScale` is the operator's
 * gamma here; resultBnScaleDiff receives the gradient of the additive term and resultBnBiasDiff
 * that of the multiplicative one, in the reference's argument order (compat/batchnorm.hpp:317-325).
 * savedMean / savedInvVariance are ignored, as in the reference. */
template <typename ValueT>
SNNStatus batchNormalizationBackward(SNNHandle& handle, BatchNormMode mode, const ValueT* alphaDataDiff,
                                     const ValueT* betaDataDiff, const ValueT* alphaParamDiff,
                                     const ValueT* betaParamDiff, const TensorDescriptor& xDesc, const void* x,
                                     const TensorDescriptor& dyDesc, const void* dy, const TensorDescriptor& dxDesc,
                                     void* dx, const TensorDescriptor& bnScaleBiasDiffDesc, const void* bnScale,
                                     void* resultBnScaleDiff, void* resultBnBiasDiff, double epsilon,
                                     const void* /*savedMean*/, const void* /*savedInvVariance*/) {
  for (const TensorDescriptor* d : {&dxDesc, &dyDesc}) {
    SNNStatus v = internal::validateBatchnormParams(xDesc, *d, bnScaleBiasDiffDesc, mode);
    if (v.status != StatusCode::OK) return v;
  }
  using Backend = SNNHandle::Backend;
  Backend& be = handle.getBackend();
  cudaStream_t s = be.get_queue();
  const int dt = backend::dtype_of<ValueT>::value;
  const batchnorm::BatchNormParams p = internal::descToSnnBatchnormParams(xDesc, true, float(epsilon));
  const size_t c = size_t(p.channels), n = dxDesc.getSize();
  auto near = [](ValueT a, ValueT b) { return (a > b ? a - b : b - a) < ValueT(1e-9); };
  const bool plain_data = near(*alphaDataDiff, ValueT(1)) && near(*betaDataDiff, ValueT(0));
  const bool plain_param = near(*alphaParamDiff, ValueT(1)) && near(*betaParamDiff, ValueT(0));
  ValueT* dx_dst = plain_data ? static_cast<ValueT*>(dx) : be.template allocate<ValueT>(n);
  ValueT* pg = plain_param ? nullptr : be.template allocate<ValueT>(2 * c);
  ValueT* dscale = plain_param ? static_cast<ValueT*>(resultBnScaleDiff) : pg;
  ValueT* dbias = plain_param ? static_cast<ValueT*>(resultBnBiasDiff) : pg + c;
  SNNStatus st = batchnorm::launch<ValueT, Backend, batchnorm::Gradient>(
      static_cast<const ValueT*>(x), static_cast<const ValueT*>(dy), static_cast<const ValueT*>(bnScale), nullptr,
      nullptr, dscale, dbias, dx_dst, p, be);
  if (st.status == StatusCode::OK && !plain_data)
    st.status = StatusCode(pdnn_scale_blend(dt, dx_dst, float(*alphaDataDiff), dx, float(*betaDataDiff), dx, n, s));
  if (st.status == StatusCode::OK && !plain_param) {
    st.status = StatusCode(pdnn_scale_blend(dt, dscale, float(*alphaParamDiff), resultBnScaleDiff,
                                            float(*betaParamDiff), resultBnScaleDiff, c, s));
    if (st.status == StatusCode::OK)
      st.status = StatusCode(pdnn_scale_blend(dt, dbias, float(*alphaParamDiff), resultBnBiasDiff,
                                              float(*betaParamDiff), resultBnBiasDiff, c, s));
  }
  if (!plain_data) be.deallocate(dx_dst);
  if (pg != nullptr) be.deallocate(pg);
  return SNNStatus{Event{s}, st.status};
}

}  // namespace compat
}  // namespace sycldnn
#endif
