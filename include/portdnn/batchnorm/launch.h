// Batch normalisation with the parameter struct and the four launch forms of portDNN's
// include/portdnn/batchnorm/{params.h:32-72, direction.h, launch.h:222-470}.
#ifndef PORTDNN_B200_BATCHNORM_LAUNCH_H_
#define PORTDNN_B200_BATCHNORM_LAUNCH_H_
#include <type_traits>
#include <vector>

#include "portdnn/backend/cuda_backend.h"
#include "portdnn/status.h"

namespace sycldnn {
namespace batchnorm {

struct BatchNormParams {
  using Index = int;
  Index batch;
  Index rows;
  Index cols;
  Index channels;
  bool is_training;
  float epsilon = 0.001f;
  float momentum = 0.9f;
  sycldnn::DataFormat input_format = sycldnn::DataFormat::NHWC;
};

struct Forward {};
struct Gradient {};

namespace internal {
inline PdnnBatchNormParams to_c(BatchNormParams const& p) {
  return PdnnBatchNormParams{p.batch,   p.rows,     p.cols, p.channels, p.is_training ? 1 : 0,
                             p.epsilon, p.momentum, int(p.input_format)};
}
}  // namespace internal

/** The eight-pointer form (launch.h:222-320).  Forward: training statistics are written to
 * running_mean / running_variance when params.is_training; Gradient: the frozen gradient with the
 * population mean / variance in input_mean / input_variance. */
template <typename T, typename Backend, typename Direction>
SNNStatus launch(typename Backend::template pointer_type<T const> input,
                 typename Backend::template pointer_type<T const> beta_or_gradient,
                 typename Backend::template pointer_type<T const> gamma,
                 typename Backend::template pointer_type<T const> input_mean,
                 typename Backend::template pointer_type<T const> input_variance,
                 typename Backend::template pointer_type<T> running_mean_or_beta_grad,
                 typename Backend::template pointer_type<T> running_variance_or_gamma_grad,
                 typename Backend::template pointer_type<T> output, BatchNormParams const& params, Backend& backend,
                 const std::vector<Event>& events = {}) {
  for (const Event& e : events) e.make_stream_wait(backend.get_queue());
  const PdnnBatchNormParams p = internal::to_c(params);
  int st;
  if (std::is_same<Direction, Forward>::value)
    st = pdnn_batchnorm_forward(backend::dtype_of<T>::value, input, beta_or_gradient, gamma, input_mean, input_variance,
                                running_mean_or_beta_grad, running_variance_or_gamma_grad, output, &p,
                                backend.get_queue());
  else
    st = pdnn_batchnorm_gradient(backend::dtype_of<T>::value, input, beta_or_gradient, gamma, input_mean,
                                 input_variance, running_mean_or_beta_grad, running_variance_or_gamma_grad, output, &p,
                                 backend.get_queue());
  return SNNStatus{Event{backend.get_queue()}, StatusCode(st)};
}

/** Forward with frozen statistics (launch.h:322-400): six pointers. */
template <typename T, typename Backend, typename Direction,
          typename = typename std::enable_if<std::is_same<Direction, Forward>::value>::type>
SNNStatus launch(typename Backend::template pointer_type<T const> input,
                 typename Backend::template pointer_type<T const> beta,
                 typename Backend::template pointer_type<T const> gamma,
                 typename Backend::template pointer_type<T const> input_mean,
                 typename Backend::template pointer_type<T const> input_variance,
                 typename Backend::template pointer_type<T> output, BatchNormParams const& params, Backend& backend,
                 const std::vector<Event>& events = {}) {
  if (params.is_training) return StatusCode::InvalidParameter;  // the training form needs the running tensors
  for (const Event& e : events) e.make_stream_wait(backend.get_queue());
  const PdnnBatchNormParams p = internal::to_c(params);
  const int st = pdnn_batchnorm_forward(backend::dtype_of<T>::value, input, beta, gamma, input_mean, input_variance,
                                        nullptr, nullptr, output, &p, backend.get_queue());
  return SNNStatus{Event{backend.get_queue()}, StatusCode(st)};
}

/** Gradient with batch statistics (launch.h:402-470): six pointers. */
template <typename T, typename Backend, typename Direction,
          typename = typename std::enable_if<std::is_same<Direction, Gradient>::value>::type>
SNNStatus launch(typename Backend::template pointer_type<T const> input,
                 typename Backend::template pointer_type<T const> gradient,
                 typename Backend::template pointer_type<T const> gamma,
                 typename Backend::template pointer_type<T> beta_grad,
                 typename Backend::template pointer_type<T> gamma_grad,
                 typename Backend::template pointer_type<T> output, BatchNormParams const& params, Backend& backend,
                 const std::vector<Event>& events = {}, int = 0) {
  if (!params.is_training) return StatusCode::InvalidParameter;  // the frozen form needs the population statistics
  for (const Event& e : events) e.make_stream_wait(backend.get_queue());
  const PdnnBatchNormParams p = internal::to_c(params);
  const int st = pdnn_batchnorm_gradient(backend::dtype_of<T>::value, input, gradient, gamma, nullptr, nullptr,
                                         beta_grad, gamma_grad, output, &p, backend.get_queue());
  return SNNStatus{Event{backend.get_queue()}, StatusCode(st)};
}

}  // namespace batchnorm
}  // namespace sycldnn
#endif
