// Softmax over the channels of each pixel, with the parameter struct, sizes and launch forms of
// portDNN's include/portdnn/softmax/{params.h:27-54, sizes.h:31-54, direction.h, launch.h:64-165}.
// The workspace pointer of the reference's signature is accepted and ignored: one kernel does the
// reference's five passes.
#ifndef PORTDNN_B200_SOFTMAX_LAUNCH_H_
#define PORTDNN_B200_SOFTMAX_LAUNCH_H_
#include <type_traits>
#include <vector>

#include "portdnn/backend/cuda_backend.h"
#include "portdnn/status.h"

namespace sycldnn {
namespace softmax {

struct SoftmaxParams {
  using Index = int;
  Index channels;
  Index batch;
  Index rows;
  Index cols;
  sycldnn::DataFormat input_format = sycldnn::DataFormat::NHWC;
};
static_assert(sizeof(SoftmaxParams) == sizeof(PdnnSoftmaxParams), "must mirror the C struct");

struct Forward {};
struct Gradient {};

struct SoftmaxSizes {
  int input_size;
  int workspace_size;
  int output_size;
};
inline SoftmaxSizes get_sizes(SoftmaxParams const& p) {
  const int pixels = p.batch * p.rows * p.cols;
  return SoftmaxSizes{pixels * p.channels, pixels, pixels * p.channels};
}

/** output = softmax(input). */
template <typename T, typename Direction, typename Backend,
          typename = typename std::enable_if<std::is_same<Direction, Forward>::value>::type>
SNNStatus launch(typename Backend::template pointer_type<T const> input,
                 typename Backend::template pointer_type<T> /*workspace*/,
                 typename Backend::template pointer_type<T> output, SoftmaxParams const& params, Backend& backend,
                 const std::vector<Event>& events = {}) {
  for (const Event& e : events) e.make_stream_wait(backend.get_queue());
  const int st = pdnn_softmax(0, backend::dtype_of<T>::value, input, nullptr, output,
                              reinterpret_cast<const PdnnSoftmaxParams*>(&params), backend.get_queue());
  return SNNStatus{Event{backend.get_queue()}, StatusCode(st)};
}

/** output = (gradient - sum_c(gradient * input)) * input, `input` being the forward output. */
template <typename T, typename Direction, typename Backend,
          typename = typename std::enable_if<std::is_same<Direction, Gradient>::value>::type>
SNNStatus launch(typename Backend::template pointer_type<T const> input,
                 typename Backend::template pointer_type<T const> gradient,
                 typename Backend::template pointer_type<T> /*workspace*/,
                 typename Backend::template pointer_type<T> output, SoftmaxParams const& params, Backend& backend,
                 const std::vector<Event>& events = {}) {
  for (const Event& e : events) e.make_stream_wait(backend.get_queue());
  const int st = pdnn_softmax(1, backend::dtype_of<T>::value, input, gradient, output,
                              reinterpret_cast<const PdnnSoftmaxParams*>(&params), backend.get_queue());
  return SNNStatus{Event{backend.get_queue()}, StatusCode(st)};
}

}  // namespace softmax
}  // namespace sycldnn
#endif
