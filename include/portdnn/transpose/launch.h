// Tensor transposition with the launch forms of portDNN's include/portdnn/transpose/launch.h:66-233:
// transpose::launch<T>(input, output, dimensions, permutation, backend) and the two layout
// conversions.  Output extent d is dimensions[permutation[d]].
#ifndef PORTDNN_B200_TRANSPOSE_LAUNCH_H_
#define PORTDNN_B200_TRANSPOSE_LAUNCH_H_
#include <vector>

#include "portdnn/backend/cuda_backend.h"
#include "portdnn/status.h"

namespace sycldnn {

/** The permutations of include/portdnn/internal/transpose/launch.h:32-33. */
const std::vector<int> NHWC_TO_NCHW{0, 3, 1, 2};
const std::vector<int> NCHW_TO_NHWC{0, 2, 3, 1};

namespace transpose {

/** As the reference: up to six dimensions, the permutation must name every dimension once
 * (src/transpose/launch.cc validates the same); InvalidParameter otherwise. */
template <typename T, typename Backend>
SNNStatus launch(typename Backend::template pointer_type<T const> input,
                 typename Backend::template pointer_type<T> output, std::vector<int> const& dimensions,
                 std::vector<int> const& permutation, Backend& backend, const std::vector<Event>& events = {}) {
  if (dimensions.empty() || dimensions.size() != permutation.size())
    return SNNStatus{Event{backend.get_queue()}, StatusCode::InvalidParameter};
  for (const Event& e : events) e.make_stream_wait(backend.get_queue());
  const int st = pdnn_transpose(int(sizeof(T)), input, output, dimensions.data(), int(dimensions.size()),
                                permutation.data(), backend.get_queue());
  return SNNStatus{Event{backend.get_queue()}, StatusCode(st)};
}

template <typename T, typename Backend>
SNNStatus convert_nhwc_to_nchw(typename Backend::template pointer_type<T const> input,
                               typename Backend::template pointer_type<T> output, std::vector<int> const& dimensions,
                               Backend& backend, const std::vector<Event>& events = {}) {
  if (dimensions.size() != 4) return SNNStatus{Event{backend.get_queue()}, StatusCode::InvalidParameter};
  return launch<T>(input, output, dimensions, NHWC_TO_NCHW, backend, events);
}

template <typename T, typename Backend>
SNNStatus convert_nchw_to_nhwc(typename Backend::template pointer_type<T const> input,
                               typename Backend::template pointer_type<T> output, std::vector<int> const& dimensions,
                               Backend& backend, const std::vector<Event>& events = {}) {
  if (dimensions.size() != 4) return SNNStatus{Event{backend.get_queue()}, StatusCode::InvalidParameter};
  return launch<T>(input, output, dimensions, NCHW_TO_NHWC, backend, events);
}

}  // namespace transpose
}  // namespace sycldnn
#endif
