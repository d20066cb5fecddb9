// Pointwise activations with the launch forms of portDNN's include/portdnn/pointwise/launch.h:61-179.
// Relu, Tanh, Exp, Log, Floor and Sqrt are the reference's operators (operators.h:30-45); Relu6 is
// an addition (MobileNet-v2).  Floor has no gradient; asking for it returns InvalidParameter.
#ifndef PORTDNN_B200_POINTWISE_LAUNCH_H_
#define PORTDNN_B200_POINTWISE_LAUNCH_H_
#include <vector>

#include "portdnn/backend/cuda_backend.h"
#include "portdnn/status.h"

namespace sycldnn {
namespace pointwise {

struct Forward {};
struct Gradient {};
template <typename Direction>
struct Relu {};
template <typename Direction>
struct Tanh {};
template <typename Direction>
struct Relu6 {};
template <typename Direction>
struct Exp {};
template <typename Direction>
struct Log {};
template <typename Direction>
struct Floor {};
template <typename Direction>
struct Sqrt {};

namespace internal {
template <template <typename> class Op>
struct op_code;
template <>
struct op_code<Relu> { static constexpr int value = PDNN_ACT_RELU; };
template <>
struct op_code<Tanh> { static constexpr int value = PDNN_ACT_TANH; };
template <>
struct op_code<Relu6> { static constexpr int value = PDNN_ACT_RELU6; };
template <>
struct op_code<Exp> { static constexpr int value = PDNN_PW_EXP; };
template <>
struct op_code<Log> { static constexpr int value = PDNN_PW_LOG; };
template <>
struct op_code<Floor> { static constexpr int value = PDNN_PW_FLOOR; };
template <>
struct op_code<Sqrt> { static constexpr int value = PDNN_PW_SQRT; };
}  // namespace internal

/** output[i] = op(input[i]). */
template <typename T, template <typename> class Op, typename Direction, typename Backend,
          typename = typename std::enable_if<std::is_same<Direction, Forward>::value>::type>
SNNStatus launch(typename Backend::template pointer_type<T const> input,
                 typename Backend::template pointer_type<T> output, size_t n_items, Backend& backend,
                 const std::vector<Event>& events = {}) {
  for (const Event& e : events) e.make_stream_wait(backend.get_queue());
  const int st = pdnn_pointwise(internal::op_code<Op>::value, backend::dtype_of<T>::value, input, output, n_items,
                                backend.get_queue());
  return SNNStatus{Event{backend.get_queue()}, StatusCode(st)};
}

/** Gradient.  The first tensor is named input_forward in the reference's API but its kernel
 * treats it as the forward OUTPUT (src/pointwise/kernels.h:205-233); so does this one. */
template <typename T, template <typename> class Op, typename Direction, typename Backend,
          typename = typename std::enable_if<std::is_same<Direction, Gradient>::value>::type>
SNNStatus launch(typename Backend::template pointer_type<T const> input_forward,
                 typename Backend::template pointer_type<T const> input_backprop,
                 typename Backend::template pointer_type<T> output_backprop, size_t n_items, Backend& backend,
                 const std::vector<Event>& events = {}) {
  for (const Event& e : events) e.make_stream_wait(backend.get_queue());
  const int st = pdnn_pointwise_grad(internal::op_code<Op>::value, backend::dtype_of<T>::value, input_forward,
                                     input_backprop, output_backprop, n_items, backend.get_queue());
  return SNNStatus{Event{backend.get_queue()}, StatusCode(st)};
}

}  // namespace pointwise
}  // namespace sycldnn
#endif
