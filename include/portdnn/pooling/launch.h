// Pooling: params, operator and direction tags, sizes and the two launch forms of portDNN's
// include/portdnn/pooling/{params.h:30-73, operators.h, sizes.h, launch.h:112-257}.
#ifndef PORTDNN_B200_POOLING_LAUNCH_H_
#define PORTDNN_B200_POOLING_LAUNCH_H_
#include <type_traits>
#include <vector>

#include "portdnn/backend/cuda_backend.h"
#include "portdnn/status.h"

namespace sycldnn {
namespace pooling {

struct PoolingParams {
  using Index = int;
  Index in_rows;
  Index in_cols;
  Index out_rows;
  Index out_cols;
  Index window_rows;
  Index window_cols;
  Index stride_rows;
  Index stride_cols;
  Index batch;
  Index channels;
  Index pad_rows;
  Index pad_cols;
  sycldnn::DataFormat input_format = sycldnn::DataFormat::NHWC;
};
static_assert(sizeof(PoolingParams) == sizeof(PdnnPoolingParams), "must mirror the C struct");

// Operator tags are class templates in the reference (template <typename> class Op).
template <typename T>
struct Max {};
template <typename T>
struct MaxWithNan {};
template <typename T>
struct Average {};
struct Forward {};
struct Backpropagate {};

namespace internal {
template <template <typename> class Op>
struct op_code;
template <>
struct op_code<Max> { static constexpr int value = PDNN_POOL_MAX; };
template <>
struct op_code<MaxWithNan> { static constexpr int value = PDNN_POOL_MAX_WITH_NAN; };
template <>
struct op_code<Average> { static constexpr int value = PDNN_POOL_AVERAGE; };
template <typename T, template <typename> class Op, typename Direction>
struct IsMaxGradient
    : std::integral_constant<bool, std::is_same<Direction, Backpropagate>::value && op_code<Op>::value != PDNN_POOL_AVERAGE> {};
}  // namespace internal

struct PoolingSizes {
  size_t input_size;
  size_t output_size;
};
template <typename Direction>
inline PoolingSizes get_sizes(PoolingParams const& p) {
  const size_t in = size_t(p.batch) * p.in_rows * p.in_cols * p.channels;
  const size_t out = size_t(p.batch) * p.out_rows * p.out_cols * p.channels;
  return std::is_same<Direction, Forward>::value ? PoolingSizes{in, out} : PoolingSizes{out, in};
}

/** Forward for every operator; Backpropagate for Average (input = dy, output = dx). */
template <typename T, template <typename> class Op, typename Direction, typename Backend,
          typename = typename std::enable_if<!internal::IsMaxGradient<T, Op, Direction>::value>::type>
SNNStatus launch(typename Backend::template pointer_type<T const> input,
                 typename Backend::template pointer_type<T> output, PoolingParams const& pp, Backend& backend,
                 const std::vector<Event>& events = {}) {
  for (const Event& e : events) e.make_stream_wait(backend.get_queue());
  const int st = pdnn_pooling(internal::op_code<Op>::value, std::is_same<Direction, Forward>::value ? 0 : 1,
                              backend::dtype_of<T>::value, input, output,
                              reinterpret_cast<const PdnnPoolingParams*>(&pp), backend.get_queue());
  return SNNStatus{Event{backend.get_queue()}, StatusCode(st)};
}

/** Max / MaxWithNan gradient: (x, y, dy) -> dx. */
template <typename T, template <typename> class Op, typename Direction, typename Backend,
          typename = typename std::enable_if<internal::IsMaxGradient<T, Op, Direction>::value>::type>
SNNStatus launch(typename Backend::template pointer_type<T const> input_data,
                 typename Backend::template pointer_type<T const> output_data,
                 typename Backend::template pointer_type<T const> input_backprop,
                 typename Backend::template pointer_type<T> output_backprop, PoolingParams const& pp, Backend& backend,
                 const std::vector<Event>& events = {}) {
  for (const Event& e : events) e.make_stream_wait(backend.get_queue());
  const int st = pdnn_pooling_max_grad(internal::op_code<Op>::value, backend::dtype_of<T>::value, input_data, output_data,
                                       input_backprop, output_backprop,
                                       reinterpret_cast<const PdnnPoolingParams*>(&pp), backend.get_queue());
  return SNNStatus{Event{backend.get_queue()}, StatusCode(st)};
}

}  // namespace pooling
}  // namespace sycldnn
#endif
