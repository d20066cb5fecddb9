// Binary operators with numpy-style broadcasting, after portDNN's include/portdnn/binaryop/
// {operators.h:29-35, params.h:31-44, launch.h:58-97}: Add, Sub, Mul, Div over operands of at most
// four extents each (an empty shape is a scalar).  The bias add of tools/layer.h:100-125 is the
// case lhs_dims = {rows, C}, rhs_dims = {1, C}.
#ifndef PORTDNN_B200_BINARYOP_LAUNCH_H_
#define PORTDNN_B200_BINARYOP_LAUNCH_H_
#include <vector>

#include "portdnn/backend/cuda_backend.h"
#include "portdnn/status.h"

namespace sycldnn {
namespace binaryop {

static constexpr int MAX_DIMS = 4;

struct Add {};
struct Sub {};
struct Mul {};
struct Div {};

namespace internal {
template <typename Op>
struct op_code;
template <>
struct op_code<Add> { static constexpr int value = PDNN_BINARY_ADD; };
template <>
struct op_code<Sub> { static constexpr int value = PDNN_BINARY_SUB; };
template <>
struct op_code<Mul> { static constexpr int value = PDNN_BINARY_MUL; };
template <>
struct op_code<Div> { static constexpr int value = PDNN_BINARY_DIV; };
}  // namespace internal

struct BinaryParams {
  std::vector<int> lhs_dims;
  std::vector<int> rhs_dims;
};

namespace internal {
inline size_t count(std::vector<int> const& dims) {
  size_t n = 1;
  for (int d : dims) n *= size_t(d);
  return n;
}
}  // namespace internal

template <typename T, typename Op, typename Backend>
SNNStatus launch(typename Backend::template pointer_type<T const> lhs, typename Backend::template pointer_type<T const> rhs,
                 typename Backend::template pointer_type<T> out, BinaryParams const& params, Backend& backend,
                 const std::vector<Event>& events = {}) {
  for (const Event& e : events) e.make_stream_wait(backend.get_queue());
  const int st = pdnn_binaryop(internal::op_code<Op>::value, backend::dtype_of<T>::value, lhs, params.lhs_dims.data(),
                               int(params.lhs_dims.size()), rhs, params.rhs_dims.data(), int(params.rhs_dims.size()),
                               out, backend.get_queue());
  return SNNStatus{Event{backend.get_queue()}, StatusCode(st)};
}

}  // namespace binaryop
}  // namespace sycldnn
#endif
