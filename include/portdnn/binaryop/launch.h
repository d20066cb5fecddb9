// Binary ops in the two forms the convolution path uses (portDNN's include/portdnn/binaryop/
// launch.h:58-97, params.h:34-44): Add with a [rows, C] left side and a [1, C] right side (the
// bias add of tools/layer.h:100-125) and elementwise / scalar Mul and Add (the compat layer's
// alpha/beta blend).  General N-d broadcasting is outside the hot path and reports
// InvalidParameter.
#ifndef PORTDNN_B200_BINARYOP_LAUNCH_H_
#define PORTDNN_B200_BINARYOP_LAUNCH_H_
#include <vector>

#include "portdnn/backend/cuda_backend.h"
#include "portdnn/status.h"

namespace sycldnn {
namespace binaryop {

struct Add {};
struct Mul {};

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
  const size_t ln = internal::count(params.lhs_dims), rn = internal::count(params.rhs_dims);
  if (ln == 0 || rn == 0) return StatusCode::InvalidParameter;
  int st = PDNN_INVALID_PARAMETER;
  if (std::is_same<Op, Add>::value && rn < ln && !params.rhs_dims.empty() && ln % rn == 0 &&
      params.rhs_dims.back() == int(rn)) {
    // right side is one row of `rn` channels broadcast over every row of the left side
    st = pdnn_bias_add(backend::dtype_of<T>::value, lhs, rhs, out, ln / rn, int(rn), PDNN_ACT_NONE, backend.get_queue());
  } else if (std::is_same<Op, Add>::value && ln == rn) {
    st = pdnn_scale_blend(backend::dtype_of<T>::value, lhs, 1.f, rhs, 1.f, out, ln, backend.get_queue());
  }
  return SNNStatus{Event{backend.get_queue()}, StatusCode(st)};
}

}  // namespace binaryop
}  // namespace sycldnn
#endif
