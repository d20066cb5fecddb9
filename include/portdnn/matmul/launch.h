// Batched matrix multiply with the shape of portDNN's include/portdnn/matmul/{params.h:28-60,
// launch.h:37-90}: output[i] = beta*output[i] + op(lhs[i])*op(rhs[i]), row-major, strided batches.
#ifndef PORTDNN_B200_MATMUL_LAUNCH_H_
#define PORTDNN_B200_MATMUL_LAUNCH_H_
#include <vector>

#include "portdnn/backend/cuda_backend.h"
#include "portdnn/status.h"

namespace sycldnn {
namespace matmul {

struct MatmulParams {
  using Index = int;
  Index batches;
  Index m;
  Index k;
  Index n;
  float beta;
  sycldnn::BatchFormat batch_type = sycldnn::BatchFormat::STRIDED;
};

template <typename T, bool TransposeLHS, bool TransposeRHS, typename Backend>
SNNStatus launch(typename Backend::template pointer_type<T const> lhs, typename Backend::template pointer_type<T const> rhs,
                 typename Backend::template pointer_type<T> output, MatmulParams const& params, Backend& backend,
                 const std::vector<Event>& events = {}) {
  if (params.batch_type != BatchFormat::STRIDED) return StatusCode::InvalidParameter;
  for (const Event& e : events) e.make_stream_wait(backend.get_queue());
  const int st = pdnn_matmul(backend::dtype_of<T>::value, TransposeLHS, TransposeRHS, lhs, rhs, output, params.batches,
                             params.m, params.k, params.n, params.beta, backend.get_queue());
  return SNNStatus{Event{backend.get_queue()}, StatusCode(st)};
}

}  // namespace matmul
}  // namespace sycldnn
#endif
