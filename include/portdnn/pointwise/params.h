// sycldnn::pointwise::PointwiseParams (portDNN's include/portdnn/pointwise/params.h:28-35).
#ifndef PORTDNN_B200_POINTWISE_PARAMS_H_
#define PORTDNN_B200_POINTWISE_PARAMS_H_
namespace sycldnn {
namespace pointwise {
struct PointwiseParams {
  using Index = int;
  Index size;
};
}  // namespace pointwise
}  // namespace sycldnn
#endif
