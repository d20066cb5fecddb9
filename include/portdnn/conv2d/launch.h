// conv2d::launch and conv2d::query_workspace_size with the signatures of portDNN's
// include/portdnn/conv2d/launch.h:59-118 and include/portdnn/conv2d/workspace_size.h:42-163,
// forwarding to the C ABI (pdnn_conv2d, pdnn_conv2d_workspace_size).  Status precedence is the
// reference's (include/portdnn/internal/conv2d/launch.h:169-207): parameter validation, then the
// selector, then layout/group restrictions, then the launcher.
#ifndef PORTDNN_B200_CONV2D_LAUNCH_H_
#define PORTDNN_B200_CONV2D_LAUNCH_H_
#include <vector>

#include "portdnn/backend/cuda_backend.h"
#include "portdnn/conv2d/params.h"
#include "portdnn/conv2d/selector/selector.h"
#include "portdnn/status.h"

namespace sycldnn {
namespace conv2d {

/** Scratch sizes in ELEMENTS of the tensor type, like the reference. */
struct WorkspaceSize {
  size_t required_size;
  size_t recommended_size;
};

/** The implicit-GEMM kernels need no scratch; the split reduction of the filter backprop and
 * the packed input of few-channel stems are reported as the recommended size (without it the
 * library allocates for the duration of the call). */
template <typename ConvType, typename T = float>
WorkspaceSize query_workspace_size(Conv2DParams const& params, Selector& selector) {
  WorkspaceSize ws{0, 0};
  const Algorithm algo = selector.select<ConvType>(params);
  if (algo == Algorithm::NotSupported) return ws;
  pdnn_conv2d_workspace_size(pass_of<ConvType>::value, backend::dtype_of<T>::value,
                             reinterpret_cast<const PdnnConv2DParams*>(&params), int(algo), &ws.required_size,
                             &ws.recommended_size);
  return ws;
}

/** Optional fused epilogue (no counterpart in the reference, which chains separate launches):
 * out = act(alpha*conv + bias) + beta*out. */
struct FusedEpilogue {
  const void* bias = nullptr;
  int activation = PDNN_ACT_NONE;
  float alpha = 1.f;
  float beta = 0.f;
  void* relu_bitmask = nullptr;  // PdnnConvEpilogue::relu_bitmask
  bool constant_filter = false;  // PdnnConvEpilogue::constant_filter
};

template <typename T, typename ConvType, typename Backend>
SNNStatus launch(typename Backend::template pointer_type<T const> input,
                 typename Backend::template pointer_type<T const> filter,
                 typename Backend::template pointer_type<T> output, Conv2DParams const& params, Selector& selector,
                 Backend& backend, typename Backend::template pointer_type<T> workspace, size_t workspace_size,
                 const std::vector<Event>& events = {}) {
  const PdnnConv2DParams* cp = reinterpret_cast<const PdnnConv2DParams*>(&params);
  // validation first, with an algorithm tag that cannot itself fail
  const int pre = pdnn_conv2d_validate(pass_of<ConvType>::value, cp, params.groups > 1 ? PDNN_ALGO_IM2COL
                                                                     : params.input_format == DataFormat::NCHW
                                                                         ? PDNN_ALGO_DIRECT
                                                                         : PDNN_ALGO_IM2COL);
  if (pre == PDNN_INVALID_PARAMETER) return StatusCode::InvalidParameter;
  const Algorithm algo = selector.select<ConvType>(params);
  for (const Event& e : events) e.make_stream_wait(backend.get_queue());
  const int st = pdnn_conv2d(pass_of<ConvType>::value, backend::dtype_of<T>::value, input, filter, output, cp, int(algo),
                             workspace, workspace_size, backend.get_queue());
  return SNNStatus{Event{backend.get_queue()}, StatusCode(st)};
}

/** Forward convolution with the fused epilogue. */
template <typename T, typename Backend>
SNNStatus launch_fused(T const* input, T const* filter, T* output, Conv2DParams const& params, Selector& selector,
                       Backend& backend, FusedEpilogue const& epilogue, T* workspace = nullptr, size_t workspace_size = 0) {
  const Algorithm algo = selector.select<conv_type::Forward>(params);
  const PdnnConvEpilogue e{epilogue.bias,         epilogue.activation, epilogue.alpha, epilogue.beta,
                           epilogue.relu_bitmask, epilogue.constant_filter ? 1 : 0};
  const int st = pdnn_conv2d_fused(backend::dtype_of<T>::value, input, filter, output,
                                   reinterpret_cast<const PdnnConv2DParams*>(&params), int(algo), &e, workspace,
                                   workspace_size, backend.get_queue());
  return SNNStatus{Event{backend.get_queue()}, StatusCode(st)};
}

}  // namespace conv2d
}  // namespace sycldnn
#endif
