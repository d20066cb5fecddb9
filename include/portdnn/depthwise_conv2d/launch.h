// Depthwise convolution: params, sizes and launch with the shapes of portDNN's
// include/portdnn/depthwise_conv2d/{params.h:33-94, sizes.h, launch.h:54-91}.
#ifndef PORTDNN_B200_DEPTHWISE_CONV2D_LAUNCH_H_
#define PORTDNN_B200_DEPTHWISE_CONV2D_LAUNCH_H_
#include <vector>

#include "portdnn/backend/cuda_backend.h"
#include "portdnn/conv2d/params.h"
#include "portdnn/status.h"

namespace sycldnn {
namespace depthwise_conv2d {

struct DepthwiseConv2DParams {
  using Index = int;
  Index channels;
  Index channel_multiplier;
  Index batch;
  Index in_rows;
  Index in_cols;
  Index window_rows;
  Index window_cols;
  Index stride_rows;
  Index stride_cols;
  Index out_rows;
  Index out_cols;
  Index pad_rows;
  Index pad_cols;
};
static_assert(sizeof(DepthwiseConv2DParams) == sizeof(PdnnDepthwiseConv2DParams), "must mirror the C struct");

struct ConvSizes {
  size_t input_size;
  size_t filter_size;
  size_t output_size;
};

template <typename ConvType>
inline ConvSizes get_sizes(DepthwiseConv2DParams const& p) {
  const size_t x = size_t(p.batch) * p.in_rows * p.in_cols * p.channels;
  const size_t w = size_t(p.window_rows) * p.window_cols * p.channels * p.channel_multiplier;
  const size_t y = size_t(p.batch) * p.out_rows * p.out_cols * p.channels * p.channel_multiplier;
  switch (conv2d::pass_of<ConvType>::value) {
    case PDNN_INPUT_BACKPROP: return {y, w, x};
    case PDNN_FILTER_BACKPROP: return {x, y, w};
    default: return {x, w, y};
  }
}

/** Slots as for conv2d::launch.  The filter backprop's scratch comes from the stream-ordered
 * allocator (the reference's launch has no workspace argument either). */
template <typename T, typename ConvType, typename Backend>
SNNStatus launch(typename Backend::template pointer_type<T const> input,
                 typename Backend::template pointer_type<T const> filter,
                 typename Backend::template pointer_type<T> output, DepthwiseConv2DParams const& params,
                 Backend& backend, const std::vector<Event>& events = {}) {
  for (const Event& e : events) e.make_stream_wait(backend.get_queue());
  const int st = pdnn_depthwise_conv2d(conv2d::pass_of<ConvType>::value, backend::dtype_of<T>::value, input, filter,
                                       output, reinterpret_cast<const PdnnDepthwiseConv2DParams*>(&params), nullptr, 0,
                                       backend.get_queue());
  return SNNStatus{Event{backend.get_queue()}, StatusCode(st)};
}

}  // namespace depthwise_conv2d
}  // namespace sycldnn
#endif
