// Convolution parameters, conv-type tags, algorithm tags and tensor sizes: the types of
// portDNN's include/portdnn/conv2d/{params.h:32-112, conv_type.h:32-48, algorithm.h:30-45,
// sizes.h:34-179} with the same names, field order and enumerator values, so that code written
// against the reference compiles unchanged.  Conv2DParams is layout-compatible with the C ABI's
// PdnnConv2DParams (checked below).
#ifndef PORTDNN_B200_CONV2D_PARAMS_H_
#define PORTDNN_B200_CONV2D_PARAMS_H_
#include <cstddef>

#include "portdnn/data_format.h"
#include "portdnn_b200.h"

namespace sycldnn {
namespace conv2d {

struct Conv2DParams {
  using Index = int;
  Index channels;
  Index features;
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
  Index dilation_rows = 1;
  Index dilation_cols = 1;
  Index groups = 1;
  sycldnn::DataFormat input_format = sycldnn::DataFormat::NHWC;
  sycldnn::FilterFormat filter_format = sycldnn::FilterFormat::HWCF;
  sycldnn::BatchFormat group_format = sycldnn::BatchFormat::STRIDED;
};
static_assert(sizeof(Conv2DParams) == sizeof(PdnnConv2DParams), "Conv2DParams must mirror PdnnConv2DParams");

namespace conv_type {
struct Forward {};
struct InputBackprop {};
struct FilterBackprop {};
}  // namespace conv_type

enum class Algorithm { NotSupported, Direct, Tiled, Im2col, Winograd, WinogradLarge, Matmul };

/** PdnnPass of a conv-type tag. */
template <typename ConvType>
struct pass_of;
template <>
struct pass_of<conv_type::Forward> { static constexpr int value = PDNN_FORWARD; };
template <>
struct pass_of<conv_type::InputBackprop> { static constexpr int value = PDNN_INPUT_BACKPROP; };
template <>
struct pass_of<conv_type::FilterBackprop> { static constexpr int value = PDNN_FILTER_BACKPROP; };

/** Element counts of the three argument slots of launch<ConvType>. */
struct ConvSizes {
  size_t input_size;
  size_t filter_size;
  size_t output_size;
};

template <typename ConvType>
inline ConvSizes get_sizes(Conv2DParams const& p) {
  const size_t x = size_t(p.batch) * p.in_rows * p.in_cols * p.channels;
  const size_t w = size_t(p.window_rows) * p.window_cols * (p.channels / (p.groups > 0 ? p.groups : 1)) * p.features;
  const size_t y = size_t(p.batch) * p.out_rows * p.out_cols * p.features;
  switch (pass_of<ConvType>::value) {
    case PDNN_INPUT_BACKPROP: return {y, w, x};   // (dy, w) -> dx
    case PDNN_FILTER_BACKPROP: return {x, y, w};  // (x, dy) -> dW: dy sits in the filter slot
    default: return {x, w, y};
  }
}

}  // namespace conv2d
}  // namespace sycldnn
#endif
