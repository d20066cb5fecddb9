// TensorFlow-style padding arithmetic, after portDNN's include/portdnn/helpers/padding.h:46-88 and
// include/portdnn/helpers/ratio.h:43-79.  Only the low-side pad is stored; the high side follows
// from the output size.
#ifndef PORTDNN_B200_HELPERS_PADDING_H_
#define PORTDNN_B200_HELPERS_PADDING_H_
#include "portdnn/data_format.h"

namespace sycldnn {
namespace helpers {
/** Quotient rounded up for non-negative numerators, truncated for negative ones. */
template <typename Index>
Index round_ratio_up(Index num, Index div) {
  const Index q = num / div;
  return (num < 0 || num % div == 0) ? q : q + 1;
}
template <typename Index>
Index round_ratio_up_above_zero(Index num, Index div) {
  return num < 0 ? 0 : round_ratio_up(num, div);
}
template <typename Index>
Index round_up_to_nearest_multiple(Index val, Index multiplier) {
  return round_ratio_up_above_zero(val, multiplier) * multiplier;
}

template <typename Index>
struct PaddingAndOutput {
  Index padding;
  Index output;
};

template <typename Index>
PaddingAndOutput<Index> calculate_padding(Index input, Index window, Index stride, PaddingMode type) {
  if (type == PaddingMode::VALID) return {Index{0}, round_ratio_up(input - window + 1, stride)};
  const Index out = round_ratio_up(input, stride);
  return {((out - 1) * stride + window - input) / 2, out};
}

/** Fills out_rows/out_cols/pad_rows/pad_cols of any parameter struct that has the usual fields. */
template <typename Params>
Params add_padding_to(Params params, PaddingMode type) {
  const auto rows = calculate_padding(params.in_rows, params.window_rows, params.stride_rows, type);
  const auto cols = calculate_padding(params.in_cols, params.window_cols, params.stride_cols, type);
  params.out_rows = rows.output;
  params.pad_rows = rows.padding;
  params.out_cols = cols.output;
  params.pad_cols = cols.padding;
  return params;
}
}  // namespace helpers
}  // namespace sycldnn
#endif
