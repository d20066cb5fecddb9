// Algorithm selectors, after portDNN's include/portdnn/conv2d/selector/*.h.  Each selector answers,
// per pass, which Algorithm tag to run or NotSupported; the answers (and so the skip behaviour of
// code written against the reference) are the reference's.  What the tags run here: Direct -> the
// general CUDA-core kernel; every other tag -> the tcgen05 implicit-GEMM kernel (shapes it cannot
// tile fall to the direct kernel).
#ifndef PORTDNN_B200_CONV2D_SELECTOR_H_
#define PORTDNN_B200_CONV2D_SELECTOR_H_
#include <memory>

#include "portdnn/conv2d/params.h"

namespace sycldnn {
namespace conv2d {

class Selector {
 public:
  virtual ~Selector() = default;
  template <typename ConvType>
  Algorithm select(Conv2DParams const& params) {
    switch (pass_of<ConvType>::value) {
      case PDNN_INPUT_BACKPROP: return select_input_backprop(params);
      case PDNN_FILTER_BACKPROP: return select_filter_backprop(params);
      default: return select_forward(params);
    }
  }
  virtual Algorithm select_forward(Conv2DParams const& params) = 0;
  virtual Algorithm select_input_backprop(Conv2DParams const& params) = 0;
  virtual Algorithm select_filter_backprop(Conv2DParams const& params) = 0;
  virtual char const* name() const = 0;
};

namespace detail {
inline bool square(Conv2DParams const& p, int window, int stride) {
  return p.window_rows == window && p.window_cols == window && p.stride_rows == stride && p.stride_cols == stride;
}
inline bool window_is(Conv2DParams const& p, int rows, int cols) { return p.window_rows == rows && p.window_cols == cols; }
// The reference's Winograd selectors reject a shape only when BOTH strides differ from 1
// (include/portdnn/conv2d/selector/winograd_selector.h:44-46).
inline bool winograd_stride_ok(Conv2DParams const& p) { return !(p.stride_rows != 1 && p.stride_cols != 1); }
inline bool pointwise_gemm(Conv2DParams const& p) {
  return square(p, 1, 1) && p.pad_rows == 0 && p.pad_cols == 0 && p.input_format == DataFormat::NHWC &&
         p.filter_format == FilterFormat::HWCF;
}
}  // namespace detail

/** Always the same answer (include/portdnn/conv2d/selector/constant_selector.h:37-97). */
template <Algorithm Algo>
class ConstantSelector final : public Selector {
 public:
  Algorithm select_forward(Conv2DParams const&) override { return Algo; }
  Algorithm select_input_backprop(Conv2DParams const&) override { return Algo; }
  Algorithm select_filter_backprop(Conv2DParams const&) override { return Algo; }
  char const* name() const override {
    return Algo == Algorithm::Direct ? "DirectSelector" : Algo == Algorithm::Im2col ? "Im2colSelector" : "ConstantSelector";
  }
};
using DirectSelector = ConstantSelector<Algorithm::Direct>;
using Im2colSelector = ConstantSelector<Algorithm::Im2col>;

/** Forward only, square 1/3 windows at stride 1/2 and 5x5 stride 1 (tiled_selector.h:45-96). */
class TiledSelector final : public Selector {
 public:
  Algorithm select_forward(Conv2DParams const& p) override {
    using detail::square;
    const bool ok = square(p, 1, 1) || square(p, 1, 2) || square(p, 3, 1) || square(p, 3, 2) || square(p, 5, 1);
    return ok ? Algorithm::Tiled : Algorithm::NotSupported;
  }
  Algorithm select_input_backprop(Conv2DParams const&) override { return Algorithm::NotSupported; }
  Algorithm select_filter_backprop(Conv2DParams const&) override { return Algorithm::NotSupported; }
  char const* name() const override { return "TiledSelector"; }
};

/** 3x3, 1x3 and 3x1 windows (winograd_selector.h:34-108). */
class WinogradSelector final : public Selector {
 public:
  Algorithm select_forward(Conv2DParams const& p) override { return pick(p); }
  Algorithm select_input_backprop(Conv2DParams const& p) override { return pick(p); }
  Algorithm select_filter_backprop(Conv2DParams const& p) override { return pick(p); }
  char const* name() const override { return "WinogradSelector"; }

 private:
  static Algorithm pick(Conv2DParams const& p) {
    using detail::window_is;
    const bool ok = detail::winograd_stride_ok(p) && (window_is(p, 1, 3) || window_is(p, 3, 1) || window_is(p, 3, 3));
    return ok ? Algorithm::Winograd : Algorithm::NotSupported;
  }
};

/** 3x3 windows only (winograd_selector.h:110-174). */
class WinogradLargeSelector final : public Selector {
 public:
  Algorithm select_forward(Conv2DParams const& p) override { return pick(p); }
  Algorithm select_input_backprop(Conv2DParams const& p) override { return pick(p); }
  Algorithm select_filter_backprop(Conv2DParams const& p) override { return pick(p); }
  char const* name() const override { return "WinogradLargeSelector"; }

 private:
  static Algorithm pick(Conv2DParams const& p) {
    return detail::winograd_stride_ok(p) && detail::window_is(p, 3, 3) ? Algorithm::WinogradLarge : Algorithm::NotSupported;
  }
};

/** 1x1, stride 1, no padding, NHWC/HWCF: one GEMM (matmul_selector.h:34-108). */
class MatmulSelector final : public Selector {
 public:
  Algorithm select_forward(Conv2DParams const& p) override { return pick(p); }
  Algorithm select_input_backprop(Conv2DParams const& p) override { return pick(p); }
  Algorithm select_filter_backprop(Conv2DParams const& p) override { return pick(p); }
  char const* name() const override { return "MatmulSelector"; }

 private:
  static Algorithm pick(Conv2DParams const& p) {
    return detail::pointwise_gemm(p) ? Algorithm::Matmul : Algorithm::NotSupported;
  }
};

/** The default selector of this implementation.  It follows the shape rules of the reference's
 * DefaultSelector (src/conv2d/selector/default_selector.cc:49-128) - grouped -> Im2col; NCHW ->
 * Direct; 1x1 stride 1 -> Matmul; forward tiled shapes -> Tiled; anything else -> Im2col - except
 * that it never picks Winograd: every tag but Direct and the Winograd pair runs the same
 * tensor-core implicit GEMM, which needs no workspace and is the fastest path for 16-bit data.
 * fp32 callers with a workspace to spare can ask for WinogradSelector explicitly. */
class B200Selector final : public Selector {
 public:
  Algorithm select_forward(Conv2DParams const& p) override {
    const Algorithm common = pick_common(p);
    if (common != Algorithm::NotSupported) return common;
    TiledSelector tiled;
    return tiled.select_forward(p) == Algorithm::Tiled ? Algorithm::Tiled : Algorithm::Im2col;
  }
  Algorithm select_input_backprop(Conv2DParams const& p) override { return or_im2col(pick_common(p)); }
  Algorithm select_filter_backprop(Conv2DParams const& p) override { return or_im2col(pick_common(p)); }
  char const* name() const override { return "B200Selector"; }

 private:
  static Algorithm or_im2col(Algorithm a) { return a == Algorithm::NotSupported ? Algorithm::Im2col : a; }
  static Algorithm pick_common(Conv2DParams const& p) {
    if (p.groups > 1) return Algorithm::Im2col;
    if (p.input_format == DataFormat::NCHW) return Algorithm::Direct;
    if (detail::pointwise_gemm(p)) return Algorithm::Matmul;
    return Algorithm::NotSupported;
  }
};

/** The reference picks by SYCL device vendor (default_selector.cc:257-286); here there is one device. */
inline std::unique_ptr<Selector> get_default_selector() { return std::unique_ptr<Selector>(new B200Selector()); }
template <typename Device>
inline std::unique_ptr<Selector> get_default_selector(Device const&) { return get_default_selector(); }

}  // namespace conv2d
}  // namespace sycldnn
#endif
