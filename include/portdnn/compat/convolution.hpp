// cuDNN-style convolution API, after portDNN's include/portdnn/compat/convolution.hpp:46-1000.
// Quirks of the reference that callers may rely on are kept: only CROSS_CORRELATION is accepted;
// dilation must be 1; the filter of an NHWC tensor is HWCF; get*WorkspaceSize reports the
// recommended size in ELEMENTS through the "bytes" out-parameter while the launch functions
// divide their byte count by sizeof(ValueT) (convolution.hpp:728,751-755); the algorithm search
// only ever tries Direct; WinogradLarge has no selector here (convolution.hpp:507-523).
#ifndef PORTDNN_B200_COMPAT_CONVOLUTION_HPP_
#define PORTDNN_B200_COMPAT_CONVOLUTION_HPP_
#include "portdnn/compat/utils.hpp"
#include "portdnn/conv2d/launch.h"

namespace sycldnn {
namespace compat {

enum class ConvolutionMode { CROSS_CORRELATION = 0, CONVOLUTION };

class ConvolutionDescriptor {
 public:
  StatusCode set2d(int pad_h, int pad_w, int stride_h, int stride_w, int dilation_h, int dilation_w,
                   ConvolutionMode mode = ConvolutionMode::CROSS_CORRELATION) {
    if (pad_h < 0 || pad_w < 0 || stride_h <= 0 || stride_w <= 0 || dilation_h != 1 || dilation_w != 1 ||
        mode != ConvolutionMode::CROSS_CORRELATION)
      return StatusCode::InvalidParameter;
    pad_h_ = pad_h;
    pad_w_ = pad_w;
    stride_h_ = stride_h;
    stride_w_ = stride_w;
    return StatusCode::OK;
  }
  StatusCode setGroupCount(int groups) {
    if (groups <= 0) return StatusCode::InvalidParameter;
    groups_ = groups;
    return StatusCode::OK;
  }
  int pad_h() const { return pad_h_; }
  int pad_w() const { return pad_w_; }
  int stride_h() const { return stride_h_; }
  int stride_w() const { return stride_w_; }
  int groups() const { return groups_; }

 private:
  int pad_h_ = 0, pad_w_ = 0, stride_h_ = 1, stride_w_ = 1, groups_ = 1;
};

inline StatusCode setConvolution2dDescriptor(ConvolutionDescriptor& desc, int pad_h, int pad_w, int stride_h,
                                             int stride_w, int dilation_h, int dilation_w, ConvolutionMode mode) {
  return desc.set2d(pad_h, pad_w, stride_h, stride_w, dilation_h, dilation_w, mode);
}
inline StatusCode setConvolutionNdDescriptor(ConvolutionDescriptor& desc, int num_spatial_dims, const int* pads,
                                             const int* strides, const int* dilations, ConvolutionMode mode) {
  if (num_spatial_dims != 2) return StatusCode::InvalidParameter;
  return desc.set2d(pads[0], pads[1], strides[0], strides[1], dilations[0], dilations[1], mode);
}
inline StatusCode setConvolutionGroupCount(ConvolutionDescriptor& desc, int groups) { return desc.setGroupCount(groups); }

/** Filter extents are given as k, c, h, w whatever the layout.  As in the reference
 * (include/portdnn/compat/convolution.hpp:278-369) the descriptor keeps a FilterFormat of its own,
 * derived from the DataFormat it is set with: NCHW -> FCHW, NHWC -> HWCF. */
class FilterDescriptor {
 public:
  StatusCode set4d(DataFormat format, int k, int c, int h, int w) {
    if (k <= 0 || c <= 0 || h <= 0 || w <= 0) return StatusCode::InvalidParameter;
    if (format != DataFormat::NCHW && format != DataFormat::NHWC) return StatusCode::InvalidParameter;
    format_ = format == DataFormat::NCHW ? FilterFormat::FCHW : FilterFormat::HWCF;
    k_ = k;
    c_ = c;
    h_ = h;
    w_ = w;
    return StatusCode::OK;
  }
  FilterFormat getFormat() const { return format_; }
  size_t getSize() const { return size_t(k_) * c_ * h_ * w_; }
  StatusCode get4dDescriptorDims(int* k, int* c, int* h, int* w) const {
    if (k == nullptr || c == nullptr || h == nullptr || w == nullptr) return StatusCode::InvalidParameter;
    *k = k_;
    *c = c_;
    *h = h_;
    *w = w_;
    return StatusCode::OK;
  }
  StatusCode getFilter4dDescriptor(SNNDataType* dataType, FilterFormat* format, int* k, int* c, int* h, int* w) const {
    if (dataType == nullptr || format == nullptr) return StatusCode::InvalidParameter;
    *dataType = SNNDataType::SNN_FLOAT;
    *format = format_;
    return get4dDescriptorDims(k, c, h, w);
  }
  int k() const { return k_; }
  int c() const { return c_; }
  int h() const { return h_; }
  int w() const { return w_; }

 private:
  FilterFormat format_ = FilterFormat::FCHW;
  int k_ = 0, c_ = 0, h_ = 0, w_ = 0;
};
inline StatusCode setFilter4dDescriptor(FilterDescriptor& desc, SNNDataType, DataFormat format, int k, int c, int h,
                                        int w) {
  return desc.set4d(format, k, c, h, w);
}
inline StatusCode getFilter4dDescriptor(FilterDescriptor const& desc, SNNDataType* dataType, FilterFormat* format, int* k,
                                        int* c, int* h, int* w) {
  return desc.getFilter4dDescriptor(dataType, format, k, c, h, w);
}

/** out = 1 + (in + 2*pad - window) / stride (dilation is 1), convolution.hpp:403-431. */
inline StatusCode getConvolution2dForwardOutputDim(ConvolutionDescriptor const& conv, TensorDescriptor const& x,
                                                   FilterDescriptor const& w, int* n, int* c, int* h, int* wd) {
  *n = x.n();
  *c = w.k();
  *h = 1 + (x.h() + 2 * conv.pad_h() - w.h()) / conv.stride_h();
  *wd = 1 + (x.w() + 2 * conv.pad_w() - w.w()) / conv.stride_w();
  return StatusCode::OK;
}

namespace internal {
inline conv2d::Conv2DParams descToSnnParams(TensorDescriptor const& x, TensorDescriptor const& y,
                                            FilterDescriptor const& w, ConvolutionDescriptor const& conv) {
  conv2d::Conv2DParams p{};
  p.channels = x.c();
  p.features = y.c();
  p.batch = x.n();
  p.in_rows = x.h();
  p.in_cols = x.w();
  p.window_rows = w.h();
  p.window_cols = w.w();
  p.stride_rows = conv.stride_h();
  p.stride_cols = conv.stride_w();
  p.out_rows = y.h();
  p.out_cols = y.w();
  p.pad_rows = conv.pad_h();
  p.pad_cols = conv.pad_w();
  p.dilation_rows = p.dilation_cols = 1;
  p.groups = conv.groups();
  p.input_format = x.getFormat();
  p.filter_format = w.getFormat();  // the filter descriptor's own format, convolution.hpp:466-495
  p.group_format = BatchFormat::STRIDED;
  return p;
}

inline std::unique_ptr<conv2d::Selector> getSelector(conv2d::Algorithm algo) {
  using conv2d::Algorithm;
  switch (algo) {
    case Algorithm::Direct: return std::unique_ptr<conv2d::Selector>(new conv2d::DirectSelector());
    case Algorithm::Tiled: return std::unique_ptr<conv2d::Selector>(new conv2d::TiledSelector());
    case Algorithm::Im2col: return std::unique_ptr<conv2d::Selector>(new conv2d::Im2colSelector());
    case Algorithm::Winograd: return std::unique_ptr<conv2d::Selector>(new conv2d::WinogradSelector());
    case Algorithm::Matmul: return std::unique_ptr<conv2d::Selector>(new conv2d::MatmulSelector());
    default: return nullptr;  // NotSupported and WinogradLarge
  }
}

template <typename ConvType>
conv2d::WorkspaceSize getConvolutionWorkspaceSize(TensorDescriptor const& x, FilterDescriptor const& w,
                                                  ConvolutionDescriptor const& conv, TensorDescriptor const& y,
                                                  conv2d::Algorithm algo) {
  auto selector = getSelector(algo);
  if (!selector) return {0, 0};
  const conv2d::Conv2DParams p = descToSnnParams(x, y, w, conv);
  return conv2d::query_workspace_size<ConvType>(p, *selector);
}
}  // namespace internal

/** y = alpha * conv(x, w) + beta * y.  Alpha and beta are applied inside the convolution's own
 * epilogue (the reference runs separate Mul/Add passes over temporaries). */
template <typename ValueT>
SNNStatus convolutionForward(SNNHandle& handle, const ValueT* alpha, TensorDescriptor const& xDesc, const void* x,
                             FilterDescriptor const& wDesc, const void* w, ConvolutionDescriptor const& convDesc,
                             conv2d::Algorithm algo, void* workSpace, size_t workSpaceSizeInBytes, const ValueT* beta,
                             TensorDescriptor const& yDesc, void* y) {
  auto selector = internal::getSelector(algo);
  if (!selector) return StatusCode::InvalidParameter;
  const conv2d::Conv2DParams p = internal::descToSnnParams(xDesc, yDesc, wDesc, convDesc);
  auto& be = handle.getBackend();
  return internal::scaled_launch<ValueT>(be, ValueT(1), ValueT(0), static_cast<ValueT*>(y), yDesc.getSize(), [&](ValueT*) {
    // the whole blend is one fused launch; alpha == 0 still has to leave beta*y behind
    conv2d::FusedEpilogue e;
    e.alpha = float(*alpha);
    e.beta = float(*beta);
    return conv2d::launch_fused<ValueT>(static_cast<const ValueT*>(x), static_cast<const ValueT*>(w),
                                        static_cast<ValueT*>(y), p, *selector, be, e, static_cast<ValueT*>(workSpace),
                                        workSpaceSizeInBytes / sizeof(ValueT));
  });
}

/** dx = alpha * conv_backward_data(dy, w) + beta * dx. */
template <typename ValueT>
SNNStatus convolutionBackwardData(SNNHandle& handle, const ValueT* alpha, FilterDescriptor const& wDesc, const void* w,
                                  TensorDescriptor const& dyDesc, const void* dy, ConvolutionDescriptor const& convDesc,
                                  conv2d::Algorithm algo, void* workSpace, size_t workSpaceSizeInBytes,
                                  const ValueT* beta, TensorDescriptor const& dxDesc, void* dx) {
  auto selector = internal::getSelector(algo);
  if (!selector) return StatusCode::InvalidParameter;
  const conv2d::Conv2DParams p = internal::descToSnnParams(dxDesc, dyDesc, wDesc, convDesc);
  auto& be = handle.getBackend();
  return internal::scaled_launch<ValueT>(be, *alpha, *beta, static_cast<ValueT*>(dx), dxDesc.getSize(), [&](ValueT* dst) {
    return conv2d::launch<ValueT, conv2d::conv_type::InputBackprop>(
        static_cast<const ValueT*>(dy), static_cast<const ValueT*>(w), dst, p, *selector, be,
        static_cast<ValueT*>(workSpace), workSpaceSizeInBytes / sizeof(ValueT));
  });
}

/** dw = alpha * conv_backward_filter(x, dy) + beta * dw. */
template <typename ValueT>
SNNStatus convolutionBackwardFilter(SNNHandle& handle, const ValueT* alpha, TensorDescriptor const& xDesc, const void* x,
                                    TensorDescriptor const& dyDesc, const void* dy,
                                    ConvolutionDescriptor const& convDesc, conv2d::Algorithm algo, void* workSpace,
                                    size_t workSpaceSizeInBytes, const ValueT* beta, FilterDescriptor const& dwDesc,
                                    void* dw) {
  auto selector = internal::getSelector(algo);
  if (!selector) return StatusCode::InvalidParameter;
  const conv2d::Conv2DParams p = internal::descToSnnParams(xDesc, dyDesc, dwDesc, convDesc);
  auto& be = handle.getBackend();
  return internal::scaled_launch<ValueT>(be, *alpha, *beta, static_cast<ValueT*>(dw), dwDesc.getSize(), [&](ValueT* dst) {
    return conv2d::launch<ValueT, conv2d::conv_type::FilterBackprop>(
        static_cast<const ValueT*>(x), static_cast<const ValueT*>(dy), dst, p, *selector, be,
        static_cast<ValueT*>(workSpace), workSpaceSizeInBytes / sizeof(ValueT));
  });
}

inline StatusCode getConvolutionForwardWorkspaceSize(SNNHandle&, TensorDescriptor const& x, FilterDescriptor const& w,
                                                     ConvolutionDescriptor const& conv, TensorDescriptor const& y,
                                                     conv2d::Algorithm algo, size_t* workSpaceSizeInBytes) {
  *workSpaceSizeInBytes =
      internal::getConvolutionWorkspaceSize<conv2d::conv_type::Forward>(x, w, conv, y, algo).recommended_size;
  return StatusCode::OK;
}
inline StatusCode getConvolutionBackwardDataWorkspaceSize(SNNHandle&, FilterDescriptor const& w,
                                                          TensorDescriptor const& dy, ConvolutionDescriptor const& conv,
                                                          TensorDescriptor const& dx, conv2d::Algorithm algo,
                                                          size_t* workSpaceSizeInBytes) {
  *workSpaceSizeInBytes =
      internal::getConvolutionWorkspaceSize<conv2d::conv_type::InputBackprop>(dx, w, conv, dy, algo).recommended_size;
  return StatusCode::OK;
}
inline StatusCode getConvolutionBackwardFilterWorkspaceSize(SNNHandle&, TensorDescriptor const& x,
                                                            TensorDescriptor const& dy,
                                                            ConvolutionDescriptor const& conv, FilterDescriptor const& dw,
                                                            conv2d::Algorithm algo, size_t* workSpaceSizeInBytes) {
  *workSpaceSizeInBytes =
      internal::getConvolutionWorkspaceSize<conv2d::conv_type::FilterBackprop>(x, dw, conv, dy, algo).recommended_size;
  return StatusCode::OK;
}

/** Like the reference, the "search" reports a single candidate, Direct (convolution.hpp:577-630). */
inline SNNStatus findConvolutionForwardAlgorithm(SNNHandle&, TensorDescriptor const&, FilterDescriptor const&,
                                                 ConvolutionDescriptor const&, TensorDescriptor const&,
                                                 int requestedAlgoCount, int* returnedAlgoCount,
                                                 convolutionFwdAlgoPerf_t* perfResults) {
  if (requestedAlgoCount < 1) return StatusCode::InvalidParameter;
  perfResults[0] = convolutionFwdAlgoPerf_t{conv2d::Algorithm::Direct, StatusCode::OK, 0.f};
  *returnedAlgoCount = 1;
  return StatusCode::OK;
}
inline SNNStatus findConvolutionBackwardDataAlgorithm(SNNHandle& h, FilterDescriptor const& w, TensorDescriptor const& dy,
                                                      ConvolutionDescriptor const& conv, TensorDescriptor const& dx,
                                                      int requestedAlgoCount, int* returnedAlgoCount,
                                                      convolutionFwdAlgoPerf_t* perfResults) {
  return findConvolutionForwardAlgorithm(h, dx, w, conv, dy, requestedAlgoCount, returnedAlgoCount, perfResults);
}

}  // namespace compat
}  // namespace sycldnn
#endif
