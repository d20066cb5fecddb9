// The cuDNN-style convolution and pooling calls (include/portdnn/compat/convolution.hpp, pooling.hpp)
// replayed on the cases of portDNN's own tests: test/compat/conv2d_forward_compat.cc,
// conv2d_backward_data_compat.cc, conv2d_backward_filter_compat.cc, pooling_compat.cc (shapes,
// alpha / beta, expected values; extracted into compat_kat.inc by tests/golden/make_golden_compat.py),
// plus the checks of workspace_size_compat.cc and conv2d_find_algo.cc and the descriptor getters.
// The harness follows the reference's do_test / test_pool: tensors are the repeating ramp
// 1..2048 in memory order, the output tensor starts as that ramp too (so beta has something to
// scale), results must EQUAL the expected integers.  Exits 0 and prints "all checks passed".
//
//   g++ -std=c++17 -Iinclude -I$CUDA/include tests/cpp/compat_conv_test.cc -Lportdnn_b200 -lportdnn_b200 -lcudart
#include <cmath>
#include <cstdio>
#include <string>
#include <vector>

#include "portdnn/compat/convolution.hpp"
#include "portdnn/compat/pooling.hpp"
#include "portdnn/helpers/padding.h"

using namespace sycldnn;
using namespace sycldnn::compat;
using Vec = std::vector<float>;

static int g_failures = 0;
#define CHECK(cond, ...)                               \
  do {                                                 \
    if (!(cond)) {                                     \
      std::printf("FAIL %s:%d: ", __FILE__, __LINE__); \
      std::printf(__VA_ARGS__);                        \
      std::printf("\n");                               \
      ++g_failures;                                    \
    }                                                  \
  } while (0)

struct CompatConvCase {
  const char* name;
  int pass;
  std::vector<int> in_sizes, filt_sizes, conv_sizes;
  DataFormat format;
  conv2d::Algorithm algo;
  int groups;
  float alpha, beta;
  Vec expect;
};
struct CompatPoolCase {
  const char* name;
  std::vector<int> in_sizes;
  int window, stride;
  bool same;
  PoolingMode mode;
  NanPropagation nan_opt;
  DataFormat format;
  float alpha, beta;
  bool nan_input;
  Vec expect;
};
#include "compat_kat.inc"

static Vec ramp(size_t n, int max = 2048) {
  Vec v(n);
  for (size_t i = 0; i < n; ++i) v[i] = float(i % size_t(max) + 1);
  return v;
}
static float* to_device(const Vec& h) {
  void* d = nullptr;
  cudaMalloc(&d, h.size() * sizeof(float) + 16);
  cudaMemcpy(d, h.data(), h.size() * sizeof(float), cudaMemcpyHostToDevice);
  return static_cast<float*>(d);
}
static Vec to_host(const float* d, size_t n) {
  Vec h(n);
  cudaMemcpy(h.data(), d, n * sizeof(float), cudaMemcpyDeviceToHost);
  return h;
}
static bool same_values(const Vec& a, const Vec& b) {
  if (a.size() != b.size()) return false;
  for (size_t i = 0; i < a.size(); ++i)
    if (!(a[i] == b[i] || (std::isnan(a[i]) && std::isnan(b[i])))) return false;
  return true;
}
static size_t product(const std::vector<int>& v) {
  size_t n = 1;
  for (int x : v) n *= size_t(x);
  return n;
}

static void run_conv_case(SNNHandle& handle, const CompatConvCase& c) {
  TensorDescriptor in_desc, out_desc;
  FilterDescriptor filt_desc;
  ConvolutionDescriptor conv_desc;
  in_desc.set4d(c.format, c.in_sizes[0], c.in_sizes[1], c.in_sizes[2], c.in_sizes[3]);
  filt_desc.set4d(c.format, c.filt_sizes[0], c.filt_sizes[1], c.filt_sizes[2], c.filt_sizes[3]);
  conv_desc.set2d(c.conv_sizes[0], c.conv_sizes[1], c.conv_sizes[2], c.conv_sizes[3], c.conv_sizes[4], c.conv_sizes[5]);
  if (c.groups > 1) setConvolutionGroupCount(conv_desc, c.groups);
  int n, k, h, w;
  getConvolution2dForwardOutputDim(conv_desc, in_desc, filt_desc, &n, &k, &h, &w);
  out_desc.set4d(c.format, n, k, h, w);
  float* in = to_device(ramp(product(c.in_sizes)));
  float* fil = to_device(ramp(product(c.filt_sizes)));
  // the forward test leaves its output buffer uninitialised unless beta is used; a ramp covers both
  float* out = to_device(ramp(out_desc.getSize()));
  SNNStatus st;
  Vec got;
  if (c.pass == 0) {
    st = convolutionForward(handle, &c.alpha, in_desc, in, filt_desc, fil, conv_desc, c.algo, nullptr, 0, &c.beta, out_desc,
                            out);
    st.event.wait();
    got = to_host(out, out_desc.getSize());
  } else if (c.pass == 1) {
    st = convolutionBackwardData(handle, &c.alpha, filt_desc, fil, out_desc, out, conv_desc, c.algo, nullptr, 0, &c.beta,
                                 in_desc, in);
    st.event.wait();
    got = to_host(in, in_desc.getSize());
  } else {
    st = convolutionBackwardFilter(handle, &c.alpha, in_desc, in, out_desc, out, conv_desc, c.algo, nullptr, 0, &c.beta,
                                   filt_desc, fil);
    st.event.wait();
    got = to_host(fil, filt_desc.getSize());
  }
  CHECK(st.status == StatusCode::OK, "%s: status %d", c.name, int(st.status));
  CHECK(same_values(got, c.expect), "%s: got[0] = %g, expected[0] = %g (%zu / %zu values)", c.name, got.empty() ? 0.f : got[0],
        c.expect.empty() ? 0.f : c.expect[0], got.size(), c.expect.size());
  cudaFree(in);
  cudaFree(fil);
  cudaFree(out);
}

static void run_pool_case(SNNHandle& handle, const CompatPoolCase& c) {
  const PaddingMode mode = c.same ? PaddingMode::SAME : PaddingMode::VALID;
  const auto rows = helpers::calculate_padding(c.in_sizes[2], c.window, c.stride, mode);
  const auto cols = helpers::calculate_padding(c.in_sizes[3], c.window, c.stride, mode);
  PoolingDescriptor pool_desc;
  CHECK(setPooling2dDescriptor(pool_desc, c.mode, c.nan_opt, c.window, c.window, rows.padding, cols.padding, c.stride,
                               c.stride) == StatusCode::OK,
        "%s: descriptor", c.name);
  TensorDescriptor in_desc, out_desc;
  in_desc.set4d(c.format, c.in_sizes[0], c.in_sizes[1], c.in_sizes[2], c.in_sizes[3]);
  out_desc.set4d(c.format, c.in_sizes[0], c.in_sizes[1], rows.output, cols.output);
  Vec input = ramp(product(c.in_sizes));
  if (c.nan_input) input.assign(input.size(), NAN);
  float* in = to_device(input);
  float* out = to_device(ramp(out_desc.getSize()));
  SNNStatus st = poolingForward(handle, pool_desc, &c.alpha, in_desc, in, &c.beta, out_desc, out);
  CHECK(st.status == StatusCode::OK, "%s: status %d", c.name, int(st.status));
  st.event.wait();
  const Vec got = to_host(out, out_desc.getSize());
  CHECK(same_values(got, c.expect), "%s: got[0] = %g, expected[0] = %g", c.name, got[0], c.expect[0]);
  cudaFree(in);
  cudaFree(out);
}

// test/compat/workspace_size_compat.cc: Direct and Tiled need no workspace in any pass.  Im2col: the
// reference reports the size of its im2col buffer; this implementation's implicit GEMM has no
// such buffer, so the forward and input-backprop figures are 0 and only the filter backprop (its
// pixel-split partial sums) recommends any scratch.
static void workspace_checks() {
  SNNHandle handle;
  SNNCreate(handle);
  conv2d::Conv2DParams p{};
  p.window_rows = p.window_cols = 3;
  p.stride_rows = p.stride_cols = 1;
  p.in_rows = p.in_cols = 56;
  p.channels = p.features = 256;
  p.batch = 1;
  p.dilation_rows = p.dilation_cols = 1;
  p = helpers::add_padding_to(p, PaddingMode::SAME);
  TensorDescriptor x, y;
  FilterDescriptor w;
  ConvolutionDescriptor conv;
  setTensor4dDescriptor(x, DataFormat::NHWC, SNNDataType::SNN_FLOAT, p.batch, p.channels, p.in_rows, p.in_cols);
  setTensor4dDescriptor(y, DataFormat::NHWC, SNNDataType::SNN_FLOAT, p.batch, p.features, p.out_rows, p.out_cols);
  setFilter4dDescriptor(w, SNNDataType::SNN_FLOAT, DataFormat::NHWC, p.features, p.channels, 3, 3);
  conv.set2d(p.pad_rows, p.pad_cols, 1, 1, 1, 1);
  for (auto algo : {conv2d::Algorithm::Direct, conv2d::Algorithm::Tiled, conv2d::Algorithm::Im2col}) {
    size_t fwd = 1, ibp = 1, fbp = 1;
    CHECK(getConvolutionForwardWorkspaceSize(handle, x, w, conv, y, algo, &fwd) == StatusCode::OK, "forward query");
    CHECK(getConvolutionBackwardDataWorkspaceSize(handle, w, y, conv, x, algo, &ibp) == StatusCode::OK, "backward data query");
    CHECK(getConvolutionBackwardFilterWorkspaceSize(handle, x, y, conv, w, algo, &fbp) == StatusCode::OK, "backward filter query");
    CHECK(fwd == 0 && ibp == 0, "algorithm %d: forward %zu, backward data %zu", int(algo), fwd, ibp);
    if (algo == conv2d::Algorithm::Direct) CHECK(fbp == 0, "direct filter backprop workspace %zu", fbp);
  }
  // test/compat/conv2d_find_algo.cc: one candidate, Direct, status OK
  int returned = 0;
  convolutionFwdAlgoPerf_t perf[2];
  SNNStatus st = findConvolutionForwardAlgorithm(handle, x, w, conv, y, 2, &returned, perf);
  CHECK(st.status == StatusCode::OK && returned == 1 && perf[0].algo == conv2d::Algorithm::Direct &&
            perf[0].status == StatusCode::OK,
        "findConvolutionForwardAlgorithm");
  returned = 0;
  st = findConvolutionBackwardDataAlgorithm(handle, w, y, conv, x, 1, &returned, perf);
  CHECK(st.status == StatusCode::OK && returned == 1 && perf[0].algo == conv2d::Algorithm::Direct, "findConvolutionBackwardDataAlgorithm");
  CHECK(findConvolutionForwardAlgorithm(handle, x, w, conv, y, 0, &returned, perf).status == StatusCode::InvalidParameter,
        "zero requested algorithms");
  // test/compat/compat_descriptor.cc: the filter descriptor reports a FilterFormat of its own
  SNNDataType dt;
  FilterFormat ff;
  int k, c, h, wd;
  CHECK(getFilter4dDescriptor(w, &dt, &ff, &k, &c, &h, &wd) == StatusCode::OK && ff == FilterFormat::HWCF && k == 256 &&
            c == 256 && h == 3 && wd == 3 && dt == SNNDataType::SNN_FLOAT,
        "filter descriptor getter");
  FilterDescriptor w2;
  w2.set4d(DataFormat::NCHW, 8, 4, 3, 3);
  CHECK(w2.getFormat() == FilterFormat::FCHW, "NCHW filter descriptors are FCHW");
}

int main() {
  SNNHandle handle;
  SNNCreate(handle);
  for (const auto& c : kCompatConvCases) run_conv_case(handle, c);
  for (const auto& c : kCompatPoolCases) run_pool_case(handle, c);
  workspace_checks();
  cudaDeviceSynchronize();
  std::printf("compat_conv_test: %zu convolution cases, %zu pooling cases\n", kCompatConvCases.size(), kCompatPoolCases.size());
  if (g_failures == 0) std::printf("compat_conv_test: all checks passed\n");
  return g_failures == 0 ? 0 : 1;
}
