// Exercises the C++ mirror of portDNN's API (include/portdnn/**) the way the reference's own tests
// drive it: ramp-initialised tensors (test/gen/iota_initialised_data.h:45-79), every selector,
// NotSupported -> skip, status checks, results compared with a host loop written from the
// operator definitions.  Exits 0 when everything matches; prints the first mismatch otherwise.
//
//   g++ -std=c++17 -Iinclude -I$CUDA/include tests/cpp/api_test.cc -Lportdnn_b200 -lportdnn_b200 -lcudart
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "portdnn/backend/cuda_backend.h"
#include "portdnn/binaryop/launch.h"
#include "portdnn/compat/convolution.hpp"
#include "portdnn/compat/pooling.hpp"
#include "portdnn/conv2d/launch.h"
#include "portdnn/depthwise_conv2d/launch.h"
#include "portdnn/helpers/padding.h"
#include "portdnn/matmul/launch.h"
#include "portdnn/pointwise/launch.h"
#include "portdnn/pooling/launch.h"

using namespace sycldnn;
using Backend = backend::CUDABackend;

static int g_failures = 0;
#define CHECK(cond, ...)                          \
  do {                                            \
    if (!(cond)) {                                \
      std::printf("FAIL %s:%d: ", __FILE__, __LINE__); \
      std::printf(__VA_ARGS__);                   \
      std::printf("\n");                          \
      ++g_failures;                               \
    }                                             \
  } while (0)

static std::vector<float> iota(size_t n, int max_val) {
  std::vector<float> v(n);
  for (size_t i = 0; i < n; ++i) v[i] = float(max_val >= 1 ? (i % size_t(max_val)) + 1 : i + 1);
  return v;
}
static float* dev_alloc(size_t bytes) {
  void* d = nullptr;
  cudaMalloc(&d, bytes);
  return static_cast<float*>(d);
}
template <typename T>
static T* to_device(const std::vector<T>& h) {
  T* d = reinterpret_cast<T*>(dev_alloc(h.size() * sizeof(T) + 16));
  cudaMemcpy(d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice);
  return d;
}
template <typename T>
static std::vector<T> to_host(const T* d, size_t n) {
  std::vector<T> h(n);
  cudaMemcpy(h.data(), d, n * sizeof(T), cudaMemcpyDeviceToHost);
  return h;
}
static bool close(const std::vector<float>& a, const std::vector<float>& b, float rel) {
  float scale = 1e-30f, err = 0.f;
  for (size_t i = 0; i < a.size(); ++i) {
    scale = std::fmax(scale, std::fabs(b[i]));
    err = std::fmax(err, std::fabs(a[i] - b[i]));
  }
  return err <= rel * scale;
}

// y[n,oh,ow,k] = sum x[n,oh*st-pad+r,ow*st-pad+s,c] * w[r,s,c,k]
static std::vector<float> host_conv(const std::vector<float>& x, const std::vector<float>& w, const conv2d::Conv2DParams& p) {
  std::vector<float> y(size_t(p.batch) * p.out_rows * p.out_cols * p.features, 0.f);
  for (int n = 0; n < p.batch; ++n)
    for (int oh = 0; oh < p.out_rows; ++oh)
      for (int ow = 0; ow < p.out_cols; ++ow)
        for (int k = 0; k < p.features; ++k) {
          double acc = 0;
          for (int r = 0; r < p.window_rows; ++r)
            for (int s = 0; s < p.window_cols; ++s) {
              const int ih = oh * p.stride_rows - p.pad_rows + r, iw = ow * p.stride_cols - p.pad_cols + s;
              if (ih < 0 || ih >= p.in_rows || iw < 0 || iw >= p.in_cols) continue;
              for (int c = 0; c < p.channels; ++c)
                acc += double(x[((size_t(n) * p.in_rows + ih) * p.in_cols + iw) * p.channels + c]) *
                       w[((size_t(r) * p.window_cols + s) * p.channels + c) * p.features + k];
            }
          y[((size_t(n) * p.out_rows + oh) * p.out_cols + ow) * p.features + k] = float(acc);
        }
  return y;
}

static conv2d::Conv2DParams make_params(int n, int h, int w, int c, int k, int window, int stride, PaddingMode mode) {
  conv2d::Conv2DParams p{};
  p.channels = c;
  p.features = k;
  p.batch = n;
  p.in_rows = h;
  p.in_cols = w;
  p.window_rows = p.window_cols = window;
  p.stride_rows = p.stride_cols = stride;
  p.dilation_rows = p.dilation_cols = 1;
  return helpers::add_padding_to(p, mode);
}

template <typename SelectorT>
static void forward_with_selector(const char* name, const conv2d::Conv2DParams& p, int max_val) {
  Backend backend{nullptr};
  SelectorT selector;
  if (selector.template select<conv2d::conv_type::Forward>(p) == conv2d::Algorithm::NotSupported) return;  // skip
  const auto sizes = conv2d::get_sizes<conv2d::conv_type::Forward>(p);
  const auto x = iota(sizes.input_size, max_val), w = iota(sizes.filter_size, max_val);
  float *dx = to_device(x), *dw = to_device(w), *dy = nullptr;
  dy = dev_alloc(sizes.output_size * sizeof(float));
  const auto ws = conv2d::query_workspace_size<conv2d::conv_type::Forward>(p, selector);
  float* dws = backend.allocate<float>(ws.recommended_size);
  auto st = conv2d::launch<float, conv2d::conv_type::Forward>(dx, dw, dy, p, selector, backend, dws, ws.recommended_size);
  if (st.status == StatusCode::InvalidAlgorithm) return;  // the reference's tests skip here too
  CHECK(st.status == StatusCode::OK, "%s: status %d (%s)", name, int(st.status), pdnn_last_error());
  st.event.wait_and_throw();
  const auto got = to_host(dy, sizes.output_size);
  CHECK(close(got, host_conv(x, w, p), 1e-5f), "%s: forward result differs", name);
  backend.deallocate(dws);
  cudaFree(dx);
  cudaFree(dw);
  cudaFree(dy);
}

int main() {
  int devices = 0;
  if (cudaGetDeviceCount(&devices) != cudaSuccess || devices == 0) {
    std::printf("no CUDA device\n");
    return 2;
  }
  // --- padding helper (include/portdnn/helpers/padding.h:46-66) ---
  {
    auto a = helpers::calculate_padding(56, 3, 2, PaddingMode::SAME);
    CHECK(a.padding == 0 && a.output == 28, "SAME 56/3/2 gave pad %d out %d", a.padding, a.output);
    auto b = helpers::calculate_padding(224, 7, 2, PaddingMode::SAME);
    CHECK(b.padding == 2 && b.output == 112, "SAME 224/7/2");
    auto c = helpers::calculate_padding(230, 7, 2, PaddingMode::VALID);
    CHECK(c.padding == 0 && c.output == 112, "VALID 230/7/2");
  }
  // --- conv2d forward through every selector, small ramp cases and tensor-core sized ones ---
  for (auto mode : {PaddingMode::SAME, PaddingMode::VALID}) {
    for (int window : {1, 3, 5}) {
      for (int stride : {1, 2}) {
        const auto small = make_params(2, 7, 6, 2, 4, window, stride, mode);
        if (small.out_rows <= 0 || small.out_cols <= 0) continue;
        forward_with_selector<conv2d::DirectSelector>("direct/small", small, 64);
        forward_with_selector<conv2d::TiledSelector>("tiled/small", small, 64);
        forward_with_selector<conv2d::Im2colSelector>("im2col/small", small, 64);
        forward_with_selector<conv2d::WinogradSelector>("winograd/small", small, 64);
        forward_with_selector<conv2d::WinogradLargeSelector>("winograd-large/small", small, 64);
        forward_with_selector<conv2d::MatmulSelector>("matmul/small", small, 64);
        const auto big = make_params(2, 12, 12, 32, 32, window, stride, mode);
        forward_with_selector<conv2d::Im2colSelector>("im2col/tc", big, 8);
        forward_with_selector<conv2d::B200Selector>("default/tc", big, 8);
      }
    }
  }
  // --- validation: InvalidParameter before anything is launched ---
  {
    Backend backend{nullptr};
    conv2d::DirectSelector sel;
    auto p = make_params(1, 4, 4, 4, 4, 3, 1, PaddingMode::SAME);
    p.dilation_rows = 2;
    float* dummy = nullptr;
    dummy = dev_alloc(1024);
    auto st = conv2d::launch<float, conv2d::conv_type::Forward>(dummy, dummy, dummy, p, sel, backend, nullptr, 0);
    CHECK(st.status == StatusCode::InvalidParameter, "dilation 2 must be rejected, got %d", int(st.status));
    cudaFree(dummy);
  }
  // --- backprop passes agree with the direct kernel ---
  {
    Backend backend{nullptr};
    const auto p = make_params(2, 10, 10, 16, 24, 3, 1, PaddingMode::SAME);
    conv2d::DirectSelector direct;
    conv2d::Im2colSelector gemm;
    const auto si = conv2d::get_sizes<conv2d::conv_type::InputBackprop>(p);
    const auto sf = conv2d::get_sizes<conv2d::conv_type::FilterBackprop>(p);
    const auto dyv = iota(si.input_size, 5), wv = iota(si.filter_size, 3), xv = iota(sf.input_size, 7);
    float *dy = to_device(dyv), *w = to_device(wv), *x = to_device(xv), *o1, *o2;
    o1 = dev_alloc(std::max(si.output_size, sf.output_size) * sizeof(float));
    o2 = dev_alloc(std::max(si.output_size, sf.output_size) * sizeof(float));
    conv2d::launch<float, conv2d::conv_type::InputBackprop>(dy, w, o1, p, direct, backend, nullptr, 0);
    auto st = conv2d::launch<float, conv2d::conv_type::InputBackprop>(dy, w, o2, p, gemm, backend, nullptr, 0);
    CHECK(st.status == StatusCode::OK, "input backprop status %d", int(st.status));
    st.event.wait();
    CHECK(close(to_host(o2, si.output_size), to_host(o1, si.output_size), 1e-5f), "input backprop differs");
    conv2d::launch<float, conv2d::conv_type::FilterBackprop>(x, dy, o1, p, direct, backend, nullptr, 0);
    st = conv2d::launch<float, conv2d::conv_type::FilterBackprop>(x, dy, o2, p, gemm, backend, nullptr, 0);
    CHECK(st.status == StatusCode::OK, "filter backprop status %d", int(st.status));
    st.event.wait();
    CHECK(close(to_host(o2, sf.output_size), to_host(o1, sf.output_size), 1e-5f), "filter backprop differs");
    cudaFree(dy); cudaFree(w); cudaFree(x); cudaFree(o1); cudaFree(o2);
  }
  // --- pooling, pointwise, bias, matmul ---
  {
    Backend backend{nullptr};
    pooling::PoolingParams pp{};
    pp.in_rows = pp.in_cols = 4;
    pp.window_rows = pp.window_cols = 2;
    pp.stride_rows = pp.stride_cols = 2;
    pp.batch = 1;
    pp.channels = 2;
    pp = helpers::add_padding_to(pp, PaddingMode::VALID);
    const auto xv = iota(32, 0);
    float *x = to_device(xv), *y, *dx;
    y = dev_alloc(8 * sizeof(float));
    dx = dev_alloc(32 * sizeof(float));
    auto st = pooling::launch<float, pooling::Max, pooling::Forward>(x, y, pp, backend);
    CHECK(st.status == StatusCode::OK, "max pool status");
    st.event.wait();
    const auto yv = to_host(y, 8);
    CHECK(yv[0] == 11.f && yv[1] == 12.f && yv[7] == 32.f, "max pool values %g %g %g", yv[0], yv[1], yv[7]);
    st = pooling::launch<float, pooling::Average, pooling::Forward>(x, y, pp, backend);
    st.event.wait();
    CHECK(to_host(y, 8)[0] == 6.f, "average pool value");
    pooling::launch<float, pooling::Max, pooling::Forward>(x, y, pp, backend);
    const auto gv = iota(8, 0);
    float* g = to_device(gv);
    st = pooling::launch<float, pooling::Max, pooling::Backpropagate>(x, y, g, dx, pp, backend);
    CHECK(st.status == StatusCode::OK, "max grad status");
    st.event.wait();
    const auto dxv = to_host(dx, 32);
    CHECK(dxv[10] == 1.f && dxv[0] == 0.f && dxv[31] == 8.f, "max grad routing %g %g %g", dxv[10], dxv[0], dxv[31]);

    std::vector<float> pv = {-2.f, -0.f, 0.5f, 3.f};
    float *pin = to_device(pv), *pout;
    pout = dev_alloc(16);
    pointwise::launch<float, pointwise::Relu, pointwise::Forward>(pin, pout, 4, backend).event.wait();
    auto r = to_host(pout, 4);
    CHECK(r[0] == 0.f && r[2] == 0.5f && r[3] == 3.f, "relu");
    pointwise::launch<float, pointwise::Tanh, pointwise::Forward>(pin, pout, 4, backend).event.wait();
    CHECK(std::fabs(to_host(pout, 4)[3] - std::tanh(3.f)) < 1e-6f, "tanh");
    pointwise::launch<float, pointwise::Relu, pointwise::Gradient>(pin, pin, pout, 4, backend).event.wait();
    r = to_host(pout, 4);
    CHECK(r[0] == 0.f && r[1] == 0.f && r[3] == 3.f, "relu gradient");
    // the reference's other operators; its gradient tests feed the same ramp as both tensors, so
    // log' = (1 / v) * v = 1 and sqrt' = (0.5 / v) * v = 0.5 (test/pointwise/{log,sqrt}_grad.cc)
    std::vector<float> qv = {1.f, 2.f, 3.f, 4.f};
    float* qin = to_device(qv);
    pointwise::launch<float, pointwise::Sqrt, pointwise::Forward>(qin, pout, 4, backend).event.wait();
    CHECK(to_host(pout, 4)[3] == 2.f, "sqrt");
    pointwise::launch<float, pointwise::Log, pointwise::Forward>(qin, pout, 4, backend).event.wait();
    CHECK(std::fabs(to_host(pout, 4)[1] - std::log(2.f)) < 1e-6f, "log");
    pointwise::launch<float, pointwise::Exp, pointwise::Forward>(pin, pout, 4, backend).event.wait();
    CHECK(std::fabs(to_host(pout, 4)[2] - std::exp(0.5f)) < 1e-6f, "exp");
    pointwise::launch<float, pointwise::Floor, pointwise::Forward>(pin, pout, 4, backend).event.wait();
    r = to_host(pout, 4);
    CHECK(r[0] == -2.f && r[2] == 0.f && r[3] == 3.f, "floor");
    pointwise::launch<float, pointwise::Log, pointwise::Gradient>(qin, qin, pout, 4, backend).event.wait();
    CHECK(std::fabs(to_host(pout, 4)[2] - 1.f) < 1e-6f, "log gradient");
    pointwise::launch<float, pointwise::Sqrt, pointwise::Gradient>(qin, qin, pout, 4, backend).event.wait();
    CHECK(std::fabs(to_host(pout, 4)[2] - 0.5f) < 1e-6f, "sqrt gradient");
    CHECK((pointwise::launch<float, pointwise::Floor, pointwise::Gradient>(qin, qin, pout, 4, backend).status ==
           StatusCode::InvalidParameter),
          "floor gradient accepted");

    binaryop::BinaryParams bp;
    bp.lhs_dims = {16, 2};
    bp.rhs_dims = {1, 2};
    std::vector<float> bias = {100.f, 200.f};
    float* b = to_device(bias);
    st = binaryop::launch<float, binaryop::Add>(x, b, dx, bp, backend);
    CHECK(st.status == StatusCode::OK, "bias status");
    st.event.wait();
    const auto bo = to_host(dx, 32);
    CHECK(bo[0] == 101.f && bo[1] == 202.f && bo[31] == 232.f, "bias add");
    // the other operators with broadcasting on both sides: x is the ramp 1..32 read as [16, 1, 2],
    // the right side [1, 3, 1] holds 2, 4, 8 (test/binaryop/binaryop_{sub,mul,div}.cc style shapes)
    {
      binaryop::BinaryParams bq;
      bq.lhs_dims = {16, 1, 2};
      bq.rhs_dims = {1, 3, 1};
      std::vector<float> pw = {2.f, 4.f, 8.f};
      float *pwd = to_device(pw), *bout = dev_alloc(96 * sizeof(float));
      st = binaryop::launch<float, binaryop::Div>(x, pwd, bout, bq, backend);
      CHECK(st.status == StatusCode::OK, "div status");
      st.event.wait();
      auto dv = to_host(bout, 96);  // out[i][j][k] = x[2 i + k] / pw[j]
      CHECK(dv[0] == 0.5f && dv[3] == 0.5f && dv[5] == 0.25f && dv[95] == 4.f, "div %g %g %g %g", dv[0], dv[3], dv[5], dv[95]);
      st = binaryop::launch<float, binaryop::Sub>(x, pwd, bout, bq, backend);
      st.event.wait();
      dv = to_host(bout, 96);
      CHECK(st.status == StatusCode::OK && dv[0] == -1.f && dv[95] == 24.f, "sub");
      st = binaryop::launch<float, binaryop::Mul>(x, pwd, bout, bq, backend);
      st.event.wait();
      dv = to_host(bout, 96);
      CHECK(st.status == StatusCode::OK && dv[1] == 4.f && dv[94] == 248.f, "mul");
      bq.rhs_dims = {2, 3, 1};
      CHECK((binaryop::launch<float, binaryop::Add>(x, pwd, bout, bq, backend).status == StatusCode::InvalidParameter),
            "extents 16 and 2 broadcast");
    }

    matmul::MatmulParams mp{2, 3, 4, 2, 0.f};
    const auto lv = iota(24, 0), rv = iota(16, 0);
    float *l = to_device(lv), *rr = to_device(rv), *mo;
    mo = dev_alloc(12 * sizeof(float));
    st = matmul::launch<float, false, false>(l, rr, mo, mp, backend);
    CHECK(st.status == StatusCode::OK, "matmul status");
    st.event.wait();
    const auto mv = to_host(mo, 12);
    CHECK(mv[0] == 1 * 1 + 2 * 3 + 3 * 5 + 4 * 7, "matmul[0] = %g", mv[0]);
    auto ev = backend.matmul<false, true>(l, l, mo, 0.f, 3, 4, 3);
    ev.wait();
    CHECK(to_host(mo, 9)[0] == 1 + 4 + 9 + 16, "backend.matmul transposed rhs");
  }
  // --- depthwise ---
  {
    Backend backend{nullptr};
    depthwise_conv2d::DepthwiseConv2DParams dp{};
    dp.channels = 2;
    dp.channel_multiplier = 1;
    dp.batch = 1;
    dp.in_rows = dp.in_cols = 3;
    dp.window_rows = dp.window_cols = 3;
    dp.stride_rows = dp.stride_cols = 1;
    dp = helpers::add_padding_to(dp, PaddingMode::VALID);
    const auto xv = iota(18, 0), wv = iota(18, 0);
    float *x = to_device(xv), *w = to_device(wv), *y;
    y = dev_alloc(8);
    auto st = depthwise_conv2d::launch<float, conv2d::conv_type::Forward>(x, w, y, dp, backend);
    CHECK(st.status == StatusCode::OK, "depthwise status");
    st.event.wait();
    float e0 = 0, e1 = 0;
    for (int i = 0; i < 9; ++i) {
      e0 += xv[2 * i] * wv[2 * i];
      e1 += xv[2 * i + 1] * wv[2 * i + 1];
    }
    const auto yv = to_host(y, 2);
    CHECK(yv[0] == e0 && yv[1] == e1, "depthwise values %g %g vs %g %g", yv[0], yv[1], e0, e1);
  }
  // --- compat: y = alpha*conv + beta*y, NHWC with an HWCF filter ---
  {
    using namespace compat;
    SNNHandle handle;
    SNNCreate(handle);
    TensorDescriptor xd, yd;
    FilterDescriptor wd;
    ConvolutionDescriptor cd;
    CHECK(cd.set2d(1, 1, 1, 1, 1, 1, ConvolutionMode::CONVOLUTION) == StatusCode::InvalidParameter, "CONVOLUTION mode");
    setConvolution2dDescriptor(cd, 1, 1, 1, 1, 1, 1, ConvolutionMode::CROSS_CORRELATION);
    setTensor4dDescriptor(xd, DataFormat::NHWC, SNNDataType::SNN_FLOAT, 1, 8, 5, 5);
    setFilter4dDescriptor(wd, SNNDataType::SNN_FLOAT, DataFormat::NHWC, 8, 8, 3, 3);
    int n, c, h, w;
    getConvolution2dForwardOutputDim(cd, xd, wd, &n, &c, &h, &w);
    CHECK(n == 1 && c == 8 && h == 5 && w == 5, "output dims %d %d %d %d", n, c, h, w);
    setTensor4dDescriptor(yd, DataFormat::NHWC, SNNDataType::SNN_FLOAT, n, c, h, w);
    const auto xv = iota(xd.getSize(), 4), wv = iota(wd.getSize(), 3);
    std::vector<float> y0(yd.getSize(), 10.f);
    float *x = to_device(xv), *wt = to_device(wv), *y = to_device(y0);
    const float alpha = 2.f, beta = 0.5f;
    auto st = convolutionForward(handle, &alpha, xd, x, wd, wt, cd, conv2d::Algorithm::Direct, nullptr, 0, &beta, yd, y);
    CHECK(st.status == StatusCode::OK, "compat forward status %d", int(st.status));
    st.event.wait();
    auto p = make_params(1, 5, 5, 8, 8, 3, 1, PaddingMode::SAME);
    auto ref = host_conv(xv, wv, p);
    for (auto& v : ref) v = 2.f * v + 5.f;
    CHECK(close(to_host(y, yd.getSize()), ref, 1e-6f), "compat forward blend");
    CHECK(convolutionForward(handle, &alpha, xd, x, wd, wt, cd, conv2d::Algorithm::WinogradLarge, nullptr, 0, &beta, yd, y)
                  .status == StatusCode::InvalidParameter,
          "WinogradLarge has no compat selector");
    PoolingDescriptor pd;
    CHECK(setPooling2dDescriptor(pd, PoolingMode::POOLING_MAX, NanPropagation::NOT_PROPAGATE_NAN, 2, 2, 0, 0, 2, 2) ==
              StatusCode::InvalidParameter,
          "POOLING_MAX is rejected");
  }
  cudaDeviceSynchronize();
  if (g_failures == 0) std::printf("api_test: all checks passed\n");
  return g_failures == 0 ? 0 : 1;
}
