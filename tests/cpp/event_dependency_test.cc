// The `events` argument of the launchers, in the manner of portDNN's event-dependency tests
// (test/helpers/dependency_check.h, test/conv2d/conv2d_event_dependencies_fixture.h,
// test/pooling/pooling_event_dependencies_test.cc, test/pointwise/pointwise_event_dependencies.cc,
// test/matmul/matmul_event_dependency.cc, test/transpose/transpose_event_dependencies.cc).
//
// Two backends on two CUDA streams.  The first runs a long chain of passes over a large tensor and
// only then produces the operand X of the operator under test; the operator is launched straight
// away on the second stream with the producer's event in its `events` list.  The checks:
//   - the result is computed from the FINAL X (without the dependency the second stream would read
//     X while it still holds its initial zeros);
//   - once the operator's event is complete the producer's event is complete too (the reference's
//     "Test 2"; its "Test 1" inspects sycl's running state, which has no CUDA counterpart).
// Exits 0 and prints "all checks passed".
//
//   g++ -std=c++17 -Iinclude -I$CUDA/include tests/cpp/event_dependency_test.cc -Lportdnn_b200 -lportdnn_b200 -lcudart
#include <cmath>
#include <cstdio>
#include <functional>
#include <vector>

#include "portdnn/binaryop/launch.h"
#include "portdnn/conv2d/launch.h"
#include "portdnn/conv2d/selector/direct_selector.h"
#include "portdnn/depthwise_conv2d/launch.h"
#include "portdnn/helpers/padding.h"
#include "portdnn/matmul/launch.h"
#include "portdnn/pointwise/launch.h"
#include "portdnn/pooling/launch.h"
#include "portdnn/transpose/launch.h"

using namespace sycldnn;
using Backend = backend::CUDABackend;
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

static float* dev_alloc(size_t n) {
  void* d = nullptr;
  cudaMalloc(&d, n * sizeof(float) + 16);
  cudaMemset(d, 0, n * sizeof(float));
  return static_cast<float*>(d);
}
static float* to_device(const Vec& h) {
  float* d = dev_alloc(h.size());
  cudaMemcpy(d, h.data(), h.size() * sizeof(float), cudaMemcpyHostToDevice);
  return d;
}
static Vec to_host(const float* d, size_t n) {
  Vec h(n);
  cudaMemcpy(h.data(), d, n * sizeof(float), cudaMemcpyDeviceToHost);
  return h;
}

// The slow producer: `passes` ReLU passes over a 256 MB tensor on the producer's stream, then one
// pass that writes the operand (X = relu(src), src positive, so X == src).
struct Producer {
  Backend backend;
  float *big_a, *big_b;
  size_t big_n = size_t(64) << 20;
  explicit Producer(cudaStream_t s) : backend(s), big_a(dev_alloc(big_n)), big_b(dev_alloc(big_n)) {}
  Event produce(const float* src, float* x, size_t n, int passes = 24) {
    for (int i = 0; i < passes; ++i)
      pointwise::launch<float, pointwise::Relu, pointwise::Forward>(i % 2 ? big_b : big_a, i % 2 ? big_a : big_b, big_n, backend);
    return pointwise::launch<float, pointwise::Relu, pointwise::Forward>(src, x, n, backend).event;
  }
};

// Runs one operator under test: `launch(x, deps)` queues it on the consumer stream and returns its
// status; `expect` is the host result computed from the final X.
static void check_op(const char* name, Producer& prod, const Vec& x_final, float* x_dev,
                     const std::function<SNNStatus(const std::vector<Event>&)>& launch, const float* out_dev,
                     const Vec& expect) {
  cudaMemset(x_dev, 0, x_final.size() * sizeof(float));
  float* src = to_device(x_final);
  cudaDeviceSynchronize();
  const Event produced = prod.produce(src, x_dev, x_final.size());
  const SNNStatus st = launch({produced});
  CHECK(st.status == StatusCode::OK, "%s: status %d", name, int(st.status));
  st.event.wait();
  CHECK(produced.complete(), "%s: the operator finished before the launch it depends on", name);
  const Vec got = to_host(out_dev, expect.size());
  float worst = 0.f;
  for (size_t i = 0; i < expect.size(); ++i) worst = std::fmax(worst, std::fabs(got[i] - expect[i]) / (std::fabs(expect[i]) + 1.f));
  CHECK(worst <= 1e-5f, "%s: result differs by %g (computed from a stale operand?)", name, worst);
  cudaDeviceSynchronize();
  cudaFree(src);
}

int main() {
  cudaStream_t sa, sb;
  cudaStreamCreateWithFlags(&sa, cudaStreamNonBlocking);
  cudaStreamCreateWithFlags(&sb, cudaStreamNonBlocking);
  Producer prod(sa);
  Backend consumer(sb);
  auto ramp = [](size_t n, int max) {
    Vec v(n);
    for (size_t i = 0; i < n; ++i) v[i] = float(i % size_t(max) + 1);
    return v;
  };

  // pointwise forward and gradient
  {
    const size_t n = 1 << 16;
    const Vec x = ramp(n, 97);
    float *xd = dev_alloc(n), *yd = dev_alloc(n);
    Vec e(n);
    for (size_t i = 0; i < n; ++i) e[i] = std::sqrt(x[i]);
    check_op("pointwise forward", prod, x, xd,
             [&](const std::vector<Event>& ev) { return pointwise::launch<float, pointwise::Sqrt, pointwise::Forward>(xd, yd, n, consumer, ev); }, yd, e);
    const Vec dy = ramp(n, 13);
    float* dyd = to_device(dy);
    for (size_t i = 0; i < n; ++i) e[i] = dy[i];  // relu gradient with a positive forward output
    check_op("pointwise gradient", prod, x, xd,
             [&](const std::vector<Event>& ev) { return pointwise::launch<float, pointwise::Relu, pointwise::Gradient>(xd, dyd, yd, n, consumer, ev); }, yd, e);
  }
  // binaryop (bias form) and transpose
  {
    const int rows = 4096, c = 32;
    const Vec x = ramp(size_t(rows) * c, 251), b = ramp(c, c);
    float *xd = dev_alloc(x.size()), *bd = to_device(b), *yd = dev_alloc(x.size());
    Vec e(x.size());
    for (size_t i = 0; i < x.size(); ++i) e[i] = x[i] + b[i % c];
    binaryop::BinaryParams bp;
    bp.lhs_dims = {rows, c};
    bp.rhs_dims = {1, c};
    check_op("binaryop add", prod, x, xd,
             [&](const std::vector<Event>& ev) { return binaryop::launch<float, binaryop::Add>(xd, bd, yd, bp, consumer, ev); }, yd, e);
    for (int r = 0; r < rows; ++r)
      for (int j = 0; j < c; ++j) e[size_t(j) * rows + r] = x[size_t(r) * c + j];
    check_op("transpose", prod, x, xd,
             [&](const std::vector<Event>& ev) { return transpose::launch<float>(xd, yd, {rows, c}, {1, 0}, consumer, ev); }, yd, e);
  }
  // matmul
  {
    const int m = 64, k = 32, n = 48;
    const Vec a = ramp(size_t(m) * k, 7), b = ramp(size_t(k) * n, 5);
    float *ad = dev_alloc(a.size()), *bd = to_device(b), *cd = dev_alloc(size_t(m) * n);
    Vec e(size_t(m) * n, 0.f);
    for (int i = 0; i < m; ++i)
      for (int j = 0; j < n; ++j)
        for (int l = 0; l < k; ++l) e[size_t(i) * n + j] += a[size_t(i) * k + l] * b[size_t(l) * n + j];
    check_op("matmul", prod, a, ad,
             [&](const std::vector<Event>& ev) {
               return matmul::launch<float, false, false>(ad, bd, cd, matmul::MatmulParams{1, m, k, n, 0.f}, consumer, ev);
             }, cd, e);
  }
  // convolution (the three passes), depthwise convolution, pooling forward and max gradient
  {
    conv2d::Conv2DParams p{};
    p.channels = 8, p.features = 8, p.batch = 2, p.in_rows = p.in_cols = 12;
    p.window_rows = p.window_cols = 3, p.stride_rows = p.stride_cols = 1, p.dilation_rows = p.dilation_cols = 1;
    p.groups = 1;
    p = helpers::add_padding_to(p, PaddingMode::SAME);
    const size_t nx = size_t(2) * 12 * 12 * 8, nw = 9 * 8 * 8;
    const Vec x = ramp(nx, 5), w = ramp(nw, 3), dy = ramp(nx, 4);
    float *xd = dev_alloc(nx), *wd = to_device(w), *yd = dev_alloc(nx), *dyd = to_device(dy), *dwd = dev_alloc(nw);
    auto at = [&](const Vec& t, int n, int h, int wc, int c) {
      return (h < 0 || h >= 12 || wc < 0 || wc >= 12) ? 0.f : t[((size_t(n) * 12 + h) * 12 + wc) * 8 + c];
    };
    Vec e(nx, 0.f);
    for (int n = 0; n < 2; ++n)
      for (int h = 0; h < 12; ++h)
        for (int wc = 0; wc < 12; ++wc)
          for (int f = 0; f < 8; ++f) {
            float acc = 0.f;
            for (int r = 0; r < 3; ++r)
              for (int s = 0; s < 3; ++s)
                for (int c = 0; c < 8; ++c) acc += at(x, n, h + r - 1, wc + s - 1, c) * w[((size_t(r) * 3 + s) * 8 + c) * 8 + f];
            e[((size_t(n) * 12 + h) * 12 + wc) * 8 + f] = acc;
          }
    conv2d::DirectSelector sel;
    check_op("conv2d forward", prod, x, xd,
             [&](const std::vector<Event>& ev) {
               return conv2d::launch<float, conv2d::conv_type::Forward>(xd, wd, yd, p, sel, consumer, nullptr, 0, ev);
             }, yd, e);
    // input backprop: the operand produced late is dy (slot "input")
    Vec ei(nx, 0.f);
    for (int n = 0; n < 2; ++n)
      for (int h = 0; h < 12; ++h)
        for (int wc = 0; wc < 12; ++wc)
          for (int c = 0; c < 8; ++c) {
            float acc = 0.f;
            for (int r = 0; r < 3; ++r)
              for (int s = 0; s < 3; ++s)
                for (int f = 0; f < 8; ++f) acc += at(dy, n, h - r + 1, wc - s + 1, f) * w[((size_t(r) * 3 + s) * 8 + c) * 8 + f];
            ei[((size_t(n) * 12 + h) * 12 + wc) * 8 + c] = acc;
          }
    check_op("conv2d input backprop", prod, dy, xd,
             [&](const std::vector<Event>& ev) {
               return conv2d::launch<float, conv2d::conv_type::InputBackprop>(xd, wd, yd, p, sel, consumer, nullptr, 0, ev);
             }, yd, ei);
    Vec ew(nw, 0.f);
    for (int r = 0; r < 3; ++r)
      for (int s = 0; s < 3; ++s)
        for (int c = 0; c < 8; ++c)
          for (int f = 0; f < 8; ++f) {
            float acc = 0.f;
            for (int n = 0; n < 2; ++n)
              for (int h = 0; h < 12; ++h)
                for (int wc = 0; wc < 12; ++wc) acc += at(x, n, h + r - 1, wc + s - 1, c) * dy[((size_t(n) * 12 + h) * 12 + wc) * 8 + f];
            ew[((size_t(r) * 3 + s) * 8 + c) * 8 + f] = acc;
          }
    check_op("conv2d filter backprop", prod, x, xd,
             [&](const std::vector<Event>& ev) {
               return conv2d::launch<float, conv2d::conv_type::FilterBackprop>(xd, dyd, dwd, p, sel, consumer, nullptr, 0, ev);
             }, dwd, ew);
    // depthwise: 8 channels, multiplier 1, same geometry
    depthwise_conv2d::DepthwiseConv2DParams dp{};
    dp.channels = 8, dp.channel_multiplier = 1, dp.batch = 2, dp.in_rows = dp.in_cols = 12;
    dp.window_rows = dp.window_cols = 3, dp.stride_rows = dp.stride_cols = 1;
    dp = helpers::add_padding_to(dp, PaddingMode::SAME);
    const Vec dwf = ramp(72, 3);
    float* dwfd = to_device(dwf);
    Vec ed(nx, 0.f);
    for (int n = 0; n < 2; ++n)
      for (int h = 0; h < 12; ++h)
        for (int wc = 0; wc < 12; ++wc)
          for (int c = 0; c < 8; ++c) {
            float acc = 0.f;
            for (int r = 0; r < 3; ++r)
              for (int s = 0; s < 3; ++s) acc += at(x, n, h + r - 1, wc + s - 1, c) * dwf[(size_t(r) * 3 + s) * 8 + c];
            ed[((size_t(n) * 12 + h) * 12 + wc) * 8 + c] = acc;
          }
    check_op("depthwise forward", prod, x, xd,
             [&](const std::vector<Event>& ev) {
               return depthwise_conv2d::launch<float, conv2d::conv_type::Forward>(xd, dwfd, yd, dp, consumer, ev);
             }, yd, ed);
    // pooling: 2x2/2 max forward, then its gradient with the pooled tensor produced late
    pooling::PoolingParams pp{};
    pp.in_rows = pp.in_cols = 12, pp.window_rows = pp.window_cols = 2, pp.stride_rows = pp.stride_cols = 2;
    pp.batch = 2, pp.channels = 8;
    pp = helpers::add_padding_to(pp, PaddingMode::VALID);
    const Vec xp = ramp(nx, 1031);
    const size_t ny = size_t(2) * 6 * 6 * 8;
    Vec ep(ny);
    for (int n = 0; n < 2; ++n)
      for (int h = 0; h < 6; ++h)
        for (int wc = 0; wc < 6; ++wc)
          for (int c = 0; c < 8; ++c) {
            float m = -1e30f;
            for (int r = 0; r < 2; ++r)
              for (int s = 0; s < 2; ++s) m = std::fmax(m, at(xp, n, 2 * h + r, 2 * wc + s, c));
            ep[((size_t(n) * 6 + h) * 6 + wc) * 8 + c] = m;
          }
    float* pyd = dev_alloc(ny);
    check_op("pooling forward", prod, xp, xd,
             [&](const std::vector<Event>& ev) {
               return pooling::launch<float, pooling::Max, pooling::Forward>(xd, pyd, pp, consumer, ev);
             }, pyd, ep);
    const Vec pdy = ramp(ny, 9);
    float *pdyd = to_device(pdy), *pxd = to_device(xp), *pdxd = dev_alloc(nx);
    Vec eg(nx, 0.f);
    for (int n = 0; n < 2; ++n)
      for (int h = 0; h < 6; ++h)
        for (int wc = 0; wc < 6; ++wc)
          for (int c = 0; c < 8; ++c) {
            const float m = ep[((size_t(n) * 6 + h) * 6 + wc) * 8 + c];
            bool given = false;
            for (int r = 0; r < 2 && !given; ++r)
              for (int s = 0; s < 2 && !given; ++s)
                if (at(xp, n, 2 * h + r, 2 * wc + s, c) == m) {
                  eg[((size_t(n) * 12 + 2 * h + r) * 12 + 2 * wc + s) * 8 + c] += pdy[((size_t(n) * 6 + h) * 6 + wc) * 8 + c];
                  given = true;
                }
          }
    float* lated = dev_alloc(ny);  // the pooled tensor y, produced late
    check_op("pooling max gradient", prod, ep, lated,
             [&](const std::vector<Event>& ev) {
               return pooling::launch<float, pooling::Max, pooling::Backpropagate>(pxd, lated, pdyd, pdxd, pp, consumer, ev);
             }, pdxd, eg);
  }
  cudaDeviceSynchronize();
  if (g_failures == 0) std::printf("event_dependency_test: all checks passed\n");
  return g_failures == 0 ? 0 : 1;
}
