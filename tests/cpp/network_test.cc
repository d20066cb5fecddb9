// Builds two small networks out of the layer wrappers (include/tools/layer.h, network.h), the way
// portDNN's samples/networks/{vgg,resnet50} build theirs: a VGG-style stack (conv - bias - relu -
// max pool, twice, then a fully connected layer and softmax) and a ResNet-style unit (conv -
// frozen batchnorm - relu - average pool).  Seeded weights; every network output is compared with
// host loops written from the operator definitions.  Exits 0 and prints "all checks passed".
//
//   g++ -std=c++17 -Iinclude -I$CUDA/include tests/cpp/network_test.cc -Lportdnn_b200 -lportdnn_b200 -lcudart
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>

#include "portdnn/helpers/padding.h"
#include "tools/network.h"

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

static Vec random_vec(size_t n, float scale, unsigned seed) {
  std::mt19937 gen(seed);
  std::uniform_real_distribution<float> dist(-scale, scale);
  Vec v(n);
  for (float& x : v) x = dist(gen);
  return v;
}
static float* to_device(const Vec& h) {
  void* d = nullptr;
  cudaMalloc(&d, h.size() * sizeof(float) + 16);
  cudaMemcpy(d, h.data(), h.size() * sizeof(float), cudaMemcpyHostToDevice);
  return static_cast<float*>(d);
}
static float* device_buffer(size_t n) {
  void* d = nullptr;
  cudaMalloc(&d, n * sizeof(float) + 16);
  cudaMemset(d, 0, n * sizeof(float));
  return static_cast<float*>(d);
}
static bool close(const Vec& a, const Vec& b, float rel) {
  if (a.size() != b.size()) return false;
  float scale = 1e-30f, err = 0.f;
  for (size_t i = 0; i < a.size(); ++i) {
    scale = std::fmax(scale, std::fabs(b[i]));
    err = std::fmax(err, std::fabs(a[i] - b[i]));
  }
  return err <= rel * scale;
}

// ---- host definitions of the operators --------------------------------------------------------
static Vec host_conv(const Vec& x, const Vec& w, const conv2d::Conv2DParams& p) {
  Vec y(size_t(p.batch) * p.out_rows * p.out_cols * p.features, 0.f);
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
static void host_bias_relu(Vec& y, const Vec& bias, bool relu) {
  const size_t C = bias.size();
  for (size_t i = 0; i < y.size(); ++i) {
    y[i] += bias[i % C];
    if (relu && y[i] < 0.f) y[i] = 0.f;
  }
}
static Vec host_pool(const Vec& x, const pooling::PoolingParams& p, bool average) {
  Vec y(size_t(p.batch) * p.out_rows * p.out_cols * p.channels);
  for (int n = 0; n < p.batch; ++n)
    for (int oh = 0; oh < p.out_rows; ++oh)
      for (int ow = 0; ow < p.out_cols; ++ow)
        for (int c = 0; c < p.channels; ++c) {
          float best = -INFINITY, sum = 0.f;
          int count = 0;
          for (int r = 0; r < p.window_rows; ++r)
            for (int s = 0; s < p.window_cols; ++s) {
              const int ih = oh * p.stride_rows - p.pad_rows + r, iw = ow * p.stride_cols - p.pad_cols + s;
              if (ih < 0 || ih >= p.in_rows || iw < 0 || iw >= p.in_cols) continue;
              const float v = x[((size_t(n) * p.in_rows + ih) * p.in_cols + iw) * p.channels + c];
              best = std::fmax(best, v);
              sum += v;
              ++count;
            }
          y[((size_t(n) * p.out_rows + oh) * p.out_cols + ow) * p.channels + c] = average ? sum / float(count) : best;
        }
  return y;
}
static Vec host_matmul(const Vec& a, const Vec& b, int m, int k, int n) {
  Vec out(size_t(m) * n);
  for (int i = 0; i < m; ++i)
    for (int j = 0; j < n; ++j) {
      double acc = 0;
      for (int l = 0; l < k; ++l) acc += double(a[size_t(i) * k + l]) * b[size_t(l) * n + j];
      out[size_t(i) * n + j] = float(acc);
    }
  return out;
}
static Vec host_softmax(const Vec& x, int C) {
  Vec y(x.size());
  for (size_t row = 0; row < x.size() / size_t(C); ++row) {
    float m = -INFINITY, sum = 0.f;
    for (int c = 0; c < C; ++c) m = std::fmax(m, x[row * C + c]);
    for (int c = 0; c < C; ++c) sum += std::exp(x[row * C + c] - m);
    for (int c = 0; c < C; ++c) y[row * C + c] = std::exp(x[row * C + c] - m) / sum;
  }
  return y;
}
static Vec host_batchnorm(const Vec& x, const Vec& beta, const Vec& gamma, const Vec& mean, const Vec& var, float eps) {
  const size_t C = beta.size();
  Vec y(x.size());
  for (size_t i = 0; i < x.size(); ++i) {
    const size_t c = i % C;
    y[i] = (x[i] - mean[c]) / std::sqrt(var[c] + eps) * gamma[c] + beta[c];
  }
  return y;
}

static conv2d::Conv2DParams conv_params(int batch, int hw, int channels, int features, int window) {
  conv2d::Conv2DParams p{};
  p.channels = channels;
  p.features = features;
  p.batch = batch;
  p.in_rows = p.in_cols = hw;
  p.window_rows = p.window_cols = window;
  p.stride_rows = p.stride_cols = 1;
  p.dilation_rows = p.dilation_cols = 1;
  p.groups = 1;
  return helpers::add_padding_to(p, PaddingMode::SAME);
}
static pooling::PoolingParams pool_params(int batch, int hw, int channels, int window, int stride) {
  pooling::PoolingParams p{};
  p.in_rows = p.in_cols = hw;
  p.window_rows = p.window_cols = window;
  p.stride_rows = p.stride_cols = stride;
  p.batch = batch;
  p.channels = channels;
  return helpers::add_padding_to(p, PaddingMode::VALID);
}

int main() {
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
    std::printf("no CUDA device\n");
    return 2;
  }
  cudaStream_t stream;
  cudaStreamCreate(&stream);
  Backend backend(stream);
  auto selector = conv2d::get_default_selector();

  // ---- VGG-style: [conv3x3 - bias - relu - maxpool2x2] x 2, FC, bias, softmax ---------------------
  {
    const int N = 2, HW = 16, C0 = 8, C1 = 16, C2 = 32, CLASSES = 10;
    const Vec x = random_vec(size_t(N) * HW * HW * C0, 1.f, 1);
    const auto cp1 = conv_params(N, HW, C0, C1, 3);
    const auto pp1 = pool_params(N, HW, C1, 2, 2);
    const auto cp2 = conv_params(N, HW / 2, C1, C2, 3);
    const auto pp2 = pool_params(N, HW / 2, C2, 2, 2);
    const int flat = (HW / 4) * (HW / 4) * C2;
    const Vec w1 = random_vec(size_t(9) * C0 * C1, 0.2f, 2), b1 = random_vec(C1, 0.5f, 3);
    const Vec w2 = random_vec(size_t(9) * C1 * C2, 0.15f, 4), b2 = random_vec(C2, 0.5f, 5);
    const Vec wf = random_vec(size_t(flat) * CLASSES, 0.05f, 6), bf = random_vec(CLASSES, 0.5f, 7);

    float* d_x = to_device(x);
    float *d_w1 = to_device(w1), *d_b1 = to_device(b1), *d_w2 = to_device(w2), *d_b2 = to_device(b2);
    float *d_wf = to_device(wf), *d_bf = to_device(bf);
    const size_t n1 = size_t(N) * HW * HW * C1, n2 = size_t(N) * (HW / 2) * (HW / 2) * C2;
    float *c1 = device_buffer(n1), *a1 = device_buffer(n1), *r1 = device_buffer(n1), *p1 = device_buffer(n1 / 4);
    float *c2 = device_buffer(n2), *a2 = device_buffer(n2), *r2 = device_buffer(n2), *p2 = device_buffer(n2 / 4);
    float *fc = device_buffer(size_t(N) * CLASSES), *fb = device_buffer(size_t(N) * CLASSES),
          *sm = device_buffer(size_t(N) * CLASSES), *sm_ws = device_buffer(N);

    Vec result;
    Network<float, Backend> net(backend, result);
    net.add_layer(new ConvolutionLayer<float, Backend>(cp1, d_x, d_w1, c1, nullptr, 0, backend, *selector));
    net.add_layer(new BiasAddLayer<float, Backend>({{N, HW, HW, C1}, {C1}}, c1, d_b1, a1, backend));
    net.add_layer(new ActivationLayer<float, Backend, pointwise::Relu>({int(n1)}, a1, r1, backend));
    net.add_layer(new PoolingLayer<float, Backend, pooling::Max>(pp1, r1, p1, backend));
    net.add_layer(new ConvolutionLayer<float, Backend>(cp2, p1, d_w2, c2, nullptr, 0, backend, *selector));
    net.add_layer(new BiasAddLayer<float, Backend>({{N, HW / 2, HW / 2, C2}, {C2}}, c2, d_b2, a2, backend));
    net.add_layer(new ActivationLayer<float, Backend, pointwise::Relu>({int(n2)}, a2, r2, backend));
    net.add_layer(new PoolingLayer<float, Backend, pooling::Max>(pp2, r2, p2, backend));
    matmul::MatmulParams mp{1, N, flat, CLASSES, 0.f};
    net.add_layer(new FCLayer<float, Backend>(mp, p2, d_wf, fc, backend));
    net.add_layer(new BiasAddLayer<float, Backend>({{N, CLASSES}, {CLASSES}}, fc, d_bf, fb, backend));
    softmax::SoftmaxParams sp{CLASSES, N, 1, 1};
    net.add_layer(new SoftmaxLayer<float, Backend>(sp, fb, sm_ws, sm, backend));
    CHECK(net.get_network_size() == 11, "eleven layers expected");

    SNNStatus st = net.test();
    CHECK(st.status == StatusCode::OK, "VGG-style network: status %d (%s)", int(st.status), pdnn_last_error());

    Vec h = host_conv(x, w1, cp1);
    host_bias_relu(h, b1, true);
    h = host_pool(h, pp1, false);
    h = host_conv(h, w2, cp2);
    host_bias_relu(h, b2, true);
    h = host_pool(h, pp2, false);
    h = host_matmul(h, wf, N, flat, CLASSES);
    host_bias_relu(h, bf, false);
    h = host_softmax(h, CLASSES);
    CHECK(result.size() == size_t(N) * CLASSES, "softmax output size %zu", result.size());
    CHECK(close(result, h, 2e-4f), "VGG-style network output differs from the host composition");
    float total = 0.f;
    for (int c = 0; c < CLASSES; ++c) total += result[c];
    CHECK(std::fabs(total - 1.f) < 1e-5f, "softmax row sums to %f", total);

    // run() queues the same work without waiting in between
    st = net.run();
    CHECK(st.status == StatusCode::OK, "run() status %d", int(st.status));
    st.event.wait_and_throw();
    st = net.dump_network_output();
    CHECK(st.status == StatusCode::OK && close(result, h, 2e-4f), "run() + dump_network_output() differs");
  }

  // ---- ResNet-style unit: conv1x1 - frozen batchnorm - relu - global average pool ----------------
  {
    const int N = 3, HW = 7, C0 = 16, C1 = 24;
    const Vec x = random_vec(size_t(N) * HW * HW * C0, 1.f, 11);
    const auto cp = conv_params(N, HW, C0, C1, 1);
    auto pp = pool_params(N, HW, C1, HW, 1);
    const Vec w = random_vec(size_t(C0) * C1, 0.3f, 12);
    const Vec beta = random_vec(C1, 0.5f, 13), gamma = random_vec(C1, 1.f, 14), mean = random_vec(C1, 0.5f, 15);
    Vec var = random_vec(C1, 0.4f, 16);
    for (float& v : var) v += 1.f;
    const size_t n1 = size_t(N) * HW * HW * C1;
    float *d_x = to_device(x), *d_w = to_device(w), *d_beta = to_device(beta), *d_gamma = to_device(gamma),
          *d_mean = to_device(mean), *d_var = to_device(var);
    float *c1 = device_buffer(n1), *bn = device_buffer(n1), *r1 = device_buffer(n1), *gp = device_buffer(size_t(N) * C1);

    Vec result;
    Network<float, Backend> net(backend, result);
    net.add_layer(new ConvolutionLayer<float, Backend>(cp, d_x, d_w, c1, nullptr, 0, backend, *selector));
    batchnorm::BatchNormParams bp{N, HW, HW, C1, false, 1e-3f, 0.9f};
    net.add_layer(new BatchNormFrozenLayer<float, Backend>(bp, c1, d_beta, d_gamma, d_mean, d_var, bn, backend));
    net.add_layer(new ActivationLayer<float, Backend, pointwise::Relu>({int(n1)}, bn, r1, backend));
    net.add_layer(new PoolingLayer<float, Backend, pooling::Average>(pp, r1, gp, backend));
    SNNStatus st = net.test();
    CHECK(st.status == StatusCode::OK, "ResNet-style unit: status %d (%s)", int(st.status), pdnn_last_error());

    Vec h = host_conv(x, w, cp);
    h = host_batchnorm(h, beta, gamma, mean, var, 1e-3f);
    for (float& v : h) v = std::fmax(v, 0.f);
    h = host_pool(h, pp, true);
    CHECK(close(result, h, 2e-4f), "ResNet-style unit output differs from the host composition");

    // the training-mode layer on the same tensor: output as above, running statistics from the batch
    float *run_mean = device_buffer(C1), *run_var = device_buffer(C1), *bn2 = device_buffer(n1);
    bp.is_training = true;
    BatchNormTrainingLayer<float, Backend> train(bp, c1, d_beta, d_gamma, d_mean, d_var, run_mean, run_var, bn2, backend);
    st = train.run();
    CHECK(st.status == StatusCode::OK, "training batchnorm: status %d", int(st.status));
    st.event.wait_and_throw();
    Vec conv = host_conv(x, w, cp), rm(C1), rv(C1), got_mean(C1), got_var(C1);
    const size_t rows = size_t(N) * HW * HW;
    for (int c = 0; c < C1; ++c) {
      double s = 0, q = 0;
      for (size_t i = 0; i < rows; ++i) s += conv[i * C1 + c];
      const double m = s / double(rows);
      for (size_t i = 0; i < rows; ++i) q += (conv[i * C1 + c] - m) * (conv[i * C1 + c] - m);
      rm[c] = float(m * 0.1 + mean[c] * 0.9);
      rv[c] = float(q / double(rows) * 0.1 + var[c] * 0.9);
    }
    cudaMemcpy(got_mean.data(), run_mean, C1 * sizeof(float), cudaMemcpyDeviceToHost);
    cudaMemcpy(got_var.data(), run_var, C1 * sizeof(float), cudaMemcpyDeviceToHost);
    CHECK(close(got_mean, rm, 1e-4f) && close(got_var, rv, 1e-4f), "running statistics differ");
  }

  // ---- the gradient launch forms of batchnorm and softmax ------------------------------------------
  {
    const int N = 2, HW = 5, C = 8;
    const size_t n = size_t(N) * HW * HW * C, rows = size_t(N) * HW * HW;
    const Vec x = random_vec(n, 1.f, 21), dy = random_vec(n, 1.f, 22), gamma = random_vec(C, 1.f, 23);
    const Vec mean = random_vec(C, 0.5f, 24);
    Vec var = random_vec(C, 0.4f, 25);
    for (float& v : var) v += 1.f;
    float *d_x = to_device(x), *d_dy = to_device(dy), *d_gamma = to_device(gamma), *d_mean = to_device(mean),
          *d_var = to_device(var);
    float *dx = device_buffer(n), *dbeta = device_buffer(C), *dgamma = device_buffer(C);
    batchnorm::BatchNormParams bp{N, HW, HW, C, false, 1e-3f, 0.9f};
    // frozen: eight-pointer form, dx = dy * gamma / sqrt(var + eps), dbeta = sum dy
    SNNStatus st = batchnorm::launch<float, Backend, batchnorm::Gradient>(d_x, d_dy, d_gamma, d_mean, d_var, dbeta, dgamma,
                                                                          dx, bp, backend);
    CHECK(st.status == StatusCode::OK, "frozen batchnorm gradient: status %d", int(st.status));
    st.event.wait_and_throw();
    Vec got(n), got_beta(C), exp_dx(n), exp_beta(C, 0.f);
    cudaMemcpy(got.data(), dx, n * sizeof(float), cudaMemcpyDeviceToHost);
    cudaMemcpy(got_beta.data(), dbeta, C * sizeof(float), cudaMemcpyDeviceToHost);
    for (size_t i = 0; i < n; ++i) {
      exp_dx[i] = dy[i] * (gamma[i % C] / std::sqrt(var[i % C] + 1e-3f));
      exp_beta[i % C] += dy[i];
    }
    CHECK(close(got, exp_dx, 1e-5f) && close(got_beta, exp_beta, 1e-4f), "frozen batchnorm gradient differs");
    // training: six-pointer form; dbeta is again sum dy, and the input gradient sums to ~0 per channel
    bp.is_training = true;
    st = batchnorm::launch<float, Backend, batchnorm::Gradient>(d_x, d_dy, d_gamma, dbeta, dgamma, dx, bp, backend);
    CHECK(st.status == StatusCode::OK, "training batchnorm gradient: status %d", int(st.status));
    st.event.wait_and_throw();
    cudaMemcpy(got.data(), dx, n * sizeof(float), cudaMemcpyDeviceToHost);
    cudaMemcpy(got_beta.data(), dbeta, C * sizeof(float), cudaMemcpyDeviceToHost);
    CHECK(close(got_beta, exp_beta, 1e-4f), "training batchnorm beta gradient differs");
    for (int c = 0; c < C; ++c) {
      double s = 0;
      for (size_t r = 0; r < rows; ++r) s += got[r * C + c];
      CHECK(std::fabs(s) < 1e-3, "training batchnorm input gradient of channel %d sums to %g", c, s);
    }
    // softmax gradient: rows of (dy - sum(dy*y)) * y sum to zero
    softmax::SoftmaxParams sp{C, N, HW, HW};
    float *y = device_buffer(n), *ws = device_buffer(rows);
    st = softmax::launch<float, softmax::Forward, Backend>(d_x, ws, y, sp, backend);
    CHECK(st.status == StatusCode::OK, "softmax forward: status %d", int(st.status));
    st = softmax::launch<float, softmax::Gradient, Backend>(y, d_dy, ws, dx, sp, backend);
    CHECK(st.status == StatusCode::OK, "softmax gradient: status %d", int(st.status));
    st.event.wait_and_throw();
    cudaMemcpy(got.data(), dx, n * sizeof(float), cudaMemcpyDeviceToHost);
    for (size_t r = 0; r < rows; ++r) {
      double s = 0;
      for (int c = 0; c < C; ++c) s += got[r * C + c];
      if (std::fabs(s) > 1e-5) {
        CHECK(false, "softmax gradient row %zu sums to %g", r, s);
        break;
      }
    }
  }

  if (g_failures == 0) std::printf("all checks passed\n");
  return g_failures == 0 ? 0 : 1;
}
