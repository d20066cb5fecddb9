// The cuDNN-style batchnorm wrappers (include/portdnn/compat/batchnorm.hpp) in the manner of
// portDNN's test/compat/batchnorm_compat.cc: inputs are the repeating ramps 1, 2, .., max the
// reference's tests use, results are compared with host loops written from the operator's
// definition, and the 1x1x1x8 training case is also checked against the values the reference's
// test lists.  Exits 0 and prints "all checks passed".
//
//   g++ -std=c++17 -Iinclude -I$CUDA/include tests/cpp/compat_batchnorm_test.cc -Lportdnn_b200 -lportdnn_b200 -lcudart
#include <cmath>
#include <cstdio>
#include <vector>

#include "portdnn/compat/batchnorm.hpp"

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

// 1, 2, .., max, 1, 2, ..: the reference's iota_initialised_data
static Vec ramp(size_t n, int max) {
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
static float max_err(const Vec& a, const Vec& b) {
  float scale = 1e-30f, err = 0.f;
  for (size_t i = 0; i < a.size(); ++i) {
    scale = std::fmax(scale, std::fabs(b[i]));
    err = std::fmax(err, std::fabs(a[i] - b[i]));
  }
  return err / scale;
}

struct Case {
  int n, h, w, c;
  float alpha, beta;
};

// y = gamma * (x - mean) / sqrt(var + eps) + beta with the statistics handed in
static Vec host_forward(const Vec& x, const Vec& beta, const Vec& gamma, const Vec& mean, const Vec& var, int c,
                        float eps) {
  Vec y(x.size());
  for (size_t i = 0; i < x.size(); ++i) {
    const int ch = int(i % size_t(c));
    y[i] = float(double(gamma[ch]) * (double(x[i]) - mean[ch]) / std::sqrt(double(var[ch]) + eps) + beta[ch]);
  }
  return y;
}
static void host_batch_stats(const Vec& x, int c, Vec* mean, Vec* var) {
  const size_t rows = x.size() / size_t(c);
  mean->assign(c, 0.f);
  var->assign(c, 0.f);
  for (int ch = 0; ch < c; ++ch) {
    double m = 0, v = 0;
    for (size_t r = 0; r < rows; ++r) m += x[r * c + ch];
    m /= double(rows);
    for (size_t r = 0; r < rows; ++r) v += (x[r * c + ch] - m) * (x[r * c + ch] - m);
    (*mean)[ch] = float(m);
    (*var)[ch] = float(v / double(rows));
  }
}

static void test_forward(SNNHandle& handle, const Case& k, bool training, bool use_cache) {
  const float eps = 0.001f, factor = 0.01f;
  const size_t n = size_t(k.n) * k.h * k.w * k.c;
  const Vec x = ramp(n, 5), beta = ramp(k.c, 4), gamma = ramp(k.c, 5), mean = ramp(k.c, 6), var = ramp(k.c, 7);
  const Vec y_prev = ramp(n, 2048);
  TensorDescriptor x_desc, bn_desc;
  x_desc.set4d(DataFormat::NHWC, k.n, k.c, k.h, k.w);
  bn_desc.set4d(DataFormat::NHWC, 1, k.c, 1, 1);
  float *d_x = to_device(x), *d_scale = to_device(beta), *d_bias = to_device(gamma), *d_mean = to_device(mean),
        *d_var = to_device(var), *d_y = to_device(y_prev);
  float *d_save_mean = use_cache ? to_device(Vec(k.c, 0.f)) : nullptr,
        *d_save_var = use_cache ? to_device(Vec(k.c, 0.f)) : nullptr;
  SNNStatus st;
  if (training)
    st = batchNormalizationForwardTraining(handle, BATCHNORM_SPATIAL, &k.alpha, &k.beta, x_desc, d_x, x_desc, d_y, bn_desc,
                                           d_scale, d_bias, double(factor), d_mean, d_var, double(eps), d_save_mean,
                                           d_save_var);
  else
    st = batchNormalizationForwardInference(handle, BATCHNORM_SPATIAL, &k.alpha, &k.beta, x_desc, d_x, x_desc, d_y,
                                            bn_desc, d_scale, d_bias, d_mean, d_var, double(eps));
  CHECK(st.status == StatusCode::OK, "forward status %d", int(st.status));
  st.event.wait_and_throw();
  Vec expect = host_forward(x, beta, gamma, mean, var, k.c, eps);
  for (size_t i = 0; i < n; ++i) expect[i] = k.alpha * expect[i] + k.beta * y_prev[i];
  const float e = max_err(to_host(d_y, n), expect);
  CHECK(e <= 1e-5f, "%s forward %dx%dx%dx%d alpha %g beta %g: error %g", training ? "training" : "inference", k.n, k.h,
        k.w, k.c, k.alpha, k.beta, e);
  if (training) {
    Vec bm, bv, em(k.c), ev(k.c);
    host_batch_stats(x, k.c, &bm, &bv);
    for (int c = 0; c < k.c; ++c) {
      em[c] = bm[c] * factor + mean[c] * (1.f - factor);
      ev[c] = bv[c] * factor + var[c] * (1.f - factor);
    }
    CHECK(max_err(to_host(d_mean, k.c), em) <= 2e-5f, "running mean differs");
    CHECK(max_err(to_host(d_var, k.c), ev) <= 2e-5f, "running variance differs");
    if (use_cache) {
      CHECK(max_err(to_host(d_save_mean, k.c), em) <= 2e-5f, "saved mean differs");
      CHECK(max_err(to_host(d_save_var, k.c), ev) <= 2e-5f, "saved variance differs");
    }
  } else {
    CHECK(max_err(to_host(d_mean, k.c), mean) == 0.f && max_err(to_host(d_var, k.c), var) == 0.f,
          "inference changed the statistics");
  }
  for (float* p : {d_x, d_scale, d_bias, d_mean, d_var, d_y, d_save_mean, d_save_var}) cudaFree(p);
}

// The values listed by the reference's ForwardTr1x1x1x8Cache / NoCache tests.
static void test_known_answer(SNNHandle& handle, bool use_cache) {
  const Vec exp_mean = {1.f, 2.f, 3.f, 4.f, 5.f, 5.949999999999999f, 1.01f, 2.01f};
  const Vec exp_var = {0.99f, 1.98f, 2.9699999999999998f, 3.96f, 4.95f, 5.9399999999999995f, 6.93f, 0.99f};
  const Vec exp_out = {1.f, 2.f, 3.f, 4.f, 1.f, -0.04107137012493428f, 3.7558749568782206f, 6.998501124063319f};
  const int c = 8;
  const float alpha = 1.f, beta_scalar = 0.f;
  TensorDescriptor x_desc, bn_desc;
  x_desc.set4d(DataFormat::NHWC, 1, c, 1, 1);
  bn_desc.set4d(DataFormat::NHWC, 1, c, 1, 1);
  float *d_x = to_device(ramp(c, 5)), *d_scale = to_device(ramp(c, 4)), *d_bias = to_device(ramp(c, 5)),
        *d_mean = to_device(ramp(c, 6)), *d_var = to_device(ramp(c, 7)), *d_y = to_device(ramp(c, 2048));
  float *d_sm = use_cache ? to_device(Vec(c, 0.f)) : nullptr, *d_sv = use_cache ? to_device(Vec(c, 0.f)) : nullptr;
  SNNStatus st = batchNormalizationForwardTraining(handle, BATCHNORM_SPATIAL, &alpha, &beta_scalar, x_desc, d_x, x_desc,
                                                   d_y, bn_desc, d_scale, d_bias, 0.01, d_mean, d_var, 0.001, d_sm, d_sv);
  CHECK(st.status == StatusCode::OK, "known-answer status %d", int(st.status));
  st.event.wait_and_throw();
  CHECK(max_err(to_host(d_mean, c), exp_mean) <= 2e-5f, "known-answer running mean");
  CHECK(max_err(to_host(d_var, c), exp_var) <= 1e-5f, "known-answer running variance");
  CHECK(max_err(to_host(d_y, c), exp_out) <= 1e-5f, "known-answer output");
  if (use_cache) {
    CHECK(max_err(to_host(d_sm, c), exp_mean) <= 1e-5f, "known-answer saved mean");
    CHECK(max_err(to_host(d_sv, c), exp_var) <= 1e-5f, "known-answer saved variance");
  }
  for (float* p : {d_x, d_scale, d_bias, d_mean, d_var, d_y, d_sm, d_sv}) cudaFree(p);
}

static void test_backward(SNNHandle& handle, const Case& k, float alpha_param, float beta_param) {
  const float eps = 0.001f;
  const int c = k.c;
  const size_t n = size_t(k.n) * k.h * k.w * c, rows = n / size_t(c);
  Vec x = ramp(n, 7), dy = ramp(n, 3);
  for (size_t i = 0; i < n; ++i) {
    x[i] += 0.25f * float(i % 11);  // no constant channels
    dy[i] += 0.5f * float(i % 7);   // correlated with x: a gamma gradient well away from zero
  }
  const Vec gamma = ramp(c, 5), dx_prev = ramp(n, 9), dscale_prev = ramp(c, 3), dbias_prev = ramp(c, 4);
  TensorDescriptor x_desc, bn_desc;
  x_desc.set4d(DataFormat::NHWC, k.n, c, k.h, k.w);
  bn_desc.set4d(DataFormat::NHWC, 1, c, 1, 1);
  float *d_x = to_device(x), *d_dy = to_device(dy), *d_gamma = to_device(gamma), *d_dx = to_device(dx_prev),
        *d_dscale = to_device(dscale_prev), *d_dbias = to_device(dbias_prev);
  SNNStatus st = batchNormalizationBackward(handle, BATCHNORM_SPATIAL, &k.alpha, &k.beta, &alpha_param, &beta_param,
                                            x_desc, d_x, x_desc, d_dy, x_desc, d_dx, bn_desc, d_gamma, d_dscale, d_dbias,
                                            double(eps), nullptr, nullptr);
  CHECK(st.status == StatusCode::OK, "backward status %d", int(st.status));
  st.event.wait_and_throw();
  Vec mean, var, exp_dx(n), exp_dbeta(c), exp_dgamma(c);
  host_batch_stats(x, c, &mean, &var);
  for (int ch = 0; ch < c; ++ch) {
    const double inv = 1.0 / std::sqrt(double(var[ch]) + eps);
    double sb = 0, sg = 0;
    for (size_t r = 0; r < rows; ++r) {
      sb += dy[r * c + ch];
      sg += dy[r * c + ch] * (x[r * c + ch] - mean[ch]) * inv;
    }
    for (size_t r = 0; r < rows; ++r) {
      const double xh = (x[r * c + ch] - mean[ch]) * inv;
      const double g = gamma[ch] * inv * (dy[r * c + ch] - sb / double(rows) - xh * sg / double(rows));
      exp_dx[r * c + ch] = float(k.alpha * g + k.beta * dx_prev[r * c + ch]);
    }
    // the additive term's gradient lands in resultBnScaleDiff, the multiplicative one's in resultBnBiasDiff
    exp_dbeta[ch] = float(alpha_param * sb + beta_param * dscale_prev[ch]);
    exp_dgamma[ch] = float(alpha_param * sg + beta_param * dbias_prev[ch]);
  }
  const float e_dx = max_err(to_host(d_dx, n), exp_dx), e_b = max_err(to_host(d_dscale, c), exp_dbeta),
              e_g = max_err(to_host(d_dbias, c), exp_dgamma);
  CHECK(e_dx <= 1e-4f && e_b <= 1e-5f && e_g <= 1e-4f, "backward %dx%dx%dx%d alpha %g beta %g / %g %g: errors %g %g %g",
        k.n, k.h, k.w, c, k.alpha, k.beta, alpha_param, beta_param, e_dx, e_b, e_g);
  for (float* p : {d_x, d_dy, d_gamma, d_dx, d_dscale, d_dbias}) cudaFree(p);
}

int main() {
  SNNHandle handle;
  CHECK(SNNCreate(handle) == StatusCode::OK, "SNNCreate");
  const float blends[][2] = {{1.f, 0.f}, {0.5f, 0.f}, {1.f, 1.f}, {2.f, 0.5f}, {0.f, 0.5f}, {0.f, 0.f}, {0.f, 1.f}};
  const int shapes[][4] = {{1, 1, 1, 8}, {1, 8, 8, 1}, {3, 5, 7, 5}, {2, 9, 4, 64}, {4, 6, 6, 24}};
  for (const auto& s : shapes)
    for (const auto& b : blends) {
      const Case k{s[0], s[1], s[2], s[3], b[0], b[1]};
      test_forward(handle, k, false, false);
      test_forward(handle, k, true, false);
      test_forward(handle, k, true, true);
      test_backward(handle, k, 1.f, 0.f);
      test_backward(handle, k, b[0], b[1]);
    }
  test_known_answer(handle, true);
  test_known_answer(handle, false);

  // descriptor checks: per-activation mode, a parameter descriptor that is not 1xCx1x1, mismatched output
  {
    TensorDescriptor x_desc, y_desc, bn_desc, bad_bn;
    x_desc.set4d(DataFormat::NHWC, 2, 8, 4, 4);
    y_desc.set4d(DataFormat::NHWC, 2, 8, 4, 5);
    bn_desc.set4d(DataFormat::NHWC, 1, 8, 1, 1);
    bad_bn.set4d(DataFormat::NHWC, 1, 8, 4, 4);
    const float one = 1.f, zero = 0.f;
    float* d = to_device(Vec(2 * 8 * 4 * 5, 1.f));
    auto run = [&](BatchNormMode mode, const TensorDescriptor& yd, const TensorDescriptor& bd) {
      return batchNormalizationForwardInference(handle, mode, &one, &zero, x_desc, d, yd, d, bd, d, d, d, d, 0.001)
          .status;
    };
    CHECK(run(BATCHNORM_PER_ACTIVATION, x_desc, bad_bn) == StatusCode::InvalidParameter, "per-activation accepted");
    CHECK(run(BATCHNORM_SPATIAL, x_desc, bad_bn) == StatusCode::InvalidParameter, "bad parameter descriptor accepted");
    CHECK(run(BATCHNORM_SPATIAL, y_desc, bn_desc) == StatusCode::InvalidParameter, "mismatched output accepted");
    CHECK(run(BATCHNORM_SPATIAL_PERSISTENT, x_desc, bn_desc) == StatusCode::OK, "valid call refused");
    float* null_f = nullptr;
    CHECK(batchNormalizationForwardTraining(handle, BATCHNORM_SPATIAL, &one, &zero, x_desc, d, x_desc, d, bn_desc, d, d,
                                            0.1, d, d, 0.001, d, null_f)
                  .status == StatusCode::InvalidParameter,
          "one cache pointer accepted");
    cudaFree(d);
  }
  if (g_failures == 0) std::printf("all checks passed\n");
  return g_failures == 0 ? 0 : 1;
}
