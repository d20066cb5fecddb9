// Shared pieces of the two inference samples (vgg16.cc, resnet50.cc): device memory that lives as
// long as the network, parameter structs built the way portDNN's samples build them
// (samples/networks/vgg/vgg.cc:66-76,118-126,174-184,198-201,234-239), and seeded weights.
//
// portDNN's samples read Keras weight files converted by a Python helper; there are none here, so
// every tensor is filled from a hash of (tensor seed, element index).  The hash is a closed form, so
// a checker can rebuild the same tensors without running a generator in sequence.
#ifndef PORTDNN_B200_SAMPLES_NETWORKS_SAMPLE_COMMON_H_
#define PORTDNN_B200_SAMPLES_NETWORKS_SAMPLE_COMMON_H_
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "portdnn/helpers/padding.h"
#include "tools/network.h"

namespace sample {

using Backend = sycldnn::backend::CUDABackend;
using DType = float;

// uniform in [-1, 1): murmur3's 32-bit finaliser of the element index mixed with the tensor's seed
inline float hashed_unit(uint32_t index, uint32_t seed) {
  uint32_t x = index * 2654435761u ^ seed * 0x9E3779B9u;
  x ^= x >> 16;
  x *= 0x85EBCA6Bu;
  x ^= x >> 13;
  x *= 0xC2B2AE35u;
  x ^= x >> 16;
  return float(x >> 8) * (2.0f / 16777216.0f) - 1.0f;
}

// value = offset + scale * hashed_unit
inline std::vector<float> hashed_tensor(size_t n, uint32_t seed, float scale, float offset = 0.f) {
  std::vector<float> v(n);
  for (size_t i = 0; i < n; ++i) v[i] = offset + scale * hashed_unit(uint32_t(i), seed);
  return v;
}

// Device allocations of one program run, freed together.
class Arena {
 public:
  ~Arena() {
    for (void* p : blocks_) cudaFree(p);
  }
  float* alloc(size_t n) {
    void* p = nullptr;
    if (cudaMalloc(&p, n * sizeof(float) + 256) != cudaSuccess) {
      std::fprintf(stderr, "cudaMalloc of %zu floats failed\n", n);
      std::exit(3);
    }
    blocks_.push_back(p);
    return static_cast<float*>(p);
  }
  float* upload(const std::vector<float>& h) {
    float* d = alloc(h.size());
    cudaMemcpy(d, h.data(), h.size() * sizeof(float), cudaMemcpyHostToDevice);
    return d;
  }

 private:
  std::vector<void*> blocks_;
};

inline sycldnn::conv2d::Conv2DParams make_conv_params(int batch, int input, int channels, int features, int window,
                                                      int stride, sycldnn::PaddingMode pad) {
  sycldnn::conv2d::Conv2DParams p{};
  p.channels = channels;
  p.features = features;
  p.batch = batch;
  p.in_rows = p.in_cols = input;
  p.window_rows = p.window_cols = window;
  p.stride_rows = p.stride_cols = stride;
  p.dilation_rows = p.dilation_cols = 1;
  p.groups = 1;
  return sycldnn::helpers::add_padding_to(p, pad);
}

inline sycldnn::pooling::PoolingParams make_pooling_params(int batch, int input, int channels, int window, int stride,
                                                          sycldnn::PaddingMode pad) {
  sycldnn::pooling::PoolingParams p{};
  p.in_rows = p.in_cols = input;
  p.window_rows = p.window_cols = window;
  p.stride_rows = p.stride_cols = stride;
  p.batch = batch;
  p.channels = channels;
  return sycldnn::helpers::add_padding_to(p, pad);
}

// Builder of a chain of layers: every add_* reads the current output and appends a layer that
// writes a fresh buffer.  Seeds count up in the order the tensors are created.
class Chain {
 public:
  using Net = sycldnn::Network<DType, Backend>;
  Chain(Net& net, Backend& backend, sycldnn::conv2d::Selector& selector, Arena& arena, float* input)
      : net_(net), backend_(backend), selector_(selector), arena_(arena), current_(input) {}

  float* output() const { return current_; }
  void set_output(float* p) { current_ = p; }
  uint32_t next_seed() { return seed_++; }
  // Weights are uniform with variance gain / fan_in: 2 keeps the activations of a plain ReLU stack
  // level, 1 suits a network whose blocks add their input back.
  void set_gain(float gain) { gain_ = gain; }

  // convolution without bias
  void conv(const sycldnn::conv2d::Conv2DParams& p) {
    const size_t fan_in = size_t(p.window_rows) * p.window_cols * p.channels;
    const float a = std::sqrt(3.0f * gain_ / float(fan_in));
    float* w = arena_.upload(hashed_tensor(fan_in * p.features, next_seed(), a));
    float* out = arena_.alloc(size_t(p.batch) * p.out_rows * p.out_cols * p.features);
    net_.add_layer(new sycldnn::ConvolutionLayer<DType, Backend>(p, current_, w, out, nullptr, 0, backend_, selector_));
    current_ = out;
  }
  // bias[C] over [rows, C]
  void bias(int rows, int channels) {
    float* b = arena_.upload(hashed_tensor(size_t(channels), next_seed(), 0.1f));
    float* out = arena_.alloc(size_t(rows) * channels);
    net_.add_layer(new sycldnn::BiasAddLayer<DType, Backend>({{rows, channels}, {channels}}, current_, b, out, backend_));
    current_ = out;
  }
  // element-wise sum with another tensor of the same shape (the residual connection)
  void add(float* other, int count) {
    float* out = arena_.alloc(size_t(count));
    net_.add_layer(new sycldnn::BiasAddLayer<DType, Backend>({{count}, {count}}, current_, other, out, backend_));
    current_ = out;
  }
  void relu(int count) {
    float* out = arena_.alloc(size_t(count));
    net_.add_layer(new sycldnn::ActivationLayer<DType, Backend, sycldnn::pointwise::Relu>({count}, current_, out, backend_));
    current_ = out;
  }
  // frozen batchnorm: gamma in [0.5, 1.5), beta and mean in [-0.1, 0.1), variance in [0.5, 1.5)
  void batchnorm(int batch, int spatial, int channels, float epsilon) {
    float* beta = arena_.upload(hashed_tensor(size_t(channels), next_seed(), 0.1f));
    float* gamma = arena_.upload(hashed_tensor(size_t(channels), next_seed(), 0.5f, 1.0f));
    float* mean = arena_.upload(hashed_tensor(size_t(channels), next_seed(), 0.1f));
    float* var = arena_.upload(hashed_tensor(size_t(channels), next_seed(), 0.5f, 1.0f));
    float* out = arena_.alloc(size_t(batch) * spatial * spatial * channels);
    sycldnn::batchnorm::BatchNormParams p{batch, spatial, spatial, channels, false, epsilon, 0.9f};
    net_.add_layer(new sycldnn::BatchNormFrozenLayer<DType, Backend>(p, current_, beta, gamma, mean, var, out, backend_));
    current_ = out;
  }
  template <template <typename> class PoolingType>
  void pool(const sycldnn::pooling::PoolingParams& p) {
    float* out = arena_.alloc(size_t(p.batch) * p.out_rows * p.out_cols * p.channels);
    net_.add_layer(new sycldnn::PoolingLayer<DType, Backend, PoolingType>(p, current_, out, backend_));
    current_ = out;
  }
  // fully connected [batch, in] x [in, out]
  void fc(int batch, int in, int out_features) {
    const float a = std::sqrt(3.0f * gain_ / float(in));
    float* w = arena_.upload(hashed_tensor(size_t(in) * out_features, next_seed(), a));
    float* out = arena_.alloc(size_t(batch) * out_features);
    sycldnn::matmul::MatmulParams mp{1, batch, in, out_features, 0.f};
    net_.add_layer(new sycldnn::FCLayer<DType, Backend>(mp, current_, w, out, backend_));
    current_ = out;
  }
  void softmax(int batch, int classes) {
    float* ws = arena_.alloc(size_t(batch));
    float* out = arena_.alloc(size_t(batch) * classes);
    sycldnn::softmax::SoftmaxParams sp{classes, batch, 1, 1};
    net_.add_layer(new sycldnn::SoftmaxLayer<DType, Backend>(sp, current_, ws, out, backend_));
    current_ = out;
  }

 private:
  Net& net_;
  Backend& backend_;
  sycldnn::conv2d::Selector& selector_;
  Arena& arena_;
  float* current_;
  uint32_t seed_ = 1;
  float gain_ = 2.0f;
};

struct Options {
  int batch = 1;
  int iterations = 8;
  std::string dump;  // file that receives the class probabilities as raw floats
};

inline Options parse_options(int argc, char** argv) {
  Options o;
  for (int i = 1; i < argc; ++i) {
    const std::string a = argv[i];
    if (a == "--batch" && i + 1 < argc) {
      o.batch = std::atoi(argv[++i]);
    } else if (a == "--iterations" && i + 1 < argc) {
      o.iterations = std::atoi(argv[++i]);
    } else if (a == "--dump" && i + 1 < argc) {
      o.dump = argv[++i];
    } else {
      std::fprintf(stderr, "usage: %s [--batch N] [--iterations N] [--dump FILE]\n", argv[0]);
      std::exit(2);
    }
  }
  if (o.batch < 1 || o.iterations < 1) {
    std::fprintf(stderr, "batch and iterations must be positive\n");
    std::exit(2);
  }
  return o;
}

// Runs the network once with a wait after every layer (Network::test), prints the class of every
// image, then times whole runs the way portDNN's samples do (vgg.cc:486-507): nanoseconds from
// queueing the first layer to the completion of the last, data transfers not included.
inline int classify_and_time(sycldnn::Network<DType, Backend>& net, std::vector<DType>& output, const Options& opt,
                             int classes) {
  sycldnn::SNNStatus st = net.test();
  if (st.status != sycldnn::StatusCode::OK) {
    std::fprintf(stderr, "network failed: status %d (%s)\n", int(st.status), pdnn_last_error());
    return 1;
  }
  for (int n = 0; n < opt.batch; ++n) {
    int best = 0;
    double total = 0;
    for (int c = 0; c < classes; ++c) {
      total += output[size_t(n) * classes + c];
      if (output[size_t(n) * classes + c] > output[size_t(n) * classes + best]) best = c;
    }
    std::printf("image %d: classed as %d (probability %.6f, probabilities sum to %.6f)\n", n, best,
                output[size_t(n) * classes + best], total);
  }
  if (!opt.dump.empty()) {
    FILE* f = std::fopen(opt.dump.c_str(), "wb");
    if (f == nullptr || std::fwrite(output.data(), sizeof(DType), output.size(), f) != output.size()) {
      std::fprintf(stderr, "cannot write %s\n", opt.dump.c_str());
      return 1;
    }
    std::fclose(f);
  }
  for (int i = 0; i < opt.iterations; ++i) {
    const auto start = std::chrono::high_resolution_clock::now();
    st = net.run();
    if (st.status != sycldnn::StatusCode::OK) {
      std::fprintf(stderr, "run %d failed: status %d (%s)\n", i, int(st.status), pdnn_last_error());
      return 1;
    }
    st.event.wait_and_throw();
    const auto stop = std::chrono::high_resolution_clock::now();
    std::printf("%lld ns\n", (long long)std::chrono::duration_cast<std::chrono::nanoseconds>(stop - start).count());
  }
  return 0;
}

}  // namespace sample
#endif
