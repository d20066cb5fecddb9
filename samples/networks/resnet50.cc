// ResNet-50 inference on the layer wrappers (include/tools/layer.h, network.h), the network of portDNN's
// samples/networks/resnet50/resnet50.cc:392-1520 (the Keras model: stride 2 on the first 1x1 of a stage):
// 7x7/2 SAME stem, 3x3/2 SAME max pool, bottleneck stages of [3, 4, 6, 3] blocks with widths 64 / 128 /
// 256 / 512 and four times as many output features, every convolution followed by bias and frozen
// batchnorm (epsilon 1.001e-5), a 1x1 projection on the shortcut of each stage's first block (VALID,
// stride 2 from the second stage on), the shortcut added before the block's last ReLU, global 7x7
// average pool, one fully connected layer and softmax.  Weights and image are seeded (sample_common.h).
//
// Build: g++ -std=c++17 -O2 -Iinclude -Isamples/networks -I$CUDA/include samples/networks/resnet50.cc
//        -Lportdnn_b200 -lportdnn_b200 -L$CUDA/lib64 -lcudart -o resnet50
#include "sample_common.h"

namespace {
constexpr float kEpsilon = 1.001e-5f;

// convolution - bias - batchnorm (- ReLU)
void conv_unit(sample::Chain& chain, int batch, int input, int channels, int features, int window, int stride,
               sycldnn::PaddingMode pad, bool relu) {
  const auto p = sample::make_conv_params(batch, input, channels, features, window, stride, pad);
  chain.conv(p);
  chain.bias(batch * p.out_rows * p.out_cols, features);
  chain.batchnorm(batch, p.out_rows, features, kEpsilon);
  if (relu) chain.relu(batch * p.out_rows * p.out_cols * features);
}
}  // namespace

int main(int argc, char** argv) {
  using namespace sample;
  const Options opt = parse_options(argc, argv);
  int devices = 0;
  if (cudaGetDeviceCount(&devices) != cudaSuccess || devices == 0) {
    std::fprintf(stderr, "no CUDA device\n");
    return 2;
  }
  cudaStream_t stream;
  cudaStreamCreate(&stream);
  Backend backend(stream);
  auto selector = sycldnn::conv2d::get_default_selector();
  Arena arena;
  std::vector<DType> output;
  sycldnn::Network<DType, Backend> net(backend, output);

  const int N = opt.batch, kClasses = 1000;
  float* image = arena.upload(hashed_tensor(size_t(N) * 224 * 224 * 3, 0u, 1.0f));
  Chain chain(net, backend, *selector, arena, image);
  chain.set_gain(1.0f);

  conv_unit(chain, N, 224, 3, 64, 7, 2, sycldnn::PaddingMode::SAME, true);
  chain.pool<sycldnn::pooling::Max>(make_pooling_params(N, 112, 64, 3, 2, sycldnn::PaddingMode::SAME));

  const int blocks[4] = {3, 4, 6, 3}, widths[4] = {64, 128, 256, 512};
  int size = 56, channels = 64;
  for (int stage = 0; stage < 4; ++stage) {
    const int mid = widths[stage], out = 4 * mid;
    for (int block = 0; block < blocks[stage]; ++block) {
      const int stride = (block == 0 && stage > 0) ? 2 : 1;
      float* block_input = chain.output();
      float* shortcut = block_input;
      if (block == 0) {  // projection shortcut
        conv_unit(chain, N, size, channels, out, 1, stride, sycldnn::PaddingMode::VALID, false);
        shortcut = chain.output();
        chain.set_output(block_input);
      }
      conv_unit(chain, N, size, channels, mid, 1, stride, sycldnn::PaddingMode::SAME, true);
      const int out_size = (size + stride - 1) / stride;
      conv_unit(chain, N, out_size, mid, mid, 3, 1, sycldnn::PaddingMode::SAME, true);
      conv_unit(chain, N, out_size, mid, out, 1, 1, sycldnn::PaddingMode::SAME, false);
      chain.add(shortcut, N * out_size * out_size * out);
      chain.relu(N * out_size * out_size * out);
      size = out_size;
      channels = out;
    }
  }
  chain.pool<sycldnn::pooling::Average>(make_pooling_params(N, size, channels, size, 1, sycldnn::PaddingMode::VALID));
  chain.fc(N, channels, kClasses);
  chain.bias(N, kClasses);
  chain.softmax(N, kClasses);
  std::printf("ResNet-50: %zu layers, batch %d\n", size_t(net.get_network_size()), N);
  return classify_and_time(net, output, opt, kClasses);
}
