// VGG-16 inference on the layer wrappers (include/tools/layer.h, network.h), layer for layer the network
// of portDNN's samples/networks/vgg/vgg.cc:286-484: thirteen 3x3 SAME convolutions with bias and ReLU in
// five stages (64, 128, 256, 512, 512 features), a 2x2/2 VALID max pool after each stage, three fully
// connected layers (4096, 4096, 1000) and softmax, on a 224 x 224 x 3 NHWC image.  Weights and image are
// seeded (sample_common.h).  Prints the class of every image and the time of each timed run.
//
// Build: g++ -std=c++17 -O2 -Iinclude -Isamples/networks -I$CUDA/include samples/networks/vgg16.cc
//        -Lportdnn_b200 -lportdnn_b200 -L$CUDA/lib64 -lcudart -o vgg16
#include "sample_common.h"

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

  const int stage_layers[5] = {2, 2, 3, 3, 3}, stage_features[5] = {64, 128, 256, 512, 512};
  int size = 224, channels = 3;
  for (int stage = 0; stage < 5; ++stage) {
    for (int i = 0; i < stage_layers[stage]; ++i) {
      const int features = stage_features[stage];
      chain.conv(make_conv_params(N, size, channels, features, 3, 1, sycldnn::PaddingMode::SAME));
      chain.bias(N * size * size, features);
      chain.relu(N * size * size * features);
      channels = features;
    }
    chain.pool<sycldnn::pooling::Max>(make_pooling_params(N, size, channels, 2, 2, sycldnn::PaddingMode::VALID));
    size /= 2;
  }
  int width = size * size * channels;  // 7 * 7 * 512, flattened in NHWC order
  const int fc_features[3] = {4096, 4096, kClasses};
  for (int i = 0; i < 3; ++i) {
    chain.fc(N, width, fc_features[i]);
    chain.bias(N, fc_features[i]);
    if (i < 2) chain.relu(N * fc_features[i]);
    width = fc_features[i];
  }
  chain.softmax(N, kClasses);
  std::printf("VGG-16: %zu layers, batch %d\n", size_t(net.get_network_size()), N);
  return classify_and_time(net, output, opt, kClasses);
}
