// A network as a list of layers run in order, with the interface of portDNN's tools/network.h:26-79
// (add_layer / run / test / get_output / get_network_size / get_output_size).  `test` waits after
// every layer so that a failure is reported by the layer that caused it, then copies the last
// layer's result into the host vector the network was built with.
#ifndef PORTDNN_B200_TOOLS_NETWORK_H_
#define PORTDNN_B200_TOOLS_NETWORK_H_
#include <memory>
#include <stdexcept>
#include <vector>

#include "tools/layer.h"

namespace sycldnn {

template <typename DType, typename Backend>
class Network {
  using DeviceMem = typename Backend::template pointer_type<DType>;
  std::vector<std::unique_ptr<Layer<DType, Backend>>> layers_;
  std::vector<DType>& host_result_;
  Backend& backend_;

 public:
  Network(Backend& backend, std::vector<DType>& output) : layers_{}, host_result_{output}, backend_{backend} {}

  /** Takes ownership of the layer object (not of the device memory it points to). */
  void add_layer(Layer<DType, Backend>* layer) { layers_.emplace_back(layer); }

  /** Queues every layer on the backend's stream; the returned event completes with the last one. */
  SNNStatus run() {
    SNNStatus status{Event{backend_.get_queue()}, StatusCode::OK};
    for (auto& layer : layers_) {
      status = layer->run();
      if (status.status != StatusCode::OK) return status;
    }
    return status;
  }

  /** Runs layer by layer, waiting (and throwing on a failed layer) after each, then reads the result back. */
  SNNStatus test() {
    for (auto& layer : layers_) {
      SNNStatus status = layer->run();
      if (status.status != StatusCode::OK) return status;
      status.event.wait_and_throw();
    }
    return dump_network_output();
  }

  DeviceMem get_output() { return layers_.back()->get_output(); }
  DeviceMem get_output(int layer_number) { return layers_[size_t(layer_number)]->get_output(); }
  size_t get_network_size() const { return layers_.size(); }
  size_t get_output_size() const { return layers_.back()->get_output_size(); }

  /** Copies the last layer's output into the host vector given to the constructor. */
  SNNStatus dump_network_output() {
    if (layers_.empty()) return StatusCode::InvalidParameter;
    const size_t count = get_output_size();
    host_result_.resize(count);
    cudaStream_t stream = backend_.get_queue();
    if (cudaMemcpyAsync(host_result_.data(), get_output(), count * sizeof(DType), cudaMemcpyDeviceToHost, stream) !=
        cudaSuccess)
      return StatusCode::AllocationProblem;
    Event done{stream};
    done.wait_and_throw();
    return SNNStatus{done, StatusCode::OK};
  }
};

}  // namespace sycldnn
#endif
