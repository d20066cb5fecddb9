// Status codes and the launch result, after portDNN's include/portdnn/status.h:31-89.  The SYCL
// event of the reference becomes a handle on the CUDA stream the work was queued on: work on one
// stream runs in order, so waiting for the stream waits for the launch.
#ifndef PORTDNN_B200_STATUS_H_
#define PORTDNN_B200_STATUS_H_
#include <cuda_runtime_api.h>

#include <stdexcept>

namespace sycldnn {
enum class StatusCode { OK, InvalidAlgorithm, IndexExceeded, InsufficientWorkspace, AllocationProblem, InvalidParameter };

/** Completion handle of a launch.  native() records a CUDA event on demand (it then covers at
 * least the launch it came from, possibly later work on the same stream too). */
class Event {
 public:
  Event() = default;
  explicit Event(cudaStream_t stream) : stream_(stream), valid_(true) {}
  void wait() const {
    if (valid_) cudaStreamSynchronize(stream_);
  }
  void wait_and_throw() const {
    if (valid_ && cudaStreamSynchronize(stream_) != cudaSuccess)
      throw std::runtime_error(cudaGetErrorString(cudaGetLastError()));
  }
  cudaStream_t stream() const { return stream_; }
  bool valid() const { return valid_; }
  /** Makes `other` wait for everything queued so far on this event's stream. */
  void make_stream_wait(cudaStream_t other) const {
    if (!valid_ || other == stream_) return;
    cudaEvent_t ev;
    cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
    cudaEventRecord(ev, stream_);
    cudaStreamWaitEvent(other, ev, 0);
    cudaEventDestroy(ev);
  }

 private:
  cudaStream_t stream_ = nullptr;
  bool valid_ = false;
};

struct SNNStatus {
  SNNStatus(Event e, StatusCode s) : event(e), status(s) {}
  SNNStatus(StatusCode s) : SNNStatus(Event{}, s) {}  // NOLINT: implicit, as in the reference
  SNNStatus() : SNNStatus(StatusCode::OK) {}
  Event event;
  StatusCode status;
};
}  // namespace sycldnn
#endif
