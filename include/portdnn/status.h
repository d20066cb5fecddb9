// Status codes and the launch result, after portDNN's include/portdnn/status.h:31-89.  The SYCL
// event of the reference becomes a handle on the CUDA stream the work was queued on: work on one
// stream runs in order, so waiting for the stream waits for the launch.
#ifndef PORTDNN_B200_STATUS_H_
#define PORTDNN_B200_STATUS_H_
#include <cuda_runtime_api.h>

#include <memory>
#include <stdexcept>

namespace sycldnn {
enum class StatusCode { OK, InvalidAlgorithm, IndexExceeded, InsufficientWorkspace, AllocationProblem, InvalidParameter };

/** Completion handle of a launch: a CUDA event recorded on the launch's stream right after the
 * launch was queued (the reference returns the sycl::event of its last kernel,
 * include/portdnn/status.h:75-89).  Copies share the event; it is destroyed with the last copy. */
class Event {
 public:
  Event() = default;
  explicit Event(cudaStream_t stream) : stream_(stream), valid_(true) {
    cudaEvent_t ev = nullptr;
    if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) == cudaSuccess) {
      cudaEventRecord(ev, stream);
      event_ = std::shared_ptr<CUevent_st>(ev, [](cudaEvent_t e) { cudaEventDestroy(e); });
    } else {
      cudaGetLastError();  // fall back to waiting for the whole stream
    }
  }
  void wait() const {
    if (!valid_) return;
    if (event_) cudaEventSynchronize(event_.get());
    else cudaStreamSynchronize(stream_);
  }
  void wait_and_throw() const {
    if (!valid_) return;
    const cudaError_t e = event_ ? cudaEventSynchronize(event_.get()) : cudaStreamSynchronize(stream_);
    if (e != cudaSuccess) throw std::runtime_error(cudaGetErrorString(cudaGetLastError()));
  }
  /** True once the work the event covers has finished (sycl's command_execution_status::complete). */
  bool complete() const { return !valid_ || (event_ ? cudaEventQuery(event_.get()) == cudaSuccess : cudaStreamQuery(stream_) == cudaSuccess); }
  cudaStream_t stream() const { return stream_; }
  cudaEvent_t native() const { return event_.get(); }
  bool valid() const { return valid_; }
  /** Makes `other` wait for the launch this event came from (the USM launchers do this for every
   * event in their `events` argument before they queue their own work). */
  void make_stream_wait(cudaStream_t other) const {
    if (!valid_ || other == stream_) return;
    if (event_) {
      cudaStreamWaitEvent(other, event_.get(), 0);
      return;
    }
    cudaEvent_t ev;
    cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
    cudaEventRecord(ev, stream_);
    cudaStreamWaitEvent(other, ev, 0);
    cudaEventDestroy(ev);
  }

 private:
  cudaStream_t stream_ = nullptr;
  bool valid_ = false;
  std::shared_ptr<CUevent_st> event_;
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
