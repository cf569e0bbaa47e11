// Per-thread device context of the engine: mode, device ordinal, the stream
// all of this thread's kernels and copies run on, and the status word that
// kernels with bounded waits report into.
//
// mini-caffe keeps mode and cuBLAS handle in a thread-local `Caffe` singleton
// (src/common.hpp:76-117, src/common.cpp:7-10); this is the counterpart.  A
// thread that never calls SetMode runs on GPU 0.
#ifndef MCB200_CONTEXT_H_
#define MCB200_CONTEXT_H_

#include <cuda_runtime.h>

#include "caffe/base.hpp"

#define CUDA_CHECK(expr)                                                            \
  do {                                                                              \
    cudaError_t cuda_check_err_ = (expr);                                           \
    CHECK_EQ(static_cast<int>(cuda_check_err_), static_cast<int>(cudaSuccess))      \
        << " " << cudaGetErrorString(cuda_check_err_);                              \
  } while (0)

// Kernel-level entry points return 0, a negative argument error, or a cudaError_t.
#define KERNEL_CHECK(expr)                                                          \
  do {                                                                              \
    int kernel_check_rc_ = (expr);                                                  \
    CHECK_EQ(kernel_check_rc_, 0) << " kernel launcher failed: " #expr              \
        << (kernel_check_rc_ > 0 ? cudaGetErrorString(static_cast<cudaError_t>(kernel_check_rc_)) : ""); \
  } while (0)

namespace caffe {

class Context {
 public:
  static Context& Get();  // of the calling thread

  DeviceMode mode() const { return mode_; }
  int device() const { return device_; }
  void Set(DeviceMode mode, int device);

  // Binds the thread to its device and creates the stream on first use.
  // Throws caffe::Error in CPU mode or without a usable device.
  void Activate();
  cudaStream_t stream() { Activate(); return stream_; }
  void* stream_ptr() { return static_cast<void*>(stream()); }
  // The stream if this thread has one already, else NULL (never creates one, never throws).
  void* stream_if_active() const { return active_ ? static_cast<void*>(stream_) : nullptr; }
  // Device int that kernels raise on a timed-out wait; checked by Net::Forward.
  int* status_word() { Activate(); return status_dev_; }
  // Blocks until the stream is idle and throws if a kernel raised the status word.
  void SyncAndCheck();
  void Sync();

  ~Context();

 private:
  Context() : mode_(GPU), device_(0), active_(false), stream_(nullptr), status_dev_(nullptr), status_host_(nullptr) {}
  DeviceMode mode_;
  int device_;
  bool active_;
  cudaStream_t stream_;
  int* status_dev_;
  int* status_host_;
  void Release();
};

// Number of usable CUDA devices (0 without a driver); cached.
int DeviceCount();

}  // namespace caffe

#endif  // MCB200_CONTEXT_H_
