#include "context.h"

#include <mutex>

namespace caffe {

int DeviceCount() {
  static int count = -1;
  static std::once_flag once;
  std::call_once(once, [] {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {
      cudaGetLastError();  // clear the sticky "no device" state
      n = 0;
    }
    count = n;
  });
  return count;
}

Context& Context::Get() {
  static thread_local Context ctx;
  return ctx;
}

void Context::Release() {
  if (!active_) return;
  // At process exit the runtime may already be gone; ignore errors here.
  if (cudaSetDevice(device_) == cudaSuccess) {
    if (stream_) cudaStreamDestroy(stream_);
    if (status_dev_) cudaFree(status_dev_);
    if (status_host_) cudaFreeHost(status_host_);
  }
  cudaGetLastError();
  stream_ = nullptr;
  status_dev_ = nullptr;
  status_host_ = nullptr;
  active_ = false;
}

Context::~Context() { Release(); }

void Context::Set(DeviceMode mode, int device) {
  if (mode == GPU) {
    CHECK_GE(device, 0) << "GPU mode needs a device id >= 0";
    CHECK_GT(DeviceCount(), 0) << "SetMode(GPU): no CUDA device is available";
    CHECK_LT(device, DeviceCount()) << "SetMode(GPU): invalid device id";
  }
  if (active_ && (mode != mode_ || device != device_)) {
    Sync();
    Release();
  }
  mode_ = mode;
  device_ = mode == GPU ? device : -1;
}

void Context::Activate() {
  if (active_) return;
  CHECK(mode_ == GPU) << "this engine has no CPU compute path: call SetMode(GPU, device) before Forward";
  CHECK_GT(DeviceCount(), 0) << "no CUDA device is available; this engine cannot run without one";
  CHECK_LT(device_, DeviceCount()) << "invalid device id";
  CUDA_CHECK(cudaSetDevice(device_));
  CUDA_CHECK(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
  CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&status_dev_), sizeof(int)));
  CUDA_CHECK(cudaMemset(status_dev_, 0, sizeof(int)));
  CUDA_CHECK(cudaMallocHost(reinterpret_cast<void**>(&status_host_), sizeof(int)));
  *status_host_ = 0;
  active_ = true;
}

void Context::Sync() {
  if (!active_) return;
  CUDA_CHECK(cudaStreamSynchronize(stream_));
}

void Context::SyncAndCheck() {
  if (!active_) return;
  CUDA_CHECK(cudaMemcpyAsync(status_host_, status_dev_, sizeof(int), cudaMemcpyDeviceToHost, stream_));
  CUDA_CHECK(cudaStreamSynchronize(stream_));
  if (*status_host_ != 0) {
    const int code = *status_host_;
    *status_host_ = 0;
    CUDA_CHECK(cudaMemsetAsync(status_dev_, 0, sizeof(int), stream_));
    // 3: a region-of-interest layer met a roi whose image index is outside the batch
    // (the reference fails its CHECK_GE / CHECK_LT on roi_batch_ind at that point).
    if (code == 3) LOG(FATAL) << "Check failed: roi_batch_ind is outside [0, batch_size)";
    LOG(FATAL) << "a kernel gave up waiting on a hardware barrier (status " << code
               << "); the results of this forward pass are invalid";
  }
}

bool GPUAvailable() { return DeviceCount() > 0; }

void SetMode(DeviceMode mode, int device) { Context::Get().Set(mode, device); }

}  // namespace caffe
