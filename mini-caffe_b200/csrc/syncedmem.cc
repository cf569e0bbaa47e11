#include "syncedmem.h"

#include <cstdlib>
#include <cstring>
#include <set>

#include "context.h"
#include "mcb200_kernels.h"

namespace caffe {

// ---------------------------------------------------------------- MemoryPool

// Pools that exist right now.  A block returned by a thread that does not own
// it finds out here whether its pool is still there; the lock is held while the
// block is handed over, so a pool cannot disappear in the middle of that.
static std::mutex& LivePoolsLock() {
  static std::mutex* mu = new std::mutex();   // outlives every thread-local pool
  return *mu;
}
static std::set<MemoryPool*>& LivePools() {
  static std::set<MemoryPool*>* pools = new std::set<MemoryPool*>();
  return *pools;
}

MemoryPool* MemoryPool::Get() {
  static thread_local MemoryPool pool;
  return &pool;
}

MemoryPool::MemoryPool() {
  std::lock_guard<std::mutex> lock(LivePoolsLock());
  LivePools().insert(this);
}

MemoryPool::~MemoryPool() {
  {
    std::lock_guard<std::mutex> lock(LivePoolsLock());
    LivePools().erase(this);
  }
  Clear();
}

static bool Reusable(size_t has, size_t wants) { return has / 2 <= wants; }

MemBlock MemoryPool::RequestCPU(size_t size) {
  std::lock_guard<std::mutex> lock(mu_);
  auto it = cpu_free_.lower_bound(size);
  if (it != cpu_free_.end() && Reusable(it->second.size, size)) {
    MemBlock b = it->second;
    cpu_free_.erase(it);
    cpu_unused_ -= static_cast<long long>(b.size);
    return b;
  }
  MemBlock b;
  b.size = size;
  b.device = -1;
  b.pool = this;
  if (DeviceCount() > 0) {
    // Pinned, so that host<->device copies can run asynchronously on the stream.
    CUDA_CHECK(cudaMallocHost(&b.ptr, size));
  } else {
    CHECK_EQ(posix_memalign(&b.ptr, 64, size), 0) << "out of host memory";
  }
  cpu_total_ += static_cast<long long>(size);
  return b;
}

void MemoryPool::ReturnCPU(MemBlock block) {
  if (!block.ptr) return;
  std::lock_guard<std::mutex> lock(mu_);
  cpu_unused_ += static_cast<long long>(block.size);
  cpu_free_.insert(std::make_pair(block.size, block));
}

MemBlock MemoryPool::RequestGPU(size_t size, int device) {
  void* stream = Context::Get().stream_ptr();   // the requesting thread's work will use the block
  std::lock_guard<std::mutex> lock(mu_);
  auto it = gpu_free_.lower_bound(std::make_pair(device, size));
  if (it != gpu_free_.end() && it->second.device == device && Reusable(it->second.size, size)) {
    MemBlock b = it->second;
    gpu_free_.erase(it);
    gpu_unused_ -= static_cast<long long>(b.size);
    b.stream = stream;
    return b;
  }
  MemBlock b;
  b.size = size;
  b.device = device;
  b.pool = this;
  b.stream = stream;
  int current = 0;
  CUDA_CHECK(cudaGetDevice(&current));
  if (current != device) CUDA_CHECK(cudaSetDevice(device));
  CUDA_CHECK(cudaMalloc(&b.ptr, size));
  if (current != device) CUDA_CHECK(cudaSetDevice(current));
  gpu_total_ += static_cast<long long>(size);
  return b;
}

void MemoryPool::ReturnGPU(MemBlock block) {
  if (!block.ptr) return;
  std::lock_guard<std::mutex> lock(mu_);
  gpu_unused_ += static_cast<long long>(block.size);
  gpu_free_.insert(std::make_pair(std::make_pair(block.device, block.size), block));
}

void MemoryPool::Release(MemBlock block) {
  if (!block.ptr) return;
  MemoryPool* mine = MemoryPool::Get();
  const bool gpu = block.device >= 0;
  if (block.pool == mine || block.pool == nullptr) {
    if (gpu) {
      mine->ReturnGPU(block);
    } else {
      mine->ReturnCPU(block);
    }
    return;
  }
  // Another thread allocated this block.  Work that uses it may be queued on
  // that thread's stream and on this thread's; the owner's pool will hand it to
  // work on the owner's stream only, so both are drained before it goes back.
  const bool have_device = DeviceCount() > 0;
  if (have_device) {
    try { Context::Get().Sync(); } catch (...) {}
    if (block.stream) cudaStreamSynchronize(static_cast<cudaStream_t>(block.stream));
    cudaGetLastError();   // the owner's stream may be gone already
  }
  std::lock_guard<std::mutex> lock(LivePoolsLock());
  if (LivePools().count(block.pool)) {
    if (gpu) {
      block.pool->ReturnGPU(block);
    } else {
      block.pool->ReturnCPU(block);
    }
    return;
  }
  // The owning thread has ended and taken its pool with it.
  if (gpu) {
    int current = 0;
    if (cudaGetDevice(&current) == cudaSuccess) {
      if (current != block.device) cudaSetDevice(block.device);
      cudaDeviceSynchronize();
      cudaFree(block.ptr);
      if (current != block.device) cudaSetDevice(current);
    }
    cudaGetLastError();
  } else if (have_device) {
    cudaFreeHost(block.ptr);
    cudaGetLastError();
  } else {
    free(block.ptr);
  }
}

void MemoryPool::Clear() {
  const bool have_device = DeviceCount() > 0;
  std::lock_guard<std::mutex> lock(mu_);
  for (auto& kv : cpu_free_) {
    if (have_device) {
      cudaFreeHost(kv.second.ptr);
    } else {
      free(kv.second.ptr);
    }
    cpu_total_ -= static_cast<long long>(kv.second.size);
  }
  cpu_free_.clear();
  cpu_unused_ = 0;
  if (have_device && !gpu_free_.empty()) {
    int current = 0;
    if (cudaGetDevice(&current) == cudaSuccess) {
      // Blocks may still be read by kernels queued on this thread's stream.
      Context::Get().Sync();
      for (auto& kv : gpu_free_) {
        if (kv.second.device != current) cudaSetDevice(kv.second.device);
        cudaFree(kv.second.ptr);
        if (kv.second.device != current) cudaSetDevice(current);
        gpu_total_ -= static_cast<long long>(kv.second.size);
      }
    }
    cudaGetLastError();
  }
  gpu_free_.clear();
  gpu_unused_ = 0;
}

static int Saturate(long long v) { return v > 0x7fffffffLL ? 0x7fffffff : static_cast<int>(v); }

MemPoolState MemoryPool::GetState() const {
  std::lock_guard<std::mutex> lock(mu_);
  MemPoolState st;
  st.cpu_mem = Saturate(cpu_total_);
  st.gpu_mem = Saturate(gpu_total_);
  st.unused_cpu_mem = Saturate(cpu_unused_);
  st.unused_gpu_mem = Saturate(gpu_unused_);
  return st;
}

void MemPoolClear() { MemoryPool::Get()->Clear(); }
MemPoolState MemPoolGetState() { return MemoryPool::Get()->GetState(); }

// ---------------------------------------------------------------- SyncedMemory

SyncedMemory::SyncedMemory(size_t size)
    : size_(size), valid_(0), nhwc_aliases_dev_(false), host_version_(1) {
  dims_[0] = dims_[1] = dims_[2] = dims_[3] = 0;
}

SyncedMemory::~SyncedMemory() {
  // Kernels queued on the stream may still use the device blocks; the pool
  // hands them out again only to work queued on the same stream, which is
  // ordered after those kernels.
  // ordered after those kernels.  (MemoryPool::Release covers the case that
  // another thread than the allocating one runs this destructor.)
  if (host_.ptr) {
    // A pinned block may be the target of a copy that is still in flight.
    if (valid_ & (kDevice | kDeviceNhwc | kDeviceNhwcHalf)) {
      try { Context::Get().Sync(); } catch (...) {}
      void* stream = dev_.ptr ? dev_.stream : (nhwc_.ptr ? nhwc_.stream : half_.stream);
      if (stream && stream != Context::Get().stream_if_active()) {
        cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
        cudaGetLastError();
      }
    }
    MemoryPool::Release(host_);
  }
  MemoryPool::Release(dev_);
  MemoryPool::Release(nhwc_);
  MemoryPool::Release(half_);
}

void SyncedMemory::EnsureHost() {
  if (!host_.ptr) {
    host_ = MemoryPool::Get()->RequestCPU(size_ ? size_ : 4);
    if (!(valid_ & (kDevice | kDeviceNhwc | kDeviceNhwcHalf))) {
      std::memset(host_.ptr, 0, size_);  // same as the reference: fresh memory reads as zero
      valid_ |= kHost;
    }
  }
}

void SyncedMemory::EnsureDevice() {
  if (!dev_.ptr) {
    Context& ctx = Context::Get();
    ctx.Activate();
    dev_ = MemoryPool::Get()->RequestGPU(size_ ? size_ : 4, ctx.device());
    if (valid_ == 0) {
      CUDA_CHECK(cudaMemsetAsync(dev_.ptr, 0, size_, ctx.stream()));
      valid_ |= kDevice;
    }
  }
}

void SyncedMemory::EnsureNhwcBuffer() {
  if (!nhwc_.ptr) {
    Context& ctx = Context::Get();
    ctx.Activate();
    nhwc_ = MemoryPool::Get()->RequestGPU(size_ ? size_ : 4, ctx.device());
  }
}

void SyncedMemory::EnsureHalfBuffer() {
  if (!half_.ptr) {
    Context& ctx = Context::Get();
    ctx.Activate();
    half_ = MemoryPool::Get()->RequestGPU(size_ / 2 ? size_ / 2 : 4, ctx.device());
  }
}

void SyncedMemory::WidenHalf() {
  if (!(valid_ & kDeviceNhwcHalf) || (valid_ & (kHost | kDevice | kDeviceNhwc))) return;
  Context& ctx = Context::Get();
  const size_t count = static_cast<size_t>(dims_[0]) * dims_[1] * dims_[2] * dims_[3];
  if (OrdersCoincide(dims_[1], dims_[2], dims_[3])) {
    EnsureDevice();
    KERNEL_CHECK(mcb200_bf16_to_f32(static_cast<const uint16_t*>(half_.ptr), static_cast<float*>(dev_.ptr), count,
                                    ctx.stream_ptr()));
    valid_ |= kDevice;
  } else {
    EnsureNhwcBuffer();
    KERNEL_CHECK(mcb200_bf16_to_f32(static_cast<const uint16_t*>(half_.ptr), static_cast<float*>(nhwc_.ptr), count,
                                    ctx.stream_ptr()));
    nhwc_aliases_dev_ = false;
    valid_ |= kDeviceNhwc;
  }
}

void SyncedMemory::DeviceFromFreshest() {
  if (valid_ & kDevice) return;
  WidenHalf();
  if (valid_ & kDevice) return;
  EnsureDevice();
  if (valid_ & kDevice) return;  // freshly zero-filled
  Context& ctx = Context::Get();
  if (valid_ & kDeviceNhwc) {
    CHECK(!nhwc_aliases_dev_);
    KERNEL_CHECK(mcb200_nhwc_to_nchw(static_cast<const float*>(nhwc_.ptr), static_cast<float*>(dev_.ptr), dims_[0],
                                     dims_[1], dims_[2], dims_[3], dims_[1], ctx.stream_ptr()));
  } else {
    CHECK(valid_ & kHost);
    CUDA_CHECK(cudaMemcpyAsync(dev_.ptr, host_.ptr, size_, cudaMemcpyHostToDevice, ctx.stream()));
  }
  valid_ |= kDevice;
}

const void* SyncedMemory::cpu_data() {
  EnsureHost();
  if (!(valid_ & kHost)) {
    DeviceFromFreshest();
    Context& ctx = Context::Get();
    CUDA_CHECK(cudaMemcpyAsync(host_.ptr, dev_.ptr, size_, cudaMemcpyDeviceToHost, ctx.stream()));
    ctx.SyncAndCheck();
    valid_ |= kHost;
  }
  return host_.ptr;
}

void* SyncedMemory::mutable_cpu_data() {
  cpu_data();
  valid_ = kHost;
  ++host_version_;
  return host_.ptr;
}

const void* SyncedMemory::gpu_data() {
  DeviceFromFreshest();
  return dev_.ptr;
}

void* SyncedMemory::mutable_gpu_data() {
  EnsureDevice();
  valid_ = kDevice;
  nhwc_aliases_dev_ = false;
  return dev_.ptr;
}

const void* SyncedMemory::gpu_data_nhwc(int n, int c, int h, int w) {
  CHECK_LE(static_cast<size_t>(n) * c * h * w * sizeof(float), size_);
  if (OrdersCoincide(c, h, w)) return gpu_data();
  WidenHalf();
  if (valid_ & kDeviceNhwc) {
    CHECK(dims_[0] == n && dims_[1] == c && dims_[2] == h && dims_[3] == w)
        << "channels-last copy was written with another shape";
    return nhwc_.ptr;
  }
  DeviceFromFreshest();
  EnsureNhwcBuffer();
  Context& ctx = Context::Get();
  KERNEL_CHECK(mcb200_nchw_to_nhwc(static_cast<const float*>(dev_.ptr), static_cast<float*>(nhwc_.ptr), n, c, h, w, c,
                                   ctx.stream_ptr()));
  dims_[0] = n; dims_[1] = c; dims_[2] = h; dims_[3] = w;
  nhwc_aliases_dev_ = false;
  valid_ |= kDeviceNhwc;
  return nhwc_.ptr;
}

void* SyncedMemory::mutable_gpu_data_nhwc(int n, int c, int h, int w) {
  CHECK_LE(static_cast<size_t>(n) * c * h * w * sizeof(float), size_);
  if (OrdersCoincide(c, h, w)) return mutable_gpu_data();
  EnsureNhwcBuffer();
  dims_[0] = n; dims_[1] = c; dims_[2] = h; dims_[3] = w;
  nhwc_aliases_dev_ = false;
  valid_ = kDeviceNhwc;
  return nhwc_.ptr;
}

const void* SyncedMemory::gpu_data_nhwc_bf16(int n, int c, int h, int w) {
  const size_t count = static_cast<size_t>(n) * c * h * w;
  CHECK_LE(count * sizeof(float), size_);
  if (valid_ & kDeviceNhwcHalf) {
    CHECK(dims_[0] == n && dims_[1] == c && dims_[2] == h && dims_[3] == w)
        << "bfloat16 copy was written with another shape";
    return half_.ptr;
  }
  const void* wide = gpu_data_nhwc(n, c, h, w);
  EnsureHalfBuffer();
  Context& ctx = Context::Get();
  KERNEL_CHECK(mcb200_f32_to_bf16(static_cast<const float*>(wide), static_cast<uint16_t*>(half_.ptr), count,
                                  ctx.stream_ptr()));
  dims_[0] = n; dims_[1] = c; dims_[2] = h; dims_[3] = w;
  valid_ |= kDeviceNhwcHalf;
  return half_.ptr;
}

void* SyncedMemory::mutable_gpu_data_nhwc_bf16(int n, int c, int h, int w) {
  CHECK_LE(static_cast<size_t>(n) * c * h * w * sizeof(float), size_);
  EnsureHalfBuffer();
  dims_[0] = n; dims_[1] = c; dims_[2] = h; dims_[3] = w;
  nhwc_aliases_dev_ = false;
  valid_ = kDeviceNhwcHalf;
  return half_.ptr;
}

}  // namespace caffe
