// Storage behind a Blob: up to four copies of the same values,
//   * host (pinned when a device exists), in Caffe's (N, C, H, W) order,
//   * device, same order,
//   * device, channels-last (N, H, W, C) -- the order the tensor-core and most
//     other kernels of the engine work in,
//   * device, channels-last, rounded to bfloat16 -- written and read only by
//     the tensor-core convolutions of a net built with bfloat16 storage; every
//     other accessor first widens it back to fp32,
// with a bit per copy saying whether it is current.  A read accessor brings
// its copy up to date from whichever copy is (host<->device copies on the
// thread's stream, layout conversion by a transpose kernel); a mutable
// accessor additionally marks the other copies stale.
//
// mini-caffe's SyncedMemory has the first two copies and a four-state head
// (src/syncedmem.hpp:86, src/syncedmem.cpp:40-121); the thread-local
// MemoryPool with its "reuse a block if it is at most twice the request" rule
// follows src/syncedmem.cpp:177-293.
#ifndef MCB200_SYNCEDMEM_H_
#define MCB200_SYNCEDMEM_H_

#include <cstddef>
#include <map>
#include <mutex>

#include "caffe/base.hpp"

namespace caffe {

class MemoryPool;

struct MemBlock {
  void* ptr = nullptr;
  size_t size = 0;
  int device = -1;  // -1: host
  // The pool the block was taken from and the stream its user's work is queued
  // on (the requesting thread's).  A block always goes back to this pool, also
  // when another thread destroys the object that holds it.
  MemoryPool* pool = nullptr;
  void* stream = nullptr;
};

class MemoryPool {
 public:
  static MemoryPool* Get();  // of the calling thread
  MemBlock RequestCPU(size_t size);
  void ReturnCPU(MemBlock block);
  MemBlock RequestGPU(size_t size, int device);
  void ReturnGPU(MemBlock block);
  // Gives a block back to the pool it came from, from whichever thread.  The
  // pool's reuse rule rests on blocks being reused by work on the stream that
  // used them last; when the calling thread is not the owner, both threads'
  // streams are drained first, and if the owning thread (and its pool) is gone
  // the block is freed.
  static void Release(MemBlock block);
  void Clear();
  MemPoolState GetState() const;
  ~MemoryPool();

 private:
  MemoryPool();
  void Insert(const MemBlock& block);
  mutable std::mutex mu_;   // the owner allocates, any thread may return
  std::multimap<size_t, MemBlock> cpu_free_;
  std::multimap<std::pair<int, size_t>, MemBlock> gpu_free_;
  long long cpu_total_ = 0, gpu_total_ = 0, cpu_unused_ = 0, gpu_unused_ = 0;
};

class SyncedMemory {
 public:
  enum Copy { kHost = 1, kDevice = 2, kDeviceNhwc = 4, kDeviceNhwcHalf = 8 };

  explicit SyncedMemory(size_t size);
  ~SyncedMemory();

  const void* cpu_data();
  void* mutable_cpu_data();
  const void* gpu_data();
  void* mutable_gpu_data();
  // Channels-last copy of the (n, c, h, w) tensor stored here.  When the two
  // orders coincide (c == 1 or h*w == 1) it is the plain device copy.
  const void* gpu_data_nhwc(int n, int c, int h, int w);
  void* mutable_gpu_data_nhwc(int n, int c, int h, int w);
  // bfloat16 channels-last copy (16-bit cells), rounded from the fp32 values on first use.
  const void* gpu_data_nhwc_bf16(int n, int c, int h, int w);
  void* mutable_gpu_data_nhwc_bf16(int n, int c, int h, int w);

  size_t size() const { return size_; }
  int valid() const { return valid_; }
  bool nhwc_is_freshest() const { return (valid_ & (kDeviceNhwc | kDeviceNhwcHalf)) && !(valid_ & kDevice); }
  unsigned long long host_version() const { return host_version_; }

 private:
  void EnsureHost();
  void EnsureDevice();
  void EnsureNhwcBuffer();
  void EnsureHalfBuffer();
  void WidenHalf();           // only the bfloat16 copy is current: make an fp32 device copy current too
  void DeviceFromFreshest();  // make kDevice valid
  static bool OrdersCoincide(int c, int h, int w) { return c == 1 || h * w == 1; }

  size_t size_;
  MemBlock host_, dev_, nhwc_, half_;
  int valid_;               // bit set of Copy
  bool nhwc_aliases_dev_;   // the channels-last copy is dev_ itself
  int dims_[4];             // (n, c, h, w) the channels-last copy was written with
  unsigned long long host_version_;
  DISABLE_COPY_AND_ASSIGN(SyncedMemory);
};

}  // namespace caffe

#endif  // MCB200_SYNCEDMEM_H_
