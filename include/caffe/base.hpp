// Basic types of the public C++ API: real_t, DeviceMode, SetMode, the
// per-thread memory-pool statistics.  Declarations match mini-caffe's
// include/caffe/base.hpp:48-77 so existing callers compile unchanged.
#ifndef CAFFE_BASE_HPP_
#define CAFFE_BASE_HPP_

#include <memory>
#include <string>
#include <vector>

#include <caffe/logging.hpp>

#define CAFFE_API __attribute__((visibility("default")))

#define STRINGIFY(m) #m
#define AS_STRING(m) STRINGIFY(m)

#define DISABLE_COPY_AND_ASSIGN(classname)         \
 private:                                          \
  classname(const classname&) = delete;            \
  classname(classname&&) = delete;                 \
  classname& operator=(const classname&) = delete; \
  classname& operator=(classname&&) = delete

#define NOT_IMPLEMENTED LOG(FATAL) << "Not Implemented Yet"
#define NO_GPU LOG(FATAL) << "Cannot use GPU in CPU-only Caffe: check mode."

namespace caffe {

using std::shared_ptr;
using std::string;
using std::vector;

typedef float real_t;

enum DeviceMode { CPU, GPU };

/*! \brief true when a CUDA device can be used by this process */
CAFFE_API bool GPUAvailable();

/*!
 * \brief choose the device of the calling thread (mode and device are per thread)
 * \param mode  GPU runs the engine on `device`.  This engine has no CPU compute
 *              path: after SetMode(CPU, -1) nets can still be built, inspected
 *              and loaded, but Net::Forward raises caffe::Error.
 * \param device CUDA device ordinal, -1 with CPU
 *
 * A thread that never calls SetMode runs on GPU 0.
 */
CAFFE_API void SetMode(DeviceMode mode, int device);

/*! \brief bytes held by the calling thread's memory pool */
struct MemPoolState {
  int gpu_mem;         // device bytes, all devices this thread used
  int cpu_mem;         // (pinned) host bytes
  int unused_gpu_mem;  // device bytes parked in the pool
  int unused_cpu_mem;  // host bytes parked in the pool
};
CAFFE_API MemPoolState MemPoolGetState();
/*! \brief give parked blocks of the calling thread's pool back to the system */
CAFFE_API void MemPoolClear();

}  // namespace caffe

#endif  // CAFFE_BASE_HPP_
