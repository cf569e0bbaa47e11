// Optional event bracketing of kernel launches (see include/mcb200_runtime.h).
#pragma once

#include <cuda_runtime.h>

namespace mcb200 {

// Records an event pair around the lifetime of the object when timing is on.
class TimedLaunch {
 public:
  explicit TimedLaunch(cudaStream_t stream);
  ~TimedLaunch();
 private:
  cudaStream_t stream_;
  int slot_;
};

}  // namespace mcb200
