#include "launch_count.h"

#include "../../../include/mcb200_kernels.h"

namespace mcb200 {
long long& launch_counter() {
  static thread_local long long count = 0;
  return count;
}
}  // namespace mcb200

extern "C" long long mcb200_launch_count(void) { return mcb200::launch_counter(); }
extern "C" void mcb200_launch_count_reset(void) { mcb200::launch_counter() = 0; }
