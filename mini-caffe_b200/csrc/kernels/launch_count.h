// Per-thread count of kernels this library has launched (read through
// mcb200_launch_count; the benchmark reports it).
#pragma once

namespace mcb200 {
long long& launch_counter();
inline void count_launch(int n = 1) { launch_counter() += n; }
}  // namespace mcb200
