#include "kernel_timer.h"

#include <vector>

#include "../../../include/mcb200_runtime.h"

namespace mcb200 {
namespace {

struct TimerState {
  bool enabled = false;
  std::vector<cudaEvent_t> begin, end;  // event pool, reused across sessions
  int used = 0;
};

TimerState& State() {
  static thread_local TimerState s;
  return s;
}

}  // namespace

TimedLaunch::TimedLaunch(cudaStream_t stream) : stream_(stream), slot_(-1) {
  TimerState& s = State();
  if (!s.enabled) return;
  if (s.used == static_cast<int>(s.begin.size())) {
    cudaEvent_t a, b;
    if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) return;
    s.begin.push_back(a);
    s.end.push_back(b);
  }
  slot_ = s.used++;
  cudaEventRecord(s.begin[slot_], stream_);
}

TimedLaunch::~TimedLaunch() {
  if (slot_ >= 0) cudaEventRecord(State().end[slot_], stream_);
}

}  // namespace mcb200

extern "C" void mcb200_kernel_timing_begin(void) {
  mcb200::TimerState& s = mcb200::State();
  s.used = 0;
  s.enabled = true;
}

extern "C" long long mcb200_kernel_timing_end_each(double* total_ms, double* each_ms, long long capacity) {
  mcb200::TimerState& s = mcb200::State();
  s.enabled = false;
  double sum = 0.0;
  for (int i = 0; i < s.used; ++i) {
    float ms = 0.f;
    if (cudaEventSynchronize(s.end[i]) == cudaSuccess && cudaEventElapsedTime(&ms, s.begin[i], s.end[i]) == cudaSuccess)
      sum += ms;
    if (each_ms && i < capacity) each_ms[i] = ms;
  }
  if (total_ms) *total_ms = sum;
  const long long n = s.used;
  s.used = 0;
  return n;
}

extern "C" long long mcb200_kernel_timing_end(double* total_ms) {
  return mcb200_kernel_timing_end_each(total_ms, nullptr, 0);
}
