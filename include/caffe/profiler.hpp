// Scope profiler of the public API (process-wide, not thread safe): nested
// named scopes with microsecond wall-clock stamps, dumped as a chrome://tracing
// JSON file.  Same interface as mini-caffe's include/caffe/profiler.hpp:28-84.
#ifndef CAFFE_PROFILER_HPP_
#define CAFFE_PROFILER_HPP_

#include <cstdint>
#include <string>
#include <vector>

#include "caffe/base.hpp"

namespace caffe {

class CAFFE_API Profiler {
 public:
  /*! \brief the process-wide instance */
  static Profiler* Get();
  /*! \brief open a scope; inside another scope the name becomes "outer:name" */
  void ScopeStart(const char* name);
  /*! \brief close the innermost open scope */
  void ScopeEnd();
  /*! \brief write every closed scope as begin/end trace events */
  void DumpProfile(const char* fn) const;
  void TurnON() {
    CHECK_EQ(state_, kNotRunning) << "Profile is already running.";
    state_ = kRunning;
  }
  void TurnOFF() {
    CHECK_EQ(state_, kRunning) << "Profile is not running.";
    CHECK(open_.empty()) << "Profile scope stack is not empty, with size = " << open_.size();
    state_ = kNotRunning;
  }
  /*! \brief wall clock in microseconds */
  uint64_t Now() const;
  /*! \brief true between TurnON and TurnOFF */
  bool running() const { return state_ == kRunning; }

 private:
  Profiler();
  DISABLE_COPY_AND_ASSIGN(Profiler);

  enum State { kRunning, kNotRunning };
  struct Scope {
    std::string name;
    uint64_t begin_us = 0;
    uint64_t end_us = 0;
  };
  std::vector<Scope> open_;    // innermost last
  std::vector<Scope> closed_;  // in closing order
  uint64_t origin_us_;
  State state_;
};

}  // namespace caffe

#endif  // CAFFE_PROFILER_HPP_
