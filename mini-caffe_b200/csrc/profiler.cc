// Scope profiler: see include/caffe/profiler.hpp.  The dump is a
// chrome://tracing file with one begin ("B") and one end ("E") event per
// closed scope, in the field layout of mini-caffe's src/profiler.cpp:59-99.
#include "caffe/profiler.hpp"

#include <chrono>
#include <fstream>

namespace caffe {

Profiler::Profiler() : origin_us_(Now()), state_(kNotRunning) {}

Profiler* Profiler::Get() {
  static Profiler instance;
  return &instance;
}

uint64_t Profiler::Now() const {
  return static_cast<uint64_t>(std::chrono::duration_cast<std::chrono::microseconds>(
                                   std::chrono::high_resolution_clock::now().time_since_epoch())
                                   .count());
}

void Profiler::ScopeStart(const char* name) {
  if (state_ == kNotRunning) return;
  Scope scope;
  scope.name = open_.empty() ? std::string(name) : open_.back().name + ":" + name;
  scope.begin_us = Now() - origin_us_;
  open_.push_back(scope);
}

void Profiler::ScopeEnd() {
  if (state_ == kNotRunning) return;
  CHECK(!open_.empty());
  Scope scope = open_.back();
  open_.pop_back();
  scope.end_us = Now() - origin_us_;
  closed_.push_back(scope);
}

static void WriteEvent(std::ofstream& out, const std::string& name, const char* phase, uint64_t ts) {
  out << "    {\n"
      << "      \"name\": \"" << name << "\",\n"
      << "      \"cat\": \"category\",\n"
      << "      \"ph\": \"" << phase << "\",\n"
      << "      \"ts\": " << ts << ",\n"
      << "      \"pid\": 0,\n"
      << "      \"tid\": 0\n"
      << "    }";
}

void Profiler::DumpProfile(const char* fn) const {
  CHECK(open_.empty());
  CHECK_EQ(state_, kNotRunning);
  std::ofstream out(fn);
  CHECK(out.good()) << "cannot write profile to " << fn;
  out << "{\n  \"traceEvents\": [";
  for (size_t i = 0; i < closed_.size(); ++i) {
    out << (i == 0 ? "\n" : ",\n");
    WriteEvent(out, closed_[i].name, "B", closed_[i].begin_us);
    out << ",\n";
    WriteEvent(out, closed_[i].name, "E", closed_[i].end_us);
  }
  out << "  ],\n  \"displayTimeUnit\": \"ms\"\n}\n";
}

}  // namespace caffe
