// Same probe as exp_probe_proposal.cc for the SSD box decoding in
// util/bbox_util.cpp (include chain of bbox_util.cpp:1-11).
#include <algorithm>
#include <csignal>
#include <ctime>
#include <functional>
#include <map>
#include <set>
#include <string>
#include <utility>
#include <vector>

#include "util/bbox_util.hpp"
#include <type_traits>

namespace caffe {
static const bool kExpIsDouble = std::is_same<decltype(exp(1.f)), double>::value;
}  // namespace caffe

extern "C" int OracleRefBBoxExpIsDouble() { return caffe::kExpIsDouble ? 1 : 0; }
