// Records which exp() overload the reference's RPN box decoding binds to.
//
// proposal_layer.cpp calls an unqualified exp(float) inside namespace caffe.
// With only <cmath> visible that is the C function double exp(double); if
// <math.h> is also visible it is the float overload.  Kept-box index sets are
// compared bit for bit, so the device code has to round the same way.  This
// translation unit repeats that file's include chain (proposal_layer.cpp:1-2)
// and exports the answer so tests can assert on it.
#include "layers/proposal_layer.hpp"
#include <cmath>
#include <type_traits>

namespace caffe {
static const bool kExpIsDouble = std::is_same<decltype(exp(1.f)), double>::value;
}  // namespace caffe

extern "C" int OracleRefProposalExpIsDouble() { return caffe::kExpIsDouble ? 1 : 0; }
