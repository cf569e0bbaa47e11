// Weight initialisation for layers built without a caffemodel.  As in
// mini-caffe (src/filler.hpp:51-71) every known filler type fills with the
// constant `value` of its FillerParameter -- the library is inference-only, so
// real weights come from a caffemodel or are written through Net::params().
#ifndef MCB200_FILLER_H_
#define MCB200_FILLER_H_

#include <string>

#include "caffe.pb.h"
#include "caffe/blob.hpp"

namespace caffe {

inline void FillBlob(const FillerParameter& param, Blob* blob) {
  const std::string& type = param.type();
  CHECK(type == "constant" || type == "gaussian" || type == "positive_unitball" || type == "uniform" ||
        type == "xavier" || type == "msra" || type == "bilinear")
      << "Unknown filler name: " << type;
  CHECK(blob->count());
  CHECK_EQ(param.sparse(), -1) << "Sparsity not supported by this Filler.";
  real_t* data = blob->mutable_cpu_data();
  const real_t value = param.value();
  for (int i = 0; i < blob->count(); ++i) data[i] = value;
}

}  // namespace caffe

#endif  // MCB200_FILLER_H_
