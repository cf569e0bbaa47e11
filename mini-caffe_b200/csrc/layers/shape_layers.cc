// Input, Split, Flatten, Reshape, Permute, Concat: layers that move or
// re-interpret data without arithmetic.
#include <algorithm>

#include "layers.h"

namespace caffe {

static void DeviceCopy(const float* src, float* dst, size_t count) {
  if (src == dst || count == 0) return;
  CUDA_CHECK(cudaMemcpyAsync(dst, src, count * sizeof(float), cudaMemcpyDeviceToDevice, Context::Get().stream()));
}

// ---------------------------------------------------------------- Input

void InputLayer::LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  const InputParameter& p = layer_param_.input_param();
  const int num_top = static_cast<int>(top.size());
  const int num_shape = p.shape_size();
  CHECK(num_shape == 0 || num_shape == 1 || num_shape == num_top)
      << "Must specify 'shape' once, once per top blob, or not at all: " << num_top << " tops vs. " << num_shape
      << " shapes.";
  for (int i = 0; num_shape > 0 && i < num_top; ++i) top[i]->Reshape(p.shape(num_shape == 1 ? 0 : i));
}
REGISTER_LAYER_CLASS(Input);

// ---------------------------------------------------------------- Split

void SplitLayer::Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  for (size_t i = 0; i < top.size(); ++i) {
    CHECK_NE(top[i], bottom[0]) << type() << " Layer does not allow in-place computation.";
    top[i]->ReshapeLike(*bottom[0]);
  }
}

void SplitLayer::Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  const bool nhwc = bottom[0]->device_is_nhwc();
  for (Blob* t : top) {
    if (nhwc) {
      DeviceCopy(bottom[0]->gpu_data_nhwc(), t->mutable_gpu_data_nhwc(), bottom[0]->count());
    } else {
      DeviceCopy(bottom[0]->gpu_data(), t->mutable_gpu_data(), bottom[0]->count());
    }
  }
}
REGISTER_LAYER_CLASS(Split);

// ---------------------------------------------------------------- Flatten

void FlattenLayer::Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  const FlattenParameter& p = layer_param_.flatten_param();
  const int start = bottom[0]->CanonicalAxisIndex(p.axis());
  const int end = bottom[0]->CanonicalAxisIndex(p.end_axis());
  vector<int> shape;
  for (int i = 0; i < start; ++i) shape.push_back(bottom[0]->shape(i));
  shape.push_back(bottom[0]->count(start, end + 1));
  for (int i = end + 1; i < bottom[0]->num_axes(); ++i) shape.push_back(bottom[0]->shape(i));
  top[0]->Reshape(shape);
  CHECK_EQ(top[0]->count(), bottom[0]->count());
}

void FlattenLayer::Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  // The flattened order is the (N, C, H, W) order.
  if (bottom[0] != top[0]) DeviceCopy(bottom[0]->gpu_data(), top[0]->mutable_gpu_data(), bottom[0]->count());
}
REGISTER_LAYER_CLASS(Flatten);

// ---------------------------------------------------------------- Reshape

void ReshapeLayer::LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  CHECK_NE(top[0], bottom[0]) << type() << " Layer does not allow in-place computation.";
  inferred_axis_ = -1;
  copy_axes_.clear();
  constant_count_ = 1;
  const BlobShape& shape = layer_param_.reshape_param().shape();
  for (int i = 0; i < shape.dim_size(); ++i) {
    const int d = static_cast<int>(shape.dim(i));
    if (d == 0) {
      copy_axes_.push_back(i);
    } else if (d == -1) {
      CHECK_EQ(inferred_axis_, -1) << "new shape contains multiple -1 dims; at most a single (1) value of -1 may be "
                                      "specified";
      inferred_axis_ = i;
    } else {
      constant_count_ *= d;
    }
  }
}

void ReshapeLayer::Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  const ReshapeParameter& p = layer_param_.reshape_param();
  const int in_axis = p.axis();
  const int start = in_axis >= 0 ? in_axis : bottom[0]->num_axes() + in_axis + 1;
  CHECK_GE(start, 0) << "axis " << in_axis << " out of range";
  CHECK_LE(start, bottom[0]->num_axes()) << "axis " << in_axis << " out of range for " << bottom[0]->num_axes()
                                         << "-D input blob";
  const int num_axes = p.num_axes();
  CHECK_GE(num_axes, -1) << "num_axes must be >= 0, or -1 for all";
  const int end = num_axes == -1 ? bottom[0]->num_axes() : start + num_axes;
  CHECK_LE(end, bottom[0]->num_axes()) << "end_axis = axis + num_axes is out of range";
  const BlobShape& new_dims = p.shape();
  vector<int> shape;
  for (int i = 0; i < start; ++i) shape.push_back(bottom[0]->shape(i));
  for (int i = 0; i < new_dims.dim_size(); ++i) shape.push_back(static_cast<int>(new_dims.dim(i)));
  for (int i = end; i < bottom[0]->num_axes(); ++i) shape.push_back(bottom[0]->shape(i));
  for (int idx : copy_axes_) {
    CHECK_GT(bottom[0]->num_axes(), start + idx)
        << "new shape contains a 0, but there was no corresponding bottom axis to copy";
    shape[start + idx] = bottom[0]->shape(start + idx);
  }
  if (inferred_axis_ >= 0) {
    int explicit_count = constant_count_ * bottom[0]->count(0, start) * bottom[0]->count(end);
    for (int idx : copy_axes_) explicit_count *= shape[start + idx];
    CHECK_EQ(0, bottom[0]->count() % explicit_count)
        << "bottom count (" << bottom[0]->count() << ") must be divisible by the product of the specified dimensions ("
        << explicit_count << ")";
    shape[start + inferred_axis_] = bottom[0]->count() / explicit_count;
  }
  top[0]->Reshape(shape);
  CHECK_EQ(top[0]->count(), bottom[0]->count()) << "output count must match input count";
}

void ReshapeLayer::Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  DeviceCopy(bottom[0]->gpu_data(), top[0]->mutable_gpu_data(), bottom[0]->count());
}
REGISTER_LAYER_CLASS(Reshape);

// ---------------------------------------------------------------- Permute

void PermuteLayer::LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  const PermuteParameter& p = layer_param_.permute_param();
  const int num_axes = bottom[0]->num_axes();
  CHECK_LE(num_axes, 6) << "Permute: at most 6 axes are supported";
  order_.clear();
  for (int i = 0; i < p.order_size(); ++i) {
    const int o = static_cast<int>(p.order(i));
    CHECK_LT(o, num_axes) << "order should be less than the input dimension.";
    CHECK(std::find(order_.begin(), order_.end(), o) == order_.end()) << "there are duplicate orders";
    order_.push_back(o);
  }
  for (int i = 0; i < num_axes; ++i) {
    if (std::find(order_.begin(), order_.end(), i) == order_.end()) order_.push_back(i);
  }
  need_permute_ = false;
  for (int i = 0; i < num_axes; ++i) need_permute_ = need_permute_ || order_[i] != i;
}

void PermuteLayer::Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  CHECK_EQ(static_cast<size_t>(bottom[0]->num_axes()), order_.size());
  vector<int> shape(order_.size());
  for (size_t i = 0; i < order_.size(); ++i) shape[i] = bottom[0]->shape(order_[i]);
  top[0]->Reshape(shape);
}

void PermuteLayer::Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  Context& ctx = Context::Get();
  if (!need_permute_) {
    DeviceCopy(bottom[0]->gpu_data(), top[0]->mutable_gpu_data(), bottom[0]->count());
    return;
  }
  if (order_.size() == 4 && order_[0] == 0 && order_[1] == 2 && order_[2] == 3 && order_[3] == 1) {
    // (N, C, H, W) -> (N, H, W, C) is exactly the channels-last copy the
    // producing convolution already wrote.
    DeviceCopy(bottom[0]->gpu_data_nhwc(), top[0]->mutable_gpu_data(), bottom[0]->count());
    return;
  }
  KERNEL_CHECK(mcb200_permute(bottom[0]->gpu_data(), top[0]->mutable_gpu_data(), static_cast<int>(order_.size()),
                              bottom[0]->shape().data(), order_.data(), ctx.stream_ptr()));
}
REGISTER_LAYER_CLASS(Permute);

// ---------------------------------------------------------------- Concat

void ConcatLayer::LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  const ConcatParameter& p = layer_param_.concat_param();
  CHECK(!(p.has_axis() && p.has_concat_dim())) << "Either axis or concat_dim should be specified; not both.";
}

void ConcatLayer::Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  const ConcatParameter& p = layer_param_.concat_param();
  const int num_axes = bottom[0]->num_axes();
  if (p.has_concat_dim()) {
    axis_ = static_cast<int>(p.concat_dim());
    CHECK_GE(axis_, 0) << "casting concat_dim from uint32 to int32 produced negative result; concat_dim must satisfy "
                       << "0 <= concat_dim < " << kMaxBlobAxes;
    CHECK_LT(axis_, num_axes) << "concat_dim out of range.";
  } else {
    axis_ = bottom[0]->CanonicalAxisIndex(p.axis());
  }
  vector<int> shape = bottom[0]->shape();
  long long total = bottom[0]->count();
  for (size_t i = 1; i < bottom.size(); ++i) {
    CHECK_EQ(num_axes, bottom[i]->num_axes()) << "All inputs must have the same #axes.";
    for (int j = 0; j < num_axes; ++j) {
      if (j == axis_) continue;
      CHECK_EQ(shape[j], bottom[i]->shape(j)) << "All inputs must have the same shape, except at concat_axis.";
    }
    total += bottom[i]->count();
    shape[axis_] += bottom[i]->shape(axis_);
  }
  top[0]->Reshape(shape);
  CHECK_EQ(total, static_cast<long long>(top[0]->count()));
}

void ConcatLayer::Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  Context& ctx = Context::Get();
  bool nhwc = axis_ == 1 && top[0]->num_axes() == 4 && top[0]->height() * top[0]->width() > 1;
  if (nhwc) {
    bool any = false;
    for (Blob* b : bottom) any = any || b->device_is_nhwc();
    nhwc = any;
  }
  if (nhwc) {
    // Channels-last: each bottom contributes a column block of every pixel row.
    float* out = top[0]->mutable_gpu_data_nhwc();
    const long long pixels = static_cast<long long>(top[0]->num()) * top[0]->height() * top[0]->width();
    const int total_c = top[0]->channels();
    int offset = 0;
    for (Blob* b : bottom) {
      KERNEL_CHECK(mcb200_copy_2d(b->gpu_data_nhwc(), b->channels(), out + offset, total_c, pixels, b->channels(),
                                  ctx.stream_ptr()));
      offset += b->channels();
    }
    return;
  }
  float* out = top[0]->mutable_gpu_data();
  const long long outer = top[0]->count(0, axis_);
  const long long inner = top[0]->count(axis_ + 1);
  const long long top_row = static_cast<long long>(top[0]->shape(axis_)) * inner;
  long long offset = 0;
  for (Blob* b : bottom) {
    const long long cols = static_cast<long long>(b->shape(axis_)) * inner;
    KERNEL_CHECK(mcb200_copy_2d(b->gpu_data(), cols, out + offset, top_row, outer, cols, ctx.stream_ptr()));
    offset += cols;
  }
}
REGISTER_LAYER_CLASS(Concat);

}  // namespace caffe
