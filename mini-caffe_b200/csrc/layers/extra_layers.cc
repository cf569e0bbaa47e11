// Layer types that the shipped example networks use beyond the benchmark
// configurations: Deconvolution, Slice, Crop, BN, LRN.
#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "../filler.h"
#include "layers.h"

namespace caffe {

// ---------------------------------------------------------------- Deconvolution

void DeconvolutionLayer::LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  const ConvolutionParameter& p = layer_param_.convolution_param();
  const int channel_axis = bottom[0]->CanonicalAxisIndex(p.axis());
  CHECK(channel_axis == 1 && bottom[0]->num_axes() == 4)
      << "this engine implements 2-D deconvolution over (N, C, H, W) blobs";
  mcb200_conv_shape& s = shape_;
  ParseConvolutionGeometry(p, &s);
  s.c = bottom[0]->shape(1);
  s.cout = static_cast<int>(p.num_output());
  CHECK_GT(s.cout, 0);
  s.group = static_cast<int>(p.group());
  CHECK_GT(s.group, 0);
  CHECK_EQ(s.c % s.group, 0);
  CHECK_EQ(s.cout % s.group, 0) << "Number of output should be multiples of group.";
  bias_term_ = p.bias_term();
  // Input channels first: the layer is the transpose of a convolution from cout to c.
  const vector<int> weight_shape = {s.c, s.cout / s.group, s.kh, s.kw};
  const vector<int> bias_shape(bias_term_ ? 1 : 0, s.cout);
  if (!blobs_.empty()) {
    CHECK_EQ(static_cast<size_t>(1 + (bias_term_ ? 1 : 0)), blobs_.size()) << "Incorrect number of weight blobs.";
    if (weight_shape != blobs_[0]->shape()) {
      Blob expected(weight_shape);
      LOG(FATAL) << "Incorrect weight shape: expected shape " << expected.shape_string() << "; instead, shape was "
                 << blobs_[0]->shape_string();
    }
  } else {
    blobs_.resize(bias_term_ ? 2 : 1);
    blobs_[0].reset(new Blob(weight_shape));
    FillBlob(p.weight_filler(), blobs_[0].get());
    if (bias_term_) {
      blobs_[1].reset(new Blob(bias_shape));
      FillBlob(p.bias_filler(), blobs_[1].get());
    }
  }
}

void DeconvolutionLayer::Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  for (size_t i = 0; i < bottom.size(); ++i) {
    CHECK_EQ(bottom[i]->num_axes(), 4);
    CHECK_EQ(bottom[i]->shape(1), shape_.c) << "Input size incompatible with convolution kernel.";
    mcb200_conv_shape s = shape_;
    s.n = bottom[i]->num();
    s.h = bottom[i]->height();
    s.w = bottom[i]->width();
    CHECK_EQ(mcb200_deconv_out_shape(&s), 0) << "Deconvolution: the output would be empty";
    top[i]->Reshape(s.n, s.cout, s.ho, s.wo);
  }
}

void DeconvolutionLayer::Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  Context& ctx = Context::Get();
  const char* force_direct = getenv("MCB200_CONV_DIRECT");   // "1": the plain kernel, for comparisons in tests
  if (plans_.size() < bottom.size()) plans_.resize(bottom.size());
  for (size_t i = 0; i < bottom.size(); ++i) {
    mcb200_conv_shape s = shape_;
    s.n = bottom[i]->num();
    s.h = bottom[i]->height();
    s.w = bottom[i]->width();
    s.c_stride = s.c;
    mcb200_deconv_out_shape(&s);
    if (top[i]->count() == 0) continue;
    mcb200_conv_shape conv;
    const bool tensor_core = !(force_direct && force_direct[0] == '1') && mcb200_deconv_as_conv_shape(&s, &conv) == 0 &&
                             conv.pad_h <= 127 && conv.pad_w <= 127 && (conv.kh - 1) * conv.dil_h <= 255 &&
                             (conv.kw - 1) * conv.dil_w <= 255;
    if (!tensor_core) {
      KERNEL_CHECK(mcb200_deconv_direct(&s, bottom[i]->gpu_data(), blobs_[0]->gpu_data(),
                                        bias_term_ ? blobs_[1]->gpu_data() : nullptr, top[i]->mutable_gpu_data(),
                                        ctx.stream_ptr()));
      continue;
    }
    // The equivalent convolution's filter, re-laid when the weights change.
    const unsigned long long wv = blobs_[0]->host_version();
    if (wv != weight_version_) {
      float* flipped = flipped_weights_.Reserve(blobs_[0]->count());
      KERNEL_CHECK(mcb200_deconv_flip_weights(&s, blobs_[0]->gpu_data(), flipped, ctx.stream_ptr()));
      float* packed = packed_weights_.Reserve(mcb200_conv_packed_weight_count(&conv));
      KERNEL_CHECK(mcb200_conv_pack_weights(&conv, flipped, packed, ctx.stream_ptr()));
      weight_version_ = wv;
      for (auto& slot : plans_) {
        if (slot) slot->valid = false;
      }
    }
    // Stride 1 with a channel count that is a multiple of four reads the input as it is.
    const float* in = bottom[i]->gpu_data_nhwc();
    if (s.stride_h != 1 || s.stride_w != 1 || conv.c_stride != s.c) {
      float* spread = spread_input_.Reserve(static_cast<size_t>(conv.n) * conv.h * conv.w * conv.c_stride);
      KERNEL_CHECK(mcb200_deconv_spread_input(&s, in, spread, ctx.stream_ptr()));
      in = spread;
    }
    if (!plans_[i]) plans_[i].reset(new PlanSlot);
    PlanSlot& slot = *plans_[i];
    const float* w = packed_weights_.Reserve(0);
    if (!slot.valid || slot.in != in || slot.weights != w || std::memcmp(&slot.shape, &conv, sizeof(conv)) != 0) {
      CHECK_EQ(mcb200_conv_tc_plan(&conv, in, w, &slot.plan), 0)
          << "cannot build the tensor-core plan for layer " << layer_param_.name();
      slot.in = in;
      slot.weights = w;
      slot.shape = conv;
      slot.valid = true;
    }
    mcb200_epilogue ep = mcb200_epilogue();
    ep.residual_coeff = 1.f;
    ep.shift = bias_term_ ? blobs_[1]->gpu_data() : nullptr;
    KERNEL_CHECK(mcb200_conv_tc_launch(&slot.plan, top[i]->mutable_gpu_data_nhwc(), conv.cout, &ep, ctx.status_word(),
                                       ctx.stream_ptr()));
  }
}
REGISTER_LAYER_CLASS(Deconvolution);

// ---------------------------------------------------------------- Slice

void SliceLayer::LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  const SliceParameter& p = layer_param_.slice_param();
  CHECK(!(p.has_axis() && p.has_slice_dim())) << "Either axis or slice_dim should be specified; not both.";
  slice_point_.assign(p.slice_point().begin(), p.slice_point().end());
}

void SliceLayer::Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  const SliceParameter& p = layer_param_.slice_param();
  if (p.has_slice_dim()) {
    slice_axis_ = static_cast<int>(p.slice_dim());
    CHECK_GE(slice_axis_, 0);
    CHECK_LT(slice_axis_, bottom[0]->num_axes()) << "slice_dim out of range.";
  } else {
    slice_axis_ = bottom[0]->CanonicalAxisIndex(p.axis());
  }
  vector<int> top_shape = bottom[0]->shape();
  const int extent = bottom[0]->shape(slice_axis_);
  int count = 0;
  if (!slice_point_.empty()) {
    CHECK_EQ(slice_point_.size(), top.size() - 1);
    CHECK_LE(static_cast<int>(top.size()), extent);
    int prev = 0;
    for (size_t i = 0; i < top.size(); ++i) {
      const int end = i < slice_point_.size() ? slice_point_[i] : extent;
      if (i < slice_point_.size()) CHECK_GT(end, prev);
      top_shape[slice_axis_] = end - prev;
      top[i]->Reshape(top_shape);
      count += top[i]->count();
      prev = end;
    }
  } else {
    CHECK_EQ(extent % static_cast<int>(top.size()), 0)
        << "Number of top blobs (" << top.size() << ") should evenly divide input slice axis (" << extent << ")";
    top_shape[slice_axis_] = extent / static_cast<int>(top.size());
    for (Blob* t : top) {
      t->Reshape(top_shape);
      count += t->count();
    }
  }
  CHECK_EQ(count, bottom[0]->count());
}

void SliceLayer::Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  Context& ctx = Context::Get();
  const long long outer = bottom[0]->count(0, slice_axis_);
  const long long inner = bottom[0]->count(slice_axis_ + 1);
  const long long in_pitch = static_cast<long long>(bottom[0]->shape(slice_axis_)) * inner;
  const float* in = bottom[0]->gpu_data();
  long long offset = 0;
  for (Blob* t : top) {
    const long long cols = static_cast<long long>(t->shape(slice_axis_)) * inner;
    if (t->count() > 0) {
      KERNEL_CHECK(mcb200_copy_2d(in + offset, in_pitch, t->mutable_gpu_data(), cols, outer, cols, ctx.stream_ptr()));
    }
    offset += cols;
  }
}
REGISTER_LAYER_CLASS(Slice);

// ---------------------------------------------------------------- Crop

void CropLayer::LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  const CropParameter& p = layer_param_.crop_param();
  const int dims = bottom[0]->num_axes();
  const int start = bottom[0]->CanonicalAxisIndex(p.axis());
  CHECK_LT(start, dims) << "crop axis bigger than input dim";
  CHECK_LE(dims, 6) << "Crop: at most six axes";
  if (p.offset_size() > 1) {
    CHECK_EQ(start + p.offset_size(), dims)
        << "number of offset values specified must be equal to the number of dimensions following axis.";
  }
}

void CropLayer::Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  const CropParameter& p = layer_param_.crop_param();
  const int dims = bottom[0]->num_axes();
  const int start = bottom[0]->CanonicalAxisIndex(p.axis());
  offsets_.assign(dims, 0);
  vector<int> shape = bottom[0]->shape();
  for (int i = start; i < dims; ++i) {
    int offset = 0;
    if (p.offset_size() == 1) {
      offset = static_cast<int>(p.offset(0));
    } else if (p.offset_size() > 1) {
      offset = static_cast<int>(p.offset(i - start));
    }
    CHECK_GE(bottom[0]->shape(i) - offset, bottom[1]->shape(i))
        << "the crop for dimension " << i << " is out-of-bounds with size " << bottom[1]->shape(i) << " and offset "
        << offset;
    shape[i] = bottom[1]->shape(i);
    offsets_[i] = offset;
  }
  top[0]->Reshape(shape);
}

void CropLayer::Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  Context& ctx = Context::Get();
  if (top[0]->count() == 0) return;
  const vector<int>& in_shape = bottom[0]->shape();
  const vector<int>& out_shape = top[0]->shape();
  KERNEL_CHECK(mcb200_crop(bottom[0]->gpu_data(), top[0]->mutable_gpu_data(), bottom[0]->num_axes(), in_shape.data(),
                           out_shape.data(), offsets_.data(), ctx.stream_ptr()));
}
REGISTER_LAYER_CLASS(Crop);

// ---------------------------------------------------------------- BN

void BNLayer::LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  const BNParameter& p = layer_param_.bn_param();
  channels_ = bottom[0]->num_axes() == 1 ? 1 : bottom[0]->shape(1);
  if (blobs_.empty()) {
    blobs_.resize(4);
    const vector<int> shape = {1, channels_};
    for (auto& b : blobs_) b.reset(new Blob(shape));
    FillBlob(p.slope_filler(), blobs_[0].get());
    FillBlob(p.bias_filler(), blobs_[1].get());
    real_t* mean = blobs_[2]->mutable_cpu_data();
    real_t* factor = blobs_[3]->mutable_cpu_data();
    for (int c = 0; c < channels_; ++c) {
      mean[c] = 0;
      factor[c] = 1;
    }
  }
}

// The reference's inference path multiplies by blobs[3] as it is (it holds the
// inverse standard deviation): y = ((x - b2) * b3) * b0 + b1.
bool BNLayer::AsChannelAffine(int channels, std::vector<double>* scale, std::vector<double>* shift) {
  if (channels != channels_ || blobs_.size() != 4) return false;
  for (const auto& b : blobs_)
    if (b->count() != channels) return false;
  if (!scale) return true;
  const float* slope = blobs_[0]->cpu_data();
  const float* bias = blobs_[1]->cpu_data();
  const float* mean = blobs_[2]->cpu_data();
  const float* factor = blobs_[3]->cpu_data();
  scale->resize(channels);
  shift->resize(channels);
  for (int c = 0; c < channels; ++c) {
    const double s = static_cast<double>(factor[c]) * slope[c];
    (*scale)[c] = s;
    (*shift)[c] = static_cast<double>(bias[c]) - static_cast<double>(mean[c]) * s;
  }
  return true;
}
REGISTER_LAYER_CLASS(BN);

// ---------------------------------------------------------------- LRN

void LRNLayer::LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  const LRNParameter& p = layer_param_.lrn_param();
  size_ = static_cast<int>(p.local_size());
  CHECK_EQ(size_ % 2, 1) << "LRN only supports odd values for local_size";
  alpha_ = p.alpha();
  beta_ = p.beta();
  k_ = p.k();
  within_channel_ = p.norm_region() == LRNParameter::WITHIN_CHANNEL;
}

void LRNLayer::Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  CHECK_EQ(4, bottom[0]->num_axes()) << "Input must have 4 axes, corresponding to (num, channels, height, width)";
  top[0]->ReshapeLike(*bottom[0]);
}

void LRNLayer::Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  Context& ctx = Context::Get();
  if (top[0]->count() == 0) return;
  const float* in = bottom[0]->gpu_data();
  if (top[0] == bottom[0]) {
    // Every output reads its neighbours' inputs: work from a copy when the layer runs in place.
    if (!in_place_copy_) in_place_copy_.reset(new Blob());
    in_place_copy_->ReshapeLike(*bottom[0]);
    CUDA_CHECK(cudaMemcpyAsync(in_place_copy_->mutable_gpu_data(), in, sizeof(float) * bottom[0]->count(),
                               cudaMemcpyDeviceToDevice, ctx.stream()));
    in = in_place_copy_->gpu_data();
  }
  KERNEL_CHECK(mcb200_lrn(in, top[0]->mutable_gpu_data(), bottom[0]->num(), bottom[0]->channels(),
                          bottom[0]->height(), bottom[0]->width(), size_, alpha_, beta_, k_, within_channel_ ? 1 : 0,
                          ctx.stream_ptr()));
}
REGISTER_LAYER_CLASS(LRN);

// ---------------------------------------------------------------- TanH / Sigmoid

void UnaryLayer::Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  Context& ctx = Context::Get();
  // Elementwise: whichever device copy is current is as good as the other.
  const bool nhwc = bottom[0]->device_is_nhwc();
  const float* x = nhwc ? bottom[0]->gpu_data_nhwc() : bottom[0]->gpu_data();
  float* y = nhwc ? top[0]->mutable_gpu_data_nhwc() : top[0]->mutable_gpu_data();
  KERNEL_CHECK(mcb200_unary(x, y, bottom[0]->count(), op_, ctx.stream_ptr()));
}

static shared_ptr<Layer> CreateTanH(const LayerParameter& param) {
  return shared_ptr<Layer>(new UnaryLayer(param, MCB200_UNARY_TANH, "TanH"));
}
static shared_ptr<Layer> CreateSigmoid(const LayerParameter& param) {
  return shared_ptr<Layer>(new UnaryLayer(param, MCB200_UNARY_SIGMOID, "Sigmoid"));
}
REGISTER_LAYER_CREATOR(TanH, CreateTanH);
REGISTER_LAYER_CREATOR(Sigmoid, CreateSigmoid);

}  // namespace caffe
