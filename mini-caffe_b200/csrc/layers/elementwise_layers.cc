// BatchNorm, Scale, Bias, ReLU, PReLU, Dropout and Eltwise.
//
// The first five are "y = act(x * scale[c] + shift[c])" layers.  Inside a net
// they are normally folded into the convolution or inner product in front of
// them (see FusedTail); the stand-alone forward here runs one vectorised pass
// in whichever memory order the bottom currently has.
#include <cmath>

#include "../filler.h"
#include "layers.h"

namespace caffe {

// ---------------------------------------------------------------- ChannelwiseLayer

void ChannelwiseLayer::Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  if (top[0] != bottom[0]) top[0]->ReshapeLike(*bottom[0]);
}

void ChannelwiseLayer::Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  Context& ctx = Context::Get();
  const int channels = Channels(bottom[0]);
  std::vector<double> scale, shift;
  const bool affine = AsChannelAffine(channels, nullptr, nullptr);
  if (affine) {
    const unsigned long long v = 1 + ParamVersion();
    if (v != built_version_ || channels != built_channels_) {
      CHECK(AsChannelAffine(channels, &scale, &shift));
      scale_dev_.Assign(std::vector<float>(scale.begin(), scale.end()));
      shift_dev_.Assign(std::vector<float>(shift.begin(), shift.end()));
      built_version_ = v;
      built_channels_ = channels;
    }
  }
  mcb200_epilogue ep = mcb200_epilogue();
  ActivationSpec spec;
  if (AsActivation(&spec)) {
    ep.act = spec.kind;
    ep.slope = spec.slope;
    if (spec.kind == 2) {
      ep.prelu = spec.slopes->gpu_data();
      ep.prelu_shared = spec.shared ? 1 : 0;
    }
  }
  const bool nhwc = bottom[0]->device_is_nhwc();
  const float* x = nhwc ? bottom[0]->gpu_data_nhwc() : bottom[0]->gpu_data();
  float* y = nhwc ? top[0]->mutable_gpu_data_nhwc() : top[0]->mutable_gpu_data();
  const int inner = nhwc ? 1 : (bottom[0]->num_axes() > 2 ? bottom[0]->count(2) : 1);
  if (!affine && ep.act == 0) {
    if (x != y) {
      CUDA_CHECK(cudaMemcpyAsync(y, x, sizeof(float) * bottom[0]->count(), cudaMemcpyDeviceToDevice, ctx.stream()));
    }
    return;
  }
  KERNEL_CHECK(mcb200_channel_affine_act(x, y, bottom[0]->count(), channels, inner, affine ? scale_dev_.get() : nullptr,
                                         affine ? shift_dev_.get() : nullptr, &ep, ctx.stream_ptr()));
}

// ---------------------------------------------------------------- BatchNorm

void BatchNormLayer::LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  const BatchNormParameter& p = layer_param_.batch_norm_param();
  use_global_stats_ = !p.has_use_global_stats() || p.use_global_stats();   // src/layers/batch_norm_layer.cpp:11-13
  channels_ = bottom[0]->num_axes() == 1 ? 1 : bottom[0]->shape(1);
  eps_ = p.eps();
  if (blobs_.empty()) {
    blobs_.resize(3);
    blobs_[0].reset(new Blob(vector<int>(1, channels_)));
    blobs_[1].reset(new Blob(vector<int>(1, channels_)));
    blobs_[2].reset(new Blob(vector<int>(1, 1)));
    for (auto& b : blobs_) {
      real_t* d = b->mutable_cpu_data();
      for (int i = 0; i < b->count(); ++i) d[i] = 0;
    }
  }
}

// mean = blobs[0] / f, var = blobs[1] / f with f = blobs[2][0] (f == 0 gives
// mean = var = 0); y = (x - mean) / sqrt(var + eps)
// (src/layers/batch_norm_layer.cpp:83-135).  Evaluated in float like there.
bool BatchNormLayer::AsChannelAffine(int channels, std::vector<double>* scale, std::vector<double>* shift) {
  if (!use_global_stats_) return false;   // depends on the data: cannot be folded into a producer
  if (channels != channels_ || blobs_.size() != 3) return false;
  if (!scale) return true;
  const float factor_raw = blobs_[2]->cpu_data()[0];
  const float factor = factor_raw == 0.f ? 0.f : 1.f / factor_raw;
  const float* mean = blobs_[0]->cpu_data();
  const float* var = blobs_[1]->cpu_data();
  scale->resize(channels);
  shift->resize(channels);
  for (int c = 0; c < channels; ++c) {
    const float m = mean[c] * factor;
    const float v = var[c] * factor + eps_;
    const double inv_std = 1.0 / static_cast<double>(std::pow(v, 0.5f));
    (*scale)[c] = inv_std;
    (*shift)[c] = -static_cast<double>(m) * inv_std;
  }
  return true;
}

// With use_global_stats: false the mean and variance come from the batch at hand
// (src/layers/batch_norm_layer.cpp:91-118): one reduction kernel writes the
// per-channel scale and shift, the affine kernel applies them.
void BatchNormLayer::Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  if (use_global_stats_) {
    ChannelwiseLayer::Forward_gpu(bottom, top);
    return;
  }
  Context& ctx = Context::Get();
  if (bottom[0]->count() == 0) return;
  CHECK_EQ(Channels(bottom[0]), channels_);
  float* scale = batch_scale_shift_.Reserve(2 * static_cast<size_t>(channels_));
  float* shift = scale + channels_;
  const bool nhwc = bottom[0]->device_is_nhwc();
  const float* x = nhwc ? bottom[0]->gpu_data_nhwc() : bottom[0]->gpu_data();
  float* y = nhwc ? top[0]->mutable_gpu_data_nhwc() : top[0]->mutable_gpu_data();
  const int inner = nhwc ? 1 : (bottom[0]->num_axes() > 2 ? bottom[0]->count(2) : 1);
  KERNEL_CHECK(mcb200_channel_batch_stats(x, bottom[0]->count(), channels_, inner, eps_, scale, shift,
                                          ctx.stream_ptr()));
  mcb200_epilogue ep = mcb200_epilogue();
  KERNEL_CHECK(mcb200_channel_affine_act(x, y, bottom[0]->count(), channels_, inner, scale, shift, &ep,
                                         ctx.stream_ptr()));
}

REGISTER_LAYER_CLASS(BatchNorm);

// ---------------------------------------------------------------- Scale / Bias

// Shape of a factor blob that spans `num_axes` axes of bottom[0] from `axis` on (-1: to the end).
static vector<int> BroadcastShape(const Blob& bottom, int axis, int num_axes, const char* what) {
  CHECK_GE(num_axes, -1) << "num_axes must be non-negative, or -1 to extend to the end of bottom[0]";
  if (num_axes == -1) return vector<int>(bottom.shape().begin() + axis, bottom.shape().end());
  CHECK_GE(bottom.num_axes(), axis + num_axes)
      << what << " blob's shape extends past bottom[0]'s shape when applied starting with bottom[0] axis = " << axis;
  return vector<int>(bottom.shape().begin() + axis, bottom.shape().begin() + axis + num_axes);
}

// Checks that `factors` matches bottom[0]'s axes from `axis` on and returns (dim, inner) of
// y[o, d, i] = f(x[o, d, i], factors[d]).  A blob without axes applies to everything (axis 0).
static void BroadcastDims(const Blob& bottom, const Blob& factors, int* axis, int* dim, int* inner, const char* what) {
  if (factors.num_axes() == 0) *axis = 0;
  CHECK_GE(bottom.num_axes(), *axis + factors.num_axes())
      << what << " blob's shape extends past bottom[0]'s shape when applied starting with bottom[0] axis = " << *axis;
  for (int i = 0; i < factors.num_axes(); ++i) {
    CHECK_EQ(bottom.shape(*axis + i), factors.shape(i))
        << "dimension mismatch between bottom[0]->shape(" << *axis + i << ") and " << what << "->shape(" << i << ")";
  }
  *dim = factors.count();
  *inner = bottom.count(*axis + factors.num_axes());
}

void ScaleLayer::LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  const ScaleParameter& p = layer_param_.scale_param();
  bias_term_ = p.bias_term();
  const int axis = bottom[0]->CanonicalAxisIndex(p.axis());
  const bool learned = bottom.size() == 1;
  // The factors: a learned blob over `num_axes` axes, or the second bottom.  The optional bias is
  // always learned and has the factors' shape (src/layers/scale_layer.cpp:13-61).
  const vector<int> bias_shape = learned ? BroadcastShape(*bottom[0], axis, p.num_axes(), "scale")
                                         : BroadcastShape(*bottom[0], axis, bottom[1]->num_axes(), "scale");
  if (blobs_.empty()) {
    if (learned) {
      blobs_.emplace_back(new Blob(bias_shape));
      FillerParameter filler(p.filler());
      if (!p.has_filler()) {
        filler.set_type("constant");
        filler.set_value(1);
      }
      FillBlob(filler, blobs_[0].get());
    }
    if (bias_term_) {
      blobs_.emplace_back(new Blob(bias_shape));
      FillBlob(p.bias_filler(), blobs_.back().get());
    }
  } else {
    CHECK_EQ(blobs_.size(), static_cast<size_t>((learned ? 1 : 0) + (bias_term_ ? 1 : 0))) << "Incorrect number of Scale blobs";
  }
  per_channel_ = learned && axis == 1 && blobs_[0]->num_axes() == 1;
  scalar_ = learned && blobs_[0]->num_axes() == 0;
  general_ = !(per_channel_ || scalar_);
}

void ScaleLayer::Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  if (per_channel_) {
    CHECK_EQ(bottom[0]->shape(1), blobs_[0]->shape(0)) << "dimension mismatch between bottom[0]->shape(1) and scale->shape(0)";
  }
  if (general_) {
    axis_ = bottom[0]->CanonicalAxisIndex(layer_param_.scale_param().axis());
    BroadcastDims(*bottom[0], bottom.size() > 1 ? *bottom[1] : *blobs_[0], &axis_, &scale_dim_, &inner_dim_, "scale");
  }
  ChannelwiseLayer::Reshape(bottom, top);
}

bool ScaleLayer::AsChannelAffine(int channels, std::vector<double>* scale, std::vector<double>* shift) {
  if (general_) return false;
  if (per_channel_ && blobs_[0]->count() != channels) return false;
  if (!scale) return true;
  const float* g = blobs_[0]->cpu_data();
  const float* b = bias_term_ ? blobs_[1]->cpu_data() : nullptr;
  scale->resize(channels);
  shift->resize(channels);
  for (int c = 0; c < channels; ++c) {
    (*scale)[c] = g[per_channel_ ? c : 0];
    (*shift)[c] = b ? b[per_channel_ ? c : 0] : 0.0;
  }
  return true;
}

void ScaleLayer::Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  if (!general_) {
    ChannelwiseLayer::Forward_gpu(bottom, top);
    return;
  }
  if (bottom[0]->count() == 0) return;
  Context& ctx = Context::Get();
  const float* factors = bottom.size() > 1 ? bottom[1]->gpu_data() : blobs_[0]->gpu_data();
  const float* bias = bias_term_ ? blobs_.back()->gpu_data() : nullptr;
  const float* x = bottom[0]->gpu_data();
  float* y = top[0]->mutable_gpu_data();
  mcb200_epilogue ep = mcb200_epilogue();
  KERNEL_CHECK(mcb200_channel_affine_act(x, y, bottom[0]->count(), scale_dim_, inner_dim_, factors, bias, &ep,
                                         ctx.stream_ptr()));
}

REGISTER_LAYER_CLASS(Scale);

void BiasLayer::LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  const BiasParameter& p = layer_param_.bias_param();
  const int axis = bottom[0]->CanonicalAxisIndex(p.axis());
  const bool learned = bottom.size() == 1;
  if (learned && blobs_.empty()) {
    blobs_.resize(1);
    blobs_[0].reset(new Blob(BroadcastShape(*bottom[0], axis, p.num_axes(), "bias")));
    FillBlob(p.filler(), blobs_[0].get());
  }
  per_channel_ = learned && axis == 1 && blobs_[0]->num_axes() == 1;
  scalar_ = learned && blobs_[0]->num_axes() == 0;
  general_ = !(per_channel_ || scalar_);
}

void BiasLayer::Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  if (per_channel_) {
    CHECK_EQ(bottom[0]->shape(1), blobs_[0]->shape(0)) << "dimension mismatch between bottom[0]->shape(1) and bias->shape(0)";
  }
  if (general_) {
    axis_ = bottom[0]->CanonicalAxisIndex(layer_param_.bias_param().axis());
    BroadcastDims(*bottom[0], bottom.size() > 1 ? *bottom[1] : *blobs_[0], &axis_, &bias_dim_, &inner_dim_, "bias");
  }
  ChannelwiseLayer::Reshape(bottom, top);
}

bool BiasLayer::AsChannelAffine(int channels, std::vector<double>* scale, std::vector<double>* shift) {
  if (general_) return false;
  if (per_channel_ && blobs_[0]->count() != channels) return false;
  if (!scale) return true;
  const float* b = blobs_[0]->cpu_data();
  scale->assign(channels, 1.0);
  shift->resize(channels);
  for (int c = 0; c < channels; ++c) (*shift)[c] = b[per_channel_ ? c : 0];
  return true;
}

void BiasLayer::Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  if (!general_) {
    ChannelwiseLayer::Forward_gpu(bottom, top);
    return;
  }
  if (bottom[0]->count() == 0) return;
  Context& ctx = Context::Get();
  const float* offsets = bottom.size() > 1 ? bottom[1]->gpu_data() : blobs_[0]->gpu_data();
  mcb200_epilogue ep = mcb200_epilogue();
  KERNEL_CHECK(mcb200_channel_affine_act(bottom[0]->gpu_data(), top[0]->mutable_gpu_data(), bottom[0]->count(), bias_dim_,
                                         inner_dim_, nullptr, offsets, &ep, ctx.stream_ptr()));
}

REGISTER_LAYER_CLASS(Bias);

// ---------------------------------------------------------------- ReLU / PReLU / Dropout

// y = max(x, 0) + slope * min(x, 0) (src/layers/relu_layer.cpp:12-29).
bool ReLULayer::AsActivation(ActivationSpec* spec) {
  spec->kind = 1;
  spec->slope = layer_param_.relu_param().negative_slope();
  return true;
}
REGISTER_LAYER_CLASS(ReLU);

void PReLULayer::LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  CHECK_GE(bottom[0]->num_axes(), 2) << "Number of axes of bottom blob must be >=2.";
  const PReLUParameter& p = layer_param_.prelu_param();
  const int channels = bottom[0]->shape(1);
  channel_shared_ = p.channel_shared();
  if (blobs_.empty()) {
    blobs_.resize(1);
    blobs_[0].reset(new Blob(channel_shared_ ? vector<int>() : vector<int>(1, channels)));
    FillerParameter filler(p.filler());
    if (!p.has_filler()) {
      filler.set_type("constant");
      filler.set_value(0.25f);
    }
    FillBlob(filler, blobs_[0].get());
  }
  CHECK_EQ(blobs_[0]->count(), channel_shared_ ? 1 : channels)
      << "Negative slope size is inconsistent with prototxt config";
}

bool PReLULayer::AsActivation(ActivationSpec* spec) {
  spec->kind = 2;
  spec->slopes = blobs_[0].get();
  spec->shared = channel_shared_;
  return true;
}
REGISTER_LAYER_CLASS(PReLU);

REGISTER_LAYER_CLASS(Dropout);

// ---------------------------------------------------------------- Eltwise

void EltwiseLayer::LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  const EltwiseParameter& p = layer_param_.eltwise_param();
  CHECK(p.coeff_size() == 0 || p.coeff_size() == static_cast<int>(bottom.size()))
      << "Eltwise Layer takes one coefficient per bottom blob.";
  CHECK(!(p.operation() == EltwiseParameter_EltwiseOp_PROD && p.coeff_size()))
      << "Eltwise layer only takes coefficients for summation.";
  switch (p.operation()) {
    case EltwiseParameter_EltwiseOp_PROD: op_ = MCB200_ELTWISE_PROD; break;
    case EltwiseParameter_EltwiseOp_SUM: op_ = MCB200_ELTWISE_SUM; break;
    case EltwiseParameter_EltwiseOp_MAX: op_ = MCB200_ELTWISE_MAX; break;
    default: LOG(FATAL) << "Unknown elementwise operation.";
  }
  coeffs_.assign(bottom.size(), 1.f);
  for (int i = 0; i < p.coeff_size(); ++i) coeffs_[i] = p.coeff(i);
  CHECK_LE(bottom.size(), static_cast<size_t>(MCB200_MAX_ELTWISE_INPUTS))
      << "Eltwise: at most " << MCB200_MAX_ELTWISE_INPUTS << " bottoms are supported";
}

void EltwiseLayer::Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  for (size_t i = 1; i < bottom.size(); ++i) CHECK(bottom[i]->shape() == bottom[0]->shape());
  top[0]->ReshapeLike(*bottom[0]);
}

bool EltwiseLayer::AsWeightedSum(std::vector<float>* coeffs) {
  if (op_ != MCB200_ELTWISE_SUM) return false;
  if (coeffs) *coeffs = coeffs_;
  return true;
}

void EltwiseLayer::Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  Context& ctx = Context::Get();
  bool nhwc = false;
  for (Blob* b : bottom) nhwc = nhwc || b->device_is_nhwc();
  const float* in[MCB200_MAX_ELTWISE_INPUTS];
  for (size_t i = 0; i < bottom.size(); ++i) in[i] = nhwc ? bottom[i]->gpu_data_nhwc() : bottom[i]->gpu_data();
  float* out = nhwc ? top[0]->mutable_gpu_data_nhwc() : top[0]->mutable_gpu_data();
  KERNEL_CHECK(mcb200_eltwise(op_, static_cast<int>(bottom.size()), in, coeffs_.data(), out, top[0]->count(), 0, 0.f,
                              ctx.stream_ptr()));
}

REGISTER_LAYER_CLASS(Eltwise);

}  // namespace caffe
