// Pooling, Softmax and Normalize.
#include <cmath>

#include "../filler.h"
#include "layers.h"

namespace caffe {

// ---------------------------------------------------------------- Pooling

void PoolingLayer::LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  const PoolingParameter& p = layer_param_.pooling_param();
  global_ = p.global_pooling();
  if (global_) {
    CHECK(!(p.has_kernel_size() || p.has_kernel_h() || p.has_kernel_w()))
        << "With Global_pooling: true Filter size cannot specified";
  } else {
    CHECK(!p.has_kernel_size() != !(p.has_kernel_h() && p.has_kernel_w()))
        << "Filter size is kernel_size OR kernel_h and kernel_w; not both";
    CHECK(p.has_kernel_size() || (p.has_kernel_h() && p.has_kernel_w()))
        << "For non-square filters both kernel_h and kernel_w are required.";
  }
  CHECK((!p.has_pad() && p.has_pad_h() && p.has_pad_w()) || (!p.has_pad_h() && !p.has_pad_w()))
      << "pad is pad OR pad_h and pad_w are required.";
  CHECK((!p.has_stride() && p.has_stride_h() && p.has_stride_w()) || (!p.has_stride_h() && !p.has_stride_w()))
      << "Stride is stride OR stride_h and stride_w are required.";
  if (global_) {
    kernel_h_ = bottom[0]->height();
    kernel_w_ = bottom[0]->width();
  } else if (p.has_kernel_size()) {
    kernel_h_ = kernel_w_ = p.kernel_size();
  } else {
    kernel_h_ = p.kernel_h();
    kernel_w_ = p.kernel_w();
  }
  CHECK_GT(kernel_h_, 0) << "Filter dimensions cannot be zero.";
  CHECK_GT(kernel_w_, 0) << "Filter dimensions cannot be zero.";
  if (!p.has_pad_h()) {
    pad_h_ = pad_w_ = p.pad();
  } else {
    pad_h_ = p.pad_h();
    pad_w_ = p.pad_w();
  }
  if (!p.has_stride_h()) {
    stride_h_ = stride_w_ = p.stride();
  } else {
    stride_h_ = p.stride_h();
    stride_w_ = p.stride_w();
  }
  if (global_) {
    CHECK(pad_h_ == 0 && pad_w_ == 0 && stride_h_ == 1 && stride_w_ == 1)
        << "With Global_pooling: true; only pad = 0 and stride = 1";
  }
  switch (p.pool()) {
    case PoolingParameter_PoolMethod_MAX: method_ = MCB200_POOL_MAX; break;
    case PoolingParameter_PoolMethod_AVE: method_ = MCB200_POOL_AVE; break;
    default: LOG(FATAL) << "Unknown pooling method.";
  }
  if (pad_h_ != 0 || pad_w_ != 0) {
    CHECK_LT(pad_h_, kernel_h_);
    CHECK_LT(pad_w_, kernel_w_);
  }
}

void PoolingLayer::Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  CHECK_EQ(4, bottom[0]->num_axes()) << "Input must have 4 axes, corresponding to (num, channels, height, width)";
  if (global_) {
    kernel_h_ = bottom[0]->height();
    kernel_w_ = bottom[0]->width();
  }
  mcb200_pool_out_shape(bottom[0]->height(), bottom[0]->width(), kernel_h_, kernel_w_, stride_h_, stride_w_, pad_h_,
                        pad_w_, &pooled_h_, &pooled_w_);
  if (pad_h_ || pad_w_) {
    CHECK_LT((pooled_h_ - 1) * stride_h_, bottom[0]->height() + pad_h_);
    CHECK_LT((pooled_w_ - 1) * stride_w_, bottom[0]->width() + pad_w_);
  }
  top[0]->Reshape(bottom[0]->num(), bottom[0]->channels(), pooled_h_, pooled_w_);
  channels_ = bottom[0]->channels();
}

void PoolingLayer::Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  Context& ctx = Context::Get();
  if (half_ && HalfOperandsCapable()) {
    const uint16_t* in16 = static_cast<const uint16_t*>(bottom[0]->gpu_data_nhwc_bf16());
    uint16_t* out16 = static_cast<uint16_t*>(top[0]->mutable_gpu_data_nhwc_bf16());
    KERNEL_CHECK(mcb200_pool_max_nhwc_bf16(in16, out16, bottom[0]->num(), bottom[0]->height(), bottom[0]->width(),
                                           bottom[0]->channels(), kernel_h_, kernel_w_, stride_h_, stride_w_, pad_h_,
                                           pad_w_, pooled_h_, pooled_w_, ctx.stream_ptr()));
    return;
  }
  const float* in = bottom[0]->gpu_data_nhwc();
  float* out = top[0]->mutable_gpu_data_nhwc();
  KERNEL_CHECK(mcb200_pool_nhwc(in, out, bottom[0]->num(), bottom[0]->height(), bottom[0]->width(),
                                bottom[0]->channels(), kernel_h_, kernel_w_, stride_h_, stride_w_, pad_h_, pad_w_,
                                pooled_h_, pooled_w_, method_, ctx.stream_ptr()));
}

REGISTER_LAYER_CLASS(Pooling);

// ---------------------------------------------------------------- Softmax

void SoftmaxLayer::Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  axis_ = bottom[0]->CanonicalAxisIndex(layer_param_.softmax_param().axis());
  top[0]->ReshapeLike(*bottom[0]);
}

void SoftmaxLayer::Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  Context& ctx = Context::Get();
  const int channels = bottom[0]->shape(axis_);
  if (axis_ == 1 && bottom[0]->num_axes() <= 4 && bottom[0]->device_is_nhwc()) {
    // Channels-last data: every pixel's channels are one contiguous row.
    const float* in = bottom[0]->gpu_data_nhwc();
    float* out = top[0]->mutable_gpu_data_nhwc();
    KERNEL_CHECK(mcb200_softmax(in, out, bottom[0]->count() / channels, channels, 1, ctx.stream_ptr()));
    return;
  }
  const float* in = bottom[0]->gpu_data();
  float* out = top[0]->mutable_gpu_data();
  KERNEL_CHECK(mcb200_softmax(in, out, bottom[0]->count(0, axis_), channels, bottom[0]->count(axis_ + 1),
                              ctx.stream_ptr()));
}

REGISTER_LAYER_CLASS(Softmax);

// ---------------------------------------------------------------- Normalize

void NormalizeLayer::LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  CHECK_GE(bottom[0]->num_axes(), 2) << "Number of axes of bottom blob must be >=2.";
  const NormalizeParameter& p = layer_param_.norm_param();
  across_spatial_ = p.across_spatial();
  channel_shared_ = p.channel_shared();
  eps_ = p.eps();
  const int channels = bottom[0]->channels();
  if (blobs_.empty()) {
    blobs_.resize(1);
    blobs_[0].reset(new Blob(channel_shared_ ? vector<int>() : vector<int>(1, channels)));
    FillerParameter filler(p.scale_filler());
    if (!p.has_scale_filler()) {
      filler.set_type("constant");
      filler.set_value(1.0f);
    }
    FillBlob(filler, blobs_[0].get());
  }
  CHECK_EQ(blobs_[0]->count(), channel_shared_ ? 1 : channels) << "Scale size is inconsistent with prototxt config";
}

void NormalizeLayer::Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  CHECK_GE(bottom[0]->num_axes(), 2) << "Number of axes of bottom blob must be >=2.";
  top[0]->ReshapeLike(*bottom[0]);
}

void NormalizeLayer::Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  Context& ctx = Context::Get();
  const int channels = bottom[0]->channels();
  if (across_spatial_) {
    // One norm per image: the image's C*H*W values form the "channel" row.
    const int dim = bottom[0]->count() / bottom[0]->num();
    CHECK(channel_shared_) << "Normalize: across_spatial with per-channel scale is not implemented in this engine";
    KERNEL_CHECK(mcb200_normalize_nhwc(bottom[0]->gpu_data(), top[0]->mutable_gpu_data(), bottom[0]->num(), dim,
                                       blobs_[0]->gpu_data(), 1, eps_, ctx.stream_ptr()));
    return;
  }
  const float* in = bottom[0]->gpu_data_nhwc();
  float* out = top[0]->mutable_gpu_data_nhwc();
  KERNEL_CHECK(mcb200_normalize_nhwc(in, out, static_cast<long long>(bottom[0]->count()) / channels, channels,
                                     blobs_[0]->gpu_data(), channel_shared_ ? 1 : 0, eps_, ctx.stream_ptr()));
}

REGISTER_LAYER_CLASS(Normalize);

}  // namespace caffe
