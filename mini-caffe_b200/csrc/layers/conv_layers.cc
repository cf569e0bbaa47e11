// Convolution and InnerProduct: parameter handling on the host, tensor-core /
// depthwise / direct kernels on the device, fused tails folded into
// per-channel scale and shift arrays.
#include <cstdlib>
#include <cstring>

#include "../filler.h"
#include "layers.h"

namespace caffe {

// ---------------------------------------------------------------- helpers

void DeviceArray::Assign(const std::vector<float>& host) {
  if (!blob_ || blob_->count() != static_cast<int>(host.size())) {
    blob_.reset(new Blob(vector<int>(1, static_cast<int>(host.size()))));
  }
  std::memcpy(blob_->mutable_cpu_data(), host.data(), host.size() * sizeof(float));
}

float* DeviceScratch::Reserve(size_t floats) {
  CHECK_LE(floats, static_cast<size_t>(0x7fffffff));
  if (!blob_ || static_cast<size_t>(blob_->count()) < floats) {
    blob_.reset(new Blob(vector<int>(1, static_cast<int>(floats ? floats : 1))));
  }
  return blob_->mutable_gpu_data();
}

unsigned long long TailVersion(const FusedTail& tail) {
  unsigned long long v = 0;
  for (Layer* l : tail.affine) v += l->ParamVersion();
  return v;
}

void FoldTail(const FusedTail& tail, int channels, const float* bias, std::vector<float>* scale,
              std::vector<float>* shift, bool* has_scale, bool* has_shift) {
  std::vector<double> s(channels, 1.0), b(channels, 0.0);
  *has_scale = false;
  *has_shift = false;
  if (bias) {
    for (int c = 0; c < channels; ++c) b[c] = bias[c];
    *has_shift = true;
  }
  for (Layer* l : tail.affine) {
    std::vector<double> ls, lb;
    CHECK(l->AsChannelAffine(channels, &ls, &lb)) << l->type() << " layer cannot be folded";
    for (int c = 0; c < channels; ++c) {
      s[c] *= ls[c];
      b[c] = b[c] * ls[c] + lb[c];
    }
    *has_scale = true;
    *has_shift = true;
  }
  if (tail.self_coeff != 1.f) {
    for (int c = 0; c < channels; ++c) {
      s[c] *= tail.self_coeff;
      b[c] *= tail.self_coeff;
    }
    *has_scale = true;
  }
  scale->assign(s.begin(), s.end());
  shift->assign(b.begin(), b.end());
}

void FillTailEpilogue(const FusedTail& tail, const DeviceArray& scale, const DeviceArray& shift,
                      ResidualCopy residual_copy, int channels, mcb200_epilogue* ep) {
  *ep = mcb200_epilogue();
  ep->scale = scale.get();
  ep->shift = shift.get();
  ep->residual_coeff = 1.f;
  if (tail.residual) {
    ep->residual = residual_copy == kResidualNhwcHalf
                       ? static_cast<const float*>(tail.residual->gpu_data_nhwc_bf16())   // 16-bit cells
                       : (residual_copy == kResidualNhwc ? tail.residual->gpu_data_nhwc() : tail.residual->gpu_data());
    ep->residual_ld = channels;
    ep->residual_coeff = tail.residual_coeff;
  }
  if (tail.activation) {
    ActivationSpec spec;
    CHECK(tail.activation->AsActivation(&spec));
    ep->act = spec.kind;
    ep->slope = spec.slope;
    if (spec.kind == 2) {
      ep->prelu = spec.slopes->gpu_data();
      ep->prelu_shared = spec.shared ? 1 : 0;
    }
  }
}

// ---------------------------------------------------------------- Convolution

// Kernel, stride, pad and dilation of a 2-D convolution from either the _h/_w
// fields or the repeated fields (src/layers/base_conv_layer.cpp:22-88, same rules
// and messages).
void ParseConvolutionGeometry(const ConvolutionParameter& p, mcb200_conv_shape* shape) {
  mcb200_conv_shape& s = *shape;
  auto pick = [&](bool has_h, bool has_w, int vh, int vw, int rep_size, const char* what, int dflt, int* oh, int* ow,
                  auto rep) {
    if (has_h || has_w) {
      CHECK_EQ(0, rep_size) << "Either " << what << " or " << what << "_h/w should be specified; not both.";
      *oh = vh;
      *ow = vw;
    } else {
      CHECK(rep_size == 0 || rep_size == 1 || rep_size == 2)
          << what << " must be specified once, or once per spatial dimension (" << what << " specified " << rep_size
          << " times; 2 spatial dims).";
      *oh = rep_size == 0 ? dflt : static_cast<int>(rep(0));
      *ow = rep_size == 0 ? dflt : static_cast<int>(rep(rep_size == 1 ? 0 : 1));
    }
  };
  CHECK(p.has_kernel_h() || p.has_kernel_w() || p.kernel_size_size() > 0) << "kernel_size must be specified";
  pick(p.has_kernel_h(), p.has_kernel_w(), p.kernel_h(), p.kernel_w(), p.kernel_size_size(), "kernel_size", 0, &s.kh,
       &s.kw, [&](int i) { return p.kernel_size(i); });
  CHECK_GT(s.kh, 0) << "Filter dimensions must be nonzero.";
  CHECK_GT(s.kw, 0) << "Filter dimensions must be nonzero.";
  pick(p.has_stride_h(), p.has_stride_w(), p.stride_h(), p.stride_w(), p.stride_size(), "stride", 1, &s.stride_h,
       &s.stride_w, [&](int i) { return p.stride(i); });
  CHECK_GT(s.stride_h, 0) << "Stride dimensions must be nonzero.";
  CHECK_GT(s.stride_w, 0) << "Stride dimensions must be nonzero.";
  pick(p.has_pad_h(), p.has_pad_w(), p.pad_h(), p.pad_w(), p.pad_size(), "pad", 0, &s.pad_h, &s.pad_w,
       [&](int i) { return p.pad(i); });
  pick(false, false, 0, 0, p.dilation_size(), "dilation", 1, &s.dil_h, &s.dil_w, [&](int i) { return p.dilation(i); });
  CHECK_GT(s.dil_h, 0);
  CHECK_GT(s.dil_w, 0);

}

void ConvolutionLayer::LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  const ConvolutionParameter& p = layer_param_.convolution_param();
  const int channel_axis = bottom[0]->CanonicalAxisIndex(p.axis());
  const int spatial_axes = bottom[0]->num_axes() - channel_axis - 1;
  CHECK(channel_axis == 1 && spatial_axes == 2)
      << "this engine implements 2-D convolution over (N, C, H, W) blobs; got axis " << channel_axis << " with "
      << spatial_axes << " spatial axes";
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

  const vector<int> weight_shape = {s.cout, s.c / s.group, s.kh, s.kw};
  const vector<int> bias_shape(bias_term_ ? 1 : 0, s.cout);
  if (!blobs_.empty()) {
    CHECK_EQ(static_cast<size_t>(1 + (bias_term_ ? 1 : 0)), blobs_.size()) << "Incorrect number of weight blobs.";
    if (weight_shape != blobs_[0]->shape()) {
      Blob expected(weight_shape);
      LOG(FATAL) << "Incorrect weight shape: expected shape " << expected.shape_string() << "; instead, shape was "
                 << blobs_[0]->shape_string();
    }
    if (bias_term_ && bias_shape != blobs_[1]->shape()) {
      Blob expected(bias_shape);
      LOG(FATAL) << "Incorrect bias shape: expected shape " << expected.shape_string() << "; instead, shape was "
                 << blobs_[1]->shape_string();
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
  // Depthwise layers (one channel per group) are pure data movement and have a kernel of their
  // own; every other layer, grouped or not, is a contraction and runs on the tensor cores (a
  // grouped layer as block-diagonal weight tiles, src/layers/base_conv_layer.cpp:265-270).
  if (s.group > 1 && s.group == s.c && s.cout == s.c && s.c % 4 == 0) {
    path_ = kDepthwise;
  } else {
    path_ = kTensorCore;
  }
  const char* force_direct = getenv("MCB200_CONV_DIRECT");   // "1": the plain kernel, for comparisons in tests
  if (force_direct && force_direct[0] == '1' && path_ == kTensorCore) path_ = kDirect;
  // Limits of the im2col tensor map (8-bit signed corners, 8-bit tap offsets).
  if (path_ == kTensorCore && (s.pad_h > 127 || s.pad_w > 127 || (s.kh - 1) * s.dil_h > 255 ||
                               (s.kw - 1) * s.dil_w > 255)) {
    path_ = kDirect;
  }
}

void ConvolutionLayer::Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  CHECK_EQ(4, bottom[0]->num_axes()) << "Convolution input must be (N, C, H, W)";
  for (size_t i = 1; i < bottom.size(); ++i) {
    CHECK(bottom[0]->shape() == bottom[i]->shape()) << "All inputs must have the same shape.";
  }
  CHECK_EQ(bottom[0]->shape(1), shape_.c) << "Input size incompatible with convolution kernel.";
  shape_.n = bottom[0]->shape(0);
  shape_.h = bottom[0]->shape(2);
  shape_.w = bottom[0]->shape(3);
  CHECK_EQ(mcb200_conv_out_shape(&shape_), 0) << "convolution window larger than the padded input";
  // Few input channels (an image in front of the first layer): one filter row per k-iteration.
  const bool rows = path_ == kTensorCore && !rows_rejected_ && mcb200_conv_rows_supported(&shape_) != 0;
  if (rows != use_rows_) {
    use_rows_ = rows;
    weight_version_ = 0;   // the packed weight image differs between the two modes
  }
  for (size_t i = 0; i < top.size(); ++i) top[i]->Reshape(shape_.n, shape_.cout, shape_.ho, shape_.wo);
}

void ConvolutionLayer::RefreshParameters() {
  Context& ctx = Context::Get();
  const unsigned long long wv = blobs_[0]->host_version();
  if (wv != weight_version_) {
    if (path_ == kTensorCore && use_rows_) {
      float* packed = packed_weights_.Reserve(mcb200_conv_rows_packed_weight_count(&shape_));
      KERNEL_CHECK(mcb200_conv_rows_pack_weights(&shape_, blobs_[0]->gpu_data(), packed, ctx.stream_ptr()));
    } else if (path_ == kTensorCore && half_operands_) {
      float* packed = packed_weights_.Reserve((mcb200_conv_packed_weight_count_bf16(&shape_) + 1) / 2);
      KERNEL_CHECK(mcb200_conv_pack_weights_bf16(&shape_, blobs_[0]->gpu_data(), reinterpret_cast<uint16_t*>(packed),
                                                 ctx.stream_ptr()));
    } else if (path_ == kTensorCore) {
      float* packed = packed_weights_.Reserve(mcb200_conv_packed_weight_count(&shape_));
      KERNEL_CHECK(mcb200_conv_pack_weights(&shape_, blobs_[0]->gpu_data(), packed, ctx.stream_ptr()));
    } else if (path_ == kDepthwise) {
      float* packed = packed_weights_.Reserve(static_cast<size_t>(shape_.c) * shape_.kh * shape_.kw);
      KERNEL_CHECK(mcb200_dw_pack_weights(&shape_, blobs_[0]->gpu_data(), packed, ctx.stream_ptr()));
    }
    weight_version_ = wv;
    for (auto& slot : plans_) {
      if (slot) slot->valid = false;
    }
  }
  const unsigned long long tv = 1 + TailVersion(tail_) + (bias_term_ ? blobs_[1]->host_version() : 0);
  if (tv != tail_version_) {
    std::vector<float> scale, shift;
    bool has_scale = false, has_shift = false;
    FoldTail(tail_, shape_.cout, bias_term_ ? blobs_[1]->cpu_data() : nullptr, &scale, &shift, &has_scale,
             &has_shift);
    if (has_scale) scale_.Assign(scale); else scale_.Clear();
    if (has_shift) shift_.Assign(shift); else shift_.Clear();
    tail_version_ = tv;
  }
}

void ConvolutionLayer::Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  Context& ctx = Context::Get();
  RefreshParameters();
  if (plans_.size() < bottom.size()) plans_.resize(bottom.size());
  for (size_t i = 0; i < bottom.size(); ++i) {
    mcb200_conv_shape s = shape_;
    const float* in = nullptr;
    const bool half = half_operands_ && HalfOperandsCapable();
    if (half) {
      s.c_stride = s.c;
      in = static_cast<const float*>(bottom[i]->gpu_data_nhwc_bf16());   // 16-bit cells
    } else if (path_ == kTensorCore && use_rows_) {
      int hp = 0, wp = 0;
      CHECK_EQ(mcb200_conv_rows_padded_dims(&s, &hp, &wp), 0);
      s.c_stride = 4;
      float* padded = padded_input_.Reserve(static_cast<size_t>(s.n) * hp * wp * 4);
      KERNEL_CHECK(mcb200_conv_rows_pad_input(&s, bottom[i]->gpu_data(), padded, ctx.stream_ptr()));
      in = padded;
    } else if (shape_.c % 4 == 0) {
      s.c_stride = s.c;
      in = bottom[i]->gpu_data_nhwc();
    } else {
      // Pad the channels to a multiple of four (16-byte pixels) in a private
      // channels-last copy, e.g. the three colour planes of the first layer.
      s.c_stride = (s.c + 3) / 4 * 4;
      float* padded = padded_input_.Reserve(static_cast<size_t>(s.n) * s.h * s.w * s.c_stride);
      if (bottom[i]->device_is_nhwc()) {
        // The pad lanes meet zero weights but still have to be finite.
        CUDA_CHECK(cudaMemsetAsync(padded, 0, static_cast<size_t>(s.n) * s.h * s.w * s.c_stride * sizeof(float),
                                   ctx.stream()));
        KERNEL_CHECK(mcb200_copy_2d(bottom[i]->gpu_data_nhwc(), s.c, padded, s.c_stride,
                                    static_cast<long long>(s.n) * s.h * s.w, s.c, ctx.stream_ptr()));
      } else {
        KERNEL_CHECK(mcb200_nchw_to_nhwc(bottom[i]->gpu_data(), padded, s.n, s.c, s.h, s.w, s.c_stride,
                                         ctx.stream_ptr()));
      }
      in = padded;
    }
    mcb200_epilogue ep;
    FillTailEpilogue(i == 0 ? tail_ : FusedTail(), scale_, shift_, half ? kResidualNhwcHalf : kResidualNhwc, s.cout,
                     &ep);
    const bool half_out = half_top_ && HalfTopCapable();
    float* out = half_out ? static_cast<float*>(top[i]->mutable_gpu_data_nhwc_bf16()) : top[i]->mutable_gpu_data_nhwc();
    if (path_ == kTensorCore) {
      if (!plans_[i]) plans_[i].reset(new PlanSlot);
      PlanSlot& slot = *plans_[i];
      const float* w = packed_weights_.Reserve(0);
      if (!slot.valid || slot.in != in || slot.weights != w || std::memcmp(&slot.shape, &s, sizeof(s)) != 0) {
        int rc = half ? mcb200_conv_tc_plan_bf16(&s, reinterpret_cast<const uint16_t*>(in),
                                                 reinterpret_cast<const uint16_t*>(w), &slot.plan)
                 : use_rows_ ? mcb200_conv_rows_plan(&s, in, w, &slot.plan)
                             : mcb200_conv_tc_plan(&s, in, w, &slot.plan);
        if (rc != 0 && use_rows_) {
          // The driver refused the row-mode tensor map: use the general path from now on.
          LOG(WARNING) << "layer " << layer_param_.name() << ": row-mode plan rejected (" << rc
                       << "), using the im2col path";
          rows_rejected_ = true;
          use_rows_ = false;
          weight_version_ = 0;
          Forward_gpu(bottom, top);
          return;
        }
        if (rc != 0 && !half && !half_out) {
          // A shape the tensor maps cannot express (for instance a stride above 8, which the
          // im2col map refuses as traversal stride): the plain kernel runs it from now on.
          LOG(WARNING) << "layer " << layer_param_.name() << ": tensor-core plan rejected (" << rc
                       << "), using the direct kernel";
          path_ = kDirect;
          Forward_gpu(bottom, top);
          return;
        }
        CHECK_EQ(rc, 0) << "cannot build the tensor-core plan for layer " << layer_param_.name();
        slot.in = in;
        slot.weights = w;
        slot.shape = s;
        slot.valid = true;
      }
      if (half || half_out) {
        KERNEL_CHECK(mcb200_conv_tc_launch_bf16(&slot.plan, out, half_out ? 1 : 0, s.cout, &ep, ctx.status_word(),
                                                ctx.stream_ptr()));
      } else {
        KERNEL_CHECK(mcb200_conv_tc_launch(&slot.plan, out, s.cout, &ep, ctx.status_word(), ctx.stream_ptr()));
      }
    } else if (path_ == kDepthwise && (half || half_out)) {
      KERNEL_CHECK(mcb200_conv_depthwise_bf16(&s, in, half ? 1 : 0, packed_weights_.Reserve(0), out, half_out ? 1 : 0,
                                              &ep, ctx.stream_ptr()));
    } else if (path_ == kDepthwise) {
      const char* dw_tma = getenv("MCB200_DW_TMA");   // "0": the register-window kernel, for comparisons
      // Outputs of 8 x 8 pixels and more: the TMA-staged kernel's 8 x 16 tiles; on smaller maps
      // (the 7 x 7 end of MobileNet) most of a tile is outside the image and the register-window
      // kernel is quicker (11 / 14 us against 15 / 18 us at batch 64).  The rule looks at the
      // layer's geometry only, never at the batch.
      const bool roomy = s.ho >= 8 && s.wo >= 8;
      if (!ep.residual && roomy && mcb200_conv_depthwise_tma_supported(&s) && !(dw_tma && dw_tma[0] == '0')) {
        KERNEL_CHECK(mcb200_conv_depthwise_tma(&s, in, packed_weights_.Reserve(0), out, &ep, ctx.status_word(),
                                               ctx.stream_ptr()));
      } else {
        KERNEL_CHECK(mcb200_conv_depthwise(&s, in, packed_weights_.Reserve(0), out, &ep, ctx.stream_ptr()));
      }
    } else {
      KERNEL_CHECK(mcb200_conv_direct(&s, in, blobs_[0]->gpu_data(), out, s.cout, &ep, ctx.stream_ptr()));
    }
  }
}

static shared_ptr<Layer> CreateConvolution(const LayerParameter& param) {
  return shared_ptr<Layer>(new ConvolutionLayer(param));
}
REGISTER_LAYER_CREATOR(Convolution, CreateConvolution);
// The reference registers its depthwise kernel under its own type name as
// well (src/layers/conv_dw_layer.cpp:158); here the one class picks the path.
REGISTER_LAYER_CREATOR(ConvolutionDepthwise, CreateConvolution);

// ---------------------------------------------------------------- InnerProduct

void InnerProductLayer::LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  const InnerProductParameter& p = layer_param_.inner_product_param();
  N_ = static_cast<int>(p.num_output());
  bias_term_ = p.bias_term();
  transpose_ = p.transpose();
  const int axis = bottom[0]->CanonicalAxisIndex(p.axis());
  K_ = bottom[0]->count(axis);
  if (blobs_.empty()) {
    blobs_.resize(bias_term_ ? 2 : 1);
    blobs_[0].reset(new Blob(transpose_ ? vector<int>{K_, N_} : vector<int>{N_, K_}));
    FillBlob(p.weight_filler(), blobs_[0].get());
    if (bias_term_) {
      blobs_[1].reset(new Blob(vector<int>(1, N_)));
      FillBlob(p.bias_filler(), blobs_[1].get());
    }
  }
}

void InnerProductLayer::Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  const int axis = bottom[0]->CanonicalAxisIndex(layer_param_.inner_product_param().axis());
  CHECK_EQ(K_, bottom[0]->count(axis)) << "Input size incompatible with inner product parameters.";
  M_ = bottom[0]->count(0, axis);
  vector<int> top_shape = bottom[0]->shape();
  top_shape.resize(axis + 1);
  top_shape[axis] = N_;
  top[0]->Reshape(top_shape);
}

void InnerProductLayer::Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  Context& ctx = Context::Get();
  mcb200_conv_shape s = mcb200_conv_shape();
  s.n = M_;
  s.h = s.w = 1;
  s.c = s.c_stride = K_;
  s.cout = N_;
  s.kh = s.kw = s.stride_h = s.stride_w = s.dil_h = s.dil_w = s.group = 1;
  s.ho = s.wo = 1;
  const bool tensor_core = (K_ % 4 == 0);

  // Weights as [N, K] rows (transpose: stored [K, N], re-laid on the host).
  const unsigned long long wv = blobs_[0]->host_version();
  const float* w_rows = nullptr;
  if (transpose_) {
    if (wv != weight_version_) {
      std::vector<float> rows(static_cast<size_t>(N_) * K_);
      const float* src = blobs_[0]->cpu_data();
      for (int k = 0; k < K_; ++k)
        for (int n = 0; n < N_; ++n) rows[static_cast<size_t>(n) * K_ + k] = src[static_cast<size_t>(k) * N_ + n];
      float* staged = staged_weights_.Reserve(rows.size());
      CUDA_CHECK(cudaMemcpyAsync(staged, rows.data(), rows.size() * sizeof(float), cudaMemcpyHostToDevice,
                                 ctx.stream()));
      ctx.Sync();  // `rows` is pageable and dies with this scope
    }
    w_rows = staged_weights_.Reserve(0);
  } else {
    w_rows = blobs_[0]->gpu_data();
  }
  if (wv != weight_version_) {
    if (tensor_core) {
      float* packed = packed_weights_.Reserve(mcb200_conv_packed_weight_count(&s));
      KERNEL_CHECK(mcb200_conv_pack_weights(&s, w_rows, packed, ctx.stream_ptr()));
    }
    weight_version_ = wv;
    plan_in_ = nullptr;
  }
  const unsigned long long tv = 1 + TailVersion(tail_) + (bias_term_ ? blobs_[1]->host_version() : 0);
  if (tv != tail_version_) {
    std::vector<float> scale, shift;
    bool has_scale = false, has_shift = false;
    FoldTail(tail_, N_, bias_term_ ? blobs_[1]->cpu_data() : nullptr, &scale, &shift, &has_scale, &has_shift);
    if (has_scale) scale_.Assign(scale); else scale_.Clear();
    if (has_shift) shift_.Assign(shift); else shift_.Clear();
    tail_version_ = tv;
  }
  // Rows of the (N, C, H, W)-ordered input are the K-vectors.
  const float* in = bottom[0]->gpu_data();
  mcb200_epilogue ep;
  FillTailEpilogue(tail_, scale_, shift_, kResidualNchw, N_, &ep);
  float* out = top[0]->mutable_gpu_data();
  if (tensor_core) {
    if (!plan_) {
      plan_storage_.reset(new char[sizeof(mcb200_conv_plan) + 64]);
      uintptr_t a = (reinterpret_cast<uintptr_t>(plan_storage_.get()) + 63) & ~static_cast<uintptr_t>(63);
      plan_ = reinterpret_cast<mcb200_conv_plan*>(a);
    }
    const float* w = packed_weights_.Reserve(0);
    if (plan_in_ != in || plan_w_ != w || plan_m_ != M_) {
      CHECK_EQ(mcb200_conv_tc_plan(&s, in, w, plan_), 0) << "cannot build the tensor-core plan for layer "
                                                         << layer_param_.name();
      plan_in_ = in;
      plan_w_ = w;
      plan_m_ = M_;
    }
    KERNEL_CHECK(mcb200_conv_tc_launch(plan_, out, N_, &ep, ctx.status_word(), ctx.stream_ptr()));
  } else {
    KERNEL_CHECK(mcb200_conv_direct(&s, in, w_rows, out, N_, &ep, ctx.stream_ptr()));
  }
}

REGISTER_LAYER_CLASS(InnerProduct);

}  // namespace caffe
