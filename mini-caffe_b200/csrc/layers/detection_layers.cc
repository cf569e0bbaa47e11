// PriorBox, Proposal and DetectionOutput: the detection tail.
#include <cfloat>
#include <cmath>
#include <cstring>

#include "layers.h"

namespace caffe {

// ---------------------------------------------------------------- PriorBox

void PriorBoxLayer::LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  const PriorBoxParameter& p = layer_param_.prior_box_param();
  CHECK_GT(p.min_size_size(), 0) << "must provide min_size.";
  for (int i = 0; i < p.min_size_size(); ++i) {
    min_sizes_.push_back(p.min_size(i));
    CHECK_GT(min_sizes_.back(), 0) << "min_size must be positive.";
  }
  aspect_ratios_.assign(1, 1.f);
  flip_ = p.flip();
  for (int i = 0; i < p.aspect_ratio_size(); ++i) {
    const float ar = p.aspect_ratio(i);
    bool seen = false;
    for (float have : aspect_ratios_) seen = seen || std::fabs(ar - have) < 1e-6;
    if (!seen) {
      aspect_ratios_.push_back(ar);
      if (flip_) aspect_ratios_.push_back(1. / ar);
    }
  }
  num_priors_ = static_cast<int>(aspect_ratios_.size() * min_sizes_.size());
  if (p.max_size_size() > 0) {
    CHECK_EQ(p.min_size_size(), p.max_size_size());
    for (int i = 0; i < p.max_size_size(); ++i) {
      max_sizes_.push_back(p.max_size(i));
      CHECK_GT(max_sizes_[i], min_sizes_[i]) << "max_size must be greater than min_size.";
      num_priors_ += 1;
    }
  }
  clip_ = p.clip();
  if (p.variance_size() > 1) {
    CHECK_EQ(p.variance_size(), 4);
    for (int i = 0; i < 4; ++i) {
      CHECK_GT(p.variance(i), 0);
      variance_.push_back(p.variance(i));
    }
  } else if (p.variance_size() == 1) {
    CHECK_GT(p.variance(0), 0);
    variance_.push_back(p.variance(0));
  } else {
    variance_.push_back(0.1);
  }
  if (p.has_img_h() || p.has_img_w()) {
    CHECK(!p.has_img_size()) << "Either img_size or img_h/img_w should be specified; not both.";
    img_h_ = p.img_h();
    CHECK_GT(img_h_, 0) << "img_h should be larger than 0.";
    img_w_ = p.img_w();
    CHECK_GT(img_w_, 0) << "img_w should be larger than 0.";
  } else if (p.has_img_size()) {
    CHECK_GT(p.img_size(), 0u) << "img_size should be larger than 0.";
    img_h_ = img_w_ = p.img_size();
  }
  if (p.has_step_h() || p.has_step_w()) {
    CHECK(!p.has_step()) << "Either step or step_h/step_w should be specified; not both.";
    step_h_ = p.step_h();
    CHECK_GT(step_h_, 0.) << "step_h should be larger than 0.";
    step_w_ = p.step_w();
    CHECK_GT(step_w_, 0.) << "step_w should be larger than 0.";
  } else if (p.has_step()) {
    CHECK_GT(p.step(), 0) << "step should be larger than 0.";
    step_h_ = step_w_ = p.step();
  }
  offset_ = p.offset();
}

void PriorBoxLayer::Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  const int dim = bottom[0]->width() * bottom[0]->height() * num_priors_ * 4;
  CHECK_GT(dim, 0);
  top[0]->Reshape(vector<int>{1, 2, dim});
}

// Same expression shapes as the reference (float centre, int-truncated sizes,
// `/ 2.` in double, one rounding to float per coordinate).
void PriorBoxLayer::Compute(int layer_h, int layer_w, int img_h, int img_w, float* out) const {
  float step_w, step_h;
  if (step_w_ == 0 || step_h_ == 0) {
    step_w = static_cast<float>(img_w) / layer_w;
    step_h = static_cast<float>(img_h) / layer_h;
  } else {
    step_w = step_w_;
    step_h = step_h_;
  }
  const int dim = layer_h * layer_w * num_priors_ * 4;
  int idx = 0;
  auto emit = [&](float cx, float cy, float bw, float bh) {
    out[idx++] = (cx - bw / 2.) / img_w;
    out[idx++] = (cy - bh / 2.) / img_h;
    out[idx++] = (cx + bw / 2.) / img_w;
    out[idx++] = (cy + bh / 2.) / img_h;
  };
  for (int h = 0; h < layer_h; ++h) {
    for (int w = 0; w < layer_w; ++w) {
      const float cx = (w + offset_) * step_w;
      const float cy = (h + offset_) * step_h;
      for (size_t s = 0; s < min_sizes_.size(); ++s) {
        const int min_size = static_cast<int>(min_sizes_[s]);
        float bw, bh;
        bw = bh = min_size;
        emit(cx, cy, bw, bh);
        if (!max_sizes_.empty()) {
          const int max_size = static_cast<int>(max_sizes_[s]);
          bw = bh = std::sqrt(static_cast<double>(min_size * max_size));
          emit(cx, cy, bw, bh);
        }
        for (float ar : aspect_ratios_) {
          if (std::fabs(ar - 1.) < 1e-6) continue;
          bw = min_size * std::sqrt(ar);
          bh = min_size / std::sqrt(ar);
          emit(cx, cy, bw, bh);
        }
      }
    }
  }
  CHECK_EQ(idx, dim);
  if (clip_) {
    for (int d = 0; d < dim; ++d) out[d] = std::min<float>(std::max<float>(out[d], 0.), 1.);
  }
  float* var = out + dim;
  if (variance_.size() == 1) {
    for (int d = 0; d < dim; ++d) var[d] = variance_[0];
  } else {
    for (int d = 0; d < dim; ++d) var[d] = variance_[d % 4];
  }
}

void PriorBoxLayer::Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  const int layer_w = bottom[0]->width(), layer_h = bottom[0]->height();
  const int img_w = (img_h_ == 0 || img_w_ == 0) ? bottom[1]->width() : img_w_;
  const int img_h = (img_h_ == 0 || img_w_ == 0) ? bottom[1]->height() : img_h_;
  const int key[4] = {layer_h, layer_w, img_h, img_w};
  if (std::memcmp(key, cached_key_, sizeof(key)) != 0) {
    cached_.resize(top[0]->count());
    Compute(layer_h, layer_w, img_h, img_w, cached_.data());
    std::memcpy(cached_key_, key, sizeof(key));
  }
  // The storage may be shared with other blobs between passes, so the values
  // are written every time (a few hundred KB at most).
  std::memcpy(top[0]->mutable_cpu_data(), cached_.data(), cached_.size() * sizeof(float));
}
REGISTER_LAYER_CLASS(PriorBox);

// ---------------------------------------------------------------- Proposal

void ProposalLayer::LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  const ProposalParameter& p = layer_param_.proposal_param();
  params_.feat_stride = p.feat_stride();
  params_.min_size = p.min_size();
  params_.pre_nms_topn = p.pre_nms_topn();
  params_.post_nms_topn = p.post_nms_topn();
  params_.nms_thresh = p.nms_thresh();
  const int base_size = p.base_size();
  std::vector<float> ratios(p.ratio().begin(), p.ratio().end());
  std::vector<float> scales(p.scale().begin(), p.scale().end());
  CHECK(!ratios.empty() && !scales.empty()) << "Proposal: ratio and scale lists must not be empty";
  num_anchors_ = static_cast<int>(ratios.size() * scales.size());
  // Base anchors, anchor index = ratio index * #scales + scale index
  // (src/layers/proposal_layer.cpp:56-85; same float expressions).
  std::vector<float> anchors(static_cast<size_t>(num_anchors_) * 4);
  const float base_area = static_cast<float>(base_size * base_size);
  const float center = static_cast<float>(0.5 * (base_size - 1));
  float* a = anchors.data();
  for (float ratio : ratios) {
    const float ratio_w = static_cast<float>(std::round(std::sqrt(base_area / ratio)));
    const float ratio_h = static_cast<float>(std::round(ratio_w * ratio));
    for (float scale : scales) {
      const float scale_w = 0.5f * static_cast<float>(ratio_w * scale - 1);
      const float scale_h = 0.5f * static_cast<float>(ratio_h * scale - 1);
      a[0] = center - scale_w;
      a[1] = center - scale_h;
      a[2] = center + scale_w;
      a[3] = center + scale_h;
      a += 4;
    }
  }
  anchors_.Assign(anchors);
}

void ProposalLayer::Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  CHECK_EQ(bottom[0]->num_axes(), 4);
  CHECK_EQ(bottom[0]->channels(), 2 * num_anchors_) << "score map must have 2 channels per anchor";
  CHECK_EQ(bottom[1]->channels(), 4 * num_anchors_) << "delta map must have 4 channels per anchor";
  CHECK_EQ(bottom[2]->count(), 3 * bottom[0]->num()) << "im_info must hold (height, width, scale) per image";
  const int rows = bottom[0]->shape(0) * params_.post_nms_topn;
  top[0]->Reshape(vector<int>{rows, 5});
  if (top.size() > 1) top[1]->Reshape(vector<int>{rows});
}

void ProposalLayer::Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  Context& ctx = Context::Get();
  const int batch = bottom[0]->num();
  params_.num_anchors = num_anchors_;
  params_.height = bottom[0]->height();
  params_.width = bottom[0]->width();
  const size_t ws_bytes = mcb200_proposal_workspace_bytes(&params_, batch);
  CHECK_GT(ws_bytes, 0u) << "Proposal: unsupported parameters (pre_nms_topn may be at most 16384)";
  const int ws_floats = static_cast<int>((ws_bytes + 3) / 4) + 64;
  if (!workspace_ || workspace_->count() < ws_floats) workspace_.reset(new Blob(vector<int>(1, ws_floats)));
  if (!counts_ || counts_->count() < batch) counts_.reset(new BlobInt(vector<int>(1, batch)));
  char* ws = reinterpret_cast<char*>(workspace_->mutable_gpu_data());
  ws = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(ws) + 255) & ~static_cast<uintptr_t>(255));

  const int post = params_.post_nms_topn;
  const bool want_scores = top.size() > 1;
  // Largest shape first: the kernels write image b's rows at b * post.
  top[0]->Reshape(vector<int>{batch * post, 5});
  if (want_scores) top[1]->Reshape(vector<int>{batch * post});
  float* rois = top[0]->mutable_gpu_data();
  float* roi_scores = want_scores ? top[1]->mutable_gpu_data() : nullptr;
  KERNEL_CHECK(mcb200_proposal_forward(&params_, batch, bottom[0]->gpu_data(), bottom[1]->gpu_data(),
                                       bottom[2]->gpu_data(), anchors_.get(), ws, rois, roi_scores,
                                       counts_->mutable_gpu_data(), ctx.stream_ptr()));
  // Close the gaps between the images' row blocks on the device (the ranges a
  // row block leaves and enters may overlap, so this is a kernel, not a copy).
  if (batch > 1) {
    KERNEL_CHECK(mcb200_proposal_compact(rois, roi_scores, counts_->gpu_data(), batch, post, ctx.stream_ptr()));
  }
  // The output row count is data dependent: fetch the counts (a few bytes).
  const int* counts = counts_->cpu_data();
  int total = 0;
  for (int b = 0; b < batch; ++b) total += counts[b];
  top[0]->Reshape(vector<int>{total, 5});
  if (want_scores) top[1]->Reshape(vector<int>{total});
}
REGISTER_LAYER_CLASS(Proposal);

// ---------------------------------------------------------------- DetectionOutput

void DetectionOutputLayer::LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  const DetectionOutputParameter& p = layer_param_.detection_output_param();
  CHECK(p.has_num_classes()) << "Must specify num_classes";
  params_.num_classes = p.num_classes();
  params_.share_location = p.share_location() ? 1 : 0;
  params_.background_label_id = p.background_label_id();
  params_.code_type = static_cast<int>(p.code_type());
  params_.variance_encoded_in_target = p.variance_encoded_in_target() ? 1 : 0;
  params_.keep_top_k = p.keep_top_k();
  params_.confidence_threshold = p.has_confidence_threshold() ? p.confidence_threshold() : -FLT_MAX;
  params_.nms_threshold = p.nms_param().nms_threshold();
  CHECK_GE(params_.nms_threshold, 0.) << "nms_threshold must be non negative.";
  params_.eta = p.nms_param().eta();
  CHECK_GT(params_.eta, 0.);
  CHECK_LE(params_.eta, 1.);
  params_.top_k = p.nms_param().has_top_k() ? p.nms_param().top_k() : -1;
}

void DetectionOutputLayer::Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  CHECK_EQ(bottom[0]->num(), bottom[1]->num());
  params_.num_priors = bottom[2]->height() / 4;
  const int loc_classes = params_.share_location ? 1 : params_.num_classes;
  CHECK_EQ(params_.num_priors * loc_classes * 4, bottom[0]->channels())
      << "Number of priors must match number of location predictions.";
  CHECK_EQ(params_.num_priors * params_.num_classes, bottom[1]->channels())
      << "Number of priors must match number of confidence predictions.";
  // The row count is only known after NMS; like the reference, start with one row.
  top[0]->Reshape(vector<int>{1, 7});
}

void DetectionOutputLayer::Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  Context& ctx = Context::Get();
  const int batch = bottom[0]->num();
  const size_t ws_bytes = mcb200_detout_workspace_bytes(&params_, batch);
  CHECK_GT(ws_bytes, 0u) << "DetectionOutput: unsupported parameters (top_k may be at most 4096)";
  const int ws_floats = static_cast<int>((ws_bytes + 3) / 4) + 64;
  if (!workspace_ || workspace_->count() < ws_floats) workspace_.reset(new Blob(vector<int>(1, ws_floats)));
  if (!total_) total_.reset(new BlobInt(vector<int>(1, 1)));
  char* ws = reinterpret_cast<char*>(workspace_->mutable_gpu_data());
  ws = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(ws) + 255) & ~static_cast<uintptr_t>(255));
  const int max_rows = mcb200_detout_max_rows_per_image(&params_);
  top[0]->Reshape(vector<int>{batch * max_rows, 7});
  float* out = top[0]->mutable_gpu_data();
  KERNEL_CHECK(mcb200_detout_forward(&params_, batch, bottom[0]->gpu_data(), bottom[1]->gpu_data(),
                                     bottom[2]->gpu_data(), ws, out, total_->mutable_gpu_data(), ctx.stream_ptr()));
  const int total = total_->cpu_data()[0];
  // No detection: one placeholder row per image (written by the kernel).
  top[0]->Reshape(vector<int>{total > 0 ? total : batch, 7});
}
REGISTER_LAYER_CLASS(DetectionOutput);

// ---------------------------------------------------------------- ROIPooling / PSROIPooling

void ROIPoolingLayer::LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  const ROIPoolingParameter& p = layer_param_.roi_pooling_param();
  CHECK_GT(p.pooled_h(), 0u) << "pooled_h must be > 0";
  CHECK_GT(p.pooled_w(), 0u) << "pooled_w must be > 0";
  pooled_h_ = static_cast<int>(p.pooled_h());
  pooled_w_ = static_cast<int>(p.pooled_w());
  spatial_scale_ = p.spatial_scale();
}

void ROIPoolingLayer::Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  CHECK_EQ(bottom[0]->num_axes(), 4) << "ROIPooling: feature maps must be (N, C, H, W)";
  CHECK_EQ(bottom[1]->count(1), 5) << "ROIPooling: rois must be rows of (batch index, x1, y1, x2, y2)";
  top[0]->Reshape(bottom[1]->num(), bottom[0]->channels(), pooled_h_, pooled_w_);
}

void ROIPoolingLayer::Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  Context& ctx = Context::Get();
  if (top[0]->count() == 0) return;
  KERNEL_CHECK(mcb200_roi_pool(bottom[0]->gpu_data(), bottom[1]->gpu_data(), top[0]->mutable_gpu_data(),
                               bottom[1]->num(), bottom[0]->num(), bottom[0]->channels(), bottom[0]->height(),
                               bottom[0]->width(), pooled_h_, pooled_w_, spatial_scale_, ctx.status_word(),
                               ctx.stream_ptr()));
}
REGISTER_LAYER_CLASS(ROIPooling);

void PSROIPoolingLayer::LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  const PSROIPoolingParameter& p = layer_param_.psroi_pooling_param();
  CHECK_GT(p.output_dim(), 0) << "output_dim must be > 0";
  CHECK_GT(p.group_size(), 0) << "group_size must be > 0";
  output_dim_ = p.output_dim();
  group_size_ = p.group_size();
  spatial_scale_ = p.spatial_scale();
}

void PSROIPoolingLayer::Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  CHECK_EQ(bottom[0]->num_axes(), 4) << "PSROIPooling: score maps must be (N, C, H, W)";
  CHECK_EQ(bottom[0]->channels(), output_dim_ * group_size_ * group_size_)
      << "input channel number does not match layer parameters";
  CHECK_EQ(bottom[1]->count(1), 5) << "PSROIPooling: rois must be rows of (batch index, x1, y1, x2, y2)";
  top[0]->Reshape(bottom[1]->num(), output_dim_, group_size_, group_size_);
}

void PSROIPoolingLayer::Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  Context& ctx = Context::Get();
  if (top[0]->count() == 0) return;
  KERNEL_CHECK(mcb200_psroi_pool(bottom[0]->gpu_data(), bottom[1]->gpu_data(), top[0]->mutable_gpu_data(),
                                 bottom[1]->num(), bottom[0]->num(), output_dim_, group_size_, bottom[0]->height(),
                                 bottom[0]->width(), spatial_scale_, ctx.status_word(), ctx.stream_ptr()));
}
REGISTER_LAYER_CLASS(PSROIPooling);

}  // namespace caffe
