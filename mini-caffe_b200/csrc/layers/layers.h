// Declarations of the engine's layer classes (one registry entry each).
#ifndef MCB200_LAYERS_H_
#define MCB200_LAYERS_H_

#include <memory>
#include <string>
#include <vector>

#include "../layer.h"
#include "mcb200_kernels.h"

namespace caffe {

// A float array that lives on the device and is refreshed from host values.
class DeviceArray {
 public:
  void Assign(const std::vector<float>& host);
  const float* get() const { return blob_ ? blob_->gpu_data() : nullptr; }
  void Clear() { blob_.reset(); }
 private:
  std::unique_ptr<Blob> blob_;
};

// Scratch device memory owned by a layer (grown on demand, never shrunk).
class DeviceScratch {
 public:
  float* Reserve(size_t floats);
 private:
  std::unique_ptr<Blob> blob_;
};

// ---------------------------------------------------------------- producers

// Convolution, 2-D, any stride / pad / dilation / group.  Depthwise layers
// (group == channels) run on a kernel of their own, everything else, grouped
// layers included, on the tensor cores; the direct kernel is left for shapes the
// tensor-core kernel's tensor maps cannot express.  Parameter handling follows src/layers/base_conv_layer.cpp:11-182.
class ConvolutionLayer : public Layer {
 public:
  explicit ConvolutionLayer(const LayerParameter& param) : Layer(param) {}
  void LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  void Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  const char* type() const override { return "Convolution"; }
  int MinBottomBlobs() const override { return 1; }
  int MinTopBlobs() const override { return 1; }
  bool EqualNumBottomTopBlobs() const override { return true; }
  bool AcceptsFusedTail() const override { return true; }
  void SetFusedTail(const FusedTail& tail) override { tail_ = tail; tail_version_ = 0; }
  bool HalfOperandsCapable() const override {
    if (path_ == kDepthwise) return DepthwiseHalfCapable();
    return path_ == kTensorCore && !use_rows_ && shape_.c % 8 == 0;
  }
  bool HalfTopCapable() const override {
    if (path_ == kDepthwise) return DepthwiseHalfCapable();
    return path_ == kTensorCore && shape_.cout % 8 == 0;
  }
  void SetHalfStorage(bool operands, bool top) override {
    if (operands != half_operands_) weight_version_ = 0;   // the packed weight image differs
    half_operands_ = operands;
    half_top_ = top;
  }

 protected:
  void Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  void RefreshParameters();
  void FillEpilogue(mcb200_epilogue* ep);

  // The depthwise 3x3 kernel reads and writes bfloat16 cells (fp32 weights and arithmetic).
  bool DepthwiseHalfCapable() const {
    return tail_.residual == nullptr && mcb200_conv_depthwise_bf16_supported(&shape_) != 0 && shape_.c % 8 == 0;
  }
  bool half_operands_ = false;   // bfloat16 activations, weights and residual (tcgen05 kind::f16)
  bool half_top_ = false;        // the result is stored as bfloat16

  mcb200_conv_shape shape_ = mcb200_conv_shape();
  bool bias_term_ = false;
  FusedTail tail_;
  unsigned long long tail_version_ = 0;    // parameter versions the folded arrays were built from
  unsigned long long weight_version_ = 0;
  DeviceArray scale_, shift_;
  DeviceScratch packed_weights_, padded_input_;
  enum Path { kTensorCore, kDepthwise, kDirect } path_ = kDirect;
  bool use_rows_ = false;       // tensor-core row mode (at most four input channels)
  bool rows_rejected_ = false;
  struct PlanSlot {
    mcb200_conv_plan plan;
    const float* in = nullptr;
    const float* weights = nullptr;
    mcb200_conv_shape shape = mcb200_conv_shape();
    bool valid = false;
  };
  std::vector<std::unique_ptr<PlanSlot> > plans_;  // one per bottom
};

// y = x W^T + b as a 1x1 convolution over [M, K] (src/layers/inner_product_layer.cpp:8-93).
class InnerProductLayer : public Layer {
 public:
  explicit InnerProductLayer(const LayerParameter& param) : Layer(param) {}
  void LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  void Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  const char* type() const override { return "InnerProduct"; }
  int ExactNumBottomBlobs() const override { return 1; }
  int ExactNumTopBlobs() const override { return 1; }
  bool AcceptsFusedTail() const override { return true; }
  void SetFusedTail(const FusedTail& tail) override { tail_ = tail; tail_version_ = 0; }

 protected:
  void Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  int M_ = 0, K_ = 0, N_ = 0;
  bool bias_term_ = false, transpose_ = false;
  FusedTail tail_;
  unsigned long long tail_version_ = 0, weight_version_ = 0;
  DeviceArray scale_, shift_;
  DeviceScratch packed_weights_, staged_weights_;
  mcb200_conv_plan* plan_ = nullptr;
  std::unique_ptr<char[]> plan_storage_;
  const float* plan_in_ = nullptr;
  const float* plan_w_ = nullptr;
  int plan_m_ = -1;
};

// Folds a FusedTail and an optional bias into per-channel scale / shift
// arrays; returns the combined parameter version.
unsigned long long TailVersion(const FusedTail& tail);
void FoldTail(const FusedTail& tail, int channels, const float* bias, std::vector<float>* scale,
              std::vector<float>* shift, bool* has_scale, bool* has_shift);
// Which device copy of the residual blob the kernel reads.
enum ResidualCopy { kResidualNchw, kResidualNhwc, kResidualNhwcHalf };
void FillTailEpilogue(const FusedTail& tail, const DeviceArray& scale, const DeviceArray& shift,
                      ResidualCopy residual_copy, int channels, mcb200_epilogue* ep);

// ---------------------------------------------------------------- per-channel / elementwise

// Shared forward of layers of the form y = act(x * scale[c] + shift[c]).
class ChannelwiseLayer : public Layer {
 public:
  explicit ChannelwiseLayer(const LayerParameter& param) : Layer(param) {}
  void Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  int ExactNumTopBlobs() const override { return 1; }

 protected:
  void Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  // The channel axis is axis 1; `inner` elements follow it in (N, C, ...) order.
  virtual int Channels(const Blob* bottom) const { return bottom->num_axes() > 1 ? bottom->shape(1) : 1; }
  DeviceArray scale_dev_, shift_dev_;
  unsigned long long built_version_ = 0;
  int built_channels_ = -1;
};

class BatchNormLayer : public ChannelwiseLayer {
 public:
  explicit BatchNormLayer(const LayerParameter& param) : ChannelwiseLayer(param) {}
  void LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  const char* type() const override { return "BatchNorm"; }
  int ExactNumBottomBlobs() const override { return 1; }
  bool AsChannelAffine(int channels, std::vector<double>* scale, std::vector<double>* shift) override;
 protected:
  void Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
 private:
  int channels_ = 0;
  float eps_ = 1e-5f;
  bool use_global_stats_ = true;   // false: normalise with the statistics of the current batch
  DeviceScratch batch_scale_shift_;
};

class ScaleLayer : public ChannelwiseLayer {
 public:
  explicit ScaleLayer(const LayerParameter& param) : ChannelwiseLayer(param) {}
  void LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  void Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  const char* type() const override { return "Scale"; }
  int MinBottomBlobs() const override { return 1; }
  int MaxBottomBlobs() const override { return 2; }
  bool AsChannelAffine(int channels, std::vector<double>* scale, std::vector<double>* shift) override;
  void Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
 private:
  bool per_channel_ = false;  // learned scale of shape [C] applied on axis 1
  bool scalar_ = false;       // learned scale with no axes
  bool bias_term_ = false;
  // Factors in a second bottom, or a learned blob over other axes than the channel axis: the layer
  // cannot be folded into its producer; y[o, d, i] = x[o, d, i] * scale[d] (+ bias[d]) over the
  // (N, C, H, W)-ordered data (src/layers/scale_layer.cpp:47,72-113).
  bool general_ = false;
  int axis_ = 1, scale_dim_ = 1, inner_dim_ = 1;
};

class BiasLayer : public ChannelwiseLayer {
 public:
  explicit BiasLayer(const LayerParameter& param) : ChannelwiseLayer(param) {}
  void LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  void Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  const char* type() const override { return "Bias"; }
  int MinBottomBlobs() const override { return 1; }
  int MaxBottomBlobs() const override { return 2; }
  bool AsChannelAffine(int channels, std::vector<double>* scale, std::vector<double>* shift) override;
  void Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
 private:
  bool per_channel_ = false;
  bool scalar_ = false;
  bool general_ = false;      // offsets in a second bottom or over other axes (src/layers/bias_layer.cpp:40,45-83)
  int axis_ = 1, bias_dim_ = 1, inner_dim_ = 1;
};

class ReLULayer : public ChannelwiseLayer {
 public:
  explicit ReLULayer(const LayerParameter& param) : ChannelwiseLayer(param) {}
  const char* type() const override { return "ReLU"; }
  int ExactNumBottomBlobs() const override { return 1; }
  bool AsActivation(ActivationSpec* spec) override;
};

class PReLULayer : public ChannelwiseLayer {
 public:
  explicit PReLULayer(const LayerParameter& param) : ChannelwiseLayer(param) {}
  void LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  const char* type() const override { return "PReLU"; }
  int ExactNumBottomBlobs() const override { return 1; }
  bool AsActivation(ActivationSpec* spec) override;
 private:
  bool channel_shared_ = false;
};

// Inference-time Dropout is the identity (the reference scales nothing at test time).
class DropoutLayer : public ChannelwiseLayer {
 public:
  explicit DropoutLayer(const LayerParameter& param) : ChannelwiseLayer(param) {}
  const char* type() const override { return "Dropout"; }
  int ExactNumBottomBlobs() const override { return 1; }
};

class EltwiseLayer : public Layer {
 public:
  explicit EltwiseLayer(const LayerParameter& param) : Layer(param) {}
  void LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  void Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  const char* type() const override { return "Eltwise"; }
  int MinBottomBlobs() const override { return 2; }
  int ExactNumTopBlobs() const override { return 1; }
  bool AsWeightedSum(std::vector<float>* coeffs) override;
 protected:
  void Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  int op_ = MCB200_ELTWISE_SUM;
  std::vector<float> coeffs_;
};

// ---------------------------------------------------------------- pooling / softmax / normalize

class PoolingLayer : public Layer {
 public:
  explicit PoolingLayer(const LayerParameter& param) : Layer(param) {}
  void LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  void Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  const char* type() const override { return "Pooling"; }
  int ExactNumBottomBlobs() const override { return 1; }
  int ExactNumTopBlobs() const override { return 1; }
  // Max pooling commutes with rounding to bfloat16: a bfloat16 blob is pooled as it is.
  bool HalfOperandsCapable() const override {
    return method_ == MCB200_POOL_MAX && channels_ > 0 &&
           mcb200_pool_max_nhwc_bf16_supported(channels_, kernel_h_, kernel_w_) != 0;
  }
  bool HalfTopCapable() const override { return HalfOperandsCapable(); }
  bool HalfNeedsBoth() const override { return true; }
  void SetHalfStorage(bool operands, bool top) override { half_ = operands && top; }
 protected:
  void Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  bool half_ = false;      // bottom and top are bfloat16-stored
  int channels_ = 0;       // of the bottom, 0 unless it has four axes
  int kernel_h_ = 0, kernel_w_ = 0, stride_h_ = 1, stride_w_ = 1, pad_h_ = 0, pad_w_ = 0;
  int pooled_h_ = 0, pooled_w_ = 0;
  bool global_ = false;
  int method_ = MCB200_POOL_MAX;
};

class SoftmaxLayer : public Layer {
 public:
  explicit SoftmaxLayer(const LayerParameter& param) : Layer(param) {}
  void Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  const char* type() const override { return "Softmax"; }
  int ExactNumBottomBlobs() const override { return 1; }
  int ExactNumTopBlobs() const override { return 1; }
 protected:
  void Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  int axis_ = 1;
};

class NormalizeLayer : public Layer {
 public:
  explicit NormalizeLayer(const LayerParameter& param) : Layer(param) {}
  void LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  void Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  const char* type() const override { return "Normalize"; }
  int ExactNumBottomBlobs() const override { return 1; }
  int ExactNumTopBlobs() const override { return 1; }
 protected:
  void Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  bool across_spatial_ = true, channel_shared_ = true;
  float eps_ = 1e-10f;
};

// ---------------------------------------------------------------- graph plumbing

class InputLayer : public Layer {
 public:
  explicit InputLayer(const LayerParameter& param) : Layer(param) {}
  void LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  void Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) override {}
  const char* type() const override { return "Input"; }
  int ExactNumBottomBlobs() const override { return 0; }
  int MinTopBlobs() const override { return 1; }
 protected:
  void Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) override {}
};

class SplitLayer : public Layer {
 public:
  explicit SplitLayer(const LayerParameter& param) : Layer(param) {}
  void Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  const char* type() const override { return "Split"; }
  int ExactNumBottomBlobs() const override { return 1; }
  int MinTopBlobs() const override { return 1; }
 protected:
  void Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
};

class FlattenLayer : public Layer {
 public:
  explicit FlattenLayer(const LayerParameter& param) : Layer(param) {}
  void Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  const char* type() const override { return "Flatten"; }
  int ExactNumBottomBlobs() const override { return 1; }
  int ExactNumTopBlobs() const override { return 1; }
 protected:
  void Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
};

class ReshapeLayer : public Layer {
 public:
  explicit ReshapeLayer(const LayerParameter& param) : Layer(param) {}
  void LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  void Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  const char* type() const override { return "Reshape"; }
  int ExactNumBottomBlobs() const override { return 1; }
  int ExactNumTopBlobs() const override { return 1; }
 protected:
  void Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  std::vector<int> copy_axes_;
  int inferred_axis_ = -1;
  int constant_count_ = 1;
};

class PermuteLayer : public Layer {
 public:
  explicit PermuteLayer(const LayerParameter& param) : Layer(param) {}
  void LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  void Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  const char* type() const override { return "Permute"; }
  int ExactNumBottomBlobs() const override { return 1; }
  int ExactNumTopBlobs() const override { return 1; }
 protected:
  void Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  std::vector<int> order_;
  bool need_permute_ = false;
};

class ConcatLayer : public Layer {
 public:
  explicit ConcatLayer(const LayerParameter& param) : Layer(param) {}
  void LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  void Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  const char* type() const override { return "Concat"; }
  int MinBottomBlobs() const override { return 1; }
  int ExactNumTopBlobs() const override { return 1; }
 protected:
  void Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  int axis_ = 1;
};

// ---------------------------------------------------------------- detection

// Prior (default) boxes of an SSD head: depends only on shapes and layer
// parameters, so it is computed on the host when the shapes change and kept
// on the device (src/layers/prior_box_layer.cpp:118-217).
class PriorBoxLayer : public Layer {
 public:
  explicit PriorBoxLayer(const LayerParameter& param) : Layer(param) {}
  void LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  void Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  const char* type() const override { return "PriorBox"; }
  int ExactNumBottomBlobs() const override { return 2; }
  int ExactNumTopBlobs() const override { return 1; }
 protected:
  void Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  void Compute(int layer_h, int layer_w, int img_h, int img_w, float* out) const;
  std::vector<float> min_sizes_, max_sizes_, aspect_ratios_, variance_;
  bool flip_ = true, clip_ = false;
  int num_priors_ = 0, img_h_ = 0, img_w_ = 0;
  float step_h_ = 0, step_w_ = 0, offset_ = 0.5f;
  std::vector<float> cached_;
  int cached_key_[4] = {-1, -1, -1, -1};
};

// RPN proposals (src/layers/proposal_layer.cpp).  The reference accepts one
// image per call; this layer also takes N > 1 and then puts the image index
// in column 0 of each roi.
class ProposalLayer : public Layer {
 public:
  explicit ProposalLayer(const LayerParameter& param) : Layer(param) {}
  void LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  void Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  // The reference reports this spelling (src/layers/proposal_layer.hpp:19).
  const char* type() const override { return "ProposalLayer"; }
  int ExactNumBottomBlobs() const override { return 3; }
  int MinTopBlobs() const override { return 1; }
  int MaxTopBlobs() const override { return 2; }
 protected:
  void Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  mcb200_proposal_params params_ = mcb200_proposal_params();
  DeviceArray anchors_;
  int num_anchors_ = 0;
  std::unique_ptr<Blob> workspace_, staging_rois_, staging_scores_;
  std::unique_ptr<BlobInt> counts_;
};

class DetectionOutputLayer : public Layer {
 public:
  explicit DetectionOutputLayer(const LayerParameter& param) : Layer(param) {}
  void LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  void Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  const char* type() const override { return "DetectionOutput"; }
  int ExactNumBottomBlobs() const override { return 3; }
  int ExactNumTopBlobs() const override { return 1; }
 protected:
  void Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  mcb200_detout_params params_ = mcb200_detout_params();
  std::unique_ptr<Blob> workspace_;
  std::unique_ptr<BlobInt> total_;
};

// Kernel, stride, pad and dilation of a 2-D convolution-type layer.
void ParseConvolutionGeometry(const ConvolutionParameter& p, mcb200_conv_shape* shape);

// ---------------------------------------------------------------- layer types of the shipped example nets
// (SSH: Deconvolution + Crop; WGAN generator: Deconvolution; older nets: LRN, Slice, BN.)
// They work on (N, C, H, W) device data; parity first, no fusion.

// Transposed convolution (src/layers/deconv_layer.cpp:7-44); weights [C_in, C_out / group, kh, kw].
class DeconvolutionLayer : public Layer {
 public:
  explicit DeconvolutionLayer(const LayerParameter& param) : Layer(param) {}
  void LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  void Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  const char* type() const override { return "Deconvolution"; }
  int MinBottomBlobs() const override { return 1; }
  int MinTopBlobs() const override { return 1; }
  bool EqualNumBottomTopBlobs() const override { return true; }
 protected:
  void Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  mcb200_conv_shape shape_ = mcb200_conv_shape();
  bool bias_term_ = false;
  // The layer runs as a convolution on the tensor cores: reversed filter, input spread `stride`
  // apart over zeros (see mcb200_deconv_as_conv_shape); the direct kernel takes what is left
  // (more padding than the filter reaches).
  unsigned long long weight_version_ = 0;
  DeviceScratch flipped_weights_, packed_weights_, spread_input_;
  struct PlanSlot {
    mcb200_conv_plan plan;
    const float* in = nullptr;
    const float* weights = nullptr;
    mcb200_conv_shape shape = mcb200_conv_shape();
    bool valid = false;
  };
  std::vector<std::unique_ptr<PlanSlot> > plans_;  // one per bottom
};

// top[i] = a range of bottom[0] along one axis (src/layers/slice_layer.cpp:9-96).
class SliceLayer : public Layer {
 public:
  explicit SliceLayer(const LayerParameter& param) : Layer(param) {}
  void LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  void Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  const char* type() const override { return "Slice"; }
  int ExactNumBottomBlobs() const override { return 1; }
  int MinTopBlobs() const override { return 1; }
 protected:
  void Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  int slice_axis_ = 1;
  vector<int> slice_point_;
};

// top = bottom[0] cut to the size of bottom[1] from `axis` on, at given offsets
// (src/layers/crop_layer.cpp:12-106).
class CropLayer : public Layer {
 public:
  explicit CropLayer(const LayerParameter& param) : Layer(param) {}
  void LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  void Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  const char* type() const override { return "Crop"; }
  int ExactNumBottomBlobs() const override { return 2; }
  int ExactNumTopBlobs() const override { return 1; }
 protected:
  void Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  vector<int> offsets_;
};

// Batch normalisation with the scale and shift in the same layer and stored
// statistics: y = (x - b2) * b3 * b0 + b1 with blobs slope, bias, mean and the
// factor the reference multiplies by (src/layers/bn_layer.cpp:10-140).
class BNLayer : public ChannelwiseLayer {
 public:
  explicit BNLayer(const LayerParameter& param) : ChannelwiseLayer(param) {}
  void LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  const char* type() const override { return "BN"; }
  int ExactNumBottomBlobs() const override { return 1; }
  bool AsChannelAffine(int channels, std::vector<double>* scale, std::vector<double>* shift) override;
 private:
  int channels_ = 0;
};

// Local response normalisation (src/layers/lrn_layer.cpp:10-160).
class LRNLayer : public Layer {
 public:
  explicit LRNLayer(const LayerParameter& param) : Layer(param) {}
  void LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  void Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  const char* type() const override { return "LRN"; }
  int ExactNumBottomBlobs() const override { return 1; }
  int ExactNumTopBlobs() const override { return 1; }
 protected:
  void Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  int size_ = 5;
  float alpha_ = 1.f, beta_ = 0.75f, k_ = 1.f;
  bool within_channel_ = false;
  std::unique_ptr<Blob> in_place_copy_;
};

// TanH and Sigmoid (the output non-linearity of the WGAN generator and of older heads).
class UnaryLayer : public Layer {
 public:
  UnaryLayer(const LayerParameter& param, int op, const char* type) : Layer(param), op_(op), type_(type) {}
  void Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) override { top[0]->ReshapeLike(*bottom[0]); }
  const char* type() const override { return type_; }
  int ExactNumBottomBlobs() const override { return 1; }
  int ExactNumTopBlobs() const override { return 1; }
 protected:
  void Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  int op_;
  const char* type_;
};

// Region-of-interest pooling behind Proposal (Faster R-CNN / R-FCN heads).
// bottom[0]: feature or score maps (N, C, H, W); bottom[1]: rois [R, 5].
class ROIPoolingLayer : public Layer {
 public:
  explicit ROIPoolingLayer(const LayerParameter& param) : Layer(param) {}
  void LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  void Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  const char* type() const override { return "ROIPooling"; }
  int ExactNumBottomBlobs() const override { return 2; }
  int ExactNumTopBlobs() const override { return 1; }
 protected:
  void Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  int pooled_h_ = 0, pooled_w_ = 0;
  float spatial_scale_ = 1.f;
};

class PSROIPoolingLayer : public Layer {
 public:
  explicit PSROIPoolingLayer(const LayerParameter& param) : Layer(param) {}
  void LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  void Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  const char* type() const override { return "PSROIPooling"; }
  int ExactNumBottomBlobs() const override { return 2; }
  int ExactNumTopBlobs() const override { return 1; }
 protected:
  void Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) override;
  int output_dim_ = 0, group_size_ = 0;
  float spatial_scale_ = 1.f;
};

}  // namespace caffe

#endif  // MCB200_LAYERS_H_
