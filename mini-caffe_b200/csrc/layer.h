// Base class of every layer (the operator plug-in interface).
//
// The virtuals match mini-caffe's src/layer.hpp:25-262: LayerSetUp, Reshape,
// Forward_cpu / Forward_gpu, GetTempBlobs, type(), and the blob-count
// predicates checked by SetUp.  Differences that matter to a plug-in author:
//  * The engine's own layers implement Forward_gpu only.  Forward_cpu is not
//    pure here; a layer that defines only Forward_cpu still works, because the
//    default Forward_gpu calls it (the blobs bring their host copies up to
//    date), exactly like the reference's fallback (layer.hpp:211-215).
//  * Layers may take part in epilogue fusion through the three small hooks at
//    the end of the class; ignoring them is always correct.
#ifndef MCB200_LAYER_H_
#define MCB200_LAYER_H_

#include <algorithm>
#include <string>
#include <vector>

#include "caffe.pb.h"
#include "caffe/blob.hpp"
#include "context.h"
#include "layer_factory.h"

namespace caffe {

// What a producer (Convolution, InnerProduct) applies to each accumulator
// before storing it, gathered from the layers fused behind it:
//   v = acc * scale[c] + shift[c];  v += residual_coeff * residual;  v = act(v)
struct FusedTail {
  // Per-channel affine layers (BatchNorm, Scale, Bias), in execution order.
  std::vector<class Layer*> affine;
  // Eltwise SUM partner: this blob is added with residual_coeff, and the
  // producer's own term is multiplied by self_coeff.
  Blob* residual = nullptr;
  float residual_coeff = 1.f;
  float self_coeff = 1.f;
  // ReLU / PReLU applied last (nullptr: none).
  class Layer* activation = nullptr;
  bool empty() const { return affine.empty() && !residual && !activation; }
};

struct ActivationSpec {
  int kind = 0;          // 0 none, 1 (leaky) ReLU, 2 PReLU
  float slope = 0.f;     // kind 1
  Blob* slopes = nullptr;  // kind 2: per-channel or single slope
  bool shared = false;
};

class Layer {
 public:
  explicit Layer(const LayerParameter& param) : layer_param_(param) {
    // Parameter blobs written inline in the prototxt.
    if (layer_param_.blobs_size() > 0) {
      blobs_.resize(layer_param_.blobs_size());
      for (int i = 0; i < layer_param_.blobs_size(); ++i) {
        blobs_[i].reset(new Blob);
        blobs_[i]->FromProto(layer_param_.blobs(i));
      }
    }
  }
  virtual ~Layer() {}

  void SetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) {
    CheckBlobCounts(bottom, top);
    LayerSetUp(bottom, top);
    Reshape(bottom, top);
  }

  // One-time set-up from the layer parameters and the bottom shapes.
  virtual void LayerSetUp(const vector<Blob*>& bottom, const vector<Blob*>& top) {}
  // Shape the tops (and internal buffers) for the current bottom shapes.
  virtual void Reshape(const vector<Blob*>& bottom, const vector<Blob*>& top) = 0;

  inline void Forward(const vector<Blob*>& bottom, const vector<Blob*>& top);

  // Scratch blobs the net's memory planner may share with other blobs.
  virtual std::vector<Blob*> GetTempBlobs() { return {}; }

  vector<shared_ptr<Blob> >& blobs() { return blobs_; }
  const LayerParameter& layer_param() const { return layer_param_; }
  inline void ToProto(LayerParameter* param);
  virtual inline const char* type() const { return ""; }

  virtual int ExactNumBottomBlobs() const { return -1; }
  virtual int MinBottomBlobs() const { return -1; }
  virtual int MaxBottomBlobs() const { return -1; }
  virtual int ExactNumTopBlobs() const { return -1; }
  virtual int MinTopBlobs() const { return -1; }
  virtual int MaxTopBlobs() const { return -1; }
  virtual bool EqualNumBottomTopBlobs() const { return false; }

  // ---- fusion hooks ----
  // Producer side: true if the layer can apply a FusedTail when it stores.
  virtual bool AcceptsFusedTail() const { return false; }
  virtual void SetFusedTail(const FusedTail& tail) {}
  // Consumer side: express this layer as y = x * scale[c] + shift[c] over
  // `channels` channels of axis 1 (false: cannot be fused).  Called whenever
  // the parameters may have changed.
  virtual bool AsChannelAffine(int channels, std::vector<double>* scale, std::vector<double>* shift) {
    return false;
  }
  // Consumer side: express this layer as an activation.
  virtual bool AsActivation(ActivationSpec* spec) { return false; }
  // Consumer side: true if the layer is y = sum_i coeff[i] * bottom[i].
  virtual bool AsWeightedSum(std::vector<float>* coeffs) { return false; }
  // ---- bfloat16 storage (nets built with MINICAFFE_PRECISION=bf16) ----
  // As shaped now: can the layer take its bottoms (and a fused residual) from
  // their bfloat16 copies / store top 0 as bfloat16?  HalfNeedsBoth: only both
  // together (a layer without arithmetic of its own, e.g. max pooling).
  virtual bool HalfOperandsCapable() const { return false; }
  virtual bool HalfTopCapable() const { return false; }
  virtual bool HalfNeedsBoth() const { return false; }
  // The net's decision.  operands: read bottoms / residual as bfloat16; top:
  // store top 0 as bfloat16.
  virtual void SetHalfStorage(bool operands, bool top) {}
  // Sum of host_version() over the parameter blobs: changes when weights do.
  unsigned long long ParamVersion() const {
    unsigned long long v = 0;
    for (const auto& b : blobs_) v += b->host_version();
    return v;
  }

 protected:
  LayerParameter layer_param_;
  vector<shared_ptr<Blob> > blobs_;

  virtual void Forward_cpu(const vector<Blob*>& bottom, const vector<Blob*>& top) {
    LOG(FATAL) << type() << " layer: this engine has no CPU compute path";
  }
  virtual void Forward_gpu(const vector<Blob*>& bottom, const vector<Blob*>& top) { Forward_cpu(bottom, top); }

  virtual void CheckBlobCounts(const vector<Blob*>& bottom, const vector<Blob*>& top) {
    const int nb = static_cast<int>(bottom.size());
    const int nt = static_cast<int>(top.size());
    if (ExactNumBottomBlobs() >= 0) {
      CHECK_EQ(ExactNumBottomBlobs(), nb) << type() << " Layer takes " << ExactNumBottomBlobs()
                                          << " bottom blob(s) as input.";
    }
    if (MinBottomBlobs() >= 0) {
      CHECK_LE(MinBottomBlobs(), nb) << type() << " Layer takes at least " << MinBottomBlobs()
                                     << " bottom blob(s) as input.";
    }
    if (MaxBottomBlobs() >= 0) {
      CHECK_GE(MaxBottomBlobs(), nb) << type() << " Layer takes at most " << MaxBottomBlobs()
                                     << " bottom blob(s) as input.";
    }
    if (ExactNumTopBlobs() >= 0) {
      CHECK_EQ(ExactNumTopBlobs(), nt) << type() << " Layer produces " << ExactNumTopBlobs()
                                       << " top blob(s) as output.";
    }
    if (MinTopBlobs() >= 0) {
      CHECK_LE(MinTopBlobs(), nt) << type() << " Layer produces at least " << MinTopBlobs()
                                  << " top blob(s) as output.";
    }
    if (MaxTopBlobs() >= 0) {
      CHECK_GE(MaxTopBlobs(), nt) << type() << " Layer produces at most " << MaxTopBlobs()
                                  << " top blob(s) as output.";
    }
    if (EqualNumBottomTopBlobs()) {
      CHECK_EQ(nb, nt) << type() << " Layer produces one top blob as output for each bottom blob input.";
    }
  }

 private:
  DISABLE_COPY_AND_ASSIGN(Layer);
};

inline void Layer::Forward(const vector<Blob*>& bottom, const vector<Blob*>& top) {
  // Raises caffe::Error in CPU mode or without a device: there is no CPU path.
  Context::Get().Activate();
  Forward_gpu(bottom, top);
}

inline void Layer::ToProto(LayerParameter* param) {
  param->Clear();
  param->CopyFrom(layer_param_);
  param->clear_blobs();
  for (size_t i = 0; i < blobs_.size(); ++i) blobs_[i]->ToProto(param->add_blobs());
}

}  // namespace caffe

#endif  // MCB200_LAYER_H_
