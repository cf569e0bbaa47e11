// caffe::Net: graph construction, the fused execution schedule, storage
// sharing, forward.
//
// Construction follows mini-caffe (src/net.cpp:26-145): layers are created in
// prototxt order through the registry, blobs are wired by name, a top named
// like the bottom at the same index is in-place, a second producer of a blob
// name is an error, parameters get "<layer>_<index>" display names.
//
// What differs is what happens between construction and the kernels:
//  * PlaceMemory() first builds a schedule in which per-channel affine layers
//    (BatchNorm, Scale, Bias), a residual Eltwise SUM and a ReLU/PReLU that
//    follow a Convolution or InnerProduct are folded into that producer's
//    store (one kernel instead of up to seven passes over the activation);
//  * blob lifetimes are then taken from that schedule and storage is shared
//    between blobs with disjoint lifetimes by the reference's greedy rule
//    (src/net.cpp:147-210: reuse a retired blob if it is at most twice as
//    large as needed);
//  * the schedule is cached: Forward(true) rebuilds it only when an input
//    shape or the set of marked outputs changed.
// Only blobs the reference guarantees to be readable after Forward (Input
// tops, last-layer tops, MarkOutputs blobs) are protected from fusion and
// sharing.
#include "caffe/net.hpp"

#include <algorithm>
#include <cstdlib>
#include <map>
#include <set>
#include <sstream>

#include "caffe/profiler.hpp"
#include "context.h"
#include "google/protobuf/text_format.h"
#include "io.h"
#include "layer.h"

namespace caffe {

struct NetStep {
  int layer_id;
  std::vector<Blob*> bottoms, tops;
  std::vector<int> bottom_ids, top_ids;  // bottom_ids includes a fused residual blob
};

struct NetPlan {
  bool valid = false;
  std::vector<NetStep> steps;
  std::vector<std::vector<int> > input_shapes;  // shapes of the Input tops the plan was built for
  std::vector<bool> visible;                    // per blob: guaranteed readable after Forward
  // Opt-in read when the net is constructed (environment MINICAFFE_PRECISION=bf16):
  // blobs that only tensor-core convolutions read are stored as bfloat16.
  bool half_storage = false;
};

namespace {
bool HalfStorageRequested() {
  const char* v = getenv("MINICAFFE_PRECISION");
  return v && (std::string(v) == "bf16" || std::string(v) == "BF16" || std::string(v) == "bfloat16");
}
}  // namespace

Net::Net(const string& param_file) : plan_(new NetPlan) {
  NetParameter param;
  ReadNetParamsFromTextFileOrDie(param_file, &param);
  Init(param);
}

Net::Net(const NetParameter& param) : plan_(new NetPlan) { Init(param); }

Net::~Net() { delete plan_; }

void Net::Init(const NetParameter& param) {
  if (!plan_) plan_ = new NetPlan;
  plan_->half_storage = HalfStorageRequested();
  name_ = param.name();
  CHECK_GT(param.layer_size(), 0) << "the net has no layers";
  std::map<string, int> blob_name_to_idx;
  std::set<string> available_blobs;
  const int n = param.layer_size();
  bottom_vecs_.resize(n);
  top_vecs_.resize(n);
  bottom_id_vecs_.resize(n);
  top_id_vecs_.resize(n);
  param_id_vecs_.resize(n);
  for (int layer_id = 0; layer_id < n; ++layer_id) {
    const LayerParameter& layer_param = param.layer(layer_id);
    layers_.push_back(LayerRegistry::CreateLayer(layer_param));
    layer_names_.push_back(layer_param.name());
    for (int b = 0; b < layer_param.bottom_size(); ++b) {
      AppendBottom(param, layer_id, b, &available_blobs, &blob_name_to_idx);
    }
    for (int t = 0; t < layer_param.top_size(); ++t) {
      AppendTop(param, layer_id, t, &available_blobs, &blob_name_to_idx);
    }
    layers_[layer_id]->SetUp(bottom_vecs_[layer_id], top_vecs_[layer_id]);
    const int num_params = static_cast<int>(layers_[layer_id]->blobs().size());
    for (int p = 0; p < num_params; ++p) AppendParam(param, layer_id, p);
  }
  CHECK_EQ(std::string(layers_[0]->type()), std::string("Input")) << "Network's first layer should be Input Layer.";
  // Inputs stay readable for the whole pass.
  for (int blob_id : top_id_vecs_[0]) blob_life_time_[blob_id] = static_cast<int>(layers_.size());
  for (size_t i = 0; i < blob_names_.size(); ++i) {
    blob_names_index_[blob_names_[i]] = static_cast<int>(i);
    blobs_[i]->set_name(blob_names_[i]);
  }
  for (size_t i = 0; i < layer_names_.size(); ++i) layer_names_index_[layer_names_[i]] = static_cast<int>(i);
  PlaceMemory();
}

void Net::AppendTop(const NetParameter& param, const int layer_id, const int top_id,
                    std::set<string>* available_blobs, std::map<string, int>* blob_name_to_idx) {
  const LayerParameter& layer_param = param.layer(layer_id);
  const string blob_name = layer_param.top(top_id);
  if (layer_param.bottom_size() > top_id && blob_name == layer_param.bottom(top_id)) {
    // In-place: the top is the bottom of the same index.
    const int blob_id = (*blob_name_to_idx)[blob_name];
    top_vecs_[layer_id].push_back(blobs_[blob_id].get());
    top_id_vecs_[layer_id].push_back(blob_id);
    blob_life_time_[blob_id] = std::max(blob_life_time_[blob_id], layer_id + 1);
  } else if (blob_name_to_idx->find(blob_name) != blob_name_to_idx->end()) {
    LOG(FATAL) << "Top blob '" << blob_name << "' produced by multiple sources.";
  } else {
    shared_ptr<Blob> blob(new Blob);
    const int blob_id = static_cast<int>(blobs_.size());
    blobs_.push_back(blob);
    blob_names_.push_back(blob_name);
    blob_life_time_.push_back(layer_id + 1);
    (*blob_name_to_idx)[blob_name] = blob_id;
    top_id_vecs_[layer_id].push_back(blob_id);
    top_vecs_[layer_id].push_back(blob.get());
  }
  available_blobs->insert(blob_name);
}

int Net::AppendBottom(const NetParameter& param, const int layer_id, const int bottom_id,
                      std::set<string>* available_blobs, std::map<string, int>* blob_name_to_idx) {
  const LayerParameter& layer_param = param.layer(layer_id);
  const string& blob_name = layer_param.bottom(bottom_id);
  if (available_blobs->find(blob_name) == available_blobs->end()) {
    LOG(FATAL) << "Unknown bottom blob '" << blob_name << "' (layer '" << layer_param.name() << "', bottom index "
               << bottom_id << ")";
  }
  const int blob_id = (*blob_name_to_idx)[blob_name];
  bottom_vecs_[layer_id].push_back(blobs_[blob_id].get());
  bottom_id_vecs_[layer_id].push_back(blob_id);
  blob_life_time_[blob_id] = std::max(blob_life_time_[blob_id], layer_id);
  return blob_id;
}

void Net::AppendParam(const NetParameter& param, const int layer_id, const int param_id) {
  const LayerParameter& layer_param = layers_[layer_id]->layer_param();
  string name = layer_param.param_size() > param_id ? layer_param.param(param_id).name() : "";
  if (name.empty()) {
    std::ostringstream os;
    os << layer_param.name() << "_" << param_id;
    name = os.str();
  }
  param_display_names_.push_back(name);
  param_id_vecs_[layer_id].push_back(static_cast<int>(params_.size()));
  params_.push_back(layers_[layer_id]->blobs()[param_id]);
}

void Net::Reshape() {
  for (size_t i = 0; i < layers_.size(); ++i) layers_[i]->Reshape(bottom_vecs_[i], top_vecs_[i]);
}

// ---------------------------------------------------------------- schedule

namespace {

struct FusionScan {
  const std::vector<shared_ptr<Layer> >& layers;
  const std::vector<std::vector<int> >& bottom_ids;
  const std::vector<std::vector<int> >& top_ids;
  const std::vector<bool>& visible;
  std::vector<bool> absorbed;

  // Layers (not absorbed) that read `blob`, in order, starting after `after`.
  std::vector<int> Consumers(int blob, int after) const {
    std::vector<int> out;
    for (size_t k = after + 1; k < layers.size(); ++k) {
      if (absorbed[k]) continue;
      if (std::find(bottom_ids[k].begin(), bottom_ids[k].end(), blob) != bottom_ids[k].end()) out.push_back(k);
    }
    return out;
  }
  // First layer that writes `blob` (its producer).
  int Producer(int blob) const {
    for (size_t k = 0; k < layers.size(); ++k) {
      if (std::find(top_ids[k].begin(), top_ids[k].end(), blob) != top_ids[k].end()) return static_cast<int>(k);
    }
    return -1;
  }
  bool WrittenBetween(int blob, int first, int last) const {
    for (int k = first; k <= last; ++k) {
      if (std::find(top_ids[k].begin(), top_ids[k].end(), blob) != top_ids[k].end()) return true;
    }
    return false;
  }
};

}  // namespace

void Net::PlaceMemory() {
  Reshape();
  NetPlan& plan = *plan_;
  const int num_layers = static_cast<int>(layers_.size());
  const int num_blobs = static_cast<int>(blobs_.size());

  // Blobs whose contents callers may read after Forward.
  plan.visible.assign(num_blobs, false);
  for (int b = 0; b < num_blobs; ++b) plan.visible[b] = blob_life_time_[b] >= num_layers;
  for (int b : top_id_vecs_[num_layers - 1]) plan.visible[b] = true;

  // ---- fusion ----
  FusionScan scan{layers_, bottom_id_vecs_, top_id_vecs_, plan.visible, std::vector<bool>(num_layers, false)};
  plan.steps.clear();
  for (int i = 0; i < num_layers; ++i) {
    if (scan.absorbed[i]) continue;
    NetStep step;
    step.layer_id = i;
    step.bottoms = bottom_vecs_[i];
    step.tops = top_vecs_[i];
    step.bottom_ids = bottom_id_vecs_[i];
    step.top_ids = top_id_vecs_[i];
    Layer* producer = layers_[i].get();
    if (producer->AcceptsFusedTail()) {
      FusedTail tail;
      if (step.tops.size() == 1 && step.bottoms.size() == 1 && blobs_[step.top_ids[0]]->num_axes() >= 2) {
        int cur = step.top_ids[0];
        const int channels = blobs_[cur]->shape(1);
        for (;;) {
          if (tail.activation) break;  // nothing is folded behind an activation
          std::vector<int> consumers = scan.Consumers(cur, i);
          if (consumers.empty()) break;
          const int k = consumers[0];
          Layer* next = layers_[k].get();
          if (top_id_vecs_[k].size() != 1) break;
          const int out = top_id_vecs_[k][0];
          const bool in_place = out == cur;
          // A separate output blob may replace `cur` only if nobody else needs `cur`.
          if (!in_place && (plan.visible[cur] || consumers.size() != 1)) break;
          if (blobs_[out]->shape() != blobs_[cur]->shape()) break;
          std::vector<float> coeffs;
          ActivationSpec act;
          if (!tail.residual && bottom_id_vecs_[k].size() == 1 && next->AsChannelAffine(channels, nullptr, nullptr)) {
            tail.affine.push_back(next);
          } else if (bottom_id_vecs_[k].size() == 1 && next->AsActivation(&act)) {
            tail.activation = next;
          } else if (!tail.residual && bottom_id_vecs_[k].size() == 2 && !in_place && next->AsWeightedSum(&coeffs) &&
                     bottom_id_vecs_[k][0] != bottom_id_vecs_[k][1]) {
            const int self_slot = bottom_id_vecs_[k][0] == cur ? 0 : 1;
            const int other = bottom_id_vecs_[k][1 - self_slot];
            // The partner must be complete before this producer runs and must
            // not change until the Eltwise would have run.
            const int other_producer = scan.Producer(other);
            if (other_producer < 0 || other_producer >= i || scan.WrittenBetween(other, i, k)) break;
            tail.residual = blobs_[other].get();
            tail.residual_coeff = coeffs[1 - self_slot];
            tail.self_coeff = coeffs[self_slot];
            // Only the id: the layer still sees its own bottoms; the id keeps
            // the partner alive until this step has run.
            step.bottom_ids.push_back(other);
          } else {
            break;
          }
          scan.absorbed[k] = true;
          cur = out;
        }
        step.tops[0] = blobs_[cur].get();
        step.top_ids[0] = cur;
      }
      producer->SetFusedTail(tail);
    }
    plan.steps.push_back(step);
  }

  // ---- bfloat16 storage ----
  // Which blobs exist only as bfloat16.  A blob qualifies if callers cannot see
  // it, its producer can store bfloat16, and every step that reads it (as input
  // or as fused residual) actually runs on bfloat16 operands.  A step does so
  // only if it is able to and ALL its own inputs are bfloat16 blobs: a layer
  // fed with fp32 data computes in TF32 on it rather than paying a conversion
  // pass.  Start from the optimistic assignment and withdraw blobs until the
  // rules hold everywhere (each round withdraws at least one, so it ends).
  {
    const int steps = static_cast<int>(plan.steps.size());
    std::vector<char> half_blob(num_blobs, 0);
    auto own_inputs = [&](const NetStep& st) { return static_cast<int>(st.bottoms.size()); };
    if (plan.half_storage) {
      for (int s = 0; s < steps; ++s) {
        const NetStep& step = plan.steps[s];
        if (step.top_ids.size() != 1 || plan.visible[step.top_ids[0]]) continue;
        if (!layers_[step.layer_id]->HalfTopCapable()) continue;
        const int blob = step.top_ids[0];
        int readers = 0;
        bool ok = true;
        for (int k = s + 1; k < steps && ok; ++k) {
          const NetStep& later = plan.steps[k];
          const bool reads = std::find(later.bottom_ids.begin(), later.bottom_ids.end(), blob) != later.bottom_ids.end();
          const bool writes = std::find(later.top_ids.begin(), later.top_ids.end(), blob) != later.top_ids.end();
          if (reads) ++readers;
          if (writes || (reads && !layers_[later.layer_id]->HalfOperandsCapable())) ok = false;
        }
        half_blob[blob] = ok && readers > 0;
      }
    }
    auto runs_half = [&](int s) {
      const NetStep& step = plan.steps[s];
      Layer* layer = layers_[step.layer_id].get();
      if (!layer->HalfOperandsCapable() || own_inputs(step) == 0) return false;
      for (int i = 0; i < own_inputs(step); ++i) {
        if (!half_blob[step.bottom_ids[i]]) return false;
      }
      if (layer->HalfNeedsBoth() && !(step.top_ids.size() == 1 && half_blob[step.top_ids[0]])) return false;
      return true;
    };
    for (bool changed = plan.half_storage; changed;) {
      changed = false;
      for (int s = 0; s < steps; ++s) {
        if (runs_half(s)) continue;
        const NetStep& step = plan.steps[s];
        for (int b : step.bottom_ids) {   // inputs and fused residual alike
          if (half_blob[b]) {
            half_blob[b] = 0;
            changed = true;
          }
        }
        if (layers_[step.layer_id]->HalfNeedsBoth() && step.top_ids.size() == 1 && half_blob[step.top_ids[0]]) {
          half_blob[step.top_ids[0]] = 0;
          changed = true;
        }
      }
    }
    for (int s = 0; s < steps; ++s) {
      const NetStep& step = plan.steps[s];
      layers_[step.layer_id]->SetHalfStorage(runs_half(s), step.top_ids.size() == 1 && half_blob[step.top_ids[0]] != 0);
    }
  }

  // ---- lifetimes over the fused schedule ----
  const int num_steps = static_cast<int>(plan.steps.size());
  std::vector<int> last_use(num_blobs, -1);
  for (int s = 0; s < num_steps; ++s) {
    for (int b : plan.steps[s].bottom_ids) last_use[b] = std::max(last_use[b], s);
    for (int b : plan.steps[s].top_ids) last_use[b] = std::max(last_use[b], s);
  }
  for (int b = 0; b < num_blobs; ++b) {
    if (plan.visible[b]) last_use[b] = num_steps;
  }

  // ---- greedy storage sharing ----
  std::multimap<size_t, Blob*> retired;
  std::vector<bool> released(num_blobs, false);
  for (int s = 0; s < num_steps; ++s) {
    NetStep& step = plan.steps[s];
    std::vector<Blob*> temps = layers_[step.layer_id]->GetTempBlobs();
    std::vector<std::pair<size_t, Blob*> > need;
    for (Blob* t : temps) {
      t->ResetMemory();
      need.push_back(std::make_pair(static_cast<size_t>(t->count()), t));
    }
    for (Blob* t : step.tops) {
      if (std::find(step.bottoms.begin(), step.bottoms.end(), t) != step.bottoms.end()) continue;  // in place
      t->ResetMemory();
      need.push_back(std::make_pair(static_cast<size_t>(t->count()), t));
    }
    std::sort(need.begin(), need.end(),
              [](const std::pair<size_t, Blob*>& a, const std::pair<size_t, Blob*>& b) { return a.first > b.first; });
    for (auto& item : need) {
      auto it = retired.lower_bound(item.first);
      if (it != retired.end() && it->first <= item.first * 2) {
        item.second->ShareData(*it->second);
        retired.erase(it);
      }
    }
    for (int b : step.bottom_ids) {
      if (!released[b] && last_use[b] <= s) {
        released[b] = true;
        retired.insert(std::make_pair(static_cast<size_t>(blobs_[b]->capacity()), blobs_[b].get()));
      }
    }
    for (Blob* t : temps) retired.insert(std::make_pair(static_cast<size_t>(t->capacity()), t));
  }

  plan.input_shapes.clear();
  for (Blob* b : top_vecs_[0]) plan.input_shapes.push_back(b->shape());
  plan.valid = true;
}

void Net::Forward(bool reshape) {
  NetPlan& plan = *plan_;
  if (reshape || !plan.valid) {
    bool stale = !plan.valid || plan.input_shapes.size() != top_vecs_[0].size();
    for (size_t i = 0; !stale && i < top_vecs_[0].size(); ++i) stale = top_vecs_[0][i]->shape() != plan.input_shapes[i];
    if (stale) PlaceMemory();
  }
  Context& ctx = Context::Get();
  ctx.Activate();
  Profiler* profiler = Profiler::Get();
  const bool profiling = profiler->running();
  for (NetStep& step : plan.steps) {
    if (profiling) profiler->ScopeStart(layer_names_[step.layer_id].c_str());
    layers_[step.layer_id]->Forward(step.bottoms, step.tops);
    if (profiling) {
      ctx.Sync();  // scopes then measure execution, not just launches
      profiler->ScopeEnd();
    }
  }
  // As in the reference: return with the last layer's tops on the host.
  if (profiling) profiler->ScopeStart("Sync");
  const NetStep& last = plan.steps.back();
  for (Blob* b : last.tops) b->cpu_data();
  ctx.SyncAndCheck();
  if (profiling) profiler->ScopeEnd();
}

// ---------------------------------------------------------------- weights / outputs

void Net::CopyTrainedLayersFrom(const NetParameter& param) {
  for (int i = 0; i < param.layer_size(); ++i) {
    const LayerParameter& source = param.layer(i);
    auto it = layer_names_index_.find(source.name());
    if (it == layer_names_index_.end()) continue;  // layers the net does not have are skipped
    // Several layers may carry the same name; the reference takes the first.
    int target = 0;
    while (layer_names_[target] != source.name()) ++target;
    vector<shared_ptr<Blob> >& target_blobs = layers_[target]->blobs();
    CHECK_EQ(static_cast<int>(target_blobs.size()), source.blobs_size())
        << "Incompatible number of blobs for layer " << source.name();
    for (size_t j = 0; j < target_blobs.size(); ++j) {
      if (!target_blobs[j]->ShapeEquals(source.blobs(static_cast<int>(j)))) {
        Blob source_blob;
        source_blob.FromProto(source.blobs(static_cast<int>(j)), true);
        LOG(FATAL) << "Cannot copy param " << j << " weights from layer '" << source.name()
                   << "'; shape mismatch.  Source param shape is " << source_blob.shape_string()
                   << "; target param shape is " << target_blobs[j]->shape_string() << ". "
                   << "To learn this layer's parameters from scratch rather than copying from a saved net, rename "
                      "the layer.";
      }
      target_blobs[j]->FromProto(source.blobs(static_cast<int>(j)), false);
    }
  }
}

void Net::CopyTrainedLayersFrom(const string& trained_filename) {
  NetParameter param;
  ReadNetParamsFromBinaryFileOrDie(trained_filename, &param);
  CopyTrainedLayersFrom(param);
}

void Net::MarkOutputs(const std::vector<std::string>& outs) {
  for (const std::string& name : outs) {
    auto it = blob_names_index_.find(name);
    if (it == blob_names_index_.end()) LOG(FATAL) << "blob (" << name << ") is not availiable in Net";
    blob_life_time_[it->second] = static_cast<int>(layers_.size());
  }
  plan_->valid = false;  // fusion and sharing depend on the visible set
}

void Net::ToProto(NetParameter* param) const {
  param->Clear();
  param->set_name(name_);
  for (size_t i = 0; i < layers_.size(); ++i) layers_[i]->ToProto(param->add_layer());
}

bool Net::has_blob(const string& blob_name) const {
  return blob_names_index_.find(blob_name) != blob_names_index_.end();
}

const shared_ptr<Blob> Net::blob_by_name(const string& blob_name) const {
  CHECK(has_blob(blob_name)) << "Unknown blob name " << blob_name;
  return blobs_[blob_names_index_.find(blob_name)->second];
}

// ---------------------------------------------------------------- readers

shared_ptr<NetParameter> ReadTextNetParameterFromFile(const string& file) {
  shared_ptr<NetParameter> np(new NetParameter);
  ReadNetParamsFromTextFileOrDie(file, np.get());
  return np;
}

shared_ptr<NetParameter> ReadTextNetParameterFromBuffer(const char* buffer, int buffer_len) {
  shared_ptr<NetParameter> np(new NetParameter);
  CHECK(google::protobuf::TextFormat::ParseFromString(std::string(buffer, buffer_len), np.get()))
      << "Parse Text NetParameter from Buffer failed";
  UpgradeNetAsNeeded("<buffer>", np.get());
  return np;
}

shared_ptr<NetParameter> ReadBinaryNetParameterFromFile(const string& file) {
  shared_ptr<NetParameter> np(new NetParameter);
  ReadNetParamsFromBinaryFileOrDie(file, np.get());
  return np;
}

shared_ptr<NetParameter> ReadBinaryNetParameterFromBuffer(const char* buffer, int buffer_len) {
  shared_ptr<NetParameter> np(new NetParameter);
  CHECK(np->ParseFromArray(buffer, buffer_len)) << "Parse Binary NetParameter from Buffer failed";
  UpgradeNetAsNeeded("<buffer>", np.get());
  return np;
}

}  // namespace caffe
