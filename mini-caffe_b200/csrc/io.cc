#include "io.h"

#include <fcntl.h>
#include <unistd.h>

#include <fstream>

#include "google/protobuf/io/zero_copy_stream_impl.h"
#include "google/protobuf/text_format.h"

namespace caffe {

using google::protobuf::io::FileInputStream;
using google::protobuf::io::FileOutputStream;

bool ReadProtoFromTextFile(const char* filename, Message* proto) {
  int fd = open(filename, O_RDONLY);
  CHECK_NE(fd, -1) << "File not found: " << filename;
  FileInputStream input(fd);
  bool ok = google::protobuf::TextFormat::Parse(&input, proto);
  close(fd);
  return ok;
}

bool ReadProtoFromBinaryFile(const char* filename, Message* proto) {
  int fd = open(filename, O_RDONLY);
  CHECK_NE(fd, -1) << "File not found: " << filename;
  FileInputStream input(fd);
  const std::string& bytes = input.ReadAll();
  bool ok = proto->ParseFromArray(bytes.data(), static_cast<int>(bytes.size()));
  close(fd);
  return ok;
}

void ReadProtoFromBinaryFileOrDie(const char* filename, Message* proto) {
  CHECK(ReadProtoFromBinaryFile(filename, proto)) << "Failed to parse file: " << filename;
}

void WriteProtoToTextFile(const Message& proto, const char* filename) {
  int fd = open(filename, O_WRONLY | O_CREAT | O_TRUNC, 0644);
  CHECK_NE(fd, -1) << "Cannot open for writing: " << filename;
  FileOutputStream output(fd);
  CHECK(google::protobuf::TextFormat::Print(proto, &output));
  close(fd);
}

void WriteProtoToBinaryFile(const Message& proto, const char* filename) {
  std::fstream output(filename, std::ios::out | std::ios::trunc | std::ios::binary);
  CHECK(proto.SerializeToOstream(&output)) << "Cannot write: " << filename;
}

static void UpgradeNetInput(NetParameter* net) {
  const bool has_shape = net->input_shape_size() > 0;
  const bool has_dim = net->input_dim_size() > 0;
  if (has_shape || has_dim) {
    if (has_shape) {
      CHECK_EQ(net->input_shape_size(), net->input_size()) << "one input_shape per input is required";
    } else {
      CHECK_EQ(net->input_dim_size(), 4 * net->input_size()) << "four input_dim values per input are required";
    }
    LayerParameter input_layer;
    input_layer.set_name("input");
    input_layer.set_type("Input");
    InputParameter* ip = input_layer.mutable_input_param();
    for (int i = 0; i < net->input_size(); ++i) {
      input_layer.add_top(net->input(i));
      BlobShape* shape = ip->add_shape();
      if (has_shape) {
        shape->CopyFrom(net->input_shape(i));
      } else {
        for (int j = 4 * i; j < 4 * i + 4; ++j) shape->add_dim(net->input_dim(j));
      }
    }
    // The new layer goes first so that every later layer finds its bottoms.
    NetParameter reordered;
    reordered.add_layer()->CopyFrom(input_layer);
    for (int i = 0; i < net->layer_size(); ++i) reordered.add_layer()->CopyFrom(net->layer(i));
    net->clear_layer();
    for (int i = 0; i < reordered.layer_size(); ++i) net->add_layer()->CopyFrom(reordered.layer(i));
  }
  net->clear_input();
  net->clear_input_shape();
  net->clear_input_dim();
}

namespace {

// Type string of the current format for a V1 enumerator (the number is the wire value of
// V1LayerParameter.LayerType).  Only the types the V1 format shares with this project's schema
// appear; anything else is an error, as in src/util/upgrade_proto.cpp:210-262.
const char* V1TypeName(int type) {
  static const struct { int value; const char* name; } kNames[] = {
      {0, ""},          {35, "AbsVal"},      {2, "BNLL"},     {3, "Concat"},        {4, "Convolution"},
      {39, "Deconvolution"}, {6, "Dropout"}, {25, "Eltwise"}, {38, "Exp"},          {8, "Flatten"},
      {14, "InnerProduct"},  {15, "LRN"},    {34, "MVN"},     {17, "Pooling"},      {26, "Power"},
      {18, "ReLU"},     {19, "Sigmoid"},     {20, "Softmax"}, {22, "Split"},        {33, "Slice"},
      {23, "TanH"},     {31, "Threshold"},
  };
  for (const auto& entry : kNames)
    if (entry.value == type) return entry.name;
  LOG(FATAL) << "Unknown V1LayerParameter layer type: " << type;
  return "";
}

ParamSpec* ParamAt(LayerParameter* layer, int i) {
  while (layer->param_size() <= i) layer->add_param();
  return layer->mutable_param(i);
}

// One V1 `layers { ... }` entry as a `layer { ... }` entry: same bottoms, tops, name, rules,
// blobs and per-type parameter blocks; the enumerated type becomes its string; the parallel
// per-blob arrays (share name, share mode, learning-rate and decay multipliers) become ParamSpecs.
void UpgradeV1Layer(const V1LayerParameter& v1, LayerParameter* layer) {
  layer->Clear();
  for (int i = 0; i < v1.bottom_size(); ++i) layer->add_bottom(v1.bottom(i));
  for (int i = 0; i < v1.top_size(); ++i) layer->add_top(v1.top(i));
  if (v1.has_name()) layer->set_name(v1.name());
  for (int i = 0; i < v1.include_size(); ++i) layer->add_include()->CopyFrom(v1.include(i));
  for (int i = 0; i < v1.exclude_size(); ++i) layer->add_exclude()->CopyFrom(v1.exclude(i));
  if (v1.has_type()) layer->set_type(V1TypeName(static_cast<int>(v1.type())));
  for (int i = 0; i < v1.blobs_size(); ++i) layer->add_blobs()->CopyFrom(v1.blobs(i));
  for (int i = 0; i < v1.param_size(); ++i) ParamAt(layer, i)->set_name(v1.param(i));
  for (int i = 0; i < v1.blob_share_mode_size(); ++i) {
    const int mode = static_cast<int>(v1.blob_share_mode(i));
    CHECK(mode == 0 || mode == 1) << "Unknown blob_share_mode: " << mode;
    ParamAt(layer, i)->set_share_mode(mode == 0 ? ParamSpec_DimCheckMode_STRICT : ParamSpec_DimCheckMode_PERMISSIVE);
  }
  for (int i = 0; i < v1.blobs_lr_size(); ++i) ParamAt(layer, i)->set_lr_mult(v1.blobs_lr(i));
  for (int i = 0; i < v1.weight_decay_size(); ++i) ParamAt(layer, i)->set_decay_mult(v1.weight_decay(i));
  for (int i = 0; i < v1.loss_weight_size(); ++i) layer->add_loss_weight(v1.loss_weight(i));
#define MCB200_COPY_BLOCK(field) \
  if (v1.has_##field()) layer->mutable_##field()->CopyFrom(v1.field())
  MCB200_COPY_BLOCK(concat_param);
  MCB200_COPY_BLOCK(convolution_param);
  MCB200_COPY_BLOCK(dropout_param);
  MCB200_COPY_BLOCK(eltwise_param);
  MCB200_COPY_BLOCK(exp_param);
  MCB200_COPY_BLOCK(inner_product_param);
  MCB200_COPY_BLOCK(lrn_param);
  MCB200_COPY_BLOCK(mvn_param);
  MCB200_COPY_BLOCK(pooling_param);
  MCB200_COPY_BLOCK(power_param);
  MCB200_COPY_BLOCK(relu_param);
  MCB200_COPY_BLOCK(sigmoid_param);
  MCB200_COPY_BLOCK(softmax_param);
  MCB200_COPY_BLOCK(slice_param);
  MCB200_COPY_BLOCK(tanh_param);
  MCB200_COPY_BLOCK(threshold_param);
  MCB200_COPY_BLOCK(loss_param);
#undef MCB200_COPY_BLOCK
}

// `layers { type: ENUM }` entries (the V1 format) become `layer { type: "String" }` entries in
// the same order (src/util/upgrade_proto.cpp:61-82).  A file that mixes both is refused.
void UpgradeV1Net(const string& source, NetParameter* net) {
  CHECK_EQ(net->layer_size(), 0)
      << source << ": refusing to upgrade an inconsistent net definition: it has both 'layer' and 'layers' "
      << "fields. The current format is layer { type: 'Layer' ... }, not layers { type: LAYER ... }";
  for (int i = 0; i < net->layers_size(); ++i) UpgradeV1Layer(net->layers(i), net->add_layer());
  net->clear_layers();
}

}  // namespace

bool UpgradeNetAsNeeded(const string& source, NetParameter* param) {
  if (param->layers_size() > 0) UpgradeV1Net(source, param);
  if (param->input_size() > 0) UpgradeNetInput(param);
  return true;
}

void ReadNetParamsFromTextFileOrDie(const string& file, NetParameter* param) {
  CHECK(ReadProtoFromTextFile(file.c_str(), param)) << "Failed to parse NetParameter file: " << file;
  UpgradeNetAsNeeded(file, param);
}

void ReadNetParamsFromBinaryFileOrDie(const string& file, NetParameter* param) {
  CHECK(ReadProtoFromBinaryFile(file.c_str(), param)) << "Failed to parse NetParameter file: " << file;
  UpgradeNetAsNeeded(file, param);
}

}  // namespace caffe
