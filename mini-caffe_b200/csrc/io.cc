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

bool UpgradeNetAsNeeded(const string& source, NetParameter* param) {
  CHECK_EQ(param->layers_size(), 0)
      << source << ": V1 'layers { type: ENUM }' definitions are not supported by this engine; "
      << "convert the model to the 'layer { type: \"String\" }' format first";
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
