// Folds Convolution -> BatchNorm -> Scale triples of a trained network into the
// convolution, on disk: the counterpart of mini-caffe's tools/fuse_bn.py (same
// pattern, same output names), built on this library's own reader and writer of
// the prototxt / caffemodel formats.
//
//   fuse_bn --net deploy.prototxt --weight weights.caffemodel
//     -> deploy_nobn.prototxt, weights_nobn.caffemodel
//
// For every Convolution with group == 1 that is directly followed by a BatchNorm
// that uses stored statistics and then a Scale:
//   W'[co] = W[co] * gamma[co] / sqrt(var[co] / f + eps)
//   b'[co] = (b[co] - mean[co] / f) * gamma[co] / sqrt(var[co] / f + eps) + beta[co]
// (f = the BatchNorm layer's third blob, the moving-average factor), the
// convolution gets a bias term and the Scale layer's top name, and the two other
// layers disappear from both files.  (The engine performs the same folding in
// memory when it builds its schedule; this tool is for shipping folded files.)
#include <math.h>
#include <stdio.h>
#include <string.h>

#include <string>
#include <vector>

#include "caffe.pb.h"
#include "io.h"

namespace {

using caffe::BlobProto;
using caffe::LayerParameter;
using caffe::NetParameter;

std::string with_suffix(const std::string& path) {
  const size_t slash = path.find_last_of('/');
  const size_t dot = path.find_last_of('.');
  if (dot == std::string::npos || (slash != std::string::npos && dot < slash)) return path + "_nobn";
  return path.substr(0, dot) + "_nobn" + path.substr(dot);
}

const LayerParameter* find_layer(const NetParameter& net, const std::string& name) {
  for (int i = 0; i < net.layer_size(); ++i)
    if (net.layer(i).name() == name) return &net.layer(i);
  return nullptr;
}

std::vector<double> values(const BlobProto& blob) {
  std::vector<double> v;
  if (blob.double_data_size() > 0) {
    for (int i = 0; i < blob.double_data_size(); ++i) v.push_back(blob.double_data(i));
  } else {
    for (int i = 0; i < blob.data_size(); ++i) v.push_back(blob.data(i));
  }
  return v;
}

void set_blob(BlobProto* blob, const std::vector<int>& shape, const std::vector<double>& v) {
  blob->Clear();
  for (int d : shape) blob->mutable_shape()->add_dim(d);
  for (double x : v) blob->add_data(static_cast<float>(x));
}

std::vector<int> shape_of(const BlobProto& blob) {
  std::vector<int> s;
  if (blob.has_shape()) {
    for (int i = 0; i < blob.shape().dim_size(); ++i) s.push_back(static_cast<int>(blob.shape().dim(i)));
  } else {
    s = {blob.num(), blob.channels(), blob.height(), blob.width()};   // legacy 4-d fields
  }
  return s;
}

}  // namespace

int main(int argc, char* argv[]) {
  std::string net_path, weight_path;
  for (int i = 1; i + 1 < argc; i += 2) {
    if (!strcmp(argv[i], "--net")) net_path = argv[i + 1];
    if (!strcmp(argv[i], "--weight")) weight_path = argv[i + 1];
  }
  if (net_path.empty() || weight_path.empty()) {
    fprintf(stderr, "[Usage]: %s --net net.prototxt --weight net.caffemodel\n", argv[0]);
    return 2;
  }
  try {
    NetParameter net, weights;
    caffe::ReadNetParamsFromTextFileOrDie(net_path, &net);
    caffe::ReadNetParamsFromBinaryFileOrDie(weight_path, &weights);

    NetParameter out_net;
    out_net.CopyFrom(net);
    out_net.clear_layer();
    std::vector<std::string> dropped;           // layers that leave the weight file
    std::vector<LayerParameter> folded_weights;   // replacement weight records, by convolution name

    int i = 0;
    int fused = 0;
    while (i < net.layer_size()) {
      const LayerParameter& conv = net.layer(i);
      const bool pattern = conv.type() == "Convolution" && conv.convolution_param().group() == 1 &&
                           i + 2 < net.layer_size() && net.layer(i + 1).type() == "BatchNorm" &&
                           (!net.layer(i + 1).batch_norm_param().has_use_global_stats() ||
                            net.layer(i + 1).batch_norm_param().use_global_stats()) &&
                           net.layer(i + 2).type() == "Scale";
      const LayerParameter* wc = pattern ? find_layer(weights, conv.name()) : nullptr;
      const LayerParameter* wb = pattern ? find_layer(weights, net.layer(i + 1).name()) : nullptr;
      const LayerParameter* ws = pattern ? find_layer(weights, net.layer(i + 2).name()) : nullptr;
      if (!pattern || !wc || !wb || !ws || wc->blobs_size() < 1 || wb->blobs_size() < 3 || ws->blobs_size() < 1) {
        out_net.add_layer()->CopyFrom(conv);
        ++i;
        continue;
      }
      const LayerParameter& bn = net.layer(i + 1);
      const LayerParameter& scale = net.layer(i + 2);
      printf("fuse (%s, %s, %s)\n", conv.name().c_str(), bn.name().c_str(), scale.name().c_str());

      const std::vector<int> wshape = shape_of(wc->blobs(0));
      std::vector<double> w = values(wc->blobs(0));
      const int cout = wshape[0];
      const size_t per_out = w.size() / static_cast<size_t>(cout);
      std::vector<double> b(cout, 0.0);
      if (conv.convolution_param().bias_term() && wc->blobs_size() > 1) b = values(wc->blobs(1));
      const std::vector<double> mean = values(wb->blobs(0)), var = values(wb->blobs(1));
      const std::vector<double> factor_blob = values(wb->blobs(2));
      const double factor = factor_blob.empty() || factor_blob[0] == 0.0 ? 0.0 : 1.0 / factor_blob[0];
      const std::vector<double> gamma = values(ws->blobs(0));
      std::vector<double> beta(cout, 0.0);
      if (scale.scale_param().bias_term() && ws->blobs_size() > 1) beta = values(ws->blobs(1));
      const double eps = bn.batch_norm_param().eps();
      if (static_cast<int>(mean.size()) != cout || static_cast<int>(var.size()) != cout ||
          static_cast<int>(gamma.size()) != cout || static_cast<int>(beta.size()) != cout ||
          static_cast<int>(b.size()) != cout) {
        fprintf(stderr, "fuse_bn: parameter sizes of (%s, %s, %s) do not match the convolution's %d outputs\n",
                conv.name().c_str(), bn.name().c_str(), scale.name().c_str(), cout);
        return 1;
      }
      for (int co = 0; co < cout; ++co) {
        const double s = gamma[co] / sqrt(var[co] * factor + eps);
        for (size_t j = 0; j < per_out; ++j) w[co * per_out + j] *= s;
        b[co] = (b[co] - mean[co] * factor) * s + beta[co];
      }
      LayerParameter* kept = out_net.add_layer();
      kept->CopyFrom(conv);
      kept->mutable_convolution_param()->set_bias_term(true);
      kept->set_top(0, scale.top(0));
      LayerParameter record;
      record.CopyFrom(*wc);
      record.clear_blobs();
      set_blob(record.add_blobs(), wshape, w);
      set_blob(record.add_blobs(), std::vector<int>(1, cout), b);
      folded_weights.push_back(record);
      dropped.push_back(bn.name());
      dropped.push_back(scale.name());
      i += 3;
      ++fused;
    }

    NetParameter out_weights;
    out_weights.CopyFrom(weights);
    out_weights.clear_layer();
    for (int l = 0; l < weights.layer_size(); ++l) {
      const std::string& name = weights.layer(l).name();
      bool skip = false;
      for (const std::string& d : dropped) skip = skip || d == name;
      if (skip) continue;
      const LayerParameter* replacement = nullptr;
      for (const LayerParameter& r : folded_weights)
        if (r.name() == name) replacement = &r;
      out_weights.add_layer()->CopyFrom(replacement ? *replacement : weights.layer(l));
    }

    const std::string out_net_path = with_suffix(net_path), out_weight_path = with_suffix(weight_path);
    caffe::WriteProtoToTextFile(out_net, out_net_path.c_str());
    caffe::WriteProtoToBinaryFile(out_weights, out_weight_path.c_str());
    printf("%d triples folded; wrote %s and %s\n", fused, out_net_path.c_str(), out_weight_path.c_str());
  } catch (const std::exception& e) {
    fprintf(stderr, "fuse_bn: %s\n", e.what());
    return 1;
  }
  return 0;
}
