// caffe::Net -- builds a network from a NetParameter (prototxt), loads weights
// from a caffemodel and runs the forward pass.  The interface follows
// mini-caffe's include/caffe/net.hpp:23-159.
//
// Behaviour callers can rely on (same as the reference, src/net.cpp):
//  * layers run in the order of the prototxt; the first layer must be "Input"
//    (legacy `input:` fields are upgraded to one);
//  * after Forward() the blobs guaranteed to hold valid data are the tops of
//    the Input layer, the tops of the last layer and every blob passed to
//    MarkOutputs(); other intermediate blobs may share storage or may never be
//    materialised because their producer was fused into a neighbour;
//  * Forward() returns with the last layer's tops already copied to host memory.
#ifndef CAFFE_NET_HPP_
#define CAFFE_NET_HPP_

#include <map>
#include <set>
#include <string>
#include <utility>
#include <vector>

#include "caffe/blob.hpp"

namespace caffe {

class Layer;
class NetParameter;
struct NetPlan;

class CAFFE_API Net {
 public:
  explicit Net(const string& param_file);
  explicit Net(const NetParameter& param);
  ~Net();

  /*! \brief create the layers of `param` and wire their blobs */
  void Init(const NetParameter& param);

  /*!
   * \brief run every layer once
   * \param reshape propagate the current input shapes through the net first
   *        (needed after an input blob was reshaped; cheap when nothing changed)
   */
  void Forward(bool reshape = true);

  /*! \brief recompute every blob shape from the input shapes */
  void Reshape();

  /*! \brief copy parameter blobs from layers of the same name */
  void CopyTrainedLayersFrom(const NetParameter& param);
  void CopyTrainedLayersFrom(const string& trained_filename);
  /*! \brief serialize layer definitions and parameters */
  void ToProto(NetParameter* param) const;

  const string& name() const { return name_; }
  const vector<string>& blob_names() const { return blob_names_; }
  const vector<string>& param_names() const { return param_display_names_; }
  const vector<shared_ptr<Blob> >& blobs() const { return blobs_; }
  const vector<shared_ptr<Blob> >& params() const { return params_; }
  const vector<vector<Blob*> >& bottom_vecs() const { return bottom_vecs_; }
  const vector<vector<Blob*> >& top_vecs() const { return top_vecs_; }
  const vector<vector<int> >& param_id_vecs() const { return param_id_vecs_; }
  const vector<int>& top_ids(int i) const {
    CHECK_GE(i, 0) << "Invalid layer id";
    CHECK_LT(i, static_cast<int>(top_id_vecs_.size())) << "Invalid layer id";
    return top_id_vecs_[i];
  }
  const vector<int>& bottom_ids(int i) const {
    CHECK_GE(i, 0) << "Invalid layer id";
    CHECK_LT(i, static_cast<int>(bottom_id_vecs_.size())) << "Invalid layer id";
    return bottom_id_vecs_[i];
  }
  bool has_blob(const string& blob_name) const;
  const shared_ptr<Blob> blob_by_name(const string& blob_name) const;

  /*! \brief keep these blobs valid after Forward() */
  void MarkOutputs(const std::vector<std::string>& outs);

 protected:
  void AppendTop(const NetParameter& param, const int layer_id, const int top_id,
                 std::set<string>* available_blobs, std::map<string, int>* blob_name_to_idx);
  int AppendBottom(const NetParameter& param, const int layer_id, const int bottom_id,
                   std::set<string>* available_blobs, std::map<string, int>* blob_name_to_idx);
  void AppendParam(const NetParameter& param, const int layer_id, const int param_id);
  /*! \brief (re)build the execution plan: fusion, blob lifetimes, storage sharing */
  void PlaceMemory();

  string name_;
  vector<shared_ptr<Layer> > layers_;
  vector<string> layer_names_;
  std::map<string, int> layer_names_index_;
  vector<shared_ptr<Blob> > blobs_;
  vector<string> blob_names_;
  vector<int> blob_life_time_;
  std::map<string, int> blob_names_index_;
  vector<shared_ptr<Blob> > params_;
  vector<string> param_display_names_;
  vector<vector<int> > param_id_vecs_;
  std::map<string, int> param_names_index_;
  vector<vector<Blob*> > bottom_vecs_;
  vector<vector<int> > bottom_id_vecs_;
  vector<vector<Blob*> > top_vecs_;
  vector<vector<int> > top_id_vecs_;
  /*! \brief fused execution schedule; rebuilt when shapes or outputs change */
  NetPlan* plan_;
  DISABLE_COPY_AND_ASSIGN(Net);
};

/*! \brief parse a prototxt */
CAFFE_API shared_ptr<NetParameter> ReadTextNetParameterFromFile(const string& file);
CAFFE_API shared_ptr<NetParameter> ReadTextNetParameterFromBuffer(const char* buffer, int buffer_len);
/*! \brief parse a caffemodel / binaryproto */
CAFFE_API shared_ptr<NetParameter> ReadBinaryNetParameterFromFile(const string& file);
CAFFE_API shared_ptr<NetParameter> ReadBinaryNetParameterFromBuffer(const char* buffer, int buffer_len);

}  // namespace caffe

#endif  // CAFFE_NET_HPP_
