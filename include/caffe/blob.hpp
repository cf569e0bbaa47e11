// caffe::Blob -- the N-dimensional fp32 tensor of the public API.
//
// The interface (shape queries, legacy num/channels/height/width accessors,
// cpu_data / gpu_data and their mutable forms, FromProto / ToProto, ShareData,
// ResetMemory, BlobInt) follows mini-caffe's include/caffe/blob.hpp:25-266 so
// callers compile unchanged.  What a caller sees through cpu_data() and
// gpu_data() is always the row-major (N, C, H, W) order Caffe defines.
//
// Inside the engine a 4-D blob can additionally hold a channels-last
// (N, H, W, C) copy on the device, which is what the tensor-core kernels read
// and write; the blob tracks which copies are current and converts on demand
// (see the *_nhwc accessors at the end of the class).
#ifndef CAFFE_BLOB_HPP_
#define CAFFE_BLOB_HPP_

#include <algorithm>
#include <sstream>
#include <string>
#include <vector>

#include "caffe/base.hpp"

const int kMaxBlobAxes = 32;

namespace caffe {

class BlobShape;
class BlobProto;
class SyncedMemory;

class CAFFE_API Blob {
 public:
  Blob() : count_(0), capacity_(0), own_data_(false) {}
  /*! \brief legacy 4-D constructor */
  explicit Blob(const int num, const int channels, const int height, const int width);
  explicit Blob(const vector<int>& shape);
  virtual ~Blob() {}

  /*! \brief legacy 4-D reshape */
  void Reshape(const int num, const int channels, const int height, const int width);
  /*!
   * \brief set the shape; storage grows when the new element count exceeds the
   *        capacity and is never shrunk.  Growing invalidates data pointers.
   */
  void Reshape(const vector<int>& shape);
  void Reshape(const BlobShape& shape);
  void ReshapeLike(const Blob& other);

  std::string shape_string() const {
    std::ostringstream os;
    for (size_t i = 0; i < shape_.size(); ++i) os << shape_[i] << " ";
    os << "(" << count_ << ")";
    return os.str();
  }
  const vector<int>& shape() const { return shape_; }
  /*! \brief extent of one axis; negative indices count from the end */
  int shape(int index) const { return shape_[CanonicalAxisIndex(index)]; }
  int num_axes() const { return static_cast<int>(shape_.size()); }
  int count() const { return count_; }
  int capacity() const { return capacity_; }

  /*! \brief product of the extents of axes [start_axis, end_axis) */
  int count(int start_axis, int end_axis) const {
    CHECK_LE(start_axis, end_axis);
    CHECK_GE(start_axis, 0);
    CHECK_GE(end_axis, 0);
    CHECK_LE(start_axis, num_axes());
    CHECK_LE(end_axis, num_axes());
    int volume = 1;
    for (int i = start_axis; i < end_axis; ++i) volume *= shape(i);
    return volume;
  }
  /*! \brief product of the extents from start_axis to the last axis */
  int count(int start_axis) const { return count(start_axis, num_axes()); }

  /*! \brief map an axis index in [-num_axes, num_axes) to [0, num_axes) */
  int CanonicalAxisIndex(int axis_index) const {
    CHECK_GE(axis_index, -num_axes()) << "axis " << axis_index << " out of range for " << num_axes()
                                      << "-D Blob with shape " << shape_string();
    CHECK_LT(axis_index, num_axes()) << "axis " << axis_index << " out of range for " << num_axes()
                                     << "-D Blob with shape " << shape_string();
    return axis_index < 0 ? axis_index + num_axes() : axis_index;
  }

  int num() const { return LegacyShape(0); }
  int channels() const { return LegacyShape(1); }
  int height() const { return LegacyShape(2); }
  int width() const { return LegacyShape(3); }
  /*! \brief 4-D view of a blob with at most four axes; missing axes read as 1 */
  int LegacyShape(int index) const {
    CHECK_LE(num_axes(), 4) << "Cannot use legacy accessors on Blobs with > 4 axes.";
    CHECK_LT(index, 4);
    CHECK_GE(index, -4);
    if (index >= num_axes() || index < -num_axes()) return 1;
    return shape(index);
  }

  int offset(const int n, const int c = 0, const int h = 0, const int w = 0) const {
    return ((n * channels() + c) * height() + h) * width() + w;
  }
  int offset(const vector<int>& indices) const {
    CHECK_LE(indices.size(), static_cast<size_t>(num_axes()));
    int off = 0;
    for (int i = 0; i < num_axes(); ++i) {
      off *= shape(i);
      if (static_cast<int>(indices.size()) > i) {
        CHECK_GE(indices[i], 0);
        CHECK_LT(indices[i], shape(i));
        off += indices[i];
      }
    }
    return off;
  }

  /*! \brief copy values (through host memory) from a blob of the same size */
  void CopyFrom(const Blob& source, bool reshape = false);

  real_t data_at(const int n, const int c = 0, const int h = 0, const int w = 0) const {
    return cpu_data()[offset(n, c, h, w)];
  }
  real_t data_at(const vector<int>& index) const { return cpu_data()[offset(index)]; }

  const int* gpu_shape() const;
  const real_t* cpu_data() const;
  const real_t* gpu_data() const;
  real_t* mutable_cpu_data();
  real_t* mutable_gpu_data();

  void FromProto(const BlobProto& proto, bool reshape = true);
  void ToProto(BlobProto* proto) const;

  /*! \brief use the storage of `other` (which must be large enough) */
  void ShareData(const Blob& other);
  bool ShapeEquals(const BlobProto& other);

  std::string name() { return name_; }
  void set_name(std::string name) { name_ = name; }

  /*! \brief stop sharing: take a private storage object of the current capacity */
  void ResetMemory();

  // ---- engine extensions (not part of mini-caffe's interface) ----

  /*!
   * \brief channels-last device copy (N, H, W, C) of a blob with at most four
   *        axes, converting from the current copy if needed.  For blobs whose
   *        two orders coincide (C == 1 or H*W == 1) this is gpu_data().
   */
  const real_t* gpu_data_nhwc() const;
  /*! \brief channels-last device buffer to be overwritten; other copies become stale */
  real_t* mutable_gpu_data_nhwc();
  /*!
   * \brief channels-last device copy rounded to bfloat16 (16-bit cells), made from
   *        the current fp32 values on first use; written and read by the tensor-core
   *        convolutions of a net built with bfloat16 storage.  Every other accessor
   *        widens it back to fp32 first, so callers never see it.
   */
  const void* gpu_data_nhwc_bf16() const;
  void* mutable_gpu_data_nhwc_bf16();
  /*! \brief true when the freshest device copy is the channels-last one */
  bool device_is_nhwc() const;
  /*! \brief counter that advances whenever host code may have written the data */
  unsigned long long host_version() const;
  const shared_ptr<SyncedMemory>& data() const { return data_; }

 protected:
  shared_ptr<SyncedMemory> data_;
  shared_ptr<SyncedMemory> shape_data_;
  vector<int> shape_;
  int count_;
  int capacity_;
  std::string name_;
  bool own_data_;

  DISABLE_COPY_AND_ASSIGN(Blob);
};

/*! \brief read a serialized BlobProto (.binaryproto) */
CAFFE_API shared_ptr<Blob> ReadBlobFromFile(const string& file);
CAFFE_API shared_ptr<Blob> ReadBlobFromBuffer(const string& buffer);

/*! \brief a Blob whose 32-bit cells are read as int */
class CAFFE_API BlobInt : public Blob {
 public:
  BlobInt() : Blob() {}
  explicit BlobInt(const int num, const int channels, const int height, const int width)
      : Blob(num, channels, height, width) {}
  explicit BlobInt(const vector<int>& shape) : Blob(shape) {}

  int data_at(const int n, const int c = 0, const int h = 0, const int w = 0) const {
    return cpu_data()[offset(n, c, h, w)];
  }
  int data_at(const vector<int>& index) const { return cpu_data()[offset(index)]; }

  const int* cpu_data() const;
  const int* gpu_data() const;
  int* mutable_cpu_data();
  int* mutable_gpu_data();

  void FromProto(const BlobProto& proto, bool reshape = true) = delete;
  void ToProto(BlobProto* proto) const = delete;

 protected:
  DISABLE_COPY_AND_ASSIGN(BlobInt);
};

}  // namespace caffe

#endif  // CAFFE_BLOB_HPP_
