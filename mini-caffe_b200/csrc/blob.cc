// caffe::Blob on top of the three-copy SyncedMemory.
// Behaviour follows mini-caffe's src/blob.cpp (grow-only Reshape :23-43,
// ShareData / ResetMemory :96-109, ShapeEquals with legacy 4-D shapes :111-131,
// FromProto / ToProto :145-192).
#include "caffe/blob.hpp"

#include <cstring>

#include "caffe.pb.h"
#include "io.h"
#include "syncedmem.h"

namespace caffe {

Blob::Blob(const int num, const int channels, const int height, const int width)
    : count_(0), capacity_(0), own_data_(false) {
  Reshape(num, channels, height, width);
}

Blob::Blob(const vector<int>& shape) : count_(0), capacity_(0), own_data_(false) { Reshape(shape); }

void Blob::Reshape(const int num, const int channels, const int height, const int width) {
  Reshape(vector<int>{num, channels, height, width});
}

void Blob::Reshape(const vector<int>& shape) {
  CHECK_LE(shape.size(), static_cast<size_t>(kMaxBlobAxes));
  long long volume = 1;
  for (size_t i = 0; i < shape.size(); ++i) {
    CHECK_GE(shape[i], 0);
    volume *= shape[i];
    CHECK_LE(volume, 0x7fffffffLL) << "blob size exceeds INT_MAX";
  }
  shape_ = shape;
  count_ = static_cast<int>(volume);
  if (shape_data_) shape_data_.reset();  // rebuilt on the next gpu_shape()
  if (count_ > capacity_) {
    capacity_ = count_;
    own_data_ = true;
    data_.reset(new SyncedMemory(static_cast<size_t>(capacity_) * sizeof(real_t)));
  }
}

void Blob::Reshape(const BlobShape& shape) {
  CHECK_LE(shape.dim_size(), kMaxBlobAxes);
  vector<int> dims(shape.dim_size());
  for (int i = 0; i < shape.dim_size(); ++i) dims[i] = static_cast<int>(shape.dim(i));
  Reshape(dims);
}

void Blob::ReshapeLike(const Blob& other) { Reshape(other.shape()); }

const int* Blob::gpu_shape() const {
  Blob* self = const_cast<Blob*>(this);
  if (!self->shape_data_) {
    self->shape_data_.reset(new SyncedMemory(kMaxBlobAxes * sizeof(int)));
    int* host = static_cast<int*>(self->shape_data_->mutable_cpu_data());
    for (size_t i = 0; i < shape_.size(); ++i) host[i] = shape_[i];
  }
  return static_cast<const int*>(self->shape_data_->gpu_data());
}

const real_t* Blob::cpu_data() const {
  CHECK(data_);
  return static_cast<const real_t*>(data_->cpu_data());
}

real_t* Blob::mutable_cpu_data() {
  CHECK(data_);
  return static_cast<real_t*>(data_->mutable_cpu_data());
}

const real_t* Blob::gpu_data() const {
  CHECK(data_);
  return static_cast<const real_t*>(data_->gpu_data());
}

real_t* Blob::mutable_gpu_data() {
  CHECK(data_);
  return static_cast<real_t*>(data_->mutable_gpu_data());
}

const real_t* Blob::gpu_data_nhwc() const {
  CHECK(data_);
  if (num_axes() > 4) return gpu_data();
  return static_cast<const real_t*>(data_->gpu_data_nhwc(num(), channels(), height(), width()));
}

real_t* Blob::mutable_gpu_data_nhwc() {
  CHECK(data_);
  if (num_axes() > 4) return mutable_gpu_data();
  return static_cast<real_t*>(data_->mutable_gpu_data_nhwc(num(), channels(), height(), width()));
}

const void* Blob::gpu_data_nhwc_bf16() const {
  CHECK(data_);
  CHECK_LE(num_axes(), 4);
  return data_->gpu_data_nhwc_bf16(num(), channels(), height(), width());
}

void* Blob::mutable_gpu_data_nhwc_bf16() {
  CHECK(data_);
  CHECK_LE(num_axes(), 4);
  return data_->mutable_gpu_data_nhwc_bf16(num(), channels(), height(), width());
}

bool Blob::device_is_nhwc() const { return data_ && data_->nhwc_is_freshest(); }

unsigned long long Blob::host_version() const { return data_ ? data_->host_version() : 0; }

void Blob::ShareData(const Blob& other) {
  CHECK_LE(count_, other.capacity_);
  CHECK(other.data_);
  capacity_ = other.capacity_;
  own_data_ = false;
  data_ = other.data_;
}

void Blob::ResetMemory() {
  if (!own_data_) {
    own_data_ = true;
    data_.reset(new SyncedMemory(static_cast<size_t>(capacity_) * sizeof(real_t)));
  }
}

bool Blob::ShapeEquals(const BlobProto& other) {
  if (other.has_num() || other.has_channels() || other.has_height() || other.has_width()) {
    // Legacy files give four extents counted from the last axis (a bias of N
    // values is 1 x 1 x 1 x N).
    return shape_.size() <= 4 && LegacyShape(-4) == other.num() && LegacyShape(-3) == other.channels() &&
           LegacyShape(-2) == other.height() && LegacyShape(-1) == other.width();
  }
  if (static_cast<int>(shape_.size()) != other.shape().dim_size()) return false;
  for (int i = 0; i < other.shape().dim_size(); ++i) {
    if (shape_[i] != other.shape().dim(i)) return false;
  }
  return true;
}

void Blob::CopyFrom(const Blob& source, bool reshape) {
  if (source.count() != count_ || source.shape() != shape_) {
    if (reshape) {
      ReshapeLike(source);
    } else {
      LOG(FATAL) << "Trying to copy blobs of different sizes.";
    }
  }
  if (count_ > 0) std::memcpy(mutable_cpu_data(), source.cpu_data(), sizeof(real_t) * count_);
}

void Blob::FromProto(const BlobProto& proto, bool reshape) {
  if (reshape) {
    vector<int> dims;
    if (proto.has_num() || proto.has_channels() || proto.has_height() || proto.has_width()) {
      dims = {proto.num(), proto.channels(), proto.height(), proto.width()};
    } else {
      dims.resize(proto.shape().dim_size());
      for (int i = 0; i < proto.shape().dim_size(); ++i) dims[i] = static_cast<int>(proto.shape().dim(i));
    }
    Reshape(dims);
  } else {
    CHECK(ShapeEquals(proto)) << "shape mismatch (reshape not set)";
  }
  real_t* dst = mutable_cpu_data();
  if (proto.double_data_size() > 0) {
    CHECK_EQ(count_, proto.double_data_size());
    for (int i = 0; i < count_; ++i) dst[i] = static_cast<real_t>(proto.double_data(i));
  } else {
    CHECK_EQ(count_, proto.data_size());
    if (count_ > 0) std::memcpy(dst, proto.data().data(), sizeof(real_t) * count_);
  }
}

void Blob::ToProto(BlobProto* proto) const {
  proto->clear_shape();
  for (size_t i = 0; i < shape_.size(); ++i) proto->mutable_shape()->add_dim(shape_[i]);
  proto->clear_data();
  proto->clear_diff();
  const real_t* src = cpu_data();
  proto->mutable_data()->Reserve(count_);
  for (int i = 0; i < count_; ++i) proto->add_data(src[i]);
}

const int* BlobInt::cpu_data() const {
  CHECK(data_);
  return static_cast<const int*>(data_->cpu_data());
}

int* BlobInt::mutable_cpu_data() {
  CHECK(data_);
  return static_cast<int*>(data_->mutable_cpu_data());
}

const int* BlobInt::gpu_data() const {
  CHECK(data_);
  return static_cast<const int*>(data_->gpu_data());
}

int* BlobInt::mutable_gpu_data() {
  CHECK(data_);
  return static_cast<int*>(data_->mutable_gpu_data());
}

shared_ptr<Blob> ReadBlobFromFile(const string& file) {
  BlobProto proto;
  ReadProtoFromBinaryFileOrDie(file.c_str(), &proto);
  shared_ptr<Blob> blob(new Blob);
  blob->FromProto(proto);
  return blob;
}

shared_ptr<Blob> ReadBlobFromBuffer(const string& buffer) {
  BlobProto proto;
  CHECK(proto.ParseFromString(buffer)) << "Parse Blob failed";
  // (The reference dereferences an empty shared_ptr here, src/blob.cpp:229-230.)
  shared_ptr<Blob> blob(new Blob);
  blob->FromProto(proto);
  return blob;
}

}  // namespace caffe
