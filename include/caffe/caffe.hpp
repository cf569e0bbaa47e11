// Umbrella header of the public C++ API.
#ifndef CAFFE_CAFFE_HPP_
#define CAFFE_CAFFE_HPP_

#include "caffe/base.hpp"
#include "caffe/blob.hpp"
#include "caffe/net.hpp"
#include "caffe/profiler.hpp"

#endif  // CAFFE_CAFFE_HPP_
