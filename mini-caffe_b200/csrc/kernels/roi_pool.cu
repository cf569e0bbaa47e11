// Region-of-interest pooling for the detection heads that follow Proposal:
// ROIPooling (max over an adaptive grid, Fast/Faster R-CNN) and PSROIPooling
// (position-sensitive average, R-FCN).
//
// One thread per output element, feature maps in (N, C, H, W) order as the
// layers define them.  The bin geometry is evaluated with the reference's float
// expressions, operation by operation (explicit IEEE multiplies and adds: the
// reference's CPU build has no fused multiply-add), and a bin is reduced in the
// reference's h-major order, so the results are bit-identical to
// src/layers/roi_pooling_layer.cpp:37-109 and src/layers/psroi_pooling_layer.cpp:45-106.
// The inputs are small (a few hundred rois over a 63 x 38 map) and stay in L2;
// the kernels are latency-bound gathers.
#include <cuda_runtime.h>
#include <float.h>

#include "../../../include/mcb200_kernels.h"
#include "launch_count.h"

namespace mcb200 {
namespace {

__device__ __forceinline__ int clamp_to(int v, int hi) { return min(max(v, 0), hi); }

// rois: [num_rois, 5] = (batch index, x1, y1, x2, y2) in image coordinates.
__global__ void roi_pool_kernel(const float* __restrict__ data, const float* __restrict__ rois,
                                float* __restrict__ out, int num_rois, int batch, int channels, int height, int width,
                                int pooled_h, int pooled_w, float spatial_scale, int* status) {
  const long long total = static_cast<long long>(num_rois) * channels * pooled_h * pooled_w;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int pw = static_cast<int>(i % pooled_w);
    const int ph = static_cast<int>((i / pooled_w) % pooled_h);
    const int c = static_cast<int>((i / (static_cast<long long>(pooled_w) * pooled_h)) % channels);
    const int n = static_cast<int>(i / (static_cast<long long>(pooled_w) * pooled_h * channels));
    const float* roi = rois + static_cast<size_t>(n) * 5;
    const int roi_batch = static_cast<int>(roi[0]);
    if (roi_batch < 0 || roi_batch >= batch) {   // the reference stops with a CHECK failure here
      if (status) atomicExch(status, 3);
      out[i] = 0.f;
      continue;
    }
    // round() of the scaled corner: half away from zero, as the C function.
    const int roi_start_w = static_cast<int>(roundf(__fmul_rn(roi[1], spatial_scale)));
    const int roi_start_h = static_cast<int>(roundf(__fmul_rn(roi[2], spatial_scale)));
    const int roi_end_w = static_cast<int>(roundf(__fmul_rn(roi[3], spatial_scale)));
    const int roi_end_h = static_cast<int>(roundf(__fmul_rn(roi[4], spatial_scale)));
    const int roi_height = max(roi_end_h - roi_start_h + 1, 1);
    const int roi_width = max(roi_end_w - roi_start_w + 1, 1);
    const float bin_h = __fdiv_rn(static_cast<float>(roi_height), static_cast<float>(pooled_h));
    const float bin_w = __fdiv_rn(static_cast<float>(roi_width), static_cast<float>(pooled_w));
    int hstart = static_cast<int>(floorf(__fmul_rn(static_cast<float>(ph), bin_h)));
    int wstart = static_cast<int>(floorf(__fmul_rn(static_cast<float>(pw), bin_w)));
    int hend = static_cast<int>(ceilf(__fmul_rn(static_cast<float>(ph + 1), bin_h)));
    int wend = static_cast<int>(ceilf(__fmul_rn(static_cast<float>(pw + 1), bin_w)));
    hstart = clamp_to(hstart + roi_start_h, height);
    hend = clamp_to(hend + roi_start_h, height);
    wstart = clamp_to(wstart + roi_start_w, width);
    wend = clamp_to(wend + roi_start_w, width);
    const bool empty = hend <= hstart || wend <= wstart;
    const float* plane = data + (static_cast<size_t>(roi_batch) * channels + c) * height * width;
    float best = empty ? 0.f : -FLT_MAX;
    for (int h = hstart; h < hend; ++h) {
      for (int w = wstart; w < wend; ++w) {
        const float v = __ldg(plane + h * width + w);
        best = best < v ? v : best;   // std::max: keeps the earlier of two equal values
      }
    }
    out[i] = best;
  }
}

// data: [batch, output_dim * group * group, H, W]; out: [num_rois, output_dim, group, group].
__global__ void psroi_pool_kernel(const float* __restrict__ data, const float* __restrict__ rois,
                                  float* __restrict__ out, int num_rois, int batch, int output_dim, int group,
                                  int height, int width, float spatial_scale, int* status) {
  const long long total = static_cast<long long>(num_rois) * output_dim * group * group;
  const int channels = output_dim * group * group;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int pw = static_cast<int>(i % group);
    const int ph = static_cast<int>((i / group) % group);
    const int c = static_cast<int>((i / (static_cast<long long>(group) * group)) % output_dim);
    const int n = static_cast<int>(i / (static_cast<long long>(group) * group * output_dim));
    const float* roi = rois + static_cast<size_t>(n) * 5;
    const int roi_batch = static_cast<int>(roi[0]);
    if (roi_batch < 0 || roi_batch >= batch) {
      if (status) atomicExch(status, 3);
      out[i] = 0.f;
      continue;
    }
    // Corners are rounded first, then scaled; the far corner is one pixel further out.
    const float roi_start_w = __fmul_rn(roundf(roi[1]), spatial_scale);
    const float roi_start_h = __fmul_rn(roundf(roi[2]), spatial_scale);
    const float roi_end_w = __fmul_rn(roundf(__fadd_rn(roi[3], 1.f)), spatial_scale);
    const float roi_end_h = __fmul_rn(roundf(__fadd_rn(roi[4], 1.f)), spatial_scale);
    const float span_h = __fsub_rn(roi_end_h, roi_start_h), span_w = __fsub_rn(roi_end_w, roi_start_w);
    const float roi_height = span_h < 0.1f ? 0.1f : span_h;   // rois are at least a tenth of a cell
    const float roi_width = span_w < 0.1f ? 0.1f : span_w;
    const float bin_h = __fdiv_rn(roi_height, static_cast<float>(group));
    const float bin_w = __fdiv_rn(roi_width, static_cast<float>(group));
    int hstart = static_cast<int>(floorf(__fadd_rn(__fmul_rn(static_cast<float>(ph), bin_h), roi_start_h)));
    int wstart = static_cast<int>(floorf(__fadd_rn(__fmul_rn(static_cast<float>(pw), bin_w), roi_start_w)));
    int hend = static_cast<int>(ceilf(__fadd_rn(__fmul_rn(static_cast<float>(ph + 1), bin_h), roi_start_h)));
    int wend = static_cast<int>(ceilf(__fadd_rn(__fmul_rn(static_cast<float>(pw + 1), bin_w), roi_start_w)));
    hstart = clamp_to(hstart, height);
    hend = clamp_to(hend, height);
    wstart = clamp_to(wstart, width);
    wend = clamp_to(wend, width);
    const bool empty = hend <= hstart || wend <= wstart;
    const int map = (c * group + ph) * group + pw;   // the score map of this bin position
    const float* plane = data + (static_cast<size_t>(roi_batch) * channels + map) * height * width;
    float sum = 0.f;
    for (int h = hstart; h < hend; ++h) {
      for (int w = wstart; w < wend; ++w) sum = __fadd_rn(sum, __ldg(plane + h * width + w));
    }
    const int area = (hend - hstart) * (wend - wstart);
    out[i] = empty ? 0.f : __fdiv_rn(sum, static_cast<float>(area));
  }
}

int grid_for_items(long long items, int threads) {
  long long blocks = (items + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return static_cast<int>(blocks < 1 ? 1 : blocks);
}

}  // namespace
}  // namespace mcb200

using namespace mcb200;

extern "C" int mcb200_roi_pool(const float* data_nchw, const float* rois, float* out, int num_rois, int batch,
                               int channels, int height, int width, int pooled_h, int pooled_w, float spatial_scale,
                               int* status, void* stream) {
  if (!data_nchw || !rois || !out || num_rois < 0 || batch < 1 || channels < 1 || height < 1 || width < 1 ||
      pooled_h < 1 || pooled_w < 1)
    return -1;
  if (num_rois == 0) return 0;
  const long long items = static_cast<long long>(num_rois) * channels * pooled_h * pooled_w;
  roi_pool_kernel<<<grid_for_items(items, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      data_nchw, rois, out, num_rois, batch, channels, height, width, pooled_h, pooled_w, spatial_scale, status);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mcb200_psroi_pool(const float* data_nchw, const float* rois, float* out, int num_rois, int batch,
                                 int output_dim, int group_size, int height, int width, float spatial_scale,
                                 int* status, void* stream) {
  if (!data_nchw || !rois || !out || num_rois < 0 || batch < 1 || output_dim < 1 || group_size < 1 || height < 1 ||
      width < 1)
    return -1;
  if (num_rois == 0) return 0;
  const long long items = static_cast<long long>(num_rois) * output_dim * group_size * group_size;
  psroi_pool_kernel<<<grid_for_items(items, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      data_nchw, rois, out, num_rois, batch, output_dim, group_size, height, width, spatial_scale, status);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}
