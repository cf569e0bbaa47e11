// Kernels of the layer types beyond the benchmark networks that shipped example
// nets use: Deconvolution (SSH, WGAN generator), Crop, LRN.  All work on
// (N, C, H, W) tensors, one thread per output element; they are correctness
// first (fp32 FMA arithmetic, no tensor cores) and bandwidth- or latency-bound.
#include <cuda_runtime.h>
#include <math.h>

#include "../../../include/mcb200_kernels.h"
#include "launch_count.h"

namespace mcb200 {
namespace {

int grid_for_items(long long items, int threads) {
  long long blocks = (items + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return static_cast<int>(blocks < 1 ? 1 : blocks);
}

// Transposed convolution as a gather: output pixel (y, x) collects input pixel
// ((y + pad - r * dil) / stride, ...) for every tap whose offset divides evenly.
// Weights are [c, cout / group, kh, kw] (input channels first), as Caffe stores
// them for this layer.  Shape fields: n, c, h, w describe the input, ho / wo the output.
__global__ void deconv_direct_kernel(const float* __restrict__ in, const float* __restrict__ w,
                                     const float* __restrict__ bias, float* __restrict__ out, mcb200_conv_shape s) {
  const int cin_g = s.c / s.group;
  const int cout_g = s.cout / s.group;
  const long long total = static_cast<long long>(s.n) * s.cout * s.ho * s.wo;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int ox = static_cast<int>(i % s.wo);
    const int oy = static_cast<int>((i / s.wo) % s.ho);
    const int co = static_cast<int>((i / (static_cast<long long>(s.wo) * s.ho)) % s.cout);
    const int n = static_cast<int>(i / (static_cast<long long>(s.wo) * s.ho * s.cout));
    const int g = co / cout_g;
    const int co_g = co - g * cout_g;
    float acc = 0.f;
    for (int r = 0; r < s.kh; ++r) {
      const int ty = oy + s.pad_h - r * s.dil_h;
      if (ty < 0 || ty % s.stride_h != 0) continue;
      const int iy = ty / s.stride_h;
      if (iy >= s.h) continue;
      for (int q = 0; q < s.kw; ++q) {
        const int tx = ox + s.pad_w - q * s.dil_w;
        if (tx < 0 || tx % s.stride_w != 0) continue;
        const int ix = tx / s.stride_w;
        if (ix >= s.w) continue;
        const float* px = in + ((static_cast<size_t>(n) * s.c + g * cin_g) * s.h + iy) * s.w + ix;
        const float* wk = w + ((static_cast<size_t>(g) * cin_g * cout_g + co_g) * s.kh + r) * s.kw + q;
        for (int ci = 0; ci < cin_g; ++ci) {
          acc = fmaf(px[static_cast<size_t>(ci) * s.h * s.w], __ldg(wk + static_cast<size_t>(ci) * cout_g * s.kh * s.kw),
                     acc);
        }
      }
    }
    if (bias) acc += __ldg(bias + co);
    out[i] = acc;
  }
}

struct CropArgs {
  int num_axes;
  int out_shape[6];
  long long in_stride[6];
  int offset[6];
};

__global__ void crop_kernel(const float* __restrict__ in, float* __restrict__ out, CropArgs a, long long total) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    long long rest = i;
    long long src = 0;
    for (int ax = a.num_axes - 1; ax >= 0; --ax) {
      const int idx = static_cast<int>(rest % a.out_shape[ax]);
      rest /= a.out_shape[ax];
      src += static_cast<long long>(idx + a.offset[ax]) * a.in_stride[ax];
    }
    out[i] = in[src];
  }
}

// scale = k + alpha / size * sum of squares over `size` neighbouring channels; y = x * scale^-beta.
__global__ void lrn_across_channels_kernel(const float* __restrict__ in, float* __restrict__ out, int n, int c, int hw,
                                           int size, float alpha_over_size, float beta, float k) {
  const long long total = static_cast<long long>(n) * c * hw;
  const int pre = (size - 1) / 2;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int p = static_cast<int>(i % hw);
    const int ch = static_cast<int>((i / hw) % c);
    const long long img = i / (static_cast<long long>(hw) * c);
    const float* base = in + img * c * hw + p;
    float sum = 0.f;
    const int lo = max(ch - pre, 0), hi = min(ch - pre + size, c);
    for (int cc = lo; cc < hi; ++cc) {
      const float v = base[static_cast<size_t>(cc) * hw];
      sum = fmaf(v, v, sum);
    }
    const float scale = fmaf(alpha_over_size, sum, k);
    out[i] = in[i] * powf(scale, -beta);
  }
}

// y = x * (1 + alpha * average of squares over a size x size window)^-beta; the
// average divides by the window clipped to the padded plane, as the reference's
// AVE pooling does (src/layers/pooling_layer.cpp:155-178).
__global__ void lrn_within_channel_kernel(const float* __restrict__ in, float* __restrict__ out, long long planes, int h,
                                          int w, int size, float alpha, float beta) {
  const long long total = planes * h * w;
  const int pad = (size - 1) / 2;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int x = static_cast<int>(i % w);
    const int y = static_cast<int>((i / w) % h);
    const float* plane = in + (i / (static_cast<long long>(w) * h)) * h * w;
    int y0 = y - pad, x0 = x - pad;
    const int y1 = min(y0 + size, h + pad), x1 = min(x0 + size, w + pad);
    const float area = static_cast<float>((y1 - y0) * (x1 - x0));
    y0 = max(y0, 0);
    x0 = max(x0, 0);
    float sum = 0.f;
    for (int yy = y0; yy < min(y1, h); ++yy) {
      for (int xx = x0; xx < min(x1, w); ++xx) {
        const float v = plane[yy * w + xx];
        sum = fmaf(v, v, sum);
      }
    }
    out[i] = in[i] * powf(fmaf(alpha, sum / area, 1.f), -beta);
  }
}

// op 0: tanh(x); op 1: 1 / (1 + exp(-x))
// (src/layers/tanh_layer.cpp:10-18, src/layers/sigmoid_layer.cpp:10-22).
__global__ void unary_kernel(const float* __restrict__ x, float* __restrict__ y, long long count, int op) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < count;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float v = x[i];
    y[i] = op == 0 ? tanhf(v) : 1.f / (1.f + expf(-v));
  }
}

// Per-channel mean and variance over the batch and all pixels, turned into the
// scale / shift of y = (x - mean) / sqrt(var + eps).  One block per channel, two
// passes over the channel's elements (mean, then squared deviations).
__global__ void __launch_bounds__(256)
channel_batch_stats_kernel(const float* __restrict__ x, long long per_channel, int channels, int inner, float eps,
                           float* __restrict__ scale, float* __restrict__ shift) {
  __shared__ float partial[8];
  const int c = blockIdx.x;
  auto element = [&](long long j) {
    // j-th element of channel c: (image j / inner, position j % inner)
    const long long img = j / inner, pos = j - img * inner;
    return x[(img * channels + c) * static_cast<long long>(inner) + pos];
  };
  auto block_sum = [&](float v) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();   // partial[] may still be read from the previous reduction
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = v;
    __syncthreads();
    float total = 0.f;
    for (int w = 0; w < 8; ++w) total += partial[w];
    return total;
  };
  float acc = 0.f;
  for (long long j = threadIdx.x; j < per_channel; j += blockDim.x) acc += element(j);
  const float mean = block_sum(acc) / static_cast<float>(per_channel);
  acc = 0.f;
  for (long long j = threadIdx.x; j < per_channel; j += blockDim.x) {
    const float d = element(j) - mean;
    acc = fmaf(d, d, acc);
  }
  const float var = block_sum(acc) / static_cast<float>(per_channel);
  if (threadIdx.x == 0) {
    const float inv_std = 1.f / sqrtf(var + eps);
    scale[c] = inv_std;
    shift[c] = -mean * inv_std;
  }
}

// Deconvolution as a convolution, step 1: the input's pixels spread `stride` apart over a zero
// tensor (channels last, `c_stride` floats per pixel, zero in the pad lanes).  `src` is channels
// last with `c` floats per pixel.  The destination was cleared beforehand.
__global__ void deconv_spread_kernel(const float* __restrict__ src, float* __restrict__ dst, int n, int h, int w, int c,
                                     int c_stride, int stride_h, int stride_w, int hs, int ws) {
  const long long total = static_cast<long long>(n) * h * w * c;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int ch = static_cast<int>(i % c);
    long long t = i / c;
    const int x = static_cast<int>(t % w);
    t /= w;
    const int y = static_cast<int>(t % h);
    const int img = static_cast<int>(t / h);
    dst[((static_cast<size_t>(img) * hs + static_cast<size_t>(y) * stride_h) * ws + static_cast<size_t>(x) * stride_w) * c_stride +
        ch] = src[i];
  }
}

// Step 2: the filter of the equivalent convolution.  Deconvolution weights are [c_in, c_out / g,
// kh, kw]; the convolution from c_in to c_out that computes the same thing over the spread input
// has weights [c_out, c_in / g, kh, kw] with both tap axes reversed.
__global__ void deconv_flip_weights_kernel(const float* __restrict__ w, float* __restrict__ out, int c_in, int c_out,
                                           int group, int kh, int kw) {
  const int cin_g = c_in / group, cout_g = c_out / group;
  const int total = c_out * cin_g * kh * kw;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int s = i % kw;
    const int r = (i / kw) % kh;
    const int ci_local = (i / (kw * kh)) % cin_g;
    const int co = i / (kw * kh * cin_g);
    const int g = co / cout_g;
    const int ci = g * cin_g + ci_local;
    out[i] = w[((static_cast<size_t>(ci) * cout_g + (co - g * cout_g)) * kh + (kh - 1 - r)) * kw + (kw - 1 - s)];
  }
}

}  // namespace
}  // namespace mcb200

using namespace mcb200;

extern "C" int mcb200_deconv_as_conv_shape(const mcb200_conv_shape* deconv, mcb200_conv_shape* conv) {
  if (!deconv || !conv) return -1;
  mcb200_conv_shape d = *deconv;
  if (mcb200_deconv_out_shape(&d) != 0) return -2;
  *conv = d;
  conv->h = (d.h - 1) * d.stride_h + 1;
  conv->w = (d.w - 1) * d.stride_w + 1;
  conv->c_stride = (d.c + 3) / 4 * 4;
  conv->stride_h = conv->stride_w = 1;
  conv->pad_h = d.dil_h * (d.kh - 1) - d.pad_h;
  conv->pad_w = d.dil_w * (d.kw - 1) - d.pad_w;
  if (conv->pad_h < 0 || conv->pad_w < 0) return -3;   // more padding than the filter reaches: the output is a crop
  conv->ho = d.ho;
  conv->wo = d.wo;
  return 0;
}

extern "C" int mcb200_deconv_spread_input(const mcb200_conv_shape* deconv, const float* in_nhwc, float* spread,
                                          void* stream) {
  mcb200_conv_shape c;
  if (!in_nhwc || !spread || mcb200_deconv_as_conv_shape(deconv, &c) != 0) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t bytes = static_cast<size_t>(c.n) * c.h * c.w * c.c_stride * sizeof(float);
  cudaError_t e = cudaMemsetAsync(spread, 0, bytes, st);
  if (e != cudaSuccess) return static_cast<int>(e);
  const long long items = static_cast<long long>(deconv->n) * deconv->h * deconv->w * deconv->c;
  if (items == 0) return 0;
  deconv_spread_kernel<<<grid_for_items(items, 256), 256, 0, st>>>(in_nhwc, spread, deconv->n, deconv->h, deconv->w,
                                                                   deconv->c, c.c_stride, deconv->stride_h,
                                                                   deconv->stride_w, c.h, c.w);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mcb200_deconv_flip_weights(const mcb200_conv_shape* deconv, const float* w_iohw, float* w_oihw,
                                          void* stream) {
  if (!deconv || !w_iohw || !w_oihw || deconv->group < 1 || deconv->c % deconv->group || deconv->cout % deconv->group)
    return -1;
  const int total = deconv->cout * (deconv->c / deconv->group) * deconv->kh * deconv->kw;
  deconv_flip_weights_kernel<<<grid_for_items(total, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      w_iohw, w_oihw, deconv->c, deconv->cout, deconv->group, deconv->kh, deconv->kw);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mcb200_deconv_out_shape(mcb200_conv_shape* s) {
  if (!s || s->kh < 1 || s->kw < 1 || s->stride_h < 1 || s->stride_w < 1 || s->dil_h < 1 || s->dil_w < 1) return -1;
  s->ho = s->stride_h * (s->h - 1) + s->dil_h * (s->kh - 1) + 1 - 2 * s->pad_h;
  s->wo = s->stride_w * (s->w - 1) + s->dil_w * (s->kw - 1) + 1 - 2 * s->pad_w;
  return (s->ho > 0 && s->wo > 0) ? 0 : -1;
}

extern "C" int mcb200_deconv_direct(const mcb200_conv_shape* s, const float* in_nchw, const float* w_iohw,
                                    const float* bias, float* out_nchw, void* stream) {
  if (!s || !in_nchw || !w_iohw || !out_nchw || s->group < 1 || s->c % s->group || s->cout % s->group) return -1;
  const long long items = static_cast<long long>(s->n) * s->cout * s->ho * s->wo;
  if (items <= 0) return 0;
  deconv_direct_kernel<<<grid_for_items(items, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(in_nchw, w_iohw, bias,
                                                                                                 out_nchw, *s);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mcb200_crop(const float* in, float* out, int num_axes, const int* in_shape, const int* out_shape,
                           const int* offsets, void* stream) {
  if (!in || !out || !in_shape || !out_shape || !offsets || num_axes < 1 || num_axes > 6) return -1;
  CropArgs a;
  a.num_axes = num_axes;
  long long stride = 1, total = 1;
  for (int ax = num_axes - 1; ax >= 0; --ax) {
    if (offsets[ax] < 0 || out_shape[ax] < 0 || offsets[ax] + out_shape[ax] > in_shape[ax]) return -2;
    a.out_shape[ax] = out_shape[ax];
    a.offset[ax] = offsets[ax];
    a.in_stride[ax] = stride;
    stride *= in_shape[ax];
    total *= out_shape[ax];
  }
  if (total == 0) return 0;
  crop_kernel<<<grid_for_items(total, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(in, out, a, total);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mcb200_lrn(const float* in_nchw, float* out_nchw, int n, int c, int h, int w, int local_size,
                          float alpha, float beta, float k, int within_channel, void* stream) {
  if (!in_nchw || !out_nchw || n < 0 || c < 1 || h < 1 || w < 1 || local_size < 1 || local_size % 2 == 0) return -1;
  const long long items = static_cast<long long>(n) * c * h * w;
  if (items == 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (within_channel) {
    lrn_within_channel_kernel<<<grid_for_items(items, 256), 256, 0, st>>>(in_nchw, out_nchw,
                                                                           static_cast<long long>(n) * c, h, w,
                                                                           local_size, alpha, beta);
  } else {
    lrn_across_channels_kernel<<<grid_for_items(items, 256), 256, 0, st>>>(in_nchw, out_nchw, n, c, h * w, local_size,
                                                                            alpha / local_size, beta, k);
  }
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mcb200_channel_batch_stats(const float* x, long long count, int channels, int inner, float eps,
                                          float* scale, float* shift, void* stream) {
  if (!x || !scale || !shift || channels < 1 || inner < 1 || count < 0 || count % channels) return -1;
  if (count == 0) return 0;
  channel_batch_stats_kernel<<<channels, 256, 0, static_cast<cudaStream_t>(stream)>>>(x, count / channels, channels, inner,
                                                                                      eps, scale, shift);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mcb200_unary(const float* x, float* y, long long count, int op, void* stream) {
  if (!x || !y || count < 0 || (op != MCB200_UNARY_TANH && op != MCB200_UNARY_SIGMOID)) return -1;
  if (count == 0) return 0;
  unary_kernel<<<grid_for_items(count, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(x, y, count, op);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}
