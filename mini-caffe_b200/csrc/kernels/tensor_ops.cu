// HBM-bound kernels: layout conversion, per-channel affine + activation,
// eltwise, pooling, softmax, block copies, permute, channel L2 normalisation.
// All are one pass over their data with coalesced (mostly 128-bit) accesses;
// grids are capped at a multiple of the SM count and loop with a grid stride.
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "../../../include/mcb200_kernels.h"
#include "launch_count.h"

namespace mcb200 {
namespace {

constexpr int kSMs = 148;

inline int grid_for(long long work_items, int threads, int max_blocks_per_sm = 16) {
  long long blocks = (work_items + threads - 1) / threads;
  const long long cap = static_cast<long long>(kSMs) * max_blocks_per_sm;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

inline cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }

// A following launch that uses programmatic dependent launch (the convolution kernels do) may begin
// its set-up once every block of this kernel has got here; it waits with griddepcontrol.wait
// before it touches a tensor, so nothing else changes.
__device__ __forceinline__ void allow_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ float activate(float v, int act, float slope) {
  return (act != 0 && v <= 0.f) ? v * slope : v;
}

// ---------------------------------------------------------------- layout

// One image plane at a time: a [C, HW] -> [HW, c_stride] transpose through a
// 32 x 33 shared tile so that both the read and the write are coalesced.
__global__ void nchw_to_nhwc_kernel(const float* __restrict__ src, float* __restrict__ dst, int c, int hw,
                                    int c_stride) {
  __shared__ float tile[32][33];
  const int n = blockIdx.z;
  const int p0 = blockIdx.x * 32;
  const int c0 = blockIdx.y * 32;
  const float* s = src + static_cast<size_t>(n) * c * hw;
  float* d = dst + static_cast<size_t>(n) * hw * c_stride;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int ch = c0 + i;
    const int p = p0 + threadIdx.x;
    tile[i][threadIdx.x] = (ch < c && p < hw) ? s[static_cast<size_t>(ch) * hw + p] : 0.f;
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int p = p0 + i;
    const int ch = c0 + threadIdx.x;
    if (p < hw && ch < c_stride) d[static_cast<size_t>(p) * c_stride + ch] = tile[threadIdx.x][i];
  }
}

// Up to four channels padded to four (e.g. colour planes in front of the first
// convolution): one thread per pixel, one coalesced read per plane, one
// 16-byte write.
__global__ void nchw_to_nhwc4_kernel(const float* __restrict__ src, float4* __restrict__ dst, int c, int hw,
                                     long long pixels) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < pixels;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long n = i / hw;
    const int p = static_cast<int>(i - n * hw);
    const float* s = src + n * c * hw + p;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    v.x = s[0];
    if (c > 1) v.y = s[hw];
    if (c > 2) v.z = s[2 * static_cast<size_t>(hw)];
    if (c > 3) v.w = s[3 * static_cast<size_t>(hw)];
    dst[i] = v;
  }
}

__global__ void nhwc_to_nchw_kernel(const float* __restrict__ src, float* __restrict__ dst, int c, int hw,
                                    int c_stride) {
  __shared__ float tile[32][33];
  const int n = blockIdx.z;
  const int p0 = blockIdx.x * 32;
  const int c0 = blockIdx.y * 32;
  const float* s = src + static_cast<size_t>(n) * hw * c_stride;
  float* d = dst + static_cast<size_t>(n) * c * hw;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int p = p0 + i;
    const int ch = c0 + threadIdx.x;
    tile[i][threadIdx.x] = (p < hw && ch < c) ? s[static_cast<size_t>(p) * c_stride + ch] : 0.f;
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int ch = c0 + i;
    const int p = p0 + threadIdx.x;
    if (ch < c && p < hw) d[static_cast<size_t>(ch) * hw + p] = tile[threadIdx.x][i];
  }
}

// ---------------------------------------------------------------- affine + activation

struct AffineArgs {
  const float* scale;
  const float* shift;
  const float* prelu;
  int prelu_shared;
  int act;
  float slope;
};

__device__ __forceinline__ float affine_one(float v, int ch, const AffineArgs& a) {
  if (a.scale) v *= __ldg(a.scale + ch);
  if (a.shift) v += __ldg(a.shift + ch);
  float slope = a.slope;
  if (a.act == 2) slope = __ldg(a.prelu + (a.prelu_shared ? 0 : ch));
  return activate(v, a.act, slope);
}

// Four consecutive elements share a channel (inner % 4 == 0) or are four
// consecutive channels (inner == 1, channels % 4 == 0).
template <bool kChannelsLast>
__global__ void affine_vec4_kernel(const float4* __restrict__ x, float4* __restrict__ y, long long count4, int channels,
                                   int inner, AffineArgs a) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < count4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 v = x[i];
    const long long e = i * 4;
    if (kChannelsLast) {
      const int ch = static_cast<int>(e % channels);
      v.x = affine_one(v.x, ch, a);
      v.y = affine_one(v.y, ch + 1, a);
      v.z = affine_one(v.z, ch + 2, a);
      v.w = affine_one(v.w, ch + 3, a);
    } else {
      const int ch = static_cast<int>((e / inner) % channels);
      v.x = affine_one(v.x, ch, a);
      v.y = affine_one(v.y, ch, a);
      v.z = affine_one(v.z, ch, a);
      v.w = affine_one(v.w, ch, a);
    }
    y[i] = v;
  }
}

__global__ void affine_scalar_kernel(const float* __restrict__ x, float* __restrict__ y, long long count, int channels,
                                     int inner, AffineArgs a) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < count;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int ch = static_cast<int>((i / inner) % channels);
    y[i] = affine_one(x[i], ch, a);
  }
}

// ---------------------------------------------------------------- eltwise

struct EltwiseArgs {
  const float* in[MCB200_MAX_ELTWISE_INPUTS];
  float coeff[MCB200_MAX_ELTWISE_INPUTS];
  int num;
  int op;
  int act;
  float slope;
};

__device__ __forceinline__ float eltwise_combine(float acc, float v, float coeff, int op, bool first) {
  if (op == MCB200_ELTWISE_SUM) return first ? coeff * v : acc + coeff * v;
  if (op == MCB200_ELTWISE_PROD) return first ? v : acc * v;
  return first ? v : fmaxf(acc, v);
}

__global__ void eltwise_vec4_kernel(EltwiseArgs a, float4* __restrict__ out, long long count4) {
  allow_dependents();
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < count4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < a.num; ++k) {
      const float4 v = reinterpret_cast<const float4*>(a.in[k])[i];
      acc.x = eltwise_combine(acc.x, v.x, a.coeff[k], a.op, k == 0);
      acc.y = eltwise_combine(acc.y, v.y, a.coeff[k], a.op, k == 0);
      acc.z = eltwise_combine(acc.z, v.z, a.coeff[k], a.op, k == 0);
      acc.w = eltwise_combine(acc.w, v.w, a.coeff[k], a.op, k == 0);
    }
    acc.x = activate(acc.x, a.act, a.slope);
    acc.y = activate(acc.y, a.act, a.slope);
    acc.z = activate(acc.z, a.act, a.slope);
    acc.w = activate(acc.w, a.act, a.slope);
    out[i] = acc;
  }
}

__global__ void eltwise_scalar_kernel(EltwiseArgs a, float* __restrict__ out, long long count) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < count;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < a.num; ++k) acc = eltwise_combine(acc, a.in[k][i], a.coeff[k], a.op, k == 0);
    out[i] = activate(acc, a.act, a.slope);
  }
}

// ---------------------------------------------------------------- pooling

struct PoolArgs {
  int n, h, w, c, kh, kw, sh, sw, ph, pw, ho, wo, method;
};

// One thread per output pixel and group of VEC channels.
template <int VEC>
__global__ void pool_nhwc_kernel(const float* __restrict__ in, float* __restrict__ out, PoolArgs a) {
  allow_dependents();
  const int cg = a.c / VEC;
  const long long total = static_cast<long long>(a.n) * a.ho * a.wo * cg;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int g = static_cast<int>(i % cg);
    long long t = i / cg;
    const int ox = static_cast<int>(t % a.wo);
    t /= a.wo;
    const int oy = static_cast<int>(t % a.ho);
    const int n = static_cast<int>(t / a.ho);
    int y0 = oy * a.sh - a.ph;
    int x0 = ox * a.sw - a.pw;
    float acc[VEC];
    if (a.method == MCB200_POOL_MAX) {
      const int y1 = min(y0 + a.kh, a.h);
      const int x1 = min(x0 + a.kw, a.w);
      y0 = max(y0, 0);
      x0 = max(x0, 0);
#pragma unroll
      for (int v = 0; v < VEC; ++v) acc[v] = -FLT_MAX;
      for (int y = y0; y < y1; ++y) {
        for (int x = x0; x < x1; ++x) {
          const float* p = in + ((static_cast<size_t>(n) * a.h + y) * a.w + x) * a.c + g * VEC;
          if (VEC == 4) {
            const float4 v = *reinterpret_cast<const float4*>(p);
            acc[0] = fmaxf(acc[0], v.x);
            acc[1] = fmaxf(acc[1], v.y);
            acc[2] = fmaxf(acc[2], v.z);
            acc[3] = fmaxf(acc[3], v.w);
          } else {
            acc[0] = fmaxf(acc[0], *p);
          }
        }
      }
    } else {
      int y1 = min(y0 + a.kh, a.h + a.ph);
      int x1 = min(x0 + a.kw, a.w + a.pw);
      const float area = static_cast<float>((y1 - y0) * (x1 - x0));
      y0 = max(y0, 0);
      x0 = max(x0, 0);
      y1 = min(y1, a.h);
      x1 = min(x1, a.w);
#pragma unroll
      for (int v = 0; v < VEC; ++v) acc[v] = 0.f;
      for (int y = y0; y < y1; ++y) {
        for (int x = x0; x < x1; ++x) {
          const float* p = in + ((static_cast<size_t>(n) * a.h + y) * a.w + x) * a.c + g * VEC;
          if (VEC == 4) {
            const float4 v = *reinterpret_cast<const float4*>(p);
            acc[0] += v.x;
            acc[1] += v.y;
            acc[2] += v.z;
            acc[3] += v.w;
          } else {
            acc[0] += *p;
          }
        }
      }
#pragma unroll
      for (int v = 0; v < VEC; ++v) acc[v] /= area;
    }
    float* o = out + ((static_cast<size_t>(n) * a.ho + oy) * a.wo + ox) * a.c + g * VEC;
    if (VEC == 4) {
      *reinterpret_cast<float4*>(o) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    } else {
      *o = acc[0];
    }
  }
}

// A window that covers the whole image (global pooling in front of a classifier: 7 x 7 pixels,
// thousands of channels, one output pixel).  One thread per output would walk the pixels in a
// dependent loop with few threads in all; here a block takes one image and 128 channels, its
// eight warps take every eighth pixel (all loads of a thread are independent), and warp 0 adds
// the eight partial results in a fixed order.
constexpr int kGlobalPoolWarps = 8;

__global__ void __launch_bounds__(32 * kGlobalPoolWarps)
pool_global_kernel(const float4* __restrict__ in, float4* __restrict__ out, int pixels, int cg, int chunks, int method,
                   float area) {
  allow_dependents();
  __shared__ float4 part[kGlobalPoolWarps][32];
  const int n = blockIdx.x / chunks;
  const int g = (blockIdx.x - n * chunks) * 32 + (threadIdx.x & 31);   // group of four channels
  const int w = threadIdx.x >> 5;
  const bool is_max = method == MCB200_POOL_MAX;
  float4 acc = is_max ? make_float4(-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX) : make_float4(0.f, 0.f, 0.f, 0.f);
  if (g < cg) {
    const float4* p = in + static_cast<size_t>(n) * pixels * cg + g;
#pragma unroll 4
    for (int i = w; i < pixels; i += kGlobalPoolWarps) {
      const float4 v = __ldg(p + static_cast<size_t>(i) * cg);
      if (is_max) {
        acc.x = fmaxf(acc.x, v.x);
        acc.y = fmaxf(acc.y, v.y);
        acc.z = fmaxf(acc.z, v.z);
        acc.w = fmaxf(acc.w, v.w);
      } else {
        acc.x += v.x;
        acc.y += v.y;
        acc.z += v.z;
        acc.w += v.w;
      }
    }
  }
  part[w][threadIdx.x & 31] = acc;
  __syncthreads();
  if (w == 0 && g < cg) {
    for (int j = 1; j < kGlobalPoolWarps; ++j) {
      const float4 v = part[j][threadIdx.x];
      if (is_max) {
        acc.x = fmaxf(acc.x, v.x);
        acc.y = fmaxf(acc.y, v.y);
        acc.z = fmaxf(acc.z, v.z);
        acc.w = fmaxf(acc.w, v.w);
      } else {
        acc.x += v.x;
        acc.y += v.y;
        acc.z += v.z;
        acc.w += v.w;
      }
    }
    if (!is_max) {
      acc.x /= area;
      acc.y /= area;
      acc.z /= area;
      acc.w /= area;
    }
    out[static_cast<size_t>(n) * cg + g] = acc;
  }
}

// Max pooling with a K x K window (K = 2, 3), channels % 4 == 0: one thread per
// output pixel and four channels.  All K*K loads are issued before the first
// comparison (taps outside the image read nothing and count as -FLT_MAX), so
// each thread has K*K independent 16-byte requests in flight instead of a
// dependent loop; index arithmetic is 32-bit.
template <int K>
__global__ void pool_max_small_kernel(const float4* __restrict__ in, float4* __restrict__ out, PoolArgs a) {
  allow_dependents();
  const int cg = a.c >> 2;
  const unsigned total = static_cast<unsigned>(a.n) * a.ho * a.wo * cg;
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const unsigned g = i % cg;
    unsigned t = i / cg;
    const int ox = static_cast<int>(t % a.wo);
    t /= a.wo;
    const int oy = static_cast<int>(t % a.ho);
    const unsigned n = t / a.ho;
    const int y0 = oy * a.sh - a.ph;
    const int x0 = ox * a.sw - a.pw;
    const float4* base = in + static_cast<size_t>(n) * a.h * a.w * cg + g;
    float4 v[K * K];
#pragma unroll
    for (int dy = 0; dy < K; ++dy) {
#pragma unroll
      for (int dx = 0; dx < K; ++dx) {
        const int y = y0 + dy, x = x0 + dx;
        const bool inside = y >= 0 && y < a.h && x >= 0 && x < a.w;
        v[dy * K + dx] = inside ? __ldg(base + (static_cast<size_t>(y) * a.w + x) * cg)
                                : make_float4(-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX);
      }
    }
    float4 m = v[0];
#pragma unroll
    for (int j = 1; j < K * K; ++j) {
      m.x = fmaxf(m.x, v[j].x);
      m.y = fmaxf(m.y, v[j].y);
      m.z = fmaxf(m.z, v[j].z);
      m.w = fmaxf(m.w, v[j].w);
    }
    out[i] = m;
  }
}

// The same window maximum over bfloat16 cells, eight channels (16 bytes) per
// thread.  Rounding to bfloat16 is monotonic, so the maximum of rounded values
// is the rounded maximum: a bfloat16 blob pooled here equals the fp32 blob
// pooled and then rounded.  Taps outside the image count as the most negative
// finite bfloat16.
template <int K>
__global__ void pool_max_small_bf16_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, PoolArgs a) {
  const int cg = a.c >> 3;
  const unsigned total = static_cast<unsigned>(a.n) * a.ho * a.wo * cg;
  auto max2 = [](uint32_t p, uint32_t q) {
    uint32_t r;
    asm("max.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(p), "r"(q));
    return r;
  };
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const unsigned g = i % cg;
    unsigned t = i / cg;
    const int ox = static_cast<int>(t % a.wo);
    t /= a.wo;
    const int oy = static_cast<int>(t % a.ho);
    const unsigned n = t / a.ho;
    const int y0 = oy * a.sh - a.ph;
    const int x0 = ox * a.sw - a.pw;
    const uint4* base = in + static_cast<size_t>(n) * a.h * a.w * cg + g;
    uint4 v[K * K];
#pragma unroll
    for (int dy = 0; dy < K; ++dy) {
#pragma unroll
      for (int dx = 0; dx < K; ++dx) {
        const int y = y0 + dy, x = x0 + dx;
        const bool inside = y >= 0 && y < a.h && x >= 0 && x < a.w;
        v[dy * K + dx] = inside ? __ldg(base + (static_cast<size_t>(y) * a.w + x) * cg)
                                : make_uint4(0xFF7FFF7Fu, 0xFF7FFF7Fu, 0xFF7FFF7Fu, 0xFF7FFF7Fu);
      }
    }
    uint4 m = v[0];
#pragma unroll
    for (int j = 1; j < K * K; ++j) {
      m.x = max2(m.x, v[j].x);
      m.y = max2(m.y, v[j].y);
      m.z = max2(m.z, v[j].z);
      m.w = max2(m.w, v[j].w);
    }
    out[i] = m;
  }
}

// ---------------------------------------------------------------- softmax

// inner == 1: one warp per row, the row is streamed three times from L1/L2
// (max, sum of exp, normalise); rows are short (21 ... 1000 values).
__global__ void softmax_rows_kernel(const float* __restrict__ in, float* __restrict__ out, int rows, int channels) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows; row += gridDim.x * warps_per_block) {
    const float* x = in + static_cast<size_t>(row) * channels;
    float* y = out + static_cast<size_t>(row) * channels;
    float m = -FLT_MAX;
    for (int c = lane; c < channels; c += 32) m = fmaxf(m, x[c]);
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float s = 0.f;
    for (int c = lane; c < channels; c += 32) s += expf(x[c] - m);
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    for (int c = lane; c < channels; c += 32) y[c] = expf(x[c] - m) / s;
  }
}

// inner == 1, long rows (a classifier's 1000 scores) and too few of them to fill the GPU with one
// warp each: a block per row, the row held in registers (up to eight values per thread), the two
// reductions through shuffles and one shared array.
constexpr int kSoftmaxBlock = 128;
constexpr int kSoftmaxPerThread = 8;

__device__ __forceinline__ float block_reduce(float v, bool is_max, float* scratch) {
  for (int o = 16; o > 0; o >>= 1) {
    const float u = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, u) : v + u;
  }
  __syncthreads();   // the previous reduction's readers are done with scratch
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = scratch[0];
  for (int j = 1; j < kSoftmaxBlock / 32; ++j) r = is_max ? fmaxf(r, scratch[j]) : r + scratch[j];
  return r;
}

__global__ void __launch_bounds__(kSoftmaxBlock)
softmax_row_block_kernel(const float* __restrict__ in, float* __restrict__ out, int channels) {
  __shared__ float scratch[kSoftmaxBlock / 32];
  const float* x = in + static_cast<size_t>(blockIdx.x) * channels;
  float* y = out + static_cast<size_t>(blockIdx.x) * channels;
  float v[kSoftmaxPerThread];
  float m = -FLT_MAX;
#pragma unroll
  for (int j = 0; j < kSoftmaxPerThread; ++j) {
    const int c = threadIdx.x + j * kSoftmaxBlock;
    v[j] = c < channels ? x[c] : -FLT_MAX;
    m = fmaxf(m, v[j]);
  }
  m = block_reduce(m, true, scratch);
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < kSoftmaxPerThread; ++j) {
    const int c = threadIdx.x + j * kSoftmaxBlock;
    v[j] = c < channels ? expf(v[j] - m) : 0.f;
    s += v[j];
  }
  s = block_reduce(s, false, scratch);
#pragma unroll
  for (int j = 0; j < kSoftmaxPerThread; ++j) {
    const int c = threadIdx.x + j * kSoftmaxBlock;
    if (c < channels) y[c] = v[j] / s;
  }
}

// inner > 1: one thread per (outer, inner) position, walking the channel axis
// with stride `inner`; neighbouring threads touch neighbouring addresses.
__global__ void softmax_strided_kernel(const float* __restrict__ in, float* __restrict__ out, int outer, int channels,
                                       int inner) {
  const long long total = static_cast<long long>(outer) * inner;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long o = i / inner;
    const int s = static_cast<int>(i % inner);
    const float* x = in + (o * channels) * inner + s;
    float* y = out + (o * channels) * inner + s;
    float m = -FLT_MAX;
    for (int c = 0; c < channels; ++c) m = fmaxf(m, x[static_cast<size_t>(c) * inner]);
    float sum = 0.f;
    for (int c = 0; c < channels; ++c) sum += expf(x[static_cast<size_t>(c) * inner] - m);
    for (int c = 0; c < channels; ++c) y[static_cast<size_t>(c) * inner] = expf(x[static_cast<size_t>(c) * inner] - m) / sum;
  }
}

// ---------------------------------------------------------------- copies

__global__ void copy_2d_kernel(const float* __restrict__ src, long long src_pitch, float* __restrict__ dst,
                               long long dst_pitch, long long rows, long long cols) {
  const long long total = rows * cols;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / cols;
    const long long c = i - r * cols;
    dst[r * dst_pitch + c] = src[r * src_pitch + c];
  }
}

__global__ void copy_2d_vec4_kernel(const float4* __restrict__ src, long long src_pitch4, float4* __restrict__ dst,
                                    long long dst_pitch4, long long rows, long long cols4) {
  const long long total = rows * cols4;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / cols4;
    const long long c = i - r * cols4;
    dst[r * dst_pitch4 + c] = src[r * src_pitch4 + c];
  }
}

struct PermuteArgs {
  int num_axes;
  int out_shape[6];
  long long in_stride_of_out_axis[6];
};

__global__ void permute_kernel(const float* __restrict__ in, float* __restrict__ out, long long count, PermuteArgs a) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < count;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    long long rem = i;
    long long src = 0;
    for (int ax = a.num_axes - 1; ax >= 0; --ax) {
      const int idx = static_cast<int>(rem % a.out_shape[ax]);
      rem /= a.out_shape[ax];
      src += idx * a.in_stride_of_out_axis[ax];
    }
    out[i] = in[src];
  }
}

// One warp per pixel: sum of squares by shuffle, then scale.
__global__ void normalize_nhwc_kernel(const float* __restrict__ in, float* __restrict__ out, long long pixels,
                                      int channels, const float* __restrict__ scale, int scale_shared, float eps) {
  allow_dependents();
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (long long p = blockIdx.x * static_cast<long long>(warps_per_block) + (threadIdx.x >> 5); p < pixels;
       p += static_cast<long long>(gridDim.x) * warps_per_block) {
    const float* x = in + p * channels;
    float* y = out + p * channels;
    float ss = 0.f;
    for (int c = lane; c < channels; c += 32) ss += x[c] * x[c];
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float norm = sqrtf(ss + eps);
    for (int c = lane; c < channels; c += 32) y[c] = x[c] / norm * __ldg(scale + (scale_shared ? 0 : c));
  }
}

}  // namespace
}  // namespace mcb200

using namespace mcb200;

extern "C" int mcb200_nchw_to_nhwc(const float* src, float* dst, int n, int c, int h, int w, int c_stride,
                                   void* stream) {
  if (!src || !dst || n < 0 || c < 1 || h < 1 || w < 1 || c_stride < c) return -1;
  if (n == 0) return 0;
  const int hw = h * w;
  if (c <= 4 && c_stride == 4 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
    const long long pixels = static_cast<long long>(n) * hw;
    nchw_to_nhwc4_kernel<<<grid_for(pixels, 256), 256, 0, as_stream(stream)>>>(src, reinterpret_cast<float4*>(dst), c,
                                                                            hw, pixels);
    count_launch();
    return static_cast<int>(cudaGetLastError());
  }
  dim3 grid((hw + 31) / 32, (c_stride + 31) / 32, n);
  if (grid.y > 65535 || grid.z > 65535) return -2;
  nchw_to_nhwc_kernel<<<grid, dim3(32, 8), 0, as_stream(stream)>>>(src, dst, c, hw, c_stride);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mcb200_nhwc_to_nchw(const float* src, float* dst, int n, int c, int h, int w, int c_stride,
                                   void* stream) {
  if (!src || !dst || n < 0 || c < 1 || h < 1 || w < 1 || c_stride < c) return -1;
  if (n == 0) return 0;
  const int hw = h * w;
  dim3 grid((hw + 31) / 32, (c + 31) / 32, n);
  if (grid.y > 65535 || grid.z > 65535) return -2;
  nhwc_to_nchw_kernel<<<grid, dim3(32, 8), 0, as_stream(stream)>>>(src, dst, c, hw, c_stride);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mcb200_channel_affine_act(const float* x, float* y, long long count, int channels, int inner,
                                         const float* scale, const float* shift, const mcb200_epilogue* ep,
                                         void* stream) {
  if (!x || !y || count < 0 || channels < 1 || inner < 1) return -1;
  if (count == 0) return 0;
  AffineArgs a;
  a.scale = scale;
  a.shift = shift;
  a.act = ep ? ep->act : 0;
  a.slope = ep ? ep->slope : 0.f;
  a.prelu = ep ? ep->prelu : nullptr;
  a.prelu_shared = ep ? ep->prelu_shared : 0;
  if (a.act == 2 && !a.prelu) return -2;
  const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0 && count % 4 == 0;
  const int threads = 256;
  if (aligned && inner % 4 == 0) {
    affine_vec4_kernel<false><<<grid_for(count / 4, threads), threads, 0, as_stream(stream)>>>(
        reinterpret_cast<const float4*>(x), reinterpret_cast<float4*>(y), count / 4, channels, inner, a);
  } else if (aligned && inner == 1 && channels % 4 == 0) {
    affine_vec4_kernel<true><<<grid_for(count / 4, threads), threads, 0, as_stream(stream)>>>(
        reinterpret_cast<const float4*>(x), reinterpret_cast<float4*>(y), count / 4, channels, inner, a);
  } else {
    affine_scalar_kernel<<<grid_for(count, threads), threads, 0, as_stream(stream)>>>(x, y, count, channels, inner, a);
  }
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mcb200_eltwise(int op, int num_inputs, const float* const* inputs, const float* coeffs, float* out,
                              long long count, int act, float slope, void* stream) {
  if (!inputs || !out || num_inputs < 1 || num_inputs > MCB200_MAX_ELTWISE_INPUTS || op < 0 || op > 2 || count < 0)
    return -1;
  if (count == 0) return 0;
  EltwiseArgs a;
  a.num = num_inputs;
  a.op = op;
  a.act = act;
  a.slope = slope;
  uintptr_t bits = reinterpret_cast<uintptr_t>(out);
  for (int k = 0; k < num_inputs; ++k) {
    if (!inputs[k]) return -2;
    a.in[k] = inputs[k];
    a.coeff[k] = coeffs ? coeffs[k] : 1.f;
    bits |= reinterpret_cast<uintptr_t>(inputs[k]);
  }
  const int threads = 256;
  if ((bits & 15) == 0 && count % 4 == 0) {
    eltwise_vec4_kernel<<<grid_for(count / 4, threads), threads, 0, as_stream(stream)>>>(
        a, reinterpret_cast<float4*>(out), count / 4);
  } else {
    eltwise_scalar_kernel<<<grid_for(count, threads), threads, 0, as_stream(stream)>>>(a, out, count);
  }
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" void mcb200_pool_out_shape(int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int* ho,
                                      int* wo) {
  // ceil((in + 2*pad - k) / stride) + 1, in float like the reference.
  int oh = static_cast<int>(ceilf(static_cast<float>(h + 2 * ph - kh) / sh)) + 1;
  int ow = static_cast<int>(ceilf(static_cast<float>(w + 2 * pw - kw) / sw)) + 1;
  if (ph || pw) {
    // The last window must start inside the image, not in the padding.
    if ((oh - 1) * sh >= h + ph) --oh;
    if ((ow - 1) * sw >= w + pw) --ow;
  }
  *ho = oh;
  *wo = ow;
}

extern "C" int mcb200_pool_nhwc(const float* in, float* out, int n, int h, int w, int c, int kh, int kw, int sh, int sw,
                                int ph, int pw, int ho, int wo, int method, void* stream) {
  if (!in || !out || n < 0 || h < 1 || w < 1 || c < 1 || kh < 1 || kw < 1 || sh < 1 || sw < 1 || ho < 1 || wo < 1)
    return -1;
  if (method != MCB200_POOL_MAX && method != MCB200_POOL_AVE) return -2;
  if (n == 0) return 0;
  PoolArgs a = {n, h, w, c, kh, kw, sh, sw, ph, pw, ho, wo, method};
  const int threads = 256;
  const bool vec = (c % 4 == 0) && ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  const long long items = static_cast<long long>(n) * ho * wo * (vec ? c / 4 : c);
  const bool small_max = vec && method == MCB200_POOL_MAX && kh == kw && (kh == 2 || kh == 3) &&
                         items < 0x7fffffffLL;
  const bool whole_image = vec && ho == 1 && wo == 1 && ph == 0 && pw == 0 && kh >= h && kw >= w && h * w >= 16 &&
                           static_cast<long long>(n) * ((c / 4 + 31) / 32) < 0x7fffffffLL;
  if (whole_image) {
    const int chunks = (c / 4 + 31) / 32;
    pool_global_kernel<<<n * chunks, 32 * kGlobalPoolWarps, 0, as_stream(stream)>>>(
        reinterpret_cast<const float4*>(in), reinterpret_cast<float4*>(out), h * w, c / 4, chunks, method,
        static_cast<float>(h * w));
  } else if (small_max) {
    const float4* in4 = reinterpret_cast<const float4*>(in);
    float4* out4 = reinterpret_cast<float4*>(out);
    if (kh == 3) {
      pool_max_small_kernel<3><<<grid_for(items, threads, 32), threads, 0, as_stream(stream)>>>(in4, out4, a);
    } else {
      pool_max_small_kernel<2><<<grid_for(items, threads, 32), threads, 0, as_stream(stream)>>>(in4, out4, a);
    }
  } else if (vec) {
    pool_nhwc_kernel<4><<<grid_for(items, threads), threads, 0, as_stream(stream)>>>(in, out, a);
  } else {
    pool_nhwc_kernel<1><<<grid_for(items, threads), threads, 0, as_stream(stream)>>>(in, out, a);
  }
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mcb200_pool_max_nhwc_bf16_supported(int c, int kh, int kw) {
  return (c % 8 == 0 && kh == kw && (kh == 2 || kh == 3)) ? 1 : 0;
}

extern "C" int mcb200_pool_max_nhwc_bf16(const uint16_t* in, uint16_t* out, int n, int h, int w, int c, int kh, int kw,
                                         int sh, int sw, int ph, int pw, int ho, int wo, void* stream) {
  if (!in || !out || n < 0 || h < 1 || w < 1 || c < 1 || sh < 1 || sw < 1 || ho < 1 || wo < 1) return -1;
  if (!mcb200_pool_max_nhwc_bf16_supported(c, kh, kw)) return -2;
  if ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) return -3;
  if (n == 0) return 0;
  PoolArgs a = {n, h, w, c, kh, kw, sh, sw, ph, pw, ho, wo, MCB200_POOL_MAX};
  const long long items = static_cast<long long>(n) * ho * wo * (c / 8);
  if (items >= 0x7fffffffLL) return -4;
  const int threads = 256;
  const uint4* in4 = reinterpret_cast<const uint4*>(in);
  uint4* out4 = reinterpret_cast<uint4*>(out);
  if (kh == 3) {
    pool_max_small_bf16_kernel<3><<<grid_for(items, threads, 32), threads, 0, as_stream(stream)>>>(in4, out4, a);
  } else {
    pool_max_small_bf16_kernel<2><<<grid_for(items, threads, 32), threads, 0, as_stream(stream)>>>(in4, out4, a);
  }
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mcb200_softmax(const float* in, float* out, int outer, int channels, int inner, void* stream) {
  if (!in || !out || outer < 0 || channels < 1 || inner < 1) return -1;
  if (outer == 0) return 0;
  if (inner == 1 && channels > 128 && channels <= kSoftmaxBlock * kSoftmaxPerThread && outer <= 148 * 16 * 8) {
    softmax_row_block_kernel<<<outer, kSoftmaxBlock, 0, as_stream(stream)>>>(in, out, channels);
  } else if (inner == 1) {
    const int threads = 256;
    const int rows_per_block = threads / 32;
    softmax_rows_kernel<<<grid_for((static_cast<long long>(outer) + rows_per_block - 1) / rows_per_block * threads,
                                   threads),
                          threads, 0, as_stream(stream)>>>(in, out, outer, channels);
  } else {
    const int threads = 128;
    softmax_strided_kernel<<<grid_for(static_cast<long long>(outer) * inner, threads), threads, 0,
                             as_stream(stream)>>>(in, out, outer, channels, inner);
  }
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mcb200_copy_2d(const float* src, long long src_pitch, float* dst, long long dst_pitch, long long rows,
                              long long cols, void* stream) {
  if (!src || !dst || rows < 0 || cols < 0 || src_pitch < cols || dst_pitch < cols) return -1;
  if (rows == 0 || cols == 0) return 0;
  const int threads = 256;
  const bool vec = (cols % 4 == 0) && (src_pitch % 4 == 0) && (dst_pitch % 4 == 0) &&
                   ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0;
  if (vec) {
    copy_2d_vec4_kernel<<<grid_for(rows * cols / 4, threads), threads, 0, as_stream(stream)>>>(
        reinterpret_cast<const float4*>(src), src_pitch / 4, reinterpret_cast<float4*>(dst), dst_pitch / 4, rows,
        cols / 4);
  } else {
    copy_2d_kernel<<<grid_for(rows * cols, threads), threads, 0, as_stream(stream)>>>(src, src_pitch, dst, dst_pitch,
                                                                                     rows, cols);
  }
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mcb200_permute(const float* in, float* out, int num_axes, const int* in_shape, const int* order,
                              void* stream) {
  if (!in || !out || !in_shape || !order || num_axes < 1 || num_axes > 6) return -1;
  long long in_stride[6];
  long long count = 1;
  for (int ax = num_axes - 1; ax >= 0; --ax) {
    in_stride[ax] = count;
    count *= in_shape[ax];
  }
  PermuteArgs a;
  a.num_axes = num_axes;
  for (int ax = 0; ax < num_axes; ++ax) {
    if (order[ax] < 0 || order[ax] >= num_axes) return -2;
    a.out_shape[ax] = in_shape[order[ax]];
    a.in_stride_of_out_axis[ax] = in_stride[order[ax]];
  }
  if (count == 0) return 0;
  const int threads = 256;
  permute_kernel<<<grid_for(count, threads), threads, 0, as_stream(stream)>>>(in, out, count, a);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mcb200_normalize_nhwc(const float* in, float* out, long long pixels, int channels, const float* scale,
                                     int scale_shared, float eps, void* stream) {
  if (!in || !out || !scale || pixels < 0 || channels < 1) return -1;
  if (pixels == 0) return 0;
  const int threads = 256;
  normalize_nhwc_kernel<<<grid_for(pixels * 32, threads), threads, 0, as_stream(stream)>>>(in, out, pixels, channels,
                                                                                          scale, scale_shared, eps);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}
