// Convolutions that do not go to the tensor cores.
//
//  * mcb200_conv_depthwise: group == channels (MobileNet).  2.25 FLOP per byte:
//    HBM-bound, so the kernel is organised around memory traffic -- channels
//    last, one thread per output pixel and four channels, every input and
//    weight access a 128-bit load, fused scale/shift/activation on the way out.
//  * mcb200_conv_direct: any group count, any channel count; one thread per
//    output element.  Slow but shape-agnostic; the fallback for layers the
//    tensor-core path rejects (e.g. grouped convolutions, channel counts that
//    are not a multiple of four).
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../../include/mcb200_kernels.h"
#include "launch_count.h"

namespace mcb200 {
namespace {

constexpr int kSMs = 148;

inline int grid_for(long long items, int threads) {
  long long blocks = (items + threads - 1) / threads;
  const long long cap = static_cast<long long>(kSMs) * 16;
  if (blocks > cap) blocks = cap;
  return blocks < 1 ? 1 : static_cast<int>(blocks);
}

__device__ __forceinline__ float tail(float v, int c, const mcb200_epilogue& ep, const float* res) {
  if (ep.scale) v *= __ldg(ep.scale + c);
  if (ep.shift) v += __ldg(ep.shift + c);
  if (res) v += ep.residual_coeff * res[c];
  if (ep.act != 0 && v <= 0.f) {
    const float slope = ep.act == 2 ? __ldg(ep.prelu + (ep.prelu_shared ? 0 : c)) : ep.slope;
    v *= slope;
  }
  return v;
}

__global__ void depthwise_vec4_kernel(const float* __restrict__ in, const float* __restrict__ w, float* __restrict__ out,
                                      mcb200_conv_shape s, mcb200_epilogue ep) {
  const int cg = s.c / 4;
  const long long total = static_cast<long long>(s.n) * s.ho * s.wo * cg;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int g = static_cast<int>(i % cg);
    long long t = i / cg;
    const int ox = static_cast<int>(t % s.wo);
    t /= s.wo;
    const int oy = static_cast<int>(t % s.ho);
    const int n = static_cast<int>(t / s.ho);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < s.kh; ++r) {
      const int y = oy * s.stride_h - s.pad_h + r * s.dil_h;
      if (y < 0 || y >= s.h) continue;
      for (int q = 0; q < s.kw; ++q) {
        const int x = ox * s.stride_w - s.pad_w + q * s.dil_w;
        if (x < 0 || x >= s.w) continue;
        const float4 v =
            *reinterpret_cast<const float4*>(in + ((static_cast<size_t>(n) * s.h + y) * s.w + x) * s.c_stride + g * 4);
        const float4 k = __ldg(reinterpret_cast<const float4*>(w + static_cast<size_t>(r * s.kw + q) * s.c + g * 4));
        acc.x += v.x * k.x;
        acc.y += v.y * k.y;
        acc.z += v.z * k.z;
        acc.w += v.w * k.w;
      }
    }
    const size_t o = ((static_cast<size_t>(n) * s.ho + oy) * s.wo + ox) * s.c + g * 4;
    const float* res = ep.residual ? ep.residual + ((static_cast<size_t>(n) * s.ho + oy) * s.wo + ox) * ep.residual_ld
                                   : nullptr;
    const int c0 = g * 4;
    float4 r4;
    r4.x = tail(acc.x, c0, ep, res);
    r4.y = tail(acc.y, c0 + 1, ep, res);
    r4.z = tail(acc.z, c0 + 2, ep, res);
    r4.w = tail(acc.w, c0 + 3, ep, res);
    *reinterpret_cast<float4*>(out + o) = r4;
  }
}

// 3 x 3 depthwise convolution, dilation 1, stride 1 or 2: one thread computes
// four neighbouring output pixels of one row for four channels.  The 3 x
// (4 * STRIDE + 2) input window is loaded once (4.5 / 6.75 sixteen-byte loads
// per output instead of 9), the nine weight vectors sit in registers, and the
// index arithmetic is 32-bit.  Consecutive threads take consecutive channel
// groups, so a warp's loads are contiguous runs of the channels-last rows.
//
// IN_HALF / OUT_HALF: the activations are read / the result is stored as
// bfloat16 (four channels = one 8-byte access), for nets with bfloat16
// storage; weights and arithmetic stay fp32.
__device__ __forceinline__ float4 load4(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ float4 load4_bf16(const uint16_t* p) {
  const uint2 w = __ldg(reinterpret_cast<const uint2*>(p));
  return make_float4(__uint_as_float(w.x << 16), __uint_as_float(w.x & 0xFFFF0000u), __uint_as_float(w.y << 16),
                     __uint_as_float(w.y & 0xFFFF0000u));
}
__device__ __forceinline__ uint32_t pack2_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

template <int STRIDE, bool IN_HALF, bool OUT_HALF>
__global__ void __launch_bounds__(256)
depthwise3x3_kernel(const void* __restrict__ in_any, const float* __restrict__ w, void* __restrict__ out_any,
                    mcb200_conv_shape s, mcb200_epilogue ep) {
  // the pointwise convolution behind this layer may set itself up meanwhile (it waits with
  // griddepcontrol.wait before it touches a tensor)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const float* in = static_cast<const float*>(in_any);
  const uint16_t* in16 = static_cast<const uint16_t*>(in_any);
  float* out = static_cast<float*>(out_any);
  uint16_t* out16 = static_cast<uint16_t*>(out_any);
  constexpr int kOut = 4;                      // output pixels per thread
  constexpr int kCols = kOut * STRIDE + 2;     // input columns they need (3 x 3 window)
  const unsigned cg = s.c >> 2;
  const unsigned strips = (s.wo + kOut - 1) / kOut;
  const unsigned total = static_cast<unsigned>(s.n) * s.ho * strips * cg;
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const unsigned g = i % cg;
    unsigned t = i / cg;
    const int strip = static_cast<int>(t % strips);
    t /= strips;
    const int oy = static_cast<int>(t % s.ho);
    const unsigned n = t / s.ho;
    const int ox0 = strip * kOut;
    const int x0 = ox0 * STRIDE - s.pad_w;
    const int y0 = oy * STRIDE - s.pad_h;
    float4 k[9];
#pragma unroll
    for (int j = 0; j < 9; ++j) k[j] = __ldg(reinterpret_cast<const float4*>(w + static_cast<size_t>(j) * s.c) + g);
    float4 acc[kOut];
#pragma unroll
    for (int o = 0; o < kOut; ++o) acc[o] = make_float4(0.f, 0.f, 0.f, 0.f);
    const size_t image = static_cast<size_t>(n) * s.h * s.w * s.c_stride + g * 4;   // element offset
#pragma unroll
    for (int r = 0; r < 3; ++r) {
      const int y = y0 + r;
      if (y < 0 || y >= s.h) continue;
      const size_t row = image + static_cast<size_t>(y) * s.w * s.c_stride;
      float4 v[kCols];
#pragma unroll
      for (int c = 0; c < kCols; ++c) {
        const int x = x0 + c;
        const size_t at = row + static_cast<size_t>(x) * s.c_stride;
        v[c] = (x >= 0 && x < s.w) ? (IN_HALF ? load4_bf16(in16 + at) : load4(in + at))
                                   : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int o = 0; o < kOut; ++o) {
#pragma unroll
        for (int q = 0; q < 3; ++q) {
          const float4 a = v[o * STRIDE + q];
          const float4 b = k[r * 3 + q];
          acc[o].x = fmaf(a.x, b.x, acc[o].x);
          acc[o].y = fmaf(a.y, b.y, acc[o].y);
          acc[o].z = fmaf(a.z, b.z, acc[o].z);
          acc[o].w = fmaf(a.w, b.w, acc[o].w);
        }
      }
    }
    const int c0 = static_cast<int>(g) * 4;
#pragma unroll
    for (int o = 0; o < kOut; ++o) {
      const int ox = ox0 + o;
      if (ox >= s.wo) break;
      const size_t pixel = (static_cast<size_t>(n) * s.ho + oy) * s.wo + ox;
      const float* res = ep.residual ? ep.residual + pixel * ep.residual_ld : nullptr;
      float4 r4;
      r4.x = tail(acc[o].x, c0, ep, res);
      r4.y = tail(acc[o].y, c0 + 1, ep, res);
      r4.z = tail(acc[o].z, c0 + 2, ep, res);
      r4.w = tail(acc[o].w, c0 + 3, ep, res);
      if (OUT_HALF) {
        *reinterpret_cast<uint2*>(out16 + pixel * s.c + c0) = make_uint2(pack2_bf16(r4.x, r4.y), pack2_bf16(r4.z, r4.w));
      } else {
        *reinterpret_cast<float4*>(out + pixel * s.c + c0) = r4;
      }
    }
  }
}

__global__ void dw_pack_kernel(const float* __restrict__ w, float* __restrict__ packed, int c, int taps) {
  const int total = c * taps;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int ch = i % c;
    const int tap = i / c;
    packed[i] = w[static_cast<size_t>(ch) * taps + tap];
  }
}

__global__ void conv_direct_kernel(const float* __restrict__ in, const float* __restrict__ w, float* __restrict__ out,
                                   int out_ld, mcb200_conv_shape s, mcb200_epilogue ep) {
  const int cin_g = s.c / s.group;
  const int cout_g = s.cout / s.group;
  const long long total = static_cast<long long>(s.n) * s.ho * s.wo * s.cout;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int co = static_cast<int>(i % s.cout);
    long long t = i / s.cout;
    const long long pixel = t;
    const int ox = static_cast<int>(t % s.wo);
    t /= s.wo;
    const int oy = static_cast<int>(t % s.ho);
    const int n = static_cast<int>(t / s.ho);
    const int g = co / cout_g;
    const float* wk = w + static_cast<size_t>(co) * cin_g * s.kh * s.kw;
    float acc = 0.f;
    for (int r = 0; r < s.kh; ++r) {
      const int y = oy * s.stride_h - s.pad_h + r * s.dil_h;
      if (y < 0 || y >= s.h) continue;
      for (int q = 0; q < s.kw; ++q) {
        const int x = ox * s.stride_w - s.pad_w + q * s.dil_w;
        if (x < 0 || x >= s.w) continue;
        const float* px = in + ((static_cast<size_t>(n) * s.h + y) * s.w + x) * s.c_stride + g * cin_g;
        for (int ci = 0; ci < cin_g; ++ci) acc += px[ci] * __ldg(wk + (static_cast<size_t>(ci) * s.kh + r) * s.kw + q);
      }
    }
    const float* res = ep.residual ? ep.residual + pixel * ep.residual_ld : nullptr;
    out[pixel * out_ld + co] = tail(acc, co, ep, res);
  }
}

mcb200_epilogue default_epilogue() {
  mcb200_epilogue ep = mcb200_epilogue();
  ep.residual_coeff = 1.f;
  return ep;
}

}  // namespace
}  // namespace mcb200

using namespace mcb200;

extern "C" int mcb200_dw_pack_weights(const mcb200_conv_shape* s, const float* w_oihw, float* packed, void* stream) {
  if (!s || !w_oihw || !packed || s->group != s->c || s->cout != s->c) return -1;
  const int taps = s->kh * s->kw;
  dw_pack_kernel<<<grid_for(static_cast<long long>(s->c) * taps, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      w_oihw, packed, s->c, taps);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mcb200_conv_depthwise(const mcb200_conv_shape* s, const float* in, const float* packed_w, float* out,
                                     const mcb200_epilogue* ep, void* stream) {
  if (!s || !in || !packed_w || !out) return -1;
  if (s->group != s->c || s->cout != s->c || (s->c & 3) || (s->c_stride & 3)) return -2;
  if ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(packed_w)) & 15)
    return -3;
  mcb200_conv_shape shape = *s;
  if (mcb200_conv_out_shape(&shape) != 0) return -4;
  const mcb200_epilogue e = ep ? *ep : default_epilogue();
  if (e.act == 2 && !e.prelu) return -5;
  const long long items = static_cast<long long>(shape.n) * shape.ho * shape.wo * (shape.c / 4);
  if (items == 0) return 0;
  const bool small3x3 = shape.kh == 3 && shape.kw == 3 && shape.dil_h == 1 && shape.dil_w == 1 &&
                        shape.stride_h == shape.stride_w && (shape.stride_h == 1 || shape.stride_h == 2) &&
                        items < 0x7fffffffLL;
  if (small3x3) {
    const long long threads = static_cast<long long>(shape.n) * shape.ho * ((shape.wo + 3) / 4) * (shape.c / 4);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (shape.stride_h == 1) {
      depthwise3x3_kernel<1, false, false><<<grid_for(threads, 256), 256, 0, st>>>(in, packed_w, out, shape, e);
    } else {
      depthwise3x3_kernel<2, false, false><<<grid_for(threads, 256), 256, 0, st>>>(in, packed_w, out, shape, e);
    }
  } else {
    depthwise_vec4_kernel<<<grid_for(items, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(in, packed_w, out,
                                                                                              shape, e);
  }
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mcb200_conv_depthwise_bf16_supported(const mcb200_conv_shape* s) {
  if (!s || s->group != s->c || s->cout != s->c || (s->c & 3) || (s->c_stride & 3)) return 0;
  return (s->kh == 3 && s->kw == 3 && s->dil_h == 1 && s->dil_w == 1 && s->stride_h == s->stride_w &&
          (s->stride_h == 1 || s->stride_h == 2))
             ? 1
             : 0;
}

extern "C" int mcb200_conv_depthwise_bf16(const mcb200_conv_shape* s, const void* in, int in_is_bf16,
                                          const float* packed_w, void* out, int out_is_bf16,
                                          const mcb200_epilogue* ep, void* stream) {
  if (!s || !in || !packed_w || !out) return -1;
  if (!mcb200_conv_depthwise_bf16_supported(s)) return -2;
  if ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(packed_w)) & 15)
    return -3;
  mcb200_conv_shape shape = *s;
  if (mcb200_conv_out_shape(&shape) != 0) return -4;
  const mcb200_epilogue e = ep ? *ep : default_epilogue();
  if (e.act == 2 && !e.prelu) return -5;
  if (e.residual) return -6;   // the fused residual of this kernel is fp32 only
  const long long threads = static_cast<long long>(shape.n) * shape.ho * ((shape.wo + 3) / 4) * (shape.c / 4);
  if (threads == 0) return 0;
  if (threads >= 0x7fffffffLL) return -7;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(threads, 256);
  const bool ih = in_is_bf16 != 0, oh = out_is_bf16 != 0;
#define MCB200_DW(STRIDE)                                                                                        \
  if (ih && oh) depthwise3x3_kernel<STRIDE, true, true><<<grid, 256, 0, st>>>(in, packed_w, out, shape, e);       \
  else if (ih) depthwise3x3_kernel<STRIDE, true, false><<<grid, 256, 0, st>>>(in, packed_w, out, shape, e);       \
  else if (oh) depthwise3x3_kernel<STRIDE, false, true><<<grid, 256, 0, st>>>(in, packed_w, out, shape, e);       \
  else depthwise3x3_kernel<STRIDE, false, false><<<grid, 256, 0, st>>>(in, packed_w, out, shape, e)
  if (shape.stride_h == 1) {
    MCB200_DW(1);
  } else {
    MCB200_DW(2);
  }
#undef MCB200_DW
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mcb200_conv_direct(const mcb200_conv_shape* s, const float* in, const float* w_oihw, float* out,
                                  int out_ld, const mcb200_epilogue* ep, void* stream) {
  if (!s || !in || !w_oihw || !out || s->group < 1) return -1;
  if (s->c % s->group != 0 || s->cout % s->group != 0 || out_ld < s->cout || s->c_stride < s->c) return -2;
  mcb200_conv_shape shape = *s;
  if (mcb200_conv_out_shape(&shape) != 0) return -4;
  const mcb200_epilogue e = ep ? *ep : default_epilogue();
  if (e.act == 2 && !e.prelu) return -5;
  const long long items = static_cast<long long>(shape.n) * shape.ho * shape.wo * shape.cout;
  if (items == 0) return 0;
  conv_direct_kernel<<<grid_for(items, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(in, w_oihw, out, out_ld,
                                                                                         shape, e);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}
