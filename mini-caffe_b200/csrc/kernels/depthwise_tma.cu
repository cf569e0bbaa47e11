// 3 x 3 depthwise convolution (group == channels, dilation 1, stride 1 or 2) with the input staged
// in shared memory by TMA.
//
// The layer moves 2.25 FLOP per byte: all that matters is keeping enough bytes in flight.  A
// kernel whose threads load their own windows has its bytes in flight bounded by registers
// (measured on MobileNet-v1 at batch 64: 24 warps per SM at 75-80 registers, 1.5-3.4 TB/s).  Here a
// CTA walks over tiles of 8 x 16 output pixels x 32 channels; one thread asks the TMA unit for the
// next tile's input box ((7 * stride + 3) x (15 * stride + 3) pixels x 32 channels, zero-filled
// outside the image, which is the layer's padding) while all threads compute the current one out of
// shared memory; a ring of kStages boxes per CTA (requests run kStages - 1 tiles ahead) keeps
// 70-190 KB per SM in flight, independent of the registers the arithmetic needs.
//
// Shared-memory layout: a pixel's 32 channels are one 128-byte row of the box, stored with the
// 128-byte swizzle; a warp's lanes are 8 channel groups x 4 neighbouring pixels of a row, which
// the swizzle spreads over all banks.  A thread computes four outputs of one column (six / nine
// input rows x three columns, each input row loaded once), rows top to bottom and taps left to
// right like the reference's loops (src/layers/conv_dw_layer.cpp:104-152), and stores 16 bytes per
// output; eight lanes write a pixel's 128 bytes.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include <mutex>

#include "../../../include/mcb200_kernels.h"
#include "launch_count.h"
#include "sm100.cuh"

namespace mcb200 {
namespace {

using namespace sm100;

constexpr int kTileH = 8, kTileW = 16, kChannels = 32;
constexpr int kMaxDwStages = 4;
constexpr long long kDwWaitLimitCycles = 2000000000LL;   // about one second

template <int STRIDE>
struct DwBox {
  static constexpr int kH = (kTileH - 1) * STRIDE + 3;
  static constexpr int kW = (kTileW - 1) * STRIDE + 3;
  static constexpr int kBytes = kH * kW * kChannels * 4;
  static constexpr int kStageBytes = (kBytes + 1023) / 1024 * 1024;
};

struct DwArgs {
  const float* w;        // [9][C]
  float* out;            // channels last, C floats per pixel
  int n, c, ho, wo, pad_h, pad_w;
  int tiles_x, tiles_y, c_blocks;
  long long tiles;
  const float* scale;    // fused tail: y = act(acc * scale[c] + shift[c])
  const float* shift;
  int act;               // 0 none, 1 leaky ReLU with `slope`, 2 per-channel slope
  float slope;
  const float* prelu;
  int prelu_shared;
  int* status;
};

__device__ __forceinline__ float dw_tail(float v, float scale, float shift, float slope) {
  v = fmaf(v, scale, shift);
  return v > 0.f ? v : v * slope;   // slope 1: no activation, 0: ReLU
}

template <int STRIDE>
__global__ void __launch_bounds__(256) depthwise3x3_tma_kernel(const __grid_constant__ CUtensorMap map_in, const DwArgs a,
                                                               const int kStages) {
  using Box = DwBox<STRIDE>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[kMaxDwStages];
  __shared__ int abort_flag;
  const uint32_t raw = smem_addr(smem_raw);
  uint8_t* stages = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  const int tid = threadIdx.x;
  if (tid == 0) {
    abort_flag = 0;
    for (int s = 0; s < kStages; ++s) mbar_init(&full_bar[s], 1);
    fence_barrier_init();
    tma_prefetch_descriptor(&map_in);
  }
  __syncthreads();
  // Up to here the CTA has only set itself up, which may overlap the tail of the previous launch of
  // the stream (programmatic dependent launch); from here on it touches tensors.  The next launch
  // may begin its own set-up as soon as every CTA of this one has got this far.
  grid_launch_dependents();
  grid_dependency_wait();
  volatile int* abort = &abort_flag;

  // tile index -> (channel block, tile column, tile row, image); channel blocks fastest, so that
  // CTAs running together read the same pixels' other channels (the same DRAM pages)
  auto decode = [&](long long t, int& cb, int& tx, int& ty, int& img) {
    cb = static_cast<int>(t % a.c_blocks);
    t /= a.c_blocks;
    tx = static_cast<int>(t % a.tiles_x);
    t /= a.tiles_x;
    ty = static_cast<int>(t % a.tiles_y);
    img = static_cast<int>(t / a.tiles_y);
  };
  auto request = [&](long long t, int stage) {
    int cb, tx, ty, img;
    decode(t, cb, tx, ty, img);
    mbar_expect_tx(&full_bar[stage], Box::kBytes);
    tma_load_4d(&map_in, &full_bar[stage], stages + stage * Box::kStageBytes, cb * kChannels,
                tx * kTileW * STRIDE - a.pad_w, ty * kTileH * STRIDE - a.pad_h, img);
  };

  // thread -> 4 channels x one column x four rows of the tile
  const int cg = tid & 7;
  const int col = ((tid >> 5) & 3) * 4 + ((tid >> 3) & 3);
  const int row0 = (tid >> 7) * 4;

  long long t = blockIdx.x;
  if (tid == 0) {
    for (int s = 0; s < kStages - 1; ++s)
      if (t + static_cast<long long>(s) * gridDim.x < a.tiles) request(t + static_cast<long long>(s) * gridDim.x, s);
  }
  int it = 0;
  for (; t < a.tiles; t += gridDim.x, ++it) {
    const int stage = it % kStages;
    const uint32_t parity = static_cast<uint32_t>(it / kStages) & 1u;
    // the tile kStages - 1 ahead goes into the stage that was consumed before the last barrier
    const long long ahead = t + static_cast<long long>(kStages - 1) * gridDim.x;
    if (tid == 0 && ahead < a.tiles) request(ahead, (it + kStages - 1) % kStages);
    if (!mbar_wait_bounded(&full_bar[stage], parity, abort, kDwWaitLimitCycles)) break;
    int cb, tx, ty, img;
    decode(t, cb, tx, ty, img);
    const int c0 = cb * kChannels + cg * 4;
    const uint8_t* box = stages + stage * Box::kStageBytes;
    float4 k[9];
    float4 sc = make_float4(1.f, 1.f, 1.f, 1.f), sh = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 sl = make_float4(1.f, 1.f, 1.f, 1.f);
    if (c0 < a.c) {
#pragma unroll
      for (int j = 0; j < 9; ++j) k[j] = __ldg(reinterpret_cast<const float4*>(a.w + static_cast<size_t>(j) * a.c + c0));
      if (a.scale) sc = __ldg(reinterpret_cast<const float4*>(a.scale + c0));
      if (a.shift) sh = __ldg(reinterpret_cast<const float4*>(a.shift + c0));
      if (a.act == 1) {
        sl = make_float4(a.slope, a.slope, a.slope, a.slope);
      } else if (a.act == 2) {
        if (a.prelu_shared) {
          const float p = __ldg(a.prelu);
          sl = make_float4(p, p, p, p);
        } else {
          sl = __ldg(reinterpret_cast<const float4*>(a.prelu + c0));
        }
      }
    }
    float4 acc[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    constexpr int kRows = 3 * STRIDE + 3;   // input rows under four output rows
#pragma unroll
    for (int ir = 0; ir < kRows; ++ir) {
      float4 v[3];
#pragma unroll
      for (int q = 0; q < 3; ++q) {
        const int p = (row0 * STRIDE + ir) * Box::kW + col * STRIDE + q;   // pixel of the box
        v[q] = *reinterpret_cast<const float4*>(box + p * 128 + ((cg ^ (p & 7)) << 4));
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = ir - i * STRIDE;   // filter row this input row is for output row i
        if (r < 0 || r > 2) continue;
#pragma unroll
        for (int q = 0; q < 3; ++q) {
          acc[i].x = fmaf(v[q].x, k[r * 3 + q].x, acc[i].x);
          acc[i].y = fmaf(v[q].y, k[r * 3 + q].y, acc[i].y);
          acc[i].z = fmaf(v[q].z, k[r * 3 + q].z, acc[i].z);
          acc[i].w = fmaf(v[q].w, k[r * 3 + q].w, acc[i].w);
        }
      }
    }
    const int ox = tx * kTileW + col;
    if (c0 < a.c && ox < a.wo) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int oy = ty * kTileH + row0 + i;
        if (oy >= a.ho) break;
        float4 r4;
        r4.x = dw_tail(acc[i].x, sc.x, sh.x, sl.x);
        r4.y = dw_tail(acc[i].y, sc.y, sh.y, sl.y);
        r4.z = dw_tail(acc[i].z, sc.z, sh.z, sl.z);
        r4.w = dw_tail(acc[i].w, sc.w, sh.w, sl.w);
        *reinterpret_cast<float4*>(a.out + ((static_cast<size_t>(img) * a.ho + oy) * a.wo + ox) * a.c + c0) = r4;
      }
    }
    __syncthreads();   // everybody is done with this stage before it is requested again
  }
  // A CTA that gave up waiting: its outstanding request gets a bounded grace period, then the
  // status word says so.
  if (abort_flag) {
    __syncthreads();
    if (tid == 0) {
      for (int j = it; j < it + kStages; ++j) {   // the box that did not arrive and the ones requested after it
        const long long start = clock64();
        while (!mbar_try_wait(&full_bar[j % kStages], static_cast<uint32_t>(j / kStages) & 1u)) {
          if (clock64() - start > kDwWaitLimitCycles / 8) break;
        }
      }
      if (a.status) atomicExch(a.status, 1);
    }
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn dw_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

template <int STRIDE>
int launch_dw(const mcb200_conv_shape& s, const float* in, const DwArgs& args, cudaStream_t st) {
  using Box = DwBox<STRIDE>;
  EncodeTiledFn encode = dw_encode_tiled();
  if (!encode) return -10;
  CUtensorMap map;
  const cuuint64_t pix = static_cast<cuuint64_t>(s.c_stride) * 4;
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(s.c), static_cast<cuuint64_t>(s.w), static_cast<cuuint64_t>(s.h),
                              static_cast<cuuint64_t>(s.n)};
  const cuuint64_t strides[3] = {pix, pix * s.w, pix * s.w * s.h};
  const cuuint32_t box[4] = {kChannels, static_cast<cuuint32_t>(Box::kW), static_cast<cuuint32_t>(Box::kH), 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  if (encode(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(in), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return -11;
  auto kernel = depthwise3x3_tma_kernel<STRIDE>;
  // Boxes per CTA: two at stride 1 (two CTAs per SM by registers), three at stride 2 (one CTA per
  // SM by shared memory: 215 KB).  Measured in interleaved MobileNet-v1 passes at batch 64 (0.777 ms
  // with four and two boxes): three boxes at stride 2 0.773, and two instead of four at stride 1
  // on top of that 0.771; with the launches chained (programmatic dependent launch) a deeper ring at
  // stride 1 no longer pays.
  int stage_count = STRIDE == 1 ? 2 : 3;
  if (const char* env = getenv(STRIDE == 1 ? "MCB200_DW_STAGES_S1" : "MCB200_DW_STAGES_S2")) {   // experiments
    const int v = atoi(env);
    if (v >= 2 && v <= kMaxDwStages && v * Box::kStageBytes + 2048 <= 227 * 1024) stage_count = v;
  }
  const int smem = stage_count * Box::kStageBytes + 1024;
  int dev = 0;
  cudaGetDevice(&dev);
  static bool configured[64] = {false};
  static int sm_count[64] = {0};
  static std::mutex mu;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) return static_cast<int>(e);
      int n = 0;
      if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) n = 148;
      sm_count[dev] = n;
      configured[dev] = true;
    }
  }
  const int sms = (dev >= 0 && dev < 64 && sm_count[dev] > 0) ? sm_count[dev] : 148;
  int per_sm = (227 * 1024) / (smem + 1024);   // by shared memory: 2 at stride 1, 1 at stride 2
  if (per_sm > 2) per_sm = 2;                  // by registers
  if (per_sm < 1) per_sm = 1;
  long long blocks = static_cast<long long>(sms) * per_sm;
  if (blocks > args.tiles) blocks = args.tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(blocks), 1, 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.dynamicSmemBytes = static_cast<size_t>(smem);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // the kernel orders itself with griddepcontrol.wait
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t launched = cudaLaunchKernelEx(&cfg, kernel, map, args, stage_count);
  count_launch();
  return static_cast<int>(launched);
}

}  // namespace
}  // namespace mcb200

using namespace mcb200;

extern "C" int mcb200_conv_depthwise_tma_supported(const mcb200_conv_shape* s) {
  if (!s || s->group != s->c || s->cout != s->c || (s->c & 3) || (s->c_stride & 3) || s->c_stride < s->c) return 0;
  return (s->kh == 3 && s->kw == 3 && s->dil_h == 1 && s->dil_w == 1 && s->stride_h == s->stride_w &&
          (s->stride_h == 1 || s->stride_h == 2))
             ? 1
             : 0;
}

extern "C" int mcb200_conv_depthwise_tma(const mcb200_conv_shape* s, const float* in, const float* packed_w, float* out,
                                         const mcb200_epilogue* ep, int* status, void* stream) {
  if (!s || !in || !packed_w || !out) return -1;
  if (!mcb200_conv_depthwise_tma_supported(s)) return -2;
  if ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(packed_w)) & 15)
    return -3;
  mcb200_conv_shape shape = *s;
  if (mcb200_conv_out_shape(&shape) != 0) return -4;
  if (ep && ep->act == 2 && !ep->prelu) return -5;
  if (ep && ep->residual) return -6;   // a fused residual goes through mcb200_conv_depthwise
  DwArgs a;
  a.w = packed_w;
  a.out = out;
  a.n = shape.n;
  a.c = shape.c;
  a.ho = shape.ho;
  a.wo = shape.wo;
  a.pad_h = shape.pad_h;
  a.pad_w = shape.pad_w;
  a.tiles_x = (shape.wo + kTileW - 1) / kTileW;
  a.tiles_y = (shape.ho + kTileH - 1) / kTileH;
  a.c_blocks = (shape.c + kChannels - 1) / kChannels;
  a.tiles = static_cast<long long>(shape.n) * a.tiles_y * a.tiles_x * a.c_blocks;
  a.scale = ep ? ep->scale : nullptr;
  a.shift = ep ? ep->shift : nullptr;
  a.act = ep ? ep->act : 0;
  a.slope = ep ? ep->slope : 0.f;
  a.prelu = ep ? ep->prelu : nullptr;
  a.prelu_shared = ep ? ep->prelu_shared : 0;
  a.status = status;
  if (a.tiles == 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return shape.stride_h == 1 ? launch_dw<1>(shape, in, a, st) : launch_dw<2>(shape, in, a, st);
}
