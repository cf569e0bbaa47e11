// Measured ceilings for the tensor-core convolution kernel's two resources, so that its
// fractions are quoted against something measured on the same device:
//
//   * the issue rate of tcgen05.mma with operands that already sit in shared memory
//     (kind::tf32 or kind::f16 / bfloat16, M = 128 per CTA, N = 64 / 128 / 256, optionally as
//     two-CTA pairs): one thread per CTA issues back-to-back MMAs on one resident stage, nothing
//     is loaded or stored, all SMs run at once;
//   * the rate at which all SMs together can pull 16 KiB operand tiles from an L2-resident
//     tensor into shared memory with TMA (tiled map, 128-byte swizzle, a ring of stages per
//     CTA, no consumer).
//
// Both are timed with CUDA events around the launch.  Every wait is bounded.  Nothing here is
// on the product path; bench.py reports the figures next to the kernel's achieved rates.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "../../../include/mcb200_runtime.h"
#include "launch_count.h"
#include "sm100.cuh"

namespace mcb200 {
namespace {

using namespace sm100;

constexpr long long kProbeWaitCycles = 2000000000LL;   // about one second

// kKind 0: tf32 (K = 8 per instruction), 1: bfloat16 (K = 16).  Operands: one 128-byte-swizzled
// K-major stage (A: 128 rows, B: BN rows, or BN / 2 per CTA of a pair), filled with small values.
template <int BN, int kKind, bool kPair>
__global__ void __launch_bounds__(128, 1) mma_peak_kernel(int steps, int* status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t done_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const uint32_t raw = smem_addr(smem_raw);
  uint8_t* tiles = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  constexpr int kBRows = kPair ? BN / 2 : BN;
  constexpr int kABytes = 128 * 128;
  constexpr int kBBytes = kBRows * 128;
  const int warp = threadIdx.x >> 5;
  // Small values of both signs (an all-zero operand would flatter the clocks).
  for (int i = threadIdx.x; i < (kABytes + kBBytes) / 4; i += blockDim.x) {
    const uint32_t h = (static_cast<uint32_t>(i) * 2654435761u) >> 20;
    const float v = (static_cast<int>(h & 255u) - 128) * (1.f / 1024.f);
    if (kKind == 0) {
      reinterpret_cast<float*>(tiles)[i] = v;
    } else {
      reinterpret_cast<uint32_t*>(tiles)[i] = pack_bf16x2(v, -v);
    }
  }
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&done_bar, 1);
    fence_barrier_init();
  }
  fence_proxy_async_smem();
  if (warp == 1) {
    tmem_alloc(&tmem_slot, BN < 32 ? 32 : BN);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  if (kPair) {
    cluster_sync_all();
  } else {
    __syncthreads();
  }
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;
  volatile int* abort = &abort_flag;
  const uint32_t rank = kPair ? cluster_cta_rank() : 0u;
  const bool usable = !kPair || tmem == 0u;   // a paired MMA writes the same address in both CTAs
  if (usable && warp == 0 && elect_one()) {
    if (rank == 0u) {
      constexpr uint32_t idesc = kKind == 0 ? umma_idesc_tf32(kPair ? 256 : 128, BN) : umma_idesc_bf16(kPair ? 256 : 128, BN);
      const uint64_t da = umma_desc_k_sw128(smem_addr(tiles));
      const uint64_t db = umma_desc_k_sw128(smem_addr(tiles) + kABytes);
      uint32_t accumulate = 0u;   // the first instruction overwrites whatever tensor memory held
      for (int s = 0; s < steps; ++s) {
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {   // the four 32-byte K steps of a 128-byte row
          if (kKind == 0) {
            if (kPair) {
              umma_tf32_pair(tmem, da + 2 * kk, db + 2 * kk, idesc, accumulate);
            } else {
              umma_tf32(tmem, da + 2 * kk, db + 2 * kk, idesc, accumulate);
            }
          } else if (kPair) {
            umma_bf16_pair(tmem, da + 2 * kk, db + 2 * kk, idesc, accumulate);
          } else {
            umma_bf16(tmem, da + 2 * kk, db + 2 * kk, idesc, accumulate);
          }
          accumulate = 1u;
        }
      }
      if (kPair) {
        umma_commit_pair(&done_bar, 3);
      } else {
        umma_commit(&done_bar);
      }
    }
    mbar_wait_bounded(&done_bar, 0u, abort, kProbeWaitCycles);
  }
  tc_fence_before_sync();
  __syncwarp();
  if (kPair) {
    cluster_sync_all();
  } else {
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, BN < 32 ? 32 : BN);
  }
  if (threadIdx.x == 0 && (abort_flag || !usable) && status) atomicExch(status, 1);
}

// Each CTA keeps `stages` 16 KiB tile loads in flight (one barrier per stage) and re-issues a
// stage's load as soon as it has landed, walking the tensor's tiles CTA-strided.
__global__ void __launch_bounds__(64, 1) tma_pull_kernel(const __grid_constant__ CUtensorMap map, int tiles_in_tensor,
                                                         int loads, int stages, int* status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[8];
  __shared__ int abort_flag;
  const uint32_t raw = smem_addr(smem_raw);
  uint8_t* tiles = smem_raw + ((1024u - (raw & 1023u)) & 1023u);
  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < stages; ++s) mbar_init(&full_bar[s], 1);
    fence_barrier_init();
    tma_prefetch_descriptor(&map);
  }
  __syncthreads();
  volatile int* abort = &abort_flag;
  if (threadIdx.x == 0) {
    int tile = static_cast<int>(blockIdx.x) % tiles_in_tensor;
    int issued = 0, landed = 0;
    bool alive = true;
    auto issue = [&]() {
      const int s = issued % stages;
      mbar_expect_tx(&full_bar[s], 16384u);
      tma_load_2d(&map, &full_bar[s], tiles + s * 16384, 0, tile * 128);
      tile += static_cast<int>(gridDim.x);
      if (tile >= tiles_in_tensor) tile -= tiles_in_tensor * (tile / tiles_in_tensor);
      ++issued;
    };
    while (issued < loads && issued < stages) issue();
    while (landed < issued && alive) {
      const int s = landed % stages;
      alive = mbar_wait_bounded(&full_bar[s], static_cast<uint32_t>(landed / stages) & 1u, abort, kProbeWaitCycles);
      ++landed;
      if (alive && issued < loads) issue();
    }
    // After a timed-out wait the copies still in flight get a bounded grace period before the CTA
    // gives its shared memory back.
    for (; !alive && landed < issued; ++landed) {
      const long long start = clock64();
      while (!mbar_try_wait(&full_bar[landed % stages], static_cast<uint32_t>(landed / stages) & 1u)) {
        if (clock64() - start > kProbeWaitCycles / 8) break;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && abort_flag && status) atomicExch(status, 1);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
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

struct ProbeTimer {
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  cudaStream_t st;
  explicit ProbeTimer(cudaStream_t s) : st(s) {
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
  }
  ~ProbeTimer() {
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
  }
  void start() { cudaEventRecord(e0, st); }
  // Milliseconds, or a negative value on error.
  double stop() {
    cudaEventRecord(e1, st);
    if (cudaEventSynchronize(e1) != cudaSuccess) return -1.0;
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, e0, e1) != cudaSuccess) return -1.0;
    return ms;
  }
};

template <int BN, int kKind, bool kPair>
int run_mma_peak(int steps, int reps, int* status_dev, cudaStream_t st, double* best_ms, int* ctas_out) {
  auto kernel = mma_peak_kernel<BN, kKind, kPair>;
  const int smem = 128 * 128 + (kPair ? BN / 2 : BN) * 128 + 1024;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return static_cast<int>(e);
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) return -3;
  const int ctas = kPair ? (sms / 2) * 2 : sms;
  *ctas_out = ctas;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ctas, 1, 1);
  cfg.blockDim = dim3(128, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = kPair ? 1 : 0;
  ProbeTimer timer(st);
  *best_ms = -1.0;
  for (int r = 0; r < reps + 1; ++r) {   // the first launch warms up (module load, clocks)
    timer.start();
    e = cudaLaunchKernelEx(&cfg, kernel, steps, status_dev);
    count_launch();
    if (e != cudaSuccess) return static_cast<int>(e);
    const double ms = timer.stop();
    if (ms < 0) return static_cast<int>(cudaGetLastError());
    if (r > 0 && (*best_ms < 0 || ms < *best_ms)) *best_ms = ms;
  }
  return 0;
}

}  // namespace
}  // namespace mcb200

using namespace mcb200;

extern "C" int mcb200_probe_mma_peak(int bf16, int block_n, int cta_pair, int steps, int reps, double* ms,
                                     double* tflops, void* stream) {
  if (!ms || !tflops || steps < 1 || reps < 1 || steps > (1 << 22)) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int* status_dev = nullptr;
  if (cudaMalloc(reinterpret_cast<void**>(&status_dev), sizeof(int)) != cudaSuccess) return -2;
  cudaMemsetAsync(status_dev, 0, sizeof(int), st);
  int rc = -4, ctas = 0;
  double best = -1.0;
#define MCB200_PEAK(BN)                                                                                    \
  rc = bf16 ? (cta_pair ? run_mma_peak<BN, 1, true>(steps, reps, status_dev, st, &best, &ctas)             \
                        : run_mma_peak<BN, 1, false>(steps, reps, status_dev, st, &best, &ctas))           \
            : (cta_pair ? run_mma_peak<BN, 0, true>(steps, reps, status_dev, st, &best, &ctas)             \
                        : run_mma_peak<BN, 0, false>(steps, reps, status_dev, st, &best, &ctas))
  switch (block_n) {
    case 64: MCB200_PEAK(64); break;
    case 128: MCB200_PEAK(128); break;
    case 256: MCB200_PEAK(256); break;
    default: rc = -4; break;
  }
#undef MCB200_PEAK
  int status = 0;
  if (rc == 0 && cudaMemcpyAsync(&status, status_dev, sizeof(int), cudaMemcpyDeviceToHost, st) == cudaSuccess)
    cudaStreamSynchronize(st);
  cudaFree(status_dev);
  if (rc != 0) return rc;
  if (status != 0) return -5;   // a wait ran out: the figure means nothing
  *ms = best;
  // Per CTA and step: four instructions of M128 (per CTA) x N x K (8 tf32 / 16 bf16).
  const double k_per_step = bf16 ? 64.0 : 32.0;
  *tflops = 2.0 * 128.0 * block_n * k_per_step * steps * ctas / (best * 1e-3) / 1e12;
  return 0;
}

extern "C" int mcb200_probe_tma_l2_pull(void* buffer, size_t bytes, int loads_per_cta, int stages, int reps, double* ms,
                                        double* gbs, void* stream) {
  if (!buffer || !ms || !gbs || bytes < (1u << 20) || loads_per_cta < 1 || stages < 1 || stages > 8 || reps < 1)
    return -1;
  if (reinterpret_cast<uintptr_t>(buffer) & 127) return -2;
  EncodeTiledFn encode = encode_tiled();
  if (!encode) return -3;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The buffer as a [rows, 32] fp32 matrix of 128-byte rows; a tile is 128 rows.
  const cuuint64_t rows = bytes / 128;
  const int tiles = static_cast<int>(rows / 128);
  CUtensorMap map;
  const cuuint64_t dims[2] = {32, rows};
  const cuuint64_t strides[1] = {128};
  const cuuint32_t box[2] = {32, 128};
  const cuuint32_t estr[2] = {1, 1};
  if (encode(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, buffer, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return -4;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) return -5;
  const int smem = stages * 16384 + 1024;
  cudaError_t e = cudaFuncSetAttribute(tma_pull_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return static_cast<int>(e);
  int* status_dev = nullptr;
  if (cudaMalloc(reinterpret_cast<void**>(&status_dev), sizeof(int)) != cudaSuccess) return -6;
  cudaMemsetAsync(status_dev, 0, sizeof(int), st);
  ProbeTimer timer(st);
  double best = -1.0;
  int rc = 0;
  for (int r = 0; r < reps + 1 && rc == 0; ++r) {   // the first launch brings the tensor into L2
    timer.start();
    tma_pull_kernel<<<sms, 64, smem, st>>>(map, tiles, loads_per_cta, stages, status_dev);
    count_launch();
    e = cudaGetLastError();
    if (e != cudaSuccess) rc = static_cast<int>(e);
    const double t = timer.stop();
    if (t < 0) rc = static_cast<int>(cudaGetLastError());
    if (rc == 0 && r > 0 && (best < 0 || t < best)) best = t;
  }
  int status = 0;
  if (rc == 0 && cudaMemcpyAsync(&status, status_dev, sizeof(int), cudaMemcpyDeviceToHost, st) == cudaSuccess)
    cudaStreamSynchronize(st);
  cudaFree(status_dev);
  if (rc != 0) return rc;
  if (status != 0) return -7;
  *ms = best;
  *gbs = 16384.0 * loads_per_cta * sms / (best * 1e-3) / 1e9;
  return 0;
}
