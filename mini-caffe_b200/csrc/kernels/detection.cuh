// Device building blocks shared by the detection kernels (RPN Proposal, SSD
// DetectionOutput): order-preserving float keys, a block-wide radix select of
// the K smallest 64-bit keys, a block-wide bitonic sort in shared memory, and
// IEEE arithmetic helpers that the compiler may not contract into fused
// multiply-adds (the CPU code being matched is compiled without FMA, and the
// kept-box sets have to agree bit for bit).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace mcb200 {
namespace det {

__device__ __forceinline__ float fadd(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float fsub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float fmul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float fdiv(float a, float b) { return __fdiv_rn(a, b); }

// Unsigned key that sorts ascending exactly when the float sorts DEScending;
// -0.0 and +0.0 get the same key (they compare equal on the CPU).
__device__ __forceinline__ uint32_t descending_key(float score) {
  uint32_t bits = __float_as_uint(score);
  if ((bits << 1) == 0u) bits = 0u;                                    // -0.0 -> +0.0
  const uint32_t ascending = bits ^ ((bits >> 31) ? 0xFFFFFFFFu : 0x80000000u);
  return ~ascending;
}

// 64-bit sort key: descending score first, ascending index second (unique).
__device__ __forceinline__ unsigned long long make_key(float score, uint32_t index) {
  return (static_cast<unsigned long long>(descending_key(score)) << 32) | index;
}

constexpr unsigned long long kPadKey = 0xFFFFFFFFFFFFFFFFull;

// Finds the k-th smallest (1-based) of n distinct keys with an MSB-first radix
// walk, 8 bits per pass, and returns a threshold T such that exactly k keys
// are <= T.  Whole block; `hist` is 256 ints of shared memory, `bcast` two
// unsigned long longs.  `fetch(i)` returns key i.
//
// Scores of one layer share their sign and most exponent bits, so in the first
// passes nearly every key falls into the same bin: lanes of a warp that hit
// the same bin are combined (__match_any_sync) into one shared-memory add.
// The walk stops as soon as the chosen bin holds exactly the keys still
// wanted (with distinct scores: after the four score bytes), because all of
// them are then selected whatever their lower bits are.
template <typename Fetch>
__device__ unsigned long long block_kth_smallest(Fetch fetch, int n, int k, int* hist, unsigned long long* bcast) {
  unsigned long long prefix = 0, mask = 0;
  int remaining = k;
  const int lane = threadIdx.x & 31;
  for (int pass = 7; pass >= 0; --pass) {
    for (int b = threadIdx.x; b < 256; b += blockDim.x) hist[b] = 0;
    __syncthreads();
    const int shift = pass * 8;
    for (int base = 0; base < n; base += blockDim.x) {   // the same trip count for every thread
      const int i = base + threadIdx.x;
      unsigned long long key = 0;
      bool live = i < n;
      if (live) {
        key = fetch(i);
        live = (key & mask) == prefix;
      }
      const unsigned live_lanes = __ballot_sync(0xffffffffu, live);
      if (live) {
        const int bin = static_cast<int>((key >> shift) & 0xFFull);
        const unsigned peers = __match_any_sync(live_lanes, bin);
        if (lane == __ffs(peers) - 1) atomicAdd(&hist[bin], __popc(peers));
      }
    }
    __syncthreads();
    if (threadIdx.x < 32) {
      // Warp 0 finds the bin that holds the `remaining`-th key: lane l sums bins
      // 8 l .. 8 l + 7, a shuffle scan gives the keys in front of each lane's
      // range, the lane whose range contains the key walks its eight bins.
      int own[8];
      int sum = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        own[j] = hist[lane * 8 + j];
        sum += own[j];
      }
      int incl = sum;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
      }
      const int excl = incl - sum;
      const bool mine = excl < remaining && remaining <= incl;
      const unsigned who = __ballot_sync(0xffffffffu, mine);
      // Fewer keys than asked for: the walk ends in the last bin, as a serial scan would.
      const int chosen = who ? __ffs(who) - 1 : 31;
      if (lane == chosen) {
        int cum = excl, bin = lane * 8;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          bin = lane * 8 + j;
          if (bin == 255 || cum + own[j] >= remaining) break;
          cum += own[j];
        }
        const unsigned long long next = prefix | (static_cast<unsigned long long>(bin) << shift);
        if (cum + hist[bin] == remaining) {   // the whole bin is wanted: done
          bcast[0] = next | ((1ull << shift) - 1ull);
          bcast[1] = 0ull;
        } else {
          bcast[0] = next;
          bcast[1] = static_cast<unsigned long long>(remaining - cum);
        }
      }
    }
    __syncthreads();
    prefix = bcast[0];
    remaining = static_cast<int>(bcast[1]);
    mask |= 0xFFull << shift;
    __syncthreads();
    if (remaining == 0) break;
  }
  return prefix;
}

// Ascending bitonic sort of `count` (a power of two) keys in shared memory.
__device__ inline void block_bitonic_sort(unsigned long long* keys, int count) {
  for (int size = 2; size <= count; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = threadIdx.x; t < (count >> 1); t += blockDim.x) {
        const int lo = ((t / stride) * (stride << 1)) + (t % stride);
        const int hi = lo + stride;
        const bool ascending = ((lo & size) == 0);
        const unsigned long long a = keys[lo], b = keys[hi];
        if ((a > b) == ascending) {
          keys[lo] = b;
          keys[hi] = a;
        }
      }
      __syncthreads();
    }
  }
}

__host__ __device__ inline int next_pow2(int v) {
  int p = 1;
  while (p < v) p <<= 1;
  return p;
}

}  // namespace det
}  // namespace mcb200
