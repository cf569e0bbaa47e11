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

// The same network with the keys in registers: thread t owns elements
// t * E .. t * E + E - 1 (count == blockDim.x * E).  Strides below E stay inside
// a thread, strides below 32 E are exchanged with warp shuffles, and only the
// larger ones go through shared memory (15 of the 91 passes for 8192 keys and
// 1024 threads), in a layout transposed so that a warp touches consecutive
// cells.  Each side of a pair keeps its own result (the smaller key where the
// run ascends and it is the lower index, and so on), so no write conflicts.
template <int E>
__device__ inline void block_bitonic_sort_regs(unsigned long long* keys) {
  const int t = threadIdx.x;
  const int threads = blockDim.x;
  const int count = threads * E;
  unsigned long long v[E];
#pragma unroll
  for (int j = 0; j < E; ++j) v[j] = keys[t * E + j];
  __syncthreads();   // the array is scratch from here on
  for (int size = 2; size <= count; size <<= 1) {
    int stride = size >> 1;
    for (; stride >= E * 32; stride >>= 1) {   // partner in another warp
#pragma unroll
      for (int j = 0; j < E; ++j) keys[j * threads + t] = v[j];
      __syncthreads();
      const int partner = t ^ (stride / E);
#pragma unroll
      for (int j = 0; j < E; ++j) {
        const int e = t * E + j;
        const unsigned long long other = keys[j * threads + partner];
        const bool keep_small = ((e & stride) == 0) == ((e & size) == 0);
        v[j] = keep_small ? (v[j] < other ? v[j] : other) : (v[j] > other ? v[j] : other);
      }
      __syncthreads();
    }
    for (; stride >= E; stride >>= 1) {        // partner in another lane
      const int lanes = stride / E;
#pragma unroll
      for (int j = 0; j < E; ++j) {
        const int e = t * E + j;
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, v[j], lanes);
        const bool keep_small = ((e & stride) == 0) == ((e & size) == 0);
        v[j] = keep_small ? (v[j] < other ? v[j] : other) : (v[j] > other ? v[j] : other);
      }
    }
    // Partner in the same thread: the strides are compile-time constants so
    // that the keys stay in registers (an index computed at run time would put
    // the array into local memory).
#pragma unroll
    for (int st = E / 2; st > 0; st >>= 1) {
      if (st <= stride) {
#pragma unroll
        for (int j = 0; j < E; ++j) {
          if ((j & st) == 0) {
            const int e = t * E + j;
            const unsigned long long a = v[j], b = v[j | st];
            const bool swap = (a > b) == ((e & size) == 0);
            v[j] = swap ? b : a;
            v[j | st] = swap ? a : b;
          }
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < E; ++j) keys[t * E + j] = v[j];
  __syncthreads();
}

// Sorts `count` keys (a power of two) with the register variant when the block
// has one thread per 1, 2, 4, 8 or 16 keys, else with the shared-memory one.
__device__ inline void block_sort_keys(unsigned long long* keys, int count) {
  const int threads = blockDim.x;
  if ((threads & 31) == 0 && count >= threads && count % threads == 0) {
    switch (count / threads) {
      case 1: block_bitonic_sort_regs<1>(keys); return;
      case 2: block_bitonic_sort_regs<2>(keys); return;
      case 4: block_bitonic_sort_regs<4>(keys); return;
      case 8: block_bitonic_sort_regs<8>(keys); return;
      case 16: block_bitonic_sort_regs<16>(keys); return;
      default: break;
    }
  }
  block_bitonic_sort(keys, count);
}

__host__ __device__ inline int next_pow2(int v) {
  int p = 1;
  while (p < v) p <<= 1;
  return p;
}

}  // namespace det
}  // namespace mcb200
