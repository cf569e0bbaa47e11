// RPN ProposalLayer on the device, batched over images:
//   1. decode      anchor + deltas -> clipped box, min-size filter, sort key
//   2. top-k sort  per image: radix-select the pre_nms_topn best keys, bitonic
//                  sort them in shared memory, gather boxes in score order
//   3. greedy NMS  per image: one block walks the boxes 64 at a time and evaluates
//                  overlaps only for rows that are kept against columns that are
//                  still alive; stops at post_nms_topn; writes rois (+ scores)
//                  and the count
// The host only reads the per-image counts back.
//
// Every float operation that decides which boxes are kept is done with the
// rounding of the CPU code it replaces (mini-caffe src/layers/proposal_layer.cpp:
// TransformBBox :14-53, GenerateProposalsCPU :114-148, SortBBox :88-111,
// NonMaximumSuppressionCPU :150-185, RetrieveRoisCPU :187-203): separate
// multiply and add (no FMA), exp() evaluated in double and the product rounded
// to float once, IEEE division.  Boxes with equal scores are ordered by
// proposal index (the CPU quicksort leaves that order unspecified).
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <mutex>

#include "../../../include/mcb200_kernels.h"
#include "detection.cuh"
#include "launch_count.h"

namespace mcb200 {
namespace {

using namespace det;

struct Workspace {
  float4* boxes;                 // [batch][n]        decoded boxes, proposal order
  float* scores;                 // [batch][n]
  unsigned long long* keys;      // [batch][n]
  float4* sorted_boxes;          // [batch][k]        score order
  float* sorted_scores;          // [batch][k]
  int n, k, col_blocks;
};

size_t align_up(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

size_t carve(const mcb200_proposal_params& p, int batch, char* base, Workspace* ws) {
  const int n = p.num_anchors * p.height * p.width;
  const int k = n < p.pre_nms_topn ? n : p.pre_nms_topn;
  const int cb = (k + 63) / 64;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    char* ptr = base ? base + off : nullptr;
    off += align_up(bytes);
    return ptr;
  };
  Workspace w;
  w.n = n;
  w.k = k;
  w.col_blocks = cb;
  w.boxes = reinterpret_cast<float4*>(take(sizeof(float4) * n * static_cast<size_t>(batch)));
  w.scores = reinterpret_cast<float*>(take(sizeof(float) * n * static_cast<size_t>(batch)));
  w.keys = reinterpret_cast<unsigned long long*>(take(8 * static_cast<size_t>(n) * batch));
  w.sorted_boxes = reinterpret_cast<float4*>(take(sizeof(float4) * k * static_cast<size_t>(batch)));
  w.sorted_scores = reinterpret_cast<float*>(take(sizeof(float) * k * static_cast<size_t>(batch)));
  if (ws) *ws = w;
  return off;
}

// ---------------------------------------------------------------- 1. decode

__global__ void proposal_decode_kernel(const float* __restrict__ score_maps, const float* __restrict__ delta_maps,
                                       const float* __restrict__ im_info, const float* __restrict__ anchors,
                                       mcb200_proposal_params p, Workspace ws) {
  const int image = blockIdx.y;
  const int hw = p.height * p.width;
  const int n = ws.n;
  // Foreground scores are the second half of the 2A score channels.
  const float* score = score_maps + static_cast<size_t>(image) * 2 * p.num_anchors * hw + static_cast<size_t>(n);
  const float* delta = delta_maps + static_cast<size_t>(image) * 4 * p.num_anchors * hw;
  const float img_h = im_info[image * 3 + 0];
  const float img_w = im_info[image * 3 + 1];
  const float min_size = fmul(static_cast<float>(p.min_size), im_info[image * 3 + 2]);
  // Threads run over (anchor, y, x) with x fastest, so the map reads coalesce.
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < n; t += gridDim.x * blockDim.x) {
    const int k = t / hw;
    const int pos = t - k * hw;
    const int y = pos / p.width;
    const int x = pos - y * p.width;
    const float fx = static_cast<float>(x * p.feat_stride);
    const float fy = static_cast<float>(y * p.feat_stride);
    float b0 = fadd(fx, anchors[k * 4 + 0]);
    float b1 = fadd(fy, anchors[k * 4 + 1]);
    float b2 = fadd(fx, anchors[k * 4 + 2]);
    float b3 = fadd(fy, anchors[k * 4 + 3]);
    const float dx = delta[(k * 4 + 0) * hw + pos];
    const float dy = delta[(k * 4 + 1) * hw + pos];
    const float dlw = delta[(k * 4 + 2) * hw + pos];
    const float dlh = delta[(k * 4 + 3) * hw + pos];

    const float w = fadd(fsub(b2, b0), 1.f);
    const float h = fadd(fsub(b3, b1), 1.f);
    const float ctr_x = fadd(b0, fmul(0.5f, w));
    const float ctr_y = fadd(b1, fmul(0.5f, h));
    const float pred_ctr_x = fadd(fmul(dx, w), ctr_x);
    const float pred_ctr_y = fadd(fmul(dy, h), ctr_y);
    // exp in double, product in double, one rounding to float.
    const float pred_w = static_cast<float>(__dmul_rn(exp(static_cast<double>(dlw)), static_cast<double>(w)));
    const float pred_h = static_cast<float>(__dmul_rn(exp(static_cast<double>(dlh)), static_cast<double>(h)));
    b0 = fsub(pred_ctr_x, fmul(0.5f, pred_w));
    b1 = fsub(pred_ctr_y, fmul(0.5f, pred_h));
    b2 = fadd(pred_ctr_x, fmul(0.5f, pred_w));
    b3 = fadd(pred_ctr_y, fmul(0.5f, pred_h));
    const float max_x = fsub(img_w, 1.f);
    const float max_y = fsub(img_h, 1.f);
    b0 = fmaxf(0.f, fminf(b0, max_x));
    b1 = fmaxf(0.f, fminf(b1, max_y));
    b2 = fmaxf(0.f, fminf(b2, max_x));
    b3 = fmaxf(0.f, fminf(b3, max_y));
    const float box_w = fadd(fsub(b2, b0), 1.f);
    const float box_h = fadd(fsub(b3, b1), 1.f);
    const int valid = (box_w >= min_size) && (box_h >= min_size);
    const float s = fmul(static_cast<float>(valid), score[k * hw + pos]);

    const int index = pos * p.num_anchors + k;   // proposal order: (y, x, anchor)
    const size_t o = static_cast<size_t>(image) * n + index;
    ws.boxes[o] = make_float4(b0, b1, b2, b3);
    ws.scores[o] = s;
    ws.keys[o] = make_key(s, static_cast<uint32_t>(index));
  }
}

// ---------------------------------------------------------------- 2. top-k + sort

// One block per image.  The score halves of the keys (the index half of key i
// is i itself) are copied to shared memory once, with all loads of a thread in
// flight together; the passes of the radix select, which test one key after the
// other with a warp vote in between, and the compaction then run out of shared
// memory instead of paying an L2 round trip per key and pass.  `staged` = 0 (the
// keys do not fit beside the sort buffer): they are read from global memory.
__global__ void __launch_bounds__(1024, 1)
proposal_topk_sort_kernel(Workspace ws, int padded, int staged) {
  extern __shared__ unsigned long long sorted[];   // `padded` keys, then (staged) n 32-bit score keys
  __shared__ int hist[256];
  __shared__ unsigned long long bcast[2];
  __shared__ int fill;
  const int image = blockIdx.x;
  const unsigned long long* keys = ws.keys + static_cast<size_t>(image) * ws.n;
  const int n = ws.n, k = ws.k;
  uint32_t* score_key = reinterpret_cast<uint32_t*>(sorted + padded);
  if (staged) {
    for (int i = threadIdx.x; i < n; i += blockDim.x) score_key[i] = static_cast<uint32_t>(keys[i] >> 32);
  }
  if (threadIdx.x == 0) fill = 0;
  for (int i = threadIdx.x; i < padded; i += blockDim.x) sorted[i] = kPadKey;
  __syncthreads();
  auto key_at = [&](int i) {
    return staged ? ((static_cast<unsigned long long>(score_key[i]) << 32) | static_cast<uint32_t>(i)) : keys[i];
  };

  unsigned long long threshold = kPadKey;
  if (k < n) threshold = block_kth_smallest(key_at, n, k, hist, bcast);
  // Append the selected keys, one update of the shared counter per warp.
  for (int base = 0; base < n; base += blockDim.x) {
    const int i = base + threadIdx.x;
    unsigned long long key = 0;
    bool take = false;
    if (i < n) {
      key = key_at(i);
      take = key <= threshold;
    }
    const unsigned taking = __ballot_sync(0xffffffffu, take);
    if (taking) {
      const int lane = threadIdx.x & 31;
      const int leader = __ffs(taking) - 1;
      int first = 0;
      if (lane == leader) first = atomicAdd(&fill, __popc(taking));
      first = __shfl_sync(0xffffffffu, first, leader);
      const int slot = first + __popc(taking & ((1u << lane) - 1u));
      if (take && slot < padded) sorted[slot] = key;
    }
  }
  __syncthreads();
  block_sort_keys(sorted, padded);
  const float4* boxes = ws.boxes + static_cast<size_t>(image) * n;
  const float* scores = ws.scores + static_cast<size_t>(image) * n;
  // Gather in groups of four per thread: the four box and score loads (random
  // rows, an L2 round trip each) are issued before the first store.
  for (int base = threadIdx.x; base < k; base += 4 * blockDim.x) {
    float4 box[4];
    float score[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = base + u * blockDim.x;
      if (i < k) {
        const uint32_t index = static_cast<uint32_t>(sorted[i] & 0xFFFFFFFFull);
        box[u] = boxes[index];
        score[u] = scores[index];
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = base + u * blockDim.x;
      if (i < k) {
        ws.sorted_boxes[static_cast<size_t>(image) * k + i] = box[u];
        ws.sorted_scores[static_cast<size_t>(image) * k + i] = score[u];
      }
    }
  }
}

// ---------------------------------------------------------------- 3a. overlap test

// IoU with the "+1 pixel" convention; areas[i] + areas[j] - inter, IEEE division.
__device__ __forceinline__ bool suppresses(const float4& a, float area_a, const float4& b, float area_b,
                                           float threshold) {
  const float x1 = fmaxf(a.x, b.x);
  const float y1 = fmaxf(a.y, b.y);
  const float x2 = fminf(a.z, b.z);
  const float y2 = fminf(a.w, b.w);
  const float w = fmaxf(0.f, fadd(fsub(x2, x1), 1.f));
  const float h = fmaxf(0.f, fadd(fsub(y2, y1), 1.f));
  const float inter = fmul(w, h);
  const float ov = fdiv(inter, fsub(fadd(area_a, area_b), inter));
  return ov > threshold;
}

__device__ __forceinline__ float box_area(const float4& b) {
  return fmul(fadd(fsub(b.z, b.x), 1.f), fadd(fsub(b.w, b.y), 1.f));
}

// ---------------------------------------------------------------- 3b. greedy suppression + output

constexpr int kNmsThreads = 1024;
// Boxes of one image are staged in shared memory when they fit (20 bytes each).
constexpr int kNmsStagedBoxes = 8192;

// Bytes in front of the staged boxes: the indices of the kept boxes (at most
// post_nms_topn), rounded up so that the float4 array starts on a 16-byte boundary.
__host__ __device__ constexpr size_t nms_kept_bytes(int post_nms_topn) {
  return (static_cast<size_t>(post_nms_topn) * 4 + 15) & ~static_cast<size_t>(15);
}

// One block per image walks the score-ordered boxes 64 at a time.  Per step:
//   1. all threads: which of the step's 64 boxes does an already kept box
//      suppress (kept boxes x 64 columns), and the 64 x 64 overlaps inside the
//      block (bit c of diag[r] = "row r suppresses column c", c > r);
//   2. thread 0: resolves the block in order (a box is kept unless an earlier
//      kept box suppresses it) and stops at post_nms_topn; the kept boxes are
//      then written out and appended to the kept list in parallel.
// Overlaps are evaluated lazily, only between kept boxes and the boxes the walk
// actually reaches: at most post_nms_topn x pre_nms_topn pairs, and far fewer
// when the walk ends early, instead of the pre_nms_topn^2 / 2 pairs of a full
// suppression matrix.  The kept set is that of the sequential algorithm
// (src/layers/proposal_layer.cpp:161-186).
__global__ void __launch_bounds__(kNmsThreads)
proposal_nms_kernel(Workspace ws, float threshold, int post_nms_topn, int staged, float* __restrict__ rois,
                    float* __restrict__ roi_scores, int* __restrict__ counts) {
  extern __shared__ __align__(16) unsigned char nms_smem[];
  __shared__ unsigned long long diag[64];
  __shared__ unsigned long long gone_word;   // columns of the current block that kept boxes suppress
  __shared__ unsigned long long keep_word;
  __shared__ int kept_total;
  __shared__ int stop;
  const int image = blockIdx.x;
  const int k = ws.k, cb = ws.col_blocks;
  const int kpad = cb * 64;
  const float4* g_boxes = ws.sorted_boxes + static_cast<size_t>(image) * k;
  const float* scores = ws.sorted_scores + static_cast<size_t>(image) * k;
  float* out = rois + static_cast<size_t>(image) * post_nms_topn * 5;
  float* out_scores = roi_scores ? roi_scores + static_cast<size_t>(image) * post_nms_topn : nullptr;

  int* kept = reinterpret_cast<int*>(nms_smem);
  float4* s_boxes = reinterpret_cast<float4*>(nms_smem + nms_kept_bytes(post_nms_topn));   // 16-byte aligned
  float* s_area = reinterpret_cast<float*>(s_boxes + kpad);
  const int t = threadIdx.x;
  if (staged) {
    for (int i = t; i < kpad; i += kNmsThreads) {
      const float4 b = i < k ? g_boxes[i] : make_float4(0.f, 0.f, 0.f, 0.f);
      s_boxes[i] = b;
      s_area[i] = box_area(b);
    }
  }
  if (t == 0) {
    kept_total = 0;
    stop = 0;
  }
  __syncthreads();
  auto box_at = [&](int i) { return staged ? s_boxes[i] : g_boxes[i]; };
  auto area_at = [&](int i, const float4& b) { return staged ? s_area[i] : box_area(b); };

  bool done = false;
  for (int block = 0; block < cb && !done; ++block) {
    const int base = block * 64;
    const int rows = min(64, k - base);
    if (t < 64) diag[t] = 0ull;
    if (t == 0) gone_word = 0ull;
    const int total_before = kept_total;   // read before the barrier: thread 0 updates it in step 2
    __syncthreads();
    // ---- 1a. kept boxes against this block: thread = (column, every 16th kept box)
    {
      const int c = t & 63;
      if (c < rows) {
        const float4 b = box_at(base + c);
        const float area_b = area_at(base + c, b);
        bool hit = false;
        for (int q = t >> 6; q < total_before && !hit; q += kNmsThreads / 64) {
          const int i = kept[q];
          const float4 a = box_at(i);
          hit = suppresses(a, area_at(i, a), b, area_b, threshold);
        }
        if (hit) atomicOr(&gone_word, 1ull << c);
      }
    }
    // ---- 1b. overlaps inside the block: thread = (row, group of four columns)
    {
      const int r = t >> 4;
      const int c0 = (t & 15) * 4;
      if (r < rows && c0 + 3 > r) {
        const float4 a = box_at(base + r);
        const float area_a = area_at(base + r, a);
        unsigned long long bits = 0ull;
#pragma unroll
        for (int c = c0; c < c0 + 4; ++c) {
          if (c > r && c < rows) {
            const float4 b = box_at(base + c);
            if (suppresses(a, area_a, b, area_at(base + c, b), threshold)) bits |= 1ull << c;
          }
        }
        if (bits) atomicOr(&diag[r], bits);
      }
    }
    __syncthreads();
    // ---- 2. resolve the block in score order
    if (t == 0) {
      unsigned long long gone = gone_word;
      unsigned long long keep = 0ull;
      int total = total_before;
      for (int r = 0; r < rows; ++r) {
        if (!((gone >> r) & 1ull)) {
          keep |= 1ull << r;
          ++total;
          if (total == post_nms_topn) {
            stop = 1;
            break;
          }
          gone |= diag[r];
        }
      }
      keep_word = keep;
      kept_total = total;
    }
    __syncthreads();
    if (t < rows && ((keep_word >> t) & 1ull)) {
      const int pos = total_before + __popcll(keep_word & ((1ull << t) - 1ull));
      const int i = base + t;
      kept[pos] = i;
      const float4 b = g_boxes[i];
      out[pos * 5 + 0] = static_cast<float>(image);
      out[pos * 5 + 1] = b.x;
      out[pos * 5 + 2] = b.y;
      out[pos * 5 + 3] = b.z;
      out[pos * 5 + 4] = b.w;
      if (out_scores) out_scores[pos] = scores[i];
    }
    // Everyone takes the same copy of the flag here; thread 0 writes it again
    // only after the next iteration's first barrier.
    done = stop != 0;
    __syncthreads();
  }
  if (t == 0) counts[image] = kept_total;
}

}  // namespace
}  // namespace mcb200

using namespace mcb200;

static int validate(const mcb200_proposal_params* p, int batch) {
  if (!p || batch < 1) return -1;
  if (p->num_anchors < 1 || p->height < 1 || p->width < 1 || p->feat_stride < 1 || p->pre_nms_topn < 1 ||
      p->post_nms_topn < 1)
    return -2;
  const long long n = static_cast<long long>(p->num_anchors) * p->height * p->width;
  if (n > (1 << 24)) return -3;
  const int k = n < p->pre_nms_topn ? static_cast<int>(n) : p->pre_nms_topn;
  // The sorted keys of one image live in shared memory (8 bytes each).
  if (det::next_pow2(k) > 16384) return -4;
  return 0;
}

constexpr size_t kSortSharedLimit = 220 * 1024;

// The top-k and the NMS kernel use more dynamic shared memory than a kernel gets
// by default; the opt-in is per device and is made on a device's first call
// (nets on several host threads may make that call at the same time).
static cudaError_t configure_kernels() {
  static bool configured[64] = {false};
  static std::mutex mu;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> lock(mu);
  if (dev < 0 || dev >= 64 || configured[dev]) return cudaSuccess;
  e = cudaFuncSetAttribute(proposal_topk_sort_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(kSortSharedLimit));
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(proposal_nms_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
  if (e != cudaSuccess) return e;
  configured[dev] = true;
  return cudaSuccess;
}

// Moves the valid rows of images 1 .. batch-1 up against those of the image in
// front (rows of image b start at b * post and move to the sum of the counts
// before it).  A row never moves to a higher address and images are handled in
// order, so what is overwritten has been moved already; inside an image the
// block copies `blockDim.x` values at a time, reading a piece completely before
// writing it (source and destination ranges may overlap).
static __global__ void proposal_compact_kernel(float* __restrict__ rois, float* __restrict__ roi_scores,
                                        const int* __restrict__ counts, int batch, int post) {
  int total = counts[0];
  for (int b = 1; b < batch; ++b) {
    const int rows = counts[b];
    if (rows > 0 && total != b * post) {
      for (int pass = 0; pass < 2; ++pass) {
        float* base = pass == 0 ? rois : roi_scores;
        if (!base) continue;
        const int width = pass == 0 ? 5 : 1;
        const float* src = base + static_cast<size_t>(b) * post * width;
        float* dst = base + static_cast<size_t>(total) * width;
        const int values = rows * width;
        for (int i0 = 0; i0 < values; i0 += blockDim.x) {
          const int i = i0 + threadIdx.x;
          const float v = i < values ? src[i] : 0.f;
          __syncthreads();
          if (i < values) dst[i] = v;
          __syncthreads();
        }
      }
    }
    total += rows;
  }
}

extern "C" size_t mcb200_proposal_workspace_bytes(const mcb200_proposal_params* p, int batch) {
  if (validate(p, batch) != 0) return 0;
  return carve(*p, batch, nullptr, nullptr);
}

extern "C" int mcb200_proposal_forward(const mcb200_proposal_params* p, int batch, const float* scores,
                                       const float* deltas, const float* im_info, const float* anchors,
                                       void* workspace, float* rois, float* roi_scores, int* counts, void* stream) {
  const int rc = validate(p, batch);
  if (rc != 0) return rc;
  if (!scores || !deltas || !im_info || !anchors || !workspace || !rois || !counts) return -5;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return -6;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const cudaError_t configured = configure_kernels();
  if (configured != cudaSuccess) return static_cast<int>(configured);
  Workspace ws;
  carve(*p, batch, static_cast<char*>(workspace), &ws);

  {
    const int threads = 256;
    int blocks = (ws.n + threads - 1) / threads;
    if (blocks > 148 * 4) blocks = 148 * 4;
    proposal_decode_kernel<<<dim3(blocks, batch), threads, 0, st>>>(scores, deltas, im_info, anchors, *p, ws);
    count_launch();
  }
  {
    const int padded = det::next_pow2(ws.k);
    const size_t sort_bytes = static_cast<size_t>(padded) * 8;
    const size_t staged_bytes = sort_bytes + static_cast<size_t>(ws.n) * 4;
    if (sort_bytes > kSortSharedLimit) return -8;
    const int staged = staged_bytes <= kSortSharedLimit ? 1 : 0;
    const size_t smem = staged ? staged_bytes : sort_bytes;
    proposal_topk_sort_kernel<<<batch, 1024, smem, st>>>(ws, padded, staged);
    count_launch();
  }
  {
    // Boxes and areas of an image go to shared memory when they fit.
    const int staged = ws.col_blocks * 64 <= kNmsStagedBoxes ? 1 : 0;
    const size_t smem = nms_kept_bytes(p->post_nms_topn) + (staged ? static_cast<size_t>(ws.col_blocks) * 64 * 20 : 0);
    if (smem > 220 * 1024) return -7;   // post_nms_topn beyond 10000 with staged boxes: not a detector's setting
    proposal_nms_kernel<<<batch, kNmsThreads, smem, st>>>(ws, p->nms_thresh, p->post_nms_topn, staged, rois, roi_scores,
                                                           counts);
    count_launch();
  }
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mcb200_proposal_compact(float* rois, float* roi_scores, const int* counts, int batch,
                                       int post_nms_topn, void* stream) {
  if (!rois || !counts || batch < 1 || post_nms_topn < 1) return -1;
  if (batch == 1) return 0;
  proposal_compact_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(rois, roi_scores, counts, batch,
                                                                             post_nms_topn);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

// ------------------------------------------------------------------ variant without allocation

// Scratch of mcb200_proposal_forward_static.  It lives in the library's device
// image: every GPU that loads the library carries these 8 MiB until the process
// exits.  The largest single image the kernels accept (65536 proposals of which
// 6000 go to NMS) takes 1.9 MB of it, an image of the stock R-FCN setting (63 x 38
// map, 15 anchors) 1.1 MB; a call whose batch needs more than the array holds
// is refused.
static constexpr size_t kStaticScratchBytes = static_cast<size_t>(8) << 20;
static __device__ __align__(256) unsigned char g_proposal_static_scratch[kStaticScratchBytes];

namespace {

// Device address of the scratch array on the current device, looked up once per device.
// In host code the array's name is only a handle; the address has to be asked for
// with that device current.
int static_scratch(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= 64) return -21;
  static void* scratch_of_device[64] = {nullptr};
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  if (!scratch_of_device[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_proposal_static_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (!ptr) return -22;
    scratch_of_device[dev] = ptr;
  }
  *out = scratch_of_device[dev];
  return 0;
}

}  // namespace

extern "C" int mcb200_proposal_static_warmup(void) {
  void* scratch = nullptr;
  const int rc = static_scratch(&scratch);
  if (rc != 0) return rc;
  return static_cast<int>(configure_kernels());
}

extern "C" int mcb200_proposal_forward_static(const mcb200_proposal_params* p, int batch, const float* scores,
                                              const float* deltas, const float* im_info, const float* anchors,
                                              float* rois, float* roi_scores, int* counts, void* stream) {
  const int rc = validate(p, batch);
  if (rc != 0) return rc;
  const size_t need = carve(*p, batch, nullptr, nullptr);
  if (need > kStaticScratchBytes) {
    fprintf(stderr,
            "mcb200_proposal_forward_static: this request needs %zu bytes of scratch, the built-in buffer holds %zu; "
            "use mcb200_proposal_forward with a caller-provided workspace\n",
            need, kStaticScratchBytes);
    return -20;
  }
  void* scratch = nullptr;
  const int found = static_scratch(&scratch);
  if (found != 0) return found;
  // Every scratch word the kernels read is written earlier in the same call
  // (keys, boxes and scores for all proposals, the sorted copies for the best
  // pre_nms_topn), so nothing has to be cleared between calls.
  return mcb200_proposal_forward(p, batch, scores, deltas, im_info, anchors, scratch, rois, roi_scores, counts,
                                 stream);
}
