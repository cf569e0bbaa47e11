// SSD DetectionOutput on the device:
//   A. per (image, class) block: collect priors whose class score passes the
//      confidence threshold, take the top_k best (radix select + bitonic sort in
//      shared memory, ties by prior index like std::stable_sort), decode their
//      boxes, greedy NMS (overlap bit matrix by the whole block, walk by one warp)
//   B. per image block: if more than keep_top_k detections survive, keep the
//      keep_top_k best over all classes; lay the rows out label-ascending
//   C. per image block: prefix sum of the per-image counts, compact the rows
// The host reads back one int (the row count).
//
// Arithmetic follows mini-caffe's CPU code operation by operation so that the
// kept sets agree bit for bit: DecodeBBox (src/util/bbox_util.cpp:242-330;
// centre/size decode with exp() in double, results rounded to float once),
// BBoxSize (:80-98), JaccardOverlap (:184-205), GetMaxScoreIndex (:524-541),
// ApplyNMSFast (:681-716), the keep_top_k step and row layout of
// DetectionOutputLayer::Forward_cpu (src/layers/detection_output_layer.cpp:107-225).
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include <mutex>

#include "../../../include/mcb200_kernels.h"
#include "detection.cuh"
#include "launch_count.h"

namespace mcb200 {
namespace {

using namespace det;

struct Entry {       // one kept detection of one (image, class)
  float score;
  float xmin, ymin, xmax, ymax;
};

struct Workspace {
  Entry* entries;    // [batch][classes][per_class]
  int* class_count;  // [batch][classes]
  float* rows;       // [batch][max_rows][7]
  int* image_count;  // [batch]
  int per_class, max_rows;
};

size_t align_up(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

int per_class_limit(const mcb200_detout_params& p) {
  int k = p.top_k < 0 ? p.num_priors : p.top_k;
  if (k > p.num_priors) k = p.num_priors;
  return k;
}

int max_rows(const mcb200_detout_params& p) {
  const int classes = p.num_classes - (p.background_label_id >= 0 && p.background_label_id < p.num_classes ? 1 : 0);
  long long all = static_cast<long long>(classes) * per_class_limit(p);
  if (p.keep_top_k > -1 && p.keep_top_k < all) all = p.keep_top_k;
  return static_cast<int>(all);
}

size_t carve(const mcb200_detout_params& p, int batch, char* base, Workspace* ws) {
  size_t off = 0;
  auto take = [&](size_t bytes) {
    char* ptr = base ? base + off : nullptr;
    off += align_up(bytes);
    return ptr;
  };
  Workspace w;
  w.per_class = per_class_limit(p);
  w.max_rows = max_rows(p);
  w.entries = reinterpret_cast<Entry*>(take(sizeof(Entry) * static_cast<size_t>(batch) * p.num_classes * w.per_class));
  w.class_count = reinterpret_cast<int*>(take(sizeof(int) * static_cast<size_t>(batch) * p.num_classes));
  w.rows = reinterpret_cast<float*>(take(sizeof(float) * 7 * static_cast<size_t>(batch) * (w.max_rows > 0 ? w.max_rows : 1)));
  w.image_count = reinterpret_cast<int*>(take(sizeof(int) * static_cast<size_t>(batch)));
  if (ws) *ws = w;
  return off;
}

// ---------------------------------------------------------------- box arithmetic

struct Box {
  float xmin, ymin, xmax, ymax, size;
};

__device__ __forceinline__ float box_size(float xmin, float ymin, float xmax, float ymax) {
  if (xmax < xmin || ymax < ymin) return 0.f;
  return fmul(fsub(xmax, xmin), fsub(ymax, ymin));
}

__device__ Box decode_box(const mcb200_detout_params& p, const float* prior, const float* var, const float* loc) {
  const float pxmin = prior[0], pymin = prior[1], pxmax = prior[2], pymax = prior[3];
  const float bx0 = loc[0], bx1 = loc[1], bx2 = loc[2], bx3 = loc[3];
  Box b;
  if (p.code_type == 1) {  // CORNER
    if (p.variance_encoded_in_target) {
      b.xmin = fadd(pxmin, bx0);
      b.ymin = fadd(pymin, bx1);
      b.xmax = fadd(pxmax, bx2);
      b.ymax = fadd(pymax, bx3);
    } else {
      b.xmin = fadd(pxmin, fmul(var[0], bx0));
      b.ymin = fadd(pymin, fmul(var[1], bx1));
      b.xmax = fadd(pxmax, fmul(var[2], bx2));
      b.ymax = fadd(pymax, fmul(var[3], bx3));
    }
  } else if (p.code_type == 2) {  // CENTER_SIZE
    const float pw = fsub(pxmax, pxmin);
    const float ph = fsub(pymax, pymin);
    // (a + b) / 2. is evaluated in double and rounded to float.
    const float pcx = static_cast<float>(__ddiv_rn(static_cast<double>(fadd(pxmin, pxmax)), 2.0));
    const float pcy = static_cast<float>(__ddiv_rn(static_cast<double>(fadd(pymin, pymax)), 2.0));
    float cx, cy, w, h;
    if (p.variance_encoded_in_target) {
      cx = fadd(fmul(bx0, pw), pcx);
      cy = fadd(fmul(bx1, ph), pcy);
      w = static_cast<float>(__dmul_rn(exp(static_cast<double>(bx2)), static_cast<double>(pw)));
      h = static_cast<float>(__dmul_rn(exp(static_cast<double>(bx3)), static_cast<double>(ph)));
    } else {
      cx = fadd(fmul(fmul(var[0], bx0), pw), pcx);
      cy = fadd(fmul(fmul(var[1], bx1), ph), pcy);
      w = static_cast<float>(__dmul_rn(exp(static_cast<double>(fmul(var[2], bx2))), static_cast<double>(pw)));
      h = static_cast<float>(__dmul_rn(exp(static_cast<double>(fmul(var[3], bx3))), static_cast<double>(ph)));
    }
    // centre -+ size / 2. : double subtraction, one rounding to float.
    const double hw = __ddiv_rn(static_cast<double>(w), 2.0);
    const double hh = __ddiv_rn(static_cast<double>(h), 2.0);
    b.xmin = static_cast<float>(__dsub_rn(static_cast<double>(cx), hw));
    b.ymin = static_cast<float>(__dsub_rn(static_cast<double>(cy), hh));
    b.xmax = static_cast<float>(__dadd_rn(static_cast<double>(cx), hw));
    b.ymax = static_cast<float>(__dadd_rn(static_cast<double>(cy), hh));
  } else {  // CORNER_SIZE
    const float pw = fsub(pxmax, pxmin);
    const float ph = fsub(pymax, pymin);
    if (p.variance_encoded_in_target) {
      b.xmin = fadd(pxmin, fmul(bx0, pw));
      b.ymin = fadd(pymin, fmul(bx1, ph));
      b.xmax = fadd(pxmax, fmul(bx2, pw));
      b.ymax = fadd(pymax, fmul(bx3, ph));
    } else {
      b.xmin = fadd(pxmin, fmul(fmul(var[0], bx0), pw));
      b.ymin = fadd(pymin, fmul(fmul(var[1], bx1), ph));
      b.xmax = fadd(pxmax, fmul(fmul(var[2], bx2), pw));
      b.ymax = fadd(pymax, fmul(fmul(var[3], bx3), ph));
    }
  }
  b.size = box_size(b.xmin, b.ymin, b.xmax, b.ymax);
  return b;
}

// Jaccard overlap of normalised boxes; 0 when they do not intersect.
__device__ __forceinline__ float jaccard(const Box& a, const Box& b) {
  if (b.xmin > a.xmax || b.xmax < a.xmin || b.ymin > a.ymax || b.ymax < a.ymin) return 0.f;
  const float ixmin = fmaxf(a.xmin, b.xmin);
  const float iymin = fmaxf(a.ymin, b.ymin);
  const float ixmax = fminf(a.xmax, b.xmax);
  const float iymax = fminf(a.ymax, b.ymax);
  const float iw = fsub(ixmax, ixmin);
  const float ih = fsub(iymax, iymin);
  if (iw > 0.f && ih > 0.f) {
    const float isize = fmul(iw, ih);
    return fdiv(isize, fsub(fadd(a.size, b.size), isize));
  }
  return 0.f;
}

// ---------------------------------------------------------------- A. per (image, class)

// Shared memory: candidate keys [num_priors], selected keys [padded], boxes
// [padded], kept list [padded].
__global__ void __launch_bounds__(256)
detout_class_kernel(const float* __restrict__ loc, const float* __restrict__ conf, const float* __restrict__ prior,
                    mcb200_detout_params p, Workspace ws, int padded, float eta) {
  extern __shared__ unsigned long long smem_keys[];
  unsigned long long* cand = smem_keys;
  unsigned long long* sel = cand + p.num_priors;
  Box* boxes = reinterpret_cast<Box*>(sel + padded);
  int* kept = reinterpret_cast<int*>(boxes + padded);
  __shared__ int hist[256];
  __shared__ unsigned long long bcast[2];
  __shared__ int num_cand, num_sel, num_kept;

  const int cls = blockIdx.x;
  const int image = blockIdx.y;
  const int limit = ws.per_class;
  int* out_count = ws.class_count + static_cast<size_t>(image) * p.num_classes + cls;
  if (cls == p.background_label_id) {
    if (threadIdx.x == 0) *out_count = 0;
    return;
  }
  if (threadIdx.x == 0) {
    num_cand = 0;
    num_sel = 0;
    num_kept = 0;
  }
  __syncthreads();
  const float* scores = conf + static_cast<size_t>(image) * p.num_priors * p.num_classes + cls;
  // Append the passing priors, one shared-memory counter update per warp (with
  // near-uniform scores nearly every prior passes, and 8732 single updates of
  // one counter would serialise).  The order of the list does not matter.
  for (int base = 0; base < p.num_priors; base += blockDim.x) {
    const int i = base + threadIdx.x;
    float s = 0.f;
    bool pass = false;
    if (i < p.num_priors) {
      s = scores[static_cast<size_t>(i) * p.num_classes];
      pass = s > p.confidence_threshold;
    }
    const unsigned passing = __ballot_sync(0xffffffffu, pass);
    if (passing) {
      const int lane = threadIdx.x & 31;
      const int leader = __ffs(passing) - 1;
      int first = 0;
      if (lane == leader) first = atomicAdd(&num_cand, __popc(passing));
      first = __shfl_sync(0xffffffffu, first, leader);
      if (pass) cand[first + __popc(passing & ((1u << lane) - 1u))] = make_key(s, static_cast<uint32_t>(i));
    }
  }
  __syncthreads();
  const int m = num_cand;
  const int count = m < limit ? m : limit;
  unsigned long long threshold = kPadKey;
  if (m > limit) threshold = block_kth_smallest([&](int i) { return cand[i]; }, m, limit, hist, bcast);
  for (int i = threadIdx.x; i < padded; i += blockDim.x) sel[i] = kPadKey;
  __syncthreads();
  for (int i = threadIdx.x; i < m; i += blockDim.x) {
    const unsigned long long key = cand[i];
    if (key <= threshold) {
      const int slot = atomicAdd(&num_sel, 1);
      if (slot < padded) sel[slot] = key;
    }
  }
  __syncthreads();
  block_sort_keys(sel, padded);

  // Decode only the boxes that compete.
  const int loc_classes = p.share_location ? 1 : p.num_classes;
  const int loc_cls = p.share_location ? 0 : cls;
  const float* var = prior + static_cast<size_t>(p.num_priors) * 4;
  for (int i = threadIdx.x; i < count; i += blockDim.x) {
    const int pi = static_cast<int>(sel[i] & 0xFFFFFFFFull);
    const float* l = loc + ((static_cast<size_t>(image) * p.num_priors + pi) * loc_classes + loc_cls) * 4;
    boxes[i] = decode_box(p, prior + static_cast<size_t>(pi) * 4, var + static_cast<size_t>(pi) * 4, l);
  }
  __syncthreads();

  // Greedy NMS: candidate i is kept iff its overlap with every box kept so far
  // is <= the threshold.  With a fixed threshold (eta == 1, the usual case) the
  // overlaps do not depend on the walk: the whole block evaluates the lower
  // triangle into a bit matrix (row i, bit j < i: box j would suppress box i),
  // which takes the place of the candidate keys in shared memory, and one warp
  // then walks the rows holding the kept set as one 32-bit word per lane.
  const int words = (count + 31) >> 5;
  const bool fixed_threshold = !(eta < 1.f);
  const bool use_matrix = fixed_threshold && words <= 32 &&
                          static_cast<size_t>(count) * words * sizeof(uint32_t) <= static_cast<size_t>(p.num_priors) * 8;
  if (use_matrix) {
    uint32_t* suppress = reinterpret_cast<uint32_t*>(cand);
    const float threshold_fixed = p.nms_threshold;
    // Consecutive threads take consecutive rows of one word column: the boxes
    // compared against are a broadcast, the row's own box a stride-5 access.
    for (int t = threadIdx.x; t < count * words; t += blockDim.x) {
      const int w = t / count;
      const int i = t - w * count;
      const int j0 = w << 5;
      uint32_t bits = 0;
      if (j0 < i) {
        const Box cur = boxes[i];
        const int jn = min(32, i - j0);
        for (int b = 0; b < jn; ++b) {
          if (jaccard(cur, boxes[j0 + b]) > threshold_fixed) bits |= 1u << b;
        }
      }
      suppress[i * words + w] = bits;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
      const int lane = threadIdx.x;
      uint32_t kept_word = 0;   // lane w: boxes 32 w .. 32 w + 31 kept so far
      int nk = 0;
      for (int i = 0; i < count; ++i) {
        const uint32_t hit = lane < words ? (suppress[i * words + lane] & kept_word) : 0u;
        if (!__any_sync(0xffffffffu, hit != 0u)) {
          if (lane == (i >> 5)) kept_word |= 1u << (i & 31);
          if (lane == 0) kept[nk] = i;
          ++nk;
        }
      }
      if (lane == 0) num_kept = nk;
    }
  } else if (threadIdx.x < 32) {
    // Adaptive threshold (eta < 1) or a very long candidate list: one warp
    // compares each candidate with the kept list, 32 kept boxes at a time.
    const int lane = threadIdx.x;
    float adaptive = p.nms_threshold;
    int nk = 0;
    for (int i = 0; i < count; ++i) {
      const Box cur = boxes[i];
      bool reject = false;
      for (int base = 0; base < nk && !reject; base += 32) {
        const int j = base + lane;
        const bool hit = j < nk && jaccard(cur, boxes[kept[j]]) > adaptive;
        reject = __any_sync(0xffffffffu, hit);
      }
      if (!reject) {
        if (lane == 0) kept[nk] = i;
        ++nk;
        __syncwarp();
        if (eta < 1.f && adaptive > 0.5f) adaptive = fmul(adaptive, eta);
      }
    }
    if (lane == 0) num_kept = nk;
  }
  __syncthreads();
  const int nk = num_kept;
  Entry* out = ws.entries + (static_cast<size_t>(image) * p.num_classes + cls) * limit;
  for (int r = threadIdx.x; r < nk; r += blockDim.x) {
    const int i = kept[r];
    const int pi = static_cast<int>(sel[i] & 0xFFFFFFFFull);
    Entry e;
    e.score = scores[static_cast<size_t>(pi) * p.num_classes];
    e.xmin = boxes[i].xmin;
    e.ymin = boxes[i].ymin;
    e.xmax = boxes[i].xmax;
    e.ymax = boxes[i].ymax;
    out[r] = e;
  }
  if (threadIdx.x == 0) *out_count = nk;
}

// ---------------------------------------------------------------- B. per image

// `staged`: the keys of all of the image's detections fit into dynamic shared
// memory and are gathered there once (all of a thread's loads in flight
// together); the passes of the radix select then read shared memory.
__global__ void __launch_bounds__(256)
detout_image_kernel(mcb200_detout_params p, Workspace ws, int staged) {
  extern __shared__ unsigned long long image_keys[];
  __shared__ int hist[256];
  __shared__ unsigned long long bcast[2];
  __shared__ int offsets[1025];   // first row of each class among the image's rows
  __shared__ int selected[1024];  // rows kept per class
  const int image = blockIdx.x;
  const int classes = p.num_classes;
  const int limit = ws.per_class;
  const int* counts = ws.class_count + static_cast<size_t>(image) * classes;
  const Entry* entries = ws.entries + static_cast<size_t>(image) * classes * limit;

  if (threadIdx.x == 0) {
    int total = 0;
    for (int c = 0; c < classes; ++c) {
      offsets[c] = total;
      total += counts[c];
    }
    offsets[classes] = total;
  }
  __syncthreads();
  const int total = offsets[classes];
  // Flat index e over (class, rank); key = (descending score, class * limit + rank).
  auto load_key = [&](int e) {
    int c = 0;
    while (offsets[c + 1] <= e) ++c;
    const int j = e - offsets[c];
    return make_key(entries[static_cast<size_t>(c) * limit + j].score, static_cast<uint32_t>(c * limit + j));
  };
  const bool select = p.keep_top_k > -1 && total > p.keep_top_k;
  if (staged && select) {
    for (int e = threadIdx.x; e < total; e += blockDim.x) image_keys[e] = load_key(e);
    __syncthreads();
  }
  auto fetch = [&](int e) { return staged ? image_keys[e] : load_key(e); };
  unsigned long long threshold = kPadKey;
  if (select) threshold = block_kth_smallest(fetch, total, p.keep_top_k, hist, bcast);
  // Within a class the entries are in descending score order, so the kept ones
  // are a prefix of it; its length is the number of the class's keys <= threshold.
  for (int c = threadIdx.x; c < classes; c += blockDim.x) selected[c] = 0;
  __syncthreads();
  for (int e = threadIdx.x; e < total; e += blockDim.x) {
    int c = 0;
    while (offsets[c + 1] <= e) ++c;
    // Without a selection every detection is kept (the threshold is the largest key).
    if (!select || fetch(e) <= threshold) atomicAdd(&selected[c], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int c = 0; c < classes; ++c) {
      offsets[c] = run;
      run += selected[c];
    }
    offsets[classes] = run;
    ws.image_count[image] = run;
  }
  __syncthreads();
  float* rows = ws.rows + static_cast<size_t>(image) * ws.max_rows * 7;
  for (int c = 0; c < classes; ++c) {
    for (int j = threadIdx.x; j < selected[c]; j += blockDim.x) {
      const Entry e = entries[static_cast<size_t>(c) * limit + j];
      float* r = rows + static_cast<size_t>(offsets[c] + j) * 7;
      r[0] = static_cast<float>(image);
      r[1] = static_cast<float>(c);
      r[2] = e.score;
      r[3] = e.xmin;
      r[4] = e.ymin;
      r[5] = e.xmax;
      r[6] = e.ymax;
    }
  }
}

// ---------------------------------------------------------------- C. compaction

// One block per image: the block sums the counts of the images before its own
// (and of all images, for the total) and copies its rows behind them.
__global__ void __launch_bounds__(256)
detout_compact_kernel(Workspace ws, int batch, float* __restrict__ out, int* __restrict__ total_out) {
  __shared__ int sums[2];
  const int image = blockIdx.x;
  if (threadIdx.x == 0) sums[0] = sums[1] = 0;
  __syncthreads();
  int before = 0, all = 0;
  for (int i = threadIdx.x; i < batch; i += blockDim.x) {
    const int n = ws.image_count[i];
    all += n;
    if (i < image) before += n;
  }
  if (before) atomicAdd(&sums[0], before);
  if (all) atomicAdd(&sums[1], all);
  __syncthreads();
  const int first = sums[0], total = sums[1];
  const int n = ws.image_count[image];
  const float* rows = ws.rows + static_cast<size_t>(image) * ws.max_rows * 7;
  for (int i = threadIdx.x; i < n * 7; i += blockDim.x) out[static_cast<size_t>(first) * 7 + i] = rows[i];
  if (image == 0) {
    if (total == 0) {
      // No detection at all: one row per image, image id followed by -1.
      for (int i = threadIdx.x; i < batch * 7; i += blockDim.x) out[i] = (i % 7 == 0) ? static_cast<float>(i / 7) : -1.f;
    }
    if (threadIdx.x == 0) *total_out = total;
  }
}

int validate(const mcb200_detout_params* p, int batch) {
  if (!p || batch < 1) return -1;
  if (p->num_priors < 1 || p->num_classes < 1 || p->num_classes > 1024 || p->code_type < 1 || p->code_type > 3)
    return -2;
  if (batch > 65535) return -3;
  if (!(p->eta > 0.f) || p->eta > 1.f) return -8;
  const int limit = per_class_limit(*p);
  if (det::next_pow2(limit) > 4096) return -4;
  return 0;
}

size_t class_kernel_smem(const mcb200_detout_params& p, int padded) {
  return static_cast<size_t>(p.num_priors) * 8 + static_cast<size_t>(padded) * (8 + sizeof(Box) + sizeof(int));
}

}  // namespace
}  // namespace mcb200

using namespace mcb200;

extern "C" size_t mcb200_detout_workspace_bytes(const mcb200_detout_params* p, int batch) {
  if (validate(p, batch) != 0) return 0;
  return carve(*p, batch, nullptr, nullptr);
}

extern "C" int mcb200_detout_max_rows_per_image(const mcb200_detout_params* p) {
  if (validate(p, 1) != 0) return -1;
  const int rows = max_rows(*p);
  return rows > 1 ? rows : 1;
}

extern "C" int mcb200_detout_forward(const mcb200_detout_params* p, int batch, const float* loc, const float* conf,
                                     const float* prior, void* workspace, float* out, int* total, void* stream) {
  const int rc = validate(p, batch);
  if (rc != 0) return rc;
  if (!loc || !conf || !prior || !workspace || !out || !total) return -5;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return -6;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Workspace ws;
  carve(*p, batch, static_cast<char*>(workspace), &ws);
  const int padded = det::next_pow2(ws.per_class);
  const size_t smem = class_kernel_smem(*p, padded);
  if (smem > 200 * 1024) return -7;
  {
    static size_t configured[64] = {0};
    static std::mutex configure_mu;   // nets on several host threads may make their first call together
    std::lock_guard<std::mutex> lock(configure_mu);
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && configured[dev] < smem) {
      cudaError_t e = cudaFuncSetAttribute(detout_class_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem));
      if (e != cudaSuccess) return static_cast<int>(e);
      configured[dev] = smem;
    }
  }
  detout_class_kernel<<<dim3(p->num_classes, batch), 256, smem, st>>>(loc, conf, prior, *p, ws, padded, p->eta);
  count_launch();
  {
    // Keys of one image: at most (classes x per-class limit) of 8 bytes.
    const size_t key_bytes = static_cast<size_t>(p->num_classes) * ws.per_class * 8;
    const size_t kImageSharedLimit = 200 * 1024;
    const int staged = key_bytes <= kImageSharedLimit ? 1 : 0;
    static size_t configured_image[64] = {0};
    static std::mutex configure_mu;
    std::lock_guard<std::mutex> lock(configure_mu);
    int dev = 0;
    cudaGetDevice(&dev);
    if (staged && dev >= 0 && dev < 64 && configured_image[dev] < key_bytes) {
      cudaError_t e = cudaFuncSetAttribute(detout_image_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(kImageSharedLimit));
      if (e != cudaSuccess) return static_cast<int>(e);
      configured_image[dev] = kImageSharedLimit;
    }
    detout_image_kernel<<<batch, 256, staged ? key_bytes : 0, st>>>(*p, ws, staged);
  }
  count_launch();
  detout_compact_kernel<<<batch, 256, 0, st>>>(ws, batch, out, total);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}
