// Convolution / InnerProduct as an implicit GEMM on the Blackwell tensor cores.
//
//   D[m, co] = sum over taps (r, s) and channels c of  X[pixel(m) + (r, s), c] * W[co, r, s, c]
//
// m runs over the N*Ho*Wo output pixels of a channels-last activation tensor.
// One CTA computes 128 x BN tiles of D, one after the other (persistent):
//   warp 0   one elected thread issues the activation loads.  The tile (128
//            pixels x 32 channels of one filter tap) comes through an
//            im2col-mode tensor map, so the hardware walks the output pixels
//            across image rows and images and zero-fills the padding.
//   warp 2   one elected thread issues the weight loads (BN x 32, tiled map).
//            Both operands land in shared memory 128-byte swizzled, K-major.
//            Two issuing threads because a single thread's loop (wait, arm the
//            barrier, issue) costs a few hundred cycles per k-iteration, which
//            is as long as the copy itself takes.
//   warp 1   one thread issues tcgen05.mma kind::tf32 (M=128, N=BN, K=8), four per
//            stage, accumulating in tensor memory; tcgen05.commit hands each
//            shared-memory stage back to the producers.
//   warps 3-10 read the accumulator out of tensor memory (tcgen05.ld), apply
//            the fused tail (per-channel scale/shift, residual add, ReLU or
//            PReLU) and store channels-last.  Two warps share each 32-lane
//            quadrant of tensor memory and take alternate 32-column chunks.
//            Each warp stages its 32 x 32 sub-tiles in shared memory (128-byte
//            swizzled) so that the residual comes in and the result goes out as
//            whole 128-byte rows through TMA tile loads / stores, double
//            buffered per warp.
// Every barrier wait is bounded; a timed-out wait raises an abort flag, the
// roles drain, tensor memory is freed and *status is set.
//
// Arithmetic replaced: mini-caffe's per-image im2col + SGEMM + bias GEMM
// (src/layers/base_conv_layer.cpp:254-278, src/util/im2col.cpp:19-55).
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <stdlib.h>

#include <mutex>

#include "../../../include/mcb200_kernels.h"
#include "kernel_timer.h"
#include "launch_count.h"
#include "sm100.cuh"

namespace mcb200 {
namespace {

using namespace sm100;

constexpr int kBlockM = 128;
constexpr int kBlockK = 32;                            // fp32 elements = one 128-byte swizzle row
constexpr int kBlockKHalf = 64;                        // bfloat16 elements of the same 128 bytes
constexpr int kMmaPerBlock = 4;                        // 32-byte K steps of a swizzle row (K = 8 tf32 / 16 bf16)
constexpr int kTileABytes = kBlockM * kBlockK * 4;     // 16 KiB
// Warp roles.  A warp may only read the tensor-memory lanes [32 * (warp % 4), +32),
// so the eight epilogue warps form four pairs that share a lane quadrant and split
// the 32-column chunks of a tile between them (even / odd).
constexpr int kWarpLoadA = 0;
constexpr int kWarpMma = 1;
constexpr int kWarpLoadB = 2;
constexpr int kFirstEpilogueWarp = 3;
constexpr int kEpilogueWarps = 8;
constexpr int kThreads = (kFirstEpilogueWarp + kEpilogueWarps) * 32;   // 352
constexpr long long kDefaultWaitLimitCycles = 2000000000LL;   // about one second
// How the activation tile of a k-iteration is fetched.
constexpr int kModeMatrix = 0;   // rows of a plain [m, c] matrix (1x1 convolution, inner product)
constexpr int kModeIm2col = 1;   // im2col-mode tensor map: any filter, channels % 4 == 0
constexpr int kModeRows = 2;     // <= 4 channels: one filter row of 8 pixels x 4 channels per k-iteration
constexpr int kModeHalo = 3;     // stride-1 filters wider than one tap: the taps of a filter row share one pixel strip
constexpr int kMaxHaloRows = 16; // extra strip rows ((kw - 1) * dilation) the halo mode takes

struct ConvTcArgs {
  float* out;
  int out_ld;
  int m;             // output pixels
  int cout;
  int k_iters;       // taps * c_blocks
  int c_blocks;      // ceil(c / 32)
  int kw;            // filter width (tap -> (r, s))
  int ho, wo;
  int stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
  mcb200_epilogue ep;
  int* status;
  int tma_epilogue;  // output (and residual) meet the 16-byte rules of TMA tiles
  int tile_rows;     // rows of an M tile: 128, or in row mode min(output width, 128)
  int row_segments;  // row mode: M tiles per output row of an image (ceil(output width / tile_rows))
  int a_bytes;       // bytes one activation tile load delivers
  int stages;        // depth of the operand ring (2 .. kMaxStages)
  int slots;         // staging slots per epilogue warp: 1 or 2; 2 .. kMaxSlots when a residual is added
  int res_depth;     // residual sub-tiles a warp requests ahead of the one it works on (1 .. slots - 1)
  int out_half;      // the output is stored as bfloat16 (else fp32), whatever the operands are
  // Halo mode.  The M index runs over a virtual output grid whose rows are `wp` = wo + (kw - 1) *
  // dil_w positions wide (the last wp - wo positions of a row are computed and never stored), so
  // that the taps s = 0 .. kw-1 of a filter row are the same strip of `128 + wp - wo` input
  // pixels read at row offsets s * dil_w.  `m` then counts virtual positions.
  int wp;
  int stage_bytes;     // strip slot + kw weight tiles
  int stage_b_offset;  // where the weight tiles start inside a stage
  int vec_store;       // plain-store epilogue: rows are 16-byte aligned, use 128-bit accesses
  // Grouped convolution (group_cout > 0): output columns [g * group_cout, (g + 1) * group_cout)
  // read input channels [g * group_cin, (g + 1) * group_cin).  An N tile multiplies the channels
  // its groups span (from `c_origin`, rounded down to 16 bytes) by a block-diagonal weight tile:
  // the packed weights hold zeros where an output column's group does not own the channel.
  int group_cout, group_cin;
  int l2_prefetch;               // ask L2 for the next tile's activations a tile ahead
  int halo_staged;               // halo mode: results pass through a shared-memory slot so that the stores are
                                 // whole 128-byte rows (fp32 output with 16-byte aligned rows)
  long long wait_limit;          // bound of every barrier wait, in SM cycles
  int resident_b_bytes;          // row mode: all filter rows' weight tiles stay in shared memory (bytes; 0 = streamed
                                 // with the activations).  Every M tile of such a layer multiplies the same
                                 // weights, and a third of what its ring pulled out of L2 was this one image.
  int drop_last_weight_load;     // test hook: the weight producer leaves out its last k-iteration (see
                                 // mcb200_conv_test_drop_weight_load): the waits on that stage run out
};

// Optional cycle-counter trace (build with -DMCB200_CONV_TRACE): the single-thread roles and the
// first epilogue warp of CTA 0 stamp clock64() at fixed points of their loops into a device
// array that mcb200_conv_trace_read copies out.  Role 0: activation producer (per k-iteration:
// stage free, loads issued); 1: weight producer (same); 2: MMA issuer (per k-iteration: stage
// full, MMAs issued and committed); 3: epilogue warp 0 (per tile: accumulator ready, tile stored);
// 4: the same warp inside its chunk loop, five stamps per 32 x 32 chunk of a launch with the staged
// epilogue (chunk begins, accumulator in registers, slot free / residual there, tail computed and
// written to the slot, store issued).
#ifdef MCB200_CONV_TRACE
constexpr int kTraceSlots = 2048;
constexpr int kTraceRoles = 5;
__device__ long long g_conv_trace[kTraceRoles * kTraceSlots];
#define MCB200_TRACE_DECL int trace_n = 0
#define MCB200_TRACE(role)                                                                         \
  do {                                                                                             \
    if (blockIdx.x == 0 && trace_n < kTraceSlots) g_conv_trace[(role) * kTraceSlots + trace_n++] = clock64(); \
  } while (0)
#define MCB200_TRACE_CHUNK_DECL int trace_c = 0
#define MCB200_TRACE_CHUNK()                                                                       \
  do {                                                                                             \
    if (blockIdx.x == 0 && ew == 0 && lane == 0 && trace_c < kTraceSlots)                          \
      g_conv_trace[4 * kTraceSlots + trace_c++] = clock64();                                       \
  } while (0)
#else
#define MCB200_TRACE_DECL
#define MCB200_TRACE(role)
#define MCB200_TRACE_CHUNK_DECL
#define MCB200_TRACE_CHUNK()
#endif

constexpr int kMaxStages = 8;
constexpr int kMaxSlots = 4;     // every barrier here is static shared memory that the operand ring cannot use
constexpr int kSharedLimit = 232448;   // 227 KiB: the most one CTA can have on sm_100

// Shared memory of one persistent CTA = operand ring (`stages` x (A tile + B
// tile)) + epilogue staging (`slots` x 4 KiB for each of the eight warps; 2 KiB
// when residual and result are both bfloat16).  The
// copies in flight are what hides the round trip of a stage (L2 -> shared
// memory, barrier hop, MMA completion, barrier hop: about a microsecond), so
// the ring takes every byte the epilogue can spare: launches that add a
// residual, or whose tiles are short (few k-iterations per epilogue), double
// buffer the staging; all others give that memory to the ring.
template <int BN, int kMode, bool kPair>
struct SmemPlan {
  static constexpr int kTileBRows = kPair ? BN / 2 : BN;   // a CTA of a pair holds half of the weight tile
  static constexpr int kTileBBytes = kTileBRows * kBlockK * 4;
  // K = 32 sub-tiles per stage.  Every stage costs each single-thread role a
  // barrier wait and a signal (a few hundred cycles of pure latency), so where
  // a K = 32 step is short (narrow tiles) a stage carries two of them.
  // (Row mode keeps single steps: two filter rows per stage were measured and change nothing, its
  // tiles are bound by their epilogue.  64-column tiles as CTA pairs were measured too: slower.)
  // Halo mode: a stage is one pixel strip plus the weight tiles of a whole filter row (sized at run time).
  static constexpr int kSub =
      (kMode != kModeRows && kMode != kModeHalo && kTileABytes + kTileBBytes <= 24 * 1024) ? 2 : 1;
  static constexpr int kStageBytes = kSub * (kTileABytes + kTileBBytes);
  static constexpr int kStageBOffset = kSub * kTileABytes;   // [A sub-tiles][B sub-tiles]
  static constexpr int staging_bytes(int slots, int slot_bytes) { return kEpilogueWarps * slots * slot_bytes; }
  static constexpr int dynamic_bytes(int stages, int slots, int slot_bytes) {
    return stages * kStageBytes + staging_bytes(slots, slot_bytes) + 1024;   // + alignment slack
  }
};

// Compile-time tag for the activation of the fused tail (0 none, 1 ReLU, 2 per-column negative slope).
template <int kAct>
struct ActTag {
  static constexpr int value = kAct;
};

// Ring position of a k-iteration: stage index and the parity of its use.
// Advancing it costs an increment and a compare; the single-thread loops
// below are latency-bound on exactly this kind of scalar work.
struct RingPos {
  int stage = 0;
  uint32_t parity = 0;
  __device__ __forceinline__ void advance(int stages) {
    if (++stage == stages) {
      stage = 0;
      parity ^= 1u;
    }
  }
};

// Persistent kernel: CTA b works on tiles b, b + gridDim.x, ... (n fastest, so
// the CTAs running at one time share activation tiles through L2).  Two
// accumulators in tensor memory let the tensor core start the next tile while
// the epilogue warps drain the previous one; the TMA producers run ahead across
// tile boundaries.
//
// kPair: the CTAs of a cluster of two share one tcgen05.mma.cta_group::2 per
// K=8 step.  The pair works on 256 output pixels (128 per CTA) x BN channels;
// each CTA fetches its own activation tile and only half of the weight tile, the
// rank-0 CTA issues the MMAs for both, and each CTA drains its own half of the
// result from its own tensor memory.  Weight bytes per MAC halve, which is what
// bounds the layers whose operands come out of L2 faster than the ring can
// turn over.  Barriers that both CTAs signal (stage full, accumulator drained)
// live in rank 0; tcgen05.commit delivers the arrivals that both CTAs wait on to
// each CTA's own copy of the barrier.
//
// kHalf: activations, weights and the residual are bfloat16 (tcgen05.mma
// kind::f16, fp32 accumulation); a k-iteration then covers 64 channels in the
// same 128-byte rows.  Independently of that, the output is stored as fp32 or
// as bfloat16 (args.out_half).
template <int BN, int kMode, bool kPair, bool kHalf>
__global__ void __launch_bounds__(kThreads, 1)
conv_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_out, const __grid_constant__ CUtensorMap map_res,
               const ConvTcArgs args) {
  static_assert(!(kPair && kMode == kModeRows), "row mode runs unpaired");
  static_assert(!(kHalf && kMode == kModeRows), "row mode takes fp32 images");
  using Plan = SmemPlan<BN, kMode, kPair>;
  constexpr int kElemsK = kHalf ? kBlockKHalf : kBlockK;   // channels per k-iteration
  const int stages = args.stages;
  const int slots = args.slots;
  const long long wait_limit = args.wait_limit;   // SM cycles a barrier wait may take before the CTA gives up

  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t full_bar[kMaxStages];    // both operand tiles of a stage have landed (two producers)
  __shared__ uint64_t empty_bar[kMaxStages];   // the MMAs reading a stage have retired
  __shared__ uint64_t tmem_full_bar[2];
  __shared__ uint64_t tmem_empty_bar[2];
  __shared__ uint64_t res_bar[kEpilogueWarps][kMaxSlots];   // per epilogue warp, per staging slot
  __shared__ uint64_t col_bar[2];              // per-column table of a tile is complete
  __shared__ uint64_t wres_bar;                // row mode: the resident weight tiles have landed
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ __align__(16) float col_scale[2][BN];   // per-column constants of the current tiles
  __shared__ __align__(16) float col_shift[2][BN];
  __shared__ __align__(16) float col_slope[2][BN];

  // 128-byte swizzled tiles must start on a 1024-byte boundary.
  const uint32_t raw_addr = smem_addr(smem_raw);
  uint8_t* tiles = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  const int stage_bytes = (kMode == kModeHalo || kMode == kModeRows) ? args.stage_bytes : Plan::kStageBytes;
  const int stage_b_offset = (kMode == kModeHalo || kMode == kModeRows) ? args.stage_b_offset : Plan::kStageBOffset;
  const bool resident_b = kMode == kModeRows && args.resident_b_bytes > 0;
  uint8_t* resident = tiles + stages * stage_bytes;   // stages are multiples of 1024 bytes: so is this address
  uint8_t* staging_base = resident + (kMode == kModeRows ? args.resident_b_bytes : 0);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_tiles = (args.cout + BN - 1) / BN;
  // Row mode: an M tile is (a segment of at most 128 pixels of) one output row of one image.
  const int m_tiles = kMode == kModeRows ? (args.m / args.wo) * args.row_segments : (args.m + kBlockM - 1) / kBlockM;
  // Row mode helpers: image row (n * ho + p) and first pixel of the segment of M tile mt.
  auto row_of = [&](int mt) { return mt / args.row_segments; };
  auto seg_start = [&](int mt) { return (mt % args.row_segments) * args.tile_rows; };
  // A work unit is an M tile (or a pair of neighbouring M tiles) x an N tile;
  // `worker` is the CTA (or pair) index among `workers`.
  const uint32_t rank = kPair ? cluster_cta_rank() : 0u;
  const int worker = kPair ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int workers = kPair ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  const int m_units = kPair ? (m_tiles + 1) >> 1 : m_tiles;
  const int num_tiles = n_tiles * m_units;
  auto unit_to_mt = [&](int unit) { return kPair ? 2 * unit + static_cast<int>(rank) : unit; };

  // Some fifty barriers: a thread each (one thread doing them all costs every launch most of a
  // microsecond before its first load can go out).
  {
    const int t = static_cast<int>(threadIdx.x);
    if (t == 0) abort_flag = 0;
    if (t < stages) {
      mbar_init(&full_bar[t], resident_b ? 1 : 2);     // one arrival per producer thread that fills the stage
      mbar_init(&empty_bar[t], 1);
      fence_barrier_init();
    } else if (t >= 32 && t < 34) {
      const int b = t - 32;
      mbar_init(&tmem_full_bar[b], 1);
      mbar_init(&tmem_empty_bar[b], kPair ? 2 * kEpilogueWarps : kEpilogueWarps);   // one arrival per epilogue warp
      mbar_init(&col_bar[b], kEpilogueWarps);
      fence_barrier_init();
    } else if (t >= 64 && t < 64 + kEpilogueWarps * kMaxSlots) {
      mbar_init(&res_bar[(t - 64) / kMaxSlots][(t - 64) % kMaxSlots], 1);
      fence_barrier_init();
    } else if (t == 34) {
      tma_prefetch_descriptor(&map_a);
      tma_prefetch_descriptor(&map_b);
    } else if (t == 35) {
      mbar_init(&wres_bar, 1);
      fence_barrier_init();
    }
  }
  if (warp == kWarpMma) {
    tmem_alloc(&tmem_base_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  if (kPair) {
    cluster_sync_all();   // the peer's barriers are initialised before anything signals them
  } else {
    __syncthreads();
  }
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_slot;
  volatile int* abort = &abort_flag;
  // A paired MMA writes the same tensor-memory address in both CTAs.  Each CTA
  // makes the first and only allocation of its SM, which starts at column 0;
  // anything else is refused rather than computed wrongly.
  // Up to here the CTA has only set itself up, which may overlap the tail of
  // the previous launch of the stream; from here on it touches tensors.
  grid_launch_dependents();
  grid_dependency_wait();
  const bool usable = !kPair || tmem_base == 0u;
  if (!usable && threadIdx.x == 0) abort_flag = 1;
  // Cluster-window addresses of rank 0's shared barriers.
  const uint32_t full_bar_leader = kPair ? cluster_map(smem_addr(&full_bar[0]), 0u) : 0u;
  const uint32_t tmem_empty_leader = kPair ? cluster_map(smem_addr(&tmem_empty_bar[0]), 0u) : 0u;

  // After an abort: give a producer's copies that are still in flight a bounded
  // time to land before the CTA's shared memory is released.
  auto drain_loads = [&](int issued) {
    if (!*abort) return;
    const int first = issued > stages ? issued - stages : 0;
    for (int j = first; j < issued; ++j) {
      const long long start = clock64();
      while (!mbar_try_wait(&full_bar[j % stages], static_cast<uint32_t>(j / stages) & 1u)) {
        if (clock64() - start > wait_limit / 8) break;
      }
    }
  };

  if (!usable) {
    // fall through to the teardown; the peer's waits run out and it follows
  } else if (warp == kWarpLoadA) {
    // ------------------------------------------------------------ activation tiles
    if (elect_one()) {
      RingPos pos;
      int issued = 0;
      bool alive = true;
      MCB200_TRACE_DECL;
      const uint32_t a_bytes = static_cast<uint32_t>(args.a_bytes);
      for (int tile = worker; tile < num_tiles && alive; tile += workers) {
        const int mt = unit_to_mt(tile / n_tiles);
        const int m0 = mt * kBlockM;
        // The odd M tile out at the end of a paired launch has no pixels: its
        // CTA loads nothing, and the MMA computes rows nobody stores.
        const bool live = !kPair || mt < m_tiles;
        // Only rank 0's barrier counts bytes: its producers announce what both
        // CTAs are about to fetch, the peer's copies just report completion
        // there (a remote arrival per k-iteration would cost the peer's
        // producer a cluster-scope release, about a microsecond each).
        const uint32_t announce =
            !kPair ? a_bytes : (rank != 0u ? 0u : (mt + 1 < m_tiles ? 2u * a_bytes : a_bytes));
        int base_w = 0, base_h = 0, base_n = 0;
        if (kMode == kModeRows) {
          const int row = row_of(mt);
          base_n = row / args.ho;
          base_h = (row - base_n * args.ho) * args.stride_h;   // row in the spatially padded copy
          base_w = seg_start(mt);                              // first output pixel of the segment
        }
        if (kMode == kModeIm2col) {
          const int q = m0 % args.wo;
          const int p = (m0 / args.wo) % args.ho;
          base_n = m0 / (args.wo * args.ho);
          base_w = q * args.stride_w - args.pad_w;
          base_h = p * args.stride_h - args.pad_h;
        }
        if (kMode == kModeHalo) {
          // m0 is a position of the virtual output grid (rows of wp positions, stride 1)
          const int t = m0 / args.wp;
          base_n = t / args.ho;
          base_w = m0 - t * args.wp - args.pad_w;
          base_h = t - base_n * args.ho - args.pad_h;
        }
        // First channel the tile's weight columns refer to (grouped layers: the first channel of
        // the first group the N tile touches, rounded down to a 16-byte boundary of the pixel).
        int c_origin = 0;
        if (args.group_cout > 0) {
          const int n0 = (tile % n_tiles) * BN;
          c_origin = ((n0 / args.group_cout) * args.group_cin) & ~((kHalf ? 8 : 4) - 1);
        }
        // The activations of this CTA's next tile are asked for now, a tile ahead (L2 prefetch, no
        // shared memory, nothing to wait for).  A tile always brings pixels nobody has read yet,
        // the ring looks only a few stages ahead, and a load that waits for DRAM holds up the whole
        // in-order ring behind it.  Of the CTAs that share an M tile (one per N tile) the one
        // with N tile 0 asks; grouped layers read other channels per N tile, so there every CTA asks.
        if (args.l2_prefetch && kMode != kModeRows) {
          const int next = tile + workers;
          const int n_index = next % n_tiles;
          const int mt2 = next < num_tiles ? unit_to_mt(next / n_tiles) : m_tiles;
          if (mt2 < m_tiles && (n_index == 0 || args.group_cout > 0)) {
            const int origin2 = args.group_cout > 0
                                    ? (((n_index * BN) / args.group_cout) * args.group_cin) & ~((kHalf ? 8 : 4) - 1)
                                    : 0;
            const int v2 = mt2 * kBlockM;
            if (kMode == kModeMatrix) {
              for (int cb = 0; cb < args.c_blocks; ++cb) tma_prefetch_2d(&map_a, origin2 + cb * kElemsK, v2);
            } else {
              int w2, h2, n2;
              if (kMode == kModeHalo) {
                const int t2 = v2 / args.wp;
                n2 = t2 / args.ho;
                w2 = v2 - t2 * args.wp - args.pad_w;
                h2 = t2 - n2 * args.ho - args.pad_h;
              } else {
                n2 = v2 / (args.wo * args.ho);
                w2 = (v2 % args.wo) * args.stride_w - args.pad_w;
                h2 = ((v2 / args.wo) % args.ho) * args.stride_h - args.pad_h;
              }
              const int kh = kMode == kModeHalo ? args.k_iters / args.c_blocks : args.k_iters / (args.c_blocks * args.kw);
              // im2col mode: the middle tap column of every filter row touches (nearly) every pixel
              // the other columns touch; with a stride, its neighbour column takes the pixels between.
              const int s_mid = kMode == kModeHalo ? 0 : args.kw / 2;
              const int s_count = (kMode == kModeIm2col && args.stride_w > 1 && args.kw > 1) ? 2 : 1;
              for (int r = 0; r < kh; ++r)
                for (int sc = 0; sc < s_count; ++sc)
                  for (int cb = 0; cb < args.c_blocks; ++cb)
                    tma_prefetch_im2col_4d(&map_a, origin2 + cb * kElemsK, w2, h2, n2,
                                           static_cast<uint16_t>(min(s_mid + sc, args.kw - 1) * args.dil_w),
                                           static_cast<uint16_t>(r * args.dil_h));
            }
          }
        }
        // Position inside the filter, advanced incrementally: channel block,
        // then tap column, then tap row.
        int c0 = 0, sx = 0;
        uint16_t off_w = 0, off_h = 0;
        int row_h = base_h;
        for (int k = 0; k < args.k_iters; k += Plan::kSub) {
          if (!mbar_wait_bounded(&empty_bar[pos.stage], pos.parity ^ 1u, abort, wait_limit)) {
            alive = false;
            break;
          }
          MCB200_TRACE(0);
          const int nsub = args.k_iters - k < Plan::kSub ? args.k_iters - k : Plan::kSub;
          uint8_t* a_dst = tiles + pos.stage * stage_bytes;
          uint64_t* bar = &full_bar[pos.stage];
          const uint32_t bar_leader = full_bar_leader + static_cast<uint32_t>(pos.stage) * 8u;
          if (rank == 0u) mbar_expect_tx(bar, announce * static_cast<uint32_t>(nsub));
#pragma unroll
          for (int j = 0; j < Plan::kSub; ++j) {
            if (j >= nsub) break;
            if (kMode == kModeRows) {
              // A sub-tile is one filter row: tile_rows pixels x (8 pixels x 4 channels) of a padded input row.
              tma_load_4d(&map_a, bar, a_dst, 0, base_w, row_h, base_n);   // pixels past the row read as zero
              row_h += args.dil_h;
            } else if (kMode == kModeHalo) {
              // One strip of 128 + halo pixels x one channel block, at filter row off_h: every tap
              // of that row reads it (k-iterations run over filter rows x channel blocks).
              if (kPair) {
                if (live) tma_load_im2col_4d_pair(&map_a, bar_leader, a_dst, c_origin + c0, base_w, base_h, base_n, 0, off_h);
              } else {
                tma_load_im2col_4d(&map_a, bar, a_dst, c_origin + c0, base_w, base_h, base_n, 0, off_h);
              }
              c0 += kElemsK;
              if (c0 >= args.c_blocks * kElemsK) {
                c0 = 0;
                off_h = static_cast<uint16_t>(off_h + args.dil_h);
              }
            } else if (kMode == kModeIm2col) {
              if (kPair) {
                if (live) tma_load_im2col_4d_pair(&map_a, bar_leader, a_dst, c_origin + c0, base_w, base_h, base_n, off_w, off_h);
              } else {
                tma_load_im2col_4d(&map_a, bar, a_dst, c_origin + c0, base_w, base_h, base_n, off_w, off_h);
              }
              c0 += kElemsK;
              if (c0 >= args.c_blocks * kElemsK) {
                c0 = 0;
                off_w = static_cast<uint16_t>(off_w + args.dil_w);
                if (++sx == args.kw) {
                  sx = 0;
                  off_w = 0;
                  off_h = static_cast<uint16_t>(off_h + args.dil_h);
                }
              }
            } else {
              if (kPair) {
                if (live) tma_load_2d_pair(&map_a, bar_leader, a_dst, c_origin + c0, m0);
              } else {
                tma_load_2d(&map_a, bar, a_dst, c_origin + c0, m0);
              }
              c0 += kElemsK;
            }
            a_dst += kTileABytes;
          }
          MCB200_TRACE(0);
          ++issued;
          pos.advance(stages);
        }
      }
      drain_loads(issued);
    }
  } else if (warp == kWarpLoadB) {
    // ------------------------------------------------------------ weight tiles
    if (elect_one()) {
      RingPos pos;
      int issued = 0;
      bool alive = true;
      MCB200_TRACE_DECL;
      if (resident_b) {
        // All filter rows at once, into their own region; the ring then carries activations only.
        const int loads = args.drop_last_weight_load ? args.k_iters - 1 : args.k_iters;
        mbar_expect_tx(&wres_bar, Plan::kTileBBytes * static_cast<uint32_t>(args.k_iters));
        for (int k = 0; k < loads; ++k) tma_load_2d(&map_b, &wres_bar, resident + k * Plan::kTileBBytes, k * kElemsK, 0);
        // The copies land before this CTA may release its shared memory (bounded, like every wait).
        const long long start = clock64();
        while (!mbar_try_wait(&wres_bar, 0u)) {
          if (clock64() - start > wait_limit) break;
        }
        alive = false;   // nothing to stream
      }
      for (int tile = worker; tile < num_tiles && alive; tile += workers) {
        // A CTA of a pair fetches the half of the weight tile that matches its rank.
        const int n0 = (tile % n_tiles) * BN + static_cast<int>(rank) * Plan::kTileBRows;
        int k0 = 0;
        int halo_cb = 0, halo_row_k0 = 0;   // halo mode: channel block and first packed-weight column of the filter row
        for (int k = 0; k < args.k_iters; k += Plan::kSub) {
          if (!mbar_wait_bounded(&empty_bar[pos.stage], pos.parity ^ 1u, abort, wait_limit)) {
            alive = false;
            break;
          }
          MCB200_TRACE(1);
          if (args.drop_last_weight_load && tile + workers >= num_tiles && k + Plan::kSub >= args.k_iters) {
            alive = false;   // nothing arrives on this stage's barrier: every role's wait on it is bounded
            break;
          }
          const int nsub = args.k_iters - k < Plan::kSub ? args.k_iters - k : Plan::kSub;
          uint8_t* b_dst = tiles + pos.stage * stage_bytes + stage_b_offset;
          uint64_t* bar = &full_bar[pos.stage];
          const uint32_t bar_leader = full_bar_leader + static_cast<uint32_t>(pos.stage) * 8u;
          if (kMode == kModeHalo) {
            // The weight tiles of the kw taps of this filter row for this channel block.  Packed
            // weight columns run [tap][channel block]; tap = row * kw + s.
            const int row_stride = args.c_blocks * kElemsK;
            if (rank == 0u) mbar_expect_tx(bar, (kPair ? 2u : 1u) * Plan::kTileBBytes * static_cast<uint32_t>(args.kw));
            int kcol = halo_row_k0 + halo_cb * kElemsK;
            for (int s = 0; s < args.kw; ++s) {
              if (kPair) {
                tma_load_2d_pair(&map_b, bar_leader, b_dst, kcol, n0);
              } else {
                tma_load_2d(&map_b, bar, b_dst, kcol, n0);
              }
              kcol += row_stride;
              b_dst += Plan::kTileBBytes;
            }
            if (++halo_cb == args.c_blocks) {
              halo_cb = 0;
              halo_row_k0 += args.kw * row_stride;
            }
            MCB200_TRACE(1);
            ++issued;
            pos.advance(stages);
            continue;
          }
          // Rank 0 announces both halves of a paired weight tile.
          if (rank == 0u) mbar_expect_tx(bar, (kPair ? 2u : 1u) * Plan::kTileBBytes * static_cast<uint32_t>(nsub));
#pragma unroll
          for (int j = 0; j < Plan::kSub; ++j) {
            if (j >= nsub) break;
            if (kPair) {
              tma_load_2d_pair(&map_b, bar_leader, b_dst, k0, n0);
            } else {
              tma_load_2d(&map_b, bar, b_dst, k0, n0);
            }
            k0 += kElemsK;
            b_dst += Plan::kTileBBytes;
          }
          MCB200_TRACE(1);
          ++issued;
          pos.advance(stages);
        }
      }
      drain_loads(issued);
    }
  } else if (warp == kWarpMma) {
    // ------------------------------------------------------------ MMA issuer
    if ((!kPair || rank == 0u) && elect_one()) {
      constexpr uint32_t idesc = kHalf ? umma_idesc_bf16(kPair ? 2 * kBlockM : kBlockM, BN)
                                       : umma_idesc_tf32(kPair ? 2 * kBlockM : kBlockM, BN);
      RingPos pos;
      int local = 0;   // tiles done by this CTA
      bool alive = true;
      MCB200_TRACE_DECL;
      const uint32_t tiles_addr = smem_addr(tiles);
      if (resident_b) {
        if (!mbar_wait_bounded(&wres_bar, 0u, abort, wait_limit)) alive = false;
        tc_fence_after_sync();
      }
      for (int tile = worker; tile < num_tiles && alive; tile += workers, ++local) {
        const int ab = local & 1;
        const uint32_t use = static_cast<uint32_t>(local >> 1) & 1u;
        // The epilogue must have drained this accumulator (first use passes).
        if (!mbar_wait_bounded(&tmem_empty_bar[ab], use ^ 1u, abort, wait_limit)) break;
        tc_fence_after_sync();
        const uint32_t tmem_acc = tmem_base + static_cast<uint32_t>(ab * BN);
        uint32_t accumulate = 0;
        for (int k = 0; k < args.k_iters; k += Plan::kSub) {
          if (!mbar_wait_bounded(&full_bar[pos.stage], pos.parity, abort, wait_limit)) {
            alive = false;
            break;
          }
          tc_fence_after_sync();
          MCB200_TRACE(2);
          const int nsub = args.k_iters - k < Plan::kSub ? args.k_iters - k : Plan::kSub;
          const uint32_t a_addr = tiles_addr + static_cast<uint32_t>(pos.stage * stage_bytes);
          uint64_t desc_a = umma_desc_k_sw128(a_addr);
          uint64_t desc_b = umma_desc_k_sw128(
              resident_b ? smem_addr(resident) + static_cast<uint32_t>(k) * Plan::kTileBBytes : a_addr + stage_b_offset);
          if (kMode == kModeHalo) {
            // Tap s of the filter row reads the strip s * dil_w pixel rows (128 bytes each) further
            // down: the same swizzled bytes, another start address.  The swizzle is a function of
            // the shared-memory address itself (TMA wrote the strip that way and the tensor core
            // reads it that way), so a start address that is not a multiple of the 1024-byte
            // pattern needs nothing else: the descriptor's base-offset field stays 0 (measured:
            // results equal the im2col mode's; with (address >> 7) & 7 in that field they are wrong).
            const uint32_t tap_step = static_cast<uint32_t>(args.dil_w) * 128u;
            for (int s = 0; s < args.kw; ++s) {
              const uint64_t da = umma_desc_k_sw128(a_addr + static_cast<uint32_t>(s) * tap_step);
#pragma unroll
              for (int kk = 0; kk < kMmaPerBlock; ++kk) {
                if (kHalf) {
                  if (kPair) {
                    umma_bf16_pair(tmem_acc, da + 2 * kk, desc_b + 2 * kk, idesc, accumulate);
                  } else {
                    umma_bf16(tmem_acc, da + 2 * kk, desc_b + 2 * kk, idesc, accumulate);
                  }
                } else if (kPair) {
                  umma_tf32_pair(tmem_acc, da + 2 * kk, desc_b + 2 * kk, idesc, accumulate);
                } else {
                  umma_tf32(tmem_acc, da + 2 * kk, desc_b + 2 * kk, idesc, accumulate);
                }
                accumulate = 1u;
              }
              desc_b += Plan::kTileBBytes >> 4;
            }
          }
#pragma unroll
          for (int j = 0; j < Plan::kSub; ++j) {
            if (kMode == kModeHalo) break;
            if (j >= nsub) break;
#pragma unroll
            for (int kk = 0; kk < kMmaPerBlock; ++kk) {
              // Each K step (8 tf32 or 16 bf16) is 32 bytes further along the swizzled
              // row: +2 in the descriptor's 16-byte address units.
              if (kHalf) {
                if (kPair) {
                  umma_bf16_pair(tmem_acc, desc_a + 2 * kk, desc_b + 2 * kk, idesc, accumulate);
                } else {
                  umma_bf16(tmem_acc, desc_a + 2 * kk, desc_b + 2 * kk, idesc, accumulate);
                }
              } else if (kPair) {
                umma_tf32_pair(tmem_acc, desc_a + 2 * kk, desc_b + 2 * kk, idesc, accumulate);
              } else {
                umma_tf32(tmem_acc, desc_a + 2 * kk, desc_b + 2 * kk, idesc, accumulate);
              }
              accumulate = 1u;
            }
            desc_a += kTileABytes >> 4;            // next sub-tile (start address is in 16-byte units)
            desc_b += Plan::kTileBBytes >> 4;
          }
          if (kPair) {
            umma_commit_pair(&empty_bar[pos.stage], 3);   // both CTAs' producers wait on their own copy
          } else {
            umma_commit(&empty_bar[pos.stage]);
          }
          MCB200_TRACE(2);
          pos.advance(stages);
        }
        if (alive) {
          if (kPair) {
            umma_commit_pair(&tmem_full_bar[ab], 3);
          } else {
            umma_commit(&tmem_full_bar[ab]);
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int ew = warp - kFirstEpilogueWarp;   // 0..7: staging ring and barriers of this warp
    const int quad = warp & 3;                  // tensor-memory lanes [32*quad, 32*quad+32)
    const int half = ew >> 2;                   // chunks half, half + 2, ... of every tile
    const mcb200_epilogue& ep = args.ep;
    const bool has_res = ep.residual != nullptr;
    // A slot holds a 32 x 32 sub-tile: 4 KiB, or 2 KiB when residual and result are both bfloat16.
    const int slot_bytes = (kHalf && args.out_half) ? 2048 : 4096;
    uint8_t* staging = staging_base + ew * (slots * slot_bytes);
    auto slot_ptr = [&](int slot) { return reinterpret_cast<float*>(staging + slot * slot_bytes); };
    const int chunks_full = BN / 32;
    const int epi_tid = threadIdx.x - kFirstEpilogueWarp * 32;   // 0..255 over the epilogue warps
    // 0: no activation, 1: plain ReLU, 2: per-column negative slope (leaky ReLU / PReLU)
    const int act_mode = ep.act == 0 ? 0 : ((ep.act == 1 && ep.slope == 0.f) ? 1 : 2);

    // Chunk sequence of this warp: for each of its CTA's tiles, the 32-column
    // chunks it owns that exist (the last n-tile may have fewer), left to right.
    // `seq` numbers them.  With a residual the warp cycles through its staging
    // slots, and a cursor of lane 0 walks the same sequence a few chunks ahead of
    // the computation (args.res_depth): it copies a coming chunk's residual
    // sub-tile into the slot that comes free next.  Asking L2 for the residual
    // further ahead instead (cp.async.bulk.prefetch) was tried and removed: the
    // lines were evicted by the output stream before use and DRAM reads grew by
    // half.
    struct ChunkCursor {
      int local;   // how many of this CTA's tiles lie behind the cursor
      int chunk;   // next chunk of the current tile
      int mt;      // M tile and first column of the current tile (-1: not looked up yet)
      int n0;
    };
    auto cursor_next = [&](ChunkCursor& cur, int& mt, int& col) {
      for (;;) {
        if (cur.mt < 0) {   // entering a tile: one division per tile, none per chunk
          const int tile = worker + cur.local * workers;
          if (tile >= num_tiles) return false;
          const int unit = tile / n_tiles;
          cur.mt = unit_to_mt(unit);
          cur.n0 = (tile - unit * n_tiles) * BN;
        }
        col = cur.n0 + cur.chunk * 32;
        if (cur.chunk >= chunks_full || col >= args.cout) {   // this warp's chunks of the tile are done
          cur.chunk = half;
          ++cur.local;
          cur.mt = -1;
          continue;
        }
        mt = cur.mt;
        cur.chunk += 2;
        return true;
      }
    };
    ChunkCursor ld = {0, half, -1, 0};
    int ld_slot = 0;                     // slot of the next residual load
    int cur_slot = 0;                    // slot of the chunk being finished (residual launches)
    uint32_t cur_parity = 0;
    auto issue_residual = [&]() {
      int mt, col;
      if (!cursor_next(ld, mt, col)) return;
      const int slot = ld_slot;
      if (++ld_slot == slots) ld_slot = 0;
      mbar_expect_tx(&res_bar[ew][slot], kHalf ? 2048 : 4096);   // 32 x 32 bfloat16 or fp32
      if (kMode == kModeRows) {
        tma_load_3d(&map_res, &res_bar[ew][slot], slot_ptr(slot), col, seg_start(mt) + quad * 32, row_of(mt));
      } else {
        tma_load_3d(&map_res, &res_bar[ew][slot], slot_ptr(slot), col, mt * kBlockM + quad * 32, 0);
      }
    };
    const bool staged = args.tma_epilogue != 0;
    // Residual sub-tiles are requested `res_depth` chunks ahead: a request takes
    // a DRAM round trip (one to two microseconds), several times the time a warp
    // needs per chunk.  Requesting chunk g + depth reuses the slot of chunk
    // g + depth - slots, so at most slots - depth - 1 of the latest stores may
    // still be reading shared memory at that point.
    const int res_depth = args.res_depth;
    const int stores_in_flight = slots - res_depth - 1;
    if (staged && has_res && lane == 0) {
      for (int d = 0; d < res_depth; ++d) issue_residual();
    }

    int seq = 0;
    int local = 0;
    bool alive = true;
    MCB200_TRACE_DECL;
    MCB200_TRACE_CHUNK_DECL;
    int table_n0[2] = {-1, -1};          // first column the per-column tables were filled for
    uint32_t table_fills[2] = {0u, 0u};
    for (int tile = worker; tile < num_tiles && alive; tile += workers, ++local) {
      const int ab = local & 1;
      const uint32_t use = static_cast<uint32_t>(local >> 1) & 1u;
      const int unit = tile / n_tiles;
      const int mt = unit_to_mt(unit);
      const int n0 = (tile - unit * n_tiles) * BN;
      // First output row (pixel) of this warp's 32-row slice, and how many of the 32 exist.
      const int row0 = (kMode == kModeRows ? row_of(mt) * args.wo + seg_start(mt) : mt * kBlockM) + quad * 32;
      const int rows_here = kMode == kModeRows ? min(args.tile_rows, args.wo - seg_start(mt)) - quad * 32 : args.m - row0;
      // Row of the output matrix this lane stores in the plain-store epilogue, and whether it exists.
      int out_row = row0 + lane;
      bool row_ok = lane < rows_here;
      if (kMode == kModeHalo) {
        const int t = out_row / args.wp;           // (image, output row); out_row counts virtual positions
        const int j = out_row - t * args.wp;
        row_ok = row_ok && j < args.wo;
        out_row = t * args.wo + j;
      }
      // tcgen05.ld is warp-collective: the whole warp takes the same branch.
      alive = __all_sync(0xffffffffu, mbar_wait_bounded(&tmem_full_bar[ab], use, abort, wait_limit));
      if (!alive) break;
      tc_fence_after_sync();
      if (ew == 0 && lane == 0) MCB200_TRACE(3);
      // Per-column constants of the tile's columns go to shared memory, so that the
      // inner loops are a broadcast 16-byte load and fused multiply-adds.  Two
      // copies (tile parity), each kept while the CTA's tiles of that parity stay
      // in the same column range (always, when the layer has one N tile or the
      // grid is a multiple of the N tiles).  A copy may be overwritten here: the
      // accumulator of this parity is full again, so every warp has finished
      // the tile that last used the copy.
      float* t_scale = col_scale[ab];
      float* t_shift = col_shift[ab];
      float* t_slope = col_slope[ab];
      if (table_n0[ab] != n0) {
        for (int c = epi_tid; c < BN; c += kEpilogueWarps * 32) {
          const int cc = n0 + c;
          const bool in = cc < args.cout;
          t_scale[c] = (in && ep.scale) ? __ldg(ep.scale + cc) : 1.f;
          t_shift[c] = (in && ep.shift) ? __ldg(ep.shift + cc) : 0.f;
          t_slope[c] = ep.act == 2 ? ((in && ep.prelu) ? __ldg(ep.prelu + (ep.prelu_shared ? 0 : cc)) : 0.f) : ep.slope;
        }
        // Rendezvous of the epilogue warps on the table (an mbarrier rather than a
        // named barrier, so that the wait is bounded like every other one).
        __syncwarp();
        if (lane == 0) mbar_arrive(&col_bar[ab]);
        alive = __all_sync(0xffffffffu, mbar_wait_bounded(&col_bar[ab], table_fills[ab] & 1u, abort, wait_limit));
        if (!alive) break;
        ++table_fills[ab];
        table_n0[ab] = n0;
      }
      const uint32_t tmem_acc = tmem_base + static_cast<uint32_t>(ab * BN) + (static_cast<uint32_t>(quad * 32) << 16);
#pragma unroll 1
      for (int chunk = half; chunk < chunks_full; chunk += 2) {
        const int col0 = n0 + chunk * 32;
        if (col0 >= args.cout) break;          // uniform across the warp
        const int g = seq++;
        uint32_t acc[32];
        MCB200_TRACE_CHUNK();
        tmem_load_32x32(tmem_acc + static_cast<uint32_t>(chunk * 32), acc);
        tmem_load_wait();
        MCB200_TRACE_CHUNK();
        const float4* sc4 = reinterpret_cast<const float4*>(t_scale + chunk * 32);
        const float4* sh4 = reinterpret_cast<const float4*>(t_shift + chunk * 32);
        const float4* sl4 = reinterpret_cast<const float4*>(t_slope + chunk * 32);
        // v = acc * scale + shift (+ coeff * residual), then the activation.  The
        // activation is a compile-time tag: with a run-time test inside, every
        // group of four values became its own chain of small basic blocks (load,
        // multiply-add, branch, ...), each exposing its latencies, and a sub-tile
        // took over a thousand cycles; as straight-line code the 32 chains of a
        // row overlap.
        auto finish4 = [&](auto act_tag, int j, float4 r, bool add_res) {
          constexpr int kAct = decltype(act_tag)::value;
          const float4 sc = sc4[j], sh = sh4[j];
          float4 v;
          v.x = fmaf(__uint_as_float(acc[j * 4 + 0]), sc.x, sh.x);
          v.y = fmaf(__uint_as_float(acc[j * 4 + 1]), sc.y, sh.y);
          v.z = fmaf(__uint_as_float(acc[j * 4 + 2]), sc.z, sh.z);
          v.w = fmaf(__uint_as_float(acc[j * 4 + 3]), sc.w, sh.w);
          if (add_res) {
            v.x = fmaf(ep.residual_coeff, r.x, v.x);
            v.y = fmaf(ep.residual_coeff, r.y, v.y);
            v.z = fmaf(ep.residual_coeff, r.z, v.z);
            v.w = fmaf(ep.residual_coeff, r.w, v.w);
          }
          if (kAct == 1) {
            v.x = fmaxf(v.x, 0.f);
            v.y = fmaxf(v.y, 0.f);
            v.z = fmaxf(v.z, 0.f);
            v.w = fmaxf(v.w, 0.f);
          } else if (kAct == 2) {
            const float4 sl = sl4[j];
            v.x = v.x > 0.f ? v.x : v.x * sl.x;
            v.y = v.y > 0.f ? v.y : v.y * sl.y;
            v.z = v.z > 0.f ? v.z : v.z * sl.z;
            v.w = v.w > 0.f ? v.w : v.w * sl.w;
          }
          return v;
        };
        auto round4 = [&](float4& v) {
          v.x = round_to_tf32(v.x);
          v.y = round_to_tf32(v.y);
          v.z = round_to_tf32(v.z);
          v.w = round_to_tf32(v.w);
        };
        if (staged) {
          const int slot = has_res ? cur_slot : (slots == 2 ? (g & 1) : 0);
          float* buf = slot_ptr(slot) + lane * 32;
          if (has_res) {
            if (lane == 0) {
              switch (stores_in_flight) {
                case 0: tma_store_wait_read<0>(); break;
                case 1: tma_store_wait_read<1>(); break;
                case 2: tma_store_wait_read<2>(); break;
                default: tma_store_wait_read<3>(); break;
              }
              issue_residual();
            }
            alive = __all_sync(0xffffffffu,
                               mbar_wait_bounded(&res_bar[ew][slot], cur_parity, abort, wait_limit));
            if (!alive) break;
            if (++cur_slot == slots) {
              cur_slot = 0;
              cur_parity ^= 1u;
            }
          }
          MCB200_TRACE_CHUNK();
          // Row `lane` of the 32 x 32 tile is 128 bytes: eight 16-byte pieces,
          // piece j stored at position j ^ (row & 7) (the 128-byte swizzle).
          // The result overwrites the residual in place.
          const int swz = lane & 7;
          // All reads of the chunk (residual cells, per-column tables) come
          // before its first write: the loads are then independent of each other
          // and overlap, where a read-modify-write per cell would expose one
          // shared-memory round trip after the other (long ones while the
          // tensor core and the TMA keep shared memory busy).
          float4 v[8];
          // bfloat16 rows are 64 bytes: four 16-byte pieces, piece q stored at
          // position q ^ ((row >> 1) & 3) (the 64-byte swizzle).
          uint8_t* hrow = reinterpret_cast<uint8_t*>(slot_ptr(slot)) + lane * 64;
          const int hswz = (lane >> 1) & 3;
          auto fill = [&](auto act_tag) {
            if (!has_res) {
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] = finish4(act_tag, j, make_float4(0.f, 0.f, 0.f, 0.f), false);
            } else if (kHalf) {
              uint4 w[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) w[q] = *reinterpret_cast<const uint4*>(hrow + ((q ^ hswz) << 4));
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                v[2 * q] = finish4(act_tag, 2 * q,
                                   make_float4(bf16_lo(w[q].x), bf16_hi(w[q].x), bf16_lo(w[q].y), bf16_hi(w[q].y)), true);
                v[2 * q + 1] = finish4(act_tag, 2 * q + 1,
                                       make_float4(bf16_lo(w[q].z), bf16_hi(w[q].z), bf16_lo(w[q].w), bf16_hi(w[q].w)),
                                       true);
              }
            } else {
              float4 r[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) r[j] = *reinterpret_cast<const float4*>(buf + ((j ^ swz) << 2));
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] = finish4(act_tag, j, r[j], true);
            }
          };
          if (act_mode == 1) {
            fill(ActTag<1>());
          } else if (act_mode == 0) {
            fill(ActTag<0>());
          } else {
            fill(ActTag<2>());
          }
          if (ep.round_tf32) {
#pragma unroll
            for (int j = 0; j < 8; ++j) round4(v[j]);
          }
          if (!has_res && g >= slots) {
            // The store that last used this slot must have finished reading it.  Asked only now,
            // with the chunk's values in registers: the query costs its thread some 200 cycles
            // whatever the answer, which the table loads above spend in flight.
            if (lane == 0) {
              if (slots == 2) {
                tma_store_wait_read<1>();
              } else {
                tma_store_wait_read<0>();
              }
            }
            __syncwarp();
          }
          // Residual and result rows of different widths overlap other lanes' rows.
          if (has_res && (args.out_half != 0) != kHalf) __syncwarp();
          if (args.out_half) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 w;
              w.x = pack_bf16x2(v[2 * q].x, v[2 * q].y);
              w.y = pack_bf16x2(v[2 * q].z, v[2 * q].w);
              w.z = pack_bf16x2(v[2 * q + 1].x, v[2 * q + 1].y);
              w.w = pack_bf16x2(v[2 * q + 1].z, v[2 * q + 1].w);
              *reinterpret_cast<uint4*>(hrow + ((q ^ hswz) << 4)) = w;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) *reinterpret_cast<float4*>(buf + ((j ^ swz) << 2)) = v[j];
          }
          MCB200_TRACE_CHUNK();
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (kMode == kModeRows) {
              tma_store_3d(&map_out, slot_ptr(slot), col0, seg_start(mt) + quad * 32, row_of(mt));   // clipped at the row's end
            } else {
              tma_store_3d(&map_out, slot_ptr(slot), col0, row0, 0);
            }
            tma_store_commit();
          }
          MCB200_TRACE_CHUNK();
        } else {
          // ---- plain stores: rows that are not 16-byte aligned, and halo mode, whose tiles are
          // pieces of the virtual output grid (a lane's row may be one of the positions that are
          // computed and dropped) ----
          const size_t out_off = static_cast<size_t>(row_ok ? out_row : 0) * args.out_ld;
          const size_t res_off = static_cast<size_t>(row_ok ? out_row : 0) * ep.residual_ld;
          const bool whole_chunk = args.vec_store && col0 + 32 <= args.cout;
          // The lane's 32 outputs of its row (128 bytes, 64 as bfloat16), fused tail applied.
          float4 v[8];
          if (whole_chunk && (row_ok || (kMode == kModeHalo && args.halo_staged))) {
            const bool add_res = has_res && row_ok;
            auto fill = [&](auto act_tag) {
              if (!add_res) {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = finish4(act_tag, j, make_float4(0.f, 0.f, 0.f, 0.f), false);
              } else if (kHalf) {
                const uint4* rp = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(ep.residual) + res_off + col0);
                uint4 w[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) w[q] = rp[q];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  v[2 * q] = finish4(act_tag, 2 * q,
                                     make_float4(bf16_lo(w[q].x), bf16_hi(w[q].x), bf16_lo(w[q].y), bf16_hi(w[q].y)), true);
                  v[2 * q + 1] = finish4(act_tag, 2 * q + 1,
                                         make_float4(bf16_lo(w[q].z), bf16_hi(w[q].z), bf16_lo(w[q].w), bf16_hi(w[q].w)),
                                         true);
                }
              } else {
                const float4* rp = reinterpret_cast<const float4*>(ep.residual + res_off + col0);
                float4 r[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) r[j] = rp[j];
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = finish4(act_tag, j, r[j], true);
              }
            };
            if (act_mode == 1) {
              fill(ActTag<1>());
            } else if (act_mode == 0) {
              fill(ActTag<0>());
            } else {
              fill(ActTag<2>());
            }
            if (ep.round_tf32) {
#pragma unroll
              for (int j = 0; j < 8; ++j) round4(v[j]);
            }
          }
          if (kMode == kModeHalo && args.halo_staged && whole_chunk) {
            // Through the warp's shared-memory slot, so that a store instruction writes four whole
            // 128-byte rows (eight lanes each) instead of 16 bytes of 32 different rows: a lane's
            // own row may be a dropped position, its neighbours' rows are not.
            float* slot = slot_ptr(0);
            const int swz = lane & 7;
#pragma unroll
            for (int j = 0; j < 8; ++j) *reinterpret_cast<float4*>(slot + lane * 32 + ((j ^ swz) << 2)) = v[j];
            __syncwarp();
            const int piece = lane & 7;
#pragma unroll
            for (int p = 0; p < 8; ++p) {
              const int r = 4 * p + (lane >> 3);
              const int orow = __shfl_sync(0xffffffffu, out_row, r);
              const int ok = __shfl_sync(0xffffffffu, row_ok ? 1 : 0, r);
              const float4 val = *reinterpret_cast<const float4*>(slot + r * 32 + ((piece ^ (r & 7)) << 2));
              if (ok) *reinterpret_cast<float4*>(args.out + static_cast<size_t>(orow) * args.out_ld + col0 + piece * 4) = val;
            }
            __syncwarp();   // the slot is rewritten by the next chunk
          } else if (row_ok) {
            if (whole_chunk) {
              if (args.out_half) {
                uint4* op = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(args.out) + out_off + col0);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  uint4 w;
                  w.x = pack_bf16x2(v[2 * q].x, v[2 * q].y);
                  w.y = pack_bf16x2(v[2 * q].z, v[2 * q].w);
                  w.z = pack_bf16x2(v[2 * q + 1].x, v[2 * q + 1].y);
                  w.w = pack_bf16x2(v[2 * q + 1].z, v[2 * q + 1].w);
                  op[q] = w;
                }
              } else {
                float4* op = reinterpret_cast<float4*>(args.out + out_off + col0);
#pragma unroll
                for (int j = 0; j < 8; ++j) op[j] = v[j];
              }
            } else {
              auto residual_at = [&](int c) {
                if (kHalf) {
                  return __uint_as_float(static_cast<uint32_t>(reinterpret_cast<const uint16_t*>(ep.residual)[res_off + c])
                                         << 16);
                }
                return ep.residual[res_off + c];
              };
              auto store_at = [&](int c, float value) {
                if (args.out_half) {
                  reinterpret_cast<uint16_t*>(args.out)[out_off + c] = static_cast<uint16_t>(pack_bf16x2(value, 0.f));
                } else {
                  args.out[out_off + c] = value;
                }
              };
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const int c = col0 + j * 4;
                if (c >= args.cout) break;
                float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
                if (has_res) {
                  r.x = residual_at(c);
                  if (c + 1 < args.cout) r.y = residual_at(c + 1);
                  if (c + 2 < args.cout) r.z = residual_at(c + 2);
                  if (c + 3 < args.cout) r.w = residual_at(c + 3);
                }
                float4 v = act_mode == 1   ? finish4(ActTag<1>(), j, r, has_res)
                           : act_mode == 0 ? finish4(ActTag<0>(), j, r, has_res)
                                           : finish4(ActTag<2>(), j, r, has_res);
                if (ep.round_tf32) round4(v);
                store_at(c, v.x);
                if (c + 1 < args.cout) store_at(c + 1, v.y);
                if (c + 2 < args.cout) store_at(c + 2, v.z);
                if (c + 3 < args.cout) store_at(c + 3, v.w);
              }
            }
          }
        }
      }
      // All of this warp's reads of the accumulator are complete: hand it back.
      if (ew == 0 && lane == 0) MCB200_TRACE(3);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (kPair) {
          mbar_arrive_cluster(tmem_empty_leader + static_cast<uint32_t>(ab) * 8u);
        } else {
          mbar_arrive(&tmem_empty_bar[ab]);
        }
      }
    }
    if (staged && lane == 0) tma_store_wait_read<0>();
    __syncwarp();
  }

  // ------------------------------------------------------------ teardown
  // A pair leaves together: until both CTAs are here, the peer may still
  // signal this CTA's barriers or (rank 0's MMAs) write its tensor memory.
  tc_fence_before_sync();
  __syncwarp();
  if (kPair) {
    cluster_sync_all();
  } else {
    __syncthreads();
  }
  if (warp == kWarpMma) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 2 * BN);
  }
  if (threadIdx.x == 0 && abort_flag && args.status) atomicExch(args.status, 1);
}

// ------------------------------------------------------------------ weight packing

__global__ void pack_weights_kernel(const float* __restrict__ w, float* __restrict__ packed, int cout, int c, int taps,
                                    int c_pad) {
  const size_t total = static_cast<size_t>(cout) * taps * c_pad;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int cc = static_cast<int>(i % c_pad);
    const int tap = static_cast<int>((i / c_pad) % taps);
    const int co = static_cast<int>(i / (static_cast<size_t>(c_pad) * taps));
    float v = 0.f;
    if (cc < c) v = round_to_tf32(w[(static_cast<size_t>(co) * c + cc) * taps + tap]);
    packed[i] = v;
  }
}

// Same image in bfloat16 (round to nearest even), taps padded to a multiple of 64 channels.
__global__ void pack_weights_bf16_kernel(const float* __restrict__ w, uint16_t* __restrict__ packed, int cout, int c,
                                         int taps, int c_pad) {
  const size_t total = static_cast<size_t>(cout) * taps * c_pad;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int cc = static_cast<int>(i % c_pad);
    const int tap = static_cast<int>((i / c_pad) % taps);
    const int co = static_cast<int>(i / (static_cast<size_t>(c_pad) * taps));
    float v = 0.f;
    if (cc < c) v = w[(static_cast<size_t>(co) * c + cc) * taps + tap];
    packed[i] = static_cast<uint16_t>(pack_bf16x2(v, 0.f));
  }
}

// fp32 <-> bfloat16 copies of an activation tensor (the layout does not change).
__global__ void f32_to_bf16_kernel(const float4* __restrict__ src, uint2* __restrict__ dst, size_t quads,
                                   const float* __restrict__ src1, uint16_t* __restrict__ dst1, size_t count) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  const size_t first = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  for (size_t i = first; i < quads; i += stride) {
    const float4 v = src[i];
    dst[i] = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
  }
  for (size_t i = quads * 4 + first; i < count; i += stride) dst1[i] = static_cast<uint16_t>(pack_bf16x2(src1[i], 0.f));
}

__global__ void bf16_to_f32_kernel(const uint2* __restrict__ src, float4* __restrict__ dst, size_t quads,
                                   const uint16_t* __restrict__ src1, float* __restrict__ dst1, size_t count) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  const size_t first = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  for (size_t i = first; i < quads; i += stride) {
    const uint2 w = src[i];
    dst[i] = make_float4(bf16_lo(w.x), bf16_hi(w.x), bf16_lo(w.y), bf16_hi(w.y));
  }
  for (size_t i = quads * 4 + first; i < count; i += stride)
    dst1[i] = __uint_as_float(static_cast<uint32_t>(src1[i]) << 16);
}

// ------------------------------------------------------------------ grouped layers

// Grouped layers run with 64-column N tiles (the narrowest: the fewest foreign channels under a
// tile's weight columns).  First channel an N tile's weight columns refer to, and how many
// channel blocks the widest tile spans.
constexpr int kGroupedBlockN = 64;

__host__ __device__ inline int grouped_origin(int n0, int group_cout, int group_cin, int align) {
  return ((n0 / group_cout) * group_cin) & ~(align - 1);
}

int grouped_c_blocks(const mcb200_conv_shape* s, int kelems, int align) {
  const int group_cout = s->cout / s->group, group_cin = s->c / s->group;
  int widest = 0;
  for (int n0 = 0; n0 < s->cout; n0 += kGroupedBlockN) {
    const int last = (n0 + kGroupedBlockN < s->cout ? n0 + kGroupedBlockN : s->cout) - 1;
    const int span = (last / group_cout + 1) * group_cin - grouped_origin(n0, group_cout, group_cin, align);
    if (span > widest) widest = span;
  }
  return (widest + kelems - 1) / kelems;
}

// Packed image of grouped weights [cout][cin / group][taps]: [cout][taps][c_pad] where column j of
// an output channel's row stands for input channel origin(tile of the output channel) + j; zero
// where that channel belongs to another group (or lies beyond the tensor).
template <bool kHalf>
__global__ void pack_weights_grouped_kernel(const float* __restrict__ w, void* __restrict__ packed_any, int cout, int taps,
                                            int c_pad, int group_cout, int group_cin) {
  const size_t total = static_cast<size_t>(cout) * taps * c_pad;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int j = static_cast<int>(i % c_pad);
    const int tap = static_cast<int>((i / c_pad) % taps);
    const int co = static_cast<int>(i / (static_cast<size_t>(c_pad) * taps));
    const int origin = grouped_origin(co / kGroupedBlockN * kGroupedBlockN, group_cout, group_cin, kHalf ? 8 : 4);
    const int local = origin + j - (co / group_cout) * group_cin;   // channel index inside co's group
    float v = 0.f;
    if (local >= 0 && local < group_cin) v = w[(static_cast<size_t>(co) * group_cin + local) * taps + tap];
    if (kHalf) {
      static_cast<uint16_t*>(packed_any)[i] = static_cast<uint16_t>(pack_bf16x2(v, 0.f));
    } else {
      static_cast<float*>(packed_any)[i] = round_to_tf32(v);
    }
  }
}

// ------------------------------------------------------------------ tensor maps

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const int*, const int*, cuuint32_t, cuuint32_t,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct DriverApi {
  EncodeTiledFn tiled = nullptr;
  EncodeIm2colFn im2col = nullptr;
  int driver_version = 0;
  bool ok = false;
};

const DriverApi& driver_api() {
  static DriverApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess || !fn)
      return;
    api.tiled = reinterpret_cast<EncodeTiledFn>(fn);
    fn = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess || !fn)
      return;
    api.im2col = reinterpret_cast<EncodeIm2colFn>(fn);
    cudaDriverGetVersion(&api.driver_version);
    api.ok = true;
  });
  return api;
}

// Tile width.  The kernel is persistent (one CTA per SM), so a layer takes as
// long as its busiest CTA: ceil(tiles / SMs) tiles, each costing its k-iterations
// (operand bytes per iteration grow with BN) plus an epilogue proportional to BN.
// Wide tiles re-read the activations less often, narrow tiles fill the machine
// when there are few output pixels; take the cheapest of the three.
int pick_block_n(int cout, long long m, int k_iters, double* cost_out = nullptr) {
  const char* force = getenv("MCB200_BLOCK_N");   // "64" / "128" / "256": override for experiments and tests
  if (force && !cost_out) {
    const int bn = atoi(force);
    if (bn == 64 || bn == 128 || bn == 256) return bn;
  }
  const long long m_tiles = (m + kBlockM - 1) / kBlockM;
  int best = 64;
  double best_cost = 0.0;
  for (int bn = 64; bn <= 256; bn *= 2) {
    if (bn > 64 && bn / 2 >= cout) break;   // wider than the layer: only padding
    const long long tiles = m_tiles * ((cout + bn - 1) / bn);
    const long long waves = (tiles + 147) / 148;
    // 64 KiB of operand-byte equivalents per 32-column chunk of epilogue: a chunk costs a warp
    // 1400-2300 cycles (two warps per tensor-memory quadrant), as long as some 64 KiB take to
    // arrive.  (Measured in interleaved runs of the three benchmark networks: the 8 KiB this
    // started with sent the 128 -> 512 residual layers of ResNet-50 to 256-column tiles, six waves
    // of eight chunks where eleven waves of four are 6 % quicker; values of 48-96 KiB agree.)
    const double per_tile = static_cast<double>(k_iters) * (kTileABytes + 128.0 * bn) + 65536.0 * (bn / 32);
    const double cost = static_cast<double>(waves) * per_tile;
    if (bn == 64 || cost < best_cost * 0.97) {   // prefer the narrower tile on near ties
      best = bn;
      best_cost = cost;
    }
  }
  if (cost_out) *cost_out = best_cost;
  return best;
}

// Shared memory a CTA can give to the operand ring, roughly (the exact figure depends on the
// kernel variant's static shared memory; the launch computes it).
constexpr int kRingBudget = kSharedLimit - 10 * 1024;

// Halo mode: tile width, pairing and cost by the same model (a CTA's time is its operand bytes).
// A stage holds the pixel strip and the weight tiles of the kw taps of a filter row; widths whose
// stage does not fit three times are left out.  Returns 0 when no width is usable.
int pick_block_n_halo(int cout, long long m_virtual, int k_iters, int kw, int strip_bytes, int* pair_out,
                      double* cost_out) {
  const char* force = getenv("MCB200_BLOCK_N");
  const int forced = force ? atoi(force) : 0;
  const char* force_pair = getenv("MCB200_CTA_PAIR");
  const long long m_tiles = (m_virtual + kBlockM - 1) / kBlockM;
  const int strip_slot = (strip_bytes + 1023) / 1024 * 1024;
  int best = 0;
  double best_cost = 0.0;
  // 256-column tiles only when asked for: on every halo-mode layer measured with both widths
  // (VGG-16 at 300 x 300, batch 32: 256 -> 256 on 75 x 75 maps, 256 -> 512 and 512 -> 512 on 38 x 38;
  // ResNet-50's 512 -> 512 on 7 x 7) paired 128-column tiles are as quick or quicker, by up to 13 %:
  // these layers run near the tensor pipe's rate, where twice as many narrower tiles fill the
  // last wave better and a stage is 41 KiB instead of 65.
  const int widest = forced == 256 ? 256 : 128;
  for (int bn = 64; bn <= widest; bn *= 2) {
    if (bn > 64 && bn / 2 >= cout) break;
    if ((forced == 64 || forced == 128 || forced == 256) && bn != forced) continue;
    for (int pair = 0; pair <= 1; ++pair) {
      if (pair && (bn < 128 || m_tiles < 2)) continue;
      if (force_pair && (force_pair[0] == '0' || force_pair[0] == '1') && bn >= 128 && pair != force_pair[0] - '0')
        continue;
      const int stage = strip_slot + kw * (pair ? bn / 2 : bn) * 128;
      if (kRingBudget / stage < 3) continue;
      const long long units = pair ? (m_tiles + 1) / 2 : m_tiles;
      const long long tiles = units * ((cout + bn - 1) / bn);
      const long long workers = pair ? 74 : 148;
      const long long waves = (tiles + workers - 1) / workers;
      // the pair's cluster-wide synchronisation costs about two k-iterations per tile
      const double per_tile = static_cast<double>(k_iters + (pair ? 2 : 0)) * stage + 8192.0 * (bn / 32);
      const double cost = static_cast<double>(waves) * per_tile;
      if (best == 0 || cost < best_cost * 0.97) {
        best = bn;
        best_cost = cost;
        *pair_out = pair;
      }
    }
  }
  if (cost_out) *cost_out = best_cost;
  return best;
}

// Whether two-CTA clusters run the layer.  Pairing halves the weight bytes each
// SM pulls per MAC, which pays where the operand ring bounds the main loop (wide
// tiles, long K) and there are at least two M tiles to pair up.  Short-K layers
// are bound by their epilogue and only pay for the pair's extra synchronisation
// (measured on ResNet-50: gains from 16 k-iterations up when no residual is
// added, losses at 4-16 with one).
int pick_cta_pair(int block_n, long long m, int k_iters) {
  const char* force = getenv("MCB200_CTA_PAIR");   // "0" / "1": override for experiments
  if (force && (force[0] == '0' || force[0] == '1')) return block_n >= 128 && force[0] == '1' ? 1 : 0;
  // 256-column tiles pair from 16 k-iterations (the 512 -> 1024 stride-2 projection of ResNet-50:
  // 39 -> 34 us), 128-column tiles from 17 (the 512 -> 2048 residual layers lose 1-2 us at 16).
  return (block_n >= 128 && m > kBlockM && k_iters >= (block_n == 256 ? 16 : 17)) ? 1 : 0;
}

// Tile map for the staged epilogue over a row-major matrix with row pitch `ld`
// (elements), 32 x 32 boxes: fp32 with the 128-byte swizzle, or bfloat16 (64-byte
// box rows) with the 64-byte swizzle.  The rows are split as (group, row in
// group): ordinary tiles use one group of all rows; row mode uses one group per
// output row of an image so that a tile never spills into the next row.
CUresult encode_tile_map(CUtensorMap* map, const void* base, bool half, int cols, int ld, long long rows_per_group,
                         long long groups) {
  const DriverApi& api = driver_api();
  const cuuint64_t es = half ? 2 : 4;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows_per_group),
                              static_cast<cuuint64_t>(groups)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * es,
                                 static_cast<cuuint64_t>(ld) * es * static_cast<cuuint64_t>(rows_per_group)};
  const cuuint32_t box[3] = {32, 32, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  return api.tiled(map, half ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3,
                   const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   half ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
}

template <int BN, int kMode, bool kPair, bool kHalf>
cudaError_t launch_variant(const mcb200_conv_plan* plan, ConvTcArgs args, cudaStream_t stream) {
  using Plan = SmemPlan<BN, kMode, kPair>;
  auto kernel = conv_tc_kernel<BN, kMode, kPair, kHalf>;
  // The large-shared-memory opt-in is per device: do it once for each device
  // this process launches on.  What the ring may use is the CTA limit minus the
  // kernel's static shared memory (barriers, per-column tables).
  int dev = 0;
  cudaGetDevice(&dev);
  static bool configured[64] = {false};
  static int sm_count[64] = {0};
  static int dynamic_limit = 0;
  static std::mutex mu;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dynamic_limit == 0) {
      cudaFuncAttributes attr;
      cudaError_t e = cudaFuncGetAttributes(&attr, kernel);
      if (e != cudaSuccess) return e;
      dynamic_limit = kSharedLimit - static_cast<int>(attr.sharedSizeBytes);
    }
    if (dev >= 0 && dev < 64 && !configured[dev]) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dynamic_limit);
      if (e != cudaSuccess) return e;
      int n = 0;
      if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) n = 148;
      sm_count[dev] = n;
      configured[dev] = true;
    }
  }
  const long long m_tiles = kMode == kModeRows
                                ? static_cast<long long>(plan->shape.n) * plan->shape.ho * args.row_segments
                                : (static_cast<long long>(args.m) + kBlockM - 1) / kBlockM;   // halo: virtual positions
  const long long m_units = kPair ? (m_tiles + 1) / 2 : m_tiles;
  const long long tiles = static_cast<long long>((plan->shape.cout + BN - 1) / BN) * m_units;
  if (tiles > 0x3fffffffLL) return cudaErrorInvalidConfiguration;
  // One persistent CTA per SM (fewer when there are fewer tiles); a paired
  // launch is a grid of two-CTA clusters, one cluster per tile at a time.
  const int sms = (dev >= 0 && dev < 64 && sm_count[dev] > 0) ? sm_count[dev] : 148;
  const long long workers_max = kPair ? sms / 2 : sms;
  const unsigned workers = static_cast<unsigned>(tiles < workers_max ? tiles : workers_max);
  // Staging slots per epilogue warp.  With a residual: three where tiles are so short that the
  // ring needs little (load, work and store of consecutive chunks overlap), else two.  Without:
  // one, and the ring takes the rest.  (Two slots for short or single tiles were the rule until
  // interleaved runs on one GPU showed one slot to be as quick or quicker on every layer of the
  // three benchmark networks: ResNet-50 1.963 -> 1.946 ms per pass, MobileNet-v1 0.778 -> 0.776,
  // SSD300 5.00 -> 4.98; a 7 x 7 first layer keeps eight activation tiles in flight instead of six.)
  const int k_units = args.k_iters * (kHalf ? 2 : 1);   // in 32-channel steps, the unit the rules were measured in
  args.slots = args.ep.residual != nullptr ? (k_units <= 4 ? 3 : 2) : 1;
  args.res_depth = 1;
  if (args.ep.residual == nullptr) {
    const char* force = getenv("MCB200_SLOTS");   // experiments: "1" / "2"
    if (force && (force[0] == '1' || force[0] == '2')) args.slots = force[0] - '0';
  } else {
    const char* force_slots = getenv("MCB200_RES_SLOTS");   // experiments: "2" .. "8"
    const char* force_depth = getenv("MCB200_RES_DEPTH");   // experiments: "1" .. slots - 1
    if (force_slots && atoi(force_slots) >= 2 && atoi(force_slots) <= kMaxSlots) args.slots = atoi(force_slots);
    if (force_depth && atoi(force_depth) >= 1) args.res_depth = atoi(force_depth);
    if (args.res_depth > args.slots - 1) args.res_depth = args.slots - 1;
  }
  const int slot_bytes = (kHalf && args.out_half) ? 2048 : 4096;
  int stage_bytes = Plan::kStageBytes;
  int staging_bytes = Plan::staging_bytes(args.slots, slot_bytes);
  int resident_bytes = 0;
  if (kMode == kModeRows) {
    // One N tile: every M tile multiplies the same kh weight tiles; they stay in shared memory
    // when they take at most a quarter of it, and the ring carries activations only.
    const long long all_rows = static_cast<long long>(args.k_iters) * Plan::kTileBBytes;
    const char* off = getenv("MCB200_ROWS_RESIDENT");   // "0": stream the weights with the activations (experiments)
    if (plan->shape.cout <= BN && all_rows <= 56 * 1024 && !(off && off[0] == '0')) resident_bytes = static_cast<int>(all_rows);
    args.resident_b_bytes = resident_bytes;
    args.stage_b_offset = kTileABytes;
    args.stage_bytes = resident_bytes ? kTileABytes : kTileABytes + Plan::kTileBBytes;
    stage_bytes = args.stage_bytes;
  }
  if (kMode == kModeHalo) {
    // A stage = the pixel strip (rounded up to the 1024-byte swizzle period) + the weight tiles of
    // the kw taps of one filter row.  The epilogue stores from registers: no staging.
    args.stage_b_offset = (args.a_bytes + 1023) / 1024 * 1024;
    args.stage_bytes = args.stage_b_offset + plan->shape.kw * Plan::kTileBBytes;
    stage_bytes = args.stage_bytes;
    args.halo_staged = (args.vec_store && !args.out_half && !getenv("MCB200_HALO_DIRECT_STORES")) ? 1 : 0;
    args.slots = 1;
    staging_bytes = args.halo_staged ? Plan::staging_bytes(1, 4096) : 0;
  }
  {
    // At most 64 prefetch instructions per tile (long-K tiles take long enough for the ring).
    const int kh = plan->shape.kh, cb = args.c_blocks;
    const int count = kMode == kModeMatrix ? cb : kh * cb * ((kMode == kModeIm2col && plan->shape.stride_w > 1) ? 2 : 1);
    // Off unless MCB200_L2_PREFETCH=1: measured on ResNet-50 at batch 64 it costs 2 % (the 1 x 1
    // reductions lose 8 %: the requests compete with the loads of the tile at hand), and the
    // layers it was meant for do not gain.
    const char* pf = getenv("MCB200_L2_PREFETCH");
    args.l2_prefetch = (kMode != kModeRows && count <= 64 && pf && pf[0] == '1') ? 1 : 0;
  }
  int stages = (dynamic_limit - 1024 - staging_bytes - resident_bytes) / stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < 2) return cudaErrorInvalidConfiguration;
  args.stages = stages;
  const int dynamic_bytes = stages * stage_bytes + staging_bytes + resident_bytes + 1024;
  const CUtensorMap* ma = reinterpret_cast<const CUtensorMap*>(plan->tma_a);
  const CUtensorMap* mb = reinterpret_cast<const CUtensorMap*>(plan->tma_b);
  const CUtensorMap* mo = reinterpret_cast<const CUtensorMap*>(plan->tma_out);
  const CUtensorMap* mr = reinterpret_cast<const CUtensorMap*>(plan->tma_res);
  cudaError_t launched;
  {
    TimedLaunch timed(stream);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kPair ? workers * 2 : workers, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = static_cast<size_t>(dynamic_bytes);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    // The kernel's set-up may overlap the end of the previous kernel in the
    // stream; it orders itself with griddepcontrol.wait.
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 2;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = kPair ? 2 : 1;
    launched = cudaLaunchKernelEx(&cfg, kernel, *ma, *mb, *mo, *mr, args);
  }
  count_launch();
  return launched;
}

}  // namespace
}  // namespace mcb200

using namespace mcb200;

namespace {
// Bound of the kernel's barrier waits (process-wide) and the one-shot test hook of the calling thread.
long long g_wait_limit_cycles = mcb200::kDefaultWaitLimitCycles;
thread_local int t_drop_weight_load = 0;
}  // namespace

extern "C" long long mcb200_conv_set_wait_limit(long long cycles) {
  const long long previous = g_wait_limit_cycles;
  g_wait_limit_cycles = cycles > 0 ? cycles : mcb200::kDefaultWaitLimitCycles;
  return previous;
}

extern "C" void mcb200_conv_test_drop_weight_load(void) { t_drop_weight_load = 1; }

extern "C" int mcb200_conv_out_shape(mcb200_conv_shape* s) {
  if (!s || s->kh < 1 || s->kw < 1 || s->stride_h < 1 || s->stride_w < 1 || s->dil_h < 1 || s->dil_w < 1) return -1;
  const int ext_h = s->dil_h * (s->kh - 1) + 1;
  const int ext_w = s->dil_w * (s->kw - 1) + 1;
  const int num_h = s->h + 2 * s->pad_h - ext_h;
  const int num_w = s->w + 2 * s->pad_w - ext_w;
  if (num_h < 0 || num_w < 0) return -1;
  s->ho = num_h / s->stride_h + 1;
  s->wo = num_w / s->stride_w + 1;
  return 0;
}

extern "C" size_t mcb200_conv_packed_weight_count(const mcb200_conv_shape* s) {
  const size_t c_pad = s->group > 1 ? static_cast<size_t>(grouped_c_blocks(s, kBlockK, 4)) * kBlockK
                                    : static_cast<size_t>((s->c + kBlockK - 1) / kBlockK) * kBlockK;
  return static_cast<size_t>(s->cout) * s->kh * s->kw * c_pad;
}

extern "C" int mcb200_conv_pack_weights(const mcb200_conv_shape* s, const float* w_oihw, float* packed,
                                        void* stream) {
  if (!s || !w_oihw || !packed || s->group < 1 || s->c % s->group != 0 || s->cout % s->group != 0) return -1;
  const size_t total = mcb200_conv_packed_weight_count(s);
  const int threads = 256;
  const int blocks = static_cast<int>((total + threads - 1) / threads < 148 * 8 ? (total + threads - 1) / threads
                                                                                  : 148 * 8);
  if (s->group > 1) {
    pack_weights_grouped_kernel<false><<<blocks > 0 ? blocks : 1, threads, 0, static_cast<cudaStream_t>(stream)>>>(
        w_oihw, packed, s->cout, s->kh * s->kw, grouped_c_blocks(s, kBlockK, 4) * kBlockK, s->cout / s->group,
        s->c / s->group);
    count_launch();
    return static_cast<int>(cudaGetLastError());
  }
  const int c_pad = (s->c + kBlockK - 1) / kBlockK * kBlockK;
  pack_weights_kernel<<<blocks > 0 ? blocks : 1, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      w_oihw, packed, s->cout, s->c, s->kh * s->kw, c_pad);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" size_t mcb200_conv_packed_weight_count_bf16(const mcb200_conv_shape* s) {
  const size_t c_pad = s->group > 1 ? static_cast<size_t>(grouped_c_blocks(s, kBlockKHalf, 8)) * kBlockKHalf
                                    : static_cast<size_t>((s->c + kBlockKHalf - 1) / kBlockKHalf) * kBlockKHalf;
  return static_cast<size_t>(s->cout) * s->kh * s->kw * c_pad;
}

extern "C" int mcb200_conv_pack_weights_bf16(const mcb200_conv_shape* s, const float* w_oihw, uint16_t* packed,
                                             void* stream) {
  if (!s || !w_oihw || !packed || s->group < 1 || s->c % s->group != 0 || s->cout % s->group != 0) return -1;
  const size_t total = mcb200_conv_packed_weight_count_bf16(s);
  const int threads = 256;
  const int blocks = static_cast<int>((total + threads - 1) / threads < 148 * 8 ? (total + threads - 1) / threads
                                                                                  : 148 * 8);
  if (s->group > 1) {
    pack_weights_grouped_kernel<true><<<blocks > 0 ? blocks : 1, threads, 0, static_cast<cudaStream_t>(stream)>>>(
        w_oihw, packed, s->cout, s->kh * s->kw, grouped_c_blocks(s, kBlockKHalf, 8) * kBlockKHalf, s->cout / s->group,
        s->c / s->group);
    count_launch();
    return static_cast<int>(cudaGetLastError());
  }
  const int c_pad = (s->c + kBlockKHalf - 1) / kBlockKHalf * kBlockKHalf;
  pack_weights_bf16_kernel<<<blocks > 0 ? blocks : 1, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      w_oihw, packed, s->cout, s->c, s->kh * s->kw, c_pad);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mcb200_f32_to_bf16(const float* src, uint16_t* dst, size_t count, void* stream) {
  if (!src || !dst) return -1;
  if (count == 0) return 0;
  const bool vec = ((reinterpret_cast<uintptr_t>(src) & 15) == 0) && ((reinterpret_cast<uintptr_t>(dst) & 7) == 0);
  const size_t quads = vec ? count / 4 : 0;
  const size_t items = quads + (count - quads * 4);
  const int blocks = static_cast<int>((items + 255) / 256 < 148 * 16 ? (items + 255) / 256 : 148 * 16);
  f32_to_bf16_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const float4*>(src), reinterpret_cast<uint2*>(dst), quads, src, dst, count);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mcb200_bf16_to_f32(const uint16_t* src, float* dst, size_t count, void* stream) {
  if (!src || !dst) return -1;
  if (count == 0) return 0;
  const bool vec = ((reinterpret_cast<uintptr_t>(dst) & 15) == 0) && ((reinterpret_cast<uintptr_t>(src) & 7) == 0);
  const size_t quads = vec ? count / 4 : 0;
  const size_t items = quads + (count - quads * 4);
  const int blocks = static_cast<int>((items + 255) / 256 < 148 * 16 ? (items + 255) / 256 : 148 * 16);
  bf16_to_f32_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint2*>(src), reinterpret_cast<float4*>(dst), quads, src, dst, count);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

namespace {

// Shared by the fp32 (TF32) and the bfloat16 plan: `in` and `packed_w` hold
// elements of `es` bytes, a k-iteration covers `kelems` channels (128 bytes).
int plan_core(const mcb200_conv_shape* s, const void* in, const void* packed_w, mcb200_conv_plan* plan, bool half) {
  const cuuint64_t es = half ? 2 : 4;
  const int kelems = half ? kBlockKHalf : kBlockK;
  const CUtensorMapDataType dtype = half ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  if (!s || !in || !packed_w || !plan) return -1;
  if (s->group < 1 || s->c % s->group != 0 || s->cout % s->group != 0) return -2;
  if ((s->c_stride & (half ? 7 : 3)) != 0 || s->c_stride < s->c) return -2;
  if ((reinterpret_cast<uintptr_t>(in) & 15) || (reinterpret_cast<uintptr_t>(packed_w) & 15)) return -3;
  if (s->pad_h > 127 || s->pad_w > 127 || (s->kh - 1) * s->dil_h > 255 || (s->kw - 1) * s->dil_w > 255) return -4;
  const DriverApi& api = driver_api();
  if (!api.ok) return -5;

  plan->shape = *s;
  plan->out_ptr = nullptr;
  plan->res_ptr = nullptr;
  plan->out_ld = plan->res_ld = plan->cta_pair = 0;
  plan->operand_bf16 = half ? 1 : 0;
  plan->out_bf16 = 0;
  if (mcb200_conv_out_shape(&plan->shape) != 0) return -6;
  const long long m_ll = static_cast<long long>(s->n) * plan->shape.ho * plan->shape.wo;
  if (m_ll <= 0 || m_ll > 0x7fffffffLL) return -7;
  plan->m = static_cast<int>(m_ll);
  const bool grouped = s->group > 1;
  plan->c_blocks = grouped ? grouped_c_blocks(s, kelems, half ? 8 : 4) : (s->c + kelems - 1) / kelems;
  plan->k_iters = s->kh * s->kw * plan->c_blocks;
  plan->block_n = grouped ? kGroupedBlockN : pick_block_n(s->cout, plan->m, plan->k_iters);
  // The pairing rule was measured in 32-channel k-iterations; a bfloat16 k-iteration covers 64.
  plan->cta_pair = grouped ? 0 : pick_cta_pair(plan->block_n, plan->m, plan->k_iters * (half ? 2 : 1));
  const bool pointwise = s->kh == 1 && s->kw == 1 && s->stride_h == 1 && s->stride_w == 1 && s->pad_h == 0 &&
                         s->pad_w == 0;
  plan->im2col = pointwise ? 0 : 1;
  plan->m_virtual = plan->m;
  plan->strip_rows = 0;
  // Halo mode for stride-1 filters with more than one tap per row: see ConvTcArgs.  The choice
  // depends on the layer's geometry only, never on the batch size: the two modes sum over K in
  // different orders, and an image's result must not depend on how many images run with it.
  // Measured on the benchmark networks (ResNet-50 at batch 64, per 3 x 3 layer): 56-pixel rows
  // 52.8 -> 49.8 us, 28-pixel rows 37.1 -> 33.4, 7-pixel rows 43.0 -> 37.3, but 14-pixel rows 35.3
  // -> 43.3: there every CTA has a single 256-column tile, and the halo mode's epilogue (plain
  // stores, since a tile of the virtual grid is not a box of the output tensor) is exposed where
  // the im2col mode's TMA tile stores are half as long (37.2 against 35.5 us once the mode kept to
  // 128-column tiles).  SSD300 at batch 32, 512 -> 512 on 19-pixel rows: 102 -> 82 us, the two
  // detection heads on the same map 84 -> 69 and 66 -> 63; on its 10-pixel rows 36 -> 38.  Hence:
  // rows of at least 16 output pixels or at most 8 (the strips save the most), and never when the
  // widened rows would cost more than half again as many positions.
  const int halo_w = (s->kw - 1) * s->dil_w;
  const char* halo_env = getenv("MCB200_HALO");   // "0" / "1": override for experiments and tests
  const bool halo_forced = halo_env && halo_env[0] == '1';
  const bool halo_pays = 2 * halo_w <= plan->shape.wo && (plan->shape.wo >= 16 || plan->shape.wo <= 8);
  if (!pointwise && s->stride_h == 1 && s->stride_w == 1 && s->kw > 1 && halo_w <= kMaxHaloRows &&
      !(halo_env && halo_env[0] == '0') && (halo_forced || halo_pays)) {
    const long long mv = static_cast<long long>(s->n) * plan->shape.ho * (plan->shape.wo + halo_w);
    const int halo_k_iters = s->kh * plan->c_blocks;
    int pair = 0;
    // (grouped layers keep their 64-column tiles: a strip and kw weight tiles of that width always fit)
    const int bn = mv > 0x7fffffffLL ? 0
                   : grouped         ? (s->kw <= 7 ? kGroupedBlockN : 0)
                                     : pick_block_n_halo(s->cout, mv, halo_k_iters, s->kw, (kBlockM + halo_w) * 128, &pair,
                                                         nullptr);
    if (bn != 0) {
      plan->im2col = kModeHalo;
      plan->m_virtual = static_cast<int>(mv);
      plan->strip_rows = kBlockM + halo_w;
      plan->k_iters = halo_k_iters;
      plan->block_n = bn;
      plan->cta_pair = pair;
    }
  }
  const bool halo = plan->im2col == kModeHalo;

  CUtensorMap* ma = reinterpret_cast<CUtensorMap*>(plan->tma_a);
  CUtensorMap* mb = reinterpret_cast<CUtensorMap*>(plan->tma_b);
  CUresult r;
  if (pointwise) {
    // Plain row-major matrix [m, c] with row pitch c_stride.
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(s->c), static_cast<cuuint64_t>(plan->m)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(s->c_stride) * es};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(kelems), kBlockM};
    const cuuint32_t estr[2] = {1, 1};
    r = api.tiled(ma, dtype, 2, const_cast<void*>(in), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  } else {
    const cuuint64_t dims[4] = {static_cast<cuuint64_t>(s->c), static_cast<cuuint64_t>(s->w),
                                static_cast<cuuint64_t>(s->h), static_cast<cuuint64_t>(s->n)};
    const cuuint64_t pix = static_cast<cuuint64_t>(s->c_stride) * es;
    const cuuint64_t strides[3] = {pix, pix * s->w, pix * s->w * s->h};
    // Window of base pixels (top-left filter corners): starts at -pad and ends
    // where the last tap still lies inside the padded image.
    const int lower[2] = {-s->pad_w, -s->pad_h};
    // Halo mode walks every position of the padded row (w + 2 * pad_w of them), not only the wo
    // positions a filter's left edge can take: the extra ones are the taps' halo.
    const int upper[2] = {halo ? s->pad_w : s->pad_w - (s->kw - 1) * s->dil_w, s->pad_h - (s->kh - 1) * s->dil_h};
    const cuuint32_t estr[4] = {1, static_cast<cuuint32_t>(s->stride_w), static_cast<cuuint32_t>(s->stride_h), 1};
    r = api.im2col(ma, dtype, 4, const_cast<void*>(in), dims, strides, lower, upper,
                   static_cast<cuuint32_t>(kelems), halo ? static_cast<cuuint32_t>(plan->strip_rows) : kBlockM, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    // Drivers up to CUDA 13.1 encode a flag in im2col descriptors of tensors
    // smaller than 128 KiB that makes the load misbehave; NVIDIA's CUTLASS
    // clears it the same way (cute/atom/copy_traits_sm90_im2col.hpp).
    if (r == CUDA_SUCCESS && api.driver_version <= 13010) {
      const unsigned long long bytes = static_cast<unsigned long long>(pix) * s->w * s->h * s->n;
      if (bytes < 131072ull) reinterpret_cast<uint64_t*>(ma)[1] &= ~(1ull << 21);
    }
  }
  if (r != CUDA_SUCCESS) return -100 - static_cast<int>(r);
  {
    const cuuint64_t kp = static_cast<cuuint64_t>(s->kh) * s->kw * plan->c_blocks * kelems;
    const cuuint64_t dims[2] = {kp, static_cast<cuuint64_t>(s->cout)};
    const cuuint64_t strides[1] = {kp * es};
    // A CTA of a pair fetches half of the weight tile.
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(kelems),
                               static_cast<cuuint32_t>(plan->cta_pair ? plan->block_n / 2 : plan->block_n)};
    const cuuint32_t estr[2] = {1, 1};
    r = api.tiled(mb, dtype, 2, const_cast<void*>(packed_w), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return -200 - static_cast<int>(r);
  }
  return 0;
}

int launch_core(mcb200_conv_plan* plan, void* out, bool out_half, int out_ld, const mcb200_epilogue* ep, int* status,
                void* stream);

}  // namespace

extern "C" int mcb200_conv_tc_plan(const mcb200_conv_shape* s, const float* in, const float* packed_w,
                                   mcb200_conv_plan* plan) {
  return plan_core(s, in, packed_w, plan, false);
}

extern "C" int mcb200_conv_tc_plan_bf16(const mcb200_conv_shape* s, const uint16_t* in, const uint16_t* packed_w,
                                        mcb200_conv_plan* plan) {
  return plan_core(s, in, packed_w, plan, true);
}

extern "C" int mcb200_conv_tc_launch(mcb200_conv_plan* plan, float* out, int out_ld, const mcb200_epilogue* ep,
                                     int* status, void* stream) {
  if (plan && plan->operand_bf16) return -8;   // bfloat16 plans go through mcb200_conv_tc_launch_bf16
  return launch_core(plan, out, false, out_ld, ep, status, stream);
}

extern "C" int mcb200_conv_tc_launch_bf16(mcb200_conv_plan* plan, void* out, int out_is_bf16, int out_ld,
                                          const mcb200_epilogue* ep, int* status, void* stream) {
  return launch_core(plan, out, out_is_bf16 != 0, out_ld, ep, status, stream);
}

namespace {

int launch_core(mcb200_conv_plan* plan, void* out, bool out_half, int out_ld, const mcb200_epilogue* ep, int* status,
                void* stream) {
  if (!plan || !out || out_ld < plan->shape.cout) return -1;
  const bool half = plan->operand_bf16 != 0;
  ConvTcArgs a;
  a.out = static_cast<float*>(out);
  a.out_half = out_half ? 1 : 0;
  a.out_ld = out_ld;
  a.m = plan->m;
  a.cout = plan->shape.cout;
  a.k_iters = plan->k_iters;
  a.c_blocks = plan->c_blocks;
  a.kw = plan->shape.kw;
  a.ho = plan->shape.ho;
  a.wo = plan->shape.wo;
  a.stride_h = plan->shape.stride_h;
  a.stride_w = plan->shape.stride_w;
  a.pad_h = plan->shape.pad_h;
  a.pad_w = plan->shape.pad_w;
  a.dil_h = plan->shape.dil_h;
  a.dil_w = plan->shape.dil_w;
  if (ep) {
    a.ep = *ep;
  } else {
    a.ep = mcb200_epilogue();
    a.ep.residual_coeff = 1.f;
  }
  if (a.ep.act == 2 && !a.ep.prelu) return -2;
  a.status = status;
  // The staged epilogue needs 16-byte aligned rows; otherwise plain stores are used.
  const bool out_ok = (out_ld % (out_half ? 8 : 4) == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
  const bool res_ok = !a.ep.residual || ((a.ep.residual_ld % (half ? 8 : 4) == 0) && a.ep.residual_ld >= plan->shape.cout &&
                                         ((reinterpret_cast<uintptr_t>(a.ep.residual) & 15) == 0));
  a.tma_epilogue = (out_ok && res_ok) ? 1 : 0;
  a.vec_store = a.tma_epilogue;
  a.l2_prefetch = a.halo_staged = 0;
  a.wait_limit = g_wait_limit_cycles;
  a.drop_last_weight_load = t_drop_weight_load;
  t_drop_weight_load = 0;
  a.group_cout = plan->shape.group > 1 ? plan->shape.cout / plan->shape.group : 0;
  a.group_cin = plan->shape.group > 1 ? plan->shape.c / plan->shape.group : 0;
  a.wp = plan->shape.wo;
  a.stage_bytes = a.stage_b_offset = a.resident_b_bytes = 0;
  if (plan->im2col == kModeHalo) {
    // Tiles are pieces of the virtual output grid: results leave through plain (128-bit) stores.
    a.tma_epilogue = 0;
    a.m = plan->m_virtual;
    a.wp = plan->m_virtual / (plan->shape.n * plan->shape.ho);
  }
  if (a.tma_epilogue) {
    const bool rows = plan->im2col == kModeRows;
    const long long per_group = rows ? plan->shape.wo : plan->m;
    const long long groups = rows ? static_cast<long long>(plan->shape.n) * plan->shape.ho : 1;
    if (plan->out_ptr != out || plan->out_ld != out_ld || plan->out_bf16 != a.out_half) {
      if (encode_tile_map(reinterpret_cast<CUtensorMap*>(plan->tma_out), out, out_half, plan->shape.cout, out_ld,
                          per_group, groups) != CUDA_SUCCESS)
        return -4;
      plan->out_ptr = static_cast<const float*>(out);
      plan->out_ld = out_ld;
      plan->out_bf16 = a.out_half;
    }
    if (a.ep.residual && (plan->res_ptr != a.ep.residual || plan->res_ld != a.ep.residual_ld)) {
      if (encode_tile_map(reinterpret_cast<CUtensorMap*>(plan->tma_res), a.ep.residual, half, plan->shape.cout,
                          a.ep.residual_ld, per_group, groups) != CUDA_SUCCESS)
        return -5;
      plan->res_ptr = a.ep.residual;
      plan->res_ld = a.ep.residual_ld;
    }
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  a.tile_rows = plan->im2col == kModeRows ? (plan->shape.wo < kBlockM ? plan->shape.wo : kBlockM) : kBlockM;
  a.row_segments = plan->im2col == kModeRows ? (plan->shape.wo + a.tile_rows - 1) / a.tile_rows : 1;
  a.a_bytes = (plan->im2col == kModeHalo ? plan->strip_rows : a.tile_rows) * kBlockK * 4;
  cudaError_t e = cudaErrorInvalidValue;
  const int mode = plan->im2col;
#define MCB200_DISPATCH(BN)                                                               \
  e = mode == kModeRows     ? launch_variant<BN, kModeRows, false, false>(plan, a, st)    \
      : mode == kModeIm2col ? launch_variant<BN, kModeIm2col, false, false>(plan, a, st)  \
      : mode == kModeHalo   ? launch_variant<BN, kModeHalo, false, false>(plan, a, st)    \
                            : launch_variant<BN, kModeMatrix, false, false>(plan, a, st)
#define MCB200_DISPATCH_PAIR(BN)                                                          \
  e = mode == kModeIm2col ? launch_variant<BN, kModeIm2col, true, false>(plan, a, st)     \
      : mode == kModeHalo ? launch_variant<BN, kModeHalo, true, false>(plan, a, st)       \
                          : launch_variant<BN, kModeMatrix, true, false>(plan, a, st)
#define MCB200_DISPATCH_HALF(BN, PAIR)                                                    \
  e = mode == kModeIm2col ? launch_variant<BN, kModeIm2col, PAIR, true>(plan, a, st)      \
      : mode == kModeHalo ? launch_variant<BN, kModeHalo, PAIR, true>(plan, a, st)        \
                          : launch_variant<BN, kModeMatrix, PAIR, true>(plan, a, st)
  if (half) {
    if (mode == kModeRows) return -3;
    if (plan->cta_pair) {
      switch (plan->block_n) {
        case 128: MCB200_DISPATCH_HALF(128, true); break;
        case 256: MCB200_DISPATCH_HALF(256, true); break;
        default: return -3;
      }
    } else {
      switch (plan->block_n) {
        case 64: MCB200_DISPATCH_HALF(64, false); break;
        case 128: MCB200_DISPATCH_HALF(128, false); break;
        case 256: MCB200_DISPATCH_HALF(256, false); break;
        default: return -3;
      }
    }
    return static_cast<int>(e);
  }
  if (plan->cta_pair) {
    if (mode == kModeRows) return -3;
    switch (plan->block_n) {
      case 128: MCB200_DISPATCH_PAIR(128); break;
      case 256: MCB200_DISPATCH_PAIR(256); break;
      default: return -3;
    }
    return static_cast<int>(e);
  }
  switch (plan->block_n) {
    case 64: MCB200_DISPATCH(64); break;
    case 128: MCB200_DISPATCH(128); break;
    case 256: MCB200_DISPATCH(256); break;
    default: return -3;
  }
#undef MCB200_DISPATCH_HALF
#undef MCB200_DISPATCH_PAIR
#undef MCB200_DISPATCH
  return static_cast<int>(e);
}

}  // namespace

// ------------------------------------------------------------------ row mode (few input channels)

namespace mcb200 {
namespace {

__global__ void pack_rows_weights_kernel(const float* __restrict__ w, float* __restrict__ packed, int cout, int c,
                                         int kh, int kw) {
  const int total = cout * kh * kBlockK;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int e = i % kBlockK;          // 8 pixels x 4 channels of one filter row
    const int r = (i / kBlockK) % kh;
    const int co = i / (kBlockK * kh);
    const int sx = e >> 2, ch = e & 3;
    float v = 0.f;
    if (sx < kw && ch < c) v = round_to_tf32(w[((static_cast<size_t>(co) * c + ch) * kh + r) * kw + sx]);
    packed[i] = v;
  }
}

// (N, C<=4, H, W) -> zero-bordered channels-last copy with 4 floats per pixel.
__global__ void pad_nhwc4_kernel(const float* __restrict__ src, float4* __restrict__ dst, int n, int c, int h, int w,
                                 int pad_h, int pad_w, int hp, int wp) {
  grid_launch_dependents();   // the convolution behind this copy may set itself up meanwhile
  // (A form with one block row per padded image row and no index divisions was measured: 33.8 us
  // against 24.7 us for 64 x 3 x 224 x 224: many small blocks with three loads per thread.)
  const long long total = static_cast<long long>(n) * hp * wp;
  const size_t plane = static_cast<size_t>(h) * w;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int xp = static_cast<int>(i % wp);
    const int yp = static_cast<int>((i / wp) % hp);
    const int img = static_cast<int>(i / (static_cast<long long>(wp) * hp));
    const int x = xp - pad_w, y = yp - pad_h;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (x >= 0 && x < w && y >= 0 && y < h) {
      const float* s = src + static_cast<size_t>(img) * c * plane + static_cast<size_t>(y) * w + x;
      v.x = s[0];
      if (c > 1) v.y = s[plane];
      if (c > 2) v.z = s[2 * plane];
      if (c > 3) v.w = s[3 * plane];
    }
    dst[i] = v;
  }
}

}  // namespace
}  // namespace mcb200

extern "C" int mcb200_conv_rows_supported(const mcb200_conv_shape* s) {
  if (!s || s->group != 1 || s->c < 1 || s->c > 4 || s->kw > 8 || s->dil_w != 1) return 0;
  mcb200_conv_shape t = *s;
  if (mcb200_conv_out_shape(&t) != 0) return 0;
  return t.wo >= 1;
}

extern "C" int mcb200_conv_rows_padded_dims(const mcb200_conv_shape* s, int* hp, int* wp) {
  if (!mcb200_conv_rows_supported(s) || !hp || !wp) return -1;
  mcb200_conv_shape t = *s;
  mcb200_conv_out_shape(&t);
  *hp = t.h + 2 * t.pad_h;
  const int reach = (t.wo - 1) * t.stride_w + 8;   // the last tile row reads 8 pixels
  *wp = t.w + 2 * t.pad_w > reach ? t.w + 2 * t.pad_w : reach;
  return 0;
}

extern "C" size_t mcb200_conv_rows_packed_weight_count(const mcb200_conv_shape* s) {
  return static_cast<size_t>(s->cout) * s->kh * kBlockK;
}

extern "C" int mcb200_conv_rows_pack_weights(const mcb200_conv_shape* s, const float* w_oihw, float* packed,
                                             void* stream) {
  if (!mcb200_conv_rows_supported(s) || !w_oihw || !packed) return -1;
  const int total = s->cout * s->kh * kBlockK;
  pack_rows_weights_kernel<<<(total + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(w_oihw, packed, s->cout,
                                                                                              s->c, s->kh, s->kw);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mcb200_conv_rows_pad_input(const mcb200_conv_shape* s, const float* src_nchw, float* padded,
                                          void* stream) {
  int hp = 0, wp = 0;
  if (mcb200_conv_rows_padded_dims(s, &hp, &wp) != 0 || !src_nchw || !padded) return -1;
  if (reinterpret_cast<uintptr_t>(padded) & 15) return -2;
  const long long total = static_cast<long long>(s->n) * hp * wp;
  if (total == 0) return 0;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  pad_nhwc4_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      src_nchw, reinterpret_cast<float4*>(padded), s->n, s->c, s->h, s->w, s->pad_h, s->pad_w, hp, wp);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mcb200_conv_rows_plan(const mcb200_conv_shape* s, const float* padded_in, const float* packed_w,
                                     mcb200_conv_plan* plan) {
  if (!padded_in || !packed_w || !plan) return -1;
  int hp = 0, wp = 0;
  if (mcb200_conv_rows_padded_dims(s, &hp, &wp) != 0) return -2;
  if ((reinterpret_cast<uintptr_t>(padded_in) & 15) || (reinterpret_cast<uintptr_t>(packed_w) & 15)) return -3;
  const DriverApi& api = driver_api();
  if (!api.ok) return -5;
  plan->shape = *s;
  plan->shape.c_stride = 4;
  plan->out_ptr = nullptr;
  plan->res_ptr = nullptr;
  plan->out_ld = plan->res_ld = plan->cta_pair = 0;
  plan->operand_bf16 = plan->out_bf16 = 0;
  if (mcb200_conv_out_shape(&plan->shape) != 0) return -6;
  const long long m_ll = static_cast<long long>(s->n) * plan->shape.ho * plan->shape.wo;
  if (m_ll <= 0 || m_ll > 0x7fffffffLL) return -7;
  plan->m = static_cast<int>(m_ll);
  plan->m_virtual = plan->m;
  plan->strip_rows = 0;
  plan->c_blocks = 1;
  plan->k_iters = s->kh;
  plan->block_n = pick_block_n(s->cout, plan->m, plan->k_iters);
  plan->im2col = kModeRows;
  // (Measured and dropped: a strip form that sorts the padded row into stride_w planes, loads a
  // filter row's pixels once (four to seven times fewer bytes out of L2) and lets the tensor core
  // read the windows through un-swizzled descriptors, rows 16 bytes apart.  Same values, but an
  // MMA with an un-swizzled operand occupied its issuing thread 76 cycles instead of 21, a 7 x 7
  // stride-2 first layer at batch 64 took 135 us instead of 106, and even the runtime switch
  // between the two forms cost the single-thread loops 100 cycles per filter row.)
  // Activation view: 32 floats (8 pixels x 4 channels) starting at padded pixel q * stride_w of padded row y.
  // Consecutive q overlap (the pitch of dimension 1 is stride_w pixels, less than the 8-pixel extent).
  CUtensorMap* ma = reinterpret_cast<CUtensorMap*>(plan->tma_a);
  const cuuint64_t dims[4] = {kBlockK, static_cast<cuuint64_t>(plan->shape.wo), static_cast<cuuint64_t>(hp),
                              static_cast<cuuint64_t>(s->n)};
  const cuuint64_t strides[3] = {static_cast<cuuint64_t>(s->stride_w) * 16, static_cast<cuuint64_t>(wp) * 16,
                                 static_cast<cuuint64_t>(wp) * 16 * hp};
  // One M tile = up to 128 output pixels of a row; wider rows are cut into segments.
  const cuuint32_t box[4] = {kBlockK, static_cast<cuuint32_t>(plan->shape.wo < kBlockM ? plan->shape.wo : kBlockM), 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = api.tiled(ma, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(padded_in), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -100 - static_cast<int>(r);
  CUtensorMap* mb = reinterpret_cast<CUtensorMap*>(plan->tma_b);
  const cuuint64_t kp = static_cast<cuuint64_t>(plan->k_iters) * kBlockK;
  const cuuint64_t bdims[2] = {kp, static_cast<cuuint64_t>(s->cout)};
  const cuuint64_t bstrides[1] = {kp * 4};
  const cuuint32_t bbox[2] = {kBlockK, static_cast<cuuint32_t>(plan->block_n)};
  const cuuint32_t bestr[2] = {1, 1};
  r = api.tiled(mb, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(packed_w), bdims, bstrides, bbox, bestr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -200 - static_cast<int>(r);
  return 0;
}

// With -DMCB200_CONV_TRACE: copies the cycle stamps of the last traced launches' CTA 0 (5 roles x
// 2048 slots, see MCB200_TRACE above) to `out` and clears the device array; returns the number
// of values per role, or 0 when the library was built without the trace.
extern "C" int mcb200_conv_trace_read(long long* out) {
#ifdef MCB200_CONV_TRACE
  if (!out) return -1;
  if (cudaDeviceSynchronize() != cudaSuccess) return -2;
  if (cudaMemcpyFromSymbol(out, mcb200::g_conv_trace, sizeof(long long) * mcb200::kTraceRoles * mcb200::kTraceSlots) !=
      cudaSuccess)
    return -3;
  static long long zeros[mcb200::kTraceRoles * mcb200::kTraceSlots];
  if (cudaMemcpyToSymbol(mcb200::g_conv_trace, zeros, sizeof(zeros)) != cudaSuccess) return -4;
  return mcb200::kTraceSlots;
#else
  (void)out;
  return 0;
#endif
}
