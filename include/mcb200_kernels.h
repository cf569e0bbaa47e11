/*
 * Kernel-level C ABI of the B200 forward engine: plain device pointers, sizes
 * and a stream; no C++ or framework types.  These are the launchers the layer
 * classes inside libcaffe.so call, exported so that each kernel can be
 * parity-tested and timed on its own.  Every pointer is a device pointer
 * unless it says "host".  `stream` is a cudaStream_t passed as void*.
 *
 * Functions return 0 on success, a negative value for a rejected argument,
 * or a positive cudaError_t.  Kernels that wait on hardware barriers report a
 * timed-out wait by writing a non-zero code to the int `*status` points at
 * (device memory, may be NULL); they never spin without a limit.
 *
 * Each entry point cites the mini-caffe function whose arithmetic it
 * replaces (paths relative to that project).
 */
#ifndef MCB200_KERNELS_H_
#define MCB200_KERNELS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ layout
 * Activations inside the engine are channels-last: element (n, y, x, c) of a
 * tensor lives at ((n*H + y)*W + x)*c_stride + c, with c_stride >= C and
 * c_stride % 4 == 0 for the tensor-core path.  Blobs at the API boundary are
 * NCHW; mcb200_nchw_to_nhwc / mcb200_nhwc_to_nchw convert.                  */

typedef struct mcb200_conv_shape {
  int n, h, w, c;          /* input extent                                   */
  int c_stride;            /* allocated channels per input pixel             */
  int cout;                /* output channels                                */
  int kh, kw;
  int stride_h, stride_w;
  int pad_h, pad_w;
  int dil_h, dil_w;
  int group;               /* 1, or c (depthwise); other values: direct path */
  int ho, wo;              /* output extent (filled by mcb200_conv_out_shape) */
} mcb200_conv_shape;

/* Fused tail applied to each accumulator before it is stored:
 *   v = acc * scale[co] + shift[co]        (either array may be NULL)
 *   v += residual_coeff * residual[m*residual_ld + co]   (if residual != NULL)
 *   v = v > 0 ? v : v * slope              (act == 1; slope 0 is plain ReLU)
 *   v = v > 0 ? v : v * prelu[co or 0]     (act == 2)
 * It replaces the separate in-place passes of BatchNormLayer, ScaleLayer,
 * BiasLayer, EltwiseLayer(SUM) and ReLU/PReLULayer
 * (src/layers/batch_norm_layer.cpp:72-136, scale_layer.cpp:96-113,
 *  eltwise_layer.cpp:51-57, relu_layer.cpp:12-29, prelu_layer.cpp:52-84).   */
typedef struct mcb200_epilogue {
  const float* scale;
  const float* shift;
  const float* residual;
  int residual_ld;
  float residual_coeff;
  int act;                 /* 0 none, 1 (leaky) ReLU, 2 PReLU                 */
  float slope;
  const float* prelu;
  int prelu_shared;        /* PReLU: one slope for all channels               */
  int round_tf32;          /* round stored values to TF32 (next op is a conv) */
} mcb200_epilogue;

/* Output extent of a convolution: floor((in + 2p - (d(k-1)+1)) / s) + 1
 * (src/layers/conv_layer.cpp:12-25).  Returns -1 if the window does not fit. */
int mcb200_conv_out_shape(mcb200_conv_shape* s);

/* Number of floats of the packed tensor-core weight image for `s`:
 * cout rows of kh*kw taps, each tap padded to a multiple of 32 channels.     */
size_t mcb200_conv_packed_weight_count(const mcb200_conv_shape* s);

/* Re-lay Caffe weights [cout, c, kh, kw] (src/layers/base_conv_layer.cpp:98-104)
 * as [cout][kh*kw][roundup(c,32)], rounded to TF32 (round-to-nearest).       */
int mcb200_conv_pack_weights(const mcb200_conv_shape* s, const float* w_oihw, float* packed, void* stream);

/* Opaque-to-C plan: two TMA descriptors and the launch geometry.  Valid while
 * `in`, `packed_w` stay where they are.  Host memory, 64-byte aligned.       */
typedef struct mcb200_conv_plan {
  uint64_t tma_a[16];
  uint64_t tma_b[16];
  uint64_t tma_out[16];     /* output / residual tile maps, built on first launch  */
  uint64_t tma_res[16];     /* and rebuilt when the pointers below change          */
  mcb200_conv_shape shape;
  int m, k_iters, c_blocks, block_n;
  int im2col;               /* 0 matrix rows, 1 im2col tensor map, 2 row mode, 3 halo mode (the taps
                               of a filter row share one strip of input pixels)   */
  int out_ld, res_ld;
  int cta_pair;             /* 1: launched as two-CTA clusters (tcgen05 cta_group::2) */
  int operand_bf16;         /* 1: built by mcb200_conv_tc_plan_bf16                 */
  int out_bf16;             /* element type the cached output tile map was built for */
  const float* out_ptr;
  const float* res_ptr;
  int m_virtual;            /* halo mode: positions of the virtual output grid (rows widened by
                               (kw - 1) * dil_w); else m                            */
  int strip_rows;           /* halo mode: pixels per activation load (128 + (kw - 1) * dil_w) */
} __attribute__((aligned(64))) mcb200_conv_plan;

/* Implicit-GEMM convolution on the tensor cores (tcgen05.mma kind::tf32,
 * accumulators in tensor memory, operands fetched by TMA; activations through
 * an im2col-mode tensor map so no column buffer exists).  group must be 1 and
 * c_stride % 4 == 0.  Replaces im2col_cpu + caffe_cpu_gemm + forward_cpu_bias
 * (src/layers/base_conv_layer.cpp:254-278, src/util/im2col.cpp:19-55).
 * InnerProduct is the same call with h = w = kh = kw = 1
 * (src/layers/inner_product_layer.cpp:80-93).                                */
int mcb200_conv_tc_plan(const mcb200_conv_shape* s, const float* in, const float* packed_w,
                        mcb200_conv_plan* plan);
/* The plan is updated in place when `out` / the residual pointer differ from
 * the previous launch (their tile maps are cached in it).                     */
int mcb200_conv_tc_launch(mcb200_conv_plan* plan, float* out, int out_ld,
                          const mcb200_epilogue* ep, int* status, void* stream);

/* Every wait of the convolution kernel on a hardware barrier is bounded: after `cycles` SM clock
 * cycles (default 2e9, about a second) the CTA raises an abort flag, its roles leave their loops,
 * copies in flight get a bounded grace period, tensor memory is freed and *status is set to 1;
 * the launch returns normally and the context stays usable.  Sets the bound for later launches
 * of the process and returns the previous one (cycles <= 0 restores the default).
 * (No counterpart in mini-caffe, whose kernels have no device-side waits.)                     */
long long mcb200_conv_set_wait_limit(long long cycles);
/* Test hook: in the calling thread's next convolution launch the weight producer leaves out the
 * loads of the last k-iteration of its last tile, so that nothing ever completes that stage's
 * barrier and the bounded waits above run out.  This is how the abort path is exercised
 * without faulting, trapping or hanging anything; combine with a short wait limit.            */
void mcb200_conv_test_drop_weight_load(void);

/* bfloat16 storage (opt-in; the reference computes in fp32 throughout, so these
 * have no counterpart there).  Activations, the packed weights and the residual
 * are bfloat16, the tensor cores run tcgen05.mma kind::f16 with fp32
 * accumulation, the fused tail is evaluated in fp32 and the result is stored
 * as bfloat16 (out_is_bf16 != 0) or fp32.  c_stride % 8 == 0; `ep->residual`
 * is read as a bfloat16 pointer with `residual_ld` in elements.  Weights:
 * [cout][kh*kw][roundup(c,64)] bfloat16, round to nearest even.
 * mcb200_conv_tc_launch_bf16 also takes plans of the fp32 entry points
 * (mcb200_conv_tc_plan, mcb200_conv_rows_plan): fp32 operands and residual,
 * TF32 tensor cores, result stored as bfloat16 or fp32.                       */
size_t mcb200_conv_packed_weight_count_bf16(const mcb200_conv_shape* s);
int mcb200_conv_pack_weights_bf16(const mcb200_conv_shape* s, const float* w_oihw, uint16_t* packed, void* stream);
int mcb200_conv_tc_plan_bf16(const mcb200_conv_shape* s, const uint16_t* in, const uint16_t* packed_w,
                             mcb200_conv_plan* plan);
int mcb200_conv_tc_launch_bf16(mcb200_conv_plan* plan, void* out, int out_is_bf16, int out_ld,
                               const mcb200_epilogue* ep, int* status, void* stream);
/* Element-wise copies between an fp32 and a bfloat16 tensor of `count` elements. */
int mcb200_f32_to_bf16(const float* src, uint16_t* dst, size_t count, void* stream);
int mcb200_bf16_to_f32(const uint16_t* src, float* dst, size_t count, void* stream);

/* "Row mode" of the same kernel for layers with at most four input channels (the
 * first layer of an image network), where 32-channel blocks would be almost all
 * padding: the input is copied once into a zero-bordered channels-last image
 * with 4 floats per pixel (mcb200_conv_rows_pad_input), and one k-iteration then
 * covers a whole filter row: 8 neighbouring pixels x 4 channels = one 128-byte
 * row per output pixel, fetched by a tiled tensor map whose pixel pitch is the
 * convolution stride.  An M tile is one output row of one image, or a segment of
 * 128 pixels of it when the row is wider.  Requires kw <= 8 and dil_w == 1.
 *   padded copy: [n, hp, wp, 4] floats with (hp, wp) from mcb200_conv_rows_padded_dims
 *   weights:     [cout][kh][8 * 4] via mcb200_conv_rows_pack_weights
 * Launch with mcb200_conv_tc_launch.                                            */
int mcb200_conv_rows_supported(const mcb200_conv_shape* s);
int mcb200_conv_rows_padded_dims(const mcb200_conv_shape* s, int* hp, int* wp);
size_t mcb200_conv_rows_packed_weight_count(const mcb200_conv_shape* s);
int mcb200_conv_rows_pack_weights(const mcb200_conv_shape* s, const float* w_oihw, float* packed, void* stream);
int mcb200_conv_rows_pad_input(const mcb200_conv_shape* s, const float* src_nchw, float* padded, void* stream);
int mcb200_conv_rows_plan(const mcb200_conv_shape* s, const float* padded_in, const float* packed_w,
                          mcb200_conv_plan* plan);

/* Direct convolution, one thread per output element, any group count; the
 * fallback for shapes the tensor-core path rejects.  Weights stay in Caffe
 * order [cout, c/group, kh, kw].                                             */
int mcb200_conv_direct(const mcb200_conv_shape* s, const float* in, const float* w_oihw, float* out,
                       int out_ld, const mcb200_epilogue* ep, void* stream);

/* Depthwise convolution (group == c == cout), channels-last, four channels per
 * thread; weights re-laid as [kh*kw][c] by mcb200_dw_pack_weights.  HBM-bound.
 * Replaces ConvolutionDepthwiseLayer::Forward_cpu (src/layers/conv_dw_layer.cpp:104-152)
 * and the per-group M=1 GEMMs of the generic path (base_conv_layer.cpp:265-270). */
int mcb200_dw_pack_weights(const mcb200_conv_shape* s, const float* w_oihw, float* packed, void* stream);
int mcb200_conv_depthwise(const mcb200_conv_shape* s, const float* in, const float* packed_w, float* out,
                          const mcb200_epilogue* ep, void* stream);

/* The same layer for 3 x 3 filters, dilation 1, stride 1 or 2, fp32 in and out, with the input
 * staged in shared memory by TMA (tiles of 8 x 16 output pixels x 32 channels, zero fill outside
 * the image, two boxes per CTA in flight): what a CTA has in flight no longer depends on its
 * registers.  `status` (device int, may be NULL) is set to 1 if a bounded wait on a box runs out.
 * No fused residual (mcb200_conv_depthwise takes those).  Replaces the same reference code,
 * src/layers/conv_dw_layer.cpp:104-152.                                                  */
int mcb200_conv_depthwise_tma_supported(const mcb200_conv_shape* s);
int mcb200_conv_depthwise_tma(const mcb200_conv_shape* s, const float* in, const float* packed_w, float* out,
                              const mcb200_epilogue* ep, int* status, void* stream);
/* The 3x3 (dilation 1, stride 1 or 2) case with bfloat16 activations on either
 * side, for nets that store their activations as bfloat16: `in` / `out` hold
 * bfloat16 cells when the matching flag is set, fp32 otherwise; weights and
 * arithmetic are fp32.  No fused residual.                                    */
int mcb200_conv_depthwise_bf16_supported(const mcb200_conv_shape* s);
int mcb200_conv_depthwise_bf16(const mcb200_conv_shape* s, const void* in, int in_is_bf16, const float* packed_w,
                               void* out, int out_is_bf16, const mcb200_epilogue* ep, void* stream);

/* ------------------------------------------------------------------ layout */
/* (N,C,H,W) -> (N,H,W,c_stride) with channels c..c_stride-1 zero-filled, and back. */
int mcb200_nchw_to_nhwc(const float* src, float* dst, int n, int c, int h, int w, int c_stride, void* stream);
int mcb200_nhwc_to_nchw(const float* src, float* dst, int n, int c, int h, int w, int c_stride, void* stream);

/* ------------------------------------------------------------------ elementwise */
/* y[i] = act(x[i] * scale[ch] + shift[ch]),  ch = (i / inner) % channels.
 * inner = H*W for (N,C,H,W) data, 1 for channels-last data.  scale / shift may
 * be NULL.  `ep` supplies act / slope / prelu only.  Stand-alone form of
 * BatchNorm, Scale, Bias, ReLU and PReLU (src/layers/batch_norm_layer.cpp:72-136,
 * scale_layer.cpp:96-113, bias_layer.cpp:68-83, relu_layer.cpp:12-29,
 * prelu_layer.cpp:52-84) for when they cannot be fused into a producer.      */
int mcb200_channel_affine_act(const float* x, float* y, long long count, int channels, int inner,
                              const float* scale, const float* shift, const mcb200_epilogue* ep, void* stream);

#define MCB200_ELTWISE_PROD 0
#define MCB200_ELTWISE_SUM 1
#define MCB200_ELTWISE_MAX 2
#define MCB200_MAX_ELTWISE_INPUTS 8
/* out = op over the inputs (SUM uses coeffs), then the optional activation.
 * EltwiseLayer::Forward_cpu, src/layers/eltwise_layer.cpp:37-78.             */
int mcb200_eltwise(int op, int num_inputs, const float* const* inputs, const float* coeffs, float* out,
                   long long count, int act, float slope, void* stream);

/* ------------------------------------------------------------------ pooling */
#define MCB200_POOL_MAX 0
#define MCB200_POOL_AVE 1
/* Output extent with Caffe's ceil rule and last-window clip
 * (src/layers/pooling_layer.cpp:92-107).                                     */
void mcb200_pool_out_shape(int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int* ho, int* wo);
/* Channels-last pooling.  MAX starts from -FLT_MAX over the window clipped to
 * the image; AVE sums the clipped window and divides by the window area clipped
 * to the padded image (src/layers/pooling_layer.cpp:124-181).                */
int mcb200_pool_nhwc(const float* in, float* out, int n, int h, int w, int c, int kh, int kw, int sh, int sw,
                     int ph, int pw, int ho, int wo, int method, void* stream);
/* MAX pooling with a 2x2 or 3x3 window over a bfloat16 channels-last tensor
 * (c % 8 == 0), for nets that store their activations as bfloat16: equal to
 * pooling the fp32 tensor and rounding the result.                           */
int mcb200_pool_max_nhwc_bf16_supported(int c, int kh, int kw);
int mcb200_pool_max_nhwc_bf16(const uint16_t* in, uint16_t* out, int n, int h, int w, int c, int kh, int kw,
                              int sh, int sw, int ph, int pw, int ho, int wo, void* stream);

/* ------------------------------------------------------------------ softmax */
/* Softmax over `channels` of data viewed as [outer, channels, inner]
 * (src/layers/softmax_layer.cpp:29-63): subtract the max, exp, divide by the sum. */
int mcb200_softmax(const float* in, float* out, int outer, int channels, int inner, void* stream);

/* ------------------------------------------------------------------ copies */
/* rows x cols floats from a pitched source to a pitched destination (pitches
 * in floats).  Concat / Slice style block copies (src/layers/concat_layer.cpp:53-70). */
int mcb200_copy_2d(const float* src, long long src_pitch, float* dst, long long dst_pitch, long long rows,
                   long long cols, void* stream);
/* out[permuted index] = in[index] for up to 6 axes; order[i] is the input axis
 * that becomes output axis i (src/layers/permute_layer.cpp:8-22).           */
int mcb200_permute(const float* in, float* out, int num_axes, const int* in_shape, const int* order, void* stream);
/* Per pixel L2 normalisation across channels of channels-last data, times a
 * per-channel (or single) scale: y = x / sqrt(sum_c x^2 + eps) * scale[c]
 * (src/layers/normalize_layer.cpp:86-135 with across_spatial = false).       */
int mcb200_normalize_nhwc(const float* in, float* out, long long pixels, int channels, const float* scale,
                          int scale_shared, float eps, void* stream);

/* ------------------------------------------------------------------ RPN proposals */
typedef struct mcb200_proposal_params {
  int num_anchors, height, width;  /* score map [2A, H, W], delta map [4A, H, W] per image */
  int feat_stride;
  int min_size;                    /* multiplied by im_info[2] on the device            */
  int pre_nms_topn, post_nms_topn;
  float nms_thresh;
} mcb200_proposal_params;

/* Bytes of device scratch mcb200_proposal_forward needs for `batch` images
 * (0 if the parameters are rejected; pre_nms_topn is limited to 16384).      */
size_t mcb200_proposal_workspace_bytes(const mcb200_proposal_params* p, int batch);

/* ProposalLayer::Forward_cpu (src/layers/proposal_layer.cpp:261-320) for `batch`
 * independent images: decode anchors + deltas, clip, zero the score of boxes
 * below min_size, take the pre_nms_topn best by score, greedy NMS with the "+1
 * pixel" IoU, keep at most post_nms_topn.
 *   scores   [batch, 2A, H, W]   (foreground = channels A..2A-1)
 *   deltas   [batch, 4A, H, W]
 *   im_info  [batch, 3]          (height, width, scale)
 *   anchors  [A, 4]              base anchors (x1, y1, x2, y2)
 *   rois     [batch, post_nms_topn, 5]  rows (image index, x1, y1, x2, y2); the
 *            first counts[b] rows of image b are valid
 *   roi_scores [batch, post_nms_topn] or NULL
 *   counts   [batch] ints (device)
 * `workspace` must be 256-byte aligned.  Kept boxes match the CPU code bit for
 * bit when no two scores among the pre_nms_topn best are equal (equal scores
 * are ordered by proposal index here; the CPU order is unspecified).         */
int mcb200_proposal_forward(const mcb200_proposal_params* p, int batch, const float* scores, const float* deltas,
                            const float* im_info, const float* anchors, void* workspace, float* rois,
                            float* roi_scores, int* counts, void* stream);

/* Closes the gaps between the images' row blocks of a batched
 * mcb200_proposal_forward result in place: image b's counts[b] valid rows move
 * from row b * post_nms_topn to row counts[0] + ... + counts[b-1] (rois and,
 * when not NULL, roi_scores).  One kernel; source and destination ranges may
 * overlap.  (mini-caffe's layer takes one image per call,
 * src/layers/proposal_layer.cpp:269, and so has nothing to compact.)           */
int mcb200_proposal_compact(float* rois, float* roi_scores, const int* counts, int batch, int post_nms_topn,
                            void* stream);

/* The same computation as mcb200_proposal_forward for callers that cannot
 * allocate device memory.  (It has no counterpart in mini-caffe.)
 *
 * Who needs it: code that runs inside a host program which has already handed
 * all device memory to its own pool, so that a cudaMalloc of the workspace
 * would fail or fight with that pool; and latency-critical loops that must not
 * hit the device-wide synchronisation a cudaMalloc / cudaFree implies.  Such
 * callers still own their inputs and outputs; only the scratch is taken off
 * their hands.
 *
 * The scratch is a fixed 8 MiB array inside the library's device image (each
 * GPU that loads the library holds it until the process exits).  The largest
 * single image the kernels accept (65536 proposals, pre_nms_topn 6000) takes
 * 1.9 MB of it, an image of the stock R-FCN setting (63 x 38 map, 15 anchors)
 * 1.1 MB, and a batch takes that many times as much; a request that needs more
 * than 8 MiB returns -20 and prints the required size.  The function calls no cudaMalloc, cudaFree
 * or any other allocating routine.
 *
 * The first call on each device looks up the array's device address
 * (cudaGetSymbolAddress) and keeps it; make that first call (or a call of
 * mcb200_proposal_static_warmup, below) before starting any stream capture and
 * before the host takes the rest of the device memory.  All calls share the one array: two calls whose kernels may
 * overlap on the GPU (different streams, or different host threads without
 * ordering) race on it -- serialise them.  Nothing in the array needs to be
 * zero on entry, it is not cleared, and it keeps the last call's contents.     */
int mcb200_proposal_forward_static(const mcb200_proposal_params* p, int batch, const float* scores,
                                   const float* deltas, const float* im_info, const float* anchors, float* rois,
                                   float* roi_scores, int* counts, void* stream);

/* Does what the first call of mcb200_proposal_forward_static on the current
 * device would do besides computing: loads the library's device code (with
 * CUDA's default lazy loading that is the moment the driver sets the 8 MiB
 * array aside, and it synchronises the device), looks up the array's address
 * and opts the kernels into their shared-memory size.  Launches nothing.  A
 * host that is about to give all device memory to its own pool, or that must
 * keep such one-time work out of a latency-critical loop, calls this first,
 * once per device; without it the first mcb200_proposal_forward_static call
 * does the same work and can fail with an out-of-memory error if no device
 * memory is left by then.  (No counterpart in mini-caffe.)                      */
int mcb200_proposal_static_warmup(void);

/* ------------------------------------------------------------------ SSD detection output */
typedef struct mcb200_detout_params {
  int num_priors, num_classes;
  int share_location;              /* 1: one box per prior for all classes              */
  int background_label_id;         /* skipped class, -1 for none                        */
  int code_type;                   /* 1 CORNER, 2 CENTER_SIZE, 3 CORNER_SIZE            */
  int variance_encoded_in_target;
  float confidence_threshold;
  float nms_threshold;
  float eta;                       /* < 1: the NMS threshold shrinks by eta per kept box while above 0.5 */
  int top_k;                       /* per class, -1: all priors (at most 4096 here)     */
  int keep_top_k;                  /* per image, -1: unlimited                          */
} mcb200_detout_params;

size_t mcb200_detout_workspace_bytes(const mcb200_detout_params* p, int batch);
/* Rows per image the output buffer must hold. */
int mcb200_detout_max_rows_per_image(const mcb200_detout_params* p);

/* DetectionOutputLayer::Forward_cpu (src/layers/detection_output_layer.cpp:74-226
 * with ApplyNMSFast / DecodeBBox / JaccardOverlap of src/util/bbox_util.cpp):
 *   loc    [batch, num_priors * (share_location ? 1 : num_classes) * 4]
 *   conf   [batch, num_priors * num_classes]     (prior-major)
 *   prior  [2, num_priors * 4]                   (boxes, then variances)
 *   out    [batch * max_rows_per_image, 7] rows (image, label, score, xmin, ymin,
 *          xmax, ymax), images in order, labels ascending within an image, score
 *          descending within a label; *total (device int) receives the row count.
 * top_k (or num_priors when top_k is -1) may be at most 4096.                */
int mcb200_detout_forward(const mcb200_detout_params* p, int batch, const float* loc, const float* conf,
                          const float* prior, void* workspace, float* out, int* total, void* stream);

/* ROIPooling: max over an adaptive pooled_h x pooled_w grid laid on each region
 * of interest (src/layers/roi_pooling_layer.cpp:37-109).  data_nchw is
 * [batch, channels, height, width]; rois is [num_rois, 5] = (batch index, x1, y1,
 * x2, y2) in image coordinates; out is [num_rois, channels, pooled_h, pooled_w].
 * Bit-identical to the reference's CPU result.  A roi whose batch index is
 * outside [0, batch) (a CHECK failure in the reference) yields zeros and sets
 * *status to 3 when status is not null.                                       */
int mcb200_roi_pool(const float* data_nchw, const float* rois, float* out, int num_rois, int batch, int channels,
                    int height, int width, int pooled_h, int pooled_w, float spatial_scale, int* status,
                    void* stream);

/* PSROIPooling: position-sensitive average pooling of R-FCN
 * (src/layers/psroi_pooling_layer.cpp:45-106).  data_nchw is
 * [batch, output_dim * group_size^2, height, width]; out is
 * [num_rois, output_dim, group_size, group_size]; bin (ph, pw) of output channel
 * c averages score map (c * group_size + ph) * group_size + pw over the bin,
 * summing in the reference's row-major order (bit-identical).                 */
int mcb200_psroi_pool(const float* data_nchw, const float* rois, float* out, int num_rois, int batch,
                      int output_dim, int group_size, int height, int width, float spatial_scale, int* status,
                      void* stream);

/* Deconvolution (transposed convolution), (N, C, H, W) in and out, fp32 FMA
 * arithmetic, one thread per output element.  `s` describes the input (n, c, h,
 * w) and the filter; mcb200_deconv_out_shape fills ho = stride*(h-1) +
 * dil*(kh-1) + 1 - 2*pad (src/layers/deconv_layer.cpp:7-25).  Weights are
 * [c, cout/group, kh, kw] as Caffe stores them for this layer; bias may be null.
 * Replaces backward_cpu_gemm + col2im + forward_cpu_bias
 * (src/layers/deconv_layer.cpp:27-44, src/layers/base_conv_layer.cpp:280-296). */
int mcb200_deconv_out_shape(mcb200_conv_shape* s);
int mcb200_deconv_direct(const mcb200_conv_shape* s, const float* in_nchw, const float* w_iohw, const float* bias,
                         float* out_nchw, void* stream);

/* Deconvolution on the tensor-core convolution kernel.  A transposed convolution with stride s
 * is the stride-1 convolution, with the filter's taps reversed and padding dil*(k-1) - pad, of the
 * input with its pixels spread s apart over zeros (what col2im's scatter-add computes, read from
 * the output's side; src/layers/deconv_layer.cpp:27-44, src/util/im2col.cpp:57-90).
 *   mcb200_deconv_as_conv_shape  the equivalent convolution's shape (input = the spread tensor,
 *                                c_stride = c rounded up to 4); -3 when pad exceeds dil*(k-1)
 *   mcb200_deconv_spread_input   channels-last input (c floats per pixel) -> the spread tensor
 *   mcb200_deconv_flip_weights   [c, cout/g, kh, kw] -> [cout, c/g, kh, kw], taps reversed
 * followed by mcb200_conv_pack_weights / mcb200_conv_tc_plan / mcb200_conv_tc_launch on that
 * shape (groups included).                                                              */
int mcb200_deconv_as_conv_shape(const mcb200_conv_shape* deconv, mcb200_conv_shape* conv);
int mcb200_deconv_spread_input(const mcb200_conv_shape* deconv, const float* in_nhwc, float* spread, void* stream);
int mcb200_deconv_flip_weights(const mcb200_conv_shape* deconv, const float* w_iohw, float* w_oihw, void* stream);

/* Crop: out[idx] = in[idx + offsets] over up to six axes
 * (src/layers/crop_layer.cpp:57-100).                                         */
int mcb200_crop(const float* in, float* out, int num_axes, const int* in_shape, const int* out_shape,
                const int* offsets, void* stream);

/* Local response normalisation over (N, C, H, W).  within_channel == 0:
 * y = x * (k + alpha/size * sum of x^2 over `size` neighbouring channels)^-beta
 * (src/layers/lrn_layer.cpp:107-150); within_channel == 1:
 * y = x * (1 + alpha * mean of x^2 over a size x size window)^-beta, the mean
 * taken like the reference's padded AVE pooling (src/layers/lrn_layer.cpp:19-66). */
int mcb200_lrn(const float* in_nchw, float* out_nchw, int n, int c, int h, int w, int local_size, float alpha,
               float beta, float k, int within_channel, void* stream);

/* BatchNorm with statistics of the current batch (use_global_stats: false, as
 * the shipped WGAN generator runs it): per channel, mean and variance over all
 * images and pixels, written as the scale = 1 / sqrt(var + eps) and shift =
 * -mean * scale of mcb200_channel_affine_act (src/layers/batch_norm_layer.cpp:91-135).
 * Element (image, channel, position) lives at ((image * channels + channel) *
 * inner + position); inner = 1 for channels-last data.                         */
int mcb200_channel_batch_stats(const float* x, long long count, int channels, int inner, float eps, float* scale,
                               float* shift, void* stream);

/* y = tanh(x) or y = 1 / (1 + exp(-x)), elementwise, any layout
 * (src/layers/tanh_layer.cpp:10-18, src/layers/sigmoid_layer.cpp:10-22).      */
#define MCB200_UNARY_TANH 0
#define MCB200_UNARY_SIGMOID 1
int mcb200_unary(const float* x, float* y, long long count, int op, void* stream);

/* Number of kernels launched by this library on the calling thread since the
 * last reset (bench.py reports it as gpu_launches).                          */
long long mcb200_launch_count(void);
void mcb200_launch_count_reset(void);

#ifdef __cplusplus
}
#endif

#endif /* MCB200_KERNELS_H_ */
