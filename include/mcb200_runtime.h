/*
 * Small runtime extensions next to the mini-caffe C API (include/caffe/c_api.h):
 * access to the calling thread's stream, so a harness can bracket work with
 * its own CUDA events, and an opt-in per-kernel timer for the tensor-core
 * convolution.  None of these has a counterpart in mini-caffe; they exist for
 * measurement only.
 */
#ifndef MCB200_RUNTIME_H_
#define MCB200_RUNTIME_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* cudaStream_t (as void*) on which the calling thread's layers launch.
 * Creates the thread's context on first use; NULL on failure (see
 * CaffeGetLastError). */
void* mcb200_current_stream(void);

/* Block until the calling thread's stream is idle. Returns 0 or -1. */
int mcb200_synchronize(void);

/* While enabled, every tensor-core convolution launch of the calling thread is
 * bracketed by a pair of CUDA events on its stream. */
void mcb200_kernel_timing_begin(void);
/* Stops timing, waits for the recorded events and returns the number of timed
 * launches; *total_ms receives the sum of their durations. */
long long mcb200_kernel_timing_end(double* total_ms);
/* The same, and each_ms[i] (i < capacity) receives the duration of the i-th timed
 * launch of the session, in launch order. */
long long mcb200_kernel_timing_end_each(double* total_ms, double* each_ms, long long capacity);

/* Measured ceilings of the current device for the two resources the tensor-core
 * convolution kernel lives on (measurement only; both launch probe kernels on
 * `stream`, time them with CUDA events and block until they are done).
 *
 * mcb200_probe_mma_peak: every SM issues `steps` x 4 tcgen05.mma instructions
 * (M = 128 per CTA, N = block_n in {64, 128, 256}, kind::tf32 or, with bf16 != 0,
 * kind::f16 on bfloat16; cta_pair != 0: two-CTA pairs, M = 256 per instruction)
 * on operands resident in shared memory.  *ms is the quickest of `reps` launches,
 * *tflops the rate over all SMs.  Returns 0, a negative argument / set-up error,
 * -5 if a bounded wait ran out, or a cudaError_t.
 *
 * mcb200_probe_tma_l2_pull: every SM pulls `loads_per_cta` tiles of 16 KiB (128
 * rows of 128 bytes, 128-byte swizzle) with TMA from `buffer` (`bytes` long, 128-byte
 * aligned, device memory; keep it below the L2 size to measure L2 -> shared memory),
 * `stages` (1..8) loads in flight per SM.  *gbs is the aggregate rate of the
 * quickest of `reps` launches after one launch that warms the cache.             */
/* Diagnostic build only (`make -C mini-caffe_b200/csrc trace` -> lib/libcaffe_trace.so): the
 * convolution kernel's roles of CTA 0 stamp the SM's cycle counter at fixed points of their loops
 * (activation producer, weight producer, MMA issuer: two stamps per k-iteration; first epilogue
 * warp: two per tile, and in a fifth row five per 32 x 32 chunk of a launch with the staged
 * epilogue).  Copies 5 x 2048 values (role-major, zero where nothing was recorded) to `out`,
 * clears the device array and returns 2048; the ordinary library returns 0.                     */
int mcb200_conv_trace_read(long long* out);

int mcb200_probe_mma_peak(int bf16, int block_n, int cta_pair, int steps, int reps, double* ms, double* tflops,
                          void* stream);
int mcb200_probe_tma_l2_pull(void* buffer, size_t bytes, int loads_per_cta, int stages, int reps, double* ms,
                             double* gbs, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* MCB200_RUNTIME_H_ */
