/*
 * Small runtime extensions next to the mini-caffe C API (include/caffe/c_api.h):
 * access to the calling thread's stream, so a harness can bracket work with
 * its own CUDA events, and an opt-in per-kernel timer for the tensor-core
 * convolution.  None of these has a counterpart in mini-caffe; they exist for
 * measurement only.
 */
#ifndef MCB200_RUNTIME_H_
#define MCB200_RUNTIME_H_

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

#ifdef __cplusplus
}
#endif

#endif /* MCB200_RUNTIME_H_ */
