/*
 * C API of the engine: the 25 functions of mini-caffe's include/caffe/c_api.h
 * (lines 26-162), with identical names, argument order and meaning, so that
 * the python (ctypes) and Java (JNI) bindings of that project work against
 * this library unchanged.
 *
 * Conventions: every function returning int gives 0 on success and -1 on
 * failure; the message of the last failure on the calling thread is
 * CaffeGetLastError().  BlobHandle values are borrowed from their net and die
 * with it.  Arrays returned through out-parameters (shape, name and handle
 * lists) live in per-thread storage until the next such call on that thread.
 */
#ifndef CAFFE_C_API_H_
#define CAFFE_C_API_H_

#define CAFFE_API __attribute__((visibility("default")))

#ifdef __cplusplus
extern "C" {
#endif

typedef float real_t;
typedef void* BlobHandle;
typedef void* NetHandle;

/* ---- blobs ---- */
CAFFE_API int CaffeBlobNum(BlobHandle blob);
CAFFE_API int CaffeBlobChannels(BlobHandle blob);
CAFFE_API int CaffeBlobHeight(BlobHandle blob);
CAFFE_API int CaffeBlobWidth(BlobHandle blob);
/* Host pointer to the blob's values in (N, C, H, W) order.  The caller may
 * write through it: the host copy becomes the authoritative one. */
CAFFE_API real_t* CaffeBlobData(BlobHandle blob);
CAFFE_API int CaffeBlobCount(BlobHandle blob);
/* May move the blob's data. */
CAFFE_API int CaffeBlobReshape(BlobHandle blob, int shape_size, int* shape);
CAFFE_API int CaffeBlobShape(BlobHandle blob, int* shape_size, int** shape);

/* ---- nets ---- */
/* model_path may be empty: the net then keeps its initial (constant) weights. */
CAFFE_API int CaffeNetCreate(const char* net_path, const char* model_path, NetHandle* net);
CAFFE_API int CaffeNetCreateFromBuffer(const char* net_buffer, int nb_len, const char* model_buffer,
                                       int mb_len, NetHandle* net);
CAFFE_API int CaffeNetDestroy(NetHandle net);
/* Keep an intermediate blob readable after CaffeNetForward. */
CAFFE_API int CaffeNetMarkOutput(NetHandle net, const char* name);
/* Fill the input blobs first. */
CAFFE_API int CaffeNetForward(NetHandle net);
CAFFE_API int CaffeNetGetBlob(NetHandle net, const char* name, BlobHandle* blob);
CAFFE_API int CaffeNetListBlob(NetHandle net, int* n, const char*** names, BlobHandle** blobs);
/* Parameter names are "<layer>_<index>" unless the prototxt names them. */
CAFFE_API int CaffeNetListParam(NetHandle net, int* n, const char*** names, BlobHandle** params);

/* ---- profiler (process-wide, single-threaded use) ---- */
CAFFE_API int CaffeProfilerEnable();
CAFFE_API int CaffeProfilerDisable();
CAFFE_API int CaffeProfilerScopeStart(const char* name);
CAFFE_API int CaffeProfilerScopeEnd();
CAFFE_API int CaffeProfilerDump(const char* fn);

/* ---- misc ---- */
/* 1 when a CUDA device is usable. */
CAFFE_API int CaffeGPUAvailable();
/* mode 1 = GPU on `device`; mode 0 = CPU (nets can be built but not run). Per thread. */
CAFFE_API int CaffeSetMode(int mode, int device);
CAFFE_API const char* CaffeGetLastError();
CAFFE_API int CaffeMemoryPoolClear();

#ifdef __cplusplus
}
#endif

#endif /* CAFFE_C_API_H_ */
