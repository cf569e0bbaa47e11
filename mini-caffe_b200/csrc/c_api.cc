// The C API (include/caffe/c_api.h) over the C++ classes.  Every entry point
// catches caffe::Error, stores its text in a per-thread string and returns -1,
// as mini-caffe's src/c_api.cpp:9-10,206-223 does; list results live in
// per-thread scratch storage until the next call (c_api.cpp:137-182).
#include "caffe/c_api.h"

#include <cstring>
#include <string>
#include <vector>

#include "caffe/caffe.hpp"
#include "context.h"
#include "io.h"
#include "mcb200_runtime.h"

namespace {

struct ThreadScratch {
  std::string last_error;
  std::vector<int> shape;
  std::vector<std::string> name_storage;
  std::vector<const char*> names;
  std::vector<void*> handles;
};

ThreadScratch& Scratch() {
  static thread_local ThreadScratch s;
  return s;
}

int Fail(const std::exception& e) {
  Scratch().last_error = e.what();
  return -1;
}

}  // namespace

#define API_BEGIN() try {
#define API_END()                          \
  }                                        \
  catch (const caffe::Error& err) {        \
    return Fail(err);                      \
  }                                        \
  catch (const std::exception& err) {      \
    return Fail(err);                      \
  }                                        \
  return 0;

using caffe::Blob;
using caffe::Net;

int CaffeBlobNum(BlobHandle blob) { return static_cast<Blob*>(blob)->num(); }
int CaffeBlobChannels(BlobHandle blob) { return static_cast<Blob*>(blob)->channels(); }
int CaffeBlobHeight(BlobHandle blob) { return static_cast<Blob*>(blob)->height(); }
int CaffeBlobWidth(BlobHandle blob) { return static_cast<Blob*>(blob)->width(); }
int CaffeBlobCount(BlobHandle blob) { return static_cast<Blob*>(blob)->count(); }

real_t* CaffeBlobData(BlobHandle blob) {
  try {
    return static_cast<Blob*>(blob)->mutable_cpu_data();
  } catch (const std::exception& err) {
    Fail(err);
    return nullptr;
  }
}

int CaffeBlobReshape(BlobHandle blob, int shape_size, int* shape) {
  API_BEGIN();
  static_cast<Blob*>(blob)->Reshape(std::vector<int>(shape, shape + shape_size));
  API_END();
}

int CaffeBlobShape(BlobHandle blob, int* shape_size, int** shape) {
  API_BEGIN();
  ThreadScratch& s = Scratch();
  s.shape = static_cast<Blob*>(blob)->shape();
  *shape_size = static_cast<int>(s.shape.size());
  *shape = s.shape.data();
  API_END();
}

int CaffeNetCreate(const char* net_path, const char* model_path, NetHandle* net) {
  API_BEGIN();
  Net* n = new Net(std::string(net_path));
  try {
    if (model_path && model_path[0] != '\0') n->CopyTrainedLayersFrom(std::string(model_path));
  } catch (...) {
    delete n;
    throw;
  }
  *net = static_cast<NetHandle>(n);
  API_END();
}

int CaffeNetCreateFromBuffer(const char* net_buffer, int nb_len, const char* model_buffer, int mb_len,
                             NetHandle* net) {
  API_BEGIN();
  caffe::shared_ptr<caffe::NetParameter> def = caffe::ReadTextNetParameterFromBuffer(net_buffer, nb_len);
  Net* n = new Net(*def);
  try {
    if (model_buffer && mb_len > 0) {
      caffe::shared_ptr<caffe::NetParameter> weights = caffe::ReadBinaryNetParameterFromBuffer(model_buffer, mb_len);
      n->CopyTrainedLayersFrom(*weights);
    }
  } catch (...) {
    delete n;
    throw;
  }
  *net = static_cast<NetHandle>(n);
  API_END();
}

int CaffeNetDestroy(NetHandle net) {
  API_BEGIN();
  delete static_cast<Net*>(net);
  API_END();
}

int CaffeNetMarkOutput(NetHandle net, const char* name) {
  API_BEGIN();
  static_cast<Net*>(net)->MarkOutputs({std::string(name)});
  API_END();
}

int CaffeNetForward(NetHandle net) {
  API_BEGIN();
  static_cast<Net*>(net)->Forward(true);
  API_END();
}

int CaffeNetGetBlob(NetHandle net, const char* name, BlobHandle* blob) {
  API_BEGIN();
  *blob = static_cast<BlobHandle>(static_cast<Net*>(net)->blob_by_name(name).get());
  API_END();
}

static void FillLists(const std::vector<std::string>& names, const std::vector<caffe::shared_ptr<Blob> >& blobs,
                      int* n, const char*** out_names, BlobHandle** out_handles) {
  ThreadScratch& s = Scratch();
  s.name_storage = names;
  s.names.resize(names.size());
  s.handles.resize(names.size());
  for (size_t i = 0; i < names.size(); ++i) {
    s.names[i] = s.name_storage[i].c_str();
    s.handles[i] = blobs[i].get();
  }
  *n = static_cast<int>(names.size());
  *out_names = s.names.data();
  *out_handles = s.handles.data();
}

int CaffeNetListBlob(NetHandle net, int* n, const char*** names, BlobHandle** blobs) {
  API_BEGIN();
  Net* p = static_cast<Net*>(net);
  FillLists(p->blob_names(), p->blobs(), n, names, blobs);
  API_END();
}

int CaffeNetListParam(NetHandle net, int* n, const char*** names, BlobHandle** params) {
  API_BEGIN();
  Net* p = static_cast<Net*>(net);
  FillLists(p->param_names(), p->params(), n, names, params);
  API_END();
}

int CaffeProfilerEnable() {
  API_BEGIN();
  caffe::Profiler::Get()->TurnON();
  API_END();
}

int CaffeProfilerDisable() {
  API_BEGIN();
  caffe::Profiler::Get()->TurnOFF();
  API_END();
}

int CaffeProfilerScopeStart(const char* name) {
  API_BEGIN();
  caffe::Profiler::Get()->ScopeStart(name);
  API_END();
}

int CaffeProfilerScopeEnd() {
  API_BEGIN();
  caffe::Profiler::Get()->ScopeEnd();
  API_END();
}

int CaffeProfilerDump(const char* fn) {
  API_BEGIN();
  caffe::Profiler::Get()->DumpProfile(fn);
  API_END();
}

int CaffeGPUAvailable() { return caffe::GPUAvailable() ? 1 : 0; }

int CaffeSetMode(int mode, int device) {
  API_BEGIN();
  caffe::SetMode(mode == 1 ? caffe::GPU : caffe::CPU, device);
  API_END();
}

const char* CaffeGetLastError() { return Scratch().last_error.c_str(); }

int CaffeMemoryPoolClear() {
  API_BEGIN();
  caffe::MemPoolClear();
  API_END();
}

// ---- measurement helpers (include/mcb200_runtime.h) ----

void* mcb200_current_stream(void) {
  try {
    return caffe::Context::Get().stream_ptr();
  } catch (const std::exception& err) {
    Fail(err);
    return nullptr;
  }
}

int mcb200_synchronize(void) {
  API_BEGIN();
  caffe::Context::Get().SyncAndCheck();
  API_END();
}
