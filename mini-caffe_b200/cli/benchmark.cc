// Command-line timing of Net::Forward through the public C++ API, the
// counterpart of mini-caffe's tools/benchmark.cpp (same arguments, same
// "Forward costs ... ms" lines, profile.json at the end), written against
// include/caffe/*.hpp only: it doubles as the proof that a program written for
// mini-caffe's headers compiles and links against this library unchanged.
//
//   benchmark net.prototxt iterations gpu_id [weights.caffemodel]
//
// Input blobs are filled with a fixed pseudo-random pattern (mini-caffe's tool
// leaves them zero, which lets ReLU networks collapse to all-zero activations).
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include <algorithm>
#include <string>
#include <vector>

#include <caffe/net.hpp>
#include <caffe/profiler.hpp>

int main(int argc, char* argv[]) {
  if (argc != 4 && argc != 5) {
    fprintf(stderr, "[Usage]: %s net.prototxt iterations gpu_id [weights.caffemodel]\n", argv[0]);
    return 2;
  }
  const std::string proto = argv[1];
  const int iters = atoi(argv[2]);
  int gpu_id = atoi(argv[3]);
  try {
    if (gpu_id >= 0 && caffe::GPUAvailable()) {
      caffe::SetMode(caffe::GPU, gpu_id);
    } else {
      gpu_id = -1;
      caffe::SetMode(caffe::CPU, -1);
    }
    LOG(INFO) << "net prototxt: " << proto;
    LOG(INFO) << "net forward iterations: " << iters;
    LOG(INFO) << "run on device " << gpu_id;

    caffe::Net net(proto);
    if (argc == 5) net.CopyTrainedLayersFrom(argv[4]);

    // The tops of the first layer (Input) are the network's inputs.
    uint32_t state = 12345u;
    for (int id : net.top_ids(0)) {
      caffe::Blob* blob = net.blobs()[id].get();
      caffe::real_t* data = blob->mutable_cpu_data();
      for (int i = 0; i < blob->count(); ++i) {
        state = state * 1664525u + 1013904223u;
        data[i] = static_cast<caffe::real_t>((state >> 8) & 0xffff) / 65536.f - 0.5f;
      }
    }

    caffe::Profiler* profiler = caffe::Profiler::Get();
    profiler->TurnON();
    std::vector<double> ms;
    for (int i = 0; i < iters; ++i) {
      const uint64_t tic = profiler->Now();
      net.Forward();
      const uint64_t toc = profiler->Now();
      ms.push_back((toc - tic) / 1000.);
      LOG(INFO) << "Forward costs " << ms.back() << " ms";
    }
    profiler->TurnOFF();
    profiler->DumpProfile("./profile.json");
    if (!ms.empty()) {
      std::sort(ms.begin(), ms.end());
      LOG(INFO) << "median " << ms[ms.size() / 2] << " ms, best " << ms.front() << " ms over " << ms.size()
                << " passes";
    }
  } catch (const std::exception& e) {
    fprintf(stderr, "benchmark: %s\n", e.what());
    return 1;
  }
  return 0;
}
