/*
 * Shared helpers of the two reference harnesses.  TEST INFRASTRUCTURE ONLY.
 * The harnesses compile the reference project's own .cu files where they lie
 * (the path is given on the nvcc command line as -DFTQ_REF_SRC_DIR=...), rename
 * the file's main(), launch its kernels unmodified on the GPU and dump their
 * outputs as raw little-endian arrays.  Nothing of the reference is copied into
 * this repository.
 */
#pragma once
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#define FTQ_STR2(x) #x
#define FTQ_STR(x) FTQ_STR2(x)

#define HCHECK(call)                                                                                  \
  do {                                                                                                \
    cudaError_t e_ = (call);                                                                          \
    if (e_ != cudaSuccess) {                                                                          \
      std::fprintf(stderr, "harness CUDA error %s:%d: %s\n", __FILE__, __LINE__, cudaGetErrorString(e_)); \
      std::exit(2);                                                                                   \
    }                                                                                                 \
  } while (0)

template <class T>
static void dump_device(const std::string& dir, const char* name, const T* device, size_t count) {
  std::vector<T> host(count);
  HCHECK(cudaMemcpy(host.data(), device, count * sizeof(T), cudaMemcpyDeviceToHost));
  std::string path = dir + "/" + name;
  FILE* f = std::fopen(path.c_str(), "wb");
  if (!f || std::fwrite(host.data(), sizeof(T), count, f) != count) {
    std::fprintf(stderr, "cannot write %s\n", path.c_str());
    std::exit(2);
  }
  std::fclose(f);
}
