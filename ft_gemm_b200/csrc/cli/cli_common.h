// Shared pieces of the per-stage command-line programs: the reference's option
// grammar (`--name V` or `--name=V`, unknown flags ignored, boolean flags by
// presence; src/s4_cluster_multicast_abft_fp8_gemm.cu:106-161), a host-side E4M3
// decoder and the sampled FP64 verifier (src/s4:527-554).
#pragma once
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "ft_gemm.h"

#define CLI_CUDA(call)                                                                               \
  do {                                                                                               \
    cudaError_t error_ = (call);                                                                     \
    if (error_ != cudaSuccess) {                                                                     \
      std::fprintf(stderr, "CUDA error %s:%d: %s\n", __FILE__, __LINE__, cudaGetErrorString(error_)); \
      std::exit(EXIT_FAILURE);                                                                       \
    }                                                                                                \
  } while (0)

#define CLI_FT(call)                                                                        \
  do {                                                                                      \
    int rc_ = (call);                                                                       \
    if (rc_ != FT_OK) {                                                                     \
      std::fprintf(stderr, "ft_gemm error %d at %s:%d: %s\n", rc_, __FILE__, __LINE__, ft_gemm_last_error()); \
      std::exit(EXIT_FAILURE);                                                              \
    }                                                                                       \
  } while (0)

struct ArgReader {
  int argc;
  char** argv;
  const char* find(const char* name) const {
    size_t length = std::strlen(name);
    for (int i = 1; i < argc; ++i) {
      if (std::strcmp(argv[i], name) == 0 && i + 1 < argc) return argv[i + 1];
      if (std::strncmp(argv[i], name, length) == 0 && argv[i][length] == '=') return argv[i] + length + 1;
    }
    return nullptr;
  }
  int get_int(const char* name, int value) const {
    const char* text = find(name);
    return text ? std::atoi(text) : value;
  }
  float get_float(const char* name, float value) const {
    const char* text = find(name);
    return text ? std::strtof(text, nullptr) : value;
  }
  double get_double(const char* name, double value) const {
    const char* text = find(name);
    return text ? std::strtod(text, nullptr) : value;
  }
  std::string get_string(const char* name, const char* value) const {
    const char* text = find(name);
    return text ? text : value;
  }
  bool has_flag(const char* name) const {
    for (int i = 1; i < argc; ++i) {
      if (std::strcmp(argv[i], name) == 0) return true;
    }
    return false;
  }
};

struct CommonOptions {
  int m = 256, n = 256, k = 256;
  int warmup = 2, repeat = 10;
  int verify_samples = 8;
  float verify_abs_tolerance = 2.5e-1f;
  float verify_rel_tolerance = 1.0e-2f;
  float abft_abs_tolerance = 1.0e-2f;
  float abft_rel_tolerance = 2.0e-5f;
  // additions of this build
  std::string dist = "uniform";  // uniform (the reference's data) | normal | llm
  uint32_t seed_a = 0x12345678U, seed_b = 0x9abcdef0U;
};

inline void read_common(const ArgReader& args, CommonOptions& o) {
  o.m = args.get_int("--m", o.m);
  o.n = args.get_int("--n", o.n);
  o.k = args.get_int("--k", o.k);
  o.warmup = args.get_int("--warmup", o.warmup);
  o.repeat = args.get_int("--repeat", o.repeat);
  o.verify_samples = args.get_int("--verify-samples", o.verify_samples);
  o.verify_abs_tolerance = args.get_float("--verify-abs-tol", o.verify_abs_tolerance);
  o.verify_rel_tolerance = args.get_float("--verify-rel-tol", o.verify_rel_tolerance);
  o.abft_abs_tolerance = args.get_float("--abs-tol", o.abft_abs_tolerance);
  o.abft_rel_tolerance = args.get_float("--rel-tol", o.abft_rel_tolerance);
  o.dist = args.get_string("--dist", o.dist.c_str());
}

inline bool common_valid(const CommonOptions& o) {
  return o.m > 0 && o.n > 0 && o.k > 0 && o.warmup >= 0 && o.repeat > 0 &&
         o.verify_samples >= 0 && o.verify_abs_tolerance >= 0.0f && o.verify_rel_tolerance >= 0.0f && o.abft_abs_tolerance >= 0.0f &&
         o.abft_rel_tolerance >= 0.0f && (o.dist == "uniform" || o.dist == "normal" || o.dist == "llm");
}

// Fills A and B on the device with the requested seeded distribution.
inline void generate_inputs(const CommonOptions& o, void* d_a, void* d_b, cudaStream_t stream) {
  size_t a_count = static_cast<size_t>(o.m) * o.k, b_count = static_cast<size_t>(o.n) * o.k;
  if (o.dist == "uniform") {
    CLI_FT(ft_gemm_generate_fp8(d_a, a_count, o.seed_a, 0, 1.0f, 1.0f, stream));
    CLI_FT(ft_gemm_generate_fp8(d_b, b_count, o.seed_b, 0, 1.0f, 1.0f, stream));
  } else if (o.dist == "normal") {
    CLI_FT(ft_gemm_generate_fp8(d_a, a_count, o.seed_a, 1, 1.0f, 1.0f, stream));
    CLI_FT(ft_gemm_generate_fp8(d_b, b_count, o.seed_b, 1, 1.0f, 1.0f, stream));
  } else {
    // N(0, 0.02) rescaled by a per-tensor FP32 scale to about unit max-abs: the
    // largest of ~1e8 normal draws is about 5.7 sigma, so scale = 1 / (5.7 * 0.02)
    const float sigma = 0.02f, scale = 1.0f / (5.7f * 0.02f);
    CLI_FT(ft_gemm_generate_fp8(d_a, a_count, o.seed_a, 1, sigma, scale, stream));
    CLI_FT(ft_gemm_generate_fp8(d_b, b_count, o.seed_b, 1, sigma, scale, stream));
  }
}

inline float e4m3_to_float(uint8_t v) {
  int sign = v >> 7, e = (v >> 3) & 15, mant = v & 7;
  float f;
  if (e == 15 && mant == 7) {
    f = NAN;
  } else if (e == 0) {
    f = std::ldexp(static_cast<float>(mant), -9);
  } else {
    f = std::ldexp(1.0f + static_cast<float>(mant) / 8.0f, e - 7);
  }
  return sign ? -f : f;
}

struct VerificationResult {
  float max_absolute_error = 0.0f;
  float max_tolerance_ratio = 0.0f;
  int checked = 0;
};

// Sampled FP64 check of C[N,M] column-major against A[M,K], B[N,K]
// (src/s4_cluster_multicast_abft_fp8_gemm.cu:527-554).  Only the sampled rows of
// A, rows of B and entries of C are fetched from the device.
inline VerificationResult verify_samples(const void* d_a, const void* d_b, const float* d_c, const CommonOptions& o) {
  VerificationResult result;
  if (o.verify_samples == 0) return result;
  int row_step = std::max(1, o.m / o.verify_samples);
  int col_step = std::max(1, o.n / o.verify_samples);
  std::vector<uint8_t> a_row(o.k), b_row(o.k);
  int checked_rows = 0;
  for (int row = 0; row < o.m && checked_rows < o.verify_samples; row += row_step, ++checked_rows) {
    CLI_CUDA(cudaMemcpy(a_row.data(), static_cast<const uint8_t*>(d_a) + static_cast<size_t>(row) * o.k, o.k, cudaMemcpyDeviceToHost));
    int checked_cols = 0;
    for (int col = 0; col < o.n && checked_cols < o.verify_samples; col += col_step, ++checked_cols) {
      CLI_CUDA(cudaMemcpy(b_row.data(), static_cast<const uint8_t*>(d_b) + static_cast<size_t>(col) * o.k, o.k, cudaMemcpyDeviceToHost));
      double reference = 0.0;
      for (int kk = 0; kk < o.k; ++kk) {
        reference += static_cast<double>(e4m3_to_float(a_row[kk])) * static_cast<double>(e4m3_to_float(b_row[kk]));
      }
      float value = 0.0f;
      CLI_CUDA(cudaMemcpy(&value, d_c + static_cast<size_t>(col) * o.m + row, sizeof(float), cudaMemcpyDeviceToHost));
      float absolute_error = static_cast<float>(std::fabs(value - reference));
      float tolerance = o.verify_abs_tolerance + o.verify_rel_tolerance * std::max(1.0f, static_cast<float>(std::fabs(reference)));
      result.max_absolute_error = std::max(result.max_absolute_error, absolute_error);
      result.max_tolerance_ratio = std::max(result.max_tolerance_ratio, absolute_error / tolerance);
      ++result.checked;
    }
  }
  return result;
}

struct StageTimings {
  float first_ms = 0.0f;
  float average_ms = 0.0f;       // per-call event pairs (src/s4:692-702)
  float batched_average_ms = 0.0f;  // one event pair around all repeats (src/cublaslt_fp8_gemm_benchmark.cu:286-293)
};

// First call, warm-up and timed loop with the reference's timing method.
inline StageTimings time_stage(ft_gemm_handle* handle, float* d_c, const CommonOptions& o, cudaStream_t stream) {
  StageTimings t;
  cudaEvent_t start, stop;
  CLI_CUDA(cudaEventCreate(&start));
  CLI_CUDA(cudaEventCreate(&stop));
  CLI_CUDA(cudaEventRecord(start, stream));
  CLI_FT(ft_gemm_fp8_abft_run(handle, d_c, nullptr, 0, stream));
  CLI_CUDA(cudaEventRecord(stop, stream));
  CLI_CUDA(cudaEventSynchronize(stop));
  CLI_CUDA(cudaEventElapsedTime(&t.first_ms, start, stop));
  for (int i = 0; i < o.warmup; ++i) CLI_FT(ft_gemm_fp8_abft_run(handle, d_c, nullptr, 0, stream));
  CLI_CUDA(cudaStreamSynchronize(stream));
  float total_ms = 0.0f;
  for (int i = 0; i < o.repeat; ++i) {
    CLI_CUDA(cudaEventRecord(start, stream));
    CLI_FT(ft_gemm_fp8_abft_run(handle, d_c, nullptr, 0, stream));
    CLI_CUDA(cudaEventRecord(stop, stream));
    CLI_CUDA(cudaEventSynchronize(stop));
    float iteration_ms = 0.0f;
    CLI_CUDA(cudaEventElapsedTime(&iteration_ms, start, stop));
    total_ms += iteration_ms;
  }
  t.average_ms = total_ms / o.repeat;
  CLI_CUDA(cudaEventRecord(start, stream));
  for (int i = 0; i < o.repeat; ++i) CLI_FT(ft_gemm_fp8_abft_run(handle, d_c, nullptr, 0, stream));
  CLI_CUDA(cudaEventRecord(stop, stream));
  CLI_CUDA(cudaEventSynchronize(stop));
  float batched_ms = 0.0f;
  CLI_CUDA(cudaEventElapsedTime(&batched_ms, start, stop));
  t.batched_average_ms = batched_ms / o.repeat;
  CLI_CUDA(cudaEventDestroy(start));
  CLI_CUDA(cudaEventDestroy(stop));
  return t;
}

inline void print_common_header(const CommonOptions& o, const char* version_key, const char* version) {
  int tile_count = ((o.m + 63) / 64) * ((o.n + 63) / 64);
  int cta_tiles = ((o.m + 127) / 128) * ((o.n + 255) / 256);
  std::printf("%s: %s\n", version_key, version);
  bool pair = o.m % 256 == 0;
  std::printf("instruction_tile: %s, cta_tile: 128x256x128, tma_stage_k: 128, stages: %d\n", pair ? "256x256x32 (2 CTAs)" : "128x256x32",
              pair ? 7 : 4);
  std::printf("threads_per_cta: 320, producer_warps: 1, mma_warps: 1, epilogue_warps: 8, tmem_accumulators: 2\n");
  std::printf("pipeline: TMA producer || tcgen05.mma issuer || TMEM epilogue with fused ABFT verifier (persistent)\n");
  std::printf("layout: A=[M,K] row-major, B=[N,K] column-major, C=[N,M] column-major\n");
  std::printf("shape: M=%d N=%d K=%d, abft_tiles=%d, cta_tiles=%d\n", o.m, o.n, o.k, tile_count, cta_tiles);
  std::printf("cluster_shape: %s, input_distribution: %s\n", pair ? "2x1x1" : "1x1x1", o.dist.c_str());
}
