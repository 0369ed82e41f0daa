// cuBLASLt FP8 E4M3 -> FP32 GEMM without ABFT: the same-box overhead reference for
// the fused kernel.  Bench-only; nothing in the product path calls cuBLASLt.
// Same operator description, autotune policy and report keys as the reference's
// benchmark program (src/cublaslt_fp8_gemm_benchmark.cu:189-280, 318-337): C[M,N]
// column-major = A^T * B with A stored K x M (ld K) and B stored K x N (ld K),
// FP32 compute and output, unit scale pointers, up to 32 heuristic candidates each
// timed `--autotune-repeat` times, the fastest kept.  Times are reported both ways:
// one event pair around all repeats (the reference's method, :286-293) and one
// event pair per call (the method of the ABFT stages, src/s4:692-702).
#include <cublasLt.h>

#include <limits>

#include "cli_common.h"

#define LT_CHECK(call)                                                                                       \
  do {                                                                                                       \
    cublasStatus_t status_ = (call);                                                                         \
    if (status_ != CUBLAS_STATUS_SUCCESS) {                                                                  \
      std::fprintf(stderr, "cuBLAS error %s:%d: %s\n", __FILE__, __LINE__, cublasGetStatusString(status_)); \
      std::exit(EXIT_FAILURE);                                                                               \
    }                                                                                                        \
  } while (0)

template <class T, class Attr>
static void set_attr(T object, cublasStatus_t (*setter)(T, Attr, const void*, size_t), Attr attr, const void* value, size_t size) {
  LT_CHECK(setter(object, attr, value, size));
}

int main(int argc, char** argv) {
  ArgReader args{argc, argv};
  CommonOptions o;
  o.m = o.n = o.k = 4096;
  o.warmup = 20;
  o.repeat = 50;
  read_common(args, o);
  int device = args.get_int("--device", 0);
  int autotune_repeat = args.get_int("--autotune-repeat", 5);
  int workspace_mb = args.get_int("--workspace-mb", 256);
  double peak_tflops = std::strtod(args.get_string("--peak-tflops", "4500").c_str(), nullptr);
  bool fast_accum = args.has_flag("--fast-accum");
  if (args.has_flag("--help")) {
    std::printf("Usage: %s [--device N --m N --n N --k N --warmup N --repeat N --autotune-repeat N]\n"
                "       [--verify-samples N --workspace-mb N --peak-tflops X --fast-accum --dist uniform|normal|llm]\n", argv[0]);
    return EXIT_SUCCESS;
  }
  if (o.m <= 0 || o.n <= 0 || o.k <= 0 || o.m % 16 || o.n % 16 || o.k % 16 || o.repeat <= 0 || autotune_repeat <= 0 || workspace_mb < 0) {
    std::fprintf(stderr, "Invalid options. cuBLASLt FP8 needs M, N, K multiples of 16.\n");
    return EXIT_FAILURE;
  }
  CLI_CUDA(cudaSetDevice(device));
  cudaDeviceProp properties;
  CLI_CUDA(cudaGetDeviceProperties(&properties, device));
  size_t a_count = static_cast<size_t>(o.m) * o.k, b_count = static_cast<size_t>(o.n) * o.k, c_count = static_cast<size_t>(o.m) * o.n;
  size_t workspace_bytes = static_cast<size_t>(workspace_mb) << 20;
  void *d_a, *d_b, *workspace = nullptr;
  float *d_c, *d_scales;
  CLI_CUDA(cudaMalloc(&d_a, a_count));
  CLI_CUDA(cudaMalloc(&d_b, b_count));
  CLI_CUDA(cudaMalloc(reinterpret_cast<void**>(&d_c), c_count * sizeof(float)));
  CLI_CUDA(cudaMalloc(reinterpret_cast<void**>(&d_scales), 2 * sizeof(float)));
  if (workspace_bytes) CLI_CUDA(cudaMalloc(&workspace, workspace_bytes));
  cudaStream_t stream;
  CLI_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
  generate_inputs(o, d_a, d_b, stream);
  const float unit_scales[2] = {1.0f, 1.0f};
  CLI_CUDA(cudaMemcpyAsync(d_scales, unit_scales, sizeof(unit_scales), cudaMemcpyHostToDevice, stream));
  CLI_CUDA(cudaStreamSynchronize(stream));

  cublasLtHandle_t lt;
  cublasLtMatmulDesc_t op;
  cublasLtMatrixLayout_t la, lb, lc;
  cublasLtMatmulPreference_t pref;
  LT_CHECK(cublasLtCreate(&lt));
  LT_CHECK(cublasLtMatmulDescCreate(&op, CUBLAS_COMPUTE_32F, CUDA_R_32F));
  const cublasOperation_t trans_a = CUBLAS_OP_T, trans_b = CUBLAS_OP_N;
  const void* scale_a = d_scales;
  const void* scale_b = d_scales + 1;
  set_attr(op, cublasLtMatmulDescSetAttribute, CUBLASLT_MATMUL_DESC_TRANSA, &trans_a, sizeof(trans_a));
  set_attr(op, cublasLtMatmulDescSetAttribute, CUBLASLT_MATMUL_DESC_TRANSB, &trans_b, sizeof(trans_b));
  set_attr(op, cublasLtMatmulDescSetAttribute, CUBLASLT_MATMUL_DESC_A_SCALE_POINTER, &scale_a, sizeof(scale_a));
  set_attr(op, cublasLtMatmulDescSetAttribute, CUBLASLT_MATMUL_DESC_B_SCALE_POINTER, &scale_b, sizeof(scale_b));
  if (fast_accum) {
    const int8_t on = 1;
    set_attr(op, cublasLtMatmulDescSetAttribute, CUBLASLT_MATMUL_DESC_FAST_ACCUM, &on, sizeof(on));
  }
  LT_CHECK(cublasLtMatrixLayoutCreate(&la, CUDA_R_8F_E4M3, o.k, o.m, o.k));
  LT_CHECK(cublasLtMatrixLayoutCreate(&lb, CUDA_R_8F_E4M3, o.k, o.n, o.k));
  LT_CHECK(cublasLtMatrixLayoutCreate(&lc, CUDA_R_32F, o.m, o.n, o.m));
  LT_CHECK(cublasLtMatmulPreferenceCreate(&pref));
  set_attr(pref, cublasLtMatmulPreferenceSetAttribute, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &workspace_bytes, sizeof(workspace_bytes));

  std::vector<cublasLtMatmulHeuristicResult_t> candidates(32);
  int found = 0;
  LT_CHECK(cublasLtMatmulAlgoGetHeuristic(lt, op, la, lb, lc, lc, pref, static_cast<int>(candidates.size()), candidates.data(), &found));
  if (found == 0) {
    std::fprintf(stderr, "cuBLASLt returned no FP8 algorithm.\n");
    return EXIT_FAILURE;
  }
  const float alpha = 1.0f, beta = 0.0f;
  auto launch = [&](int index) {
    return cublasLtMatmul(lt, op, &alpha, d_a, la, d_b, lb, &beta, d_c, lc, d_c, lc, &candidates[index].algo, workspace, workspace_bytes,
                          stream);
  };
  cudaEvent_t start, stop;
  CLI_CUDA(cudaEventCreate(&start));
  CLI_CUDA(cudaEventCreate(&stop));
  auto time_batch = [&](int index, int count, float* ms) {  // false when the algorithm refuses to run
    CLI_CUDA(cudaEventRecord(start, stream));
    for (int i = 0; i < count; ++i) {
      if (launch(index) != CUBLAS_STATUS_SUCCESS) return false;
    }
    CLI_CUDA(cudaEventRecord(stop, stream));
    CLI_CUDA(cudaEventSynchronize(stop));
    CLI_CUDA(cudaEventElapsedTime(ms, start, stop));
    *ms /= count;
    return true;
  };
  int best = -1;
  float best_ms = std::numeric_limits<float>::max();
  for (int index = 0; index < found; ++index) {
    float ms = 0.0f;
    if (candidates[index].state != CUBLAS_STATUS_SUCCESS || !time_batch(index, 1, &ms) || !time_batch(index, autotune_repeat, &ms)) continue;
    if (ms < best_ms) {
      best_ms = ms;
      best = index;
    }
  }
  if (best < 0) {
    std::fprintf(stderr, "All cuBLASLt FP8 algorithms failed.\n");
    return EXIT_FAILURE;
  }
  float ignored = 0.0f, batched_ms = 0.0f, per_call_total = 0.0f;
  if (o.warmup > 0) time_batch(best, o.warmup, &ignored);
  time_batch(best, o.repeat, &batched_ms);
  for (int i = 0; i < o.repeat; ++i) {
    float ms = 0.0f;
    time_batch(best, 1, &ms);
    per_call_total += ms;
  }
  float per_call_ms = per_call_total / o.repeat;
  double operations = 2.0 * static_cast<double>(o.m) * o.n * o.k;
  double tflops = operations / (batched_ms * 1.0e9);
  VerificationResult verification = verify_samples(d_a, d_b, d_c, o);
  bool passed = o.verify_samples == 0 || verification.max_tolerance_ratio <= 1.0f;
  int algorithm_id = -1;
  size_t written = 0;
  LT_CHECK(cublasLtMatmulAlgoConfigGetAttribute(&candidates[best].algo, CUBLASLT_ALGO_CONFIG_ID, &algorithm_id, sizeof(algorithm_id), &written));

  std::printf("benchmark: cuBLASLt FP8 E4M3 GEMM\n");
  std::printf("device: %d (%s)\n", device, properties.name);
  std::printf("shape: M=%d N=%d K=%d\n", o.m, o.n, o.k);
  std::printf("layout: column-major C=A*B\n");
  std::printf("types: A=FP8 E4M3 B=FP8 E4M3 accumulator=FP32 output=FP32\n");
  std::printf("fast_accum: %s\n", fast_accum ? "true" : "false");
  std::printf("input_distribution: %s\n", o.dist.c_str());
  std::printf("heuristic_algorithms: %d\n", found);
  std::printf("selected_algorithm_index: %d\n", best);
  std::printf("selected_algorithm_id: %d\n", algorithm_id);
  std::printf("workspace_bytes: %zu\n", workspace_bytes);
  std::printf("average_time_ms: %.6f\n", batched_ms);
  std::printf("throughput_tflops: %.6f\n", tflops);
  std::printf("per_call_average_time_ms: %.6f\n", per_call_ms);
  std::printf("per_call_throughput_tflops: %.6f\n", operations / (per_call_ms * 1.0e9));
  std::printf("configured_peak_tflops: %.3f\n", peak_tflops);
  std::printf("peak_utilization_percent: %.3f\n", 100.0 * tflops / peak_tflops);
  std::printf("verification_samples: %d\n", verification.checked);
  std::printf("sampled_max_absolute_error: %.6e\n", verification.max_absolute_error);
  std::printf("sampled_max_tolerance_ratio: %.6e\n", verification.max_tolerance_ratio);
  std::printf("verification: %s\n", passed ? "PASS" : "FAIL");
  return passed ? EXIT_SUCCESS : EXIT_FAILURE;
}
