// GEMM + softmax cross-nonlinearity check: the reference's prototype program
// (src/gemm_softmax_abft.cu:381-543) over the C-ABI of include/ft_gemm_softmax.h.
// Same options, printed lines and exit-code rule: a clean run must detect nothing;
// with a fault (the default) exactly the faulty row must be detected and its column
// located, and after correction the probabilities must equal the clean ones within
// 1e-6 (gs:465, 501, 519).
#include "cli_common.h"
#include "ft_gemm_softmax.h"

int main(int argc, char** argv) {
  ArgReader args{argc, argv};
  int device = args.get_int("--device", 0);
  int m = args.get_int("--m", 64), n = args.get_int("--n", 64), k = args.get_int("--k", 64);  // gs:27-40
  int fault_row = args.get_int("--fault-row", -1), fault_col = args.get_int("--fault-col", -1);
  float fault_value = args.get_float("--fault-value", 1.0f);
  ft_gs_options opt;
  ft_gs_options_default(&opt);
  opt.abs_tol = args.get_double("--abs-tol", opt.abs_tol);
  opt.rel_tol = args.get_double("--rel-tol", opt.rel_tol);
  opt.row_sum_tol = args.get_double("--row-sum-tol", opt.row_sum_tol);
  opt.location_tol = args.get_double("--location-tol", opt.location_tol);
  bool inject_fault = !args.has_flag("--no-fault");
  if (args.has_flag("--help")) {
    std::printf(
        "Usage: %s [--device N --m N --n N --k N]\n"
        "       [--fault-row N --fault-col N --fault-value X]\n"
        "       [--abs-tol X --rel-tol X --row-sum-tol X]\n"
        "       [--location-tol X --no-fault]\n",
        argv[0]);
    return EXIT_SUCCESS;
  }
  if (m <= 0 || n <= 1 || k <= 0 || fault_value == 0.0f || opt.abs_tol < 0.0 || opt.rel_tol < 0.0 || opt.row_sum_tol < 0.0 ||
      opt.location_tol < 0.0) {
    std::fprintf(stderr, "Invalid shape, fault, or tolerance option.\n");
    return EXIT_FAILURE;
  }
  if (fault_row < 0) fault_row = m / 2;
  if (fault_col < 0) fault_col = n / 2;
  if (fault_row >= m || fault_col >= n) {
    std::fprintf(stderr, "Fault position must satisfy row < M and col < N.\n");
    return EXIT_FAILURE;
  }
  CLI_CUDA(cudaSetDevice(device));
  size_t a_count = static_cast<size_t>(m) * k, b_count = static_cast<size_t>(n) * k, out_count = static_cast<size_t>(m) * n;
  void *d_a = nullptr, *d_b = nullptr;
  float *d_probabilities = nullptr, *d_reference = nullptr;
  CLI_CUDA(cudaMalloc(&d_a, a_count));
  CLI_CUDA(cudaMalloc(&d_b, b_count));
  CLI_CUDA(cudaMalloc(reinterpret_cast<void**>(&d_probabilities), out_count * sizeof(float)));
  CLI_CUDA(cudaMalloc(reinterpret_cast<void**>(&d_reference), out_count * sizeof(float)));
  CLI_FT(ft_gemm_softmax_generate_fp8(d_a, a_count, 17U, nullptr));  // seeds of gs:431-432
  CLI_FT(ft_gemm_softmax_generate_fp8(d_b, b_count, 29U, nullptr));
  ft_gs_handle* handle = nullptr;
  CLI_FT(ft_gemm_softmax_abft_prepare(&handle, d_a, d_b, m, n, k, &opt, nullptr));

  cudaEvent_t start, stop;
  CLI_CUDA(cudaEventCreate(&start));
  CLI_CUDA(cudaEventCreate(&stop));
  ft_gs_report clean;
  CLI_FT(ft_gemm_softmax_abft_run(handle, d_reference, nullptr, 0, nullptr));  // warm-up: loads the kernels
  CLI_CUDA(cudaEventRecord(start));
  CLI_FT(ft_gemm_softmax_abft_run(handle, d_reference, nullptr, 0, nullptr));
  CLI_CUDA(cudaEventRecord(stop));
  CLI_FT(ft_gemm_softmax_abft_report(handle, &clean));
  float clean_ms = 0.0f;
  CLI_CUDA(cudaEventElapsedTime(&clean_ms, start, stop));

  bool pass = clean.detected_rows == 0;
  std::printf("GEMM + Softmax cross-nonlinearity ABFT\n");
  std::printf("shape: M=%d N=%d K=%d, scale=1/sqrt(K), input=FP8 E4M3, output=FP32\n", m, n, k);
  std::printf("identity 0: sum(log(P)) + N*logZ == sum(logits)\n");
  std::printf("identity 1: sum(w*log(P)) == sum(w*logits), w_j=2*j-(N-1)\n");
  std::printf("clean run: detected_rows=%d located_rows=%d max_projection_residual=%.6e\n", clean.detected_rows, clean.located_rows,
              clean.max_projection_residual);
  std::printf("gemm: fault-tolerant FP8 tensor-core GEMM, bad_tiles=%d corrected_tiles=%d\n", clean.gemm_bad_tiles, clean.gemm_corrected_tiles);
  std::printf("clean_run_time_ms: %.6f\n", clean_ms);
  pass = pass && clean.gemm_bad_tiles == 0;

  if (inject_fault) {
    ft_gs_fault fault{fault_row, fault_col, fault_value};
    ft_gs_report faulty;
    CLI_FT(ft_gemm_softmax_abft_run(handle, d_probabilities, &fault, 1, nullptr));
    CLI_FT(ft_gemm_softmax_abft_report(handle, &faulty));
    int estimated_col = -1;
    double estimated_delta = 0.0;
    bool detected_target = false;
    for (int i = 0; i < faulty.n_records; ++i) {
      if (faulty.records[i].row == fault_row) {
        detected_target = true;
        estimated_col = faulty.records[i].estimated_col;
        estimated_delta = faulty.records[i].correction_delta;
      }
    }
    std::printf("fault: row=%d col=%d injected_delta=%+.6f\n", fault_row, fault_col, fault_value);
    std::printf("detection: detected_rows=%d located_rows=%d estimated_col=%d estimated_delta=%+.6f\n", faulty.detected_rows,
                faulty.located_rows, estimated_col, estimated_delta);
    pass = pass && faulty.detected_rows == 1 && faulty.located_rows == 1 && detected_target && estimated_col == fault_col;
    std::vector<float> reference(out_count), recovered(out_count);
    CLI_CUDA(cudaMemcpy(reference.data(), d_reference, out_count * sizeof(float), cudaMemcpyDeviceToHost));
    CLI_CUDA(cudaMemcpy(recovered.data(), d_probabilities, out_count * sizeof(float), cudaMemcpyDeviceToHost));
    double max_probability_error = 0.0;
    for (size_t index = 0; index < out_count; ++index) {
      max_probability_error = std::max(max_probability_error, std::fabs(static_cast<double>(reference[index] - recovered[index])));
    }
    std::printf("recovery: post_detected_rows=%d max_probability_error=%.6e\n", faulty.post_detected_rows, max_probability_error);
    pass = pass && faulty.post_detected_rows == 0 && max_probability_error <= 1.0e-6;
  }
  std::printf("verification: %s\n", pass ? "PASS" : "FAIL");
  CLI_FT(ft_gemm_softmax_abft_destroy(handle));
  CLI_CUDA(cudaFree(d_reference));
  CLI_CUDA(cudaFree(d_probabilities));
  CLI_CUDA(cudaFree(d_b));
  CLI_CUDA(cudaFree(d_a));
  return pass ? EXIT_SUCCESS : EXIT_FAILURE;
}
