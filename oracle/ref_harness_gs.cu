/*
 * Reference harness for the GEMM + softmax cross-nonlinearity check.  TEST
 * INFRASTRUCTURE ONLY.  Compiles src/gemm_softmax_abft.cu of the reference in place
 * and launches, unmodified, its generate_exact_fp8_kernel (:156-163),
 * fp8_qk_gemm_kernel (:165-178), project_b_kernel (:205-223),
 * expected_logit_projection_kernel (:225-241), softmax_with_log_checks_kernel
 * (:243-300), analyze_rows_kernel (:302-339), inject_logit_fault_kernel (:341-345)
 * and correct_detected_logits_kernel (:347-353) with the launch shapes and the
 * order of its main() (:430-510).
 *
 * Written to OUTDIR: a.u8, b.u8, logits.f32, expected_sum.f64, expected_weighted.f64
 * and, for each of the phases clean / fault / recovered: probabilities_<p>.f32,
 * actual_sum_<p>.f64, actual_weighted_<p>.f64, probability_sum_<p>.f64, log_z_<p>.f64,
 * detected_<p>.i32, estimated_col_<p>.i32, correction_delta_<p>.f64,
 * counts_<p>.i32 = {detected_rows, located_rows}.
 *
 * usage: ref_harness_gs M N K FAULT_ROW FAULT_COL FAULT_VALUE OUTDIR
 */
#include <cuda_runtime.h>
#define main reference_main_gs
#include FTQ_STR_INCLUDE
#undef main
#include "ref_harness_common.h"

int main(int argc, char** argv) {
  if (argc != 8) {
    std::fprintf(stderr, "usage: %s M N K FAULT_ROW FAULT_COL FAULT_VALUE OUTDIR\n", argv[0]);
    return 2;
  }
  int m = std::atoi(argv[1]), n = std::atoi(argv[2]), k = std::atoi(argv[3]);
  int fault_row = std::atoi(argv[4]), fault_col = std::atoi(argv[5]);
  float fault_value = static_cast<float>(std::atof(argv[6]));
  std::string dir = argv[7];
  Options defaults;
  size_t a_count = (size_t)m * k, b_count = (size_t)n * k, out_count = (size_t)m * n;
  float scale = 1.0f / std::sqrt(static_cast<float>(k));
  Element *d_a, *d_b;
  float *d_logits, *d_prob;
  double *b_sum, *b_weighted, *e_sum, *e_weighted, *a_sum, *a_weighted, *p_sum, *log_z, *delta;
  int *underflow, *detected, *est_col, *counts;
  HCHECK(cudaMalloc(&d_a, a_count));
  HCHECK(cudaMalloc(&d_b, b_count));
  HCHECK(cudaMalloc(&d_logits, out_count * 4));
  HCHECK(cudaMalloc(&d_prob, out_count * 4));
  HCHECK(cudaMalloc(&b_sum, k * 8));
  HCHECK(cudaMalloc(&b_weighted, k * 8));
  HCHECK(cudaMalloc(&e_sum, m * 8));
  HCHECK(cudaMalloc(&e_weighted, m * 8));
  HCHECK(cudaMalloc(&a_sum, m * 8));
  HCHECK(cudaMalloc(&a_weighted, m * 8));
  HCHECK(cudaMalloc(&p_sum, m * 8));
  HCHECK(cudaMalloc(&log_z, m * 8));
  HCHECK(cudaMalloc(&delta, m * 8));
  HCHECK(cudaMalloc(&underflow, m * 4));
  HCHECK(cudaMalloc(&detected, m * 4));
  HCHECK(cudaMalloc(&est_col, m * 4));
  HCHECK(cudaMalloc(&counts, 8));

  int init_blocks = div_up(static_cast<int>(std::max(a_count, b_count)), 256);
  generate_exact_fp8_kernel<<<init_blocks, 256>>>(d_a, a_count, 17U);
  generate_exact_fp8_kernel<<<init_blocks, 256>>>(d_b, b_count, 29U);
  dim3 gemm_block(kTile, kTile), gemm_grid(div_up(n, kTile), div_up(m, kTile));
  fp8_qk_gemm_kernel<<<gemm_grid, gemm_block>>>(d_a, d_b, d_logits, m, n, k, scale);
  project_b_kernel<<<k, kReductionThreads>>>(d_b, b_sum, b_weighted, n, k);
  expected_logit_projection_kernel<<<div_up(m, 128), 128>>>(d_a, b_sum, b_weighted, e_sum, e_weighted, m, k, scale);
  HCHECK(cudaDeviceSynchronize());
  dump_device(dir, "a.u8", reinterpret_cast<const unsigned char*>(d_a), a_count);
  dump_device(dir, "b.u8", reinterpret_cast<const unsigned char*>(d_b), b_count);
  dump_device(dir, "logits.f32", d_logits, out_count);
  dump_device(dir, "expected_sum.f64", e_sum, (size_t)m);
  dump_device(dir, "expected_weighted.f64", e_weighted, (size_t)m);

  auto phase = [&](const char* name) {
    softmax_with_log_checks_kernel<<<m, kReductionThreads>>>(d_logits, d_prob, a_sum, a_weighted, p_sum, log_z, underflow, m, n);
    HCHECK(cudaMemset(counts, 0, 8));
    analyze_rows_kernel<<<div_up(m, 256), 256>>>(e_sum, e_weighted, a_sum, a_weighted, p_sum, underflow, detected, est_col, delta,
                                                 counts, counts + 1, m, n, defaults.abs_tolerance, defaults.rel_tolerance,
                                                 defaults.row_sum_tolerance, defaults.location_tolerance);
    HCHECK(cudaGetLastError());
    HCHECK(cudaDeviceSynchronize());
    std::string p = name;
    dump_device(dir, ("probabilities_" + p + ".f32").c_str(), d_prob, out_count);
    dump_device(dir, ("actual_sum_" + p + ".f64").c_str(), a_sum, (size_t)m);
    dump_device(dir, ("actual_weighted_" + p + ".f64").c_str(), a_weighted, (size_t)m);
    dump_device(dir, ("probability_sum_" + p + ".f64").c_str(), p_sum, (size_t)m);
    dump_device(dir, ("log_z_" + p + ".f64").c_str(), log_z, (size_t)m);
    dump_device(dir, ("detected_" + p + ".i32").c_str(), detected, (size_t)m);
    dump_device(dir, ("estimated_col_" + p + ".i32").c_str(), est_col, (size_t)m);
    dump_device(dir, ("correction_delta_" + p + ".f64").c_str(), delta, (size_t)m);
    dump_device(dir, ("counts_" + p + ".i32").c_str(), counts, (size_t)2);
  };
  phase("clean");
  inject_logit_fault_kernel<<<1, 1>>>(d_logits, n, fault_row, fault_col, fault_value);
  phase("fault");
  correct_detected_logits_kernel<<<div_up(m, 256), 256>>>(d_logits, detected, est_col, delta, m, n);
  phase("recovered");
  std::printf("ref_harness_gs: M=%d N=%d K=%d fault=(%d,%d,%g) written to %s\n", m, n, k, fault_row, fault_col, fault_value, dir.c_str());
  return 0;
}
