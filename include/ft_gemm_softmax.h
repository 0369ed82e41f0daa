/*
 * ft_gemm_softmax.h -- C-ABI of the GEMM + softmax cross-nonlinearity check.
 *
 * Boundary of the reference's prototype src/gemm_softmax_abft.cu, which is a
 * program, not a library: every entry point below names the part of its main()
 * (src/gemm_softmax_abft.cu:381-543) that it replaces.
 *
 *   A [M,K], B [N,K]  FP8 E4M3, K contiguous; any positive M, K and N > 1
 *   logits[M,N] = A B^T / sqrt(K), FP32, row-major with a leading dimension that
 *                 the handle reports (N rounded up to a multiple of 128)
 *   P = softmax over each row, FP32 out, the reductions in FP64
 *   identity 0:  sum_j log(P_j) + N logZ == sum_j logit_j
 *   identity 1:  sum_j w_j log(P_j)      == sum_j w_j logit_j,   w_j = 2j - (N-1)
 * The right-hand sides come from A and column sums of B only (gs:205-241), so a
 * corrupted logit shows up AFTER the nonlinearity; its column follows from the
 * ratio of the two residuals and its value from the first (gs:302-339).
 *
 * The logits themselves are produced by the fault-tolerant FP8 GEMM of ft_gemm.h
 * on the tensor cores (the prototype uses a scalar kernel, gs:165-178), so the
 * product is already covered by the 64x64 tile checksums; the identities cover
 * what happens to it afterwards.
 *
 * Functions return FT_OK or a negative FT_ERR_* code of ft_gemm.h; the message of
 * the last error is available from ft_gemm_last_error().
 */
#ifndef FT_GEMM_SOFTMAX_H
#define FT_GEMM_SOFTMAX_H

#include "ft_gemm.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ft_gs_handle ft_gs_handle;

typedef struct {
  double abs_tol;      /* default 2e-3  (src/gemm_softmax_abft.cu:35) */
  double rel_tol;      /* default 2e-5  (gs:36) */
  double row_sum_tol;  /* default 2e-6: |sum_j P_j - 1| above this marks the row (gs:37) */
  double location_tol; /* default 0.25: distance of the observed weight from an integer weight (gs:38) */
} ft_gs_options;

/* value added to logits[row, col] after the GEMM and before the softmax (gs:341-345) */
typedef struct {
  int row;
  int col;
  float value;
} ft_gs_fault;

#define FT_GS_MAX_RECORDS 16

typedef struct {
  int row;
  int estimated_col;       /* -1: detected but not located */
  double correction_delta; /* actual - expected of identity 0: the estimate of the fault's value */
} ft_gs_record;

typedef struct {
  int status;             /* FT_OK or FT_ERR_TIMEOUT (from the GEMM) */
  int detected_rows;      /* rows whose identities or row sum failed in the first analysis (gs:320) */
  int located_rows;       /* of those, rows whose column was located (gs:336) */
  int post_detected_rows; /* detected rows after correction and a second softmax; -1 when no correction ran */
  int n_records;          /* detected rows of the first analysis, lowest rows first, at most FT_GS_MAX_RECORDS */
  int gemm_bad_tiles;     /* report of the fault-tolerant GEMM that produced the logits */
  int gemm_corrected_tiles;
  double max_projection_residual;      /* max over rows of |actual - expected| of both identities, first analysis (gs:372-379) */
  double post_max_projection_residual; /* the same after correction */
  ft_gs_record records[FT_GS_MAX_RECORDS];
} ft_gs_report;

void ft_gs_options_default(ft_gs_options* options);

/* Replaces the allocations, project_b_kernel and expected_logit_projection_kernel
 * launches (gs:390-428, 437-439): copies A and B into padded buffers of its own,
 * prepares the fault-tolerant GEMM and computes the expected projections. */
int ft_gemm_softmax_abft_prepare(ft_gs_handle** handle, const void* a_e4m3, const void* b_e4m3, int m, int n, int k,
                                 const ft_gs_options* options, void* stream);

/* Replaces fp8_qk_gemm_kernel + [inject_logit_fault_kernel] + run_softmax_and_analysis
 * (+ correct_detected_logits_kernel + a second run_softmax_and_analysis when
 * `correct` is non-zero): gs:434-436, 441-452, 483-486, 506-510.  probabilities is
 * [M,N] row-major FP32 device memory owned by the caller.  Asynchronous. */
int ft_gemm_softmax_abft_run(ft_gs_handle* handle, float* probabilities, const ft_gs_fault* fault, int correct, void* stream);

/* Replaces the copies of the counters and check arrays to the host (gs:455-463, 487-497). */
int ft_gemm_softmax_abft_report(ft_gs_handle* handle, ft_gs_report* report);

/* Inspection: the logits buffer of the handle (device), its leading dimension, and the per-row check values of the
 * LAST softmax pass copied to host arrays of M doubles each (any of them may be NULL). */
int ft_gemm_softmax_abft_logits(ft_gs_handle* handle, const float** logits, int* leading_dimension);
/* Waits for the handle's stream and copies the logits to a dense host array of M x N floats. */
int ft_gemm_softmax_abft_logits_read(ft_gs_handle* handle, float* host_out);
int ft_gemm_softmax_abft_checks(ft_gs_handle* handle, double* expected_sum, double* expected_weighted, double* actual_sum,
                                double* actual_weighted, double* probability_sum, double* log_z);

int ft_gemm_softmax_abft_destroy(ft_gs_handle* handle);

/* The prototype's input generator ((hash(seed + i) % 7) - 3) / 16 (gs:156-163). */
int ft_gemm_softmax_generate_fp8(void* out, size_t count, uint32_t seed, void* stream);

#ifdef __cplusplus
}
#endif
#endif
