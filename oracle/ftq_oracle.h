/*
 * CPU oracle for the ABFT FP8 GEMM path.  TEST INFRASTRUCTURE ONLY.
 *
 * This is a plain-C restatement of the algorithm in the reference project
 * chaiduo/FT-GEMM (files cited per function as `src/<file>:<lines>`).  It is the
 * checker used by the tests, by the smoke run and by the benchmark's CPU-baseline
 * leg; the product library never links, imports or executes it.
 *
 * Parity status: PINNED.  The reference ships no golden vectors, so the pins are
 * outputs of the reference's own kernels (generator, S0 GEMM / prepare / checker,
 * S2-S4 band-sum and expected-checksum kernels) run unmodified on a B200 through
 * `oracle/ref_harness.cu`; they are stored under `tests/golden/` and every
 * function below that has a reference kernel is compared with them bit for bit.
 * The one part that no reference output can pin on this hardware is the FP8
 * tensor-core accumulation order of the S1-S4 main loops (sm_90a only).
 *
 * Floating-point conventions: the reference is compiled by nvcc with its default
 * -fmad=true, so every `x += a * b` in its kernels is one fused multiply-add.
 * The oracle therefore calls fmaf() explicitly at those places and must itself be
 * compiled with -ffp-contract=off so that nothing else is fused.
 */
#ifndef FTQ_ORACLE_H
#define FTQ_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- layouts ---------------------------------------------------------- */
enum { FTQ_B_NK = 0 /* B[N,K], K contiguous (S1-S4) */, FTQ_B_KN = 1 /* B[K,N], N contiguous (S0) */ };
enum { FTQ_C_COLMAJOR = 0 /* c[col*M+row] (S1-S4) */, FTQ_C_ROWMAJOR = 1 /* c[row*N+col] (S0) */ };

/* ---- E4M3 codec and generators ---------------------------------------- */
uint32_t ftq_mix_u32(uint32_t x);                       /* src/s0:93-100 */
uint8_t ftq_e4m3_from_float(float x);                   /* __nv_fp8_e4m3(float): RNE, saturate to +-448, NaN -> 0x7f */
float ftq_e4m3_to_float(uint8_t v);
void ftq_quantize_f32(const float* src, size_t count, float scale, uint8_t* out);  /* E4M3(src * scale) */
void ftq_generate_uniform(uint8_t* out, size_t count, uint32_t seed);          /* src/s0:102-110 */
void ftq_generate_normal(uint8_t* out, size_t count, uint32_t seed, float sigma, float post_scale);

/* ---- GEMM -------------------------------------------------------------- */
/* FP32 accumulate in ascending k with one fma per step (src/s0:112-133). */
void ftq_gemm_f32(const uint8_t* a, const uint8_t* b, float* c, int m, int n, int k, int b_layout, int c_layout);
/* FP64 truth for sampled entries (src/s4:540-545). */
double ftq_dot_f64(const uint8_t* a, const uint8_t* b, int row, int col, int n, int k, int b_layout);

/* ---- expected checksums ------------------------------------------------ */
/* src/s4:194-235: band sums over `tile` rows of A / rows of B[N,K]. */
void ftq_band_sums(const uint8_t* a, const uint8_t* b, float* a_sums, float* a_mags, float* b_sums, float* b_mags, int m, int n,
                   int k, int tile);
/* src/s4:237-294: one warp per checksum, lane-strided k, shuffle-down tree. */
void ftq_expected_from_bands(const uint8_t* a, const uint8_t* b, const float* a_sums, const float* a_mags, const float* b_sums,
                             const float* b_mags, float* expected_rows, float* expected_cols, float* row_scales,
                             float* col_scales, int m, int n, int k, int tile);
/* src/s0:135-185: direct form, any tile size, B[K,N]. Entries beyond the valid
 * rows/cols of an edge tile are left untouched, as in the reference. */
void ftq_s0_prepare(const uint8_t* a, const uint8_t* b, float* expected_rows, float* expected_cols, float* row_scales,
                    float* col_scales, int m, int n, int k, int tile);

/* ---- checker ----------------------------------------------------------- */
typedef struct {
  int tile;    /* ABFT tile id = tile_row * tile_cols + tile_col */
  int row;     /* local row in the tile */
  int col;     /* local column in the tile */
  float value; /* added to C before the checksums */
} ftq_fault;

typedef struct {
  int tile;
  int bad_row_count;
  int bad_col_count;
  int bad_row; /* lowest bad local row, -1 if none */
  int bad_col; /* lowest bad local column, -1 if none */
  float row_delta; /* expected - actual of bad_row (0 if none) */
  float col_delta;
  int corrected;
  /* smallest |(|delta| - threshold)| over all 2*tile checksums of this tile,
   * divided by the threshold: how close the nearest decision was to flipping */
  float min_margin;
} ftq_tile_record;

typedef struct {
  int bad_tiles;
  int corrected_tiles;
  int multi_fault_tiles; /* bad but not (1 row, 1 col) */
  int n_records;         /* records written (<= max_records) */
  float max_clean_ratio; /* max |delta| / (abs + rel*max(1,scale)) over checks that were NOT bad */
  float min_margin;      /* min over all checks of | |delta| - thr | / thr */
} ftq_check_summary;

/* S1-S4 checker (src/s4:432-503 with the campaign's injection point,
 * src/s4_random_fault_campaign.cu:464-466).  `or_rule` != 0 counts a tile as bad
 * when rows>0 || cols>0 (S1-S4, src/s4:490); 0 uses rows>0 && cols>0 (S0,
 * src/s0:267).  C is modified in place (faults injected, single faults corrected).
 * m must be a multiple of tile for the S1-S4 form; n may be ragged. */
void ftq_abft_check(float* c, int m, int n, int tile, int c_layout, const float* expected_rows, const float* expected_cols,
                    const float* row_scales, const float* col_scales, float abs_tol, float rel_tol, int or_rule,
                    const ftq_fault* faults, int n_faults, ftq_tile_record* records, int max_records,
                    ftq_check_summary* summary);

/* ---- campaign ---------------------------------------------------------- */
typedef struct {
  int tile, row, col, bin;
  float magnitude, signed_value, unit;
} ftq_campaign_draw;
/* src/s4_random_fault_campaign.cu:755-769.  `state` carries over between trials. */
void ftq_campaign_next(uint32_t* state, int trial, int tile_count, int tile, float min_value, float max_value,
                       ftq_campaign_draw* out);

/* ---- sampled verifier (src/s4:527-554) --------------------------------- */
typedef struct {
  float max_absolute_error, max_tolerance_ratio;
  int checked;
} ftq_verify_result;
void ftq_verify_samples(const uint8_t* a, const uint8_t* b, const float* c, int m, int n, int k, int samples, float abs_tol,
                        float rel_tol, int b_layout, int c_layout, ftq_verify_result* out);

/* ---- timed whole-path pass for the CPU baseline ------------------------- */
/* Runs prepare -> GEMM -> check -> correct on rows [0, m_rows) of A with all
 * OpenMP threads; returns seconds spent in {prepare, gemm, check}. */
void ftq_full_pass(const uint8_t* a, const uint8_t* b, float* c, int m_rows, int n, int k, int tile, float abs_tol,
                   float rel_tol, double* seconds3, ftq_check_summary* summary);
int ftq_num_threads(void);
void ftq_set_num_threads(int threads);

#ifdef __cplusplus
}
#endif
#endif
