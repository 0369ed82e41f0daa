/*
 * CPU oracle for the ABFT FP8 GEMM path.  TEST INFRASTRUCTURE ONLY: see the
 * header for the rules.  Each function restates, in plain C, one kernel or host
 * routine of the reference project chaiduo/FT-GEMM; the citation names the
 * reference file and lines it follows.  Compile with -ffp-contract=off.
 */
#include "ftq_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------------ */
/* hash, codec, generators                                                   */
/* ------------------------------------------------------------------------ */

/* src/s0_tiled_abft_fp8_gemm.cu:93-100 */
uint32_t ftq_mix_u32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7feb352dU;
  x ^= x >> 15;
  x *= 0x846ca68bU;
  x ^= x >> 16;
  return x;
}

static float g_decode[256];
static int g_decode_ready = 0;

static void build_decode(void) {
  for (int v = 0; v < 256; ++v) {
    int sign = v >> 7, e = (v >> 3) & 15, mant = v & 7;
    float f;
    if (e == 15 && mant == 7) {
      f = NAN;
    } else if (e == 0) {
      f = ldexpf((float)mant, -9); /* subnormal: mant * 2^-9 */
    } else {
      f = ldexpf(1.0f + (float)mant / 8.0f, e - 7);
    }
    g_decode[v] = sign ? -f : f;
  }
  g_decode_ready = 1;
}

float ftq_e4m3_to_float(uint8_t v) {
  if (!g_decode_ready) build_decode();
  return g_decode[v];
}

static inline const float* decode_table(void) {
  if (!g_decode_ready) build_decode();
  return g_decode;
}

/* What `__nv_fp8_e4m3(float)` does (cuda_fp8.hpp: __nv_cvt_float_to_fp8 with
 * __NV_SATFINITE, __NV_E4M3): round to nearest even, saturate to +-448, NaN ->
 * 0x7f.  The reference constructs every input through it (src/s0:109). */
uint8_t ftq_e4m3_from_float(float x) {
  uint32_t bits;
  memcpy(&bits, &x, 4);
  if ((bits & 0x7fffffffU) > 0x7f800000U) return 0x7f;
  uint8_t sign = (uint8_t)((bits >> 31) << 7);
  float ax = fabsf(x);
  if (ax >= 448.0f) return (uint8_t)(sign | 0x7e);
  if (ax == 0.0f) return sign;
  int e;
  (void)frexpf(ax, &e); /* ax = f * 2^e, f in [0.5, 1) */
  int ex = e - 1;
  if (ex < -6) ex = -6;
  float q = ldexpf(1.0f, ex - 3); /* spacing of representable values at this exponent */
  float r = nearbyintf(ax / q);   /* exact scaling; RNE in the default rounding mode */
  if (r == 16.0f) {
    ex += 1;
    r = 8.0f;
  }
  int ri = (int)r;
  if (ri < 8) return (uint8_t)(sign | ri); /* subnormal or zero */
  return (uint8_t)(sign | ((ex + 7) << 3) | (ri - 8));
}

/* src/s0_tiled_abft_fp8_gemm.cu:102-110 */
/* The producer of an FP8 operand: out = E4M3(src * scale), one FP32 multiply and one rounding per element
 * (what a fused quantise kernel in front of src/s4:194-235 has to produce). */
void ftq_quantize_f32(const float* src, size_t count, float scale, uint8_t* out) {
  for (size_t index = 0; index < count; ++index) out[index] = ftq_e4m3_from_float(src[index] * scale);
}

void ftq_generate_uniform(uint8_t* out, size_t count, uint32_t seed) {
#pragma omp parallel for schedule(static)
  for (size_t index = 0; index < count; ++index) {
    uint32_t bits = ftq_mix_u32(seed + (uint32_t)index);
    float unit = (float)(bits & 0x00ffffffU) / 16777216.0f;
    out[index] = ftq_e4m3_from_float(2.0f * unit - 1.0f);
  }
}

/* Not in the reference: a seeded normal source for the N(0,1) and N(0,0.02)
 * workloads.  Box-Muller over two hash draws per element; value = z * sigma *
 * post_scale.  libm differs between host and device in the last bit, so this is
 * used for distribution checks, never for byte-exact comparisons. */
void ftq_generate_normal(uint8_t* out, size_t count, uint32_t seed, float sigma, float post_scale) {
#pragma omp parallel for schedule(static)
  for (size_t index = 0; index < count; ++index) {
    uint32_t i2 = (uint32_t)(2u * (uint32_t)index);
    uint32_t h1 = ftq_mix_u32(seed ^ i2);
    uint32_t h2 = ftq_mix_u32(seed ^ (i2 + 1u));
    float u1 = ((float)(h1 & 0x00ffffffU) + 1.0f) / 16777216.0f; /* (0,1] */
    float u2 = (float)(h2 & 0x00ffffffU) / 16777216.0f;
    float z = sqrtf(-2.0f * logf(u1)) * cosf(6.28318530717958647692f * u2);
    out[index] = ftq_e4m3_from_float(z * sigma * post_scale);
  }
}

/* ------------------------------------------------------------------------ */
/* GEMM                                                                      */
/* ------------------------------------------------------------------------ */

/* src/s0_tiled_abft_fp8_gemm.cu:112-133: one FP32 accumulator per output,
 * k ascending, `accumulator += a * b` (an fma under nvcc; the product of two
 * E4M3 values is exact in FP32, so fma and mul+add agree). */
void ftq_gemm_f32(const uint8_t* a, const uint8_t* b, float* c, int m, int n, int k, int b_layout, int c_layout) {
  const float* dec = decode_table();
  /* work on FP32 copies, B transposed to [N,K] when needed, for cache behaviour */
  float* af = (float*)malloc((size_t)m * k * sizeof(float));
  float* bf = (float*)malloc((size_t)n * k * sizeof(float));
#pragma omp parallel for schedule(static)
  for (int r = 0; r < m; ++r)
    for (int kk = 0; kk < k; ++kk) af[(size_t)r * k + kk] = dec[a[(size_t)r * k + kk]];
#pragma omp parallel for schedule(static)
  for (int col = 0; col < n; ++col)
    for (int kk = 0; kk < k; ++kk)
      bf[(size_t)col * k + kk] = dec[b_layout == FTQ_B_NK ? b[(size_t)col * k + kk] : b[(size_t)kk * n + col]];

  enum { RB = 4, CB = 8 };
#pragma omp parallel for schedule(dynamic, 4)
  for (int r0 = 0; r0 < m; r0 += RB) {
    for (int c0 = 0; c0 < n; c0 += CB) {
      float acc[RB][CB];
      int rmax = r0 + RB <= m ? RB : m - r0;
      int cmax = c0 + CB <= n ? CB : n - c0;
      for (int i = 0; i < RB; ++i)
        for (int j = 0; j < CB; ++j) acc[i][j] = 0.0f;
      for (int kk = 0; kk < k; ++kk) {
        for (int i = 0; i < rmax; ++i) {
          float av = af[(size_t)(r0 + i) * k + kk];
          for (int j = 0; j < cmax; ++j) acc[i][j] = fmaf(av, bf[(size_t)(c0 + j) * k + kk], acc[i][j]);
        }
      }
      for (int i = 0; i < rmax; ++i)
        for (int j = 0; j < cmax; ++j) {
          size_t idx = c_layout == FTQ_C_COLMAJOR ? (size_t)(c0 + j) * m + (r0 + i) : (size_t)(r0 + i) * n + (c0 + j);
          c[idx] = acc[i][j];
        }
    }
  }
  free(af);
  free(bf);
}

/* src/s4_cluster_multicast_abft_fp8_gemm.cu:540-545 */
double ftq_dot_f64(const uint8_t* a, const uint8_t* b, int row, int col, int n, int k, int b_layout) {
  const float* dec = decode_table();
  double reference = 0.0;
  for (int kk = 0; kk < k; ++kk) {
    float bv = dec[b_layout == FTQ_B_NK ? b[(size_t)col * k + kk] : b[(size_t)kk * n + col]];
    reference += (double)dec[a[(size_t)row * k + kk]] * (double)bv;
  }
  return reference;
}

/* ------------------------------------------------------------------------ */
/* expected checksums                                                        */
/* ------------------------------------------------------------------------ */

/* src/s4_cluster_multicast_abft_fp8_gemm.cu:194-235.  Rows of a band are added
 * in ascending order into one FP32 accumulator per k. */
void ftq_band_sums(const uint8_t* a, const uint8_t* b, float* a_sums, float* a_mags, float* b_sums, float* b_mags, int m, int n,
                   int k, int tile) {
  const float* dec = decode_table();
  int tile_rows = (m + tile - 1) / tile; /* the reference requires M % 128 == 0; a short last band is treated like a short last band of B */
  int tile_cols = (n + tile - 1) / tile;
#pragma omp parallel for schedule(static)
  for (int t = 0; t < tile_rows + tile_cols; ++t) {
    if (t < tile_rows) {
      int row_begin = t * tile;
      int valid_rows = m - row_begin < tile ? m - row_begin : tile;
      for (int kk = 0; kk < k; ++kk) {
        float sum = 0.0f, magnitude = 0.0f;
        for (int row = 0; row < valid_rows; ++row) {
          float value = dec[a[(size_t)(row_begin + row) * k + kk]];
          sum += value;
          magnitude += fabsf(value);
        }
        a_sums[(size_t)t * k + kk] = sum;
        a_mags[(size_t)t * k + kk] = magnitude;
      }
    } else {
      int tile_col = t - tile_rows;
      int col_begin = tile_col * tile;
      int valid_cols = n - col_begin < tile ? n - col_begin : tile;
      for (int kk = 0; kk < k; ++kk) {
        float sum = 0.0f, magnitude = 0.0f;
        for (int col = 0; col < valid_cols; ++col) {
          float value = dec[b[(size_t)(col_begin + col) * k + kk]];
          sum += value;
          magnitude += fabsf(value);
        }
        b_sums[(size_t)tile_col * k + kk] = sum;
        b_mags[(size_t)tile_col * k + kk] = magnitude;
      }
    }
  }
}

/* The reduction of src/s4:264-282: lane l accumulates k = l, l+32, ... with one
 * fma per step, then five shuffle-down rounds (offsets 16, 8, 4, 2, 1); lane 0
 * holds the result.  Lanes >= offset add values whose content does not reach
 * lane 0, so only the lower half is formed at each round. */
static inline float tree32(float* p) {
  for (int offset = 16; offset > 0; offset /= 2)
    for (int i = 0; i < offset; ++i) p[i] = p[i] + p[i + offset];
  return p[0];
}

/* src/s4_cluster_multicast_abft_fp8_gemm.cu:237-294 */
void ftq_expected_from_bands(const uint8_t* a, const uint8_t* b, const float* a_sums, const float* a_mags, const float* b_sums,
                             const float* b_mags, float* expected_rows, float* expected_cols, float* row_scales,
                             float* col_scales, int m, int n, int k, int tile) {
  const float* dec = decode_table();
  int tile_rows = (m + tile - 1) / tile;
  int tile_cols = (n + tile - 1) / tile;
  long total = (long)tile_rows * tile_cols;
#pragma omp parallel for schedule(static)
  for (long tile_id = 0; tile_id < total; ++tile_id) {
    int tile_row = (int)(tile_id / tile_cols);
    int tile_col = (int)(tile_id % tile_cols);
    int valid_cols = n - tile_col * tile < tile ? n - tile_col * tile : tile;
    int valid_rows = m - tile_row * tile < tile ? m - tile_row * tile : tile; /* rows past M: zeros, as for columns past N */
    for (int check = 0; check < 2 * tile; ++check) {
      int is_row = check < tile;
      int idx = is_row ? check : check - tile;
      float pe[32], ps[32];
      for (int l = 0; l < 32; ++l) pe[l] = ps[l] = 0.0f;
      if (is_row && idx >= valid_rows) {
        /* nothing to add */
      } else if (is_row) {
        const uint8_t* arow = a + (size_t)(tile_row * tile + idx) * k;
        const float* bs = b_sums + (size_t)tile_col * k;
        const float* bm = b_mags + (size_t)tile_col * k;
        for (int kk = 0; kk < k; ++kk) {
          float av = dec[arow[kk]];
          int l = kk & 31;
          pe[l] = fmaf(av, bs[kk], pe[l]);
          ps[l] = fmaf(fabsf(av), bm[kk], ps[l]);
        }
      } else if (idx < valid_cols) {
        const uint8_t* brow = b + (size_t)(tile_col * tile + idx) * k;
        const float* as = a_sums + (size_t)tile_row * k;
        const float* am = a_mags + (size_t)tile_row * k;
        for (int kk = 0; kk < k; ++kk) {
          float bv = dec[brow[kk]];
          int l = kk & 31;
          pe[l] = fmaf(as[kk], bv, pe[l]);
          ps[l] = fmaf(am[kk], fabsf(bv), ps[l]);
        }
      }
      float expected = tree32(pe), scale = tree32(ps);
      if (is_row) {
        expected_rows[(size_t)tile_id * tile + idx] = expected;
        row_scales[(size_t)tile_id * tile + idx] = scale;
      } else {
        expected_cols[(size_t)tile_id * tile + idx] = expected;
        col_scales[(size_t)tile_id * tile + idx] = scale;
      }
    }
  }
}

/* src/s0_tiled_abft_fp8_gemm.cu:135-185 (B is [K,N]). */
void ftq_s0_prepare(const uint8_t* a, const uint8_t* b, float* expected_rows, float* expected_cols, float* row_scales,
                    float* col_scales, int m, int n, int k, int tile) {
  const float* dec = decode_table();
  int tile_rows = (m + tile - 1) / tile;
  int tile_cols = (n + tile - 1) / tile;
#pragma omp parallel for schedule(static)
  for (int tile_id = 0; tile_id < tile_rows * tile_cols; ++tile_id) {
    int tile_row = tile_id / tile_cols, tile_col = tile_id % tile_cols;
    int valid_rows = m - tile_row * tile < tile ? m - tile_row * tile : tile;
    int valid_cols = n - tile_col * tile < tile ? n - tile_col * tile : tile;
    for (int t = 0; t < valid_rows; ++t) {
      int row = tile_row * tile + t;
      float expected = 0.0f, scale = 0.0f;
      for (int kk = 0; kk < k; ++kk) {
        float b_sum = 0.0f, b_abs_sum = 0.0f;
        for (int lc = 0; lc < valid_cols; ++lc) {
          float value = dec[b[(size_t)kk * n + tile_col * tile + lc]];
          b_sum += value;
          b_abs_sum += fabsf(value);
        }
        float avalue = dec[a[(size_t)row * k + kk]];
        expected = fmaf(avalue, b_sum, expected);
        scale = fmaf(fabsf(avalue), b_abs_sum, scale);
      }
      expected_rows[(size_t)tile_id * tile + t] = expected;
      row_scales[(size_t)tile_id * tile + t] = scale;
    }
    for (int t = 0; t < valid_cols; ++t) {
      int col = tile_col * tile + t;
      float expected = 0.0f, scale = 0.0f;
      for (int kk = 0; kk < k; ++kk) {
        float a_sum = 0.0f, a_abs_sum = 0.0f;
        for (int lr = 0; lr < valid_rows; ++lr) {
          float value = dec[a[(size_t)(tile_row * tile + lr) * k + kk]];
          a_sum += value;
          a_abs_sum += fabsf(value);
        }
        float bvalue = dec[b[(size_t)kk * n + col]];
        expected = fmaf(a_sum, bvalue, expected);
        scale = fmaf(a_abs_sum, fabsf(bvalue), scale);
      }
      expected_cols[(size_t)tile_id * tile + t] = expected;
      col_scales[(size_t)tile_id * tile + t] = scale;
    }
  }
}

/* ------------------------------------------------------------------------ */
/* checker                                                                   */
/* ------------------------------------------------------------------------ */

static inline size_t c_index(int row, int col, int m, int n, int c_layout) {
  return c_layout == FTQ_C_COLMAJOR ? (size_t)col * m + row : (size_t)row * n + col;
}

/* Threshold of src/s4:467 / src/s0:187-189: abs + rel * fmaxf(1, scale), one
 * fma under nvcc. */
static inline float threshold(float abs_tol, float rel_tol, float scale) { return fmaf(rel_tol, fmaxf(1.0f, scale), abs_tol); }

/* src/s4_cluster_multicast_abft_fp8_gemm.cu:432-503 (tile 64, `||`) and
 * src/s0_tiled_abft_fp8_gemm.cu:193-277 (tile 16, `&&`); injection as
 * src/s4_random_fault_campaign.cu:464-466.  Actual sums are formed in ascending
 * index order like the reference's serial loops. */
void ftq_abft_check(float* c, int m, int n, int tile, int c_layout, const float* expected_rows, const float* expected_cols,
                    const float* row_scales, const float* col_scales, float abs_tol, float rel_tol, int or_rule,
                    const ftq_fault* faults, int n_faults, ftq_tile_record* records, int max_records,
                    ftq_check_summary* summary) {
  int tile_rows = (m + tile - 1) / tile;
  int tile_cols = (n + tile - 1) / tile;
  long total = (long)tile_rows * tile_cols;
  int bad_tiles = 0, corrected_tiles = 0, multi = 0, n_records = 0;
  float max_clean_ratio = 0.0f, min_margin = INFINITY;

#pragma omp parallel for schedule(static) reduction(+ : bad_tiles, corrected_tiles, multi) reduction(max : max_clean_ratio) \
    reduction(min : min_margin)
  for (long tile_id = 0; tile_id < total; ++tile_id) {
    int tile_row = (int)(tile_id / tile_cols), tile_col = (int)(tile_id % tile_cols);
    int valid_rows = m - tile_row * tile < tile ? m - tile_row * tile : tile;
    int valid_cols = n - tile_col * tile < tile ? n - tile_col * tile : tile;
    for (int f = 0; f < n_faults; ++f) {
      if (faults[f].tile == tile_id) {
        int row = faults[f].row < valid_rows - 1 ? faults[f].row : valid_rows - 1;
        int col = faults[f].col < valid_cols - 1 ? faults[f].col : valid_cols - 1;
        c[c_index(tile_row * tile + row, tile_col * tile + col, m, n, c_layout)] += faults[f].value;
      }
    }
    int nbr = 0, nbc = 0, bad_row = -1, bad_col = -1;
    float bad_row_delta = 0.0f, bad_col_delta = 0.0f, tile_margin = INFINITY;
    for (int r = 0; r < valid_rows; ++r) {
      float actual = 0.0f;
      for (int col = 0; col < valid_cols; ++col) actual += c[c_index(tile_row * tile + r, tile_col * tile + col, m, n, c_layout)];
      float delta = expected_rows[(size_t)tile_id * tile + r] - actual;
      float thr = threshold(abs_tol, rel_tol, row_scales[(size_t)tile_id * tile + r]);
      float margin = fabsf(fabsf(delta) - thr) / thr;
      if (margin < tile_margin) tile_margin = margin;
      if (fabsf(delta) > thr) {
        if (nbr == 0) {
          bad_row = r;
          bad_row_delta = delta;
        }
        ++nbr;
      } else {
        float ratio = fabsf(delta) / thr;
        if (ratio > max_clean_ratio) max_clean_ratio = ratio;
      }
    }
    for (int col = 0; col < valid_cols; ++col) {
      float actual = 0.0f;
      for (int r = 0; r < valid_rows; ++r) actual += c[c_index(tile_row * tile + r, tile_col * tile + col, m, n, c_layout)];
      float delta = expected_cols[(size_t)tile_id * tile + col] - actual;
      float thr = threshold(abs_tol, rel_tol, col_scales[(size_t)tile_id * tile + col]);
      float margin = fabsf(fabsf(delta) - thr) / thr;
      if (margin < tile_margin) tile_margin = margin;
      if (fabsf(delta) > thr) {
        if (nbc == 0) {
          bad_col = col;
          bad_col_delta = delta;
        }
        ++nbc;
      } else {
        float ratio = fabsf(delta) / thr;
        if (ratio > max_clean_ratio) max_clean_ratio = ratio;
      }
    }
    if (tile_margin < min_margin) min_margin = tile_margin;
    int is_bad = or_rule ? (nbr > 0 || nbc > 0) : (nbr > 0 && nbc > 0);
    int corrected = 0;
    if (nbr == 1 && nbc == 1) {
      size_t idx = c_index(tile_row * tile + bad_row, tile_col * tile + bad_col, m, n, c_layout);
      c[idx] = fmaf(0.5f, bad_row_delta + bad_col_delta, c[idx]);
      corrected = 1;
    }
    bad_tiles += is_bad;
    corrected_tiles += corrected;
    multi += is_bad && !corrected;
    if ((is_bad || corrected) && records != NULL) {
      int slot;
#pragma omp atomic capture
      slot = n_records++;
      if (slot < max_records) {
        ftq_tile_record rec = {(int)tile_id, nbr, nbc, bad_row, bad_col, bad_row_delta, bad_col_delta, corrected, tile_margin};
        records[slot] = rec;
      }
    }
  }
  if (records != NULL) {
    int kept = n_records < max_records ? n_records : max_records;
    /* records arrive in thread order: sort by tile id (insertion sort, few entries) */
    for (int i = 1; i < kept; ++i) {
      ftq_tile_record key = records[i];
      int j = i - 1;
      while (j >= 0 && records[j].tile > key.tile) {
        records[j + 1] = records[j];
        --j;
      }
      records[j + 1] = key;
    }
    n_records = kept;
  }
  if (summary != NULL) {
    summary->bad_tiles = bad_tiles;
    summary->corrected_tiles = corrected_tiles;
    summary->multi_fault_tiles = multi;
    summary->n_records = n_records;
    summary->max_clean_ratio = max_clean_ratio;
    summary->min_margin = min_margin;
  }
}

/* ------------------------------------------------------------------------ */
/* campaign, sampled verifier                                                */
/* ------------------------------------------------------------------------ */

/* src/s4_random_fault_campaign.cu:755-769 */
void ftq_campaign_next(uint32_t* state, int trial, int tile_count, int tile, float min_value, float max_value,
                       ftq_campaign_draw* out) {
  uint32_t s = *state;
  s = ftq_mix_u32(s + 0x9e3779b9U + (uint32_t)trial);
  out->tile = (int)(s % (uint32_t)tile_count);
  s = ftq_mix_u32(s);
  out->row = (int)(s % (uint32_t)tile);
  s = ftq_mix_u32(s);
  out->col = (int)(s % (uint32_t)tile);
  s = ftq_mix_u32(s);
  float unit = (float)(s & 0x00ffffffU) / 16777215.0f;
  out->unit = unit;
  out->magnitude = min_value + (max_value - min_value) * unit;
  int bin = (int)(4 * unit);
  out->bin = max_value == min_value ? 0 : (bin < 3 ? bin : 3);
  s = ftq_mix_u32(s);
  out->signed_value = (s & 1U) == 0 ? out->magnitude : -out->magnitude;
  *state = s;
}

/* src/s4_cluster_multicast_abft_fp8_gemm.cu:527-554 */
void ftq_verify_samples(const uint8_t* a, const uint8_t* b, const float* c, int m, int n, int k, int samples, float abs_tol,
                        float rel_tol, int b_layout, int c_layout, ftq_verify_result* out) {
  out->max_absolute_error = 0.0f;
  out->max_tolerance_ratio = 0.0f;
  out->checked = 0;
  if (samples == 0) return;
  int row_step = m / samples > 1 ? m / samples : 1;
  int col_step = n / samples > 1 ? n / samples : 1;
  int checked_rows = 0;
  for (int row = 0; row < m && checked_rows < samples; row += row_step, ++checked_rows) {
    int checked_cols = 0;
    for (int col = 0; col < n && checked_cols < samples; col += col_step, ++checked_cols) {
      double reference = ftq_dot_f64(a, b, row, col, n, k, b_layout);
      float absolute_error = (float)fabs(c[c_index(row, col, m, n, c_layout)] - reference);
      float tolerance = abs_tol + rel_tol * fmaxf(1.0f, (float)fabs(reference));
      if (absolute_error > out->max_absolute_error) out->max_absolute_error = absolute_error;
      if (absolute_error / tolerance > out->max_tolerance_ratio) out->max_tolerance_ratio = absolute_error / tolerance;
      ++out->checked;
    }
  }
}

/* ------------------------------------------------------------------------ */
/* timed whole-path pass (CPU baseline)                                      */
/* ------------------------------------------------------------------------ */

static double now_seconds(void) {
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (double)ts.tv_sec + 1e-9 * (double)ts.tv_nsec;
}

int ftq_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Number of OpenMP threads of the following calls (a launcher may have set OMP_NUM_THREADS=1 for its children). */
void ftq_set_num_threads(int threads) {
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
#else
  (void)threads;
#endif
}

void ftq_full_pass(const uint8_t* a, const uint8_t* b, float* c, int m_rows, int n, int k, int tile, float abs_tol,
                   float rel_tol, double* seconds3, ftq_check_summary* summary) {
  int tile_rows = m_rows / tile, tile_cols = (n + tile - 1) / tile;
  size_t checks = (size_t)tile_rows * tile_cols * tile;
  float* a_sums = (float*)malloc((size_t)tile_rows * k * sizeof(float));
  float* a_mags = (float*)malloc((size_t)tile_rows * k * sizeof(float));
  float* b_sums = (float*)malloc((size_t)tile_cols * k * sizeof(float));
  float* b_mags = (float*)malloc((size_t)tile_cols * k * sizeof(float));
  float* er = (float*)malloc(checks * sizeof(float));
  float* ec = (float*)malloc(checks * sizeof(float));
  float* sr = (float*)malloc(checks * sizeof(float));
  float* sc = (float*)malloc(checks * sizeof(float));
  double t0 = now_seconds();
  ftq_band_sums(a, b, a_sums, a_mags, b_sums, b_mags, m_rows, n, k, tile);
  ftq_expected_from_bands(a, b, a_sums, a_mags, b_sums, b_mags, er, ec, sr, sc, m_rows, n, k, tile);
  double t1 = now_seconds();
  ftq_gemm_f32(a, b, c, m_rows, n, k, FTQ_B_NK, FTQ_C_COLMAJOR);
  double t2 = now_seconds();
  ftq_abft_check(c, m_rows, n, tile, FTQ_C_COLMAJOR, er, ec, sr, sc, abs_tol, rel_tol, 1, NULL, 0, NULL, 0, summary);
  double t3 = now_seconds();
  seconds3[0] = t1 - t0;
  seconds3[1] = t2 - t1;
  seconds3[2] = t3 - t2;
  free(a_sums);
  free(a_mags);
  free(b_sums);
  free(b_mags);
  free(er);
  free(ec);
  free(sr);
  free(sc);
}
