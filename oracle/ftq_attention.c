/*
 * CPU oracle for the fault-tolerant attention forward.  TEST INFRASTRUCTURE ONLY
 * (same rules as ftq_oracle.c).  Compile with -ffp-contract=off.
 *
 * What it restates:
 *   - score stage: S = Q K^T per head is a GEMM with A = Q [N,D], B = K [N,D]; its
 *     64x64 tiles are verified with the reference's GEMM checker -- band sums
 *     (src/s4_cluster_multicast_abft_fp8_gemm.cu:194-235), expected checksums with
 *     the lane-strided partial sums and shuffle-down tree (src/s4:237-294), compare
 *     and single-point correction (src/s4:456-499) -- on FP16 operands;
 *   - online softmax over 128-key tiles in FP32 (src/ft_flash_attention_a0.cu:
 *     456-470 for the recurrence), probabilities rounded to FP16 before P V;
 *   - output stage: the reference's projection check, V metadata
 *     (src/ft_flash_attention_a14.cu:600-620), expected sum / position-weighted sum
 *     carried through the recurrence (a0:585-611), compare, locate by the ratio of
 *     the deltas, correct or count a failed row (a0:613-662).
 *
 * Parity status of this part: PINNED WITHIN TOLERANCE against the reference's own
 * scalar attention kernel (src/ft_flash_attention_a0.cu:285-667), run unmodified on a
 * B200 by oracle/ref_harness_a0.cu; fixtures tests/golden/a0_*.npz (head dimensions
 * 128 and 64, causal and not, every fault stage).  Inputs agree bit for bit (the
 * reference's grid values are exact in FP16), outputs within 2e-3 (FP16
 * probabilities here, FP32 there) for clean runs and for every recovered fault, the
 * per-stage counters are equal.  A bit-for-bit comparison is not possible: the
 * reference's attention programs take FP8 inputs and protect the score stage with
 * per-row projections, while the FP16 inputs and the 2-D tile checksums used here
 * are the variant this build was asked for.  The GEMM checker it reuses is pinned bit
 * for bit (tests/test_golden_cpu.py).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "ftq_oracle.h"

typedef struct {
  int score_detected, score_corrected, score_uncorrected;
  int pv_detected, pv_corrected, failed_rows;
  int softmax_detected, softmax_corrected, softmax_replayed;
  int n_records;
  float max_score_noise;
  float min_margin; /* nearest score-stage decision to its threshold, relative */
  int score_replayed; /* tiles whose fault could not be located: recomputed, verified again and accepted */
} ftq_attn_stats;

float ftq_half_to_float(uint16_t h) {
  uint32_t sign = (uint32_t)(h >> 15) << 31, e = (h >> 10) & 31, m = h & 1023;
  float f;
  if (e == 0) {
    f = ldexpf((float)m, -24);
  } else if (e == 31) {
    f = m ? NAN : INFINITY;
  } else {
    f = ldexpf(1.0f + (float)m / 1024.0f, (int)e - 15);
  }
  uint32_t bits;
  memcpy(&bits, &f, 4);
  bits |= sign;
  memcpy(&f, &bits, 4);
  return f;
}

/* round to nearest even, overflow to infinity (cvt.rn.f16.f32) */
uint16_t ftq_float_to_half(float x) {
  uint32_t bits;
  memcpy(&bits, &x, 4);
  uint16_t sign = (uint16_t)((bits >> 16) & 0x8000);
  if ((bits & 0x7fffffffu) > 0x7f800000u) return (uint16_t)(sign | 0x7e00);
  float ax = fabsf(x);
  if (ax >= 65520.0f) return (uint16_t)(sign | 0x7c00);
  if (ax == 0.0f) return sign;
  int e;
  (void)frexpf(ax, &e);
  int ex = e - 1;
  if (ex < -14) ex = -14;
  float q = ldexpf(1.0f, ex - 10);
  float r = nearbyintf(ax / q); /* 0 .. 2048 */
  if (r == 2048.0f) {
    ex += 1;
    r = 1024.0f;
  }
  int ri = (int)r;
  if (ri < 1024) return (uint16_t)(sign | ri); /* subnormal */
  return (uint16_t)(sign | ((ex + 15) << 10) | (ri - 1024));
}

static inline float tree32(float* p) {
  for (int offset = 16; offset > 0; offset /= 2)
    for (int i = 0; i < offset; ++i) p[i] = p[i] + p[i + offset];
  return p[0];
}

/* expected = sum_k x[k] * y[k] in the order of src/s4:264-282 */
static inline void strided_dot(const float* x, const float* y, const float* ymag, int k, int x_first, float* expected, float* scale) {
  float pe[32], ps[32];
  for (int l = 0; l < 32; ++l) pe[l] = ps[l] = 0.0f;
  for (int kk = 0; kk < k; ++kk) {
    int l = kk & 31;
    if (x_first) {
      pe[l] = fmaf(x[kk], y[kk], pe[l]);
      ps[l] = fmaf(fabsf(x[kk]), ymag[kk], ps[l]);
    } else {
      pe[l] = fmaf(y[kk], x[kk], pe[l]);
      ps[l] = fmaf(ymag[kk], fabsf(x[kk]), ps[l]);
    }
  }
  *expected = tree32(pe);
  *scale = tree32(ps);
}

static inline float threshold(float abs_tol, float rel_tol, float scale) { return fmaf(rel_tol, fmaxf(1.0f, scale), abs_tol); }

/* band sums over 64 rows of x [rows, d] (src/s4:199-211) */
static void band_sums_f32(const float* x, int rows, int d, float* sums, float* mags) {
  for (int band = 0; band < rows / 64; ++band)
    for (int kk = 0; kk < d; ++kk) {
      float sum = 0.0f, magnitude = 0.0f;
      for (int r = 0; r < 64; ++r) {
        float value = x[(size_t)(band * 64 + r) * d + kk];
        sum += value;
        magnitude += fabsf(value);
      }
      sums[(size_t)band * d + kk] = sum;
      mags[(size_t)band * d + kk] = magnitude;
    }
}

/*
 * Forward for all heads.  Q, K, V: [B*H, N, D] FP16 bit patterns; out: [B*H, N, D].
 * fault_stage 0 none, 1 score (value added to S[query, index]), 2 softmax (value
 * added to the probability of key index), 3 softmax-state (value added to the running
 * sum l in the tile holding key index), 4 output (value added to the normalised
 * O[query, index]); numbering of src/ft_flash_attention_a0.cu:27-33.  Stages 2 and 3
 * act only with protect_softmax, which adds the reference's softmax-stage protection
 * (src/ft_flash_attention_a14.cu:964-1099): verifier probabilities, the moments
 * sum p, sum w p, sum w^2 p of the FP16-rounded probabilities, single-point
 * replacement or replay of the row, and a duplicate of the running state.
 * seq is a multiple of 128; valid_seq <= seq is the real sequence length: the rows
 * valid_seq..seq-1 of q, k, v are zero padding, their keys are masked like the
 * causal ones (a14:893 masks by index) and their queries leave no output row and
 * no output-stage counters; out is [batch_heads, valid_seq, dim].
 * records (may be NULL): score tiles whose checker fired, tile id =
 * ((bh * N/64) + q_band) * N/64 + key_band, sorted by tile id.
 */
void ftq_attention_forward(const uint16_t* q16, const uint16_t* k16, const uint16_t* v16, int batch_heads, int seq, int valid_seq, int dim,
                           float score_abs, float score_rel, float pv_abs, float pv_rel, float softmax_abs, float softmax_rel,
                           int protect_softmax, int causal, int fault_stage, int fault_bh,
                           int fault_query, int fault_index, float fault_value, int fault2_query, int fault2_index, float fault2_value,
                           float* out, ftq_attn_stats* stats, ftq_tile_record* records, int max_records) {
  const int bands = seq / 64;
  const float scale_log2 = 1.44269504088896340736f / sqrtf((float)dim);
  int score_detected = 0, score_corrected = 0, score_uncorrected = 0, pv_detected = 0, pv_corrected = 0, failed_rows = 0;
  int softmax_detected = 0, softmax_corrected = 0, softmax_replayed = 0, score_replayed = 0;
  int n_records = 0;
  float max_noise = 0.0f, min_margin = INFINITY;

#pragma omp parallel for schedule(dynamic, 1) reduction(+ : score_detected, score_corrected, score_uncorrected, pv_detected, \
                                                            pv_corrected, failed_rows, softmax_detected, softmax_corrected, \
                                                            softmax_replayed, score_replayed) reduction(max : max_noise)   \
    reduction(min : min_margin)
  for (int bh = 0; bh < batch_heads; ++bh) {
    const size_t head = (size_t)bh * seq * dim;
    float* qf = (float*)malloc((size_t)seq * dim * sizeof(float));
    float* kf = (float*)malloc((size_t)seq * dim * sizeof(float));
    float* vf = (float*)malloc((size_t)seq * dim * sizeof(float));
    for (size_t i = 0; i < (size_t)seq * dim; ++i) {
      qf[i] = ftq_half_to_float(q16[head + i]);
      kf[i] = ftq_half_to_float(k16[head + i]);
      vf[i] = ftq_half_to_float(v16[head + i]);
    }
    float* q_sums = (float*)malloc((size_t)bands * dim * sizeof(float));
    float* q_mags = (float*)malloc((size_t)bands * dim * sizeof(float));
    float* k_sums = (float*)malloc((size_t)bands * dim * sizeof(float));
    float* k_mags = (float*)malloc((size_t)bands * dim * sizeof(float));
    band_sums_f32(qf, seq, dim, q_sums, q_mags);
    band_sums_f32(kf, seq, dim, k_sums, k_mags);
    /* per-key sums of V (a14:606-619) */
    float* v_sum = (float*)malloc((size_t)seq * sizeof(float));
    float* v_weighted = (float*)malloc((size_t)seq * sizeof(float));
    for (int key = 0; key < seq; ++key) {
      float sum = 0.0f, weighted = 0.0f;
      for (int d = 0; d < dim; ++d) {
        float value = vf[(size_t)key * dim + d];
        sum += value;
        weighted = fmaf((float)(2 * d - (dim - 1)), value, weighted);
      }
      v_sum[key] = sum;
      v_weighted[key] = weighted;
    }
    float* s = (float*)malloc((size_t)64 * 128 * sizeof(float));    /* one 64-query band x 128 keys */
    float* acc = (float*)malloc((size_t)64 * dim * sizeof(float));  /* unnormalised output of the band */
    float m_run[64], l_run[64], e_sum[64], e_weighted[64];
    float u1_run[64], u2_run[64], m_ver[64], l_ver[64], u1_ver[64], u2_ver[64];
    float ph[128], qh[128];

    for (int qb = 0; qb < bands; ++qb) { /* the two 64-row bands of a 128-query CTA are independent */
      for (int r = 0; r < 64; ++r) {
        m_run[r] = m_ver[r] = -INFINITY;
        l_run[r] = e_sum[r] = e_weighted[r] = 0.0f;
        u1_run[r] = u2_run[r] = l_ver[r] = u1_ver[r] = u2_ver[r] = 0.0f;
      }
      memset(acc, 0, (size_t)64 * dim * sizeof(float));
      /* causal (a14:708): the band's 128-query tile stops after the key tile on its diagonal */
      const int key_tiles = causal ? (qb * 64) / 128 + 1 : seq / 128;
      for (int j = 0; j < key_tiles; ++j) {
        /* S tile: FP32 accumulate, ascending d */
        for (int r = 0; r < 64; ++r)
          for (int c = 0; c < 128; ++c) {
            const float* qr = qf + (size_t)(qb * 64 + r) * dim;
            const float* kr = kf + (size_t)(j * 128 + c) * dim;
            float a = 0.0f;
            for (int d = 0; d < dim; ++d) a = fmaf(qr[d], kr[d], a);
            s[r * 128 + c] = a;
          }
        if (fault_stage == 1 && fault_bh == bh && fault_query / 64 == qb && fault_index / 128 == j)
          s[(fault_query % 64) * 128 + fault_index % 128] += fault_value;
        if (fault_stage == 1 && fault_bh == bh && fault2_value != 0.0f && fault2_query / 64 == qb && fault2_index / 128 == j)
          s[(fault2_query % 64) * 128 + fault2_index % 128] += fault2_value;
        /* verify the two 64x64 tiles */
        for (int c2 = 0; c2 < 2; ++c2) {
          int kb = j * 2 + c2;
          int nbr = 0, nbc = 0, bad_row = -1, bad_col = -1;
          float row_delta = 0.0f, col_delta = 0.0f;
          int first_nbr = 0, first_nbc = 0, first_bad_row = -1, first_bad_col = -1, replayed_tile = 0;
          float first_row_delta = 0.0f, first_col_delta = 0.0f;
          /* pass 0: the tile as the tensor core (and the fault hook) left it; pass 1, only when the fault of pass 0
           * cannot be located: the tile recomputed without the tensor core (a14:935-959) and checked again */
          for (int pass = 0; pass < 2; ++pass) {
            nbr = nbc = 0;
            bad_row = bad_col = -1;
            row_delta = col_delta = 0.0f;
            for (int r = 0; r < 64; ++r) {
              float expected, scale, actual = 0.0f;
              strided_dot(qf + (size_t)(qb * 64 + r) * dim, k_sums + (size_t)kb * dim, k_mags + (size_t)kb * dim, dim, 1, &expected, &scale);
              for (int c = 0; c < 64; ++c) actual += s[r * 128 + c2 * 64 + c];
              float delta = expected - actual, thr = threshold(score_abs, score_rel, scale);
              float margin = fabsf(fabsf(delta) - thr) / thr;
              if (margin < min_margin) min_margin = margin;
              if (fabsf(delta) > thr) {
                if (nbr++ == 0) {
                  bad_row = r;
                  row_delta = delta;
                }
              } else if (pass == 0 && fabsf(delta) / thr > max_noise) {
                max_noise = fabsf(delta) / thr;
              }
            }
            for (int c = 0; c < 64; ++c) {
              float expected, scale, actual = 0.0f;
              strided_dot(kf + (size_t)(kb * 64 + c) * dim, q_sums + (size_t)qb * dim, q_mags + (size_t)qb * dim, dim, 0, &expected, &scale);
              for (int r = 0; r < 64; ++r) actual += s[r * 128 + c2 * 64 + c];
              float delta = expected - actual, thr = threshold(score_abs, score_rel, scale);
              float margin = fabsf(fabsf(delta) - thr) / thr;
              if (margin < min_margin) min_margin = margin;
              if (fabsf(delta) > thr) {
                if (nbc++ == 0) {
                  bad_col = c;
                  col_delta = delta;
                }
              } else if (pass == 0 && fabsf(delta) / thr > max_noise) {
                max_noise = fabsf(delta) / thr;
              }
            }
            if (pass == 0) {
              first_nbr = nbr, first_nbc = nbc, first_bad_row = bad_row, first_bad_col = bad_col;
              first_row_delta = row_delta, first_col_delta = col_delta;
              if ((nbr == 0 && nbc == 0) || (nbr == 1 && nbc == 1)) break;
              for (int r = 0; r < 64; ++r)
                for (int c = 0; c < 64; ++c) {
                  const float* qr = qf + (size_t)(qb * 64 + r) * dim;
                  const float* kr = kf + (size_t)(j * 128 + c2 * 64 + c) * dim;
                  float a = 0.0f;
                  for (int d = 0; d < dim; ++d) a = fmaf(qr[d], kr[d], a);
                  s[r * 128 + c2 * 64 + c] = a;
                }
            } else {
              replayed_tile = nbr == 0 && nbc == 0;
            }
          }
          nbr = first_nbr, nbc = first_nbc, bad_row = first_bad_row, bad_col = first_bad_col;
          row_delta = first_row_delta, col_delta = first_col_delta;
          if (nbr > 0 || nbc > 0) {
            int corrected = nbr == 1 && nbc == 1;
            if (corrected) s[bad_row * 128 + c2 * 64 + bad_col] = fmaf(0.5f, row_delta + col_delta, s[bad_row * 128 + c2 * 64 + bad_col]);
            ++score_detected;
            score_corrected += corrected;
            score_replayed += !corrected && replayed_tile;
            score_uncorrected += !corrected && !replayed_tile;
            if (records != NULL) {
              int slot;
#pragma omp atomic capture
              slot = n_records++;
              if (slot < max_records) {
                ftq_tile_record rec = {(bh * bands + qb) * bands + kb, nbr, nbc, bad_row, bad_col, row_delta, col_delta, corrected, 0.0f};
                records[slot] = rec;
              }
            }
          }
        }
        /* causal mask (a14:893), applied after the verifier has seen the raw tile: exp2(-inf) = 0 below */
        if (causal)
          for (int r = 0; r < 64; ++r)
            for (int c = 0; c < 128; ++c)
              if (j * 128 + c > qb * 64 + r) s[r * 128 + c] = -INFINITY;
        if ((j + 1) * 128 > valid_seq)
          for (int r = 0; r < 64; ++r)
            for (int c = 0; c < 128; ++c)
              if (j * 128 + c >= valid_seq) s[r * 128 + c] = -INFINITY;
        /* online softmax, FP16 probabilities, P V and the expected projections */
        for (int r = 0; r < 64; ++r) {
          float row_max = -INFINITY;
          for (int c = 0; c < 128; ++c) row_max = fmaxf(row_max, s[r * 128 + c]);
          float m_new = fmaxf(m_run[r], row_max * scale_log2);
          float alpha = exp2f(m_run[r] - m_new);
          float* o = acc + (size_t)r * dim;
          for (int d = 0; d < dim; ++d) o[d] *= alpha;
          int query = qb * 64 + r;
          int target = fault_bh == bh && fault_query == query && fault_index / 128 == j;
          float m_check = m_new, alpha_check = alpha;
          if (protect_softmax) {
            m_check = fmaxf(m_ver[r], row_max * scale_log2);
            alpha_check = exp2f(m_ver[r] - m_check);
          }
          /* FP16-rounded primary (ph) and verifier (qh) probabilities */
          for (int c = 0; c < 128; ++c) {
            float pr = exp2f(fmaf(s[r * 128 + c], scale_log2, -m_new));
            if (protect_softmax && fault_stage == 2 && target && fault_index % 128 == c) pr += fault_value;
            ph[c] = ftq_half_to_float(ftq_float_to_half(pr));
            qh[c] = protect_softmax ? ftq_half_to_float(ftq_float_to_half(exp2f(fmaf(s[r * 128 + c], scale_log2, -m_check)))) : ph[c];
          }
          float l_tile = 0.0f, u1 = 0.0f, u2 = 0.0f, c0 = 0.0f, c1 = 0.0f, c2 = 0.0f;
          for (int attempt = 0; attempt < 2; ++attempt) {
            l_tile = u1 = u2 = c0 = c1 = c2 = 0.0f;
            for (int c = 0; c < 128; ++c) {
              float w = (float)(2 * (j * 128 + c) - (seq - 1));
              l_tile += ph[c];
              u1 = fmaf(w, ph[c], u1);
              u2 = fmaf(w, w * ph[c], u2);
              c0 += qh[c];
              c1 = fmaf(w, qh[c], c1);
              c2 = fmaf(w, w * qh[c], c2);
            }
            if (!protect_softmax || attempt == 1) break;
            float d0 = l_tile - c0, d1 = u1 - c1, d2 = u2 - c2;
            if (!(fabsf(d0) > threshold(softmax_abs, softmax_rel, fabsf(c0)) || fabsf(d1) > threshold(softmax_abs, softmax_rel, fabsf(c1)) ||
                  fabsf(d2) > threshold(softmax_abs, softmax_rel, fabsf(c2))))
              break;
            ++softmax_detected;
            int action = 2, key = -1;
            if (fabsf(d0) > threshold(softmax_abs, softmax_rel, fabsf(c0))) {
              float observed = d1 / d0;
              int key_index = (int)nearbyintf(0.5f * (observed + (float)(seq - 1)));
              float second = fabsf(d2 / d0 - observed * observed);
              if (key_index >= j * 128 && key_index < (j + 1) * 128 && fabsf(observed - (float)(2 * key_index - (seq - 1))) <= 0.25f &&
                  second <= fmaxf(1.0f, fabsf(observed)) * 0.5f) {
                action = 1;
                key = key_index - j * 128;
              }
            }
            if (action == 1) {
              ++softmax_corrected;
              ph[key] = qh[key];
            } else {
              ++softmax_replayed;
              memcpy(ph, qh, sizeof(ph));
            }
          }
          float es = 0.0f, ew = 0.0f;
          for (int c = 0; c < 128; ++c) {
            es = fmaf(ph[c], v_sum[j * 128 + c], es);
            ew = fmaf(ph[c], v_weighted[j * 128 + c], ew);
            const float* vr = vf + (size_t)(j * 128 + c) * dim;
            for (int d = 0; d < dim; ++d) o[d] = fmaf(ph[c], vr[d], o[d]);
          }
          l_run[r] = fmaf(alpha, l_run[r], l_tile);
          e_sum[r] = fmaf(alpha, e_sum[r], es);
          e_weighted[r] = fmaf(alpha, e_weighted[r], ew);
          if (protect_softmax) {
            u1_run[r] = fmaf(alpha, u1_run[r], u1);
            u2_run[r] = fmaf(alpha, u2_run[r], u2);
            l_ver[r] = fmaf(alpha_check, l_ver[r], c0);
            u1_ver[r] = fmaf(alpha_check, u1_ver[r], c1);
            u2_ver[r] = fmaf(alpha_check, u2_ver[r], c2);
            m_ver[r] = m_check;
            if (fault_stage == 3 && target) l_run[r] += fault_value;
            if ((m_new != m_ver[r] && fabsf(m_new - m_ver[r]) > threshold(softmax_abs, softmax_rel, fabsf(m_ver[r]))) ||
                fabsf(l_run[r] - l_ver[r]) > threshold(softmax_abs, softmax_rel, fabsf(l_ver[r])) ||
                fabsf(u1_run[r] - u1_ver[r]) > threshold(softmax_abs, softmax_rel, fabsf(u1_ver[r])) ||
                fabsf(u2_run[r] - u2_ver[r]) > threshold(softmax_abs, softmax_rel, fabsf(u2_ver[r]))) {
              ++softmax_detected;
              ++softmax_replayed;
              l_run[r] = l_ver[r];
              u1_run[r] = u1_ver[r];
              u2_run[r] = u2_ver[r];
            }
          }
          m_run[r] = m_new;
        }
      }
      /* output stage (a0:613-662) */
      for (int r = 0; r < 64; ++r) {
        int query = qb * 64 + r;
        if (query >= valid_seq) continue;
        float inv_l = 1.0f / l_run[r];
        float* o = acc + (size_t)r * dim;
        float actual_sum = 0.0f, actual_weighted = 0.0f;
        for (int d = 0; d < dim; ++d) {
          o[d] = o[d] * inv_l;
          if (fault_stage == 4 && fault_bh == bh && fault_query == query && fault_index == d) o[d] += fault_value;
          actual_sum += o[d];
          actual_weighted = fmaf((float)(2 * d - (dim - 1)), o[d], actual_weighted);
        }
        float expected_sum = e_sum[r] * inv_l, expected_weighted = e_weighted[r] * inv_l;
        float delta_sum = actual_sum - expected_sum, delta_weighted = actual_weighted - expected_weighted;
        float thr_sum = threshold(pv_abs, pv_rel, fabsf(expected_sum)), thr_weighted = threshold(pv_abs, pv_rel, fabsf(expected_weighted));
        if (fabsf(delta_sum) > thr_sum || fabsf(delta_weighted) > thr_weighted) {
          ++pv_detected;
          int recover = -1;
          if (fabsf(delta_sum) > thr_sum) {
            float observed = delta_weighted / delta_sum;
            int d = (int)nearbyintf(0.5f * (observed + (float)(dim - 1)));
            if (d >= 0 && d < dim && fabsf(observed - (float)(2 * d - (dim - 1))) <= 0.25f) recover = d;
          }
          if (recover >= 0) {
            o[recover] -= delta_sum;
            ++pv_corrected;
          } else {
            ++failed_rows;
          }
        }
        memcpy(out + (size_t)bh * valid_seq * dim + (size_t)query * dim, o, (size_t)dim * sizeof(float));
      }
    }
    free(qf);
    free(kf);
    free(vf);
    free(q_sums);
    free(q_mags);
    free(k_sums);
    free(k_mags);
    free(v_sum);
    free(v_weighted);
    free(s);
    free(acc);
  }
  if (records != NULL) {
    int kept = n_records < max_records ? n_records : max_records;
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
  stats->score_detected = score_detected;
  stats->score_corrected = score_corrected;
  stats->score_uncorrected = score_uncorrected;
  stats->pv_detected = pv_detected;
  stats->pv_corrected = pv_corrected;
  stats->failed_rows = failed_rows;
  stats->softmax_detected = softmax_detected;
  stats->softmax_corrected = softmax_corrected;
  stats->softmax_replayed = softmax_replayed;
  stats->n_records = n_records;
  stats->max_score_noise = max_noise;
  stats->min_margin = min_margin;
  stats->score_replayed = score_replayed;
}
