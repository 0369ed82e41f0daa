/*
 * ft_attention.h -- C-ABI of the fault-tolerant flash-attention forward on B200.
 *
 * The reference project's attention chain (src/ft_flash_attention_a0.cu ...
 * a14.cu) is, like its GEMM stages, a set of standalone programs: main() prepares
 * K/V metadata (prepare_attention_metadata_kernel, transpose_v_kernel;
 * src/ft_flash_attention_a14.cu:303-316, 571-621), launches the fused forward
 * kernel with a fault description (a14:659-1201, parameters a14:640-657) and reads
 * nine counters back (DeviceStats, a14:98-108).  The entry points below are that
 * launch interface.
 *
 * Operator: O[b,h,q,:] = softmax(Q K^T / sqrt(D)) V, causal (ft_attn_options.causal,
 * a14:708, 893) or not, for
 *   Q, K, V  [B, H, N, D]  FP16, D contiguous       (the reference uses FP8 E4M3)
 *   O        [B, H, N, D]  FP32
 *   D == 64 or 128 (a14:267), any N >= 1 (the handle keeps zero-padded copies of
 *   Q, K, V when N is not a multiple of the 128-row tile; O keeps the caller's N)
 * Protection:
 *   - score stage: every 64x64 tile of S = Q K^T is checked with the SAME row /
 *     column checksum verifier as the GEMM (expected_row = Q rowsum(K-tile),
 *     expected_col = colsum(Q-tile) K^T, cached by _prepare); a single faulty score
 *     is located at the row/column intersection and corrected in registers before
 *     the softmax; a tile with several bad rows or columns is recomputed without
 *     the tensor core, checked again and counted as replayed (a14:935-959), or as
 *     uncorrected when the recomputed tile still fails the check;
 *   - output stage: the reference's projection check of P V (a0:585-662): the
 *     expected sum and position-weighted sum of each output row are carried
 *     through the online softmax from per-key sums of V, a single faulty output
 *     element is located by the ratio of the two deltas and corrected, anything
 *     else counts as a failed row.
 */
#ifndef FT_ATTENTION_H
#define FT_ATTENTION_H

#include <stddef.h>
#include <stdint.h>

#include "ft_gemm.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ft_attn_handle ft_attn_handle;

typedef struct {
  float score_abs_tol; /* default 1e-2: |delta| > abs + rel * max(1, scale), as in the GEMM (src/s4:467) */
  float score_rel_tol; /* default 2e-5 */
  float pv_abs_tol;    /* default 2e-3 (src/ft_flash_attention_a0.cu:63-64) */
  float pv_rel_tol;    /* default 2e-3 */
  float softmax_abs_tol; /* default 2e-5 (src/ft_flash_attention_a0.cu:61-62) */
  float softmax_rel_tol; /* default 2e-5 */
  int protect_softmax;   /* 0 (default): score and output stages only; 1: also the reference's softmax-stage
                            protection (verifier copies of the exponent reference and of every probability, moment
                            check with location, duplicate of the running state; about 1.5x the time) */
  int causal;            /* 0 (default): every key; 1: key <= query only (src/ft_flash_attention_a14.cu:130, 708, 836):
                            key tiles beyond the diagonal are skipped, the diagonal tile is verified unmasked and
                            masked afterwards; score / softmax faults must then have index <= query (a14:278) */
  int exact_prepare;     /* 0 (default): the expected score checksums are computed on the tensor cores from FP16 pieces of the
                            band sums (absolute error below 2^-17 per band-sum element); 1: on the CUDA cores in the
                            reference GEMM's summation order (src/s4:264-282), about 10x slower */
} ft_attn_options;

/* Fault stages use the reference's numbering (src/ft_flash_attention_a0.cu:27-33);
 * the softmax stages can be targeted only when protect_softmax is set. */
#define FT_ATTN_FAULT_NONE 0
#define FT_ATTN_FAULT_SCORE 1  /* value added to S[query, index=key] after Q K^T */
#define FT_ATTN_FAULT_SOFTMAX 2       /* value added to the probability of key `index` (needs protect_softmax) */
#define FT_ATTN_FAULT_SOFTMAX_STATE 3 /* value added to the running sum l in the tile holding key `index` (needs protect_softmax) */
#define FT_ATTN_FAULT_OUTPUT 4 /* value added to the normalised O[query, index=dim] */

typedef struct {
  int stage;
  int batch;
  int head;
  int query;
  int index;
  float value;
  /* A second fault of the score stage in the same (batch, head), for runs that must show a tile with several faults
   * (the reference injects one fault per run; its replay path, src/ft_flash_attention_a14.cu:935-959, is reached by
   * faults its row locator cannot place).  Ignored unless stage == FT_ATTN_FAULT_SCORE and value2 != 0. */
  int query2;
  int index2;
  float value2;
} ft_attn_fault;

typedef struct {
  int status;            /* FT_OK or FT_ERR_TIMEOUT */
  int score_detected;    /* score tiles whose checker fired */
  int score_corrected;   /* of which: one bad row and one bad column, corrected */
  int score_uncorrected; /* of which: not locatable, and the replayed tile still disagrees with the cached checksums */
  int pv_detected;       /* output rows whose projection check fired */
  int pv_corrected;
  int failed_rows;       /* output rows detected but not locatable */
  int softmax_detected;  /* (row, key tile) pairs whose moment or state check fired (protect_softmax) */
  int softmax_corrected; /* of which: one probability located and replaced by the verifier's */
  int softmax_replayed;  /* of which: the row of the tile, or the running state, taken from the verifier */
  int score_replayed;    /* score tiles whose fault could not be located (several bad rows or columns): recomputed on
                            the CUDA cores from Q and K, verified again and accepted (src/ft_flash_attention_a14.cu:935-959) */
  int n_records;
  float max_score_noise; /* max |delta|/threshold over score checksums that passed */
  float prepare_ms;
  /* score-tile records: tile = ((batch*heads + head) * (N/64) + q_band) * (N/64) + key_band */
  ft_tile_record records[16];
} ft_attn_report;

void ft_attn_options_default(ft_attn_options* options);

/* Replaces the reference's metadata allocation and prepare launches
 * (src/ft_flash_attention_a14.cu:1369-1430): builds V^T, the per-key sums of V and
 * the expected row/column checksums of every 64x64 score tile.  The cache is valid
 * while Q, K and V are unchanged; it is owned by the handle. */
int ft_attention_fp16_abft_prepare(ft_attn_handle** handle, const void* q, const void* k, const void* v, int batch, int heads,
                                   int sequence, int head_dim, const ft_attn_options* options, void* stream);

/* Rebuilds the metadata (V^T with its checksum rows, band sums, the score-checksum cache) for new contents of Q, K, V of the
 * shape given to _prepare, without allocating: what a forward pass calls when its operands changed, which in attention is
 * every call.  The pointers may differ from those given to _prepare (16-byte aligned).  Replaces re-running the metadata
 * kernels of the reference's main() (src/ft_flash_attention_a14.cu:1294-1322, 1369-1430) on the buffers it already holds.
 * Asynchronous on `stream`; a later _run on the same stream sees the new metadata. */
int ft_attention_fp16_abft_refresh(ft_attn_handle* handle, const void* q, const void* k, const void* v, void* stream);

/* Replaces one launch of the fused forward kernel with its fault parameters
 * (src/ft_flash_attention_a14.cu:1324-1359).  Asynchronous; `fault` may be NULL. */
int ft_attention_fp16_abft_run(ft_attn_handle* handle, float* out, const ft_attn_fault* fault, void* stream);

/* Replaces the read-back of DeviceStats (src/ft_flash_attention_a14.cu:1437-1440). */
int ft_attention_fp16_abft_report(ft_attn_handle* handle, ft_attn_report* out);

int ft_attention_fp16_abft_destroy(ft_attn_handle* handle);

/* Seeded FP16 inputs on the device.  dist 0: the grid ((mix(seed+i) % 17) - 8) / 16
 * of the reference's attention generator (src/ft_flash_attention_a0.cu:231-238);
 * dist 1: N(0, sigma^2).  The reference seeds Q, K, V with 0x12345678, 0x9abcdef0,
 * 0x31415926 (a0:771-773). */
int ft_attention_generate_f16(void* out_f16, size_t count, uint32_t seed, int dist, float sigma, void* stream);

#ifdef __cplusplus
}
#endif
#endif
