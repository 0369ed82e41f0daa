// Internal interface between the attention C-ABI layer and its kernels.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/ft_attention.h"

namespace ftg {

// V^T carries, below the D rows of a head, kAttnVExtra rows of per-key constants for the output-stage check:
// row D: ones; D+1, D+2: FP16 hi and lo pieces of sum_d V[key, d]; D+3, D+4: hi and lo pieces of
// sum_d w_d V[key, d] / kAttnVWeightScale (w_d = 2d - (D-1); the division keeps the value inside the FP16 range);
// the rest zeros.  As extra columns of the PV product they give l and the two expected output projections.
constexpr int kAttnVExtra = 16;
constexpr float kAttnVWeightScale = 128.0f;

struct AttnDeviceReport {
  int status;
  int score_detected;
  int score_corrected;
  int score_uncorrected;
  int pv_detected;
  int pv_corrected;
  int failed_rows;
  int record_count;
  int max_noise_bits;
  int softmax_detected;
  int softmax_corrected;
  int softmax_replayed;
  int score_replayed;
  int pad[3];  // the counters above (64 bytes with this padding) are cleared before every run
  ft_tile_record records[16];
};

struct AttnParams {
  const float* expected_rows;  // [B*H][(N/64)^2][64]
  const float* expected_cols;
  const float* row_scales;
  const float* col_scales;
  const void* q;  // [B*H][N][D] FP16: read directly only when a score tile is replayed on the CUDA cores
  const void* k;
  const float* v_sum;       // [B*H][N]
  const float* v_weighted;  // [B*H][N]
  float* out;               // [B*H][N][D]
  AttnDeviceReport* report;
  int seq;        // keys and queries per head as the kernels see them: a multiple of 128
  int valid_seq;  // the caller's sequence length (<= seq): keys past it are masked, queries past it are not stored
  int dim;  // head dimension: 128, or 64 (split-row kernel only)
  float score_abs_tol, score_rel_tol, pv_abs_tol, pv_rel_tol, softmax_abs_tol, softmax_rel_tol;
  int protect_softmax;
  int causal;
  float scale_log2;  // log2(e) / sqrt(D)
  int fault_stage, fault_bh, fault_query, fault_index;
  float fault_value;
  int fault2_query, fault2_index;  // a second score fault in the same (batch, head); active when fault2_value != 0
  float fault2_value;
};

cudaError_t launch_attn_prepare_v(const void* v, void* vt, float* v_sum, float* v_weighted, int batch_heads, int seq, int dim,
                                  cudaStream_t stream);
cudaError_t launch_generate_f16(void* out, size_t count, uint32_t seed, int dist, float sigma, cudaStream_t stream);
cudaError_t configure_attention();
cudaError_t launch_attention(const CUtensorMap& tmap_q, const CUtensorMap& tmap_k, const CUtensorMap& tmap_vt, const AttnParams& params,
                             int batch_heads, cudaStream_t stream);
// the split-row form (two threads per query row; no softmax-stage protection): ft_attention_split.cu
cudaError_t configure_attention_split();
cudaError_t launch_attention_split(const CUtensorMap& tmap_q, const CUtensorMap& tmap_k, const CUtensorMap& tmap_vt, const AttnParams& params,
                                   int batch_heads, cudaStream_t stream);

}  // namespace ftg
