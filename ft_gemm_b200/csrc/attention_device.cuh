// Device helpers shared by the two attention forward kernels.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "abft_tile_check.cuh"

namespace ftg {

// One score row of a 64-key tile recomputed on the CUDA cores: FP32 accumulation over the head dimension in ascending
// order (src/ft_flash_attention_a14.cu:948-953).  q_row: the query's D halves; k_tile: the first of 64 consecutive keys.
template <int kDim>
__device__ __forceinline__ void replay_score_row(const __half* __restrict__ q_row, const __half* __restrict__ k_tile, float (&v)[64]) {
  const __half2* q2 = reinterpret_cast<const __half2*>(q_row);
#pragma unroll
  for (int c = 0; c < 64; ++c) {
    const __half2* k2 = reinterpret_cast<const __half2*>(k_tile + static_cast<size_t>(c) * kDim);
    float acc = 0.0f;
#pragma unroll 4
    for (int d = 0; d < kDim / 2; ++d) {
      const float2 qv = __half22float2(__ldg(q2 + d));
      const float2 kv = __half22float2(__ldg(k2 + d));
      acc = __fmaf_rn(qv.x, kv.x, acc);
      acc = __fmaf_rn(qv.y, kv.y, acc);
    }
    v[c] = acc;
  }
}


// The replay of a score tile whose fault could not be located, kept out of line: it runs once in a blue moon, and
// inlined its register needs would be charged to the softmax loop around it.  Each of the 64 threads of the band
// recomputes its row into `rv` (64 floats in local memory), the rows and columns are checked against the cached
// checksums once more, and the outcome comes back: true when the recomputed tile passes.  The two warps of the band meet
// on `bar` (an mbarrier with 64 arrivals per phase; `parity` is the phase of this use) with a bounded wait: *wait_ok is
// cleared when the partner never came.
template <int kDim>
__device__ __noinline__ bool replay_and_verify(const __half* q_row, const __half* k_tile, float* rv, int lane, int half, TileScratch* again,
                                               const float* expected_rows, const float* row_scales, const float* expected_cols,
                                               const float* col_scales, float abs_tol, float rel_tol, uint64_t* bar, uint32_t parity,
                                               volatile int* abort_flag, uint64_t timeout_ns, bool* wait_ok) {
  float x[64];
  replay_score_row<kDim>(q_row, k_tile, x);
#pragma unroll
  for (int i = 0; i < 64; ++i) rv[i] = x[i];
  float ignored = 0.0f;
  abft_tile_rows(x, lane, half, *again, __ldg(expected_rows + half * 32 + lane), __ldg(row_scales + half * 32 + lane), abs_tol, rel_tol, ignored);
  abft_tile_cols_from_rows(x, lane, half, *again);
  mbar_arrive(bar);
  const bool ok = __all_sync(0xffffffffU, mbar_wait_bounded(bar, parity, abort_flag, timeout_ns));
  *wait_ok = ok;
  if (!ok) return false;
  const TileDecision d = abft_tile_decide(lane, *again, __ldg(expected_cols + lane), __ldg(expected_cols + 32 + lane), __ldg(col_scales + lane),
                                          __ldg(col_scales + 32 + lane), abs_tol, rel_tol, ignored);
  return (d.bad_rows | d.bad_cols) == 0;
}

}  // namespace ftg
