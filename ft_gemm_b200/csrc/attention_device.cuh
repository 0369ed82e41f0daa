// Device helpers shared by the two attention forward kernels.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

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

}  // namespace ftg
