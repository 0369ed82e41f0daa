// The 64x64 ABFT tile verifier shared by the kernels that hold an accumulator
// tile in registers after a TMEM load (one thread = one row, 64 columns): the
// checker of the reference's epilogue (src/s4_cluster_multicast_abft_fp8_gemm.cu:
// 456-499) in register form.
//
//   row checksum    sum of the thread's 64 values (four interleaved partial sums)
//   column checksum transpose-reduce butterfly over the warp's 32 rows (from the row
//                   registers, or from a second read of tensor memory in the
//                   fragment layout), combined with the partner warp (the other 32
//                   rows of the tile) through shared memory; the caller
//                   synchronises the two warps
//   decision        bad <=> |expected - actual| > abs + rel * max(1, scale)
//   correction      iff exactly one bad row and one bad column:
//                   v[row][col] += 0.5 * (row_delta + col_delta), applied by the caller
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "sm100_ptx.cuh"

namespace ftg {

struct TileRowInfo {
  int count;
  int first;
  float delta;
  int pad;
};

struct TileScratch {
  float colpart[2][64];  // [warp half][column]: column sums over that warp's 32 rows
  TileRowInfo rows[2];   // [warp half]
};

struct TileDecision {
  int bad_rows;
  int bad_cols;
  int bad_row;  // lowest bad local row (0..63), -1 if none
  int bad_col;
  float row_delta;
  float col_delta;
  bool corrected;
};

// The check is split so that a caller can overlap the partner exchange with other work (a second tile, the row
// maximum): the row part and the column part by each of the two warps (64 threads) that own the tile's rows, then a
// barrier over those 64 threads, then abft_tile_decide().  `half` says which 32 rows this warp holds.  `sc` must not
// be written again before both warps have finished abft_tile_decide().

// Row part: the thread's row checksum against its cached expectation; publishes the warp's bad-row count, its lowest
// bad row and that row's delta.
__device__ __forceinline__ void abft_tile_rows(const float (&v)[64], int lane, int half, TileScratch& sc, float exp_row, float scale_row,
                                               float abs_tol, float rel_tol, float& max_ratio) {
  // Four interleaved partial sums in two packed FP32 pairs: 32 dependent additions become two chains of 15.  (The score
  // products come from the tensor core, whose own summation order is not defined, so no particular order is owed here.)
  unsigned long long sum_a = pack_f32x2(v[0], v[1]), sum_b = pack_f32x2(v[2], v[3]);
#pragma unroll
  for (int c = 4; c < 64; c += 4) {
    sum_a = add_f32x2(sum_a, pack_f32x2(v[c], v[c + 1]));
    sum_b = add_f32x2(sum_b, pack_f32x2(v[c + 2], v[c + 3]));
  }
  float sum_lo, sum_hi;
  unpack_f32x2(add_f32x2(sum_a, sum_b), sum_lo, sum_hi);
  const float row_sum = sum_lo + sum_hi;
  const float row_delta = exp_row - row_sum;
  const float row_thr = __fmaf_rn(rel_tol, fmaxf(1.0f, scale_row), abs_tol);
  const bool row_bad = fabsf(row_delta) > row_thr;
  if (!row_bad) max_ratio = fmaxf(max_ratio, __fdividef(fabsf(row_delta), row_thr));
  const uint32_t row_mask = __ballot_sync(0xffffffffU, row_bad);
  const int first_lane = row_mask != 0 ? __ffs(row_mask) - 1 : 0;
  const float first_delta = __shfl_sync(0xffffffffU, row_delta, first_lane);
  if (lane == 0) {
    sc.rows[half].count = __popc(row_mask);
    sc.rows[half].first = row_mask != 0 ? half * 32 + first_lane : -1;
    sc.rows[half].delta = first_delta;
  }
}

// Column part from registers (one thread = one row): transpose-reduce butterfly over the warp's 32 rows, 63 shuffles.
__device__ __forceinline__ void abft_tile_cols_from_rows(const float (&v)[64], int lane, int half, TileScratch& sc) {
  float w[32];
  {
    const bool upper = (lane & 16) != 0;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      float send = upper ? v[i] : v[i + 32];
      float keep = upper ? v[i + 32] : v[i];
      w[i] = keep + __shfl_xor_sync(0xffffffffU, send, 16);
    }
    int n = 16;
#pragma unroll
    for (int off = 8; off >= 1; off >>= 1) {
      const bool up = (lane & off) != 0;
#pragma unroll
      for (int i = 0; i < n; ++i) {
        float send = up ? w[i] : w[i + n];
        float keep = up ? w[i + n] : w[i];
        w[i] = keep + __shfl_xor_sync(0xffffffffU, send, off);
      }
      n >>= 1;
    }
  }
  *reinterpret_cast<float2*>(&sc.colpart[half][2 * lane]) = make_float2(w[0], w[1]);
}

// Column sums straight from tensor memory: the warp's 32 lanes x 64 columns at `taddr` (lane field = first lane of the
// warp's quarter) are read a second time in the 16-lane x 256-bit fragment layout, in which a thread holds two adjacent
// columns of four rows per 8-column block.  Three packed additions per block fold the four rows, then a
// transpose-reduce over the eight row groups (lane bits 2..4) leaves the sums of columns 2*lane and 2*lane+1 in each
// thread (c0, c1): 14 shuffles instead of 63, and the additions work on FP32 pairs.  abft_tile_cols_from_tmem publishes
// them as the warp's column part of a tile check.
__device__ __forceinline__ void tmem_column_sums_32x64(uint32_t taddr, int lane, float& c0, float& c1) {
  float a[32], b[32];
  tmem_ld_16x256b_x8(taddr, a);                // lanes +0 .. +15
  tmem_ld_16x256b_x8(taddr + (16u << 16), b);  // lanes +16 .. +31
  tmem_wait_ld();
  unsigned long long s[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    s[k] = add_f32x2(add_f32x2(pack_f32x2(a[4 * k], a[4 * k + 1]), pack_f32x2(a[4 * k + 2], a[4 * k + 3])),
                     add_f32x2(pack_f32x2(b[4 * k], b[4 * k + 1]), pack_f32x2(b[4 * k + 2], b[4 * k + 3])));
  }
  int n = 4;
#pragma unroll
  for (int off = 16; off >= 4; off >>= 1) {
    const bool up = (lane & off) != 0;
#pragma unroll
    for (int i = 0; i < n; ++i) {
      const unsigned long long send = up ? s[i] : s[i + n];
      const unsigned long long keep = up ? s[i + n] : s[i];
      s[i] = add_f32x2(keep, shfl_xor_f32x2(send, off));
    }
    n >>= 1;
  }
  // block index kept = lane >> 2, columns 8*(lane>>2) + 2*(lane&3) + {0,1} = 2*lane + {0,1}
  unpack_f32x2(s[0], c0, c1);
}

__device__ __forceinline__ void abft_tile_cols_from_tmem(uint32_t taddr, int lane, int half, TileScratch& sc) {
  float c0, c1;
  tmem_column_sums_32x64(taddr, lane, c0, c1);
  *reinterpret_cast<float2*>(&sc.colpart[half][2 * lane]) = make_float2(c0, c1);
}

// Row and column parts from registers (the form the kernels with one thread per whole row use).
__device__ __forceinline__ void abft_tile_sums(const float (&v)[64], int lane, int half, TileScratch& sc, float exp_row, float scale_row,
                                               float abs_tol, float rel_tol, float& max_ratio) {
  abft_tile_rows(v, lane, half, sc, exp_row, scale_row, abs_tol, rel_tol, max_ratio);
  abft_tile_cols_from_rows(v, lane, half, sc);
}

// The decision is the same in all 64 threads.  Nothing is corrected here: the caller applies
// 0.5 * (row_delta + col_delta) to element (bad_row, bad_col) when `corrected` is set.
__device__ __forceinline__ TileDecision abft_tile_decide(int lane, const TileScratch& sc, float exp_col0, float exp_col1, float scale_col0,
                                                         float scale_col1, float abs_tol, float rel_tol, float& max_ratio) {
  const float col_delta0 = exp_col0 - (sc.colpart[0][lane] + sc.colpart[1][lane]);
  const float col_delta1 = exp_col1 - (sc.colpart[0][32 + lane] + sc.colpart[1][32 + lane]);
  const float col_thr0 = __fmaf_rn(rel_tol, fmaxf(1.0f, scale_col0), abs_tol);
  const float col_thr1 = __fmaf_rn(rel_tol, fmaxf(1.0f, scale_col1), abs_tol);
  const bool col_bad0 = fabsf(col_delta0) > col_thr0;
  const bool col_bad1 = fabsf(col_delta1) > col_thr1;
  if (!col_bad0) max_ratio = fmaxf(max_ratio, __fdividef(fabsf(col_delta0), col_thr0));
  if (!col_bad1) max_ratio = fmaxf(max_ratio, __fdividef(fabsf(col_delta1), col_thr1));
  const uint32_t col_mask0 = __ballot_sync(0xffffffffU, col_bad0);
  const uint32_t col_mask1 = __ballot_sync(0xffffffffU, col_bad1);

  TileDecision d;
  d.bad_rows = sc.rows[0].count + sc.rows[1].count;
  d.bad_cols = __popc(col_mask0) + __popc(col_mask1);
  d.bad_row = -1;
  d.bad_col = -1;
  d.row_delta = 0.0f;
  d.col_delta = 0.0f;
  d.corrected = false;
  if ((d.bad_rows | d.bad_cols) != 0) {  // uniform over the two warps
    if (d.bad_rows != 0) {
      d.bad_row = sc.rows[0].count != 0 ? sc.rows[0].first : sc.rows[1].first;
      d.row_delta = sc.rows[0].count != 0 ? sc.rows[0].delta : sc.rows[1].delta;
    }
    const float d0 = __shfl_sync(0xffffffffU, col_delta0, col_mask0 != 0 ? __ffs(col_mask0) - 1 : 0);
    const float d1 = __shfl_sync(0xffffffffU, col_delta1, col_mask1 != 0 ? __ffs(col_mask1) - 1 : 0);
    if (col_mask0 != 0) {
      d.bad_col = __ffs(col_mask0) - 1;
      d.col_delta = d0;
    } else if (col_mask1 != 0) {
      d.bad_col = 32 + __ffs(col_mask1) - 1;
      d.col_delta = d1;
    }
    d.corrected = d.bad_rows == 1 && d.bad_cols == 1;
  }
  return d;
}

}  // namespace ftg
