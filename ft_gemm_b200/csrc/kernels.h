// Internal interface between the C-ABI layer and the kernels.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ft_gemm.h"

namespace ftg {

// Device-side report of one run: counters first, then the per-tile records.
struct DeviceReport {
  int status;            // 0, or 1 when a bounded wait expired
  int bad_tiles;
  int corrected_tiles;
  int multi_fault_tiles;
  int record_count;      // records attempted (may exceed FT_MAX_RECORDS)
  int max_clean_ratio_bits;  // float bits of max |delta|/threshold over passing checks
  int pad[2];
  ft_tile_record records[FT_MAX_RECORDS];
};

struct FaultParams {
  int count;
  int tile[FT_MAX_FAULTS];
  int row[FT_MAX_FAULTS];
  int col[FT_MAX_FAULTS];
  float value[FT_MAX_FAULTS];
};

struct GemmParams {
  const float* expected_rows;
  const float* expected_cols;
  const float* row_scales;
  const float* col_scales;
  float* c;
  DeviceReport* report;
  // The handle keeps two report buffers and alternates between them: a launch that starts a new report also clears the
  // counters (the first 32 bytes) of the buffer the NEXT call will use, so no separate memset sits between two calls.
  // nullptr: nothing to clear (window launches that add to the current report).
  int* clear_counters;
  int m, n, k;
  // window of C this launch computes (rows a multiple of the tile height, cols of 256); the whole product by default
  int row0, rows, col0, cols;
  float abs_tol, rel_tol;
  // limit of every device-side wait of this launch, nanoseconds (ft_options::wait_limit_us; 2 s by default)
  unsigned long long wait_timeout_ns;
  // Tiles are walked in groups of group_rows rows of C, column block by column block inside a group, so that the A panel of
  // a group (group_rows x K bytes) stays in L2 while B streams past it once per group.  The host sizes the panel to 32 MiB,
  // a quarter of the L2, between 1024 and 8192 rows: at K = 8192 that is 4096 rows (measured at 8192^3: 2048 rows -1.6 %,
  // 8192 rows -7 %; 8192 x 8192 x 4096 gains 3.7 % with 8192 rows over 2048).
  int group_rows;
  // Column slices for the tail of a launch.  The tiles are dealt out round robin to the persistent CTAs (pairs); when
  // their number is not a multiple of the worker count the last round keeps only some workers busy, and with few tiles
  // per worker the epilogue of the last tile overlaps nothing.  Tiles from index split_from on are therefore cut into
  // `split` (1, 2 or 4) column slices of 256 / split columns, each scheduled as an item of its own: the last round
  // spreads over more workers, and a worker's last epilogue covers a slice instead of a tile.
  int split_from, split;
  FaultParams faults;
  // optional per-CTA cycle counters (8 x uint64 per CTA), nullptr in normal runs:
  // [0] producer waiting for a free stage, [1] MMA waiting for a full stage, [2] MMA waiting for a drained
  // accumulator, [3] MMA role total, [4] epilogue waiting for an accumulator, [5] epilogue total, [6] tiles, [7] spare
  unsigned long long* profile;
};

cudaError_t launch_generate(void* out, size_t count, uint32_t seed, int dist, float sigma, float post_scale, cudaStream_t stream);
cudaError_t launch_band_sums(const void* x, float* sums, float* mags, int rows, int k, cudaStream_t stream);
cudaError_t launch_expected(const void* x, const float* band_sums, const float* band_mags, float* expected, float* scales, int rows,
                            int nbands, int k, int mode, cudaStream_t stream);
// src [rows, k] (dtype 0 FP32, 1 BF16, 2 FP16) * scale -> E4M3 dst, with the band sums of dst in the same pass; rows % 64 == 0, k % 8 == 0.
cudaError_t launch_quantize_band_sums(const void* src, int src_dtype, void* dst, float* sums, float* mags, int rows, int k, float scale,
                                      cudaStream_t stream);

// FP16 variants for the attention path: `rows` may span many heads for the band sums; the expected
// kernel treats `batch` problems of [rows, k] x [nbands, k] laid out back to back.
cudaError_t launch_band_sums_f16(const void* x, float* sums, float* mags, size_t rows, int k, cudaStream_t stream);
cudaError_t launch_expected_f16(const void* x, const float* band_sums, const float* band_mags, float* expected, float* scales, int rows,
                                int nbands, int k, int mode, int batch, cudaStream_t stream);

// Expected checksums on the tensor cores (prepare_mma.cu): the band sums are split into five E4M3 digit planes
// (plane rows = prepare_mma_plane_rows(nbands), k bytes each), then X times the planes gives the four cache arrays.
// tmap_x: X [rows, k] with a 128-row box; tmap_ws / tmap_wm: the planes of the sums / magnitudes with a 160-row box.
cudaError_t configure_prepare_mma();
size_t prepare_mma_plane_bytes(int nbands, int k);
int prepare_mma_plane_rows(int nbands);
cudaError_t launch_split_band_digits(const float* sums, const float* mags, void* ws, void* wm, int nbands, int k, cudaStream_t stream);
cudaError_t launch_expected_mma(const CUtensorMap& tmap_x, const CUtensorMap& tmap_ws, const CUtensorMap& tmap_wm, float* expected,
                                float* scales, int rows, int nbands, int k, int mode, int sm_count, int* status, cudaStream_t stream);
// FP16 form for the attention path: the band sums (times 2^-7) as 3 + 2 FP16 pieces per band; `batch` problems back to back.
// Plane rows per problem: prepare_mma_plane_rows_f16(nbands, 0 sums | 1 magnitudes), k FP16 elements each; maps with a 96- / 64-row box.
int prepare_mma_plane_rows_f16(int nbands, int which);
cudaError_t launch_split_band_pieces_f16(const float* sums, const float* mags, void* ws, void* wm, int nbands, int k, int batch,
                                         cudaStream_t stream);
cudaError_t launch_expected_mma_f16(const CUtensorMap& tmap_x, const CUtensorMap& tmap_ws, const CUtensorMap& tmap_wm, float* expected,
                                    float* scales, int rows, int nbands, int k, int mode, int batch, int sm_count, int* status,
                                    cudaStream_t stream);

// Fused FP8 GEMM + ABFT checker/corrector.  tmap_a / tmap_b describe A[M,K] and
// B[N,K] with 128-byte-swizzled boxes of (128 K-bytes x 128 rows) and
// (128 K-bytes x 256 rows).
cudaError_t configure_abft_gemm();
// pair = true launches the 2-CTA form (clusters of two CTAs sharing a 256x256 tile;
// tmap_b must then have a 128-row box, grid must be even and M a multiple of 256).
cudaError_t launch_abft_gemm(const CUtensorMap& tmap_a, const CUtensorMap& tmap_b, const GemmParams& params, int grid, bool pair,
                             cudaStream_t stream);
int abft_gemm_smem_bytes(bool pair);
// Test hook: one thread waits with mbar_wait_bounded on a barrier nobody arrives on and records the time-out in `report`.
cudaError_t launch_selftest_wait(DeviceReport* report, unsigned long long limit_ns, cudaStream_t stream);

}  // namespace ftg
