/*
 * Reference harness for the S2-S4 expected-checksum cache.  TEST INFRASTRUCTURE
 * ONLY.  Compiles src/s4_cluster_multicast_abft_fp8_gemm.cu of the reference in
 * place and launches, unmodified, its generate_fp8_kernel (:184-192),
 * cache_input_tile_checksums_kernel (:194-235) and
 * cache_expected_tile_checksums_kernel (:237-294) with the launch shapes of its
 * main() (:603-606, 635-649).  The WGMMA kernel of that file is never launched
 * (it needs sm_90a).
 *
 * usage: ref_harness_s4 M N K OUTDIR   (M % 64 == 0; N may be ragged)
 */
#include <cuda_runtime.h>
#define main reference_main_s4
#include FTQ_STR_INCLUDE
#undef main
#include "ref_harness_common.h"

int main(int argc, char** argv) {
  if (argc != 5) {
    std::fprintf(stderr, "usage: %s M N K OUTDIR\n", argv[0]);
    return 2;
  }
  int m = std::atoi(argv[1]), n = std::atoi(argv[2]), k = std::atoi(argv[3]);
  std::string dir = argv[4];
  int tile_rows = m / kM, tile_cols = div_up(n, kN), tile_count = tile_rows * tile_cols;
  size_t a_count = (size_t)m * k, b_count = (size_t)n * k;
  Element *d_a, *d_b;
  float *a_sums, *a_mags, *b_sums, *b_mags, *er, *ec, *sr, *sc;
  HCHECK(cudaMalloc(&d_a, a_count));
  HCHECK(cudaMalloc(&d_b, b_count));
  HCHECK(cudaMalloc(&a_sums, (size_t)tile_rows * k * 4));
  HCHECK(cudaMalloc(&a_mags, (size_t)tile_rows * k * 4));
  HCHECK(cudaMalloc(&b_sums, (size_t)tile_cols * k * 4));
  HCHECK(cudaMalloc(&b_mags, (size_t)tile_cols * k * 4));
  HCHECK(cudaMalloc(&er, (size_t)tile_count * kM * 4));
  HCHECK(cudaMalloc(&sr, (size_t)tile_count * kM * 4));
  HCHECK(cudaMalloc(&ec, (size_t)tile_count * kN * 4));
  HCHECK(cudaMalloc(&sc, (size_t)tile_count * kN * 4));
  HCHECK(cudaMemset(er, 0xff, (size_t)tile_count * kM * 4));
  HCHECK(cudaMemset(ec, 0xff, (size_t)tile_count * kN * 4));
  HCHECK(cudaMemset(sr, 0xff, (size_t)tile_count * kM * 4));
  HCHECK(cudaMemset(sc, 0xff, (size_t)tile_count * kN * 4));
  generate_fp8_kernel<<<(int)((a_count + 255) / 256), 256>>>(d_a, a_count, 0x12345678U);
  generate_fp8_kernel<<<(int)((b_count + 255) / 256), 256>>>(d_b, b_count, 0x9abcdef0U);
  HCHECK(cudaGetLastError());
  cache_input_tile_checksums_kernel<<<tile_rows + tile_cols, 256>>>(d_a, d_b, a_sums, a_mags, b_sums, b_mags, n, k, tile_rows,
                                                                    tile_cols);
  HCHECK(cudaGetLastError());
  int blocks = div_up(tile_count * (kM + kN), 8);
  cache_expected_tile_checksums_kernel<<<blocks, 256>>>(d_a, d_b, a_sums, a_mags, b_sums, b_mags, er, ec, sr, sc, n, k,
                                                        tile_rows, tile_cols);
  HCHECK(cudaGetLastError());
  HCHECK(cudaDeviceSynchronize());
  dump_device(dir, "a.u8", reinterpret_cast<unsigned char*>(d_a), a_count);
  dump_device(dir, "b.u8", reinterpret_cast<unsigned char*>(d_b), b_count);
  dump_device(dir, "a_sums.f32", a_sums, (size_t)tile_rows * k);
  dump_device(dir, "a_mags.f32", a_mags, (size_t)tile_rows * k);
  dump_device(dir, "b_sums.f32", b_sums, (size_t)tile_cols * k);
  dump_device(dir, "b_mags.f32", b_mags, (size_t)tile_cols * k);
  dump_device(dir, "expected_rows.f32", er, (size_t)tile_count * kM);
  dump_device(dir, "row_scales.f32", sr, (size_t)tile_count * kM);
  dump_device(dir, "expected_cols.f32", ec, (size_t)tile_count * kN);
  dump_device(dir, "col_scales.f32", sc, (size_t)tile_count * kN);
  std::printf("ref_harness_s4 ok M=%d N=%d K=%d tiles=%d\n", m, n, k, tile_count);
  return 0;
}
