/*
 * Reference harness for the S0 path.  TEST INFRASTRUCTURE ONLY.  Compiles
 * src/s0_tiled_abft_fp8_gemm.cu of the reference in place and launches,
 * unmodified, its generate_fp8_kernel (:102-110), native_tiled_fp8_gemm_kernel
 * (:112-133), prepare_expected_checksum_kernel (:135-185) and tile_abft_kernel
 * (:193-277) with the launch shapes of its main() (:327-359).
 *
 * Scenarios written to OUTDIR (each: c_<name>.f32 after the checker, and
 * counters_<name>.i32 = {bad_tiles, corrected_tiles}):
 *   clean     no fault
 *   inject    the program's own --inject-fault (+1.0 at the centre of tile
 *             tile_count/2)
 *   two_rc    host adds two faults at distinct rows and columns of tile 0
 *   same_row  host adds two faults in one row of tile 0
 *   cancel    host adds +v and -v in one row of tile 0 (row sum unchanged)
 *
 * usage: ref_harness_s0 M N K OUTDIR
 */
#include <cuda_runtime.h>
#define main reference_main_s0
#include FTQ_STR_INCLUDE
#undef main
#include "ref_harness_common.h"

struct HostFault {
  int row, col;
  float value;
};

int main(int argc, char** argv) {
  if (argc != 5) {
    std::fprintf(stderr, "usage: %s M N K OUTDIR\n", argv[0]);
    return 2;
  }
  int m = std::atoi(argv[1]), n = std::atoi(argv[2]), k = std::atoi(argv[3]);
  std::string dir = argv[4];
  Options defaults;
  int tile_rows = (m + kTile - 1) / kTile, tile_cols = (n + kTile - 1) / kTile, tile_count = tile_rows * tile_cols;
  size_t a_count = (size_t)m * k, b_count = (size_t)k * n, c_count = (size_t)m * n;
  Element *d_a, *d_b;
  float *d_c, *d_clean, *er, *ec, *sr, *sc;
  int* counters;
  HCHECK(cudaMalloc(&d_a, a_count));
  HCHECK(cudaMalloc(&d_b, b_count));
  HCHECK(cudaMalloc(&d_c, c_count * 4));
  HCHECK(cudaMalloc(&d_clean, c_count * 4));
  HCHECK(cudaMalloc(&er, (size_t)tile_count * kTile * 4));
  HCHECK(cudaMalloc(&ec, (size_t)tile_count * kTile * 4));
  HCHECK(cudaMalloc(&sr, (size_t)tile_count * kTile * 4));
  HCHECK(cudaMalloc(&sc, (size_t)tile_count * kTile * 4));
  HCHECK(cudaMalloc(&counters, 8));
  HCHECK(cudaMemset(er, 0, (size_t)tile_count * kTile * 4));
  HCHECK(cudaMemset(ec, 0, (size_t)tile_count * kTile * 4));
  HCHECK(cudaMemset(sr, 0, (size_t)tile_count * kTile * 4));
  HCHECK(cudaMemset(sc, 0, (size_t)tile_count * kTile * 4));
  generate_fp8_kernel<<<(int)((a_count + 255) / 256), 256>>>(d_a, a_count, 0x12345678U);
  generate_fp8_kernel<<<(int)((b_count + 255) / 256), 256>>>(d_b, b_count, 0x9abcdef0U);
  HCHECK(cudaGetLastError());
  dim3 block(kTile, kTile), grid(tile_cols, tile_rows);
  prepare_expected_checksum_kernel<<<tile_count, 256>>>(d_a, d_b, er, ec, sr, sc, m, n, k, tile_rows, tile_cols);
  HCHECK(cudaGetLastError());
  native_tiled_fp8_gemm_kernel<<<grid, block>>>(d_a, d_b, d_clean, m, n, k);
  HCHECK(cudaGetLastError());
  HCHECK(cudaDeviceSynchronize());
  dump_device(dir, "a.u8", reinterpret_cast<unsigned char*>(d_a), a_count);
  dump_device(dir, "b.u8", reinterpret_cast<unsigned char*>(d_b), b_count);
  dump_device(dir, "c_gemm.f32", d_clean, c_count);
  dump_device(dir, "expected_rows.f32", er, (size_t)tile_count * kTile);
  dump_device(dir, "expected_cols.f32", ec, (size_t)tile_count * kTile);
  dump_device(dir, "row_scales.f32", sr, (size_t)tile_count * kTile);
  dump_device(dir, "col_scales.f32", sc, (size_t)tile_count * kTile);

  struct Scenario {
    const char* name;
    bool inject;
    std::vector<HostFault> faults;
  };
  std::vector<Scenario> scenarios = {
      {"clean", false, {}},
      {"inject", true, {}},
      {"two_rc", false, {{1, 2, 3.0f}, {5, 7, -2.5f}}},
      {"same_row", false, {{3, 1, 4.0f}, {3, 9, 6.0f}}},
      {"cancel", false, {{4, 2, 5.0f}, {4, 11, -5.0f}}},
  };
  std::vector<float> host_c(c_count);
  for (const Scenario& s : scenarios) {
    HCHECK(cudaMemcpy(host_c.data(), d_clean, c_count * 4, cudaMemcpyDeviceToHost));
    for (const HostFault& f : s.faults) {
      if (f.row < m && f.col < n) host_c[(size_t)f.row * n + f.col] += f.value;
    }
    HCHECK(cudaMemcpy(d_c, host_c.data(), c_count * 4, cudaMemcpyHostToDevice));
    HCHECK(cudaMemset(counters, 0, 8));
    tile_abft_kernel<<<tile_count, block>>>(d_c, er, ec, sr, sc, m, n, tile_rows, tile_cols, defaults.abs_tolerance,
                                            defaults.rel_tolerance, s.inject, counters, counters + 1);
    HCHECK(cudaGetLastError());
    HCHECK(cudaDeviceSynchronize());
    dump_device(dir, (std::string("c_") + s.name + ".f32").c_str(), d_c, c_count);
    dump_device(dir, (std::string("counters_") + s.name + ".i32").c_str(), counters, 2);
  }
  std::printf("ref_harness_s0 ok M=%d N=%d K=%d tiles=%d\n", m, n, k, tile_count);
  return 0;
}
