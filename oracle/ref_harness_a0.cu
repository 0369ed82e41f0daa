/*
 * Reference harness for the attention path.  TEST INFRASTRUCTURE ONLY.  Compiles
 * src/ft_flash_attention_a0.cu of the reference in place (the clean scalar statement
 * of its three protected stages) and launches, unmodified, its generate_fp8_kernel
 * (:231-238) and ft_flash_attention_a0_kernel (:285-667) with the launch shape and
 * arguments of its main() (:772-797) and the default tolerances of its Options.
 *
 * Scenarios (fault stage, query, index, value are given on the command line as
 * STAGE:QUERY:INDEX:VALUE, stage by the reference's number 0..4; batch 0, head 0):
 * for scenario i the harness writes out_<i>.f32 (the output O) and stats_<i>.i32
 * (DeviceStats: score detected/corrected/replayed, softmax detected/corrected/
 * replayed, pv detected/corrected, failed rows).  q.u8, k.u8, v.u8 are written once.
 *
 * usage: ref_harness_a0 B H N D CAUSAL OUTDIR SCENARIO...
 */
#include <cuda_runtime.h>
#define main reference_main_a0
#include FTQ_STR_INCLUDE
#undef main
#include "ref_harness_common.h"

int main(int argc, char** argv) {
  if (argc < 8) {
    std::fprintf(stderr, "usage: %s B H N D CAUSAL OUTDIR STAGE:QUERY:INDEX:VALUE...\n", argv[0]);
    return 2;
  }
  int batch = std::atoi(argv[1]), heads = std::atoi(argv[2]), sequence = std::atoi(argv[3]), head_dim = std::atoi(argv[4]);
  bool causal = std::atoi(argv[5]) != 0;
  std::string dir = argv[6];
  if (head_dim != 64 && head_dim != 128) {
    std::fprintf(stderr, "head_dim must be 64 or 128\n");
    return 2;
  }
  Options defaults;
  size_t count = (size_t)batch * heads * sequence * head_dim;
  Element *d_q, *d_k, *d_v;
  float* d_out;
  DeviceStats* d_stats;
  HCHECK(cudaMalloc(&d_q, count));
  HCHECK(cudaMalloc(&d_k, count));
  HCHECK(cudaMalloc(&d_v, count));
  HCHECK(cudaMalloc(&d_out, count * sizeof(float)));
  HCHECK(cudaMalloc(&d_stats, sizeof(DeviceStats)));
  int blocks = (int)((count + 255) / 256);
  generate_fp8_kernel<<<blocks, 256>>>(d_q, count, 0x12345678U);
  generate_fp8_kernel<<<blocks, 256>>>(d_k, count, 0x9abcdef0U);
  generate_fp8_kernel<<<blocks, 256>>>(d_v, count, 0x31415926U);
  HCHECK(cudaGetLastError());
  HCHECK(cudaDeviceSynchronize());
  dump_device(dir, "q.u8", reinterpret_cast<const unsigned char*>(d_q), count);
  dump_device(dir, "k.u8", reinterpret_cast<const unsigned char*>(d_k), count);
  dump_device(dir, "v.u8", reinterpret_cast<const unsigned char*>(d_v), count);

  dim3 grid(sequence, batch * heads);
  float score_scale = 1.0f / std::sqrt(static_cast<float>(head_dim));
  for (int i = 7; i < argc; ++i) {
    int stage = 0, query = 0, index = 0;
    float value = 0.0f;
    if (std::sscanf(argv[i], "%d:%d:%d:%f", &stage, &query, &index, &value) != 4) {
      std::fprintf(stderr, "bad scenario %s\n", argv[i]);
      return 2;
    }
    HCHECK(cudaMemset(d_stats, 0, sizeof(DeviceStats)));
    HCHECK(cudaMemset(d_out, 0, count * sizeof(float)));
    if (head_dim == 64) {
      ft_flash_attention_a0_kernel<64><<<grid, kThreads>>>(d_q, d_k, d_v, d_out, batch, heads, sequence, causal, score_scale, stage, 0, 0, query,
                                                          index, value, defaults.score_abs_tolerance, defaults.score_rel_tolerance,
                                                          defaults.softmax_abs_tolerance, defaults.softmax_rel_tolerance,
                                                          defaults.pv_abs_tolerance, defaults.pv_rel_tolerance, d_stats);
    } else {
      ft_flash_attention_a0_kernel<128><<<grid, kThreads>>>(d_q, d_k, d_v, d_out, batch, heads, sequence, causal, score_scale, stage, 0, 0,
                                                           query, index, value, defaults.score_abs_tolerance, defaults.score_rel_tolerance,
                                                           defaults.softmax_abs_tolerance, defaults.softmax_rel_tolerance,
                                                           defaults.pv_abs_tolerance, defaults.pv_rel_tolerance, d_stats);
    }
    HCHECK(cudaGetLastError());
    HCHECK(cudaDeviceSynchronize());
    std::string tag = std::to_string(i - 7);
    dump_device(dir, ("out_" + tag + ".f32").c_str(), d_out, count);
    dump_device(dir, ("stats_" + tag + ".i32").c_str(), reinterpret_cast<const int*>(d_stats), sizeof(DeviceStats) / sizeof(int));
  }
  std::printf("ref_harness_a0: B=%d H=%d N=%d D=%d causal=%d, %d scenario(s) written to %s\n", batch, heads, sequence, head_dim, causal ? 1 : 0,
              argc - 7, dir.c_str());
  return 0;
}
