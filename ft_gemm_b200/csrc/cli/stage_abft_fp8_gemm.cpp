// Per-stage program of the B200 ABFT FP8 GEMM.  Same command line, report keys
// and exit code as the reference's final stage
// (src/s4_cluster_multicast_abft_fp8_gemm.cu:132-173, 556-784): generate ->
// prepare (timed) -> first call -> warm-up -> timed repeats -> sampled FP64
// verification -> `key: value` report; exit 0 iff numerical_pass && abft_pass.
// Everything on the GPU goes through the C-ABI of ft_gemm.h.
//
// Flags beyond the reference's: --dist uniform|normal|llm, --seed N (added to both
// input seeds), --fault2 (a second fault in the same ABFT tile: the tile must then
// be reported and left uncorrected), --json (the report once more as one JSON
// line), --gpus G (rows of A and of C split into G equal bands, one device each,
// B replicated: the kernels read local memory only; the one exchange is a single
// ncclAllGather of the fixed-size per-band report, after which every device holds
// all G reports with tile ids re-based to the whole product, merged in rank order).
#include <nccl.h>

#include <cstdarg>
#include <string>
#include <utility>
#include <vector>

#include "cli_common.h"

namespace {

// `key: value` lines as the reference prints them, remembered for --json.
struct Report {
  std::vector<std::pair<std::string, std::string>> items;
  void add(const char* key, const char* format, ...) __attribute__((format(printf, 3, 4))) {
    char text[512];
    va_list args;
    va_start(args, format);
    std::vsnprintf(text, sizeof(text), format, args);
    va_end(args);
    std::printf("%s: %s\n", key, text);
    items.emplace_back(key, text);
  }
  void print_json() const {
    std::printf("{");
    for (size_t i = 0; i < items.size(); ++i) {
      const std::string& v = items[i].second;
      char* end = nullptr;
      std::strtod(v.c_str(), &end);
      const bool number = !v.empty() && end != nullptr && *end == '\0';
      std::printf("%s\"%s\": ", i ? ", " : "", items[i].first.c_str());
      if (number) {
        std::printf("%s", v.c_str());
      } else {
        std::printf("\"");
        for (char ch : v) {
          if (ch == '"' || ch == '\\') std::printf("\\");
          std::printf("%c", ch);
        }
        std::printf("\"");
      }
    }
    std::printf("}\n");
  }
};

#define CLI_NCCL(call)                                                                              \
  do {                                                                                              \
    ncclResult_t result_ = (call);                                                                  \
    if (result_ != ncclSuccess) {                                                                   \
      std::fprintf(stderr, "NCCL error %s:%d: %s\n", __FILE__, __LINE__, ncclGetErrorString(result_)); \
      std::exit(EXIT_FAILURE);                                                                      \
    }                                                                                               \
  } while (0)

struct Device {
  int id = 0;
  int rows = 0, row_begin = 0;
  void *a = nullptr, *b = nullptr;
  float* c = nullptr;
  cudaStream_t stream = nullptr;
  ft_gemm_handle* handle = nullptr;
  cudaEvent_t start = nullptr, stop = nullptr;
};

}  // namespace

int main(int argc, char** argv) {
  ArgReader args{argc, argv};
  CommonOptions o;
  read_common(args, o);
  float fault_value = args.get_float("--fault-value", 1.0f);
  bool inject_fault = args.has_flag("--inject-fault");
  const bool second_fault = args.has_flag("--fault2");
  const bool json = args.has_flag("--json");
  const int gpus = args.get_int("--gpus", 1);
  const uint32_t seed = static_cast<uint32_t>(args.get_int("--seed", 0));
  o.seed_a += seed;
  o.seed_b += seed;
  if (second_fault) inject_fault = true;
  if (args.has_flag("--help")) {
    std::printf(
        "Usage: %s [--m N --n N --k N --warmup N --repeat N]\n"
        "       [--verify-samples N --verify-abs-tol X --verify-rel-tol X]\n"
        "       [--abs-tol X --rel-tol X --fault-value X --inject-fault --fault2]\n"
        "       [--dist uniform|normal|llm --seed N --gpus G --json]\n"
        "Constraints: any positive M, N and K (boundary tiles; K is padded to a multiple of 16 internally).\n",
        argv[0]);
    return EXIT_SUCCESS;
  }
  if (!common_valid(o) || fault_value <= 0.0f || gpus < 1) {
    std::fprintf(stderr, "Invalid options. Require a positive shape.\n");
    return EXIT_FAILURE;
  }
  int device_count = 0;
  CLI_CUDA(cudaGetDeviceCount(&device_count));
  if (gpus > device_count || o.m % gpus != 0 || (gpus > 1 && (o.m / gpus) % 64 != 0)) {
    std::fprintf(stderr, "Invalid options. --gpus %d needs that many devices (found %d) and M divisible into bands of whole 64-row tiles.\n",
                 gpus, device_count);
    return EXIT_FAILURE;
  }
  const int rows = o.m / gpus;
  const int tile_cols = (o.n + 63) / 64;
  const int tile_count = ((o.m + 63) / 64) * tile_cols;
  CommonOptions shard = o;  // what one device sees
  shard.m = rows;

  ft_options options;
  ft_options_default(&options);
  options.abs_tol = o.abft_abs_tolerance;
  options.rel_tol = o.abft_rel_tolerance;
  std::vector<Device> devices(gpus);
  size_t cache_bytes = 0;
  float input_metadata_ms = 0.0f, expected_metadata_ms = 0.0f;
  for (int g = 0; g < gpus; ++g) {
    Device& d = devices[g];
    d.id = g;
    d.rows = rows;
    d.row_begin = g * rows;
    CLI_CUDA(cudaSetDevice(g));
    size_t a_count = static_cast<size_t>(rows) * o.k, b_count = static_cast<size_t>(o.n) * o.k, c_count = static_cast<size_t>(rows) * o.n;
    CLI_CUDA(cudaMalloc(&d.a, a_count));
    CLI_CUDA(cudaMalloc(&d.b, b_count));
    CLI_CUDA(cudaMalloc(reinterpret_cast<void**>(&d.c), c_count * sizeof(float)));
    CLI_CUDA(cudaStreamCreateWithFlags(&d.stream, cudaStreamNonBlocking));
    CLI_CUDA(cudaEventCreate(&d.start));
    CLI_CUDA(cudaEventCreate(&d.stop));
    CommonOptions mine = shard;  // the band's own part of the seeded sequence, so that the bands differ
    mine.seed_a = o.seed_a + static_cast<uint32_t>(static_cast<size_t>(d.row_begin) * o.k);
    generate_inputs(mine, d.a, d.b, d.stream);
    CLI_CUDA(cudaStreamSynchronize(d.stream));
    CLI_FT(ft_gemm_fp8_abft_prepare(&d.handle, d.a, d.b, rows, o.n, o.k, &options, d.stream));
    ft_report report;
    CLI_FT(ft_gemm_fp8_abft_report(d.handle, &report));
    // The timings reported below are those of a second fill of the cache: the first one also pays for loading the
    // prepare kernels onto the device (lazy module loading), which is not part of the operator's cost.
    CLI_FT(ft_gemm_fp8_abft_refresh(d.handle, 3, d.stream));
    CLI_FT(ft_gemm_fp8_abft_report(d.handle, &report));
    input_metadata_ms = std::max(input_metadata_ms, report.prepare_input_ms);
    expected_metadata_ms = std::max(expected_metadata_ms, report.prepare_expected_ms);
    ft_cache_view cache;
    CLI_FT(ft_gemm_fp8_abft_cache(d.handle, &cache));
    cache_bytes += cache.bytes;
  }
  float metadata_prepare_ms = input_metadata_ms + expected_metadata_ms;

  StageTimings timing;
  if (gpus == 1) {
    CLI_CUDA(cudaSetDevice(0));
    timing = time_stage(devices[0].handle, devices[0].c, shard, devices[0].stream);
  } else {
    // every device runs its band at the same time; a measurement is the slowest device's CUDA-event time
    auto run_all = [&](int calls) {
      for (Device& d : devices) {
        CLI_CUDA(cudaSetDevice(d.id));
        CLI_CUDA(cudaEventRecord(d.start, d.stream));
        for (int i = 0; i < calls; ++i) CLI_FT(ft_gemm_fp8_abft_run(d.handle, d.c, nullptr, 0, d.stream));
        CLI_CUDA(cudaEventRecord(d.stop, d.stream));
      }
      float slowest = 0.0f;
      for (Device& d : devices) {
        CLI_CUDA(cudaSetDevice(d.id));
        CLI_CUDA(cudaEventSynchronize(d.stop));
        float ms = 0.0f;
        CLI_CUDA(cudaEventElapsedTime(&ms, d.start, d.stop));
        slowest = std::max(slowest, ms);
      }
      return slowest;
    };
    timing.first_ms = run_all(1);
    if (o.warmup > 0) run_all(o.warmup);
    float total_ms = 0.0f;
    for (int i = 0; i < o.repeat; ++i) total_ms += run_all(1);
    timing.average_ms = total_ms / o.repeat;
    timing.batched_average_ms = run_all(o.repeat) / o.repeat;
  }

  // the run whose output is verified: with the deterministic fault of the reference (value at local (32, 32) of ABFT
  // tile tile_count/2, src/s4:449-453) and, with --fault2, a second one in the same tile
  const int fault_tile = tile_count / 2;
  const int fault_tile_row = fault_tile / tile_cols;
  ft_report total{};
  for (Device& d : devices) {
    CLI_CUDA(cudaSetDevice(d.id));
    ft_fault faults[2];
    int n_faults = 0;
    const int first_tile_row = d.row_begin / 64, band_tile_rows = (d.rows + 63) / 64;
    if (inject_fault && fault_tile_row >= first_tile_row && fault_tile_row < first_tile_row + band_tile_rows) {
      const int local_tile = (fault_tile_row - first_tile_row) * tile_cols + fault_tile % tile_cols;
      faults[n_faults++] = ft_fault{local_tile, 32, 32, fault_value};
      if (second_fault) faults[n_faults++] = ft_fault{local_tile, 16, 48, fault_value};
    }
    CLI_FT(ft_gemm_fp8_abft_run(d.handle, d.c, n_faults ? faults : nullptr, n_faults, d.stream));
  }
  std::vector<ft_report> shards(gpus);
  for (Device& d : devices) {
    CLI_CUDA(cudaSetDevice(d.id));
    CLI_FT(ft_gemm_fp8_abft_report(d.handle, &shards[d.id]));
    CLI_FT(ft_gemm_report_rebase(&shards[d.id], tile_cols, d.row_begin / 64));  // band-local tile ids -> ids of the whole product
  }
  float report_gather_ms = 0.0f;
  if (gpus == 1) {
    total = shards[0];
  } else {
    // One all-gather of the fixed-size report: afterwards every device holds the G reports in rank order.
    std::vector<ncclComm_t> comms(gpus);
    std::vector<int> ids(gpus);
    for (int g = 0; g < gpus; ++g) ids[g] = g;
    CLI_NCCL(ncclCommInitAll(comms.data(), gpus, ids.data()));
    std::vector<ft_report*> send(gpus), recv(gpus);
    for (Device& d : devices) {
      CLI_CUDA(cudaSetDevice(d.id));
      CLI_CUDA(cudaMalloc(reinterpret_cast<void**>(&send[d.id]), sizeof(ft_report)));
      CLI_CUDA(cudaMalloc(reinterpret_cast<void**>(&recv[d.id]), sizeof(ft_report) * gpus));
      CLI_CUDA(cudaMemcpyAsync(send[d.id], &shards[d.id], sizeof(ft_report), cudaMemcpyHostToDevice, d.stream));
      CLI_CUDA(cudaEventRecord(d.start, d.stream));
    }
    CLI_NCCL(ncclGroupStart());
    for (Device& d : devices) CLI_NCCL(ncclAllGather(send[d.id], recv[d.id], sizeof(ft_report), ncclChar, comms[d.id], d.stream));
    CLI_NCCL(ncclGroupEnd());
    for (Device& d : devices) {
      CLI_CUDA(cudaSetDevice(d.id));
      CLI_CUDA(cudaEventRecord(d.stop, d.stream));
      CLI_CUDA(cudaStreamSynchronize(d.stream));
      float ms = 0.0f;
      CLI_CUDA(cudaEventElapsedTime(&ms, d.start, d.stop));
      report_gather_ms = std::max(report_gather_ms, ms);
    }
    // every rank holds the same union; the last device's copy is the one printed (it proves the data travelled)
    std::vector<ft_report> gathered(gpus);
    CLI_CUDA(cudaSetDevice(gpus - 1));
    CLI_CUDA(cudaMemcpy(gathered.data(), recv[gpus - 1], sizeof(ft_report) * gpus, cudaMemcpyDeviceToHost));
    CLI_FT(ft_gemm_report_merge(gathered.data(), gpus, &total));
    for (Device& d : devices) {
      CLI_CUDA(cudaSetDevice(d.id));
      CLI_CUDA(cudaFree(send[d.id]));
      CLI_CUDA(cudaFree(recv[d.id]));
      CLI_NCCL(ncclCommDestroy(comms[d.id]));
    }
  }

  float first_call_total_ms = metadata_prepare_ms + timing.first_ms;
  float amortized_ms = timing.average_ms + metadata_prepare_ms / o.repeat;
  double operations = 2.0 * static_cast<double>(o.m) * o.n * o.k;
  double tflops = operations / (timing.average_ms * 1.0e9);
  double batched_tflops = operations / (timing.batched_average_ms * 1.0e9);
  double first_call_tflops = operations / (first_call_total_ms * 1.0e9);
  double amortized_tflops = operations / (amortized_ms * 1.0e9);
  VerificationResult verification;
  for (Device& d : devices) {
    CLI_CUDA(cudaSetDevice(d.id));
    VerificationResult v = verify_samples(d.a, d.b, d.c, shard);
    verification.checked += v.checked;
    verification.max_absolute_error = std::max(verification.max_absolute_error, v.max_absolute_error);
    verification.max_tolerance_ratio = std::max(verification.max_tolerance_ratio, v.max_tolerance_ratio);
  }
  bool numerical_pass = o.verify_samples == 0 || verification.max_tolerance_ratio <= 1.0f;
  bool abft_pass = second_fault   ? total.bad_tiles == 1 && total.corrected_tiles == 0 && total.multi_fault_tiles == 1
                   : inject_fault ? total.bad_tiles == 1 && total.corrected_tiles == 1
                                  : total.bad_tiles == 0;
  bool passed = numerical_pass && abft_pass;

  print_common_header(o, "version", "B200 tcgen05 TMEM-epilogue ABFT FP8 GEMM");
  Report out;
  out.add("gpus", "%d", gpus);
  out.add("rows_per_gpu", "%d", rows);
  out.add("metadata_cache_bytes", "%zu", cache_bytes);
  out.add("input_metadata_time_ms", "%.6f", input_metadata_ms);
  out.add("expected_metadata_time_ms", "%.6f", expected_metadata_ms);
  out.add("metadata_prepare_time_ms", "%.6f", metadata_prepare_ms);
  out.add("first_fused_gemm_abft_time_ms", "%.6f", timing.first_ms);
  out.add("first_call_total_ms", "%.6f", first_call_total_ms);
  out.add("first_call_tflops", "%.6f", first_call_tflops);
  out.add("avg_fused_gemm_abft_time_ms", "%.6f", timing.average_ms);
  out.add("amortized_time_ms", "%.6f", amortized_ms);
  out.add("amortized_tflops", "%.6f", amortized_tflops);
  out.add("fused_gemm_tflops", "%.6f", tflops);
  out.add("batched_avg_fused_gemm_abft_time_ms", "%.6f", timing.batched_average_ms);
  out.add("batched_fused_gemm_tflops", "%.6f", batched_tflops);
  out.add("abft_tolerance", "abs=%.6e rel=%.6e", o.abft_abs_tolerance, o.abft_rel_tolerance);
  out.add("clean_checksum_noise_ratio", "%.6e", total.max_clean_ratio);
  out.add("bad_tiles", "%d", total.bad_tiles);
  out.add("corrected_tiles", "%d", total.corrected_tiles);
  out.add("multi_fault_tiles", "%d", total.multi_fault_tiles);
  if (gpus > 1) out.add("report_gather", "ncclAllGather of %zu bytes per device, %.3f ms", sizeof(ft_report), report_gather_ms);
  for (int i = 0; i < total.n_records; ++i) {  // tile ids of the whole product, rank order
    const ft_tile_record& r = total.records[i];
    char key[32];
    std::snprintf(key, sizeof(key), "fault_record_%d", i);
    out.add(key, "tile=%d gpu=%d bad_rows=%d bad_cols=%d row=%d col=%d row_delta=%.6e col_delta=%.6e corrected=%d", r.tile,
            (r.tile / tile_cols) * 64 / rows, r.bad_row_count, r.bad_col_count, r.bad_row, r.bad_col, r.row_delta, r.col_delta, r.corrected);
  }
  out.add("verification_samples", "%d", verification.checked);
  out.add("sampled_max_absolute_error", "%.6e", verification.max_absolute_error);
  out.add("sampled_max_tolerance_ratio", "%.6e", verification.max_tolerance_ratio);
  out.add("verification", "%s", passed ? "PASS" : "FAIL");
  if (json) out.print_json();

  for (Device& d : devices) {
    CLI_CUDA(cudaSetDevice(d.id));
    CLI_FT(ft_gemm_fp8_abft_destroy(d.handle));
    CLI_CUDA(cudaEventDestroy(d.start));
    CLI_CUDA(cudaEventDestroy(d.stop));
    CLI_CUDA(cudaStreamDestroy(d.stream));
    CLI_CUDA(cudaFree(d.a));
    CLI_CUDA(cudaFree(d.b));
    CLI_CUDA(cudaFree(d.c));
  }
  return passed ? 0 : 1;
}
