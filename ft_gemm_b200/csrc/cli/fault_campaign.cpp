// Random single-fault campaign on the B200 ABFT FP8 GEMM.  Same command line,
// trial generator, classification and report keys as the reference's campaign
// program (src/s4_random_fault_campaign.cu:133-173, 735-895): every trial draws
// (tile, row, col, magnitude, sign) from the seeded hash chain, runs the fused
// kernel with that fault, and is counted as detected / attempted / recovered.
// `--double-trials N` appends N trials with a second fault in the same tile at a
// different row and column; those must be reported and left uncorrected.
#include "cli_common.h"

static uint32_t mix_host_u32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7feb352dU;
  x ^= x >> 15;
  x *= 0x846ca68bU;
  x ^= x >> 16;
  return x;
}

int main(int argc, char** argv) {
  ArgReader args{argc, argv};
  CommonOptions o;
  read_common(args, o);
  float fault_min_value = args.get_float("--fault-min-value", 1.0f);
  float fault_max_value = args.get_float("--fault-max-value", 256.0f);
  int fault_trials = args.get_int("--fault-trials", 100);
  int fault_seed = args.get_int("--fault-seed", 12345);
  int double_trials = args.get_int("--double-trials", 0);
  if (args.has_flag("--help")) {
    std::printf(
        "Usage: %s [--m N --n N --k N --warmup N --repeat N]\n"
        "       [--verify-samples N --verify-abs-tol X --verify-rel-tol X]\n"
        "       [--abs-tol X --rel-tol X]\n"
        "       [--fault-min-value X --fault-max-value X]\n"
        "       [--fault-trials N --fault-seed N --double-trials N]\n"
        "       [--dist uniform|normal|llm]\n"
        "Constraints: any positive M, N and K (boundary tiles; K is padded to a multiple of 16 internally).\n",
        argv[0]);
    return EXIT_SUCCESS;
  }
  if (!common_valid(o) || fault_min_value <= 0.0f || fault_max_value < fault_min_value || fault_trials <= 0 || double_trials < 0) {
    std::fprintf(stderr, "Invalid options. Require a positive shape.\n");
    return EXIT_FAILURE;
  }
  CLI_CUDA(cudaSetDevice(0));
  size_t a_count = static_cast<size_t>(o.m) * o.k, b_count = static_cast<size_t>(o.n) * o.k, c_count = static_cast<size_t>(o.m) * o.n;
  int tile_cols = (o.n + 63) / 64, tile_count = ((o.m + 63) / 64) * tile_cols;
  void *d_a = nullptr, *d_b = nullptr;
  float *d_c = nullptr, *d_clean = nullptr;
  CLI_CUDA(cudaMalloc(&d_a, a_count));
  CLI_CUDA(cudaMalloc(&d_b, b_count));
  CLI_CUDA(cudaMalloc(reinterpret_cast<void**>(&d_c), c_count * sizeof(float)));
  CLI_CUDA(cudaMalloc(reinterpret_cast<void**>(&d_clean), c_count * sizeof(float)));
  cudaStream_t stream;
  CLI_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
  generate_inputs(o, d_a, d_b, stream);
  CLI_CUDA(cudaStreamSynchronize(stream));

  ft_options options;
  ft_options_default(&options);
  options.abs_tol = o.abft_abs_tolerance;
  options.rel_tol = o.abft_rel_tolerance;
  ft_gemm_handle* handle = nullptr;
  CLI_FT(ft_gemm_fp8_abft_prepare(&handle, d_a, d_b, o.m, o.n, o.k, &options, stream));
  ft_report report;
  CLI_FT(ft_gemm_fp8_abft_report(handle, &report));
  // The timings reported below are those of a second fill of the cache: the first one also pays for loading the
  // prepare kernels onto the device (lazy module loading), which is not part of the operator's cost.
  CLI_FT(ft_gemm_fp8_abft_refresh(handle, 3, stream));
  CLI_FT(ft_gemm_fp8_abft_report(handle, &report));
  float metadata_prepare_ms = report.prepare_input_ms + report.prepare_expected_ms;
  float input_metadata_ms = report.prepare_input_ms, expected_metadata_ms = report.prepare_expected_ms;
  ft_cache_view cache;
  CLI_FT(ft_gemm_fp8_abft_cache(handle, &cache));
  // The largest detection threshold of the run, abs + rel * max(1, scale) over every cached row and column scale
  // (src/s4_cluster_multicast_abft_fp8_gemm.cu:467, 480): a fault below it may pass the reference's checker by design.
  float threshold_max = 0.0f, threshold_min = 0.0f;
  {
    std::vector<float> scales(static_cast<size_t>(tile_count) * 64);
    float largest = 1.0f, smallest = 3.0e38f;
    for (int which = 6; which <= 7; ++which) {
      CLI_FT(ft_gemm_fp8_abft_cache_read(handle, which, scales.data(), scales.size()));
      for (float v : scales) {
        largest = std::fmax(largest, v);
        if (v > 0.0f) smallest = std::fmin(smallest, v);  // zeros pad the boundary tiles
      }
    }
    threshold_max = o.abft_abs_tolerance + o.abft_rel_tolerance * largest;
    threshold_min = o.abft_abs_tolerance + o.abft_rel_tolerance * std::fmax(1.0f, smallest);
  }

  StageTimings timing = time_stage(handle, d_clean, o, stream);
  // clean reference output and clean counters (src/s4_random_fault_campaign.cu keeps h_c of the clean run)
  CLI_FT(ft_gemm_fp8_abft_run(handle, d_clean, nullptr, 0, stream));
  CLI_FT(ft_gemm_fp8_abft_report(handle, &report));
  int bad_tiles = report.bad_tiles, corrected_tiles = report.corrected_tiles;
  float clean_noise = report.max_clean_ratio;

  int campaign_detected = 0, campaign_correction_attempts = 0, campaign_corrected = 0, campaign_missed = 0;
  int campaign_detected_not_corrected = 0, campaign_miscorrected = 0;
  float campaign_max_residual = 0.0f;
  constexpr int kMagnitudeBins = 4;
  int bin_trials[kMagnitudeBins] = {}, bin_detected[kMagnitudeBins] = {}, bin_corrected[kMagnitudeBins] = {};
  struct FaultFailure {
    int trial, row, col;
    float fault;
    int bad_tiles, corrected_tiles;
    float residual, tolerance;
  };
  std::vector<FaultFailure> failures;
  int double_reported = 0, double_silently_corrected = 0, double_missed = 0;
  float max_missed_magnitude = 0.0f, min_detected_magnitude = 3.0e38f;

  uint32_t state = static_cast<uint32_t>(fault_seed);
  for (int trial = 0; trial < fault_trials + double_trials; ++trial) {
    bool is_double = trial >= fault_trials;
    state = mix_host_u32(state + 0x9e3779b9U + static_cast<uint32_t>(trial));
    int fault_tile = static_cast<int>(state % static_cast<uint32_t>(tile_count));
    state = mix_host_u32(state);
    int fault_row = static_cast<int>(state % 64);
    state = mix_host_u32(state);
    int fault_col = static_cast<int>(state % 64);
    state = mix_host_u32(state);
    float magnitude_unit = static_cast<float>(state & 0x00ffffffU) / 16777215.0f;
    float fault_magnitude = fault_min_value + (fault_max_value - fault_min_value) * magnitude_unit;
    int magnitude_bin = fault_max_value == fault_min_value ? 0 : std::min(kMagnitudeBins - 1, static_cast<int>(kMagnitudeBins * magnitude_unit));
    state = mix_host_u32(state);
    float signed_fault_value = (state & 1U) == 0 ? fault_magnitude : -fault_magnitude;

    ft_fault faults[2];
    faults[0] = ft_fault{fault_tile, fault_row, fault_col, signed_fault_value};
    int n_faults = 1;
    if (is_double) {
      // three more draws: a second element of the same tile in another row and column
      state = mix_host_u32(state);
      int row2 = (fault_row + 1 + static_cast<int>(state % 63)) % 64;
      state = mix_host_u32(state);
      int col2 = (fault_col + 1 + static_cast<int>(state % 63)) % 64;
      state = mix_host_u32(state);
      float unit2 = static_cast<float>(state & 0x00ffffffU) / 16777215.0f;
      float value2 = fault_min_value + (fault_max_value - fault_min_value) * unit2;
      faults[1] = ft_fault{fault_tile, row2, col2, (state & 0x01000000U) ? -value2 : value2};
      n_faults = 2;
    }
    CLI_FT(ft_gemm_fp8_abft_run(handle, d_c, faults, n_faults, stream));
    ft_report trial_report;
    CLI_FT(ft_gemm_fp8_abft_report(handle, &trial_report));

    if (is_double) {
      bool reported = trial_report.bad_tiles == 1 && trial_report.corrected_tiles == 0 && trial_report.multi_fault_tiles == 1;
      double_reported += reported;
      double_silently_corrected += trial_report.corrected_tiles > 0;
      double_missed += trial_report.bad_tiles == 0;
      continue;
    }
    int fault_global_row = (fault_tile / tile_cols) * 64 + fault_row;
    int fault_global_col = (fault_tile % tile_cols) * 64 + fault_col;
    size_t fault_output_index = static_cast<size_t>(fault_global_col) * o.m + fault_global_row;
    float corrected_value = 0.0f, reference_value = 0.0f;
    CLI_CUDA(cudaMemcpy(&corrected_value, d_c + fault_output_index, sizeof(float), cudaMemcpyDeviceToHost));
    CLI_CUDA(cudaMemcpy(&reference_value, d_clean + fault_output_index, sizeof(float), cudaMemcpyDeviceToHost));
    float residual = std::fabs(corrected_value - reference_value);
    float recovery_tolerance = o.verify_abs_tolerance + o.verify_rel_tolerance * std::fmax(1.0f, std::fabs(reference_value));
    bool detected = trial_report.bad_tiles > 0;
    bool attempted = trial_report.corrected_tiles > 0;
    bool recovered = trial_report.bad_tiles == 1 && trial_report.corrected_tiles == 1 && residual <= recovery_tolerance;
    campaign_detected += detected;
    campaign_correction_attempts += attempted;
    campaign_corrected += recovered;
    campaign_missed += !detected;
    if (!detected) max_missed_magnitude = std::fmax(max_missed_magnitude, fault_magnitude);
    if (detected) min_detected_magnitude = std::fmin(min_detected_magnitude, fault_magnitude);
    campaign_detected_not_corrected += detected && !attempted;
    campaign_miscorrected += attempted && !recovered;
    campaign_max_residual = std::fmax(campaign_max_residual, residual);
    ++bin_trials[magnitude_bin];
    bin_detected[magnitude_bin] += detected;
    bin_corrected[magnitude_bin] += recovered;
    if (!recovered && failures.size() < 16) {
      failures.push_back({trial, fault_global_row, fault_global_col, signed_fault_value, trial_report.bad_tiles,
                          trial_report.corrected_tiles, residual, recovery_tolerance});
    }
  }

  float first_call_total_ms = metadata_prepare_ms + timing.first_ms;
  float amortized_ms = timing.average_ms + metadata_prepare_ms / o.repeat;
  double operations = 2.0 * static_cast<double>(o.m) * o.n * o.k;
  double tflops = operations / (timing.average_ms * 1.0e9);
  double first_call_tflops = operations / (first_call_total_ms * 1.0e9);
  double amortized_tflops = operations / (amortized_ms * 1.0e9);
  VerificationResult verification = verify_samples(d_a, d_b, d_clean, o);
  bool numerical_pass = o.verify_samples == 0 || verification.max_tolerance_ratio <= 1.0f;
  bool abft_pass = bad_tiles == 0;
  bool passed = numerical_pass && abft_pass;

  print_common_header(o, "program", "B200 random single-fault correction campaign");
  std::printf("metadata_cache_bytes: %zu\n", cache.bytes);
  std::printf("input_metadata_time_ms: %.6f\n", input_metadata_ms);
  std::printf("expected_metadata_time_ms: %.6f\n", expected_metadata_ms);
  std::printf("metadata_prepare_time_ms: %.6f\n", metadata_prepare_ms);
  std::printf("first_fused_gemm_abft_time_ms: %.6f\n", timing.first_ms);
  std::printf("first_call_total_ms: %.6f\n", first_call_total_ms);
  std::printf("first_call_tflops: %.6f\n", first_call_tflops);
  std::printf("avg_fused_gemm_abft_time_ms: %.6f\n", timing.average_ms);
  std::printf("amortized_time_ms: %.6f\n", amortized_ms);
  std::printf("amortized_tflops: %.6f\n", amortized_tflops);
  std::printf("fused_gemm_tflops: %.6f\n", tflops);
  std::printf("abft_tolerance: abs=%.6e rel=%.6e\n", o.abft_abs_tolerance, o.abft_rel_tolerance);
  std::printf("clean_checksum_noise_ratio: %.6e\n", clean_noise);
  std::printf("bad_tiles: %d\n", bad_tiles);
  std::printf("corrected_tiles: %d\n", corrected_tiles);
  double detection_rate = 100.0 * campaign_detected / fault_trials;
  double correction_rate = 100.0 * campaign_corrected / fault_trials;
  int failed_trials = fault_trials - campaign_corrected;
  std::printf("fault_campaign_trials: %d\n", fault_trials);
  std::printf("fault_campaign_seed: %d\n", fault_seed);
  std::printf("fault_campaign_magnitude_distribution: uniform [%.6e, %.6e], random sign\n", fault_min_value, fault_max_value);
  std::printf("fault_campaign_detected: %d\n", campaign_detected);
  std::printf("fault_campaign_correction_attempts: %d\n", campaign_correction_attempts);
  std::printf("fault_campaign_corrected: %d\n", campaign_corrected);
  std::printf("fault_campaign_missed: %d\n", campaign_missed);
  std::printf("fault_campaign_detected_not_corrected: %d\n", campaign_detected_not_corrected);
  std::printf("fault_campaign_miscorrected: %d\n", campaign_miscorrected);
  std::printf("fault_campaign_detection_rate_percent: %.3f\n", detection_rate);
  std::printf("fault_campaign_correction_rate_percent: %.3f\n", correction_rate);
  std::printf("fault_campaign_max_post_correction_residual: %.6e\n", campaign_max_residual);
  std::printf("abft_threshold_range: min=%.6e max=%.6e\n", threshold_min, threshold_max);
  std::printf("fault_campaign_max_missed_magnitude: %.6e\n", max_missed_magnitude);
  std::printf("fault_campaign_min_detected_magnitude: %.6e\n", campaign_detected > 0 ? min_detected_magnitude : 0.0f);
  float bin_width = (fault_max_value - fault_min_value) / kMagnitudeBins;
  for (int bin = 0; bin < kMagnitudeBins; ++bin) {
    float lower = fault_min_value + bin * bin_width;
    float upper = bin == kMagnitudeBins - 1 ? fault_max_value : lower + bin_width;
    double bin_detection_rate = bin_trials[bin] == 0 ? 0.0 : 100.0 * bin_detected[bin] / bin_trials[bin];
    double bin_correction_rate = bin_trials[bin] == 0 ? 0.0 : 100.0 * bin_corrected[bin] / bin_trials[bin];
    std::printf("fault_campaign_bin_%d: range=[%.6e, %.6e%s trials=%d detected=%d corrected=%d detection_rate=%.3f correction_rate=%.3f\n",
                bin, lower, upper, bin == kMagnitudeBins - 1 ? "]" : ")", bin_trials[bin], bin_detected[bin], bin_corrected[bin],
                bin_detection_rate, bin_correction_rate);
  }
  for (const FaultFailure& failure : failures) {
    std::printf("fault_campaign_failure: trial=%d row=%d col=%d fault=%+.6e bad_tiles=%d corrected_tiles=%d residual=%.6e tolerance=%.6e\n",
                failure.trial, failure.row, failure.col, failure.fault, failure.bad_tiles, failure.corrected_tiles, failure.residual,
                failure.tolerance);
  }
  if (failed_trials > static_cast<int>(failures.size())) {
    std::printf("fault_campaign_failure_records_truncated: %d\n", failed_trials - static_cast<int>(failures.size()));
  }
  if (double_trials > 0) {
    std::printf("double_fault_trials: %d\n", double_trials);
    std::printf("double_fault_reported_uncorrected: %d\n", double_reported);
    std::printf("double_fault_silently_corrected: %d\n", double_silently_corrected);
    std::printf("double_fault_missed: %d\n", double_missed);
  }
  std::printf("verification_samples: %d\n", verification.checked);
  std::printf("sampled_max_absolute_error: %.6e\n", verification.max_absolute_error);
  std::printf("sampled_max_tolerance_ratio: %.6e\n", verification.max_tolerance_ratio);
  std::printf("verification: %s\n", passed ? "PASS" : "FAIL");

  CLI_FT(ft_gemm_fp8_abft_destroy(handle));
  CLI_CUDA(cudaStreamDestroy(stream));
  CLI_CUDA(cudaFree(d_a));
  CLI_CUDA(cudaFree(d_b));
  CLI_CUDA(cudaFree(d_c));
  CLI_CUDA(cudaFree(d_clean));
  return passed ? 0 : 1;
}
