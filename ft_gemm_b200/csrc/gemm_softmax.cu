// GEMM + softmax cross-nonlinearity check: kernels and C-ABI (include/ft_gemm_softmax.h).
//
// Replaces the reference's prototype src/gemm_softmax_abft.cu.  The logits come from
// the fault-tolerant FP8 GEMM of this library (tcgen05 tensor cores, 64x64 tile
// checksums) instead of the prototype's scalar kernel; called with the operands
// swapped, its column-major output is exactly the row-major logits matrix.  The
// softmax pass keeps the prototype's arithmetic: FP64 reductions as 256 strided
// partial sums per row followed by a halving tree (gs:183-203, 243-300), so that its
// check values can be compared with a CPU restatement term by term.  Each row is
// scaled by 1/sqrt(K) on its way into shared memory and every later pass reads it
// from there.
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <new>

#include "../../include/ft_gemm_softmax.h"

namespace ftg {
int noalloc_fail(int code, const char* fmt, ...);  // sets the thread's last-error text (api.cu)
}
using ftg::noalloc_fail;

namespace {

constexpr int kGsThreads = 256;              // kReductionThreads of the prototype (gs:25)
constexpr int kGsMaxStagedBytes = 160 * 1024;  // rows up to 40960 logits are staged in shared memory

struct GsDeviceReport {
  int detected[2];  // [pass]: first analysis, analysis after correction
  int located[2];
  unsigned long long max_residual_bits[2];  // non-negative doubles order like their bit patterns
  int record_count;
  int pad;
  ft_gs_record records[FT_GS_MAX_RECORDS];
};

__device__ __forceinline__ uint32_t gs_mix_u32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7feb352dU;
  x ^= x >> 15;
  x *= 0x846ca68bU;
  x ^= x >> 16;
  return x;
}

__device__ __forceinline__ float gs_e4m3_to_float(uint8_t v) {  // exact decode without the FP16 detour
  const uint32_t sign = (v & 0x80u) << 24, exponent = (v >> 3) & 15u, mantissa = v & 7u;
  if (exponent == 0) {
    const float magnitude = static_cast<float>(mantissa) * 0.001953125f;  // subnormals: m * 2^-9
    return __uint_as_float(__float_as_uint(magnitude) | sign);
  }
  return __uint_as_float(sign | ((exponent + 120u) << 23) | (mantissa << 20));
}

// gs:156-163
__global__ void gs_generate_kernel(uint8_t* out, size_t count, uint32_t seed) {
  size_t index = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  // codes of -3/16 .. 3/16 in E4M3: 1/16 = 2^-4 (exponent 3), 2/16 = 2^-3 (exponent 4), 3/16 = 1.5 * 2^-3
  const uint8_t codes[7] = {0xa4, 0xa0, 0x98, 0x00, 0x18, 0x20, 0x24};
  for (; index < count; index += stride) out[index] = codes[gs_mix_u32(seed + static_cast<uint32_t>(index)) % 7u];
}

// b_sum[k] = sum_j B[j,k], b_weighted[k] = sum_j (2j - (N-1)) B[j,k] (gs:205-223).  Every term is a multiple of 2^-9
// and the totals stay far below 2^53 * 2^-9, so the FP64 sums are exact and their order is free: thread = one k,
// CTA = 256 rows of B, partial results added with atomics.
__global__ void __launch_bounds__(kGsThreads) gs_column_sums_kernel(const uint8_t* __restrict__ b, int ld, double* __restrict__ b_sum,
                                                                    double* __restrict__ b_weighted, int n, int k) {
  const int kk = blockIdx.x * kGsThreads + threadIdx.x;
  if (kk >= k) return;
  const int row_begin = blockIdx.y * 256, row_end = min(n, row_begin + 256);
  double sum = 0.0, weighted = 0.0;
  for (int row = row_begin; row < row_end; ++row) {
    const double value = static_cast<double>(gs_e4m3_to_float(b[static_cast<size_t>(row) * ld + kk]));
    sum += value;
    weighted += static_cast<double>(2 * row - (n - 1)) * value;
  }
  atomicAdd(b_sum + kk, sum);
  atomicAdd(b_weighted + kk, weighted);
}

// gs:225-241: one thread per row of A, k ascending, one fma per step; the products with the FP32 scale widened to FP64.
__global__ void __launch_bounds__(128) gs_expected_kernel(const uint8_t* __restrict__ a, int ld, const double* __restrict__ b_sum,
                                                          const double* __restrict__ b_weighted, double* __restrict__ expected_sum,
                                                          double* __restrict__ expected_weighted, int m, int k, double scale) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= m) return;
  double sum = 0.0, weighted = 0.0;
  const uint8_t* a_row = a + static_cast<size_t>(row) * ld;
  for (int k0 = 0; k0 < k; k0 += 16) {  // ld is a multiple of 32 and the padding is zero: whole 16-byte loads
    const uint4 raw = *reinterpret_cast<const uint4*>(a_row + k0);
    const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if (k0 + i < k) {
        const double value = static_cast<double>(gs_e4m3_to_float(static_cast<uint8_t>(words[i >> 2] >> (8 * (i & 3)))));
        sum += value * b_sum[k0 + i];
        weighted += value * b_weighted[k0 + i];
      }
    }
  }
  expected_sum[row] = sum * scale;
  expected_weighted[row] = weighted * scale;
}

__device__ double gs_block_sum(double value, double* scratch) {  // gs:183-193
  scratch[threadIdx.x] = value;
  __syncthreads();
  for (int stride = kGsThreads / 2; stride > 0; stride >>= 1) {
    if (threadIdx.x < stride) scratch[threadIdx.x] += scratch[threadIdx.x + stride];
    __syncthreads();
  }
  const double result = scratch[0];
  __syncthreads();
  return result;
}

__device__ double gs_block_max(double value, double* scratch) {  // gs:195-203
  scratch[threadIdx.x] = value;
  __syncthreads();
  for (int stride = kGsThreads / 2; stride > 0; stride >>= 1) {
    if (threadIdx.x < stride) scratch[threadIdx.x] = fmax(scratch[threadIdx.x], scratch[threadIdx.x + stride]);
    __syncthreads();
  }
  const double result = scratch[0];
  __syncthreads();
  return result;
}

// gs:243-300.  raw != 0: the buffer holds the GEMM's accumulators; they are scaled (and the test fault added) here and
// written back as the logits.  staged != 0: the row lives in dynamic shared memory after the first pass.
__global__ void __launch_bounds__(kGsThreads) gs_softmax_checks_kernel(float* __restrict__ logits, int ld, float* __restrict__ probabilities,
                                                                       double* __restrict__ actual_sum, double* __restrict__ actual_weighted,
                                                                       double* __restrict__ probability_sum, double* __restrict__ log_z,
                                                                       int* __restrict__ underflow_count, int n, float scale, int raw,
                                                                       int staged, int fault_row, int fault_col, float fault_value) {
  extern __shared__ float gs_row[];
  __shared__ double scratch[kGsThreads];
  const int row = blockIdx.x;
  float* x = logits + static_cast<size_t>(row) * ld;
  double local_max = -DBL_MAX;
  for (int column = threadIdx.x; column < n; column += blockDim.x) {
    float value = x[column];
    if (raw) value *= scale;                                           // accumulator * scale, as gs:177
    if (row == fault_row && column == fault_col) value += fault_value;  // gs:341-345
    if (raw || row == fault_row) x[column] = value;
    if (staged) gs_row[column] = value;
    local_max = fmax(local_max, static_cast<double>(value));
  }
  const float* v = staged ? gs_row : x;  // each thread re-reads only what it wrote itself
  const double row_max = gs_block_max(local_max, scratch);

  double local_exp_sum = 0.0;
  for (int column = threadIdx.x; column < n; column += blockDim.x) local_exp_sum += exp(static_cast<double>(v[column]) - row_max);
  const double denominator = gs_block_sum(local_exp_sum, scratch);
  const double row_log_z = row_max + log(denominator);

  double local_log_sum = 0.0, local_weighted = 0.0, local_probability_sum = 0.0;
  int local_underflow = 0;
  for (int column = threadIdx.x; column < n; column += blockDim.x) {
    const double log_probability = static_cast<double>(v[column]) - row_log_z;
    const float probability = static_cast<float>(exp(log_probability));
    probabilities[static_cast<size_t>(row) * n + column] = probability;
    local_probability_sum += static_cast<double>(probability);
    local_log_sum += log_probability;
    local_weighted += static_cast<double>(2 * column - (n - 1)) * log_probability;
    if (probability == 0.0f) ++local_underflow;
  }
  const double row_log_sum = gs_block_sum(local_log_sum, scratch);
  const double row_weighted = gs_block_sum(local_weighted, scratch);
  const double row_probability_sum = gs_block_sum(local_probability_sum, scratch);
  const double row_underflow = gs_block_sum(static_cast<double>(local_underflow), scratch);
  if (threadIdx.x == 0) {
    actual_sum[row] = row_log_sum + static_cast<double>(n) * row_log_z;  // sum(log P) + N logZ
    actual_weighted[row] = row_weighted;                                 // the weights sum to zero: logZ cancels
    probability_sum[row] = row_probability_sum;
    log_z[row] = row_log_z;
    underflow_count[row] = static_cast<int>(row_underflow);
  }
}

__device__ bool gs_exceeds(double actual, double expected, double abs_tol, double rel_tol) {  // gs:297-300
  const double threshold = abs_tol + rel_tol * fmax(1.0, fabs(expected));
  return fabs(actual - expected) > threshold;
}

// gs:302-339, plus the records and the residual maximum of the report.
__global__ void gs_analyze_kernel(const double* expected_sum, const double* expected_weighted, const double* actual_sum,
                                  const double* actual_weighted, const double* probability_sum, int* detected, int* estimated_col,
                                  double* correction_delta, GsDeviceReport* report, int pass, int m, int n, double abs_tol, double rel_tol,
                                  double row_sum_tol, double location_tol) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= m) return;
  const double delta_sum = actual_sum[row] - expected_sum[row];
  const double delta_weighted = actual_weighted[row] - expected_weighted[row];
  const bool bad = fabs(probability_sum[row] - 1.0) > row_sum_tol || gs_exceeds(actual_sum[row], expected_sum[row], abs_tol, rel_tol) ||
                   gs_exceeds(actual_weighted[row], expected_weighted[row], abs_tol, rel_tol);
  atomicMax(&report->max_residual_bits[pass], static_cast<unsigned long long>(__double_as_longlong(fmax(fabs(delta_sum), fabs(delta_weighted)))));
  detected[row] = bad ? 1 : 0;
  estimated_col[row] = -1;
  correction_delta[row] = delta_sum;
  if (!bad) return;
  atomicAdd(&report->detected[pass], 1);
  int column = -1;
  const double minimum_delta = abs_tol + rel_tol * fmax(1.0, fabs(expected_sum[row]));
  if (fabs(delta_sum) > minimum_delta) {
    const double observed_weight = delta_weighted / delta_sum;
    const int candidate = __double2int_rn(0.5 * (observed_weight + static_cast<double>(n - 1)));
    if (candidate >= 0 && candidate < n && fabs(observed_weight - static_cast<double>(2 * candidate - (n - 1))) <= location_tol) {
      column = candidate;
      estimated_col[row] = column;
      atomicAdd(&report->located[pass], 1);
    }
  }
  if (pass == 0) {
    const int slot = atomicAdd(&report->record_count, 1);
    if (slot < FT_GS_MAX_RECORDS) {
      report->records[slot].row = row;
      report->records[slot].estimated_col = column;
      report->records[slot].correction_delta = delta_sum;
    }
  }
}

// gs:347-353
__global__ void gs_correct_kernel(float* logits, int ld, const int* detected, const int* estimated_col, const double* correction_delta,
                                  int m) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row < m && detected[row] != 0 && estimated_col[row] >= 0) {
    logits[static_cast<size_t>(row) * ld + estimated_col[row]] -= static_cast<float>(correction_delta[row]);
  }
}

#define GS_CUDA(call)                                                                                     \
  do {                                                                                                    \
    cudaError_t err_ = (call);                                                                            \
    if (err_ != cudaSuccess) return noalloc_fail(FT_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(err_)); \
  } while (0)

}  // namespace

struct ft_gs_handle {
  int m = 0, n = 0, k = 0, n_pad = 0, k_pad = 0;
  ft_gs_options options{};
  uint8_t *a_pad = nullptr, *b_pad = nullptr;
  float* logits = nullptr;
  ft_gemm_handle* gemm = nullptr;
  double* doubles = nullptr;  // b_sum, b_weighted [k]; expected_sum, expected_weighted, actual_sum, actual_weighted,
                              // probability_sum, log_z, correction_delta [m]
  double *b_sum = nullptr, *b_weighted = nullptr, *expected_sum = nullptr, *expected_weighted = nullptr, *actual_sum = nullptr,
         *actual_weighted = nullptr, *probability_sum = nullptr, *log_z = nullptr, *correction_delta = nullptr;
  int* ints = nullptr;  // underflow_count, detected, estimated_col [m]
  int *underflow = nullptr, *detected = nullptr, *estimated_col = nullptr;
  GsDeviceReport* report = nullptr;
  bool corrected = false;
  cudaStream_t last_stream = nullptr;
};

extern "C" {

void ft_gs_options_default(ft_gs_options* options) {
  if (options == nullptr) return;
  options->abs_tol = 2.0e-3;
  options->rel_tol = 2.0e-5;
  options->row_sum_tol = 2.0e-6;
  options->location_tol = 2.5e-1;
}

int ft_gemm_softmax_abft_destroy(ft_gs_handle* h) {
  if (h == nullptr) return FT_OK;
  cudaStreamSynchronize(h->last_stream);
  if (h->gemm != nullptr) ft_gemm_fp8_abft_destroy(h->gemm);
  cudaFree(h->a_pad);
  cudaFree(h->b_pad);
  cudaFree(h->logits);
  cudaFree(h->doubles);
  cudaFree(h->ints);
  cudaFree(h->report);
  delete h;
  return FT_OK;
}

int ft_gemm_softmax_abft_prepare(ft_gs_handle** handle, const void* a, const void* b, int m, int n, int k, const ft_gs_options* options,
                                 void* stream_ptr) {
  if (handle == nullptr || a == nullptr || b == nullptr) return noalloc_fail(FT_ERR_INVALID, "null handle or operand pointer");
  *handle = nullptr;
  ft_gs_options opts;
  ft_gs_options_default(&opts);
  if (options != nullptr) opts = *options;
  if (m <= 0 || n <= 1 || k <= 0 || opts.abs_tol < 0.0 || opts.rel_tol < 0.0 || opts.row_sum_tol < 0.0 || opts.location_tol < 0.0) {
    return noalloc_fail(FT_ERR_INVALID, "Invalid shape, fault, or tolerance option.");  // gs:121-125
  }
  ft_gs_handle* h = new (std::nothrow) ft_gs_handle();
  if (h == nullptr) return noalloc_fail(FT_ERR_INVALID, "out of host memory");
  h->m = m, h->n = n, h->k = k;
  h->n_pad = (n + 127) / 128 * 128;  // the GEMM sees B as its row operand: rows in multiples of 128
  h->k_pad = (k + 31) / 32 * 32;
  h->options = opts;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  const size_t a_bytes = static_cast<size_t>(m) * h->k_pad, b_bytes = static_cast<size_t>(h->n_pad) * h->k_pad;
  cudaError_t err = cudaMalloc(reinterpret_cast<void**>(&h->a_pad), a_bytes);
  if (err == cudaSuccess) err = cudaMalloc(reinterpret_cast<void**>(&h->b_pad), b_bytes);
  if (err == cudaSuccess) err = cudaMalloc(reinterpret_cast<void**>(&h->logits), static_cast<size_t>(m) * h->n_pad * sizeof(float));
  if (err == cudaSuccess) err = cudaMalloc(reinterpret_cast<void**>(&h->doubles), (2 * static_cast<size_t>(k) + 7 * static_cast<size_t>(m)) * sizeof(double));
  if (err == cudaSuccess) err = cudaMalloc(reinterpret_cast<void**>(&h->ints), 3 * static_cast<size_t>(m) * sizeof(int));
  if (err == cudaSuccess) err = cudaMalloc(reinterpret_cast<void**>(&h->report), sizeof(GsDeviceReport));
  // zero padding: E4M3 code 0 is +0, so padded rows and columns add nothing to any product
  if (err == cudaSuccess) err = cudaMemsetAsync(h->a_pad, 0, a_bytes, stream);
  if (err == cudaSuccess) err = cudaMemsetAsync(h->b_pad, 0, b_bytes, stream);
  if (err == cudaSuccess) err = cudaMemcpy2DAsync(h->a_pad, h->k_pad, a, k, k, m, cudaMemcpyDeviceToDevice, stream);
  if (err == cudaSuccess) err = cudaMemcpy2DAsync(h->b_pad, h->k_pad, b, k, k, n, cudaMemcpyDeviceToDevice, stream);
  if (err == cudaSuccess) err = cudaMemsetAsync(h->doubles, 0, 2 * static_cast<size_t>(k) * sizeof(double), stream);
  if (err == cudaSuccess) err = cudaMemsetAsync(h->report, 0, sizeof(GsDeviceReport), stream);
  if (err != cudaSuccess) {
    ft_gemm_softmax_abft_destroy(h);
    return noalloc_fail(FT_ERR_CUDA, "allocating or filling the buffers failed: %s", cudaGetErrorString(err));
  }
  double* cursor = h->doubles;
  h->b_sum = cursor, cursor += k;
  h->b_weighted = cursor, cursor += k;
  h->expected_sum = cursor, cursor += m;
  h->expected_weighted = cursor, cursor += m;
  h->actual_sum = cursor, cursor += m;
  h->actual_weighted = cursor, cursor += m;
  h->probability_sum = cursor, cursor += m;
  h->log_z = cursor, cursor += m;
  h->correction_delta = cursor;
  h->underflow = h->ints;
  h->detected = h->ints + m;
  h->estimated_col = h->ints + 2 * static_cast<size_t>(m);
  h->last_stream = stream;
  // logits[i][j] = sum_k A[i,k] B[j,k]: with B as the row operand the GEMM's column-major [N', M'] output (M' = n_pad,
  // N' = m) is the row-major logits matrix with leading dimension n_pad
  int rc = ft_gemm_fp8_abft_prepare(&h->gemm, h->b_pad, h->a_pad, h->n_pad, m, h->k_pad, nullptr, stream);
  if (rc != FT_OK) {
    ft_gemm_softmax_abft_destroy(h);
    return rc;
  }
  const float scale = 1.0f / std::sqrt(static_cast<float>(k));  // gs:388
  dim3 grid_b((k + kGsThreads - 1) / kGsThreads, (n + 255) / 256);
  gs_column_sums_kernel<<<grid_b, kGsThreads, 0, stream>>>(h->b_pad, h->k_pad, h->b_sum, h->b_weighted, n, k);
  gs_expected_kernel<<<(m + 127) / 128, 128, 0, stream>>>(h->a_pad, h->k_pad, h->b_sum, h->b_weighted, h->expected_sum, h->expected_weighted,
                                                          m, k, static_cast<double>(scale));
  err = cudaGetLastError();
  if (err != cudaSuccess) {
    ft_gemm_softmax_abft_destroy(h);
    return noalloc_fail(FT_ERR_CUDA, "launching the projection kernels failed: %s", cudaGetErrorString(err));
  }
  *handle = h;
  return FT_OK;
}

int ft_gemm_softmax_abft_run(ft_gs_handle* h, float* probabilities, const ft_gs_fault* fault, int correct, void* stream_ptr) {
  if (h == nullptr || probabilities == nullptr) return noalloc_fail(FT_ERR_INVALID, "null handle or output pointer");
  if (fault != nullptr && (fault->row < 0 || fault->row >= h->m || fault->col < 0 || fault->col >= h->n)) {
    return noalloc_fail(FT_ERR_INVALID, "Fault position must satisfy row < M and col < N.");  // gs:132-135
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  int rc = ft_gemm_fp8_abft_run(h->gemm, h->logits, nullptr, 0, stream);
  if (rc != FT_OK) return rc;
  GS_CUDA(cudaMemsetAsync(h->report, 0, sizeof(GsDeviceReport), stream));
  const float scale = 1.0f / std::sqrt(static_cast<float>(h->k));
  const size_t row_bytes = static_cast<size_t>(h->n) * sizeof(float);
  const int staged = row_bytes <= static_cast<size_t>(kGsMaxStagedBytes) ? 1 : 0;
  const size_t smem = staged ? row_bytes : 0;
  if (smem > 48 * 1024) {
    GS_CUDA(cudaFuncSetAttribute(gs_softmax_checks_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGsMaxStagedBytes));
  }
  const ft_gs_options& o = h->options;
  for (int pass = 0; pass < (correct ? 2 : 1); ++pass) {
    const bool first = pass == 0;
    gs_softmax_checks_kernel<<<h->m, kGsThreads, smem, stream>>>(
        h->logits, h->n_pad, probabilities, h->actual_sum, h->actual_weighted, h->probability_sum, h->log_z, h->underflow, h->n, scale,
        first ? 1 : 0, staged, first && fault != nullptr ? fault->row : -1, first && fault != nullptr ? fault->col : -1,
        first && fault != nullptr ? fault->value : 0.0f);
    gs_analyze_kernel<<<(h->m + 255) / 256, 256, 0, stream>>>(h->expected_sum, h->expected_weighted, h->actual_sum, h->actual_weighted,
                                                              h->probability_sum, h->detected, h->estimated_col, h->correction_delta,
                                                              h->report, pass, h->m, h->n, o.abs_tol, o.rel_tol, o.row_sum_tol,
                                                              o.location_tol);
    if (first && correct) {
      gs_correct_kernel<<<(h->m + 255) / 256, 256, 0, stream>>>(h->logits, h->n_pad, h->detected, h->estimated_col, h->correction_delta,
                                                                h->m);
    }
  }
  GS_CUDA(cudaGetLastError());
  h->corrected = correct != 0;
  h->last_stream = stream;
  return FT_OK;
}

int ft_gemm_softmax_abft_report(ft_gs_handle* h, ft_gs_report* out) {
  if (h == nullptr || out == nullptr) return noalloc_fail(FT_ERR_INVALID, "null handle or report pointer");
  ft_report gemm_report;
  int rc = ft_gemm_fp8_abft_report(h->gemm, &gemm_report);  // synchronises the stream
  if (rc != FT_OK && rc != FT_ERR_TIMEOUT) return rc;
  GS_CUDA(cudaStreamSynchronize(h->last_stream));
  GsDeviceReport dev;
  GS_CUDA(cudaMemcpy(&dev, h->report, sizeof(dev), cudaMemcpyDeviceToHost));
  std::memset(out, 0, sizeof(*out));
  out->status = gemm_report.status;
  out->detected_rows = dev.detected[0];
  out->located_rows = dev.located[0];
  out->post_detected_rows = h->corrected ? dev.detected[1] : -1;
  out->gemm_bad_tiles = gemm_report.bad_tiles;
  out->gemm_corrected_tiles = gemm_report.corrected_tiles;
  std::memcpy(&out->max_projection_residual, &dev.max_residual_bits[0], sizeof(double));
  std::memcpy(&out->post_max_projection_residual, &dev.max_residual_bits[1], sizeof(double));
  const int kept = std::min(dev.record_count, FT_GS_MAX_RECORDS);
  out->n_records = kept;
  std::copy(dev.records, dev.records + kept, out->records);
  std::sort(out->records, out->records + kept, [](const ft_gs_record& x, const ft_gs_record& y) { return x.row < y.row; });
  return rc;
}

int ft_gemm_softmax_abft_logits(ft_gs_handle* h, const float** logits, int* leading_dimension) {
  if (h == nullptr || logits == nullptr || leading_dimension == nullptr) return noalloc_fail(FT_ERR_INVALID, "null pointer");
  *logits = h->logits;
  *leading_dimension = h->n_pad;
  return FT_OK;
}

int ft_gemm_softmax_abft_logits_read(ft_gs_handle* h, float* host_out) {
  if (h == nullptr || host_out == nullptr) return noalloc_fail(FT_ERR_INVALID, "null pointer");
  GS_CUDA(cudaStreamSynchronize(h->last_stream));
  GS_CUDA(cudaMemcpy2D(host_out, static_cast<size_t>(h->n) * sizeof(float), h->logits, static_cast<size_t>(h->n_pad) * sizeof(float),
                       static_cast<size_t>(h->n) * sizeof(float), h->m, cudaMemcpyDeviceToHost));
  return FT_OK;
}

int ft_gemm_softmax_abft_checks(ft_gs_handle* h, double* expected_sum, double* expected_weighted, double* actual_sum, double* actual_weighted,
                                double* probability_sum, double* log_z) {
  if (h == nullptr) return noalloc_fail(FT_ERR_INVALID, "null handle");
  GS_CUDA(cudaStreamSynchronize(h->last_stream));
  const size_t bytes = static_cast<size_t>(h->m) * sizeof(double);
  double* const host[6] = {expected_sum, expected_weighted, actual_sum, actual_weighted, probability_sum, log_z};
  const double* const device[6] = {h->expected_sum, h->expected_weighted, h->actual_sum, h->actual_weighted, h->probability_sum, h->log_z};
  for (int i = 0; i < 6; ++i) {
    if (host[i] != nullptr) GS_CUDA(cudaMemcpy(host[i], device[i], bytes, cudaMemcpyDeviceToHost));
  }
  return FT_OK;
}

int ft_gemm_softmax_generate_fp8(void* out, size_t count, uint32_t seed, void* stream_ptr) {
  if (out == nullptr && count > 0) return noalloc_fail(FT_ERR_INVALID, "null output pointer");
  if (count == 0) return FT_OK;
  size_t blocks = std::min<size_t>((count + 255) / 256, 148 * 32);
  gs_generate_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream_ptr)>>>(static_cast<uint8_t*>(out), count, seed);
  GS_CUDA(cudaGetLastError());
  return FT_OK;
}

}  // extern "C"
