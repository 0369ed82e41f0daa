// C-ABI layer: handle, expected-checksum cache ownership, tensor maps, report.
// See include/ft_gemm.h for the contract of each entry point and the reference
// lines it replaces.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>

#include "kernels.h"

using namespace ftg;

namespace {

thread_local char g_error[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  std::vsnprintf(g_error, sizeof(g_error), fmt, args);
  va_end(args);
  return code;
}

}  // namespace

namespace ftg {
// error reporting shared with the other translation units of the C-ABI
int noalloc_fail(int code, const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  std::vsnprintf(g_error, sizeof(g_error), fmt, args);
  va_end(args);
  return code;
}
}  // namespace ftg

namespace {

#define FT_CUDA(call)                                                                              \
  do {                                                                                             \
    cudaError_t err_ = (call);                                                                     \
    if (err_ != cudaSuccess) return fail(FT_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(err_)); \
  } while (0)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult query;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &query) == cudaSuccess &&
        query == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
  }
  return fn;
}

// [rows, k] FP8, k contiguous; box = 128 bytes of k x box_rows rows, 128-byte swizzle.
int make_operand_map(CUtensorMap* map, const void* base, int rows, int k, int box_rows) {
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) return fail(FT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(k)};
  cuuint32_t box[2] = {128u, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t elem[2] = {1u, 1u};
  CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(FT_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
  return FT_OK;
}

}  // namespace

constexpr int kMaxPipeChunks = 8;

struct ft_gemm_handle {
  int device = 0;
  int m = 0, n = 0, k = 0;
  int sm_count = 0;
  int grid = 0;
  int max_workers = 0;  // persistent CTAs (pairs in the 2-CTA form) a launch may use
  ft_options options{};
  const void* a = nullptr;
  const void* b = nullptr;
  // cache (one allocation)
  float* cache_base = nullptr;
  size_t cache_bytes = 0;
  float *a_sums = nullptr, *a_mags = nullptr, *b_sums = nullptr, *b_mags = nullptr;
  float *expected_rows = nullptr, *expected_cols = nullptr, *row_scales = nullptr, *col_scales = nullptr;
  DeviceReport* report = nullptr;          // the buffer of the current (last started) report: report_pair[report_index]
  DeviceReport* report_pair = nullptr;     // two buffers, used alternately (see GemmParams::clear_counters)
  int report_index = 0;
  CUtensorMap tmap_a{}, tmap_b{};
  // tensor-core prepare: digit planes of the band sums (in the cache allocation) and their maps
  uint8_t *planes_as = nullptr, *planes_am = nullptr, *planes_bs = nullptr, *planes_bm = nullptr;
  CUtensorMap tmap_b128{}, tmap_as{}, tmap_am{}, tmap_bs{}, tmap_bm{};
  int* prepare_status = nullptr;
  bool pair = false;  // 2-CTA form: clusters of two CTAs per 256x256 tile
  cudaEvent_t ev0 = nullptr, ev_mid = nullptr, ev1 = nullptr;
  bool prepare_timed = false;
  cudaStream_t last_stream = nullptr;
  // K not a multiple of 16 (or operands not 16-byte aligned): zero-padded copies with K rounded up; `k` is then the
  // padded K, user_k the caller's
  const void *user_a = nullptr, *user_b = nullptr;
  void *pad_a = nullptr, *pad_b = nullptr;
  int user_k = 0;
  // device buffers owned by the host-buffer entry point
  void* own_a = nullptr;
  void* own_b = nullptr;
  float* own_c = nullptr;
  cudaStream_t own_stream = nullptr;
  // copy streams and events of the pipelined form of the host-buffer entry point
  cudaStream_t in_stream = nullptr, out_stream = nullptr;
  cudaEvent_t pipe_events[3 * kMaxPipeChunks + 1] = {};
};

namespace {

int check_shape(int m, int n, int k) {
  // Any positive shape (boundary tiles in both directions, as the reference's first stage takes them,
  // src/s0_tiled_abft_fp8_gemm.cu:143-144).  The copy engine needs a row pitch of whole 16-byte chunks: for other K the
  // handle works on zero-padded copies of the operands.
  if (m <= 0 || n <= 0 || k <= 0) {
    return fail(FT_ERR_INVALID, "Invalid options. Require a positive shape (got M=%d N=%d K=%d).", m, n, k);
  }
  long long tiles = static_cast<long long>((m + 63) / 64) * ((n + 63) / 64);
  if (tiles * 64 > 0x7fffffffLL) return fail(FT_ERR_INVALID, "shape too large: %lld ABFT tiles", tiles);
  return FT_OK;
}

// The four checksum arrays from the operands and their band sums; `which` says whose band sums changed (bit 0 A, bit 1 B).
int fill_expected(ft_gemm_handle* h, int which, cudaStream_t stream) {
  const int band_rows_a = (h->m + 63) / 64, band_rows_b = (h->n + 63) / 64;
  if (h->options.exact_prepare != 0) {
    // expected_rows[(I,J),r] = sum_k A[64I+r,k] * b_sums[J,k]
    FT_CUDA(launch_expected(h->a, h->b_sums, h->b_mags, h->expected_rows, h->row_scales, h->m, band_rows_b, h->k, 0, stream));
    // expected_cols[(I,J),c] = sum_k a_sums[I,k] * B[64J+c,k]
    FT_CUDA(launch_expected(h->b, h->a_sums, h->a_mags, h->expected_cols, h->col_scales, h->n, band_rows_a, h->k, 1, stream));
    return FT_OK;
  }
  if (which & 1) FT_CUDA(launch_split_band_digits(h->a_sums, h->a_mags, h->planes_as, h->planes_am, band_rows_a, h->k, stream));
  if (which & 2) FT_CUDA(launch_split_band_digits(h->b_sums, h->b_mags, h->planes_bs, h->planes_bm, band_rows_b, h->k, stream));
  FT_CUDA(launch_expected_mma(h->tmap_a, h->tmap_bs, h->tmap_bm, h->expected_rows, h->row_scales, h->m, band_rows_b, h->k, 0,
                              h->sm_count, h->prepare_status, stream));
  FT_CUDA(launch_expected_mma(h->tmap_b128, h->tmap_as, h->tmap_am, h->expected_cols, h->col_scales, h->n, band_rows_a, h->k, 1,
                              h->sm_count, h->prepare_status, stream));
  return FT_OK;
}

// Handles with padded operand copies: refreshes the copies of the operands that changed (bit 0 A, bit 1 B).  The padding
// columns are zeros (E4M3 code 0), which add nothing to any product or sum.
int copy_padded(ft_gemm_handle* h, int which, cudaStream_t stream) {
  if (h->pad_a == nullptr) return FT_OK;
  if (which & 1) {
    FT_CUDA(cudaMemsetAsync(h->pad_a, 0, static_cast<size_t>(h->m) * h->k, stream));
    FT_CUDA(cudaMemcpy2DAsync(h->pad_a, h->k, h->user_a, h->user_k, h->user_k, h->m, cudaMemcpyDeviceToDevice, stream));
  }
  if (which & 2) {
    FT_CUDA(cudaMemsetAsync(h->pad_b, 0, static_cast<size_t>(h->n) * h->k, stream));
    FT_CUDA(cudaMemcpy2DAsync(h->pad_b, h->k, h->user_b, h->user_k, h->user_k, h->n, cudaMemcpyDeviceToDevice, stream));
  }
  return FT_OK;
}

int fill_cache(ft_gemm_handle* h, int which, cudaStream_t stream) {
  // the status of the prepare kernels describes the latest fill: a handle whose earlier fill timed out recovers here
  FT_CUDA(cudaMemsetAsync(h->prepare_status, 0, sizeof(int), stream));
  FT_CUDA(cudaEventRecord(h->ev0, stream));
  if (which & 1) FT_CUDA(launch_band_sums(h->a, h->a_sums, h->a_mags, h->m, h->k, stream));
  if (which & 2) FT_CUDA(launch_band_sums(h->b, h->b_sums, h->b_mags, h->n, h->k, stream));
  FT_CUDA(cudaEventRecord(h->ev_mid, stream));
  int rc = fill_expected(h, which, stream);
  if (rc != FT_OK) return rc;
  FT_CUDA(cudaEventRecord(h->ev1, stream));
  h->prepare_timed = true;
  h->last_stream = stream;
  return FT_OK;
}

void fill_params(const ft_gemm_handle* h, float* c, GemmParams* params) {
  params->expected_rows = h->expected_rows;
  params->expected_cols = h->expected_cols;
  params->row_scales = h->row_scales;
  params->col_scales = h->col_scales;
  params->c = c;
  params->report = h->report;
  params->m = h->m;
  params->n = h->n;
  params->k = h->k;
  params->row0 = 0;
  params->rows = h->m;
  params->col0 = 0;
  params->cols = h->n;
  params->abs_tol = h->options.abs_tol;
  params->rel_tol = h->options.rel_tol;
  params->wait_timeout_ns = h->options.wait_limit_us > 0 ? 1000ull * static_cast<unsigned long long>(h->options.wait_limit_us) : 2000000000ull;
  const long long panel_rows = (32ll << 20) / h->k;  // rows of A whose K bytes fill 32 MiB
  const int tile_m = h->pair ? 256 : 128;
  const int per_group = static_cast<int>(std::min<long long>(std::max<long long>(panel_rows, 1024), 8192)) / tile_m;
  const int row_blocks = (h->m + tile_m - 1) / tile_m;
  const int groups = (row_blocks + per_group - 1) / per_group;
  params->group_rows = (row_blocks + groups - 1) / groups * tile_m;  // groups of equal height
  params->split_from = 0x7fffffff;  // whole tiles only, unless the caller of the launch decides otherwise
  params->split = 1;
}

// How the tail of a launch is cut into column slices (GemmParams::split_from / split).  Model, in units of one whole
// tile's main loop: a worker's time is its whole tiles, then its slices (a slice of 256/s columns costs c(s)/s, the
// narrower MMA shapes being a little less efficient), each overlapped with the previous item's epilogue, plus the one
// epilogue that overlaps nothing.  e = epilogue / main loop of a whole tile, about 0.2 at K = 8192 and growing as K
// shrinks.  The smallest s within 2 % of the best wins.
void choose_split(int tiles, int workers, int k, int* split_from, int* split) {
  *split_from = tiles;
  *split = 1;
  if (workers <= 0 || tiles <= 0) return;
  const int full = tiles >= workers ? (tiles / workers) * workers : 0;
  const int tail = tiles - full;
  if (tail == 0) return;
  const double e = std::min(4.0, 0.2 * 8192.0 / std::max(k, 1));
  const int rounds_full = full / workers;
  double best_time = 0.0;
  for (int s = 1; s <= 4; s *= 2) {
    const double c = s == 1 ? 1.0 : (s == 2 ? 1.04 : 1.3);
    const int tail_rounds = (tail * s + workers - 1) / workers;
    const double main = c / s, epi = e / s;
    const double time = rounds_full * std::max(1.0, e) + tail_rounds * std::max(main, epi) + std::min(main, epi);
    if (s == 1 || time < 0.98 * best_time) {
      best_time = time;
      *split = s;
    }
  }
  *split_from = full;
}

// Largest chunk count g <= kMaxPipeChunks for which M/g and N/g are whole tiles; 1 = no pipelining.
int pipe_chunks(const ft_gemm_handle* h) {
  if (h->pad_a != nullptr) return 1;  // padded operand copies are refreshed as a whole
  const int tile_m = h->pair ? 256 : 128;
  for (int g = kMaxPipeChunks; g > 1; g >>= 1) {
    if (h->m % (g * tile_m) == 0 && h->n % (g * 256) == 0) return g;
  }
  return 1;
}

int ensure_pipe(ft_gemm_handle* h) {
  if (h->in_stream != nullptr) return FT_OK;
  FT_CUDA(cudaStreamCreateWithFlags(&h->in_stream, cudaStreamNonBlocking));
  FT_CUDA(cudaStreamCreateWithFlags(&h->out_stream, cudaStreamNonBlocking));
  for (cudaEvent_t& e : h->pipe_events) FT_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  return FT_OK;
}

// Steady-state form of the host-buffer call (cache valid): A and B arrive in g row chunks each, alternating; as soon as
// chunk i of both is on the device the L-shaped part of C that needs only chunks 0..i is computed by two window launches
// and copied back while later chunks are still on their way.  Three streams: copies in, compute, copies out.
int host_pipelined(ft_gemm_handle* h, const void* a_host, const void* b_host, float* c_host, const ft_fault* faults, int n_faults,
                   int g) {
  int rc = ensure_pipe(h);
  if (rc != FT_OK) return rc;
  const size_t k = static_cast<size_t>(h->k), m = static_cast<size_t>(h->m);
  const int mc = h->m / g, nc = h->n / g;
  const size_t pitch = m * sizeof(float);
  cudaStream_t compute = h->own_stream;
  cudaEvent_t* in_done = h->pipe_events;
  cudaEvent_t* c_done = h->pipe_events + g;
  cudaEvent_t out_done = h->pipe_events[3 * g];
  const char* a_src = static_cast<const char*>(a_host);
  const char* b_src = static_cast<const char*>(b_host);
  FT_CUDA(cudaMemsetAsync(h->report, 0, 32, compute));
  for (int i = 0; i < g; ++i) {
    const size_t a_off = static_cast<size_t>(i) * mc * k, b_off = static_cast<size_t>(i) * nc * k;
    FT_CUDA(cudaMemcpyAsync(static_cast<char*>(h->own_a) + a_off, a_src + a_off, static_cast<size_t>(mc) * k, cudaMemcpyHostToDevice,
                            h->in_stream));
    FT_CUDA(cudaMemcpyAsync(static_cast<char*>(h->own_b) + b_off, b_src + b_off, static_cast<size_t>(nc) * k, cudaMemcpyHostToDevice,
                            h->in_stream));
    FT_CUDA(cudaEventRecord(in_done[i], h->in_stream));
    FT_CUDA(cudaStreamWaitEvent(compute, in_done[i], 0));
    // rows of chunk i against every column that has arrived (the corner included)
    rc = ft_gemm_fp8_abft_run_window(h, h->own_c, faults, n_faults, i * mc, mc, 0, (i + 1) * nc, 0, compute);
    if (rc != FT_OK) return rc;
    FT_CUDA(cudaEventRecord(c_done[2 * i], compute));
    FT_CUDA(cudaStreamWaitEvent(h->out_stream, c_done[2 * i], 0));
    FT_CUDA(cudaMemcpy2DAsync(c_host + static_cast<size_t>(i) * mc, pitch, h->own_c + static_cast<size_t>(i) * mc, pitch,
                              static_cast<size_t>(mc) * sizeof(float), static_cast<size_t>(i + 1) * nc, cudaMemcpyDeviceToHost,
                              h->out_stream));
    if (i > 0) {
      // columns of chunk i against the rows of the earlier chunks
      rc = ft_gemm_fp8_abft_run_window(h, h->own_c, faults, n_faults, 0, i * mc, i * nc, nc, 0, compute);
      if (rc != FT_OK) return rc;
      FT_CUDA(cudaEventRecord(c_done[2 * i + 1], compute));
      FT_CUDA(cudaStreamWaitEvent(h->out_stream, c_done[2 * i + 1], 0));
      const size_t off = static_cast<size_t>(i) * nc * m;
      FT_CUDA(cudaMemcpy2DAsync(c_host + off, pitch, h->own_c + off, pitch, static_cast<size_t>(i) * mc * sizeof(float),
                                static_cast<size_t>(nc), cudaMemcpyDeviceToHost, h->out_stream));
    }
  }
  FT_CUDA(cudaEventRecord(out_done, h->out_stream));
  FT_CUDA(cudaStreamWaitEvent(compute, out_done, 0));
  h->last_stream = compute;
  return FT_OK;
}

}  // namespace

extern "C" {

void ft_options_default(ft_options* options) {
  if (options == nullptr) return;
  std::memset(options, 0, sizeof(*options));
  options->abs_tol = 1.0e-2f;
  options->rel_tol = 2.0e-5f;
  options->sm_limit = 0;
  options->single_cta = 0;
  options->exact_prepare = 0;
}

const char* ft_gemm_last_error(void) { return g_error; }
int ft_gemm_abi_version(void) { return 1; }

int ft_gemm_fp8_abft_prepare(ft_gemm_handle** handle, const void* a, const void* b, int m, int n, int k, const ft_options* options,
                             void* stream_ptr) {
  if (handle == nullptr || a == nullptr || b == nullptr) return fail(FT_ERR_INVALID, "null handle or operand pointer");
  *handle = nullptr;
  int rc = check_shape(m, n, k);
  if (rc != FT_OK) return rc;
  const bool padded = k % 16 != 0 || (reinterpret_cast<uintptr_t>(a) & 15) != 0 || (reinterpret_cast<uintptr_t>(b) & 15) != 0;
  const int user_k = k;
  k = (k + 15) / 16 * 16;
  ft_options opts;
  ft_options_default(&opts);
  if (options != nullptr) opts = *options;
  if (opts.abs_tol < 0.0f || opts.rel_tol < 0.0f || opts.sm_limit < 0 || opts.wait_limit_us < 0) {
    return fail(FT_ERR_INVALID, "negative tolerance, sm_limit or wait_limit_us");
  }

  int device = 0;
  FT_CUDA(cudaGetDevice(&device));
  cudaDeviceProp prop;
  FT_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10) {
    return fail(FT_ERR_UNSUPPORTED, "this library needs an sm_100 GPU (found sm_%d%d)", prop.major, prop.minor);
  }
  FT_CUDA(configure_abft_gemm());

  ft_gemm_handle* h = new (std::nothrow) ft_gemm_handle();
  if (h == nullptr) return fail(FT_ERR_INVALID, "out of host memory");
  h->device = device;
  h->m = m;
  h->n = n;
  h->k = k;
  h->options = opts;
  h->a = a;
  h->b = b;
  h->user_a = a;
  h->user_b = b;
  h->user_k = user_k;
  if (padded) {
    cudaError_t perr = cudaMalloc(&h->pad_a, static_cast<size_t>(m) * k);
    if (perr == cudaSuccess) perr = cudaMalloc(&h->pad_b, static_cast<size_t>(n) * k);
    if (perr != cudaSuccess) {
      ft_gemm_fp8_abft_destroy(h);
      return fail(FT_ERR_CUDA, "allocating the padded operand copies failed: %s", cudaGetErrorString(perr));
    }
    h->a = h->pad_a;
    h->b = h->pad_b;
    a = h->pad_a;
    b = h->pad_b;
  }
  h->sm_count = prop.multiProcessorCount;
  h->pair = (m % 256 == 0) && opts.single_cta == 0;
  int sm_cap = opts.sm_limit > 0 ? std::min(opts.sm_limit, h->sm_count) : h->sm_count;
  if (h->pair) {
    int tiles = (m / 256) * ((n + 255) / 256);
    h->max_workers = std::max(1, sm_cap / 2);
    h->grid = 2 * std::max(1, std::min(tiles, sm_cap / 2));
  } else {
    int tiles = ((m + 127) / 128) * ((n + 255) / 256);
    h->max_workers = std::max(1, sm_cap);
    h->grid = std::min(tiles, sm_cap);
  }

  size_t a_meta = static_cast<size_t>((m + 63) / 64) * k, b_meta = static_cast<size_t>((n + 63) / 64) * k;
  size_t checks = static_cast<size_t>((m + 63) / 64) * ((n + 63) / 64) * 64;
  size_t floats = 2 * a_meta + 2 * b_meta + 4 * checks;
  const size_t planes_a = opts.exact_prepare != 0 ? 0 : prepare_mma_plane_bytes((m + 63) / 64, k);
  const size_t planes_b = opts.exact_prepare != 0 ? 0 : prepare_mma_plane_bytes((n + 63) / 64, k);
  h->cache_bytes = floats * sizeof(float) + 2 * planes_a + 2 * planes_b;
  cudaError_t err = opts.exact_prepare != 0 ? cudaSuccess : configure_prepare_mma();
  if (err == cudaSuccess) err = cudaMalloc(&h->cache_base, h->cache_bytes);
  if (err == cudaSuccess) err = cudaMalloc(&h->report_pair, 2 * sizeof(DeviceReport));
  h->report = h->report_pair;
  if (err == cudaSuccess) err = cudaMalloc(reinterpret_cast<void**>(&h->prepare_status), sizeof(int));
  if (err == cudaSuccess) err = cudaEventCreate(&h->ev0);
  if (err == cudaSuccess) err = cudaEventCreate(&h->ev_mid);
  if (err == cudaSuccess) err = cudaEventCreate(&h->ev1);
  if (err != cudaSuccess) {
    ft_gemm_fp8_abft_destroy(h);
    return fail(FT_ERR_CUDA, "allocating the expected-checksum cache (%zu bytes) failed: %s", h->cache_bytes,
                cudaGetErrorString(err));
  }
  float* cursor = h->cache_base;
  h->a_sums = cursor, cursor += a_meta;
  h->a_mags = cursor, cursor += a_meta;
  h->b_sums = cursor, cursor += b_meta;
  h->b_mags = cursor, cursor += b_meta;
  h->expected_rows = cursor, cursor += checks;
  h->expected_cols = cursor, cursor += checks;
  h->row_scales = cursor, cursor += checks;
  h->col_scales = cursor, cursor += checks;
  if (opts.exact_prepare == 0) {  // every offset is a multiple of 16 bytes: K % 32 == 0 and plane rows come in groups of 160
    uint8_t* bytes = reinterpret_cast<uint8_t*>(cursor);
    h->planes_as = bytes, bytes += planes_a;
    h->planes_am = bytes, bytes += planes_a;
    h->planes_bs = bytes, bytes += planes_b;
    h->planes_bm = bytes, bytes += planes_b;
  }

  rc = make_operand_map(&h->tmap_a, a, m, k, 128);
  if (rc == FT_OK) rc = make_operand_map(&h->tmap_b, b, n, k, h->pair ? 128 : 256);
  if (rc == FT_OK && opts.exact_prepare == 0) {
    const int rows_a = prepare_mma_plane_rows((m + 63) / 64), rows_b = prepare_mma_plane_rows((n + 63) / 64);
    rc = make_operand_map(&h->tmap_b128, b, n, k, 128);
    if (rc == FT_OK) rc = make_operand_map(&h->tmap_as, h->planes_as, rows_a, k, 160);
    if (rc == FT_OK) rc = make_operand_map(&h->tmap_am, h->planes_am, rows_a, k, 160);
    if (rc == FT_OK) rc = make_operand_map(&h->tmap_bs, h->planes_bs, rows_b, k, 160);
    if (rc == FT_OK) rc = make_operand_map(&h->tmap_bm, h->planes_bm, rows_b, k, 160);
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  if (rc == FT_OK) {
    cudaError_t merr = cudaMemsetAsync(h->report_pair, 0, 2 * sizeof(DeviceReport), stream);
    if (merr == cudaSuccess) merr = cudaMemsetAsync(h->prepare_status, 0, sizeof(int), stream);
    if (merr != cudaSuccess) rc = fail(FT_ERR_CUDA, "cudaMemsetAsync failed: %s", cudaGetErrorString(merr));
  }
  if (rc == FT_OK) rc = copy_padded(h, 3, stream);
  if (rc == FT_OK) rc = fill_cache(h, 3, stream);
  if (rc != FT_OK) {
    ft_gemm_fp8_abft_destroy(h);
    return rc;
  }
  *handle = h;
  return FT_OK;
}

int ft_gemm_fp8_abft_refresh(ft_gemm_handle* h, int which, void* stream_ptr) {
  if (h == nullptr || (which & 3) == 0) return fail(FT_ERR_INVALID, "null handle or empty refresh mask");
  int rc = copy_padded(h, which & 3, static_cast<cudaStream_t>(stream_ptr));
  if (rc != FT_OK) return rc;
  return fill_cache(h, which & 3, static_cast<cudaStream_t>(stream_ptr));
}

int ft_gemm_fp8_abft_quantize_a(ft_gemm_handle* h, const void* src, int src_dtype, float scale, void* stream_ptr) {
  if (h == nullptr || src == nullptr) return fail(FT_ERR_INVALID, "null handle or source pointer");
  if (src_dtype < FT_SRC_F32 || src_dtype > FT_SRC_F16) return fail(FT_ERR_INVALID, "src_dtype must be 0 (FP32), 1 (BF16) or 2 (FP16)");
  if ((reinterpret_cast<uintptr_t>(src) & 15) != 0) return fail(FT_ERR_INVALID, "the source must be 16-byte aligned");
  if (!(scale == scale) || scale == 0.0f) return fail(FT_ERR_INVALID, "scale must be a non-zero number");
  if (h->pad_a != nullptr) return fail(FT_ERR_UNSUPPORTED, "the fused producer of A needs K %% 16 == 0 and a 16-byte aligned A");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  FT_CUDA(cudaMemsetAsync(h->prepare_status, 0, sizeof(int), stream));
  FT_CUDA(cudaEventRecord(h->ev0, stream));
  // A and its band sums in one pass over the source; the caller's A buffer is written here
  FT_CUDA(launch_quantize_band_sums(src, src_dtype, const_cast<void*>(h->a), h->a_sums, h->a_mags, h->m, h->k, scale, stream));
  FT_CUDA(cudaEventRecord(h->ev_mid, stream));
  int rc = fill_expected(h, 1, stream);
  if (rc != FT_OK) return rc;
  FT_CUDA(cudaEventRecord(h->ev1, stream));
  h->prepare_timed = true;
  h->last_stream = stream;
  return FT_OK;
}

int ft_gemm_fp8_abft_set_tolerance(ft_gemm_handle* h, float abs_tol, float rel_tol) {
  if (h == nullptr || abs_tol < 0.0f || rel_tol < 0.0f) return fail(FT_ERR_INVALID, "null handle or negative tolerance");
  h->options.abs_tol = abs_tol;
  h->options.rel_tol = rel_tol;
  return FT_OK;
}

int ft_gemm_fp8_abft_run(ft_gemm_handle* h, float* c, const ft_fault* faults, int n_faults, void* stream_ptr) {
  if (h == nullptr) return fail(FT_ERR_INVALID, "null handle or output pointer");
  return ft_gemm_fp8_abft_run_window(h, c, faults, n_faults, 0, h->m, 0, h->n, 1, stream_ptr);
}

int ft_gemm_fp8_abft_run_window(ft_gemm_handle* h, float* c, const ft_fault* faults, int n_faults, int row0, int rows, int col0,
                                int cols, int zero_report, void* stream_ptr) {
  if (h == nullptr || c == nullptr) return fail(FT_ERR_INVALID, "null handle or output pointer");
  if (n_faults < 0 || n_faults > FT_MAX_FAULTS || (n_faults > 0 && faults == nullptr)) {
    return fail(FT_ERR_INVALID, "n_faults must be in [0, %d]", FT_MAX_FAULTS);
  }
  const int tile_m = h->pair ? 256 : 128;
  if (row0 < 0 || rows <= 0 || col0 < 0 || cols <= 0 || row0 % tile_m != 0 || col0 % 256 != 0 || row0 + rows > h->m ||
      col0 + cols > h->n || (rows % tile_m != 0 && row0 + rows != h->m) || (cols % 256 != 0 && col0 + cols != h->n)) {
    return fail(FT_ERR_INVALID,
                "window rows [%d,+%d) cols [%d,+%d) must lie inside %dx%d on multiples of %d rows and 256 columns (the last "
                "row and column blocks may be short)",
                row0, rows, col0, cols, h->m, h->n, tile_m);
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  GemmParams params{};
  fill_params(h, c, &params);
  params.row0 = row0;
  params.rows = rows;
  params.col0 = col0;
  params.cols = cols;
  params.faults.count = n_faults;
  int tile_count = ((h->m + 63) / 64) * ((h->n + 63) / 64);
  for (int i = 0; i < n_faults; ++i) {
    if (faults[i].tile < 0 || faults[i].tile >= tile_count || faults[i].row < 0 || faults[i].col < 0) {
      return fail(FT_ERR_INVALID, "fault %d is outside the %d ABFT tiles", i, tile_count);
    }
    params.faults.tile[i] = faults[i].tile;
    params.faults.row[i] = faults[i].row;
    params.faults.col[i] = faults[i].col;
    params.faults.value[i] = faults[i].value;
  }
  // In place of the reference's two counter memsets (src/s4:693-694): a new report goes to the other buffer, whose
  // counters the previous such launch (or the prepare) has cleared, and this launch clears the one it leaves.
  if (zero_report) {
    h->report_index ^= 1;
    h->report = h->report_pair + h->report_index;
    params.report = h->report;
    params.clear_counters = reinterpret_cast<int*>(h->report_pair + (h->report_index ^ 1));
  }
  int tiles = ((rows + tile_m - 1) / tile_m) * ((cols + 255) / 256);
  choose_split(tiles, h->max_workers, h->k, &params.split_from, &params.split);
  const int items = params.split_from + (tiles - params.split_from) * params.split;
  const int workers = std::min(h->max_workers, items);
  const int grid = h->pair ? 2 * workers : workers;
  FT_CUDA(launch_abft_gemm(h->tmap_a, h->tmap_b, params, grid, h->pair, stream));
  h->last_stream = stream;
  return FT_OK;
}

int ft_gemm_fp8_abft_run_profiled(ft_gemm_handle* h, float* c, unsigned long long* counters_host, int max_ctas, int* ctas,
                                  void* stream_ptr) {
  if (h == nullptr || c == nullptr || counters_host == nullptr || max_ctas <= 0) return fail(FT_ERR_INVALID, "null pointer");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  unsigned long long* dev = nullptr;
  size_t bytes = static_cast<size_t>(h->grid) * 8 * sizeof(unsigned long long);
  FT_CUDA(cudaMalloc(reinterpret_cast<void**>(&dev), bytes));
  GemmParams params{};
  fill_params(h, c, &params);
  params.profile = dev;
  cudaError_t err = cudaMemsetAsync(dev, 0, bytes, stream);  // every failure below still reaches the cudaFree
  if (err == cudaSuccess) err = cudaMemsetAsync(h->report, 0, 32, stream);
  if (err == cudaSuccess) err = launch_abft_gemm(h->tmap_a, h->tmap_b, params, h->grid, h->pair, stream);
  if (err == cudaSuccess) err = cudaStreamSynchronize(stream);
  int n = std::min(h->grid, max_ctas);
  if (err == cudaSuccess) err = cudaMemcpy(counters_host, dev, static_cast<size_t>(n) * 8 * sizeof(unsigned long long), cudaMemcpyDeviceToHost);
  cudaFree(dev);
  h->last_stream = stream;
  if (ctas != nullptr) *ctas = h->grid;
  if (err != cudaSuccess) return fail(FT_ERR_CUDA, "profiled run failed: %s", cudaGetErrorString(err));
  return FT_OK;
}

int ft_gemm_fp8_abft_report(ft_gemm_handle* h, ft_report* out) {
  if (h == nullptr || out == nullptr) return fail(FT_ERR_INVALID, "null handle or report pointer");
  FT_CUDA(cudaStreamSynchronize(h->last_stream));
  DeviceReport dev;
  FT_CUDA(cudaMemcpy(&dev, h->report, sizeof(DeviceReport), cudaMemcpyDeviceToHost));
  int prepare_status = 0;
  FT_CUDA(cudaMemcpy(&prepare_status, h->prepare_status, sizeof(int), cudaMemcpyDeviceToHost));
  if (prepare_status != 0) dev.status = prepare_status;  // a prepare kernel gave up: the cache is not valid
  std::memset(out, 0, sizeof(*out));
  out->status = dev.status != 0 ? FT_ERR_TIMEOUT : FT_OK;
  out->bad_tiles = dev.bad_tiles;
  out->corrected_tiles = dev.corrected_tiles;
  out->multi_fault_tiles = dev.multi_fault_tiles;
  int kept = std::min(dev.record_count, FT_MAX_RECORDS);
  out->n_records = kept;
  out->records_dropped = dev.record_count - kept;
  std::memcpy(&out->max_clean_ratio, &dev.max_clean_ratio_bits, sizeof(float));
  std::copy(dev.records, dev.records + kept, out->records);
  std::sort(out->records, out->records + kept, [](const ft_tile_record& x, const ft_tile_record& y) { return x.tile < y.tile; });
  if (h->prepare_timed) {
    float ms = 0.0f;
    if (cudaEventElapsedTime(&ms, h->ev0, h->ev1) == cudaSuccess) out->prepare_ms = ms;
    if (cudaEventElapsedTime(&ms, h->ev0, h->ev_mid) == cudaSuccess) out->prepare_input_ms = ms;
    if (cudaEventElapsedTime(&ms, h->ev_mid, h->ev1) == cudaSuccess) out->prepare_expected_ms = ms;
  }
  if (dev.status != 0) {
    return fail(FT_ERR_TIMEOUT, "a device-side wait expired; the output of this run is not valid (after a prepare time-out, "
                                "_refresh the handle)");
  }
  return FT_OK;
}

int ft_gemm_fp8_abft_selftest_wait(ft_gemm_handle* h, int limit_us, void* stream_ptr) {
  if (h == nullptr || limit_us <= 0 || limit_us > 1000000) return fail(FT_ERR_INVALID, "null handle, or limit_us outside [1, 1000000]");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  FT_CUDA(cudaMemsetAsync(h->report, 0, 32, stream));
  FT_CUDA(launch_selftest_wait(h->report, 1000ull * static_cast<unsigned long long>(limit_us), stream));
  h->last_stream = stream;
  return FT_OK;
}

int ft_gemm_report_rebase(ft_report* report, int tile_cols, int first_tile_row) {
  if (report == nullptr || tile_cols <= 0 || first_tile_row < 0) return fail(FT_ERR_INVALID, "null report, or bad tile_cols / first_tile_row");
  for (int i = 0; i < report->n_records && i < FT_MAX_RECORDS; ++i) report->records[i].tile += first_tile_row * tile_cols;
  return FT_OK;
}

int ft_gemm_report_merge(const ft_report* shards, int n, ft_report* out) {
  if (shards == nullptr || out == nullptr || n <= 0) return fail(FT_ERR_INVALID, "null report pointer or no shards");
  ft_report merged;
  std::memset(&merged, 0, sizeof(merged));
  for (int s = 0; s < n; ++s) {
    const ft_report& r = shards[s];
    if (merged.status == FT_OK) merged.status = r.status;
    merged.bad_tiles += r.bad_tiles;
    merged.corrected_tiles += r.corrected_tiles;
    merged.multi_fault_tiles += r.multi_fault_tiles;
    merged.records_dropped += r.records_dropped;
    merged.max_clean_ratio = std::max(merged.max_clean_ratio, r.max_clean_ratio);
    merged.prepare_ms = std::max(merged.prepare_ms, r.prepare_ms);
    merged.prepare_input_ms = std::max(merged.prepare_input_ms, r.prepare_input_ms);
    merged.prepare_expected_ms = std::max(merged.prepare_expected_ms, r.prepare_expected_ms);
    const int count = std::max(0, std::min(r.n_records, FT_MAX_RECORDS));
    for (int i = 0; i < count; ++i) {
      if (merged.n_records < FT_MAX_RECORDS) {
        merged.records[merged.n_records++] = r.records[i];
      } else {
        ++merged.records_dropped;
      }
    }
  }
  *out = merged;
  return FT_OK;
}

int ft_gemm_fp8_abft_cache(ft_gemm_handle* h, ft_cache_view* out) {
  if (h == nullptr || out == nullptr) return fail(FT_ERR_INVALID, "null handle or view pointer");
  out->a_sums = h->a_sums;
  out->a_magnitudes = h->a_mags;
  out->b_sums = h->b_sums;
  out->b_magnitudes = h->b_mags;
  out->expected_rows = h->expected_rows;
  out->expected_cols = h->expected_cols;
  out->row_scales = h->row_scales;
  out->col_scales = h->col_scales;
  out->bytes = h->cache_bytes;
  return FT_OK;
}

int ft_gemm_fp8_abft_cache_read(ft_gemm_handle* h, int which, float* host_out, size_t count) {
  if (h == nullptr || host_out == nullptr || which < 0 || which > 7) return fail(FT_ERR_INVALID, "null pointer or bad array index");
  const float* arrays[8] = {h->a_sums, h->a_mags, h->b_sums, h->b_mags, h->expected_rows, h->expected_cols, h->row_scales, h->col_scales};
  size_t a_meta = static_cast<size_t>((h->m + 63) / 64) * h->k, b_meta = static_cast<size_t>((h->n + 63) / 64) * h->k;
  size_t checks = static_cast<size_t>((h->m + 63) / 64) * ((h->n + 63) / 64) * 64;
  size_t sizes[8] = {a_meta, a_meta, b_meta, b_meta, checks, checks, checks, checks};
  if (count > sizes[which]) return fail(FT_ERR_INVALID, "array %d holds %zu floats, %zu requested", which, sizes[which], count);
  FT_CUDA(cudaStreamSynchronize(h->last_stream));
  FT_CUDA(cudaMemcpy(host_out, arrays[which], count * sizeof(float), cudaMemcpyDeviceToHost));
  return FT_OK;
}

int ft_gemm_fp8_abft_destroy(ft_gemm_handle* h) {
  if (h == nullptr) return FT_OK;
  if (h->last_stream != nullptr || h->cache_base != nullptr) cudaStreamSynchronize(h->last_stream);
  cudaFree(h->cache_base);
  cudaFree(h->report_pair);
  cudaFree(h->prepare_status);
  if (h->ev0) cudaEventDestroy(h->ev0);
  if (h->ev_mid) cudaEventDestroy(h->ev_mid);
  if (h->ev1) cudaEventDestroy(h->ev1);
  cudaFree(h->pad_a);
  cudaFree(h->pad_b);
  cudaFree(h->own_a);
  cudaFree(h->own_b);
  cudaFree(h->own_c);
  if (h->own_stream) cudaStreamDestroy(h->own_stream);
  if (h->in_stream) cudaStreamDestroy(h->in_stream);
  if (h->out_stream) cudaStreamDestroy(h->out_stream);
  for (cudaEvent_t e : h->pipe_events) {
    if (e) cudaEventDestroy(e);
  }
  delete h;
  return FT_OK;
}

int ft_gemm_generate_fp8(void* out, size_t count, uint32_t seed, int dist, float sigma, float post_scale, void* stream_ptr) {
  if (out == nullptr && count > 0) return fail(FT_ERR_INVALID, "null output pointer");
  if (dist != 0 && dist != 1) return fail(FT_ERR_INVALID, "dist must be 0 (uniform) or 1 (normal)");
  FT_CUDA(launch_generate(out, count, seed, dist, sigma, post_scale, static_cast<cudaStream_t>(stream_ptr)));
  return FT_OK;
}

int ft_gemm_fp8_abft_host(ft_gemm_handle** reuse, const void* a_host, const void* b_host, float* c_host, int m, int n, int k,
                          const ft_options* options, const ft_fault* faults, int n_faults, int prepare, ft_report* report) {
  if (a_host == nullptr || b_host == nullptr || c_host == nullptr || report == nullptr) {
    return fail(FT_ERR_INVALID, "null host buffer or report pointer");
  }
  int rc = check_shape(m, n, k);
  if (rc != FT_OK) return rc;
  ft_gemm_handle* h = reuse != nullptr ? *reuse : nullptr;
  size_t a_bytes = static_cast<size_t>(m) * k, b_bytes = static_cast<size_t>(n) * k, c_bytes = static_cast<size_t>(m) * n * 4;
  bool fresh = h == nullptr;
  if (!fresh && (h->m != m || h->n != n || h->user_k != k || h->own_a == nullptr)) {
    return fail(FT_ERR_INVALID, "the handle passed for reuse was not created by this entry point with the same shape");
  }
  void *da = nullptr, *db = nullptr;
  float* dc = nullptr;
  cudaStream_t stream = nullptr;
  if (fresh) {
    FT_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    cudaError_t err = cudaMalloc(&da, a_bytes);
    if (err == cudaSuccess) err = cudaMalloc(&db, b_bytes);
    if (err == cudaSuccess) err = cudaMalloc(reinterpret_cast<void**>(&dc), c_bytes);
    if (err != cudaSuccess) {
      cudaFree(da);
      cudaFree(db);
      cudaFree(dc);
      cudaStreamDestroy(stream);
      return fail(FT_ERR_CUDA, "allocating device operands failed: %s", cudaGetErrorString(err));
    }
  } else {
    da = h->own_a;
    db = h->own_b;
    dc = h->own_c;
    stream = h->own_stream;
  }
  const int chunks = (!fresh && !prepare) ? pipe_chunks(h) : 1;
  if (chunks > 1) {
    rc = host_pipelined(h, a_host, b_host, c_host, faults, n_faults, chunks);
    if (rc != FT_OK) {  // nothing may still be writing into the caller's memory when the error is returned
      cudaStreamSynchronize(h->in_stream);
      cudaStreamSynchronize(h->out_stream);
    }
  } else {
    cudaError_t err = cudaMemcpyAsync(da, a_host, a_bytes, cudaMemcpyHostToDevice, stream);
    if (err == cudaSuccess) err = cudaMemcpyAsync(db, b_host, b_bytes, cudaMemcpyHostToDevice, stream);
    if (err != cudaSuccess) rc = fail(FT_ERR_CUDA, "host-to-device copy failed: %s", cudaGetErrorString(err));
    if (rc == FT_OK && fresh) {
      rc = ft_gemm_fp8_abft_prepare(&h, da, db, m, n, k, options, stream);
      if (rc == FT_OK) {
        h->own_a = da;
        h->own_b = db;
        h->own_c = dc;
        h->own_stream = stream;
      } else {
        cudaFree(da);
        cudaFree(db);
        cudaFree(dc);
        cudaStreamDestroy(stream);
        return rc;
      }
    } else if (rc == FT_OK && prepare) {
      rc = ft_gemm_fp8_abft_refresh(h, 3, stream);
    } else if (rc == FT_OK) {
      rc = copy_padded(h, 3, stream);
    }
    if (rc == FT_OK) rc = ft_gemm_fp8_abft_run(h, dc, faults, n_faults, stream);
    if (rc == FT_OK) {
      err = cudaMemcpyAsync(c_host, dc, c_bytes, cudaMemcpyDeviceToHost, stream);
      if (err != cudaSuccess) rc = fail(FT_ERR_CUDA, "device-to-host copy failed: %s", cudaGetErrorString(err));
    }
  }
  if (h == nullptr) {  // a fresh call whose copies failed before a handle existed: the error text stays, nothing leaks
    cudaFree(da);
    cudaFree(db);
    cudaFree(dc);
    cudaStreamDestroy(stream);
    return rc;
  }
  int report_rc = ft_gemm_fp8_abft_report(h, report);
  if (rc == FT_OK) rc = report_rc;
  if (reuse != nullptr) {
    *reuse = h;
  } else {
    ft_gemm_fp8_abft_destroy(h);
  }
  return rc;
}

}  // extern "C"
