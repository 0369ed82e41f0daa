/*
 * ft_gemm.h -- C-ABI of the B200 fault-tolerant FP8 GEMM library.
 *
 * The reference project (chaiduo/FT-GEMM) has no library boundary: every stage is
 * a standalone program whose main() owns the device buffers and launches the
 * kernels in the fixed ABFT order  prepare expected checksums -> GEMM -> actual
 * checksums -> compare -> single-point correct.  The entry points below are that
 * kernel-launch interface made callable: each one cites the reference lines it
 * replaces.  All pointers are plain device or host pointers, `stream` is a
 * cudaStream_t passed as void* (NULL = the default stream); no function exits the
 * process, traps or allocates behind the caller's back except where stated.
 *
 * Operator contract (same as the reference's S1-S4 programs,
 * src/s4_cluster_multicast_abft_fp8_gemm.cu:744-745):
 *   A  [M,K]  FP8 E4M3, K contiguous
 *   B  [N,K]  FP8 E4M3, K contiguous
 *   C  [N,M]  FP32 column-major: element (row r, column c) at C[c*M + r]
 *   ABFT tiles are 64x64; tile_id = (r/64) * ceil(N/64) + (c/64)
 *   Any positive M, N and K (for K % 16 != 0, or operands that are not 16-byte
 *   aligned, the handle works on zero-padded copies of A and B that _prepare and
 *   _refresh fill; the band-sum arrays then have ceil16(K) columns).  The
 *   reference's tensor-core stages take
 *   boundary tiles in N (src/s3_warpspecialized_abft_fp8_gemm.cu:144-154, 418-419:
 *   M % 128 == 0, K % 32 == 0), its first stage any shape
 *   (src/s0_tiled_abft_fp8_gemm.cu:143-144); here the last tile row / column holds
 *   M % 64 / N % 64 valid rows / columns, cached checksums past them are zeros
 *   (src/s4_cluster_multicast_abft_fp8_gemm.cu:284-293) and fault positions are
 *   clamped into the valid part.  The final stage's M % 128 == 0, N % 256 == 0,
 *   K % 128 == 0 (src/s4:163-169) is a special case.
 *
 * Every function returns FT_OK (0) or a negative FT_ERR_* code; the text of the
 * last error of the calling thread is available from ft_gemm_last_error().
 * A handle may be used by one host thread at a time, and its _run / _run_window /
 * _refresh / _report calls belong to ONE stream at a time: the handle keeps two
 * report buffers that successive launches use alternately, and _report waits for
 * the stream of the last launch only.  Launch on another stream only after the
 * previous stream's work on the handle has finished (an event or _report).
 */
#ifndef FT_GEMM_H
#define FT_GEMM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FT_OK 0
#define FT_ERR_INVALID (-1)   /* bad shape, pointer or option */
#define FT_ERR_CUDA (-2)      /* a CUDA call failed; see ft_gemm_last_error() */
#define FT_ERR_TIMEOUT (-3)   /* a device-side wait gave up; results are not valid */
#define FT_ERR_UNSUPPORTED (-4) /* not an sm_100 device */

#define FT_ABFT_TILE 64
#define FT_MAX_FAULTS 4
#define FT_MAX_RECORDS 64

typedef struct ft_gemm_handle ft_gemm_handle;

/* Options of the checker; defaults are the reference's
 * (src/s4_cluster_multicast_abft_fp8_gemm.cu:98-99). */
typedef struct {
  float abs_tol;  /* default 1e-2 */
  float rel_tol;  /* default 2e-5 */
  int sm_limit;   /* 0 = one persistent CTA per SM; >0 caps the grid (testing) */
  int single_cta; /* 0 = pair two CTAs on one 256x256 tile when M % 256 == 0; 1 = always one CTA per 128x256 tile */
  int exact_prepare; /* 0 (default): the expected checksums are computed on the tensor cores (band sums split into exact
                        E4M3 digits; equal to the reference's values up to FP32 accumulation order); 1: on the CUDA
                        cores in the reference's summation order (src/s4:264-282), bit-identical to its cache, ~10x slower */
  int wait_limit_us; /* 0 (default): a device-side wait of the fused GEMM kernel gives up after 2 s; >0: after this many
                        microseconds.  A kernel whose wait gave up leaves through its normal teardown and the run is
                        reported as FT_ERR_TIMEOUT; nothing traps or spins without limit. */
  int reserved[2];
} ft_options;

/* A test fault: `value` is added to the accumulator element (row, col) of ABFT
 * tile `tile` after the main loop and before the checksums
 * (src/s4_random_fault_campaign.cu:321-322, 464-466; row and col are clamped to
 * 63 like there). */
typedef struct {
  int tile;
  int row;
  int col;
  float value;
} ft_fault;

/* One record per tile whose checker fired (src/s4:489-499 keeps only two global
 * counters; the per-tile detail is what its shared-memory state holds). */
typedef struct {
  int tile;          /* ABFT tile id */
  int bad_row_count; /* checksums over threshold */
  int bad_col_count;
  int bad_row;       /* lowest bad local row, -1 if none */
  int bad_col;       /* lowest bad local column, -1 if none */
  float row_delta;   /* expected - actual of bad_row */
  float col_delta;   /* expected - actual of bad_col */
  int corrected;     /* 1 iff exactly one row and one column were bad */
} ft_tile_record;

typedef struct {
  int status;            /* FT_OK or FT_ERR_TIMEOUT */
  int bad_tiles;         /* tiles with rows>0 || cols>0 (src/s4:490) */
  int corrected_tiles;   /* tiles with rows==1 && cols==1 (src/s4:493-499) */
  int multi_fault_tiles; /* bad but not corrected: reported, never silently fixed */
  int n_records;         /* valid entries of records[], sorted by tile id */
  int records_dropped;   /* bad tiles beyond FT_MAX_RECORDS */
  float max_clean_ratio; /* max |delta| / threshold over checks that passed: the clean-run noise level */
  float prepare_ms;      /* device time of the last prepare (band sums + expected checksums) */
  float prepare_input_ms;    /* of which: band sums (the reference's input_metadata_time_ms) */
  float prepare_expected_ms; /* of which: expected checksums (expected_metadata_time_ms) */
  ft_tile_record records[FT_MAX_RECORDS];
} ft_report;

/* Pointers into the handle's expected-checksum cache (device memory, owned by
 * the handle), laid out exactly as the reference's buffers
 * (src/s4_cluster_multicast_abft_fp8_gemm.cu:584-598). */
typedef struct {
  const float* a_sums;        /* [M/64, K] */
  const float* a_magnitudes;  /* [M/64, K] */
  const float* b_sums;        /* [N/64, K] */
  const float* b_magnitudes;  /* [N/64, K] */
  const float* expected_rows; /* [tiles*64] */
  const float* expected_cols; /* [tiles*64] */
  const float* row_scales;    /* [tiles*64] */
  const float* col_scales;    /* [tiles*64] */
  size_t bytes;               /* total size of the eight arrays */
} ft_cache_view;

void ft_options_default(ft_options* options);

/* Replaces the reference's cudaMalloc of the metadata buffers, its two prepare
 * launches cache_input_tile_checksums_kernel + cache_expected_tile_checksums_kernel
 * and its tensor-map construction (src/s4_cluster_multicast_abft_fp8_gemm.cu:
 * 584-598, 608-617, 634-655).  Allocates the cache (freed by _destroy), fills it
 * from A and B on `stream` and returns a handle bound to these A, B pointers.
 * The cache is valid while the contents of A and B are unchanged. */
int ft_gemm_fp8_abft_prepare(ft_gemm_handle** handle, const void* a_e4m3, const void* b_e4m3, int m, int n, int k,
                             const ft_options* options, void* stream);

/* Recomputes the cache of an existing handle after A and/or B changed in place
 * (same pointers, same shape).  which: bit 0 = A changed, bit 1 = B changed. */
int ft_gemm_fp8_abft_refresh(ft_gemm_handle* handle, int which, void* stream);

/* Producer of A fused with its band sums, for callers whose A is produced on the
 * device in a wider type (activations of an FP8 projection).  The reference makes
 * a separate pass over the finished FP8 A for a_sums / a_magnitudes
 * (src/s4_cluster_multicast_abft_fp8_gemm.cu:194-235, 634-640).  Here one pass
 * over src [M,K] (row-major, src_dtype FT_SRC_*) writes E4M3(src * scale), rounded
 * to nearest even and saturated, into the A buffer the handle was prepared with
 * (which must be writable), accumulates the band sums of the rounded values in the
 * reference's order, and is followed by the two expected-checksum launches; B's
 * band sums are reused.  The resulting A and cache are bit-identical to quantising
 * first and calling _refresh(handle, 1, ...). */
#define FT_SRC_F32 0
#define FT_SRC_BF16 1
#define FT_SRC_F16 2
int ft_gemm_fp8_abft_quantize_a(ft_gemm_handle* handle, const void* src, int src_dtype, float scale, void* stream);

/* Replaces one enqueue_gemm() of the reference together with the two counter
 * memsets in front of it (src/s4_cluster_multicast_abft_fp8_gemm.cu:657-672,
 * 693-694): zeroes the handle's report and launches the fused GEMM + checker +
 * corrector on `stream`.  Asynchronous.  `faults` may be NULL (n_faults = 0). */
int ft_gemm_fp8_abft_run(ft_gemm_handle* handle, float* c, const ft_fault* faults, int n_faults, void* stream);

/* The same launch restricted to the window rows [row0, row0+rows) x columns
 * [col0, col0+cols) of the product (the reference always launches the whole grid,
 * src/s4_cluster_multicast_abft_fp8_gemm.cu:657-672).  `c` is still the base of
 * the full [N,M] output, tile ids in faults and records stay global.  row0 and
 * rows must be multiples of 256 (128 for a handle in the one-CTA form), col0 and
 * cols of 256, except that a window may end at M or N.  With zero_report = 0 the counters of earlier windows are kept, so
 * a caller whose operands arrive in pieces can cover the product with several
 * windows and read one report. */
int ft_gemm_fp8_abft_run_window(ft_gemm_handle* handle, float* c, const ft_fault* faults, int n_faults, int row0, int rows,
                                int col0, int cols, int zero_report, void* stream);

/* Diagnostic variant of _run without faults: additionally records, per CTA, how
 * many clock cycles each role spent waiting (8 counters per CTA: producer waiting
 * for a free stage, MMA waiting for a full stage, MMA waiting for a drained
 * accumulator, MMA role total, epilogue waiting for an accumulator, epilogue
 * total, tiles processed, spare).  Synchronous; `counters_host` receives
 * min(ctas, max_ctas) * 8 values and *ctas the grid size.  The reference has no
 * such hook; its timing is event-based only (src/s4:692-702). */
int ft_gemm_fp8_abft_run_profiled(ft_gemm_handle* handle, float* c, unsigned long long* counters_host, int max_ctas, int* ctas,
                                  void* stream);

/* Replaces the reference's read-back of bad_tiles / corrected_tiles
 * (src/s4_cluster_multicast_abft_fp8_gemm.cu:711-714): waits for the stream of the
 * last _run and copies its report to host memory.  Returns FT_ERR_TIMEOUT (and
 * sets out->status) when a device-side wait gave up. */
int ft_gemm_fp8_abft_report(ft_gemm_handle* handle, ft_report* out);

/* Multi-GPU reports (the reference is single-GPU, src/s4:558; its two counters
 * become one report per row band).  _report_rebase turns the band-local tile ids of
 * a shard's report into ids of the whole product: the band starts at tile row
 * first_tile_row (= first row of the band / 64) of a product with tile_cols =
 * ceil(N/64) tile columns.  _report_merge forms the union of n re-based reports in
 * the order given (rank order): counters added, records concatenated up to
 * FT_MAX_RECORDS (the rest counted in records_dropped), status = the first
 * non-zero status, max_clean_ratio / prepare times = the maximum.  Both are plain
 * host functions: whoever moves the fixed-size ft_report between ranks (one
 * ncclAllGather in the stage program, torch.distributed in the Python host) calls
 * them on the gathered array. */
int ft_gemm_report_rebase(ft_report* report, int tile_cols, int first_tile_row);
int ft_gemm_report_merge(const ft_report* shards, int n, ft_report* out);

/* Test hook for the failure path (no counterpart in the reference, whose kernels
 * wait without limit): launches a one-thread kernel that waits, with the same
 * bounded-wait routine every kernel of this library uses, on a barrier nobody
 * arrives on.  After limit_us microseconds the wait gives up and the kernel
 * records the time-out in the handle's current report exactly as the fused
 * kernel's teardown does, so the next _report returns FT_ERR_TIMEOUT.  The kernel
 * touches no tensor memory, issues no copy and no MMA; the context stays usable
 * and the next _run starts a clean report. */
int ft_gemm_fp8_abft_selftest_wait(ft_gemm_handle* handle, int limit_us, void* stream);

/* Frees the cache (the reference's cudaFree block, src/s4:771-783). */
int ft_gemm_fp8_abft_destroy(ft_gemm_handle* handle);

int ft_gemm_fp8_abft_cache(ft_gemm_handle* handle, ft_cache_view* out);

/* Inspection helper (the reference never reads its metadata back): waits for the
 * handle's stream and copies `count` floats of one cache array to host memory.
 * which: 0 a_sums, 1 a_magnitudes, 2 b_sums, 3 b_magnitudes, 4 expected_rows,
 * 5 expected_cols, 6 row_scales, 7 col_scales. */
int ft_gemm_fp8_abft_cache_read(ft_gemm_handle* handle, int which, float* host_out, size_t count);

/* Tolerances can be changed between runs without re-preparing (they are kernel
 * arguments in the reference, src/s4:306-307). */
int ft_gemm_fp8_abft_set_tolerance(ft_gemm_handle* handle, float abs_tol, float rel_tol);

/* The same operator with HOST buffers: copies A and B to the device, prepares
 * (when `reuse` is NULL) or reuses the cache of *reuse, runs, copies C back and
 * fills `report`.  a, b, c should be pinned for full copy bandwidth.  With a
 * reused handle and prepare = 0 the call is pipelined: A and B travel in up to 8
 * row chunks each, every part of C is computed by a window launch as soon as its
 * operands are on the device and copied back while later chunks are still on
 * their way (three streams).  When
 * `reuse` is non-NULL and *reuse is NULL a new handle with its own device
 * buffers is created and returned there for later calls; destroy it with
 * ft_gemm_fp8_abft_destroy. */
int ft_gemm_fp8_abft_host(ft_gemm_handle** reuse, const void* a_host, const void* b_host, float* c_host, int m, int n, int k,
                          const ft_options* options, const ft_fault* faults, int n_faults, int prepare, ft_report* report);

/* Seeded input generators on the device.  dist 0: the reference's
 * E4M3(2u-1), u = (mix(seed+i) & 0xffffff) / 2^24
 * (src/s0_tiled_abft_fp8_gemm.cu:93-110, bit-exact).  dist 1: E4M3(z * sigma *
 * post_scale) with z ~ N(0,1) by Box-Muller over two hash draws. */
int ft_gemm_generate_fp8(void* out_e4m3, size_t count, uint32_t seed, int dist, float sigma, float post_scale, void* stream);

/* No counterpart in the reference (its programs allocate everything up front in
 * main()).  Fills the four expected-checksum arrays for A[M,K], B[N,K] exactly as
 * ft_gemm_fp8_abft_prepare does, but allocates nothing: the caller passes the
 * outputs and the intermediate band sums are kept in an array built into the
 * library, 16 MiB on every GPU that loads it.  It exists for callers that cannot
 * call cudaMalloc where they need new checksums -- a serving loop that refreshes
 * them whenever A changes while the framework's allocator owns the device memory,
 * or that cannot take the device-wide stall cudaMalloc causes.
 *   - Any positive M and N, K % 16 == 0, A and B 16-byte aligned.  Each of the
 *     four outputs holds ceil(M/64) * ceil(N/64) * 64 floats of device memory
 *     (boundary tiles count in full; entries past the last valid column are
 *     written as zeros): M = 100, N = 256 needs 2 * 4 * 64 = 512 floats each.
 *   - Shapes with 2*(ceil(M/64) + ceil(N/64))*K*4 bytes > FT_NOALLOC_MAX_SCRATCH_BYTES
 *     are rejected with FT_ERR_INVALID (8192^3 fits exactly); use _prepare for them.
 *   - The first call on each device looks the array's device address up (with
 *     that device current).  Under lazy module loading that lookup is also the
 *     moment the 16 MiB are reserved on the device, and it can fail with
 *     FT_ERR_CUDA when no memory is left: make the first call at start-up, before
 *     the framework's allocator takes the device memory and before any stream
 *     capture (a call on a tiny shape will do).  The address is kept per device for
 *     the life of the process and does not survive cudaDeviceReset.
 *   - All calls on a device share the array, which keeps the previous call's
 *     contents: every used element is rewritten before it is read, but two calls
 *     whose kernels overlap on the GPU (different streams) race on it. */
#define FT_NOALLOC_MAX_SCRATCH_BYTES (16u << 20)
int ft_gemm_fp8_abft_expected_noalloc(const void* a_e4m3, const void* b_e4m3, int m, int n, int k, float* expected_rows,
                                      float* expected_cols, float* row_scales, float* col_scales, void* stream);

const char* ft_gemm_last_error(void);
int ft_gemm_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif
