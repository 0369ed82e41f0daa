// C-ABI of the fault-tolerant attention forward: see include/ft_attention.h.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <new>

#include "attention_kernels.h"
#include "kernels.h"

using namespace ftg;

namespace ftg {
int noalloc_fail(int code, const char* fmt, ...);  // sets the thread's last-error text (api.cu)
}

namespace {

#define ATTN_CUDA(call)                                                                                      \
  do {                                                                                                       \
    cudaError_t err_ = (call);                                                                               \
    if (err_ != cudaSuccess) return noalloc_fail(FT_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(err_)); \
  } while (0)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// [rows, cols] FP16, cols contiguous; box = 64 columns (128 bytes) x 128 rows, 128-byte swizzle.
int make_f16_map(CUtensorMap* map, const void* base, size_t rows, size_t cols, unsigned box_rows = 128u) {
  static EncodeTiledFn encode = nullptr;
  if (encode == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult query;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &query) != cudaSuccess ||
        query != cudaDriverEntryPointSuccess) {
      return noalloc_fail(FT_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    }
    encode = reinterpret_cast<EncodeTiledFn>(sym);
  }
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
  cuuint32_t box[2] = {64u, box_rows};
  cuuint32_t elem[2] = {1u, 1u};
  CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return noalloc_fail(FT_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
  return FT_OK;
}

}  // namespace

struct ft_attn_handle {
  int batch = 0, heads = 0, seq = 0, dim = 0;  // seq: rounded up to whole 128-row tiles
  int valid_seq = 0;                           // the caller's sequence length
  void* padded[3] = {nullptr, nullptr, nullptr};  // zero-padded copies of Q, K, V when valid_seq != seq
  ft_attn_options options{};
  const void *q = nullptr, *k = nullptr, *v = nullptr;
  void* vt = nullptr;
  float* cache = nullptr;  // one allocation: band sums, expected checksums, V sums
  size_t cache_bytes = 0;
  float *q_sums = nullptr, *q_mags = nullptr, *k_sums = nullptr, *k_mags = nullptr;
  float *expected_rows = nullptr, *expected_cols = nullptr, *row_scales = nullptr, *col_scales = nullptr;
  float *v_sum = nullptr, *v_weighted = nullptr;
  AttnDeviceReport* report = nullptr;
  CUtensorMap tmap_q{}, tmap_k{}, tmap_vt{};  // tmap_vt: boxes of D rows (whole-row kernel)
  CUtensorMap tmap_vt_ext{};                  // boxes of D + kAttnVExtra rows: V^T with its checksum rows (split-row kernel)
  // tensor-core prepare: FP16 pieces of the band sums (one allocation) and their maps
  void* planes = nullptr;
  void *q_ws = nullptr, *q_wm = nullptr, *k_ws = nullptr, *k_wm = nullptr;
  CUtensorMap tmap_q_ws{}, tmap_q_wm{}, tmap_k_ws{}, tmap_k_wm{};
  int* prepare_status = nullptr;
  int sm_count = 0;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  cudaStream_t last_stream = nullptr;
};

// The metadata of the current Q, K, V: V^T with its checksum rows, band sums of Q and K, the score-checksum cache
// (src/ft_flash_attention_a14.cu:571-621, 1294-1322 in this build's form).  Everything it writes was allocated by _prepare.
static int fill_attention_metadata(ft_attn_handle* h, cudaStream_t stream) {
  const void *q = h->q, *k = h->k, *v = h->v;
  const int seq = h->seq, head_dim = h->dim;
  const size_t bh = static_cast<size_t>(h->batch) * h->heads;
  const int nbands = seq / 64;
  const ft_attn_options& opts = h->options;
  cudaError_t err = cudaMemsetAsync(h->report, 0, sizeof(AttnDeviceReport), stream);
  if (err == cudaSuccess) err = cudaMemsetAsync(h->prepare_status, 0, sizeof(int), stream);
  if (err == cudaSuccess) err = cudaEventRecord(h->ev0, stream);
  if (err == cudaSuccess) err = launch_attn_prepare_v(v, h->vt, h->v_sum, h->v_weighted, static_cast<int>(bh), seq, head_dim, stream);
  if (err == cudaSuccess) err = launch_band_sums_f16(q, h->q_sums, h->q_mags, bh * seq, head_dim, stream);
  if (err == cudaSuccess) err = launch_band_sums_f16(k, h->k_sums, h->k_mags, bh * seq, head_dim, stream);
  // per head: S = Q K^T is the GEMM A = Q [N, D], B = K [N, D]
  if (opts.exact_prepare != 0) {
    if (err == cudaSuccess) {
      err = launch_expected_f16(q, h->k_sums, h->k_mags, h->expected_rows, h->row_scales, seq, seq / 64, head_dim, 0, static_cast<int>(bh), stream);
    }
    if (err == cudaSuccess) {
      err = launch_expected_f16(k, h->q_sums, h->q_mags, h->expected_cols, h->col_scales, seq, seq / 64, head_dim, 1, static_cast<int>(bh), stream);
    }
  } else {
    if (err == cudaSuccess) err = launch_split_band_pieces_f16(h->k_sums, h->k_mags, h->k_ws, h->k_wm, nbands, head_dim, static_cast<int>(bh), stream);
    if (err == cudaSuccess) err = launch_split_band_pieces_f16(h->q_sums, h->q_mags, h->q_ws, h->q_wm, nbands, head_dim, static_cast<int>(bh), stream);
    if (err == cudaSuccess) {
      err = launch_expected_mma_f16(h->tmap_q, h->tmap_k_ws, h->tmap_k_wm, h->expected_rows, h->row_scales, seq, nbands, head_dim, 0,
                                    static_cast<int>(bh), h->sm_count, h->prepare_status, stream);
    }
    if (err == cudaSuccess) {
      err = launch_expected_mma_f16(h->tmap_k, h->tmap_q_ws, h->tmap_q_wm, h->expected_cols, h->col_scales, seq, nbands, head_dim, 1,
                                    static_cast<int>(bh), h->sm_count, h->prepare_status, stream);
    }
  }
  if (err == cudaSuccess) err = cudaEventRecord(h->ev1, stream);
  if (err != cudaSuccess) return noalloc_fail(FT_ERR_CUDA, "attention prepare failed: %s", cudaGetErrorString(err));
  return FT_OK;
}

extern "C" {

void ft_attn_options_default(ft_attn_options* o) {
  if (o == nullptr) return;
  std::memset(o, 0, sizeof(*o));
  o->score_abs_tol = 1.0e-2f;
  o->score_rel_tol = 2.0e-5f;
  o->pv_abs_tol = 2.0e-3f;
  o->pv_rel_tol = 2.0e-3f;
  o->softmax_abs_tol = 2.0e-5f;
  o->softmax_rel_tol = 2.0e-5f;
  o->protect_softmax = 0;
  o->causal = 0;
  o->exact_prepare = 0;
}

int ft_attention_fp16_abft_destroy(ft_attn_handle* h) {
  if (h == nullptr) return FT_OK;
  cudaStreamSynchronize(h->last_stream);
  cudaFree(h->vt);
  for (void* buffer : h->padded) cudaFree(buffer);
  cudaFree(h->planes);
  cudaFree(h->prepare_status);
  cudaFree(h->cache);
  cudaFree(h->report);
  if (h->ev0) cudaEventDestroy(h->ev0);
  if (h->ev1) cudaEventDestroy(h->ev1);
  delete h;
  return FT_OK;
}

int ft_attention_fp16_abft_prepare(ft_attn_handle** handle, const void* q, const void* k, const void* v, int batch, int heads, int seq,
                                   int head_dim, const ft_attn_options* options, void* stream_ptr) {
  if (handle == nullptr || q == nullptr || k == nullptr || v == nullptr) return noalloc_fail(FT_ERR_INVALID, "null handle or operand pointer");
  *handle = nullptr;
  if (batch <= 0 || heads <= 0 || seq <= 0 || (head_dim != 128 && head_dim != 64)) {
    return noalloc_fail(FT_ERR_INVALID,
                        "Invalid options. Require head_dim 64 or 128 (src/ft_flash_attention_a14.cu:267) and positive batch, heads and "
                        "sequence (got B=%d H=%d N=%d D=%d).",
                        batch, heads, seq, head_dim);
  }
  // Any sequence length, as in the reference (a14:708, 893 mask by index): the kernels work on whole 128-row tiles, so for
  // other lengths the handle keeps zero-padded copies of Q, K and V; padded keys are masked, padded queries not stored.
  const int valid_seq = seq;
  seq = (seq + 127) / 128 * 128;
  if (((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15) != 0) {
    return noalloc_fail(FT_ERR_INVALID, "Q, K and V must be 16-byte aligned");
  }
  ft_attn_options opts;
  ft_attn_options_default(&opts);
  if (options != nullptr) opts = *options;
  if (opts.score_abs_tol < 0 || opts.score_rel_tol < 0 || opts.pv_abs_tol < 0 || opts.pv_rel_tol < 0) {
    return noalloc_fail(FT_ERR_INVALID, "negative tolerance");
  }
  int device = 0;
  ATTN_CUDA(cudaGetDevice(&device));
  cudaDeviceProp prop;
  ATTN_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10) return noalloc_fail(FT_ERR_UNSUPPORTED, "this library needs an sm_100 GPU (found sm_%d%d)", prop.major, prop.minor);
  ATTN_CUDA(configure_attention());
  ATTN_CUDA(configure_attention_split());
  if (opts.exact_prepare == 0) ATTN_CUDA(configure_prepare_mma());

  ft_attn_handle* h = new (std::nothrow) ft_attn_handle();
  if (h == nullptr) return noalloc_fail(FT_ERR_INVALID, "out of host memory");
  h->batch = batch;
  h->heads = heads;
  h->seq = seq;
  h->dim = head_dim;
  h->options = opts;
  h->valid_seq = valid_seq;
  if (valid_seq != seq) {
    const size_t pad_bytes = static_cast<size_t>(batch) * heads * seq * head_dim * 2;
    const size_t src_pitch = static_cast<size_t>(valid_seq) * head_dim * 2, dst_pitch = static_cast<size_t>(seq) * head_dim * 2;
    cudaStream_t copy_stream = static_cast<cudaStream_t>(stream_ptr);
    const void* sources[3] = {q, k, v};
    for (int i = 0; i < 3; ++i) {
      cudaError_t perr = cudaMalloc(&h->padded[i], pad_bytes);
      if (perr == cudaSuccess) perr = cudaMemsetAsync(h->padded[i], 0, pad_bytes, copy_stream);
      if (perr == cudaSuccess) {
        perr = cudaMemcpy2DAsync(h->padded[i], dst_pitch, sources[i], src_pitch, src_pitch, static_cast<size_t>(batch) * heads,
                                 cudaMemcpyDeviceToDevice, copy_stream);
      }
      if (perr != cudaSuccess) {
        ft_attention_fp16_abft_destroy(h);
        return noalloc_fail(FT_ERR_CUDA, "making the padded copies of Q, K, V failed: %s", cudaGetErrorString(perr));
      }
    }
    q = h->padded[0];
    k = h->padded[1];
    v = h->padded[2];
  }
  h->q = q;
  h->k = k;
  h->v = v;
  h->sm_count = prop.multiProcessorCount;
  const size_t bh = static_cast<size_t>(batch) * heads;
  const size_t bands = bh * (seq / 64);
  const size_t band_floats = bands * head_dim;
  const size_t checks = bh * (seq / 64) * (seq / 64) * 64;
  const size_t key_floats = bh * seq;
  const size_t floats = 4 * band_floats + 4 * checks + 2 * key_floats;
  h->cache_bytes = floats * sizeof(float);
  cudaError_t err = cudaMalloc(reinterpret_cast<void**>(&h->cache), h->cache_bytes);
  if (err == cudaSuccess) err = cudaMalloc(&h->vt, bh * seq * (head_dim + kAttnVExtra) * 2);
  if (err == cudaSuccess) err = cudaMalloc(reinterpret_cast<void**>(&h->report), sizeof(AttnDeviceReport));
  if (err == cudaSuccess) err = cudaMalloc(reinterpret_cast<void**>(&h->prepare_status), sizeof(int));
  const int nbands = seq / 64;
  const size_t ws_elems = bh * prepare_mma_plane_rows_f16(nbands, 0) * head_dim, wm_elems = bh * prepare_mma_plane_rows_f16(nbands, 1) * head_dim;
  if (err == cudaSuccess && opts.exact_prepare == 0) err = cudaMalloc(&h->planes, 2 * (ws_elems + wm_elems) * 2);
  if (err == cudaSuccess) err = cudaEventCreate(&h->ev0);
  if (err == cudaSuccess) err = cudaEventCreate(&h->ev1);
  if (err != cudaSuccess) {
    ft_attention_fp16_abft_destroy(h);
    return noalloc_fail(FT_ERR_CUDA, "allocating the attention cache (%zu bytes) failed: %s", floats * sizeof(float), cudaGetErrorString(err));
  }
  float* cursor = h->cache;
  h->q_sums = cursor, cursor += band_floats;
  h->q_mags = cursor, cursor += band_floats;
  h->k_sums = cursor, cursor += band_floats;
  h->k_mags = cursor, cursor += band_floats;
  h->expected_rows = cursor, cursor += checks;
  h->expected_cols = cursor, cursor += checks;
  h->row_scales = cursor, cursor += checks;
  h->col_scales = cursor, cursor += checks;
  h->v_sum = cursor, cursor += key_floats;
  h->v_weighted = cursor, cursor += key_floats;

  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  int rc = make_f16_map(&h->tmap_q, q, bh * seq, head_dim);
  if (rc == FT_OK) rc = make_f16_map(&h->tmap_k, k, bh * seq, head_dim);
  if (rc == FT_OK) rc = make_f16_map(&h->tmap_vt, h->vt, bh * (head_dim + kAttnVExtra), seq, static_cast<unsigned>(head_dim));
  if (rc == FT_OK) rc = make_f16_map(&h->tmap_vt_ext, h->vt, bh * (head_dim + kAttnVExtra), seq, static_cast<unsigned>(head_dim + kAttnVExtra));
  if (rc == FT_OK && opts.exact_prepare == 0) {
    __half* cursor16 = static_cast<__half*>(h->planes);
    h->q_ws = cursor16, cursor16 += ws_elems;
    h->q_wm = cursor16, cursor16 += wm_elems;
    h->k_ws = cursor16, cursor16 += ws_elems;
    h->k_wm = cursor16, cursor16 += wm_elems;
    const size_t ws_rows = bh * prepare_mma_plane_rows_f16(nbands, 0), wm_rows = bh * prepare_mma_plane_rows_f16(nbands, 1);
    rc = make_f16_map(&h->tmap_q_ws, h->q_ws, ws_rows, head_dim, 96u);
    if (rc == FT_OK) rc = make_f16_map(&h->tmap_q_wm, h->q_wm, wm_rows, head_dim, 64u);
    if (rc == FT_OK) rc = make_f16_map(&h->tmap_k_ws, h->k_ws, ws_rows, head_dim, 96u);
    if (rc == FT_OK) rc = make_f16_map(&h->tmap_k_wm, h->k_wm, wm_rows, head_dim, 64u);
  }
  if (rc == FT_OK) rc = fill_attention_metadata(h, stream);
  h->last_stream = stream;
  if (rc != FT_OK) {
    ft_attention_fp16_abft_destroy(h);
    return rc;
  }
  *handle = h;
  return FT_OK;
}

int ft_attention_fp16_abft_refresh(ft_attn_handle* h, const void* q, const void* k, const void* v, void* stream_ptr) {
  if (h == nullptr || q == nullptr || k == nullptr || v == nullptr) return noalloc_fail(FT_ERR_INVALID, "null handle or operand pointer");
  if (((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15) != 0) {
    return noalloc_fail(FT_ERR_INVALID, "Q, K and V must be 16-byte aligned");
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  const size_t bh = static_cast<size_t>(h->batch) * h->heads;
  if (h->valid_seq != h->seq) {
    // the padding rows of the handle's copies are zero since _prepare; only the real rows are replaced
    const size_t src_pitch = static_cast<size_t>(h->valid_seq) * h->dim * 2, dst_pitch = static_cast<size_t>(h->seq) * h->dim * 2;
    const void* sources[3] = {q, k, v};
    for (int i = 0; i < 3; ++i) {
      ATTN_CUDA(cudaMemcpy2DAsync(h->padded[i], dst_pitch, sources[i], src_pitch, src_pitch, bh, cudaMemcpyDeviceToDevice, stream));
    }
  } else {
    if (q != h->q) {
      const int rc = make_f16_map(&h->tmap_q, q, bh * h->seq, h->dim);
      if (rc != FT_OK) return rc;
    }
    if (k != h->k) {
      const int rc = make_f16_map(&h->tmap_k, k, bh * h->seq, h->dim);
      if (rc != FT_OK) return rc;
    }
    h->q = q;
    h->k = k;
    h->v = v;
  }
  h->last_stream = stream;
  return fill_attention_metadata(h, stream);
}

int ft_attention_generate_f16(void* out, size_t count, uint32_t seed, int dist, float sigma, void* stream_ptr) {
  if (out == nullptr && count > 0) return noalloc_fail(FT_ERR_INVALID, "null output pointer");
  if (dist != 0 && dist != 1) return noalloc_fail(FT_ERR_INVALID, "dist must be 0 (reference grid) or 1 (normal)");
  ATTN_CUDA(launch_generate_f16(out, count, seed, dist, sigma, static_cast<cudaStream_t>(stream_ptr)));
  return FT_OK;
}

int ft_attention_fp16_abft_run(ft_attn_handle* h, float* out, const ft_attn_fault* fault, void* stream_ptr) {
  if (h == nullptr || out == nullptr) return noalloc_fail(FT_ERR_INVALID, "null handle or output pointer");
  AttnParams params{};
  params.expected_rows = h->expected_rows;
  params.expected_cols = h->expected_cols;
  params.row_scales = h->row_scales;
  params.col_scales = h->col_scales;
  params.q = h->q;
  params.k = h->k;
  params.v_sum = h->v_sum;
  params.v_weighted = h->v_weighted;
  params.out = out;
  params.report = h->report;
  params.seq = h->seq;
  params.valid_seq = h->valid_seq;
  params.dim = h->dim;
  params.score_abs_tol = h->options.score_abs_tol;
  params.score_rel_tol = h->options.score_rel_tol;
  params.pv_abs_tol = h->options.pv_abs_tol;
  params.pv_rel_tol = h->options.pv_rel_tol;
  params.softmax_abs_tol = h->options.softmax_abs_tol;
  params.softmax_rel_tol = h->options.softmax_rel_tol;
  params.protect_softmax = h->options.protect_softmax;
  params.causal = h->options.causal != 0 ? 1 : 0;
  params.scale_log2 = 1.44269504088896340736f / std::sqrt(static_cast<float>(h->dim));
  params.fault_stage = FT_ATTN_FAULT_NONE;
  params.fault_bh = -1;
  if (fault != nullptr && fault->stage != FT_ATTN_FAULT_NONE) {
    const bool softmax_stage = fault->stage == FT_ATTN_FAULT_SOFTMAX || fault->stage == FT_ATTN_FAULT_SOFTMAX_STATE;
    if (fault->stage != FT_ATTN_FAULT_SCORE && fault->stage != FT_ATTN_FAULT_OUTPUT && !softmax_stage) {
      return noalloc_fail(FT_ERR_INVALID, "fault stage must be 1 (score), 2 (softmax), 3 (softmax-state) or 4 (output)");
    }
    if (softmax_stage && h->options.protect_softmax == 0) {
      return noalloc_fail(FT_ERR_INVALID, "the softmax stages can be targeted only by a handle prepared with protect_softmax");
    }
    int limit = fault->stage == FT_ATTN_FAULT_OUTPUT ? h->dim : h->valid_seq;
    if (fault->batch < 0 || fault->batch >= h->batch || fault->head < 0 || fault->head >= h->heads || fault->query < 0 ||
        fault->query >= h->valid_seq || fault->index < 0 || fault->index >= limit) {
      return noalloc_fail(FT_ERR_INVALID, "fault target is outside the tensor");
    }
    if (h->options.causal != 0 && fault->stage != FT_ATTN_FAULT_OUTPUT && fault->index > fault->query) {
      return noalloc_fail(FT_ERR_INVALID, "For causal attention, the fault key must not exceed the fault query.");
    }
    params.fault_stage = fault->stage;
    params.fault_bh = fault->batch * h->heads + fault->head;
    params.fault_query = fault->query;
    params.fault_index = fault->index;
    params.fault_value = fault->value;
    if (fault->stage == FT_ATTN_FAULT_SCORE && fault->value2 != 0.0f) {
      if (fault->query2 < 0 || fault->query2 >= h->valid_seq || fault->index2 < 0 || fault->index2 >= h->valid_seq ||
          (h->options.causal != 0 && fault->index2 > fault->query2)) {
        return noalloc_fail(FT_ERR_INVALID, "the second fault target is outside the tensor (or beyond the causal diagonal)");
      }
      params.fault2_query = fault->query2;
      params.fault2_index = fault->index2;
      params.fault2_value = fault->value2;
    }
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  ATTN_CUDA(cudaMemsetAsync(h->report, 0, 64, stream));  // the counters; the records are guarded by record_count
  // The split-row kernel (two threads per query row) is the default, with or without the softmax-stage protection; the
  // whole-row kernel (head dimension 128) can be selected for comparison with FT_ATTENTION_KERNEL=row in the environment.
  static const bool force_row = [] {
    const char* choice = std::getenv("FT_ATTENTION_KERNEL");
    return choice != nullptr && std::strcmp(choice, "row") == 0;
  }();
  if (force_row && h->dim == 128) {
    ATTN_CUDA(launch_attention(h->tmap_q, h->tmap_k, h->tmap_vt, params, h->batch * h->heads, stream));
  } else {
    ATTN_CUDA(launch_attention_split(h->tmap_q, h->tmap_k, h->tmap_vt_ext, params, h->batch * h->heads, stream));
  }
  h->last_stream = stream;
  return FT_OK;
}

int ft_attention_fp16_abft_report(ft_attn_handle* h, ft_attn_report* out) {
  if (h == nullptr || out == nullptr) return noalloc_fail(FT_ERR_INVALID, "null handle or report pointer");
  ATTN_CUDA(cudaStreamSynchronize(h->last_stream));
  AttnDeviceReport dev;
  ATTN_CUDA(cudaMemcpy(&dev, h->report, sizeof(dev), cudaMemcpyDeviceToHost));
  int prepare_status = 0;
  ATTN_CUDA(cudaMemcpy(&prepare_status, h->prepare_status, sizeof(int), cudaMemcpyDeviceToHost));
  if (prepare_status != 0) dev.status = prepare_status;  // a prepare kernel gave up: the cache is not valid
  std::memset(out, 0, sizeof(*out));
  out->status = dev.status != 0 ? FT_ERR_TIMEOUT : FT_OK;
  out->score_detected = dev.score_detected;
  out->score_corrected = dev.score_corrected;
  out->score_uncorrected = dev.score_uncorrected;
  out->pv_detected = dev.pv_detected;
  out->pv_corrected = dev.pv_corrected;
  out->failed_rows = dev.failed_rows;
  out->softmax_detected = dev.softmax_detected;
  out->softmax_corrected = dev.softmax_corrected;
  out->softmax_replayed = dev.softmax_replayed;
  out->score_replayed = dev.score_replayed;
  out->n_records = std::min(dev.record_count, 16);
  std::memcpy(&out->max_score_noise, &dev.max_noise_bits, sizeof(float));
  std::copy(dev.records, dev.records + out->n_records, out->records);
  std::sort(out->records, out->records + out->n_records, [](const ft_tile_record& a, const ft_tile_record& b) { return a.tile < b.tile; });
  float ms = 0.0f;
  if (cudaEventElapsedTime(&ms, h->ev0, h->ev1) == cudaSuccess) out->prepare_ms = ms;
  if (dev.status != 0) return noalloc_fail(FT_ERR_TIMEOUT, "a device-side wait expired; the output of this run is not valid");
  return FT_OK;
}

}  // extern "C"
