// Fault-tolerant flash-attention forward for sm_100a (FP16 in, FP32 softmax,
// accumulate and output).
//
// Replaces the reference's fused attention kernels (final form
// src/ft_flash_attention_a14.cu:659-1201) and its metadata kernels (a14:303-316,
// 571-621).  One CTA owns 256 queries of one (batch, head) as two 128-query tiles
// A and B that share every 128-key K / V^T tile:
//   warpgroup 0  warp 0: TMA producer of Q (once) and the K tiles, warp 2: of the V^T tiles; warp 1: one thread
//                issues tcgen05.mma kind::f16 -- S_A, S_B = Q_{A,B} K_j^T into two
//                128-column TMEM buffers, O_{A,B} += P_{A,B} V_j into two more;
//                the group gives most of its registers away (setmaxnreg);
//   warpgroups 1, 2  softmax / verifier of tile A and of tile B, one thread per
//                query row, running concurrently.  Pass 1 over S_j: the 64x64 ABFT
//                tile verifier of the GEMM epilogue (abft_tile_check.cuh) on both
//                64-column halves, corrected scores written back to TMEM, row
//                maximum.  Then the online-softmax rescale of O in TMEM.  Pass 2:
//                P = exp2(...) rounded to FP16 into shared memory in the MMA's
//                swizzled layout, while the expected output projections
//                sum_j p_j * vsum_j and sum_j p_j * vweighted_j are accumulated
//                (src/ft_flash_attention_a0.cu:585-611).  After the last tile the
//                output row is checked against those projections, a single faulty
//                element located and corrected (a0:613-662), normalised and stored.
// Every wait is bounded; on expiry the kernel reports status and leaves.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "abft_tile_check.cuh"
#include "attention_device.cuh"
#include "attention_kernels.h"
#include "sm100_ptx.cuh"

namespace ftg {

constexpr int kAttnTile = 128;             // queries per tile, keys per tile, head dimension
constexpr int kAttnQTiles = 2;             // query tiles per CTA
constexpr int kAttnSlabBytes = 128 * 128;  // 128 rows x 64 FP16 (one 128-byte swizzle row each)
constexpr int kAttnTileBytes = 2 * kAttnSlabBytes;
constexpr int kAttnThreads = 384;
constexpr uint64_t kAttnTimeoutNs = 2000000000ull;
constexpr uint32_t kTmemS = 0;    // score buffers of tile A, B at columns 0, 128
constexpr uint32_t kTmemO = 256;  // output accumulators of tile A, B at columns 256, 384

struct AttnShared {
  uint64_t q_full, k_full, k_empty, v_full, v_empty;
  uint64_t s_full[kAttnQTiles], s_empty[kAttnQTiles];
  uint64_t p_full[kAttnQTiles], p_empty[kAttnQTiles];
  uint32_t tmem_base;
  int abort_flag;
  float2 v_meta[kAttnQTiles][2][kAttnTile];  // [query tile][parity][key]: {sum_d V, sum_d w_d V}
  TileScratch scratch[kAttnQTiles][2][2];    // [query tile][row pair][parity]
  TileScratch replay_scratch[kAttnQTiles][2];  // [query tile][row pair]: second check of a replayed score tile
};

// Q (2 tiles), K, V^T, P (2 tiles)
constexpr int kAttnSmemBytes = 6 * kAttnTileBytes + static_cast<int>(sizeof(AttnShared)) + 1024;

// ---------------------------------------------------------------------------
// V metadata and transpose (src/ft_flash_attention_a14.cu:303-316, 600-620):
// v_sum[key] = sum_d V[key,d] (ascending d), v_weighted[key] = sum_d (2d-(D-1)) V[key,d]
// (one fma per step), V^T[d][key] so that the keys are contiguous for the PV MMA.
// grid (N/64, B*H), 256 threads: 64 keys per CTA, read as 16-byte pieces, written back as 128-byte runs of keys.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) attn_prepare_v_kernel(const __half* __restrict__ v, __half* __restrict__ vt,
                                                             float* __restrict__ v_sum, float* __restrict__ v_weighted, int seq,
                                                             int dim) {
  __shared__ __half tile[64][kAttnTile + 2];  // dim <= 128; the odd word stride keeps column reads free of bank conflicts
  const int bh = blockIdx.y;
  const int key0 = blockIdx.x * 64;
  const uint4* src = reinterpret_cast<const uint4*>(v + (static_cast<size_t>(bh) * seq + key0) * dim);  // 16-byte aligned: dim % 8 == 0
  for (int i = threadIdx.x; i < 64 * dim / 8; i += 256) {
    const uint4 piece = __ldg(src + i);
    const int key = (i * 8) / dim, d = (i * 8) % dim;
    uint32_t* dst = reinterpret_cast<uint32_t*>(&tile[key][d]);  // rows start on 4-byte boundaries
    dst[0] = piece.x;
    dst[1] = piece.y;
    dst[2] = piece.z;
    dst[3] = piece.w;
  }
  __syncthreads();
  if (threadIdx.x < 64) {
    float sum = 0.0f, weighted = 0.0f;
    for (int d = 0; d < dim; ++d) {
      float value = __half2float(tile[threadIdx.x][d]);
      sum += value;
      weighted = __fmaf_rn(static_cast<float>(2 * d - (dim - 1)), value, weighted);
    }
    v_sum[static_cast<size_t>(bh) * seq + key0 + threadIdx.x] = sum;
    v_weighted[static_cast<size_t>(bh) * seq + key0 + threadIdx.x] = weighted;
    // The checksum rows below the head's D rows of V^T (see kAttnVExtra): ones, then hi and lo FP16 pieces of the two
    // sums, so that the PV product accumulates l and both expected projections.  hi + lo carries 22 bits of the FP32
    // value; values beyond the FP16 range saturate (the check then reports the rows instead of passing them).
    __half* extra = vt + (static_cast<size_t>(bh) * (dim + kAttnVExtra) + dim) * seq + key0 + threadIdx.x;
    const float scaled = weighted * (1.0f / kAttnVWeightScale);
    const float clamp = 65504.0f;
    const __half sum_hi = __float2half_rn(fminf(fmaxf(sum, -clamp), clamp));
    const __half sum_lo = __float2half_rn(sum - __half2float(sum_hi));
    const __half weighted_hi = __float2half_rn(fminf(fmaxf(scaled, -clamp), clamp));
    const __half weighted_lo = __float2half_rn(scaled - __half2float(weighted_hi));
    extra[0] = __float2half_rn(1.0f);
    extra[static_cast<size_t>(1) * seq] = sum_hi;
    extra[static_cast<size_t>(2) * seq] = sum_lo;
    extra[static_cast<size_t>(3) * seq] = weighted_hi;
    extra[static_cast<size_t>(4) * seq] = weighted_lo;
    for (int e = 5; e < kAttnVExtra; ++e) extra[static_cast<size_t>(e) * seq] = __float2half_rn(0.0f);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int d = warp; d < dim; d += 8) {
    const __half2 pair = __halves2half2(tile[2 * lane][d], tile[2 * lane + 1][d]);
    *reinterpret_cast<__half2*>(vt + (static_cast<size_t>(bh) * (dim + kAttnVExtra) + d) * seq + key0 + 2 * lane) = pair;
  }
}

cudaError_t launch_attn_prepare_v(const void* v, void* vt, float* v_sum, float* v_weighted, int batch_heads, int seq, int dim,
                                  cudaStream_t stream) {
  dim3 grid(seq / 64, batch_heads);
  attn_prepare_v_kernel<<<grid, 256, 0, stream>>>(static_cast<const __half*>(v), static_cast<__half*>(vt), v_sum, v_weighted, seq, dim);
  return cudaGetLastError();
}

// Seeded FP16 inputs.  dist 0: the reference attention generator's grid
// ((mix(seed+i) % 17) - 8) / 16 (src/ft_flash_attention_a0.cu:231-238; exactly
// representable in FP16 as it is in E4M3).  dist 1: N(0, sigma^2) by Box-Muller
// over two hash draws, rounded to FP16.
__device__ __forceinline__ uint32_t attn_mix_u32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7feb352dU;
  x ^= x >> 15;
  x *= 0x846ca68bU;
  x ^= x >> 16;
  return x;
}

__global__ void generate_f16_kernel(__half* out, size_t count, uint32_t seed, int dist, float sigma) {
  size_t index = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (; index < count; index += stride) {
    float value;
    if (dist == 0) {
      int quantized = static_cast<int>(attn_mix_u32(seed + static_cast<uint32_t>(index)) % 17u) - 8;
      value = static_cast<float>(quantized) * 0.0625f;
    } else {
      uint32_t i2 = 2u * static_cast<uint32_t>(index);
      uint32_t h1 = attn_mix_u32(seed ^ i2);
      uint32_t h2 = attn_mix_u32(seed ^ (i2 + 1u));
      float u1 = (static_cast<float>(h1 & 0x00ffffffU) + 1.0f) / 16777216.0f;
      float u2 = static_cast<float>(h2 & 0x00ffffffU) / 16777216.0f;
      value = sqrtf(-2.0f * logf(u1)) * cosf(6.28318530717958647692f * u2) * sigma;
    }
    out[index] = __float2half_rn(value);
  }
}

cudaError_t launch_generate_f16(void* out, size_t count, uint32_t seed, int dist, float sigma, cudaStream_t stream) {
  if (count == 0) return cudaSuccess;
  size_t blocks = (count + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  generate_f16_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(static_cast<__half*>(out), count, seed, dist, sigma);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// forward kernel helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// OR of `flag` over the 128 threads of one softmax warpgroup (named barrier `id`).
__device__ __forceinline__ bool attn_any(bool flag, int id) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %1, 0;\n\t"
      "barrier.cta.red.or.pred q, %2, 128, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(out)
      : "r"(static_cast<uint32_t>(flag)), "r"(id)
      : "memory");
  return out != 0;
}

// One thread of the warpgroup polls; the others sleep in the hardware barrier.
// Returns false (for all 128) when the wait was abandoned.
__device__ __forceinline__ bool attn_wait_all(uint64_t* bar, uint32_t parity, volatile int* abort_flag, bool poller, int id) {
  bool ok = true;
  if (poller) ok = mbar_wait_bounded(bar, parity, abort_flag, kAttnTimeoutNs);
  return !attn_any(!ok, id);
}

// Adds `value` to one element of a TMEM column in place; executed by the whole
// warp that owns the row's lane quarter.
__device__ __forceinline__ void tmem_add_to_element(uint32_t taddr_column, int lane, int target_lane, float value) {
  float x;
  tmem_ld_32x32b_x1(taddr_column, x);
  tmem_wait_ld();
  if (lane == target_lane) x += value;
  tmem_st_32x32b_x1(taddr_column, x);
  tmem_wait_st();
}

// Hides a value from the optimiser so that a verifier copy is really recomputed.
__device__ __forceinline__ float opaque(float x) {
  asm volatile("" : "+f"(x));
  return x;
}

template <int Regs>
__device__ __forceinline__ void reg_release() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(Regs));
}
template <int Regs>
__device__ __forceinline__ void reg_acquire() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(Regs));
}

// kProtect adds the reference's softmax-stage protection (verifier copies, moment check, state duplicate).
template <bool kProtect>
__global__ void __launch_bounds__(kAttnThreads, 1)
ft_attention_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                        const __grid_constant__ CUtensorMap tmap_vt, const __grid_constant__ AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  // aligned to 1024 bytes by pointer arithmetic on the shared array itself, so that the compiler keeps every access below
  // in the shared address space (32-bit addresses, LDS / STS) instead of falling back to generic 64-bit addressing
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* smem_q = smem;                       // 2 query tiles
  uint8_t* smem_k = smem + 2 * kAttnTileBytes;  // 1 stage
  uint8_t* smem_v = smem + 3 * kAttnTileBytes;  // 1 stage
  uint8_t* smem_p = smem + 4 * kAttnTileBytes;  // 2 query tiles
  AttnShared& sh = *reinterpret_cast<AttnShared*>(smem + 6 * kAttnTileBytes);
  volatile int* abort_flag = &sh.abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int group = warp >> 2;  // 0: producer + MMA, 1 and 2: softmax of query tile A and B
  const int bh = blockIdx.y;
  // causal CTAs get longer towards the end of the sequence: the longest are scheduled first
  const int q_block = p.causal != 0 ? static_cast<int>(gridDim.x - 1 - blockIdx.x) : static_cast<int>(blockIdx.x);
  const int q0 = q_block * kAttnQTiles * kAttnTile;
  const int seq = p.seq;
  const int num_tiles = seq / kAttnTile;
  const int row_base = bh * seq;  // first row of this head in the [B*H*N, D] matrices
  const int qtiles = q0 + kAttnQTiles * kAttnTile <= seq ? kAttnQTiles : 1;  // the last CTA of a head may own one tile
  // Causal attention (src/ft_flash_attention_a14.cu:708): query tile t stops after the key tile on its diagonal, so tile B
  // of a CTA runs one key tile longer than tile A; inside the diagonal tile keys beyond the query are masked.
  const bool causal = p.causal != 0;
  const int first_qtile = q0 / kAttnTile;
  auto tiles_of = [&](int t) { return causal ? min(num_tiles, first_qtile + t + 1) : num_tiles; };
  const int cta_tiles = tiles_of(qtiles - 1);

  if (threadIdx.x == 0) {
    mbar_init(&sh.q_full, 1);
    mbar_init(&sh.k_full, 1);
    mbar_init(&sh.k_empty, 1);
    mbar_init(&sh.v_full, 1);
    mbar_init(&sh.v_empty, 1);
    for (int t = 0; t < kAttnQTiles; ++t) {
      mbar_init(&sh.s_full[t], 1);
      mbar_init(&sh.s_empty[t], 128);
      mbar_init(&sh.p_full[t], 128);
      mbar_init(&sh.p_empty[t], 1);
    }
    sh.abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmap_q);
    prefetch_tensormap(&tmap_k);
    prefetch_tensormap(&tmap_vt);
  }
  if (warp == 1) {
    tmem_alloc(&sh.tmem_base, 512);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = sh.tmem_base;

  if (group == 0) {
    reg_release<40>();
    if (warp == 0 && elect_one()) {
      // ------------------------------------------------------------- producer
      mbar_arrive_expect_tx(&sh.q_full, qtiles * kAttnTileBytes);
      for (int t = 0; t < qtiles; ++t) {
        tma_load_2d(smem_q + t * kAttnTileBytes, &tmap_q, &sh.q_full, 0, row_base + q0 + t * kAttnTile);
        tma_load_2d(smem_q + t * kAttnTileBytes + kAttnSlabBytes, &tmap_q, &sh.q_full, 64, row_base + q0 + t * kAttnTile);
      }
      for (int j = 0; j < cta_tiles; ++j) {
        const uint32_t ph = j & 1;
        if (!mbar_wait_bounded(&sh.k_empty, ph ^ 1, abort_flag, kAttnTimeoutNs)) break;
        mbar_arrive_expect_tx(&sh.k_full, kAttnTileBytes);
        tma_load_2d(smem_k, &tmap_k, &sh.k_full, 0, row_base + j * kAttnTile);
        tma_load_2d(smem_k + kAttnSlabBytes, &tmap_k, &sh.k_full, 64, row_base + j * kAttnTile);
      }
    } else if (warp == 2 && elect_one()) {
      // ------------------------------------------------------------- producer of V^T: its own thread, so that the load of
      // K_{j+1} (free as soon as both score products of tile j are done) never queues behind the wait for the V buffer
      for (int j = 0; j < cta_tiles; ++j) {
        const uint32_t ph = j & 1;
        if (!mbar_wait_bounded(&sh.v_empty, ph ^ 1, abort_flag, kAttnTimeoutNs)) break;
        mbar_arrive_expect_tx(&sh.v_full, kAttnTileBytes);
        tma_load_2d(smem_v, &tmap_vt, &sh.v_full, j * kAttnTile, bh * (kAttnTile + kAttnVExtra));  // the D rows of the head; its checksum rows are skipped
        tma_load_2d(smem_v + kAttnSlabBytes, &tmap_vt, &sh.v_full, j * kAttnTile + 64, bh * (kAttnTile + kAttnVExtra));
      }
    } else if (warp == 1 && elect_one()) {
      // ------------------------------------------------------------- MMA issuer
      constexpr uint32_t idesc = make_idesc_f16_f32(kAttnTile, kAttnTile);
      bool alive = mbar_wait_bounded(&sh.q_full, 0, abort_flag, kAttnTimeoutNs);
      for (int j = 0; j <= cta_tiles && alive; ++j) {
        if (j < cta_tiles) {  // S_A, S_B = Q_{A,B} K_j^T
          if (!mbar_wait_bounded(&sh.k_full, j & 1, abort_flag, kAttnTimeoutNs)) break;
          for (int t = 0; t < qtiles && alive; ++t) {
            if (j >= tiles_of(t)) continue;
            // the score buffer of tile t is free once its softmax group has read S_{j-1} twice
            if (!mbar_wait_bounded(&sh.s_empty[t], (j & 1) ^ 1, abort_flag, kAttnTimeoutNs)) {
              alive = false;
              break;
            }
            tcgen05_fence_after();
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
              uint64_t da = make_smem_desc_sw128(smem_u32(smem_q + t * kAttnTileBytes + (kk >> 2) * kAttnSlabBytes)) + 2 * (kk & 3);
              uint64_t db = make_smem_desc_sw128(smem_u32(smem_k + (kk >> 2) * kAttnSlabBytes)) + 2 * (kk & 3);
              umma_f16(tmem_base + kTmemS + t * kAttnTile, da, db, idesc, kk != 0 ? 1u : 0u);
            }
            umma_commit(&sh.s_full[t]);
          }
          if (!alive) break;
          umma_commit(&sh.k_empty);
        }
        if (j > 0) {  // O_{A,B} += P_i V_i for the previous key tile
          const int i = j - 1;
          if (!mbar_wait_bounded(&sh.v_full, i & 1, abort_flag, kAttnTimeoutNs)) break;
          for (int t = 0; t < qtiles && alive; ++t) {
            if (i >= tiles_of(t)) continue;
            if (!mbar_wait_bounded(&sh.p_full[t], i & 1, abort_flag, kAttnTimeoutNs)) {
              alive = false;
              break;
            }
            tcgen05_fence_after();
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
              uint64_t da = make_smem_desc_sw128(smem_u32(smem_p + t * kAttnTileBytes + (kk >> 2) * kAttnSlabBytes)) + 2 * (kk & 3);
              uint64_t db = make_smem_desc_sw128(smem_u32(smem_v + (kk >> 2) * kAttnSlabBytes)) + 2 * (kk & 3);
              umma_f16(tmem_base + kTmemO + t * kAttnTile, da, db, idesc, (i | kk) != 0 ? 1u : 0u);
            }
            umma_commit(&sh.p_empty[t]);
          }
          if (!alive) break;
          umma_commit(&sh.v_empty);
        }
      }
    }
  } else {
    reg_acquire<224>();
    // ------------------------------------------------------------- softmax / verifier: one thread per query row
    const int t = group - 1;  // query tile of this warpgroup
    if (t < qtiles) {
      const int quarter = warp & 3;
      const int pair = quarter >> 1;
      const int half = quarter & 1;
      const int r_local = half * 32 + lane;
      const int row_in_tile = quarter * 32 + lane;
      const int tg = threadIdx.x & 127;
      const bool poller = tg == 0;
      const int bar_all = 3 + 3 * t;          // 128-thread barrier of this warpgroup
      const int bar_pair = 1 + 3 * t + pair;  // 64-thread barrier of this 64-row band
      const int tile_cols = seq / 64;
      const size_t head_cache = static_cast<size_t>(bh) * tile_cols * tile_cols * 64;
      const int q_tile0 = q0 + t * kAttnTile;
      const int q_band = q_tile0 / 64 + pair;
      const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
      const uint32_t s_addr = lane_addr + kTmemS + t * kAttnTile;
      const uint32_t o_addr = lane_addr + kTmemO + t * kAttnTile;
      uint8_t* p_tile = smem_p + t * kAttnTileBytes;
      const bool fault_here = p.fault_bh == bh && p.fault_query >= q_tile0 && p.fault_query < q_tile0 + kAttnTile;
      const bool score_fault = fault_here && p.fault_stage == FT_ATTN_FAULT_SCORE;
      const bool score_fault2 = p.fault_bh == bh && p.fault_stage == FT_ATTN_FAULT_SCORE && p.fault2_value != 0.0f &&
                                p.fault2_query >= q_tile0 && p.fault2_query < q_tile0 + kAttnTile;
      const bool output_fault = fault_here && p.fault_stage == FT_ATTN_FAULT_OUTPUT;
      const int fault_row = p.fault_query - q_tile0;  // row in this tile, when fault_here

      float m_run = -INFINITY, l_run = 0.0f, exp_sum = 0.0f, exp_weighted = 0.0f, max_ratio = 0.0f;
      float u1_run = 0.0f, u2_run = 0.0f;                                             // running moments (kProtect)
      float m_verify = -INFINITY, l_verify = 0.0f, u1_verify = 0.0f, u2_verify = 0.0f;  // verifier copy of the state
      bool alive = true;

      const int my_tiles = tiles_of(t);
      for (int j = 0; j < my_tiles; ++j) {
        const int buf = j & 1;
        // Keys of this tile the row may attend to are those with local index <= key_limit: all 128, up to the query in
        // the causal diagonal tile (src/ft_flash_attention_a14.cu:893), up to the last real key in the last tile of a
        // sequence that was padded to whole tiles.
        int key_limit = kAttnTile - 1;
        if (causal && j == first_qtile + t) key_limit = row_in_tile;
        if ((j + 1) * kAttnTile > p.valid_seq) key_limit = min(key_limit, p.valid_seq - 1 - j * kAttnTile);
        const bool diagonal = key_limit < kAttnTile - 1;  // some keys of this tile are masked for this row
        // per-key sums of V for this tile (read in pass 2; published by the barrier inside the wait below)
        sh.v_meta[t][buf][tg] = make_float2(__ldg(p.v_sum + static_cast<size_t>(bh) * seq + j * kAttnTile + tg),
                                            __ldg(p.v_weighted + static_cast<size_t>(bh) * seq + j * kAttnTile + tg));
        // cached expected checksums of the four 64x64 tiles this thread takes part in: fetched before the wait
        float exp_row[2], scale_row[2], exp_col0[2], exp_col1[2], scale_col0[2], scale_col1[2];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const size_t cache = head_cache + (static_cast<size_t>(q_band) * tile_cols + j * 2 + c) * 64;
          exp_row[c] = __ldg(p.expected_rows + cache + r_local);
          scale_row[c] = __ldg(p.row_scales + cache + r_local);
          exp_col0[c] = __ldg(p.expected_cols + cache + lane);
          exp_col1[c] = __ldg(p.expected_cols + cache + 32 + lane);
          scale_col0[c] = __ldg(p.col_scales + cache + lane);
          scale_col1[c] = __ldg(p.col_scales + cache + 32 + lane);
        }
        if (!attn_wait_all(&sh.s_full[t], j & 1, abort_flag, poller, bar_all)) {
          alive = false;
          break;
        }
        tcgen05_fence_after();

        // test hook: the fault enters the accumulator itself, before any checksum
        if (score_fault && p.fault_index / kAttnTile == j && fault_row / 32 == quarter) {
          tmem_add_to_element(s_addr + p.fault_index % kAttnTile, lane, fault_row % 32, p.fault_value);
        }
        if (score_fault2 && p.fault2_index / kAttnTile == j && (p.fault2_query - q_tile0) / 32 == quarter) {
          tmem_add_to_element(s_addr + p.fault2_index % kAttnTile, lane, (p.fault2_query - q_tile0) % 32, p.fault2_value);
        }

        // ---- pass 1: verify both 64x64 score tiles of this thread's band, track the row maximum.  Both halves are
        // loaded at once; row sums, column partials and the maximum of both are done before the one barrier with the
        // partner warp, the two decisions after it.
        float row_max = -INFINITY;
        if (!kProtect) {
          float v0[64], v1[64];
          tmem_ld_32x32b_x32(s_addr, v0);
          tmem_ld_32x32b_x32(s_addr + 32, v0 + 32);
          tmem_ld_32x32b_x32(s_addr + 64, v1);
          tmem_ld_32x32b_x32(s_addr + 96, v1 + 32);
          tmem_wait_ld();
          abft_tile_sums(v0, lane, half, sh.scratch[t][pair][0], exp_row[0], scale_row[0], p.score_abs_tol, p.score_rel_tol, max_ratio);
          abft_tile_sums(v1, lane, half, sh.scratch[t][pair][1], exp_row[1], scale_row[1], p.score_abs_tol, p.score_rel_tol, max_ratio);
          if (diagonal) {  // the verifier has seen the raw tile; the maximum only sees keys up to the query
#pragma unroll
            for (int i = 0; i < 64; ++i) {
              if (i > key_limit) v0[i] = -INFINITY;
              if (64 + i > key_limit) v1[i] = -INFINITY;
            }
          }
#pragma unroll
          for (int i = 0; i < 64; ++i) row_max = max3_f32(row_max, v0[i], v1[i]);
          asm volatile("bar.sync %0, 64;" ::"r"(bar_pair) : "memory");
        }
        bool reload_row = false;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          if (kProtect) {  // this variant keeps fewer registers live: one half at a time, one barrier each
            float v[64];
            tmem_ld_32x32b_x32(s_addr + c * 64, v);
            tmem_ld_32x32b_x32(s_addr + c * 64 + 32, v + 32);
            tmem_wait_ld();
            abft_tile_sums(v, lane, half, sh.scratch[t][pair][c], exp_row[c], scale_row[c], p.score_abs_tol, p.score_rel_tol, max_ratio);
            if (diagonal) {
#pragma unroll
              for (int i = 0; i < 64; ++i) {
                if (c * 64 + i > key_limit) v[i] = -INFINITY;
              }
            }
#pragma unroll
            for (int i = 0; i < 64; i += 2) row_max = max3_f32(row_max, v[i], v[i + 1]);
            asm volatile("bar.sync %0, 64;" ::"r"(bar_pair) : "memory");
          }
          const TileDecision d = abft_tile_decide(lane, sh.scratch[t][pair][c], exp_col0[c], exp_col1[c], scale_col0[c], scale_col1[c],
                                                  p.score_abs_tol, p.score_rel_tol, max_ratio);
          if ((d.bad_rows | d.bad_cols) != 0) {  // uniform over the two warps of the band
            bool replayed = false;
            if (d.corrected && d.bad_row / 32 == half) {
              // src/s4:493-497 on the accumulator itself: pass 2 reads the corrected score back
              tmem_add_to_element(s_addr + c * 64 + d.bad_col, lane, d.bad_row % 32, 0.5f * (d.row_delta + d.col_delta));
              reload_row = true;
            }
            if (!d.corrected) {
              // The fault cannot be located: the band's 64 x 64 scores are recomputed without the tensor core
              // (src/ft_flash_attention_a14.cu:935-959), checked again and put back into the accumulator for pass 2.
              // Waits of this kernel are abandoned by whole warpgroups, so the two warps of the band can meet at their
              // named barrier here as well.
              float rv[64];
              const __half* q_row = static_cast<const __half*>(p.q) + (static_cast<size_t>(row_base) + q_tile0 + row_in_tile) * kAttnTile;
              const __half* k_tile = static_cast<const __half*>(p.k) + (static_cast<size_t>(row_base) + j * kAttnTile + c * 64) * kAttnTile;
              replay_score_row<kAttnTile>(q_row, k_tile, rv);
              TileScratch& again = sh.replay_scratch[t][pair];
              float ignored = 0.0f;
              abft_tile_sums(rv, lane, half, again, exp_row[c], scale_row[c], p.score_abs_tol, p.score_rel_tol, ignored);
              asm volatile("bar.sync %0, 64;" ::"r"(bar_pair) : "memory");
              const TileDecision d2 = abft_tile_decide(lane, again, exp_col0[c], exp_col1[c], scale_col0[c], scale_col1[c], p.score_abs_tol,
                                                       p.score_rel_tol, ignored);
              replayed = (d2.bad_rows | d2.bad_cols) == 0;
              asm volatile("bar.sync %0, 64;" ::"r"(bar_pair) : "memory");  // `again` may be written again for the other half
              tmem_st_32x32b_x32(s_addr + c * 64, rv);
              tmem_st_32x32b_x32(s_addr + c * 64 + 32, rv + 32);
              tmem_wait_st();
              reload_row = true;
            }
            if (half == 0 && lane == 0) {
              atomicAdd(&p.report->score_detected, 1);
              atomicAdd(d.corrected ? &p.report->score_corrected : (replayed ? &p.report->score_replayed : &p.report->score_uncorrected), 1);
              int slot = atomicAdd(&p.report->record_count, 1);
              if (slot < 16) {
                ft_tile_record rec;
                rec.tile = (bh * tile_cols + q_band) * tile_cols + j * 2 + c;
                rec.bad_row_count = d.bad_rows;
                rec.bad_col_count = d.bad_cols;
                rec.bad_row = d.bad_row;
                rec.bad_col = d.bad_col;
                rec.row_delta = d.row_delta;
                rec.col_delta = d.col_delta;
                rec.corrected = d.corrected ? 1 : 0;
                p.report->records[slot] = rec;
              }
            }
          }
        }
        if (reload_row) {  // warp-uniform and rare: the maximum of the corrected row is taken from the corrected scores
          row_max = -INFINITY;
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            float v[32];
            tmem_ld_32x32b_x32(s_addr + c * 32, v);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              if (!diagonal || c * 32 + i <= key_limit) row_max = fmaxf(row_max, v[i]);
            }
          }
        }

        // ---- online softmax state (log2 domain)
        const float m_new = fmaxf(m_run, row_max * p.scale_log2);
        const float alpha = fast_exp2(m_run - m_new);  // 0 for the first tile (m_run = -inf)

        if (j > 0) {
          // PV of the previous tile must have finished: the P buffer is free and O is quiescent
          if (!attn_wait_all(&sh.p_empty[t], (j - 1) & 1, abort_flag, poller, bar_all)) {
            alive = false;
            break;
          }
          tcgen05_fence_after();
          if (__any_sync(0xffffffffU, alpha != 1.0f)) {
#pragma unroll 1
            for (int cc = 0; cc < 4; ++cc) {
              float o[32];
              tmem_ld_32x32b_x32(o_addr + cc * 32, o);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] *= alpha;
              tmem_st_32x32b_x32(o_addr + cc * 32, o);
            }
            tmem_wait_st();
          }
        }
        // ---- pass 2: probabilities, FP16 P tile for the MMA, expected output projections
        // With kProtect the reference's softmax-stage protection runs alongside (src/ft_flash_attention_a14.cu:
        // 964-1099): a verifier copy of the maximum, of every probability and of the moments sum p, sum w p,
        // sum w^2 p (w = 2*key - (N-1)) of the FP16-rounded probabilities; on a mismatch one probability is
        // located by the ratio of the moment deltas and replaced by the verifier's, otherwise the whole row of
        // the tile is replayed from the verifier; a duplicate of the running state (m, l, u1, u2) follows.
        float l_tile = 0.0f, es_tile = 0.0f, ew_tile = 0.0f, u1_tile = 0.0f, u2_tile = 0.0f;
        float check_u0 = 0.0f, check_u1 = 0.0f, check_u2 = 0.0f;
        float m_check = m_new, alpha_check = alpha;
        if (kProtect) {
          // verifier maximum: recomputed from its own copy of the running maximum
          float verifier_max = opaque(row_max);
          if (fabsf(row_max - verifier_max) > p.softmax_abs_tol) {
            atomicAdd(&p.report->softmax_detected, 1);
            atomicAdd(&p.report->softmax_replayed, 1);
          }
          m_check = fmaxf(m_verify, verifier_max * p.scale_log2);
          alpha_check = fast_exp2(opaque(m_verify - m_check));
        }
        const bool softmax_fault = kProtect && fault_here && p.fault_stage == FT_ATTN_FAULT_SOFTMAX && fault_row == row_in_tile &&
                                   p.fault_index / kAttnTile == j;
        int recovery_action = 0, recovery_key = -1;  // 1: take the verifier's value at recovery_key, 2: replay the row
#pragma unroll 1
        for (int attempt = 0; attempt < (kProtect ? 2 : 1); ++attempt) {
          l_tile = es_tile = ew_tile = u1_tile = u2_tile = 0.0f;
          check_u0 = check_u1 = check_u2 = 0.0f;
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {
            float v[64];
            tmem_ld_32x32b_x32(s_addr + c * 64, v);
            tmem_ld_32x32b_x32(s_addr + c * 64 + 32, v + 32);
            tmem_wait_ld();
            if (diagonal) {  // exp2(-inf) = 0: a masked key gets probability zero in every copy below
#pragma unroll
              for (int i = 0; i < 64; ++i) {
                if (c * 64 + i > key_limit) v[i] = -INFINITY;
              }
            }
            if (!kProtect && c == 1) {  // both halves are in registers: the score buffer can take S of the next key tile
              tcgen05_fence_before();
              mbar_arrive(&sh.s_empty[t]);
            }
            uint8_t* p_row = p_tile + c * kAttnSlabBytes + (row_in_tile >> 3) * 1024 + (row_in_tile & 7) * 128;
            const int key0 = c * 64;  // key of v[0] within the tile
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) {
              uint32_t packed[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int i0 = ch * 8 + 2 * e;
                float p0 = fast_exp2(__fmaf_rn(v[i0], p.scale_log2, -m_new));
                float p1 = fast_exp2(__fmaf_rn(v[i0 + 1], p.scale_log2, -m_new));
                __half2 h;
                if (kProtect) {
                  if (softmax_fault && p.fault_index % kAttnTile == key0 + i0) p0 += p.fault_value;
                  if (softmax_fault && p.fault_index % kAttnTile == key0 + i0 + 1) p1 += p.fault_value;
                  const float q0 = fast_exp2(opaque(__fmaf_rn(v[i0], p.scale_log2, -m_check)));
                  const float q1 = fast_exp2(opaque(__fmaf_rn(v[i0 + 1], p.scale_log2, -m_check)));
                  const __half2 hv = __floats2half2_rn(q0, q1);
                  const float2 rv = __half22float2(hv);
                  const float w0 = static_cast<float>(2 * (j * kAttnTile + key0 + i0) - (seq - 1));
                  const float w1 = w0 + 2.0f;
                  check_u0 += rv.x;
                  check_u0 += rv.y;
                  check_u1 = __fmaf_rn(w0, rv.x, check_u1);
                  check_u1 = __fmaf_rn(w1, rv.y, check_u1);
                  check_u2 = __fmaf_rn(w0, w0 * rv.x, check_u2);
                  check_u2 = __fmaf_rn(w1, w1 * rv.y, check_u2);
                  h = __floats2half2_rn(p0, p1);
                  if (recovery_action == 2 || (recovery_action == 1 && recovery_key == key0 + i0)) h = __halves2half2(__low2half(hv), __high2half(h));
                  if (recovery_action == 2 || (recovery_action == 1 && recovery_key == key0 + i0 + 1)) h = __halves2half2(__low2half(h), __high2half(hv));
                  const float2 ra = __half22float2(h);
                  u1_tile = __fmaf_rn(w0, ra.x, u1_tile);
                  u1_tile = __fmaf_rn(w1, ra.y, u1_tile);
                  u2_tile = __fmaf_rn(w0, w0 * ra.x, u2_tile);
                  u2_tile = __fmaf_rn(w1, w1 * ra.y, u2_tile);
                } else {
                  h = __floats2half2_rn(p0, p1);
                }
                const float2 r = __half22float2(h);  // what the MMA will multiply by V
                l_tile += r.x;
                l_tile += r.y;
                const float4 meta = *reinterpret_cast<const float4*>(&sh.v_meta[t][buf][key0 + i0]);  // two keys
                es_tile = __fmaf_rn(r.x, meta.x, es_tile);
                es_tile = __fmaf_rn(r.y, meta.z, es_tile);
                ew_tile = __fmaf_rn(r.x, meta.y, ew_tile);
                ew_tile = __fmaf_rn(r.y, meta.w, ew_tile);
                packed[e] = *reinterpret_cast<const uint32_t*>(&h);
              }
              // 128-byte swizzle: 16-byte chunk index XOR (row mod 8)
              *reinterpret_cast<uint4*>(p_row + ((ch ^ (row_in_tile & 7)) << 4)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            }
          }
          if (!kProtect || attempt == 1) break;
          // moment check of the probabilities just written (a14:1014-1046)
          const float delta0 = l_tile - check_u0, delta1 = u1_tile - check_u1, delta2 = u2_tile - check_u2;
          const float thr0 = __fmaf_rn(p.softmax_rel_tol, fmaxf(1.0f, fabsf(check_u0)), p.softmax_abs_tol);
          const float thr1 = __fmaf_rn(p.softmax_rel_tol, fmaxf(1.0f, fabsf(check_u1)), p.softmax_abs_tol);
          const float thr2 = __fmaf_rn(p.softmax_rel_tol, fmaxf(1.0f, fabsf(check_u2)), p.softmax_abs_tol);
          const bool bad = fabsf(delta0) > thr0 || fabsf(delta1) > thr1 || fabsf(delta2) > thr2;
          if (bad) {
            atomicAdd(&p.report->softmax_detected, 1);
            recovery_action = 2;
            if (fabsf(delta0) > thr0) {
              const float observed_weight = delta1 / delta0;
              const int key_index = __float2int_rn(0.5f * (observed_weight + static_cast<float>(seq - 1)));
              const float second_residual = fabsf(delta2 / delta0 - observed_weight * observed_weight);
              if (key_index >= j * kAttnTile && key_index < (j + 1) * kAttnTile &&
                  fabsf(observed_weight - static_cast<float>(2 * key_index - (seq - 1))) <= 0.25f &&
                  second_residual <= fmaxf(1.0f, fabsf(observed_weight)) * 0.5f) {
                recovery_action = 1;
                recovery_key = key_index - j * kAttnTile;
              }
            }
            atomicAdd(recovery_action == 1 ? &p.report->softmax_corrected : &p.report->softmax_replayed, 1);
          }
          // The repair pass reads the scores again with warp-wide TMEM loads, so the whole warp takes it together;
          // rows without a finding recompute what they already have.
          if (!__any_sync(0xffffffffU, bad)) break;
        }
        if (kProtect) {  // the score buffer is released only now: a repair pass reads it again
          tcgen05_fence_before();
          mbar_arrive(&sh.s_empty[t]);
          // duplicate of the running state (a14:1075-1098)
          l_verify = __fmaf_rn(alpha_check, l_verify, check_u0);
          u1_verify = __fmaf_rn(alpha_check, u1_verify, check_u1);
          u2_verify = __fmaf_rn(alpha_check, u2_verify, check_u2);
          m_verify = m_check;
          u1_run = __fmaf_rn(alpha, u1_run, u1_tile);
          u2_run = __fmaf_rn(alpha, u2_run, u2_tile);
        }
        l_run = __fmaf_rn(alpha, l_run, l_tile);
        exp_sum = __fmaf_rn(alpha, exp_sum, es_tile);
        exp_weighted = __fmaf_rn(alpha, exp_weighted, ew_tile);
        m_run = m_new;
        if (kProtect) {
          if (fault_here && p.fault_stage == FT_ATTN_FAULT_SOFTMAX_STATE && fault_row == row_in_tile && p.fault_index / kAttnTile == j) {
            l_run += p.fault_value;
          }
          auto exceeds = [&](float actual, float expected) {
            return fabsf(actual - expected) > __fmaf_rn(p.softmax_rel_tol, fmaxf(1.0f, fabsf(expected)), p.softmax_abs_tol);
          };
          const bool m_bad = m_run != m_verify && exceeds(m_run, m_verify);  // both are -inf only before the first tile
          if (m_bad || exceeds(l_run, l_verify) || exceeds(u1_run, u1_verify) || exceeds(u2_run, u2_verify)) {
            atomicAdd(&p.report->softmax_detected, 1);
            atomicAdd(&p.report->softmax_replayed, 1);
            m_run = m_verify;
            l_run = l_verify;
            u1_run = u1_verify;
            u2_run = u2_verify;
          }
        }
        fence_proxy_async_shared();  // P written with st.shared must be visible to the MMA's reads
        tcgen05_fence_before();
        mbar_arrive(&sh.p_full[t]);
      }
      // ---- output stage: projection check of O / l (src/ft_flash_attention_a0.cu:613-662), normalise, store
      if (alive && attn_wait_all(&sh.p_empty[t], (my_tiles - 1) & 1, abort_flag, poller, bar_all)) {
        tcgen05_fence_after();
        const float inv_l = 1.0f / l_run;
        const int query = q_tile0 + row_in_tile;
        const bool my_fault = output_fault && fault_row == row_in_tile;
        float actual_sum = 0.0f, actual_weighted = 0.0f;
#pragma unroll 1
        for (int cc = 0; cc < 4; ++cc) {
          float o[32];
          tmem_ld_32x32b_x32(o_addr + cc * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float x = o[i] * inv_l;
            if (my_fault && p.fault_index == cc * 32 + i) x += p.fault_value;
            actual_sum += x;
            actual_weighted = __fmaf_rn(static_cast<float>(2 * (cc * 32 + i) - (kAttnTile - 1)), x, actual_weighted);
          }
        }
        const float expected_sum = exp_sum * inv_l;
        const float expected_weighted = exp_weighted * inv_l;
        const float delta_sum = actual_sum - expected_sum;
        const float delta_weighted = actual_weighted - expected_weighted;
        const float thr_sum = __fmaf_rn(p.pv_rel_tol, fmaxf(1.0f, fabsf(expected_sum)), p.pv_abs_tol);
        const float thr_weighted = __fmaf_rn(p.pv_rel_tol, fmaxf(1.0f, fabsf(expected_weighted)), p.pv_abs_tol);
        int recover_dim = -1;
        const bool real_row = query < p.valid_seq;  // rows that only pad the sequence to whole tiles are neither checked nor stored
        if (real_row && (fabsf(delta_sum) > thr_sum || fabsf(delta_weighted) > thr_weighted)) {
          atomicAdd(&p.report->pv_detected, 1);
          if (fabsf(delta_sum) > thr_sum) {
            const float observed_weight = delta_weighted / delta_sum;
            const int dim = __float2int_rn(0.5f * (observed_weight + static_cast<float>(kAttnTile - 1)));
            if (dim >= 0 && dim < kAttnTile && fabsf(observed_weight - static_cast<float>(2 * dim - (kAttnTile - 1))) <= 0.25f) {
              recover_dim = dim;
              atomicAdd(&p.report->pv_corrected, 1);
            }
          }
          if (recover_dim < 0) atomicAdd(&p.report->failed_rows, 1);
        }
        float* out_row = p.out + (static_cast<size_t>(bh) * p.valid_seq + query) * kAttnTile;
#pragma unroll 1
        for (int cc = 0; cc < 4; ++cc) {
          float o[32];
          tmem_ld_32x32b_x32(o_addr + cc * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float x = o[i] * inv_l;
            if (my_fault && p.fault_index == cc * 32 + i) x += p.fault_value;
            if (recover_dim == cc * 32 + i) x -= delta_sum;
            o[i] = x;
          }
          if (real_row) {
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              __stcs(reinterpret_cast<float4*>(out_row + cc * 32 + i), make_float4(o[i], o[i + 1], o[i + 2], o[i + 3]));
            }
          }
        }
      }
#pragma unroll
      for (int off = 16; off >= 1; off >>= 1) max_ratio = fmaxf(max_ratio, __shfl_xor_sync(0xffffffffU, max_ratio, off));
      if (lane == 0) atomicMax(&p.report->max_noise_bits, __float_as_int(max_ratio));
    }
  }

  // ------------------------------------------------------------------- teardown
  tcgen05_fence_before();
  __syncthreads();
  if (sh.abort_flag != 0) {
    if (threadIdx.x == 0) atomicExch(&p.report->status, 1);
    for (int i = 0; i < 64; ++i) __nanosleep(20000);
    __syncthreads();
  }
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

cudaError_t configure_attention() {
  cudaError_t err = cudaFuncSetAttribute(ft_attention_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmemBytes);
  if (err != cudaSuccess) return err;
  return cudaFuncSetAttribute(ft_attention_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmemBytes);
}

cudaError_t launch_attention(const CUtensorMap& tmap_q, const CUtensorMap& tmap_k, const CUtensorMap& tmap_vt, const AttnParams& params,
                             int batch_heads, cudaStream_t stream) {
  dim3 grid((params.seq + kAttnQTiles * kAttnTile - 1) / (kAttnQTiles * kAttnTile), batch_heads);
  if (params.protect_softmax != 0) {
    ft_attention_fwd_kernel<true><<<grid, kAttnThreads, kAttnSmemBytes, stream>>>(tmap_q, tmap_k, tmap_vt, params);
  } else {
    ft_attention_fwd_kernel<false><<<grid, kAttnThreads, kAttnSmemBytes, stream>>>(tmap_q, tmap_k, tmap_vt, params);
  }
  return cudaGetLastError();
}

}  // namespace ftg
