// Fault-tolerant flash-attention forward, split-row form (the default kernel, with
// or without the softmax-stage protection; the form with one thread per whole row
// in ft_attention.cu is kept for comparison).
//
// One CTA owns 256 queries of one (batch, head) as two 128-query tiles A and B that
// share every 128-key K / V^T tile.  Every query row is worked on by TWO threads:
// the softmax / verifier warpgroup (t, c) takes the key half c (64 columns =
// exactly one 64x64 ABFT tile per 64-row band) of query tile t.
//   warpgroup 0        warp 0 TMA producer of Q and K, warp 2 of V^T, warp 1 issues the score MMAs, warp 3 the PV MMAs
//   warpgroups 1..4    (t, c) = (A,0), (A,1), (B,0), (B,1); 16 softmax warps per SM
//
// Tensor memory: ONE score buffer S (128 columns) serves both query tiles in turn,
// because a thread reads its 64 scores exactly once: the column checksums come from
// a read in the 16x256b fragment layout, then the row's 64 values are loaded into
// registers, the buffer is handed back, and everything else (row checksum, row
// maximum, correction, exponentials) works on the registers.  The columns this
// frees hold 16 extra columns per output accumulator: V^T carries, below its D rows,
// a row of ones and FP16 hi/lo pieces of the per-key sums sum_d V and sum_d w_d V
// (attn_prepare_v_kernel), so the PV product of the tensor core also accumulates
//   l = sum_j p_j,  sum_j p_j vsum_j,  sum_j p_j vweighted_j
// -- the softmax denominator and the two expected output projections of the
// reference's output-stage check (src/ft_flash_attention_a0.cu:585-662) -- from the
// very FP16 probabilities it multiplies by V; the rescaling of O when a row maximum
// moves covers them like any other column.
//
// Per key tile the two threads of a row exchange one number, their row maxima
// (shared memory + one 256-thread barrier).  The ABFT check of a score tile pairs
// the two warps that hold rows 0-31 and 32-63 of the band (abft_tile_check.cuh);
// both belong to the same warpgroup.  A tile whose fault cannot be located (not
// exactly one bad row and one bad column) is replayed on the CUDA cores from Q and
// K in global memory (src/ft_flash_attention_a14.cu:935-959), verified again and
// counted as replayed, or as uncorrected when the replayed tile still disagrees
// with the cached checksums.
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

// Optional timeline of one CTA (library built with -DFT_ATTENTION_TRACE, `make trace`): lane 0 of every softmax warp and
// the two MMA issuer threads store clock64() at fixed points of each key tile; ft_attention_trace_read copies the table
// out.  Without the flag the macro is empty and the kernel is unchanged.
//   actors 0..15  softmax warps (tile A: 0-7, tile B: 8-15; key half = (actor / 4) % 2), slot = key tile, events:
//                 0 starts waiting for S, 1 has S, 2 S handed back, 3 before / 4 after the band barrier,
//                 5 after the tile barrier, 6 before the exponentials, 7 P handed to the PV issuer
//   actor 16      score-MMA issuer, slot = use of the S buffer: 0 loop top, 1 has K, 2 has the S buffer, 3 issued
//   actor 17      PV-MMA issuer, slot = 2 * key tile + query tile: 0 loop top, 1 has V, 2 has P, 3 issued
#ifdef FT_ATTENTION_TRACE
constexpr int kTraceActors = 18, kTraceSlots = 64, kTraceEvents = 8;
__device__ long long g_attention_trace[kTraceActors * kTraceSlots * kTraceEvents];
#define FT_TRACE(actor, slot, event)                                                                                   \
  do {                                                                                                                 \
    if (traced && (slot) < kTraceSlots) g_attention_trace[((actor) * kTraceSlots + (slot)) * kTraceEvents + (event)] = clock64(); \
  } while (0)
#else
#define FT_TRACE(actor, slot, event) \
  do {                               \
  } while (0)
#endif

namespace {

constexpr int kTile = 128;             // queries per tile, keys per tile; the head dimension kDim is 128 or 64
constexpr int kQTiles = 2;             // query tiles per CTA
constexpr int kSlabBytes = 128 * 128;  // 128 rows x 64 FP16 (one 128-byte swizzle row each)
constexpr int kTileBytes = 2 * kSlabBytes;
constexpr int kThreads = 640;
// Register budget.  The CTA is launched with kLaunchRegs registers per thread (what the compiler reports for 640 threads
// per SM); warpgroup 0 then gives registers back and the four softmax warpgroups take more.  setmaxnreg.inc WAITS until
// the CTA's pool holds what it asks for, so the two numbers must fit the pool the launch allocated -- not the register
// file: 128 * 32 + 512 * 112 = 61440 = 640 * 96 (with 40 registers left to warpgroup 0 the softmax warps would wait for ever).
constexpr int kLaunchRegs = 96;
constexpr int kProducerRegs = 32;
constexpr int kSoftmaxRegs = 112;
static_assert(128 * kProducerRegs + 512 * kSoftmaxRegs <= kThreads * kLaunchRegs, "setmaxnreg.inc would wait for registers the CTA does not own");
constexpr uint64_t kTimeoutNs = 2000000000ull;
constexpr float kRescaleStep = 8.0f;  // log2 units: the exponent reference follows the row maximum in steps of at least this
constexpr uint32_t kTmemS = 0;    // the score buffer, shared by the two query tiles
constexpr uint32_t kTmemO = 128;  // output accumulators of tile A, B: kDim + kAttnVExtra columns each

struct SplitShared {
  uint64_t q_full, k_full, k_empty, v_full, v_empty;
  uint64_t s_full[kQTiles], s_free;
  uint64_t p_full[kQTiles], p_empty[kQTiles];
  uint64_t replay_bar[kQTiles][2][2];      // [query tile][key half][row pair]: the two warps of a band in the replay path
  uint32_t tmem_base;
  int abort_flag;
  TileScratch scratch[kQTiles][2][2];      // [query tile][key half][row pair]
  TileScratch replay_scratch[kQTiles][2][2];
  float col_expect[kQTiles][2][2][2][64];  // [query tile][key half][row pair][expected | scale][column]: the band's cached column checksums
  float row_expect[kQTiles][2][2][2][64];  // the same for its rows
  float row_max[kQTiles][2][2][kTile];     // [query tile][parity][key half][row]: the half's row maximum of this key tile
  float2 final_actual[kQTiles][2][kTile];  // [query tile][dim half][row]: {sum_d o, sum_d w_d o} over the half's dims
};

template <int kDim>
constexpr int v_slab_bytes() {
  return (kDim + kAttnVExtra) * 128;  // one slab of V^T: kDim + extra rows x 64 keys
}
template <int kDim>
constexpr int smem_bytes() {
  return 3 * kTileBytes + 2 * v_slab_bytes<kDim>() + 2 * kTileBytes + static_cast<int>(sizeof(SplitShared)) + 1024;
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Hides a value from the optimiser so that a verifier copy is really recomputed.
__device__ __forceinline__ float opaque(float x) {
  asm volatile("" : "+f"(x));
  return x;
}

// Every lane polls the barrier itself (no CTA-level barrier around the wait); the outcome is made uniform over the warp.
// A warp whose wait was abandoned stops working but keeps executing the named barriers of the remaining key tiles
// (see the drain loop in the kernel), so that the warps it shares those barriers with are never left waiting.
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  const bool ok = mbar_wait_bounded(bar, parity, abort_flag, kTimeoutNs);
  return __all_sync(0xffffffffU, ok);
}

// Adds `value` to one element of a TMEM column in place; executed by the whole warp that owns the row's lane quarter.
__device__ __forceinline__ void tmem_add(uint32_t taddr_column, int lane, int target_lane, float value) {
  float x;
  tmem_ld_32x32b_x1(taddr_column, x);
  tmem_wait_ld();
  if (lane == target_lane) x += value;
  tmem_st_32x32b_x1(taddr_column, x);
  tmem_wait_st();
}

template <int Regs>
__device__ __forceinline__ void reg_release() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(Regs));
}
template <int Regs>
__device__ __forceinline__ void reg_acquire() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(Regs));
}

// Row maximum over the keys of this half a row may attend to (all 64 unless the tile is masked for the row).
__device__ __forceinline__ float masked_row_max(const float (&v)[64], bool masked, int first_key, int key_limit) {
  if (masked) {
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < 64; ++i) {
      if (first_key + i <= key_limit) m = fmaxf(m, v[i]);
    }
    return m;
  }
  // two chains of three-input maxima instead of one chain of 64
  float max_a = v[0], max_b = v[1];
#pragma unroll
  for (int i = 2; i < 62; i += 4) {
    max_a = max3_f32(max_a, v[i], v[i + 1]);
    max_b = max3_f32(max_b, v[i + 2], v[i + 3]);
  }
  return max3_f32(max_a, max_b, fmaxf(v[62], v[63]));
}

}  // namespace

// The rare half of the softmax-stage protection, kept out of line: a chunk of eight probabilities whose moments
// disagree with the verifier's (src/ft_flash_attention_a14.cu:1014-1074).  Primary (with the test hook's fault) and
// verifier values are recomputed from the scores; if the deltas of the three moments exceed the tolerance, one key is
// located by their ratios and takes the verifier's value, otherwise the whole chunk does.  Leaves the chunk's FP16
// probabilities in `packed` and what remains of sum(primary - verifier) in *remaining (zero after a replacement, the
// tolerated difference otherwise); false when the deltas are within tolerance.
__device__ __noinline__ bool repair_probability_chunk(const float* x, float scale_log2, float m_new, float m_check, int fault_at,
                                                      float fault_value, int first_key, int seq, float abs_tol, float rel_tol,
                                                      AttnDeviceReport* report, uint32_t* packed, float* remaining) {
  float pr[8], qv[8];
  float u0 = 0.0f, u1 = 0.0f, u2 = 0.0f, c0 = 0.0f, c1 = 0.0f, c2 = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    pr[i] = fast_exp2(__fmaf_rn(x[i], scale_log2, -m_new));
    qv[i] = fast_exp2(opaque(__fmaf_rn(x[i], scale_log2, -m_check)));
    if (i == fault_at) pr[i] += fault_value;
    const float w = static_cast<float>(2 * (first_key + i) - (seq - 1));
    u0 += pr[i];
    u1 = __fmaf_rn(w, pr[i], u1);
    u2 = __fmaf_rn(w * w, pr[i], u2);
    c0 += qv[i];
    c1 = __fmaf_rn(w, qv[i], c1);
    c2 = __fmaf_rn(w * w, qv[i], c2);
  }
  const float delta0 = u0 - c0, delta1 = u1 - c1, delta2 = u2 - c2;
  const float thr0 = __fmaf_rn(rel_tol, fmaxf(1.0f, fabsf(c0)), abs_tol);
  const float thr1 = __fmaf_rn(rel_tol, fmaxf(1.0f, fabsf(c1)), abs_tol);
  const float thr2 = __fmaf_rn(rel_tol, fmaxf(1.0f, fabsf(c2)), abs_tol);
  const bool bad = fabsf(delta0) > thr0 || fabsf(delta1) > thr1 || fabsf(delta2) > thr2;
  if (bad) atomicAdd(&report->softmax_detected, 1);
  int recovery_key = -1;
  if (bad && fabsf(delta0) > thr0) {
    const float observed_weight = delta1 / delta0;
    const int key_index = __float2int_rn(0.5f * (observed_weight + static_cast<float>(seq - 1)));
    const float second_residual = fabsf(delta2 / delta0 - observed_weight * observed_weight);
    if (key_index >= first_key && key_index < first_key + 8 && fabsf(observed_weight - static_cast<float>(2 * key_index - (seq - 1))) <= 0.25f &&
        second_residual <= fmaxf(1.0f, fabsf(observed_weight)) * 0.5f) {
      recovery_key = key_index - first_key;
    }
  }
  if (bad) atomicAdd(recovery_key >= 0 ? &report->softmax_corrected : &report->softmax_replayed, 1);
  float left = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if (bad && (recovery_key < 0 || recovery_key == i)) pr[i] = qv[i];
    left += pr[i] - qv[i];
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const __half2 h = __floats2half2_rn(pr[2 * e], pr[2 * e + 1]);
    packed[e] = *reinterpret_cast<const uint32_t*>(&h);
  }
  *remaining = left;
  return bad;
}

// kProtect adds the reference's softmax-stage protection (src/ft_flash_attention_a14.cu:964-1099) for the thread's half
// of the row: a verifier copy of the exponent reference and of every probability; the moments sum, sum w, sum w^2
// (w = 2 key - (N - 1)) of the differences, checked per chunk of eight keys while the chunk's scores are still in
// registers; replacement of one located probability or of the chunk from the verifier; a duplicate of the running
// state (m, l).  At the end the protected denominator of the row's two threads
// checks the one the PV product accumulated in its checksum column.
template <int kDim, bool kProtect>
__global__ void __launch_bounds__(kThreads, 1)
ft_attention_split_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                          const __grid_constant__ CUtensorMap tmap_vt, const __grid_constant__ AttnParams p) {
  constexpr int kDimSlabs = kDim / 64;             // 128-byte slabs of Q and K rows (64 FP16 each)
  constexpr int kQKBytes = kDimSlabs * kSlabBytes;
  constexpr int kVRows = kDim + kAttnVExtra;       // rows of a V^T tile: the head dimension and the checksum rows
  constexpr int kVSlabBytes = (kDim + kAttnVExtra) * 128;  // one slab of V^T: kVRows rows x 64 keys
  constexpr int kHalfDim = kDim / 2;               // output dims per thread of a row
  constexpr uint32_t kOCols = kDim + kAttnVExtra;  // TMEM columns of one output accumulator

  extern __shared__ uint8_t smem_raw[];
  // aligned to 1024 bytes by pointer arithmetic on the shared array itself, so that the compiler keeps every access below
  // in the shared address space (32-bit addresses, LDS / STS) instead of falling back to generic 64-bit addressing
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* smem_q = smem;                      // 2 query tiles
  uint8_t* smem_k = smem + 2 * kTileBytes;     // 1 stage
  uint8_t* smem_v = smem + 3 * kTileBytes;     // 1 stage: two slabs of kVRows x 64 keys
  uint8_t* smem_p = smem_v + 2 * kVSlabBytes;  // 2 query tiles
  SplitShared& sh = *reinterpret_cast<SplitShared*>(smem_p + 2 * kTileBytes);
  volatile int* abort_flag = &sh.abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int group = warp >> 2;  // 0: producer + MMA; 1..4: softmax of (tile, key half) = (A,0), (A,1), (B,0), (B,1)
  const int bh = blockIdx.y;
#ifdef FT_ATTENTION_TRACE
  // one CTA in the middle of the grid; of a softmax warp its lane 0 (in warpgroup 0 only the elected threads reach a trace point)
  const bool traced = blockIdx.x == gridDim.x / 2 && blockIdx.y == gridDim.y / 2 && (threadIdx.x < 128 || (threadIdx.x & 31) == 0);
#endif
  // causal CTAs get longer towards the end of the sequence: the longest are scheduled first
  const int q_block = p.causal != 0 ? static_cast<int>(gridDim.x - 1 - blockIdx.x) : static_cast<int>(blockIdx.x);
  const int q0 = q_block * kQTiles * kTile;
  const int seq = p.seq;
  const int num_tiles = seq / kTile;
  const int row_base = bh * seq;  // first row of this head in the [B*H*N, D] matrices
  const int qtiles = q0 + kQTiles * kTile <= seq ? kQTiles : 1;  // the last CTA of a head may own one tile
  // causal (src/ft_flash_attention_a14.cu:708): query tile t stops after the key tile on its diagonal
  const bool causal = p.causal != 0;
  const int first_qtile = q0 / kTile;
  auto tiles_of = [&](int t) { return causal ? min(num_tiles, first_qtile + t + 1) : num_tiles; };
  const int cta_tiles = tiles_of(qtiles - 1);

  if (threadIdx.x == 0) {
    mbar_init(&sh.q_full, 1);
    mbar_init(&sh.k_full, 1);
    mbar_init(&sh.k_empty, 1);
    mbar_init(&sh.v_full, 1);
    mbar_init(&sh.v_empty, 1);
    mbar_init(&sh.s_free, 256);  // both key halves of the tile that used the buffer hold their scores in registers
    for (int t = 0; t < kQTiles; ++t) {
      mbar_init(&sh.s_full[t], 1);
      mbar_init(&sh.p_full[t], 256);  // both halves of P are written
      mbar_init(&sh.p_empty[t], 1);
      for (int i = 0; i < 4; ++i) mbar_init(&sh.replay_bar[t][i >> 1][i & 1], 64);
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
    reg_release<kProducerRegs>();
    if (warp == 0 && elect_one()) {
      // ------------------------------------------------------------- producer
      mbar_arrive_expect_tx(&sh.q_full, qtiles * kQKBytes);
      for (int t = 0; t < qtiles; ++t) {
#pragma unroll
        for (int sl = 0; sl < kDimSlabs; ++sl) {
          tma_load_2d(smem_q + t * kTileBytes + sl * kSlabBytes, &tmap_q, &sh.q_full, 64 * sl, row_base + q0 + t * kTile);
        }
      }
      for (int j = 0; j < cta_tiles; ++j) {
        const uint32_t ph = j & 1;
        if (!mbar_wait_bounded(&sh.k_empty, ph ^ 1, abort_flag, kTimeoutNs)) break;
        mbar_arrive_expect_tx(&sh.k_full, kQKBytes);
#pragma unroll
        for (int sl = 0; sl < kDimSlabs; ++sl) tma_load_2d(smem_k + sl * kSlabBytes, &tmap_k, &sh.k_full, 64 * sl, row_base + j * kTile);
      }
    } else if (warp == 2 && elect_one()) {
      // ------------------------------------------------------------- producer of V^T: its own thread, so that the load of
      // K_{j+1} never queues behind the wait for the V buffer
      for (int j = 0; j < cta_tiles; ++j) {
        const uint32_t ph = j & 1;
        if (!mbar_wait_bounded(&sh.v_empty, ph ^ 1, abort_flag, kTimeoutNs)) break;
        mbar_arrive_expect_tx(&sh.v_full, 2 * kVSlabBytes);
        tma_load_2d(smem_v, &tmap_vt, &sh.v_full, j * kTile, bh * kVRows);
        tma_load_2d(smem_v + kVSlabBytes, &tmap_vt, &sh.v_full, j * kTile + 64, bh * kVRows);
      }
    } else if ((warp == 1 || warp == 3) && elect_one()) {
      // ------------------------------------------------------------- MMA issuers: warp 1 the score products, warp 3 the PV
      // products.  Two threads, so that neither chain queues behind a wait of the other (a score product never waits for
      // probabilities, a PV product never for a free score buffer) and each loop keeps only a handful of registers.
      // The score buffer is used in the order (key tile 0: A, B), (key tile 1: A, B), ...; use n may start when the
      // softmax threads of use n-1 hold their scores in registers.  The PV products follow the same order.
      auto advance = [&](int& j, int& t) {  // next (key tile, query tile) in use order; j == cta_tiles at the end
        do {
          if (++t == qtiles) {
            t = 0;
            ++j;
          }
        } while (j < cta_tiles && j >= tiles_of(t));
      };
      int j = 0, t = 0;
      if (warp == 1) {
        constexpr uint32_t idesc_s = make_idesc_f16_f32(kTile, kTile);  // S: 128 queries x 128 keys
        bool alive = mbar_wait_bounded(&sh.q_full, 0, abort_flag, kTimeoutNs);
        int k_waited = -1;
        uint32_t uses = 0;
        while (alive && j < cta_tiles) {
          FT_TRACE(16, uses, 0);
          if (k_waited != j) {
            if (!mbar_wait_bounded(&sh.k_full, j & 1, abort_flag, kTimeoutNs)) break;
            k_waited = j;
          }
          FT_TRACE(16, uses, 1);
          if (uses > 0 && !mbar_wait_bounded(&sh.s_free, (uses - 1) & 1, abort_flag, kTimeoutNs)) break;
          FT_TRACE(16, uses, 2);
          tcgen05_fence_after();
#pragma unroll
          for (int kk = 0; kk < kDim / 16; ++kk) {
            uint64_t da = make_smem_desc_sw128(smem_u32(smem_q + t * kTileBytes + (kk >> 2) * kSlabBytes)) + 2 * (kk & 3);
            uint64_t db = make_smem_desc_sw128(smem_u32(smem_k + (kk >> 2) * kSlabBytes)) + 2 * (kk & 3);
            umma_f16(tmem_base + kTmemS, da, db, idesc_s, kk != 0 ? 1u : 0u);
          }
          umma_commit(&sh.s_full[t]);
          FT_TRACE(16, uses, 3);
          const int before = j;
          advance(j, t);
          if (j != before) umma_commit(&sh.k_empty);  // that was the last product that reads K_j
          ++uses;
        }
      } else {
        constexpr uint32_t idesc_o = make_idesc_f16_f32(kTile, kVRows);  // O and its checksum columns: 128 queries x (kDim + 16)
        int v_waited = -1;
        while (j < cta_tiles) {
          FT_TRACE(17, 2 * j + t, 0);
          if (v_waited != j) {
            if (!mbar_wait_bounded(&sh.v_full, j & 1, abort_flag, kTimeoutNs)) break;
            v_waited = j;
          }
          FT_TRACE(17, 2 * j + t, 1);
          if (!mbar_wait_bounded(&sh.p_full[t], j & 1, abort_flag, kTimeoutNs)) break;
          FT_TRACE(17, 2 * j + t, 2);
          tcgen05_fence_after();
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            uint64_t da = make_smem_desc_sw128(smem_u32(smem_p + t * kTileBytes + (kk >> 2) * kSlabBytes)) + 2 * (kk & 3);
            uint64_t db = make_smem_desc_sw128(smem_u32(smem_v + (kk >> 2) * kVSlabBytes)) + 2 * (kk & 3);
            umma_f16(tmem_base + kTmemO + t * kOCols, da, db, idesc_o, (j | kk) != 0 ? 1u : 0u);
          }
          umma_commit(&sh.p_empty[t]);
          FT_TRACE(17, 2 * j + t, 3);
          const int before = j;
          advance(j, t);
          if (j != before) umma_commit(&sh.v_empty);  // that was the last product that reads V_j
        }
      }
    }
  } else {
    reg_acquire<kSoftmaxRegs>();
    // ------------------------------------------------------------- softmax / verifier: two threads per query row
    const int t = (group - 1) >> 1;  // query tile of this warpgroup
    const int c = (group - 1) & 1;   // key half of S / dim half of O this warpgroup works on
    if (t < qtiles) {
      const int quarter = warp & 3;
      const int pair = quarter >> 1;
      const int half = quarter & 1;
      const int r_local = half * 32 + lane;
      const int row_in_tile = quarter * 32 + lane;
      const int bar_tile = 1 + t;                       // 256-thread barrier of the two warpgroups of tile t (ids 1, 2)
      const int bar_pair = 3 + 2 * (group - 1) + pair;  // 64-thread barrier of this 64-row band (ids 3..10)
      const int tile_cols = seq / 64;
      const size_t head_cache = static_cast<size_t>(bh) * tile_cols * tile_cols * 64;
      const int q_tile0 = q0 + t * kTile;
      const int q_band = q_tile0 / 64 + pair;
      const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
      const uint32_t s_addr = lane_addr + kTmemS + c * 64;                     // this half's 64 score columns
      const uint32_t o_addr = lane_addr + kTmemO + t * kOCols + c * kHalfDim;  // this half's output dims
      const uint32_t x_addr = lane_addr + kTmemO + t * kOCols + kDim;          // the checksum columns of the row
      uint8_t* p_row = smem_p + t * kTileBytes + c * kSlabBytes + (row_in_tile >> 3) * 1024 + (row_in_tile & 7) * 128;
      TileScratch& scratch = sh.scratch[t][c][pair];
      uint32_t replays = 0;  // times this band went through the replay path (the phase of its barrier)

      float m_run = -INFINITY, max_ratio = 0.0f;
      // kProtect: running denominator of this half of the row and the verifier's duplicate of the state
      float l_run = 0.0f, m_verify = -INFINITY, l_verify = 0.0f;
      bool alive = true;
      const int my_tiles = tiles_of(t);
      // when a wait is abandoned: the first key tile whose band barrier / tile barrier this warp still owes the others
      int owed_pair_from = my_tiles, owed_tile_from = my_tiles;
      // Cached expected checksums of the band's 64x64 tile of key tile jj.  They travel by asynchronous copy straight into
      // shared memory -- the band's first warp brings the column expectations, its second the column scales, two adjacent
      // columns per lane, and every thread the pair of its own row -- so that they cost no register while the scores are
      // worked on and their latency is over when they are needed.
      auto prefetch_checksums = [&](int jj) {
        const size_t cache = head_cache + (static_cast<size_t>(q_band) * tile_cols + jj * 2 + c) * 64;
        cp_async_8(&sh.col_expect[t][c][pair][half][2 * lane], (half == 0 ? p.expected_cols : p.col_scales) + cache + 2 * lane);
        cp_async_4(&sh.row_expect[t][c][pair][0][r_local], p.expected_rows + cache + r_local);  // read back by this thread only
        cp_async_4(&sh.row_expect[t][c][pair][1][r_local], p.row_scales + cache + r_local);
        cp_async_commit();
      };
      if (my_tiles > 0) prefetch_checksums(0);
      for (int j = 0; j < my_tiles; ++j) {
        const int buf = j & 1;
        // Keys of this tile the row may attend to are those with local index <= key_limit: all 128, up to the query in
        // the causal diagonal tile (src/ft_flash_attention_a14.cu:893), up to the last real key in the last tile of a
        // sequence that was padded to whole tiles.
        int key_limit = kTile - 1;
        if (causal && j == first_qtile + t) key_limit = row_in_tile;
        if ((j + 1) * kTile > p.valid_seq) key_limit = min(key_limit, p.valid_seq - 1 - j * kTile);
        const bool diagonal = key_limit < kTile - 1;  // some keys of this tile are masked for this row
        // (asked for by prefetch_checksums: for the first tile before the loop, for the others while the previous tile's
        // probabilities drain into shared memory)
        FT_TRACE(warp - 4, j, 0);
        if (!warp_wait(&sh.s_full[t], j & 1, abort_flag)) {
          alive = false;
          owed_pair_from = owed_tile_from = j;
          break;
        }
        tcgen05_fence_after();
        FT_TRACE(warp - 4, j, 1);

        // test hook: the fault enters the accumulator itself, before any checksum
        if (p.fault_stage == FT_ATTN_FAULT_SCORE && p.fault_bh == bh) {  // uniform over the CTA
          const int r1 = p.fault_query - q_tile0, r2 = p.fault2_query - q_tile0;
          if (r1 >= 0 && r1 < kTile && p.fault_index / 64 == j * 2 + c && r1 / 32 == quarter) {
            tmem_add(s_addr + p.fault_index % 64, lane, r1 % 32, p.fault_value);
          }
          if (p.fault2_value != 0.0f && r2 >= 0 && r2 < kTile && p.fault2_index / 64 == j * 2 + c && r2 / 32 == quarter) {
            tmem_add(s_addr + p.fault2_index % 64, lane, r2 % 32, p.fault2_value);
          }
        }

        // ---- the one read of this thread's scores: column checksums from the fragment layout, then the row into registers
        abft_tile_cols_from_tmem(s_addr, lane, half, scratch);
        float v[64];
        tmem_ld_32x32b_x32(s_addr, v);
        tmem_ld_32x32b_x32(s_addr + 32, v + 32);
        tmem_wait_ld();
        tcgen05_fence_before();
        mbar_arrive(&sh.s_free);  // the buffer can take the next score product (the other query tile's)
        FT_TRACE(warp - 4, j, 2);
        cp_async_wait_all();  // this lane's pieces of the cached checksums have landed; the band barrier below publishes the column side
        abft_tile_rows(v, lane, half, scratch, sh.row_expect[t][c][pair][0][r_local], sh.row_expect[t][c][pair][1][r_local],
                       p.score_abs_tol, p.score_rel_tol, max_ratio);
        float local_max = masked_row_max(v, diagonal, c * 64, key_limit);
        FT_TRACE(warp - 4, j, 3);
        asm volatile("bar.sync %0, 64;" ::"r"(bar_pair) : "memory");
        FT_TRACE(warp - 4, j, 4);
        {
          const float exp_col0 = sh.col_expect[t][c][pair][0][lane], exp_col1 = sh.col_expect[t][c][pair][0][32 + lane];
          const float scale_col0 = sh.col_expect[t][c][pair][1][lane], scale_col1 = sh.col_expect[t][c][pair][1][32 + lane];
          const TileDecision d = abft_tile_decide(lane, scratch, exp_col0, exp_col1, scale_col0, scale_col1, p.score_abs_tol,
                                                  p.score_rel_tol, max_ratio);
          if ((d.bad_rows | d.bad_cols) != 0) {  // uniform over the two warps of the band; rare
            bool replayed = false;
            if (d.corrected) {
              if (d.bad_row == r_local) {
                // src/s4:493-497 in registers
                const float fix = 0.5f * (d.row_delta + d.col_delta);
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                  if (i == d.bad_col) v[i] += fix;
                }
              }
            } else {
              // The fault cannot be located: recompute the band's 64 x 64 scores without the tensor core and check again.
              const size_t cache = head_cache + (static_cast<size_t>(q_band) * tile_cols + j * 2 + c) * 64;
              const __half* q_row = static_cast<const __half*>(p.q) + (static_cast<size_t>(row_base) + q_tile0 + row_in_tile) * kDim;
              const __half* k_tile = static_cast<const __half*>(p.k) + (static_cast<size_t>(row_base) + j * kTile + c * 64) * kDim;
              float rv[64];
              bool wait_ok = true;
              replayed = replay_and_verify<kDim>(q_row, k_tile, rv, lane, half, &sh.replay_scratch[t][c][pair], p.expected_rows + cache,
                                                 p.row_scales + cache, p.expected_cols + cache, p.col_scales + cache, p.score_abs_tol,
                                                 p.score_rel_tol, &sh.replay_bar[t][c][pair], replays & 1, abort_flag, kTimeoutNs, &wait_ok);
              if (!wait_ok) {  // the partner warp gave up: this tile's band barrier is passed, its tile barrier is owed
                alive = false;
                owed_pair_from = j + 1;
                owed_tile_from = j;
                break;
              }
              ++replays;
#pragma unroll
              for (int i = 0; i < 64; ++i) v[i] = rv[i];
            }
            local_max = masked_row_max(v, diagonal, c * 64, key_limit);
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
        // ---- the two halves of the row exchange their maxima
        sh.row_max[t][buf][c][row_in_tile] = local_max;
        asm volatile("bar.sync %0, 256;" ::"r"(bar_tile) : "memory");
        FT_TRACE(warp - 4, j, 5);
        const float row_max = fmaxf(local_max, sh.row_max[t][buf][c ^ 1][row_in_tile]);

        // ---- online softmax state (log2 domain); identical in both threads of the row.  The reference point of the
        // exponentials moves only when the tile's maximum exceeds it by more than kRescaleStep: probabilities then stay
        // below 2^kRescaleStep (exact in FP16 up to 2^16, and l, O and the checksum columns all carry the same factor,
        // which the final division removes), and the pass over O that a moved reference costs becomes rare instead of
        // happening whenever any of the warp's 32 rows sees a new maximum.
        const float m_tile = row_max * p.scale_log2;
        float alpha = 1.0f;
        if (m_tile > m_run + kRescaleStep) {  // always for the first tile (m_run = -inf)
          alpha = fast_exp2(m_run - m_tile);  // 0 for the first tile
          m_run = m_tile;
        }
        const float m_new = m_run;
        float m_check = m_new, alpha_check = alpha;
        if (kProtect) {
          // the verifier follows its own copy of the maximum and of the reference point, by the same rule
          const float verifier_max = opaque(row_max);
          if (c == 0 && fabsf(row_max - verifier_max) > p.softmax_abs_tol) {
            atomicAdd(&p.report->softmax_detected, 1);
            atomicAdd(&p.report->softmax_replayed, 1);
          }
          const float m_tile_check = verifier_max * p.scale_log2;
          m_check = m_verify;
          alpha_check = 1.0f;
          if (m_tile_check > m_verify + kRescaleStep) {
            alpha_check = fast_exp2(opaque(m_verify - m_tile_check));
            m_check = m_tile_check;
          }
        }

        if (j > 0) {
          // PV of the previous tile must have finished: the P buffer is free and O is quiescent
          if (!warp_wait(&sh.p_empty[t], (j - 1) & 1, abort_flag)) {
            alive = false;
            owed_pair_from = owed_tile_from = j + 1;
            break;
          }
          tcgen05_fence_after();
          if (__any_sync(0xffffffffU, alpha != 1.0f)) {
            const unsigned long long alpha2 = pack_f32x2(alpha, alpha);
#pragma unroll 1
            for (int cc = 0; cc < kHalfDim / 32; ++cc) {  // this half's output dims
              float o[32];
              tmem_ld_32x32b_x32(o_addr + cc * 32, o);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; i += 2) unpack_f32x2(mul_f32x2(pack_f32x2(o[i], o[i + 1]), alpha2), o[i], o[i + 1]);
              tmem_st_32x32b_x32(o_addr + cc * 32, o);
            }
            if (c == 1) {  // the checksum columns (l and the expected projections) scale with the row like any output column
              float x[8];
              tmem_ld_32x32b_x8(x_addr, x);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 8; i += 2) unpack_f32x2(mul_f32x2(pack_f32x2(x[i], x[i + 1]), alpha2), x[i], x[i + 1]);
              tmem_st_32x32b_x8(x_addr, x);
            }
            tmem_wait_st();
          }
        }
        FT_TRACE(warp - 4, j, 6);
        // ---- probabilities of this half: FP16 P slab for the MMA (which also forms l and the expected projections)
        {
          if (diagonal) {  // exp2(-inf) = 0: a masked key gets probability zero
#pragma unroll
            for (int i = 0; i < 64; ++i) {
              if (c * 64 + i > key_limit) v[i] = -INFINITY;
            }
          }
          // two scores per instruction where the arithmetic allows it (packed FP32 pairs)
          const unsigned long long scale2 = pack_f32x2(p.scale_log2, p.scale_log2), neg_m2 = pack_f32x2(-m_new, -m_new);
          if (!kProtect) {
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) {
              uint32_t packed[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int i0 = ch * 8 + 2 * e;
                float a0, a1;
                unpack_f32x2(fma_f32x2(pack_f32x2(v[i0], v[i0 + 1]), scale2, neg_m2), a0, a1);
                const __half2 h = __floats2half2_rn(fast_exp2(a0), fast_exp2(a1));
                packed[e] = *reinterpret_cast<const uint32_t*>(&h);
              }
              // 128-byte swizzle: 16-byte chunk index XOR (row mod 8)
              *reinterpret_cast<uint4*>(p_row + ((ch ^ (row_in_tile & 7)) << 4)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            }
          } else {
            const unsigned long long neg_check2 = pack_f32x2(-m_check, -m_check);
            const int fault_key = p.fault_stage == FT_ATTN_FAULT_SOFTMAX && p.fault_bh == bh && p.fault_query == q_tile0 + row_in_tile &&
                                          p.fault_index / 64 == j * 2 + c
                                      ? p.fault_index % 64
                                      : -1;
            const int first_key = j * kTile + c * 64;
            unsigned long long cl2 = 0;  // a packed pair of zeros: sum of the verifier's probabilities
            float l_extra = 0.0f;        // sum over the chunks that went to the out-of-line check of (primary - verifier)
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) {
              uint32_t packed[4];
              uint32_t differ = 0;  // primary and verifier run the same instructions on the same inputs: any differing bit is a finding
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int i0 = ch * 8 + 2 * e;
                const unsigned long long x2 = pack_f32x2(v[i0], v[i0 + 1]);
                float a0, a1, b0, b1;
                unpack_f32x2(fma_f32x2(x2, scale2, neg_m2), a0, a1);
                unpack_f32x2(fma_f32x2(x2, scale2, neg_check2), b0, b1);
                const float p0 = fast_exp2(a0), p1 = fast_exp2(a1);
                const float q0 = fast_exp2(opaque(b0)), q1 = fast_exp2(opaque(b1));  // the verifier's copies
                differ |= (__float_as_uint(p0) ^ __float_as_uint(q0)) | (__float_as_uint(p1) ^ __float_as_uint(q1));
                cl2 = add_f32x2(cl2, pack_f32x2(q0, q1));
                const __half2 h = __floats2half2_rn(p0, p1);
                packed[e] = *reinterpret_cast<const uint32_t*>(&h);
              }
              // A chunk with a finding (or the test hook's fault) takes the out-of-line path: moments of both copies with
              // the reference's weights and tolerance, location, replacement (repair_probability_chunk).
              if (differ != 0 || (fault_key >> 3) == ch) {
                float x8[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) x8[i] = v[ch * 8 + i];
                float extra = 0.0f;
                repair_probability_chunk(x8, p.scale_log2, m_new, m_check, (fault_key >> 3) == ch ? (fault_key & 7) : -1, p.fault_value,
                                         first_key + ch * 8, seq, p.softmax_abs_tol, p.softmax_rel_tol, p.report, packed, &extra);
                l_extra += extra;
              }
              *reinterpret_cast<uint4*>(p_row + ((ch ^ (row_in_tile & 7)) << 4)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            }
            // running denominator and the duplicate of the state (a14:1075-1098)
            {
              float lo, hi;
              unpack_f32x2(cl2, lo, hi);
              l_run = __fmaf_rn(alpha, l_run, lo + hi + l_extra);  // the primary sum: the verifier's plus what the findings left
              l_verify = __fmaf_rn(alpha_check, l_verify, lo + hi);
              m_verify = m_check;
              if (p.fault_stage == FT_ATTN_FAULT_SOFTMAX_STATE && p.fault_bh == bh && p.fault_query == q_tile0 + row_in_tile &&
                  p.fault_index / 64 == j * 2 + c) {
                l_run += p.fault_value;  // test hook: the fault enters the running denominator
              }
              auto exceeds = [&](float actual, float expected) {
                return fabsf(actual - expected) > __fmaf_rn(p.softmax_rel_tol, fmaxf(1.0f, fabsf(expected)), p.softmax_abs_tol);
              };
              const bool m_bad = m_run != m_verify && exceeds(m_run, m_verify);  // both are -inf only before the first tile
              if (m_bad || exceeds(l_run, l_verify)) {
                atomicAdd(&p.report->softmax_detected, 1);
                atomicAdd(&p.report->softmax_replayed, 1);
                m_run = m_verify;
                l_run = l_verify;
              }
            }
          }
        }
        // The band's cached checksums were last read before this tile's 256-thread barrier: the next tile's can be asked
        // for now, while the stores above drain.
        if (j + 1 < my_tiles) prefetch_checksums(j + 1);
        fence_proxy_async_shared();  // P written with st.shared must be visible to the MMA's reads
        tcgen05_fence_before();
        mbar_arrive(&sh.p_full[t]);
        FT_TRACE(warp - 4, j, 7);
      }
      // only after an abandoned wait: the named barriers the other warps of the band / tile still count on
      for (int jj = min(owed_pair_from, owed_tile_from); jj < my_tiles; ++jj) {
        if (jj >= owed_pair_from) asm volatile("bar.sync %0, 64;" ::"r"(bar_pair) : "memory");
        if (jj >= owed_tile_from) asm volatile("bar.sync %0, 256;" ::"r"(bar_tile) : "memory");
      }
      // ---- output stage: projection check of O / l (src/ft_flash_attention_a0.cu:613-662), normalise, store.
      // Its exchange barrier is executed by every warp; a warp that gave up skips the work around it (the run is
      // reported as timed out, its output is not valid).
      alive = alive && warp_wait(&sh.p_empty[t], (my_tiles - 1) & 1, abort_flag);
      float inv_l = 0.0f, es_total = 0.0f, ew_total = 0.0f;
      float actual_sum = 0.0f, actual_weighted = 0.0f;
      const int query = q_tile0 + row_in_tile;
      const bool my_fault = p.fault_stage == FT_ATTN_FAULT_OUTPUT && p.fault_bh == bh && p.fault_query == query && p.fault_index / kHalfDim == c;
      float l_protected = 0.0f;
      if (kProtect) {
        // the protected denominator is the sum of the two halves' registers (fixed order: both threads hold the same bits);
        // the exchange uses the parity of the row-maximum buffer that the last key tile did not use
        sh.row_max[t][my_tiles & 1][c][row_in_tile] = l_run;
        asm volatile("bar.sync %0, 256;" ::"r"(bar_tile) : "memory");
        const float other_l = sh.row_max[t][my_tiles & 1][c ^ 1][row_in_tile];
        l_protected = c == 0 ? l_run + other_l : other_l + l_run;
      }
      if (alive) {
        tcgen05_fence_after();
        {
          // what the tensor core accumulated beside the output: [0] l, [1]+[2] sum p*vsum (hi and lo pieces),
          // [3]+[4] sum p*vweighted / kAttnVWeightScale
          float x[8];
          tmem_ld_32x32b_x8(x_addr, x);
          tmem_wait_ld();
          float l_total = x[0];
          if (kProtect) {
            // The tensor core summed the FP16-rounded probabilities, the registers the unrounded ones: they agree to a
            // fraction of the FP16 rounding step.  Beyond that the protected registers decide.
            if (fabsf(l_total - l_protected) > 1.0e-3f * l_protected) {
              if (c == 0) {
                atomicAdd(&p.report->softmax_detected, 1);
                atomicAdd(&p.report->softmax_replayed, 1);
              }
              l_total = l_protected;
            }
          }
          inv_l = 1.0f / l_total;
          es_total = x[1] + x[2];
          ew_total = (x[3] + x[4]) * kAttnVWeightScale;
        }
#pragma unroll 1
        for (int cc = 0; cc < kHalfDim / 32; ++cc) {
          float o[32];
          tmem_ld_32x32b_x32(o_addr + cc * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int dim = c * kHalfDim + cc * 32 + i;
            float x = o[i] * inv_l;
            if (my_fault && p.fault_index == dim) x += p.fault_value;
            actual_sum += x;
            actual_weighted = __fmaf_rn(static_cast<float>(2 * dim - (kDim - 1)), x, actual_weighted);
          }
        }
        sh.final_actual[t][c][row_in_tile] = make_float2(actual_sum, actual_weighted);
      }
      asm volatile("bar.sync %0, 256;" ::"r"(bar_tile) : "memory");
      if (alive) {
        const float2 other_actual = sh.final_actual[t][c ^ 1][row_in_tile];
        // totals in a fixed order (half 0 + half 1) so that both threads of the row hold the same bits
        const float sum_total = c == 0 ? actual_sum + other_actual.x : other_actual.x + actual_sum;
        const float weighted_total = c == 0 ? actual_weighted + other_actual.y : other_actual.y + actual_weighted;
        const float expected_sum = es_total * inv_l;
        const float expected_weighted = ew_total * inv_l;
        const float delta_sum = sum_total - expected_sum;
        const float delta_weighted = weighted_total - expected_weighted;
        const float thr_sum = __fmaf_rn(p.pv_rel_tol, fmaxf(1.0f, fabsf(expected_sum)), p.pv_abs_tol);
        const float thr_weighted = __fmaf_rn(p.pv_rel_tol, fmaxf(1.0f, fabsf(expected_weighted)), p.pv_abs_tol);
        int recover_dim = -1;
        const bool real_row = query < p.valid_seq;  // rows that only pad the sequence to whole tiles are neither checked nor stored
        if (real_row && (fabsf(delta_sum) > thr_sum || fabsf(delta_weighted) > thr_weighted)) {  // the same in both threads of the row
          if (fabsf(delta_sum) > thr_sum) {
            const float observed_weight = delta_weighted / delta_sum;
            const int dim = __float2int_rn(0.5f * (observed_weight + static_cast<float>(kDim - 1)));
            if (dim >= 0 && dim < kDim && fabsf(observed_weight - static_cast<float>(2 * dim - (kDim - 1))) <= 0.25f) recover_dim = dim;
          }
          if (c == 0) {  // one of the two threads reports
            atomicAdd(&p.report->pv_detected, 1);
            atomicAdd(recover_dim >= 0 ? &p.report->pv_corrected : &p.report->failed_rows, 1);
          }
        }
        float* out_row = p.out + (static_cast<size_t>(bh) * p.valid_seq + query) * kDim + c * kHalfDim;
#pragma unroll 1
        for (int cc = 0; cc < kHalfDim / 32; ++cc) {
          float o[32];
          tmem_ld_32x32b_x32(o_addr + cc * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int dim = c * kHalfDim + cc * 32 + i;
            float x = o[i] * inv_l;
            if (my_fault && p.fault_index == dim) x += p.fault_value;
            if (recover_dim == dim) x -= delta_sum;
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

cudaError_t configure_attention_split() {
  cudaError_t err = cudaFuncSetAttribute(ft_attention_split_kernel<128, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<128>());
  if (err == cudaSuccess) err = cudaFuncSetAttribute(ft_attention_split_kernel<64, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<64>());
  if (err == cudaSuccess) err = cudaFuncSetAttribute(ft_attention_split_kernel<128, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<128>());
  if (err == cudaSuccess) err = cudaFuncSetAttribute(ft_attention_split_kernel<64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<64>());
  return err;
}

cudaError_t launch_attention_split(const CUtensorMap& tmap_q, const CUtensorMap& tmap_k, const CUtensorMap& tmap_vt, const AttnParams& params,
                                   int batch_heads, cudaStream_t stream) {
  dim3 grid((params.seq + kQTiles * kTile - 1) / (kQTiles * kTile), batch_heads);
  const bool protect = params.protect_softmax != 0;
  if (params.dim == 64) {
    if (protect) {
      ft_attention_split_kernel<64, true><<<grid, kThreads, smem_bytes<64>(), stream>>>(tmap_q, tmap_k, tmap_vt, params);
    } else {
      ft_attention_split_kernel<64, false><<<grid, kThreads, smem_bytes<64>(), stream>>>(tmap_q, tmap_k, tmap_vt, params);
    }
  } else if (protect) {
    ft_attention_split_kernel<128, true><<<grid, kThreads, smem_bytes<128>(), stream>>>(tmap_q, tmap_k, tmap_vt, params);
  } else {
    ft_attention_split_kernel<128, false><<<grid, kThreads, smem_bytes<128>(), stream>>>(tmap_q, tmap_k, tmap_vt, params);
  }
  return cudaGetLastError();
}

}  // namespace ftg

#ifdef FT_ATTENTION_TRACE
// Copies the timeline table of the last launch to the host: [actor][slot][event] cycle counts (see FT_TRACE above).
extern "C" int ft_attention_trace_read(long long* out, int count) {
  const int total = ftg::kTraceActors * ftg::kTraceSlots * ftg::kTraceEvents;
  if (out == nullptr || count < total) return total;
  return cudaMemcpyFromSymbol(out, ftg::g_attention_trace, sizeof(long long) * total) == cudaSuccess ? 0 : -1;
}
#endif
