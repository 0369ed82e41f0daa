// Fused FP8 GEMM + ABFT checker/corrector for sm_100a.
//
// Replaces the reference's wgmma_tma_k128_cluster_abft_kernel
// (src/s4_cluster_multicast_abft_fp8_gemm.cu:301-519) with the same operator
// semantics -- C[N,M] column-major = A[M,K] * B[N,K]^T in FP32, checked per 64x64
// ABFT tile against cached expected row/column checksums, single faults located
// at the (row, column) intersection and corrected by 0.5*(row_delta+col_delta)
// (src/s4:432-503) -- on a different machine model:
//
//   * persistent CTAs, one per SM, each owning 128 rows x 256 columns of an
//     output tile.  In the pair form (kPair) two CTAs of a cluster share one
//     256x256 tile: each stages its own 128 rows of A and HALF of the B tile, and
//     the leader CTA issues one tcgen05.mma.cta_group::2 (M256 N256 K32) for
//     both, which halves the shared-memory traffic per MMA;
//   * warp 0: TMA producer, ring of (A, B) FP8 stages with 128-byte swizzle,
//     mbarrier full/empty pairs;
//   * warp 1: one thread issues tcgen05.mma kind::f8f6f4 from shared-memory
//     descriptors into one of two 256-column TMEM accumulators;
//   * warps 2-9: epilogue, two sets of four warps (one warp per TMEM lane quarter
//     in each set); set e takes the 64-column groups g = e, e+2 of a tile, so that
//     every scheduler has two epilogue warps to switch between.  Each thread owns
//     one accumulator row; per group the warp first reads its 32 x 64 block in the
//     16x256b fragment layout and forms the column sums over its rows (packed
//     additions, 14 shuffles), then loads the row's 64 values into registers,
//     forms the row sum serially (the reference's order), exchanges the column
//     sums with its partner warp (the other 32 rows of the 64-row ABFT tile),
//     decides, corrects the faulty element in its registers and only then
//     stores.  The epilogue of tile i runs while the main loop of tile i+1 fills
//     the other accumulator.
//
// Every wait is bounded: on expiry the kernel sets report->status and leaves.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "abft_tile_check.cuh"
#include "kernels.h"
#include "sm100_ptx.cuh"

namespace ftg {

constexpr int kBlockM = 128;   // rows of C per CTA
constexpr int kBlockN = 256;   // columns of C per tile
constexpr int kBlockK = 128;   // FP8 elements = bytes = one 128-byte swizzle row
constexpr int kUmmaK = 32;
constexpr int kABytes = kBlockM * kBlockK;
constexpr int kTmemColumns = 512;
constexpr int kAccumulators = 2;
constexpr int kEpilogueSets = 2;  // sets of four epilogue warps; a set covers all four TMEM lane quarters
constexpr int kEpilogueThreads = 128 * kEpilogueSets;
constexpr int kThreads = 64 + kEpilogueThreads;
constexpr int kGroupCols = 64;  // = FT_ABFT_TILE
constexpr int kMaxStages = 7;

template <bool kPair>
struct Config {
  static constexpr int kBRows = kPair ? kBlockN / 2 : kBlockN;  // rows of B staged by one CTA
  static constexpr int kBBytes = kBRows * kBlockK;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = kPair ? 7 : 4;
  static constexpr int kTileM = kPair ? 2 * kBlockM : kBlockM;  // rows of C per scheduled tile
  static constexpr uint32_t kExpectTx = kPair ? 2 * kStageBytes : kStageBytes;
  static constexpr uint32_t kEmptyArrivals = kPair ? 2 * kEpilogueThreads : kEpilogueThreads;
};

struct RowInfo {
  int count;
  int first;
  float delta;
  int pad;
};

struct EpilogueScratch {
  float colpart[2][kGroupCols];  // [warp half][column]: column sums over that warp's 32 rows
  RowInfo rows[2];               // [warp half]
};

struct SharedTail {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[kAccumulators];
  uint64_t tmem_empty[kAccumulators];
  uint32_t tmem_base;
  int abort_flag;
  EpilogueScratch scratch[kEpilogueSets][2];  // [epilogue set][row pair]
};

template <bool kPair>
constexpr int smem_bytes() {
  return Config<kPair>::kStages * Config<kPair>::kStageBytes + static_cast<int>(sizeof(SharedTail));
}

static_assert(smem_bytes<true>() <= 232448 && smem_bytes<false>() <= 232448, "more dynamic shared memory than a CTA can have on sm_100");

// tile index -> (row block of kTileM rows, column block of 256 columns)
__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int group, int& mb, int& nb) {
  int per_group = group * num_n;
  int g = t / per_group;
  int first_m = g * group;
  int group_m = min(group, num_m - first_m);
  int in_group = t - g * per_group;
  mb = first_m + in_group % group_m;
  nb = in_group / group_m;
}

// Work item `w` of a launch -> its output tile.  Items below `split_from` are whole tiles (256 columns); every tile from
// there on is cut into `split` column slices of 256 / split columns, each an item of its own (GemmParams::split).
// Returns false for a slice that lies entirely past the last column of the window (ragged N): such an item is skipped
// by every role alike.
struct WorkItem {
  int mb, nb;   // row block (of the form's tile height) and 256-column block, relative to the window
  int col_off;  // first column of the slice inside the 256-column block
  int width;    // columns of the slice: 256, 128 or 64
};
__device__ __forceinline__ bool work_item(int w, int num_m, int num_n, int group, int split_from, int split, int cols, WorkItem& item) {
  int t = w, slice = 0;
  item.width = kBlockN;
  if (w >= split_from) {
    const int r = w - split_from;
    t = split_from + r / split;
    slice = r % split;
    item.width = kBlockN / split;
  }
  tile_coords(t, num_m, num_n, group, item.mb, item.nb);
  item.col_off = slice * item.width;
  return item.nb * kBlockN + item.col_off < cols;
}

__device__ __forceinline__ bool any_over_epilogue(bool flag) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %1, 0;\n\t"
      "barrier.cta.red.or.pred q, 3, 256, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(out)
      : "r"(static_cast<uint32_t>(flag))
      : "memory");
  return out != 0;
}

// kProfile adds the per-role cycle counters of GemmParams::profile; the production
// instantiation carries none of that code.
template <bool kPair, bool kProfile>
__global__ void __launch_bounds__(kThreads, 1)
abft_gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                     const __grid_constant__ GemmParams p) {
  using Cfg = Config<kPair>;
  // The swizzled operand tiles need a 1024-byte aligned base.  The declaration asks for it; should a toolchain not
  // honour that, the kernel reports an error instead of running with misplaced tiles.
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if ((smem_u32(smem_raw) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicExch(&p.report->status, 2);
    return;
  }
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + Cfg::kStages * kABytes;
  SharedTail& tail = *reinterpret_cast<SharedTail*>(smem + Cfg::kStages * Cfg::kStageBytes);
  volatile int* abort_flag = &tail.abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = kPair ? cluster_ctarank() : 0u;  // 0 = leader of the pair
  const int worker = kPair ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int workers = kPair ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  // the launch covers the window [row0, row0+rows) x [col0, col0+cols) of C; checksum indices stay global
  const int num_m = (p.rows + Cfg::kTileM - 1) / Cfg::kTileM;  // the last row block may reach past M: zero-filled like the columns
  const int num_n = (p.cols + kBlockN - 1) / kBlockN;  // the last column block may reach past N: the copies fill zeros there
  const int first_mb = p.row0 / Cfg::kTileM;
  const int first_nb = p.col0 / kBlockN;
  const int num_tiles = num_m * num_n;
  const int split_from = min(p.split_from, num_tiles);
  const int num_items = split_from + (num_tiles - split_from) * p.split;  // whole tiles, then column slices of the rest
  const int num_kb = (p.k + kBlockK - 1) / kBlockK;    // a short last K block is zero-filled by the copy engine
  const int kGroupM = max(1, p.group_rows / Cfg::kTileM);  // row blocks walked together (see GemmParams::group_rows)
  constexpr bool profiling = kProfile;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&tail.full[s], 1);
      mbar_init(&tail.empty[s], 1);
    }
    for (int a = 0; a < kAccumulators; ++a) {
      mbar_init(&tail.tmem_full[a], 1);
      mbar_init(&tail.tmem_empty[a], Cfg::kEmptyArrivals);
    }
    tail.abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) {
    if (kPair) {
      tmem_alloc_pair(&tail.tmem_base, kTmemColumns);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(&tail.tmem_base, kTmemColumns);
      tmem_relinquish();
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (kPair) {  // the peer's barriers must be initialised before anything remote touches them
    cluster_arrive();
    cluster_wait();
  }
  tcgen05_fence_after();
  const uint32_t tmem_base = tail.tmem_base;

  if (p.clear_counters != nullptr && blockIdx.x == 0 && threadIdx.x >= 64 && threadIdx.x < 72) p.clear_counters[threadIdx.x - 64] = 0;

  if (warp == 0) {
    // ------------------------------------------------------------- producer
    if (elect_one()) {
      int s = 0;
      uint32_t phase = 0;
      bool alive = true;
      long long waited = 0;
      for (int w = worker; w < num_items && alive; w += workers) {
        WorkItem item;
        if (!work_item(w, num_m, num_n, kGroupM, split_from, p.split, p.cols, item)) continue;
        const int mb = item.mb + first_mb, nb = item.nb + first_nb;
        const int a_row = mb * Cfg::kTileM + static_cast<int>(rank) * kBlockM;
        // Each CTA of a pair stages its half of the slice's B rows.  The copy always brings a full box (the byte count
        // of a stage does not change); for a narrow slice the rows behind the ones the MMA reads are simply not used.
        const int b_row = nb * kBlockN + item.col_off + static_cast<int>(rank) * (kPair ? item.width / 2 : 0);
        for (int kb = 0; kb < num_kb; ++kb) {
          const long long t0 = profiling ? clock64() : 0;
          if (!mbar_wait_bounded(&tail.empty[s], phase ^ 1, abort_flag, p.wait_timeout_ns)) {
            alive = false;
            break;
          }
          if (profiling) waited += clock64() - t0;
          if (kPair) {
            // both CTAs' bytes are counted on the leader's barrier
            if (rank == 0) mbar_arrive_expect_tx(&tail.full[s], Cfg::kExpectTx);
            const uint32_t leader_full = map_to_cta(smem_u32(&tail.full[s]), 0);
            tma_load_2d_pair(smem_a + s * kABytes, &tmap_a, leader_full, kb * kBlockK, a_row);
            tma_load_2d_pair(smem_b + s * Cfg::kBBytes, &tmap_b, leader_full, kb * kBlockK, b_row);
          } else {
            mbar_arrive_expect_tx(&tail.full[s], Cfg::kExpectTx);
            tma_load_2d(smem_a + s * kABytes, &tmap_a, &tail.full[s], kb * kBlockK, a_row);
            tma_load_2d(smem_b + s * Cfg::kBBytes, &tmap_b, &tail.full[s], kb * kBlockK, b_row);
          }
          if (++s == Cfg::kStages) {
            s = 0;
            phase ^= 1;
          }
        }
      }
      if (profiling) p.profile[blockIdx.x * 8 + 0] = waited;
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer (the leader only, in the pair form)
    if (rank == 0 && elect_one()) {
      int s = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool alive = true;
      long long wait_full = 0, wait_tmem = 0;
      const long long role_start = profiling ? clock64() : 0;
      for (int w = worker; w < num_items && alive; w += workers) {
        WorkItem item;
        if (!work_item(w, num_m, num_n, kGroupM, split_from, p.split, p.cols, item)) continue;
        const uint32_t idesc = make_idesc_e4m3_f32(Cfg::kTileM, item.width);
        long long t0 = profiling ? clock64() : 0;
        if (!mbar_wait_bounded(&tail.tmem_empty[acc], acc_phase ^ 1, abort_flag, p.wait_timeout_ns)) break;
        if (profiling) wait_tmem += clock64() - t0;
        tcgen05_fence_after();
        uint32_t tmem_d = tmem_base + acc * kBlockN;
        for (int kb = 0; kb < num_kb; ++kb) {
          t0 = profiling ? clock64() : 0;
          if (!mbar_wait_bounded(&tail.full[s], phase, abort_flag, p.wait_timeout_ns)) {
            alive = false;
            break;
          }
          if (profiling) wait_full += clock64() - t0;
          tcgen05_fence_after();
          uint64_t desc_a = make_smem_desc_sw128(smem_u32(smem_a + s * kABytes));
          uint64_t desc_b = make_smem_desc_sw128(smem_u32(smem_b + s * Cfg::kBBytes));
#pragma unroll
          for (int kk = 0; kk < kBlockK / kUmmaK; ++kk) {
            // advancing K by 32 bytes inside the 128-byte swizzle row = +2 in the (address >> 4) field
            if (kPair) {
              umma_f8f6f4_pair(tmem_d, desc_a + 2 * kk, desc_b + 2 * kk, idesc, (kb | kk) != 0 ? 1u : 0u);
            } else {
              umma_f8f6f4(tmem_d, desc_a + 2 * kk, desc_b + 2 * kk, idesc, (kb | kk) != 0 ? 1u : 0u);
            }
          }
          if (kPair) {  // the stage is free in both CTAs once these MMAs have read it
            umma_commit_pair(smem_u32(&tail.empty[s]));
            umma_commit_pair(map_to_cta(smem_u32(&tail.empty[s]), 1));
          } else {
            umma_commit(&tail.empty[s]);
          }
          if (++s == Cfg::kStages) {
            s = 0;
            phase ^= 1;
          }
        }
        if (alive) {
          if (kPair) {
            umma_commit_pair(smem_u32(&tail.tmem_full[acc]));
            umma_commit_pair(map_to_cta(smem_u32(&tail.tmem_full[acc]), 1));
          } else {
            umma_commit(&tail.tmem_full[acc]);
          }
        }
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
      if (profiling) {
        p.profile[blockIdx.x * 8 + 1] = wait_full;
        p.profile[blockIdx.x * 8 + 2] = wait_tmem;
        p.profile[blockIdx.x * 8 + 3] = clock64() - role_start;
      }
    }
  } else {
    // ------------------------------------------------------------- epilogue
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) belong to this warp
    const int set = (warp - 2) >> 2;  // which of the two epilogue sets: it takes the column groups g with g % 2 == set
    const int pair = quarter >> 1;  // which 64-row ABFT band of this CTA's 128 rows
    const int half = quarter & 1;   // which 32 rows of that band
    const int r_local = half * 32 + lane;
    const int tile_cols = (p.n + kGroupCols - 1) / kGroupCols;
    uint32_t groups_done = 0;  // groups this warp has checked so far
    int acc = 0;
    uint32_t acc_phase = 0;
    float max_ratio = 0.0f;
    long long epi_wait = 0, tiles_done = 0;
    const long long epi_start = profiling ? clock64() : 0;
    for (int w = worker; w < num_items; w += workers) {
      WorkItem item;
      if (!work_item(w, num_m, num_n, kGroupM, split_from, p.split, p.cols, item)) continue;
      const int mb = item.mb + first_mb, nb = item.nb + first_nb;
      const int col_base = nb * kBlockN + item.col_off;  // first column of C this item covers
      const int item_groups = item.width / kGroupCols;
      {
        // The cached expected checksums of this tile's (up to) four ABFT tiles are asked for while the main loop still runs:
        // with few tiles per CTA nothing else hides their latency.  Lines of row blocks or column groups past the
        // matrix are not touched.
        const int pf_row = (mb * Cfg::kTileM + static_cast<int>(rank) * kBlockM) / kGroupCols + pair;
        if (pf_row * kGroupCols < p.m) {
          const int pf_groups = min(item_groups, (p.n - col_base + kGroupCols - 1) / kGroupCols);
          for (int g = set; g < pf_groups; g += kEpilogueSets) {
            const size_t cache = static_cast<size_t>(pf_row * tile_cols + col_base / kGroupCols + g) * kGroupCols;
            prefetch_l1(p.expected_rows + cache + r_local);
            prefetch_l1(p.row_scales + cache + r_local);
            prefetch_l1(p.expected_cols + cache + 2 * lane);
            prefetch_l1(p.col_scales + cache + 2 * lane);
          }
        }
      }
      const long long t0 = profiling ? clock64() : 0;
      // one thread polls the barrier; the other 255 sleep in the hardware barrier below until it has seen the phase
      bool ok = true;
      if (warp == 2 && lane == 0) ok = mbar_wait_bounded(&tail.tmem_full[acc], acc_phase, abort_flag, p.wait_timeout_ns);
      if (any_over_epilogue(!ok)) break;
      if (profiling) {
        epi_wait += clock64() - t0;
        ++tiles_done;
      }
      tcgen05_fence_after();
      const int row0 = mb * Cfg::kTileM + static_cast<int>(rank) * kBlockM;  // first row of this CTA's part
      const int grow = row0 + quarter * 32 + lane;
      const int tile_row = row0 / kGroupCols + pair;
      // a 64-row band that starts past M holds nothing: its two warps only take part in handing the accumulator back
      const bool band_valid = tile_row * kGroupCols < p.m;
      const int valid_rows = min(kGroupCols, p.m - tile_row * kGroupCols);
      // 64-column groups of this tile that hold at least one column of C (src/s3:418-419)
      const int groups_here = min(item_groups, (p.n - col_base + kGroupCols - 1) / kGroupCols);
      // this set's groups: set, set + 2, ...; after its last one (or at once, when it has none) the set lets go of the accumulator
      const int last_group = groups_here - 1 - ((groups_here - 1 - set) & 1);  // largest g < groups_here with g % 2 == set; < set if none
      if (last_group < set) {
        tcgen05_fence_before();
        if (kPair) {
          mbar_arrive_cluster(map_to_cta(smem_u32(&tail.tmem_empty[acc]), 0));
        } else {
          mbar_arrive(&tail.tmem_empty[acc]);
        }
      }
#pragma unroll 1
      for (int g = set; g < groups_here; g += kEpilogueSets) {
        const int valid_cols = min(kGroupCols, p.n - col_base - g * kGroupCols);
        if (!band_valid) {  // uniform over the two warps of the band
          if (g == last_group) {
            tcgen05_fence_before();
            if (kPair) {
              mbar_arrive_cluster(map_to_cta(smem_u32(&tail.tmem_empty[acc]), 0));
            } else {
              mbar_arrive(&tail.tmem_empty[acc]);
            }
          }
          continue;
        }
        const int tile_id = tile_row * tile_cols + col_base / kGroupCols + g;
        const size_t cache = static_cast<size_t>(tile_id) * kGroupCols;
        const float exp_row = __ldg(p.expected_rows + cache + r_local);
        const float scale_row = __ldg(p.row_scales + cache + r_local);
        const float exp_col0 = __ldg(p.expected_cols + cache + lane);
        const float exp_col1 = __ldg(p.expected_cols + cache + 32 + lane);
        const float scale_col0 = __ldg(p.col_scales + cache + lane);
        const float scale_col1 = __ldg(p.col_scales + cache + 32 + lane);

        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * kBlockN + g * kGroupCols;
        // Column sums over this warp's 32 rows from a read in the fragment layout.  A test fault is added to the
        // accumulator below, in registers; the column it lands in gets its share here.
        float col_sum_a, col_sum_b;  // columns 2*lane and 2*lane+1
        tmem_column_sums_32x64(taddr, lane, col_sum_a, col_sum_b);
        float v[kGroupCols];
        tmem_ld_32x32b_x32(taddr, v);
        tmem_ld_32x32b_x32(taddr + 32, v + 32);
        tmem_wait_ld();
        if (g == last_group) {
          // the accumulator is now entirely in registers: hand it back to the MMA warp (of the leader)
          tcgen05_fence_before();
          if (kPair) {
            mbar_arrive_cluster(map_to_cta(smem_u32(&tail.tmem_empty[acc]), 0));
          } else {
            mbar_arrive(&tail.tmem_empty[acc]);
          }
        }

        // test hook: faults enter the accumulator values before any checksum
        if (p.faults.count > 0) {
#pragma unroll
          for (int f = 0; f < FT_MAX_FAULTS; ++f) {
            if (f < p.faults.count && p.faults.tile[f] == tile_id) {
              int fr = min(p.faults.row[f], valid_rows - 1);
              int fc = min(p.faults.col[f], valid_cols - 1);
              if (fr == r_local) {
#pragma unroll
                for (int c = 0; c < kGroupCols; ++c) {
                  if (c == fc) v[c] += p.faults.value[f];
                }
              }
              // the warp that holds the row also holds its share of the column's checksum: the lane with column fc adds the value
              if (fr / 32 == half && (fc >> 1) == lane) {
                if ((fc & 1) == 0) {
                  col_sum_a += p.faults.value[f];
                } else {
                  col_sum_b += p.faults.value[f];
                }
              }
            }
          }
        }

        // actual row checksum: ascending columns, one accumulator (src/s4:458-464)
        float row_sum = 0.0f;
#pragma unroll
        for (int c = 0; c < kGroupCols; ++c) row_sum += v[c];
        const float row_delta = exp_row - row_sum;
        const float row_thr = __fmaf_rn(p.rel_tol, fmaxf(1.0f, scale_row), p.abs_tol);
        const bool row_bad = fabsf(row_delta) > row_thr;
        if (!row_bad) max_ratio = fmaxf(max_ratio, __fdividef(fabsf(row_delta), row_thr));

        EpilogueScratch& sc = tail.scratch[set][pair];
        // the partner warp may still be reading the previous group's sums (shared memory has no room for a second copy
        // beside seven pipeline stages): meet it once before writing, once after
        if (groups_done != 0) asm volatile("bar.sync %0, 64;" ::"r"(1 + 3 * set + pair) : "memory");
        ++groups_done;
        *reinterpret_cast<float2*>(&sc.colpart[half][2 * lane]) = make_float2(col_sum_a, col_sum_b);
        const uint32_t row_mask = __ballot_sync(0xffffffffU, row_bad);
        const int first_lane = row_mask != 0 ? __ffs(row_mask) - 1 : 0;
        const float first_delta = __shfl_sync(0xffffffffU, row_delta, first_lane);
        if (lane == 0) {
          sc.rows[half].count = __popc(row_mask);
          sc.rows[half].first = row_mask != 0 ? half * 32 + first_lane : -1;
          sc.rows[half].delta = first_delta;
        }
        // 64-thread barrier of this set's band: ids 1, 2 (set 0) and 4, 5 (set 1); id 3 is the epilogue-wide one
        asm volatile("bar.sync %0, 64;" ::"r"(1 + 3 * set + pair) : "memory");

        // every warp of the pair checks all 64 columns (lane: columns lane, lane+32)
        const float col_sum0 = sc.colpart[0][lane] + sc.colpart[1][lane];
        const float col_sum1 = sc.colpart[0][32 + lane] + sc.colpart[1][32 + lane];
        const float col_delta0 = exp_col0 - col_sum0;
        const float col_delta1 = exp_col1 - col_sum1;
        const float col_thr0 = __fmaf_rn(p.rel_tol, fmaxf(1.0f, scale_col0), p.abs_tol);
        const float col_thr1 = __fmaf_rn(p.rel_tol, fmaxf(1.0f, scale_col1), p.abs_tol);
        const bool col_bad0 = fabsf(col_delta0) > col_thr0;
        const bool col_bad1 = fabsf(col_delta1) > col_thr1;
        if (!col_bad0) max_ratio = fmaxf(max_ratio, __fdividef(fabsf(col_delta0), col_thr0));
        if (!col_bad1) max_ratio = fmaxf(max_ratio, __fdividef(fabsf(col_delta1), col_thr1));
        const uint32_t col_mask0 = __ballot_sync(0xffffffffU, col_bad0);
        const uint32_t col_mask1 = __ballot_sync(0xffffffffU, col_bad1);
        const int bad_rows = sc.rows[0].count + sc.rows[1].count;
        const int bad_cols = __popc(col_mask0) + __popc(col_mask1);

        if ((bad_rows | bad_cols) != 0) {  // uniform over the pair of warps
          const int bad_row = sc.rows[0].count != 0 ? sc.rows[0].first : sc.rows[1].first;
          const float bad_row_delta = sc.rows[0].count != 0 ? sc.rows[0].delta : sc.rows[1].delta;
          int bad_col = -1;
          float bad_col_delta = 0.0f;
          {
            const float d0 = __shfl_sync(0xffffffffU, col_delta0, col_mask0 != 0 ? __ffs(col_mask0) - 1 : 0);
            const float d1 = __shfl_sync(0xffffffffU, col_delta1, col_mask1 != 0 ? __ffs(col_mask1) - 1 : 0);
            if (col_mask0 != 0) {
              bad_col = __ffs(col_mask0) - 1;
              bad_col_delta = d0;
            } else if (col_mask1 != 0) {
              bad_col = 32 + __ffs(col_mask1) - 1;
              bad_col_delta = d1;
            }
          }
          const bool correct = bad_rows == 1 && bad_cols == 1;
          if (correct && r_local == bad_row) {
            // src/s4:493-497: C[row,col] += 0.5 * (row_delta + col_delta), in registers
            const float both = bad_row_delta + bad_col_delta;
#pragma unroll
            for (int c = 0; c < kGroupCols; ++c) {
              if (c == bad_col) v[c] = __fmaf_rn(0.5f, both, v[c]);
            }
          }
          if (half == 0 && lane == 0) {
            atomicAdd(&p.report->bad_tiles, 1);
            if (correct) {
              atomicAdd(&p.report->corrected_tiles, 1);
            } else {
              atomicAdd(&p.report->multi_fault_tiles, 1);
            }
            int slot = atomicAdd(&p.report->record_count, 1);
            if (slot < FT_MAX_RECORDS) {
              ft_tile_record rec;
              rec.tile = tile_id;
              rec.bad_row_count = bad_rows;
              rec.bad_col_count = bad_cols;
              rec.bad_row = bad_rows != 0 ? bad_row : -1;
              rec.bad_col = bad_col;
              rec.row_delta = bad_rows != 0 ? bad_row_delta : 0.0f;
              rec.col_delta = bad_col_delta;
              rec.corrected = correct ? 1 : 0;
              p.report->records[slot] = rec;
            }
          }
        }

        // C is column-major [N,M]: for a fixed column the 32 lanes write 32 consecutive floats
        float* cptr = p.c + static_cast<size_t>(col_base + g * kGroupCols) * p.m + grow;
        if (valid_cols == kGroupCols && valid_rows == kGroupCols) {
#pragma unroll
          for (int c = 0; c < kGroupCols; ++c) __stcs(cptr + static_cast<size_t>(c) * p.m, v[c]);
        } else if (r_local < valid_rows) {
#pragma unroll
          for (int c = 0; c < kGroupCols; ++c) {
            if (c < valid_cols) __stcs(cptr + static_cast<size_t>(c) * p.m, v[c]);
          }
        }
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    // one atomic per warp for the clean-noise statistic
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) max_ratio = fmaxf(max_ratio, __shfl_xor_sync(0xffffffffU, max_ratio, off));
    if (lane == 0) atomicMax(&p.report->max_clean_ratio_bits, __float_as_int(max_ratio));
    if (profiling && warp == 2 && lane == 0) {
      p.profile[blockIdx.x * 8 + 4] = epi_wait;
      p.profile[blockIdx.x * 8 + 5] = clock64() - epi_start;
      p.profile[blockIdx.x * 8 + 6] = tiles_done;
    }
  }

  // ------------------------------------------------------------------- teardown
  tcgen05_fence_before();
  __syncthreads();
  if (tail.abort_flag != 0) {
    if (threadIdx.x == 0) atomicExch(&p.report->status, 1);
    // give copies and MMAs still in flight time to land before TMEM and smem go away
    for (int i = 0; i < 64; ++i) __nanosleep(20000);
    __syncthreads();
  }
  if (kPair) {  // neither CTA may leave while its partner can still reach its barriers or shared memory
    cluster_arrive();
    cluster_wait();
  }
  if (warp == 1) {
    tcgen05_fence_after();
    if (kPair) {
      tmem_dealloc_pair(tmem_base, kTmemColumns);
    } else {
      tmem_dealloc(tmem_base, kTmemColumns);
    }
  }
}

// The failure path of every kernel here, in isolation: a bounded wait that nothing satisfies, then the same status
// write as the teardown above.  One warp, no tensor memory, no copies, no MMA.
__global__ void selftest_wait_kernel(DeviceReport* report, unsigned long long limit_ns) {
  __shared__ uint64_t barrier;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&barrier, 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const bool ok = mbar_wait_bounded(&barrier, 0, &abort_flag, limit_ns);  // phase 0 never completes
    if (!ok && abort_flag != 0) atomicExch(&report->status, 1);
  }
}

cudaError_t launch_selftest_wait(DeviceReport* report, unsigned long long limit_ns, cudaStream_t stream) {
  selftest_wait_kernel<<<1, 32, 0, stream>>>(report, limit_ns);
  return cudaGetLastError();
}

int abft_gemm_smem_bytes(bool pair) { return pair ? smem_bytes<true>() : smem_bytes<false>(); }

template <bool kPair, bool kProfile>
static cudaError_t configure_one() {
  return cudaFuncSetAttribute(abft_gemm_fp8_kernel<kPair, kProfile>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes<kPair>());
}

cudaError_t configure_abft_gemm() {
  cudaError_t err = configure_one<false, false>();
  if (err == cudaSuccess) err = configure_one<true, false>();
  if (err == cudaSuccess) err = configure_one<false, true>();
  if (err == cudaSuccess) err = configure_one<true, true>();
  return err;
}

template <bool kProfile>
static cudaError_t launch_with(const CUtensorMap& tmap_a, const CUtensorMap& tmap_b, const GemmParams& params, int grid, bool pair,
                               cudaStream_t stream) {
  if (!pair) {
    abft_gemm_fp8_kernel<false, kProfile><<<grid, kThreads, smem_bytes<false>(), stream>>>(tmap_a, tmap_b, params);
    return cudaGetLastError();
  }
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeClusterDimension;
  attribute.val.clusterDim.x = 2;
  attribute.val.clusterDim.y = 1;
  attribute.val.clusterDim.z = 1;
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  config.blockDim = dim3(kThreads, 1, 1);
  config.dynamicSmemBytes = smem_bytes<true>();
  config.stream = stream;
  config.attrs = &attribute;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, abft_gemm_fp8_kernel<true, kProfile>, tmap_a, tmap_b, params);
}

cudaError_t launch_abft_gemm(const CUtensorMap& tmap_a, const CUtensorMap& tmap_b, const GemmParams& params, int grid, bool pair,
                             cudaStream_t stream) {
  return params.profile != nullptr ? launch_with<true>(tmap_a, tmap_b, params, grid, pair, stream)
                                   : launch_with<false>(tmap_a, tmap_b, params, grid, pair, stream);
}

}  // namespace ftg
