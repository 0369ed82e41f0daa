// Expected checksums on the tensor cores.
//
// expected_rows[(I,J),r] = sum_k A[64I+r,k] * b_sums[J,k] is a GEMM of A against
// the band sums of B, and the three other cache arrays are the same with |.| or
// with the operands swapped (src/s4_cluster_multicast_abft_fp8_gemm.cu:237-294).
// The reference and expected_checksums_kernel (prepare.cu) evaluate it with FP32
// FMAs on the CUDA cores, M*N*K/16 of them.  Here it runs as tcgen05.mma: the FP32
// band sums are written as a few planes in the operand's own format whose weighted
// sum is the band sum, X (A or B itself, straight from the caller's memory by TMA,
// no conversion) times the planes gives one FP32 accumulator per plane, each a sum
// of exact products, and the epilogue recombines them.
//   FP8 (the GEMM path): a sum of 64 E4M3 values is an integer multiple of 2^-9
//     below 2^24 * 2^-9; five signed radix-32 digits d in [-15, 16] (exact E4M3
//     integers) hold it exactly: sum = 2^-9 * (d0 + 32 d1 + ... + 32^4 d4); Horner.
//   FP16 (the attention path): the band sum times 2^-7 (so that 64 * 65504 cannot
//     overflow) is split into FP16 pieces hi + mid + lo (two pieces for the
//     magnitudes); what falls below the FP16 subnormal step is dropped, an absolute
//     error under 2^-17 per band-sum element.
// The scales need |X|: a helper warpgroup clears the sign bits of each staged X
// tile into a second shared-memory tile (same swizzled layout).
// The result equals the reference's value up to FP32 accumulation order, not bit
// for bit; the CUDA-core kernel remains for that.
//
// One CTA (448 threads) per SM, persistent over tiles of 128 rows of X x 32 bands:
//   warp 0      TMA producer: X tile 128 rows x 128 B, plane tiles of sums and of
//               magnitudes, 3 stages;
//   warp 1      one thread issues, per 32 B of K, X * Ws^T and |X| * Wm^T into two
//               column ranges of one TMEM accumulator (M128, N = planes x 32);
//   warps 2-9   the epilogue: two threads per row, 16 bands each; the accumulator is handed back as soon as it is in
//               registers, so the stores of tile i run beside the main loop of tile i+1;
//   warps 10-13 the |X| tiles of the main loop (a group of their own: with short K, as for the attention heads, the
//               epilogue of one tile must not hold up the |X| tiles of the next).
// `batch` independent problems of the same shape (attention heads) are laid out back
// to back in X, in the planes and in the outputs.
// Every wait is bounded; on expiry the kernel sets *status and leaves.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels.h"
#include "sm100_ptx.cuh"

namespace ftg {

namespace {

constexpr int kPmRows = 128;   // rows of X per tile
constexpr int kPmBands = 32;   // bands per tile
constexpr int kPmStages = 3;
constexpr int kPmXBytes = kPmRows * 128;  // 16 KiB: 128 rows x one 128-byte swizzle row of K
constexpr int kPmThreads = 448;
constexpr uint32_t kPmTmemColumns = 512;
constexpr uint64_t kPmTimeoutNs = 2000000000ull;

struct PmFp8 {
  static constexpr int kSumPlanes = 5, kMagPlanes = 5;
  static constexpr int kBlockKElems = 128;  // elements of K per 128-byte row
  static constexpr uint32_t kAbsMask = 0x7f7f7f7fu;
  static constexpr bool kHalf = false;
};
struct PmF16 {
  static constexpr int kSumPlanes = 3, kMagPlanes = 2;
  static constexpr int kBlockKElems = 64;
  static constexpr uint32_t kAbsMask = 0x7fff7fffu;
  static constexpr bool kHalf = true;
};

template <class Cfg>
struct PmLayout {
  static constexpr int kSumCols = Cfg::kSumPlanes * kPmBands, kMagCols = Cfg::kMagPlanes * kPmBands;
  static constexpr int kWsBytes = kSumCols * 128, kWmBytes = kMagCols * 128;
  static constexpr int kStageBytes = 2 * kPmXBytes + kWsBytes + kWmBytes;
  static constexpr int kAccCols = kSumCols + kMagCols;                      // TMEM columns of one accumulator
  static constexpr int kAccBuffers = 2 * kAccCols <= 512 ? 2 : 1;           // FP16: two (epilogue beside the next main loop); FP8: one
};

struct PmTail {
  uint64_t full[kPmStages];      // TMA data landed
  uint64_t abs_full[kPmStages];  // |X| written
  uint64_t empty[kPmStages];     // MMAs have read the stage
  uint64_t acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

template <class Cfg>
constexpr int pm_smem_bytes() {
  return kPmStages * PmLayout<Cfg>::kStageBytes + static_cast<int>(sizeof(PmTail));
}

template <int kCount>
__device__ __forceinline__ bool pm_any(bool flag, int barrier_id) {  // OR over the kCount threads of one helper group
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %1, 0;\n\t"
      "barrier.cta.red.or.pred q, %2, %3, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(out)
      : "r"(static_cast<uint32_t>(flag)), "r"(barrier_id), "n"(kCount)
      : "memory");
  return out != 0;
}

}  // namespace

// ---------------------------------------------------------------------------
// Planes.  sums / mags: [bands_total, k] FP32 (bands_total = batch * nbands).  Per
// problem the planes of band J lie at rows (J / 32) * (planes * 32) + p * 32 + J % 32
// of that problem's block of ceil(nbands / 32) * planes * 32 rows, each row k
// elements; bands past nbands (padding of the last group) are written as zeros.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) split_band_digits_kernel(const float* __restrict__ sums, const float* __restrict__ mags,
                                                                uint8_t* __restrict__ ws, uint8_t* __restrict__ wm, int nbands,
                                                                int k) {
  const int band = blockIdx.y;
  const int kk = blockIdx.x * 256 + threadIdx.x;
  if (kk >= k) return;
  constexpr int kCols = PmFp8::kSumPlanes * kPmBands;
  const size_t row0 = static_cast<size_t>(band / kPmBands) * kCols + band % kPmBands;
  const bool valid = band < nbands;
  const float values[2] = {valid ? sums[static_cast<size_t>(band) * k + kk] : 0.0f, valid ? mags[static_cast<size_t>(band) * k + kk] : 0.0f};
  uint8_t* const planes[2] = {ws, wm};
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    const float v = values[which];
    uint32_t t = static_cast<uint32_t>(fabsf(v) * 512.0f);  // exact: a multiple of 2^-9 below 2^15
    const float sign = v < 0.0f ? -1.0f : 1.0f;
#pragma unroll
    for (int d = 0; d < PmFp8::kSumPlanes; ++d) {
      int digit = static_cast<int>(t & 31u);
      t >>= 5;
      if (digit > 16) {  // signed digits keep every plane an exact E4M3 integer
        digit -= 32;
        t += 1;
      }
      planes[which][(row0 + static_cast<size_t>(d) * kPmBands) * k + kk] =
          static_cast<uint8_t>(__nv_cvt_float_to_fp8(sign * static_cast<float>(digit), __NV_SATFINITE, __NV_E4M3));
    }
  }
}

// grid (ceil(k / 256), padded bands per problem, batch)
__global__ void __launch_bounds__(256) split_band_pieces_f16_kernel(const float* __restrict__ sums, const float* __restrict__ mags,
                                                                    __half* __restrict__ ws, __half* __restrict__ wm, int nbands, int k) {
  const int band = blockIdx.y, problem = blockIdx.z;
  const int kk = blockIdx.x * 256 + threadIdx.x;
  if (kk >= k) return;
  const int groups = (nbands + kPmBands - 1) / kPmBands;
  const bool valid = band < nbands;
  const size_t src = (static_cast<size_t>(problem) * nbands + band) * k + kk;
  float s = valid ? sums[src] * 0.0078125f : 0.0f;  // 2^-7: exact, and 64 * 65504 * 2^-7 fits FP16
  float m = valid ? mags[src] * 0.0078125f : 0.0f;
  const size_t ws_row = (static_cast<size_t>(problem) * groups + band / kPmBands) * (PmF16::kSumPlanes * kPmBands) + band % kPmBands;
  const size_t wm_row = (static_cast<size_t>(problem) * groups + band / kPmBands) * (PmF16::kMagPlanes * kPmBands) + band % kPmBands;
#pragma unroll
  for (int p = 0; p < PmF16::kSumPlanes; ++p) {
    const __half piece = __float2half_rn(s);
    s -= __half2float(piece);  // exact
    ws[(ws_row + static_cast<size_t>(p) * kPmBands) * k + kk] = piece;
  }
#pragma unroll
  for (int p = 0; p < PmF16::kMagPlanes; ++p) {
    const __half piece = __float2half_rn(m);
    m -= __half2float(piece);
    wm[(wm_row + static_cast<size_t>(p) * kPmBands) * k + kk] = piece;
  }
}

// mode 0 (X = A, bands of B): out index = ((row / 64) * nbands + band) * 64 + row % 64
// mode 1 (X = B, bands of A): out index = (band * ceil(rows / 64) + row / 64) * 64 + row % 64
// per problem; problem p adds p * ceil(rows / 64) * nbands * 64.
template <class Cfg>
__global__ void __launch_bounds__(kPmThreads, 1)
expected_checksums_mma_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_ws,
                              const __grid_constant__ CUtensorMap tmap_wm, float* __restrict__ expected, float* __restrict__ scales,
                              int rows, int nbands, int k, int mode, int batch, int* __restrict__ status) {
  using L = PmLayout<Cfg>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  if ((smem_u32(smem_raw) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicExch(status, 2);
    return;
  }
  uint8_t* smem_x = smem_raw;
  uint8_t* smem_ax = smem_raw + kPmStages * kPmXBytes;
  uint8_t* smem_ws = smem_raw + 2 * kPmStages * kPmXBytes;
  uint8_t* smem_wm = smem_ws + kPmStages * L::kWsBytes;
  PmTail& tail = *reinterpret_cast<PmTail*>(smem_raw + kPmStages * L::kStageBytes);
  volatile int* abort_flag = &tail.abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row_blocks = (rows + kPmRows - 1) / kPmRows;
  const int groups = (nbands + kPmBands - 1) / kPmBands;
  const int tiles_per_problem = row_blocks * groups;
  const int num_tiles = tiles_per_problem * batch;
  const int num_kb = (k + Cfg::kBlockKElems - 1) / Cfg::kBlockKElems;
  const int worker = blockIdx.x, workers = gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPmStages; ++s) {
      mbar_init(&tail.full[s], 1);
      mbar_init(&tail.abs_full[s], 128);
      mbar_init(&tail.empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tail.acc_full[a], 1);
      mbar_init(&tail.acc_empty[a], 256);
    }
    tail.abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmap_x);
    prefetch_tensormap(&tmap_ws);
    prefetch_tensormap(&tmap_wm);
  }
  if (warp == 1) {
    tmem_alloc(&tail.tmem_base, kPmTmemColumns);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = tail.tmem_base;

  if (warp == 0) {
    if (elect_one()) {
      // ------------------------------------------------------------- producer
      int s = 0;
      uint32_t phase = 0;
      bool alive = true;
      for (int t = worker; t < num_tiles && alive; t += workers) {
        const int problem = t / tiles_per_problem, local = t % tiles_per_problem;
        const int group = local % groups, row_block = local / groups;  // neighbouring CTAs share the X tile in L2
        const int x_row = problem * rows + row_block * kPmRows;         // batch > 1 only with rows a multiple of 128
        const int w_group = problem * groups + group;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&tail.empty[s], phase ^ 1, abort_flag, kPmTimeoutNs)) {
            alive = false;
            break;
          }
          mbar_arrive_expect_tx(&tail.full[s], kPmXBytes + L::kWsBytes + L::kWmBytes);
          tma_load_2d(smem_x + s * kPmXBytes, &tmap_x, &tail.full[s], kb * Cfg::kBlockKElems, x_row);
          tma_load_2d(smem_ws + s * L::kWsBytes, &tmap_ws, &tail.full[s], kb * Cfg::kBlockKElems, w_group * L::kSumCols);
          tma_load_2d(smem_wm + s * L::kWmBytes, &tmap_wm, &tail.full[s], kb * Cfg::kBlockKElems, w_group * L::kMagCols);
          if (++s == kPmStages) {
            s = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      // ------------------------------------------------------------- MMA issuer
      constexpr uint32_t idesc_s = Cfg::kHalf ? make_idesc_f16_f32(kPmRows, L::kSumCols) : make_idesc_e4m3_f32(kPmRows, L::kSumCols);
      constexpr uint32_t idesc_m = Cfg::kHalf ? make_idesc_f16_f32(kPmRows, L::kMagCols) : make_idesc_e4m3_f32(kPmRows, L::kMagCols);
      int s = 0;
      uint32_t phase = 0;
      int done = 0;  // tiles issued by this CTA: accumulator done % kAccBuffers, in its use number done / kAccBuffers
      bool alive = true;
      for (int t = worker; t < num_tiles && alive; t += workers, ++done) {
        const int acc = done % L::kAccBuffers;
        const uint32_t acc_phase = (done / L::kAccBuffers) & 1;
        const uint32_t tmem_acc = tmem_base + acc * L::kAccCols;
        if (!mbar_wait_bounded(&tail.acc_empty[acc], acc_phase ^ 1, abort_flag, kPmTimeoutNs)) break;
        tcgen05_fence_after();
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&tail.full[s], phase, abort_flag, kPmTimeoutNs) ||
              !mbar_wait_bounded(&tail.abs_full[s], phase, abort_flag, kPmTimeoutNs)) {
            alive = false;
            break;
          }
          tcgen05_fence_after();
          const uint64_t desc_x = make_smem_desc_sw128(smem_u32(smem_x + s * kPmXBytes));
          const uint64_t desc_ax = make_smem_desc_sw128(smem_u32(smem_ax + s * kPmXBytes));
          const uint64_t desc_ws = make_smem_desc_sw128(smem_u32(smem_ws + s * L::kWsBytes));
          const uint64_t desc_wm = make_smem_desc_sw128(smem_u32(smem_wm + s * L::kWmBytes));
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {  // one MMA consumes 32 bytes of K; +32 bytes inside the swizzle row = +2 in the address field
            const uint32_t accumulate = (kb | kk) != 0 ? 1u : 0u;
            if (Cfg::kHalf) {
              umma_f16(tmem_acc, desc_x + 2 * kk, desc_ws + 2 * kk, idesc_s, accumulate);
              umma_f16(tmem_acc + L::kSumCols, desc_ax + 2 * kk, desc_wm + 2 * kk, idesc_m, accumulate);
            } else {
              umma_f8f6f4(tmem_acc, desc_x + 2 * kk, desc_ws + 2 * kk, idesc_s, accumulate);
              umma_f8f6f4(tmem_acc + L::kSumCols, desc_ax + 2 * kk, desc_wm + 2 * kk, idesc_m, accumulate);
            }
          }
          umma_commit(&tail.empty[s]);
          if (++s == kPmStages) {
            s = 0;
            phase ^= 1;
          }
        }
        if (alive) umma_commit(&tail.acc_full[acc]);
      }
    }
  } else if (warp >= 10) {
    // ------------------------------------------------------------- |X| tiles
    const int tid = threadIdx.x - 320;  // 0..127
    int s = 0;
    uint32_t phase = 0;
    bool alive = true;
    for (int t = worker; t < num_tiles && alive; t += workers) {
      for (int kb = 0; kb < num_kb; ++kb) {
        bool ok = true;
        if (tid == 0) ok = mbar_wait_bounded(&tail.full[s], phase, abort_flag, kPmTimeoutNs);
        if (pm_any<128>(!ok, 2)) {  // uniform over the 128 threads
          alive = false;
          break;
        }
        const uint4* src = reinterpret_cast<const uint4*>(smem_x + s * kPmXBytes);
        uint4* dst = reinterpret_cast<uint4*>(smem_ax + s * kPmXBytes);
#pragma unroll
        for (int c = 0; c < kPmXBytes / 16 / 128; ++c) {  // the swizzle permutes whole 16-byte chunks: clearing sign bits keeps the layout
          uint4 v = src[c * 128 + tid];
          v.x &= Cfg::kAbsMask;
          v.y &= Cfg::kAbsMask;
          v.z &= Cfg::kAbsMask;
          v.w &= Cfg::kAbsMask;
          dst[c * 128 + tid] = v;
        }
        fence_proxy_async_shared();
        mbar_arrive(&tail.abs_full[s]);
        if (++s == kPmStages) {
          s = 0;
          phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------- epilogue
    const int tid = threadIdx.x - 64;  // 0..255
    const int half = (warp - 2) >> 2;  // which 16 of the tile's 32 bands this thread recombines and stores
    const int quarter = warp & 3;      // TMEM lanes [32 * quarter, +32) belong to this warp
    const int row_in_block = quarter * 32 + lane;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const int rows64 = (rows + 63) >> 6;
    int done = 0;
    for (int t = worker; t < num_tiles; t += workers, ++done) {
      const int problem = t / tiles_per_problem, local = t % tiles_per_problem;
      const int group = local % groups, row_block = local / groups;
      const int acc = done % L::kAccBuffers;
      const uint32_t acc_phase = (done / L::kAccBuffers) & 1;
      bool ok = true;
      if (tid == 0) ok = mbar_wait_bounded(&tail.acc_full[acc], acc_phase, abort_flag, kPmTimeoutNs);
      if (pm_any<256>(!ok, 1)) break;
      tcgen05_fence_after();
      // recombination, last plane first: FP8 digits by Horner (value = 2^-9 * sum_d 32^d * acc_d), FP16 pieces lo + mid + hi
      float e[2][16];  // [sums | magnitudes][band]
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const int planes = which == 0 ? Cfg::kSumPlanes : Cfg::kMagPlanes;
        {
          const uint32_t base = lane_addr + acc * L::kAccCols + which * L::kSumCols + half * 16;
          tmem_ld_32x32b_x16(base + (planes - 1) * kPmBands, e[which]);
          tmem_wait_ld();
#pragma unroll
          for (int d = planes - 2; d >= 0; --d) {
            float a[16];
            tmem_ld_32x32b_x16(base + d * kPmBands, a);
            tmem_wait_ld();
#pragma unroll
            for (int b = 0; b < 16; ++b) e[which][b] = Cfg::kHalf ? e[which][b] + a[b] : __fmaf_rn(e[which][b], 32.0f, a[b]);
          }
        }
      }
      tcgen05_fence_before();
      mbar_arrive(&tail.acc_empty[acc]);  // the accumulators are in registers: this buffer may take another tile
      const float unit = Cfg::kHalf ? 128.0f : 0.001953125f;  // undo the 2^-7 of the FP16 pieces / the 2^9 of the FP8 digits
      const int row = row_block * kPmRows + row_in_block;
      if (row < rows64 * 64) {  // rows of the last 64-row group past `rows` were zero-filled by the copy: their checksums are zeros
        const size_t problem_base = static_cast<size_t>(problem) * rows64 * nbands * 64;
        // consecutive bands of one row lie a fixed distance apart in both layouts
        const int band0 = group * kPmBands + half * 16;
        const size_t first = mode == 0 ? static_cast<size_t>(row >> 6) * nbands + band0 : static_cast<size_t>(band0) * rows64 + (row >> 6);
        const size_t step = mode == 0 ? 64 : static_cast<size_t>(rows64) * 64;
        float* out_e = expected + problem_base + first * 64 + (row & 63);
        float* out_s = scales + problem_base + first * 64 + (row & 63);
#pragma unroll
        for (int b = 0; b < 16; ++b) {
          if (band0 + b < nbands) {
            out_e[b * step] = e[0][b] * unit;
            out_s[b * step] = e[1][b] * unit;
          }
        }
      }
    }
  }

  // ------------------------------------------------------------------- teardown
  tcgen05_fence_before();
  __syncthreads();
  if (tail.abort_flag != 0) {
    if (threadIdx.x == 0) atomicExch(status, 1);
    for (int i = 0; i < 64; ++i) __nanosleep(20000);  // copies and MMAs still in flight land before TMEM and smem go away
    __syncthreads();
  }
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, kPmTmemColumns);
  }
}

cudaError_t configure_prepare_mma() {
  cudaError_t err = cudaFuncSetAttribute(expected_checksums_mma_kernel<PmFp8>, cudaFuncAttributeMaxDynamicSharedMemorySize, pm_smem_bytes<PmFp8>());
  if (err != cudaSuccess) return err;
  return cudaFuncSetAttribute(expected_checksums_mma_kernel<PmF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, pm_smem_bytes<PmF16>());
}

int prepare_mma_plane_rows(int nbands) { return (nbands + kPmBands - 1) / kPmBands * (PmFp8::kSumPlanes * kPmBands); }
size_t prepare_mma_plane_bytes(int nbands, int k) { return static_cast<size_t>(prepare_mma_plane_rows(nbands)) * k; }
int prepare_mma_plane_rows_f16(int nbands, int which) {
  return (nbands + kPmBands - 1) / kPmBands * ((which == 0 ? PmF16::kSumPlanes : PmF16::kMagPlanes) * kPmBands);
}

cudaError_t launch_split_band_digits(const float* sums, const float* mags, void* ws, void* wm, int nbands, int k, cudaStream_t stream) {
  const int padded = (nbands + kPmBands - 1) / kPmBands * kPmBands;
  dim3 grid((k + 255) / 256, padded);
  split_band_digits_kernel<<<grid, 256, 0, stream>>>(sums, mags, static_cast<uint8_t*>(ws), static_cast<uint8_t*>(wm), nbands, k);
  return cudaGetLastError();
}

cudaError_t launch_split_band_pieces_f16(const float* sums, const float* mags, void* ws, void* wm, int nbands, int k, int batch,
                                         cudaStream_t stream) {
  const int padded = (nbands + kPmBands - 1) / kPmBands * kPmBands;
  for (int first = 0; first < batch; first += 65535) {  // grid.z limit
    const int count = batch - first < 65535 ? batch - first : 65535;
    const int groups = padded / kPmBands;
    dim3 grid((k + 255) / 256, padded, count);
    split_band_pieces_f16_kernel<<<grid, 256, 0, stream>>>(
        sums + static_cast<size_t>(first) * nbands * k, mags + static_cast<size_t>(first) * nbands * k,
        static_cast<__half*>(ws) + static_cast<size_t>(first) * groups * PmF16::kSumPlanes * kPmBands * k,
        static_cast<__half*>(wm) + static_cast<size_t>(first) * groups * PmF16::kMagPlanes * kPmBands * k, nbands, k);
  }
  return cudaGetLastError();
}

cudaError_t launch_expected_mma(const CUtensorMap& tmap_x, const CUtensorMap& tmap_ws, const CUtensorMap& tmap_wm, float* expected,
                                float* scales, int rows, int nbands, int k, int mode, int sm_count, int* status, cudaStream_t stream) {
  const int tiles = ((rows + kPmRows - 1) / kPmRows) * ((nbands + kPmBands - 1) / kPmBands);
  const int grid = tiles < sm_count ? tiles : sm_count;
  expected_checksums_mma_kernel<PmFp8><<<grid, kPmThreads, pm_smem_bytes<PmFp8>(), stream>>>(tmap_x, tmap_ws, tmap_wm, expected, scales, rows,
                                                                                            nbands, k, mode, 1, status);
  return cudaGetLastError();
}

cudaError_t launch_expected_mma_f16(const CUtensorMap& tmap_x, const CUtensorMap& tmap_ws, const CUtensorMap& tmap_wm, float* expected,
                                    float* scales, int rows, int nbands, int k, int mode, int batch, int sm_count, int* status,
                                    cudaStream_t stream) {
  const long long tiles = static_cast<long long>((rows + kPmRows - 1) / kPmRows) * ((nbands + kPmBands - 1) / kPmBands) * batch;
  const int grid = tiles < sm_count ? static_cast<int>(tiles) : sm_count;
  expected_checksums_mma_kernel<PmF16><<<grid, kPmThreads, pm_smem_bytes<PmF16>(), stream>>>(tmap_x, tmap_ws, tmap_wm, expected, scales, rows,
                                                                                            nbands, k, mode, batch, status);
  return cudaGetLastError();
}

}  // namespace ftg
