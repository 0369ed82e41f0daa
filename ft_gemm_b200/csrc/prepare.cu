// Expected-checksum cache and input generators.
//
// The cache is what the reference's S2-S4 programs compute once per (A, B) pair
// with cache_input_tile_checksums_kernel and cache_expected_tile_checksums_kernel
// (src/s4_cluster_multicast_abft_fp8_gemm.cu:194-294):
//   a_sums[I,k]  = sum over the 64 rows of band I of A[.,k]      (+ |.| version)
//   b_sums[J,k]  = sum over the 64 rows of band J of B[.,k]      (+ |.| version)
//   expected_rows[(I,J),r] = sum_k A[64I+r,k] * b_sums[J,k],  row_scales with |.|
//   expected_cols[(I,J),c] = sum_k a_sums[I,k] * B[64J+c,k],  col_scales with |.|
// The kernels here read A and B with 16-byte loads and keep the reference's
// summation order, so the cache is bit-identical to the reference's:
//   band sums: one FP32 accumulator per k, rows added in ascending order;
//   expected:  32 partial sums per checksum, partial l taking k = l, l+32, ...
//              in ascending order with one fma per step, then the pairwise tree
//              (l, l+16), (l, l+8), ..., (l, l+1) of a shuffle-down reduction.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels.h"

namespace ftg {

__device__ __forceinline__ uint32_t mix_u32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7feb352dU;
  x ^= x >> 15;
  x *= 0x846ca68bU;
  x ^= x >> 16;
  return x;
}

__device__ __forceinline__ float fp8_to_float(uint8_t v) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(v), __NV_E4M3);
  return __half2float(__half(h));
}

// ---------------------------------------------------------------------------
// generators
// ---------------------------------------------------------------------------
__global__ void generate_fp8_kernel(uint8_t* out, size_t count, uint32_t seed, int dist, float sigma, float post_scale) {
  size_t index = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (; index < count; index += stride) {
    float value;
    if (dist == 0) {
      uint32_t bits = mix_u32(seed + static_cast<uint32_t>(index));
      float unit = static_cast<float>(bits & 0x00ffffffU) / 16777216.0f;
      value = 2.0f * unit - 1.0f;
    } else {
      uint32_t i2 = 2u * static_cast<uint32_t>(index);
      uint32_t h1 = mix_u32(seed ^ i2);
      uint32_t h2 = mix_u32(seed ^ (i2 + 1u));
      float u1 = (static_cast<float>(h1 & 0x00ffffffU) + 1.0f) / 16777216.0f;
      float u2 = static_cast<float>(h2 & 0x00ffffffU) / 16777216.0f;
      float z = sqrtf(-2.0f * logf(u1)) * cosf(6.28318530717958647692f * u2);
      value = z * sigma * post_scale;
    }
    out[index] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(value, __NV_SATFINITE, __NV_E4M3));
  }
}

// ---------------------------------------------------------------------------
// band sums: x is [rows, k] FP8; one band = 64 consecutive rows.
// grid (ceil(k / 1024), bands), 256 threads: 64 chunks of 16 consecutive k x 4 quarters of 16 rows.
// ---------------------------------------------------------------------------
constexpr int kBandThreads = 128;

// A sum of 64 E4M3 values (multiples of 2^-9, at most 448 in magnitude) is a multiple of 2^-9 below 2^24 * 2^-9, so
// every partial sum is exact in FP32 and the order of the additions cannot change the result: the 64 rows of a band
// are summed as four quarters of 16 rows by four threads and combined through shared memory, which gives the bits of
// the reference's serial loop (src/s4:194-235) with four times as many loads in flight.
constexpr int kBandQuarters = 4;
constexpr int kBandChunks = 64;  // 16-byte chunks of k per CTA

__global__ void __launch_bounds__(kBandQuarters* kBandChunks) band_sums_kernel(const uint8_t* __restrict__ x, float* __restrict__ sums,
                                                                               float* __restrict__ mags, int rows, int k) {
  __shared__ float part[2][kBandQuarters - 1][kBandChunks][17];  // [sums | mags][quarter 1..3][chunk][16 + pad]
  const int band = blockIdx.y;
  const int chunk = threadIdx.x % kBandChunks, quarter = threadIdx.x / kBandChunks;
  const int k0 = (blockIdx.x * kBandChunks + chunk) * 16;
  const bool active = k0 < k;
  const int valid = min(64, rows - band * 64);  // the last band of B may be short (src/s3:203)
  float s[16], m[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) s[i] = m[i] = 0.0f;
  if (active) {
    const uint8_t* base = x + (static_cast<size_t>(band) * 64 + quarter * 16) * k + k0;
    const int my_rows = max(0, min(16, valid - quarter * 16));
#pragma unroll 16
    for (int row = 0; row < my_rows; ++row) {
      uint4 packed = __ldg(reinterpret_cast<const uint4*>(base + static_cast<size_t>(row) * k));
      uint32_t words[4] = {packed.x, packed.y, packed.z, packed.w};
#pragma unroll
      for (int w = 0; w < 4; ++w) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          __half2_raw pair = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(words[w] >> (16 * h)), __NV_E4M3);
          float2 f = __half22float2(__half2(pair));
          s[w * 4 + h * 2 + 0] += f.x;
          m[w * 4 + h * 2 + 0] += fabsf(f.x);
          s[w * 4 + h * 2 + 1] += f.y;
          m[w * 4 + h * 2 + 1] += fabsf(f.y);
        }
      }
    }
  }
  if (quarter > 0) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      part[0][quarter - 1][chunk][i] = s[i];
      part[1][quarter - 1][chunk][i] = m[i];
    }
  }
  __syncthreads();
  if (quarter == 0 && active) {
#pragma unroll
    for (int q = 0; q < kBandQuarters - 1; ++q) {
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        s[i] += part[0][q][chunk][i];
        m[i] += part[1][q][chunk][i];
      }
    }
    float4* so = reinterpret_cast<float4*>(sums + static_cast<size_t>(band) * k + k0);
    float4* mo = reinterpret_cast<float4*>(mags + static_cast<size_t>(band) * k + k0);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      so[q] = make_float4(s[4 * q], s[4 * q + 1], s[4 * q + 2], s[4 * q + 3]);
      mo[q] = make_float4(m[4 * q], m[4 * q + 1], m[4 * q + 2], m[4 * q + 3]);
    }
  }
}

// ---------------------------------------------------------------------------
// Producer of an FP8 operand fused with its band sums: src [rows, k] in FP32, BF16
// or FP16 is scaled, rounded to E4M3 (round to nearest even, saturating) and
// written to dst while the 64-row band sums and magnitudes of the ROUNDED values
// are accumulated in the order of band_sums_kernel (rows ascending, one
// accumulator per k), so the result equals a separate band-sum pass over dst bit
// for bit.  The reference reads A again for this (src/s4:194-235, 634-640).
// One thread owns 8 consecutive k; grid (ceil(k / 1024), rows / 64), 128 threads.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
  const float4 lo = __ldg(reinterpret_cast<const float4*>(p)), hi = __ldg(reinterpret_cast<const float4*>(p) + 1);
  v[0] = lo.x, v[1] = lo.y, v[2] = lo.z, v[3] = lo.w, v[4] = hi.x, v[5] = hi.y, v[6] = hi.z, v[7] = hi.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 raw = __ldg(reinterpret_cast<const uint4*>(p));
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {  // a BF16 is the upper half of an FP32
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ void load8(const __half* p, float (&v)[8]) {
  const uint4 raw = __ldg(reinterpret_cast<const uint4*>(p));
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

template <class S>
__global__ void __launch_bounds__(kBandThreads) quantize_band_sums_kernel(const S* __restrict__ src, uint8_t* __restrict__ dst,
                                                                          float* __restrict__ sums, float* __restrict__ mags,
                                                                          int rows, int k, float scale) {
  const int band = blockIdx.y;
  const int k0 = (blockIdx.x * kBandThreads + threadIdx.x) * 8;
  if (k0 >= k) return;
  const size_t base = static_cast<size_t>(band) * 64 * k + k0;
  float s[8], m[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) s[i] = m[i] = 0.0f;
  const int valid = min(64, rows - band * 64);
#pragma unroll 8
  for (int row = 0; row < valid; ++row) {
    float v[8];
    load8(src + base + static_cast<size_t>(row) * k, v);
    uint32_t packed[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
      const __nv_fp8x2_storage_t two = __nv_cvt_float2_to_fp8x2(make_float2(v[i] * scale, v[i + 1] * scale), __NV_SATFINITE, __NV_E4M3);
      packed[i >> 2] |= static_cast<uint32_t>(two) << (8 * (i & 3));
      const float2 f = __half22float2(__half2(__nv_cvt_fp8x2_to_halfraw2(two, __NV_E4M3)));
      s[i] += f.x;
      m[i] += fabsf(f.x);
      s[i + 1] += f.y;
      m[i + 1] += fabsf(f.y);
    }
    *reinterpret_cast<uint2*>(dst + base + static_cast<size_t>(row) * k) = make_uint2(packed[0], packed[1]);
  }
  float4* so = reinterpret_cast<float4*>(sums + static_cast<size_t>(band) * k + k0);
  float4* mo = reinterpret_cast<float4*>(mags + static_cast<size_t>(band) * k + k0);
  so[0] = make_float4(s[0], s[1], s[2], s[3]);
  so[1] = make_float4(s[4], s[5], s[6], s[7]);
  mo[0] = make_float4(m[0], m[1], m[2], m[3]);
  mo[1] = make_float4(m[4], m[5], m[6], m[7]);
}

// FP16 operands (attention): one thread owns 8 consecutive k of one band, rows in ascending order.  With a short k (a head
// dimension) `per` = k / 8 threads cover a band and a CTA takes kBandThreads / per bands, so that no thread is idle.
__global__ void __launch_bounds__(kBandThreads) band_sums_f16_kernel(const __half* __restrict__ x, float* __restrict__ sums,
                                                                     float* __restrict__ mags, int k, int per, int nbands) {
  int band = blockIdx.y * (kBandThreads / per) + threadIdx.x / per;
  int k0 = (blockIdx.x * per + threadIdx.x % per) * 8;
  if (k0 >= k || band >= nbands) return;
  const __half* base = x + static_cast<size_t>(band) * 64 * k + k0;
  float s[8], m[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) s[i] = m[i] = 0.0f;
#pragma unroll 16
  for (int row = 0; row < 64; ++row) {
    uint4 packed = __ldg(reinterpret_cast<const uint4*>(base + static_cast<size_t>(row) * k));
    const __half2* h2 = reinterpret_cast<const __half2*>(&packed);
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      float2 f = __half22float2(h2[w]);
      s[2 * w] += f.x;
      m[2 * w] += fabsf(f.x);
      s[2 * w + 1] += f.y;
      m[2 * w + 1] += fabsf(f.y);
    }
  }
  float4* so = reinterpret_cast<float4*>(sums + static_cast<size_t>(band) * k + k0);
  float4* mo = reinterpret_cast<float4*>(mags + static_cast<size_t>(band) * k + k0);
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    so[q] = make_float4(s[4 * q], s[4 * q + 1], s[4 * q + 2], s[4 * q + 3]);
    mo[q] = make_float4(m[4 * q], m[4 * q + 1], m[4 * q + 2], m[4 * q + 3]);
  }
}

// ---------------------------------------------------------------------------
// expected checksums.
// x is [rows, k] FP8 (A for the row checksums, B for the column checksums);
// band_sums / band_mags are the [nbands, k] sums of the OTHER operand.
// A CTA covers 64 rows of x (8 warps x 8 rows) and 8 bands; lane l owns the
// partial sums of k = l (mod 32).
// mode 0 (x = A): out index = ((row/64) * nbands + band) * 64 + row % 64
// mode 1 (x = B): out index = (band * (rows/64) + row/64) * 64 + row % 64
// ---------------------------------------------------------------------------
constexpr int kExpRows = 8;   // rows of x per warp
constexpr int kExpBands = 8;  // bands per CTA

template <int N>
__device__ __forceinline__ void transpose_reduce(float (&v)[N], int lane) {
  // After the call v[i], i < N/32, holds the sum over all 32 lanes of the
  // original v[(N/32) * lane + i].  Lane pairs are combined as (l, l^16), then
  // (l, l^8), ... (l, l^1): the same pairing as a shuffle-down tree read at lane 0.
  int n = N / 2;
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) {
    bool upper = (lane & off) != 0;
#pragma unroll
    for (int i = 0; i < n; ++i) {
      float send = upper ? v[i] : v[i + n];
      float keep = upper ? v[i + n] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffU, send, off);
    }
    n >>= 1;
  }
}

constexpr int kExpChunk = 128;  // k per staged slice

__device__ __forceinline__ float element_to_float(uint8_t v) { return fp8_to_float(v); }
__device__ __forceinline__ float element_to_float(__half v) { return __half2float(v); }

// copies `bytes` (0..16) from global memory and fills the rest of the 16 bytes with zeros
__device__ __forceinline__ void cp_async_16_zfill(void* smem_dst, const void* global_src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))),
               "l"(global_src), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// blockIdx.z walks independent problems of the same shape laid out back to back
// (one per attention head); the GEMM path launches with gridDim.z = 1.
template <class T>
__global__ void __launch_bounds__(256) expected_checksums_kernel(const T* __restrict__ x, const float* __restrict__ band_sums,
                                                                 const float* __restrict__ band_mags, float* __restrict__ expected,
                                                                 float* __restrict__ scales, int rows, int nbands, int k, int mode) {
  {
    const size_t z = blockIdx.z;
    const size_t tiles64 = static_cast<size_t>((rows + 63) >> 6) * nbands * 64;
    x += z * rows * k;
    band_sums += z * nbands * k;
    band_mags += z * nbands * k;
    expected += z * tiles64;
    scales += z * tiles64;
  }
  // Two-stage shared-memory ring over k: per stage the 64 x 128 slice of x and the
  // 8 x 128 slices of the band sums and magnitudes, filled with 16-byte cp.async
  // copies while the previous slice is consumed.
  __shared__ __align__(16) T sx[2][64][kExpChunk];
  __shared__ __align__(16) float sbs[2][kExpBands][kExpChunk];
  __shared__ __align__(16) float sbm[2][kExpBands][kExpChunk];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = blockIdx.x * 64 + warp * kExpRows;
  const int band0 = blockIdx.y * kExpBands;
  constexpr int kXChunksPerRow = kExpChunk * static_cast<int>(sizeof(T)) / 16;
  // Rows past the end of x repeat the last row (their results are stored as zeros below); k past the end is filled
  // with zeros, which leaves every partial sum unchanged.  k must be a multiple of 16 elements of T's 16-byte chunks.
  constexpr int kElemsPerChunk = 16 / static_cast<int>(sizeof(T));
  auto stage_copy = [&](int stage, int k0) {
#pragma unroll
    for (int i = threadIdx.x; i < 64 * kXChunksPerRow; i += 256) {
      const int r = i / kXChunksPerRow, ch = i % kXChunksPerRow;
      const int kk = k0 + ch * kElemsPerChunk;
      const int row = min(blockIdx.x * 64 + r, rows - 1);
      cp_async_16_zfill(reinterpret_cast<uint8_t*>(&sx[stage][r][0]) + ch * 16, x + static_cast<size_t>(row) * k + min(kk, k - kElemsPerChunk),
                        kk < k ? 16 : 0);
    }
    {
      const int j = threadIdx.x >> 5, ch = threadIdx.x & 31;  // 8 bands x 32 chunks of 4 floats
      const int kk = k0 + ch * 4;
      const size_t src = static_cast<size_t>(min(band0 + j, nbands - 1)) * k + min(kk, k - 4);
      cp_async_16_zfill(&sbs[stage][j][ch * 4], band_sums + src, kk < k ? 16 : 0);
      cp_async_16_zfill(&sbm[stage][j][ch * 4], band_mags + src, kk < k ? 16 : 0);
    }
    cp_async_commit();
  };
  // v[0..63]: expected partials [r*8+j]; v[64..127]: scale partials
  float v[2 * kExpRows * kExpBands];
#pragma unroll
  for (int i = 0; i < 2 * kExpRows * kExpBands; ++i) v[i] = 0.0f;

  const int chunks = (k + kExpChunk - 1) / kExpChunk;
  stage_copy(0, 0);
  for (int c = 0; c < chunks; ++c) {
    const int stage = c & 1;
    if (c + 1 < chunks) {
      stage_copy(stage ^ 1, (c + 1) * kExpChunk);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
#pragma unroll
    for (int it = 0; it < kExpChunk / 32; ++it) {  // lane l takes k = l (mod 32), ascending
      const int kk = it * 32 + lane;
      float av[kExpRows], sv[kExpBands], mv[kExpBands];
#pragma unroll
      for (int r = 0; r < kExpRows; ++r) av[r] = element_to_float(sx[stage][warp * kExpRows + r][kk]);
#pragma unroll
      for (int j = 0; j < kExpBands; ++j) {
        sv[j] = sbs[stage][j][kk];
        mv[j] = sbm[stage][j][kk];
      }
#pragma unroll
      for (int r = 0; r < kExpRows; ++r) {
        const float aabs = fabsf(av[r]);
#pragma unroll
        for (int j = 0; j < kExpBands; ++j) {
          v[r * kExpBands + j] = __fmaf_rn(av[r], sv[j], v[r * kExpBands + j]);
          v[64 + r * kExpBands + j] = __fmaf_rn(aabs, mv[j], v[64 + r * kExpBands + j]);
        }
      }
    }
    __syncthreads();  // the stage is refilled by the copy issued in the next iteration
  }
  transpose_reduce<2 * kExpRows * kExpBands>(v, lane);
  // lane holds original indices 4*lane + i
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int idx = 4 * lane + i;
    int which = idx >> 6;
    int r = (idx >> 3) & 7;
    int j = idx & 7;
    int band = band0 + j;
    if (band < nbands) {
      int row = row0 + r;
      size_t tile = mode == 0 ? static_cast<size_t>(row >> 6) * nbands + band
                              : static_cast<size_t>(band) * ((rows + 63) >> 6) + (row >> 6);
      size_t out = tile * 64 + (row & 63);
      const float value = row < rows ? v[i] : 0.0f;  // entries past the last valid column are stored as zeros (src/s4:284-293)
      if (which == 0) {
        expected[out] = value;
      } else {
        scales[out] = value;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// host launchers
// ---------------------------------------------------------------------------
cudaError_t launch_generate(void* out, size_t count, uint32_t seed, int dist, float sigma, float post_scale, cudaStream_t stream) {
  if (count == 0) return cudaSuccess;
  size_t blocks = (count + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  generate_fp8_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(static_cast<uint8_t*>(out), count, seed, dist, sigma,
                                                                         post_scale);
  return cudaGetLastError();
}

cudaError_t launch_band_sums(const void* x, float* sums, float* mags, int rows, int k, cudaStream_t stream) {
  dim3 grid((k / 16 + kBandChunks - 1) / kBandChunks, (rows + 63) / 64);
  band_sums_kernel<<<grid, kBandQuarters * kBandChunks, 0, stream>>>(static_cast<const uint8_t*>(x), sums, mags, rows, k);
  return cudaGetLastError();
}

cudaError_t launch_quantize_band_sums(const void* src, int src_dtype, void* dst, float* sums, float* mags, int rows, int k, float scale,
                                      cudaStream_t stream) {
  dim3 grid((k / 8 + kBandThreads - 1) / kBandThreads, (rows + 63) / 64);
  uint8_t* out = static_cast<uint8_t*>(dst);
  if (src_dtype == 0) {
    quantize_band_sums_kernel<float><<<grid, kBandThreads, 0, stream>>>(static_cast<const float*>(src), out, sums, mags, rows, k, scale);
  } else if (src_dtype == 1) {
    quantize_band_sums_kernel<__nv_bfloat16><<<grid, kBandThreads, 0, stream>>>(static_cast<const __nv_bfloat16*>(src), out, sums, mags, rows, k, scale);
  } else {
    quantize_band_sums_kernel<__half><<<grid, kBandThreads, 0, stream>>>(static_cast<const __half*>(src), out, sums, mags, rows, k, scale);
  }
  return cudaGetLastError();
}

cudaError_t launch_expected(const void* x, const float* band_sums, const float* band_mags, float* expected, float* scales, int rows,
                            int nbands, int k, int mode, cudaStream_t stream) {
  dim3 grid((rows + 63) / 64, (nbands + kExpBands - 1) / kExpBands);
  expected_checksums_kernel<uint8_t><<<grid, 256, 0, stream>>>(static_cast<const uint8_t*>(x), band_sums, band_mags, expected, scales,
                                                               rows, nbands, k, mode);
  return cudaGetLastError();
}

cudaError_t launch_band_sums_f16(const void* x, float* sums, float* mags, size_t rows, int k, cudaStream_t stream) {
  size_t bands = rows / 64;
  for (size_t first = 0; first < bands; first += 65535) {  // grid.y limit
    unsigned count = static_cast<unsigned>(bands - first < 65535 ? bands - first : 65535);
    const int chunks = k / 8;
    const int per = chunks < kBandThreads && kBandThreads % chunks == 0 ? chunks : kBandThreads;  // threads per band in a CTA
    const unsigned bands_per_cta = kBandThreads / per;
    dim3 grid((chunks + per - 1) / per, (count + bands_per_cta - 1) / bands_per_cta);
    band_sums_f16_kernel<<<grid, kBandThreads, 0, stream>>>(static_cast<const __half*>(x) + first * 64 * k, sums + first * k,
                                                            mags + first * k, k, per, static_cast<int>(count));
  }
  return cudaGetLastError();
}

cudaError_t launch_expected_f16(const void* x, const float* band_sums, const float* band_mags, float* expected, float* scales, int rows,
                                int nbands, int k, int mode, int batch, cudaStream_t stream) {
  dim3 grid(rows / 64, (nbands + kExpBands - 1) / kExpBands, batch);
  expected_checksums_kernel<__half><<<grid, 256, 0, stream>>>(static_cast<const __half*>(x), band_sums, band_mags, expected, scales, rows,
                                                              nbands, k, mode);
  return cudaGetLastError();
}

}  // namespace ftg
