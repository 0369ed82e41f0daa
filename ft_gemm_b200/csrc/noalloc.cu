// Expected-checksum preparation for callers that must not allocate.
//
// ft_gemm_fp8_abft_prepare() owns its cache and therefore calls cudaMalloc.  Some
// users of this library cannot afford that at the point where they need fresh
// checksums: an inference server recomputes them every time the activation
// matrix A changes, from inside a step loop in which the framework's caching
// allocator has already reserved the device's memory (a cudaMalloc there fails
// or forces the pool to be trimmed) and in which cudaMalloc's device-wide
// synchronisation would stall every other stream.  For them this file offers one
// entry point that allocates nothing: the caller passes the four output arrays,
// and the intermediate band sums live in a fixed array that is part of the
// library image.
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "kernels.h"

namespace {

// Band sums of A and B: a_sums, a_magnitudes [M/64, K] then b_sums,
// b_magnitudes [N/64, K].  Every GPU that loads the library holds these 16 MiB
// until the process exits.
constexpr size_t kScratchFloats = FT_NOALLOC_MAX_SCRATCH_BYTES / sizeof(float);
static __device__ __align__(256) float g_band_scratch[kScratchFloats];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
float* g_scratch_address[kMaxDevices] = {};  // device address of g_band_scratch on each device, filled at set-up

}  // namespace

namespace ftg {
int noalloc_fail(int code, const char* fmt, ...);
}

extern "C" int ft_gemm_fp8_abft_expected_noalloc(const void* a, const void* b, int m, int n, int k, float* expected_rows,
                                                 float* expected_cols, float* row_scales, float* col_scales, void* stream_ptr) {
  using namespace ftg;
  if (a == nullptr || b == nullptr || expected_rows == nullptr || expected_cols == nullptr || row_scales == nullptr ||
      col_scales == nullptr) {
    return noalloc_fail(FT_ERR_INVALID, "null operand or output pointer");
  }
  if (m <= 0 || n <= 0 || k <= 0 || k % 16 != 0) {
    return noalloc_fail(FT_ERR_INVALID, "Invalid options. Require K%%16==0 and positive shape.");
  }
  if ((reinterpret_cast<uintptr_t>(a) & 15) != 0 || (reinterpret_cast<uintptr_t>(b) & 15) != 0) {
    return noalloc_fail(FT_ERR_INVALID, "A and B must be 16-byte aligned");
  }
  const size_t a_meta = static_cast<size_t>((m + 63) / 64) * k, b_meta = static_cast<size_t>((n + 63) / 64) * k;
  const size_t needed = 2 * (a_meta + b_meta);
  if (needed > kScratchFloats) {
    return noalloc_fail(FT_ERR_INVALID,
                        "shape needs %zu bytes of band-sum scratch, the built-in array holds %zu: (M/64 + N/64) * K must not "
                        "exceed %zu; use ft_gemm_fp8_abft_prepare for larger shapes",
                        needed * sizeof(float), kScratchFloats * sizeof(float), kScratchFloats / 2);
  }
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return noalloc_fail(FT_ERR_CUDA, "cudaGetDevice failed: %s", cudaGetErrorString(err));
  if (device < 0 || device >= kMaxDevices) return noalloc_fail(FT_ERR_INVALID, "device index %d is out of range", device);
  float* scratch = nullptr;
  {
    // Set-up, once per device, with that device current: in host code the name
    // g_band_scratch is only a handle for the symbol, so ask the runtime for the
    // array's address on this device and hand that address to the kernels.
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_address[device] == nullptr) {
      void* address = nullptr;
      err = cudaGetSymbolAddress(&address, g_band_scratch);
      if (err != cudaSuccess || address == nullptr) {
        return noalloc_fail(FT_ERR_CUDA, "cudaGetSymbolAddress(band scratch) failed on device %d: %s", device,
                            cudaGetErrorString(err));
      }
      g_scratch_address[device] = static_cast<float*>(address);
    }
    scratch = g_scratch_address[device];
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  float* a_sums = scratch;
  float* a_mags = a_sums + a_meta;
  float* b_sums = a_mags + a_meta;
  float* b_mags = b_sums + b_meta;
  // Every element of the used part of the scratch is overwritten by the two
  // band-sum launches before it is read, so nothing has to be cleared first.
  err = launch_band_sums(a, a_sums, a_mags, m, k, stream);
  if (err == cudaSuccess) err = launch_band_sums(b, b_sums, b_mags, n, k, stream);
  if (err == cudaSuccess) err = launch_expected(a, b_sums, b_mags, expected_rows, row_scales, m, (n + 63) / 64, k, 0, stream);
  if (err == cudaSuccess) err = launch_expected(b, a_sums, a_mags, expected_cols, col_scales, n, (m + 63) / 64, k, 1, stream);
  if (err != cudaSuccess) return noalloc_fail(FT_ERR_CUDA, "launching the prepare kernels failed: %s", cudaGetErrorString(err));
  return FT_OK;
}
