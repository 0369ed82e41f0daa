// Compares the oracle's E4M3 encoder/decoder with the conversion the reference
// uses, `__nv_fp8_e4m3(float)` from the CUDA toolkit's cuda_fp8.h (host path).
// TEST INFRASTRUCTURE ONLY.  Prints "e4m3 ok <count>" and exits 0 on agreement.
#include <cuda_fp8.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>

#include "ftq_oracle.h"

int main() {
  long checked = 0, bad = 0;
  // every 2^9-th float bit pattern plus a dense sweep around each representable value
  for (uint64_t bits = 0; bits <= 0xffffffffull; bits += 509) {
    uint32_t b32 = (uint32_t)bits;
    float x;
    std::memcpy(&x, &b32, 4);
    uint8_t mine = ftq_e4m3_from_float(x);
    uint8_t theirs = (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
    ++checked;
    if (mine != theirs && bad++ < 10) std::printf("encode mismatch x=%a mine=%02x theirs=%02x\n", x, mine, theirs);
  }
  for (int v = 0; v < 256; ++v) {
    float mine = ftq_e4m3_to_float((uint8_t)v);
    __nv_fp8_e4m3 t;
    t.__x = (__nv_fp8_storage_t)v;
    float theirs = (float)t;
    ++checked;
    if (!((std::isnan(mine) && std::isnan(theirs)) || mine == theirs)) {
      if (bad++ < 10) std::printf("decode mismatch v=%02x mine=%a theirs=%a\n", v, mine, theirs);
    }
    if (std::isnan(mine)) continue;
    // neighbours and midpoints: ties must go to even
    for (int d = -3; d <= 3; ++d) {
      for (int w = 0; w < 256; ++w) {
        float other = ftq_e4m3_to_float((uint8_t)w);
        if (std::isnan(other)) continue;
        float mid = 0.5f * (mine + other);
        uint32_t mb;
        std::memcpy(&mb, &mid, 4);
        mb += (uint32_t)d;
        float x;
        std::memcpy(&x, &mb, 4);
        uint8_t a = ftq_e4m3_from_float(x);
        uint8_t b = (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
        ++checked;
        if (a != b && bad++ < 10) std::printf("midpoint mismatch x=%a mine=%02x theirs=%02x\n", x, a, b);
      }
    }
  }
  if (bad) {
    std::printf("e4m3 FAILED %ld of %ld\n", bad, checked);
    return 1;
  }
  std::printf("e4m3 ok %ld\n", checked);
  return 0;
}
