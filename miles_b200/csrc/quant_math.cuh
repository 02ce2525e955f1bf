// Scalar conversions shared by the block-scaled quantisers (quant.cu) and the weight push (weight_push.cu):
// E8M0 power-of-two scales, E4M3 values and scales, the E2M1 grid.
#pragma once
#include <cuda_fp8.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace mb {
namespace qmath {

// Biased E8M0 exponent of the smallest power of two >= v (v > 0), 0 for v == 0.
__device__ __forceinline__ uint8_t e8m0_ceil(float v) {
  if (!(v > 0.f)) return 0;
  const uint32_t u = __float_as_uint(v);
  uint32_t e = (u >> 23) & 0xff;
  const uint32_t mant = u & 0x7fffff;
  if (mant != 0 && e != 0xfe) e += 1;
  if (e == 0 && mant != 0) e = 1;  // denormal input: round up to the smallest normal power
  return static_cast<uint8_t>(e);
}
__device__ __forceinline__ float e8m0_to_float(uint8_t e) {
  return e == 0 ? __uint_as_float(0x00400000u) /* 2^-127 */ : __uint_as_float(static_cast<uint32_t>(e) << 23);
}
__device__ __forceinline__ uint8_t to_e4m3(float x) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ float from_e4m3(uint8_t b) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(b), __NV_E4M3);
  return __half2float(__half(h));
}
// Round-to-nearest-even onto the E2M1 grid {0, .5, 1, 1.5, 2, 3, 4, 6}; returns the 4-bit code.
__device__ __forceinline__ uint8_t to_e2m1(float x) {
  const uint8_t sign = x < 0.f ? 8 : 0;
  const float a = fabsf(x);
  uint8_t code;
  if (a <= 0.25f) code = 0;
  else if (a < 0.75f) code = 1;
  else if (a <= 1.25f) code = 2;
  else if (a < 1.75f) code = 3;
  else if (a <= 2.5f) code = 4;
  else if (a < 3.5f) code = 5;
  else if (a <= 5.0f) code = 6;
  else code = 7;
  return sign | code;
}
__device__ __forceinline__ float from_e2m1(uint8_t c) {
  const float tbl[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  const float v = tbl[c & 7];
  return (c & 8) ? -v : v;
}

}  // namespace qmath
}  // namespace mb
