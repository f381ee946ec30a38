// Numeric types of the checkpoint files on the host (reference: include/bfloat16.h, src/common/float16.h — software
// conversions used while loading).  On the device the CUDA types (__nv_bfloat16, __half, __nv_fp8_e4m3) are used directly.
// File element codes: 0 fp32, 1 fp16, 2 bf16.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cstring>

namespace xft {

inline size_t dtypeSize(int dt) { return dt == 0 ? 4 : 2; }

inline float halfToFloat(uint16_t h) {
  uint32_t s = (h >> 15) & 1, e = (h >> 10) & 31, m = h & 1023, u;
  if (e == 0) {
    if (m == 0) u = s << 31;
    else { e = 127 - 15 + 1; while (!(m & 1024)) { m <<= 1; --e; } m &= 1023; u = (s << 31) | (e << 23) | (m << 13); }
  } else if (e == 31) u = (s << 31) | 0x7f800000u | (m << 13);
  else u = (s << 31) | ((e + 112) << 23) | (m << 13);
  float f; std::memcpy(&f, &u, 4); return f;
}

// round to nearest even; overflow gives infinity, values below the smallest subnormal give zero
inline uint16_t floatToHalf(float f) {
  uint32_t u; std::memcpy(&u, &f, 4);
  const uint32_t s = (u >> 16) & 0x8000u;
  const uint32_t a = u & 0x7fffffffu;
  if (a >= 0x7f800000u) return (uint16_t)(s | 0x7c00u | (a > 0x7f800000u ? 0x200u : 0u));    // inf / nan
  if (a >= 0x477ff000u) return (uint16_t)(s | 0x7c00u);                                      // rounds to >= 65520: inf
  if (a < 0x33000001u) return (uint16_t)s;                                                   // below half of 2^-24
  int32_t e = (int32_t)(a >> 23) - 127;
  uint32_t m = (a & 0x7fffffu) | 0x800000u;                                                  // 24-bit significand
  int shift = e < -14 ? 13 + (-14 - e) : 13;                                                 // bits dropped
  uint32_t q = m >> shift, rem = m & ((1u << shift) - 1), half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1u))) ++q;
  // normal: q has its hidden bit at position 10 (a carry moves it to 11, which bumps the exponent by itself)
  const uint32_t h = e < -14 ? q : (((uint32_t)(e + 15) << 10) + (q - 0x400u));
  return (uint16_t)(s | h);
}

inline uint16_t floatToBf16(float f) {
  uint32_t u; std::memcpy(&u, &f, 4);
  u += 0x7fffu + ((u >> 16) & 1);
  return (uint16_t)(u >> 16);
}

inline float bf16ToFloat(uint16_t h) { uint32_t u = (uint32_t)h << 16; float f; std::memcpy(&f, &u, 4); return f; }

inline float elemToFloat(const char* p, int dt, size_t i) {
  if (dt == 0) { float f; std::memcpy(&f, p + 4 * i, 4); return f; }
  uint16_t h; std::memcpy(&h, p + 2 * i, 2);
  return dt == 1 ? halfToFloat(h) : bf16ToFloat(h);
}

}  // namespace xft
