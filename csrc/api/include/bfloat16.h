// bfloat16_t: a host-side bf16 value (the upper half of an IEEE float) for programs that fill or read the bf16 buffers of
// the layer-level API.  Same name and members as the reference's include/bfloat16.h:29-116, without its AVX-512 helpers:
// conversion from float rounds to nearest even and keeps NaN quiet, conversion to float is exact.
#pragma once
#include <cstdint>
#include <type_traits>

#include "bit_cast.h"

class bfloat16_t {
public:
  bfloat16_t() = default;
  bfloat16_t(float f) { *this = f; }
  constexpr bfloat16_t(uint16_t raw, bool) : bits_(raw) {}
  template <typename Int, typename = typename std::enable_if<std::is_integral<Int>::value>::type>
  bfloat16_t(Int i) { *this = static_cast<float>(i); }

  bfloat16_t& operator=(float f) {
    uint32_t u = bit_cast<uint32_t>(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) { bits_ = static_cast<uint16_t>((u >> 16) | 0x40u); return *this; }   // NaN stays NaN
    u += 0x7fffu + ((u >> 16) & 1u);
    bits_ = static_cast<uint16_t>(u >> 16);
    return *this;
  }
  template <typename Int, typename = typename std::enable_if<std::is_integral<Int>::value>::type>
  bfloat16_t& operator=(Int i) { return *this = static_cast<float>(i); }

  operator float() const { return bit_cast<float>(static_cast<uint32_t>(bits_) << 16); }
  bfloat16_t& operator+=(float a) { return *this = static_cast<float>(*this) + a; }
  uint16_t raw() const { return bits_; }

  static void cvt_float_to_bfloat16(const float* src, bfloat16_t* dst, int size) { for (int i = 0; i < size; ++i) dst[i] = src[i]; }
  static void cvt_bfloat16_to_float(const bfloat16_t* src, float* dst, int size) { for (int i = 0; i < size; ++i) dst[i] = src[i]; }
  static void float_add_bfloat16(const float* a, const bfloat16_t* b, float* dst, int size) {
    for (int i = 0; i < size; ++i) dst[i] = a[i] + static_cast<float>(b[i]);
  }

private:
  uint16_t bits_ = 0;
};

static_assert(sizeof(bfloat16_t) == 2, "bfloat16_t is two bytes");
