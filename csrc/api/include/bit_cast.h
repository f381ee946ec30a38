// bit_cast<To>(from): the bytes of one trivially copyable value read as another type of the same size (the reference
// ships this helper as include/bit_cast.h; user code that includes it keeps compiling).
#pragma once
#include <cstring>
#include <type_traits>

template <typename To, typename From>
inline To bit_cast(const From& from) {
  static_assert(sizeof(To) == sizeof(From), "bit_cast needs types of one size");
  static_assert(std::is_trivially_copyable<To>::value && std::is_trivially_copyable<From>::value, "bit_cast needs trivially copyable types");
  To to;
  std::memcpy(&to, &from, sizeof(To));
  return to;
}
