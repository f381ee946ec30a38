// A program written against the reference's header names (include/xfastertransformer.h, bfloat16.h) compiles with
// -I csrc/api/include; the bf16 value type converts as documented (round to nearest even, exact the other way).
#include "xfastertransformer.h"
#include "bfloat16.h"
#include <cstdio>
int main() {
  bfloat16_t a(1.00390625f), b(3);   // 1 + 2^-8 rounds to even -> 1.0
  float f[2] = {0.1f, -2.5f}; bfloat16_t h[2]; bfloat16_t::cvt_float_to_bfloat16(f, h, 2);
  float g[2]; bfloat16_t::cvt_bfloat16_to_float(h, g, 2);
  std::printf("%g %g %g %g %d\n", (float)a, (float)b, g[0], g[1], (int)sizeof(SearcherConfig) > 0);
  xft::DataType d = xft::DataType::bf16; (void)d;
  return ((float)a == 1.0f && (float)b == 3.0f && g[1] == -2.5f) ? 0 : 1;
}
