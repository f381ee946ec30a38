#include "gptq.h"

#include <cstring>

namespace xft {
namespace {
inline int codeAt(const uint8_t* file, int outF, bool uint4, int i, int o) {
  if (!uint4) return (int)(int8_t)file[(size_t)i * outF + o];
  const uint8_t b = file[(size_t)i * (outF / 2) + o / 2];
  return (o & 1) ? (b >> 4) : (b & 15);
}
}  // namespace

void gptqRepack(const uint8_t* file, int inF, int outF, bool uint4, int in0, int in1, int out0, int out1, int pitch,
                uint8_t* dst) {
  (void)inF;
  const int K = in1 - in0;
  for (int o = out0; o < out1; ++o) {
    uint8_t* row = dst + (size_t)(o - out0) * pitch;
    std::memset(row, 0, (size_t)pitch);
    if (!uint4) {
      for (int i = 0; i < K; ++i) row[i] = (uint8_t)codeAt(file, outF, false, in0 + i, o);
    } else {
      for (int i = 0; i + 1 < K; i += 2)
        row[i / 2] = (uint8_t)(codeAt(file, outF, true, in0 + i, o) | (codeAt(file, outF, true, in0 + i + 1, o) << 4));
    }
  }
}

void gptqDequant(const uint8_t* file, int inF, int outF, bool uint4, int in0, int in1, int out0, int out1, const float* scale,
                 const float* zero, float* dst) {
  (void)inF;
  const int K = in1 - in0;
  for (int o = out0; o < out1; ++o)
    for (int i = 0; i < K; ++i)
      dst[(size_t)(o - out0) * K + i] = (float)codeAt(file, outF, uint4, in0 + i, o) * scale[o] + zero[o];
}

void gptqRowSums(const uint8_t* file, int inF, int outF, bool uint4, int in0, int in1, int out0, int out1, float* dst) {
  (void)inF;
  for (int o = out0; o < out1; ++o) {
    long long s = 0;
    for (int i = in0; i < in1; ++i) s += codeAt(file, outF, uint4, i, o);
    dst[o - out0] = (float)s;
  }
}

}  // namespace xft
