// GPTQ-converted tensors of a checkpoint directory (reference: src/layers/decoder_block.h:204-277 reads them,
// src/xfastertransformer/tools/llama_convert.py:335-392 writes them):
//   <name>.qweight.0.bin  int8 [in, out], or uint4 two per byte ALONG OUT ([in, out / 2], low nibble = even column)
//   <name>.scales.0.bin, <name>.zeros.0.bin  fp32 [out];  w = q * scale + zero
// The device kernels read [out, in] rows (uint4: two codes per byte along IN, low nibble = even index), so a tensor is
// unpacked, cut to the rank's ranges, transposed and repacked on the host.
#pragma once
#include <cstdint>
#include <vector>

namespace xft {

// Rows [out0, out1) x columns [in0, in1) of the logical [out, in] code matrix, in the device layout, `pitch` bytes per
// row (>= the row's bytes; the padding is zero).  int8: one signed byte per code; uint4: see above (in1 - in0 even).
void gptqRepack(const uint8_t* file, int inF, int outF, bool uint4, int in0, int in1, int out0, int out1, int pitch,
                uint8_t* dst);

// The same selection as fp32 values q * scale[o] + zero[o], row-major [out1 - out0, in1 - in0].
void gptqDequant(const uint8_t* file, int inF, int outF, bool uint4, int in0, int in1, int out0, int out1, const float* scale,
                 const float* zero, float* dst);

// Sum of the codes of every selected row (the correction term of the int8 x int8 GEMM).
void gptqRowSums(const uint8_t* file, int inF, int outF, bool uint4, int in0, int in1, int out0, int out1, float* dst);

}  // namespace xft
