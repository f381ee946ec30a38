// Public enums of the C++ API.  Same names and values as the reference's include/dtype.h:18-55 so that user code
// compiles unchanged against this library.
#pragma once

namespace xft {

enum DataType {
  fp32 = 0, bf16, fp16, int8, w8a8, int4, nf4,
  bf16_fp16, bf16_int8, bf16_w8a8, bf16_int4, bf16_nf4, w8a8_int8, w8a8_int4, w8a8_nf4,
  fp8_e4m3, unknown,
};

// "bf16", "int8", ..., "bf16_int8", ... -> DataType (DataType::unknown for anything else): the strings the Python
// package and the command-line programs use for weight types.
inline DataType dataTypeFromName(const char* name) {
  static const char* names[] = {"fp32", "bf16", "fp16", "int8", "w8a8", "int4", "nf4", "bf16_fp16", "bf16_int8", "bf16_w8a8",
                                "bf16_int4", "bf16_nf4", "w8a8_int8", "w8a8_int4", "w8a8_nf4", "fp8_e4m3"};
  for (int i = 0; i < (int)(sizeof(names) / sizeof(names[0])); ++i) {
    const char* a = names[i];
    const char* b = name;
    while (*a && *a == *b) { ++a; ++b; }
    if (!*a && !*b) return (DataType)i;
  }
  return unknown;
}

enum DeviceKind { iCPU = 0, iGPU };
enum NormType { RMS = 0, LN };
enum ActivationType { RELU = 0, GELU, SWIGLU, SILU };
enum class ParamType { None, INT4, INT8, FP16, BF16, FP32, FP8_E4M3 };

}  // namespace xft
