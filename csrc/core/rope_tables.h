// Position-encoding tables of the C++ runtime, built on the host and consumed by the RoPE / attention kernels
// (reference: the eight rotary classes under src/layers — rotary_embedding.cpp, yarn_scaled_rotary_embedding.cpp:26-84,
// rotary_embedding_deepseekv2.cpp:62-85, rotary_embedding_qwen.cpp:33-135, rope_2d.cpp — and alibi_embedding.cpp).
// One builder covers them: the variants differ in the inverse frequencies and in a scale on the table.
// C++ twin of ops/reference.py (rope_inv_freq, rope_table, yarn_mscale, alibi_slopes).
#pragma once
#include <string>
#include <vector>

namespace xft {

struct RopeScaling {
  std::string type;            // "", "linear", "yarn"
  double factor = 1.0;
  int originalMaxPos = 2048;   // yarn: training context
  double betaFast = 32.0, betaSlow = 1.0;
  double mscale = 1.0, mscaleAllDim = 0.0;
  double tableScale = -1.0;    // >= 0 overrides the YaRN attention scale (Llama YaRN uses 0.1 ln(factor) + 1)
};

// 0.1 * mscale * ln(scale) + 1 for scale > 1, else 1
double yarnMscale(double scale, double mscale);
// rotDim / 2 inverse frequencies
std::vector<double> ropeInvFreq(int rotDim, double theta, const RopeScaling& s);
// [maxPos, rotDim] = cos(pos * inv) ‖ sin(pos * inv), rotDim / 2 values each, times the table scale
std::vector<float> ropeTable(int maxPos, int rotDim, double theta, const RopeScaling& s);
// Qwen-1 dynamic NTK: base for a context of maxKv tokens when the model was trained on seqLen (alpha = 2^ceil(log2(
// maxKv / seqLen) + 1) - 1, base * alpha^(rot / (rot - 2))); returns theta unchanged for maxKv <= seqLen
double qwenNtkTheta(double theta, int rotDim, int maxKv, int seqLen);
// TeleChat NTK (src/layers/rotary_embedding_telechat.cpp:29-35,68-117): the base for a context of kvLen tokens is
// computed from max(kvLen, trainLen), alpha = max(2^ceil(log2(len / 4096) + 1) - 1, 1), base * alpha^(rot / (rot - 2));
// a table first built during a pass with more than trainLen input tokens is scaled by 0.1 ln(inputLen / trainLen) + 1
double telechatNtkTheta(double theta, int rotDim, int kvLen, int trainLen);
double telechatMscale(int inputLen, int trainLen);
// ALiBi slopes for nHeads heads: powers of 2^(-8/n) of the next lower power of two, interleaved tail for the rest
std::vector<float> alibiSlopes(int nHeads);

}  // namespace xft
