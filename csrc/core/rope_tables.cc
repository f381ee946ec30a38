#include "rope_tables.h"

#include <algorithm>
#include <cmath>

namespace xft {

double yarnMscale(double scale, double mscale) { return scale <= 1.0 ? 1.0 : 0.1 * mscale * std::log(scale) + 1.0; }

// dimension whose wavelength makes `numRot` rotations over the training context
static double yarnFindDim(double numRot, int dim, double base, int maxPos) {
  const double pi = 3.14159265358979323846;
  return (dim * std::log(maxPos / (numRot * 2.0 * pi))) / (2.0 * std::log(base));
}

std::vector<double> ropeInvFreq(int rotDim, double theta, const RopeScaling& s) {
  const int half = rotDim / 2;
  std::vector<double> inv(half);
  for (int i = 0; i < half; ++i) inv[i] = 1.0 / std::pow(theta, 2.0 * i / rotDim);
  if (s.type == "linear" && s.factor != 1.0) {
    for (auto& v : inv) v = v / s.factor;
  } else if (s.type == "yarn" && s.factor != 1.0) {
    // low dimensions (short wavelengths) keep their frequency, high ones are interpolated, a linear ramp in between
    double low = std::max(std::floor(yarnFindDim(s.betaFast, rotDim, theta, s.originalMaxPos)), 0.0);
    double high = std::min(std::ceil(yarnFindDim(s.betaSlow, rotDim, theta, s.originalMaxPos)), (double)rotDim - 1.0);
    if (low == high) high += 0.001;
    for (int i = 0; i < half; ++i) {
      const double ramp = std::min(std::max((i - low) / (high - low), 0.0), 1.0);
      const double keep = 1.0 - ramp;
      inv[i] = inv[i] / s.factor * (1.0 - keep) + inv[i] * keep;
    }
  }
  return inv;
}

std::vector<float> ropeTable(int maxPos, int rotDim, double theta, const RopeScaling& s) {
  const int half = rotDim / 2;
  const std::vector<double> inv = ropeInvFreq(rotDim, theta, s);
  double scale = 1.0;
  if (s.tableScale >= 0.0) scale = s.tableScale;
  else if (s.type == "yarn" && s.factor > 1.0)
    scale = yarnMscale(s.factor, s.mscale) / (s.mscaleAllDim != 0.0 ? yarnMscale(s.factor, s.mscaleAllDim) : 1.0);
  std::vector<float> tab((size_t)maxPos * rotDim);
  for (int pos = 0; pos < maxPos; ++pos)
    for (int i = 0; i < half; ++i) {
      tab[(size_t)pos * rotDim + i] = (float)(std::cos(pos * inv[i]) * scale);
      tab[(size_t)pos * rotDim + half + i] = (float)(std::sin(pos * inv[i]) * scale);
    }
  return tab;
}

double qwenNtkTheta(double theta, int rotDim, int maxKv, int seqLen) {
  if (maxKv <= seqLen || rotDim <= 2) return theta;
  const double ctx = std::log2((double)maxKv / seqLen) + 1.0;
  const double alpha = std::max(std::pow(2.0, std::ceil(ctx)) - 1.0, 1.0);
  return theta * std::pow(alpha, (double)rotDim / (rotDim - 2));
}

double telechatNtkTheta(double theta, int rotDim, int kvLen, int trainLen) {
  if (rotDim <= 2) return theta;
  const int len = std::max(kvLen, trainLen);
  const double ctx = std::log((double)len / 4096.0) / std::log(2.0) + 1.0;
  const double alpha = std::max(std::pow(2.0, std::ceil(ctx)) - 1.0, 1.0);
  return theta * std::pow(alpha, (double)rotDim / (rotDim - 2));
}

double telechatMscale(int inputLen, int trainLen) {
  return inputLen > trainLen ? 0.1 * std::log((double)inputLen / trainLen) + 1.0 : 1.0;
}

static void pow2Slopes(int n, std::vector<float>& out) {
  const double start = std::pow(2.0, -8.0 / n);
  double v = start;
  for (int i = 0; i < n; ++i, v *= start) out.push_back((float)v);
}

std::vector<float> alibiSlopes(int nHeads) {
  std::vector<float> out;
  if (nHeads <= 0) return out;
  int p = 1;
  while (p * 2 <= nHeads) p *= 2;
  pow2Slopes(p, out);
  if (p < nHeads) {
    std::vector<float> extra;
    pow2Slopes(2 * p, extra);
    for (int i = 0; i < 2 * p && (int)out.size() < nHeads; i += 2) out.push_back(extra[i]);
  }
  return out;
}

}  // namespace xft
