// Stateful entries of the layer-level C++ API (csrc/api/xft/layers.h): a whole attention block, a whole decoder layer
// and the DeepSeek MoE object, on DEVICE pointers.
//
// Reference: invokeAttentionLLaMA (src/layers/attention.cpp:28-160), invokeLayerLLaMA (src/layers/decoder_layer.cpp:
// 29-207), createDeepSeekMoE / forwardDeepSeekMoE / destroyDeepSeekMoE and invokeMoEDeepSeek
// (src/layers/moe_deepseek.cpp:24-260).  As there, the attention and layer calls keep one object per set of weight
// pointers; unlike there, each object owns its KV cache (the reference shares one cache manager between all of them),
// so two layers driven through this API do not overwrite each other's keys.
//
// Weight layout of these calls: row-major [in, out] bf16 on the device (the reference's untransposed layout); the
// object keeps its own [out, in] copy, which is what the tcgen05 GEMM streams.
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <map>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <tuple>
#include <vector>

#include "kernels_c.h"
#include "xft/layers.h"

namespace xft {
namespace {

struct Buf {
  void* p = nullptr;
  size_t bytes = 0;
  Buf() = default;
  Buf(const Buf&) = delete;
  Buf& operator=(const Buf&) = delete;
  ~Buf() { if (p) cudaFree(p); }
  bool ensure(size_t n, bool zero = false) {
    if (n <= bytes) return true;
    if (p) cudaFree(p);
    p = nullptr; bytes = 0;
    if (cudaMalloc(&p, n) != cudaSuccess) return false;
    bytes = n;
    if (zero) cudaMemset(p, 0, n);
    return true;
  }
  template <class T> T* as() const { return static_cast<T*>(p); }
};

struct Work {                   // split-K / split-KV scratch shared by the objects of one device
  Buf ws, counters, attnCounters, status, partO, partMl;
  static constexpr size_t kWs = 64u << 20;
  bool init() {
    if (ws.p) return true;
    return ws.ensure(kWs) && counters.ensure(8192 * 4, true) && attnCounters.ensure(16384 * 4, true) &&
           status.ensure(16, true) && partO.ensure(64u << 20) && partMl.ensure(4u << 20);
  }
};
Work& work() {
  static Work w[64];
  int dev = 0;
  cudaGetDevice(&dev);
  return w[dev & 63];
}
std::mutex g_mu;

constexpr int kBlock = 64;

int gemm(Work& w, const void* X, int ldx, const void* Wt, int wRows, int K, void* Y, int ldo, int T, int N, int gated,
         int dualOff, const float* bias, const void* res, int ldr, int act, int fp32, cudaStream_t st) {
  return xft_gemm_bf16(X, ldx, Wt, wRows, K, Y, ldo, fp32, T, N, K, gated, dualOff, bias, res, ldr, 1.0f, act, nullptr,
                       w.ws.as<float>(), Work::kWs, w.counters.as<int>(), 8192, w.status.as<int>(), 0, st);
}

// ---------------------------------------------------------------------------------------------- attention object
struct AttnObj {
  int hidden = 0, heads = 0, kvHeads = 0, dim = 0, maxPos = 0;
  Buf qkvW, oW, qkvB, oB, rope, kc, vc, bt, cu, kvl, pos, slots, qkv, q, att;
  bool hasQkvB = false, hasOB = false;
  int cacheBatch = 0, blocksPerSeq = 0;

  bool build(int hidden_, int heads_, int kvHeads_, int dim_, int maxPos_, float theta, const void* qW, const void* kW,
             const void* vW, const void* oWt, const float* qB, const float* kB, const float* vB, const float* oBias,
             cudaStream_t st) {
    hidden = hidden_; heads = heads_; kvHeads = kvHeads_; dim = dim_; maxPos = maxPos_;
    const int qN = heads * dim, kvN = kvHeads * dim, N = qN + 2 * kvN;
    if (!qkvW.ensure((size_t)N * hidden * 2) || !oW.ensure((size_t)hidden * qN * 2)) return false;
    char* d = qkvW.as<char>();
    // [hidden, n] -> [n, hidden]
    if (xft_transpose_to_bf16(qW, 2, qN, hidden, qN, d, hidden, st)) return false;
    if (xft_transpose_to_bf16(kW, 2, kvN, hidden, kvN, d + (size_t)qN * hidden * 2, hidden, st)) return false;
    if (xft_transpose_to_bf16(vW, 2, kvN, hidden, kvN, d + (size_t)(qN + kvN) * hidden * 2, hidden, st)) return false;
    if (xft_transpose_to_bf16(oWt, 2, hidden, qN, hidden, oW.p, qN, st)) return false;
    hasQkvB = qB || kB || vB;
    if (hasQkvB) {
      std::vector<float> z((size_t)N, 0.f);
      if (!qkvB.ensure((size_t)N * 4)) return false;
      cudaMemcpyAsync(qkvB.p, z.data(), (size_t)N * 4, cudaMemcpyHostToDevice, st);
      cudaStreamSynchronize(st);
      if (qB) cudaMemcpyAsync(qkvB.as<float>(), qB, (size_t)qN * 4, cudaMemcpyDefault, st);
      if (kB) cudaMemcpyAsync(qkvB.as<float>() + qN, kB, (size_t)kvN * 4, cudaMemcpyDefault, st);
      if (vB) cudaMemcpyAsync(qkvB.as<float>() + qN + kvN, vB, (size_t)kvN * 4, cudaMemcpyDefault, st);
    }
    hasOB = oBias != nullptr;
    if (hasOB) {
      if (!oB.ensure((size_t)hidden * 4)) return false;
      cudaMemcpyAsync(oB.p, oBias, (size_t)hidden * 4, cudaMemcpyDefault, st);
    }
    // rotary table [maxPos, dim] = cos(dim/2) | sin(dim/2)
    std::vector<float> tab((size_t)maxPos * dim);
    const int half = dim / 2;
    for (int pos = 0; pos < maxPos; ++pos)
      for (int i = 0; i < half; ++i) {
        const double inv = std::pow((double)theta, -2.0 * i / dim);
        tab[(size_t)pos * dim + i] = (float)std::cos(pos * inv);
        tab[(size_t)pos * dim + half + i] = (float)std::sin(pos * inv);
      }
    if (!rope.ensure(tab.size() * 4)) return false;
    cudaMemcpyAsync(rope.p, tab.data(), tab.size() * 4, cudaMemcpyHostToDevice, st);
    cudaStreamSynchronize(st);
    return true;
  }

  // x [batch*seq, ldx] -> out = attention(x) Wo + bias + residual; keys of the call land at positions past..past+seq-1
  int forward(Work& w, int batch, int seq, int past, const void* x, int ldx, const void* residual, int ldr, void* out,
              int ldo, cudaStream_t st) {
    if (past + seq > maxPos) return -20;
    const int T = batch * seq, qN = heads * dim, kvN = kvHeads * dim, N = qN + 2 * kvN;
    const int bps = (maxPos + kBlock - 1) / kBlock;
    if (batch > cacheBatch || bps != blocksPerSeq) {
      if (past > 0) return -21;                     // growing the batch in the middle of a sequence would lose its keys
      const size_t per = (size_t)kvHeads * kBlock * dim * 2;
      if (!kc.ensure(per * bps * batch, true) || !vc.ensure(per * bps * batch, true)) return -22;
      cudaMemsetAsync(kc.p, 0, per * bps * batch, st);
      cudaMemsetAsync(vc.p, 0, per * bps * batch, st);
      cacheBatch = batch; blocksPerSeq = bps;
    }
    std::vector<int> hbt((size_t)batch * bps), hcu(batch + 1), hkv(batch), hpos(T), hslot(T);
    for (int b = 0; b < batch; ++b) {
      for (int j = 0; j < bps; ++j) hbt[(size_t)b * bps + j] = b * bps + j;
      hcu[b] = b * seq;
      hkv[b] = past + seq;
      for (int i = 0; i < seq; ++i) {
        hpos[b * seq + i] = past + i;
        hslot[b * seq + i] = b * bps * kBlock + past + i;
      }
    }
    hcu[batch] = T;
    if (!bt.ensure(hbt.size() * 4) || !cu.ensure(hcu.size() * 4) || !kvl.ensure(hkv.size() * 4) || !pos.ensure((size_t)T * 4) ||
        !slots.ensure((size_t)T * 4) || !qkv.ensure((size_t)T * N * 2) || !q.ensure((size_t)T * qN * 2) ||
        !att.ensure((size_t)T * qN * 2))
      return -22;
    cudaMemcpyAsync(bt.p, hbt.data(), hbt.size() * 4, cudaMemcpyHostToDevice, st);
    cudaMemcpyAsync(cu.p, hcu.data(), hcu.size() * 4, cudaMemcpyHostToDevice, st);
    cudaMemcpyAsync(kvl.p, hkv.data(), hkv.size() * 4, cudaMemcpyHostToDevice, st);
    cudaMemcpyAsync(pos.p, hpos.data(), (size_t)T * 4, cudaMemcpyHostToDevice, st);
    cudaMemcpyAsync(slots.p, hslot.data(), (size_t)T * 4, cudaMemcpyHostToDevice, st);
    cudaStreamSynchronize(st);                      // the host vectors go out of scope below
    int rc = gemm(w, x, ldx, qkvW.p, N, hidden, qkv.p, N, T, N, 0, 0, hasQkvB ? qkvB.as<float>() : nullptr, nullptr, 0, 0, 0, st);
    if (rc) return rc;
    const int numBlocks = cacheBatch * blocksPerSeq;
    rc = xft_qkv_rope_cache(qkv.p, N, T, heads, kvHeads, dim, pos.as<int>(), rope.as<float>(), dim, 0, 0, maxPos, nullptr,
                            nullptr, nullptr, 1e-6f, q.p, kc.p, vc.p, nullptr, nullptr, 0, kBlock,
                            (long long)numBlocks * kBlock, slots.as<int>(), w.status.as<int>(), st);
    if (rc) return rc;
    const int group = heads / (kvHeads > 0 ? kvHeads : 1);
    const bool decode = seq == 1;
    int nsplit = 1;
    if (decode) {
      const int ctas = batch * kvHeads * ((group + 15) / 16), ntiles = (past + seq + 63) / 64;
      nsplit = (dim <= 128 ? 296 : 148) / (ctas > 0 ? ctas : 1);
      if (nsplit > ntiles / 8) nsplit = ntiles / 8;
      if (nsplit > 32) nsplit = 32;
      if (nsplit < 1 || ctas > 16384) nsplit = 1;
    }
    rc = xft_paged_attention(q.p, att.p, kc.p, vc.p, nullptr, nullptr, bt.as<int>(), bps, cu.as<int>(), kvl.as<int>(), batch,
                             seq, heads, kvHeads, group, 0, dim, kBlock, numBlocks, 1.0f / std::sqrt((float)dim), nullptr,
                             nullptr, decode ? 1 : 0, nsplit, w.partO.as<float>(), w.partMl.as<float>(),
                             w.attnCounters.as<int>(), w.status.as<int>(), st);
    if (rc) return rc;
    return gemm(w, att.p, qN, oW.p, hidden, qN, out, ldo, T, hidden, 0, 0, hasOB ? oB.as<float>() : nullptr, residual, ldr, 0,
                0, st);
  }
};

using Key = std::tuple<const void*, const void*, const void*, const void*, int, int, int, int>;
std::map<Key, std::unique_ptr<AttnObj>> g_attn;

AttnObj* attnFor(int hidden, int heads, int kvHeads, int dim, int maxPos, const void* qW, const void* kW, const void* vW,
                 const void* oW, const float* qB, const float* kB, const float* vB, const float* oB, cudaStream_t st) {
  Key key{qW, kW, vW, oW, heads, kvHeads, dim, maxPos};
  auto it = g_attn.find(key);
  if (it != g_attn.end()) return it->second.get();
  auto obj = std::make_unique<AttnObj>();
  if (!obj->build(hidden, heads, kvHeads, dim, maxPos, 10000.0f, qW, kW, vW, oW, qB, kB, vB, oB, st)) return nullptr;
  AttnObj* p = obj.get();
  g_attn[key] = std::move(obj);
  return p;
}

// ---------------------------------------------------------------------------------------------- layer object
struct MlpObj {
  Buf gateUp, down, h, g;
  int hidden = 0, inter = 0;
  bool build(int hidden_, int inter_, const void* gate, const void* up, const void* dn, cudaStream_t st) {
    hidden = hidden_; inter = inter_;
    if (!gateUp.ensure((size_t)2 * inter * hidden * 2) || !down.ensure((size_t)hidden * inter * 2)) return false;
    if (xft_transpose_to_bf16(gate, 2, inter, hidden, inter, gateUp.p, hidden, st)) return false;
    if (xft_transpose_to_bf16(up, 2, inter, hidden, inter, gateUp.as<char>() + (size_t)inter * hidden * 2, hidden, st)) return false;
    if (xft_transpose_to_bf16(dn, 2, hidden, inter, hidden, down.p, inter, st)) return false;
    return true;
  }
};
std::map<std::tuple<const void*, const void*, const void*>, std::unique_ptr<MlpObj>> g_mlp;

}  // namespace

int invokeAttentionLLaMA(DataType dt, int batchSize, int inputSeqLen, int attHeadDim, int attHeadNum, int kvHeadNum,
                         int maxPositions, int maxPosEmbed, int pastSeqLen, int currentSeqLen, int step, int hiddenSize,
                         void* output, int outputStride, const void* input, int inputStride, const void* queryWeight,
                         const void* keyWeight, const void* valueWeight, const void* attnOutWeight, const float* queryBias,
                         const float* keyBias, const float* valueBias, const float* attnOutBias, cudaStream_t stream) {
  (void)maxPosEmbed; (void)currentSeqLen; (void)step;
  if (dt != DataType::bf16) return -1;
  std::lock_guard<std::mutex> g(g_mu);
  Work& w = work();
  if (!w.init()) return -22;
  AttnObj* a = attnFor(hiddenSize, attHeadNum, kvHeadNum, attHeadDim, maxPositions, queryWeight, keyWeight, valueWeight,
                       attnOutWeight, queryBias, keyBias, valueBias, attnOutBias, stream);
  if (!a) return -23;
  return a->forward(w, batchSize, inputSeqLen, pastSeqLen, input, inputStride, input, inputStride, output, outputStride, stream);
}

int invokeLayerLLaMA(DataType dt, ActivationType at, NormType nt, int batchSize, int inputSeqLen, int attHeadDim,
                     int attHeadNum, int kvHeadNum, int maxPositions, int maxPosEmbed, int pastSeqLen, int currentSeqLen,
                     int step, int hiddenSize, int intermediateSize, void* output, int outputStride, const void* input,
                     int inputStride, const float* ln1Gamma, const float* ln1Beta, const void* queryWeight,
                     const void* keyWeight, const void* valueWeight, const void* attnOutWeight, const float* ln2Gamma,
                     const float* ln2Beta, const void* gateWeight, const void* upWeight, const void* downWeight,
                     const float* queryBias, const float* keyBias, const float* valueBias, const float* attnOutBias,
                     cudaStream_t stream) {
  (void)maxPosEmbed; (void)currentSeqLen; (void)step;
  if (dt != DataType::bf16) return -1;
  std::lock_guard<std::mutex> g(g_mu);
  Work& w = work();
  if (!w.init()) return -22;
  AttnObj* a = attnFor(hiddenSize, attHeadNum, kvHeadNum, attHeadDim, maxPositions, queryWeight, keyWeight, valueWeight,
                       attnOutWeight, queryBias, keyBias, valueBias, attnOutBias, stream);
  if (!a) return -23;
  auto mk = std::make_tuple(gateWeight, upWeight, downWeight);
  auto it = g_mlp.find(mk);
  if (it == g_mlp.end()) {
    auto obj = std::make_unique<MlpObj>();
    if (!obj->build(hiddenSize, intermediateSize, gateWeight, upWeight, downWeight, stream)) return -23;
    it = g_mlp.emplace(mk, std::move(obj)).first;
  }
  MlpObj* m = it->second.get();
  const int T = batchSize * inputSeqLen;
  // three hidden-sized rows per token: normed input, state after attention, normed state; plus the activation
  if (!m->h.ensure((size_t)3 * T * hiddenSize * 2) || !m->g.ensure((size_t)T * intermediateSize * 2)) return -22;
  char* h1 = m->h.as<char>();
  char* x1 = h1 + (size_t)T * hiddenSize * 2;
  char* h2 = x1 + (size_t)T * hiddenSize * 2;
  auto norm = [&](const void* src, int ld, const float* gamma, const float* beta, void* dst) {
    if (nt == NormType::RMS) return xft_rmsnorm(src, ld, nullptr, 0, gamma, dst, hiddenSize, nullptr, T, hiddenSize, 1e-6f, stream);
    return xft_layernorm(src, ld, gamma, beta, dst, hiddenSize, T, hiddenSize, 1e-5f, stream);
  };
  int rc = norm(input, inputStride, ln1Gamma, ln1Beta, h1);
  if (rc) return rc;
  rc = a->forward(w, batchSize, inputSeqLen, pastSeqLen, h1, hiddenSize, input, inputStride, x1, hiddenSize, stream);
  if (rc) return rc;
  rc = norm(x1, hiddenSize, ln2Gamma, ln2Beta, h2);
  if (rc) return rc;
  const int act = at == RELU ? 1 : at == GELU ? 3 : 2;
  rc = gemm(w, h2, hiddenSize, m->gateUp.p, 2 * intermediateSize, hiddenSize, m->g.p, intermediateSize, T, intermediateSize, 1,
            intermediateSize, nullptr, nullptr, 0, act, 0, stream);
  if (rc) return rc;
  return gemm(w, m->g.p, intermediateSize, m->down.p, hiddenSize, intermediateSize, output, outputStride, T, hiddenSize, 0, 0,
              nullptr, x1, hiddenSize, 0, 0, stream);
}

// ---------------------------------------------------------------------------------------------- DeepSeek MoE object
namespace {
struct MoeObj {
  int E = 0, k = 0, H = 0, I = 0, nGroup = 1, topkGroup = 1, e0 = 0, e1 = 0;
  bool normTopK = true;
  float scaling = 1.0f;
  Buf gu, dn, bias, idx, wts, pos, src, rowW, tiles, meta, xs, h1, ys;
};
}  // namespace

void* createDeepSeekMoE(int layerId, int numExperts, int numExpPerTok, int hiddenSize, int intermediateSize, bool normTopKProb,
                        int nGroup, int topkGroup, const void* gateUpWeights, const void* downWeights,
                        const void* gateUpScales, const void* downScales, const void* gatingCorrBias, int blockSize,
                        int tpRank, int tpSize, float routedScalingFactor, cudaStream_t stream) {
  (void)layerId;
  if (numExperts <= 0 || tpSize <= 0 || numExperts % tpSize || hiddenSize % 8 || intermediateSize % 8) return nullptr;
  auto m = std::make_unique<MoeObj>();
  m->E = numExperts; m->k = numExpPerTok; m->H = hiddenSize; m->I = intermediateSize; m->nGroup = nGroup > 0 ? nGroup : 1;
  m->topkGroup = topkGroup > 0 ? topkGroup : 1; m->normTopK = normTopKProb; m->scaling = routedScalingFactor;
  // expert parallelism: rank r owns experts [r*E/tp, (r+1)*E/tp); the caller sums the ranks' outputs
  const int per = numExperts / tpSize;
  m->e0 = tpRank * per; m->e1 = m->e0 + per;
  const size_t guRows = (size_t)2 * intermediateSize, guElems = guRows * hiddenSize, dnElems = (size_t)hiddenSize * intermediateSize;
  if (!m->gu.ensure(per * guElems * 2) || !m->dn.ensure(per * dnElems * 2)) return nullptr;
  if (gateUpScales) {
    if (guRows % blockSize || hiddenSize % blockSize) return nullptr;       // stacked experts must align with the scale grid
    const size_t scPer = (guRows / blockSize) * ((hiddenSize + blockSize - 1) / blockSize);
    if (xft_fp8_block_dequant((const uint8_t*)gateUpWeights + m->e0 * guElems, (const float*)gateUpScales + m->e0 * scPer,
                              (long long)per * guRows, hiddenSize, blockSize, m->gu.p, stream)) return nullptr;
  } else {
    cudaMemcpyAsync(m->gu.p, (const char*)gateUpWeights + m->e0 * guElems * 2, per * guElems * 2, cudaMemcpyDefault, stream);
  }
  if (downScales) {
    if (hiddenSize % blockSize) return nullptr;
    const size_t scPer = ((size_t)hiddenSize / blockSize) * ((intermediateSize + blockSize - 1) / blockSize);
    if (xft_fp8_block_dequant((const uint8_t*)downWeights + m->e0 * dnElems, (const float*)downScales + m->e0 * scPer,
                              (long long)per * hiddenSize, intermediateSize, blockSize, m->dn.p, stream)) return nullptr;
  } else {
    cudaMemcpyAsync(m->dn.p, (const char*)downWeights + m->e0 * dnElems * 2, per * dnElems * 2, cudaMemcpyDefault, stream);
  }
  if (gatingCorrBias) {
    if (!m->bias.ensure((size_t)numExperts * 4)) return nullptr;
    cudaMemcpyAsync(m->bias.p, gatingCorrBias, (size_t)numExperts * 4, cudaMemcpyDefault, stream);
  }
  if (cudaStreamSynchronize(stream) != cudaSuccess) return nullptr;
  return m.release();
}

static int moeExperts(MoeObj* m, const void* input, void* output, int T, const int* idx, const float* wts, int iStride,
                      int oStride, cudaStream_t st) {
  if (oStride != 0 && oStride != m->H) return -24;
  Work& w = work();
  if (!w.init()) return -22;
  const int k = m->k, E = m->e1 - m->e0, H = m->H, I = m->I;
  const int avg = std::max(1, (T * k + E - 1) / E);
  const int bn = avg <= 16 ? 16 : avg <= 32 ? 32 : avg <= 64 ? 64 : 128;
  const int maxRows = T * k, maxTiles = (maxRows + bn - 1) / bn + E;
  if (!m->pos.ensure((size_t)maxRows * 4) || !m->src.ensure((size_t)maxRows * 4) || !m->rowW.ensure((size_t)maxRows * 4) ||
      !m->tiles.ensure((size_t)maxTiles * 16) || !m->meta.ensure(8) || !m->xs.ensure((size_t)maxRows * H * 2) ||
      !m->h1.ensure((size_t)maxRows * I * 2) || !m->ys.ensure((size_t)maxRows * H * 4))
    return -22;
  int rc = xft_moe_plan(idx, wts, T, k, m->e0, m->e1, bn, m->pos.as<int>(), m->src.as<int>(), m->rowW.as<float>(), m->tiles.p,
                        m->meta.as<int>(), maxTiles, maxRows, st);
  if (rc) return rc;
  rc = xft_moe_gather(input, iStride > 0 ? iStride : H, m->src.as<int>(), m->meta.as<int>(), m->xs.p, maxRows, H, st);
  if (rc) return rc;
  rc = xft_gemm_bf16_grouped(m->xs.p, H, maxRows, m->gu.p, E * 2 * I, H, m->h1.p, I, 0, I, H, 1, I, 2 * I, m->tiles.p,
                             m->meta.as<int>(), maxTiles, bn, nullptr, 2 /* silu */, w.status.as<int>(), st);
  if (rc) return rc;
  rc = xft_gemm_bf16_grouped(m->h1.p, I, maxRows, m->dn.p, E * H, I, m->ys.p, H, 1, H, I, 0, 0, H, m->tiles.p, m->meta.as<int>(),
                             maxTiles, bn, m->rowW.as<float>(), 0, w.status.as<int>(), st);
  if (rc) return rc;
  return xft_moe_combine(m->ys.as<float>(), m->pos.as<int>(), k, nullptr, nullptr, 0, output, nullptr, T, H, st);
}

int forwardDeepSeekMoE(void* moe, void* input, void* output, int nTokens, void* routingLogits, int iStride, int oStride,
                       cudaStream_t stream) {
  MoeObj* m = static_cast<MoeObj*>(moe);
  if (!m || nTokens <= 0) return m ? 0 : -25;
  std::lock_guard<std::mutex> g(g_mu);
  if (!m->idx.ensure((size_t)nTokens * m->k * 4) || !m->wts.ensure((size_t)nTokens * m->k * 4)) return -22;
  int rc = xft_moe_route((const float*)routingLogits, m->E, nTokens, m->E, m->k, 2 /* deepseek */, m->bias.as<float>(), m->nGroup,
                         m->topkGroup, m->scaling, m->normTopK ? 1 : 0, 1, m->idx.as<int>(), m->wts.as<float>(), stream);
  if (rc) return rc;
  return moeExperts(m, input, output, nTokens, m->idx.as<int>(), m->wts.as<float>(), iStride, oStride, stream);
}

int forwardDeepSeekMoE(void* moe, void* input, void* output, int nTokens, int* selExperts, float* expertWeights, int iStride,
                       int oStride, cudaStream_t stream) {
  MoeObj* m = static_cast<MoeObj*>(moe);
  if (!m || nTokens <= 0) return m ? 0 : -25;
  std::lock_guard<std::mutex> g(g_mu);
  return moeExperts(m, input, output, nTokens, selExperts, expertWeights, iStride, oStride, stream);
}

void destroyDeepSeekMoE(void* moe) { delete static_cast<MoeObj*>(moe); }

// ---------------------------------------------------------------------------------------------- stateless DeepSeek MoE
namespace {
struct MoeCallObj {
  MlpObj mlp;                 // the one weight set every expert uses, as [out, in] copies
  Buf router, bias, logits, idx, wts, pos, src, rowW, tiles, meta, xs, h1, ys, shared, hid;
  int E = 0;
};
std::map<std::tuple<const void*, const void*, const void*, const void*>, std::unique_ptr<MoeCallObj>> g_moeCall;
}  // namespace

int invokeMoEDeepSeek(DataType dt, ActivationType at, int numTokens, int hiddenSize, int intermediateSize,
                      int moeIntermediateSize, int numSharedExperts, int numRoutedExperts, void* output, int outputStride,
                      const void* input, int inputStride, const void* gatingWeight, const float* gatingBias,
                      const void* gateWeight, const void* upWeight, const void* downWeight, cudaStream_t st) {
  if (dt != DataType::bf16 || at != SILU) return -1;
  if (numTokens <= 0) return 0;
  if (!input || !output || !gateWeight || !upWeight || !downWeight) return -25;
  const int H = hiddenSize, T = numTokens;
  const int I = numRoutedExperts > 0 ? moeIntermediateSize : intermediateSize;
  if (H % 8 || I % 8 || (outputStride != 0 && outputStride != H)) return -24;
  const int ldx = inputStride > 0 ? inputStride : H;
  Work& w = work();
  std::lock_guard<std::mutex> g(g_mu);
  if (!w.init()) return -22;
  auto key = std::make_tuple(gateWeight, upWeight, downWeight, gatingWeight);
  auto it = g_moeCall.find(key);
  if (it == g_moeCall.end()) {
    auto o = std::make_unique<MoeCallObj>();
    if (!o->mlp.build(H, I, gateWeight, upWeight, downWeight, st)) return -22;
    o->E = numRoutedExperts;
    if (numRoutedExperts > 0) {
      if (!gatingWeight) return -25;
      // router weight: fp32 [hidden, experts] -> bf16 [experts, hidden]; correction bias fp32 [experts]
      if (!o->router.ensure((size_t)numRoutedExperts * H * 2)) return -22;
      if (xft_transpose_to_bf16(gatingWeight, 0, numRoutedExperts, H, numRoutedExperts, o->router.p, H, st)) return -22;
      if (gatingBias) {
        if (!o->bias.ensure((size_t)numRoutedExperts * 4)) return -22;
        cudaMemcpyAsync(o->bias.p, gatingBias, (size_t)numRoutedExperts * 4, cudaMemcpyDefault, st);
      }
    }
    it = g_moeCall.emplace(key, std::move(o)).first;
  }
  MoeCallObj* m = it->second.get();
  const int act = 2;   // silu
  if (numRoutedExperts <= 0) {
    // dense layer (the first layers of the model): down(silu(x gate) * (x up))
    if (!m->hid.ensure((size_t)T * I * 2)) return -22;
    int rc = gemm(w, input, ldx, m->mlp.gateUp.p, 2 * I, H, m->hid.p, I, T, I, 1, I, nullptr, nullptr, 0, act, 0, st);
    if (rc) return rc;
    return gemm(w, m->hid.p, I, m->mlp.down.p, H, I, output, H, T, H, 0, 0, nullptr, nullptr, 0, 0, 0, st);
  }
  // routing as DeepSeek-V3 does it: sigmoid scores + correction bias, 8 groups / best 4, top 8, weights normalised and
  // scaled by 2.5 (the constants of the reference's entry point, src/layers/moe_deepseek.cpp:43-55)
  const int E = numRoutedExperts, k = E < 8 ? E : 8;
  const int nGroup = E % 8 == 0 ? 8 : 1, topkGroup = nGroup == 8 ? 4 : 1;
  if (!m->logits.ensure((size_t)T * E * 4) || !m->idx.ensure((size_t)T * k * 4) || !m->wts.ensure((size_t)T * k * 4)) return -22;
  int rc = gemm(w, input, ldx, m->router.p, E, H, m->logits.p, E, T, E, 0, 0, nullptr, nullptr, 0, 0, 1, st);
  if (rc) return rc;
  rc = xft_moe_route(m->logits.as<float>(), E, T, E, k, 2 /* deepseek */, m->bias.as<float>(), nGroup, topkGroup, 2.5f, 1, 1,
                     m->idx.as<int>(), m->wts.as<float>(), st);
  if (rc) return rc;
  const int avg = std::max(1, (T * k + E - 1) / E);
  const int bn = avg <= 16 ? 16 : avg <= 32 ? 32 : avg <= 64 ? 64 : 128;
  const int maxRows = T * k, maxTiles = (maxRows + bn - 1) / bn + E;
  if (!m->pos.ensure((size_t)maxRows * 4) || !m->src.ensure((size_t)maxRows * 4) || !m->rowW.ensure((size_t)maxRows * 4) ||
      !m->tiles.ensure((size_t)maxTiles * 16) || !m->meta.ensure(8) || !m->xs.ensure((size_t)maxRows * H * 2) ||
      !m->h1.ensure((size_t)maxRows * I * 2) || !m->ys.ensure((size_t)maxRows * H * 4))
    return -22;
  rc = xft_moe_plan(m->idx.as<int>(), m->wts.as<float>(), T, k, 0, E, bn, m->pos.as<int>(), m->src.as<int>(),
                    m->rowW.as<float>(), m->tiles.p, m->meta.as<int>(), maxTiles, maxRows, st);
  if (rc) return rc;
  rc = xft_moe_gather(input, ldx, m->src.as<int>(), m->meta.as<int>(), m->xs.p, maxRows, H, st);
  if (rc) return rc;
  // every routed expert reads the same weight set: a group stride of 0 rows points all groups at it
  rc = xft_gemm_bf16_grouped(m->xs.p, H, maxRows, m->mlp.gateUp.p, 2 * I, H, m->h1.p, I, 0, I, H, 1, I, 0, m->tiles.p,
                             m->meta.as<int>(), maxTiles, bn, nullptr, act, w.status.as<int>(), st);
  if (rc) return rc;
  rc = xft_gemm_bf16_grouped(m->h1.p, I, maxRows, m->mlp.down.p, H, I, m->ys.p, H, 1, H, I, 0, 0, 0, m->tiles.p,
                             m->meta.as<int>(), maxTiles, bn, m->rowW.as<float>(), 0, w.status.as<int>(), st);
  if (rc) return rc;
  const void* add = nullptr;
  if (numSharedExperts > 0) {
    // the shared expert sees every token (same weight pointers in this entry point)
    if (!m->hid.ensure((size_t)T * I * 2) || !m->shared.ensure((size_t)T * H * 2)) return -22;
    rc = gemm(w, input, ldx, m->mlp.gateUp.p, 2 * I, H, m->hid.p, I, T, I, 1, I, nullptr, nullptr, 0, act, 0, st);
    if (rc) return rc;
    rc = gemm(w, m->hid.p, I, m->mlp.down.p, H, I, m->shared.p, H, T, H, 0, 0, nullptr, nullptr, 0, 0, 0, st);
    if (rc) return rc;
    add = m->shared.p;
  }
  return xft_moe_combine(m->ys.as<float>(), m->pos.as<int>(), k, nullptr, add, H, output, nullptr, T, H, st);
}

}  // namespace xft
