// Layer-level C++ API (csrc/api/xft/layers.h) on device pointers: thin adapters over the kernel library.
// Reference: src/kernels/{layernorm,rmsnorm,token_embedding,rotary_embedding,attention}_kernels.cpp,
// src/kernels/gemm_kernel_ext.cpp:502-517 (invokeGemm), src/layers/mlp_llama.cpp:24-88 (invokeMLPLLaMA).
#include <cuda_runtime.h>

#include <mutex>

#include "kernels_c.h"
#include "xft/layers.h"

namespace xft {
namespace {
struct Scratch {
  float* ws = nullptr; int* counters = nullptr; int* attnCounters = nullptr; int* status = nullptr;
  float* partO = nullptr; float* partMl = nullptr;
  static constexpr size_t kWs = 64u << 20, kPartO = 64u << 20, kPartMl = 4u << 20;
};
Scratch& scratch() {
  static Scratch s[64];
  static std::mutex mu;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> g(mu);
  Scratch& r = s[dev & 63];
  if (!r.ws) {
    cudaMalloc(&r.ws, Scratch::kWs);
    cudaMalloc(&r.counters, 8192 * 4); cudaMemset(r.counters, 0, 8192 * 4);
    cudaMalloc(&r.attnCounters, 16384 * 4); cudaMemset(r.attnCounters, 0, 16384 * 4);
    cudaMalloc(&r.status, 16); cudaMemset(r.status, 0, 16);
    cudaMalloc(&r.partO, Scratch::kPartO);
    cudaMalloc(&r.partMl, Scratch::kPartMl);
  }
  return r;
}
bool bf16Only(DataType dt) { return dt == DataType::bf16; }
}  // namespace

int invokeRmsNorm(DataType dt, void* out, const void* in, const float* w, int rows, int cols, int iStride, int oStride,
                  float eps, cudaStream_t st) {
  if (!bf16Only(dt)) return -1;
  return xft_rmsnorm(in, iStride < 0 ? cols : iStride, nullptr, 0, w, out, oStride < 0 ? cols : oStride, nullptr, rows, cols, eps, st);
}
int invokeLayerNorm(DataType dt, void* out, const void* in, const float* gamma, const float* beta, int rows, int cols,
                    int iStride, int oStride, float eps, cudaStream_t st) {
  if (!bf16Only(dt)) return -1;
  return xft_layernorm(in, iStride < 0 ? cols : iStride, gamma, beta, out, oStride < 0 ? cols : oStride, rows, cols, eps, st);
}
int invokeGemm(DataType dt, int M, int N, int K, const void* A, int lda, const void* W, int ldw, void* C, int ldc,
               const float* bias, const void* res, int ldres, cudaStream_t st) {
  if (!bf16Only(dt)) return -1;
  Scratch& s = scratch();
  return xft_gemm_bf16(A, lda, W, N, ldw, C, ldc, 0, M, N, K, 0, 0, bias, res, ldres < 0 ? N : ldres, 1.0f, 0, nullptr, s.ws,
                       Scratch::kWs, s.counters, 8192, s.status, 0, st);
}
int invokeTokenEmbedding(DataType dt, void* out, const int* ids, const void* table, int tokens, int hidden, int vocab,
                         cudaStream_t st) {
  if (!bf16Only(dt)) return -1;
  return xft_embedding(ids, table, out, tokens, hidden, vocab, 1.0f, nullptr, nullptr, 0, 0, scratch().status, st);
}
int invokeRotaryEmbedding(DataType dt, void* x, const int* positions, const float* table, int tokens, int heads, int dim,
                          int maxPos, cudaStream_t st) {
  if (!bf16Only(dt)) return -1;
  return xft_rope(x, tokens, heads, dim, positions, table, dim, 0, 0, maxPos, nullptr, scratch().status, st);
}
int invokeAttention(DataType dt, void* out, const void* q, const void* kc, const void* vc, const int* bt, int btStride,
                    const int* cuQ, const int* ctxLens, int batch, int maxQ, int qHeads, int kvHeads, int dim, int numBlocks,
                    float scale, bool isPrefill, cudaStream_t st) {
  if (!bf16Only(dt)) return -1;
  Scratch& s = scratch();
  const int group = qHeads / (kvHeads > 0 ? kvHeads : 1);
  int nsplit = 1;
  if (!isPrefill) {
    const int ctas = batch * kvHeads * ((group + 15) / 16);
    nsplit = 444 / (ctas > 0 ? ctas : 1);
    if (nsplit > 8) nsplit = 8;
    if (nsplit < 1 || ctas > 16384) nsplit = 1;
    while (nsplit > 1 && ((size_t)batch * qHeads * nsplit * dim * 4 > Scratch::kPartO || (size_t)batch * qHeads * nsplit * 8 > Scratch::kPartMl)) --nsplit;
  }
  return xft_paged_attention(q, out, kc, vc, nullptr, nullptr, bt, btStride, cuQ, ctxLens, batch, maxQ, qHeads, kvHeads, group, 0,
                             dim, 64, numBlocks, scale, nullptr, nullptr, isPrefill ? 0 : 1, nsplit, s.partO, s.partMl,
                             s.attnCounters, s.status, st);
}
int invokeMLPLLaMA(DataType dt, ActivationType act, int tokens, int hidden, int inter, void* out, const void* in,
                   const void* gateUp, const void* down, void* sc, const void* residual, cudaStream_t st) {
  if (!bf16Only(dt)) return -1;
  Scratch& s = scratch();
  const int a = act == RELU ? 1 : act == GELU ? 3 : 2;
  int rc = xft_gemm_bf16(in, hidden, gateUp, 2 * inter, hidden, sc, inter, 0, tokens, inter, hidden, 1, inter, nullptr, nullptr, 0,
                         1.0f, a, nullptr, s.ws, Scratch::kWs, s.counters, 8192, s.status, 0, st);
  if (rc) return rc;
  return xft_gemm_bf16(sc, inter, down, hidden, inter, out, hidden, 0, tokens, hidden, inter, 0, 0, nullptr, residual, hidden, 1.0f,
                       0, nullptr, s.ws, Scratch::kWs, s.counters, 8192, s.status, 0, st);
}

}  // namespace xft
