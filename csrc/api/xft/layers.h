// Layer-level C++ API on DEVICE pointers (reference: include/layers_norm.h, layers_gemm.h, layers_attention.h,
// layers_rotary_embedding.h, layers_token_embedding.h, layers_mlp.h — there on host pointers).  All tensors are bf16
// unless noted, row-major; every call enqueues on `stream` and returns 0 or an error code.
#pragma once
#include <cuda_runtime.h>

#include "dtype.h"

namespace xft {

int invokeRmsNorm(DataType dt, void* output, const void* input, const float* weight, int rows, int cols, int iStride = -1,
                  int oStride = -1, float epsilon = 1e-6f, cudaStream_t stream = 0);
int invokeLayerNorm(DataType dt, void* output, const void* input, const float* gamma, const float* beta, int rows, int cols,
                    int iStride = -1, int oStride = -1, float epsilon = 1e-5f, cudaStream_t stream = 0);
// C[M,N] = A[M,K] · W[N,K]^T (+bias[N] fp32) (+res[M,N]);  W is the [out,in] device layout of this library
int invokeGemm(DataType dt, int M, int N, int K, const void* A, int lda, const void* W, int ldw, void* C, int ldc,
               const float* bias = nullptr, const void* res = nullptr, int ldres = -1, cudaStream_t stream = 0);
// ids int32 [tokens] -> output [tokens, hidden]
int invokeTokenEmbedding(DataType dt, void* output, const int* ids, const void* table, int tokens, int hidden, int vocab,
                         cudaStream_t stream = 0);
// in-place llama-style rotary embedding on x [tokens, heads, dim] with table [maxPos, dim] = cos ‖ sin (fp32)
int invokeRotaryEmbedding(DataType dt, void* x, const int* positions, const float* table, int tokens, int heads, int dim,
                          int maxPos, cudaStream_t stream = 0);
// paged attention: q [tokens, qHeads, dim]; caches [blocks, kvHeads, 64, dim]; see csrc/kernels/attention.cu
int invokeAttention(DataType dt, void* output, const void* query, const void* kcache, const void* vcache,
                    const int* blockTables, int tableStride, const int* cuQ, const int* contextLens, int batch, int maxQ,
                    int qHeads, int kvHeads, int dim, int numBlocks, float scale, bool isPrefill, cudaStream_t stream = 0);
// out = down( act(x·gate^T) * (x·up^T) ) + residual;  gateUp [2*inter, hidden] (gate rows then up rows), down [hidden, inter]
int invokeMLPLLaMA(DataType dt, ActivationType act, int tokens, int hidden, int inter, void* output, const void* input,
                   const void* gateUp, const void* down, void* scratch /* tokens*inter bf16 */, const void* residual = nullptr,
                   cudaStream_t stream = 0);


// ---- stateful entries (csrc/core/layer_objects.cc).  Weights here are row-major [in, out] bf16 on the device, as in
// the reference's calls; one object per set of weight pointers keeps the [out, in] copies, the rotary table and its
// own paged KV cache (batch x maxPositions).  Keys of a call are appended at positions pastSeqLen ...
// output = attention(input) Wo + bias + input
int invokeAttentionLLaMA(DataType dt, int batchSize, int inputSeqLen, int attHeadDim, int attHeadNum, int kvHeadNum,
                         int maxPositions, int maxPosEmbed, int pastSeqLen, int currentSeqLen, int step, int hiddenSize,
                         void* output, int outputStride, const void* input, int inputStride, const void* queryWeight,
                         const void* keyWeight, const void* valueWeight, const void* attnOutWeight,
                         const float* queryBias = nullptr, const float* keyBias = nullptr, const float* valueBias = nullptr,
                         const float* attnOutBias = nullptr, cudaStream_t stream = 0);
// a whole pre-norm decoder layer: x1 = x + attn(norm1(x)); output = x1 + mlp(norm2(x1))
int invokeLayerLLaMA(DataType dt, ActivationType at, NormType nt, int batchSize, int inputSeqLen, int attHeadDim,
                     int attHeadNum, int kvHeadNum, int maxPositions, int maxPosEmbed, int pastSeqLen, int currentSeqLen,
                     int step, int hiddenSize, int intermediateSize, void* output, int outputStride, const void* input,
                     int inputStride, const float* ln1Gamma, const float* ln1Beta, const void* queryWeight,
                     const void* keyWeight, const void* valueWeight, const void* attnOutWeight, const float* ln2Gamma,
                     const float* ln2Beta, const void* gateWeight, const void* upWeight, const void* downWeight,
                     const float* queryBias = nullptr, const float* keyBias = nullptr, const float* valueBias = nullptr,
                     const float* attnOutBias = nullptr, cudaStream_t stream = 0);

// Stateless DeepSeek MoE block (reference: include/layers_mlp.h:25, src/layers/moe_deepseek.cpp:24-118).  As in the
// reference's entry point, ONE gate / up / down weight set (bf16 [in, out] on the device) serves every routed expert and
// the shared expert, and routing uses DeepSeek-V3's constants (sigmoid + correction bias, 8 groups / 4 kept, top 8,
// normalised, scaled by 2.5).  gatingWeight fp32 [hidden, experts], gatingBias fp32 [experts] or null.
// numRoutedExperts == 0: a dense SwiGLU layer of width intermediateSize.  The [out, in] copies are kept per set of weight
// ADDRESSES (as the reference keys its objects): weights must stay at their address, unchanged, while they are in use.
int invokeMoEDeepSeek(DataType dt, ActivationType at, int numTokens, int hiddenSize, int intermediateSize,
                      int moeIntermediateSize, int numSharedExperts, int numRoutedExperts, void* output, int outputStride,
                      const void* input, int inputStride, const void* gatingWeight, const float* gatingBias,
                      const void* gateWeight, const void* upWeight, const void* downWeight, cudaStream_t stream = 0);

// DeepSeek routed experts.  gateUpWeights [E, 2*inter, hidden] (gate rows, then up rows) and downWeights
// [E, hidden, inter], in [out, in] layout: bf16 when the scales are null, else e4m3 with one fp32 scale per
// blockSize x blockSize tile ([E, rows/blockSize, cols/blockSize]); they are expanded to bf16 once, here.
// tpRank / tpSize select the local experts (expert parallelism); the caller sums the ranks' outputs.
void* createDeepSeekMoE(int layerId, int numExperts, int numExpPerTok, int hiddenSize, int intermediateSize, bool normTopKProb,
                        int nGroup, int topkGroup, const void* gateUpWeights, const void* downWeights,
                        const void* gateUpScales, const void* downScales, const void* gatingCorrBias = nullptr,
                        int blockSize = 128, int tpRank = 0, int tpSize = 1, float routedScalingFactor = 1.0f,
                        cudaStream_t stream = 0);
// routingLogits: fp32 [nTokens, numExperts] (sigmoid scores + correction bias + group-limited top-k happen inside)
int forwardDeepSeekMoE(void* moe, void* input, void* output, int nTokens, void* routingLogits, int iStride = 0,
                       int oStride = 0, cudaStream_t stream = 0);
// experts already selected: selExperts int32 [nTokens, k], expertWeights fp32 [nTokens, k]
int forwardDeepSeekMoE(void* moe, void* input, void* output, int nTokens, int* selExperts, float* expertWeights,
                       int iStride = 0, int oStride = 0, cudaStream_t stream = 0);
void destroyDeepSeekMoE(void* moe);

}  // namespace xft
