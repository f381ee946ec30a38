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

}  // namespace xft
