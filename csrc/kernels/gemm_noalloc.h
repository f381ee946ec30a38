// Allocation-free bf16 GEMM entry point of libxft_b200_kernels.so.
//
// This entry point has no counterpart in the reference (intel/xFasterTransformer); it exists for
// callers of this library that cannot allocate device memory: code running inside a CUDA-graph
// capture or a serving loop where a cudaMalloc would stall the device, plug-ins loaded into a
// process whose GPU memory is already fully reserved by its host application, and C callers that
// hold raw device pointers but no allocator.  They pass only inputs and outputs.
//
//   Y[T,N] = act(X[T,K] · W[N,K]^T + bias) + res_scale * residual
//
//   X  bf16 [T, ldx]   row-major activations (ldx >= K, multiple of 8 elements, 16-byte aligned base)
//   W  bf16 [N, ldw]   weight in [out, in] layout (ldw >= K, multiple of 8)
//   Y  bf16 or fp32 [T, ldo]  (out_fp32 selects)
//   bias fp32 [N] or null; residual bf16 [T, ldr] or null; act: 0 none, 1 relu, 2 silu, 3 gelu(tanh)
//
// Scratch.  The split-K partial tiles, the per-tile arrival counters and the status word of the
// kernel live in one static device array inside the library: XFT_NOALLOC_SCRATCH_BYTES bytes that
// every GPU which loads the library holds until the process exits.  Consequences:
//   * Limits: T <= XFT_NOALLOC_MAX_TOKENS and ceil(N/128) * ceil(T/tile) <= XFT_NOALLOC_MAX_TILES (tile = 16, 32,
//     64, 128 or 256 tokens, the smallest that holds T).  Larger problems are rejected with -100 before anything
//     is launched; use xft_gemm_bf16 with caller-provided scratch for those.
//   * All calls on a device share the array.  Each call clears the counters and the status word on its
//     stream before the kernel; the partial-tile area keeps the previous call's contents and is always
//     written before it is read.  Two calls that may run at the same time on one GPU (different streams,
//     or different host threads) race on the array: serialise them.
//   * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
//     device current).  Make that first call outside of any stream capture.
// The function calls no cudaMalloc / cudaFree and no allocating library routine.
//
// Returns 0 on success; negative codes are explained by xft_gemm_bf16_noalloc_strerror(); positive
// codes are cudaError_t values from the launch.
#pragma once
#include <cuda_runtime.h>

#define XFT_NOALLOC_SCRATCH_BYTES ((8u << 20) + 8192u)
#define XFT_NOALLOC_MAX_TOKENS 256
#define XFT_NOALLOC_MAX_TILES 1024

#ifdef __cplusplus
extern "C" {
#endif

int xft_gemm_bf16_noalloc(const void* X, int ldx, const void* W, int ldw, void* Y, int ldo, int out_fp32, int T, int N,
                          int K, const float* bias, const void* residual, int ldr, float res_scale, int act,
                          cudaStream_t stream);

// Kernel status of the last call on the current device (0 = ok, see ptx.cuh for the codes). Synchronises `stream`.
int xft_gemm_bf16_noalloc_status(cudaStream_t stream);

const char* xft_gemm_bf16_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
