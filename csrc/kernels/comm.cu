// Peer-memory plumbing and the stand-alone one-shot all-reduce.
//
// Replaces the reference's intra-host shared-memory all-reduce (ShmCCL: src/utils/shm_ccl.h:40-138,
// shm_ccl.cpp:29-145 — a memfd segment, per-block flags, chain accumulation) and its oneCCL calls
// (src/comm_helper/comm_helper.cpp:84-129) for small messages: on an NVSwitch box every GPU maps every
// peer's buffer (CUDA IPC) and moves data with plain stores over NVLink from inside the kernel.
//
//   xft_comm_alloc / _free / _ipc_handle / _ipc_open / _ipc_close : symmetric buffers
//   xft_allreduce_oneshot : out = sum_r in_r for small tensors (push to all peers, flag, bounded wait,
//                           sum in rank order => bit-identical on all ranks)
//
// Every wait is bounded and reports XFT_ERR_WAIT_PEER through the status word instead of spinning.
#include "ptx.cuh"

namespace xft {

struct ArParams {
  int world, rank;
  float* recv[8];          // rank r's receive area [2][world][cap] as mapped here
  int* flag[8];            // rank r's flag area   [2][nblocks_cap][8]
  int* epoch;              // local launch counter
  int* done;               // local CTA exit counter
  long long cap;           // floats per slot
  int flag_parity_stride;
  long long wait_cycles;
  int* status;
};

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

// Each CTA owns a contiguous chunk of the vector: push chunk to all ranks, flag, wait, reduce.
template <typename T>
__global__ void __launch_bounds__(256) allreduce_oneshot_kernel(const T* __restrict__ in, T* __restrict__ out,
                                                                const float* __restrict__ add_f32, long long n,
                                                                const ArParams p, const int gather) {
  __shared__ int s_epoch, s_fail;
  grid_dep_launch();
  grid_dep_wait();
  if (threadIdx.x == 0) { s_epoch = *reinterpret_cast<volatile int*>(p.epoch) + 1; s_fail = 0; }
  __syncthreads();
  const int epoch = s_epoch, par = epoch & 1;
  const long long per = (n + gridDim.x - 1) / gridDim.x;
  const long long lo = (long long)blockIdx.x * per, hi = min(n, lo + per);
  const long long pbase = (long long)par * p.world * p.cap;
  for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    float v = to_f<T>(in[i]);
    if (add_f32) v += add_f32[i];
    for (int r = 0; r < p.world; ++r) p.recv[r][pbase + (long long)p.rank * p.cap + i] = v;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < p.world) {
    const int r = threadIdx.x;
    volatile int* f = p.flag[r] + par * p.flag_parity_stride + blockIdx.x * 8 + p.rank;
    *f = epoch;
    volatile int* mine = p.flag[p.rank] + par * p.flag_parity_stride + blockIdx.x * 8 + r;
    const long long t0 = clock64();
    while (*mine < epoch) {
      if (clock64() - t0 > p.wait_cycles) {
        if (p.status) atomicCAS(p.status, 0, XFT_ERR_WAIT_PEER);
        s_fail = 1;
        break;
      }
    }
    __threadfence_system();
  }
  __syncthreads();
  if (!s_fail) {
    const float* mine = p.recv[p.rank] + pbase;
    for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) {
      if (gather) {          // all-gather: out[r][i] = rank r's contribution
        for (int r = 0; r < p.world; ++r) out[(long long)r * n + i] = from_f<T>(__ldcg(mine + (long long)r * p.cap + i));
      } else {
        float x = 0.f;       // rank order: identical bits on every rank
        for (int r = 0; r < p.world; ++r) x += __ldcg(mine + (long long)r * p.cap + i);
        out[i] = from_f<T>(x);
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(p.done, 1) == (int)gridDim.x - 1) {
      *reinterpret_cast<volatile int*>(p.done) = 0;
      __threadfence();
      atomicAdd(p.epoch, 1);
    }
  }
}

}  // namespace xft

using namespace xft;

extern "C" int xft_comm_alloc(size_t bytes, void** ptr) {
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemset(*ptr, 0, bytes);
}
extern "C" int xft_comm_free(void* ptr) { return (int)cudaFree(ptr); }
extern "C" int xft_comm_ipc_handle(void* ptr, void* handle64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) return (int)e;
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
extern "C" int xft_comm_ipc_open(const void* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  return (int)cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
}
extern "C" int xft_comm_ipc_close(void* ptr) { return (int)cudaIpcCloseMemHandle(ptr); }
extern "C" int xft_comm_handle_bytes() { return (int)sizeof(cudaIpcMemHandle_t); }

// dtype: 0 = fp32, 1 = bf16.  nblocks <= capacity of the flag area.  add_f32: optional fp32 addend applied
// to this rank's contribution before the sum (e.g. a residual on one rank).
// gather != 0: all-gather instead of sum, out is [world, n].
extern "C" int xft_allreduce_oneshot(const void* in, void* out, const float* add_f32, long long n, int dtype,
                                     const ArParams* p, int nblocks, int gather, cudaStream_t st) {
  if (!p || p->world < 2 || p->world > 8 || n > p->cap) return -10;
  if (n <= 0) return 0;
  if (nblocks < 1) nblocks = 1;
  cudaError_t e;
  if (dtype == 0)
    e = launch_pdl(allreduce_oneshot_kernel<float>, dim3(nblocks), dim3(256), 0, st, (const float*)in, (float*)out, add_f32,
                   n, *p, gather);
  else
    e = launch_pdl(allreduce_oneshot_kernel<__nv_bfloat16>, dim3(nblocks), dim3(256), 0, st, (const __nv_bfloat16*)in,
                   (__nv_bfloat16*)out, add_f32, n, *p, gather);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}
