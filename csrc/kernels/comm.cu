// Peer-memory plumbing and the stand-alone one-shot all-reduce.
//
// Replaces the reference's intra-host shared-memory all-reduce (ShmCCL: src/utils/shm_ccl.h:40-138,
// shm_ccl.cpp:29-145 — a memfd segment, per-block flags, chain accumulation) and its oneCCL calls
// (src/comm_helper/comm_helper.cpp:84-129) for small messages: on an NVSwitch box every GPU maps every
// peer's buffer (CUDA IPC) and moves data with plain stores over NVLink from inside the kernel.
//
//   xft_comm_alloc / _free / _ipc_handle / _ipc_open / _ipc_close : symmetric buffers
//   xft_allreduce_oneshot : out = sum_r in_r (or all-gather) for small tensors: {value, epoch} words pushed to
//                           all peers, bounded wait per word, sum in rank order => bit-identical on all ranks
//
// Every wait is bounded and reports XFT_ERR_WAIT_PEER through the status word instead of spinning.
#include "ptx.cuh"

namespace xft {

// Low-latency transport: every 8-byte word on the wire is {fp32 value, 32-bit epoch}.  A receiver knows a
// value has arrived when the epoch next to it equals the epoch of the current call, so no fence, no
// separate flag and no barrier sit between the producer's store and the consumer's load: the latency of
// the collective is one NVLink store propagation.  Receive area per rank: [2 parities][world][cap] words;
// the parity alternates per call (device-side epoch counter), so a slot is rewritten only two calls later,
// when every rank has long finished reading it.
struct ArParams {
  int world, rank;
  unsigned long long* recv[8];   // rank r's receive area as mapped into this process
  int* epoch;                    // local: completed launches
  int* done;                     // local: CTAs of the current launch that have exited
  long long cap;                 // words per source slot
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

__device__ __forceinline__ unsigned long long ll_pack(float v, int epoch) {
  return ((unsigned long long)(unsigned)epoch << 32) | (unsigned long long)__float_as_uint(v);
}
// Spin (bounded) until the word carries `epoch`; returns false on time-out.
__device__ __forceinline__ bool ll_read(const unsigned long long* p, int epoch, long long wait_cycles, float* v) {
  unsigned long long w = *reinterpret_cast<const volatile unsigned long long*>(p);
  if ((int)(w >> 32) != epoch) {
    const long long t0 = clock64();
    do {
      if (clock64() - t0 > wait_cycles) return false;
      w = *reinterpret_cast<const volatile unsigned long long*>(p);
    } while ((int)(w >> 32) != epoch);
  }
  *v = __uint_as_float((unsigned)w);
  return true;
}

// out = sum over ranks (gather == 0) or out[r] = rank r's vector (gather != 0).
template <typename T>
__global__ void __launch_bounds__(256) allreduce_ll_kernel(const T* __restrict__ in, T* __restrict__ out,
                                                           const float* __restrict__ add_f32, long long n,
                                                           const ArParams p, const int gather) {
  __shared__ int s_epoch;
  grid_dep_launch();
  grid_dep_wait();
  if (threadIdx.x == 0) s_epoch = *reinterpret_cast<volatile int*>(p.epoch) + 1;
  __syncthreads();
  const int epoch = s_epoch, par = epoch & 1;
  const long long pbase = (long long)par * p.world * p.cap;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (long long i = i0; i < n; i += stride) {
    float v = to_f<T>(in[i]);
    if (add_f32) v += add_f32[i];
    const unsigned long long w = ll_pack(v, epoch);
#pragma unroll 8
    for (int r = 0; r < p.world; ++r) p.recv[r][pbase + (long long)p.rank * p.cap + i] = w;
  }
  bool ok = true;
  const unsigned long long* mine = p.recv[p.rank] + pbase;
  for (long long i = i0; i < n; i += stride) {
    float x = 0.f;
    for (int r = 0; r < p.world; ++r) {          // rank order: identical bits on every rank
      float v;
      if (!ll_read(mine + (long long)r * p.cap + i, epoch, p.wait_cycles, &v)) { ok = false; break; }
      if (gather) out[(long long)r * n + i] = from_f<T>(v);
      else x += v;
    }
    if (!ok) break;
    if (!gather) out[i] = from_f<T>(x);
  }
  if (!ok && p.status) atomicCAS(p.status, 0, XFT_ERR_WAIT_PEER);
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

// dtype: 0 = fp32, 1 = bf16.  add_f32: optional fp32 addend applied to this rank's contribution before the
// sum.  gather != 0: all-gather instead of sum, out is [world, n].
extern "C" int xft_allreduce_oneshot(const void* in, void* out, const float* add_f32, long long n, int dtype,
                                     const ArParams* p, int nblocks, int gather, cudaStream_t st) {
  if (!p || p->world < 2 || p->world > 8 || n > p->cap) return -10;
  if (n <= 0) return 0;
  if (nblocks < 1) nblocks = 1;
  cudaError_t e;
  if (dtype == 0)
    e = launch_pdl(allreduce_ll_kernel<float>, dim3(nblocks), dim3(256), 0, st, (const float*)in, (float*)out, add_f32, n,
                   *p, gather);
  else
    e = launch_pdl(allreduce_ll_kernel<__nv_bfloat16>, dim3(nblocks), dim3(256), 0, st, (const __nv_bfloat16*)in,
                   (__nv_bfloat16*)out, add_f32, n, *p, gather);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

// Size and field offsets of ArParams, for the layout check of the Python mirror.
extern "C" int xft_ar_params_layout(long long* out, int n) {
  const long long v[] = {sizeof(ArParams),         offsetof(ArParams, world), offsetof(ArParams, rank),
                         offsetof(ArParams, recv), offsetof(ArParams, epoch), offsetof(ArParams, done),
                         offsetof(ArParams, cap),  offsetof(ArParams, wait_cycles), offsetof(ArParams, status)};
  const int m = (int)(sizeof(v) / sizeof(v[0]));
  for (int i = 0; i < m && i < n; ++i) out[i] = v[i];
  return m;
}

// ---------------------------------------------------------------------------------------------- local sum
// dst[i] <- sum over s of srcs[s][i] (fp32 accumulation, one rounding), n bf16 values; every pointer is memory of THIS
// GPU.  The reduction step of the in-process (thread-rank) communicator of the C++ engine; dst may be one of the sources.
namespace xft {
struct SumSrcs { const __nv_bfloat16* p[8]; int n; };
__global__ void __launch_bounds__(256) sum_bf16_kernel(__nv_bfloat16* dst, const SumSrcs s, size_t n) {
  const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= n) return;
  float a = 0.f;
  for (int k = 0; k < s.n; ++k) a += __bfloat162float(s.p[k][i]);
  dst[i] = __float2bfloat16(a);
}
}  // namespace xft

extern "C" int xft_sum_bf16(void* dst, const void* const* srcs, int nsrc, size_t n, cudaStream_t st) {
  if (n == 0) return 0;
  if (nsrc < 1 || nsrc > 8 || !dst || !srcs) return -1;
  xft::SumSrcs s{};
  s.n = nsrc;
  for (int k = 0; k < nsrc; ++k) s.p[k] = (const __nv_bfloat16*)srcs[k];
  xft::sum_bf16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>((__nv_bfloat16*)dst, s, n);
  return (int)cudaGetLastError();
}
