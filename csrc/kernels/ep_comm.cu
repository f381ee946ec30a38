// Expert-parallel token exchange over peer memory (decode sizes), for data-parallel attention + expert-parallel MoE.
//
// The reference has no expert parallelism (its MoE layers slice every expert across the tensor-parallel ranks:
// src/layers/moe_deepseek.h, src/layers/mlp_llama.h:70-79).  Here each rank owns whole experts and only its own
// sequences' tokens, so every (token, expert) pair has to reach the expert's rank and come back:
//
//   plan      (home rank)    pair i -> destination rank d and a slot p in d's receive area for this source
//   dispatch  (home rank)    the token's hidden row is stored straight into rank d's receive area [src][p] over NVLink,
//                            next to {expert id, pair index}; the CTA that finishes last publishes the per-destination
//                            counts as {count, epoch} words
//   receive   (expert rank)  waits (bounded) for the count word of every source and writes the expert id of every
//                            valid slot (-1 elsewhere) so that the grouped expert GEMMs can run over the whole area
//   return    (expert rank)  the expert output of slot [src][p] is stored into the source's return area at the pair
//                            index; the last CTA raises {epoch} words at every source
//   combine   (home rank)    waits (bounded) for every rank's return word, then
//                            y[t] = sum_k w[t,k] * ret[t*k + k] (+ shared expert output) (+ residual)
//
// Nothing synchronises with the host, so the exchange can sit inside a CUDA graph; no buffer needs double buffering:
// a source starts the next exchange only after its combine, which needs the return word of every expert rank, and a
// rank returns only after its GEMMs have read the whole receive area.  Peer memory is touched with plain stores; every
// wait is bounded and reports XFT_ERR_WAIT_PEER / XFT_ERR_BOUNDS through the status word.
#include "ptx.cuh"

namespace xft {

struct EpParams {
  int world, rank;
  __nv_bfloat16* rx_tok[8];          // rank r's receive area [world][cap][H], as mapped here
  int* rx_meta[8];                   // rank r's [world][cap][2] = {expert id, pair index at the source}
  unsigned long long* rx_cnt[8];     // rank r's [world] words {count, epoch}
  __nv_bfloat16* ret[8];             // rank r's return area [pairs_cap][H]
  unsigned long long* ret_flag[8];   // rank r's [world] words {0, epoch}
  int* epoch;                        // local: completed exchanges
  int* done;                         // local: [3] CTA counters of dispatch / return / combine
  int cap;                           // slots per source in a receive area
  int pairs_cap;                     // rows of a return area
  int H;
  long long wait_cycles;
  int* status;
};

__device__ __forceinline__ unsigned long long ld_acquire_sys_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// Bounded wait for a {payload, epoch} word; returns false on time-out.
__device__ __forceinline__ bool ep_wait_word(const unsigned long long* p, int epoch, long long limit, unsigned* payload) {
  unsigned long long w = ld_acquire_sys_u64(p);
  if ((int)(w >> 32) != epoch) {
    const long long t0 = clock64();
    do {
      if (clock64() - t0 > limit) return false;
      w = ld_acquire_sys_u64(p);
    } while ((int)(w >> 32) != epoch);
  }
  *payload = (unsigned)w;
  return true;
}

// rank that owns expert e when E experts are laid out in contiguous blocks over `world` ranks (remainder first)
__device__ __forceinline__ int ep_owner(int e, int E, int world) {
  const int base = E / world, rem = E % world;
  const int cut = rem * (base + 1);
  if (e < cut) return e / (base + 1);
  return rem + (e - cut) / max(base, 1);
}

// pair i = (token i / k, choice i % k) -> dest[i], slot[i]; cnt[d] = pairs going to rank d
__global__ void __launch_bounds__(1024) ep_plan_kernel(const int* __restrict__ idx, int n_pairs, int E, const EpParams p,
                                                       int* __restrict__ dest, int* __restrict__ slot,
                                                       int* __restrict__ cnt) {
  __shared__ int s_cnt[8];
  grid_dep_launch();
  grid_dep_wait();
  if (threadIdx.x < 8) s_cnt[threadIdx.x] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int e = idx[i];
    int d = -1, s = -1;
    if (e >= 0 && e < E && i < p.pairs_cap) {
      d = ep_owner(e, E, p.world);
      s = atomicAdd(&s_cnt[d], 1);
      if (s >= p.cap) {                                // does not fit the receive area: drop and report
        if (p.status) atomicCAS(p.status, 0, XFT_ERR_BOUNDS);
        d = -1;
      }
    } else if (p.status) {                             // bad expert id, or a pair beyond the return area: no slot is taken
      atomicCAS(p.status, 0, XFT_ERR_BOUNDS);
    }
    dest[i] = d;
    slot[i] = s;
  }
  __syncthreads();
  if (threadIdx.x < p.world) cnt[threadIdx.x] = min(s_cnt[threadIdx.x], p.cap);
}

// one CTA per pair: hidden row -> the destination's receive area; last CTA publishes the counts
__global__ void __launch_bounds__(128) ep_dispatch_kernel(const __nv_bfloat16* __restrict__ x, int ldx,
                                                          const int* __restrict__ idx, int n_pairs, int k,
                                                          const int* __restrict__ dest, const int* __restrict__ slot,
                                                          const int* __restrict__ cnt, const EpParams p) {
  __shared__ int s_last;
  grid_dep_launch();
  grid_dep_wait();
  const int i = blockIdx.x;
  if (i < n_pairs) {
    const int d = dest[i];
    if (d >= 0) {
      const size_t row = (size_t)p.rank * p.cap + slot[i];
      const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(i / k) * ldx);
      uint4* dst = reinterpret_cast<uint4*>(p.rx_tok[d] + row * p.H);
      for (int c = threadIdx.x; c < p.H / 8; c += blockDim.x) dst[c] = src[c];
      if (threadIdx.x == 0) {
        p.rx_meta[d][row * 2] = idx[i];
        p.rx_meta[d][row * 2 + 1] = i;
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(&p.done[0], 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (s_last) {
    const int epoch = *reinterpret_cast<volatile int*>(p.epoch) + 1;
    if (threadIdx.x == 0) p.done[0] = 0;
    __threadfence_system();
    if (threadIdx.x < p.world)
      st_release_sys_u64(p.rx_cnt[threadIdx.x] + p.rank,
                         ((unsigned long long)(unsigned)epoch << 32) | (unsigned)cnt[threadIdx.x]);
  }
}

// expert rank: wait for every source's count; idx_out[src * cap + slot] = expert id of a valid slot, -1 otherwise
__global__ void __launch_bounds__(1024) ep_receive_kernel(const EpParams p, int* __restrict__ idx_out,
                                                          int* __restrict__ cnt_out) {
  __shared__ int s_cnt[8];
  __shared__ int s_fail;
  grid_dep_launch();
  grid_dep_wait();
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  const int epoch = *reinterpret_cast<volatile int*>(p.epoch) + 1;
  if (threadIdx.x < p.world) {
    unsigned c = 0;
    if (!ep_wait_word(p.rx_cnt[p.rank] + threadIdx.x, epoch, p.wait_cycles, &c)) {
      if (p.status) atomicCAS(p.status, 0, XFT_ERR_WAIT_PEER);
      s_fail = 1;
      c = 0;
    }
    s_cnt[threadIdx.x] = min((int)c, p.cap);
  }
  __syncthreads();
  const int total = p.world * p.cap;
  for (int j = threadIdx.x; j < total; j += blockDim.x) {
    const int s = j / p.cap, q = j % p.cap;
    idx_out[j] = (!s_fail && q < s_cnt[s]) ? __ldcg(p.rx_meta[p.rank] + (size_t)j * 2) : -1;   // written by a peer: read at L2
  }
  if (threadIdx.x < p.world) cnt_out[threadIdx.x] = s_fail ? 0 : s_cnt[threadIdx.x];
}

// expert rank: one CTA per slot; the expert output goes to the source's return area at the pair index
__global__ void __launch_bounds__(128) ep_return_kernel(const float* __restrict__ y, const int* __restrict__ cnt,
                                                        const EpParams p) {
  __shared__ int s_last;
  grid_dep_launch();
  grid_dep_wait();
  const int j = blockIdx.x;
  const int s = j / p.cap, q = j % p.cap;
  if (s < p.world && q < cnt[s]) {
    const int pair = __ldcg(p.rx_meta[p.rank] + (size_t)j * 2 + 1);
    if (pair >= 0 && pair < p.pairs_cap) {
      const float4* src = reinterpret_cast<const float4*>(y + (size_t)j * p.H);
      uint2* dst = reinterpret_cast<uint2*>(p.ret[s] + (size_t)pair * p.H);
      for (int c = threadIdx.x; c < p.H / 4; c += blockDim.x) {
        const float4 v = src[c];
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 o;
        o.x = *reinterpret_cast<unsigned*>(&a);
        o.y = *reinterpret_cast<unsigned*>(&b);
        dst[c] = o;
      }
    } else if (p.status && threadIdx.x == 0) {
      atomicCAS(p.status, 0, XFT_ERR_BOUNDS);
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(&p.done[1], 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (s_last) {
    const int epoch = *reinterpret_cast<volatile int*>(p.epoch) + 1;
    if (threadIdx.x == 0) p.done[1] = 0;
    __threadfence_system();
    if (threadIdx.x < p.world)
      st_release_sys_u64(p.ret_flag[threadIdx.x] + p.rank, (unsigned long long)(unsigned)epoch << 32);
  }
}

// home rank: y[t] = sum_k w[t,k] * ret[t*k + k] + add1[t] + add2[t]; one CTA per token (at least one CTA, which also
// closes the exchange: the last CTA bumps the epoch)
__global__ void __launch_bounds__(256) ep_combine_kernel(const float* __restrict__ w, const int* __restrict__ dest, int T,
                                                         int k, const float* __restrict__ add1,
                                                         const __nv_bfloat16* __restrict__ add2, int ld2,
                                                         __nv_bfloat16* __restrict__ out, const EpParams p) {
  __shared__ int s_fail, s_last;
  grid_dep_launch();
  grid_dep_wait();
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  const int epoch = *reinterpret_cast<volatile int*>(p.epoch) + 1;
  if (threadIdx.x < p.world) {
    unsigned unused;
    if (!ep_wait_word(p.ret_flag[p.rank] + threadIdx.x, epoch, p.wait_cycles, &unused)) {
      if (p.status) atomicCAS(p.status, 0, XFT_ERR_WAIT_PEER);
      s_fail = 1;
    }
  }
  __syncthreads();
  const int t = blockIdx.x;
  if (t < T && !s_fail) {
    const __nv_bfloat16* mine = p.ret[p.rank];
    for (int c = threadIdx.x; c < p.H; c += blockDim.x) {
      float a = 0.f;
      for (int j = 0; j < k; ++j) {
        const int i = t * k + j;
        if (dest[i] >= 0) a += w[i] * __bfloat162float(__ldcg(mine + (size_t)i * p.H + c));
      }
      if (add1) a += add1[(size_t)t * p.H + c];
      if (add2) a += __bfloat162float(add2[(size_t)t * ld2 + c]);
      out[(size_t)t * p.H + c] = __float2bfloat16(a);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(&p.done[2], 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (s_last && threadIdx.x == 0) {
    p.done[2] = 0;
    __threadfence();
    atomicAdd(p.epoch, 1);
  }
}

}  // namespace xft

using namespace xft;

static int ep_check(const EpParams* p) {
  if (!p || p->world < 2 || p->world > 8 || p->rank < 0 || p->rank >= p->world || p->cap <= 0 || (p->H & 7)) return -10;
  return 0;
}

// idx [T, k] int32 (global expert ids).  dest / slot: [T * k] scratch, cnt: [world] scratch, all on the device.
extern "C" int xft_ep_dispatch(const void* x, int ldx, const int* idx, int T, int k, int E, int* dest, int* slot, int* cnt,
                               const EpParams* p, cudaStream_t st) {
  if (int r = ep_check(p)) return r;
  if (T < 0 || k <= 0 || (ldx & 7)) return -11;
  const int n = T * k;
  cudaError_t e = launch_pdl(ep_plan_kernel, dim3(1), dim3(1024), 0, st, idx, n, E, *p, dest, slot, cnt);
  if (e != cudaSuccess) return (int)e;
  e = launch_pdl(ep_dispatch_kernel, dim3(n > 0 ? n : 1), dim3(128), 0, st, (const __nv_bfloat16*)x, ldx, idx, n, k,
                 (const int*)dest, (const int*)slot, (const int*)cnt, *p);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

// idx_out: [world * cap] expert id per slot of this rank's receive area (-1 = empty); cnt_out: [world]
extern "C" int xft_ep_receive(int* idx_out, int* cnt_out, const EpParams* p, cudaStream_t st) {
  if (int r = ep_check(p)) return r;
  cudaError_t e = launch_pdl(ep_receive_kernel, dim3(1), dim3(1024), 0, st, *p, idx_out, cnt_out);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

// y: fp32 [world * cap, H] expert outputs per slot; cnt: the counts xft_ep_receive produced
extern "C" int xft_ep_return(const float* y, const int* cnt, const EpParams* p, cudaStream_t st) {
  if (int r = ep_check(p)) return r;
  cudaError_t e = launch_pdl(ep_return_kernel, dim3(p->world * p->cap), dim3(128), 0, st, y, cnt, *p);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

// w: fp32 [T, k] routing weights; dest: the array xft_ep_dispatch filled; add1 (fp32 [T, H]) and add2 (bf16, ld2) optional
extern "C" int xft_ep_combine(const float* w, const int* dest, int T, int k, const float* add1, const void* add2, int ld2,
                              void* out, const EpParams* p, cudaStream_t st) {
  if (int r = ep_check(p)) return r;
  cudaError_t e = launch_pdl(ep_combine_kernel, dim3(T > 0 ? T : 1), dim3(256), 0, st, w, dest, T, k, add1,
                             (const __nv_bfloat16*)add2, ld2, (__nv_bfloat16*)out, *p);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

// Size and field offsets of EpParams, for the layout check of the Python mirror.
extern "C" int xft_ep_layout(long long* out, int n) {
  const long long v[] = {sizeof(EpParams),           offsetof(EpParams, world),   offsetof(EpParams, rank),
                         offsetof(EpParams, rx_tok), offsetof(EpParams, rx_meta), offsetof(EpParams, rx_cnt),
                         offsetof(EpParams, ret),    offsetof(EpParams, ret_flag), offsetof(EpParams, epoch),
                         offsetof(EpParams, done),   offsetof(EpParams, cap),     offsetof(EpParams, pairs_cap),
                         offsetof(EpParams, H),      offsetof(EpParams, wait_cycles), offsetof(EpParams, status)};
  const int m = (int)(sizeof(v) / sizeof(v[0]));
  for (int i = 0; i < m && i < n; ++i) out[i] = v[i];
  return m;
}
