// Top-k / top-p sampling on the device (reference: src/searchers/sample_search.cpp:118-268): top-k -> /temperature ->
// top-p prefix that never keeps fewer than 2 candidates -> softmax over the kept -> inverse CDF with ONE uniform
// draw per row.  The draw comes from the caller (a counter-based stream shared by all ranks), so every tensor-
// parallel rank picks the same token; the reference reseeds std::random_device per step instead.
//
// One CTA per row: a 32-step bisection on the order-preserving integer image of the floats finds the k-th largest
// logit, the candidates (>= threshold) are compacted into shared memory, bitonic-sorted by (value desc, index asc),
// and thread 0 walks the at most 1024 survivors.  k is clamped to [1, min(V, 1024)] (the CPU oracle applies the same
// cap).  Logits equal to the threshold are admitted in index order through a block-wide prefix count, so the kept
// set — and with it the token every tensor-parallel rank picks — does not depend on thread timing.
#include "ptx.cuh"

namespace xft {

__device__ __forceinline__ unsigned f2key(float f) {
  unsigned u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

constexpr int kMaxK = 1024;

__global__ void __launch_bounds__(1024) sample_topk_topp_kernel(const float* __restrict__ logits, int ld, int V, int k,
                                                                float top_p, float temperature,
                                                                const float* __restrict__ uniform, int* __restrict__ out) {
  __shared__ unsigned long long cand[kMaxK];      // (key << 32) | (0xffffffff - idx): sorts value desc, idx asc
  __shared__ int s_cnt;
  __shared__ unsigned s_red[32];
  grid_dep_launch();
  grid_dep_wait();
  const int row = blockIdx.x, tid = threadIdx.x;
  const float* x = logits + (size_t)row * ld;
  if (k > V) k = V;
  if (k > kMaxK) k = kMaxK;
  if (k < 1) k = 1;
  // largest threshold key with count(key >= thr) >= k
  unsigned thr = 0;
  for (int bit = 31; bit >= 0; --bit) {
    const unsigned cand_thr = thr | (1u << bit);
    unsigned c = 0;
    for (int i = tid; i < V; i += 1024) c += f2key(x[i]) >= cand_thr;
    for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
    if ((tid & 31) == 0) s_red[tid >> 5] = c;
    __syncthreads();
    unsigned tot = 0;
    for (int w = 0; w < 32; ++w) tot += s_red[w];
    __syncthreads();
    if (tot >= (unsigned)k) thr = cand_thr;
  }
  if (tid == 0) s_cnt = 0;
  for (int i = tid; i < kMaxK; i += 1024) cand[i] = 0ull;
  __syncthreads();
  // strictly greater first (always fits: fewer than k of them; their order is settled by the sort below)
  for (int i = tid; i < V; i += 1024) {
    const unsigned key = f2key(x[i]);
    if (key > thr) { const int p = atomicAdd(&s_cnt, 1); if (p < kMaxK) cand[p] = ((unsigned long long)key << 32) | (0xffffffffu - (unsigned)i); }
  }
  __syncthreads();
  // then ties with the threshold, lowest index first, until k candidates are held: chunks of 1024 logits in index
  // order, a ballot + warp totals give every tie its rank among the ties seen so far
  int held = min(s_cnt, kMaxK);                       // same value in every thread
  __syncthreads();
  for (int i0 = 0; i0 < V && held < k; i0 += 1024) {
    const int i = i0 + tid;
    const bool tie = i < V && f2key(x[i]) == thr;
    const unsigned b = __ballot_sync(0xffffffffu, tie);
    if ((tid & 31) == 0) s_red[tid >> 5] = __popc(b);
    __syncthreads();
    int before = 0, tot = 0;
    for (int w = 0; w < 32; ++w) { const int c = (int)s_red[w]; if (w < (tid >> 5)) before += c; tot += c; }
    __syncthreads();
    const int pos = held + before + __popc(b & ((1u << (tid & 31)) - 1u));
    if (tie && pos < k) cand[pos] = ((unsigned long long)thr << 32) | (0xffffffffu - (unsigned)i);
    held += tot;
  }
  __syncthreads();
  // bitonic sort, descending
  for (int size = 2; size <= kMaxK; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      const int i = tid, j = i ^ stride;
      if (j > i) {
        const bool desc = (i & size) == 0;
        const unsigned long long a = cand[i], b = cand[j];
        if ((a < b) == desc) { cand[i] = b; cand[j] = a; }
      }
      __syncthreads();
    }
  }
  if (tid == 0) {
    const int n = max(1, min(k, held));
    auto val = [&](int i) {
      unsigned key = (unsigned)(cand[i] >> 32);
      unsigned u = (key & 0x80000000u) ? (key & 0x7fffffffu) : ~key;
      return __uint_as_float(u);
    };
    const float invT = 1.f / fmaxf(temperature, 1e-6f);
    const float mx = val(0) * invT;
    float den = 0.f;
    for (int i = 0; i < n; ++i) den += __expf(val(i) * invT - mx);
    int keep = n;
    if (top_p < 1.f && n > 1) {
      float c = 0.f;
      keep = 0;
      for (int i = 0; i < n; ++i) {
        if (i >= 2 && c >= top_p) break;          // prefix whose mass before the element is < top_p, at least 2
        c += __expf(val(i) * invT - mx) / den;
        keep = i + 1;
      }
    }
    float den2 = 0.f;
    for (int i = 0; i < keep; ++i) den2 += __expf(val(i) * invT - mx);
    const float u = fminf(fmaxf(uniform[row], 0.f), 1.f - 1e-7f) * den2;
    float c = 0.f;
    int pick = keep - 1;
    for (int i = 0; i < keep; ++i) {
      c += __expf(val(i) * invT - mx);
      if (c > u) { pick = i; break; }
    }
    out[row] = (int)(0xffffffffu - (unsigned)(cand[pick] & 0xffffffffull));
  }
}

// Beam-search step on the device (reference: src/searchers/beam_search.cpp:356-540 computes log-softmax over the whole
// vocabulary and the top 2 x beams of every request on the host): per row (= one beam) the log-softmax normaliser and
// the k best entries, as (log-probability, token id) sorted by value descending, ties by lower id.  Only rows x k pairs
// leave the GPU; the host merges the beams of a request (k = 2 x beams candidates per beam are enough for the global
// top 2 x beams).  Same selection scheme as the sampler above: bisection for the k-th largest key, ordered admission of
// ties, bitonic sort of the candidates.  k <= 64.
constexpr int kBeamMaxK = 64;

__global__ void __launch_bounds__(1024) beam_topk_kernel(const float* __restrict__ logits, int ld, int V, int k,
                                                         float* __restrict__ out_logp, int* __restrict__ out_idx) {
  __shared__ unsigned long long cand[kBeamMaxK];
  __shared__ int s_cnt;
  __shared__ unsigned s_red[32];
  __shared__ float s_f[32];
  grid_dep_launch();
  grid_dep_wait();
  const int row = blockIdx.x, tid = threadIdx.x;
  const float* x = logits + (size_t)row * ld;
  if (k > V) k = V;
  if (k > kBeamMaxK) k = kBeamMaxK;
  if (k < 1) k = 1;
  // log-sum-exp of the row
  float mx = -INFINITY;
  for (int i = tid; i < V; i += 1024) mx = fmaxf(mx, x[i]);
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((tid & 31) == 0) s_f[tid >> 5] = mx;
  __syncthreads();
  mx = s_f[0];
  for (int w = 1; w < 32; ++w) mx = fmaxf(mx, s_f[w]);
  __syncthreads();
  float se = 0.f;
  for (int i = tid; i < V; i += 1024) se += expf(x[i] - mx);
  for (int o = 16; o > 0; o >>= 1) se += __shfl_xor_sync(0xffffffffu, se, o);
  if ((tid & 31) == 0) s_f[tid >> 5] = se;
  __syncthreads();
  se = 0.f;
  for (int w = 0; w < 32; ++w) se += s_f[w];
  const float lse = mx + logf(se);
  // largest threshold key with count(key >= thr) >= k
  unsigned thr = 0;
  for (int bit = 31; bit >= 0; --bit) {
    const unsigned cand_thr = thr | (1u << bit);
    unsigned c = 0;
    for (int i = tid; i < V; i += 1024) c += f2key(x[i]) >= cand_thr;
    for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
    if ((tid & 31) == 0) s_red[tid >> 5] = c;
    __syncthreads();
    unsigned tot = 0;
    for (int w = 0; w < 32; ++w) tot += s_red[w];
    __syncthreads();
    if (tot >= (unsigned)k) thr = cand_thr;
  }
  if (tid == 0) s_cnt = 0;
  if (tid < kBeamMaxK) cand[tid] = 0ull;
  __syncthreads();
  for (int i = tid; i < V; i += 1024) {
    const unsigned key = f2key(x[i]);
    if (key > thr) { const int p = atomicAdd(&s_cnt, 1); if (p < kBeamMaxK) cand[p] = ((unsigned long long)key << 32) | (0xffffffffu - (unsigned)i); }
  }
  __syncthreads();
  int held = min(s_cnt, kBeamMaxK);
  __syncthreads();
  for (int i0 = 0; i0 < V && held < k; i0 += 1024) {
    const int i = i0 + tid;
    const bool tie = i < V && f2key(x[i]) == thr;
    const unsigned b = __ballot_sync(0xffffffffu, tie);
    if ((tid & 31) == 0) s_red[tid >> 5] = __popc(b);
    __syncthreads();
    int before = 0, tot = 0;
    for (int w = 0; w < 32; ++w) { const int c = (int)s_red[w]; if (w < (tid >> 5)) before += c; tot += c; }
    __syncthreads();
    const int pos = held + before + __popc(b & ((1u << (tid & 31)) - 1u));
    if (tie && pos < k) cand[pos] = ((unsigned long long)thr << 32) | (0xffffffffu - (unsigned)i);
    held += tot;
  }
  __syncthreads();
  // bitonic sort of the 64 slots, descending (empty slots are 0 and sink to the end)
  for (int size = 2; size <= kBeamMaxK; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      if (tid < kBeamMaxK) {
        const int i = tid, j = i ^ stride;
        if (j > i) {
          const bool desc = (i & size) == 0;
          const unsigned long long a = cand[i], b = cand[j];
          if ((a < b) == desc) { cand[i] = b; cand[j] = a; }
        }
      }
      __syncthreads();
    }
  }
  if (tid < k) {
    const unsigned key = (unsigned)(cand[tid] >> 32);
    const unsigned u = (key & 0x80000000u) ? (key & 0x7fffffffu) : ~key;
    out_logp[(size_t)row * k + tid] = __uint_as_float(u) - lse;
    out_idx[(size_t)row * k + tid] = (int)(0xffffffffu - (unsigned)(cand[tid] & 0xffffffffull));
  }
}

// logits[row, id] <- l < 0 ? l*p : l/p for every id in the row's token list (src/searchers/search_utils.cpp:104-172).
// tokens: [rows, max_len] padded with -1; ids outside [vocab_offset, vocab_offset + V) belong to other ranks.
__global__ void repetition_penalty_kernel(float* __restrict__ logits, int ld, int V, const int* __restrict__ tokens,
                                          int max_len, float penalty, int vocab_offset) {
  grid_dep_launch();
  grid_dep_wait();
  const int row = blockIdx.x;
  float* x = logits + (size_t)row * ld;
  const int* tk = tokens + (size_t)row * max_len;
  for (int i = threadIdx.x; i < max_len; i += blockDim.x) {
    const int id = tk[i];
    if (id < 0) continue;
    bool first = true;                         // apply once per distinct id: only its first occurrence acts
    for (int j = 0; j < i; ++j) if (tk[j] == id) { first = false; break; }
    const int c = id - vocab_offset;
    if (first && c >= 0 && c < V) { const float l = x[c]; x[c] = l < 0.f ? l * penalty : l / penalty; }
  }
}

}  // namespace xft

using namespace xft;

extern "C" int xft_sample_topk_topp(const float* logits, int ld, int rows, int V, int k, float top_p, float temperature,
                                    const float* uniform, int* out, cudaStream_t st) {
  if (rows <= 0) return 0;
  cudaError_t e = launch_pdl(sample_topk_topp_kernel, dim3(rows), dim3(1024), 0, st, logits, ld, V, k, top_p, temperature,
                             uniform, out);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

extern "C" int xft_repetition_penalty(float* logits, int ld, int rows, int V, const int* tokens, int max_len, float penalty,
                                      int vocab_offset, cudaStream_t st) {
  if (rows <= 0 || max_len <= 0) return 0;
  cudaError_t e = launch_pdl(repetition_penalty_kernel, dim3(rows), dim3(256), 0, st, logits, ld, V, tokens, max_len, penalty,
                             vocab_offset);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

// Per row: log-softmax and its k best entries, sorted (value descending, lower id first on ties).  k <= 64 (returns -1
// above).  out_logp, out_idx: [rows, k].
extern "C" int xft_beam_topk(const float* logits, int ld, int rows, int V, int k, float* out_logp, int* out_idx,
                             cudaStream_t st) {
  if (rows <= 0) return 0;
  if (k < 1 || k > xft::kBeamMaxK || k > V) return -1;
  cudaError_t e = launch_pdl(beam_topk_kernel, dim3(rows), dim3(1024), 0, st, logits, ld, V, k, out_logp, out_idx);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}
