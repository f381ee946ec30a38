// Mixture-of-experts plumbing for sm_100a: routers, the sync-free dispatch plan, row gather and the weighted combine.
//
// Reference: Mixtral top-2 on raw logits + softmax over the two (src/layers/mlp_mixtral.h:223-281); Qwen3 full
// softmax -> top-k -> renormalise (src/layers/moe_qwen3.h:283-315); DeepSeek noaux_tc — sigmoid, group score =
// sum of the top-2 biased scores of the group, keep topk_group groups, top-k experts by biased score, weights =
// unbiased scores / (sum + 1e-20) * routed_scaling_factor (src/layers/moe_deepseek.h:226-283,402-536); gather /
// scatter-add of rows (moe_deepseek.h:380-398, mlp_mixtral.h:204-219).
//
// The reference gathers on the host per expert.  Here nothing leaves the device: a plan kernel counts the rows of
// every local expert, lays the (token, slot) pairs out sorted by expert, and writes the tile table that the grouped
// tcgen05 GEMM (gemm_sm100.cu, xft_gemm_bf16_grouped) walks; the combine is a gather over each token's k slots in
// slot order, so results do not depend on where the rows landed.
#include "ptx.cuh"

namespace xft {

typedef __nv_bfloat16 bf16;

// ------------------------------------------------------------------------------------------ routers
// One warp per token.  kind: 0 mixtral, 1 softmax->topk(->renorm), 2 deepseek (sigmoid or softmax scores).
struct RouteParams {
  const float* logits; int ld; int T, E, k, kind;
  const float* bias; int n_group, topk_group; float scaling; int norm_topk; int sigmoid;
  int* idx; float* w;
};

__global__ void __launch_bounds__(128) route_kernel(const RouteParams p) {
  extern __shared__ float sm[];                 // per warp: score[E], sel[E], gscore[32]
  grid_dep_launch();
  grid_dep_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  if (t >= p.T) return;
  const int E = p.E;
  float* score = sm + warp * (2 * E + 32);
  float* sel = score + E;
  float* gs = sel + E;
  const float* x = p.logits + (size_t)t * p.ld;
  // scores
  if (p.kind == 0) {
    for (int e = lane; e < E; e += 32) { score[e] = x[e]; sel[e] = x[e]; }
  } else {
    const bool softmax = p.kind == 1 || !p.sigmoid;
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, x[e]);
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
      const float v = softmax ? __expf(x[e] - mx) : 1.f / (1.f + __expf(-x[e]));
      score[e] = v;
      sum += v;
    }
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    for (int e = lane; e < E; e += 32) {
      if (softmax) score[e] /= sum;
      sel[e] = score[e] + ((p.kind == 2 && p.bias) ? p.bias[e] : 0.f);
    }
  }
  __syncwarp();
  if (p.kind == 2 && p.n_group > 1) {
    const int gsz = E / p.n_group;
    if (lane < p.n_group) {                     // group score = sum of its two best biased scores
      float a = -INFINITY, b = -INFINITY;
      for (int i = 0; i < gsz; ++i) {
        const float v = sel[lane * gsz + i];
        if (v > a) { b = a; a = v; } else if (v > b) b = v;
      }
      gs[lane] = a + b;
    }
    __syncwarp();
    if (lane == 0) {                            // keep the topk_group best groups (first wins ties)
      unsigned keep = 0;
      for (int j = 0; j < p.topk_group; ++j) {
        int bi = -1; float bv = -INFINITY;
        for (int g = 0; g < p.n_group; ++g)
          if (!(keep >> g & 1) && (bi < 0 || gs[g] > bv)) { bv = gs[g]; bi = g; }
        keep |= 1u << bi;
      }
      gs[31] = __uint_as_float(keep);
    }
    __syncwarp();
    const unsigned keep = __float_as_uint(gs[31]);
    for (int e = lane; e < E; e += 32)
      if (!(keep >> (e / gsz) & 1)) sel[e] = -INFINITY;
    __syncwarp();
  }
  // top-k by repeated arg-max (lowest index wins ties)
  float wsum = 0.f;
  float myw = 0.f; int myi = 0;
  for (int j = 0; j < p.k; ++j) {
    float bv = -INFINITY; int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = sel[e];
      if (v > bv || (v == bv && e < bi)) { bv = v; bi = e; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (bi == 0x7fffffff) bi = 0;
    const float sc = score[bi];
    wsum += sc;
    if (lane == j) { myw = sc; myi = bi; }
    __syncwarp();
    if (lane == 0) sel[bi] = -INFINITY;
    __syncwarp();
  }
  if (lane < p.k) {
    float w = myw;
    if (p.kind == 0) {
      // softmax over the selected logits only
      float mx = -INFINITY;
      for (int j = 0; j < p.k; ++j) mx = fmaxf(mx, __shfl_sync((1u << p.k) - 1, myw, j));
      float den = 0.f;
      for (int j = 0; j < p.k; ++j) den += __expf(__shfl_sync((1u << p.k) - 1, myw, j) - mx);
      w = __expf(myw - mx) / den;
    } else if (p.kind == 1) {
      if (p.norm_topk) w = myw / wsum;
    } else {
      if (p.norm_topk) w = myw / (wsum + 1e-20f);
      w *= p.scaling;
    }
    p.idx[(size_t)t * p.k + lane] = myi;
    p.w[(size_t)t * p.k + lane] = w;
  }
}

// ------------------------------------------------------------------------------------------ dispatch plan
// One block.  Pairs (t, s) whose expert lies in [e0, e1) are placed, grouped by expert, in rows
// [0, total).  Outputs: pos[T*k] (row of the pair or -1), src_tok[row], row_w[row], tile table
// {local expert, first row, rows, 0} for token tiles of `bn` rows, meta = {num_tiles, total rows}.
struct PlanParams {
  const int* idx; const float* w; int T, k, e0, e1, bn;
  int* pos; int* src_tok; float* row_w; int4* tiles; int* meta; int max_tiles; int max_rows;
};

__global__ void __launch_bounds__(1024) moe_plan_kernel(const PlanParams p) {
  __shared__ int cnt[256], off[257], cur[256], toff[257];
  grid_dep_launch();
  grid_dep_wait();
  const int E = p.e1 - p.e0, n = p.T * p.k;
  for (int i = threadIdx.x; i < E; i += blockDim.x) { cnt[i] = 0; cur[i] = 0; }
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = p.idx[i] - p.e0;
    if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int o = 0, to = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = o; toff[e] = to;
      o += cnt[e];
      to += (cnt[e] + p.bn - 1) / p.bn;
    }
    off[E] = o; toff[E] = to;
    p.meta[0] = to > p.max_tiles ? p.max_tiles : to;
    p.meta[1] = o;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int nt = toff[e + 1] - toff[e];
    for (int j = 0; j < nt; ++j) {
      const int ti = toff[e] + j;
      if (ti < p.max_tiles) p.tiles[ti] = make_int4(e, off[e] + j * p.bn, min(p.bn, cnt[e] - j * p.bn), 0);
    }
  }
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = p.idx[i] - p.e0;
    int r = -1;
    if (e >= 0 && e < E) {
      r = off[e] + atomicAdd(&cur[e], 1);
      if (r < p.max_rows) { p.src_tok[r] = i / p.k; p.row_w[r] = p.w[i]; } else r = -1;
    }
    p.pos[i] = r;
  }
}

// Xs[row] = X[src_tok[row]] for row < total (one CTA per row slot; idle past the total)
__global__ void __launch_bounds__(128) moe_gather_kernel(const bf16* __restrict__ x, int ldx, const int* __restrict__ src_tok,
                                                         const int* __restrict__ meta, bf16* __restrict__ xs, int H) {
  grid_dep_launch();
  grid_dep_wait();
  const int r = blockIdx.x;
  if (r >= meta[1]) return;
  const uint4* s = reinterpret_cast<const uint4*>(x + (size_t)src_tok[r] * ldx);
  uint4* d = reinterpret_cast<uint4*>(xs + (size_t)r * H);
  for (int i = threadIdx.x; i < H / 8; i += 128) d[i] = s[i];
}

// y[t] = sum_s ys[pos[t,s]] (already scaled by the routing weight) + add1[t] + add2[t]   (fp32 sum, bf16 out)
__global__ void __launch_bounds__(256) moe_combine_kernel(const float* __restrict__ ys, const int* __restrict__ pos, int k,
                                                          const float* __restrict__ add1, const bf16* __restrict__ add2,
                                                          int ld2, bf16* __restrict__ y, float* __restrict__ y32, int H) {
  grid_dep_launch();
  grid_dep_wait();
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < H; i += 256) {
    float a = 0.f;
    for (int s = 0; s < k; ++s) {
      const int r = pos[t * k + s];
      if (r >= 0) a += ys[(size_t)r * H + i];
    }
    if (add1) a += add1[(size_t)t * H + i];
    if (add2) a += __bfloat162float(add2[(size_t)t * ld2 + i]);
    if (y32) y32[(size_t)t * H + i] = a;
    else y[(size_t)t * H + i] = __float2bfloat16(a);
  }
}

}  // namespace xft

using namespace xft;

extern "C" int xft_moe_route(const float* logits, int ld, int T, int E, int k, int kind, const float* bias, int n_group,
                             int topk_group, float scaling, int norm_topk, int sigmoid, int* idx, float* w, cudaStream_t st) {
  if (T <= 0) return 0;
  if (E > 4096 || k > 32 || n_group > 31) return -1;
  RouteParams p{logits, ld, T, E, k, kind, bias, n_group, topk_group, scaling, norm_topk, sigmoid, idx, w};
  const size_t smem = 4 * (2 * E + 32) * sizeof(float);
  cudaError_t e = launch_pdl(route_kernel, dim3((T + 3) / 4), dim3(128), smem, st, p);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

extern "C" int xft_moe_plan(const int* idx, const float* w, int T, int k, int e0, int e1, int bn, int* pos, int* src_tok,
                            float* row_w, void* tiles, int* meta, int max_tiles, int max_rows, cudaStream_t st) {
  if (e1 - e0 > 256 || e1 <= e0) return -1;
  PlanParams p{idx, w, T, k, e0, e1, bn, pos, src_tok, row_w, reinterpret_cast<int4*>(tiles), meta, max_tiles, max_rows};
  cudaError_t e = launch_pdl(moe_plan_kernel, dim3(1), dim3(1024), 0, st, p);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

extern "C" int xft_moe_gather(const void* x, int ldx, const int* src_tok, const int* meta, void* xs, int max_rows, int H,
                              cudaStream_t st) {
  if (max_rows <= 0) return 0;
  if (H % 8) return -1;
  cudaError_t e = launch_pdl(moe_gather_kernel, dim3(max_rows), dim3(128), 0, st, (const bf16*)x, ldx, src_tok, meta, (bf16*)xs, H);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

extern "C" int xft_moe_combine(const float* ys, const int* pos, int k, const float* add1, const void* add2, int ld2, void* y,
                               float* y32, int T, int H, cudaStream_t st) {
  if (T <= 0) return 0;
  cudaError_t e = launch_pdl(moe_combine_kernel, dim3(T), dim3(256), 0, st, ys, pos, k, add1, (const bf16*)add2, ld2, (bf16*)y,
                             y32, H);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}
