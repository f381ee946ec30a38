// Memory-bound glue kernels for sm_100a: embedding gather, RMSNorm / LayerNorm, fused
// QKV-split + per-head q/k norm + RoPE + paged KV-cache append (optional int8 quantisation),
// generic RoPE, latent (MLA) cache append, gated activation, row arg-max.
//
// Reference counterparts: src/kernels/token_embedding_kernels.cpp:24-54, rmsnorm_kernels.cpp:27-180,
// layernorm_kernels.cpp:27-160, rotary_embedding_kernels.cpp:57-927, attention_kernels.h:45-69
// (storeKVCache), src/utils/quantize_util.h:22-51, decoder_util.h:495-607, src/searchers/sampling.cpp:22-131.
// All of them move each byte once with 16-byte accesses; there is no GEMM-shaped work here.
#include "ptx.cuh"

namespace xft {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
template <int NW>
__device__ __forceinline__ float block_sum(float v, float* sh) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = 0.f;
#pragma unroll
  for (int i = 0; i < NW; ++i) r += sh[i];
  __syncthreads();
  return r;
}

struct alignas(16) bf16x8 { bf16 v[8]; };

// ------------------------------------------------------------------------------ embedding
__global__ void embedding_kernel(const int* __restrict__ ids, const bf16* __restrict__ table, bf16* __restrict__ out,
                                 int H, int vocab, float scale, const bf16* __restrict__ pos_table,
                                 const int* __restrict__ positions, int pos_offset, int npos, int* status) {
  grid_dep_launch();
  grid_dep_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) { if (threadIdx.x == 0 && status) atomicCAS(status, 0, XFT_ERR_BOUNDS); id = 0; }
  const bf16x8* src = reinterpret_cast<const bf16x8*>(table + (size_t)id * H);
  const bf16x8* ps = nullptr;
  if (pos_table) {
    int p = positions[t] + pos_offset;
    if (p < 0 || p >= npos) { if (threadIdx.x == 0 && status) atomicCAS(status, 0, XFT_ERR_BOUNDS); p = 0; }
    ps = reinterpret_cast<const bf16x8*>(pos_table + (size_t)p * H);
  }
  bf16x8* dst = reinterpret_cast<bf16x8*>(out + (size_t)t * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
    bf16x8 v = src[i];
    if (scale != 1.f || ps) {
      bf16x8 pv;
      if (ps) pv = ps[i];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float x = __bfloat162float(v.v[j]) * scale;
        if (ps) x += __bfloat162float(pv.v[j]);
        v.v[j] = __float2bfloat16(x);
      }
    }
    dst[i] = v;
  }
}

// ------------------------------------------------------------------------------ norms
// y = x * rsqrt(mean(x^2)+eps) * w ; optional residual: h = x + r is written to h_out first.
template <int NT>
__global__ void __launch_bounds__(NT) rmsnorm_kernel(const bf16* __restrict__ x, int ldx, const bf16* __restrict__ res,
                                                     int ldr, const float* __restrict__ w, bf16* __restrict__ y, int ldy,
                                                     bf16* __restrict__ h_out, int H, float eps) {
  __shared__ float sh[NT / 32];
  extern __shared__ float row[];     // H floats
  grid_dep_launch();
  grid_dep_wait();
  const int t = blockIdx.x;
  const bf16x8* xp = reinterpret_cast<const bf16x8*>(x + (size_t)t * ldx);
  const bf16x8* rp = res ? reinterpret_cast<const bf16x8*>(res + (size_t)t * ldr) : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H / 8; i += NT) {
    bf16x8 v = xp[i];
    bf16x8 r;
    if (rp) r = rp[i];
    bf16x8 hv;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float f = __bfloat162float(v.v[j]);
      if (rp) { f += __bfloat162float(r.v[j]); hv.v[j] = __float2bfloat16(f); f = __bfloat162float(hv.v[j]); }
      row[i * 8 + j] = f;
      ss += f * f;
    }
    if (rp && h_out) reinterpret_cast<bf16x8*>(h_out + (size_t)t * H)[i] = hv;
  }
  ss = block_sum<NT / 32>(ss, sh);
  const float inv = rsqrtf(ss / H + eps);
  bf16x8* yp = reinterpret_cast<bf16x8*>(y + (size_t)t * ldy);
  for (int i = threadIdx.x; i < H / 8; i += NT) {
    bf16x8 o;
#pragma unroll
    for (int j = 0; j < 8; ++j) o.v[j] = __float2bfloat16(row[i * 8 + j] * inv * w[i * 8 + j]);
    yp[i] = o;
  }
}

// The same for rows of at most NT * 8 * CH elements (every hidden size in use): each thread keeps its CH chunks of
// eight values in registers between the two passes, so a row is read once and written once with nothing staged in
// shared memory.  A warp owns a row when the row is short enough (NT = 32), else a CTA of NT threads.
template <int NT, int CH>
__global__ void __launch_bounds__(NT) rmsnorm_reg_kernel(const bf16* __restrict__ x, int ldx, const bf16* __restrict__ res,
                                                         int ldr, const float* __restrict__ w, bf16* __restrict__ y, int ldy,
                                                         bf16* __restrict__ h_out, int H, float eps) {
  __shared__ float sh[NT / 32];
  grid_dep_launch();
  grid_dep_wait();
  const int t = blockIdx.x;
  const bf16x8* xp = reinterpret_cast<const bf16x8*>(x + (size_t)t * ldx);
  const bf16x8* rp = res ? reinterpret_cast<const bf16x8*>(res + (size_t)t * ldr) : nullptr;
  const int nch = H / 8;
  bf16x8 v[CH];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int i = threadIdx.x + c * NT;
    if (i < nch) {
      v[c] = xp[i];
      if (rp) {
        const bf16x8 r = rp[i];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[c].v[j] = __float2bfloat16(__bfloat162float(v[c].v[j]) + __bfloat162float(r.v[j]));
        if (h_out) reinterpret_cast<bf16x8*>(h_out + (size_t)t * H)[i] = v[c];
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) { const float f = __bfloat162float(v[c].v[j]); ss += f * f; }
    }
  }
  ss = block_sum<NT / 32>(ss, sh);
  const float inv = rsqrtf(ss / H + eps);
  bf16x8* yp = reinterpret_cast<bf16x8*>(y + (size_t)t * ldy);
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int i = threadIdx.x + c * NT;
    if (i < nch) {
      const float4 w0 = __ldg(reinterpret_cast<const float4*>(w) + 2 * i), w1 = __ldg(reinterpret_cast<const float4*>(w) + 2 * i + 1);
      const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
      bf16x8 o;
#pragma unroll
      for (int j = 0; j < 8; ++j) o.v[j] = __float2bfloat16(__bfloat162float(v[c].v[j]) * inv * wv[j]);
      yp[i] = o;
    }
  }
}

template <int NT>
__global__ void __launch_bounds__(NT) layernorm_kernel(const bf16* __restrict__ x, int ldx, const float* __restrict__ w,
                                                       const float* __restrict__ b, bf16* __restrict__ y, int ldy, int H,
                                                       float eps) {
  __shared__ float sh[NT / 32];
  extern __shared__ float row[];
  const int t = blockIdx.x;
  const bf16x8* xp = reinterpret_cast<const bf16x8*>(x + (size_t)t * ldx);
  float s = 0.f;
  for (int i = threadIdx.x; i < H / 8; i += NT) {
    bf16x8 v = xp[i];
#pragma unroll
    for (int j = 0; j < 8; ++j) { float f = __bfloat162float(v.v[j]); row[i * 8 + j] = f; s += f; }
  }
  const float mu = block_sum<NT / 32>(s, sh) / H;
  float vs = 0.f;
  for (int i = threadIdx.x; i < H; i += NT) { float d = row[i] - mu; vs += d * d; }
  const float inv = rsqrtf(block_sum<NT / 32>(vs, sh) / H + eps);
  bf16x8* yp = reinterpret_cast<bf16x8*>(y + (size_t)t * ldy);
  for (int i = threadIdx.x; i < H / 8; i += NT) {
    bf16x8 o;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      int k = i * 8 + j;
      o.v[j] = __float2bfloat16((row[k] - mu) * inv * w[k] + (b ? b[k] : 0.f));
    }
    yp[i] = o;
  }
}

// ------------------------------------------------------------------------------ gated activation (unfused fallback)
__device__ __forceinline__ float act_fn(float x, int act) {
  if (act == 1) return fmaxf(x, 0.f);
  if (act == 2) return x / (1.f + __expf(-x));
  if (act == 3) { float u = 0.7978845608028654f * (x + 0.044715f * x * x * x); return 0.5f * x * (1.f + tanhf(u)); }
  return x;
}
__global__ void gated_act_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int T, int I, int act) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)T * I) return;
  int t = i / I, c = i % I;
  float g = __bfloat162float(gu[(size_t)t * 2 * I + c]);
  float u = __bfloat162float(gu[(size_t)t * 2 * I + I + c]);
  out[i] = __float2bfloat16(act_fn(g, act) * u);
}

// ------------------------------------------------------------------------------ QKV split + qk-norm + RoPE + cache append
// One warp per (token, head).  qkv [T, (hq+2hkv)*D] bf16.  style 0 = half (pairs i, i+rot/2), 1 = interleaved.
// table [max_pos, rot] = cos(rot/2) ‖ sin(rot/2) fp32.  Cache [nb, hkv, bs, D] bf16 or int8 (+ fp32 scale [nb,hkv,bs]).
struct RopeCacheParams {
  const bf16* qkv; int ldq;
  int T, hq, hkv, D;
  const int* positions; const float* table; int rot, style, rot_off, max_pos;
  const float* q_scale; const float* q_norm_w; const float* k_norm_w; float eps;
  bf16* q_out;
  void* kc; void* vc; float* ks; float* vs; int int8_cache; int bs; long long nslots;
  const int* slots;
  int* status;
  const int* positions2;      // two-stream rotary (ChatGLM-1): a second rotation of `rot` dims at rot_off + rot, or null
};

__global__ void __launch_bounds__(128) qkv_rope_cache_kernel(const RopeCacheParams p) {
  __shared__ float sh[4][256];
  grid_dep_launch();
  grid_dep_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nheads = p.hq + 2 * p.hkv;
  const long long gw = (long long)blockIdx.x * 4 + warp;
  if (gw >= (long long)p.T * nheads) return;
  const int t = gw / nheads, h = gw % nheads;
  const int D = p.D;
  float* v = sh[warp];
  const bf16* src = p.qkv + (size_t)t * p.ldq + (size_t)h * D;
  for (int d = lane * 2; d < D; d += 64) {
    __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(src + d);
    v[d] = __low2float(x);
    v[d + 1] = __high2float(x);
  }
  __syncwarp();
  const bool is_q = h < p.hq, is_k = !is_q && h < p.hq + p.hkv;
  if ((is_q && p.q_norm_w) || (is_k && p.k_norm_w)) {
    const float* w = is_q ? p.q_norm_w : p.k_norm_w;
    float ss = 0.f;
    for (int d = lane; d < D; d += 32) ss += v[d] * v[d];
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / D + p.eps);
    // round to bf16 like a standalone norm kernel would before RoPE
    for (int d = lane; d < D; d += 32) v[d] = __bfloat162float(__float2bfloat16(v[d] * inv * w[d]));
    __syncwarp();
  }
  if ((is_q || is_k) && p.table && p.rot > 0) {
    int pos = p.positions[t];
    if (pos < 0 || pos >= p.max_pos) { if (lane == 0 && p.status) atomicCAS(p.status, 0, XFT_ERR_BOUNDS); pos = 0; }
    const float* cs = p.table + (size_t)pos * p.rot;
    const int half = p.rot / 2;
    for (int i = lane; i < half; i += 32) {
      const float c = cs[i], s = cs[half + i];
      const int a = p.rot_off + (p.style == 0 ? i : 2 * i);
      const int b = p.rot_off + (p.style == 0 ? i + half : 2 * i + 1);
      const float x1 = v[a], x2 = v[b];
      v[a] = x1 * c - x2 * s;
      v[b] = x2 * c + x1 * s;
    }
    if (p.positions2) {
      int pos2 = p.positions2[t];
      if (pos2 < 0 || pos2 >= p.max_pos) { if (lane == 0 && p.status) atomicCAS(p.status, 0, XFT_ERR_BOUNDS); pos2 = 0; }
      const float* cs2 = p.table + (size_t)pos2 * p.rot;
      const int off2 = p.rot_off + p.rot;
      for (int i = lane; i < half; i += 32) {
        const float c = cs2[i], s = cs2[half + i];
        const int a = off2 + (p.style == 0 ? i : 2 * i);
        const int b = off2 + (p.style == 0 ? i + half : 2 * i + 1);
        const float x1 = v[a], x2 = v[b];
        v[a] = x1 * c - x2 * s;
        v[b] = x2 * c + x1 * s;
      }
    }
    __syncwarp();
  }
  if (is_q) {
    const float qs = p.q_scale ? p.q_scale[t] : 1.f;
    bf16* dst = p.q_out + ((size_t)t * p.hq + h) * D;
    for (int d = lane * 2; d < D; d += 64)
      *reinterpret_cast<__nv_bfloat162*>(dst + d) = __floats2bfloat162_rn(v[d] * qs, v[d + 1] * qs);
    return;
  }
  const int kh = is_k ? h - p.hq : h - p.hq - p.hkv;
  const long long slot = p.slots[t];
  if (slot < 0 || slot >= p.nslots) { if (lane == 0 && p.status) atomicCAS(p.status, 0, XFT_ERR_BOUNDS); return; }
  const long long blk = slot / p.bs, off = slot % p.bs;
  const size_t base = ((size_t)(blk * p.hkv + kh) * p.bs + off);
  if (p.int8_cache) {
    float am = 0.f;
    for (int d = lane; d < D; d += 32) am = fmaxf(am, fabsf(v[d]));
    am = warp_max(am);
    const float sc = am / 127.f;
    const float inv = sc > 1e-20f ? 1.f / sc : 0.f;
    int8_t* dst = reinterpret_cast<int8_t*>(is_k ? p.kc : p.vc) + base * D;
    for (int d = lane; d < D; d += 32) {
      float r = rintf(v[d] * inv);
      dst[d] = (int8_t)fminf(fmaxf(r, -127.f), 127.f);
    }
    if (lane == 0) (is_k ? p.ks : p.vs)[base] = sc;
  } else {
    bf16* dst = reinterpret_cast<bf16*>(is_k ? p.kc : p.vc) + base * D;
    for (int d = lane * 2; d < D; d += 64)
      *reinterpret_cast<__nv_bfloat162*>(dst + d) = __floats2bfloat162_rn(v[d], v[d + 1]);
  }
}

// ------------------------------------------------------------------------------ generic RoPE on x [T, nh, D] (in place)
__global__ void rope_kernel(bf16* __restrict__ x, int T, int nh, int D, const int* __restrict__ positions,
                            const float* __restrict__ table, int rot, int style, int rot_off, int max_pos,
                            const float* __restrict__ q_scale, int* status) {
  const long long gw = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= (long long)T * nh) return;
  const int t = gw / nh;
  bf16* v = x + (size_t)gw * D;
  int pos = positions[t];
  if (pos < 0 || pos >= max_pos) { if (lane == 0 && status) atomicCAS(status, 0, XFT_ERR_BOUNDS); pos = 0; }
  const float* cs = table + (size_t)pos * rot;
  const int half = rot / 2;
  const float qs = q_scale ? q_scale[t] : 1.f;
  for (int i = lane; i < half; i += 32) {
    const float c = cs[i], s = cs[half + i];
    const int a = rot_off + (style == 0 ? i : 2 * i);
    const int b = rot_off + (style == 0 ? i + half : 2 * i + 1);
    const float x1 = __bfloat162float(v[a]), x2 = __bfloat162float(v[b]);
    v[a] = __float2bfloat16((x1 * c - x2 * s) * qs);
    v[b] = __float2bfloat16((x2 * c + x1 * s) * qs);
  }
  if (q_scale)
    for (int d = lane; d < D; d += 32)
      if (d < rot_off || d >= rot_off + rot) v[d] = __float2bfloat16(__bfloat162float(v[d]) * qs);
}

// latent [T, W] -> cache [nb, 1, bs, W] rows at slots
__global__ void latent_write_kernel(const bf16* __restrict__ latent, int ld, bf16* __restrict__ cache, int W,
                                    const int* __restrict__ slots, long long nslots, int T, int* status) {
  const int t = blockIdx.x;
  const long long slot = slots[t];
  if (slot < 0 || slot >= nslots) { if (threadIdx.x == 0 && status) atomicCAS(status, 0, XFT_ERR_BOUNDS); return; }
  for (int d = threadIdx.x; d < W; d += blockDim.x) cache[(size_t)slot * W + d] = latent[(size_t)t * ld + d];
}

// Everything between the MLA projections and the MLA attention kernel in one launch (reference: the QKPO + cache-store
// steps of DeepSeekAttention, src/layers/attention_deepseek.h): one warp per (token, head) splits a query head into its
// no-position part [nope] and its rotated part [rope] (interleaved pairs); one more warp per token RMS-normalises the
// compressed KV [kvl], rotates the shared key part [rope] and stores both as the token's latent row in the paged cache.
struct MlaPrepParams {
  const bf16* q; int ldq;            // [T, Hl * (nope + rope)]
  const bf16* kv; int ldkv;          // [T, kvl + rope]
  int T, Hl, nope, rope, kvl;
  const int* positions; const float* table; int max_pos;      // table [max_pos, rope] = cos(rope/2) ‖ sin(rope/2)
  const float* kv_norm_w; float eps;
  bf16* q_nope; bf16* q_rope;        // [T, Hl, nope] (or [Hl, T, nope] with nope_head_major), [T, Hl, rope]
  bf16* cache; long long nslots; const int* slots;            // [nslots, kvl + rope]
  int* status;
  int nope_head_major;               // the per-head absorb GEMM reads its rows grouped by head
};

__global__ void __launch_bounds__(128) mla_prep_kernel(const MlaPrepParams p) {
  grid_dep_launch();
  grid_dep_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long gw = (long long)blockIdx.x * 4 + warp;
  if (gw >= (long long)p.T * (p.Hl + 1)) return;
  const int t = (int)(gw / (p.Hl + 1)), h = (int)(gw % (p.Hl + 1));
  int pos = p.positions[t];
  if (pos < 0 || pos >= p.max_pos) { if (lane == 0 && p.status) atomicCAS(p.status, 0, XFT_ERR_BOUNDS); pos = 0; }
  const float* cs = p.table + (size_t)pos * p.rope;
  const int half = p.rope / 2;
  if (h < p.Hl) {
    const bf16* src = p.q + (size_t)t * p.ldq + (size_t)h * (p.nope + p.rope);
    bf16* dn = p.q_nope + (p.nope_head_major ? (size_t)h * p.T + t : (size_t)t * p.Hl + h) * p.nope;
    for (int d = lane * 2; d < p.nope; d += 64)
      *reinterpret_cast<__nv_bfloat162*>(dn + d) = *reinterpret_cast<const __nv_bfloat162*>(src + d);
    bf16* dr = p.q_rope + ((size_t)t * p.Hl + h) * p.rope;
    for (int i = lane; i < half; i += 32) {
      const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(src + p.nope + 2 * i);
      const float x1 = __low2float(x), x2 = __high2float(x), c = cs[i], s = cs[half + i];
      *reinterpret_cast<__nv_bfloat162*>(dr + 2 * i) = __floats2bfloat162_rn(x1 * c - x2 * s, x2 * c + x1 * s);
    }
    return;
  }
  const long long slot = p.slots[t];
  if (slot < 0 || slot >= p.nslots) { if (lane == 0 && p.status) atomicCAS(p.status, 0, XFT_ERR_BOUNDS); return; }
  const bf16* src = p.kv + (size_t)t * p.ldkv;
  bf16* dst = p.cache + (size_t)slot * (p.kvl + p.rope);
  float ss = 0.f;
  for (int d = lane * 2; d < p.kvl; d += 64) {
    const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(src + d);
    ss += __low2float(x) * __low2float(x) + __high2float(x) * __high2float(x);
  }
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / p.kvl + p.eps);
  for (int d = lane * 2; d < p.kvl; d += 64) {
    const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(src + d);
    *reinterpret_cast<__nv_bfloat162*>(dst + d) =
        __floats2bfloat162_rn(__low2float(x) * inv * p.kv_norm_w[d], __high2float(x) * inv * p.kv_norm_w[d + 1]);
  }
  for (int i = lane; i < half; i += 32) {
    const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(src + p.kvl + 2 * i);
    const float x1 = __low2float(x), x2 = __high2float(x), c = cs[i], s = cs[half + i];
    *reinterpret_cast<__nv_bfloat162*>(dst + p.kvl + 2 * i) = __floats2bfloat162_rn(x1 * c - x2 * s, x2 * c + x1 * s);
  }
}

// ------------------------------------------------------------------------------ row arg-max (first max wins)
template <int NT>
__global__ void __launch_bounds__(NT) argmax_kernel(const float* __restrict__ logits, int ld, int V, float* __restrict__ vals,
                                                    int* __restrict__ idx) {
  __shared__ float sv[NT / 32];
  __shared__ int si[NT / 32];
  grid_dep_launch();
  grid_dep_wait();
  const float* row = logits + (size_t)blockIdx.x * ld;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += NT) {
    float x = row[i];
    if (x > best || (x == best && i < bi)) { best = x; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < NT / 32; ++w)
      if (sv[w] > best || (sv[w] == best && si[w] < bi)) { best = sv[w]; bi = si[w]; }
    vals[blockIdx.x] = best;
    idx[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
  }
}

}  // namespace xft

using namespace xft;

extern "C" int xft_embedding(const int* ids, const void* table, void* out, int T, int H, int vocab, float scale,
                             const void* pos_table, const int* positions, int pos_offset, int npos, int* status,
                             cudaStream_t st) {
  if (T <= 0) return 0;
  if (H % 8) return -1;
  cudaError_t e = launch_pdl(embedding_kernel, dim3(T), dim3(128), 0, st, ids, (const bf16*)table, (bf16*)out, H, vocab,
                             scale, (const bf16*)pos_table, positions, pos_offset, npos, status);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

extern "C" int xft_rmsnorm(const void* x, int ldx, const void* res, int ldr, const float* w, void* y, int ldy, void* h_out,
                           int T, int H, float eps, cudaStream_t st) {
  if (T <= 0) return 0;
  if (H % 8 || ldx % 8 || ldy % 8 || (res && ldr % 8)) return -1;
  cudaError_t e;
  const bool w16 = (reinterpret_cast<uintptr_t>(w) & 15) == 0;
  if (w16 && H >= 2048 && H <= 256 * 8 * 4)
    e = launch_pdl(rmsnorm_reg_kernel<256, 4>, dim3(T), dim3(256), 0, st, (const bf16*)x, ldx, (const bf16*)res, ldr, w,
                   (bf16*)y, ldy, (bf16*)h_out, H, eps);
  else if (w16 && H >= 2048 && H <= 512 * 8 * 4)
    e = launch_pdl(rmsnorm_reg_kernel<512, 4>, dim3(T), dim3(512), 0, st, (const bf16*)x, ldx, (const bf16*)res, ldr, w,
                   (bf16*)y, ldy, (bf16*)h_out, H, eps);
  else if (H >= 2048)
    e = launch_pdl(rmsnorm_kernel<256>, dim3(T), dim3(256), H * sizeof(float), st, (const bf16*)x, ldx, (const bf16*)res,
                   ldr, w, (bf16*)y, ldy, (bf16*)h_out, H, eps);
  else
    e = launch_pdl(rmsnorm_kernel<64>, dim3(T), dim3(64), H * sizeof(float), st, (const bf16*)x, ldx, (const bf16*)res,
                   ldr, w, (bf16*)y, ldy, (bf16*)h_out, H, eps);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

extern "C" int xft_layernorm(const void* x, int ldx, const float* w, const float* b, void* y, int ldy, int T, int H,
                             float eps, cudaStream_t st) {
  if (T <= 0) return 0;
  if (H % 8 || ldx % 8 || ldy % 8) return -1;
  layernorm_kernel<256><<<T, 256, H * sizeof(float), st>>>((const bf16*)x, ldx, w, b, (bf16*)y, ldy, H, eps);
  return (int)cudaGetLastError();
}

extern "C" int xft_gated_act(const void* gu, void* out, int T, int I, int act, cudaStream_t st) {
  size_t n = (size_t)T * I;
  if (!n) return 0;
  gated_act_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>((const bf16*)gu, (bf16*)out, T, I, act);
  return (int)cudaGetLastError();
}

extern "C" int xft_qkv_rope_cache(const void* qkv, int ldq, int T, int hq, int hkv, int D, const int* positions,
                                  const float* table, int rot, int style, int rot_off, int max_pos, const float* q_scale,
                                  const float* q_norm_w, const float* k_norm_w, float eps, void* q_out, void* kc,
                                  void* vc, float* ks, float* vs, int int8_cache, int bs, long long nslots,
                                  const int* slots, int* status, cudaStream_t st) {
  if (T <= 0) return 0;
  if (D > 256 || D % 2) return -1;
  RopeCacheParams p{(const bf16*)qkv, ldq, T, hq, hkv, D, positions, table, rot, style, rot_off, max_pos, q_scale,
                    q_norm_w, k_norm_w, eps, (bf16*)q_out, kc, vc, ks, vs, int8_cache, bs, nslots, slots, status};
  long long warps = (long long)T * (hq + 2 * hkv);
  cudaError_t e = launch_pdl(qkv_rope_cache_kernel, dim3((unsigned)((warps + 3) / 4)), dim3(128), 0, st, p);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

// Two-stream rotary of ChatGLM-1 (reference: src/layers/rope_2d.cpp) in the same launch as the split and the cache
// append: dims [0, rot) of every q / k head turn by positions[t], dims [rot, 2 rot) by positions2[t], both from one
// table [max_pos, rot]; 2 rot <= D.
extern "C" int xft_qkv_rope2d_cache(const void* qkv, int ldq, int T, int hq, int hkv, int D, const int* positions,
                                    const int* positions2, const float* table, int rot, int max_pos, void* q_out,
                                    void* kc, void* vc, float* ks, float* vs, int int8_cache, int bs, long long nslots,
                                    const int* slots, int* status, cudaStream_t st) {
  if (T <= 0) return 0;
  if (D > 256 || D % 2 || rot <= 0 || rot % 2 || 2 * rot > D || !positions || !positions2 || !table) return -1;
  RopeCacheParams p{(const bf16*)qkv, ldq, T, hq, hkv, D, positions, table, rot, 0, 0, max_pos, nullptr,
                    nullptr, nullptr, 0.f, (bf16*)q_out, kc, vc, ks, vs, int8_cache, bs, nslots, slots, status,
                    positions2};
  long long warps = (long long)T * (hq + 2 * hkv);
  cudaError_t e = launch_pdl(qkv_rope_cache_kernel, dim3((unsigned)((warps + 3) / 4)), dim3(128), 0, st, p);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

extern "C" int xft_rope(void* x, int T, int nh, int D, const int* positions, const float* table, int rot, int style,
                        int rot_off, int max_pos, const float* q_scale, int* status, cudaStream_t st) {
  long long warps = (long long)T * nh;
  if (warps <= 0) return 0;
  rope_kernel<<<(unsigned)((warps * 32 + 127) / 128), 128, 0, st>>>((bf16*)x, T, nh, D, positions, table, rot, style,
                                                                    rot_off, max_pos, q_scale, status);
  return (int)cudaGetLastError();
}

extern "C" int xft_latent_write(const void* latent, int ld, void* cache, int W, const int* slots, long long nslots, int T,
                                int* status, cudaStream_t st) {
  if (T <= 0) return 0;
  latent_write_kernel<<<T, 128, 0, st>>>((const bf16*)latent, ld, (bf16*)cache, W, slots, nslots, T, status);
  return (int)cudaGetLastError();
}

// src [A, B, D] bf16 -> dst [B, A, D] (D a multiple of 8, 16-byte aligned rows): per-head results [heads, tokens, D] back
// to token-major rows for the output projection.
__global__ void __launch_bounds__(128) swap_outer_dims_kernel(const bf16* __restrict__ src, bf16* __restrict__ dst, int A,
                                                              int B, int D) {
  grid_dep_launch();
  grid_dep_wait();
  const long long row = blockIdx.x;            // a * B + b
  const int a = (int)(row / B), b = (int)(row % B);
  const bf16x8* s = reinterpret_cast<const bf16x8*>(src + row * D);
  bf16x8* d = reinterpret_cast<bf16x8*>(dst + ((long long)b * A + a) * D);
  for (int i = threadIdx.x; i < D / 8; i += 128) d[i] = s[i];
}

extern "C" int xft_swap_outer_dims(const void* src, void* dst, int A, int B, int D, cudaStream_t st) {
  if (A <= 0 || B <= 0 || D <= 0) return 0;
  if (D % 8 || (((uintptr_t)src | (uintptr_t)dst) & 15)) return -1;
  cudaError_t e = launch_pdl(swap_outer_dims_kernel, dim3((unsigned)((long long)A * B)), dim3(128), 0, st, (const bf16*)src,
                             (bf16*)dst, A, B, D);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

// q rows [T, Hl * (nope + rope)] (row stride ldq), kv rows [T, kvl + rope] (row stride ldkv); all of nope, rope, kvl,
// ldq, ldkv and the cache row width even, pointers 4-byte aligned.  With nope_head_major the no-position parts are
// written as [Hl, T, nope].
extern "C" int xft_mla_prep(const void* q, int ldq, const void* kv, int ldkv, int T, int Hl, int nope, int rope, int kvl,
                            const int* positions, const float* table, int max_pos, const float* kv_norm_w, float eps,
                            void* q_nope, void* q_rope, void* cache, long long nslots, const int* slots, int* status,
                            int nope_head_major, cudaStream_t st) {
  if (T <= 0) return 0;
  if (Hl <= 0 || nope < 0 || rope <= 0 || kvl <= 0 || ((nope | rope | kvl | ldq | ldkv) & 1)) return -1;
  if (((uintptr_t)q | (uintptr_t)kv | (uintptr_t)q_nope | (uintptr_t)q_rope | (uintptr_t)cache) & 3) return -1;
  MlaPrepParams p{(const bf16*)q, ldq, (const bf16*)kv, ldkv, T, Hl, nope, rope, kvl, positions, table, max_pos,
                  kv_norm_w, eps, (bf16*)q_nope, (bf16*)q_rope, (bf16*)cache, nslots, slots, status, nope_head_major};
  const long long warps = (long long)T * (Hl + 1);
  cudaError_t e = launch_pdl(mla_prep_kernel, dim3((unsigned)((warps + 3) / 4)), dim3(128), 0, st, p);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

extern "C" int xft_argmax(const float* logits, int ld, int rows, int V, float* vals, int* idx, cudaStream_t st) {
  if (rows <= 0) return 0;
  cudaError_t e = launch_pdl(argmax_kernel<1024>, dim3(rows), dim3(1024), 0, st, logits, ld, V, vals, idx);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------ load-time layout kernels
// Checkpoint tensors are [in, out] (fp32 / fp16 / bf16); the device layout is bf16 [out, in].  One pass:
// convert + transpose through a padded shared-memory tile (reference: MMHelper::convertWeight / packWeight,
// src/utils/matmul_helper.h:149-562, done on the host there).
namespace xft {
template <typename S>
__device__ __forceinline__ float load_as_float(const S* p);
template <> __device__ __forceinline__ float load_as_float<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float load_as_float<__half>(const __half* p) { return __half2float(*p); }
template <> __device__ __forceinline__ float load_as_float<bf16>(const bf16* p) { return __bfloat162float(*p); }

template <typename S>
__global__ void transpose_to_bf16_kernel(const S* __restrict__ src, long long ld_src, int rows, int cols,
                                         bf16* __restrict__ dst, long long ld_dst) {
  __shared__ float tile[32][33];
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int i = threadIdx.y; i < 32; i += 8) {
    const int r = r0 + i, c = c0 + threadIdx.x;
    tile[i][threadIdx.x] = (r < rows && c < cols) ? load_as_float<S>(src + (long long)r * ld_src + c) : 0.f;
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += 8) {
    const int c = c0 + i, r = r0 + threadIdx.x;           // dst[c][r]
    if (c < cols && r < rows) dst[(long long)c * ld_dst + r] = __float2bfloat16(tile[threadIdx.x][i]);
  }
}
}  // namespace xft

// Quantise-at-load (reference: MMHelper::convertWeight, src/utils/matmul_helper.h:205-373, a host loop there): one CTA per
// output channel finds the row's range, derives scale and zero point and writes the codes.
//   mode 0: int8, asymmetric:  scale = (max - min) / 255, zero = (max + min) / 2 + scale / 2, q = rint((w - zero) / scale) in
//           [-128, 127]; `wsum` (optional) gets the sum of the codes (the W8A8 kernel's correction term)
//   mode 1: uint4, asymmetric: scale = (max - min) / 15, zero = min, q in [0, 15], two codes per byte, even index low
//   mode 2: NF4: scale = max|w|, zero = 0, q = nearest of the 16 NormalFloat levels (first on ties), packed like uint4
// Divisions are IEEE-rounded so the codes equal those of the PyTorch formulation of the same arithmetic.
namespace xft {
__constant__ float kNf4Code[16] = {-1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
                                   -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
                                   0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f,
                                   0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};

template <typename S>
__global__ void __launch_bounds__(256) quantize_rows_kernel(const S* __restrict__ w, long long ldw, int K, int mode,
                                                            uint8_t* __restrict__ q, long long ldq_bytes,
                                                            float* __restrict__ scale, float* __restrict__ zero,
                                                            float* __restrict__ wsum) {
  __shared__ float s_mx[8], s_mn[8];
  __shared__ int s_sum[8];
  const int row = blockIdx.x, tid = threadIdx.x;
  const S* src = w + (long long)row * ldw;
  float mx = -INFINITY, mn = INFINITY;
  for (int i = tid; i < K; i += 256) {
    const float v = load_as_float<S>(src + i);
    mx = fmaxf(mx, mode == 2 ? fabsf(v) : v);
    mn = fminf(mn, v);
  }
  mx = warp_max(mx);
  mn = -warp_max(-mn);
  if ((tid & 31) == 0) { s_mx[tid >> 5] = mx; s_mn[tid >> 5] = mn; }
  __syncthreads();
  mx = s_mx[0]; mn = s_mn[0];
  for (int i = 1; i < 8; ++i) { mx = fmaxf(mx, s_mx[i]); mn = fminf(mn, s_mn[i]); }
  float sc, zp;
  if (mode == 0) {
    sc = fmaxf(__fdiv_rn(__fsub_rn(mx, mn), 255.0f), 1e-10f);
    zp = __fadd_rn(__fmul_rn(__fadd_rn(mx, mn), 0.5f), __fmul_rn(0.5f, sc));
  } else if (mode == 1) {
    sc = fmaxf(__fdiv_rn(__fsub_rn(mx, mn), 15.0f), 1e-10f);
    zp = mn;
  } else {
    sc = fmaxf(mx, 1e-10f);
    zp = 0.f;
  }
  if (tid == 0) { scale[row] = sc; zero[row] = zp; }
  uint8_t* dst = q + (long long)row * ldq_bytes;
  int acc = 0;
  if (mode == 0) {
    for (int i = tid; i < K; i += 256) {
      const float r = rintf(__fdiv_rn(__fsub_rn(load_as_float<S>(src + i), zp), sc));
      const int c = (int)fminf(fmaxf(r, -128.f), 127.f);
      reinterpret_cast<int8_t*>(dst)[i] = (int8_t)c;
      acc += c;
    }
    if (wsum) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if ((tid & 31) == 0) s_sum[tid >> 5] = acc;
      __syncthreads();
      if (tid == 0) {
        int t = 0;
        for (int i = 0; i < 8; ++i) t += s_sum[i];
        wsum[row] = (float)t;
      }
    }
    return;
  }
  for (int i = tid; i < K / 2; i += 256) {         // one byte = codes 2i (low nibble) and 2i + 1 (high nibble)
    int code[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const float v = load_as_float<S>(src + 2 * i + j);
      if (mode == 1) {
        code[j] = (int)fminf(fmaxf(rintf(__fdiv_rn(__fsub_rn(v, zp), sc)), 0.f), 15.f);
      } else {
        const float xn = __fdiv_rn(v, sc);
        int best = 0;
        float bd = fabsf(__fsub_rn(xn, kNf4Code[0]));
        for (int c = 1; c < 16; ++c) {
          const float d = fabsf(__fsub_rn(xn, kNf4Code[c]));
          if (d < bd) { bd = d; best = c; }
        }
        code[j] = best;
      }
    }
    dst[i] = (uint8_t)(code[0] | (code[1] << 4));
  }
}
}  // namespace xft

// w [rows, K] (dtype 0 fp32, 1 fp16, 2 bf16; row stride ldw elements) -> codes q (row stride ldq_bytes), scale[rows],
// zero[rows], and for mode 0 optionally wsum[rows].  Modes 1 and 2 need an even K.
extern "C" int xft_quantize_rows(const void* w, int dtype, long long ldw, int rows, int K, int mode, void* q,
                                 long long ldq_bytes, float* scale, float* zero, float* wsum, cudaStream_t st) {
  if (rows <= 0 || K <= 0) return 0;
  if (mode < 0 || mode > 2 || (mode != 0 && (K & 1)) || !q || !scale || !zero) return -1;
  uint8_t* qq = (uint8_t*)q;
  if (dtype == 0) xft::quantize_rows_kernel<float><<<rows, 256, 0, st>>>((const float*)w, ldw, K, mode, qq, ldq_bytes, scale, zero, wsum);
  else if (dtype == 1) xft::quantize_rows_kernel<__half><<<rows, 256, 0, st>>>((const __half*)w, ldw, K, mode, qq, ldq_bytes, scale, zero, wsum);
  else xft::quantize_rows_kernel<xft::bf16><<<rows, 256, 0, st>>>((const xft::bf16*)w, ldw, K, mode, qq, ldq_bytes, scale, zero, wsum);
  return (int)cudaGetLastError();
}

namespace xft {
// e4m3 byte -> float (no NaN/Inf handling beyond what the format encodes: 0x7f / 0xff are NaN)
__device__ __forceinline__ float e4m3_to_float(uint8_t v) {
  const int s = v >> 7, e = (v >> 3) & 15, m = v & 7;
  float f;
  if (e == 0) f = ldexpf((float)m, -9);                 // subnormal: m * 2^-3 * 2^-6
  else if (e == 15 && m == 7) f = __int_as_float(0x7fc00000);
  else f = ldexpf(1.0f + (float)m * 0.125f, e - 7);
  return s ? -f : f;
}
__global__ void fp8_block_dequant_kernel(const uint8_t* __restrict__ src, const float* __restrict__ scale, long long rows,
                                         int cols, int block, __nv_bfloat16* __restrict__ dst) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * cols) return;
  const long long r = i / cols;
  const int c = (int)(i % cols);
  const int sc_cols = (cols + block - 1) / block;
  dst[i] = __float2bfloat16(e4m3_to_float(src[i]) * scale[(r / block) * sc_cols + c / block]);
}
}  // namespace xft

// e4m3 [rows, cols] with one fp32 scale per block x block tile (scale [ceil(rows/block), ceil(cols/block)]) -> bf16.
// `rows` may span several stacked matrices when each one's row count is a multiple of `block`.
extern "C" int xft_fp8_block_dequant(const void* src, const float* scale, long long rows, int cols, int block, void* dst,
                                     cudaStream_t st) {
  if (rows <= 0 || cols <= 0) return 0;
  if (block <= 0) return -1;
  const long long n = rows * cols;
  xft::fp8_block_dequant_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>((const uint8_t*)src, scale, rows, cols, block,
                                                                            (__nv_bfloat16*)dst);
  return (int)cudaGetLastError();
}

// src: [rows, cols] of dtype (0 fp32, 1 fp16, 2 bf16) on the device -> dst bf16 [cols, rows]
extern "C" int xft_transpose_to_bf16(const void* src, int dtype, long long ld_src, int rows, int cols, void* dst,
                                     long long ld_dst, cudaStream_t st) {
  if (rows <= 0 || cols <= 0) return 0;
  dim3 grid((cols + 31) / 32, (rows + 31) / 32), block(32, 8);
  if (dtype == 0) transpose_to_bf16_kernel<float><<<grid, block, 0, st>>>((const float*)src, ld_src, rows, cols, (bf16*)dst, ld_dst);
  else if (dtype == 1) transpose_to_bf16_kernel<__half><<<grid, block, 0, st>>>((const __half*)src, ld_src, rows, cols, (bf16*)dst, ld_dst);
  else transpose_to_bf16_kernel<bf16><<<grid, block, 0, st>>>((const bf16*)src, ld_src, rows, cols, (bf16*)dst, ld_dst);
  return (int)cudaGetLastError();
}
