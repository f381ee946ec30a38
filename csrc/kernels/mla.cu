// DeepSeek multi-head latent attention over the paged latent cache, absorbed form, for sm_100a.
//
// Reference: crossAttnByHead_DS (src/kernels/attention_kernels.h:1132-1206) — per (head, batch):
// S = (Q_nope·W_uk)·C_kv^T + Q_rope·K_rope^T, O = (softmax(S)·C_kv)·W_uv — and selfAttention_MLA (:569-766) for
// prefill.  The cache holds one 576-wide row per token: c_kv[512] ‖ k_rope[64] (src/layers/attn_deepseek.h:129-376).
//
// Here the two absorb products are grouped tcgen05 GEMMs (one group per head, gemm_sm100.cu); this kernel does the
// middle: every head reads the SAME latent rows (multi-query attention with a 576-wide key and a 512-wide value),
// so a CTA takes 16 heads of one query token as its 16 MMA rows and streams the sequence's latent tiles once.
// Per 32-key tile: warp w computes the scores of keys 8w..8w+7 over all 576 dims, the four score slices meet in
// shared memory, every warp redoes the (tiny) online-softmax bookkeeping, and warp w accumulates output
// dims 128w..128w+127.  Long sequences are split over CTAs; the slice that arrives last merges.
#include "ptx.cuh"

namespace xft {

typedef __nv_bfloat16 bf16;

constexpr int LAT = 512, ROPE = 64, DK = LAT + ROPE, MKT = 32;

struct MlaParams {
  const bf16* q_abs; long long qa_sh, qa_st;     // [head][token][512] strides in elements
  const bf16* q_rope; long long qr_sh, qr_st;    // [.][.][64]
  bf16* out; long long o_sh, o_st;               // [head][token][512]
  const bf16* cache;                             // [nb][bs][576]
  const int* block_table; int bt_stride;
  const int* cu_q; const int* kv_lens;
  int B, T, hl, bs, num_blocks;
  float scale;
  int nsplit; float* part_o; float* part_ml; int* counters;
  int* status;
};

__device__ __forceinline__ void mla_cp16(void* s, const void* g) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(s)), "l"(g) : "memory");
}
__device__ __forceinline__ void mla_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N_>
__device__ __forceinline__ void mla_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N_) : "memory"); }
__device__ __forceinline__ void mla_ldsm(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mla_ldsm_t(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mla_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t mla_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// [rows][576] bf16, 16-byte chunks XOR-swizzled by (row & 7) inside groups of 8 chunks
__device__ __forceinline__ bf16* mla_ptr(bf16* base, int row, int chunk) {
  return base + row * DK + ((chunk ^ (row & 7)) << 3);
}

// grid (tokens * head_chunks, nsplit); 128 threads
__global__ void __launch_bounds__(128) mla_attn_kernel(const MlaParams p) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);              // [16][576]
  bf16* lat = qs + 16 * DK;                                  // [2][MKT][576]
  float* sx = reinterpret_cast<float*>(lat + 2 * MKT * DK);  // [16][MKT]
  __shared__ int s_last;
  grid_dep_launch();
  grid_dep_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int chunks = (p.hl + 15) / 16;
  const int t = blockIdx.x / chunks, hc = blockIdx.x % chunks;
  const int split = blockIdx.y;
  // sequence of token t
  int b = 0;
  {
    int lo = 0, hi = p.B - 1;
    while (lo < hi) { int mid = (lo + hi + 1) >> 1; if (p.cu_q[mid] <= t) lo = mid; else hi = mid - 1; }
    b = lo;
  }
  const int q0 = p.cu_q[b], q_len = p.cu_q[b + 1] - q0;
  const int kv_len = p.kv_lens[b];
  const int qpos = kv_len - q_len + (t - q0);
  const int h0 = hc * 16, nq = min(16, p.hl - h0);
  const int n_keys = qpos + 1;                               // causal: keys 0..qpos
  const int ntiles = (n_keys + MKT - 1) / MKT;
  const int per = (ntiles + p.nsplit - 1) / p.nsplit;
  const int t_begin = split * per, t_end = min(ntiles, t_begin + per);
  const int* bt = p.block_table + (size_t)b * p.bt_stride;
  const int tiles_per_block = p.bs / MKT;

  // Q tile: row r = head h0+r : [q_abs(512) | q_rope(64)]
  for (int i = tid; i < 16 * (DK / 8); i += 128) {
    const int r = i / (DK / 8), c = i % (DK / 8);
    bf16* dst = mla_ptr(qs, r, c);
    if (r < nq) {
      const bf16* src = c < LAT / 8 ? p.q_abs + (h0 + r) * p.qa_sh + (long long)t * p.qa_st + c * 8
                                    : p.q_rope + (h0 + r) * p.qr_sh + (long long)t * p.qr_st + (c - LAT / 8) * 8;
      mla_cp16(dst, src);
    } else {
      *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
  }
  auto issue = [&](int ti, int buf) {
    if (ti < t_end) {
      int blk = bt[ti / tiles_per_block];
      if (blk < 0 || blk >= p.num_blocks) { if (tid == 0 && p.status) atomicCAS(p.status, 0, XFT_ERR_BOUNDS); blk = 0; }
      const bf16* src = p.cache + ((size_t)blk * p.bs + (ti % tiles_per_block) * MKT) * DK;
      const int valid = min(MKT, n_keys - ti * MKT);
      bf16* dstb = lat + buf * MKT * DK;
      for (int i = tid; i < MKT * (DK / 8); i += 128) {
        const int r = i / (DK / 8), c = i % (DK / 8);
        bf16* dst = mla_ptr(dstb, r, c);
        if (r < valid) mla_cp16(dst, src + (size_t)r * DK + c * 8);
        else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
      }
    }
    mla_commit();
  };

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  const int r0 = lane >> 2, r1 = r0 + 8;

  issue(t_begin, 0);
  for (int ti = t_begin; ti < t_end; ++ti) {
    const int buf = (ti - t_begin) & 1;
    issue(ti + 1, buf ^ 1);
    mla_wait<1>();
    __syncthreads();
    const bf16* kt = lat + buf * MKT * DK;
    // ---- scores of keys 8*warp .. 8*warp+7 over 576 dims ----
    float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 6
    for (int ks = 0; ks < DK / 16; ks += 2) {
      uint32_t a0[4], a1[4], bb[4];
      mla_ldsm(a0, mla_ptr(qs, (lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)));
      mla_ldsm(a1, mla_ptr(qs, (lane & 7) + ((lane >> 3) & 1) * 8, (ks + 1) * 2 + (lane >> 4)));
      // matrices: (keys, dims ks*16), (keys, ks*16+8), (keys, (ks+1)*16), (keys, (ks+1)*16+8)
      mla_ldsm(bb, mla_ptr(const_cast<bf16*>(kt), warp * 8 + (lane & 7), ks * 2 + (lane >> 3)));
      mla_mma(s, a0, bb[0], bb[1]);
      mla_mma(s, a1, bb[2], bb[3]);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int kl = warp * 8 + 2 * (lane & 3) + (e & 1);
      const int key = ti * MKT + kl;
      const int row = (e < 2) ? r0 : r1;
      sx[row * MKT + kl] = (key < n_keys && row < nq) ? s[e] * p.scale : -INFINITY;
    }
    __syncthreads();
    // ---- online softmax on the full [16][32] tile (every warp keeps identical m, l) ----
    float pv[2][8];                       // [row r0 / r1][k-step(2) x {cols 2q, 2q+1, 2q+8, 2q+9}]
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int ks = 0; ks < 2; ++ks)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int col = ks * 16 + 2 * (lane & 3) + (e & 1) + (e >> 1) * 8;
        pv[0][ks * 4 + e] = sx[r0 * MKT + col];
        pv[1][ks * 4 + e] = sx[r1 * MKT + col];
        mx0 = fmaxf(mx0, pv[0][ks * 4 + e]);
        mx1 = fmaxf(mx1, pv[1][ks * 4 + e]);
      }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m[0], mx0), mn1 = fmaxf(m[1], mx1);
    const float c0 = (mn0 == -INFINITY) ? 1.f : __expf(m[0] - mn0);
    const float c1 = (mn1 == -INFINITY) ? 1.f : __expf(m[1] - mn1);
    m[0] = mn0; m[1] = mn1;
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      pv[0][i] = (pv[0][i] == -INFINITY) ? 0.f : __expf(pv[0][i] - mn0);
      pv[1][i] = (pv[1][i] == -INFINITY) ? 0.f : __expf(pv[1][i] - mn1);
      sum0 += pv[0][i]; sum1 += pv[1][i];
    }
    l[0] = l[0] * c0 + sum0;
    l[1] = l[1] * c1 + sum1;
#pragma unroll
    for (int i = 0; i < 16; ++i) { o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1; }
    // ---- O[:, 128*warp .. +127] += P · C_kv ----
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      uint32_t a[4];
      a[0] = mla_pack(pv[0][ks * 4 + 0], pv[0][ks * 4 + 1]);
      a[1] = mla_pack(pv[1][ks * 4 + 0], pv[1][ks * 4 + 1]);
      a[2] = mla_pack(pv[0][ks * 4 + 2], pv[0][ks * 4 + 3]);
      a[3] = mla_pack(pv[1][ks * 4 + 2], pv[1][ks * 4 + 3]);
#pragma unroll
      for (int j = 0; j < 16; j += 2) {
        uint32_t bb[4];
        mla_ldsm_t(bb, mla_ptr(const_cast<bf16*>(kt), ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, warp * 16 + j + (lane >> 4)));
        mla_mma(o[j], a, bb[0], bb[1]);
        mla_mma(o[j + 1], a, bb[2], bb[3]);
      }
    }
    __syncthreads();
  }
  mla_wait<0>();
  l[0] += __shfl_xor_sync(0xffffffffu, l[0], 1); l[0] += __shfl_xor_sync(0xffffffffu, l[0], 2);
  l[1] += __shfl_xor_sync(0xffffffffu, l[1], 1); l[1] += __shfl_xor_sync(0xffffffffu, l[1], 2);

  if (p.nsplit == 1) {
    const float i0 = l[0] > 0.f ? 1.f / l[0] : 0.f, i1 = l[1] > 0.f ? 1.f / l[1] : 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int d = warp * 128 + j * 8 + 2 * (lane & 3);
      if (r0 < nq) *reinterpret_cast<uint32_t*>(p.out + (h0 + r0) * p.o_sh + (long long)t * p.o_st + d) = mla_pack(o[j][0] * i0, o[j][1] * i0);
      if (r1 < nq) *reinterpret_cast<uint32_t*>(p.out + (h0 + r1) * p.o_sh + (long long)t * p.o_st + d) = mla_pack(o[j][2] * i1, o[j][3] * i1);
    }
    return;
  }
  // ---- split: publish partials, last arriver merges ----
  const size_t tile_id = blockIdx.x;
  float* po = p.part_o + (tile_id * p.nsplit + split) * 16 * LAT;
  float* pm = p.part_ml + (tile_id * p.nsplit + split) * 32;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const int d = warp * 128 + j * 8 + 2 * (lane & 3);
    po[r0 * LAT + d] = o[j][0]; po[r0 * LAT + d + 1] = o[j][1];
    po[r1 * LAT + d] = o[j][2]; po[r1 * LAT + d + 1] = o[j][3];
  }
  if (warp == 0 && (lane & 3) == 0) { pm[r0 * 2] = m[0]; pm[r0 * 2 + 1] = l[0]; pm[r1 * 2] = m[1]; pm[r1 * 2 + 1] = l[1]; }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int old = atomicAdd(&p.counters[tile_id], 1);
    s_last = (old == p.nsplit - 1);
    if (s_last) p.counters[tile_id] = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int i = tid; i < nq * LAT; i += 128) {
    const int r = i / LAT, d = i % LAT;
    float mm = -INFINITY;
    for (int s2 = 0; s2 < p.nsplit; ++s2) mm = fmaxf(mm, __ldcg(p.part_ml + (tile_id * p.nsplit + s2) * 32 + r * 2));
    float acc = 0.f, ll = 0.f;
    for (int s2 = 0; s2 < p.nsplit; ++s2) {
      const float ms = __ldcg(p.part_ml + (tile_id * p.nsplit + s2) * 32 + r * 2);
      const float c = (ms == -INFINITY) ? 0.f : __expf(ms - mm);
      acc += c * __ldcg(p.part_o + ((tile_id * p.nsplit + s2) * 16 + r) * LAT + d);
      ll += c * __ldcg(p.part_ml + (tile_id * p.nsplit + s2) * 32 + r * 2 + 1);
    }
    p.out[(h0 + r) * p.o_sh + (long long)t * p.o_st + d] = __float2bfloat16(ll > 0.f ? acc / ll : 0.f);
  }
}

}  // namespace xft

using namespace xft;

extern "C" int xft_mla_attention(const void* q_abs, long long qa_sh, long long qa_st, const void* q_rope, long long qr_sh,
                                 long long qr_st, void* out, long long o_sh, long long o_st, const void* cache,
                                 const int* block_table, int bt_stride, const int* cu_q, const int* kv_lens, int B, int T,
                                 int hl, int bs, int num_blocks, float scale, int nsplit, float* part_o, float* part_ml,
                                 int* counters, int* status, cudaStream_t st) {
  if (T <= 0 || B <= 0) return 0;
  if (bs % MKT) return -2;
  MlaParams p{(const bf16*)q_abs, qa_sh, qa_st, (const bf16*)q_rope, qr_sh, qr_st, (bf16*)out, o_sh, o_st, (const bf16*)cache,
              block_table, bt_stride, cu_q, kv_lens, B, T, hl, bs, num_blocks, scale, nsplit < 1 ? 1 : nsplit, part_o, part_ml,
              counters, status};
  if (p.nsplit > 1 && (!part_o || !part_ml || !counters)) return -3;
  const size_t smem = (size_t)(16 * DK + 2 * MKT * DK) * 2 + 16 * MKT * sizeof(float);
  static bool attr = false;
  if (!attr) { cudaFuncSetAttribute(mla_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); attr = true; }
  const int chunks = (hl + 15) / 16;
  cudaError_t e = launch_pdl(mla_attn_kernel, dim3(T * chunks, p.nsplit), dim3(128), smem, st, p);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}
