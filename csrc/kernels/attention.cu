// Paged-KV attention for sm_100a: causal prefill (flash, online softmax) and split-KV flash-decode.
//
// Reference kernels covered: selfAttention / selfScaledDpAttention (prefill), crossAttnByHead,
// crossAttnShardedHead (split-K decode with exp(m_i - m) merge), paged crossAttention
// (src/kernels/attention_kernels.h:142-552,838-1123,1285-1408; attention_kernels.cpp:24-156), with fp16/int8
// KV (per token·head fp32 scale, src/utils/quantize_util.h:22-51), GQA, ALiBi and the ChatGLM prefix mask.
//
// One definition serves every case: sequence b owns query rows cu_q[b]..cu_q[b+1]; its keys are cache
// positions 0..kv_len[b]-1 found through block_table[b]; query row i sits at position
// kv_len - q_len + i and sees keys <= its position.
//
// Cache layout: K, V : [num_blocks, kv_heads, BS(=64), HD]; a (block, head) pair is one contiguous
// BS x HD tile, fetched with 16-byte cp.async into XOR-swizzled shared memory and consumed through
// ldmatrix by mma.sync.m16n8k16 (bf16 in, fp32 accumulate).  Decode is bandwidth-bound (every K/V byte is
// read once): a CTA owns one kv head of one sequence and a slice of its blocks, the GQA group's query
// heads are the 16 MMA rows, the four warps walk different tiles and merge at the end; the slice that arrives
// last merges all slices.  bf16 caches are fed by TMA into a CTA-wide ring (attn_decode_tma_kernel); int8 caches
// keep the cp.async path, which converts to bf16 on the way into shared memory.  Prefill gives each warp 16 query rows of one head and shares K/V tiles
// across the CTA.
#include "ptx.cuh"

namespace xft {

typedef __nv_bfloat16 bf16;

// gemm_sm100.cu: cached 2-D tensor map with a 128-byte-wide, SWIZZLE_128B box of `box_rows` rows
int make_tensor_map(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                    uint32_t esize);

struct AttnParams {
  const bf16* q;            // [T, hq, HD]
  bf16* out;                // [T, hq, HD]
  const void* kc; const void* vc;     // paged caches
  const float* ks; const float* vs;   // int8 scales [nb, hkv, BS] or null
  const int* block_table; int bt_stride;
  const int* cu_q; const int* kv_lens;
  const float* slopes;      // [hq] or null
  const int* prefix_lens;   // [B] or null
  int hq, hkv, group, q_off, bs;
  float scale;
  int num_blocks;
  // decode split
  int nsplit; float* part_o; float* part_ml;   // [B, hq, nsplit, HD], [B, hq, nsplit, 2]
  int* split_counters;      // [B * gridDim.y] arrival counters (zero between launches)
  int* status;
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// smem tile [rows][HD] bf16, 16-byte chunks XOR-swizzled with (row & 7)
template <int HD>
__device__ __forceinline__ bf16* tile_ptr(bf16* base, int row, int chunk) {
  return base + row * HD + ((chunk ^ (row & 7)) << 3);
}

// K/V tile as a TMA box sequence: HD/64 column halves of [rows][64] bf16, each 128-byte row swizzled by the
// hardware (SWIZZLE_128B: 16-byte chunk index ^= row & 7); `rows` is the tile's key count.
template <int HD, int KT>
__device__ __forceinline__ bf16* tile_ptr_tma(bf16* base, int row, int chunk) {
  return base + (chunk >> 3) * (KT * 64) + row * 64 + (((chunk & 7) ^ (row & 7)) << 3);
}

// Copy `rows` x HD bf16 from global (row stride = gstride elements) into a swizzled tile; rows >= valid are zeroed.
template <int HD, int NT>
__device__ __forceinline__ void load_tile_bf16(bf16* tile, const bf16* g, long long gstride, int rows, int valid, int tid) {
  constexpr int CPR = HD / 8;
  for (int i = tid; i < rows * CPR; i += NT) {
    const int r = i / CPR, c = i % CPR;
    bf16* dst = tile_ptr<HD>(tile, r, c);
    if (r < valid) cp_async16(dst, g + (long long)r * gstride + c * 8);
    else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
  }
}
// int8 rows -> bf16 swizzled tile (exact conversion; the per-row scale is applied to the scores / probabilities)
template <int HD, int NT>
__device__ __forceinline__ void load_tile_int8(bf16* tile, const int8_t* g, int rows, int valid, int tid) {
  constexpr int CPR = HD / 16;     // 16 int8 per 16-byte load -> two bf16 chunks
  for (int i = tid; i < rows * CPR; i += NT) {
    const int r = i / CPR, c = i % CPR;
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (r < valid) raw = *reinterpret_cast<const uint4*>(g + (long long)r * HD + c * 16);
    const int8_t* b = reinterpret_cast<const int8_t*>(&raw);
    uint32_t w[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) w[j] = pack_bf16((float)b[2 * j], (float)b[2 * j + 1]);
    *reinterpret_cast<uint4*>(tile_ptr<HD>(tile, r, 2 * c)) = make_uint4(w[0], w[1], w[2], w[3]);
    *reinterpret_cast<uint4*>(tile_ptr<HD>(tile, r, 2 * c + 1)) = make_uint4(w[4], w[5], w[6], w[7]);
  }
}

// One warp: 16 query rows (A fragments re-read from the swizzled Q tile) against a KT-key tile.
// Updates the running max m[2], sum l[2] and O accumulator (two rows per thread: lane/4 and lane/4+8).
template <int HD, int KT, bool KV_TMA = false, int TROWS = KT>
struct WarpAttn {
  float m[2], l[2];
  float o[HD / 8][4];

  static __device__ __forceinline__ bf16* kv_ptr(const bf16* base, int row, int chunk) {
    if (KV_TMA) return tile_ptr_tma<HD, TROWS>(const_cast<bf16*>(base), row, chunk);
    return tile_ptr<HD>(const_cast<bf16*>(base), row, chunk);
  }

  __device__ __forceinline__ void init() {
    m[0] = m[1] = -INFINITY;
    l[0] = l[1] = 0.f;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  }

  // qtile: [16][HD] rows of this warp; kt/vt: [KT][HD]; key0: global index of key 0 of the tile.
  // qpos0/qpos1: positions of this thread's two query rows (-1 => row unused); kv_len bounds the keys.
  // kscale/vscale: per-key fp32 (smem) or null.
  __device__ __forceinline__ void step(const bf16* qtile, const bf16* kt, const bf16* vt, int key0, int kv_len, int qpos0,
                                       int qpos1, float scale, float slope0, float slope1, bool use_alibi, int prefix_len,
                                       const float* kscale, const float* vscale, int lane) {
    float s[KT / 8][4];
    scores(s, qtile, kt, key0, kv_len, qpos0, qpos1, scale, slope0, slope1, use_alibi, prefix_len, kscale, vscale, lane);
    pv(s, vt, lane);
  }

  // S = Q K^T for one tile
  __device__ __forceinline__ void qk(float (&s)[KT / 8][4], const bf16* qtile, const bf16* kt, int lane) {
#pragma unroll
    for (int j = 0; j < KT / 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      uint32_t a[4];
      ldsm_x4(a, tile_ptr<HD>(const_cast<bf16*>(qtile), (lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)));
#pragma unroll
      for (int j = 0; j < KT / 8; j += 2) {
        // matrices: (keys j*8.., dims ks*16), (keys j*8.., dims ks*16+8), (keys (j+1)*8.., dims ks*16), (.., +8)
        uint32_t b[4];
        ldsm_x4(b, kv_ptr(kt, j * 8 + (lane & 7) + ((lane >> 4) & 1) * 8, ks * 2 + ((lane >> 3) & 1)));
        mma16816(s[j], a, b[0], b[1]);
        mma16816(s[j + 1], a, b[2], b[3]);
      }
    }
  }

  // same with the Q fragments already in registers (qa[ks] = the ldmatrix result of k-step ks)
  __device__ __forceinline__ void qk_frag(float (&s)[KT / 8][4], const uint32_t (&qa)[HD / 16][4], const bf16* kt, int lane) {
#pragma unroll
    for (int j = 0; j < KT / 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
      for (int j = 0; j < KT / 8; j += 2) {
        uint32_t b[4];
        ldsm_x4(b, kv_ptr(kt, j * 8 + (lane & 7) + ((lane >> 4) & 1) * 8, ks * 2 + ((lane >> 3) & 1)));
        mma16816(s[j], qa[ks], b[0], b[1]);
        mma16816(s[j + 1], qa[ks], b[2], b[3]);
      }
    }
  }

  // scale, bias, mask; thread holds rows r0 = lane/4 (c0,c1) and r0+8 (c2,c3), key cols j*8 + 2*(lane%4) + {0,1}
  __device__ __forceinline__ void mask(float (&s)[KT / 8][4], int key0, int kv_len, int qpos0, int qpos1, float scale,
                                       float slope0, float slope1, bool use_alibi, int prefix_len, const float* kscale,
                                       int lane) {
#pragma unroll
    for (int j = 0; j < KT / 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int kl = j * 8 + 2 * (lane & 3) + (e & 1);
        const int key = key0 + kl;
        const int qp = (e < 2) ? qpos0 : qpos1;
        float v = s[j][e] * scale;
        if (kscale) v *= kscale[kl];
        if (use_alibi) v += ((e < 2) ? slope0 : slope1) * (float)(key - qp);
        const bool vis = key < kv_len && qp >= 0 && (key <= qp || key < prefix_len);
        s[j][e] = vis ? v : -INFINITY;
      }
    }
  }

  // online-softmax update: leaves P (scaled by vscale) in s, updates m and l, rescales O when a maximum moved
  __device__ __forceinline__ void softmax_update(float (&s)[KT / 8][4], const float* vscale, int lane) {
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < KT / 8; ++j) {
      mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
      mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m[0], mx0), mn1 = fmaxf(m[1], mx1);
    const float c0 = (mn0 == -INFINITY) ? 1.f : __expf(m[0] - mn0);
    const float c1 = (mn1 == -INFINITY) ? 1.f : __expf(m[1] - mn1);
    m[0] = mn0; m[1] = mn1;
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int j = 0; j < KT / 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float mm = (e < 2) ? mn0 : mn1;
        float pv = (s[j][e] == -INFINITY) ? 0.f : __expf(s[j][e] - mm);
        if (e < 2) sum0 += pv; else sum1 += pv;
        if (vscale) pv *= vscale[j * 8 + 2 * (lane & 3) + (e & 1)];
        s[j][e] = pv;
      }
    }
    l[0] = l[0] * c0 + sum0;     // per-thread partial row sums; reduced across the quad at the end
    l[1] = l[1] * c1 + sum1;
    if (__any_sync(0xffffffffu, c0 != 1.f || c1 != 1.f)) {   // after the first tiles the maxima rarely move
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) { o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1; }
    }
  }

  // phase 1: S = Q K^T, mask, online-softmax update; leaves P (scaled by vscale) in s and rescales O
  __device__ __forceinline__ void scores(float (&s)[KT / 8][4], const bf16* qtile, const bf16* kt, int key0, int kv_len,
                                         int qpos0, int qpos1, float scale, float slope0, float slope1, bool use_alibi,
                                         int prefix_len, const float* kscale, const float* vscale, int lane) {
    qk(s, qtile, kt, lane);
    mask(s, key0, kv_len, qpos0, qpos1, scale, slope0, slope1, use_alibi, prefix_len, kscale, lane);
    softmax_update(s, vscale, lane);
  }

  // phase 2: O += P V
  __device__ __forceinline__ void pv(float (&s)[KT / 8][4], const bf16* vt, int lane) {
#pragma unroll
    for (int ks = 0; ks < KT / 16; ++ks) {
      uint32_t a[4];
      a[0] = pack_bf16(s[2 * ks][0], s[2 * ks][1]);
      a[1] = pack_bf16(s[2 * ks][2], s[2 * ks][3]);
      a[2] = pack_bf16(s[2 * ks + 1][0], s[2 * ks + 1][1]);
      a[3] = pack_bf16(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
      for (int j = 0; j < HD / 8; j += 2) {
        // transposed matrices: (keys ks*16.., dims j*8), (keys ks*16+8.., dims j*8), (keys ks*16.., dims (j+1)*8), (+8, ..)
        uint32_t b[4];
        ldsm_x4_t(b, kv_ptr(vt, ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, j + (lane >> 4)));
        mma16816(o[j], a, b[0], b[1]);
        mma16816(o[j + 1], a, b[2], b[3]);
      }
    }
  }

  __device__ __forceinline__ void reduce_l() {
    l[0] += __shfl_xor_sync(0xffffffffu, l[0], 1);
    l[0] += __shfl_xor_sync(0xffffffffu, l[0], 2);
    l[1] += __shfl_xor_sync(0xffffffffu, l[1], 1);
    l[1] += __shfl_xor_sync(0xffffffffu, l[1], 2);
  }
};

// ------------------------------------------------------------------------------------------ prefill
// grid (q tiles of 64 rows, hq, B); 128 threads; K/V tiles of KT keys double-buffered.
template <int HD, int KT, bool INT8>
__global__ void __launch_bounds__(128) attn_prefill_kernel(const AttnParams p) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);                 // [64][HD]
  bf16* kbuf = qs + 64 * HD;                                    // [2][KT][HD]
  bf16* vbuf = kbuf + 2 * KT * HD;                              // [2][KT][HD]
  float* sc = reinterpret_cast<float*>(vbuf + 2 * KT * HD);     // [2][2][KT] k/v scales (int8)
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.z, h = blockIdx.y;
  const int q0 = p.cu_q[b], q_len = p.cu_q[b + 1] - q0;
  const int r0 = blockIdx.x * 64;
  if (r0 >= q_len) return;
  const int kv_len = p.kv_lens[b];
  const int kvh = min((h + p.q_off) / p.group, p.hkv - 1);
  const int pos_base = kv_len - q_len;
  const int rows = min(64, q_len - r0);
  const int prefix_len = p.prefix_lens ? p.prefix_lens[b] : 0;
  // keys needed by this tile: up to the position of its last row (or the prefix)
  int k_end = min(kv_len, max(pos_base + r0 + rows, prefix_len));
  const int ntiles = (k_end + KT - 1) / KT;
  const int* bt = p.block_table + (size_t)b * p.bt_stride;
  const int tiles_per_block = p.bs / KT;

  load_tile_bf16<HD, 128>(qs, p.q + ((size_t)(q0 + r0) * p.hq + h) * HD, (long long)p.hq * HD, 64, rows, tid);

  auto issue = [&](int ti, int buf) {
    const int blk_i = ti / tiles_per_block, sub = ti % tiles_per_block;
    int blk = bt[blk_i];
    if (blk < 0 || blk >= p.num_blocks) { if (tid == 0 && p.status) atomicCAS(p.status, 0, XFT_ERR_BOUNDS); blk = 0; }
    const size_t row0 = ((size_t)blk * p.hkv + kvh) * p.bs + sub * KT;
    const int valid = min(KT, k_end - ti * KT);
    if (INT8) {
      load_tile_int8<HD, 128>(kbuf + buf * KT * HD, reinterpret_cast<const int8_t*>(p.kc) + row0 * HD, KT, valid, tid);
      load_tile_int8<HD, 128>(vbuf + buf * KT * HD, reinterpret_cast<const int8_t*>(p.vc) + row0 * HD, KT, valid, tid);
      for (int i = tid; i < KT; i += 128) {
        sc[(buf * 2 + 0) * KT + i] = i < valid ? p.ks[row0 + i] : 0.f;
        sc[(buf * 2 + 1) * KT + i] = i < valid ? p.vs[row0 + i] : 0.f;
      }
    } else {
      load_tile_bf16<HD, 128>(kbuf + buf * KT * HD, reinterpret_cast<const bf16*>(p.kc) + row0 * HD, HD, KT, valid, tid);
      load_tile_bf16<HD, 128>(vbuf + buf * KT * HD, reinterpret_cast<const bf16*>(p.vc) + row0 * HD, HD, KT, valid, tid);
    }
  };

  WarpAttn<HD, KT> wa;
  wa.init();
  const int rq0 = r0 + warp * 16 + (lane >> 2), rq1 = rq0 + 8;
  const int qpos0 = rq0 < q_len ? pos_base + rq0 : -1;
  const int qpos1 = rq1 < q_len ? pos_base + rq1 : -1;
  const bool use_alibi = p.slopes != nullptr;
  const float slope = use_alibi ? p.slopes[h] : 0.f;
  const int warp_last_pos = pos_base + min(r0 + warp * 16 + 15, q_len - 1);

  if (ntiles > 0) issue(0, 0);
  cp_async_commit();
  for (int ti = 0; ti < ntiles; ++ti) {
    const int buf = ti & 1;
    if (ti + 1 < ntiles) issue(ti + 1, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    // skip tiles entirely above this warp's causal frontier (still take part in the barriers)
    if (ti * KT <= max(warp_last_pos, prefix_len - 1) && r0 + warp * 16 < q_len)
      wa.step(qs + warp * 16 * HD, kbuf + buf * KT * HD, vbuf + buf * KT * HD, ti * KT, kv_len, qpos0, qpos1, p.scale, slope,
              slope, use_alibi, prefix_len, INT8 ? sc + (buf * 2 + 0) * KT : nullptr, INT8 ? sc + (buf * 2 + 1) * KT : nullptr, lane);
    __syncthreads();
  }
  wa.reduce_l();
  const float i0 = wa.l[0] > 0.f ? 1.f / wa.l[0] : 0.f, i1 = wa.l[1] > 0.f ? 1.f / wa.l[1] : 0.f;
#pragma unroll
  for (int j = 0; j < HD / 8; ++j) {
    const int d = j * 8 + 2 * (lane & 3);
    if (rq0 < q_len)
      *reinterpret_cast<uint32_t*>(p.out + ((size_t)(q0 + rq0) * p.hq + h) * HD + d) = pack_bf16(wa.o[j][0] * i0, wa.o[j][1] * i0);
    if (rq1 < q_len)
      *reinterpret_cast<uint32_t*>(p.out + ((size_t)(q0 + rq1) * p.hq + h) * HD + d) = pack_bf16(wa.o[j][2] * i1, wa.o[j][3] * i1);
  }
}

// Tail of a decode CTA: merge the four consumer warps' (m, l, O) through shared memory `mo` ([4][16][HD+2] floats),
// then either store the result (nsplit == 1) or write this slice's partial and let the slice that arrives last
// merge all slices of the (sequence, kv head) — no second kernel, no spinning.  Every thread of the CTA calls it.
template <int HD, class WA>
__device__ __forceinline__ void decode_finish(const AttnParams& p, WA& wa, float* mo, bool consumer, int warp, int lane,
                                              int tid, int nthreads, int nq, int h_lo, int b, int tok, int split) {
  constexpr int RS = HD + 2;
  const int r0 = lane >> 2, r1 = r0 + 8;
  if (consumer) {
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) {
      const int d = j * 8 + 2 * (lane & 3);
      mo[(warp * 16 + r0) * RS + d] = wa.o[j][0];
      mo[(warp * 16 + r0) * RS + d + 1] = wa.o[j][1];
      mo[(warp * 16 + r1) * RS + d] = wa.o[j][2];
      mo[(warp * 16 + r1) * RS + d + 1] = wa.o[j][3];
    }
    if ((lane & 3) == 0) {
      mo[(warp * 16 + r0) * RS + HD] = wa.m[0];
      mo[(warp * 16 + r0) * RS + HD + 1] = wa.l[0];
      mo[(warp * 16 + r1) * RS + HD] = wa.m[1];
      mo[(warp * 16 + r1) * RS + HD + 1] = wa.l[1];
    }
  }
  __syncthreads();
  for (int i = tid; i < nq * HD; i += nthreads) {
    const int r = i / HD, d = i % HD;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, mo[(w * 16 + r) * RS + HD]);
    float acc = 0.f, ll = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = mo[(w * 16 + r) * RS + HD];
      const float c = (mw == -INFINITY) ? 0.f : __expf(mw - mm);
      acc += c * mo[(w * 16 + r) * RS + d];
      ll += c * mo[(w * 16 + r) * RS + HD + 1];
    }
    const int h = h_lo + r;
    if (p.nsplit == 1) {
      p.out[((size_t)tok * p.hq + h) * HD + d] = __float2bfloat16(ll > 0.f ? acc / ll : 0.f);
    } else {
      const size_t pi = ((size_t)b * p.hq + h) * p.nsplit + split;
      p.part_o[pi * HD + d] = acc;
      if (d == 0) { p.part_ml[pi * 2] = mm; p.part_ml[pi * 2 + 1] = ll; }
    }
  }
  if (p.nsplit > 1) {
    __shared__ int s_last;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      int* c = p.split_counters + (size_t)b * gridDim.y + blockIdx.y;
      const int old = atomicAdd(c, 1);
      s_last = (old == p.nsplit - 1);
      if (s_last) *c = 0;
    }
    __syncthreads();
    if (s_last) {
      __threadfence();
      for (int i = tid; i < nq * HD; i += nthreads) {
        const int r = i / HD, d = i % HD;
        const int h = h_lo + r;
        const size_t base = ((size_t)b * p.hq + h) * p.nsplit;
        float mm = -INFINITY;
        for (int s = 0; s < p.nsplit; ++s) mm = fmaxf(mm, __ldcg(p.part_ml + (base + s) * 2));
        float acc = 0.f, ll = 0.f;
        for (int s = 0; s < p.nsplit; ++s) {
          const float ms = __ldcg(p.part_ml + (base + s) * 2);
          const float c = (ms == -INFINITY) ? 0.f : __expf(ms - mm);
          acc += c * __ldcg(p.part_o + (base + s) * HD + d);
          ll += c * __ldcg(p.part_ml + (base + s) * 2 + 1);
        }
        p.out[((size_t)tok * p.hq + h) * HD + d] = __float2bfloat16(ll > 0.f ? acc / ll : 0.f);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------ decode
// grid (B, hkv * qchunks, nsplit); 128 threads; each warp walks its own tiles with private buffers.
// Requires q_len == 1 for every sequence.
template <int HD, int KT, bool INT8>
__global__ void __launch_bounds__(128) attn_decode_kernel(const AttnParams p) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);                 // [16][HD]
  bf16* kv = qs + 16 * HD;                                      // per warp: K [KT][HD], V [KT][HD]
  float* scb = reinterpret_cast<float*>(kv + 4 * 2 * KT * HD);  // per warp [2][KT]
  grid_dep_launch();
  grid_dep_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.x;
  const int qchunks = (p.group + 15) / 16;
  const int kvh = blockIdx.y / qchunks, qc = blockIdx.y % qchunks;
  const int split = blockIdx.z;
  const int kv_len = p.kv_lens[b];
  const int tok = p.cu_q[b];
  // local q heads served by this kv head: i with (i + q_off) / group == kvh
  const int h_lo = max(0, kvh * p.group - p.q_off) + qc * 16;
  const int h_hi = min(min(p.hq, (kvh + 1) * p.group - p.q_off), h_lo + 16);
  const int nq = h_hi - h_lo;
  if (nq <= 0) return;
  const int ntiles = (kv_len + KT - 1) / KT;
  const int per = (ntiles + p.nsplit - 1) / p.nsplit;
  const int t_begin = split * per, t_end = min(ntiles, t_begin + per);
  const int* bt = p.block_table + (size_t)b * p.bt_stride;
  const int tiles_per_block = p.bs / KT;

  // Q rows = heads h_lo..h_hi-1 of the single query token (contiguous in memory)
  load_tile_bf16<HD, 128>(qs, p.q + ((size_t)tok * p.hq + h_lo) * HD, HD, 16, nq, tid);
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();

  bf16* kt = kv + warp * 2 * KT * HD;
  bf16* vt = kt + KT * HD;
  float* ksc = scb + warp * 2 * KT;
  float* vsc = ksc + KT;

  auto issue_k = [&](int ti) {
    if (ti < t_end) {
      int blk = bt[ti / tiles_per_block];
      if (blk < 0 || blk >= p.num_blocks) { if (lane == 0 && p.status) atomicCAS(p.status, 0, XFT_ERR_BOUNDS); blk = 0; }
      const size_t row0 = ((size_t)blk * p.hkv + kvh) * p.bs + (ti % tiles_per_block) * KT;
      const int valid = min(KT, kv_len - ti * KT);
      if (INT8) {
        load_tile_int8<HD, 32>(kt, reinterpret_cast<const int8_t*>(p.kc) + row0 * HD, KT, valid, lane);
        for (int i = lane; i < KT; i += 32) ksc[i] = i < valid ? p.ks[row0 + i] : 0.f;
      } else {
        load_tile_bf16<HD, 32>(kt, reinterpret_cast<const bf16*>(p.kc) + row0 * HD, HD, KT, valid, lane);
      }
    }
    cp_async_commit();
  };
  auto issue_v = [&](int ti) {
    if (ti < t_end) {
      int blk = bt[ti / tiles_per_block];
      if (blk < 0 || blk >= p.num_blocks) blk = 0;
      const size_t row0 = ((size_t)blk * p.hkv + kvh) * p.bs + (ti % tiles_per_block) * KT;
      const int valid = min(KT, kv_len - ti * KT);
      if (INT8) {
        load_tile_int8<HD, 32>(vt, reinterpret_cast<const int8_t*>(p.vc) + row0 * HD, KT, valid, lane);
        for (int i = lane; i < KT; i += 32) vsc[i] = i < valid ? p.vs[row0 + i] : 0.f;
      } else {
        load_tile_bf16<HD, 32>(vt, reinterpret_cast<const bf16*>(p.vc) + row0 * HD, HD, KT, valid, lane);
      }
    }
    cp_async_commit();
  };

  // Each warp runs its tiles as one "row block" of 16 rows where row r = head h_lo + r; all rows share
  // the query position kv_len-1.  S and P V are computed for all 16 rows (unused rows are zero queries).
  WarpAttn<HD, KT> wa;
  wa.init();
  const int r0 = lane >> 2, r1 = r0 + 8;
  const int qpos = kv_len - 1;
  const int qpos0 = r0 < nq ? qpos : -1, qpos1 = r1 < nq ? qpos : -1;
  const bool use_alibi = p.slopes != nullptr;
  // ALiBi slope differs per row (= per head): fold it by processing the bias with per-row slopes
  const float slope0 = (use_alibi && r0 < nq) ? p.slopes[h_lo + r0] : 0.f;
  const float slope1 = (use_alibi && r1 < nq) ? p.slopes[h_lo + r1] : 0.f;

  // Per warp: the V tile streams in while S is computed, the next K tile while P V is computed.
  int ti = t_begin + warp;
  issue_k(ti);
  issue_v(ti);
  for (; ti < t_end; ti += 4) {
    float s[KT / 8][4];
    cp_async_wait<1>();          // K(ti) landed (V(ti) may still be in flight)
    __syncwarp();
    wa.scores(s, qs, kt, ti * KT, kv_len, qpos0, qpos1, p.scale, slope0, slope1, use_alibi, 0, INT8 ? ksc : nullptr,
              INT8 ? vsc : nullptr, lane);
    __syncwarp();
    issue_k(ti + 4);             // K buffer is free again
    cp_async_wait<1>();          // V(ti) landed
    __syncwarp();
    wa.pv(s, vt, lane);
    __syncwarp();
    issue_v(ti + 4);
  }
  cp_async_wait<0>();
  wa.reduce_l();
  __syncthreads();
  decode_finish<HD>(p, wa, reinterpret_cast<float*>(kv), true, warp, lane, tid, 128, nq, h_lo, b, tok, split);
}

// ------------------------------------------------------------------------------------------ decode, TMA ring
// bf16 caches.  grid (B, hkv * qchunks, nsplit); 160 threads: one lane of warp 4 feeds a CTA-wide ring of 64-key
// K/V tiles with TMA (a tile is one box per 64-column half of 64 cache rows, hardware-swizzled, so no thread
// computes a load address); warps 0-3 each take 16 keys of every tile, so all four wait on the same barrier in the
// same order (a waiter is never more than one phase away from its barrier) and release the stage with one arrival
// each.  About 96 KB of tiles are in flight per CTA and two CTAs share an SM, which covers the HBM latency without
// any warp waiting on its own request.
// Rows of a block past kv_len hold finite stale data (the pool starts zeroed), so P = 0 masks them exactly.
constexpr int kDecTile = 64;            // keys per ring stage (= the cache block size granule)
constexpr int kDecMaxBlocks = 512;      // block ids of this CTA's slice cached in shared memory
template <int HD>
struct DecCfg {
  static constexpr int STAGE_BYTES = 2 * kDecTile * HD * 2;
  static constexpr int STAGES = (96 * 1024) / STAGE_BYTES >= 3 ? (96 * 1024) / STAGE_BYTES : 3;
};

template <int HD>
__global__ void __launch_bounds__(160, (HD <= 128 ? 2 : 1)) attn_decode_tma_kernel(const __grid_constant__ CUtensorMap tmK,
                                                                                  const __grid_constant__ CUtensorMap tmV,
                                                                                  const AttnParams p) {
  constexpr int KT = kDecTile, KW = KT / 4;             // keys per tile, keys per warp and tile
  constexpr int TILE = KT * HD;                         // elements of one K (or V) tile
  constexpr int STAGES = DecCfg<HD>::STAGES;
  constexpr uint32_t STAGE_BYTES = DecCfg<HD>::STAGE_BYTES;
  extern __shared__ __align__(1024) uint8_t smem_dyn[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  bf16* ring = reinterpret_cast<bf16*>(base);                               // [STAGES][K tile | V tile]
  bf16* qs = reinterpret_cast<bf16*>(base + (size_t)STAGES * STAGE_BYTES);  // [16][HD]
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES];
  __shared__ int s_blk[kDecMaxBlocks];
  __shared__ int s_abort;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 4); }
    s_abort = 0;
    fence_barrier_init();
  }
  if (warp == 4 && lane == 0) { tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); }
  grid_dep_launch();
  // Until grid_dep_wait() below only step inputs are read (lengths, block table: written before the first kernel of
  // the step) and cache rows of EARLIER tokens; the query and the newest token's K / V row come from the kernel in
  // front of this one and are touched after the wait.
  const int b = blockIdx.x;
  const int qchunks = (p.group + 15) / 16;
  const int kvh = blockIdx.y / qchunks, qc = blockIdx.y % qchunks;
  const int split = blockIdx.z;
  const int kv_len = p.kv_lens[b];
  const int tok = p.cu_q[b];
  const int h_lo = max(0, kvh * p.group - p.q_off) + qc * 16;
  const int h_hi = min(min(p.hq, (kvh + 1) * p.group - p.q_off), h_lo + 16);
  const int nq = h_hi - h_lo;
  if (nq <= 0) return;
  const int ntiles = (kv_len + KT - 1) / KT;
  const int per = (ntiles + p.nsplit - 1) / p.nsplit;
  const int t_begin = split * per, t_end = min(ntiles, t_begin + per);
  const int nloc = max(t_end - t_begin, 0);
  const int* bt = p.block_table + (size_t)b * p.bt_stride;
  const int tiles_per_block = p.bs / KT;

  const int blk_first = t_begin / tiles_per_block;
  const int nblk = nloc > 0 ? (t_end - 1) / tiles_per_block - blk_first + 1 : 0;
  for (int i = tid; i < min(nblk, kDecMaxBlocks); i += 160) {
    int blk = bt[blk_first + i];
    if (blk < 0 || blk >= p.num_blocks) { if (p.status) atomicCAS(p.status, 0, XFT_ERR_BOUNDS); blk = 0; }
    s_blk[i] = blk;
  }
  __syncthreads();
  // tiles of this slice that cannot hold the token appended in this step: their loads start before the kernel in
  // front has finished (the first STAGES tiles find their stage free without a wait)
  const int newest_tile = (kv_len - 1) / KT;
  const int npre = max(0, min(min(STAGES, nloc), newest_tile - t_begin));
  auto issue_tile = [&](int n) {
    const int st = n % STAGES;
    const int ti = t_begin + n;
    const int bi = ti / tiles_per_block - blk_first;
    int blk;
    if (bi < kDecMaxBlocks) {
      blk = s_blk[bi];
    } else {
      blk = bt[blk_first + bi];
      if (blk < 0 || blk >= p.num_blocks) { if (p.status) atomicCAS(p.status, 0, XFT_ERR_BOUNDS); blk = 0; }
    }
    const int row = (blk * p.hkv + kvh) * p.bs + (ti % tiles_per_block) * KT;
    bf16* kt = ring + (size_t)st * 2 * TILE;
    mbar_expect_tx(&full_bar[st], STAGE_BYTES);
#pragma unroll
    for (int h = 0; h < HD / 64; ++h) {
      tma_load_2d(kt + h * KT * 64, &tmK, &full_bar[st], h * 64, row, kEvictFirst);
      tma_load_2d(kt + TILE + h * KT * 64, &tmV, &full_bar[st], h * 64, row, kEvictFirst);
    }
  };
  if (warp == 4 && lane == 0)
    for (int n = 0; n < npre; ++n) issue_tile(n);
  grid_dep_wait();
  if (tid < 128) load_tile_bf16<HD, 128>(qs, p.q + ((size_t)tok * p.hq + h_lo) * HD, HD, 16, nq, tid);
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();

  WarpAttn<HD, KW, true, KT> wa;
  wa.init();
  if (warp == 4) {
    if (lane == 0) {
      for (int n = npre; n < nloc; ++n) {
        const int st = n % STAGES;
        if (!mbar_wait(&empty_bar[st], ((n / STAGES) & 1) ^ 1, p.status, XFT_ERR_WAIT_EMPTY)) { s_abort = 1; break; }
        issue_tile(n);
      }
    }
  } else {
    const int r0 = lane >> 2, r1 = r0 + 8;
    const int qpos = kv_len - 1;
    const int qpos0 = r0 < nq ? qpos : -1, qpos1 = r1 < nq ? qpos : -1;
    const bool use_alibi = p.slopes != nullptr;
    const float slope0 = (use_alibi && r0 < nq) ? p.slopes[h_lo + r0] : 0.f;
    const float slope1 = (use_alibi && r1 < nq) ? p.slopes[h_lo + r1] : 0.f;
    constexpr bool QREG = HD <= 128;            // Q fragments live in registers when they fit
    uint32_t qa[QREG ? HD / 16 : 1][4];
    if (QREG) {
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks)
        ldsm_x4(qa[QREG ? ks : 0], tile_ptr<HD>(qs, (lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)));
    }
    for (int n = 0; n < nloc; ++n) {
      const int st = n % STAGES;
      if (!mbar_wait(&full_bar[st], (n / STAGES) & 1, p.status, XFT_ERR_WAIT_FULL)) { s_abort = 1; break; }
      // this warp's 16 keys of the tile: rows warp*16 .. +15 of both halves (the row offset keeps row & 7)
      const bf16* kt = ring + (size_t)st * 2 * TILE + warp * KW * 64;
      const int key0 = (t_begin + n) * KT + warp * KW;
      if (key0 < kv_len) {
        float s[KW / 8][4];
        if constexpr (QREG) wa.qk_frag(s, reinterpret_cast<const uint32_t (&)[HD / 16][4]>(qa), kt, lane);
        else wa.qk(s, qs, kt, lane);
        if (use_alibi || key0 + KW > kv_len) {
          wa.mask(s, key0, kv_len, qpos0, qpos1, p.scale, slope0, slope1, use_alibi, 0, nullptr, lane);
        } else {
          // every key is visible; rows past nq carry a zero query and are never stored
#pragma unroll
          for (int j = 0; j < KW / 8; ++j) { s[j][0] *= p.scale; s[j][1] *= p.scale; s[j][2] *= p.scale; s[j][3] *= p.scale; }
        }
        wa.softmax_update(s, nullptr, lane);
        wa.pv(s, kt + TILE, lane);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[st]);
    }
    wa.reduce_l();
  }
  __syncthreads();
  if (s_abort) {
    // a wait ran out (status holds the reason): let copies already issued land before the CTA's memory is released
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) {}
    return;
  }
  // every issued tile was consumed, so the ring is idle and can carry the merge
  decode_finish<HD>(p, wa, reinterpret_cast<float*>(ring), warp < 4, warp, lane, tid, 160, nq, h_lo, b, tok, split);
}

// merge split partials: grid (B, hq), HD threads
__global__ void attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, bf16* __restrict__ out,
                                  const int* __restrict__ cu_q, int hq, int HD, int nsplit) {
  const int b = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
  const size_t base = ((size_t)b * hq + h) * nsplit;
  float mm = -INFINITY;
  for (int s = 0; s < nsplit; ++s) mm = fmaxf(mm, part_ml[(base + s) * 2]);
  float acc = 0.f, ll = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float ms = part_ml[(base + s) * 2];
    const float c = (ms == -INFINITY) ? 0.f : __expf(ms - mm);
    acc += c * part_o[(base + s) * HD + d];
    ll += c * part_ml[(base + s) * 2 + 1];
  }
  out[((size_t)cu_q[b] * hq + h) * HD + d] = __float2bfloat16(ll > 0.f ? acc / ll : 0.f);
}

}  // namespace xft

using namespace xft;

template <int HD, int KT>
static int launch_prefill(const AttnParams& p, int B, int max_q, bool int8, cudaStream_t st) {
  size_t smem = (size_t)(64 * HD + 4 * KT * HD) * 2 + 4 * KT * sizeof(float);
  dim3 grid((max_q + 63) / 64, p.hq, B);
  if (int8) {
    cudaFuncSetAttribute(attn_prefill_kernel<HD, KT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    attn_prefill_kernel<HD, KT, true><<<grid, 128, smem, st>>>(p);
  } else {
    cudaFuncSetAttribute(attn_prefill_kernel<HD, KT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    attn_prefill_kernel<HD, KT, false><<<grid, 128, smem, st>>>(p);
  }
  return (int)cudaGetLastError();
}

template <int HD, int KT>
static int launch_decode(const AttnParams& p, int B, bool int8, cudaStream_t st) {
  size_t kvbytes = (size_t)4 * 2 * KT * HD * 2;
  size_t merge = (size_t)4 * 16 * (HD + 2) * sizeof(float);
  size_t smem = (size_t)16 * HD * 2 + (kvbytes > merge ? kvbytes : merge) + 4 * 2 * KT * sizeof(float);
  const int qchunks = (p.group + 15) / 16;
  dim3 grid(B, p.hkv * qchunks, p.nsplit);
  if (int8) {
    cudaFuncSetAttribute(attn_decode_kernel<HD, KT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaError_t e = launch_pdl(attn_decode_kernel<HD, KT, true>, grid, dim3(128), smem, st, p);
    if (e != cudaSuccess) return (int)e;
  } else {
    cudaFuncSetAttribute(attn_decode_kernel<HD, KT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaError_t e = launch_pdl(attn_decode_kernel<HD, KT, false>, grid, dim3(128), smem, st, p);
    if (e != cudaSuccess) return (int)e;
  }
  return (int)cudaGetLastError();
}

template <int HD>
static int launch_decode_tma(const AttnParams& p, int B, cudaStream_t st) {
  CUtensorMap tmK, tmV;
  const uint64_t rows = (uint64_t)p.num_blocks * p.hkv * p.bs;
  if (make_tensor_map(&tmK, p.kc, rows, HD, HD, kDecTile, 2) || make_tensor_map(&tmV, p.vc, rows, HD, HD, kDecTile, 2)) return -4;
  const size_t smem = (size_t)DecCfg<HD>::STAGES * DecCfg<HD>::STAGE_BYTES + 16 * HD * 2 + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(attn_decode_tma_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return -5;
    attr_set = true;
  }
  const int qchunks = (p.group + 15) / 16;
  dim3 grid(B, p.hkv * qchunks, p.nsplit);
  cudaError_t e = launch_pdl(attn_decode_tma_kernel<HD>, grid, dim3(160), smem, st, tmK, tmV, p);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaGetLastError();
}

// decode != 0: every sequence has exactly one query row (2 forces the cp.async kernel for bf16 caches too).  nsplit/part_*: split-KV scratch (decode only).
extern "C" int xft_paged_attention(const void* q, void* out, const void* kc, const void* vc, const float* ks, const float* vs,
                                   const int* block_table, int bt_stride, const int* cu_q, const int* kv_lens, int B,
                                   int max_q, int hq, int hkv, int group, int q_off, int HD, int bs, int num_blocks,
                                   float scale, const float* slopes, const int* prefix_lens, int decode, int nsplit,
                                   float* part_o, float* part_ml, int* split_counters, int* status, cudaStream_t st) {
  if (B <= 0) return 0;
  AttnParams p{};
  p.q = (const bf16*)q; p.out = (bf16*)out; p.kc = kc; p.vc = vc; p.ks = ks; p.vs = vs;
  p.block_table = block_table; p.bt_stride = bt_stride; p.cu_q = cu_q; p.kv_lens = kv_lens; p.slopes = slopes;
  p.prefix_lens = prefix_lens; p.hq = hq; p.hkv = hkv; p.group = group; p.q_off = q_off; p.bs = bs; p.scale = scale;
  p.num_blocks = num_blocks; p.nsplit = nsplit < 1 ? 1 : nsplit; p.part_o = part_o; p.part_ml = part_ml; p.split_counters = split_counters; p.status = status;
  const bool int8 = ks != nullptr;
  if (bs % 64) return -2;
  if (decode) {
    if (p.nsplit > 1 && (!part_o || !part_ml || !split_counters)) return -3;
    if (!int8 && decode != 2) {
      if (HD == 64) return launch_decode_tma<64>(p, B, st);
      if (HD == 128) return launch_decode_tma<128>(p, B, st);
      if (HD == 256) return launch_decode_tma<256>(p, B, st);
      return -1;
    }
    // per-warp K+V tiles of 16 KB: a CTA stays at ~64 KB so three CTAs (12 warps) overlap loads and math per SM
    if (HD == 64) return launch_decode<64, 64>(p, B, int8, st);
    if (HD == 128) return launch_decode<128, 32>(p, B, int8, st);
    if (HD == 256) return launch_decode<256, 16>(p, B, int8, st);
    return -1;
  }
  if (HD == 64) return launch_prefill<64, 64>(p, B, max_q, int8, st);
  if (HD == 128) return launch_prefill<128, 64>(p, B, max_q, int8, st);
  if (HD == 256) return launch_prefill<256, 32>(p, B, max_q, int8, st);
  return -1;
}
