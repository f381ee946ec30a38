// Prefill attention for sm_100a on the 5th-generation tensor cores: causal flash attention over the paged KV cache,
// head_dim 128, bf16 cache, GQA.
//
// Replaces the reference's prompt-phase attention (src/kernels/attention_kernels.h:142-552 crossAttnByHead /
// selfAttention with its small-GEMM softmax loop, and the flash variant at :1285-1408) with one kernel per
// (128 query rows, head, sequence):
//
//   S = Q K^T   tcgen05.mma, A = the query tile [128 rows x 128] (K-major, shared memory, loaded once by TMA),
//               B = 128 keys of the cache (two 64-token blocks of the block table, K-major), D = S in TMEM (fp32,
//               128 columns, double buffered so the next tile's S is computed while this one's softmax runs)
//   P = softmax row by row: four warps, one query row (= one TMEM lane) per thread, read S with tcgen05.ld, keep the
//               running maximum and sum in registers, write P as bf16 into shared memory in the K-major 128-byte
//               swizzled layout the next product expects
//   O += P V    tcgen05.mma, A = P (shared memory), B = the same 128 cache rows of V used as an MN-major operand
//               (rows = keys = the contraction dimension, the 128 head features contiguous: no transpose is needed),
//               D = the tile's contribution in TMEM; the four warps add it to their fp32 accumulator rows in registers
//               with the usual exp(m_old - m_new) correction
//
// K and V tiles arrive through a two-stage TMA ring (one box per 64-token cache block and 64-feature half), the
// softmax of tile j overlaps the QK^T of tile j + 1, and CTAs with the most keys to visit (the last query rows of a
// causal prompt) are scheduled first.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer, warps 2-5 = softmax / output.
// Every wait is bounded and reports through the status word.
#include "ptx.cuh"

namespace xft {

int make_tensor_map(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                    uint32_t esize);

struct PrefillAttnParams {
  __nv_bfloat16* out;        // [T, hq, 128]
  const int* block_table; int bt_stride;
  const int* cu_q; const int* kv_lens;
  int hq, hkv, group, q_off;  // kv head of query head h = (h + q_off) / group
  int bs;                     // tokens per cache block (64)
  float scale_log2;           // softmax scale * log2(e)
  int num_blocks;
  int* status;
};

// Shared-memory matrix descriptor of an MN-major operand with the 128-byte swizzle: rows of 128 bytes hold 64
// consecutive M/N elements of one K index, 8 such rows (K indices) form a 1024-byte group (stride byte offset), the next
// 64 M/N elements start `lbo_bytes` further (leading byte offset).
__device__ __forceinline__ uint64_t umma_desc_mn128(uint32_t smem_addr, uint32_t lbo_bytes) {
  uint64_t d = (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)(lbo_bytes >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,"
      "%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr));
}

constexpr int kPfTile = 128;                 // keys per tile = two cache blocks
constexpr int kPfQ = 128;                    // query rows per CTA
constexpr int kPfHalf = kPfTile * 128;       // bytes of one 64-feature half of a 128-row tile (128 rows x 128 B)
constexpr int kPfTileBytes = 2 * kPfHalf;    // 32 KB: Q, P, and each K / V stage
constexpr int kPfSmem = kPfTileBytes * 6 + 1024;   // Q, P, K x 2, V x 2

__global__ void __launch_bounds__(192, 1) attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmQ,
                                                                 const __grid_constant__ CUtensorMap tmK,
                                                                 const __grid_constant__ CUtensorMap tmV,
                                                                 const PrefillAttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sP = smem + kPfTileBytes;
  uint8_t* sK = smem + 2 * kPfTileBytes;      // two stages
  uint8_t* sV = smem + 4 * kPfTileBytes;      // two stages
  __shared__ uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_full, o_full;
  __shared__ uint32_t tmem_base_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z, h = blockIdx.y;
  const int q0 = p.cu_q[b], q_len = p.cu_q[b + 1] - q0, kv_len = p.kv_lens[b];
  // heavy tiles first: the last query rows of a causal prompt visit the most keys
  const int n_qt = (q_len + kPfQ - 1) / kPfQ;
  if ((int)blockIdx.x >= n_qt) return;
  const int row0 = (n_qt - 1 - (int)blockIdx.x) * kPfQ;
  const int past = kv_len - q_len;            // keys before this call's first query
  const int last_row = min(row0 + kPfQ, q_len) - 1;
  const int n_tiles = (min(kv_len, past + last_row + 1) + kPfTile - 1) / kPfTile;
  const int kvh = (h + p.q_off) / p.group;

  if (threadIdx.x == 0) {
    mbar_init(&q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1);
    }
    mbar_init(&p_full, 4);                     // one arrival per softmax warp
    mbar_init(&o_full, 1);
    fence_barrier_init();
    fence_proxy_async();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_s, 512);             // S x 2 (256 columns) + O tile (128), rounded up to a power of two
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  grid_dep_launch();
  grid_dep_wait();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(&q_full, kPfTileBytes);
      // q is [T, hq * 128]: rows past the end of the tensor read as zero, rows of the next sequence are never stored
      tma_load_2d(sQ, &tmQ, &q_full, h * 128, q0 + row0, kEvictFirst);
      tma_load_2d(sQ + kPfHalf, &tmQ, &q_full, h * 128 + 64, q0 + row0, kEvictFirst);
      const int* bt = p.block_table + (size_t)b * p.bt_stride;
      const int n_blocks = (kv_len + p.bs - 1) / p.bs;
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        // cache rows of the two blocks of this tile; past the sequence's last block the last one is read again
        // (finite values; those keys are masked)
        int rowk[2];
        bool bad = false;
        for (int i = 0; i < 2; ++i) {
          int blk = bt[min(2 * j + i, n_blocks - 1)];
          if (blk < 0 || blk >= p.num_blocks) { bad = true; blk = 0; }
          rowk[i] = (blk * p.hkv + kvh) * p.bs;
        }
        if (bad && p.status) atomicCAS(p.status, 0, XFT_ERR_BOUNDS);
        if (!mbar_wait(&k_empty[s], ph ^ 1, p.status, XFT_ERR_WAIT_EMPTY)) break;
        mbar_expect_tx(&k_full[s], kPfTileBytes);
        uint8_t* k = sK + s * kPfTileBytes;
        for (int i = 0; i < 2; ++i) {
          tma_load_2d(k + i * 8192, &tmK, &k_full[s], 0, rowk[i], kEvictNormal);
          tma_load_2d(k + kPfHalf + i * 8192, &tmK, &k_full[s], 64, rowk[i], kEvictNormal);
        }
        if (!mbar_wait(&v_empty[s], ph ^ 1, p.status, XFT_ERR_WAIT_EMPTY)) break;
        mbar_expect_tx(&v_full[s], kPfTileBytes);
        uint8_t* v = sV + s * kPfTileBytes;
        for (int i = 0; i < 2; ++i) {
          tma_load_2d(v + i * 8192, &tmV, &v_full[s], 0, rowk[i], kEvictNormal);
          tma_load_2d(v + kPfHalf + i * 8192, &tmV, &v_full[s], 64, rowk[i], kEvictNormal);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // S = Q K^T: both operands K-major, M = 128 query rows, N = 128 keys, K = 128 features in 8 steps of 16
      constexpr uint32_t IDESC_S = umma_idesc(128, 128, 1, 1, 1);
      // O = P V: A = P K-major (keys contiguous), B = V MN-major (bit 16), N = 128 features, K = 128 keys
      constexpr uint32_t IDESC_O = umma_idesc(128, 128, 1, 1, 1) | (1u << 16);
      auto issue_s = [&](int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait(&k_full[s], (j >> 1) & 1, p.status, XFT_ERR_WAIT_FULL)) return false;
        tcgen05_fence_after();
        const uint32_t qa = smem_u32(sQ), ka = smem_u32(sK + s * kPfTileBytes);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (kk >> 2) * kPfHalf + (kk & 3) * 32;       // feature half, then 16 features = 32 bytes
          umma_bf16(tmem_base + (uint32_t)(s * 128), umma_desc_k128(qa + off), umma_desc_k128(ka + off), IDESC_S, kk > 0);
        }
        tcgen05_commit(&k_empty[s]);
        tcgen05_commit(&s_full[s]);
        return true;
      };
      bool ok = mbar_wait(&q_full, 0, p.status, XFT_ERR_WAIT_FULL) && issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) ok = issue_s(j + 1);          // runs while the softmax warps work on tile j
        if (!ok) break;
        const int s = j & 1;
        if (!mbar_wait(&p_full, j & 1, p.status, XFT_ERR_WAIT_TMEM)) break;
        if (!mbar_wait(&v_full[s], (j >> 1) & 1, p.status, XFT_ERR_WAIT_FULL)) break;
        tcgen05_fence_after();
        const uint32_t pa = smem_u32(sP), va = smem_u32(sV + s * kPfTileBytes);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          // A: 16 keys = 32 bytes inside the 64-key half; B: 16 keys = 16 rows of 128 bytes
          const uint32_t aoff = (kk >> 2) * kPfHalf + (kk & 3) * 32;
          umma_bf16(tmem_base + 256, umma_desc_k128(pa + aoff), umma_desc_mn128(va + kk * 2048, kPfHalf), IDESC_O, kk > 0);
        }
        tcgen05_commit(&v_empty[s]);
        tcgen05_commit(&o_full);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + output: one query row per thread
    const int qd = warp & 3;
    const int r = qd * 32 + lane;                          // row of the tile = TMEM lane
    const int qrow = row0 + r;
    // rows past the sequence's end attend like its last row (finite numbers, never stored)
    const int qpos = past + min(qrow, q_len - 1);
    const uint32_t lane_addr = tmem_base + (uint32_t(qd * 32) << 16);
    float o[128];
#pragma unroll
    for (int i = 0; i < 128; ++i) o[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int s = j & 1;
      if (!mbar_wait(&s_full[s], (j >> 1) & 1, p.status, XFT_ERR_WAIT_TMEM)) { ok = false; break; }
      tcgen05_fence_after();
      const uint32_t sa = lane_addr + (uint32_t)(s * 128);
      const int k0 = j * kPfTile;
      const int nvalid = min(qpos, kv_len - 1) - k0 + 1;    // keys [k0, k0 + nvalid) are visible to this row
      // pass 1: row maximum of the visible scores
      float mx = m;
#pragma unroll 1
      for (int c = 0; c < 128; c += 32) {
        uint32_t v[32];
        tmem_ld32(sa + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (c + i < nvalid) mx = fmaxf(mx, __uint_as_float(v[i]) * p.scale_log2);
      }
      const float alpha = exp2f(m - mx);                    // m = -inf on the first tile: alpha = 0, o and l are 0
      m = mx;
      // pass 2: P = exp2(s - m) as bf16 into the swizzled K-major tile, row sum
      float sum = 0.f;
#pragma unroll 1
      for (int c = 0; c < 128; c += 32) {
        uint32_t v[32];
        tmem_ld32(sa + c, v);
        tmem_ld_wait();
        uint8_t* prow = sP + (c >> 6) * kPfHalf + r * 128;
#pragma unroll
        for (int g8 = 0; g8 < 4; ++g8) {
          uint32_t w[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int e = g8 * 8 + 2 * i;
            const float p0 = (c + e < nvalid) ? exp2f(__uint_as_float(v[e]) * p.scale_log2 - m) : 0.f;
            const float p1 = (c + e + 1 < nvalid) ? exp2f(__uint_as_float(v[e + 1]) * p.scale_log2 - m) : 0.f;
            const __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
            // the sum uses the rounded values, as the product does
            sum += __low2float(pb) + __high2float(pb);
            w[i] = *reinterpret_cast<const uint32_t*>(&pb);
          }
          const int chunk = ((c & 63) >> 3) + g8;            // 16-byte chunk of the 128-byte row
          *reinterpret_cast<uint4*>(prow + ((chunk ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
      l = l * alpha + sum;
      // P is complete: make the generic-proxy stores visible to the tensor core, then tell the MMA warp
      fence_proxy_async();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full);
      // this tile's P V, added to the row's accumulator with the correction for the new maximum
      if (!mbar_wait(&o_full, j & 1, p.status, XFT_ERR_WAIT_TMEM)) { ok = false; break; }
      tcgen05_fence_after();
#pragma unroll
      for (int c = 0; c < 128; c += 32) {
        uint32_t v[32];
        tmem_ld32(lane_addr + 256 + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c + i] = o[c + i] * alpha + __uint_as_float(v[i]);
      }
      tcgen05_fence_before();
    }
    if (ok && qrow < q_len) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = p.out + ((size_t)(q0 + qrow) * p.hq + h) * 128;
#pragma unroll
      for (int c = 0; c < 128; c += 8) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const __nv_bfloat162 ob = __floats2bfloat162_rn(o[c + 2 * i] * inv, o[c + 2 * i + 1] * inv);
          w[i] = *reinterpret_cast<const uint32_t*>(&ob);
        }
        *reinterpret_cast<uint4*>(dst + c) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace xft

using namespace xft;

// Causal prefill attention over the paged bf16 cache, head_dim 128 (see the file comment).  q, out: [T, hq, 128];
// caches [num_blocks, hkv, bs, 128] with bs = 64; cu_q [B + 1], kv_lens [B] (keys visible after this call's append).
// Returns 0, -1 for an unsupported shape, or a CUDA / tensor-map error.
extern "C" int xft_attn_prefill_tc(const void* q, void* out, const void* kc, const void* vc, const int* block_table,
                                   int bt_stride, const int* cu_q, const int* kv_lens, int B, int T, int max_q, int hq,
                                   int hkv, int group, int q_off, int bs, int num_blocks, float scale, int* status,
                                   cudaStream_t st) {
  if (B <= 0 || T <= 0 || max_q <= 0) return 0;
  if (bs != 64 || hq <= 0 || hkv <= 0) return -1;
  PrefillAttnParams p{};
  p.out = (__nv_bfloat16*)out; p.block_table = block_table; p.bt_stride = bt_stride; p.cu_q = cu_q; p.kv_lens = kv_lens;
  p.hq = hq; p.hkv = hkv; p.group = group; p.q_off = q_off; p.bs = bs; p.scale_log2 = scale * 1.4426950408889634f;
  p.num_blocks = num_blocks; p.status = status;
  CUtensorMap tmQ, tmK, tmV;
  const uint64_t rows = (uint64_t)num_blocks * hkv * bs;
  int r = make_tensor_map(&tmQ, q, (uint64_t)T, (uint64_t)hq * 128, (uint64_t)hq * 128, 128, 2);
  if (r) return 1000 - r;
  if (make_tensor_map(&tmK, kc, rows, 128, 128, 64, 2) || make_tensor_map(&tmV, vc, rows, 128, 128, 64, 2)) return -4;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPfSmem) != cudaSuccess)
      return 3000 + (int)cudaGetLastError();
    attr_set = true;
  }
  dim3 grid((max_q + kPfQ - 1) / kPfQ, hq, B);
  cudaError_t e = launch_pdl(attn_prefill_tc_kernel, grid, dim3(192), (size_t)kPfSmem, st, tmQ, tmK, tmV, p);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}
