// Quantised-weight GEMMs for sm_100a.
//
// (1) Weight-only dequant-GEMM: Y[T,N] = epi( X[T,K] · dequant(Wq[N,K])^T ), bf16 activations, weights int8,
//     uint4 (two codes per byte, low nibble first), nf4 (16-entry code book) with per-output-channel
//     w = q*scale + zero, or fp8 e4m3 with one fp32 scale per 128x128 block.  Reference: the xDNN
//     f32s8f32 / f32u4f32 / f32nf4f32 kernels behind MMHelper::compute* (src/utils/matmul_helper.h:565-1705)
//     and xdnn_small_amx_sgemm_bf16f8bf16_* (matmul_helper.h:692-727, fp8 dequantised to bf16 before a bf16 MMA).
//     Here TMA brings the packed tile into shared memory, four warps expand it to bf16 in the 128-byte-swizzled
//     K-major layout the tensor core wants (exact for int8/uint4; fp8 is scaled per block and rounded to bf16,
//     matching the reference's numerics), and the same tcgen05 / TMEM pipeline as the bf16 kernel runs on it.
//     Per-channel scale and zero are applied on the accumulator: y = s[n]*acc + z[n]*sum_k x[t,k].
//
// (2) W8A8: per-row dynamic asymmetric int8 activations (zero = (min+max)/2, scale = max|x-zero|/127,
//     matmul_helper.h:2813-2855) x int8 weights on the int8 tensor path (tcgen05 kind::i8, s32 accumulators in
//     TMEM); epilogue  y = sa*sw*acc + sa*zw*sum(qx) + za*sw*sum(qw) + K*za*zw  (+ bias, act, residual).
//
// Both kernels share the split-K scheme of gemm_sm100.cu (partials in fp32 scratch, last arriver reduces).
#include "ptx.cuh"

#include <cuda_fp8.h>

namespace xft {

int make_tensor_map(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                    uint32_t esize);
void plan_splits(int tiles, int num_kb, int bn, int nacc, size_t ws_bytes, int max_tiles, int* splits, int* kb_per_split);
int pick_bn(int T);

enum { Q_INT8 = 0, Q_INT4 = 1, Q_NF4 = 2, Q_FP8 = 3, Q_INT4F = 4 };

struct QGemmParams {
  int N, T, K;
  int dual_off;
  void* out; int ldo; int out_fp32;
  const float* bias;
  const __nv_bfloat16* residual; int ldr; float res_scale;
  int act;
  int splits, kb_per_split, num_kb;
  float* ws; int* counters; int* status;
  int n_tiles, t_tiles, stages;
  const float* scale;      // [N] per channel (int8/int4/nf4)  |  fp8: [ceil(N/128), ceil(K/128)] block scales
  const float* zero;       // [N] or null
  const float* xsum;       // [T] sum_k x[t,k] (needed when zero != null)
  int scale_ld;            // fp8: blocks per scale row
  // w8a8
  const float* a_scale; const float* a_zero; const float* a_qsum;   // [T]
  const float* w_sum;      // [N] sum_k qw
  // Grouped mode (MoE experts, fp8 block-scaled weights): token tile i is group_tiles[i] = {group, first row, rows, -};
  // the weight rows (and, /128, the scale rows) of group g start at g * group_w_rows.  No split-K.
  const int4* group_tiles;
  const int* num_group_tiles;
  int group_w_rows;
  const float* col_scale;  // optional per-token factor on the result (routing weight)
};

__device__ __forceinline__ float q_act(float x, int act) {
  if (act == 1) return fmaxf(x, 0.f);
  if (act == 2) return x / (1.f + __expf(-x));
  if (act == 3) { float u = 0.7978845608028654f * (x + 0.044715f * x * x * x); return 0.5f * x * (1.f + tanhf(u)); }
  return x;
}

__constant__ float c_nf4[16] = {-1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
                                -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
                                0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f,
                                0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};

__device__ __forceinline__ uint32_t pk(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Expand one packed row (64 K-elements) into the swizzled bf16 A tile: row r, 8 chunks of 16 B, chunk c at c ^ (r & 7).
template <int QT>
__device__ __forceinline__ void expand_row(const uint8_t* raw_row, uint8_t* a_tile, int r, float fp8_scale) {
  uint8_t* dst_row = a_tile + r * 128;
#pragma unroll
  for (int c = 0; c < 8; ++c) {          // 8 K-elements per chunk
    float f[8];
    if (QT == Q_INT8) {
      const uint2 w = *reinterpret_cast<const uint2*>(raw_row + c * 8);
      const int8_t* b = reinterpret_cast<const int8_t*>(&w);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = (float)b[j];
    } else if (QT == Q_FP8) {
      const uint2 w = *reinterpret_cast<const uint2*>(raw_row + c * 8);
      const __nv_fp8_e4m3* b = reinterpret_cast<const __nv_fp8_e4m3*>(&w);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = float(b[j]) * fp8_scale;
    } else {
      const uint32_t w = *reinterpret_cast<const uint32_t*>(raw_row + c * 4);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int q = (w >> (4 * j)) & 0xF;          // low nibble = even element
        f[j] = (QT == Q_NF4) ? c_nf4[q] : (float)q;
      }
    }
    *reinterpret_cast<uint4*>(dst_row + ((c ^ (r & 7)) << 4)) = make_uint4(pk(f[0], f[1]), pk(f[2], f[3]), pk(f[4], f[5]), pk(f[6], f[7]));
  }
}

// Cooperative expansion of a whole raw tile by the 128 expand threads, 16 bytes per thread and step, so that the
// loads are consecutive and the swizzled 16-byte stores of a quarter warp never share a bank.
//   Q_INT8:  the byte u = q + 128 is dropped into the mantissa of 2^23 (one PRMT), 2^23 + 128 is subtracted (exact),
//            and the upper halves of two such floats are one bf16 pair (one PRMT): no integer-to-float conversion.
//   Q_INT4F: words are stored nibble-interleaved (nibble i = element 2i, nibble i + 4 = element 2i + 1), so
//            (w >> 4i) & 0x000F000F | 0x43004300 IS the bf16 pair (128 + e_2i, 128 + e_2i+1): one shift and one
//            logic op per two elements.  The constant 128 is removed in the epilogue through the activations' row
//            sums (the caller passes zero - 128 * scale).
template <int QT>
__device__ __forceinline__ void expand_tile(const uint8_t* raw, uint8_t* a_tile, int et) {
  if (QT == Q_INT8) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int ci = et + 128 * i, row = ci >> 2, part = ci & 3;
      const uint4 w = *reinterpret_cast<const uint4*>(raw + ci * 16);
      const uint32_t x[4] = {w.x ^ 0x80808080u, w.y ^ 0x80808080u, w.z ^ 0x80808080u, w.w ^ 0x80808080u};
      uint32_t o[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float f0 = __uint_as_float(__byte_perm(x[j], 0x4B000000u, 0x7540)) - 8388736.0f;
        const float f1 = __uint_as_float(__byte_perm(x[j], 0x4B000000u, 0x7541)) - 8388736.0f;
        const float f2 = __uint_as_float(__byte_perm(x[j], 0x4B000000u, 0x7542)) - 8388736.0f;
        const float f3 = __uint_as_float(__byte_perm(x[j], 0x4B000000u, 0x7543)) - 8388736.0f;
        o[2 * j] = __byte_perm(__float_as_uint(f0), __float_as_uint(f1), 0x7632);
        o[2 * j + 1] = __byte_perm(__float_as_uint(f2), __float_as_uint(f3), 0x7632);
      }
      uint8_t* dst = a_tile + row * 128;
      *reinterpret_cast<uint4*>(dst + (((2 * part) ^ (row & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
      *reinterpret_cast<uint4*>(dst + (((2 * part + 1) ^ (row & 7)) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
    }
  } else {   // Q_INT4F
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int ci = et + 128 * i, row = ci >> 1, part = ci & 1;
      const uint4 w = *reinterpret_cast<const uint4*>(raw + ci * 16);
      const uint32_t x[4] = {w.x, w.y, w.z, w.w};
      uint8_t* dst = a_tile + row * 128;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t v = x[j];
        *reinterpret_cast<uint4*>(dst + (((4 * part + j) ^ (row & 7)) << 4)) =
            make_uint4((v & 0x000F000Fu) | 0x43004300u, ((v >> 4) & 0x000F000Fu) | 0x43004300u,
                       ((v >> 8) & 0x000F000Fu) | 0x43004300u, ((v >> 12) & 0x000F000Fu) | 0x43004300u);
      }
    }
  }
}

constexpr int kQMaxStages = 8;

template <int BN, bool DUAL, int QT>
__global__ void __launch_bounds__(192) qgemm_kernel(const __grid_constant__ CUtensorMap tmW,
                                                    const __grid_constant__ CUtensorMap tmX, const QGemmParams p) {
  constexpr int RAW_BYTES = (QT == Q_INT8 || QT == Q_FP8) ? 128 * 64 : 128 * 32;      // Q_INT4F is packed like Q_INT4
  constexpr int RAW_ROW = RAW_BYTES / 128;
  constexpr int A_BYTES = 128 * 64 * 2;
  constexpr int B_BYTES = BN * 64 * 2;
  constexpr int NACC = DUAL ? 2 : 1;
  constexpr int STAGE_BYTES = (RAW_BYTES + A_BYTES) * NACC + B_BYTES;
  constexpr int TX_BYTES = RAW_BYTES * NACC + B_BYTES;
  constexpr uint32_t TMEM_COLS = (BN * NACC <= 32) ? 32 : (BN * NACC <= 64) ? 64 : (BN * NACC <= 128) ? 128
                                 : (BN * NACC <= 256) ? 256 : 512;
  constexpr uint32_t IDESC = umma_idesc(128, BN, 1, 1, 1);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t raw_full[kQMaxStages], a_ready[kQMaxStages], empty_bar[kQMaxStages], tmem_full_bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_last;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int stages = p.stages;
  int tile_n, tile_t;
  {
    const int GN = 16;
    int bid = blockIdx.x;
    int per_group = GN * p.t_tiles;
    int g = bid / per_group, r = bid % per_group;
    int gn = min(GN, p.n_tiles - g * GN);
    tile_n = g * GN + r % gn;
    tile_t = r / gn;
  }
  const int split = blockIdx.y;
  const int kb0 = split * p.kb_per_split;
  const int kb1 = min(kb0 + p.kb_per_split, p.num_kb);
  const int tile_id = tile_t * p.n_tiles + tile_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&a_ready[s], 128);       // every expanding thread arrives
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&tmem_full_bar, 1);
    fence_barrier_init();
    fence_proxy_async();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_s, TMEM_COLS);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  grid_dep_launch();
  __shared__ int s_group[4];
  const bool grouped = p.group_tiles != nullptr;
  if (grouped) {
    grid_dep_wait();          // the tile table comes from the routing plan kernel
    if (threadIdx.x == 0) {
      int4 e = make_int4(0, 0, 0, 0);
      if (tile_t < *p.num_group_tiles) e = p.group_tiles[tile_t];
      s_group[0] = e.x; s_group[1] = e.y; s_group[2] = e.z;
    }
    __syncthreads();
  }
  const int w_row0 = grouped ? s_group[0] * p.group_w_rows : 0;
  const int x_row0 = grouped ? s_group[1] : tile_t * BN;
  const int x_rows = grouped ? s_group[2] : BN;
  const bool active = !grouped || x_rows > 0;
  const int kend = active ? kb1 : kb0;

  // stage layout: [raw A (xNACC)] [bf16 A (xNACC)] [B]
  if (warp == 0) {
    if (lane == 0) {
      const uint64_t hint_w = p.t_tiles == 1 ? kEvictFirst : kEvictNormal;
      const uint64_t hint_x = p.n_tiles > 1 ? kEvictLast : kEvictNormal;
      constexpr int KEL = (QT == Q_INT8 || QT == Q_FP8) ? 64 : 32;      // raw bytes per k-block row
      // weights never depend on the previous kernel: the first `stages` raw tiles are requested before the grid
      // dependency resolves
      const int pre = min(stages, kend - kb0);
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(&raw_full[i], TX_BYTES);
        uint8_t* st = smem + i * STAGE_BYTES;
        tma_load_2d(st, &tmW, &raw_full[i], (kb0 + i) * KEL, w_row0 + tile_n * 128, hint_w);
        if (DUAL) tma_load_2d(st + RAW_BYTES, &tmW, &raw_full[i], (kb0 + i) * KEL, w_row0 + p.dual_off + tile_n * 128, hint_w);
      }
      grid_dep_wait();
      for (int i = 0; i < pre; ++i)
        tma_load_2d(smem + i * STAGE_BYTES + (RAW_BYTES + A_BYTES) * NACC, &tmX, &raw_full[i], (kb0 + i) * 64, x_row0, hint_x);
      int it = pre;
      for (int kb = kb0 + pre; kb < kend; ++kb, ++it) {
        const int s = it % stages;
        const uint32_t ph = (it / stages) & 1;
        if (!mbar_wait(&empty_bar[s], ph ^ 1, p.status, XFT_ERR_WAIT_EMPTY)) break;
        mbar_expect_tx(&raw_full[s], TX_BYTES);
        uint8_t* st = smem + s * STAGE_BYTES;
        tma_load_2d(st, &tmW, &raw_full[s], kb * KEL, w_row0 + tile_n * 128, hint_w);
        if (DUAL) tma_load_2d(st + RAW_BYTES, &tmW, &raw_full[s], kb * KEL, w_row0 + p.dual_off + tile_n * 128, hint_w);
        tma_load_2d(st + (RAW_BYTES + A_BYTES) * NACC, &tmX, &raw_full[s], kb * 64, x_row0, hint_x);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && active) {
      int it = 0;
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % stages;
        const uint32_t ph = (it / stages) & 1;
        if (!mbar_wait(&a_ready[s], ph, p.status, XFT_ERR_WAIT_FULL)) break;
        tcgen05_fence_after();
        const uint32_t base = smem_u32(smem + s * STAGE_BYTES);
        const uint64_t adesc = umma_desc_k128(base + RAW_BYTES * NACC);
        const uint64_t bdesc = umma_desc_k128(base + (RAW_BYTES + A_BYTES) * NACC);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          umma_bf16(tmem_base, adesc + 2 * k, bdesc + 2 * k, IDESC, (it > 0 || k > 0) ? 1u : 0u);
          if (DUAL) {
            const uint64_t a1 = umma_desc_k128(base + RAW_BYTES * NACC + A_BYTES);
            umma_bf16(tmem_base + BN, a1 + 2 * k, bdesc + 2 * k, IDESC, (it > 0 || k > 0) ? 1u : 0u);
          }
        }
        tcgen05_commit(&empty_bar[s]);
      }
      tcgen05_commit(&tmem_full_bar);
    }
  } else {
    // ---- expand warps (one weight row per thread), then the epilogue on the same threads -----------
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int n = tile_n * 128 + row;
    const bool n_ok = n < p.N;
    const int et = threadIdx.x - 64;
    {
      int it = 0;
      bool alive = true;
      for (int kb = kb0; kb < kend; ++kb, ++it) {
        const int s = it % stages;
        const uint32_t ph = (it / stages) & 1;
        if (alive && !mbar_wait(&raw_full[s], ph, p.status, XFT_ERR_WAIT_FULL)) alive = false;
        if (alive) {
          uint8_t* st = smem + s * STAGE_BYTES;
          float sc0 = 1.f, sc1 = 1.f;
          if (QT == Q_FP8) {
            sc0 = p.scale[(size_t)((w_row0 >> 7) + tile_n) * p.scale_ld + (kb >> 1)];
            if (DUAL) sc1 = p.scale[(size_t)((w_row0 >> 7) + (p.dual_off >> 7) + tile_n) * p.scale_ld + (kb >> 1)];
          }
          if (QT == Q_INT8 || QT == Q_INT4F) {
            expand_tile<QT>(st, st + RAW_BYTES * NACC, et);
            if (DUAL) expand_tile<QT>(st + RAW_BYTES, st + RAW_BYTES * NACC + A_BYTES, et);
          } else {
            expand_row<QT>(st + row * RAW_ROW, st + RAW_BYTES * NACC, row, sc0);
            if (DUAL) expand_row<QT>(st + RAW_BYTES + row * RAW_ROW, st + RAW_BYTES * NACC + A_BYTES, row, sc1);
          }
          fence_proxy_async();            // generic-proxy stores -> visible to the tensor core's async reads
        }
        mbar_arrive(&a_ready[s]);
      }
    }
    grid_dep_wait();
    bool ok = active && mbar_wait(&tmem_full_bar, 0, p.status, XFT_ERR_WAIT_TMEM);
    tcgen05_fence_after();
    const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16);
    const int t0 = x_row0;
    bool last = true;
    if (p.splits > 1) {
      float* wsp = p.ws + ((size_t)split * (p.n_tiles * p.t_tiles) + tile_id) * (size_t)(BN * NACC) * 128;
      if (ok) {
#pragma unroll 1
        for (int c = 0; c < BN * NACC; c += 16) {
          uint32_t v[16];
          tmem_ld16(taddr + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) wsp[(size_t)(c + j) * 128 + row] = __uint_as_float(v[j]);
        }
      }
      __threadfence();
      named_bar_sync(1, 128);
      if (et == 0) {
        int old = atomicAdd(&p.counters[tile_id], 1);
        s_last = (old == p.splits - 1);
        if (s_last) p.counters[tile_id] = 0;
      }
      named_bar_sync(1, 128);
      last = s_last != 0;
      if (last) __threadfence();
    }
    if (last && ok) {
      const float bias_g = (p.bias && n_ok) ? p.bias[n] : 0.f;
      const float bias_u = (DUAL && p.bias && n_ok) ? p.bias[p.dual_off + n] : 0.f;
      const bool per_ch = QT != Q_FP8;
      const float sg = (per_ch && n_ok) ? p.scale[n] : 1.f;
      const float su = (per_ch && DUAL && n_ok) ? p.scale[p.dual_off + n] : 1.f;
      const float zg = (per_ch && p.zero && n_ok) ? p.zero[n] : 0.f;
      const float zu = (per_ch && DUAL && p.zero && n_ok) ? p.zero[p.dual_off + n] : 0.f;
      const float* ws_tile = p.ws + (size_t)tile_id * (size_t)(BN * NACC) * 128;
      const size_t ws_split_stride = (size_t)(p.n_tiles * p.t_tiles) * (size_t)(BN * NACC) * 128;
#pragma unroll 1
      for (int c = 0; c < BN; c += 16) {
        float g[16], u[16];
        if (p.splits > 1) {
#pragma unroll
          for (int j = 0; j < 16; ++j) { g[j] = 0.f; u[j] = 0.f; }
          for (int s = 0; s < p.splits; ++s) {
            const float* w = ws_tile + s * ws_split_stride;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              g[j] += __ldcg(w + (size_t)(c + j) * 128 + row);
              if (DUAL) u[j] += __ldcg(w + (size_t)(BN + c + j) * 128 + row);
            }
          }
        } else {
          uint32_t v[16];
          tmem_ld16(taddr + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) g[j] = __uint_as_float(v[j]);
          if (DUAL) {
            tmem_ld16(taddr + BN + c, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) u[j] = __uint_as_float(v[j]);
          }
        }
        if (n_ok) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int t = t0 + c + j;
            if (t < p.T && c + j < x_rows) {
              const float xs = (p.zero && p.xsum) ? p.xsum[t] : 0.f;
              float x = g[j] * sg + zg * xs + bias_g;
              x = q_act(x, p.act);
              if (DUAL) x *= (u[j] * su + zu * xs + bias_u);
              if (p.col_scale) x *= p.col_scale[t];
              if (p.residual) x += p.res_scale * __bfloat162float(p.residual[(size_t)t * p.ldr + n]);
              if (p.out_fp32) reinterpret_cast<float*>(p.out)[(size_t)t * p.ldo + n] = x;
              else reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)t * p.ldo + n] = __float2bfloat16(x);
            }
          }
        }
      }
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------ W8A8
// A = int8 weights [N,K] (128 K-elements per 128-byte swizzled row), B = int8 activations [T,K]; s32 accumulators.
template <int BN>
__global__ void __launch_bounds__(192) w8a8_gemm_kernel(const __grid_constant__ CUtensorMap tmW,
                                                        const __grid_constant__ CUtensorMap tmX, const QGemmParams p) {
  constexpr int A_BYTES = 128 * 128;
  constexpr int B_BYTES = BN * 128;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = BN <= 32 ? 32 : BN <= 64 ? 64 : BN <= 128 ? 128 : 256;
  constexpr uint32_t IDESC = umma_idesc(128, BN, 1, 1, 2);      // signed int8 x signed int8 -> s32

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full_bar[kQMaxStages], empty_bar[kQMaxStages], tmem_full_bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_last;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int stages = p.stages;
  const int tile_n = blockIdx.x % p.n_tiles, tile_t = blockIdx.x / p.n_tiles;
  const int split = blockIdx.y;
  const int kb0 = split * p.kb_per_split;
  const int kb1 = min(kb0 + p.kb_per_split, p.num_kb);
  const int tile_id = tile_t * p.n_tiles + tile_n;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(&tmem_full_bar, 1);
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) { tmem_alloc(&tmem_base_s, TMEM_COLS); tmem_relinquish(); }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  grid_dep_launch();
  if (warp == 0) {
    if (lane == 0) {
      grid_dep_wait();
      int it = 0;
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % stages;
        const uint32_t ph = (it / stages) & 1;
        if (!mbar_wait(&empty_bar[s], ph ^ 1, p.status, XFT_ERR_WAIT_EMPTY)) break;
        mbar_expect_tx(&full_bar[s], STAGE_BYTES);
        uint8_t* st = smem + s * STAGE_BYTES;
        tma_load_2d(st, &tmW, &full_bar[s], kb * 128, tile_n * 128, p.t_tiles == 1 ? kEvictFirst : kEvictNormal);
        tma_load_2d(st + A_BYTES, &tmX, &full_bar[s], kb * 128, tile_t * BN, kEvictLast);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int it = 0;
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % stages;
        const uint32_t ph = (it / stages) & 1;
        if (!mbar_wait(&full_bar[s], ph, p.status, XFT_ERR_WAIT_FULL)) break;
        tcgen05_fence_after();
        const uint32_t base = smem_u32(smem + s * STAGE_BYTES);
        const uint64_t adesc = umma_desc_k128(base), bdesc = umma_desc_k128(base + A_BYTES);
#pragma unroll
        for (int k = 0; k < 4; ++k)       // 4 x (K = 32 int8 = 32 bytes)
          umma_i8(tmem_base, adesc + 2 * k, bdesc + 2 * k, IDESC, (it > 0 || k > 0) ? 1u : 0u);
        tcgen05_commit(&empty_bar[s]);
      }
      tcgen05_commit(&tmem_full_bar);
    }
  } else {
    const int q = warp & 3, row = q * 32 + lane, n = tile_n * 128 + row;
    const bool n_ok = n < p.N;
    const int et = threadIdx.x - 64;
    grid_dep_wait();
    bool ok = mbar_wait(&tmem_full_bar, 0, p.status, XFT_ERR_WAIT_TMEM);
    tcgen05_fence_after();
    const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16);
    const int t0 = tile_t * BN;
    bool last = true;
    if (p.splits > 1) {
      float* wsp = p.ws + ((size_t)split * (p.n_tiles * p.t_tiles) + tile_id) * (size_t)BN * 128;
      if (ok) {
#pragma unroll 1
        for (int c = 0; c < BN; c += 16) {
          uint32_t v[16];
          tmem_ld16(taddr + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) wsp[(size_t)(c + j) * 128 + row] = (float)(int)v[j];
        }
      }
      __threadfence();
      named_bar_sync(1, 128);
      if (et == 0) {
        int old = atomicAdd(&p.counters[tile_id], 1);
        s_last = (old == p.splits - 1);
        if (s_last) p.counters[tile_id] = 0;
      }
      named_bar_sync(1, 128);
      last = s_last != 0;
      if (last) __threadfence();
    }
    if (last && ok) {
      const float sw = n_ok ? p.scale[n] : 0.f, zw = (n_ok && p.zero) ? p.zero[n] : 0.f;
      const float wsum = (n_ok && p.w_sum) ? p.w_sum[n] : 0.f;
      const float bias = (n_ok && p.bias) ? p.bias[n] : 0.f;
      const float* ws_tile = p.ws + (size_t)tile_id * (size_t)BN * 128;
      const size_t ws_split_stride = (size_t)(p.n_tiles * p.t_tiles) * (size_t)BN * 128;
#pragma unroll 1
      for (int c = 0; c < BN; c += 16) {
        float g[16];
        if (p.splits > 1) {
#pragma unroll
          for (int j = 0; j < 16; ++j) g[j] = 0.f;
          for (int s = 0; s < p.splits; ++s)
#pragma unroll
            for (int j = 0; j < 16; ++j) g[j] += __ldcg(ws_tile + s * ws_split_stride + (size_t)(c + j) * 128 + row);
        } else {
          uint32_t v[16];
          tmem_ld16(taddr + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) g[j] = (float)(int)v[j];
        }
        if (n_ok) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int t = t0 + c + j;
            if (t < p.T) {
              const float sa = p.a_scale[t], za = p.a_zero[t], qs = p.a_qsum[t];
              float x = sa * sw * g[j] + sa * zw * qs + za * sw * wsum + (float)p.K * za * zw + bias;
              x = q_act(x, p.act);
              if (p.residual) x += p.res_scale * __bfloat162float(p.residual[(size_t)t * p.ldr + n]);
              if (p.out_fp32) reinterpret_cast<float*>(p.out)[(size_t)t * p.ldo + n] = x;
              else reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)t * p.ldo + n] = __float2bfloat16(x);
            }
          }
        }
      }
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) { tcgen05_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

// Per-row dynamic int8 quantisation of activations (+ the sums the W8A8 epilogue needs) and plain row sums.
__global__ void __launch_bounds__(256) quant_act_kernel(const __nv_bfloat16* __restrict__ x, int ldx, int8_t* __restrict__ q,
                                                        int ldq, float* __restrict__ scale, float* __restrict__ zero,
                                                        float* __restrict__ qsum, int K) {
  __shared__ float smx[8], smn[8], ssum[8];
  grid_dep_launch();
  grid_dep_wait();
  const int t = blockIdx.x;
  const __nv_bfloat16* row = x + (size_t)t * ldx;
  float mx = -INFINITY, mn = INFINITY;
  for (int i = threadIdx.x; i < K; i += 256) { float v = __bfloat162float(row[i]); mx = fmaxf(mx, v); mn = fminf(mn, v); }
  for (int o = 16; o > 0; o >>= 1) { mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o)); mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o)); }
  if ((threadIdx.x & 31) == 0) { smx[threadIdx.x >> 5] = mx; smn[threadIdx.x >> 5] = mn; }
  __syncthreads();
  mx = smx[0]; mn = smn[0];
  for (int w = 1; w < 8; ++w) { mx = fmaxf(mx, smx[w]); mn = fminf(mn, smn[w]); }
  const float z = 0.5f * (mx + mn);
  const float s = fmaxf(fmaxf(mx - z, z - mn) / 127.f, 1e-10f);
  const float inv = 1.f / s;
  float acc = 0.f;
  for (int i = threadIdx.x; i < K; i += 256) {
    float r = rintf((__bfloat162float(row[i]) - z) * inv);
    r = fminf(fmaxf(r, -127.f), 127.f);
    q[(size_t)t * ldq + i] = (int8_t)r;
    acc += r;
  }
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) ssum[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = 0.f;
    for (int w = 0; w < 8; ++w) a += ssum[w];
    scale[t] = s; zero[t] = z; qsum[t] = a;
  }
}

__global__ void __launch_bounds__(256) row_sum_kernel(const __nv_bfloat16* __restrict__ x, int ldx, float* __restrict__ out, int K) {
  __shared__ float ssum[8];
  grid_dep_launch();
  grid_dep_wait();
  const int t = blockIdx.x;
  float acc = 0.f;
  for (int i = threadIdx.x; i < K; i += 256) acc += __bfloat162float(x[(size_t)t * ldx + i]);
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) ssum[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) { float a = 0.f; for (int w = 0; w < 8; ++w) a += ssum[w]; out[t] = a; }
}

// ------------------------------------------------------------------------------------------ host
typedef CUresult (*EncFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                          const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                          CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static int make_raw_map(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t row_bytes, uint64_t ld_bytes,
                        uint32_t box_rows, uint32_t box_bytes) {
  static EncFn enc = nullptr;
  if (!enc) {
    void* fp = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fp, cudaEnableDefault, &q) != cudaSuccess) return -1;
    enc = reinterpret_cast<EncFn>(fp);
  }
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (ld_bytes & 15)) return -2;
  cuuint64_t dims[2] = {row_bytes, rows};
  cuuint64_t strides[1] = {ld_bytes};
  cuuint32_t box[2] = {box_bytes, box_rows};
  cuuint32_t es[2] = {1, 1};
  return enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, es,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? 0 : -3;
}

template <int BN, bool DUAL, int QT>
static int launch_q(const CUtensorMap& tmW, const CUtensorMap& tmX, QGemmParams& p, cudaStream_t st) {
  constexpr int RAW = (QT == Q_INT8 || QT == Q_FP8) ? 128 * 64 : 128 * 32;
  constexpr int STAGE = (RAW + 128 * 64 * 2) * (DUAL ? 2 : 1) + BN * 64 * 2;
  int budget = (BN <= 64) ? 110 * 1024 : 220 * 1024;
  if (budget / STAGE < 3) budget = 220 * 1024;
  int stages = budget / STAGE;
  if (stages > kQMaxStages) stages = kQMaxStages;
  if (stages < 2) stages = 2;
  p.stages = stages;
  static bool attr = false;
  if (!attr) { cudaFuncSetAttribute(qgemm_kernel<BN, DUAL, QT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024); attr = true; }
  cudaError_t e = launch_pdl(qgemm_kernel<BN, DUAL, QT>, dim3(p.n_tiles * p.t_tiles, p.splits), dim3(192),
                             (size_t)stages * STAGE + 1024, st, tmW, tmX, p);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

template <int BN, bool DUAL>
static int launch_qt(int qt, const CUtensorMap& a, const CUtensorMap& b, QGemmParams& p, cudaStream_t st) {
  switch (qt) {
    case Q_INT8: return launch_q<BN, DUAL, Q_INT8>(a, b, p, st);
    case Q_INT4: return launch_q<BN, DUAL, Q_INT4>(a, b, p, st);
    case Q_NF4: return launch_q<BN, DUAL, Q_NF4>(a, b, p, st);
    case Q_FP8: return launch_q<BN, DUAL, Q_FP8>(a, b, p, st);
    case Q_INT4F: return launch_q<BN, DUAL, Q_INT4F>(a, b, p, st);
  }
  return -1;
}

}  // namespace xft

using namespace xft;

// qtype: 0 int8, 1 uint4, 2 nf4, 3 fp8-e4m3 (block 128x128), 4 uint4 with nibble-interleaved words (nibble i of a
// 32-bit word = element 2i, nibble i + 4 = element 2i + 1; the kernel feeds 128 + q, so the caller passes
// zero - 128 * scale and always the row sums).  Wq: [w_rows, K] int8/fp8 or [w_rows, K/2] packed.
// scale/zero: see QGemmParams.  xsum: [T] row sums of X, required when zero != null.
extern "C" int xft_qgemm(const void* X, int ldx, const void* Wq, int w_rows, int ldw_bytes, int qtype, void* Y, int ldo,
                         int out_fp32, int T, int N, int K, int gated, int dual_off, const float* scale, const float* zero,
                         const float* xsum, int scale_ld, const float* bias, const void* residual, int ldr,
                         float res_scale, int act, float* ws, size_t ws_bytes, int* counters, int n_counters, int* status,
                         cudaStream_t st) {
  if (T <= 0 || N <= 0 || K <= 0) return 0;
  if (qtype == Q_FP8 && gated && (dual_off & 127)) return -4;
  QGemmParams p{};
  p.N = N; p.T = T; p.K = K; p.dual_off = dual_off; p.out = Y; p.ldo = ldo; p.out_fp32 = out_fp32; p.bias = bias;
  p.residual = (const __nv_bfloat16*)residual; p.ldr = ldr; p.res_scale = res_scale; p.act = act; p.ws = ws;
  p.counters = counters; p.status = status; p.scale = scale; p.zero = zero; p.xsum = xsum; p.scale_ld = scale_ld;
  const int bn = pick_bn(T) > 128 ? 128 : pick_bn(T);
  p.n_tiles = (N + 127) / 128;
  p.t_tiles = (T + bn - 1) / bn;
  p.num_kb = (K + 63) / 64;
  plan_splits(p.n_tiles * p.t_tiles, p.num_kb, bn, gated ? 2 : 1, ws ? ws_bytes : 0, counters ? n_counters : 0, &p.splits,
              &p.kb_per_split);
  CUtensorMap tmW, tmX;
  const bool byte_el = qtype == Q_INT8 || qtype == Q_FP8;
  int r = make_raw_map(&tmW, Wq, (uint64_t)w_rows, byte_el ? (uint64_t)K : (uint64_t)K / 2, (uint64_t)ldw_bytes, 128,
                       byte_el ? 64 : 32);
  if (r) return 1000 - r;
  r = make_tensor_map(&tmX, X, (uint64_t)T, (uint64_t)K, (uint64_t)ldx, (uint32_t)bn, 2);
  if (r) return 2000 - r;
#define XFT_Q(BN_) case BN_: return gated ? launch_qt<BN_, true>(qtype, tmW, tmX, p, st) : launch_qt<BN_, false>(qtype, tmW, tmX, p, st);
  switch (bn) { XFT_Q(16) XFT_Q(32) XFT_Q(64) XFT_Q(128) }
#undef XFT_Q
  return -1;
}

// Grouped (MoE expert) form of the fp8 block-scaled GEMM: Wq stacks the experts' [group_w_rows, K] e4m3 matrices,
// scale stacks their [group_w_rows/128, ceil(K/128)] block scales, group_tiles / num_group_tiles come from
// xft_moe_plan (csrc/kernels/moe.cu).  gated: rows [0, N) of an expert are the gate, rows [dual_off, dual_off + N) the
// up projection.  col_scale: per-row factor on the result (routing weight).  Keeps DeepSeek-V3/R1 experts in fp8 on the
// device (the reference's fp8 expert GEMM: src/layers/moe_deepseek.h, xdnn_*_f8e4m3 calls in src/utils/matmul_helper.h).
extern "C" int xft_qgemm_grouped(const void* X, int ldx, int x_rows, const void* Wq, int w_rows, int ldw_bytes, void* Y,
                                 int ldo, int out_fp32, int N, int K, int gated, int dual_off, int group_w_rows,
                                 const float* scale, int scale_ld, const void* group_tiles, const int* num_group_tiles,
                                 int max_tiles, int bn, const float* col_scale, int act, int* status, cudaStream_t st) {
  if (x_rows <= 0 || N <= 0 || K <= 0 || max_tiles <= 0) return 0;
  if ((group_w_rows & 127) || (gated && (dual_off & 127)) || (K & 15)) return -4;
  QGemmParams p{};
  p.N = N; p.T = x_rows; p.K = K; p.dual_off = dual_off; p.out = Y; p.ldo = ldo; p.out_fp32 = out_fp32;
  p.res_scale = 1.f; p.act = act; p.status = status; p.scale = scale; p.scale_ld = scale_ld;
  p.group_tiles = reinterpret_cast<const int4*>(group_tiles); p.num_group_tiles = num_group_tiles;
  p.group_w_rows = group_w_rows; p.col_scale = col_scale;
  p.n_tiles = (N + 127) / 128;
  p.t_tiles = max_tiles;
  p.num_kb = (K + 63) / 64;
  p.splits = 1; p.kb_per_split = p.num_kb;
  CUtensorMap tmW, tmX;
  int r = make_raw_map(&tmW, Wq, (uint64_t)w_rows, (uint64_t)K, (uint64_t)ldw_bytes, 128, 64);
  if (r) return 1000 - r;
  r = make_tensor_map(&tmX, X, (uint64_t)x_rows, (uint64_t)K, (uint64_t)ldx, (uint32_t)bn, 2);
  if (r) return 2000 - r;
#define XFT_QG(BN_) case BN_: return gated ? launch_q<BN_, true, Q_FP8>(tmW, tmX, p, st) : launch_q<BN_, false, Q_FP8>(tmW, tmX, p, st);
  switch (bn) { XFT_QG(16) XFT_QG(32) XFT_QG(64) XFT_QG(128) }
#undef XFT_QG
  return -1;
}

extern "C" int xft_quant_act(const void* x, int ldx, void* q, int ldq, float* scale, float* zero, float* qsum, int T, int K,
                             cudaStream_t st) {
  if (T <= 0) return 0;
  cudaError_t e = launch_pdl(quant_act_kernel, dim3(T), dim3(256), 0, st, (const __nv_bfloat16*)x, ldx, (int8_t*)q, ldq, scale,
                             zero, qsum, K);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

extern "C" int xft_row_sum(const void* x, int ldx, float* out, int T, int K, cudaStream_t st) {
  if (T <= 0) return 0;
  cudaError_t e = launch_pdl(row_sum_kernel, dim3(T), dim3(256), 0, st, (const __nv_bfloat16*)x, ldx, out, K);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

// Y = epi(dequant(qx) · dequant(Wq)^T): qx int8 [T, K] with a_scale/a_zero/a_qsum from xft_quant_act.
extern "C" int xft_w8a8_gemm(const void* qx, int ldqx, const void* Wq, int ldw, void* Y, int ldo, int out_fp32, int T, int N,
                             int K, const float* a_scale, const float* a_zero, const float* a_qsum, const float* w_scale,
                             const float* w_zero, const float* w_sum, const float* bias, const void* residual, int ldr,
                             float res_scale, int act, float* ws, size_t ws_bytes, int* counters, int n_counters,
                             int* status, cudaStream_t st) {
  if (T <= 0 || N <= 0 || K <= 0) return 0;
  if (K % 16) return -4;
  QGemmParams p{};
  p.N = N; p.T = T; p.K = K; p.out = Y; p.ldo = ldo; p.out_fp32 = out_fp32; p.bias = bias;
  p.residual = (const __nv_bfloat16*)residual; p.ldr = ldr; p.res_scale = res_scale; p.act = act; p.ws = ws;
  p.counters = counters; p.status = status; p.scale = w_scale; p.zero = w_zero; p.w_sum = w_sum; p.a_scale = a_scale;
  p.a_zero = a_zero; p.a_qsum = a_qsum;
  const int bn = pick_bn(T);
  p.n_tiles = (N + 127) / 128;
  p.t_tiles = (T + bn - 1) / bn;
  p.num_kb = (K + 127) / 128;
  plan_splits(p.n_tiles * p.t_tiles, p.num_kb, bn, 1, ws ? ws_bytes : 0, counters ? n_counters : 0, &p.splits, &p.kb_per_split);
  CUtensorMap tmW, tmX;
  int r = make_tensor_map(&tmW, Wq, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, 128, 1);
  if (r) return 1000 - r;
  r = make_tensor_map(&tmX, qx, (uint64_t)T, (uint64_t)K, (uint64_t)ldqx, (uint32_t)bn, 1);
  if (r) return 2000 - r;
  const int stage = 128 * 128 + bn * 128;
  int budget = bn <= 64 ? 110 * 1024 : 220 * 1024;
  int stages = budget / stage;
  if (stages > kQMaxStages) stages = kQMaxStages;
  if (stages < 2) stages = 2;
  p.stages = stages;
  const size_t smem = (size_t)stages * stage + 1024;
  dim3 grid(p.n_tiles * p.t_tiles, p.splits);
  cudaError_t e = cudaSuccess;
#define XFT_W(BN_)                                                                                             \
  case BN_:                                                                                                    \
    cudaFuncSetAttribute(w8a8_gemm_kernel<BN_>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);      \
    e = launch_pdl(w8a8_gemm_kernel<BN_>, grid, dim3(192), smem, st, tmW, tmX, p);                             \
    break;
  switch (bn) { XFT_W(16) XFT_W(32) XFT_W(64) XFT_W(128) XFT_W(256) default: return -1; }
#undef XFT_W
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}
