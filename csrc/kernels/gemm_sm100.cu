// bf16 GEMM for sm_100a:  Y[T, N] = epilogue( X[T, K] · W[N, K]^T )
//
// Replaces the reference's MMHelper::compute* family (src/utils/matmul_helper.h:565-1705: compute,
// compute_bias, compute_biasadd_relu, compute_silu, compute_gelu, compute_resmul, compute_residential,
// compute_resext) — there dispatched to xDNN/oneDNN AMX kernels — with one tcgen05 kernel.
//
// Mapping.  The weight is always the 128-row UMMA "A" operand (M = 128 output features per CTA) and
// the activations are the UMMA "B" operand (N = BN tokens, 16..256), both K-major in shared memory
// with the 128-byte swizzle, staged by TMA.  The accumulator lives in TMEM as [128 lanes = output
// features] x [BN columns = tokens].  With few tokens (decode) the tile is still a full-rate MMA
// and the kernel is a pure weight stream; with many tokens BN = 256 reaches the tensor-core peak
// of a single-CTA MMA.  A gated variant (DUAL) keeps two accumulators, gate and up, fed by two
// weight tiles and the same token tile, and applies act(gate)*up on the way out of TMEM
// (siluSum/geluSum of src/utils/decoder_util.h:495-607 fused into the GEMM).
//
// Warp roles (192 threads): warp 0 = TMA producer (one lane), warp 1 = TMEM owner + MMA issuer (one
// lane), warps 2-5 = epilogue (TMEM lane quadrant = warp_id % 4).
//
// Split-K: when the tile count cannot fill 148 SMs (decode, TP slices), grid.y CTAs share an output
// tile, each reducing a K range.  Partials go to an fp32 scratch in accumulator layout
// [split][tile][column][128 rows]; the CTA that arrives last on the tile's counter sums the splits
// in index order (deterministic) and runs the epilogue.  Nobody spins: there is no wait on a peer.
#include "gemm_common.cuh"
#include "gemm_noalloc.h"

#include <cmath>
#include <mutex>
#include <unordered_map>

namespace xft {

int g_xft_pdl = 1;

struct GemmParams {
  int N, T, K;
  int dual_off;            // DUAL: W row of the first "up" feature (gate rows are [0, dual_off))
  void* out;               // [T, ldo] bf16 or fp32
  int ldo;
  int out_fp32;
  const float* bias;       // [N] (DUAL: [2N] gate then up at dual_off)
  const __nv_bfloat16* residual;
  int ldr;
  float res_scale;
  int act;                 // 0 none, 1 relu, 2 silu, 3 gelu(tanh)
  int splits, kb_per_split, num_kb;
  float* ws;               // split-K partials
  int* counters;           // one per output tile, zero between launches
  int* status;
  int n_tiles, t_tiles, stages;
  const float* row_scale;  // optional per-output-feature scale applied to the accumulator (weight-only int8)
  CommParams ar;           // ar.world > 1: the epilogue all-reduces the tile over peer memory
  // Grouped mode (MoE experts): token tile i is described by group_tiles[i] = {group, first row, rows, -};
  // the weight rows of group g start at g * group_w_rows.  num_group_tiles[0] tiles are valid; CTAs past it idle.
  const int4* group_tiles;
  const int* num_group_tiles;
  int group_w_rows;
  const float* col_scale;  // optional per-token factor applied to the result (routing weight)
  // pair != 0 (DUAL instantiation, no gating): the two accumulators are two independent 128-feature tiles
  // (rows n and n + 128 of W) sharing one token tile — 256 x BN of output per CTA, which halves the
  // operand bytes per FLOP of the compute-bound (prefill) shapes.
  int pair;
  // rms_x != null: the GEMM input is the un-normalised hidden state and the RMSNorm gain is already folded into W's
  // columns, so  RMSNorm(x) W^T = rsqrt(mean(x^2) + eps) * (x W'^T): the epilogue warps compute each token's sum
  // of squares over this CTA's K slice while the main loop runs (split-K slices add up through rms_ws) and apply
  // the factor to the accumulator.  Only for token tiles of at most 64 rows (decode).
  const __nv_bfloat16* rms_x;
  int rms_ldx;
  float rms_eps;
  float* rms_ws;           // [tile][split][BN] partial sums of squares
};

constexpr int kMaxStages = 12;

template <int BN, bool DUAL>
__global__ void __launch_bounds__(192) gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmW,
                                                        const __grid_constant__ CUtensorMap tmX, const GemmParams p) {
  constexpr int A_BYTES = 128 * 64 * 2;
  constexpr int B_BYTES = BN * 64 * 2;
  constexpr int NACC = DUAL ? 2 : 1;
  constexpr int STAGE_BYTES = A_BYTES * NACC + B_BYTES;
  constexpr uint32_t TMEM_COLS = (BN * NACC <= 32) ? 32 : (BN * NACC <= 64) ? 64 : (BN * NACC <= 128) ? 128
                                 : (BN * NACC <= 256) ? 256 : 512;
  constexpr uint32_t IDESC = umma_idesc(128, BN, 1, 1, 1);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full_bar[kMaxStages], empty_bar[kMaxStages], tmem_full_bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_last;
  __shared__ int s_epoch, s_peer_fail;
  __shared__ float s_ssq[64];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int stages = p.stages;

  // tile coordinates: groups of 16 feature tiles sweep all token tiles before moving on, so the
  // CTAs resident together share few distinct weight and token tiles (L2 reuse)
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
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&tmem_full_bar, 1);
    s_peer_fail = 0;
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
  grid_dep_launch();          // all CTAs of this grid are (or have been) resident once each has passed here
  __shared__ int s_group[4];
  const bool grouped = p.group_tiles != nullptr;
  if (grouped) {
    grid_dep_wait();          // the tile table is produced by the routing plan kernel
    if (threadIdx.x == 0) {
      int4 e = make_int4(0, 0, 0, 0);
      if (tile_t < *p.num_group_tiles) e = p.group_tiles[tile_t];
      s_group[0] = e.x; s_group[1] = e.y; s_group[2] = e.z;
    }
    __syncthreads();
  }
  const int w_row0 = grouped ? s_group[0] * p.group_w_rows : 0;      // first weight row of this tile's group
  const int x_row0 = grouped ? s_group[1] : tile_t * BN;            // first token row of this tile
  const int x_rows = grouped ? s_group[2] : BN;                     // valid token rows in this tile
  const bool active = !grouped || x_rows > 0;
  const int tn_stride = (DUAL && p.pair) ? 256 : 128;      // output features covered per CTA

  if (warp == 0) {
    if (lane == 0) {
      // a weight byte is read once when one token tile covers the batch (decode): stream it past
      // L2; the small activation tile is re-read by every feature tile: keep it
      const uint64_t hint_w = p.t_tiles == 1 ? kEvictFirst : kEvictNormal;
      const uint64_t hint_x = p.n_tiles > 1 ? kEvictLast : kEvictNormal;
      // Weights never depend on the previous kernel: their first `stages` tiles are requested before the
      // grid dependency resolves, so the stream from HBM starts while the predecessor drains.
      const int kend = active ? kb1 : kb0;
      const int pre = min(stages, kend - kb0);
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(&full_bar[i], STAGE_BYTES);
        uint8_t* a = smem + i * STAGE_BYTES;
        tma_load_2d(a, &tmW, &full_bar[i], (kb0 + i) * 64, w_row0 + tile_n * tn_stride, hint_w);
        if (DUAL) tma_load_2d(a + A_BYTES, &tmW, &full_bar[i], (kb0 + i) * 64, w_row0 + p.dual_off + tile_n * tn_stride, hint_w);
      }
      grid_dep_wait();
      for (int i = 0; i < pre; ++i)
        tma_load_2d(smem + i * STAGE_BYTES + A_BYTES * NACC, &tmX, &full_bar[i], (kb0 + i) * 64, x_row0, hint_x);
      int it = pre;
      for (int kb = kb0 + pre; kb < kend; ++kb, ++it) {
        const int s = it % stages;
        const uint32_t ph = (it / stages) & 1;
        if (!mbar_wait(&empty_bar[s], ph ^ 1, p.status, XFT_ERR_WAIT_EMPTY)) break;
        mbar_expect_tx(&full_bar[s], STAGE_BYTES);
        uint8_t* a = smem + s * STAGE_BYTES;
        tma_load_2d(a, &tmW, &full_bar[s], kb * 64, w_row0 + tile_n * tn_stride, hint_w);
        if (DUAL) tma_load_2d(a + A_BYTES, &tmW, &full_bar[s], kb * 64, w_row0 + p.dual_off + tile_n * tn_stride, hint_w);
        tma_load_2d(a + A_BYTES * NACC, &tmX, &full_bar[s], kb * 64, x_row0, hint_x);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && active) {
      int it = 0;
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % stages;
        const uint32_t ph = (it / stages) & 1;
        if (!mbar_wait(&full_bar[s], ph, p.status, XFT_ERR_WAIT_FULL)) break;
        tcgen05_fence_after();
        const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
        const uint64_t adesc = umma_desc_k128(a_addr);
        const uint64_t bdesc = umma_desc_k128(a_addr + A_BYTES * NACC);
#pragma unroll
        for (int k = 0; k < 4; ++k) {       // 4 x (K = 16) per 64-wide k-block; +32 B = +2 in the address field
          umma_bf16(tmem_base, adesc + 2 * k, bdesc + 2 * k, IDESC, (it > 0 || k > 0) ? 1u : 0u);
          if (DUAL) {
            const uint64_t a1desc = umma_desc_k128(a_addr + A_BYTES);
            umma_bf16(tmem_base + BN, a1desc + 2 * k, bdesc + 2 * k, IDESC, (it > 0 || k > 0) ? 1u : 0u);
          }
        }
        tcgen05_commit(&empty_bar[s]);       // frees the stage when these MMAs have read it
      }
      tcgen05_commit(&tmem_full_bar);        // accumulator complete
    }
  } else {
    // ---------------- epilogue: 4 warps, one TMEM lane (= output feature) per thread -------------
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int n = tile_n * tn_stride + row;
    const bool n_ok = n < p.N;
    const int et = threadIdx.x - 64;                    // 0..127 among epilogue threads
    grid_dep_wait();            // scratch, residual and output belong to the stream order from here on
    if (p.ar.world > 1 && et == 0) s_epoch = *reinterpret_cast<volatile int*>(p.ar.epoch) + 1;
    const bool rms = BN <= 64 && p.rms_x != nullptr;
    if (BN <= 64 && rms) {
      // sum of squares of this CTA's K slice for each of its BN tokens: 128 / BN threads per token, 16-byte loads
      constexpr int TPT = 128 / (BN <= 64 ? BN : 64);
      const int tok = et / TPT, sub = et % TPT;
      const int t = x_row0 + tok;
      const int k_begin = kb0 * 64, k_end = min(kb1 * 64, p.K);
      float acc = 0.f;
      if (t < p.T) {
        const __nv_bfloat16* xr = p.rms_x + (size_t)t * p.rms_ldx;
#pragma unroll 4
        for (int k = k_begin + sub * 8; k < k_end; k += TPT * 8) {
          const uint4 v = __ldg(reinterpret_cast<const uint4*>(xr + k));
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h[i]);
            acc += f.x * f.x + f.y * f.y;
          }
        }
      }
#pragma unroll
      for (int o = TPT / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (sub == 0) s_ssq[tok] = acc;
      named_bar_sync(1, 128);
    }
    bool ok = active && mbar_wait(&tmem_full_bar, 0, p.status, XFT_ERR_WAIT_TMEM);
    tcgen05_fence_after();
    const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16);
    const int t0 = x_row0;
    bool last = true;
    if (p.splits > 1) {
      // publish this split's partial tile
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
      if (BN <= 64 && rms && et < BN) p.rms_ws[((size_t)tile_id * p.splits + split) * BN + et] = s_ssq[et];
      __threadfence();
      named_bar_sync(1, 128);
      if (et == 0) {
        int old = atomicAdd(&p.counters[tile_id], 1);
        s_last = (old == p.splits - 1);
        if (s_last) p.counters[tile_id] = 0;            // ready for the next launch
      }
      named_bar_sync(1, 128);
      last = s_last != 0;
      if (last) __threadfence();
      if (BN <= 64 && rms && last) {
        if (et < BN) {
          float a = 0.f;
          for (int sp = 0; sp < p.splits; ++sp) a += __ldcg(p.rms_ws + ((size_t)tile_id * p.splits + sp) * BN + et);
          s_ssq[et] = a;
        }
        named_bar_sync(1, 128);
      }
    }
    if (last) {
      const float bias_g = (p.bias && n_ok) ? p.bias[n] : 0.f;
      const bool pair = DUAL && p.pair;
      const int n2 = n + 128;                            // pair mode: the second tile's feature
      const bool n2_ok = pair && n2 < p.N;
      const float bias_u = (DUAL && p.bias && (pair ? n2_ok : n_ok)) ? p.bias[pair ? n2 : p.dual_off + n] : 0.f;
      const float rs = (p.row_scale && n_ok) ? p.row_scale[n] : 1.f;
      const float* ws_tile = p.ws + (size_t)tile_id * (size_t)(BN * NACC) * 128;
      const size_t ws_split_stride = (size_t)(p.n_tiles * p.t_tiles) * (size_t)(BN * NACC) * 128;
      // accumulator columns [c, c+16): from TMEM, or the sum of the split-K partials in split order
      auto load_acc = [&](int c, float (&g)[16], float (&u)[16]) {
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
      };
      const bool fused_ar = (!DUAL) && p.ar.world > 1;
      bool peers_ok = true;
      if (fused_ar) named_bar_sync(1, 128);          // s_epoch was written by epilogue thread 0
      const int epoch = fused_ar ? s_epoch : 0;
      const int par = epoch & 1;
      const bool two_shot = fused_ar && p.ar.two_shot;
      const int owner = two_shot ? tile_id % p.ar.world : p.ar.rank;
      const bool i_reduce = !two_shot || owner == p.ar.rank;
      if (fused_ar && ok) {
        // push this rank's partial tile, tagged with the epoch, into slot `rank` of every rank (its own included)
#pragma unroll 1
        for (int c = 0; c < BN; c += 16) {
          float g[16], u[16];
          load_acc(c, g, u);
          if (n_ok) {
#pragma unroll
            for (int j = 0; j < 16; j += 2) {
              const int t = t0 + c + j;           // even: one word carries tokens t and t + 1 of feature n
              if (t < p.T) {
                const unsigned long long w = ((unsigned long long)(unsigned)epoch << 32) | ll_pack2(g[j] * rs, g[j + 1] * rs);
                const long long off = par * p.ar.parity_stride + p.ar.rank * p.ar.slot_stride + (long long)(t >> 1) * p.N + n;
                if (two_shot) p.ar.recv[owner][off] = w;
                else for (int r = 0; r < p.ar.world; ++r) p.ar.recv[r][off] = w;
              }
            }
          }
        }
      }
      if (ok) {
        const unsigned long long* my_recv = fused_ar ? p.ar.recv[p.ar.rank] + par * p.ar.parity_stride : nullptr;
#pragma unroll 1
        for (int c = 0; c < BN && peers_ok; c += 16) {
          float g[16], u[16];
          if (!fused_ar) {
            load_acc(c, g, u);
          } else if (!i_reduce) {
            // two-shot, not the owner: the finished values arrive in this rank's result area
            const volatile unsigned long long* base = p.ar.result[p.ar.rank] + par * p.ar.slot_stride + n;
            unsigned long long w[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int t = t0 + c + 2 * j;
              w[j] = (n_ok && t < p.T) ? base[(long long)(t >> 1) * p.N] : ((unsigned long long)(unsigned)epoch << 32);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if ((int)(w[j] >> 32) != epoch) {
                const int t = t0 + c + 2 * j;
                const long long tstart = clock64();
                do {
                  if (clock64() - tstart > p.ar.wait_cycles) { peers_ok = false; break; }
                  w[j] = base[(long long)(t >> 1) * p.N];
                } while ((int)(w[j] >> 32) != epoch);
              }
              ll_unpack2((unsigned)w[j], g[2 * j], g[2 * j + 1]);
            }
            if (!peers_ok) { if (p.status) atomicCAS(p.status, 0, XFT_ERR_WAIT_PEER); break; }
          } else {
            // Sum the world slots in rank order.  All 16 words of a rank are requested before any is
            // examined, so the L2 round trips overlap; only words that have not arrived yet are re-polled.
#pragma unroll
            for (int j = 0; j < 16; ++j) g[j] = 0.f;
            for (int r = 0; r < p.ar.world && peers_ok; ++r) {
              const volatile unsigned long long* base = my_recv + r * p.ar.slot_stride + n;
              unsigned long long w[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const int t = t0 + c + 2 * j;
                w[j] = (n_ok && t < p.T) ? base[(long long)(t >> 1) * p.N] : ((unsigned long long)(unsigned)epoch << 32);
              }
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                if ((int)(w[j] >> 32) != epoch) {
                  const int t = t0 + c + 2 * j;
                  const long long tstart = clock64();
                  do {
                    if (clock64() - tstart > p.ar.wait_cycles) { peers_ok = false; break; }
                    w[j] = base[(long long)(t >> 1) * p.N];
                  } while ((int)(w[j] >> 32) != epoch);
                }
                float lo, hi;
                ll_unpack2((unsigned)w[j], lo, hi);
                g[2 * j] += lo;
                g[2 * j + 1] += hi;
              }
            }
            if (!peers_ok) { if (p.status) atomicCAS(p.status, 0, XFT_ERR_WAIT_PEER); break; }
          }
          if (n_ok) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int t = t0 + c + j;
              if (t < p.T && c + j < x_rows) {
                float x;
                if (fused_ar && !i_reduce) {
                  x = g[j];                     // finished by the owner
                } else {
                  const float ts = (BN <= 64 && rms) ? rsqrtf(s_ssq[(c + j) & 63] / (float)p.K + p.rms_eps) : 1.f;
                  x = fused_ar ? g[j] + bias_g : g[j] * (rs * ts) + bias_g;
                  x = apply_act(x, p.act);
                  if (DUAL && !pair) x *= (u[j] * (rs * ts) + bias_u);
                  if (p.col_scale) x *= p.col_scale[t];
                  if (p.residual) x += p.res_scale * __bfloat162float(p.residual[(size_t)t * p.ldr + n]);
                  g[j] = x;                     // kept for the two-shot broadcast below
                }
                if (p.out_fp32) reinterpret_cast<float*>(p.out)[(size_t)t * p.ldo + n] = x;
                else reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)t * p.ldo + n] = __float2bfloat16(x);
              }
            }
            if (two_shot && i_reduce) {
              // all-gather half of the two-shot scheme: the owner hands the finished values (two tokens per word)
              // to every other rank
#pragma unroll
              for (int j = 0; j < 16; j += 2) {
                const int t = t0 + c + j;
                if (t < p.T) {
                  const unsigned long long w = ((unsigned long long)(unsigned)epoch << 32) | ll_pack2(g[j], g[j + 1]);
                  const long long off = par * p.ar.slot_stride + (long long)(t >> 1) * p.N + n;
                  for (int r = 0; r < p.ar.world; ++r)
                    if (r != p.ar.rank) p.ar.result[r][off] = w;
                }
              }
            }
          }
          if (n2_ok) {          // pair mode: second independent tile
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int t = t0 + c + j;
              if (t < p.T && c + j < x_rows) {
                float x = apply_act(u[j] + bias_u, p.act);
                if (p.col_scale) x *= p.col_scale[t];
                if (p.residual) x += p.res_scale * __bfloat162float(p.residual[(size_t)t * p.ldr + n2]);
                if (p.out_fp32) reinterpret_cast<float*>(p.out)[(size_t)t * p.ldo + n2] = x;
                else reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)t * p.ldo + n2] = __float2bfloat16(x);
              }
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
  if (p.ar.world > 1 && threadIdx.x == 0) {
    grid_dep_wait();
    // last CTA of the launch: the next launch uses the next epoch (and the other buffer parity)
    const int total = gridDim.x * gridDim.y;
    if (atomicAdd(p.ar.done, 1) == total - 1) {
      *reinterpret_cast<volatile int*>(p.ar.done) = 0;
      __threadfence();
      atomicAdd(p.ar.epoch, 1);
    }
  }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess) return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

struct MapKey {
  const void* ptr; uint64_t rows, cols, ld; uint32_t box_rows, esize;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows && esize == o.esize;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    h ^= k.rows * 0x9E3779B97F4A7C15ull + (h << 6);
    h ^= k.cols * 0xC2B2AE3D27D4EB4Full + (h >> 2);
    h ^= (k.ld << 20) ^ (uint64_t(k.box_rows) << 8) ^ k.esize;
    return h;
  }
};

// K-major matrix [rows, cols] with row stride `ld` elements; box = 128 bytes x box_rows, 128B swizzle.
int make_tensor_map(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                    uint32_t esize) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex mu;
  MapKey key{ptr, rows, cols, ld, box_rows, esize};
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return 0; }
  }
  EncodeTiledFn enc = get_encode();
  if (!enc) return -1;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || ((ld * esize) & 15)) return -2;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * esize};
  cuuint32_t box[2] = {128 / esize, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = esize == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = enc(out, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -3;
  std::lock_guard<std::mutex> g(mu);
  if (cache.size() > 65536) cache.clear();
  cache[key] = *out;
  return 0;
}

template <int BN, bool DUAL>
static int launch_gemm(const CUtensorMap& tmW, const CUtensorMap& tmX, GemmParams& p, cudaStream_t st) {
  constexpr int STAGE_BYTES = 128 * 64 * 2 * (DUAL ? 2 : 1) + BN * 64 * 2;
  // small token tiles: keep a CTA under half an SM's shared memory so two CTAs (and twice the
  // loads in flight) share an SM; large tiles take the whole SM
  int budget = (BN <= 64) ? 110 * 1024 : 220 * 1024;
  if (budget / STAGE_BYTES < 3) budget = 220 * 1024;      // a deep pipeline beats a second resident CTA
  int stages = budget / STAGE_BYTES;
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < 2) stages = 2;
  p.stages = stages;
  size_t smem = (size_t)stages * STAGE_BYTES + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_bf16_kernel<BN, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024) != cudaSuccess) return 3000 + (int)cudaGetLastError();
    attr_set = true;
  }
  dim3 grid(p.n_tiles * p.t_tiles, p.splits);
  cudaError_t e = launch_pdl(gemm_bf16_kernel<BN, DUAL>, grid, dim3(192), smem, st, tmW, tmX, p);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

int pick_bn(int T) {
  if (T <= 16) return 16;
  if (T <= 32) return 32;
  if (T <= 64) return 64;
  if (T <= 128) return 128;
  return 256;
}

// Split-K plan from a cost model (microseconds) whose constants were fitted to a sweep of every split factor on
// the decode shapes of 7B and 70B models at TP 1/2/4/8 (benchmarks/bench_gemm.py --sweep-splits):
//   t(s) = 4 + [s > 1] * 2 + s * partial-tile bytes / 25 GB/s + sum over waves of weight bytes / rate(CTAs in the wave)
//   rate(n) = smooth-min(n * bytes a CTA keeps in flight / 3 us,  min(6.3 TB/s, 90 GB/s * busy SMs))
// A CTA's pull rate follows from its pipeline depth (Little's law), so few CTAs cannot saturate HBM; a nearly
// empty tail wave is expensive and a nearly full one is not; the last-arriver reduction grows with the split
// count and the tile's token width.
void plan_splits(int tiles, int num_kb, int bn, int nacc, size_t ws_bytes, int max_tiles, int* splits,
                 int* kb_per_split) {
  const int stage_bytes = 128 * 64 * 2 * nacc + bn * 64 * 2;
  const double w_stage = 128.0 * 64 * 2 * nacc;   // the token tile comes from L2
  const bool two_per_sm = bn <= 64 && (110 * 1024) / stage_bytes >= 3;
  const int slots = two_per_sm ? 296 : 148;
  int best = 1;
  if (tiles < slots && tiles <= max_tiles && ws_bytes > 0) {
    const size_t per_split = (size_t)tiles * bn * nacc * 128 * sizeof(float);
    int smax = num_kb / 2 > 0 ? num_kb / 2 : 1;
    if (smax > 64) smax = 64;
    int stages = (two_per_sm ? 110 * 1024 : 220 * 1024) / stage_bytes;
    if (stages > kMaxStages) stages = kMaxStages;
    const double r_cta = (double)stages * stage_bytes / 3.0;      // bytes per microsecond
    auto wave = [&](long long n, double kb_avg) {
      const double cap = fmin(6.3e6, (double)(n < 148 ? n : 148) * 9.0e4);
      const double nr = (double)n * r_cta;
      const double rate = pow(pow(cap, -8.0) + pow(nr, -8.0), -1.0 / 8.0);
      return (double)n * kb_avg * w_stage / rate;
    };
    double best_t = -1.0;
    for (int s = 1; s <= smax; ++s) {
      if (s > 1 && per_split * s > ws_bytes) break;
      const int per = (num_kb + s - 1) / s;
      const int real = (num_kb + per - 1) / per;
      const long long ctas = (long long)tiles * real;
      const double kb_avg = (double)num_kb / real;
      const long long full = ctas / slots, tail = ctas % slots;
      double t = 4.0 + (double)full * wave(slots, kb_avg) + (tail ? wave(tail, kb_avg) : 0.0);
      if (real > 1) t += 2.0 + (double)real * bn * nacc * 512.0 / 2.5e4;
      if (best_t < 0 || t < best_t) { best_t = t; best = real; }
    }
  }
  const int per = (num_kb + best - 1) / best;
  *splits = (num_kb + per - 1) / per;
  *kb_per_split = per;
}

}  // namespace xft

using namespace xft;

// Y[T,N] = epi(X[T,K] W[N,K]^T).  gated != 0: W holds gate rows [0,N) and up rows [dual_off, dual_off+N),
// Y = act(gate)*up.  ws/counters: split-K scratch (ws_bytes, n_counters ints, zero-initialised once).
static int gemm_bf16_impl(const void* X, int ldx, const void* W, int w_rows, int ldw, void* Y, int ldo, int out_fp32,
                          int T, int N, int K, int gated, int dual_off, const float* bias, const void* residual,
                          int ldr, float res_scale, int act, const float* row_scale, float* ws, size_t ws_bytes,
                          int* counters, int n_counters, int* status, int force_splits, const CommParams* ar,
                          cudaStream_t st, const float* rms_eps = nullptr) {
  if (T <= 0 || N <= 0 || K <= 0) return 0;
  GemmParams p{};
  if (ar) p.ar = *ar;
  p.N = N; p.T = T; p.K = K; p.dual_off = dual_off; p.out = Y; p.ldo = ldo; p.out_fp32 = out_fp32;
  p.bias = bias; p.residual = reinterpret_cast<const __nv_bfloat16*>(residual); p.ldr = ldr; p.res_scale = res_scale;
  p.act = act; p.ws = ws; p.counters = counters; p.status = status; p.row_scale = row_scale;
  const int bn = pick_bn(T);
  p.n_tiles = (N + 127) / 128;
  p.t_tiles = (T + bn - 1) / bn;
  p.num_kb = (K + 63) / 64;
  // compute-bound shapes: one CTA owns two adjacent feature tiles (pair mode) when that still fills the GPU
  constexpr size_t kRmsWsBytes = 1 << 20;        // tail of the split-K scratch kept for partial sums of squares
  if (rms_eps) {
    if (bn > 64 || ar || (K & 7) || (ldx & 7)) return -7;
    ws_bytes = (ws && ws_bytes > kRmsWsBytes) ? ws_bytes - kRmsWsBytes : 0;
  }
  if (!gated && !ar && !row_scale && bn == 256 && ((N + 255) / 256) * p.t_tiles >= 148) {
    p.pair = 1;
    p.dual_off = 128;
    p.n_tiles = (N + 255) / 256;
  }
  const int tiles = p.n_tiles * p.t_tiles;
  plan_splits(tiles, p.num_kb, bn, gated ? 2 : 1, ws ? ws_bytes : 0, counters ? n_counters : 0, &p.splits, &p.kb_per_split);
  if (force_splits > 0 && ws && counters && tiles <= n_counters) {
    int s = force_splits < p.num_kb ? force_splits : p.num_kb;
    size_t need = (size_t)tiles * bn * (gated ? 2 : 1) * 128 * sizeof(float) * s;
    if (need <= ws_bytes) {
      p.kb_per_split = (p.num_kb + s - 1) / s;
      p.splits = (p.num_kb + p.kb_per_split - 1) / p.kb_per_split;
    }
  }
  if (rms_eps) {
    if (p.splits > 1 && (size_t)tiles * p.splits * bn * sizeof(float) > kRmsWsBytes) { p.splits = 1; p.kb_per_split = p.num_kb; }
    p.rms_x = reinterpret_cast<const __nv_bfloat16*>(X);
    p.rms_ldx = ldx;
    p.rms_eps = *rms_eps;
    p.rms_ws = ws ? reinterpret_cast<float*>(reinterpret_cast<char*>(ws) + ws_bytes) : nullptr;
  }
  CUtensorMap tmW, tmX;
  int r = make_tensor_map(&tmW, W, (uint64_t)w_rows, (uint64_t)K, (uint64_t)ldw, 128, 2);
  if (r) return 1000 - r;
  r = make_tensor_map(&tmX, X, (uint64_t)T, (uint64_t)K, (uint64_t)ldx, (uint32_t)bn, 2);
  if (r) return 2000 - r;
#define XFT_LAUNCH(BN_)                                                        \
  case BN_:                                                                    \
    return (gated || p.pair) ? launch_gemm<BN_, true>(tmW, tmX, p, st) : launch_gemm<BN_, false>(tmW, tmX, p, st);
  switch (bn) {
    XFT_LAUNCH(16)
    XFT_LAUNCH(32)
    XFT_LAUNCH(64)
    XFT_LAUNCH(128)
    XFT_LAUNCH(256)
  }
#undef XFT_LAUNCH
  return -1;
}

extern "C" void xft_set_pdl(int on) { xft::g_xft_pdl = on ? 1 : 0; }

// RMSNorm fused into the GEMM: X is the un-normalised hidden state, W carries the norm's gain folded into its
// columns, and the kernel scales each token's accumulator by rsqrt(mean(x^2) + eps).  T <= 64 only (returns -7
// otherwise).  Replaces the reference's separate norm kernel in front of the QKV and gate/up products
// (src/layers/attention.h: norm.forward + qkv gemm; src/layers/mlp_llama.h).
extern "C" int xft_gemm_bf16_rms(const void* X, int ldx, const void* W, int w_rows, int ldw, void* Y, int ldo, int out_fp32,
                                 int T, int N, int K, int gated, int dual_off, const float* bias, int act, float eps,
                                 float* ws, size_t ws_bytes, int* counters, int n_counters, int* status,
                                 cudaStream_t st) {
  return gemm_bf16_impl(X, ldx, W, w_rows, ldw, Y, ldo, out_fp32, T, N, K, gated, dual_off, bias, nullptr, 0, 1.0f, act,
                        nullptr, ws, ws_bytes, counters, n_counters, status, 0, nullptr, st, &eps);
}

// The split-K planner on its own (host arithmetic only), for tests and tuning.
extern "C" void xft_plan_splits(int tiles, int num_kb, int bn, int nacc, size_t ws_bytes, int max_tiles, int* splits,
                                int* kb_per_split) {
  xft::plan_splits(tiles, num_kb, bn, nacc, ws_bytes, max_tiles, splits, kb_per_split);
}

extern "C" int xft_gemm_bf16(const void* X, int ldx, const void* W, int w_rows, int ldw, void* Y, int ldo, int out_fp32,
                             int T, int N, int K, int gated, int dual_off, const float* bias, const void* residual,
                             int ldr, float res_scale, int act, const float* row_scale, float* ws, size_t ws_bytes,
                             int* counters, int n_counters, int* status, int force_splits, cudaStream_t st) {
  return gemm_bf16_impl(X, ldx, W, w_rows, ldw, Y, ldo, out_fp32, T, N, K, gated, dual_off, bias, residual, ldr, res_scale,
                        act, row_scale, ws, ws_bytes, counters, n_counters, status, force_splits, nullptr, st);
}

// Grouped GEMM over token rows sorted by group (MoE experts): W is [groups * group_w_rows, K]; token tile i of
// size `bn` (16..128, chosen by the caller and used to build the table) is group_tiles[i] = {group, row0, rows, 0}.
// gated != 0: each group's rows are gate [0,N) then up [dual_off, dual_off+N).  col_scale: per-row factor.
extern "C" int xft_gemm_bf16_grouped(const void* X, int ldx, int x_rows, const void* W, int w_rows, int ldw, void* Y,
                                     int ldo, int out_fp32, int N, int K, int gated, int dual_off, int group_w_rows,
                                     const void* group_tiles, const int* num_group_tiles, int max_tiles, int bn,
                                     const float* col_scale, int act, int* status, cudaStream_t st) {
  if (x_rows <= 0 || N <= 0 || K <= 0 || max_tiles <= 0) return 0;
  GemmParams p{};
  p.N = N; p.T = x_rows; p.K = K; p.dual_off = dual_off; p.out = Y; p.ldo = ldo; p.out_fp32 = out_fp32;
  p.res_scale = 1.f; p.act = act; p.status = status;
  p.group_tiles = reinterpret_cast<const int4*>(group_tiles); p.num_group_tiles = num_group_tiles;
  p.group_w_rows = group_w_rows; p.col_scale = col_scale;
  p.n_tiles = (N + 127) / 128;
  p.t_tiles = max_tiles;
  p.num_kb = (K + 63) / 64;
  p.splits = 1; p.kb_per_split = p.num_kb;
  CUtensorMap tmW, tmX;
  int r = make_tensor_map(&tmW, W, (uint64_t)w_rows, (uint64_t)K, (uint64_t)ldw, 128, 2);
  if (r) return 1000 - r;
  r = make_tensor_map(&tmX, X, (uint64_t)x_rows, (uint64_t)K, (uint64_t)ldx, (uint32_t)bn, 2);
  if (r) return 2000 - r;
#define XFT_LAUNCH(BN_)                                                        \
  case BN_:                                                                    \
    return gated ? launch_gemm<BN_, true>(tmW, tmX, p, st) : launch_gemm<BN_, false>(tmW, tmX, p, st);
  switch (bn) {
    XFT_LAUNCH(16)
    XFT_LAUNCH(32)
    XFT_LAUNCH(64)
    XFT_LAUNCH(128)
  }
#undef XFT_LAUNCH
  return -1;
}

// Row-parallel GEMM fused with the tensor-parallel sum: Y = act(sum_r X_r W_r^T + bias) + res_scale*residual
// on every rank.  `comm` describes the peer-mapped receive/flag areas (see CommParams); requires
// T <= t_cap tokens and at most max_tiles output tiles (the capacity of the areas).
extern "C" int xft_gemm_bf16_ar(const void* X, int ldx, const void* W, int ldw, void* Y, int ldo, int out_fp32, int T,
                                int N, int K, const float* bias, const void* residual, int ldr, float res_scale, int act,
                                float* ws, size_t ws_bytes, int* counters, int n_counters, int* status,
                                const CommParams* comm, int t_cap, int max_tiles, cudaStream_t st) {
  if (!comm || comm->world < 2 || comm->world > 8) return -10;
  const int bn = pick_bn(T);
  const int tiles = ((N + 127) / 128) * ((T + bn - 1) / bn);
  if (T > t_cap || tiles > max_tiles || (long long)T * N > comm->slot_stride) return -11;
  return gemm_bf16_impl(X, ldx, W, N, ldw, Y, ldo, out_fp32, T, N, K, 0, 0, bias, residual, ldr, res_scale, act, nullptr,
                        ws, ws_bytes, counters, n_counters, status, 0, comm, st);
}

// ------------------------------------------------------------------------------------------
// Allocation-free entry point (declared in gemm_noalloc.h; no counterpart in the reference).
//
// Some hosts of this library may not allocate device memory at all once they are running: code
// inside a CUDA-graph capture or a latency-critical serving loop where cudaMalloc would synchronise
// the device, plug-ins living in a process whose memory pool is owned by someone else (an inference
// server that has already reserved the whole GPU), and callers that only have raw device pointers
// and no allocator to hand.  For them the split-K scratch of the GEMM above — partial tiles, tile
// counters and the status word — lives in one file-scope device array of fixed size.
//
// The array is part of the library image: every GPU that loads the library keeps
// XFT_NOALLOC_SCRATCH_BYTES (8 MiB + 8 KiB) resident until the process exits.
static __device__ __align__(256) unsigned char g_noalloc_scratch[XFT_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr size_t kNoallocPartialBytes = 8u << 20;    // split-K partial tiles
constexpr int kNoallocCounters = 1024;               // one int per output tile (first 4 KiB)
constexpr int kNoallocMaxTokens = 256;
constexpr int kNoallocMaxDevices = 64;
constexpr size_t kNoallocHeadBytes = 8192;           // counters [0, 4096), status word at 4096
// the limits published in gemm_noalloc.h are the ones enforced here
static_assert(kNoallocMaxTokens == XFT_NOALLOC_MAX_TOKENS, "token limit differs from gemm_noalloc.h");
static_assert(kNoallocCounters == XFT_NOALLOC_MAX_TILES, "tile limit differs from gemm_noalloc.h");
static_assert(kNoallocHeadBytes + kNoallocPartialBytes == XFT_NOALLOC_SCRATCH_BYTES, "scratch size differs from gemm_noalloc.h");
static_assert(kNoallocCounters * sizeof(int) <= 4096, "tile counters overlap the status word");
void* g_noalloc_ptr[kNoallocMaxDevices] = {};        // device address of the array, per device
}  // namespace

extern "C" const char* xft_gemm_bf16_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case -100: return "shape exceeds the allocation-free variant: need T <= 256 tokens and ceil(N/128)*ceil(T/tile) <= 1024 tiles";
    case -101: return "cudaGetSymbolAddress failed for the static scratch array";
    case -102: return "no current CUDA device / device index out of range";
    case -103: return "bad argument (null pointer, K not a multiple of 8, unaligned rows, or ldo / ldr smaller than N)";
    default: return "CUDA or tensor-map error (positive codes are cudaError_t values; 1000+/2000+ tensor-map encoding)";
  }
}

// Y[T,N] = act(X[T,K] · W[N,K]^T + bias) + res_scale * residual, bf16 in, bf16 or fp32 out.
// Same kernel and numerics as xft_gemm_bf16; the scratch is the static array above.
extern "C" int xft_gemm_bf16_noalloc(const void* X, int ldx, const void* W, int ldw, void* Y, int ldo, int out_fp32,
                                     int T, int N, int K, const float* bias, const void* residual, int ldr,
                                     float res_scale, int act, cudaStream_t st) {
  if (!X || !W || !Y || T <= 0 || N <= 0 || K <= 0 || (K % 8) || (ldx % 8) || (ldw % 8)) return -103;
  if (ldx < K || ldw < K || ldo < N || (residual && ldr < N)) return -103;
  if (T > kNoallocMaxTokens) return -100;
  const int bn = pick_bn(T);
  const int tiles = ((N + 127) / 128) * ((T + bn - 1) / bn);
  if (tiles > kNoallocCounters) return -100;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoallocMaxDevices) return -102;
  if (!g_noalloc_ptr[dev]) {
    // In host code the array's name is only a stand-in; the kernel needs its device address.
    // Looked up once per device, with that device current.
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || !p) return -101;
    g_noalloc_ptr[dev] = p;
  }
  unsigned char* base = static_cast<unsigned char*>(g_noalloc_ptr[dev]);
  int* counters = reinterpret_cast<int*>(base);                       // [0, 4096)
  int* status = reinterpret_cast<int*>(base + 4096);                  // [4096, 4352)
  float* ws = reinterpret_cast<float*>(base + kNoallocHeadBytes);     // partial tiles
  // the array keeps whatever the previous call left: counters and status must start at zero
  cudaError_t e = cudaMemsetAsync(base, 0, kNoallocHeadBytes, st);
  if (e != cudaSuccess) return (int)e;
  return xft_gemm_bf16(X, ldx, W, N, ldw, Y, ldo, out_fp32, T, N, K, /*gated=*/0, /*dual_off=*/0, bias, residual, ldr,
                       res_scale, act, /*row_scale=*/nullptr, ws, kNoallocPartialBytes, counters, kNoallocCounters,
                       status, /*force_splits=*/0, st);
}

// Status word of the last allocation-free call on the current device (0 = ok); synchronises the stream.
extern "C" int xft_gemm_bf16_noalloc_status(cudaStream_t st) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoallocMaxDevices || !g_noalloc_ptr[dev]) return -102;
  int v = 0;
  if (cudaMemcpyAsync(&v, static_cast<unsigned char*>(g_noalloc_ptr[dev]) + 4096, sizeof(int), cudaMemcpyDeviceToHost, st) !=
      cudaSuccess)
    return -102;
  if (cudaStreamSynchronize(st) != cudaSuccess) return -102;
  return v;
}

// Size and field offsets of CommParams, for the layout check of the Python mirror.
extern "C" int xft_comm_params_layout(long long* out, int n) {
  using xft::CommParams;
  const long long v[] = {sizeof(CommParams),           offsetof(CommParams, world),        offsetof(CommParams, rank),
                         offsetof(CommParams, recv),   offsetof(CommParams, epoch),        offsetof(CommParams, done),
                         offsetof(CommParams, slot_stride), offsetof(CommParams, parity_stride),
                         offsetof(CommParams, wait_cycles), offsetof(CommParams, two_shot), offsetof(CommParams, result)};
  const int m = (int)(sizeof(v) / sizeof(v[0]));
  for (int i = 0; i < m && i < n; ++i) out[i] = v[i];
  return m;
}
