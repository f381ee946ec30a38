// Decode-size bf16 GEMM for sm_100a (at most 64 tokens):  Y[T, N] = epilogue( X[T, K] · W[N, K]^T ), written as a
// balanced weight stream with the layer's neighbouring work fused into its two ends.
//
// The reference runs a decoder layer's linears as separate xDNN/oneDNN calls with a norm in front, a RoPE + cache
// copy behind the QKV product and an all-reduce behind o_proj / down_proj (src/layers/attention.h, mlp_llama.h,
// decoder_block.h:122-134, src/utils/matmul_helper.h:565-1705).  At decode sizes every one of these products is a pure
// weight stream, so what matters is (a) that all SMs pull the same number of bytes and (b) how few dependent kernels a
// layer needs.  This kernel therefore differs from the tile-per-CTA GEMM of gemm_sm100.cu in three ways:
//
//   * Work is cut into units of one 128-feature x 64-deep weight block.  The units, in (tile, k-block) order, are
//     dealt to one CTA per SM in equal contiguous runs, whatever the shape ("stream-K"): a CTA's run may end in the
//     middle of one output tile and begin in the middle of another.  Runs that cover a whole tile finish it from TMEM;
//     the others leave an fp32 partial in scratch and the CTA that arrives last on the tile's counter adds the
//     partials in CTA order (deterministic) and finishes the tile.  Nobody waits for another CTA.
//   * Two TMEM accumulators: the epilogue warps drain run i while the MMA warp already accumulates run i + 1.
//     A CTA uses about half an SM's shared memory, so the CTAs of the next kernel in the stream (programmatic
//     dependent launch) can become resident and request their first weight blocks while this one drains.
//   * Fused ends.  Front: RMSNorm folded in (the gain lives in W's columns, 1/rms is computed beside the main loop).
//     Back, one of: bias / activation / act(gate) * up / residual; split + RoPE + paged KV-cache append of a QKV
//     product (one 128-feature tile = one head); or the tensor-parallel all-reduce over peer memory.
//
// All-reduce form.  The CTA that finishes a tile pushes it, as 8-byte words {two bf16 values, epoch}, into the receive
// areas of the other ranks (one-shot: every rank; two-shot: the rank that owns that range of the output).  The sum
// itself is not done by that CTA: once a CTA has run out of GEMM work, its four epilogue warps take an equal share of
// the WHOLE output, poll the world's words for it (all loads of a 16-byte unit in flight at once, bounded), add them in
// rank order — bit-identical on every rank — apply bias / residual and store.  In the two-shot form the owners also
// hand the finished words to every other rank, and all CTAs copy out the ranges they do not own.  No fence, flag or
// barrier separates a store from the load that consumes it, and the reduction runs on every SM instead of in the
// few CTAs that happened to finish a tile.
#include "gemm_common.cuh"

#include <cstdlib>
#include <type_traits>

namespace xft {

constexpr int kSkMaxStages = 12;
constexpr int kSkInlineMax = 4;         // a tile shared by at most this many CTAs is finished by the one that arrives last
constexpr int kSkMaxCtas = 320;         // upper bound of the grid (one or two CTAs per SM)

// split + RoPE + cache append as the epilogue of a QKV product (head_dim 128, bf16 cache)
struct SkQkv {
  __nv_bfloat16* q_out;      // [T, hq, 128]; null = mode off
  int hq, hkv;
  const int* positions;      // [T]
  const float* table;        // [max_pos, rot] = cos(rot/2) ‖ sin(rot/2), or null (no rotation)
  int rot, style, rot_off, max_pos;   // style 0: pairs (i, i + rot/2); 1: pairs (2i, 2i + 1)
  const float* q_scale;      // optional per-token factor on q
  __nv_bfloat16* kc;         // [nb, hkv, bs, 128]
  __nv_bfloat16* vc;
  int bs;
  long long nslots;
  const int* slots;          // [T] flat slot = block * bs + offset
};

struct SkParams {
  int N, T, K;
  int dual_off;              // DUAL: W row of the first "up" feature
  void* out; int ldo; int out_fp32;
  const float* bias;
  const __nv_bfloat16* residual; int ldr; float res_scale;
  int act;
  int n_tiles, num_kb, stages;
  int units;                 // n_tiles * num_kb
  float* ws;                 // partial tiles [2 * gridDim.x][BN * NACC][128]
  float* rms_ws;             // partial sums of squares [2 * gridDim.x][BN]
  int* counters;             // one per output tile, zero between launches
  int* status;
  const float* row_scale;    // optional per-feature factor on the accumulator
  const __nv_bfloat16* rms_x; int rms_ldx; float rms_eps;     // folded RMSNorm (see gemm_sm100.cu)
  CommParams ar;             // ar.world > 1: all-reduce form
  SkQkv qkv;
  // cluster > 1: classic split-K, `cluster` consecutive CTAs (one thread-block cluster) share each tile and add their
  // parts through distributed shared memory instead of global scratch; the grid is n_tiles * cluster CTAs
  int cluster;
  // optional time line: 8 globaltimer stamps (ns) per CTA — 0 entry, 1 set-up done, 2 grid dependency resolved
  // (producer), 3 first weight block landed, 4 last MMA issued, 5 last accumulator ready, 6 epilogue done, 7 exit
  unsigned long long* trace;
};

__device__ __forceinline__ unsigned long long sk_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// thread-block cluster: rank of this CTA, the cluster-wide barrier in its two halves, shared memory of a peer CTA
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t dsmem_addr(uint32_t smem_addr, uint32_t cta_rank) {
  uint32_t a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(smem_addr), "r"(cta_rank));
  return a;
}
__device__ __forceinline__ float ld_dsmem(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}

#define SK_STAMP(ev) do { if (p.trace) p.trace[(size_t)blockIdx.x * 8 + (ev)] = sk_now(); } while (0)

// CTA that holds unit u when `units` units are dealt to `G` CTAs as [i * units / G, (i + 1) * units / G).  32-bit
// arithmetic on purpose (64-bit division is emulated on the GPU and these sit on the kernel's critical tail): the
// entry point refuses shapes with units * (G + 1) >= 2^31.
__host__ __device__ __forceinline__ int sk_cta_of(int u, int units, int G) {
  return (int)(((unsigned)(u + 1) * (unsigned)G + (unsigned)units - 1u) / (unsigned)units) - 1;
}
__host__ __device__ __forceinline__ int sk_first_unit(int cta, int units, int G) {
  return (int)((unsigned)cta * (unsigned)units / (unsigned)G);
}

// two 8-byte transport words with one 16-byte load
__device__ __forceinline__ void ld_volatile_2w(const unsigned long long* p, unsigned long long& a, unsigned long long& b) {
  asm volatile("ld.volatile.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
__device__ __forceinline__ void st_2w(unsigned long long* p, unsigned long long a, unsigned long long b) {
  asm volatile("st.global.v2.u64 [%0], {%1, %2};" ::"l"(p), "l"(a), "l"(b) : "memory");
}

template <int BN, bool DUAL>
__global__ void __launch_bounds__(192, 2) gemm_sk_kernel(const __grid_constant__ CUtensorMap tmW,
                                                         const __grid_constant__ CUtensorMap tmX, const SkParams p) {
  constexpr int A_BYTES = 128 * 64 * 2;
  constexpr int B_BYTES = BN * 64 * 2;
  constexpr int NACC = DUAL ? 2 : 1;
  constexpr int STAGE_BYTES = A_BYTES * NACC + B_BYTES;
  constexpr int ACC_COLS = BN * NACC;
  constexpr uint32_t TMEM_COLS = 2 * ACC_COLS < 32 ? 32 : 2 * ACC_COLS;
  constexpr uint32_t IDESC = umma_idesc(128, BN, 1, 1, 1);
  static_assert(BN == 16 || BN == 32 || BN == 64, "token tile of the decode kernel");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full_bar[kSkMaxStages], empty_bar[kSkMaxStages], tmem_full[2], tmem_empty[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_epoch, s_nsplit, s_last;
  __shared__ int s_split[kSkMaxCtas];                       // tiles shared by several CTAs, in tile order
  __shared__ float s_ssq[BN];
  constexpr int kHeadLd = 128 + 2;                        // bf16 elements per staged token row (odd word count)
  __shared__ __nv_bfloat16 s_head[DUAL ? 1 : BN * kHeadLd];   // QKV mode: one head of every token

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int stages = p.stages;
  const int G = gridDim.x, bid = blockIdx.x;
  const int u0 = sk_first_unit(bid, p.units, G), u1 = sk_first_unit(bid + 1, p.units, G);

  if (threadIdx.x == 0) {
    SK_STAMP(0);
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 4);                        // one arrival per epilogue warp
    }
    s_nsplit = 0;
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
  if (threadIdx.x == 0) SK_STAMP(1);

  // ---- epilogue threads (warps 2-5): one TMEM lane = one output feature of the tile per thread ------------------------
  const int q = warp & 3;
  const int row = q * 32 + lane;
  const int et = threadIdx.x - 64;                        // 0..127 among the epilogue threads
  const bool fused_ar = (!DUAL) && p.ar.world > 1;
  const bool qkv_mode = (!DUAL) && p.qkv.q_out != nullptr;
  const bool rms = p.rms_x != nullptr;
  const int E2 = ((p.T + 1) >> 1) * (p.N >> 1);           // 16-byte units of the all-reduce (N is even); 32-bit on purpose
  int epoch = 0, par = 0;                                 // set once the grid dependency has resolved
  bool alive = true;

  // ---- the ways a finished value leaves the kernel -------------------------------------------------------------
  // plain: feature n of token t;  g = accumulator (gate), u = up accumulator (DUAL), ssq = sum of squares of token t
  auto store_plain = [&](int n, int t, float g, float u, float ssq) {
    const float rs = p.row_scale ? p.row_scale[n] : 1.f;
    const float ts = rms ? rsqrtf(ssq / (float)p.K + p.rms_eps) : 1.f;
    float x = apply_act(g * (rs * ts) + (p.bias ? p.bias[n] : 0.f), p.act);
    if constexpr (DUAL) x *= (u * (rs * ts) + (p.bias ? p.bias[p.dual_off + n] : 0.f));
    if (p.residual) x += p.res_scale * __bfloat162float(p.residual[(size_t)t * p.ldr + n]);
    if (p.out_fp32) reinterpret_cast<float*>(p.out)[(size_t)t * p.ldo + n] = x;
    else reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)t * p.ldo + n] = __float2bfloat16(x);
  };
  // all-reduce: this rank's partial sums of tokens t, t + 1 (t even) of feature n go to the ranks that reduce them
  auto push_pair = [&](int n, int t, float g0, float g1) {
    const float rs = p.row_scale ? p.row_scale[n] : 1.f;
    const unsigned long long w = ((unsigned long long)(unsigned)epoch << 32) | ll_pack2(g0 * rs, g1 * rs);
    const int wi = (t >> 1) * p.N + n;
    const long long off = par * p.ar.parity_stride + p.ar.rank * p.ar.slot_stride + wi;
    if (p.ar.two_shot) {
      p.ar.recv[(int)((unsigned)(wi >> 1) * (unsigned)p.ar.world / (unsigned)E2)][off] = w;
    } else {
      for (int r = 0; r < p.ar.world; ++r) p.ar.recv[r][off] = w;
    }
  };
  // QKV: tokens [t0, t0 + nt) of head `tile` are staged in s_head rows [0, nt) (bias added, rounded to bf16 as a
  // separate product would store them); rotate and hand them to the attention kernel's inputs.  All 128 threads.
  auto qkv_rotate_store = [&](int tile, int t0, int nt) {
    if constexpr (!DUAL) {
      named_bar_sync(1, 128);
      const SkQkv& qp = p.qkv;
      const int h = tile;
      const bool is_q = h < qp.hq, is_k = !is_q && h < qp.hq + qp.hkv;
      const int d = row;
      const int half = qp.rot >> 1;
      const int rd = d - qp.rot_off;                     // index inside the rotary range
      const bool rotate = (is_q || is_k) && qp.table != nullptr && qp.rot > 0 && rd >= 0 && rd < qp.rot;
      int pi = 0, partner = d;
      float sign = 0.f;
      if (rotate) {
        if (qp.style == 0) { pi = rd < half ? rd : rd - half; partner = rd < half ? d + half : d - half; sign = rd < half ? -1.f : 1.f; }
        else { pi = rd >> 1; partner = d ^ 1; sign = (rd & 1) ? 1.f : -1.f; }
      }
      for (int i = 0; i < nt; ++i) {
        const int t = t0 + i;
        if (t >= p.T) break;
        float x = __bfloat162float(s_head[i * kHeadLd + d]);
        if (rotate) {
          int pos = qp.positions[t];
          if (pos < 0 || pos >= qp.max_pos) { if (p.status) atomicCAS(p.status, 0, XFT_ERR_BOUNDS); pos = 0; }
          const float* cs = qp.table + (size_t)pos * qp.rot;
          const float y = __bfloat162float(s_head[i * kHeadLd + partner]);
          x = x * cs[pi] + sign * y * cs[half + pi];
        }
        if (is_q) {
          if (qp.q_scale) x *= qp.q_scale[t];
          qp.q_out[((size_t)t * qp.hq + h) * 128 + d] = __float2bfloat16(x);
        } else {
          const int kh = is_k ? h - qp.hq : h - qp.hq - qp.hkv;
          const int slot = qp.slots[t];
          if (slot < 0 || slot >= qp.nslots) { if (p.status) atomicCAS(p.status, 0, XFT_ERR_BOUNDS); continue; }
          const int blk = slot / qp.bs, off = slot % qp.bs;
          __nv_bfloat16* dst = (is_k ? qp.kc : qp.vc) + ((size_t)(blk * qp.hkv + kh) * qp.bs + off) * 128;
          dst[d] = __float2bfloat16(x);
        }
      }
      named_bar_sync(1, 128);                            // s_head is reused
    }
  };
  auto stage_head = [&](int i, int n, float g, float ssq) {
    if constexpr (!DUAL) {
      const float rs = p.row_scale ? p.row_scale[n] : 1.f;
      const float ts = rms ? rsqrtf(ssq / (float)p.K + p.rms_eps) : 1.f;
      s_head[i * kHeadLd + row] = __float2bfloat16(g * (rs * ts) + (p.bias ? p.bias[n] : 0.f));
    }
  };


// ---- all-reduce: once its own tiles are pushed, every CTA reduces its share of the whole output (epilogue warps)
auto ar_reduce = [&]() {
  if (fused_ar && alive) {
    const int world = p.ar.world, rank = p.ar.rank;
    const unsigned long long* my_recv = p.ar.recv[rank] + par * p.ar.parity_stride;
    const int halfN = p.N >> 1;
    bool peers_ok = true;
    // finished values of unit i2 (features n, n + 1 of tokens t, t + 1) -> output, from the sum `f`
    auto store_unit = [&](int i2, const float (&f)[4]) {
      const int tp = i2 / halfN, n = (i2 % halfN) * 2;
      const int t = 2 * tp;
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        if (t + k < p.T) {
          if (p.out_fp32) {
            float* o = reinterpret_cast<float*>(p.out) + (size_t)(t + k) * p.ldo + n;
            o[0] = f[k]; o[1] = f[2 + k];
          } else {
            *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)(t + k) * p.ldo + n) =
                __floats2bfloat162_rn(f[k], f[2 + k]);
          }
        }
      }
    };
    // owned range of this rank (one-shot: everything), then this CTA's share of it
    int r0 = 0, r1 = E2;
    if (p.ar.two_shot) {
      r0 = (int)(((unsigned)rank * (unsigned)E2 + world - 1) / (unsigned)world);
      r1 = (int)(((unsigned)(rank + 1) * (unsigned)E2 + world - 1) / (unsigned)world);
    }
    const int a0 = r0 + (int)((unsigned)(r1 - r0) * (unsigned)bid / (unsigned)G);
    const int a1 = r0 + (int)((unsigned)(r1 - r0) * (unsigned)(bid + 1) / (unsigned)G);
    for (int i2 = a0 + et; i2 < a1 && peers_ok; i2 += 128) {
      unsigned long long w[8][2];
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (r < world) ld_volatile_2w(my_recv + r * p.ar.slot_stride + 2 * (long long)i2, w[r][0], w[r][1]);
      float f[4] = {0.f, 0.f, 0.f, 0.f};                   // (n, t), (n, t + 1), (n + 1, t), (n + 1, t + 1)
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        if (r < world) {
          if ((int)(w[r][0] >> 32) != epoch || (int)(w[r][1] >> 32) != epoch) {
            const long long tstart = clock64();
            do {
              if (clock64() - tstart > p.ar.wait_cycles) { peers_ok = false; break; }
              ld_volatile_2w(my_recv + r * p.ar.slot_stride + 2 * (long long)i2, w[r][0], w[r][1]);
            } while ((int)(w[r][0] >> 32) != epoch || (int)(w[r][1] >> 32) != epoch);
          }
          float lo, hi;
          ll_unpack2((unsigned)w[r][0], lo, hi); f[0] += lo; f[1] += hi;
          ll_unpack2((unsigned)w[r][1], lo, hi); f[2] += lo; f[3] += hi;
        }
      }
      if (!peers_ok) break;
      const int tp = i2 / halfN, n = (i2 % halfN) * 2;
      const int t = 2 * tp;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int nn = n + (k >> 1), tt = t + (k & 1);
        float x = f[k] + (p.bias ? p.bias[nn] : 0.f);
        x = apply_act(x, p.act);
        if (p.residual && tt < p.T) x += p.res_scale * __bfloat162float(p.residual[(size_t)tt * p.ldr + nn]);
        f[k] = x;
      }
      if (p.ar.two_shot) {
        // all-gather half: the owner hands the finished values to every other rank, rounded as they are stored
        const unsigned long long w0 = ((unsigned long long)(unsigned)epoch << 32) | ll_pack2(f[0], f[1]);
        const unsigned long long w1 = ((unsigned long long)(unsigned)epoch << 32) | ll_pack2(f[2], f[3]);
        for (int r = 0; r < world; ++r)
          if (r != rank) st_2w(p.ar.result[r] + par * p.ar.slot_stride + 2 * (long long)i2, w0, w1);
      }
      store_unit(i2, f);
    }
    if (p.ar.two_shot && peers_ok) {
      // copy out the ranges the other ranks own as their finished words arrive
      const unsigned long long* res = p.ar.result[rank] + par * p.ar.slot_stride;
      const int b0 = (int)((unsigned)E2 * (unsigned)bid / (unsigned)G), b1 = (int)((unsigned)E2 * (unsigned)(bid + 1) / (unsigned)G);
      for (int i2 = b0 + et; i2 < b1 && peers_ok; i2 += 128) {
        if (i2 >= r0 && i2 < r1) continue;
        unsigned long long w0, w1;
        ld_volatile_2w(res + 2 * (long long)i2, w0, w1);
        if ((int)(w0 >> 32) != epoch || (int)(w1 >> 32) != epoch) {
          const long long tstart = clock64();
          do {
            if (clock64() - tstart > p.ar.wait_cycles) { peers_ok = false; break; }
            ld_volatile_2w(res + 2 * (long long)i2, w0, w1);
          } while ((int)(w0 >> 32) != epoch || (int)(w1 >> 32) != epoch);
        }
        if (!peers_ok) break;
        float f[4];
        ll_unpack2((unsigned)w0, f[0], f[1]);
        ll_unpack2((unsigned)w1, f[2], f[3]);
        store_unit(i2, f);
      }
    }
    if (!peers_ok && p.status) atomicCAS(p.status, 0, XFT_ERR_WAIT_PEER);
  }
};

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      // a weight byte is read once: stream it past L2; the token tile is re-read by every CTA: keep it
      const uint64_t hint_w = kEvictFirst, hint_x = kEvictLast;
      const int n_units = u1 - u0;
      const int pre = min(stages, n_units);
      int tile = u0 / p.num_kb, kb = u0 % p.num_kb;
      const int tile0 = tile, kb0 = kb;
      // weights never depend on the previous kernel: the first blocks are requested before the grid dependency
      // resolves, so the stream from HBM starts while the predecessor drains
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(&full_bar[i], STAGE_BYTES);
        uint8_t* a = smem + i * STAGE_BYTES;
        tma_load_2d(a, &tmW, &full_bar[i], kb * 64, tile * 128, hint_w);
        if (DUAL) tma_load_2d(a + A_BYTES, &tmW, &full_bar[i], kb * 64, p.dual_off + tile * 128, hint_w);
        if (++kb == p.num_kb) { kb = 0; ++tile; }
      }
      grid_dep_wait();
      SK_STAMP(2);
      {
        int kb2 = kb0, tile2 = tile0;
        for (int i = 0; i < pre; ++i) {
          tma_load_2d(smem + i * STAGE_BYTES + A_BYTES * NACC, &tmX, &full_bar[i], kb2 * 64, 0, hint_x);
          if (++kb2 == p.num_kb) { kb2 = 0; ++tile2; }
        }
      }
      for (int it = pre; it < n_units; ++it) {
        const int s = it % stages;
        const uint32_t ph = (it / stages) & 1;
        if (!mbar_wait(&empty_bar[s], ph ^ 1, p.status, XFT_ERR_WAIT_EMPTY)) break;
        mbar_expect_tx(&full_bar[s], STAGE_BYTES);
        uint8_t* a = smem + s * STAGE_BYTES;
        tma_load_2d(a, &tmW, &full_bar[s], kb * 64, tile * 128, hint_w);
        if (DUAL) tma_load_2d(a + A_BYTES, &tmW, &full_bar[s], kb * 64, p.dual_off + tile * 128, hint_w);
        tma_load_2d(a + A_BYTES * NACC, &tmX, &full_bar[s], kb * 64, 0, hint_x);
        if (++kb == p.num_kb) { kb = 0; ++tile; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int it = 0, seg = 0;
      bool ok = true;
      for (int u = u0; u < u1 && ok; ++seg) {
        const int kb_begin = u % p.num_kb;
        const int kb_end = min(p.num_kb, kb_begin + (u1 - u));
        const int a = seg & 1;
        const uint32_t aph = (seg >> 1) & 1;
        if (!mbar_wait(&tmem_empty[a], aph ^ 1, p.status, XFT_ERR_WAIT_TMEM)) break;
        tcgen05_fence_after();
        const uint32_t acc = tmem_base + (uint32_t)(a * ACC_COLS);
        for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
          const int s = it % stages;
          const uint32_t ph = (it / stages) & 1;
          if (!mbar_wait(&full_bar[s], ph, p.status, XFT_ERR_WAIT_FULL)) { ok = false; break; }
          if (it == 0) SK_STAMP(3);
          tcgen05_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
          const uint64_t adesc = umma_desc_k128(a_addr);
          const uint64_t bdesc = umma_desc_k128(a_addr + A_BYTES * NACC);
#pragma unroll
          for (int k = 0; k < 4; ++k) {          // 4 x (K = 16) per 64-wide k-block; +32 B = +2 in the address field
            umma_bf16(acc, adesc + 2 * k, bdesc + 2 * k, IDESC, (kb > kb_begin || k > 0) ? 1u : 0u);
            if (DUAL) {
              const uint64_t a1desc = umma_desc_k128(a_addr + A_BYTES);
              umma_bf16(acc + BN, a1desc + 2 * k, bdesc + 2 * k, IDESC, (kb > kb_begin || k > 0) ? 1u : 0u);
            }
          }
          tcgen05_commit(&empty_bar[s]);
        }
        if (ok) tcgen05_commit(&tmem_full[a]);
        u += kb_end - kb_begin;
      }
      SK_STAMP(4);
    }
  } else {
    // ------------------------------------------------------------------ epilogue: 4 warps, one TMEM lane per thread
    // Tiles that more than kSkInlineMax CTAs work on, in tile order (phase 2 below): tile t is split when a CTA boundary
    // lies strictly inside it; the CTA after the first such boundary names it.  Every CTA builds the same list.
    if (warp == 2 && p.cluster <= 1) {
      int n = 0;
      for (int c0 = 1; c0 < G; c0 += 32) {
        const int c = c0 + lane;
        bool named = false;
        int t = 0;
        if (c < G) {
          const int b = sk_first_unit(c, p.units, G);
          t = b / p.num_kb;
          named = (b % p.num_kb) != 0 && sk_cta_of(t * p.num_kb, p.units, G) == c - 1 &&
                  sk_cta_of((t + 1) * p.num_kb - 1, p.units, G) - (c - 1) + 1 > kSkInlineMax;
        }
        const unsigned m = __ballot_sync(0xffffffffu, named);
        if (named) s_split[n + __popc(m & ((1u << lane) - 1u))] = t;
        n += __popc(m);
      }
      if (lane == 0) s_nsplit = n;
    }
    grid_dep_wait();              // scratch, residual, tokens and outputs belong to the stream order from here on
    if (fused_ar && et == 0) s_epoch = *reinterpret_cast<volatile int*>(p.ar.epoch) + 1;
    named_bar_sync(1, 128);
    const int nsplit = s_nsplit;
    epoch = fused_ar ? s_epoch : 0;
    par = epoch & 1;
    bool ssq_full = false;                                  // s_ssq holds the sums over the whole K

    // ---- phase 1: the runs of this CTA.  Whole tiles are finished from TMEM; parts of tiles are left in scratch ----
    int seg = 0;
    for (int u = u0; u < u1 && alive; ++seg) {
      const int tile = u / p.num_kb;
      const int kb_begin = u % p.num_kb;
      const int kb_end = min(p.num_kb, kb_begin + (u1 - u));
      u += kb_end - kb_begin;
      const bool complete = kb_begin == 0 && kb_end == p.num_kb;
      const int a = seg & 1;
      const uint32_t aph = (seg >> 1) & 1;
      const int n = tile * 128 + row;
      const bool n_ok = n < p.N;

      if (rms && !(complete && ssq_full)) {
        // sum of squares over this run's K range for each token: 128 / BN threads per token, 16-byte loads
        constexpr int TPT = 128 / BN;
        const int tok = et / TPT, sub = et % TPT;
        const int k_begin = kb_begin * 64, k_end = min(kb_end * 64, p.K);
        float acc = 0.f;
        if (tok < p.T) {
          const __nv_bfloat16* xr = p.rms_x + (size_t)tok * p.rms_ldx;
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
        named_bar_sync(1, 128);                             // the previous run's readers of s_ssq are done
        if (sub == 0) s_ssq[tok] = acc;
        named_bar_sync(1, 128);
        ssq_full = complete;
      }

      const bool got = mbar_wait(&tmem_full[a], aph, p.status, XFT_ERR_WAIT_TMEM);
      // one answer for all 128 threads, so nobody is left alone in front of a later barrier
      if (named_bar_or(1, 128, !got)) { alive = false; break; }
      if (et == 0 && u >= u1) SK_STAMP(5);
      tcgen05_fence_after();
      const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + (uint32_t)(a * ACC_COLS);

      int c_lo = bid, c_hi = bid, lo_slot = 0;
      if (p.cluster > 1) {
        // cluster mode: this CTA's only run is one K slice of a tile; its part goes to shared memory (the operand ring
        // is drained: every stage has been consumed by the MMAs this accumulator waited for), [column][128 rows] fp32
        float* part = reinterpret_cast<float*>(smem);
#pragma unroll 1
        for (int c = 0; c < ACC_COLS; c += 16) {
          uint32_t v[16];
          tmem_ld16(taddr + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) part[(c + j) * 128 + row] = __uint_as_float(v[j]);
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[a]);
        continue;                                           // finished after the cluster barrier, below
      }
      if (!complete) {
        // leave this run's part of the tile (and of the sums of squares) in scratch
        const int slot = 2 * bid + (seg == 0 ? 0 : 1);
        float* wsp = p.ws + (size_t)slot * (ACC_COLS * 128);
#pragma unroll 1
        for (int c = 0; c < ACC_COLS; c += 16) {
          uint32_t v[16];
          tmem_ld16(taddr + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) wsp[(size_t)(c + j) * 128 + row] = __uint_as_float(v[j]);
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[a]);
        if (rms && et < BN) p.rms_ws[(size_t)slot * BN + et] = s_ssq[et];
        c_lo = sk_cta_of(tile * p.num_kb, p.units, G);
        c_hi = sk_cta_of((tile + 1) * p.num_kb - 1, p.units, G);
        if (c_hi - c_lo + 1 > kSkInlineMax) continue;       // many parts: phase 2 shares the additions
        // few parts: the CTA that arrives last on the tile's counter adds them right away (nobody waits)
        __threadfence();
        named_bar_sync(1, 128);
        if (et == 0) {
          const int old = atomicAdd(&p.counters[2 + tile], 1);
          s_last = (old == c_hi - c_lo);
          if (s_last) p.counters[2 + tile] = 0;             // ready for the next launch
        }
        named_bar_sync(1, 128);
        if (!s_last) continue;
        __threadfence();
        lo_slot = sk_first_unit(c_lo, p.units, G) == tile * p.num_kb ? 0 : 1;
        if (rms) {
          if (et < BN) {
            float acc = 0.f;
            for (int cc = c_lo; cc <= c_hi; ++cc)
              acc += __ldcg(p.rms_ws + (size_t)(2 * cc + (cc == c_lo ? lo_slot : 0)) * BN + et);
            s_ssq[et] = acc;
          }
          named_bar_sync(1, 128);
          ssq_full = false;
        }
      }

      // ---------------- finish the tile: accumulator columns [c, c + 16) from TMEM, or the sum of its few parts ------
#pragma unroll 1
      for (int c = 0; c < BN; c += 16) {
        float g[16], uu[DUAL ? 16 : 1];
        if (complete) {
          uint32_t v[16];
          tmem_ld16(taddr + c, v);
          if constexpr (DUAL) {
            uint32_t v2[16];
            tmem_ld16(taddr + BN + c, v2);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) uu[j] = __uint_as_float(v2[j]);
          } else {
            tmem_ld_wait();
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) g[j] = __uint_as_float(v[j]);
          if (c + 16 >= BN) {
            // the accumulator is in registers: hand the TMEM buffer back to the MMA warp before the stores
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[a]);
          }
        } else {
          // parts in CTA order (deterministic); all their loads are in flight together
          float pv[kSkInlineMax][16], pu[DUAL ? kSkInlineMax : 1][DUAL ? 16 : 1];
#pragma unroll
          for (int i = 0; i < kSkInlineMax; ++i) {
            const int cc = c_lo + i;
            const bool on = cc <= c_hi;
            const float* w = p.ws + (size_t)(2 * cc + (i == 0 ? lo_slot : 0)) * (ACC_COLS * 128) + row;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              pv[i][j] = on ? __ldcg(w + (size_t)(c + j) * 128) : 0.f;
              if constexpr (DUAL) pu[i][j] = on ? __ldcg(w + (size_t)(BN + c + j) * 128) : 0.f;
            }
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            g[j] = 0.f;
            if constexpr (DUAL) uu[j] = 0.f;
          }
#pragma unroll
          for (int i = 0; i < kSkInlineMax; ++i)
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              g[j] += pv[i][j];
              if constexpr (DUAL) uu[j] += pu[i][j];
            }
        }
        if (fused_ar) {
          if (n_ok) {
#pragma unroll
            for (int j = 0; j < 16; j += 2)
              if (c + j < p.T) push_pair(n, c + j, g[j], g[j + 1]);
          }
        } else if (qkv_mode) {
#pragma unroll
          for (int j = 0; j < 16; ++j) stage_head(c + j, n, g[j], rms ? s_ssq[(c + j) % BN] : 0.f);
        } else if (n_ok) {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (c + j < p.T) {
              float up = 0.f;
              if constexpr (DUAL) up = uu[j];
              store_plain(n, c + j, g[j], up, rms ? s_ssq[(c + j) % BN] : 0.f);
            }
        }
      }
      if (qkv_mode) qkv_rotate_store(tile, 0, BN);
    }

    // ---- phase 2: the split tiles.  Once every CTA has left its parts in scratch, ALL CTAs share the additions: an
    // item is one token (all-reduce form: one pair of tokens) of one split tile, 128 features = one per thread; the
    // parts of up to 16 (item, CTA) pairs are requested together, so a CTA's share costs one or two round trips to L2
    // instead of one per contributing CTA.  The wait below is the only place where a CTA waits for other CTAs of
    // its grid; the grid is at most one CTA per SM, so all of them are resident, and the wait is bounded anyway.
    if (nsplit > 0) {
      __threadfence();
      named_bar_sync(1, 128);
      bool ok = true;
      if (et == 0) {
        atomicAdd(&p.counters[0], 1);
        const long long t0 = clock64();
        while (*reinterpret_cast<volatile int*>(&p.counters[0]) < G) {
          if (clock64() - t0 > kWaitCycles) { ok = false; if (p.status) atomicCAS(p.status, 0, XFT_ERR_WAIT_GRID); break; }
        }
      }
      if (named_bar_or(1, 128, !ok)) alive = false;
      __threadfence();
      if (alive) {
        const int ipt = fused_ar ? (p.T + 1) >> 1 : p.T;             // items per split tile
        const int total = nsplit * ipt;
        const int i0 = (int)((unsigned)total * (unsigned)bid / (unsigned)G), i1 = (int)((unsigned)total * (unsigned)(bid + 1) / (unsigned)G);
        auto run = [&](auto cpi_tag) {
          constexpr int CPI = decltype(cpi_tag)::value;              // contributor slots per item in one batch
          constexpr int IPB = 16 / CPI;                              // items per batch
          for (int base = i0; base < i1; base += IPB) {
            float acc[IPB], acc2[IPB], ssq[IPB];
            int tl[IPB], tk[IPB], lo[IPB], hi[IPB], lo_slot[IPB];
#pragma unroll
            for (int ib = 0; ib < IPB; ++ib) {
              acc[ib] = acc2[ib] = ssq[ib] = 0.f;
              const int it = base + ib;
              tl[ib] = -1; tk[ib] = 0; lo[ib] = 0; hi[ib] = -1; lo_slot[ib] = 0;
              if (it < i1) {
                tl[ib] = s_split[it / ipt];
                tk[ib] = fused_ar ? 2 * (it % ipt) : it % ipt;
                lo[ib] = sk_cta_of(tl[ib] * p.num_kb, p.units, G);
                hi[ib] = sk_cta_of((tl[ib] + 1) * p.num_kb - 1, p.units, G);
                // a CTA's part of a tile sits in its slot 0 when the tile is the first of its run, else in slot 1: only
                // the first contributor can have begun before this tile
                lo_slot[ib] = sk_first_unit(lo[ib], p.units, G) == tl[ib] * p.num_kb ? 0 : 1;
              }
            }
            int most = 0;
#pragma unroll
            for (int ib = 0; ib < IPB; ++ib) most = max(most, hi[ib] - lo[ib] + 1);
            for (int ch = 0; ch < most; ch += CPI) {
              float v[16], v2[16], v3[16];
#pragma unroll
              for (int s = 0; s < 16; ++s) {
                const int ib = s / CPI, cc = lo[ib] + ch + (s % CPI);
                v[s] = v2[s] = v3[s] = 0.f;
                if (cc <= hi[ib]) {
                  const int sl = 2 * cc + (cc == lo[ib] ? lo_slot[ib] : 0);
                  const float* w = p.ws + (size_t)sl * (ACC_COLS * 128) + row;
                  v[s] = __ldcg(w + (size_t)tk[ib] * 128);
                  if constexpr (DUAL) v2[s] = __ldcg(w + (size_t)(BN + tk[ib]) * 128);
                  else if (fused_ar) v2[s] = __ldcg(w + (size_t)(tk[ib] + 1) * 128);
                  if (rms) v3[s] = __ldcg(p.rms_ws + (size_t)sl * BN + tk[ib]);
                }
              }
#pragma unroll
              for (int s = 0; s < 16; ++s) { acc[s / CPI] += v[s]; acc2[s / CPI] += v2[s]; ssq[s / CPI] += v3[s]; }
            }
#pragma unroll
            for (int ib = 0; ib < IPB; ++ib) {
              if (tl[ib] < 0) continue;                              // same answer in all 128 threads
              const int n = tl[ib] * 128 + row;
              if (fused_ar) {
                if (n < p.N) push_pair(n, tk[ib], acc[ib], acc2[ib]);
              } else if (qkv_mode) {
                stage_head(0, n, acc[ib], ssq[ib]);
                qkv_rotate_store(tl[ib], tk[ib], 1);
              } else if (n < p.N) {
                store_plain(n, tk[ib], acc[ib], acc2[ib], ssq[ib]);
              }
            }
          }
        };
        // contributors per split tile are about G / n_tiles (at least 2): pick the batch shape from that
        const int typical = (G + p.n_tiles - 1) / p.n_tiles + 1;
        if (typical <= 2) run(std::integral_constant<int, 2>{});
        else if (typical <= 4) run(std::integral_constant<int, 4>{});
        else if (typical <= 8) run(std::integral_constant<int, 8>{});
        else run(std::integral_constant<int, 16>{});
      }
      // the last CTA through here re-arms the two counters for the next launch
      named_bar_sync(1, 128);
      if (et == 0 && atomicAdd(&p.counters[1], 1) == G - 1) {
        p.counters[0] = 0;
        p.counters[1] = 0;
        __threadfence();
      }
    }

    if (p.cluster <= 1) ar_reduce();
  }
  if (p.cluster > 1) {
    // ---- cluster mode: the CTAs of a cluster hold the K slices of one tile.  After the barrier CTA r finishes the
    // tokens [r * BN / cluster, (r + 1) * BN / cluster): every thread adds its feature's parts from all CTAs' shared
    // memory in rank order (deterministic) — one round trip through distributed shared memory instead of global scratch,
    // a counter and a last arriver.  A CTA leaves only after the second barrier: nobody reads a CTA that has exited.
    const int cs = p.cluster;
    __syncwarp();
    cluster_arrive();
    cluster_wait();
    if (warp >= 2 && alive) {
      const int crank = (int)cluster_ctarank();
      const int tile = u0 / p.num_kb;
      const int n = tile * 128 + row;
      const int per = BN / cs;
      const uint32_t part0 = smem_u32(smem), ssq0 = smem_u32(s_ssq);
      // all parts of a chunk of tokens are requested before any is used: one round trip per chunk, not per token
      auto run = [&](auto cs_tag) {
        constexpr int CS = decltype(cs_tag)::value;
        constexpr int TPC = 16 / CS;                        // tokens per chunk
        uint32_t pb[CS], sb[CS];
#pragma unroll
        for (int j = 0; j < CS; ++j) { pb[j] = dsmem_addr(part0, (uint32_t)j); sb[j] = dsmem_addr(ssq0, (uint32_t)j); }
        for (int t0 = 0; t0 < per; t0 += TPC) {
          float v[16], v2[16], v3[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int t = crank * per + t0 + i / CS, j = i % CS;
            v[i] = v2[i] = v3[i] = 0.f;
            if (t0 + i / CS < per && t < p.T) {
              v[i] = ld_dsmem(pb[j] + (uint32_t)(t * 128 + row) * 4u);
              if constexpr (DUAL) v2[i] = ld_dsmem(pb[j] + (uint32_t)((BN + t) * 128 + row) * 4u);
              else if (fused_ar) v2[i] = ld_dsmem(pb[j] + (uint32_t)((t + 1) * 128 + row) * 4u);
              if (rms) v3[i] = ld_dsmem(sb[j] + (uint32_t)t * 4u);
            }
          }
#pragma unroll
          for (int k = 0; k < TPC; ++k) {
            const int t = crank * per + t0 + k;
            if (t0 + k >= per || t >= p.T) break;           // the same answer in all 128 threads
            if (fused_ar && (k & 1)) continue;              // pairs: the odd token went out with the even one
            float g = 0.f, g2 = 0.f, ssq = 0.f;
#pragma unroll
            for (int j = 0; j < CS; ++j) { g += v[k * CS + j]; g2 += v2[k * CS + j]; ssq += v3[k * CS + j]; }
            if (fused_ar) {
              if (n < p.N) push_pair(n, t, g, g2);
            } else if (qkv_mode) {
              stage_head(0, n, g, ssq);
              qkv_rotate_store(tile, t, 1);
            } else if (n < p.N) {
              store_plain(n, t, g, g2, ssq);
            }
          }
        }
      };
      if (cs == 2) run(std::integral_constant<int, 2>{});
      else if (cs == 4) run(std::integral_constant<int, 4>{});
      else run(std::integral_constant<int, 8>{});
    }
    __syncwarp();
    cluster_arrive();
    if (warp >= 2) ar_reduce();
    cluster_wait();
  }
  if (threadIdx.x == 64) SK_STAMP(6);
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0) SK_STAMP(7);
  if (p.ar.world > 1 && threadIdx.x == 0) {
    grid_dep_wait();
    // last CTA of the launch: the next launch uses the next epoch (and the other buffer parity)
    if (atomicAdd(p.ar.done, 1) == (int)gridDim.x - 1) {
      *reinterpret_cast<volatile int*>(p.ar.done) = 0;
      __threadfence();
      atomicAdd(p.ar.epoch, 1);
    }
  }
}

// pipeline depth and shared memory of one CTA: about half an SM when that still gives three stages
static void sk_smem_plan(int bn, int nacc, int* stages, size_t* smem) {
  const int stage_bytes = 128 * 64 * 2 * nacc + bn * 64 * 2;
  static const int env_kb = [] { const char* v = getenv("XFT_SK_SMEM_KB"); return v ? atoi(v) : 0; }();
  int budget = (env_kb > 0 ? env_kb : 106) * 1024;
  if (budget / stage_bytes < 3) budget = 200 * 1024;
  if (budget > 216 * 1024) budget = 216 * 1024;
  int s = budget / stage_bytes;
  if (s > kSkMaxStages) s = kSkMaxStages;
  if (s < 2) s = 2;
  *stages = s;
  *smem = (size_t)s * stage_bytes + 1024;
}

template <int BN, bool DUAL>
static int launch_sk(const CUtensorMap& tmW, const CUtensorMap& tmX, SkParams& p, int grid, cudaStream_t st) {
  size_t smem;
  sk_smem_plan(BN, DUAL ? 2 : 1, &p.stages, &smem);
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_sk_kernel<BN, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return 3000 + (int)cudaGetLastError();
    attr_set = true;
  }
  if (p.cluster <= 1) {
    cudaError_t e = launch_pdl(gemm_sk_kernel<BN, DUAL>, dim3(grid), dim3(192), smem, st, tmW, tmX, p);
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
  }
  // cluster mode: the CTAs that share a tile form one thread-block cluster (at most 8: the portable size)
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = p.cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_xft_pdl ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_sk_kernel<BN, DUAL>, tmW, tmX, p);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

static unsigned long long* g_sk_trace = nullptr;

static int sk_num_sms() {
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        sms <= 0)
      sms = 148;
  }
  return sms;
}

}  // namespace xft

using namespace xft;

// Cluster size of a launch (1 = balanced stream over one CTA per SM with parts in global scratch).  Classic split-K
// with `s` CTAs per tile, added up through distributed shared memory, has the cheaper tail, but only pays when
// n_tiles * s CTAs load the SMs evenly: it is taken when some s in {8, 4, 2} fills at least 80 % of the CTA slots of
// its waves.  s must divide the token tile (each CTA finishes bn / s tokens; pairs of tokens in the all-reduce form).
// XFT_SK_CLUSTER = 0 never, = s forces s where it is valid.
extern "C" int xft_gemm_sk_cluster(int T, int N, int K, int gated, int all_reduce) {
  static const int env = [] { const char* v = getenv("XFT_SK_CLUSTER"); return v ? atoi(v) : -1; }();
  if (env == 0) return 1;
  const int bn = pick_bn(T), nacc = gated ? 2 : 1;
  const int n_tiles = (N + 127) / 128, num_kb = (K + 63) / 64;
  const int sms = sk_num_sms();
  int stages;
  size_t smem;
  sk_smem_plan(bn, nacc, &stages, &smem);
  const int per_sm = (smem + 20 * 1024 <= 113 * 1024) ? 2 : 1;      // CTAs that fit an SM together
  int best = 1;
  double best_e = 0.0;
  for (int s = 8; s >= 2; s >>= 1) {
    if (s > num_kb / 2 || bn % s || (all_reduce && bn / s < 2)) continue;
    const long long g = (long long)n_tiles * s;
    if (g > (long long)sms * per_sm || g > kSkMaxCtas) continue;
    if (env > 0) { if (s == env) return s; continue; }
    // busiest SM holds ceil(g / sms) CTAs; the even share would be g / sms
    const double e = (double)g / ((double)sms * (double)((g + sms - 1) / sms));
    if (e > best_e + 1e-9) { best_e = e; best = s; }
  }
  // small products are latency-bound: there the cheap tail wins even when the SMs are loaded unevenly
  const double mbytes = (double)n_tiles * 128 * nacc * (double)K * 2.0 / 1e6;
  return (env <= 0 && best > 1 && (best_e >= 0.75 || mbytes < 32.0)) ? best : 1;
}

// Which kernel runs a decode-size product: 0 = the tile-per-CTA kernel of gemm_sm100.cu (many tiles: its CTAs of
// neighbouring launches overlap), 1 = the balanced stream of this file (few tiles, many CTAs per tile), s >= 2 = this
// file's cluster mode.  Rules fitted to a sweep of the Llama-2 7B / 70B decode shapes at TP 1..8 on B200.
extern "C" int xft_gemm_sk_choice(int T, int N, int K, int gated, int all_reduce) {
  const int s = xft_gemm_sk_cluster(T, N, K, gated, all_reduce);
  if (s > 1) return s;
  static const int force = [] { const char* v = getenv("XFT_GEMM_STREAMK"); return v ? atoi(v) : 1; }();
  if (force == 2) return 1;                               // XFT_GEMM_STREAMK=2: never the tile-per-CTA kernel
  return ((N + 127) / 128) * (gated ? 2 : 1) <= 32 ? 1 : 0;
}

// CTAs of a launch: one per SM, fewer when that would leave a CTA less than two weight blocks.  XFT_SK_CTAS overrides
// the upper bound (tuning).
extern "C" int xft_gemm_sk_grid(int N, int K) {
  static const int env_ctas = [] { const char* v = getenv("XFT_SK_CTAS"); return v ? atoi(v) : 0; }();
  const long long units = (long long)((N + 127) / 128) * ((K + 63) / 64);
  long long g = env_ctas > 0 ? env_ctas : sk_num_sms();
  if (g > units / 2) g = units / 2;
  if (g > kSkMaxCtas) g = kSkMaxCtas;
  if (g < 1) g = 1;
  return (int)g;
}

// Scratch a launch needs: bytes of partial tiles + sums of squares, and tile counters.
extern "C" void xft_gemm_sk_scratch(int T, int N, int K, int gated, size_t* ws_bytes, int* n_counters) {
  const int bn = pick_bn(T), nacc = gated ? 2 : 1;
  const int g = xft_gemm_sk_grid(N, K);
  *ws_bytes = (size_t)2 * g * bn * nacc * 128 * sizeof(float) + (size_t)2 * g * bn * sizeof(float);
  *n_counters = (N + 127) / 128 + 2;
}

// Y[T, N] = epi(X[T, K] W[N, K]^T) for T <= 64.  gated: W holds gate rows [0, N) and up rows [dual_off, dual_off + N),
// Y = act(gate) * up.  rms_eps != null: X is the un-normalised hidden state and W carries the norm's gain.
// comm != null: row-parallel product, summed over the ranks (see the file comment); qkv != null: the output goes
// through RoPE into q_out and the paged cache instead of Y (N = (hq + 2 hkv) * 128).
// Returns 0, a negative argument error (-21 shape, -22 scratch too small, -23 all-reduce capacity), or a CUDA error.
extern "C" int xft_gemm_sk(const void* X, int ldx, const void* W, int w_rows, int ldw, void* Y, int ldo, int out_fp32,
                           int T, int N, int K, int gated, int dual_off, const float* bias, const void* residual, int ldr,
                           float res_scale, int act, const float* row_scale, const float* rms_eps, float* ws,
                           size_t ws_bytes, int* counters, int n_counters, int* status, const CommParams* comm,
                           const SkQkv* qkv, cudaStream_t st) {
  if (T <= 0 || N <= 0 || K <= 0) return 0;
  if (T > 64 || (K & 7) || (ldx & 7) || (ldw & 7)) return -21;
  if (comm && (gated || rms_eps || qkv || (N & 1))) return -21;
  if (qkv && (gated || N != (qkv->hq + 2 * qkv->hkv) * 128 || act != 0 || residual || qkv->nslots >= (1ll << 31))) return -21;
  SkParams p{};
  p.N = N; p.T = T; p.K = K; p.dual_off = dual_off; p.out = Y; p.ldo = ldo; p.out_fp32 = out_fp32;
  p.bias = bias; p.residual = reinterpret_cast<const __nv_bfloat16*>(residual); p.ldr = ldr; p.res_scale = res_scale;
  p.act = act; p.row_scale = row_scale; p.counters = counters; p.status = status;
  const int bn = pick_bn(T), nacc = gated ? 2 : 1;
  p.n_tiles = (N + 127) / 128;
  p.num_kb = (K + 63) / 64;
  p.cluster = xft_gemm_sk_cluster(T, N, K, gated, comm != nullptr);
  const int grid = p.cluster > 1 ? p.n_tiles * p.cluster : xft_gemm_sk_grid(N, K);
  if ((long long)p.n_tiles * p.num_kb * (grid + 1) >= (1ll << 31) || (long long)p.n_tiles * 64 * (grid + 1) >= (1ll << 31)) return -21;
  p.units = p.n_tiles * p.num_kb;
  const size_t part_bytes = (size_t)2 * grid * bn * nacc * 128 * sizeof(float);
  const size_t rms_bytes = (size_t)2 * grid * bn * sizeof(float);
  if (!ws || !counters || ws_bytes < part_bytes + rms_bytes || n_counters < p.n_tiles + 2) return -22;
  p.ws = ws;
  p.rms_ws = reinterpret_cast<float*>(reinterpret_cast<char*>(ws) + part_bytes);
  if (rms_eps) {
    p.rms_x = reinterpret_cast<const __nv_bfloat16*>(X);
    p.rms_ldx = ldx;
    p.rms_eps = *rms_eps;
  }
  if (comm) {
    if (comm->world < 2 || comm->world > 8) return -23;
    if ((long long)((T + 1) / 2) * N > comm->slot_stride) return -23;
    if ((long long)((T + 1) / 2) * (N / 2) * (grid + 8) >= (1ll << 31)) return -23;
    p.ar = *comm;
  }
  if (qkv) p.qkv = *qkv;
  p.trace = g_sk_trace;
  CUtensorMap tmW, tmX;
  int r = make_tensor_map(&tmW, W, (uint64_t)w_rows, (uint64_t)K, (uint64_t)ldw, 128, 2);
  if (r) return 1000 - r;
  r = make_tensor_map(&tmX, X, (uint64_t)T, (uint64_t)K, (uint64_t)ldx, (uint32_t)bn, 2);
  if (r) return 2000 - r;
#define XFT_LAUNCH(BN_) \
  case BN_: return gated ? launch_sk<BN_, true>(tmW, tmX, p, grid, st) : launch_sk<BN_, false>(tmW, tmX, p, grid, st);
  switch (bn) {
    XFT_LAUNCH(16)
    XFT_LAUNCH(32)
    XFT_LAUNCH(64)
  }
#undef XFT_LAUNCH
  return -21;
}

// Time line of the following launches: `buf` holds 8 stamps (nanoseconds of the GPU's global timer) per CTA, see
// SkParams::trace; null switches it off.  A debugging aid: the stamps cost a predicated store each.
extern "C" void xft_gemm_sk_set_trace(unsigned long long* buf) { xft::g_sk_trace = buf; }

// The work decomposition on its own (host arithmetic only), for tests: CTA that holds unit u, first unit of a CTA.
extern "C" int xft_sk_cta_of(long long u, long long units, int G) { return xft::sk_cta_of((int)u, (int)units, G); }
extern "C" long long xft_sk_first_unit(int cta, long long units, int G) { return xft::sk_first_unit(cta, (int)units, G); }

// Size and field offsets of SkQkv, for the layout check of the Python mirror.
extern "C" int xft_sk_qkv_layout(long long* out, int n) {
  const long long v[] = {sizeof(SkQkv),           offsetof(SkQkv, q_out),   offsetof(SkQkv, hq),       offsetof(SkQkv, hkv),
                         offsetof(SkQkv, positions), offsetof(SkQkv, table), offsetof(SkQkv, rot),      offsetof(SkQkv, style),
                         offsetof(SkQkv, rot_off), offsetof(SkQkv, max_pos), offsetof(SkQkv, q_scale),  offsetof(SkQkv, kc),
                         offsetof(SkQkv, vc),      offsetof(SkQkv, bs),      offsetof(SkQkv, nslots),   offsetof(SkQkv, slots)};
  const int m = (int)(sizeof(v) / sizeof(v[0]));
  for (int i = 0; i < m && i < n; ++i) out[i] = v[i];
  return m;
}
