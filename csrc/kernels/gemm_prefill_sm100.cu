// Persistent prefill GEMM for sm_100a with the tensor-parallel reduction fused in:
//     Y[T, N] = act( sum over ranks ( X_r[T, K_r] · W_r[N, K_r]^T ) + bias ) + res_scale * residual        (bf16 in / out)
//
// The reference runs a row-parallel linear and then a separate collective (o_proj / down_proj followed by
// Messenger::reduceAdd, src/layers/decoder_block.h:122-134; DistLinear in src/layers/dist_linear.h).  At prefill sizes
// that collective moves T x N values per layer twice and leaves the tensor cores idle while it runs.  Here one kernel
// does both, tile by tile:
//
//   * One CTA per SM walks a list of 128-feature x BN-token output tiles.  Warp 0 streams operands with TMA into a
//     shared-memory ring, warp 1 issues tcgen05.mma into one of TWO TMEM accumulators, warps 2-5 drain the other one:
//     the epilogue of tile i (conversion, NVLink stores, waits on peers) overlaps the main loop of tile i + 1.
//   * Token blocks are owned round-robin by the ranks (block j belongs to rank j % world).  A rank that finishes a tile
//     of a block it does not own stores its bf16 partial straight into the owner's memory (reduce-scatter half) and
//     raises a flag there; the owner adds the partials of all ranks to its own fp32 accumulator in rank order, applies
//     bias / activation / residual and stores the finished tile into the output buffer of EVERY rank (all-gather half),
//     again followed by a flag.  The kernel ends on a rank when the finished tiles of all other owners have arrived,
//     so its output is complete in local memory and the next kernel needs no collective.
//   * Each rank visits the blocks it owns a few positions late (the host passes the visiting order), so the partials
//     of its peers are normally there when it gets to them and the waits cost nothing.
//
// Peer memory is touched with plain global stores only (no TMA, no multicast); the operands of the MMA always come
// from this GPU's own memory.  Ordering: data stores, __threadfence_system() by every storing thread, a CTA barrier,
// then one st.release.sys of the flag; the consumer polls with ld.acquire.sys.  Every wait is bounded and reports
// through the status word.  With world == 1 the same kernel is a plain persistent GEMM with a double-buffered
// accumulator.
#include "ptx.cuh"

#include <cstdlib>

namespace xft {

int make_tensor_map(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                    uint32_t esize);

struct BulkArParams {
  int world, rank;
  __nv_bfloat16* part[8];     // rank r's partial area as mapped here: [world source slots][part_stride]
  unsigned* flag_part[8];     // rank r's arrival flags: [owned tile][world]
  __nv_bfloat16* out[8];      // rank r's output buffer [T, ldo] (out[rank] is this rank's own)
  unsigned* flag_res[8];      // rank r's result flags: [tile]
  int* epoch;                 // local: completed launches
  int* done;                  // local: CTAs of the current launch that have finished their tiles
  long long part_stride;      // elements per source slot of the partial area
  long long wait_cycles;      // bound of every wait on a peer
};

struct PrefillParams {
  int N, T, K;
  __nv_bfloat16* out;
  int ldo;
  const float* bias;
  const __nv_bfloat16* residual;
  int ldr;
  float res_scale;
  int act;
  int n_tiles, t_tiles, num_kb, stages;
  int gn;                     // feature tiles per group: a group sweeps all token blocks before the next one starts
  int dual_off;               // gated form: W row of the first "up" feature (gate rows are [0, dual_off)); bias likewise
  const int* order;           // optional: i-th visited token block (a permutation of 0..t_tiles-1)
  int wide;                   // != 0: bf16 rows leave through shared memory as 256-byte runs (full 128-feature tiles)
  int* status;
  BulkArParams ar;
};

__device__ __forceinline__ float prefill_act(float x, int act) {
  switch (act) {
    case 1: return fmaxf(x, 0.f);
    case 2: return x / (1.f + __expf(-x));
    case 3: {
      const float c = 0.7978845608028654f;
      const float u = c * (x + 0.044715f * x * x * x);
      return 0.5f * x * (1.f + tanhf(u));
    }
    default: return x;
  }
}

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Bounded poll of a flag another GPU writes; false on time-out.
__device__ __forceinline__ bool wait_flag(const unsigned* p, unsigned want, long long limit) {
  if (ld_acquire_sys(p) == want) return true;
  const long long t0 = clock64();
  while (ld_acquire_sys(p) != want) {
    if (clock64() - t0 > limit) return false;
  }
  return true;
}

// work item -> (feature tile, visited block index)
__device__ __forceinline__ void decode_item(const PrefillParams& p, int item, int& nt, int& blk) {
  const int per_group = p.gn * p.t_tiles;
  const int g = item / per_group, r = item % per_group;
  const int gn = min(p.gn, p.n_tiles - g * p.gn);
  nt = g * p.gn + r % gn;
  const int bi = r / gn;
  blk = p.order ? p.order[bi] : bi;
}

// mbarrier wait that also gives up as soon as another role of this CTA has raised the abort flag
__device__ __forceinline__ bool mbar_wait_or_abort(uint64_t* bar, uint32_t parity, int* status, int code,
                                                   volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitCycles) {
      if (status) atomicCAS(status, 0, code);
      *abort_flag = 1;
      return false;
    }
  }
  return true;
}

constexpr int kPrefillMaxStages = 8;

// DUAL: gated form (column-parallel gate ‖ up projection, no reduction over ranks): two weight tiles, gate rows n and up
// rows dual_off + n, share one token tile and feed two accumulators; the epilogue stores act(gate) * up.  With BN = 128
// the four accumulators (2 x double buffer) fill the 512 TMEM columns and a stage moves the same bytes per FLOP as the
// plain 128 x 256 tile.
template <int BN, bool DUAL>
__global__ void __launch_bounds__(192, 1) gemm_prefill_kernel(const __grid_constant__ CUtensorMap tmW,
                                                              const __grid_constant__ CUtensorMap tmX,
                                                              const PrefillParams p) {
  constexpr int A_BYTES = 128 * 64 * 2;
  constexpr int B_BYTES = BN * 64 * 2;
  constexpr int NACC = DUAL ? 2 : 1;
  constexpr int STAGE_BYTES = A_BYTES * NACC + B_BYTES;
  constexpr uint32_t TMEM_COLS = 2 * BN * NACC;          // double-buffered accumulators of BN fp32 columns each
  constexpr uint32_t IDESC = umma_idesc(128, BN, 1, 1, 1);
  static_assert(BN == 128 || (BN == 256 && !DUAL), "token tile of the prefill kernel");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full_bar[kPrefillMaxStages], empty_bar[kPrefillMaxStages], tmem_full[2], tmem_empty[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_abort_mem, s_epoch, s_last;
  // wide stores: 16 token rows x 128 features of bf16, rows padded by 8 elements so that both the per-feature writes
  // and the 16-byte row reads spread over the banks
  constexpr int kStageLd = 128 + 8;
  __shared__ __align__(16) __nv_bfloat16 s_stage[16 * kStageLd];
  volatile int* s_abort = &s_abort_mem;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int stages = p.stages;
  const int total = p.n_tiles * p.t_tiles;
  const int world = p.ar.world, rank = p.ar.rank;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 4);          // one arrival per epilogue warp
    }
    s_abort_mem = 0;
    s_last = 0;
    s_epoch = world > 1 ? *reinterpret_cast<volatile int*>(p.ar.epoch) + 1 : 0;
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
  const unsigned epoch = (unsigned)s_epoch;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const uint64_t hint = kEvictNormal;          // both operands are re-read by other CTAs out of L2
      int it = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total && ok; item += gridDim.x) {
        int nt, blk;
        decode_item(p, item, nt, blk);
        for (int kb = 0; kb < p.num_kb; ++kb, ++it) {
          const int s = it % stages;
          const uint32_t ph = (it / stages) & 1;
          if (*s_abort || !mbar_wait_or_abort(&empty_bar[s], ph ^ 1, p.status, XFT_ERR_WAIT_EMPTY, s_abort)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&full_bar[s], STAGE_BYTES);
          uint8_t* a = smem + s * STAGE_BYTES;
          tma_load_2d(a, &tmW, &full_bar[s], kb * 64, nt * 128, hint);
          if (DUAL) tma_load_2d(a + A_BYTES, &tmW, &full_bar[s], kb * 64, p.dual_off + nt * 128, hint);
          tma_load_2d(a + A_BYTES * NACC, &tmX, &full_bar[s], kb * 64, blk * BN, hint);
        }
      }
      if (!ok) {
        // loads already issued still write into this CTA's shared memory: give them time to land before the CTA exits
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) {}
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int it = 0, lt = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total && ok; item += gridDim.x, ++lt) {
        const int a = lt & 1;
        const uint32_t aph = (lt >> 1) & 1;
        if (*s_abort || !mbar_wait_or_abort(&tmem_empty[a], aph ^ 1, p.status, XFT_ERR_WAIT_TMEM, s_abort)) break;
        tcgen05_fence_after();
        const uint32_t acc = tmem_base + (uint32_t)(a * BN * NACC);
        for (int kb = 0; kb < p.num_kb; ++kb, ++it) {
          const int s = it % stages;
          const uint32_t ph = (it / stages) & 1;
          if (!mbar_wait_or_abort(&full_bar[s], ph, p.status, XFT_ERR_WAIT_FULL, s_abort)) {
            ok = false;
            break;
          }
          tcgen05_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
          const uint64_t adesc = umma_desc_k128(a_addr);
          const uint64_t bdesc = umma_desc_k128(a_addr + A_BYTES * NACC);
#pragma unroll
          for (int k = 0; k < 4; ++k) {        // 4 x (K = 16) per 64-wide k-block; +32 B = +2 in the address field
            umma_bf16(acc, adesc + 2 * k, bdesc + 2 * k, IDESC, (kb > 0 || k > 0) ? 1u : 0u);
            if (DUAL) {
              const uint64_t a1desc = umma_desc_k128(a_addr + A_BYTES);
              umma_bf16(acc + BN, a1desc + 2 * k, bdesc + 2 * k, IDESC, (kb > 0 || k > 0) ? 1u : 0u);
            }
          }
          tcgen05_commit(&empty_bar[s]);
        }
        if (ok) tcgen05_commit(&tmem_full[a]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (4 warps, one TMEM lane per thread)
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int et = threadIdx.x - 64;
    int lt = 0;
    for (int item = blockIdx.x; item < total; item += gridDim.x, ++lt) {
      int nt, blk;
      decode_item(p, item, nt, blk);
      const int a = lt & 1;
      const uint32_t aph = (lt >> 1) & 1;
      mbar_wait_or_abort(&tmem_full[a], aph, p.status, XFT_ERR_WAIT_TMEM, s_abort);
      const int owner = world > 1 ? blk % world : 0;
      const bool owned = world <= 1 || owner == rank;
      const int own_idx = world > 1 ? blk / world : 0;          // index of this block among its owner's blocks
      if (world > 1 && owned && et < world && et != rank && !*s_abort) {
        // the partial of rank `et` for this tile must have landed in this rank's memory
        const unsigned* f = p.ar.flag_part[rank] + ((size_t)own_idx * p.n_tiles + nt) * world + et;
        if (!wait_flag(f, epoch, p.ar.wait_cycles)) {
          if (p.status) atomicCAS(p.status, 0, XFT_ERR_WAIT_PEER);
          *s_abort = 1;
        }
      }
      // one answer for all 128 epilogue threads: a flag read per thread could change between two reads (the other
      // roles raise it too) and leave part of the group in front of a barrier the rest never reaches
      if (named_bar_or(1, 128, *s_abort != 0)) break;
      tcgen05_fence_after();
      const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + (uint32_t)(a * BN * NACC);
      const int n = nt * 128 + row;
      const bool n_ok = n < p.N;
      const int t0 = blk * BN;
      const float bias = (p.bias && n_ok) ? p.bias[n] : 0.f;
      const float bias_u = (DUAL && p.bias && n_ok) ? p.bias[p.dual_off + n] : 0.f;
#pragma unroll 1
      for (int c = 0; c < BN; c += 16) {
        uint32_t v[16];
        uint32_t vu[DUAL ? 16 : 1];
        tmem_ld16(taddr + c, v);
        if constexpr (DUAL) tmem_ld16(taddr + BN + c, vu);
        tmem_ld_wait();
        if (c + 16 >= BN) {
          // the accumulator is in registers: hand the TMEM buffer back to the MMA warp before the stores
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tmem_empty[a]);
        }
        // full 128-feature tile and the caller asked for it: rows go out as 256-byte runs through shared memory.
        // Uniform over the 128 epilogue threads (it depends on the tile only), so the barriers inside are safe.
        const bool wide = p.wide && (nt * 128 + 128 <= p.N) && (p.N % 8 == 0) && (p.ldo % 8 == 0);
        if (!owned && wide) {
#pragma unroll
          for (int j = 0; j < 16; ++j) s_stage[j * kStageLd + row] = __float2bfloat16(__uint_as_float(v[j]));
          named_bar_sync(1, 128);
          __nv_bfloat16* base = p.ar.part[owner] + (size_t)rank * p.ar.part_stride +
                                ((size_t)own_idx * BN + c) * p.N + nt * 128;
#pragma unroll
          for (int it = 0; it < 2; ++it) {
            const int j = (et >> 4) + 8 * it, seg = et & 15;          // 16 threads write one 256-byte row
            if (t0 + c + j < p.T)
              *reinterpret_cast<uint4*>(base + (size_t)j * p.N + seg * 8) =
                  *reinterpret_cast<const uint4*>(&s_stage[j * kStageLd + seg * 8]);
          }
          named_bar_sync(1, 128);                                      // the buffer is reused by the next chunk
          continue;
        }
        if (!n_ok) continue;
        if (!owned) {
          __nv_bfloat16* dst = p.ar.part[owner] + (size_t)rank * p.ar.part_stride +
                               ((size_t)own_idx * BN + c) * p.N + n;
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (t0 + c + j < p.T) dst[(size_t)j * p.N] = __float2bfloat16(__uint_as_float(v[j]));
          continue;
        }
        float x[16];
        if (world > 1) {
          // sum in rank order; this rank's own term is its fp32 accumulator, the others arrive rounded to bf16
#pragma unroll
          for (int j = 0; j < 16; ++j) x[j] = 0.f;
          for (int r = 0; r < world; ++r) {
            if (r == rank) {
#pragma unroll
              for (int j = 0; j < 16; ++j) x[j] += __uint_as_float(v[j]);
            } else {
              const __nv_bfloat16* src = p.ar.part[rank] + (size_t)r * p.ar.part_stride +
                                         ((size_t)own_idx * BN + c) * p.N + n;
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (t0 + c + j < p.T) x[j] += __bfloat162float(__ldcg(src + (size_t)j * p.N));
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) x[j] = __uint_as_float(v[j]);
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int t = t0 + c + j;
          if (t < p.T) {
            float y = prefill_act(x[j] + bias, p.act);
            if constexpr (DUAL) y *= __uint_as_float(vu[j]) + bias_u;
            if (p.residual) y += p.res_scale * __bfloat162float(p.residual[(size_t)t * p.ldr + n]);
            const __nv_bfloat16 yb = __float2bfloat16(y);
            if (wide) {
              s_stage[j * kStageLd + row] = yb;
            } else if (world > 1) {
              for (int r = 0; r < world; ++r) p.ar.out[r][(size_t)t * p.ldo + n] = yb;
            } else {
              p.out[(size_t)t * p.ldo + n] = yb;
            }
          }
        }
        if (wide) {
          named_bar_sync(1, 128);
#pragma unroll
          for (int it = 0; it < 2; ++it) {
            const int j = (et >> 4) + 8 * it, seg = et & 15;
            const int t = t0 + c + j;
            if (t < p.T) {
              const uint4 val = *reinterpret_cast<const uint4*>(&s_stage[j * kStageLd + seg * 8]);
              const size_t off = (size_t)t * p.ldo + nt * 128 + seg * 8;
              if (world > 1) {
                for (int r = 0; r < world; ++r) *reinterpret_cast<uint4*>(p.ar.out[r] + off) = val;
              } else {
                *reinterpret_cast<uint4*>(p.out + off) = val;
              }
            }
          }
          named_bar_sync(1, 128);
        }
      }
      if (world > 1) {
        __threadfence_system();               // this thread's stores to peer memory, before the flag below
        named_bar_sync(1, 128);
        if (!owned) {
          if (et == 0)
            st_release_sys(p.ar.flag_part[owner] + ((size_t)own_idx * p.n_tiles + nt) * world + rank, epoch);
        } else if (et < world && et != rank) {
          st_release_sys(p.ar.flag_res[et] + (size_t)blk * p.n_tiles + nt, epoch);
        }
      }
    }
    if (world > 1) {
      // The launch is complete on this rank when the finished tiles of every other owner are here.  The CTA that
      // finishes last checks them all, then opens the next epoch.
      named_bar_sync(1, 128);
      if (et == 0) {
        __threadfence();
        s_last = (atomicAdd(p.ar.done, 1) == (int)gridDim.x - 1);
      }
      named_bar_sync(1, 128);
      if (s_last) {
        bool ok = !*s_abort;
        for (int idx = et; idx < total && ok; idx += 128) {
          const int blk = idx / p.n_tiles;
          if (blk % world == rank) continue;
          if (!wait_flag(p.ar.flag_res[rank] + idx, epoch, p.ar.wait_cycles)) {
            if (p.status) atomicCAS(p.status, 0, XFT_ERR_WAIT_PEER);
            ok = false;
          }
        }
        named_bar_sync(1, 128);
        if (et == 0) {
          *reinterpret_cast<volatile int*>(p.ar.done) = 0;
          __threadfence();
          atomicAdd(p.ar.epoch, 1);
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

// ------------------------------------------------------------------------------------------------------------------
// Token-major form (one GPU, or the local product in front of a library collective).  Same pipeline, but the operands
// trade places: the 128 rows of the MMA are 128 TOKENS (A = the activation tile) and its columns are BNF output features
// (B = the weight tile), so the accumulator is [token lane][feature column] — the layout of Y itself.  Each epilogue
// thread owns one token row and handles 16 consecutive features per step: bias and residual arrive as 16-byte vectors
// and the result leaves as two 16-byte stores, instead of one 2-byte store per element in the feature-major form, whose
// epilogue (a dependent chain per element on four warps) took ten times longer than the main loop of the short-K
// row-parallel products.  Gated form: gate and up accumulators of 128 features each, act(gate) * up on the way out.
template <int BNF, bool DUAL>
__global__ void __launch_bounds__(192, 1) gemm_prefill_tm_kernel(const __grid_constant__ CUtensorMap tmX,
                                                                 const __grid_constant__ CUtensorMap tmW,
                                                                 const PrefillParams p) {
  constexpr int A_BYTES = 128 * 64 * 2;                  // 128 tokens x 64 k
  constexpr int B_BYTES = BNF * 64 * 2;                  // BNF features x 64 k
  constexpr int NACC = DUAL ? 2 : 1;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES * NACC;
  constexpr uint32_t TMEM_COLS = 2 * BNF * NACC;         // double-buffered accumulators
  constexpr uint32_t IDESC = umma_idesc(128, BNF, 1, 1, 1);
  static_assert((BNF == 256 && !DUAL) || (BNF == 128 && DUAL), "feature tile of the token-major kernel");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full_bar[kPrefillMaxStages], empty_bar[kPrefillMaxStages], tmem_full[2], tmem_empty[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_abort_mem;
  volatile int* s_abort = &s_abort_mem;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int stages = p.stages;
  const int total = p.n_tiles * p.t_tiles;               // n_tiles: feature tiles of BNF, t_tiles: token blocks of 128

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 4);
    }
    s_abort_mem = 0;
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

  if (warp == 0) {
    if (lane == 0) {
      const uint64_t hint = kEvictNormal;
      int it = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total && ok; item += gridDim.x) {
        int nt, blk;
        decode_item(p, item, nt, blk);
        for (int kb = 0; kb < p.num_kb; ++kb, ++it) {
          const int s = it % stages;
          const uint32_t ph = (it / stages) & 1;
          if (*s_abort || !mbar_wait_or_abort(&empty_bar[s], ph ^ 1, p.status, XFT_ERR_WAIT_EMPTY, s_abort)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&full_bar[s], STAGE_BYTES);
          uint8_t* a = smem + s * STAGE_BYTES;
          tma_load_2d(a, &tmX, &full_bar[s], kb * 64, blk * 128, hint);
          tma_load_2d(a + A_BYTES, &tmW, &full_bar[s], kb * 64, nt * BNF, hint);
          if (DUAL) tma_load_2d(a + A_BYTES + B_BYTES, &tmW, &full_bar[s], kb * 64, p.dual_off + nt * BNF, hint);
        }
      }
      if (!ok) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) {}
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int it = 0, lt = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total && ok; item += gridDim.x, ++lt) {
        const int a = lt & 1;
        const uint32_t aph = (lt >> 1) & 1;
        if (*s_abort || !mbar_wait_or_abort(&tmem_empty[a], aph ^ 1, p.status, XFT_ERR_WAIT_TMEM, s_abort)) break;
        tcgen05_fence_after();
        const uint32_t acc = tmem_base + (uint32_t)(a * BNF * NACC);
        for (int kb = 0; kb < p.num_kb; ++kb, ++it) {
          const int s = it % stages;
          const uint32_t ph = (it / stages) & 1;
          if (!mbar_wait_or_abort(&full_bar[s], ph, p.status, XFT_ERR_WAIT_FULL, s_abort)) {
            ok = false;
            break;
          }
          tcgen05_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
          const uint64_t adesc = umma_desc_k128(a_addr);                      // tokens
          const uint64_t bdesc = umma_desc_k128(a_addr + A_BYTES);            // features (gate)
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            umma_bf16(acc, adesc + 2 * k, bdesc + 2 * k, IDESC, (kb > 0 || k > 0) ? 1u : 0u);
            if (DUAL) {
              const uint64_t b1desc = umma_desc_k128(a_addr + A_BYTES + B_BYTES);
              umma_bf16(acc + BNF, adesc + 2 * k, b1desc + 2 * k, IDESC, (kb > 0 || k > 0) ? 1u : 0u);
            }
          }
          tcgen05_commit(&empty_bar[s]);
        }
        if (ok) tcgen05_commit(&tmem_full[a]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue: one token row per thread
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const bool vec = (p.N % 8 == 0) && (p.ldo % 8 == 0) && (!p.residual || p.ldr % 8 == 0);
    int lt = 0;
    for (int item = blockIdx.x; item < total; item += gridDim.x, ++lt) {
      int nt, blk;
      decode_item(p, item, nt, blk);
      const int a = lt & 1;
      const uint32_t aph = (lt >> 1) & 1;
      mbar_wait_or_abort(&tmem_full[a], aph, p.status, XFT_ERR_WAIT_TMEM, s_abort);
      if (named_bar_or(1, 128, *s_abort != 0)) break;
      tcgen05_fence_after();
      const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + (uint32_t)(a * BNF * NACC);
      const int t = blk * 128 + row;
      const bool t_ok = t < p.T;
      __nv_bfloat16* orow = p.out + (size_t)t * p.ldo;
      const __nv_bfloat16* rrow = p.residual ? p.residual + (size_t)t * p.ldr : nullptr;
#pragma unroll 1
      for (int c = 0; c < BNF; c += 16) {
        uint32_t v[16];
        uint32_t vu[DUAL ? 16 : 1];
        tmem_ld16(taddr + c, v);
        if constexpr (DUAL) tmem_ld16(taddr + BNF + c, vu);
        tmem_ld_wait();
        if (c + 16 >= BNF) {
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tmem_empty[a]);
        }
        const int n0 = nt * BNF + c;
        if (!t_ok || n0 >= p.N) continue;
        float x[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) x[j] = __uint_as_float(v[j]);
        const bool full = vec && n0 + 16 <= p.N;
        if (p.bias) {
#pragma unroll
          for (int j = 0; j < 16; ++j) if (full || n0 + j < p.N) x[j] += __ldg(p.bias + n0 + j);
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) x[j] = prefill_act(x[j], p.act);
        if constexpr (DUAL) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float u = __uint_as_float(vu[j]);
            if (p.bias && (full || n0 + j < p.N)) u += __ldg(p.bias + p.dual_off + n0 + j);
            x[j] *= u;
          }
        }
        if (full) {
          if (rrow) {
            const uint4 r0 = *reinterpret_cast<const uint4*>(rrow + n0), r1 = *reinterpret_cast<const uint4*>(rrow + n0 + 8);
            const __nv_bfloat162* h0 = reinterpret_cast<const __nv_bfloat162*>(&r0);
            const __nv_bfloat162* h1 = reinterpret_cast<const __nv_bfloat162*>(&r1);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 f0 = __bfloat1622float2(h0[j]), f1 = __bfloat1622float2(h1[j]);
              x[2 * j] += p.res_scale * f0.x; x[2 * j + 1] += p.res_scale * f0.y;
              x[8 + 2 * j] += p.res_scale * f1.x; x[8 + 2 * j + 1] += p.res_scale * f1.y;
            }
          }
          uint32_t w[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const __nv_bfloat162 b = __floats2bfloat162_rn(x[2 * j], x[2 * j + 1]);
            w[j] = *reinterpret_cast<const uint32_t*>(&b);
          }
          *reinterpret_cast<uint4*>(orow + n0) = make_uint4(w[0], w[1], w[2], w[3]);
          *reinterpret_cast<uint4*>(orow + n0 + 8) = make_uint4(w[4], w[5], w[6], w[7]);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (n0 + j < p.N) {
              float y = x[j];
              if (rrow) y += p.res_scale * __bfloat162float(rrow[n0 + j]);
              orow[n0 + j] = __float2bfloat16(y);
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

template <int BNF, bool DUAL>
static int launch_prefill_tm(const CUtensorMap& tmX, const CUtensorMap& tmW, PrefillParams& p, int num_ctas,
                             cudaStream_t st) {
  constexpr int STAGE_BYTES = 128 * 64 * 2 + BNF * 64 * 2 * (DUAL ? 2 : 1);
  int stages = (196 * 1024) / STAGE_BYTES;
  if (stages > kPrefillMaxStages) stages = kPrefillMaxStages;
  p.stages = stages;
  const size_t smem = (size_t)stages * STAGE_BYTES + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_prefill_tm_kernel<BNF, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return 3000 + (int)cudaGetLastError();
    attr_set = true;
  }
  const int total = p.n_tiles * p.t_tiles;
  const int grid = total < num_ctas ? total : num_ctas;
  gemm_prefill_tm_kernel<BNF, DUAL><<<grid, 192, smem, st>>>(tmX, tmW, p);
  return (int)cudaGetLastError();
}

template <int BN, bool DUAL>
static int launch_prefill(const CUtensorMap& tmW, const CUtensorMap& tmX, PrefillParams& p, int num_ctas,
                          cudaStream_t st) {
  constexpr int STAGE_BYTES = 128 * 64 * 2 * (DUAL ? 2 : 1) + BN * 64 * 2;
  int stages = (220 * 1024) / STAGE_BYTES;
  if (stages > kPrefillMaxStages) stages = kPrefillMaxStages;
  p.stages = stages;
  const size_t smem = (size_t)stages * STAGE_BYTES + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    // the request is the ring itself: the kernel's static shared memory (barriers, the 4 KB store staging tile)
    // counts against the same 227 KB, so asking for more than the ring needs can be refused
    if (cudaFuncSetAttribute(gemm_prefill_kernel<BN, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return 3000 + (int)cudaGetLastError();
    attr_set = true;
  }
  const int total = p.n_tiles * p.t_tiles;
  const int grid = total < num_ctas ? total : num_ctas;
  gemm_prefill_kernel<BN, DUAL><<<grid, 192, smem, st>>>(tmW, tmX, p);
  return (int)cudaGetLastError();
}

}  // namespace xft

using namespace xft;

// Elements of one source slot of the partial area and the flag counts a launch of (T, N) needs at `world` ranks.
extern "C" void xft_prefill_ar_sizes(int T, int N, int world, long long* part_elems_per_slot, long long* n_flag_part,
                                     long long* n_flag_res) {
  const int bn = T > 128 ? 256 : 128;
  const long long t_tiles = (T + bn - 1) / bn, n_tiles = (N + 127) / 128;
  const long long own = (t_tiles + world - 1) / world;
  *part_elems_per_slot = own * bn * (long long)N;
  *n_flag_part = own * n_tiles * world;
  *n_flag_res = t_tiles * n_tiles;
}

// Y = act(X W^T (+ the same product of every other rank) + bias) + res_scale * residual, bf16.  ar == nullptr or
// ar->world <= 1: plain persistent GEMM.  order: optional device array, the order in which token blocks are visited
// (with ar it must hold the same multiset on every rank, see the file comment).  Returns 0, a negative argument
// error, or a CUDA error code.
extern "C" int xft_gemm_bf16_prefill(const void* X, int ldx, const void* W, int w_rows, int ldw, void* Y, int ldo, int T,
                                     int N, int K, const float* bias, const void* residual, int ldr, float res_scale,
                                     int act, const int* order, int* status, const BulkArParams* ar, int num_ctas,
                                     cudaStream_t st) {
  if (T <= 0 || N <= 0 || K <= 0) return 0;
  if ((K & 7) || (ldx & 7) || (ldw & 7)) return -2;
  PrefillParams p{};
  p.N = N; p.T = T; p.K = K; p.out = reinterpret_cast<__nv_bfloat16*>(Y); p.ldo = ldo; p.bias = bias;
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual); p.ldr = ldr; p.res_scale = res_scale; p.act = act;
  p.order = order; p.status = status;
  static const int wide_env = [] { const char* v = getenv("XFT_PREFILL_WIDE_STORES"); return v && v[0] == '1' ? 1 : 0; }();
  p.wide = wide_env;
  const int bn = T > 128 ? 256 : 128;
  p.n_tiles = (N + 127) / 128;
  p.t_tiles = (T + bn - 1) / bn;
  p.num_kb = (K + 63) / 64;
  p.gn = 16;
  if (ar && ar->world > 1) {
    if (ar->world > 8 || ar->rank < 0 || ar->rank >= ar->world) return -3;
    long long need_part, nfp, nfr;
    xft_prefill_ar_sizes(T, N, ar->world, &need_part, &nfp, &nfr);
    if (ar->part_stride < need_part) return -4;
    if (ar->out[ar->rank] != p.out) return -5;
    p.ar = *ar;
    p.gn = p.n_tiles;                 // block-major: all feature tiles of a token block are visited together
  }
  if (num_ctas <= 0) {
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    num_ctas = sms > 0 ? sms : 148;
  }
  CUtensorMap tmW, tmX;
  int r = make_tensor_map(&tmW, W, (uint64_t)w_rows, (uint64_t)K, (uint64_t)ldw, 128, 2);
  if (r) return 1000 - r;
  r = make_tensor_map(&tmX, X, (uint64_t)T, (uint64_t)K, (uint64_t)ldx, (uint32_t)bn, 2);
  if (r) return 2000 - r;
  return bn == 256 ? launch_prefill<256, false>(tmW, tmX, p, num_ctas, st)
                   : launch_prefill<128, false>(tmW, tmX, p, num_ctas, st);
}

// Gated form: Y[T, N] = act(X Wg^T + bias_g) * (X Wu^T + bias_u), W holds gate rows [0, N) and up rows
// [dual_off, dual_off + N) (bias likewise).  Token tiles of 128.
extern "C" int xft_gemm_bf16_prefill_gated(const void* X, int ldx, const void* W, int w_rows, int ldw, void* Y, int ldo,
                                           int T, int N, int K, int dual_off, const float* bias, int act, int* status,
                                           int num_ctas, cudaStream_t st) {
  if (T <= 0 || N <= 0 || K <= 0) return 0;
  if ((K & 7) || (ldx & 7) || (ldw & 7)) return -2;
  PrefillParams p{};
  p.N = N; p.T = T; p.K = K; p.out = reinterpret_cast<__nv_bfloat16*>(Y); p.ldo = ldo; p.bias = bias; p.act = act;
  p.status = status; p.dual_off = dual_off;
  static const int wide_env = [] { const char* v = getenv("XFT_PREFILL_WIDE_STORES"); return v && v[0] == '1' ? 1 : 0; }();
  p.wide = wide_env;
  p.n_tiles = (N + 127) / 128;
  p.t_tiles = (T + 127) / 128;
  p.num_kb = (K + 63) / 64;
  p.gn = 16;
  if (num_ctas <= 0) {
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    num_ctas = sms > 0 ? sms : 148;
  }
  CUtensorMap tmW, tmX;
  int r = make_tensor_map(&tmW, W, (uint64_t)w_rows, (uint64_t)K, (uint64_t)ldw, 128, 2);
  if (r) return 1000 - r;
  r = make_tensor_map(&tmX, X, (uint64_t)T, (uint64_t)K, (uint64_t)ldx, 128, 2);
  if (r) return 2000 - r;
  return launch_prefill<128, true>(tmW, tmX, p, num_ctas, st);
}

// Size and field offsets of BulkArParams, for the layout check of the Python mirror.
extern "C" int xft_bulk_ar_layout(long long* out, int n) {
  const long long v[] = {sizeof(BulkArParams),           offsetof(BulkArParams, world),       offsetof(BulkArParams, rank),
                         offsetof(BulkArParams, part),   offsetof(BulkArParams, flag_part),   offsetof(BulkArParams, out),
                         offsetof(BulkArParams, flag_res), offsetof(BulkArParams, epoch),     offsetof(BulkArParams, done),
                         offsetof(BulkArParams, part_stride), offsetof(BulkArParams, wait_cycles)};
  const int m = (int)(sizeof(v) / sizeof(v[0]));
  for (int i = 0; i < m && i < n; ++i) out[i] = v[i];
  return m;
}

// Token-major persistent GEMM (see gemm_prefill_tm_kernel): Y[T, N] = act(X W^T + bias) [* (X Wu^T + bias_u)] +
// res_scale * residual, bf16.  gated != 0: gate rows [0, N) and up rows [dual_off, dual_off + N) of W.
extern "C" int xft_gemm_bf16_prefill_tm(const void* X, int ldx, const void* W, int w_rows, int ldw, void* Y, int ldo, int T,
                                        int N, int K, int gated, int dual_off, const float* bias, const void* residual,
                                        int ldr, float res_scale, int act, int* status, int num_ctas, cudaStream_t st) {
  if (T <= 0 || N <= 0 || K <= 0) return 0;
  if ((K & 7) || (ldx & 7) || (ldw & 7)) return -2;
  PrefillParams p{};
  p.N = N; p.T = T; p.K = K; p.out = reinterpret_cast<__nv_bfloat16*>(Y); p.ldo = ldo; p.bias = bias;
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual); p.ldr = ldr; p.res_scale = res_scale; p.act = act;
  p.status = status; p.dual_off = dual_off;
  const int bnf = gated ? 128 : 256;
  p.n_tiles = (N + bnf - 1) / bnf;
  p.t_tiles = (T + 127) / 128;
  p.num_kb = (K + 63) / 64;
  p.gn = 8;
  if (num_ctas <= 0) {
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    num_ctas = sms > 0 ? sms : 148;
  }
  CUtensorMap tmW, tmX;
  int r = make_tensor_map(&tmW, W, (uint64_t)w_rows, (uint64_t)K, (uint64_t)ldw, (uint32_t)bnf, 2);
  if (r) return 1000 - r;
  r = make_tensor_map(&tmX, X, (uint64_t)T, (uint64_t)K, (uint64_t)ldx, 128, 2);
  if (r) return 2000 - r;
  return gated ? launch_prefill_tm<128, true>(tmX, tmW, p, num_ctas, st) : launch_prefill_tm<256, false>(tmX, tmW, p, num_ctas, st);
}
