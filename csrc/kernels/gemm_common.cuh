// Definitions shared by the GEMM kernels of this library (gemm_sm100.cu, gemm_decode_sm100.cu): the peer-memory
// description of the fused all-reduce, the 8-byte transport word, activation functions, the tensor-map helper.
#pragma once
#include "ptx.cuh"

namespace xft {

// Fused one-shot all-reduce (row-parallel o_proj / down_proj at decode sizes): replaces the reference's
// GEMM followed by Messenger::reduceAdd (src/layers/decoder_block.h:122-134).  `recv[r]` is rank r's
// receive area [2 parities][world slots][slot words] as mapped into this process (CUDA IPC over NVLink);
// each word is {two bf16 values (tokens t, t + 1 of one feature), epoch}.  The CTA that finishes an output tile stores its partial tile into
// slot `rank` of every rank straight from the accumulator, then reads the world slots of its own area,
// spinning (bounded) on each word until its epoch matches, and sums them in rank order, so all ranks
// produce bit-identical results.  No fence, flag or barrier separates a producer's store from the
// consumer's load.  The epoch is a device-side counter bumped by the last CTA of each launch, which keeps
// the scheme valid under CUDA-graph replay; the parity (epoch & 1) double-buffers the area.
struct CommParams {
  int world, rank;
  unsigned long long* recv[8];
  int* epoch;              // local: number of completed fused launches
  int* done;               // local: CTAs of the current launch that have exited
  long long slot_stride;   // words per source slot
  long long parity_stride; // words per parity (= world * slot_stride)
  long long wait_cycles;   // bound of the wait on a peer's word
  // two_shot != 0 (used for world >= 4): tile i is owned by rank i % world.  Partials go only to the owner
  // (reduce-scatter), which sums them, applies the epilogue and stores the finished value into `result`
  // of every rank (all-gather); the other ranks wait for that word.  Traffic per rank falls from
  // (world-1) x tile to about 2 x (world-1)/world x tile for one extra NVLink hop.
  int two_shot;
  unsigned long long* result[8];   // rank r's result area [2 parities][slot words]
};

// Payload of one LL word of the fused all-reduce: two bf16 values (tokens t and t + 1 of one feature).  Partials are
// rounded to bf16 before they cross NVLink, as a bf16 all-reduce does; the sum itself runs in fp32.
__device__ __forceinline__ unsigned long long ll_pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return (unsigned long long)(*reinterpret_cast<unsigned*>(&v));
}
__device__ __forceinline__ void ll_unpack2(unsigned w, float& lo, float& hi) {
  const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&w);
  const float2 f = __bfloat1622float2(v);
  lo = f.x; hi = f.y;
}

__device__ __forceinline__ float apply_act(float x, int act) {
  switch (act) {
    case 1: return fmaxf(x, 0.f);
    case 2: return x / (1.f + __expf(-x));
    case 3: {
      const float c = 0.7978845608028654f;
      float u = c * (x + 0.044715f * x * x * x);
      return 0.5f * x * (1.f + tanhf(u));
    }
    default: return x;
  }
}

// K-major matrix [rows, cols] with row stride `ld` elements; box = 128 bytes x box_rows, 128B swizzle (gemm_sm100.cu).
int make_tensor_map(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                    uint32_t esize);
// token tile (UMMA N) that holds T tokens: 16, 32, 64, 128 or 256
int pick_bn(int T);

}  // namespace xft
