// C ABI of libxft_b200_kernels.so as used by the C++ runtime (definitions: csrc/kernels/*.cu).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

extern "C" {
int xft_gemm_bf16(const void* X, int ldx, const void* W, int w_rows, int ldw, void* Y, int ldo, int out_fp32, int T, int N,
                  int K, int gated, int dual_off, const float* bias, const void* residual, int ldr, float res_scale,
                  int act, const float* row_scale, float* ws, size_t ws_bytes, int* counters, int n_counters, int* status,
                  int force_splits, cudaStream_t st);
int xft_embedding(const int* ids, const void* table, void* out, int T, int H, int vocab, float scale, const void* pos_table,
                  const int* positions, int pos_offset, int npos, int* status, cudaStream_t st);
int xft_rmsnorm(const void* x, int ldx, const void* res, int ldr, const float* w, void* y, int ldy, void* h_out, int T, int H,
                float eps, cudaStream_t st);
int xft_layernorm(const void* x, int ldx, const float* w, const float* b, void* y, int ldy, int T, int H, float eps,
                  cudaStream_t st);
int xft_qkv_rope_cache(const void* qkv, int ldq, int T, int hq, int hkv, int D, const int* positions, const float* table,
                       int rot, int style, int rot_off, int max_pos, const float* q_scale, const float* q_norm_w,
                       const float* k_norm_w, float eps, void* q_out, void* kc, void* vc, float* ks, float* vs,
                       int int8_cache, int bs, long long nslots, const int* slots, int* status, cudaStream_t st);
int xft_qkv_rope2d_cache(const void* qkv, int ldq, int T, int hq, int hkv, int D, const int* positions,
                         const int* positions2, const float* table, int rot, int max_pos, void* q_out, void* kc,
                         void* vc, float* ks, float* vs, int int8_cache, int bs, long long nslots, const int* slots,
                         int* status, cudaStream_t st);
int xft_rope(void* x, int T, int nh, int D, const int* positions, const float* table, int rot, int style, int rot_off,
             int max_pos, const float* q_scale, int* status, cudaStream_t st);
int xft_paged_attention(const void* q, void* out, const void* kc, const void* vc, const float* ks, const float* vs,
                        const int* block_table, int bt_stride, const int* cu_q, const int* kv_lens, int B, int max_q, int hq,
                        int hkv, int group, int q_off, int HD, int bs, int num_blocks, float scale, const float* slopes,
                        const int* prefix_lens, int decode, int nsplit, float* part_o, float* part_ml, int* split_counters,
                        int* status, cudaStream_t st);
int xft_argmax(const float* logits, int ld, int rows, int V, float* vals, int* idx, cudaStream_t st);
int xft_transpose_to_bf16(const void* src, int dtype, long long ld_src, int rows, int cols, void* dst, long long ld_dst,
                          cudaStream_t st);
int xft_fp8_block_dequant(const void* src, const float* scale, long long rows, int cols, int block, void* dst,
                          cudaStream_t st);
int xft_moe_route(const float* logits, int ld, int T, int E, int k, int kind, const float* bias, int n_group, int topk_group,
                  float scaling, int norm_topk, int sigmoid, int* idx, float* w, cudaStream_t st);
int xft_moe_plan(const int* idx, const float* w, int T, int k, int e0, int e1, int bn, int* pos, int* src_tok, float* row_w,
                 void* tiles, int* meta, int max_tiles, int max_rows, cudaStream_t st);
int xft_moe_gather(const void* x, int ldx, const int* src_tok, const int* meta, void* xs, int max_rows, int H, cudaStream_t st);
int xft_moe_combine(const float* ys, const int* pos, int k, const float* add1, const void* add2, int ld2, void* y, float* y32,
                    int T, int H, cudaStream_t st);
int xft_gemm_bf16_grouped(const void* X, int ldx, int x_rows, const void* W, int w_rows, int ldw, void* Y, int ldo,
                          int out_fp32, int N, int K, int gated, int dual_off, int group_w_rows, const void* group_tiles,
                          const int* num_group_tiles, int max_tiles, int bn, const float* col_scale, int act, int* status,
                          cudaStream_t st);
// quantised weights: load-time quantiser (mode 0 int8, 1 uint4, 2 nf4), weight-only GEMM (qtype 0 int8, 1 int4, 2 nf4,
// 3 fp8, 4 int4 fast layout), per-row activation sums / dynamic int8 activations, int8 x int8 GEMM, act(gate) * up
int xft_quantize_rows(const void* w, int dtype, long long ldw, int rows, int K, int mode, void* q, long long ldq_bytes,
                      float* scale, float* zero, float* wsum, cudaStream_t st);
int xft_qgemm(const void* X, int ldx, const void* Wq, int w_rows, int ldw_bytes, int qtype, void* Y, int ldo, int out_fp32,
              int T, int N, int K, int gated, int dual_off, const float* scale, const float* zero, const float* xsum,
              int scale_ld, const float* bias, const void* residual, int ldr, float res_scale, int act, float* ws,
              size_t ws_bytes, int* counters, int n_counters, int* status, cudaStream_t st);
// grouped (expert) form for e4m3 weights: Wq stacks the experts' [group_w_rows, K] bytes, scale their
// [group_w_rows / 128, scale_ld] block scales (scale_ld = blocks along K); tiles / counts from xft_moe_plan
int xft_qgemm_grouped(const void* X, int ldx, int x_rows, const void* Wq, int w_rows, int ldw_bytes, void* Y, int ldo,
                      int out_fp32, int N, int K, int gated, int dual_off, int group_w_rows, const float* scale, int scale_ld,
                      const void* group_tiles, const int* num_group_tiles, int max_tiles, int bn, const float* col_scale,
                      int act, int* status, cudaStream_t st);
int xft_row_sum(const void* x, int ldx, float* out, int T, int K, cudaStream_t st);
int xft_quant_act(const void* x, int ldx, void* q, int ldq, float* scale, float* zero, float* qsum, int T, int K,
                  cudaStream_t st);
int xft_w8a8_gemm(const void* qx, int ldqx, const void* Wq, int ldw, void* Y, int ldo, int out_fp32, int T, int N, int K,
                  const float* a_scale, const float* a_zero, const float* a_qsum, const float* w_scale, const float* w_zero,
                  const float* w_sum, const float* bias, const void* residual, int ldr, float res_scale, int act, float* ws,
                  size_t ws_bytes, int* counters, int n_counters, int* status, cudaStream_t st);
int xft_gated_act(const void* gu, void* out, int T, int I, int act, cudaStream_t st);
// DeepSeek latent attention: the steps between the projections and the attention in one launch; the attention over the
// latent cache (q_abs / out: head stride, token stride in elements); [A, B, D] -> [B, A, D]
int xft_mla_prep(const void* q, int ldq, const void* kv, int ldkv, int T, int Hl, int nope, int rope, int kvl,
                 const int* positions, const float* table, int max_pos, const float* kv_norm_w, float eps, void* q_nope,
                 void* q_rope, void* cache, long long nslots, const int* slots, int* status, int nope_head_major,
                 cudaStream_t st);
int xft_mla_attention(const void* q_abs, long long qa_sh, long long qa_st, const void* q_rope, long long qr_sh, long long qr_st,
                      void* out, long long o_sh, long long o_st, const void* cache, const int* block_table, int bt_stride,
                      const int* cu_q, const int* kv_lens, int B, int T, int hl, int bs, int num_blocks, float scale,
                      int nsplit, float* part_o, float* part_ml, int* counters, int* status, cudaStream_t st);
int xft_swap_outer_dims(const void* src, void* dst, int A, int B, int D, cudaStream_t st);
// dst[i] <- sum of srcs[s][i], bf16, all pointers on this GPU (srcs: host array of nsrc <= 8 device pointers)
int xft_sum_bf16(void* dst, const void* const* srcs, int nsrc, size_t n, cudaStream_t st);
int xft_sample_topk_topp(const float* logits, int ld, int rows, int V, int k, float top_p, float temperature,
                         const float* uniform, int* out, cudaStream_t st);
}
