// A host stand-in for the device side of the C++ engine, for tests WITHOUT a GPU: the CUDA runtime calls that
// csrc/core makes (memory is plain malloc'd memory) and every entry point of the kernel library the engine calls.
// The stand-in kernels do no arithmetic worth the name; what they do is TOUCH exactly the bytes the real kernels
// read and write, computed from the same arguments — every row of every operand with its stride, every KV block a
// block table names, every expert's weight rows a tile points at.  Built with AddressSanitizer and with
// XFT_ARENA_EXACT=1 (buffers get exactly the size asked for), a run of the engine over this library checks the host
// side of every family x weight type x rank count: buffer sizes, strides, block and slot arithmetic, the tensor-
// parallel ranges, the order of collectives.  Indices that the real kernels would refuse through their status word
// (a slot or block outside the pool) abort here.
//
// The few results the host logic depends on are produced for real: the routing (valid expert ids), the expert plan
// (rows grouped by expert, tile table, counts) and logits that differ per row and step so that searchers move.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

namespace {

[[noreturn]] void die(const char* what) {
  std::fprintf(stderr, "mock device: %s\n", what);
  std::abort();
}
void need(bool ok, const char* what) { if (!ok) die(what); }

// read / write every byte of [p, p + bytes): ASan checks the range
volatile unsigned char g_sink;
void rd(const void* p, size_t bytes) {
  if (!bytes) return;
  need(p != nullptr, "null pointer read");
  const unsigned char* c = static_cast<const unsigned char*>(p);
  unsigned char acc = 0;
  for (size_t i = 0; i < bytes; i += 64) acc ^= c[i];
  acc ^= c[bytes - 1];
  g_sink = acc;
}
void wr(void* p, size_t bytes, int value = 0) {
  if (!bytes) return;
  need(p != nullptr, "null pointer write");
  std::memset(p, value, bytes);
}
// rows x cols elements of `esz` bytes with a row stride of ld elements
void rdRows(const void* p, long long rows, long long cols, long long ld, size_t esz) {
  need(ld >= cols || rows <= 1, "row stride smaller than the row");
  for (long long r = 0; r < rows; ++r) rd(static_cast<const char*>(p) + (size_t)r * ld * esz, (size_t)cols * esz);
}
void wrRows(void* p, long long rows, long long cols, long long ld, size_t esz, int value = 0) {
  need(ld >= cols || rows <= 1, "row stride smaller than the row");
  for (long long r = 0; r < rows; ++r) wr(static_cast<char*>(p) + (size_t)r * ld * esz, (size_t)cols * esz, value);
}
const uint16_t kBf16Small = 0x3c00;      // bf16 of 0.0078125: keeps activations finite and tiny

}  // namespace

// ------------------------------------------------------------------------------------------------ CUDA runtime
extern "C" {
cudaError_t cudaMalloc(void** p, size_t n) { *p = std::calloc(1, n ? n : 1); return *p ? cudaSuccess : cudaErrorMemoryAllocation; }
cudaError_t cudaFree(void* p) { std::free(p); return cudaSuccess; }
cudaError_t cudaMallocHost(void** p, size_t n) { *p = std::calloc(1, n ? n : 1); return *p ? cudaSuccess : cudaErrorMemoryAllocation; }
cudaError_t cudaFreeHost(void* p) { std::free(p); return cudaSuccess; }
cudaError_t cudaMemcpy(void* d, const void* s, size_t n, cudaMemcpyKind) { if (n) std::memmove(d, s, n); return cudaSuccess; }
cudaError_t cudaMemcpyAsync(void* d, const void* s, size_t n, cudaMemcpyKind, cudaStream_t) { if (n) std::memmove(d, s, n); return cudaSuccess; }
cudaError_t cudaMemset(void* d, int v, size_t n) { if (n) std::memset(d, v, n); return cudaSuccess; }
cudaError_t cudaMemsetAsync(void* d, int v, size_t n, cudaStream_t) { if (n) std::memset(d, v, n); return cudaSuccess; }
cudaError_t cudaStreamCreate(cudaStream_t* s) { static char token; *s = reinterpret_cast<cudaStream_t>(&token); return cudaSuccess; }
cudaError_t cudaStreamSynchronize(cudaStream_t) { return cudaSuccess; }
cudaError_t cudaDeviceSynchronize() { return cudaSuccess; }
cudaError_t cudaGetLastError() { return cudaSuccess; }
cudaError_t cudaGetDeviceCount(int* n) { *n = 1; return cudaSuccess; }
cudaError_t cudaSetDevice(int) { return cudaSuccess; }
cudaError_t cudaGetDevice(int* d) { *d = 0; return cudaSuccess; }
const char* cudaGetErrorString(cudaError_t) { return "mock device error"; }
}

// ------------------------------------------------------------------------------------------------ kernel library
extern "C" {

int xft_embedding(const int* ids, const void* table, void* out, int T, int H, int vocab, float, const void* pos_table,
                  const int* positions, int pos_offset, int npos, int*, cudaStream_t) {
  rd(ids, (size_t)T * 4);
  for (int t = 0; t < T; ++t) {
    need(ids[t] >= 0 && ids[t] < vocab, "embedding: token id outside the vocabulary");
    rd(static_cast<const char*>(table) + (size_t)ids[t] * H * 2, (size_t)H * 2);
    if (pos_table) {
      const int p = positions[t] + pos_offset;
      need(p >= 0 && p < npos, "embedding: position outside the table");
      rd(static_cast<const char*>(pos_table) + (size_t)p * H * 2, (size_t)H * 2);
    }
  }
  uint16_t* o = static_cast<uint16_t*>(out);
  wrRows(out, T, H, H, 2);
  for (size_t i = 0; i < (size_t)T * H; ++i) o[i] = kBf16Small;
  return 0;
}

int xft_rmsnorm(const void* x, int ldx, const void* res, int ldr, const float* w, void* y, int ldy, void* h_out, int T, int H,
                float, cudaStream_t) {
  rdRows(x, T, H, ldx, 2);
  if (res) rdRows(res, T, H, ldr, 2);
  rd(w, (size_t)H * 4);
  wrRows(y, T, H, ldy, 2);
  if (h_out) wrRows(h_out, T, H, H, 2);
  return 0;
}

int xft_layernorm(const void* x, int ldx, const float* w, const float* b, void* y, int ldy, int T, int H, float, cudaStream_t) {
  rdRows(x, T, H, ldx, 2);
  rd(w, (size_t)H * 4);
  rd(b, (size_t)H * 4);
  wrRows(y, T, H, ldy, 2);
  return 0;
}

int xft_gemm_bf16(const void* X, int ldx, const void* W, int w_rows, int ldw, void* Y, int ldo, int out_fp32, int T, int N,
                  int K, int gated, int dual_off, const float* bias, const void* residual, int ldr, float, int, const float* row_scale,
                  float* ws, size_t ws_bytes, int* counters, int n_counters, int* status, int, cudaStream_t) {
  need(w_rows >= (gated ? dual_off + N : N), "gemm: weight has fewer rows than outputs");
  rdRows(X, T, K, ldx, 2);
  rdRows(W, gated ? dual_off + N : N, K, ldw, 2);
  if (bias) rd(bias, (size_t)(gated ? dual_off + N : N) * 4);
  if (residual) rdRows(residual, T, N, ldr, 2);
  if (row_scale) rd(row_scale, (size_t)T * 4);
  if (ws) { rd(ws, 1); rd(reinterpret_cast<char*>(ws) + ws_bytes - 1, 1); }
  if (counters) rd(counters, (size_t)n_counters * 4);
  if (status) rd(status, 4);
  if (out_fp32) {
    // logits and router scores: a different, deterministic number per (row, column) so that searches and routing move
    wrRows(Y, T, N, ldo, 4);
    float* y = static_cast<float*>(Y);
    static unsigned call = 0;
    ++call;
    for (int t = 0; t < T; ++t)
      for (int n = 0; n < N; ++n) y[(size_t)t * ldo + n] = (float)((((unsigned)n * 2654435761u) ^ ((unsigned)t * 40503u) ^ (call * 97u)) % 1000u) * 1e-3f;
  } else {
    wrRows(Y, T, N, ldo, 2);
  }
  return 0;
}

static void touchCache(void* kc, void* vc, float* ks, float* vs, int int8_cache, int hkv, int D, int bs, long long nslots,
                       const int* slots, int T) {
  rd(slots, (size_t)T * 4);
  const size_t esz = int8_cache ? 1 : 2;
  for (int t = 0; t < T; ++t) {
    const long long slot = slots[t];
    need(slot >= 0 && slot < nslots, "cache append: slot outside the pool");
    const long long blk = slot / bs, off = slot % bs;
    for (int h = 0; h < hkv; ++h) {
      const size_t row = (size_t)(blk * hkv + h) * bs + off;
      wr(static_cast<char*>(kc) + row * D * esz, (size_t)D * esz);
      wr(static_cast<char*>(vc) + row * D * esz, (size_t)D * esz);
      if (int8_cache) { wr(ks + row, 4); wr(vs + row, 4); }
    }
  }
}

int xft_qkv_rope_cache(const void* qkv, int ldq, int T, int hq, int hkv, int D, const int* positions, const float* table, int rot,
                       int, int rot_off, int max_pos, const float* q_scale, const float* q_norm_w, const float* k_norm_w, float,
                       void* q_out, void* kc, void* vc, float* ks, float* vs, int int8_cache, int bs, long long nslots,
                       const int* slots, int*, cudaStream_t) {
  rdRows(qkv, T, (long long)(hq + 2 * hkv) * D, ldq, 2);
  if (table && rot > 0) {
    need(rot_off + rot <= D, "rotary range outside the head");
    for (int t = 0; t < T; ++t) {
      need(positions[t] >= 0 && positions[t] < max_pos, "rotary position outside the table");
      rd(table + (size_t)positions[t] * rot, (size_t)rot * 4);
    }
  }
  if (q_scale) rd(q_scale, (size_t)T * 4);
  if (q_norm_w) rd(q_norm_w, (size_t)D * 4);
  if (k_norm_w) rd(k_norm_w, (size_t)D * 4);
  wrRows(q_out, T, (long long)hq * D, (long long)hq * D, 2);
  touchCache(kc, vc, ks, vs, int8_cache, hkv, D, bs, nslots, slots, T);
  return 0;
}

int xft_qkv_rope2d_cache(const void* qkv, int ldq, int T, int hq, int hkv, int D, const int* positions, const int* positions2,
                         const float* table, int rot, int max_pos, void* q_out, void* kc, void* vc, float* ks, float* vs,
                         int int8_cache, int bs, long long nslots, const int* slots, int*, cudaStream_t) {
  need(2 * rot <= D, "two-stream rotary wider than the head");
  rdRows(qkv, T, (long long)(hq + 2 * hkv) * D, ldq, 2);
  for (int t = 0; t < T; ++t) {
    need(positions[t] >= 0 && positions[t] < max_pos && positions2[t] >= 0 && positions2[t] < max_pos, "rotary position outside the table");
    rd(table + (size_t)positions[t] * rot, (size_t)rot * 4);
    rd(table + (size_t)positions2[t] * rot, (size_t)rot * 4);
  }
  wrRows(q_out, T, (long long)hq * D, (long long)hq * D, 2);
  touchCache(kc, vc, ks, vs, int8_cache, hkv, D, bs, nslots, slots, T);
  return 0;
}

int xft_paged_attention(const void* q, void* out, const void* kc, const void* vc, const float* ks, const float* vs,
                        const int* block_table, int bt_stride, const int* cu_q, const int* kv_lens, int B, int max_q, int hq,
                        int hkv, int group, int q_off, int HD, int bs, int num_blocks, float, const float* slopes,
                        const int* prefix_lens, int decode, int nsplit, float* part_o, float* part_ml, int* split_counters,
                        int* status, cudaStream_t) {
  rd(cu_q, (size_t)(B + 1) * 4);
  rd(kv_lens, (size_t)B * 4);
  const int T = cu_q[B];
  const bool int8 = ks != nullptr;
  const size_t esz = int8 ? 1 : 2;
  need(group >= 1 && q_off >= 0 && (hq - 1 + q_off) / group < hkv, "attention: query heads map outside the local KV heads");
  for (int b = 0; b < B; ++b) {
    const int nq = cu_q[b + 1] - cu_q[b];
    need(nq >= 1 && nq <= max_q && kv_lens[b] >= nq, "attention: query / context lengths inconsistent");
    if (decode) need(nq == 1, "attention: decode launch with more than one query row");
    const int nblk = (kv_lens[b] + bs - 1) / bs;
    need(nblk <= bt_stride, "attention: block table row too short");
    for (int j = 0; j < nblk; ++j) {
      const int blk = block_table[(size_t)b * bt_stride + j];
      need(blk >= 0 && blk < num_blocks, "attention: block outside the pool");
      const size_t bytes = (size_t)hkv * bs * HD * esz;
      rd(static_cast<const char*>(kc) + (size_t)blk * bytes, bytes);
      rd(static_cast<const char*>(vc) + (size_t)blk * bytes, bytes);
      if (int8) { rd(ks + (size_t)blk * hkv * bs, (size_t)hkv * bs * 4); rd(vs + (size_t)blk * hkv * bs, (size_t)hkv * bs * 4); }
    }
  }
  rdRows(q, T, (long long)hq * HD, (long long)hq * HD, 2);
  if (slopes) rd(slopes, (size_t)hq * 4);
  if (prefix_lens) rd(prefix_lens, (size_t)B * 4);
  if (nsplit > 1) {
    need(decode && part_o && part_ml && split_counters, "attention: split launch without its scratch");
    wr(part_o, (size_t)B * hq * nsplit * HD * 4);
    wr(part_ml, (size_t)B * hq * nsplit * 2 * 4);
    rd(split_counters, 4);
  }
  if (status) rd(status, 4);
  wrRows(out, T, (long long)hq * HD, (long long)hq * HD, 2);
  return 0;
}

int xft_transpose_to_bf16(const void* src, int dtype, long long ld_src, int rows, int cols, void* dst, long long ld_dst, cudaStream_t) {
  const size_t esz = dtype == 0 ? 4 : 2;
  rdRows(src, rows, cols, ld_src, esz);
  wrRows(dst, cols, rows, ld_dst, 2);
  return 0;
}

int xft_fp8_block_dequant(const void* src, const float* scale, long long rows, int cols, int block, void* dst, cudaStream_t) {
  rd(src, (size_t)rows * cols);
  rd(scale, (size_t)((rows + block - 1) / block) * ((cols + block - 1) / block) * 4);
  wr(dst, (size_t)rows * cols * 2);
  return 0;
}

// ---- quantised weights
int xft_quantize_rows(const void* w, int dtype, long long ldw, int rows, int K, int mode, void* q, long long ldq_bytes,
                      float* scale, float* zero, float* wsum, cudaStream_t) {
  need(mode >= 0 && mode <= 2 && (mode == 0 || K % 2 == 0), "quantize_rows: bad mode / odd K");
  rdRows(w, rows, K, ldw, dtype == 0 ? 4 : 2);
  wrRows(q, rows, mode == 0 ? K : K / 2, ldq_bytes, 1);
  wr(scale, (size_t)rows * 4);
  wr(zero, (size_t)rows * 4);
  if (wsum) wr(wsum, (size_t)rows * 4);
  return 0;
}

int xft_row_sum(const void* x, int ldx, float* out, int T, int K, cudaStream_t) {
  rdRows(x, T, K, ldx, 2);
  wr(out, (size_t)T * 4);
  return 0;
}

int xft_quant_act(const void* x, int ldx, void* q, int ldq, float* scale, float* zero, float* qsum, int T, int K, cudaStream_t) {
  rdRows(x, T, K, ldx, 2);
  wrRows(q, T, K, ldq, 1);
  wr(scale, (size_t)T * 4); wr(zero, (size_t)T * 4); wr(qsum, (size_t)T * 4);
  return 0;
}

int xft_qgemm(const void* X, int ldx, const void* Wq, int w_rows, int ldw_bytes, int qtype, void* Y, int ldo, int out_fp32, int T,
              int N, int K, int gated, int dual_off, const float* scale, const float* zero, const float* xsum, int, const float* bias,
              const void* residual, int ldr, float, int, float* ws, size_t ws_bytes, int* counters, int n_counters, int* status,
              cudaStream_t) {
  const int rows = gated ? dual_off + N : N;
  need(w_rows >= rows, "qgemm: weight has fewer rows than outputs");
  need(qtype == 0 || qtype == 1 || qtype == 2, "qgemm: weight type not used by the engine");
  need(ldw_bytes % 16 == 0, "qgemm: code rows must start on 16-byte boundaries");
  rdRows(X, T, K, ldx, 2);
  rdRows(Wq, rows, qtype == 0 ? K : K / 2, ldw_bytes, 1);
  rd(scale, (size_t)rows * 4);
  if (zero) { rd(zero, (size_t)rows * 4); need(xsum != nullptr, "qgemm: zero points without activation sums"); rd(xsum, (size_t)T * 4); }
  if (bias) rd(bias, (size_t)rows * 4);
  if (residual) rdRows(residual, T, N, ldr, 2);
  if (ws) rd(reinterpret_cast<char*>(ws) + ws_bytes - 1, 1);
  if (counters) rd(counters, (size_t)n_counters * 4);
  if (status) rd(status, 4);
  wrRows(Y, T, N, ldo, out_fp32 ? 4 : 2);
  return 0;
}

int xft_w8a8_gemm(const void* qx, int ldqx, const void* Wq, int ldw, void* Y, int ldo, int out_fp32, int T, int N, int K,
                  const float* a_scale, const float* a_zero, const float* a_qsum, const float* w_scale, const float* w_zero,
                  const float* w_sum, const float* bias, const void* residual, int ldr, float, int, float* ws, size_t ws_bytes,
                  int* counters, int n_counters, int* status, cudaStream_t) {
  need(K % 16 == 0, "w8a8: K must be a multiple of 16");
  rdRows(qx, T, K, ldqx, 1);
  rdRows(Wq, N, K, ldw, 1);
  rd(a_scale, (size_t)T * 4); rd(a_zero, (size_t)T * 4); rd(a_qsum, (size_t)T * 4);
  rd(w_scale, (size_t)N * 4); rd(w_zero, (size_t)N * 4); rd(w_sum, (size_t)N * 4);
  if (bias) rd(bias, (size_t)N * 4);
  if (residual) rdRows(residual, T, N, ldr, 2);
  if (ws) rd(reinterpret_cast<char*>(ws) + ws_bytes - 1, 1);
  if (counters) rd(counters, (size_t)n_counters * 4);
  if (status) rd(status, 4);
  wrRows(Y, T, N, ldo, out_fp32 ? 4 : 2);
  return 0;
}

int xft_gated_act(const void* gu, void* out, int T, int I, int, cudaStream_t) {
  rdRows(gu, T, 2LL * I, 2LL * I, 2);
  wrRows(out, T, I, I, 2);
  return 0;
}

// ---- routed experts: these three produce real results, the host logic and the later stand-ins depend on them
int xft_moe_route(const float* logits, int ld, int T, int E, int k, int, const float* bias, int n_group, int topk_group, float, int,
                  int, int* idx, float* w, cudaStream_t) {
  need(k >= 1 && k <= E && n_group >= 1 && topk_group >= 1 && topk_group <= n_group && E % n_group == 0, "route: bad configuration");
  rdRows(logits, T, E, ld, 4);
  if (bias) rd(bias, (size_t)E * 4);
  for (int t = 0; t < T; ++t) {
    // top k by value (first index wins ties): distinct, valid expert ids
    std::vector<int> order(E);
    for (int e = 0; e < E; ++e) order[e] = e;
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return logits[(size_t)t * ld + a] > logits[(size_t)t * ld + b]; });
    for (int j = 0; j < k; ++j) { idx[(size_t)t * k + j] = order[j]; w[(size_t)t * k + j] = 1.0f / k; }
  }
  return 0;
}

int xft_moe_plan(const int* idx, const float* w, int T, int k, int e0, int e1, int bn, int* pos, int* src_tok, float* row_w,
                 void* tiles, int* meta, int max_tiles, int max_rows, cudaStream_t) {
  int* tl = static_cast<int*>(tiles);
  int rows = 0, nt = 0;
  for (int i = 0; i < T * k; ++i) pos[i] = -1;
  for (int e = e0; e < e1; ++e) {
    const int first = rows;
    for (int t = 0; t < T; ++t)
      for (int j = 0; j < k; ++j)
        if (idx[(size_t)t * k + j] == e) {
          need(rows < max_rows, "plan: more rows than the buffers hold");
          pos[(size_t)t * k + j] = rows; src_tok[rows] = t; row_w[rows] = w[(size_t)t * k + j];
          ++rows;
        }
    for (int r = first; r < rows; r += bn) {
      need(nt < max_tiles, "plan: more tiles than the table holds");
      tl[4 * nt] = e - e0; tl[4 * nt + 1] = r; tl[4 * nt + 2] = std::min(bn, rows - r); tl[4 * nt + 3] = 0;
      ++nt;
    }
  }
  meta[0] = nt; meta[1] = rows;
  return 0;
}

int xft_moe_gather(const void* x, int ldx, const int* src_tok, const int* meta, void* xs, int max_rows, int H, cudaStream_t) {
  need(meta[1] <= max_rows, "gather: more rows than the buffer holds");
  for (int r = 0; r < meta[1]; ++r) {
    rd(static_cast<const char*>(x) + (size_t)src_tok[r] * ldx * 2, (size_t)H * 2);
    wr(static_cast<char*>(xs) + (size_t)r * H * 2, (size_t)H * 2);
  }
  return 0;
}

int xft_gemm_bf16_grouped(const void* X, int ldx, int x_rows, const void* W, int w_rows, int ldw, void* Y, int ldo, int out_fp32,
                          int N, int K, int gated, int dual_off, int group_w_rows, const void* group_tiles,
                          const int* num_group_tiles, int max_tiles, int bn, const float* col_scale, int, int* status, cudaStream_t) {
  const int* tl = static_cast<const int*>(group_tiles);
  const int nt = num_group_tiles[0];
  need(nt <= max_tiles, "grouped gemm: tile count beyond the table");
  const int rows_w = gated ? dual_off + N : N;
  for (int i = 0; i < nt; ++i) {
    const int g = tl[4 * i], r0 = tl[4 * i + 1], nr = tl[4 * i + 2];
    need(nr >= 1 && nr <= bn && r0 >= 0 && r0 + nr <= x_rows, "grouped gemm: tile outside the rows");
    need((long long)g * group_w_rows + rows_w <= w_rows, "grouped gemm: group outside the stacked weights");
    rdRows(static_cast<const char*>(X) + (size_t)r0 * ldx * 2, nr, K, ldx, 2);
    rdRows(static_cast<const char*>(W) + (size_t)g * group_w_rows * ldw * 2, rows_w, K, ldw, 2);
    if (col_scale) rd(col_scale + r0, (size_t)nr * 4);
    wrRows(static_cast<char*>(Y) + (size_t)r0 * ldo * (out_fp32 ? 4 : 2), nr, N, ldo, out_fp32 ? 4 : 2);
  }
  if (status) rd(status, 4);
  return 0;
}

int xft_moe_combine(const float* ys, const int* pos, int k, const float* add1, const void* add2, int ld2, void* y, float* y32, int T,
                    int H, cudaStream_t) {
  for (int i = 0; i < T * k; ++i) if (pos[i] >= 0) rd(ys + (size_t)pos[i] * H, (size_t)H * 4);
  if (add1) rd(add1, (size_t)T * H * 4);
  if (add2) rdRows(add2, T, H, ld2, 2);
  if (y32) wr(y32, (size_t)T * H * 4); else wrRows(y, T, H, H, 2);
  return 0;
}

// ---- latent attention
int xft_mla_prep(const void* q, int ldq, const void* kv, int ldkv, int T, int Hl, int nope, int rope, int kvl, const int* positions,
                 const float* table, int max_pos, const float* kv_norm_w, float, void* q_nope, void* q_rope, void* cache,
                 long long nslots, const int* slots, int*, int, cudaStream_t) {
  rdRows(q, T, (long long)Hl * (nope + rope), ldq, 2);
  rdRows(kv, T, kvl + rope, ldkv, 2);
  rd(kv_norm_w, (size_t)kvl * 4);
  for (int t = 0; t < T; ++t) {
    need(positions[t] >= 0 && positions[t] < max_pos, "mla_prep: position outside the table");
    rd(table + (size_t)positions[t] * rope, (size_t)rope * 4);
    need(slots[t] >= 0 && slots[t] < nslots, "mla_prep: slot outside the pool");
    wr(static_cast<char*>(cache) + (size_t)slots[t] * (kvl + rope) * 2, (size_t)(kvl + rope) * 2);
  }
  wr(q_nope, (size_t)T * Hl * nope * 2);
  wr(q_rope, (size_t)T * Hl * rope * 2);
  return 0;
}

int xft_mla_attention(const void* q_abs, long long qa_sh, long long qa_st, const void* q_rope, long long qr_sh, long long qr_st,
                      void* out, long long o_sh, long long o_st, const void* cache, const int* block_table, int bt_stride,
                      const int* cu_q, const int* kv_lens, int B, int T, int hl, int bs, int num_blocks, float, int nsplit,
                      float* part_o, float* part_ml, int* counters, int*, cudaStream_t) {
  const int L = 512, R = 64;
  need(cu_q[B] == T, "mla: token count mismatch");
  for (int h = 0; h < hl; ++h)
    for (int t = 0; t < T; ++t) {
      rd(static_cast<const char*>(q_abs) + ((size_t)h * qa_sh + (size_t)t * qa_st) * 2, (size_t)L * 2);
      rd(static_cast<const char*>(q_rope) + ((size_t)h * qr_sh + (size_t)t * qr_st) * 2, (size_t)R * 2);
      wr(static_cast<char*>(out) + ((size_t)h * o_sh + (size_t)t * o_st) * 2, (size_t)L * 2);
    }
  for (int b = 0; b < B; ++b) {
    const int nblk = (kv_lens[b] + bs - 1) / bs;
    need(nblk <= bt_stride, "mla: block table row too short");
    for (int j = 0; j < nblk; ++j) {
      const int blk = block_table[(size_t)b * bt_stride + j];
      need(blk >= 0 && blk < num_blocks, "mla: block outside the pool");
      rd(static_cast<const char*>(cache) + (size_t)blk * bs * (L + R) * 2, (size_t)bs * (L + R) * 2);
    }
  }
  if (nsplit > 1) {
    need(part_o && part_ml && counters, "mla: split launch without its scratch");
    const size_t ctas = (size_t)T * ((hl + 15) / 16);
    wr(part_o, ctas * nsplit * 16 * L * 4);
    wr(part_ml, ctas * nsplit * 32 * 4);
  }
  return 0;
}

int xft_swap_outer_dims(const void* src, void* dst, int A, int B, int D, cudaStream_t) {
  rd(src, (size_t)A * B * D * 2);
  wr(dst, (size_t)A * B * D * 2);
  return 0;
}

int xft_sum_bf16(void* dst, const void* const* srcs, int nsrc, size_t n, cudaStream_t) {
  for (int k = 0; k < nsrc; ++k) rd(srcs[k], n * 2);
  wr(dst, n * 2);
  return 0;
}
}
