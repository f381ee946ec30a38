// A host stand-in for the device side of the C++ engine, for tests WITHOUT a GPU: the CUDA runtime calls that
// csrc/core makes (memory is plain malloc'd memory) and every entry point of the kernel library the engine calls.
// The stand-in kernels do no arithmetic worth the name; what they do is TOUCH exactly the bytes the real kernels
// read and write, computed from the same arguments — every row of every operand with its stride, every KV block a
// block table names, every expert's weight rows a tile points at.  Built with AddressSanitizer and with
// XFT_ARENA_EXACT=1 (buffers get exactly the size asked for), a run of the engine over this library checks the host
// side of every family x weight type x rank count: buffer sizes, strides, block and slot arithmetic, the tensor-
// parallel ranges, the order of collectives.  Indices that the real kernels would refuse through their status word
// (a slot or block outside the pool) abort here, and so do arguments the real entry points reject: operands that are not
// aligned for a tensor map (16-byte base and row pitch), sizes and strides the kernels' vector accesses cannot take.
//
// The few results the host logic depends on are produced for real: the routing (valid expert ids), the expert plan
// (rows grouped by expert, tile table, counts) and logits that differ per row and step so that searchers move.
//
// With XFT_MOCK_MATH=1 the stand-ins of the bf16 path ALSO compute what the real kernels compute (fp32 arithmetic,
// results rounded to bf16 where the kernels round): embedding, norms, GEMMs with their epilogues, rotary + cache append,
// paged attention (grouped heads, ALiBi, prefix mask, int8 cache), routing, grouped expert GEMMs, combine, the latent-
// attention steps, the sum of the thread-rank all-reduce.  The engine's logits can then be compared, on a CPU box, with
// the PyTorch fp32 path of the package for every family, and tensor-parallel ranks with a single rank: that checks what
// the touch checks cannot — which rows of which file went where, offsets of heads and experts, position tables.  The
// load-time quantiser and the quantised GEMMs (int8 / uint4 / NF4 weight-only, int8 x int8) follow the kernels' formulas
// too, so quantised and GPTQ checkpoints are compared the same way.
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
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
// what the tensor maps of the real GEMMs need: a 16-byte aligned base and a row pitch that is a multiple of 16 bytes
void needTma(const void* p, long long ld, size_t esz, const char* what) {
  need((reinterpret_cast<uintptr_t>(p) & 15) == 0 && (ld * (long long)esz) % 16 == 0, what);
}
const uint16_t kBf16Small = 0x3c00;      // bf16 of 0.0078125: keeps activations finite and tiny

const bool g_math = [] { const char* v = std::getenv("XFT_MOCK_MATH"); return v && *v && *v != '0'; }();

inline float bf(uint16_t h) { uint32_t u = (uint32_t)h << 16; float f; std::memcpy(&f, &u, 4); return f; }
inline uint16_t tobf(float f) {           // round to nearest even, as __float2bfloat16
  uint32_t u; std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fc0;
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
inline float rbf(float f) { return bf(tobf(f)); }
inline float halfToFloat(uint16_t h) {
  const int e = (h >> 10) & 31, m = h & 1023;
  float v = e == 0 ? std::ldexp((float)m, -24) : e == 31 ? (m ? NAN : INFINITY) : std::ldexp((float)(m | 1024), e - 25);
  return (h & 0x8000) ? -v : v;
}
inline float e4m3ToFloat(uint8_t b) {
  const int e = (b >> 3) & 15, m = b & 7;
  float v = e == 0 ? std::ldexp((float)m, -9) : (e == 15 && m == 7) ? NAN : std::ldexp((float)(m | 8), e - 10);
  return (b & 0x80) ? -v : v;
}
inline float actf(float x, int act) {
  switch (act) {
    case 1: return std::max(x, 0.f);
    case 2: return x / (1.f + std::exp(-x));
    case 3: { const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x); return 0.5f * x * (1.f + std::tanh(u)); }
    default: return x;
  }
}
const float kNf4Code[16] = {-1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
                            -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
                            0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f,
                            0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};
inline const uint16_t* bfp(const void* p) { return static_cast<const uint16_t*>(p); }
inline uint16_t* bfp(void* p) { return static_cast<uint16_t*>(p); }

// acc[n] = sum_k x[k] * W[n, k] for n in [0, rows): bf16 operands, fp32 sums
void dots(const uint16_t* x, int K, const uint16_t* W, long long ldw, int rows, std::vector<float>& acc) {
  std::vector<float> xf(K);
  for (int k = 0; k < K; ++k) xf[k] = bf(x[k]);
  acc.resize(rows);
  for (int n = 0; n < rows; ++n) {
    const uint16_t* w = W + (size_t)n * ldw;
    float a = 0.f;
    for (int k = 0; k < K; ++k) a += xf[k] * bf(w[k]);
    acc[n] = a;
  }
}

}  // namespace

// ------------------------------------------------------------------------------------------------ CUDA runtime
extern "C" {
cudaError_t cudaMalloc(void** p, size_t n) { *p = std::calloc(1, n ? n : 1); return *p ? cudaSuccess : cudaErrorMemoryAllocation; }
cudaError_t cudaFree(void* p) { std::free(p); return cudaSuccess; }
cudaError_t cudaMallocHost(void** p, size_t n) { *p = std::calloc(1, n ? n : 1); return *p ? cudaSuccess : cudaErrorMemoryAllocation; }
cudaError_t cudaFreeHost(void* p) { std::free(p); return cudaSuccess; }
cudaError_t cudaMemcpy(void* d, const void* s, size_t n, cudaMemcpyKind) { if (n) std::memmove(d, s, n); return cudaSuccess; }
cudaError_t cudaMemcpyAsync(void* d, const void* s, size_t n, cudaMemcpyKind, cudaStream_t) { if (n) std::memmove(d, s, n); return cudaSuccess; }
cudaError_t cudaMemcpy2DAsync(void* d, size_t dpitch, const void* s, size_t spitch, size_t width, size_t height, cudaMemcpyKind,
                              cudaStream_t) {
  for (size_t r = 0; r < height; ++r) std::memmove(static_cast<char*>(d) + r * dpitch, static_cast<const char*>(s) + r * spitch, width);
  return cudaSuccess;
}
cudaError_t cudaMemset(void* d, int v, size_t n) { if (n) std::memset(d, v, n); return cudaSuccess; }
cudaError_t cudaMemsetAsync(void* d, int v, size_t n, cudaStream_t) { if (n) std::memset(d, v, n); return cudaSuccess; }
cudaError_t cudaStreamCreate(cudaStream_t* s) { static char token; *s = reinterpret_cast<cudaStream_t>(&token); return cudaSuccess; }
cudaError_t cudaStreamSynchronize(cudaStream_t) { return cudaSuccess; }
cudaError_t cudaStreamQuery(cudaStream_t) { return cudaSuccess; }
cudaError_t cudaDeviceSynchronize() { return cudaSuccess; }
cudaError_t cudaGetLastError() { return cudaSuccess; }
cudaError_t cudaGetDeviceCount(int* n) { *n = 1; return cudaSuccess; }
cudaError_t cudaSetDevice(int) { return cudaSuccess; }
cudaError_t cudaGetDevice(int* d) { *d = 0; return cudaSuccess; }
const char* cudaGetErrorString(cudaError_t) { return "mock device error"; }
}

// ------------------------------------------------------------------------------------------------ kernel library
extern "C" {

int xft_embedding(const int* ids, const void* table, void* out, int T, int H, int vocab, float scale, const void* pos_table,
                  const int* positions, int pos_offset, int npos, int*, cudaStream_t) {
  need(H % 8 == 0, "embedding: hidden size must be a multiple of 8");
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
  if (!g_math) return 0;
  for (int t = 0; t < T; ++t)
    for (int i = 0; i < H; ++i) {
      const uint16_t raw = bfp(table)[(size_t)ids[t] * H + i];
      if (scale == 1.f && !pos_table) { o[(size_t)t * H + i] = raw; continue; }
      float x = bf(raw) * scale;
      if (pos_table) x += bf(bfp(pos_table)[(size_t)(positions[t] + pos_offset) * H + i]);
      o[(size_t)t * H + i] = tobf(x);
    }
  return 0;
}

int xft_rmsnorm(const void* x, int ldx, const void* res, int ldr, const float* w, void* y, int ldy, void* h_out, int T, int H,
                float eps, cudaStream_t) {
  need(H % 8 == 0 && ldx % 8 == 0 && ldy % 8 == 0 && (!res || ldr % 8 == 0), "rmsnorm: sizes and strides must be multiples of 8");
  rdRows(x, T, H, ldx, 2);
  if (res) rdRows(res, T, H, ldr, 2);
  rd(w, (size_t)H * 4);
  std::vector<float> row(g_math ? H : 0);
  if (g_math)                                     // before the writes: y may alias x
    for (int t = 0; t < T; ++t) {
      float ss = 0.f;
      for (int i = 0; i < H; ++i) {
        float f = bf(bfp(x)[(size_t)t * ldx + i]);
        if (res) f = rbf(f + bf(bfp(res)[(size_t)t * ldr + i]));
        row[i] = f; ss += f * f;
      }
      const float inv = 1.f / std::sqrt(ss / H + eps);
      for (int i = 0; i < H; ++i) {
        if (res && h_out) bfp(h_out)[(size_t)t * H + i] = tobf(row[i]);
        bfp(y)[(size_t)t * ldy + i] = tobf(row[i] * inv * w[i]);
      }
    }
  else {
    wrRows(y, T, H, ldy, 2);
    if (h_out) wrRows(h_out, T, H, H, 2);
  }
  return 0;
}

int xft_layernorm(const void* x, int ldx, const float* w, const float* b, void* y, int ldy, int T, int H, float eps, cudaStream_t) {
  rdRows(x, T, H, ldx, 2);
  rd(w, (size_t)H * 4);
  rd(b, (size_t)H * 4);
  if (!g_math) { wrRows(y, T, H, ldy, 2); return 0; }
  std::vector<float> row(H);
  for (int t = 0; t < T; ++t) {
    float s = 0.f, vs = 0.f;
    for (int i = 0; i < H; ++i) { row[i] = bf(bfp(x)[(size_t)t * ldx + i]); s += row[i]; }
    const float mu = s / H;
    for (int i = 0; i < H; ++i) vs += (row[i] - mu) * (row[i] - mu);
    const float inv = 1.f / std::sqrt(vs / H + eps);
    for (int i = 0; i < H; ++i) bfp(y)[(size_t)t * ldy + i] = tobf((row[i] - mu) * inv * w[i] + b[i]);
  }
  return 0;
}

int xft_gemm_bf16(const void* X, int ldx, const void* W, int w_rows, int ldw, void* Y, int ldo, int out_fp32, int T, int N,
                  int K, int gated, int dual_off, const float* bias, const void* residual, int ldr, float res_scale, int act,
                  const float* row_scale, float* ws, size_t ws_bytes, int* counters, int n_counters, int* status, int, cudaStream_t) {
  const int rows = gated ? dual_off + N : N;
  need(w_rows >= rows, "gemm: weight has fewer rows than outputs");
  needTma(X, ldx, 2, "gemm: activations are not aligned for a tensor map");
  needTma(W, ldw, 2, "gemm: weights are not aligned for a tensor map");
  rdRows(X, T, K, ldx, 2);
  rdRows(W, rows, K, ldw, 2);
  if (bias) rd(bias, (size_t)rows * 4);
  if (residual) rdRows(residual, T, N, ldr, 2);
  if (row_scale) rd(row_scale, (size_t)N * 4);
  if (ws) { rd(ws, 1); rd(reinterpret_cast<char*>(ws) + ws_bytes - 1, 1); }
  if (counters) rd(counters, (size_t)n_counters * 4);
  if (status) rd(status, 4);
  if (g_math) {
    // y = act(acc * row_scale[n] + bias[n]) [* (acc_up + bias_up)] + res_scale * residual   (Y may alias the residual)
    std::vector<float> acc, out(N);
    for (int t = 0; t < T; ++t) {
      dots(bfp(X) + (size_t)t * ldx, K, bfp(W), ldw, rows, acc);
      for (int n = 0; n < N; ++n) {
        const float rs = row_scale ? row_scale[n] : 1.f;
        float x = actf(acc[n] * rs + (bias ? bias[n] : 0.f), act);
        if (gated) x *= acc[dual_off + n] * rs + (bias ? bias[dual_off + n] : 0.f);
        if (residual) x += res_scale * bf(bfp(residual)[(size_t)t * ldr + n]);
        out[n] = x;
      }
      for (int n = 0; n < N; ++n)
        if (out_fp32) static_cast<float*>(Y)[(size_t)t * ldo + n] = out[n];
        else bfp(Y)[(size_t)t * ldo + n] = tobf(out[n]);
    }
    return 0;
  }
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

// the split of a fused QKV row, per-head RMSNorm, rotary (one or two streams) and the paged append, as the kernel does them
static void ropeCacheMath(const void* qkv, int ldq, int T, int hq, int hkv, int D, const int* positions, const int* positions2,
                          const float* table, int rot, int style, int rot_off, const float* q_scale, const float* q_norm_w,
                          const float* k_norm_w, float eps, void* q_out, void* kc, void* vc, float* ks, float* vs, int int8_cache,
                          int bs, const int* slots) {
  std::vector<float> v(D);
  for (int t = 0; t < T; ++t)
    for (int h = 0; h < hq + 2 * hkv; ++h) {
      const uint16_t* src = bfp(qkv) + (size_t)t * ldq + (size_t)h * D;
      for (int d = 0; d < D; ++d) v[d] = bf(src[d]);
      const bool is_q = h < hq, is_k = !is_q && h < hq + hkv;
      const float* nw = is_q ? q_norm_w : is_k ? k_norm_w : nullptr;
      if (nw) {
        float ss = 0.f;
        for (int d = 0; d < D; ++d) ss += v[d] * v[d];
        const float inv = 1.f / std::sqrt(ss / D + eps);
        for (int d = 0; d < D; ++d) v[d] = rbf(v[d] * inv * nw[d]);
      }
      if ((is_q || is_k) && table && rot > 0) {
        const int half = rot / 2;
        for (int stream = 0; stream < (positions2 ? 2 : 1); ++stream) {
          const float* cs = table + (size_t)(stream ? positions2[t] : positions[t]) * rot;
          const int off = rot_off + stream * rot;
          for (int i = 0; i < half; ++i) {
            const int a = off + (style == 0 ? i : 2 * i), b = off + (style == 0 ? i + half : 2 * i + 1);
            const float x1 = v[a], x2 = v[b];
            v[a] = x1 * cs[i] - x2 * cs[half + i];
            v[b] = x2 * cs[i] + x1 * cs[half + i];
          }
        }
      }
      if (is_q) {
        const float qs = q_scale ? q_scale[t] : 1.f;
        for (int d = 0; d < D; ++d) bfp(q_out)[((size_t)t * hq + h) * D + d] = tobf(v[d] * qs);
        continue;
      }
      const int kh = is_k ? h - hq : h - hq - hkv;
      const long long blk = slots[t] / bs, off = slots[t] % bs;
      const size_t base = (size_t)(blk * hkv + kh) * bs + off;
      if (int8_cache) {
        float am = 0.f;
        for (int d = 0; d < D; ++d) am = std::max(am, std::fabs(v[d]));
        const float sc = am / 127.f, inv = sc > 1e-20f ? 1.f / sc : 0.f;
        int8_t* dst = static_cast<int8_t*>(is_k ? kc : vc) + base * D;
        for (int d = 0; d < D; ++d) dst[d] = (int8_t)std::min(std::max(std::nearbyint(v[d] * inv), -127.f), 127.f);
        (is_k ? ks : vs)[base] = sc;
      } else {
        uint16_t* dst = bfp(is_k ? kc : vc) + base * D;
        for (int d = 0; d < D; ++d) dst[d] = tobf(v[d]);
      }
    }
}

int xft_qkv_rope_cache(const void* qkv, int ldq, int T, int hq, int hkv, int D, const int* positions, const float* table, int rot,
                       int style, int rot_off, int max_pos, const float* q_scale, const float* q_norm_w, const float* k_norm_w,
                       float eps, void* q_out, void* kc, void* vc, float* ks, float* vs, int int8_cache, int bs, long long nslots,
                       const int* slots, int*, cudaStream_t) {
  need(D <= 256 && D % 2 == 0, "rope + cache: head size must be even and at most 256");
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
  if (g_math)
    ropeCacheMath(qkv, ldq, T, hq, hkv, D, positions, nullptr, table, rot, style, rot_off, q_scale, q_norm_w, k_norm_w, eps, q_out,
                  kc, vc, ks, vs, int8_cache, bs, slots);
  return 0;
}

int xft_qkv_rope2d_cache(const void* qkv, int ldq, int T, int hq, int hkv, int D, const int* positions, const int* positions2,
                         const float* table, int rot, int max_pos, void* q_out, void* kc, void* vc, float* ks, float* vs,
                         int int8_cache, int bs, long long nslots, const int* slots, int*, cudaStream_t) {
  need(2 * rot <= D && D <= 256 && D % 2 == 0 && rot > 0 && rot % 2 == 0, "two-stream rotary: bad head or rotary size");
  rdRows(qkv, T, (long long)(hq + 2 * hkv) * D, ldq, 2);
  for (int t = 0; t < T; ++t) {
    need(positions[t] >= 0 && positions[t] < max_pos && positions2[t] >= 0 && positions2[t] < max_pos, "rotary position outside the table");
    rd(table + (size_t)positions[t] * rot, (size_t)rot * 4);
    rd(table + (size_t)positions2[t] * rot, (size_t)rot * 4);
  }
  wrRows(q_out, T, (long long)hq * D, (long long)hq * D, 2);
  touchCache(kc, vc, ks, vs, int8_cache, hkv, D, bs, nslots, slots, T);
  if (g_math)
    ropeCacheMath(qkv, ldq, T, hq, hkv, D, positions, positions2, table, rot, 0, 0, nullptr, nullptr, nullptr, 0.f, q_out, kc, vc,
                  ks, vs, int8_cache, bs, slots);
  return 0;
}

int xft_paged_attention(const void* q, void* out, const void* kc, const void* vc, const float* ks, const float* vs,
                        const int* block_table, int bt_stride, const int* cu_q, const int* kv_lens, int B, int max_q, int hq,
                        int hkv, int group, int q_off, int HD, int bs, int num_blocks, float scale, const float* slopes,
                        const int* prefix_lens, int decode, int nsplit, float* part_o, float* part_ml, int* split_counters,
                        int* status, cudaStream_t) {
  need(bs % 64 == 0 && (HD == 64 || HD == 128 || HD == 256), "attention: block size must be a multiple of 64, head size 64 / 128 / 256");
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
  if (!g_math) return 0;
  std::vector<float> sc, o(HD);
  for (int b = 0; b < B; ++b) {
    const int nq = cu_q[b + 1] - cu_q[b], L = kv_lens[b], prefix = prefix_lens ? prefix_lens[b] : 0;
    for (int i = 0; i < nq; ++i)
      for (int h = 0; h < hq; ++h) {
        const int t = cu_q[b] + i, qp = L - nq + i, kvh = std::min((h + q_off) / group, hkv - 1);
        const uint16_t* qv = bfp(q) + ((size_t)t * hq + h) * HD;
        sc.assign(L, -INFINITY);
        float mx = -INFINITY;
        for (int key = 0; key < L; ++key) {
          if (!(key <= qp || key < prefix)) continue;
          const size_t row = ((size_t)block_table[(size_t)b * bt_stride + key / bs] * hkv + kvh) * bs + key % bs;
          float a = 0.f;
          if (int8) { const int8_t* kr = static_cast<const int8_t*>(kc) + row * HD; for (int d = 0; d < HD; ++d) a += bf(qv[d]) * kr[d]; a *= ks[row]; }
          else { const uint16_t* kr = bfp(kc) + row * HD; for (int d = 0; d < HD; ++d) a += bf(qv[d]) * bf(kr[d]); }
          a *= scale;
          if (slopes) a += slopes[h] * (float)(key - qp);
          sc[key] = a; mx = std::max(mx, a);
        }
        float den = 0.f;
        std::fill(o.begin(), o.end(), 0.f);
        for (int key = 0; key < L; ++key) {
          if (sc[key] == -INFINITY) continue;
          const float pw = std::exp(sc[key] - mx);
          den += pw;
          const size_t row = ((size_t)block_table[(size_t)b * bt_stride + key / bs] * hkv + kvh) * bs + key % bs;
          if (int8) { const int8_t* vr = static_cast<const int8_t*>(vc) + row * HD; for (int d = 0; d < HD; ++d) o[d] += pw * vs[row] * vr[d]; }
          else { const uint16_t* vr = bfp(vc) + row * HD; for (int d = 0; d < HD; ++d) o[d] += pw * bf(vr[d]); }
        }
        for (int d = 0; d < HD; ++d) bfp(out)[((size_t)t * hq + h) * HD + d] = tobf(o[d] / den);
      }
  }
  return 0;
}

int xft_transpose_to_bf16(const void* src, int dtype, long long ld_src, int rows, int cols, void* dst, long long ld_dst, cudaStream_t) {
  const size_t esz = dtype == 0 ? 4 : 2;
  rdRows(src, rows, cols, ld_src, esz);
  wrRows(dst, cols, rows, ld_dst, 2);
  for (int r = 0; r < rows; ++r)             // real in both modes: weights pass through here at load
    for (int c = 0; c < cols; ++c) {
      const size_t i = (size_t)r * ld_src + c;
      const float f = dtype == 0 ? static_cast<const float*>(src)[i] : dtype == 1 ? halfToFloat(bfp(src)[i]) : bf(bfp(src)[i]);
      bfp(dst)[(size_t)c * ld_dst + r] = tobf(f);
    }
  return 0;
}

int xft_fp8_block_dequant(const void* src, const float* scale, long long rows, int cols, int block, void* dst, cudaStream_t) {
  rd(src, (size_t)rows * cols);
  rd(scale, (size_t)((rows + block - 1) / block) * ((cols + block - 1) / block) * 4);
  wr(dst, (size_t)rows * cols * 2);
  const int sc_cols = (cols + block - 1) / block;
  for (long long r = 0; r < rows; ++r)
    for (int c = 0; c < cols; ++c)
      bfp(dst)[r * cols + c] = tobf(e4m3ToFloat(static_cast<const uint8_t*>(src)[r * cols + c]) * scale[(r / block) * sc_cols + c / block]);
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
  if (!g_math) return 0;
  // mode 0: int8, scale = (max - min) / 255, zero = (max + min) / 2 + scale / 2, code in [-128, 127]; mode 1: uint4,
  // scale = (max - min) / 15, zero = min; mode 2: NF4, scale = max|w|, nearest code (first on ties); low nibble first
  auto at = [&](int r, int i) {
    const size_t k = (size_t)r * ldw + i;
    return dtype == 0 ? static_cast<const float*>(w)[k] : dtype == 1 ? halfToFloat(bfp(w)[k]) : bf(bfp(w)[k]);
  };
  for (int r = 0; r < rows; ++r) {
    float mx = -INFINITY, mn = INFINITY;
    for (int i = 0; i < K; ++i) { const float v = at(r, i); mx = std::max(mx, mode == 2 ? std::fabs(v) : v); mn = std::min(mn, v); }
    float sc, zp;
    if (mode == 0) { sc = std::max((mx - mn) / 255.0f, 1e-10f); zp = (mx + mn) * 0.5f + 0.5f * sc; }
    else if (mode == 1) { sc = std::max((mx - mn) / 15.0f, 1e-10f); zp = mn; }
    else { sc = std::max(mx, 1e-10f); zp = 0.f; }
    scale[r] = sc; zero[r] = zp;
    uint8_t* dst = static_cast<uint8_t*>(q) + (size_t)r * ldq_bytes;
    if (mode == 0) {
      int acc = 0;
      for (int i = 0; i < K; ++i) {
        const int c = (int)std::min(std::max(std::nearbyint((at(r, i) - zp) / sc), -128.f), 127.f);
        reinterpret_cast<int8_t*>(dst)[i] = (int8_t)c; acc += c;
      }
      if (wsum) wsum[r] = (float)acc;
      continue;
    }
    for (int i = 0; i < K / 2; ++i) {
      int code[2];
      for (int j = 0; j < 2; ++j) {
        const float v = at(r, 2 * i + j);
        if (mode == 1) { code[j] = (int)std::min(std::max(std::nearbyint((v - zp) / sc), 0.f), 15.f); continue; }
        const float xn = v / sc;
        int best = 0; float bd = std::fabs(xn - kNf4Code[0]);
        for (int c = 1; c < 16; ++c) { const float d = std::fabs(xn - kNf4Code[c]); if (d < bd) { bd = d; best = c; } }
        code[j] = best;
      }
      dst[i] = (uint8_t)(code[0] | (code[1] << 4));
    }
  }
  return 0;
}

int xft_row_sum(const void* x, int ldx, float* out, int T, int K, cudaStream_t) {
  rdRows(x, T, K, ldx, 2);
  wr(out, (size_t)T * 4);
  if (g_math)
    for (int t = 0; t < T; ++t) { float a = 0.f; for (int i = 0; i < K; ++i) a += bf(bfp(x)[(size_t)t * ldx + i]); out[t] = a; }
  return 0;
}

int xft_quant_act(const void* x, int ldx, void* q, int ldq, float* scale, float* zero, float* qsum, int T, int K, cudaStream_t) {
  rdRows(x, T, K, ldx, 2);
  wrRows(q, T, K, ldq, 1);
  wr(scale, (size_t)T * 4); wr(zero, (size_t)T * 4); wr(qsum, (size_t)T * 4);
  if (!g_math) return 0;
  for (int t = 0; t < T; ++t) {            // zero = (min + max) / 2, scale = max|x - zero| / 127
    float mx = -INFINITY, mn = INFINITY;
    for (int i = 0; i < K; ++i) { const float v = bf(bfp(x)[(size_t)t * ldx + i]); mx = std::max(mx, v); mn = std::min(mn, v); }
    const float z = 0.5f * (mx + mn), sc = std::max(std::max(mx - z, z - mn) / 127.f, 1e-10f), inv = 1.f / sc;
    float acc = 0.f;
    for (int i = 0; i < K; ++i) {
      const float r = std::min(std::max(std::nearbyint((bf(bfp(x)[(size_t)t * ldx + i]) - z) * inv), -127.f), 127.f);
      static_cast<int8_t*>(q)[(size_t)t * ldq + i] = (int8_t)r; acc += r;
    }
    scale[t] = sc; zero[t] = z; qsum[t] = acc;
  }
  return 0;
}

int xft_qgemm(const void* X, int ldx, const void* Wq, int w_rows, int ldw_bytes, int qtype, void* Y, int ldo, int out_fp32, int T,
              int N, int K, int gated, int dual_off, const float* scale, const float* zero, const float* xsum, int, const float* bias,
              const void* residual, int ldr, float res_scale, int act, float* ws, size_t ws_bytes, int* counters, int n_counters,
              int* status, cudaStream_t) {
  const int rows = gated ? dual_off + N : N;
  need(w_rows >= rows, "qgemm: weight has fewer rows than outputs");
  need(qtype == 0 || qtype == 1 || qtype == 2, "qgemm: weight type not used by the engine");
  need(ldw_bytes % 16 == 0, "qgemm: code rows must start on 16-byte boundaries");
  needTma(X, ldx, 2, "qgemm: activations are not aligned for a tensor map");
  needTma(Wq, ldw_bytes, 1, "qgemm: codes are not aligned for a tensor map");
  rdRows(X, T, K, ldx, 2);
  rdRows(Wq, rows, qtype == 0 ? K : K / 2, ldw_bytes, 1);
  rd(scale, (size_t)rows * 4);
  if (zero) { rd(zero, (size_t)rows * 4); need(xsum != nullptr, "qgemm: zero points without activation sums"); rd(xsum, (size_t)T * 4); }
  if (bias) rd(bias, (size_t)rows * 4);
  if (residual) rdRows(residual, T, N, ldr, 2);
  if (ws) rd(reinterpret_cast<char*>(ws) + ws_bytes - 1, 1);
  if (counters) rd(counters, (size_t)n_counters * 4);
  if (status) rd(status, 4);
  if (!g_math) { wrRows(Y, T, N, ldo, out_fp32 ? 4 : 2); return 0; }
  // the codes (NF4: the code book rounded to bf16) meet bf16 activations with fp32 sums; scale and zero act on the sums:
  // y = act(scale[n] * acc + zero[n] * sum_k x + bias[n]) [* (the same for the up rows)] + res_scale * residual
  std::vector<float> wf((size_t)rows * K), xf(K), out(N);
  for (int n = 0; n < rows; ++n) {
    const uint8_t* wr_ = static_cast<const uint8_t*>(Wq) + (size_t)n * ldw_bytes;
    for (int k = 0; k < K; ++k) {
      if (qtype == 0) { wf[(size_t)n * K + k] = (float)reinterpret_cast<const int8_t*>(wr_)[k]; continue; }
      const int code = (wr_[k / 2] >> (4 * (k & 1))) & 15;
      wf[(size_t)n * K + k] = qtype == 2 ? rbf(kNf4Code[code]) : (float)code;
    }
  }
  for (int t = 0; t < T; ++t) {
    for (int k = 0; k < K; ++k) xf[k] = bf(bfp(X)[(size_t)t * ldx + k]);
    const float xs = (zero && xsum) ? xsum[t] : 0.f;
    auto dot = [&](int n) { float a = 0.f; for (int k = 0; k < K; ++k) a += xf[k] * wf[(size_t)n * K + k]; return a; };
    for (int n = 0; n < N; ++n) {
      float x = actf(dot(n) * scale[n] + (zero ? zero[n] : 0.f) * xs + (bias ? bias[n] : 0.f), act);
      if (gated) x *= dot(dual_off + n) * scale[dual_off + n] + (zero ? zero[dual_off + n] : 0.f) * xs + (bias ? bias[dual_off + n] : 0.f);
      if (residual) x += res_scale * bf(bfp(residual)[(size_t)t * ldr + n]);
      out[n] = x;
    }
    for (int n = 0; n < N; ++n)
      if (out_fp32) static_cast<float*>(Y)[(size_t)t * ldo + n] = out[n]; else bfp(Y)[(size_t)t * ldo + n] = tobf(out[n]);
  }
  return 0;
}

int xft_w8a8_gemm(const void* qx, int ldqx, const void* Wq, int ldw, void* Y, int ldo, int out_fp32, int T, int N, int K,
                  const float* a_scale, const float* a_zero, const float* a_qsum, const float* w_scale, const float* w_zero,
                  const float* w_sum, const float* bias, const void* residual, int ldr, float res_scale, int act, float* ws,
                  size_t ws_bytes, int* counters, int n_counters, int* status, cudaStream_t) {
  need(K % 16 == 0, "w8a8: K must be a multiple of 16");
  needTma(qx, ldqx, 1, "w8a8: activations are not aligned for a tensor map");
  needTma(Wq, ldw, 1, "w8a8: weights are not aligned for a tensor map");
  rdRows(qx, T, K, ldqx, 1);
  rdRows(Wq, N, K, ldw, 1);
  rd(a_scale, (size_t)T * 4); rd(a_zero, (size_t)T * 4); rd(a_qsum, (size_t)T * 4);
  rd(w_scale, (size_t)N * 4); rd(w_zero, (size_t)N * 4); rd(w_sum, (size_t)N * 4);
  if (bias) rd(bias, (size_t)N * 4);
  if (residual) rdRows(residual, T, N, ldr, 2);
  if (ws) rd(reinterpret_cast<char*>(ws) + ws_bytes - 1, 1);
  if (counters) rd(counters, (size_t)n_counters * 4);
  if (status) rd(status, 4);
  if (!g_math) { wrRows(Y, T, N, ldo, out_fp32 ? 4 : 2); return 0; }
  // y = sa * sw * acc + sa * zw * sum(qx) + za * sw * sum(qw) + K * za * zw (+ bias, activation, residual), integer sums
  std::vector<float> out(N);
  for (int t = 0; t < T; ++t) {
    const int8_t* xr = static_cast<const int8_t*>(qx) + (size_t)t * ldqx;
    for (int n = 0; n < N; ++n) {
      const int8_t* wr_ = static_cast<const int8_t*>(Wq) + (size_t)n * ldw;
      int acc = 0;
      for (int k = 0; k < K; ++k) acc += (int)xr[k] * (int)wr_[k];
      float x = a_scale[t] * w_scale[n] * (float)acc + a_scale[t] * w_zero[n] * a_qsum[t] + a_zero[t] * w_scale[n] * w_sum[n] +
                (float)K * a_zero[t] * w_zero[n] + (bias ? bias[n] : 0.f);
      x = actf(x, act);
      if (residual) x += res_scale * bf(bfp(residual)[(size_t)t * ldr + n]);
      out[n] = x;
    }
    for (int n = 0; n < N; ++n)
      if (out_fp32) static_cast<float*>(Y)[(size_t)t * ldo + n] = out[n]; else bfp(Y)[(size_t)t * ldo + n] = tobf(out[n]);
  }
  return 0;
}

int xft_gated_act(const void* gu, void* out, int T, int I, int act, cudaStream_t) {
  rdRows(gu, T, 2LL * I, 2LL * I, 2);
  wrRows(out, T, I, I, 2);
  if (g_math)
    for (int t = 0; t < T; ++t)
      for (int c = 0; c < I; ++c)
        bfp(out)[(size_t)t * I + c] = tobf(actf(bf(bfp(gu)[(size_t)t * 2 * I + c]), act) * bf(bfp(gu)[(size_t)t * 2 * I + I + c]));
  return 0;
}

// ---- routed experts: these three produce real results, the host logic and the later stand-ins depend on them
int xft_moe_route(const float* logits, int ld, int T, int E, int k, int kind, const float* bias, int n_group, int topk_group,
                  float scaling, int norm_topk, int sigmoid, int* idx, float* w, cudaStream_t) {
  need(k >= 1 && k <= E && n_group >= 1 && topk_group >= 1 && topk_group <= n_group && E % n_group == 0, "route: bad configuration");
  need(E <= 4096 && k <= 32 && n_group <= 31, "route: more experts, choices or groups than the kernel takes");
  rdRows(logits, T, E, ld, 4);
  if (bias) rd(bias, (size_t)E * 4);
  std::vector<float> score(E), sel(E);
  for (int t = 0; t < T; ++t) {
    const float* x = logits + (size_t)t * ld;
    if (!g_math) {
      // top k by value (first index wins ties): distinct, valid expert ids
      std::vector<int> order(E);
      for (int e = 0; e < E; ++e) order[e] = e;
      std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return x[a] > x[b]; });
      for (int j = 0; j < k; ++j) { idx[(size_t)t * k + j] = order[j]; w[(size_t)t * k + j] = 1.0f / k; }
      continue;
    }
    // kind 0: softmax over the k best logits; 1: softmax over all, k best, renormalised; 2: softmax or sigmoid scores,
    // selection on score + bias inside the best groups, weights from the unbiased scores
    if (kind == 0) {
      for (int e = 0; e < E; ++e) score[e] = sel[e] = x[e];
    } else {
      const bool softmax = kind == 1 || !sigmoid;
      float mx = -INFINITY, sum = 0.f;
      for (int e = 0; e < E; ++e) mx = std::max(mx, x[e]);
      for (int e = 0; e < E; ++e) { score[e] = softmax ? std::exp(x[e] - mx) : 1.f / (1.f + std::exp(-x[e])); sum += score[e]; }
      for (int e = 0; e < E; ++e) { if (softmax) score[e] /= sum; sel[e] = score[e] + ((kind == 2 && bias) ? bias[e] : 0.f); }
    }
    if (kind == 2 && n_group > 1) {
      const int gsz = E / n_group;
      std::vector<float> gs(n_group);
      for (int g = 0; g < n_group; ++g) {
        float a = -INFINITY, b = -INFINITY;
        for (int i = 0; i < gsz; ++i) { const float v = sel[g * gsz + i]; if (v > a) { b = a; a = v; } else if (v > b) b = v; }
        gs[g] = a + b;
      }
      std::vector<char> keep(n_group, 0);
      for (int j = 0; j < topk_group; ++j) {
        int bi = -1; float bv = -INFINITY;
        for (int g = 0; g < n_group; ++g) if (!keep[g] && (bi < 0 || gs[g] > bv)) { bv = gs[g]; bi = g; }
        keep[bi] = 1;
      }
      for (int e = 0; e < E; ++e) if (!keep[e / gsz]) sel[e] = -INFINITY;
    }
    float wsum = 0.f;
    for (int j = 0; j < k; ++j) {
      int bi = 0; float bv = sel[0];                      // lowest index wins ties
      for (int e = 1; e < E; ++e) if (sel[e] > bv) { bv = sel[e]; bi = e; }
      idx[(size_t)t * k + j] = bi; w[(size_t)t * k + j] = score[bi]; wsum += score[bi];
      sel[bi] = -INFINITY;
    }
    float* wt = w + (size_t)t * k;
    if (kind == 0) {
      float mx = -INFINITY, den = 0.f;
      for (int j = 0; j < k; ++j) mx = std::max(mx, wt[j]);
      for (int j = 0; j < k; ++j) den += std::exp(wt[j] - mx);
      for (int j = 0; j < k; ++j) wt[j] = std::exp(wt[j] - mx) / den;
    } else if (kind == 1) {
      if (norm_topk) for (int j = 0; j < k; ++j) wt[j] /= wsum;
    } else {
      for (int j = 0; j < k; ++j) wt[j] = (norm_topk ? wt[j] / (wsum + 1e-20f) : wt[j]) * scaling;
    }
  }
  return 0;
}

int xft_moe_plan(const int* idx, const float* w, int T, int k, int e0, int e1, int bn, int* pos, int* src_tok, float* row_w,
                 void* tiles, int* meta, int max_tiles, int max_rows, cudaStream_t) {
  need(e1 > e0 && e1 - e0 <= 256, "plan: between 1 and 256 experts per rank");
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
  need(meta[1] <= max_rows && H % 8 == 0, "gather: more rows than the buffer holds, or a hidden size that is not a multiple of 8");
  for (int r = 0; r < meta[1]; ++r) {
    rd(static_cast<const char*>(x) + (size_t)src_tok[r] * ldx * 2, (size_t)H * 2);
    wr(static_cast<char*>(xs) + (size_t)r * H * 2, (size_t)H * 2);
    std::memcpy(static_cast<char*>(xs) + (size_t)r * H * 2, static_cast<const char*>(x) + (size_t)src_tok[r] * ldx * 2, (size_t)H * 2);
  }
  return 0;
}

int xft_gemm_bf16_grouped(const void* X, int ldx, int x_rows, const void* W, int w_rows, int ldw, void* Y, int ldo, int out_fp32,
                          int N, int K, int gated, int dual_off, int group_w_rows, const void* group_tiles,
                          const int* num_group_tiles, int max_tiles, int bn, const float* col_scale, int act, int* status, cudaStream_t) {
  const int* tl = static_cast<const int*>(group_tiles);
  const int nt = num_group_tiles[0];
  need(nt <= max_tiles, "grouped gemm: tile count beyond the table");
  needTma(X, ldx, 2, "grouped gemm: activations are not aligned for a tensor map");
  needTma(W, ldw, 2, "grouped gemm: weights are not aligned for a tensor map");
  const int rows_w = gated ? dual_off + N : N;
  for (int i = 0; i < nt; ++i) {
    const int g = tl[4 * i], r0 = tl[4 * i + 1], nr = tl[4 * i + 2];
    need(nr >= 1 && nr <= bn && r0 >= 0 && r0 + nr <= x_rows, "grouped gemm: tile outside the rows");
    need((long long)g * group_w_rows + rows_w <= w_rows, "grouped gemm: group outside the stacked weights");
    rdRows(static_cast<const char*>(X) + (size_t)r0 * ldx * 2, nr, K, ldx, 2);
    rdRows(static_cast<const char*>(W) + (size_t)g * group_w_rows * ldw * 2, rows_w, K, ldw, 2);
    if (col_scale) rd(col_scale + r0, (size_t)nr * 4);
    wrRows(static_cast<char*>(Y) + (size_t)r0 * ldo * (out_fp32 ? 4 : 2), nr, N, ldo, out_fp32 ? 4 : 2);
    if (!g_math) continue;
    std::vector<float> acc;
    for (int r = r0; r < r0 + nr; ++r) {
      dots(bfp(X) + (size_t)r * ldx, K, bfp(W) + (size_t)g * group_w_rows * ldw, ldw, rows_w, acc);
      for (int n = 0; n < N; ++n) {
        float x = actf(acc[n], act);
        if (gated) x *= acc[dual_off + n];
        if (col_scale) x *= col_scale[r];
        if (out_fp32) static_cast<float*>(Y)[(size_t)r * ldo + n] = x;
        else bfp(Y)[(size_t)r * ldo + n] = tobf(x);
      }
    }
  }
  if (status) rd(status, 4);
  return 0;
}

// the same for experts kept in e4m3: bytes [w_rows, K], one fp32 scale per 128 x 128 block ([w_rows / 128, scale_ld]); a
// weight enters the product as bf16(e4m3 * scale), as in the kernel that expands tiles in shared memory
int xft_qgemm_grouped(const void* X, int ldx, int x_rows, const void* Wq, int w_rows, int ldw_bytes, void* Y, int ldo, int out_fp32,
                      int N, int K, int gated, int dual_off, int group_w_rows, const float* scale, int scale_ld,
                      const void* group_tiles, const int* num_group_tiles, int max_tiles, int bn, const float* col_scale, int act,
                      int* status, cudaStream_t) {
  static const bool report = [] {
    const char* v = std::getenv("XFT_MOCK_REPORT");          // tests ask which path ran
    if (v && *v && *v != '0') std::atexit([] { std::fprintf(stderr, "mock device: grouped e4m3 gemm ran\n"); });
    return true;
  }();
  (void)report;
  need(group_w_rows % 128 == 0 && (!gated || dual_off % 128 == 0) && K % 16 == 0, "grouped e4m3 gemm: sizes are not whole blocks");
  need(scale_ld >= (K + 127) / 128, "grouped e4m3 gemm: scale rows shorter than the blocks along K");
  needTma(X, ldx, 2, "grouped e4m3 gemm: activations are not aligned for a tensor map");
  needTma(Wq, ldw_bytes, 1, "grouped e4m3 gemm: weights are not aligned for a tensor map");
  const int* tl = static_cast<const int*>(group_tiles);
  const int nt = num_group_tiles[0];
  need(nt <= max_tiles, "grouped e4m3 gemm: tile count beyond the table");
  const int rows_w = gated ? dual_off + N : N;
  const uint8_t* W = static_cast<const uint8_t*>(Wq);
  for (int i = 0; i < nt; ++i) {
    const int g = tl[4 * i], r0 = tl[4 * i + 1], nr = tl[4 * i + 2];
    need(nr >= 1 && nr <= bn && r0 >= 0 && r0 + nr <= x_rows, "grouped e4m3 gemm: tile outside the rows");
    need((long long)g * group_w_rows + rows_w <= w_rows, "grouped e4m3 gemm: group outside the stacked weights");
    rdRows(static_cast<const char*>(X) + (size_t)r0 * ldx * 2, nr, K, ldx, 2);
    rdRows(W + (size_t)g * group_w_rows * ldw_bytes, rows_w, K, ldw_bytes, 1);
    rd(scale + (size_t)(g * group_w_rows / 128) * scale_ld, (size_t)((rows_w + 127) / 128) * scale_ld * 4);
    if (col_scale) rd(col_scale + r0, (size_t)nr * 4);
    wrRows(static_cast<char*>(Y) + (size_t)r0 * ldo * (out_fp32 ? 4 : 2), nr, N, ldo, out_fp32 ? 4 : 2);
    if (!g_math) continue;
    std::vector<float> wf((size_t)rows_w * K), xf(K);
    for (int n = 0; n < rows_w; ++n) {
      const size_t row = (size_t)g * group_w_rows + n;
      for (int k = 0; k < K; ++k) wf[(size_t)n * K + k] = rbf(e4m3ToFloat(W[row * ldw_bytes + k]) * scale[(row >> 7) * scale_ld + (k >> 7)]);
    }
    for (int r = r0; r < r0 + nr; ++r) {
      for (int k = 0; k < K; ++k) xf[k] = bf(bfp(X)[(size_t)r * ldx + k]);
      auto dot = [&](int n) { float a = 0.f; for (int k = 0; k < K; ++k) a += xf[k] * wf[(size_t)n * K + k]; return a; };
      for (int n = 0; n < N; ++n) {
        float x = actf(dot(n), act);
        if (gated) x *= dot(dual_off + n);
        if (col_scale) x *= col_scale[r];
        if (out_fp32) static_cast<float*>(Y)[(size_t)r * ldo + n] = x; else bfp(Y)[(size_t)r * ldo + n] = tobf(x);
      }
    }
  }
  if (status) rd(status, 4);
  return 0;
}

int xft_moe_combine(const float* ys, const int* pos, int k, const float* add1, const void* add2, int ld2, void* y, float* y32, int T,
                    int H, cudaStream_t) {
  for (int i = 0; i < T * k; ++i) if (pos[i] >= 0) rd(ys + (size_t)pos[i] * H, (size_t)H * 4);
  if (add1) rd(add1, (size_t)T * H * 4);
  if (add2) rdRows(add2, T, H, ld2, 2);
  if (!g_math) { if (y32) wr(y32, (size_t)T * H * 4); else wrRows(y, T, H, H, 2); return 0; }
  for (int t = 0; t < T; ++t)                     // y may alias add2: element by element
    for (int i = 0; i < H; ++i) {
      float a = 0.f;
      for (int j = 0; j < k; ++j) if (pos[(size_t)t * k + j] >= 0) a += ys[(size_t)pos[(size_t)t * k + j] * H + i];
      if (add1) a += add1[(size_t)t * H + i];
      if (add2) a += bf(bfp(add2)[(size_t)t * ld2 + i]);
      if (y32) y32[(size_t)t * H + i] = a; else bfp(y)[(size_t)t * H + i] = tobf(a);
    }
  return 0;
}

// ---- latent attention
int xft_mla_prep(const void* q, int ldq, const void* kv, int ldkv, int T, int Hl, int nope, int rope, int kvl, const int* positions,
                 const float* table, int max_pos, const float* kv_norm_w, float eps, void* q_nope, void* q_rope, void* cache,
                 long long nslots, const int* slots, int*, int nope_head_major, cudaStream_t) {
  need(Hl > 0 && rope > 0 && kvl > 0 && ((nope | rope | kvl | ldq | ldkv) & 1) == 0, "mla_prep: sizes and strides must be even");
  need(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(kv) | reinterpret_cast<uintptr_t>(q_nope) |
         reinterpret_cast<uintptr_t>(q_rope) | reinterpret_cast<uintptr_t>(cache)) & 3) == 0, "mla_prep: pointers must be 4-byte aligned");
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
  if (!g_math) return 0;
  const int half = rope / 2;
  for (int t = 0; t < T; ++t) {
    const float* cs = table + (size_t)positions[t] * rope;
    for (int h = 0; h < Hl; ++h) {
      const uint16_t* src = bfp(q) + (size_t)t * ldq + (size_t)h * (nope + rope);
      uint16_t* dn = bfp(q_nope) + (nope_head_major ? (size_t)h * T + t : (size_t)t * Hl + h) * nope;
      std::memcpy(dn, src, (size_t)nope * 2);
      uint16_t* dr = bfp(q_rope) + ((size_t)t * Hl + h) * rope;
      for (int i = 0; i < half; ++i) {
        const float x1 = bf(src[nope + 2 * i]), x2 = bf(src[nope + 2 * i + 1]);
        dr[2 * i] = tobf(x1 * cs[i] - x2 * cs[half + i]);
        dr[2 * i + 1] = tobf(x2 * cs[i] + x1 * cs[half + i]);
      }
    }
    const uint16_t* src = bfp(kv) + (size_t)t * ldkv;
    uint16_t* dst = bfp(cache) + (size_t)slots[t] * (kvl + rope);
    float ss = 0.f;
    for (int d = 0; d < kvl; ++d) ss += bf(src[d]) * bf(src[d]);
    const float inv = 1.f / std::sqrt(ss / kvl + eps);
    for (int d = 0; d < kvl; ++d) dst[d] = tobf(bf(src[d]) * inv * kv_norm_w[d]);
    for (int i = 0; i < half; ++i) {
      const float x1 = bf(src[kvl + 2 * i]), x2 = bf(src[kvl + 2 * i + 1]);
      dst[kvl + 2 * i] = tobf(x1 * cs[i] - x2 * cs[half + i]);
      dst[kvl + 2 * i + 1] = tobf(x2 * cs[i] + x1 * cs[half + i]);
    }
  }
  return 0;
}

int xft_mla_attention(const void* q_abs, long long qa_sh, long long qa_st, const void* q_rope, long long qr_sh, long long qr_st,
                      void* out, long long o_sh, long long o_st, const void* cache, const int* block_table, int bt_stride,
                      const int* cu_q, const int* kv_lens, int B, int T, int hl, int bs, int num_blocks, float scale, int nsplit,
                      float* part_o, float* part_ml, int* counters, int*, cudaStream_t) {
  const int L = 512, R = 64;
  need(cu_q[B] == T && bs % 32 == 0, "mla: token count mismatch, or a block size that is not a multiple of 32");
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
  if (!g_math) return 0;
  // S = q_abs . c_kv + q_rope . k_rope over the latent rows [c_kv (512) | k_rope (64)], causal; O = softmax(S) . c_kv
  std::vector<float> sc, o(L);
  for (int b = 0; b < B; ++b) {
    const int nq = cu_q[b + 1] - cu_q[b], len = kv_lens[b];
    for (int i = 0; i < nq; ++i)
      for (int h = 0; h < hl; ++h) {
        const int t = cu_q[b] + i, qp = len - nq + i;
        const uint16_t* qa = bfp(q_abs) + (size_t)h * qa_sh + (size_t)t * qa_st;
        const uint16_t* qr = bfp(q_rope) + (size_t)h * qr_sh + (size_t)t * qr_st;
        sc.assign(qp + 1, 0.f);
        float mx = -INFINITY;
        for (int key = 0; key <= qp; ++key) {
          const uint16_t* row = bfp(cache) + ((size_t)block_table[(size_t)b * bt_stride + key / bs] * bs + key % bs) * (L + R);
          float a = 0.f;
          for (int d = 0; d < L; ++d) a += bf(qa[d]) * bf(row[d]);
          for (int d = 0; d < R; ++d) a += bf(qr[d]) * bf(row[L + d]);
          sc[key] = a * scale; mx = std::max(mx, sc[key]);
        }
        float den = 0.f;
        std::fill(o.begin(), o.end(), 0.f);
        for (int key = 0; key <= qp; ++key) {
          const uint16_t* row = bfp(cache) + ((size_t)block_table[(size_t)b * bt_stride + key / bs] * bs + key % bs) * (L + R);
          const float pw = std::exp(sc[key] - mx);
          den += pw;
          for (int d = 0; d < L; ++d) o[d] += pw * bf(row[d]);
        }
        uint16_t* dst = bfp(out) + (size_t)h * o_sh + (size_t)t * o_st;
        for (int d = 0; d < L; ++d) dst[d] = tobf(o[d] / den);
      }
  }
  return 0;
}

int xft_swap_outer_dims(const void* src, void* dst, int A, int B, int D, cudaStream_t) {
  rd(src, (size_t)A * B * D * 2);
  wr(dst, (size_t)A * B * D * 2);
  for (int a = 0; a < A; ++a)
    for (int b = 0; b < B; ++b)
      std::memcpy(bfp(dst) + ((size_t)b * A + a) * D, bfp(src) + ((size_t)a * B + b) * D, (size_t)D * 2);
  return 0;
}

int xft_sum_bf16(void* dst, const void* const* srcs, int nsrc, size_t n, cudaStream_t) {
  for (int k = 0; k < nsrc; ++k) rd(srcs[k], n * 2);
  if (!g_math) { wr(dst, n * 2); return 0; }
  for (size_t i = 0; i < n; ++i) {                // dst may be one of the sources
    float a = 0.f;
    for (int k = 0; k < nsrc; ++k) a += bf(bfp(srcs[k])[i]);
    bfp(dst)[i] = tobf(a);
  }
  return 0;
}
}
