// C ABI over the host-side runtime so that Python (ctypes) and tests can drive the C++ twins of the layout
// arithmetic, the block allocator and the samplers without a GPU.
#include <algorithm>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "arena.h"
#include "comm.h"
#include "beam.h"
#include "bpe_tokenizer.h"
#include "dtypes.h"
#include "env.h"
#include "gptq.h"
#include "rope_tables.h"
#include "runtime.h"
#include "tokenizer.h"
#include "xft/layers.h"

using namespace xft;

extern "C" {

void xftc_task_range(int n, int splits, int idx, int* out2) { auto r = taskRange(n, splits, idx); out2[0] = r.first; out2[1] = r.second; }
void xftc_head_range(int q, int kv, int splits, int idx, int* out4) { auto r = headRange(q, kv, splits, idx); out4[0] = r.q0; out4[1] = r.q1; out4[2] = r.kv0; out4[3] = r.kv1; }

void xftc_pp_layer_range(int layers, int pp, int rank, int* out2) { auto r = ppLayerRange(layers, pp, rank); out2[0] = r.first; out2[1] = r.second; }
int xftc_moe_slice_index(int tpRank, int tpSize, int layer, int expert, int dim) { return moeSliceIndex(tpRank, tpSize, layer, expert, dim); }
void xftc_expert_range(int experts, int ep, int rank, int* out2) { auto r = expertRange(experts, ep, rank); out2[0] = r.first; out2[1] = r.second; }
int xftc_expert_owner(int expert, int experts, int ep) { return expertOwner(expert, experts, ep); }
int xftc_block_visit_order(int blocks, int world, int rank, int lag, int* out) {
  auto v = blockVisitOrder(blocks, world, rank, lag);
  std::memcpy(out, v.data(), v.size() * sizeof(int));
  return (int)v.size();
}

void* xftc_tables_new(int blockSize, int numBlocks) { return new BlockTables(blockSize, numBlocks); }
void xftc_tables_delete(void* t) { delete static_cast<BlockTables*>(t); }
int xftc_tables_add(void* t, int seq) { try { static_cast<BlockTables*>(t)->add(seq); return 0; } catch (...) { return -1; } }
void xftc_tables_free(void* t, int seq) { static_cast<BlockTables*>(t)->free(seq); }
int xftc_tables_fork(void* t, int src, int dst) { try { static_cast<BlockTables*>(t)->fork(src, dst); return 0; } catch (...) { return -1; } }
// returns number of slots written, -1 on exhaustion; cow_pairs receives (src,dst) of a block split (or -1,-1)
int xftc_tables_append(void* t, int seq, int n, int* slots, int* cow_pairs) {
  try {
    cow_pairs[0] = cow_pairs[1] = -1;
    auto s = static_cast<BlockTables*>(t)->append(seq, n, [&](int a, int b) { cow_pairs[0] = a; cow_pairs[1] = b; });
    std::memcpy(slots, s.data(), s.size() * sizeof(int));
    return (int)s.size();
  } catch (...) { return -1; }
}
int xftc_tables_table(void* t, int seq, int* out, int cap) {
  try {
    auto& v = static_cast<BlockTables*>(t)->table(seq);
    int n = (int)v.size() < cap ? (int)v.size() : cap;
    std::memcpy(out, v.data(), n * sizeof(int));
    return (int)v.size();
  } catch (...) { return -1; }
}
int xftc_tables_len(void* t, int seq) { try { return static_cast<BlockTables*>(t)->len(seq); } catch (...) { return -1; } }
int xftc_tables_truncate(void* t, int seq, int newLen) { try { static_cast<BlockTables*>(t)->truncate(seq, newLen); return 0; } catch (...) { return -1; } }
int xftc_tables_refs(void* t, int block) { return static_cast<BlockTables*>(t)->allocator().refs(block); }
int xftc_tables_num_free(void* t) { return static_cast<BlockTables*>(t)->allocator().numFree(); }
void xftc_tables_grow(void* t, int total) { static_cast<BlockTables*>(t)->allocator().grow(total); }
int xftc_tables_reorder(void* t, const int* seqs, const int* src, int n) {
  try { static_cast<BlockTables*>(t)->reorder(std::vector<int>(seqs, seqs + n), std::vector<int>(src, src + n)); return 0; } catch (...) { return -1; }
}

int xftc_argmax(const float* l, int n) { return argmaxFirst(l, n); }
int xftc_sample(const float* l, int n, int k, float p, float temp, float u) { return sampleTopKTopP(l, n, k, p, temp, u); }
void xftc_repetition_penalty(float* l, int n, const int* toks, int nt, float pen, int off) {
  repetitionPenalty(l, n, std::vector<int32_t>(toks, toks + nt), pen, off);
}


// ---- beam search scorer (csrc/core/beam.cc)
void* xftc_beam_new(int batch, int beams, float lenPenalty, int earlyStopping, int eos, int pad, int nret) {
  return new BeamSearchScorer(batch, beams, lenPenalty, earlyStopping != 0, eos, pad, nret);
}
void xftc_beam_set_prompt_lens(void* s, const int* lens, int n) {
  static_cast<BeamSearchScorer*>(s)->setPromptLens(std::vector<int>(lens, lens + n));
}
void xftc_beam_delete(void* s) { delete static_cast<BeamSearchScorer*>(s); }
int xftc_beam_done(void* s) { return static_cast<BeamSearchScorer*>(s)->isDone() ? 1 : 0; }
void xftc_beam_process(void* s, const float* logprobs, int vocab, int32_t* tokens, int* src, int n) {
  std::vector<int32_t> t; std::vector<int> b;
  static_cast<BeamSearchScorer*>(s)->process(logprobs, vocab, t, b);
  for (int i = 0; i < n && i < (int)t.size(); ++i) { tokens[i] = t[i]; src[i] = b[i]; }
}
// prompts: [batch, promptLen] row-major; out: [rows, width] written up to cap ints; returns rows * 65536 + width
int xftc_beam_finalize(void* s, const int32_t* prompts, int batch, int promptLen, int maxLength, int32_t* out, int cap) {
  std::vector<std::vector<int32_t>> p(batch);
  for (int b = 0; b < batch; ++b) p[b].assign(prompts + (size_t)b * promptLen, prompts + (size_t)(b + 1) * promptLen);
  auto res = static_cast<BeamSearchScorer*>(s)->finalize(p, maxLength);
  const int rows = (int)res.size(), width = rows ? (int)res[0].size() : 0;
  for (int r = 0; r < rows; ++r)
    for (int c = 0; c < width; ++c)
      if ((size_t)r * width + c < (size_t)cap) out[(size_t)r * width + c] = res[r][c];
  return rows * 65536 + width;
}
void xftc_log_softmax(float* row, int n) { logSoftmaxRow(row, n); }
// host-side numeric conversions (csrc/core/dtypes.h): kind 1 = fp16, 2 = bf16
void xftc_convert_from_float(const float* in, uint16_t* out, int n, int kind) {
  for (int i = 0; i < n; ++i) out[i] = kind == 1 ? floatToHalf(in[i]) : floatToBf16(in[i]);
}
void xftc_convert_to_float(const uint16_t* in, float* out, int n, int kind) {
  for (int i = 0; i < n; ++i) out[i] = kind == 1 ? halfToFloat(in[i]) : bf16ToFloat(in[i]);
}

// ---- position tables (csrc/core/rope_tables.cc).  scaling: 0 none, 1 linear, 2 yarn; table_scale < 0 = default
void xftc_rope_table(int max_pos, int rot_dim, double theta, int scaling, double factor, int original_max_pos,
                     double beta_fast, double beta_slow, double mscale, double mscale_all_dim, double table_scale,
                     float* out) {
  RopeScaling s;
  s.type = scaling == 1 ? "linear" : scaling == 2 ? "yarn" : "";
  s.factor = factor; s.originalMaxPos = original_max_pos; s.betaFast = beta_fast; s.betaSlow = beta_slow;
  s.mscale = mscale; s.mscaleAllDim = mscale_all_dim; s.tableScale = table_scale;
  auto t = ropeTable(max_pos, rot_dim, theta, s);
  std::memcpy(out, t.data(), t.size() * sizeof(float));
}
double xftc_telechat_ntk_theta(double theta, int rot_dim, int kv_len, int train_len) { return telechatNtkTheta(theta, rot_dim, kv_len, train_len); }
double xftc_telechat_mscale(int input_len, int train_len) { return telechatMscale(input_len, train_len); }
double xftc_qwen_ntk_theta(double theta, int rot_dim, int max_kv, int seq_len) { return qwenNtkTheta(theta, rot_dim, max_kv, seq_len); }
void xftc_alibi_slopes(int n_heads, float* out) { auto v = alibiSlopes(n_heads); std::memcpy(out, v.data(), v.size() * sizeof(float)); }

// ---- byte-level BPE tokenizer (csrc/core/bpe_tokenizer.cc); errors come back as a null handle + message
static thread_local std::string g_bpeError;
void* xftc_bpe_load(const char* path) {
  try { return new BpeTokenizer(path); } catch (const std::exception& e) { g_bpeError = e.what(); return nullptr; }
}
const char* xftc_bpe_error() { return g_bpeError.c_str(); }
void xftc_bpe_free(void* h) { delete static_cast<BpeTokenizer*>(h); }
int xftc_bpe_vocab_size(void* h) { return static_cast<BpeTokenizer*>(h)->vocabSize(); }
const char* xftc_bpe_pattern(void* h) { return static_cast<BpeTokenizer*>(h)->pattern(); }
int xftc_bpe_special_id(void* h, const char* text) { return static_cast<BpeTokenizer*>(h)->specialId(text); }
int xftc_bpe_encode(void* h, const char* text, int* out, int cap) {
  auto ids = static_cast<BpeTokenizer*>(h)->encode(text);
  for (int i = 0; i < (int)ids.size() && i < cap; ++i) out[i] = ids[i];
  return (int)ids.size();
}
int xftc_bpe_decode(void* h, const int* ids, int n, char* out, int cap) {
  std::string s = static_cast<BpeTokenizer*>(h)->decode(std::vector<int32_t>(ids, ids + n));
  const int m = std::min((int)s.size(), cap - 1);
  if (cap > 0) { std::memcpy(out, s.data(), m); out[m] = 0; }
  return (int)s.size();
}

// ---- GPTQ tensor repacking (csrc/core/gptq.cc)
void xftc_gptq_repack(const void* file, int in_f, int out_f, int uint4, int in0, int in1, int out0, int out1, int pitch, void* dst) {
  gptqRepack((const uint8_t*)file, in_f, out_f, uint4 != 0, in0, in1, out0, out1, pitch, (uint8_t*)dst);
}
void xftc_gptq_dequant(const void* file, int in_f, int out_f, int uint4, int in0, int in1, int out0, int out1, const float* scale,
                       const float* zero, float* dst) {
  gptqDequant((const uint8_t*)file, in_f, out_f, uint4 != 0, in0, in1, out0, out1, scale, zero, dst);
}
void xftc_gptq_row_sums(const void* file, int in_f, int out_f, int uint4, int in0, int in1, int out0, int out1, float* dst) {
  gptqRowSums((const uint8_t*)file, in_f, out_f, uint4 != 0, in0, in1, out0, out1, dst);
}

// ---- weight-type names (csrc/api/xft/dtype.h) and the launcher's rank variables (csrc/core/comm.cc)
int xftc_dtype_from_name(const char* name) { return (int)dataTypeFromName(name); }
void xftc_rank_from_env(int* rank, int* world) { auto rw = rankFromEnv(); *rank = rw.first; *world = rw.second; }

// ---- caching arena (csrc/core/arena.cc) over malloc/free, for tests without a GPU
void* xftc_arena_new_host() { return new Arena([](size_t n) { return std::malloc(n); }, [](void* p) { std::free(p); }); }
void xftc_arena_delete(void* a) { delete static_cast<Arena*>(a); }
void* xftc_arena_alloc(void* a, size_t n) { return static_cast<Arena*>(a)->allocate(n); }
void xftc_arena_release(void* a, void* p) { static_cast<Arena*>(a)->release(p); }
void xftc_arena_trim(void* a) { static_cast<Arena*>(a)->trim(); }
size_t xftc_arena_stat(void* a, int what) {
  Arena* ar = static_cast<Arena*>(a);
  return what == 0 ? ar->bytesInUse() : what == 1 ? ar->bytesCached() : ar->backendCalls();
}
size_t xftc_arena_round(size_t n) { return Arena::roundUp(n); }

// ---- environment flags and the timeline (csrc/core/env.cc)
void xftc_env_reload() { Env::get().reload(); }
int xftc_env_int(const char* name) {
  const Env& e = Env::get();
  const std::string n(name);
  if (n == "verbose") return e.verbose;
  if (n == "pipeline_stage") return e.pipelineStage;
  if (n == "fake_model") return e.fakeModel;
  if (n == "timeline") return e.timeline ? 1 : 0;
  if (n == "kv_block_size") return e.kvBlockSize;
  if (n == "cuda_graph") return e.cudaGraph ? 1 : 0;
  if (n == "max_batch_tokens") return e.maxBatchTokens;
  if (n == "attn_splits") return e.attnSplits;
  if (n == "whitelist_size") return (int)e.timelineWhitelist.size();
  return -1;
}
void xftc_timeline_enable(int on) { TimeLine::enable(on != 0); }
void xftc_timeline_scope(const char* name, int spin_us) {
  TimeLine t(name);
  const auto t0 = std::chrono::steady_clock::now();
  while (std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count() < spin_us) {}
}
int xftc_timeline_pending() { return (int)TimeLine::pending(); }
int xftc_timeline_dump(const char* path, char* out, int cap) {
  const std::string f = TimeLine::dump(path ? path : "");
  if (out && cap > 0) { std::strncpy(out, f.c_str(), cap - 1); out[cap - 1] = 0; }
  return (int)f.size();
}

// ---- the stateful layer API (csrc/core/layer_objects.cc) on device pointers, stream 0
int xftc_layer_llama(int batch, int seq, int headDim, int heads, int kvHeads, int maxPos, int past, int hidden, int inter,
                     void* out, const void* in, const float* ln1, const void* qW, const void* kW, const void* vW,
                     const void* oW, const float* ln2, const void* gate, const void* up, const void* down) {
  return xft::invokeLayerLLaMA(xft::DataType::bf16, xft::SILU, xft::RMS, batch, seq, headDim, heads, kvHeads, maxPos, maxPos,
                               past, past + seq, past == 0 ? 0 : 1, hidden, inter, out, hidden, in, hidden, ln1, nullptr, qW,
                               kW, vW, oW, ln2, nullptr, gate, up, down);
}
int xftc_attention_llama(int batch, int seq, int headDim, int heads, int kvHeads, int maxPos, int past, int hidden, void* out,
                         const void* in, const void* qW, const void* kW, const void* vW, const void* oW) {
  return xft::invokeAttentionLLaMA(xft::DataType::bf16, batch, seq, headDim, heads, kvHeads, maxPos, maxPos, past, past + seq,
                                   past == 0 ? 0 : 1, hidden, out, hidden, in, hidden, qW, kW, vW, oW);
}
void* xftc_dsmoe_create(int E, int k, int hidden, int inter, int normTopK, int nGroup, int topkGroup, const void* gateUp,
                        const void* down, const void* guScales, const void* dnScales, const void* bias, int block, int rank,
                        int world, float scaling) {
  return xft::createDeepSeekMoE(0, E, k, hidden, inter, normTopK != 0, nGroup, topkGroup, gateUp, down, guScales, dnScales, bias,
                                block, rank, world, scaling);
}
int xftc_dsmoe_forward_logits(void* moe, void* in, void* out, int T, void* logits) {
  return xft::forwardDeepSeekMoE(moe, in, out, T, logits);
}
int xftc_dsmoe_forward_selected(void* moe, void* in, void* out, int T, int* idx, float* w) {
  return xft::forwardDeepSeekMoE(moe, in, out, T, idx, w);
}
void xftc_dsmoe_destroy(void* moe) { xft::destroyDeepSeekMoE(moe); }

// ---- SentencePiece model reader (csrc/core/tokenizer.h): handle-based wrappers for tests and bindings
void* xftc_tok_load(const char* path) {
  try { return new xft::SentencePieceTokenizer(path); } catch (const std::exception&) { return nullptr; }
}
void xftc_tok_free(void* h) { delete static_cast<xft::SentencePieceTokenizer*>(h); }
int xftc_tok_info(void* h, int what) {
  auto* t = static_cast<xft::SentencePieceTokenizer*>(h);
  switch (what) { case 0: return t->vocabSize(); case 1: return t->bosId(); case 2: return t->eosId(); case 3: return t->unkId(); default: return t->isBpe() ? 1 : 0; }
}
int xftc_tok_encode(void* h, const char* text, int add_bos, int add_eos, int* out, int cap) {
  const std::vector<int32_t> ids = static_cast<xft::SentencePieceTokenizer*>(h)->encode(text, add_bos != 0, add_eos != 0);
  for (int i = 0; i < (int)ids.size() && i < cap; ++i) out[i] = ids[i];
  return (int)ids.size();
}
int xftc_tok_decode(void* h, const int* ids, int n, char* out, int cap) {
  const std::string s = static_cast<xft::SentencePieceTokenizer*>(h)->decode(std::vector<int32_t>(ids, ids + n));
  const int m = (int)s.size() < cap - 1 ? (int)s.size() : cap - 1;
  if (cap > 0) { std::memcpy(out, s.data(), m); out[m] = 0; }
  return (int)s.size();
}
int xftc_invoke_moe_deepseek(int T, int hidden, int inter, int moeInter, int nShared, int nRouted, void* out, const void* in,
                             const void* gatingW, const float* gatingBias, const void* gate, const void* up, const void* down) {
  return xft::invokeMoEDeepSeek(xft::DataType::bf16, xft::SILU, T, hidden, inter, moeInter, nShared, nRouted, out, 0, in, 0,
                                gatingW, gatingBias, gate, up, down);
}
}  // extern "C"
