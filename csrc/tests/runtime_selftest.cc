// Native unit tests of the host-side C++ runtime (the counterpart of the reference's gtest programs under tests/ut:
// kv_reorder_test.cpp, small_gemm_test.cpp, ... — here for the parts that need no device: layout maths, sequences,
// the ref-counted block allocator and block tables, samplers, the beam scorer, the INI reader, Env / TimeLine and the
// arena).  Built by `python csrc/build.py --selftest` with -fsanitize=address,undefined so that every run is also a
// memory-error and undefined-behaviour check of the runtime; exits non-zero on the first failed expectation.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <numeric>
#include <set>
#include <stdexcept>
#include <string>
#include <vector>

#include "arena.h"
#include "beam.h"
#include "bpe_tokenizer.h"
#include "dtypes.h"
#include "env.h"
#include "gptq.h"
#include "ini.h"
#include "rope_tables.h"
#include "runtime.h"

static int g_failed = 0, g_checks = 0;
#define EXPECT(cond)                                                                      \
  do {                                                                                    \
    ++g_checks;                                                                           \
    if (!(cond)) { ++g_failed; std::fprintf(stderr, "%s:%d: EXPECT(%s) failed\n", __FILE__, __LINE__, #cond); } \
  } while (0)

using namespace xft;

static void testPartition() {
  // every split of n covers [0, n) exactly once, in order; sizes differ by at most one granule (64, 16, 2 or 1)
  for (int n : {1, 7, 64, 100, 11008}) {
    for (int splits : {1, 2, 3, 8}) {
      int next = 0, lo = 1 << 30, hi = 0;
      for (int i = 0; i < splits; ++i) {
        auto r = taskRange(n, splits, i);
        EXPECT(r.first == next && r.second >= r.first);
        next = r.second;
        lo = std::min(lo, r.second - r.first);
        hi = std::max(hi, r.second - r.first);
      }
      EXPECT(next == n && hi - lo <= 64);
      if (n % 2) EXPECT(hi - lo <= 1);
    }
  }
  for (int gran : {16, 64, 128}) {
    int next = 0;
    for (int i = 0; i < 4; ++i) {
      auto r = taskRangeGran(11008, gran, 4, i);
      EXPECT(r.first == next && (r.first % gran == 0));
      next = r.second;
    }
    EXPECT(next == 11008);
  }
  // grouped-query heads: kv heads split first, q heads follow their group; more ranks than kv heads replicate
  auto h = headRange(64, 8, 8, 3);
  EXPECT(h.kv1 - h.kv0 == 1 && h.q1 - h.q0 == 8 && h.q0 == h.kv0 * 8);
  auto m = headRange(32, 2, 4, 3);       // 4 ranks, 2 kv heads: ranks 2,3 share kv head 1
  EXPECT(m.kv0 == 1 && m.kv1 == 2 && m.q1 - m.q0 == 8 && m.q0 == 24);
}

static void testSequences() {
  SequencePool pool;
  auto& a = pool.create({1, 2, 3}, 16);
  const int ida = a.id;
  auto& b = pool.create({4, 5}, 8);
  EXPECT(b.id != ida && pool.has(ida) && pool.has(b.id));
  auto& s = pool.get(ida);
  EXPECT(s.totalLen() == 3 && s.pastLen == 0);
  s.pending = s.prompt;
  s.stepForward(9);
  EXPECT(s.pastLen == 3 && s.pending.size() == 1 && s.pending[0] == 9 && s.totalLen() == 4);
  s.stepForward(10);
  EXPECT(s.pastLen == 4 && s.generated.size() == 2);
  pool.remove(ida);
  EXPECT(!pool.has(ida));
  bool threw = false;
  try { pool.get(ida); } catch (const std::exception&) { threw = true; }
  EXPECT(threw);
}

static void testBlockTables() {
  BlockAllocator al(4);
  EXPECT(al.numFree() == 4);
  int b0 = al.alloc(), b1 = al.alloc();
  EXPECT(b0 != b1 && al.numFree() == 2);
  al.share(b0);
  al.release(b0);
  EXPECT(al.numFree() == 2 && al.refs(b0) == 1);
  al.release(b0);
  EXPECT(al.numFree() == 3);
  al.grow(8);
  EXPECT(al.numBlocks() == 8 && al.numFree() == 7);
  al.release(b1);

  BlockTables t(4, 16);
  int copies = 0;
  auto cow = [&](int, int) { ++copies; };
  t.add(1);
  auto s = t.append(1, 6, cow);                  // two blocks, positions 0..5
  EXPECT(s.size() == 6 && t.table(1).size() == 2 && t.len(1) == 6);
  for (int p = 0; p < 6; ++p) EXPECT(s[p] == t.table(1)[p / 4] * 4 + p % 4);
  t.fork(1, 2);                                  // shares both blocks
  EXPECT(t.table(2) == t.table(1) && t.allocator().refs(t.table(1)[1]) == 2);
  auto s2 = t.append(2, 1, cow);                 // tail block is shared and partly filled: copy on write
  EXPECT(copies == 1 && t.table(2)[0] == t.table(1)[0] && t.table(2)[1] != t.table(1)[1]);
  EXPECT(s2[0] == t.table(2)[1] * 4 + 2 && t.len(2) == 7 && t.len(1) == 6);
  t.truncate(2, 3);                              // drops the private tail block
  EXPECT(t.table(2).size() == 1 && t.len(2) == 3);
  // reorder: beams 1 and 2 both continue from beam 2
  t.reorder({1, 2}, {1, 1});
  EXPECT(t.table(1) == t.table(2) && t.len(1) == 3);
  const int freeBefore = t.allocator().numFree();
  t.free(1);
  EXPECT(t.allocator().numFree() == freeBefore);  // still referenced by sequence 2
  t.free(2);
  EXPECT(t.allocator().numFree() == 16);
}

static void testSamplers() {
  std::vector<float> l = {0.5f, -1.0f, 2.0f, 2.0f, -3.0f};
  EXPECT(argmaxFirst(l.data(), 5) == 2);                     // first of equal maxima
  std::vector<float> r = l;
  repetitionPenalty(r.data(), 5, {1, 2, 2, 9}, 2.0f);        // distinct ids; id 9 is outside the slice
  EXPECT(r[1] == -2.0f && r[2] == 1.0f && r[0] == 0.5f && r[3] == 2.0f);
  std::vector<float> r2 = l;
  repetitionPenalty(r2.data(), 5, {10, 12}, 2.0f, 10);       // vocabulary slice starting at id 10
  EXPECT(r2[0] == 0.25f && r2[2] == 1.0f && r2[1] == -1.0f);
  EXPECT(matchStopWords({5, 6, 7}, {{6, 7}}) && !matchStopWords({5, 6, 7}, {{5, 6}}) && !matchStopWords({7}, {{6, 7}}));
  auto sw = cleanStopWords({{}, {2}, {3, 4}, {0, 5}, {2, 6}}, 2);   // empty, a lone eos and ids <= 0 are dropped
  EXPECT(sw.size() == 2 && sw[0] == std::vector<int>({3, 4}) && sw[1] == std::vector<int>({2, 6}));
  // top-k = 1 is greedy whatever u is; top-p keeps at least two candidates; the inverse CDF is monotone in u
  for (float u : {0.0f, 0.3f, 0.999f}) EXPECT(sampleTopKTopP(l.data(), 5, 1, 1.0f, 1.0f, u) == 2);
  std::vector<float> peaked = {10.f, 0.f, -1.f, -2.f};
  std::set<int> seen;
  for (int i = 0; i < 100; ++i) seen.insert(sampleTopKTopP(peaked.data(), 4, 4, 0.01f, 1.0f, i / 100.0f));
  EXPECT(seen.count(0) == 1 && seen.size() <= 2 && seen.count(2) == 0 && seen.count(3) == 0);
  int prev = -1;
  std::vector<float> flat = {1.f, 1.f, 1.f, 1.f};
  std::vector<int> order;
  for (int i = 0; i < 8; ++i) order.push_back(sampleTopKTopP(flat.data(), 4, 4, 1.0f, 1.0f, (i + 0.5f) / 8.0f));
  std::set<int> all(order.begin(), order.end());
  EXPECT(all.size() == 4);                                   // uniform logits: every id is reachable
  (void)prev;
}

static void testBeams() {
  std::vector<float> row = {1.f, 2.f, 3.f};
  logSoftmaxRow(row.data(), 3);
  double s = 0;
  for (float v : row) s += std::exp((double)v);
  EXPECT(std::fabs(s - 1.0) < 1e-5 && row[2] > row[1] && row[1] > row[0]);

  BeamHypotheses h(2, 1.0f, false);
  h.add({1, 2}, -1.0, 2);
  h.add({3}, -3.0, 1);
  h.add({4, 5, 6}, -1.5, 3);                  // -0.5 per token beats -3.0: the worst one is evicted
  EXPECT(h.beams().size() == 2);
  for (auto& b : h.beams()) EXPECT(b.second != std::vector<int32_t>({3}));
  EXPECT(!h.isDone(-0.1, 4) && h.isDone(-100.0, 4));

  // one request, two beams, vocabulary of 4 with eos = 3.  Step 1: only beam 0 is live (the scorer masks the clones).
  const int V = 4;
  BeamSearchScorer sc(1, 2, 1.0f, false, 3, 0, 1);
  std::vector<float> lp(2 * V);
  auto fill = [&](std::vector<float> a, std::vector<float> b) {
    for (int i = 0; i < V; ++i) { lp[i] = a[i]; lp[V + i] = b[i]; }
    logSoftmaxRow(lp.data(), V);
    logSoftmaxRow(lp.data() + V, V);
  };
  std::vector<int32_t> tok;
  std::vector<int> src;
  fill({0.f, 3.f, 2.f, -5.f}, {0.f, 3.f, 2.f, -5.f});
  sc.process(lp.data(), V, tok, src);
  EXPECT(tok.size() == 2 && src.size() == 2);
  EXPECT(tok[0] == 1 && tok[1] == 2 && src[0] == 0 && src[1] == 0);      // the two best continuations of beam 0
  // Step 2: beam 0 wants eos most; the hypothesis is banked and the live beams continue with the next best tokens
  fill({-5.f, 0.f, 0.5f, 4.f}, {1.f, 0.f, -1.f, -6.f});
  sc.process(lp.data(), V, tok, src);
  EXPECT(tok.size() == 2);
  for (int t : tok) EXPECT(t != 3);
  EXPECT(!sc.isDone() || true);
  auto out = sc.finalize({{7, 8}}, 6);
  EXPECT(out.size() == 1 && out[0].size() >= 3 && out[0][0] == 7 && out[0][1] == 8);
  EXPECT(out[0][2] == 1);                                               // the banked hypothesis started with token 1
}

static void testIni(const std::string& dir) {
  const std::string path = dir + "/config.ini";
  {
    std::ofstream f(path);
    f << "; comment\n[llama]\nmodel_name = tiny\nHead_Num = 4\n  size_per_head=8 \nlayernorm_eps = 1e-6\n"
         "do_qk_norm = true\n# another\n[other]\nx = 1\n";
  }
  Ini ini(path);
  EXPECT(ini.ok() && ini.sections().size() == 2 && ini.sections()[0] == "llama");
  EXPECT(ini.getInt("llama", "head_num") == 4 && ini.getInt("llama", "SIZE_PER_HEAD") == 8);
  EXPECT(std::fabs(ini.getFloat("llama", "layernorm_eps") - 1e-6) < 1e-12);
  EXPECT(ini.getBool("llama", "do_qk_norm") && !ini.getBool("llama", "missing", false));
  EXPECT(ini.get("llama", "model_name") == "tiny" && ini.get("llama", "nope", "dflt") == "dflt");
  EXPECT(ini.has("other", "x") && !ini.has("other", "y"));
  Ini missing(dir + "/does_not_exist.ini");
  EXPECT(!missing.ok());
}

static void testEnvAndTimeline(const std::string& dir) {
  setenv("XFT_VERBOSE", "2", 1);
  setenv("XFT_PIPELINE_STAGE", "2", 1);
  setenv("XFT_TIMELINE_WHITELIST", "A, C", 1);
  setenv("XFT_KV_CACHE_GB", "1.5", 1);
  setenv("XFT_CUDA_GRAPH", "0", 1);
  Env::get().reload();
  Env& e = Env::get();
  EXPECT(e.verbose == 2 && e.pipelineStage == 2 && !e.cudaGraph && std::fabs(e.kvCacheGb - 1.5) < 1e-9);
  EXPECT(e.timelineWhitelist.count("A") == 1 && e.timelineWhitelist.count("C") == 1 && e.timelineWhitelist.size() == 2);
  TimeLine::enable(true);
  { TimeLine a("A"); TimeLine b("B"); }          // B is filtered out by the whitelist
  { TimeLine c("C"); }
  EXPECT(TimeLine::pending() == 2);
  const std::string out = TimeLine::dump(dir + "/timeline.json");
  EXPECT(!out.empty() && TimeLine::pending() == 0);
  std::ifstream f(out);
  std::string text((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
  EXPECT(text.find("\"name\": \"A\"") != std::string::npos || text.find("\"name\":\"A\"") != std::string::npos);
  EXPECT(text.find("\"B\"") == std::string::npos && text.find("\"ph\"") != std::string::npos);
  TimeLine::enable(false);
  { TimeLine off("A"); }
  EXPECT(TimeLine::pending() == 0);
  unsetenv("XFT_VERBOSE");
  unsetenv("XFT_PIPELINE_STAGE");
  unsetenv("XFT_TIMELINE_WHITELIST");
  unsetenv("XFT_KV_CACHE_GB");
  unsetenv("XFT_CUDA_GRAPH");
  Env::get().reload();
  EXPECT(Env::get().verbose == 0 && Env::get().cudaGraph && Env::get().timelineWhitelist.empty());
  log(LogLevel::Debug, "not printed at verbosity %d", 0);
}

static int g_backendAllocs = 0, g_backendFrees = 0;
static void* countingAlloc(size_t n) { ++g_backendAllocs; return std::malloc(n); }
static void countingFree(void* p) { ++g_backendFrees; std::free(p); }

static void testArena() {
  EXPECT(Arena::roundUp(1) == 512 && Arena::roundUp(512) == 512 && Arena::roundUp(513) == 1024);
  EXPECT(Arena::roundUp((1u << 20) + 1) == (2u << 20) && Arena::roundUp(3u << 20) == (4u << 20));
  {
    Arena a(countingAlloc, countingFree);
    void* p = a.allocate(1000);
    std::memset(p, 0xab, 1000);
    EXPECT(p && a.bytesInUse() == 1024 && g_backendAllocs == 1);
    a.release(p);
    EXPECT(a.bytesInUse() == 0 && a.bytesCached() == 1024 && g_backendFrees == 0);
    void* q = a.allocate(600);                   // same class: served from the free list
    EXPECT(q == p && g_backendAllocs == 1 && a.bytesCached() == 0);
    void* r = a.allocate(600);
    EXPECT(r != q && g_backendAllocs == 2);
    int unknown = 0;
    a.release(&unknown);                         // ignored
    a.release(q);
    a.trim();
    EXPECT(g_backendFrees == 1 && a.bytesCached() == 0 && a.bytesInUse() == 1024);
    {
      ArenaBuf b(a, 100), c;
      EXPECT(b.get() && b.size() == 100);
      c = std::move(b);
      EXPECT(c.get() && !b.get());
    }
    EXPECT(a.bytesInUse() == 1024);
    a.release(r);
  }                                              // destructor frees what is cached
  EXPECT(g_backendAllocs == g_backendFrees);
}

static void testRopeTables() {
  RopeScaling none;
  auto t = ropeTable(16, 8, 10000.0, none);
  EXPECT(t.size() == 16 * 8);
  for (int i = 0; i < 4; ++i) EXPECT(t[i] == 1.0f && t[4 + i] == 0.0f);               // position 0: cos 1, sin 0
  EXPECT(std::fabs(t[8 + 0] - std::cos(1.0)) < 1e-6 && std::fabs(t[8 + 4] - std::sin(1.0)) < 1e-6);   // pos 1, freq 1
  for (size_t p = 0; p < 16; ++p)
    for (int i = 0; i < 4; ++i) {
      const float c = t[p * 8 + i], s = t[p * 8 + 4 + i];
      EXPECT(std::fabs(c * c + s * s - 1.0f) < 1e-5);
    }
  RopeScaling lin;
  lin.type = "linear";
  lin.factor = 4.0;
  auto tl = ropeTable(16, 8, 10000.0, lin);
  for (int i = 0; i < 8; ++i) EXPECT(std::fabs(tl[4 * 8 + i] - t[1 * 8 + i]) < 1e-6);   // position 4 at factor 4 = position 1
  RopeScaling yarn;
  yarn.type = "yarn";
  yarn.factor = 8.0;
  yarn.originalMaxPos = 64;
  auto inv0 = ropeInvFreq(64, 10000.0, none), inv = ropeInvFreq(64, 10000.0, yarn);
  EXPECT(inv.size() == 32 && inv[0] == inv0[0]);                                       // fastest dimension is kept
  EXPECT(std::fabs(inv[31] - inv0[31] / 8.0) < 1e-12);                                 // slowest is interpolated
  for (int i = 0; i < 32; ++i) EXPECT(inv[i] <= inv0[i] * (1 + 1e-12) && inv[i] >= inv0[i] / 8.0 * (1 - 1e-12));
  EXPECT(std::fabs(yarnMscale(8.0, 1.0) - (0.1 * std::log(8.0) + 1.0)) < 1e-12 && yarnMscale(1.0, 1.0) == 1.0);
  auto ty = ropeTable(4, 64, 10000.0, yarn);
  EXPECT(std::fabs(ty[0] - (float)yarnMscale(8.0, 1.0)) < 1e-6);                       // cos(0) times the YaRN scale
  EXPECT(telechatNtkTheta(10000.0, 128, 100, 4096) == 10000.0);
  EXPECT(std::fabs(telechatNtkTheta(10000.0, 128, 100, 8192) - 10000.0 * std::pow(3.0, 128.0 / 126.0)) < 1e-6);
  EXPECT(telechatMscale(4096, 8192) == 1.0 && std::fabs(telechatMscale(16384, 8192) - (0.1 * std::log(2.0) + 1.0)) < 1e-12);
  EXPECT(qwenNtkTheta(10000.0, 128, 4096, 8192) == 10000.0);
  EXPECT(std::fabs(qwenNtkTheta(10000.0, 128, 16384, 8192) - 10000.0 * std::pow(3.0, 128.0 / 126.0)) < 1e-6);
  auto a8 = alibiSlopes(8);
  EXPECT(a8.size() == 8 && std::fabs(a8[0] - 0.5f) < 1e-7 && std::fabs(a8[7] - 1.0f / 256) < 1e-9);
  auto a12 = alibiSlopes(12);
  EXPECT(a12.size() == 12 && a12[7] == a8[7] && std::fabs(a12[8] - std::pow(2.0, -0.5)) < 1e-6);
}

static void testDtypes() {
  // every finite half survives the round trip; conversions of exact values are exact
  for (uint32_t h = 0; h < 65536; ++h) {
    const uint32_t e = (h >> 10) & 31;
    if (e == 31 && (h & 1023)) continue;                       // NaN payloads are not preserved bit for bit
    EXPECT(floatToHalf(halfToFloat((uint16_t)h)) == (uint16_t)h);
  }
  EXPECT(floatToHalf(1.0f) == 0x3c00 && floatToHalf(-2.0f) == 0xc000 && floatToHalf(65504.0f) == 0x7bff);
  EXPECT(floatToHalf(65520.0f) == 0x7c00 && floatToHalf(1e9f) == 0x7c00 && floatToHalf(-1e9f) == 0xfc00);
  EXPECT(floatToHalf(5.9604645e-8f) == 0x0001 && floatToHalf(2.0e-8f) == 0x0000);      // smallest subnormal; below half of it
  // ties go to even: 1 + 2^-11 is halfway between 1 and 1 + 2^-10
  EXPECT(floatToHalf(1.0f + 0.00048828125f) == 0x3c00 && floatToHalf(1.0f + 3 * 0.00048828125f) == 0x3c02);
  EXPECT(floatToHalf(1.0f + 0.0005f) == 0x3c01);
  EXPECT(floatToBf16(1.0f) == 0x3f80 && bf16ToFloat(0x3f80) == 1.0f && floatToBf16(-0.0f) == 0x8000);
  EXPECT(floatToBf16(1.0f + 0.00390625f) == 0x3f80 && floatToBf16(1.0f + 3 * 0.00390625f) == 0x3f82);   // ties to even
  const float vals[3] = {0.5f, -3.25f, 100.0f};
  char buf[12];
  std::memcpy(buf, vals, 12);
  EXPECT(elemToFloat(buf, 0, 1) == -3.25f && dtypeSize(0) == 4 && dtypeSize(1) == 2 && dtypeSize(2) == 2);
  uint16_t hs[2] = {floatToHalf(-3.25f), floatToBf16(100.0f)};
  EXPECT(elemToFloat(reinterpret_cast<const char*>(hs), 1, 0) == -3.25f);
  EXPECT(elemToFloat(reinterpret_cast<const char*>(hs), 2, 1) == 100.0f);
}

// Byte-level BPE reader: a hand-written tokenizer.json (alphabet a, b, c, space-character and two merges), malformed
// files that must be refused with an exception, input bytes that are no UTF-8.
static void testBpeTokenizer(const std::string& dir) {
  const std::string good = dir + "/bpe_good.json";
  {
    std::ofstream f(good);
    // "\u0120" is the alphabet character of the space byte
    f << R"({"added_tokens": [{"id": 9, "content": "<|end|>"}],
             "pre_tokenizer": {"type": "ByteLevel", "add_prefix_space": false, "use_regex": true},
             "model": {"type": "BPE", "unk_token": null, "ignore_merges": false,
                       "vocab": {"a": 0, "b": 1, "c": 2, "\u0120": 3, "ab": 4, "\u0120c": 5, "abab": 6, "!": 7, "1": 8},
                       "merges": ["a b", ["\u0120", "c"], "ab ab"]}})";
  }
  BpeTokenizer t(good);
  EXPECT(t.vocabSize() == 10 && t.specialId("<|end|>") == 9 && t.specialId("nope") == -1 && std::string(t.pattern()) == "gpt2");
  EXPECT(t.encode("abab c") == std::vector<int32_t>({6, 5}));
  EXPECT(t.encode("ab<|end|>ba") == std::vector<int32_t>({4, 9, 1, 0}));
  EXPECT(t.encode("") .empty());
  EXPECT(t.decode({6, 5, 9, 7}) == "abab c<|end|>!");
  EXPECT(t.decode({-1, 99}) .empty());
  // bytes outside the vocabulary (and not even UTF-8) are dropped, never read past the end
  const std::string junk = std::string("a\xff\xfe") + "\xe4" + "b\xf0\x9f";
  EXPECT(t.encode(junk) == std::vector<int32_t>({0, 1}));
  const char* bad[] = {"", "{", "{\"model\": {\"vocab\": {\"a\": 0}, \"merges\": [}}", "{\"model\": \"x\"}",
                       "{\"a\": \"\\u12\"}", "{\"a\": \"\\q\"}", "[1, 2", "{\"model\": {\"type\": \"WordPiece\", \"vocab\": {}, \"merges\": []}}",
                       "{\"model\": {\"vocab\": {}, \"merges\": []}}"};
  int refused = 0;
  for (const char* text : bad) {
    const std::string p = dir + "/bpe_bad.json";
    { std::ofstream f(p); f << text; }
    try { BpeTokenizer x(p); } catch (const std::runtime_error&) { ++refused; }
  }
  EXPECT(refused == (int)(sizeof(bad) / sizeof(bad[0])));
  std::string deep(200, '[');
  { std::ofstream f(dir + "/bpe_deep.json"); f << deep; }
  bool threw = false;
  try { BpeTokenizer x(dir + "/bpe_deep.json"); } catch (const std::runtime_error&) { threw = true; }
  EXPECT(threw);
}

// GPTQ tensors: [in, out] codes -> [out, in] rows (uint4: repacked along `in`), slices, dequantised values, code sums.
static void testGptq() {
  const int inF = 6, outF = 4;
  std::vector<uint8_t> i8(inF * outF);
  for (int i = 0; i < inF; ++i) for (int o = 0; o < outF; ++o) i8[i * outF + o] = (uint8_t)(int8_t)(i * 10 + o - 20);
  std::vector<uint8_t> rows(outF * 16, 0xAA);
  gptqRepack(i8.data(), inF, outF, false, 0, inF, 0, outF, 16, rows.data());
  EXPECT((int8_t)rows[2 * 16 + 5] == 5 * 10 + 2 - 20 && rows[2 * 16 + 6] == 0 && rows[15] == 0);
  std::vector<uint8_t> u4(inF * outF / 2);
  auto code = [](int i, int o) { return (i * 3 + o * 5) & 15; };
  for (int i = 0; i < inF; ++i) for (int o = 0; o < outF; o += 2) u4[i * (outF / 2) + o / 2] = (uint8_t)(code(i, o) | (code(i, o + 1) << 4));
  std::vector<uint8_t> r4(2 * 16, 0xAA);
  gptqRepack(u4.data(), inF, outF, true, 2, 6, 1, 3, 16, r4.data());          // inputs 2..5 of outputs 1..2
  EXPECT(r4[0] == (uint8_t)(code(2, 1) | (code(3, 1) << 4)) && r4[16 + 1] == (uint8_t)(code(4, 2) | (code(5, 2) << 4)) && r4[2] == 0);
  const float sc[4] = {0.5f, 1.0f, 2.0f, 4.0f}, zp[4] = {0.f, -1.f, 1.f, 0.25f};
  std::vector<float> deq(2 * 4);
  gptqDequant(u4.data(), inF, outF, true, 2, 6, 1, 3, sc, zp, deq.data());
  EXPECT(deq[0] == code(2, 1) * 1.0f - 1.f && deq[4 + 3] == code(5, 2) * 2.0f + 1.f);
  float sums[2];
  gptqRowSums(u4.data(), inF, outF, true, 2, 6, 1, 3, sums);
  EXPECT(sums[0] == (float)(code(2, 1) + code(3, 1) + code(4, 1) + code(5, 1)));
}

int main(int argc, char** argv) {
  const std::string dir = argc > 1 ? argv[1] : "/tmp";
  testPartition();
  testSequences();
  testBlockTables();
  testSamplers();
  testBeams();
  testIni(dir);
  testEnvAndTimeline(dir);
  testArena();
  testRopeTables();
  testDtypes();
  testBpeTokenizer(dir);
  testGptq();
  std::printf("runtime_selftest: %d checks, %d failed\n", g_checks, g_failed);
  return g_failed ? 1 : 0;
}
