// Drives the C++ engine through its whole public API over the host stand-in of the device library
// (csrc/tests/mock_device.cc), without a GPU: every request shape the engine knows — batch generation with greedy
// search, sampling and beams, continuous batching with ragged prompts that cross KV block borders, a sequence joining
// and leaving, prefix sharing, all-position logits — for one model directory, weight type and KV type, on one rank or
// on N thread ranks (tensor parallel).  The numbers are meaningless; what is checked is that the host side asks the
// device library for memory it owns (AddressSanitizer + exact-size buffers), keeps its bookkeeping consistent, and
// that ranks agree.
//
//   engine_hostcheck <model dir> <weight type> <kv type> <ranks>
//
// With the arithmetic of the stand-in switched on (XFT_MOCK_MATH=1) a second form records logits for a comparison with
// another implementation of the model: the prompts of <ids file> ("B P steps" and then B * P token ids) go through the
// continuous-batching calls, `steps` greedy tokens follow one at a time, and <out file> receives B, V, steps + 1 as
// int32, the logits of every pass [steps + 1, B, V] as fp32 and the token chosen after each pass [steps + 1, B] as int32.
//
//   engine_hostcheck logits <model dir> <weight type> <kv type> <ranks> <ids file> <out file>
//
// A third form runs the batch generation calls (config / input / generate / finalize) with `beams` beams and writes the
// rows that finalize() returns: B, row length as int32, then the rows.  `steps` of the ids file is the number of new
// tokens, eos is token `eos` (-1: none).
//
//   engine_hostcheck generate <model dir> <weight type> <kv type> <ranks> <ids file> <out file> <beams> <eos>
#include <cstdio>
#include <cstdlib>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include "comm.h"
#include "xft/models.h"

namespace {

#define CHECK(cond)                                                                                         \
  do {                                                                                                      \
    if (!(cond)) throw std::runtime_error(std::string("check failed: " #cond " (line ") + std::to_string(__LINE__) + ")"); \
  } while (0)

std::vector<int32_t> promptOf(int len, int vocab, int salt) {
  std::vector<int32_t> p(len);
  for (int i = 0; i < len; ++i) p[i] = 3 + (i * 7 + salt * 13) % (vocab - 3);
  return p;
}

// everything one rank does; every rank of a tensor-parallel group makes the same calls
std::vector<int32_t> exercise(xft::Model& m, bool experts) {
  const int V = m.getVocabSize();
  CHECK(V > 8 && m.getMaxSeqLen() >= 128);
  std::vector<int32_t> trace;
  // 1. batch generation, greedy: two equal-length prompts
  {
    const int P = 9, B = 2;
    std::vector<int32_t> ids;
    for (int b = 0; b < B; ++b) { auto p = promptOf(P, V, b); ids.insert(ids.end(), p.begin(), p.end()); }
    m.config(P + 4, 1, 1, 1.0f, false, V + 5 /* never produced */, 0);
    m.input(ids, B);
    int steps = 0;
    while (!m.isDone()) { auto next = m.generate(); CHECK((int)next.size() == B); ++steps; }
    CHECK(steps == 4);
    auto out = m.finalize();
    CHECK((int)out.size() == B * (P + 4));
    for (int b = 0; b < B; ++b) for (int i = 0; i < P; ++i) CHECK(out[b * (P + 4) + i] == ids[b * P + i]);
    trace.insert(trace.end(), out.begin(), out.end());
  }
  // 2. sampling with a fixed seed and a repetition penalty
  {
    SearcherConfig c(14, 1, 1, 1.0f, false, V + 5, 0, true, 0.8f, 5, 0.9f, 1.2f);
    c.seed = 1234;
    std::vector<std::vector<int32_t>> prompts = {promptOf(6, V, 2), promptOf(11, V, 3)};       // ragged
    m.set_input(prompts, c);
    while (!m.isDone()) m.generate();
    auto out = m.finalize();
    CHECK(out.size() == 2 * 14);
    trace.insert(trace.end(), out.begin(), out.end());
  }
  // 3. beam search, three beams, prompts that fill a KV block exactly and spill into the next one
  {
    const int P = 64, B = 2, nb = 3;
    std::vector<int32_t> ids;
    for (int b = 0; b < B; ++b) { auto p = promptOf(P, V, 4 + b); ids.insert(ids.end(), p.begin(), p.end()); }
    m.config(P + 5, nb, 2, 1.0f, false, 1 /* eos may well appear */, 0);
    m.input(ids, B);
    int steps = 0;
    while (!m.isDone() && steps < 8) { auto next = m.generate(); CHECK((int)next.size() == B * nb); ++steps; }
    auto out = m.finalize();
    CHECK(!out.empty() && out.size() % (B * 2) == 0);
    trace.insert(trace.end(), out.begin(), out.end());
  }
  // 4. continuous batching: ragged prompts (one crosses a block border), decode, a third sequence joins, one leaves
  {
    std::vector<std::vector<int32_t>> prompts = {promptOf(5, V, 6), promptOf(70, V, 7)};
    std::vector<int> ids = m.set_input(prompts, std::vector<int>{}, 100);
    CHECK(ids.size() == 2);
    auto r = m.forward(false);
    CHECK(std::get<1>(r) == 2 && std::get<2>(r) == V);
    for (int step = 0; step < 3; ++step) {
      std::vector<std::vector<int32_t>> next = {{4 + step}, {5 + step}};
      m.set_input(next, ids, 100);
      r = m.forward(false);
      CHECK(std::get<1>(r) == 2);
    }
    std::vector<std::vector<int32_t>> late = {promptOf(130, V, 8)};                              // three blocks
    std::vector<int> id3 = m.set_input(late, std::vector<int>{}, 140);
    r = m.forward(true);                                                                        // every position
    CHECK(std::get<1>(r) == 130);
    std::vector<int> first = {ids[0]};
    CHECK(m.freeSeqs(first));
    std::vector<int> both = {ids[1], id3[0]};
    std::vector<std::vector<int32_t>> next = {{9}, {10}};
    m.set_input(next, both, 140);
    r = m.forward(false);
    CHECK(std::get<1>(r) == 2);
    const float* lg = std::get<0>(r);
    for (int i = 0; i < 2 * V; ++i) CHECK(lg[i] == lg[i]);                                      // no NaN
    trace.push_back((int32_t)(lg[3] * 1000));
    CHECK(m.freeSeqs(both));
  }
  // 5. prefix sharing: 64 shared tokens (one whole block), two requests behind it
  if (!experts) {
    auto shared = promptOf(64, V, 9);
    m.setPrefix(shared);
    std::vector<int32_t> ids;
    for (int b = 0; b < 2; ++b) { auto p = shared; auto tail = promptOf(6, V, 10 + b); p.insert(p.end(), tail.begin(), tail.end()); ids.insert(ids.end(), p.begin(), p.end()); }
    m.config(70 + 3, 1, 1, 1.0f, false, V + 5, 0);
    m.input(ids, 2);
    while (!m.isDone()) m.generate();
    auto out = m.finalize();
    CHECK(out.size() == 2 * 73);
    m.unsetPrefix();
    trace.insert(trace.end(), out.begin(), out.end());
  }
  return trace;
}

struct LogitsRun {
  int B = 0, P = 0, steps = 0;
  std::vector<int32_t> ids;
  std::vector<float> logits;       // [steps + 1, B, V]
  std::vector<int32_t> tokens;     // [steps + 1, B]
  int V = 0;
};

void recordLogits(xft::Model& m, LogitsRun& run) {
  std::vector<std::vector<int32_t>> prompts(run.B);
  for (int b = 0; b < run.B; ++b) prompts[b].assign(run.ids.begin() + (size_t)b * run.P, run.ids.begin() + (size_t)(b + 1) * run.P);
  const int maxLen = run.P + run.steps + 2;
  std::vector<int> seqs = m.set_input(prompts, std::vector<int>{}, maxLen);
  run.V = m.getVocabSize();
  for (int s = 0; s <= run.steps; ++s) {
    auto r = m.forward(false);
    CHECK(std::get<1>(r) == run.B && std::get<2>(r) == run.V);
    const float* lg = std::get<0>(r);
    run.logits.insert(run.logits.end(), lg, lg + (size_t)run.B * run.V);
    std::vector<std::vector<int32_t>> next(run.B);
    for (int b = 0; b < run.B; ++b) {
      int best = 0;
      for (int v = 1; v < run.V; ++v) if (lg[(size_t)b * run.V + v] > lg[(size_t)b * run.V + best]) best = v;
      run.tokens.push_back(best);
      next[b].assign(1, best);
    }
    if (s < run.steps) m.set_input(next, seqs, maxLen);
  }
  CHECK(m.freeSeqs(seqs));
}

void recordGenerate(xft::Model& m, LogitsRun& run, int beams, int eos) {
  run.V = m.getVocabSize();
  const int maxLen = run.P + run.steps;
  m.config(maxLen, beams, 1, 1.0f, false, eos < 0 ? run.V + 5 : eos, 0);
  m.input(run.ids, run.B);
  int guard = 0;
  while (!m.isDone() && guard++ <= run.steps) m.generate();
  CHECK(m.isDone());
  run.tokens = m.finalize();
  CHECK(!run.tokens.empty() && run.tokens.size() % run.B == 0);
}

int logitsMain(int argc, char** argv) {
  const bool gen = std::string(argv[1]) == "generate";
  const int beams = gen && argc >= 9 ? std::atoi(argv[8]) : 1, eos = gen && argc >= 10 ? std::atoi(argv[9]) : -1;
  if (argc < 8) { std::fprintf(stderr, "usage: engine_hostcheck logits <model dir> <weight type> <kv type> <ranks> <ids file> <out file>\n"); return 2; }
  const std::string dir = argv[2];
  const xft::DataType wdt = xft::dataTypeFromName(argv[3]);
  const xft::DataType kdt = std::string(argv[4]) == "int8" ? xft::DataType::int8 : xft::DataType::fp16;
  // <ranks> = "env": this process is ONE rank of a group of processes; rank and world size come from the launcher's
  // variables, the ranks meet through the NCCL communicator (in tests: a stand-in library named by XFT_NCCL_LIB)
  const bool procs = std::string(argv[5]) == "env";
  const int ranks = procs ? 1 : std::atoi(argv[5]);
  if (wdt == xft::DataType::unknown || ranks < 1 || ranks > 8) { std::fprintf(stderr, "bad arguments\n"); return 2; }
  LogitsRun proto;
  {
    FILE* f = std::fopen(argv[6], "r");
    if (!f || std::fscanf(f, "%d %d %d", &proto.B, &proto.P, &proto.steps) != 3) { std::fprintf(stderr, "cannot read %s\n", argv[6]); return 2; }
    proto.ids.resize((size_t)proto.B * proto.P);
    for (auto& v : proto.ids) if (std::fscanf(f, "%d", &v) != 1) { std::fprintf(stderr, "short ids file\n"); std::fclose(f); return 2; }
    std::fclose(f);
  }
  std::vector<LogitsRun> runs(ranks, proto);
  std::vector<std::string> errors(ranks);
  if (procs) {
    xft::AutoModel m(dir, wdt, kdt);
    if (gen) recordGenerate(m, runs[0], beams, eos); else recordLogits(m, runs[0]);
    if (!m.isMaster()) { std::printf("hostcheck rank %d of %d done\n", m.getRank(), m.getWorldSize()); return 0; }
  } else if (ranks == 1) {
    xft::AutoModel m(dir, wdt, kdt, nullptr);
    if (gen) recordGenerate(m, runs[0], beams, eos); else recordLogits(m, runs[0]);
  } else {
    auto comms = xft::makeThreadCommunicators(ranks);
    std::vector<std::thread> threads;
    for (int r = 0; r < ranks; ++r)
      threads.emplace_back([&, r] {
        try {
          comms[r]->begin();
          xft::AutoModel m(dir, wdt, kdt, comms[r]);
          if (gen) recordGenerate(m, runs[r], beams, eos); else recordLogits(m, runs[r]);
        } catch (const std::exception& e) {
          errors[r] = e.what();
        }
        comms[r]->end();
      });
    for (auto& t : threads) t.join();
  }
  bool failed = false;
  for (int r = 0; r < ranks; ++r)
    if (!errors[r].empty()) { std::fprintf(stderr, "rank %d: %s\n", r, errors[r].c_str()); failed = true; }
  if (failed) return 1;
  for (int r = 1; r < ranks; ++r)
    if (runs[r].logits != runs[0].logits || runs[r].tokens != runs[0].tokens) { std::fprintf(stderr, "rank %d sees other logits than rank 0\n", r); return 1; }
  FILE* f = std::fopen(argv[7], "wb");
  if (!f) { std::fprintf(stderr, "cannot write %s\n", argv[7]); return 2; }
  if (gen) {
    const int32_t head[2] = {runs[0].B, (int32_t)(runs[0].tokens.size() / runs[0].B)};
    std::fwrite(head, 4, 2, f);
    std::fwrite(runs[0].tokens.data(), 4, runs[0].tokens.size(), f);
    std::fclose(f);
    std::printf("hostcheck generate ok: %d ranks, %d rows of %d\n", ranks, head[0], head[1]);
    return 0;
  }
  const int32_t head[3] = {runs[0].B, runs[0].V, runs[0].steps + 1};
  std::fwrite(head, 4, 3, f);
  std::fwrite(runs[0].logits.data(), 4, runs[0].logits.size(), f);
  std::fwrite(runs[0].tokens.data(), 4, runs[0].tokens.size(), f);
  std::fclose(f);
  std::printf("hostcheck logits ok: %d ranks, %d x %d x %d\n", ranks, head[2], head[0], head[1]);
  return 0;
}

}  // namespace

int main(int argc, char** argv) {
  if (argc >= 2 && (std::string(argv[1]) == "logits" || std::string(argv[1]) == "generate")) {
    try { return logitsMain(argc, argv); } catch (const std::exception& e) { std::fprintf(stderr, "error: %s\n", e.what()); return 1; }
  }
  if (argc < 5) { std::fprintf(stderr, "usage: engine_hostcheck <model dir> <weight type> <kv type> <ranks>\n"); return 2; }
  const std::string dir = argv[1];
  const xft::DataType wdt = xft::dataTypeFromName(argv[2]);
  const xft::DataType kdt = std::string(argv[3]) == "int8" ? xft::DataType::int8 : xft::DataType::fp16;
  const int ranks = std::atoi(argv[4]);
  const bool experts = dir.find("moe") != std::string::npos || dir.find("mixtral") != std::string::npos;
  if (wdt == xft::DataType::unknown || ranks < 1 || ranks > 8) { std::fprintf(stderr, "bad arguments\n"); return 2; }
  try {
    if (ranks == 1) {
      xft::AutoModel m(dir, wdt, kdt, nullptr);
      CHECK(m.isMaster() && m.getRank() == 0 && m.getWorldSize() == 1);
      auto t = exercise(m, experts);
      std::printf("hostcheck ok: %zu values\n", t.size());
      return 0;
    }
    auto comms = xft::makeThreadCommunicators(ranks);
    std::vector<std::vector<int32_t>> traces(ranks);
    std::vector<std::string> errors(ranks);
    std::vector<std::thread> threads;
    for (int r = 0; r < ranks; ++r)
      threads.emplace_back([&, r] {
        try {
          comms[r]->begin();
          xft::AutoModel m(dir, wdt, kdt, comms[r]);
          if (m.getRank() != r || m.getWorldSize() != ranks || m.isMaster() != (r == 0)) throw std::runtime_error("rank bookkeeping");
          traces[r] = exercise(m, experts);
        } catch (const std::exception& e) {
          errors[r] = e.what();
        }
        comms[r]->end();
      });
    for (auto& t : threads) t.join();
    bool failed = false;
    for (int r = 0; r < ranks; ++r)
      if (!errors[r].empty()) { std::fprintf(stderr, "rank %d: %s\n", r, errors[r].c_str()); failed = true; }
    if (failed) return 1;
    for (int r = 1; r < ranks; ++r)
      if (traces[r] != traces[0]) { std::fprintf(stderr, "rank %d produced other tokens than rank 0\n", r); return 1; }
    std::printf("hostcheck ok: %d ranks, %zu values each\n", ranks, traces[0].size());
    return 0;
  } catch (const std::exception& e) {
    std::fprintf(stderr, "error: %s\n", e.what());
    return 1;
  }
}
