// Continuous-batching consistency checker for the C++ API (reference: examples/cpp/cb_check.cpp).
//
// The same prompts are decoded twice with greedy search: (1) one sequence at a time, (2) through the continuous-
// batching calls with staggered admission — a new prompt joins every `--stride` steps while earlier sequences are
// in the middle of their decode, and finished sequences are freed while others keep running.  Batch composition
// must not change what a sequence generates, so both passes have to produce the same tokens.
//
//   cb_check -m <model dir> [-d bf16|int8|...] [--kv_cache_dtype fp16|int8] [-n prompts] [-o out_len] [--stride k]
//            [--min_len a] [--max_len b] [--seed s] [--tolerate t] [-t <tokenizer.model | tokenizer.json | dir>] [-i <prompt>]
// The prompts are random token ids; `-i` (token ids, or text with `-t`, as the reference's checker takes it) replaces the
// first of them.
// Exit code 0 when every sequence agrees (up to `--tolerate` late divergences caused by bf16 near-ties), 1 otherwise.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <memory>
#include <random>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "bpe_tokenizer.h"
#include "tokenizer.h"
#include "xft/models.h"

namespace {

int argmaxRow(const float* row, int vocab) {
  int best = 0;
  for (int i = 1; i < vocab; ++i)
    if (row[i] > row[best]) best = i;
  return best;
}

// one sequence on its own: prefill, then one token per forward()
std::vector<int> runAlone(xft::Model& m, const std::vector<int32_t>& prompt, int outLen) {
  std::vector<std::vector<int32_t>> in{prompt};
  std::vector<int> ids = m.set_input(in, std::vector<int>{}, (int)prompt.size() + outLen);
  std::vector<int> out;
  for (int step = 0; step < outLen; ++step) {
    auto [logits, rows, vocab] = m.forward(false);
    if (rows != 1) throw std::runtime_error("expected one row of logits");
    const int tok = argmaxRow(logits, vocab);
    out.push_back(tok);
    if (step + 1 < outLen) {
      std::vector<std::vector<int32_t>> next{{tok}};
      m.set_input(next, ids);
    }
  }
  m.freeSeqs(ids);
  return out;
}

}  // namespace

int main(int argc, char** argv) {
  std::string model, dtype = "bf16", kv = "fp16", tokenPath, input;
  int nPrompts = 6, outLen = 16, stride = 3, minLen = 4, maxLen = 40, tolerate = 0;
  unsigned seed = 1234;
  for (int i = 1; i < argc; ++i) {
    std::string a = argv[i];
    auto next = [&]() -> std::string {
      if (i + 1 >= argc) { std::fprintf(stderr, "missing value for %s\n", a.c_str()); std::exit(2); }
      return argv[++i];
    };
    if (a == "-m" || a == "--model") model = next();
    else if (a == "-d" || a == "--dtype") dtype = next();
    else if (a == "--kv_cache_dtype") kv = next();
    else if (a == "-n" || a == "--num_prompts") nPrompts = std::atoi(next().c_str());
    else if (a == "-o" || a == "--output_len") outLen = std::atoi(next().c_str());
    else if (a == "--stride") stride = std::max(1, std::atoi(next().c_str()));
    else if (a == "--min_len") minLen = std::atoi(next().c_str());
    else if (a == "--max_len") maxLen = std::atoi(next().c_str());
    else if (a == "--seed") seed = (unsigned)std::atoi(next().c_str());
    else if (a == "--tolerate") tolerate = std::atoi(next().c_str());
    else if (a == "-t" || a == "--token") tokenPath = next();
    else if (a == "-i" || a == "--input") input = next();
    else { std::fprintf(stderr, "unknown flag %s\n", a.c_str()); return 2; }
  }
  if (model.empty()) { std::fprintf(stderr, "usage: cb_check -m <model dir> [options]\n"); return 2; }
  const xft::DataType wdt = xft::dataTypeFromName(dtype.c_str());
  if (wdt == xft::DataType::unknown) { std::fprintf(stderr, "unknown weight type %s\n", dtype.c_str()); return 2; }
  try {
    // the prompt of -i: token ids, or text through the tokenizer of -t
    std::vector<int32_t> given;
    if (!input.empty()) {
      if (input.find_first_not_of("0123456789 \t") == std::string::npos) {
        std::istringstream is(input);
        for (int v; is >> v;) given.push_back(v);
      } else if (tokenPath.empty()) {
        std::fprintf(stderr, "-i takes token ids separated by spaces, or text with -t <tokenizer.model | tokenizer.json>\n");
        return 2;
      } else if (tokenPath.size() > 6 && tokenPath.compare(tokenPath.size() - 6, 6, ".model") == 0) {
        given = xft::SentencePieceTokenizer(tokenPath).encode(input, /*addBos=*/true);
      } else {
        given = xft::BpeTokenizer(tokenPath).encode(input);
      }
    }
    xft::AutoModel m(model, wdt, kv == "int8" ? xft::DataType::int8 : xft::DataType::fp16);
    const int vocab = m.getVocabSize();
    std::mt19937 rng(seed);
    std::vector<std::vector<int32_t>> prompts(nPrompts);
    for (auto& p : prompts) {
      const int len = minLen + (int)(rng() % (unsigned)std::max(1, maxLen - minLen + 1));
      p.resize(len);
      for (auto& t : p) t = 3 + (int)(rng() % (unsigned)std::max(1, vocab - 3));
    }
    if (!given.empty() && !prompts.empty()) {
      for (int t : given) if (t < 0 || t >= vocab) throw std::runtime_error("-i: token id outside the vocabulary");
      prompts[0] = given;
    }
    // pass 1: alone
    std::vector<std::vector<int>> alone;
    for (const auto& p : prompts) alone.push_back(runAlone(m, p, outLen));

    // pass 2: continuous batching with staggered admission
    struct Live { int prompt; int id; std::vector<int> out; };
    std::vector<Live> live;
    std::vector<std::vector<int>> batched(nPrompts);
    int admitted = 0, step = 0, finished = 0;
    while (finished < nPrompts) {
      if (admitted < nPrompts && step % stride == 0) {
        std::vector<std::vector<int32_t>> in{prompts[admitted]};
        std::vector<int> ids = m.set_input(in, std::vector<int>{}, (int)prompts[admitted].size() + outLen);
        auto [logits, rows, v] = m.forward(false);
        if (rows != 1) throw std::runtime_error("prefill returned more than one row");
        live.push_back({admitted, ids[0], {argmaxRow(logits, v)}});
        ++admitted;
      }
      // retire the finished, decode the rest together
      std::vector<int> done;
      for (auto it = live.begin(); it != live.end();) {
        if ((int)it->out.size() >= outLen) {
          done.push_back(it->id);
          batched[it->prompt] = it->out;
          ++finished;
          it = live.erase(it);
        } else {
          ++it;
        }
      }
      if (!done.empty()) m.freeSeqs(done);
      if (!live.empty()) {
        std::vector<std::vector<int32_t>> toks;
        std::vector<int> ids;
        for (auto& s : live) { toks.push_back({s.out.back()}); ids.push_back(s.id); }
        m.set_input(toks, ids);
        auto [logits, rows, v] = m.forward(false);
        if (rows != (int)live.size()) throw std::runtime_error("decode returned a wrong number of rows");
        for (int r = 0; r < rows; ++r) live[r].out.push_back(argmaxRow(logits + (size_t)r * v, v));
      }
      ++step;
    }
    // pass 3: the AbstractDecoder view (xft/abstract_decoder.h).  Two copies of prompt 0 run as a (batch 1, beam 2)
    // step; after the first token the two rows are swapped with reorderCache, which must not change what they
    // generate (both rows hold the same history), and the tokens must equal pass 1.
    int decoderBad = 0;
    {
      std::unique_ptr<xft::AbstractDecoder> dec = xft::makeDecoder(m);
      const std::vector<int32_t>& p0 = prompts[0];
      std::vector<int> ids(p0.begin(), p0.end());
      ids.insert(ids.end(), p0.begin(), p0.end());
      int64_t dims[3] = {1, 2, (int64_t)p0.size()};
      std::vector<int> out;
      for (int t = 0; t < outLen; ++t) {
        auto [logits, off, size] = dec->forward(ids.data(), dims, t);
        const int a = argmaxRow(logits, size), b = argmaxRow(logits + size, size);
        if (off != 0 || size != vocab || a != b) { ++decoderBad; break; }
        out.push_back(a);
        if (t == 0) { int swap[2] = {1, 0}; dec->reorderCache(swap, 2); }
        ids = {a, b};
        dims[2] = 1;
      }
      if ((int)out.size() == outLen && out != alone[0]) ++decoderBad;
      if (dec->getEndId() < 0 || !dec->isMaster() || dec->getRank() != 0) ++decoderBad;
      std::printf("decoder view: %s\n", decoderBad ? "MISMATCH" : "identical to the model API");
    }
    int bad = decoderBad;
    for (int i = 0; i < nPrompts; ++i) {
      int first = -1;
      for (int t = 0; t < outLen; ++t)
        if (alone[i][t] != batched[i][t]) { first = t; break; }
      if (first >= 0) {
        ++bad;
        std::printf("prompt %d (len %zu): diverges at generated token %d (alone %d, batched %d)\n", i, prompts[i].size(),
                    first, alone[i][first], batched[i][first]);
      } else {
        std::printf("prompt %d (len %zu): %d tokens identical\n", i, prompts[i].size(), outLen);
      }
    }
    std::printf("cb_check: %d of %d sequences identical, %d steps\n", nPrompts - bad, nPrompts, step);
    return bad <= tolerate ? 0 : 1;
  } catch (const std::exception& e) {
    std::fprintf(stderr, "cb_check failed: %s\n", e.what());
    return 3;
  }
}
