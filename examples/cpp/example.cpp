// Command-line generation with the C++ API (reference: examples/cpp/example.cpp:352-545).
//
//   example -m <model dir> [-t <tokenizer.model | tokenizer.json | dir>] [--bos id] [-d bf16|fp16|int8|w8a8|int4|nf4|bf16_int8|...]
//           [--kv_cache_dtype fp16|int8] [-i "1 2 3 4"] [-l input_len] [-o out_len] [--prefix_len n] [-n num_beams]
//           [-b batch] [--loop n] [--topK k] [--topP p] [--temperature t] [--repetPen r] [--do_sample] [--no_stream]
// Same flag names as the reference.  -l pads the prompt to `input_len` tokens by repeating its third token (the
// reference's way of making a long prompt for timing); --prefix_len shares the first n prompt tokens between the rows
// of the batch through Model::setPrefix (whole 64-token blocks).  With -t, -i may be TEXT: it is tokenised by a
// built-in reader and the generated ids are printed as text too.  -t takes a SentencePiece model file (*.model: Llama,
// Mistral, Gemma, Yi, Baichuan, ChatGLM families; csrc/core/tokenizer.h, BOS prepended), or a tokenizer.json or the
// directory that holds it (byte-level BPE: OPT, Qwen, Llama-3, ...; csrc/core/bpe_tokenizer.h; `--bos id` prepends a
// token, e.g. 2 for OPT).  Without -t, or when -i holds only numbers, -i is a list of token ids.  Prints the generated
// ids / text, first-token latency and average next-token latency (the reference's metrics).  Started as several
// processes (mpirun -n N, or torchrun) the dense families run tensor-parallel, one GPU per process; rank 0's flags
// decide and rank 0 prints.
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

#include "bpe_tokenizer.h"
#include "tokenizer.h"
#include "xft/models.h"

int main(int argc, char** argv) {
  std::string model, dtype = "bf16", kv = "fp16", input = "1 15043 29892 920 526 366 29973", tokenPath;
  int batch = 1, outLen = 32, loop = 1, topK = 50, numBeams = 1, inputLen = -1, prefixLen = 0, bosId = -1;
  float topP = 1.0f, temp = 1.0f, rep = 1.0f;
  bool sample = false, stream = true;
  for (int i = 1; i < argc; ++i) {
    std::string a = argv[i], inlineValue;
    // `--name=value`, as the reference's option parser takes it besides `--name value`
    const size_t eq = a.rfind("--", 0) == 0 ? a.find('=') : std::string::npos;
    const bool hasInline = eq != std::string::npos;
    if (hasInline) { inlineValue = a.substr(eq + 1); a = a.substr(0, eq); }
    auto next = [&]() -> std::string {
      if (hasInline) return inlineValue;
      if (i + 1 >= argc) { std::fprintf(stderr, "missing value for %s\n", a.c_str()); std::exit(2); }
      return argv[++i];
    };
    if (a == "-m" || a == "--model") model = next();
    else if (a == "-d" || a == "--dtype") dtype = next();
    else if (a == "--kv_cache_dtype") kv = next();
    else if (a == "-i" || a == "--input" || a == "--input_ids") input = next();
    else if (a == "-b" || a == "--batch_size") batch = std::atoi(next().c_str());
    else if (a == "-o" || a == "--output_len") outLen = std::atoi(next().c_str());
    else if (a == "--loop") loop = std::atoi(next().c_str());
    else if (a == "-l" || a == "--input_len") inputLen = std::atoi(next().c_str());
    else if (a == "--prefix_len") prefixLen = std::atoi(next().c_str());
    else if (a == "-t" || a == "--token") tokenPath = next();
    else if (a == "--bos") bosId = std::atoi(next().c_str());
    else if (a == "--topK") topK = std::atoi(next().c_str());
    else if (a == "-n" || a == "--num_beams") numBeams = std::atoi(next().c_str());
    else if (a == "--topP") topP = (float)std::atof(next().c_str());
    else if (a == "--temperature") temp = (float)std::atof(next().c_str());
    else if (a == "--repetPen") rep = (float)std::atof(next().c_str());
    else if (a == "--do_sample") sample = true;
    else if (a == "--no_stream") stream = false;
    else { std::fprintf(stderr, "unknown flag %s\n", a.c_str()); return 2; }
  }
  if (model.empty()) { std::fprintf(stderr, "usage: example -m <model dir> [options]\n"); return 2; }
  std::vector<int32_t> prompt;
  // -t: a SentencePiece model file (*.model), or a tokenizer.json / a directory with one (byte-level BPE)
  std::unique_ptr<xft::SentencePieceTokenizer> tok;
  std::unique_ptr<xft::BpeTokenizer> bpe;
  const bool numeric = input.find_first_not_of("0123456789 \t") == std::string::npos;
  try {
    if (!tokenPath.empty()) {
      const bool spm = tokenPath.size() > 6 && tokenPath.compare(tokenPath.size() - 6, 6, ".model") == 0;
      if (spm) tok.reset(new xft::SentencePieceTokenizer(tokenPath));
      else bpe.reset(new xft::BpeTokenizer(tokenPath));
    }
  } catch (const std::exception& e) {
    std::fprintf(stderr, "error: %s\n", e.what());
    return 1;
  }
  if (tok && !numeric) {
    prompt = tok->encode(input, /*addBos=*/true);
  } else if (bpe && !numeric) {
    prompt = bpe->encode(input);
    if (bosId >= 0) prompt.insert(prompt.begin(), bosId);       // these tokenizers add no BOS by themselves
  } else {
    std::istringstream is(input);
    int v;
    while (is >> v) prompt.push_back(v);
  }
  if (prompt.empty()) { std::fprintf(stderr, "-i takes token ids separated by spaces (or text, with -t <tokenizer.model | tokenizer.json>)\n"); return 2; }
  if (inputLen > (int)prompt.size()) {
    const size_t at = prompt.size() > 2 ? 2 : prompt.size() - 1;
    prompt.insert(prompt.begin() + at, inputLen - prompt.size(), prompt[at]);
  } else if (inputLen > 0) {
    std::fprintf(stderr, "[Warning] input_len %d is not longer than the prompt, using %zu tokens\n", inputLen, prompt.size());
  }
  if (prefixLen < 0 || prefixLen >= (int)prompt.size()) { std::fprintf(stderr, "--prefix_len must be below the prompt length\n"); return 2; }
  try {
    const xft::DataType wdt = xft::dataTypeFromName(dtype.c_str());
    if (wdt == xft::DataType::unknown) { std::fprintf(stderr, "unknown weight type %s\n", dtype.c_str()); return 2; }
    xft::AutoModel m(model, wdt,
                     kv == "int8" ? xft::DataType::int8 : xft::DataType::fp16);
    if (prefixLen > 0) {
      std::vector<int32_t> prefix(prompt.begin(), prompt.begin() + prefixLen);
      m.setPrefix(prefix);
    }
    for (int it = 0; it < loop; ++it) {
      std::vector<int32_t> ids;
      for (int b = 0; b < batch; ++b) ids.insert(ids.end(), prompt.begin(), prompt.end());
      m.config((int)prompt.size() + outLen, numBeams, 1, 1.0f, false, -1, -1, sample, temp, topK, topP, rep);
      m.input(ids, batch);
      double first = 0, rest = 0;
      int steps = 0;
      while (!m.isDone()) {
        auto t0 = std::chrono::steady_clock::now();
        auto next = m.generate();
        double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
        if (steps == 0) first = ms; else rest += ms;
        ++steps;
        if (stream && batch == 1 && numBeams == 1 && m.isMaster()) {
          // ids stream one by one; text is printed once per run below (pieces only join into characters and words in
          // context)
          std::printf("%d ", next[0]);
          std::fflush(stdout);
        }
      }
      auto out = m.finalize();
      if (!m.isMaster()) continue;          // tensor-parallel ranks (mpirun -n N example ...): rank 0 reports
      if (stream && batch == 1 && numBeams == 1) std::printf("\n");
      const size_t w = out.size() / batch;
      for (int b = 0; b < batch; ++b) {
        std::printf("[%d] ", b);
        for (size_t i = prompt.size(); i < w; ++i) std::printf("%d ", out[b * w + i]);
        std::printf("\n");
        if (bpe) {
          std::vector<int32_t> gen(out.begin() + b * w + prompt.size(), out.begin() + (b + 1) * w);
          std::printf("[%d] %s\n", b, bpe->decode(gen).c_str());
        }
        if (tok) {
          std::vector<int32_t> gen(out.begin() + b * w + prompt.size(), out.begin() + (b + 1) * w);
          std::printf("[%d] %s\n", b, tok->decode(gen).c_str());
        }
      }
      std::printf("first token: %.2f ms, next tokens: %.2f ms avg over %d\n", first, steps > 1 ? rest / (steps - 1) : 0.0, steps - 1);
    }
  } catch (const std::exception& e) {
    std::fprintf(stderr, "error: %s\n", e.what());
    return 1;
  }
  return 0;
}
