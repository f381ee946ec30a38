// Tensor-parallel self-check of the C++ API on ONE GPU: the model runs once on a single rank and once as N ranks that
// are threads of this process (csrc/core/comm.h: they take turns, collectives are done on the host side of the device
// queue), and the logits of the prompt pass and of a few decode steps are compared.  What it covers: the head / FFN /
// vocabulary ranges every rank loads, bias and residual entering once, the sums after the two row-parallel projections,
// the gathered head — everything of the multi-process NCCL mode except the NCCL calls themselves.  With -s the ranks
// form that many pipeline stages (ranks / stages tensor-parallel ranks each), as XFT_PIPELINE_STAGE does for processes.
//
//   tp_check -m <model dir> [-n ranks] [-s stages] [-d bf16|int8|...] [--kv_cache_dtype fp16|int8] [-o decode steps] [--tol t]
//
// (The reference has no counterpart: its ranks are always MPI processes.)
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include "comm.h"
#include "xft/models.h"

namespace {

struct Trace {
  std::vector<std::vector<float>> logits;      // one [batch * vocab] block per step
  std::vector<std::vector<int32_t>> tokens;    // the token fed after each step
  std::string error;
};

// prompt pass + `steps` decode steps through the continuous-batching calls; `forced` (from the single-rank run) decides
// the tokens when given, else the arg-max does
void run(xft::Model& m, std::vector<std::vector<int32_t>> prompts, int steps, const Trace* forced, Trace& out) {
  const int B = (int)prompts.size();
  std::vector<int> ids = m.set_input(prompts, std::vector<int>{}, 256);
  for (int s = 0; s <= steps; ++s) {
    auto r = m.forward(false);
    const float* lg = std::get<0>(r);
    const int rows = std::get<1>(r), V = std::get<2>(r);
    if (rows != B) throw std::runtime_error("unexpected number of logits rows");
    out.logits.emplace_back(lg, lg + (size_t)rows * V);
    if (s == steps) break;
    std::vector<int32_t> next(B);
    for (int b = 0; b < B; ++b)
      next[b] = forced ? forced->tokens[s][b] : (int32_t)(std::max_element(lg + (size_t)b * V, lg + (size_t)(b + 1) * V) - (lg + (size_t)b * V));
    out.tokens.push_back(next);
    std::vector<std::vector<int32_t>> step(B);
    for (int b = 0; b < B; ++b) step[b] = {next[b]};
    m.set_input(step, ids, 256);
  }
  m.freeSeqs(ids);
}

}  // namespace

int main(int argc, char** argv) {
  std::string model, dtype = "bf16", kv = "fp16";
  int ranks = 2, steps = 4, stages = 0;
  double tol = 0.05;
  for (int i = 1; i < argc; ++i) {
    const std::string a = argv[i];
    auto next = [&]() -> std::string { if (i + 1 >= argc) { std::fprintf(stderr, "missing value for %s\n", a.c_str()); std::exit(2); } return argv[++i]; };
    if (a == "-m") model = next();
    else if (a == "-n") ranks = std::atoi(next().c_str());
    else if (a == "-s") stages = std::atoi(next().c_str());
    else if (a == "-d") dtype = next();
    else if (a == "--kv_cache_dtype") kv = next();
    else if (a == "-o") steps = std::atoi(next().c_str());
    else if (a == "--tol") tol = std::atof(next().c_str());
    else { std::fprintf(stderr, "unknown flag %s\n", a.c_str()); return 2; }
  }
  if (model.empty() || ranks < 2 || ranks > 8 || stages < 0 || (stages > 0 && ranks % stages)) {
    std::fprintf(stderr, "usage: tp_check -m <model dir> [-n 2..8] [-s stages, a divisor of the ranks] [-d dtype] [-o steps]\n");
    return 2;
  }
  // the runtime reads its flags once, at first use: set the stage count before any model exists
  if (stages > 0) setenv("XFT_PIPELINE_STAGE", std::to_string(stages).c_str(), 1);
  const xft::DataType wdt = xft::dataTypeFromName(dtype.c_str());
  const xft::DataType kdt = kv == "int8" ? xft::DataType::int8 : xft::DataType::fp16;
  if (wdt == xft::DataType::unknown) { std::fprintf(stderr, "unknown weight type %s\n", dtype.c_str()); return 2; }
  const std::vector<std::vector<int32_t>> prompts = {{5, 17, 99, 200, 3, 42, 7, 150, 23, 64, 11}, {9, 8, 250, 6, 5, 4, 3}};
  Trace single;
  try {
    xft::AutoModel m(model, wdt, kdt, nullptr);
    run(m, prompts, steps, nullptr, single);
  } catch (const std::exception& e) {
    std::fprintf(stderr, "single rank: %s\n", e.what());
    return 1;
  }
  auto comms = xft::makeThreadCommunicators(ranks);
  std::vector<Trace> traces(ranks);
  std::vector<std::thread> threads;
  for (int r = 0; r < ranks; ++r)
    threads.emplace_back([&, r] {
      try {
        comms[r]->begin();
        xft::AutoModel m(model, wdt, kdt, comms[r]);
        // ranks other than 0 pass nothing: rank 0's arguments reach them through the communicator
        run(m, r == 0 ? prompts : std::vector<std::vector<int32_t>>(prompts.size()), steps, &single, traces[r]);
      } catch (const std::exception& e) {
        traces[r].error = e.what();
      }
      comms[r]->end();
    });
  for (auto& t : threads) t.join();
  for (int r = 0; r < ranks; ++r)
    if (!traces[r].error.empty()) { std::fprintf(stderr, "rank %d: %s\n", r, traces[r].error.c_str()); return 1; }
  double worst = 0, top = 0;
  for (int r = 0; r < ranks; ++r) {
    if (traces[r].logits.size() != single.logits.size()) { std::fprintf(stderr, "rank %d ran %zu steps\n", r, traces[r].logits.size()); return 1; }
    for (size_t s = 0; s < single.logits.size(); ++s) {
      if (traces[r].logits[s].size() != single.logits[s].size()) { std::fprintf(stderr, "rank %d: logits size differs\n", r); return 1; }
      for (size_t i = 0; i < single.logits[s].size(); ++i) {
        worst = std::max(worst, (double)std::fabs(traces[r].logits[s][i] - single.logits[s][i]));
        top = std::max(top, (double)std::fabs(single.logits[s][i]));
      }
    }
  }
  std::printf("%d thread ranks vs one rank: %zu steps, max |logit difference| %.4f (largest |logit| %.3f)\n", ranks,
              single.logits.size(), worst, top);
  if (!(worst <= tol * std::max(top, 1.0))) { std::printf("MISMATCH\n"); return 1; }
  std::printf("tensor-parallel ranks agree\n");
  return 0;
}
