// Beam search bookkeeping of the C++ runtime (reference: src/searchers/beam_search.cpp:27-345 — BeamSearchScorer and
// BeamHypotheses, HF semantics).  Host-only: `process` takes the log-probabilities of the current step for every beam
// ([batch * beams, vocab]) and returns the next token and the source beam of every beam; the engine then reorders
// the KV block tables accordingly (block-table fork, no data copy).
#pragma once
#include <cstdint>
#include <utility>
#include <vector>

namespace xft {

class BeamHypotheses {
public:
  BeamHypotheses(int numBeams, float lengthPenalty, bool earlyStopping)
      : numBeams_(numBeams), lengthPenalty_(lengthPenalty), earlyStopping_(earlyStopping) {}
  // score = sumLogprobs / length ^ lengthPenalty
  void add(const std::vector<int32_t>& hyp, double sumLogprobs, int length);
  bool isDone(double bestSumLogprobs, int curLen) const;
  const std::vector<std::pair<double, std::vector<int32_t>>>& beams() const { return beams_; }
private:
  int numBeams_;
  float lengthPenalty_;
  bool earlyStopping_;
  double worst_ = 1e9;
  std::vector<std::pair<double, std::vector<int32_t>>> beams_;
};

class BeamSearchScorer {
public:
  BeamSearchScorer(int batch, int numBeams, float lengthPenalty, bool earlyStopping, int eosId, int padId,
                   int numReturn);
  bool isDone() const;
  // Prompt length of every request (default 0).  As in the reference (src/searchers/beam_search.cpp:87-112,137-194, where
  // a hypothesis is the whole row of input ids), the length that normalises a hypothesis' score is prompt + tokens
  // generated before the closing one.
  void setPromptLens(const std::vector<int>& lens) { promptLens_ = lens; }
  // logprobs: [batch * beams, vocab] (log-softmax of this step).  Outputs have batch * beams entries; srcBeam holds
  // flat indices into the previous step's beams.
  void process(const float* logprobs, int vocab, std::vector<int32_t>& nextTokens, std::vector<int>& srcBeam);
  // best `numReturn` hypotheses per request, prompt prepended, padded to a common width (at most maxLength)
  std::vector<std::vector<int32_t>> finalize(const std::vector<std::vector<int32_t>>& prompts, int maxLength);
  const std::vector<double>& beamScores() const { return scores_; }
private:
  int promptLen(int b) const { return b < (int)promptLens_.size() ? promptLens_[b] : 0; }
  int bs_, nb_, eos_, pad_, nret_;
  std::vector<int> promptLens_;
  std::vector<BeamHypotheses> hyps_;
  std::vector<char> done_;
  std::vector<double> scores_;                       // [batch * beams]
  std::vector<std::vector<int32_t>> seqs_;           // generated tokens per beam
};

// in-place log-softmax of one row
void logSoftmaxRow(float* row, int n);

}  // namespace xft
