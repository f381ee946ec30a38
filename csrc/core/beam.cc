#include "beam.h"

#include <algorithm>
#include <cmath>
#include <numeric>

namespace xft {

void BeamHypotheses::add(const std::vector<int32_t>& hyp, double sumLogprobs, int length) {
  const double score = sumLogprobs / std::pow((double)std::max(length, 1), (double)lengthPenalty_);
  if ((int)beams_.size() < numBeams_ || score > worst_) {
    beams_.emplace_back(score, hyp);
    if ((int)beams_.size() > numBeams_) {
      std::stable_sort(beams_.begin(), beams_.end(), [](const auto& a, const auto& b) { return a.first < b.first; });
      beams_.erase(beams_.begin());
      worst_ = beams_.front().first;
    } else {
      worst_ = std::min(score, worst_);
    }
  }
}

bool BeamHypotheses::isDone(double bestSumLogprobs, int curLen) const {
  if ((int)beams_.size() < numBeams_) return false;
  if (earlyStopping_) return true;
  return worst_ >= bestSumLogprobs / std::pow((double)std::max(curLen, 1), (double)lengthPenalty_);
}

BeamSearchScorer::BeamSearchScorer(int batch, int numBeams, float lengthPenalty, bool earlyStopping, int eosId, int padId,
                                   int numReturn)
    : bs_(batch), nb_(numBeams), eos_(eosId), pad_(padId), nret_(std::max(1, std::min(numReturn, numBeams))),
      hyps_(batch, BeamHypotheses(numBeams, lengthPenalty, earlyStopping)), done_(batch, 0),
      scores_((size_t)batch * numBeams, -1e9), seqs_((size_t)batch * numBeams) {
  for (int b = 0; b < batch; ++b) scores_[(size_t)b * numBeams] = 0.0;      // only beam 0 is live at the first step
}

bool BeamSearchScorer::isDone() const {
  return std::all_of(done_.begin(), done_.end(), [](char d) { return d != 0; });
}

void BeamSearchScorer::process(const float* logprobs, int vocab, std::vector<int32_t>& nextTokens, std::vector<int>& srcBeam) {
  const int nb = nb_, k2 = 2 * nb;
  nextTokens.assign((size_t)bs_ * nb, pad_ >= 0 ? pad_ : 0);
  srcBeam.assign((size_t)bs_ * nb, 0);
  std::vector<double> nextScores((size_t)bs_ * nb, 0.0);
  const int gen = (int)seqs_[0].size();              // tokens every open beam has generated so far
  std::vector<std::pair<double, long long>> cand;
  for (int b = 0; b < bs_; ++b) {
    if (done_[b]) {
      for (int j = 0; j < nb; ++j) {
        srcBeam[(size_t)b * nb + j] = b * nb + j;
        nextScores[(size_t)b * nb + j] = scores_[(size_t)b * nb + j];
      }
      continue;
    }
    const int curLen = promptLen(b) + gen;             // the reference ranks by the length of the whole row of ids
    // top 2 * beams of (beam score + log-prob) over beams x vocab; ties go to the lower flat index, as torch.topk
    cand.clear();
    cand.reserve((size_t)nb * vocab);
    for (int j = 0; j < nb; ++j) {
      const float* row = logprobs + ((size_t)b * nb + j) * vocab;
      const double base = scores_[(size_t)b * nb + j];
      for (int v = 0; v < vocab; ++v) cand.emplace_back((double)(float)(row[v] + (float)base), (long long)j * vocab + v);
    }
    const int take = std::min<int>(k2, (int)cand.size());
    std::partial_sort(cand.begin(), cand.begin() + take, cand.end(), [](const auto& a, const auto& c) {
      return a.first > c.first || (a.first == c.first && a.second < c.second);
    });
    int k = 0;
    for (int rank = 0; rank < take; ++rank) {
      const int sb = (int)(cand[rank].second / vocab), t = (int)(cand[rank].second % vocab);
      const double s = cand[rank].first;
      if (t == eos_ && eos_ >= 0) {
        if (rank >= nb) continue;
        std::vector<int32_t> h = seqs_[(size_t)b * nb + sb];
        h.push_back(t);
        hyps_[b].add(h, s, curLen);
      } else {
        nextTokens[(size_t)b * nb + k] = t;
        srcBeam[(size_t)b * nb + k] = b * nb + sb;
        nextScores[(size_t)b * nb + k] = s;
        ++k;
      }
      if (k == nb) break;
    }
    done_[b] = done_[b] || hyps_[b].isDone(take ? cand[0].first : 0.0, curLen);
  }
  std::vector<std::vector<int32_t>> next((size_t)bs_ * nb);
  for (size_t i = 0; i < next.size(); ++i) {
    next[i] = seqs_[srcBeam[i]];
    next[i].push_back(nextTokens[i]);
  }
  seqs_.swap(next);
  scores_.swap(nextScores);
}

std::vector<std::vector<int32_t>> BeamSearchScorer::finalize(const std::vector<std::vector<int32_t>>& prompts, int maxLength) {
  std::vector<std::vector<int32_t>> out;
  for (int b = 0; b < bs_; ++b) {
    if (!done_[b] || (int)hyps_[b].beams().size() < nret_)
      for (int j = 0; j < nb_; ++j) {
        const auto& s = seqs_[(size_t)b * nb_ + j];
        hyps_[b].add(s, scores_[(size_t)b * nb_ + j], promptLen(b) + (int)s.size());
      }
    auto best = hyps_[b].beams();
    std::stable_sort(best.begin(), best.end(), [](const auto& a, const auto& c) { return a.first > c.first; });
    for (int r = 0; r < nret_ && r < (int)best.size(); ++r) {
      std::vector<int32_t> o = prompts[b];
      o.insert(o.end(), best[r].second.begin(), best[r].second.end());
      out.push_back(std::move(o));
    }
  }
  const int32_t pad = pad_ >= 0 ? pad_ : std::max(eos_, 0);
  size_t width = 0;
  for (const auto& o : out) width = std::max(width, o.size());
  width = std::min(width, (size_t)std::max(maxLength, 0));
  for (auto& o : out) o.resize(width, pad);
  return out;
}

void logSoftmaxRow(float* row, int n) {
  float m = row[0];
  for (int i = 1; i < n; ++i) m = std::max(m, row[i]);
  double s = 0.0;
  for (int i = 0; i < n; ++i) s += std::exp((double)(row[i] - m));
  const float lse = m + (float)std::log(s);
  for (int i = 0; i < n; ++i) row[i] -= lse;
}

}  // namespace xft
