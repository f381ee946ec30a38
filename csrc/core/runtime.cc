#include "runtime.h"

#include <algorithm>
#include <cmath>
#include <numeric>
#include <set>

namespace xft {

std::pair<int, int> taskRange(int n, int splits, int idx) {
  if (splits <= 0 || idx < 0 || idx >= splits) throw std::invalid_argument("bad split");
  if (n % (splits * 64) == 0) { int per = n / splits; return {idx * per, (idx + 1) * per}; }
  int gran = 1;
  for (int c : {64, 16, 2}) if (n % c == 0) { n /= c; gran = c; break; }
  int base = n / splits, rem = n % splits, s, e;
  if (idx < rem) { s = idx * (base + 1); e = s + base + 1; }
  else { s = (base + 1) * rem + (idx - rem) * base; e = s + base; }
  return {s * gran, e * gran};
}
std::pair<int, int> taskRangeGran(int n, int gran, int splits, int idx) {
  if (n % gran) throw std::invalid_argument("N must be a multiple of the granularity");
  auto r = taskRange(n / gran, splits, idx);
  return {r.first * gran, r.second * gran};
}
HeadRange headRange(int qHeads, int kvHeads, int splits, int idx) {
  int base = qHeads / splits, rem = qHeads % splits, s, e;
  if (idx < rem) { s = idx * (base + 1); e = s + base + 1; }
  else { s = (base + 1) * rem + (idx - rem) * base; e = s + base; }
  int expand = kvHeads > 0 ? qHeads / kvHeads : 1;
  return {s, e, s / expand, e > s ? (e - 1) / expand + 1 : s / expand};
}

std::pair<int, int> ppLayerRange(int numLayers, int ppSize, int ppRank) {
  if (ppSize <= 0 || ppRank < 0 || ppRank >= ppSize) throw std::invalid_argument("bad pipeline stage");
  const int base = numLayers / ppSize, rem = numLayers % ppSize;
  const int start = ppRank * base + std::min(ppRank, rem);
  return {start, start + base + (ppRank < rem ? 1 : 0)};
}
int moeSliceIndex(int tpRank, int tpSize, int layerId, int expertId, int balanceDim) {
  return (tpRank + (balanceDim == 0 ? layerId : expertId)) % tpSize;
}
std::pair<int, int> expertRange(int numExperts, int epSize, int epRank) {
  if (epSize <= 0 || epRank < 0 || epRank >= epSize) throw std::invalid_argument("bad expert-parallel rank");
  const int base = numExperts / epSize, rem = numExperts % epSize;
  const int start = epRank * base + std::min(epRank, rem);
  return {start, start + base + (epRank < rem ? 1 : 0)};
}
int expertOwner(int expertId, int numExperts, int epSize) {
  const int base = numExperts / epSize, rem = numExperts % epSize;
  const int cut = rem * (base + 1);
  if (expertId < cut) return expertId / (base + 1);
  return rem + (expertId - cut) / std::max(base, 1);
}
std::vector<int> blockVisitOrder(int numBlocks, int world, int rank, int lag) {
  if (lag < 0) lag = world;
  std::vector<int> out;
  out.reserve(numBlocks);
  for (int k = 0; k < numBlocks + lag; ++k) {
    if (k < numBlocks && k % world != rank) out.push_back(k);
    if (k >= lag && (k - lag) % world == rank) out.push_back(k - lag);
  }
  return out;
}

SequenceMeta& SequencePool::create(const std::vector<int32_t>& prompt, int maxLen) {
  for (int tries = 0; tries < kMaxId; ++tries) {
    int id = next_;
    next_ = (next_ + 1) % kMaxId;
    if (!seqs_.count(id)) {
      SequenceMeta& s = seqs_[id];
      s.id = id; s.prompt = prompt; s.pending = prompt; s.maxLen = maxLen;
      return s;
    }
  }
  throw std::runtime_error("no free sequence id");
}
SequenceMeta& SequencePool::get(int id) {
  auto it = seqs_.find(id);
  if (it == seqs_.end()) throw std::out_of_range("unknown sequence id " + std::to_string(id));
  return it->second;
}

void BlockAllocator::grow(int total) {
  int old = (int)ref_.size();
  if (total <= old) return;
  ref_.resize(total, 0);
  std::vector<int> add;
  for (int b = total - 1; b >= old; --b) add.push_back(b);
  free_.insert(free_.begin(), add.begin(), add.end());
}
int BlockAllocator::alloc() {
  if (free_.empty()) throw std::runtime_error("KV cache exhausted");
  int b = free_.back();
  free_.pop_back();
  ref_[b] = 1;
  return b;
}
void BlockAllocator::release(int b) {
  if (--ref_[b] == 0) free_.push_back(b);
  else if (ref_[b] < 0) throw std::logic_error("double free of KV block");
}

void BlockTables::add(int seq) {
  if (tables_.count(seq)) throw std::logic_error("sequence already cached");
  tables_[seq];
  lens_[seq] = 0;
}
void BlockTables::free(int seq) {
  auto it = tables_.find(seq);
  if (it == tables_.end()) return;
  for (int b : it->second) alloc_.release(b);
  tables_.erase(it);
  lens_.erase(seq);
}
void BlockTables::fork(int src, int dst) {
  free(dst);
  auto& d = tables_[dst];
  for (int b : tables_.at(src)) d.push_back(alloc_.share(b));
  lens_[dst] = lens_.at(src);
}
void BlockTables::truncate(int seq, int newLen) {
  auto& tab = tables_.at(seq);
  size_t keep = (newLen + bs_ - 1) / bs_;
  for (size_t i = keep; i < tab.size(); ++i) alloc_.release(tab[i]);     // same release order as the Python twin
  if (tab.size() > keep) tab.resize(keep);
  lens_[seq] = newLen;
}
void BlockTables::reorder(const std::vector<int>& seqs, const std::vector<int>& srcIndex) {
  std::map<int, std::vector<int>> fresh;
  std::map<int, int> nl;
  for (size_t i = 0; i < seqs.size(); ++i) {
    int src = seqs[srcIndex[i]];
    for (int b : tables_.at(src)) fresh[seqs[i]].push_back(alloc_.share(b));
    nl[seqs[i]] = lens_.at(src);
  }
  for (int s : seqs) for (int b : tables_.at(s)) alloc_.release(b);
  for (int s : seqs) { tables_[s] = fresh[s]; lens_[s] = nl[s]; }
}

void repetitionPenalty(float* logits, int n, const std::vector<int32_t>& tokens, float penalty, int vocabOffset) {
  if (penalty == 1.0f) return;
  std::set<int32_t> uniq(tokens.begin(), tokens.end());
  for (int32_t t : uniq) {
    int c = t - vocabOffset;
    if (c < 0 || c >= n) continue;
    logits[c] = logits[c] < 0 ? logits[c] * penalty : logits[c] / penalty;
  }
}
bool matchStopWords(const std::vector<int32_t>& g, const std::vector<std::vector<int>>& sw) {
  for (auto& w : sw) {
    if (w.empty() || w.size() > g.size()) continue;
    if (std::equal(w.begin(), w.end(), g.end() - w.size())) return true;
  }
  return false;
}
std::vector<std::vector<int>> cleanStopWords(const std::vector<std::vector<int>>& in, int eos) {
  std::vector<std::vector<int>> out;
  for (auto& w : in) {
    if (w.empty()) continue;
    if (std::any_of(w.begin(), w.end(), [](int t) { return t <= 0; })) continue;
    if (w.size() == 1 && w[0] == eos) continue;
    out.push_back(w);
  }
  return out;
}
int argmaxFirst(const float* l, int n) {
  int bi = 0;
  for (int i = 1; i < n; ++i) if (l[i] > l[bi]) bi = i;
  return bi;
}
int sampleTopKTopP(const float* logits, int n, int topK, float topP, float temperature, float u) {
  int k = std::max(1, std::min(topK, n));
  std::vector<int> idx(n);
  std::iota(idx.begin(), idx.end(), 0);
  std::partial_sort(idx.begin(), idx.begin() + k, idx.end(), [&](int a, int b) { return logits[a] > logits[b] || (logits[a] == logits[b] && a < b); });
  float invT = 1.0f / std::max(temperature, 1e-6f), mx = logits[idx[0]] * invT;
  std::vector<double> p(k);
  double den = 0;
  for (int i = 0; i < k; ++i) { p[i] = std::exp(logits[idx[i]] * invT - mx); den += p[i]; }
  int keep = k;
  if (topP < 1.0f && k > 1) {
    double c = 0;
    keep = 0;
    for (int i = 0; i < k; ++i) { if (i >= 2 && c >= topP) break; c += p[i] / den; keep = i + 1; }
  }
  double den2 = 0;
  for (int i = 0; i < keep; ++i) den2 += p[i];
  double target = std::min(std::max((double)u, 0.0), 1.0 - 1e-7) * den2, c = 0;
  for (int i = 0; i < keep; ++i) { c += p[i]; if (c > target) return idx[i]; }
  return idx[keep - 1];
}

}  // namespace xft
