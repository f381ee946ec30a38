// Host-side runtime pieces of the C++ engine: layout arithmetic, sequences, the paged KV block allocator and
// samplers.  C++ twins of parallel/partition.py, runtime/sequence.py, runtime/kv_cache.py, runtime/sampler.py
// (reference: src/utils/split_util.h, src/common/sequence.h, src/common/kvcache_mgr.h, src/searchers/*).
#pragma once
#include <cstdint>
#include <map>
#include <stdexcept>
#include <utility>
#include <vector>

namespace xft {

// ---- SplitUtil (src/utils/split_util.h:8-99) --------------------------------------------------------------
std::pair<int, int> taskRange(int n, int splits, int idx);
std::pair<int, int> taskRangeGran(int n, int gran, int splits, int idx);
struct HeadRange { int q0, q1, kv0, kv1; };
HeadRange headRange(int qHeads, int kvHeads, int splits, int idx);
// layers of one pipeline stage (src/layers/decoder_block.h:33-40; a remainder goes to the first stages)
std::pair<int, int> ppLayerRange(int numLayers, int ppSize, int ppRank);
// rotated tensor-parallel slice of an expert, so uneven slices even out over layers (dim 0) or experts (dim 1)
// (src/layers/mlp_llama.h:70-79, XFT_MOE_SPLIT_BALANCE_DIM)
int moeSliceIndex(int tpRank, int tpSize, int layerId, int expertId, int balanceDim);
// expert parallelism: contiguous block of experts per rank, and the rank that owns an expert
std::pair<int, int> expertRange(int numExperts, int epSize, int epRank);
int expertOwner(int expertId, int numExperts, int epSize);
// fused prefill GEMM + all-reduce: order in which a rank visits the token blocks (its own blocks `lag` steps late;
// lag < 0 = one round of `world`)
std::vector<int> blockVisitOrder(int numBlocks, int world, int rank, int lag = -1);

// ---- sequences (src/common/sequence.h) ----------------------------------------------------------------------
struct SequenceMeta {
  int id = 0;
  std::vector<int32_t> prompt, generated, pending;
  int pastLen = 0, maxLen = 0;
  bool done = false;
  int totalLen() const { return (int)(prompt.size() + generated.size()); }
  void stepForward(int32_t tok) { pastLen += (int)pending.size(); generated.push_back(tok); pending.assign(1, tok); }
};

class SequencePool {
public:
  static constexpr int kMaxId = 10240;     // ids wrap like the reference's SequenceIDManager
  SequenceMeta& create(const std::vector<int32_t>& prompt, int maxLen);
  SequenceMeta& get(int id);
  bool has(int id) const { return seqs_.count(id) != 0; }
  void remove(int id) { seqs_.erase(id); }
private:
  std::map<int, SequenceMeta> seqs_;
  int next_ = 0;
};

// ---- paged KV block allocator with reference counts ---------------------------------------------------------
class BlockAllocator {
public:
  explicit BlockAllocator(int n = 0) { grow(n); }
  void grow(int total);
  int numBlocks() const { return (int)ref_.size(); }
  int numFree() const { return (int)free_.size(); }
  int alloc();
  int share(int b) { ++ref_[b]; return b; }
  void release(int b);
  int refs(int b) const { return ref_[b]; }
private:
  std::vector<int> free_, ref_;
};

class BlockTables {
public:
  BlockTables(int blockSize, int numBlocks) : bs_(blockSize), alloc_(numBlocks) {}
  void add(int seq);
  void free(int seq);
  void fork(int src, int dst);                       // dst shares src's blocks (prefix / beam)
  // Reserve n positions; returns slot ids.  cow(srcBlock, dstBlock) is invoked when a shared tail block is split.
  template <class Cow>
  std::vector<int> append(int seq, int n, Cow cow);
  void truncate(int seq, int newLen);
  void reorder(const std::vector<int>& seqs, const std::vector<int>& srcIndex);
  const std::vector<int>& table(int seq) const { return tables_.at(seq); }
  int len(int seq) const { return lens_.at(seq); }
  int blockSize() const { return bs_; }
  BlockAllocator& allocator() { return alloc_; }
private:
  int bs_;
  BlockAllocator alloc_;
  std::map<int, std::vector<int>> tables_;
  std::map<int, int> lens_;
};

template <class Cow>
std::vector<int> BlockTables::append(int seq, int n, Cow cow) {
  auto& tab = tables_.at(seq);
  int cur = lens_.at(seq);
  if (cur % bs_ && !tab.empty() && alloc_.refs(tab.back()) > 1) {
    int nb = alloc_.alloc();
    cow(tab.back(), nb);
    alloc_.release(tab.back());
    tab.back() = nb;
  }
  int need = (cur + n + bs_ - 1) / bs_ - (int)tab.size();
  for (int i = 0; i < need; ++i) tab.push_back(alloc_.alloc());
  std::vector<int> slots;
  for (int p = cur; p < cur + n; ++p) slots.push_back(tab[p / bs_] * bs_ + p % bs_);
  lens_[seq] = cur + n;
  return slots;
}

// ---- samplers / logits processors (src/searchers/*) -------------------------------------------------------------
// l < 0 ? l*p : l/p on the distinct ids of `tokens` that fall in [vocabOffset, vocabOffset + n)
void repetitionPenalty(float* logits, int n, const std::vector<int32_t>& tokens, float penalty, int vocabOffset = 0);
bool matchStopWords(const std::vector<int32_t>& generated, const std::vector<std::vector<int>>& stopWords);
std::vector<std::vector<int>> cleanStopWords(const std::vector<std::vector<int>>& in, int eos);
int argmaxFirst(const float* logits, int n);
// top-k -> /T -> top-p (keeps >= 2) -> softmax -> inverse CDF with uniform u
int sampleTopKTopP(const float* logits, int n, int topK, float topP, float temperature, float u);

}  // namespace xft
