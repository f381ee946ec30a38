// C++ generation API: xft::Model / xft::AutoModel (reference: include/models.h:25-133, src/models/models.cpp).
//
//   xft::AutoModel model("/path/to/converted-model", xft::DataType::bf16);
//   model.config(/*maxLen*/ 128);  model.input(ids, batch);
//   while (!model.isDone()) { auto next = model.generate(); }
//   auto all = model.finalize();
//
// and the continuous-batching calls set_input(ids, seqIDs, maxLen) / forward() / freeSeqs().  The native engine
// runs all sixteen families on one B200: llama, yarn_llama, gemma, qwen, qwen2, qwen3, baichuan (RoPE or ALiBi), chatglm,
// chatglm2 / 3 / 4, gpt (OPT), telechat, the routed-expert families mixtral and qwen3_moe, and deepseek_moe (latent
// attention, shared + routed experts; from e4m3 checkpoints the routed experts stay e4m3 on the device, the rest is
// dequantised to bf16 at load).  Dense families take bf16 / fp16,
// int8, w8a8, int4, nf4 weights (quantised at load) and the hybrid types (one form for the prompt pass, one for decode
// steps), from dense or GPTQ-converted checkpoints; Mixtral and Qwen3-MoE take the quantised and hybrid types (experts keep the
// quantised values in bf16), DeepSeek runs in bf16.  Every family also runs on several
// ranks: heads, FFN rows and lm_head rows are split as the reference splits them; routed experts are kept whole, a run
// of experts per rank, every rank routing every token (DeepSeek: query heads with their slices of the up-projections,
// the shared experts by columns).  It uses the same sm_100a kernels as the Python
// package — greedy, top-k / top-p sampling and beam search (host scorer, beams fork and reorder paged KV block tables);
// errors are exceptions (std::runtime_error), never exit().
#pragma once
#include <cstdint>
#include <memory>
#include <string>
#include <tuple>
#include <vector>

#include "abstract_decoder.h"
#include "abstract_searcher.h"
#include "dtype.h"

namespace xft {

class Engine;         // csrc/core/engine.cc
class Communicator;   // csrc/core/comm.h

class Model {
public:
  Model();
  ~Model();

  void input(std::vector<int32_t>& inputIds, int batchSize);

  void config(int maxLen = -1, int numBeams = 1, int numBeamHypsToKeep = 1, float lenPenalty = 1.0f,
              bool doEarlyStopping = false, int eosTokenId = -1, int padTokenId = -1, bool doSample = false,
              float temperature = 1.0f, int topK = 50, float topP = 1.0f, float repetitionPenalty = 1.0f,
              const std::vector<std::vector<int>>& stopWordsList = {});
  void config(SearcherConfig& cfg, const std::vector<std::vector<int>>& stopWordsList = {});

  // batch of equal-length prompts + generation config; returns the sequence ids
  std::vector<int> set_input(std::vector<int32_t>& inputIds, int batchSize, int maxLen = -1, int numBeams = 1,
                             int numBeamHypsToKeep = 1, float lenPenalty = 1.0f, bool doEarlyStopping = false,
                             int eosTokenId = -1, int padTokenId = -1, bool doSample = false, float temperature = 1.0f,
                             int topK = 50, float topP = 1.0f, float repetitionPenalty = 1.0f,
                             const std::vector<std::vector<int>>& stopWordsList = {});
  std::vector<int> set_input(std::vector<int32_t>& inputIds, int batchSize, SearcherConfig& cfg,
                             const std::vector<std::vector<int>>& stopWordsList = {});
  std::vector<int> set_input(std::vector<std::vector<int32_t>>& inputIds, SearcherConfig& cfg,
                             const std::vector<std::vector<int>>& stopWordsList = {});
  std::vector<int> set_input(std::vector<std::vector<int32_t>>& inputIds, int maxLen = -1, int numBeams = 1,
                             int numBeamHypsToKeep = 1, float lenPenalty = 1.0f, bool doEarlyStopping = false,
                             int eosTokenId = -1, int padTokenId = -1, bool doSample = false, float temperature = 1.0f,
                             int topK = 50, float topP = 1.0f, float repetitionPenalty = 1.0f,
                             const std::vector<std::vector<int>>& stopWordsList = {});
  std::vector<int> set_input(std::vector<std::vector<int32_t>>& inputIds, std::vector<int> seqIDs, SearcherConfig& cfg,
                             const std::vector<std::vector<int>>& stopWordsList = {});
  // continuous batching (used with forward()): new prompts when seqIDs is empty, else one next token per sequence.
  // maxLen as a vector: empty = the model's limit, one value for all, or one per new sequence.  (As in the reference,
  // a call with only the ids is ambiguous between this group and the one above: pass seqIDs or maxLen.)
  std::vector<int> set_input(std::vector<std::vector<int32_t>>& inputIds, std::vector<int> seqIDs = {}, int maxLen = -1);
  std::vector<int> set_input(std::vector<int32_t>& inputIds, int batchSize, std::vector<int> seqIDs = {}, int maxLen = -1);
  std::vector<int> set_input(std::vector<int32_t>& inputIds, int batchSize, std::vector<int> seqIDs, const std::vector<int>& maxLen);
  std::vector<int> set_input(std::vector<int32_t>& inputIds, std::vector<int32_t>& seqLens, std::vector<int> seqIDs,
                             std::vector<int>& maxLen);

  bool isDone();
  // logits of the scheduled sequences: (pointer to fp32 [rows, vocab] on the host, rows, vocab)
  // (the default follows the reference: every position of a prompt pass; pass false for the last position only)
  std::tuple<float*, int, int> forward(bool logitsAll = true);
  void createSearcher(SearcherConfig& cfg);      // the reference's name for config(cfg)
  std::vector<int32_t> generate();     // one step: next token of every sequence of the current request
  std::vector<int32_t> finalize();     // prompt + generated, flattened, rows padded to equal length
  bool freeSeqs(std::vector<int>& seqIDs);
  void setPrefix(std::vector<int32_t>& prefixIDs);
  void unsetPrefix();
  bool setStopWords(std::vector<std::vector<int>> stopWordsList);

  // Tensor-parallel ranks (one process per GPU, or thread ranks of one process) all make the same calls; the arguments
  // of rank 0 (the master) are the ones every rank uses, as in the reference.
  bool isMaster();
  int getRank();
  int getWorldSize();
  int getBatchSize() { return batchSize; }
  int getSeqLen() { return seqLen; }
  int getVocabSize();
  int getMaxSeqLen();
  SearcherConfig getConfig() { return configuration; }
  void exitSlaves() {}

protected:
  friend class ModelDecoder;          // the AbstractDecoder view of this model (makeDecoder)
  void load(const std::string& path, DataType dt, DataType kv, std::shared_ptr<Communicator> comm = nullptr);
  std::vector<int> cbSetInput(std::vector<std::vector<int32_t>>& ids, std::vector<int>& seqIDs, std::vector<int>& maxLens);
  std::unique_ptr<Engine> engine;
  SearcherConfig configuration;
  std::vector<std::vector<int>> stopWords;
  int batchSize = 0, seqLen = 0;
};

class AutoModel : public Model {
public:
  // Rank and world size come from the launcher's environment (RANK / WORLD_SIZE, OMPI_COMM_WORLD_*, PMI_*): with more
  // than one rank the dense families run tensor-parallel, one GPU per process, over NCCL.
  AutoModel(std::string modelPath, xft::DataType dataType, xft::DataType KVCacheDataType = xft::DataType::fp16);
  // The same with an explicit communicator (csrc/core/comm.h: process ranks, or thread ranks inside one process).
  AutoModel(std::string modelPath, xft::DataType dataType, xft::DataType KVCacheDataType, std::shared_ptr<Communicator> comm);
};

}  // namespace xft
