// Decoder interface of the C++ API (reference: include/abstract_decoder.h:23-59).  A searcher drives a model through
// it: run the ids of a step, get the logits of the next token, permute the cached keys / values between beams.
//
// Differences from the reference's interface, which exposes host-side internals of the Xeon engine: the logits pointer
// refers to host memory holding fp32 [rows, vocab] of THIS process (the whole vocabulary: split offset 0, split size
// vocab); sequences of the second forward() are named by the ids set_input() returned, not by SequenceMeta pointers;
// getContext() / getMessenger() have no counterpart (the runtime's context is not part of the public API).
#pragma once
#include <cstdint>
#include <memory>
#include <tuple>
#include <vector>

namespace xft {

class Model;

class AbstractDecoder {
public:
  virtual ~AbstractDecoder() {}

  // ids: (batchSize, beamSize, seqLen) = dims[0..2], row-major.  step 0 starts new sequences from these prompts; a
  // later step appends seqLen (normally 1) tokens to each of them.  Returns (logits, splitOffset, splitSize): fp32
  // [batchSize * beamSize (x seqLen with logitsAll), splitSize] of the last (or every) position.
  virtual std::tuple<float*, int, int> forward(int* ids, int64_t* dims, int step, bool logitsAll = false) = 0;

  // continuous batching: run whatever is pending for these sequences (see Model::set_input)
  virtual std::tuple<float*, int, int> forward(const std::vector<int>& seqIDs, bool logitsAll = false) = 0;

  // Reorder cached keys and values: row i continues from the history of row idx[i]; size = batchSize * beamSize
  virtual void reorderCache(int* idx, int size) = 0;

  virtual bool isMaster() = 0;
  virtual int getRank() = 0;
  virtual int getEndId() = 0;

  virtual void setPrefix(int* ids, int seqLen) = 0;
  virtual void unsetPrefix() = 0;
};

// The decoder behind a loaded model (it shares the model's weights, KV cache and sequences; the model must outlive it).
std::unique_ptr<AbstractDecoder> makeDecoder(Model& model);

}  // namespace xft
