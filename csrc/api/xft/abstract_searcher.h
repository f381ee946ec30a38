// Searcher configuration of the C++ API (reference: include/abstract_searcher.h:20-67).
#pragma once
#include <vector>

struct SearcherConfig {
  bool doEarlyStopping = false;
  bool doSample = false;
  int maxLen = -1;
  int numBeams = 1;
  int numBeamHypsToKeep = 1;
  int eosTokenId = -1;
  int padTokenId = -1;
  int topK = 50;
  float lenPenalty = 1.0f;
  float temperature = 1.0f;
  float topP = 1.0f;
  float repetitionPenalty = 1.0f;
  unsigned long long seed = 0;     // extension: 0 = time-based

  SearcherConfig(int maxLen_ = -1, int numBeams_ = 1, int numBeamHypsToKeep_ = 1, float lenPenalty_ = 1.0f,
                 bool doEarlyStopping_ = false, int eosTokenId_ = -1, int padTokenId_ = -1, bool doSample_ = false,
                 float temperature_ = 1.0f, int topK_ = 50, float topP_ = 1.0f, float repetitionPenalty_ = 1.0f)
      : doEarlyStopping(doEarlyStopping_), doSample(doSample_), maxLen(maxLen_), numBeams(numBeams_),
        numBeamHypsToKeep(numBeamHypsToKeep_), eosTokenId(eosTokenId_), padTokenId(padTokenId_), topK(topK_),
        lenPenalty(lenPenalty_), temperature(temperature_), topP(topP_), repetitionPenalty(repetitionPenalty_) {}
};
