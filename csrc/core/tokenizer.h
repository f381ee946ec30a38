// Text <-> token ids for the C++ command-line example: a reader of SentencePiece model files (`tokenizer.model` of the
// Llama / Mistral / Gemma / Yi / Baichuan / ChatGLM families) with the two segmentation algorithms those files use.
//
// The reference's example links the sentencepiece library (and bakes vocabularies for OPT and Qwen into headers,
// examples/cpp/example.cpp:60-350); here the model file is parsed directly (it is a protobuf message with three fields
// of interest) so the example needs no third-party library:
//   * BPE models (Llama-2, Mistral, ...): start from UTF-8 characters and repeatedly merge the adjacent pair whose
//     concatenation is the best-scoring piece of the vocabulary (leftmost on ties), as sentencepiece's bpe_model does;
//   * unigram models (T5-style, ChatGLM): Viterbi segmentation that maximises the sum of piece scores;
//   * characters that no piece covers fall back to byte pieces <0xNN> when the model has them, else to <unk>.
// Normalisation covers what these chat models rely on: the optional dummy prefix, spaces escaped as U+2581, optional
// collapsing of repeated spaces.  The precompiled NFKC character map of a model file is NOT applied: text that NFKC
// would change (full-width forms, ligatures, ...) can tokenise differently from the sentencepiece library.
#pragma once
#include <cstdint>
#include <string>
#include <unordered_map>
#include <vector>

namespace xft {

class SentencePieceTokenizer {
public:
  // Parses a SentencePiece model file; throws std::runtime_error when the file is missing or malformed.
  explicit SentencePieceTokenizer(const std::string& modelPath);

  std::vector<int32_t> encode(const std::string& text, bool addBos = false, bool addEos = false) const;
  std::string decode(const std::vector<int32_t>& ids) const;

  int vocabSize() const { return (int)pieces_.size(); }
  int bosId() const { return bos_; }
  int eosId() const { return eos_; }
  int unkId() const { return unk_; }
  bool isBpe() const { return bpe_; }
  const std::string& piece(int id) const { return pieces_.at(id).text; }

private:
  enum PieceType { NORMAL = 1, UNKNOWN = 2, CONTROL = 3, USER_DEFINED = 4, UNUSED = 5, BYTE = 6 };
  struct Piece {
    std::string text;
    float score = 0.f;
    int type = NORMAL;
  };
  std::string normalize(const std::string& text) const;
  void encodeBpe(const std::string& norm, std::vector<int32_t>& out) const;
  void encodeUnigram(const std::string& norm, std::vector<int32_t>& out) const;
  void emitUnknown(const std::string& ch, std::vector<int32_t>& out) const;

  std::vector<Piece> pieces_;
  std::unordered_map<std::string, int> index_;     // NORMAL / USER_DEFINED pieces by text
  int byteId_[256];
  bool hasBytes_ = false;
  bool bpe_ = false;
  bool addDummyPrefix_ = true, removeExtraSpaces_ = true, escapeSpaces_ = true;
  int unk_ = 0, bos_ = 1, eos_ = 2;
  size_t maxPieceBytes_ = 1;
};

}  // namespace xft
