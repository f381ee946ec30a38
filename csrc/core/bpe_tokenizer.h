// Byte-level BPE tokenizer for the C++ command-line example: the `tokenizer.json` of the GPT-2 lineage (OPT, Qwen 1.5 /
// 2 / 3, Llama-3, Mixtral-style fast tokenizers), or the older `vocab.json` + `merges.txt` pair.
//
// The reference's example bakes the OPT and Qwen vocabularies into headers (examples/cpp/vocab_opt.h, vocab_qwen.h,
// example.cpp:60-350); here the files that ship with every Hugging Face checkpoint are read instead:
//   * text is cut into pieces by the pre-tokenizer pattern — GPT-2's ('s|'t|…| ?letters| ?digits| ?other|spaces) or
//     the tiktoken-style one of Llama-3 / Qwen (case-insensitive contractions, digits in groups of up to 3 or 1,
//     newlines kept with the preceding symbols) — recognised from the pattern string in tokenizer.json;
//   * every piece is mapped byte by byte to the printable alphabet of GPT-2 and merged pair by pair in merge-rank
//     order; the merged strings are looked up in the vocabulary;
//   * decoding concatenates the token strings and maps the alphabet back to bytes; added (special) tokens print as
//     their text and are recognised in the input when they appear literally.
// Character classes: ASCII letters / digits / whitespace are exact; every code point above U+007F counts as a letter
// (true for accented Latin, Greek, Cyrillic, CJK, Hangul …), so non-ASCII punctuation, digits or spaces can split
// differently from the Hugging Face implementation.
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <unordered_map>
#include <vector>

namespace xft {

class BpeTokenizer {
public:
  // `path`: a tokenizer.json, or a directory holding tokenizer.json or vocab.json + merges.txt.
  // Throws std::runtime_error when nothing usable is found or a file is malformed.
  explicit BpeTokenizer(const std::string& path);

  std::vector<int32_t> encode(const std::string& text) const;
  std::string decode(const std::vector<int32_t>& ids) const;

  int vocabSize() const { return (int)idToToken_.size(); }
  // id of an added token such as "<|endoftext|>", or -1
  int specialId(const std::string& text) const;
  const char* pattern() const { return style_ == 0 ? "gpt2" : digitGroup_ == 3 ? "llama3" : "qwen2"; }

private:
  void loadTokenizerJson(const std::string& file);
  void loadVocabMerges(const std::string& vocabFile, const std::string& mergesFile);
  void finish();
  std::vector<std::string> split(const std::string& text) const;       // pre-tokenizer
  void bpe(const std::string& piece, std::vector<int32_t>& out) const;

  std::unordered_map<std::string, int> vocab_;                          // token string (GPT-2 alphabet) -> id
  std::vector<std::string> idToToken_;
  std::unordered_map<std::string, int> mergeRank_;                      // "left right" -> rank
  std::vector<std::pair<std::string, int>> special_;                    // added tokens, longest first
  std::vector<char> isSpecial_;
  std::string byteToUni_[256];                                          // byte -> UTF-8 of its alphabet character
  std::unordered_map<std::string, int> uniToByte_;
  int style_ = 0;                                                       // 0 GPT-2 pattern, 1 tiktoken-style
  int digitGroup_ = 3;                                                  // tiktoken-style: digits per piece
  int unk_ = -1;
  bool ignoreMerges_ = false;                                           // whole pieces that are tokens skip the merges (Llama-3)
};

}  // namespace xft
