#include "tokenizer.h"

#include <cstdio>
#include <cstring>
#include <fstream>
#include <limits>
#include <sstream>
#include <stdexcept>

namespace xft {
namespace {

const char kSpace[] = "\xE2\x96\x81";      // U+2581, the escaped space of SentencePiece

// ---- just enough of the protobuf wire format: varints, length-delimited fields, fixed 32 / 64 ----------------
struct Reader {
  const uint8_t* p;
  const uint8_t* end;
  bool more() const { return p < end; }
  uint64_t varint() {
    uint64_t v = 0;
    for (int shift = 0; shift < 64; shift += 7) {
      if (p >= end) throw std::runtime_error("tokenizer model: truncated varint");
      const uint8_t b = *p++;
      v |= (uint64_t)(b & 0x7f) << shift;
      if (!(b & 0x80)) return v;
    }
    throw std::runtime_error("tokenizer model: varint too long");
  }
  Reader sub() {
    const uint64_t n = varint();
    if (n > (uint64_t)(end - p)) throw std::runtime_error("tokenizer model: field runs past the end");
    Reader r{p, p + n};
    p += n;
    return r;
  }
  void skip(int wire) {
    if (wire == 0) varint();
    else if (wire == 1) { if (end - p < 8) throw std::runtime_error("tokenizer model: truncated"); p += 8; }
    else if (wire == 2) sub();
    else if (wire == 5) { if (end - p < 4) throw std::runtime_error("tokenizer model: truncated"); p += 4; }
    else throw std::runtime_error("tokenizer model: unsupported wire type");
  }
};

// length in bytes of the UTF-8 character that starts at s[i] (1 for a stray continuation byte)
size_t utf8Len(const std::string& s, size_t i) {
  const uint8_t c = (uint8_t)s[i];
  size_t n = c < 0x80 ? 1 : (c >> 5) == 6 ? 2 : (c >> 4) == 14 ? 3 : (c >> 3) == 30 ? 4 : 1;
  if (i + n > s.size()) n = s.size() - i;
  return n;
}

}  // namespace

SentencePieceTokenizer::SentencePieceTokenizer(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) throw std::runtime_error("cannot open tokenizer model " + path);
  std::stringstream ss;
  ss << f.rdbuf();
  const std::string buf = ss.str();
  for (int& b : byteId_) b = -1;
  Reader r{(const uint8_t*)buf.data(), (const uint8_t*)buf.data() + buf.size()};
  int modelType = 1;      // UNIGRAM unless the trainer spec says otherwise
  while (r.more()) {
    const uint64_t key = r.varint();
    const int field = (int)(key >> 3), wire = (int)(key & 7);
    if (field == 1 && wire == 2) {                       // repeated SentencePiece pieces
      Reader m = r.sub();
      Piece pc;
      while (m.more()) {
        const uint64_t k = m.varint();
        const int fd = (int)(k >> 3), w = (int)(k & 7);
        if (fd == 1 && w == 2) { Reader s = m.sub(); pc.text.assign((const char*)s.p, s.end - s.p); }
        else if (fd == 2 && w == 5) { if (m.end - m.p < 4) throw std::runtime_error("tokenizer model: truncated score"); std::memcpy(&pc.score, m.p, 4); m.p += 4; }
        else if (fd == 3 && w == 0) pc.type = (int)m.varint();
        else m.skip(w);
      }
      pieces_.push_back(pc);
    } else if (field == 2 && wire == 2) {                // TrainerSpec
      Reader m = r.sub();
      while (m.more()) {
        const uint64_t k = m.varint();
        const int fd = (int)(k >> 3), w = (int)(k & 7);
        if (w != 0) { m.skip(w); continue; }
        const int64_t v = (int64_t)m.varint();
        if (fd == 3) modelType = (int)v;
        else if (fd == 40) unk_ = (int)v;
        else if (fd == 41) bos_ = (int)v;
        else if (fd == 42) eos_ = (int)v;
      }
    } else if (field == 3 && wire == 2) {                // NormalizerSpec
      Reader m = r.sub();
      while (m.more()) {
        const uint64_t k = m.varint();
        const int fd = (int)(k >> 3), w = (int)(k & 7);
        if (w != 0) { m.skip(w); continue; }
        const uint64_t v = m.varint();
        if (fd == 3) addDummyPrefix_ = v != 0;
        else if (fd == 4) removeExtraSpaces_ = v != 0;
        else if (fd == 5) escapeSpaces_ = v != 0;
      }
    } else {
      r.skip(wire);
    }
  }
  if (pieces_.empty()) throw std::runtime_error("tokenizer model " + path + " holds no pieces");
  if (modelType != 1 && modelType != 2) throw std::runtime_error("tokenizer model: only unigram and BPE models are supported");
  bpe_ = modelType == 2;
  for (int i = 0; i < (int)pieces_.size(); ++i) {
    const Piece& pc = pieces_[i];
    if (pc.type == NORMAL || pc.type == USER_DEFINED) {
      index_.emplace(pc.text, i);
      if (pc.text.size() > maxPieceBytes_) maxPieceBytes_ = pc.text.size();
    } else if (pc.type == BYTE && pc.text.size() == 6) {           // "<0xNN>"
      unsigned v = 0;
      if (std::sscanf(pc.text.c_str(), "<0x%02X>", &v) == 1 && v < 256) { byteId_[v] = i; hasBytes_ = true; }
    } else if (pc.type == UNKNOWN) {
      unk_ = i;
    }
  }
}

std::string SentencePieceTokenizer::normalize(const std::string& text) const {
  std::string s;
  if (removeExtraSpaces_) {
    bool pendingSpace = false;
    for (char c : text) {
      if (c == ' ') { pendingSpace = !s.empty(); continue; }
      if (pendingSpace) s.push_back(' ');
      pendingSpace = false;
      s.push_back(c);
    }
  } else {
    s = text;
  }
  if (s.empty()) return s;
  if (addDummyPrefix_) s.insert(s.begin(), ' ');
  if (!escapeSpaces_) return s;
  std::string out;
  out.reserve(s.size() + 16);
  for (char c : s) {
    if (c == ' ') out += kSpace;
    else out.push_back(c);
  }
  return out;
}

void SentencePieceTokenizer::emitUnknown(const std::string& ch, std::vector<int32_t>& out) const {
  if (hasBytes_) {
    for (unsigned char b : ch) out.push_back(byteId_[b] >= 0 ? byteId_[b] : unk_);
  } else if (out.empty() || out.back() != unk_) {
    out.push_back(unk_);              // a run of unknown characters is one <unk>
  }
}

void SentencePieceTokenizer::encodeBpe(const std::string& norm, std::vector<int32_t>& out) const {
  std::vector<std::string> sym;
  for (size_t i = 0; i < norm.size();) {
    const size_t n = utf8Len(norm, i);
    sym.emplace_back(norm, i, n);
    i += n;
  }
  // merge the adjacent pair whose concatenation is the best-scoring piece, leftmost first on ties, until none is left
  while (sym.size() > 1) {
    float best = -std::numeric_limits<float>::infinity();
    size_t at = sym.size();
    for (size_t i = 0; i + 1 < sym.size(); ++i) {
      if (sym[i].size() + sym[i + 1].size() > maxPieceBytes_) continue;
      auto it = index_.find(sym[i] + sym[i + 1]);
      if (it != index_.end() && pieces_[it->second].score > best) { best = pieces_[it->second].score; at = i; }
    }
    if (at == sym.size()) break;
    sym[at] += sym[at + 1];
    sym.erase(sym.begin() + at + 1);
  }
  for (const std::string& s : sym) {
    auto it = index_.find(s);
    if (it != index_.end()) out.push_back(it->second);
    else emitUnknown(s, out);
  }
}

void SentencePieceTokenizer::encodeUnigram(const std::string& norm, std::vector<int32_t>& out) const {
  const size_t n = norm.size();
  float minScore = 0.f;
  for (const Piece& pc : pieces_) if (pc.type == NORMAL && pc.score < minScore) minScore = pc.score;
  const float unkScore = minScore - 10.f;                       // sentencepiece's penalty for an unknown character
  const float ninf = -std::numeric_limits<float>::infinity();
  std::vector<float> best(n + 1, ninf);
  std::vector<int> from(n + 1, -1), id(n + 1, -1);
  best[0] = 0.f;
  for (size_t i = 0; i < n; i += utf8Len(norm, i)) {
    if (best[i] == ninf) continue;
    // pieces that start here, character boundary by character boundary
    for (size_t j = i; j < n && j - i < maxPieceBytes_;) {
      j += utf8Len(norm, j);
      auto it = index_.find(norm.substr(i, j - i));
      if (it != index_.end()) {
        const float s = best[i] + pieces_[it->second].score;
        if (s > best[j]) { best[j] = s; from[j] = (int)i; id[j] = it->second; }
      }
    }
    const size_t j = i + utf8Len(norm, i);
    if (best[i] + unkScore > best[j]) { best[j] = best[i] + unkScore; from[j] = (int)i; id[j] = -1; }
  }
  std::vector<std::pair<int, int>> seg;                          // (start, piece id or -1), back to front
  for (int j = (int)n; j > 0; j = from[j]) seg.emplace_back(from[j], id[j]);
  for (size_t k = seg.size(); k-- > 0;) {
    const size_t start = (size_t)seg[k].first;
    const size_t stop = k == 0 ? n : (size_t)seg[k - 1].first;
    if (seg[k].second >= 0) out.push_back(seg[k].second);
    else emitUnknown(norm.substr(start, stop - start), out);
  }
}

std::vector<int32_t> SentencePieceTokenizer::encode(const std::string& text, bool addBos, bool addEos) const {
  std::vector<int32_t> out;
  if (addBos && bos_ >= 0) out.push_back(bos_);
  const std::string norm = normalize(text);
  if (!norm.empty()) {
    if (bpe_) encodeBpe(norm, out);
    else encodeUnigram(norm, out);
  }
  if (addEos && eos_ >= 0) out.push_back(eos_);
  return out;
}

std::string SentencePieceTokenizer::decode(const std::vector<int32_t>& ids) const {
  std::string s;
  for (int32_t i : ids) {
    if (i < 0 || i >= (int)pieces_.size()) continue;
    const Piece& pc = pieces_[i];
    if (pc.type == CONTROL || pc.type == UNUSED) continue;
    if (pc.type == BYTE) {
      unsigned v = 0;
      if (std::sscanf(pc.text.c_str(), "<0x%02X>", &v) == 1) s.push_back((char)v);
      continue;
    }
    if (pc.type == UNKNOWN) { s += " \xE2\x81\x87 "; continue; }      // sentencepiece prints U+2047 for <unk>
    s += pc.text;
  }
  std::string out;
  for (size_t i = 0; i < s.size();) {
    if (s.compare(i, 3, kSpace) == 0) { out.push_back(' '); i += 3; }
    else out.push_back(s[i++]);
  }
  if (addDummyPrefix_ && !out.empty() && out[0] == ' ') out.erase(out.begin());
  return out;
}

}  // namespace xft
