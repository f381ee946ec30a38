#include "bpe_tokenizer.h"

#include <sys/stat.h>

#include <algorithm>
#include <climits>
#include <fstream>
#include <memory>
#include <sstream>
#include <stdexcept>

namespace xft {
namespace {

// ---- a small JSON reader: enough for tokenizer.json / vocab.json (objects, arrays, strings with escapes, numbers,
// true / false / null).  Values are kept as a tree; object members keep their order.
struct Json {
  enum Type { Null, Bool, Number, String, Array, Object } type = Null;
  bool b = false;
  double num = 0;
  std::string str;
  std::vector<Json> arr;
  std::vector<std::pair<std::string, Json>> obj;
  const Json* get(const char* key) const {
    if (type != Object) return nullptr;
    for (auto& kv : obj) if (kv.first == key) return &kv.second;
    return nullptr;
  }
};

void appendUtf8(std::string& s, uint32_t cp) {
  if (cp < 0x80) s.push_back((char)cp);
  else if (cp < 0x800) { s.push_back((char)(0xC0 | (cp >> 6))); s.push_back((char)(0x80 | (cp & 0x3F))); }
  else if (cp < 0x10000) { s.push_back((char)(0xE0 | (cp >> 12))); s.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); s.push_back((char)(0x80 | (cp & 0x3F))); }
  else { s.push_back((char)(0xF0 | (cp >> 18))); s.push_back((char)(0x80 | ((cp >> 12) & 0x3F))); s.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); s.push_back((char)(0x80 | (cp & 0x3F))); }
}

class JsonReader {
public:
  explicit JsonReader(const std::string& text) : s_(text) {}
  Json parse() {
    Json v = value(0);
    ws();
    if (p_ != s_.size()) fail("trailing characters");
    return v;
  }

private:
  [[noreturn]] void fail(const char* what) const { throw std::runtime_error(std::string("JSON: ") + what + " at byte " + std::to_string(p_)); }
  void ws() { while (p_ < s_.size() && (s_[p_] == ' ' || s_[p_] == '\n' || s_[p_] == '\t' || s_[p_] == '\r')) ++p_; }
  uint32_t hex4() {
    if (p_ + 4 > s_.size()) fail("truncated \\u escape");
    uint32_t v = 0;
    for (int i = 0; i < 4; ++i) {
      const char c = s_[p_++];
      v = v * 16 + (c >= '0' && c <= '9' ? c - '0' : c >= 'a' && c <= 'f' ? c - 'a' + 10 : c >= 'A' && c <= 'F' ? c - 'A' + 10 : (fail("bad hex digit"), 0));
    }
    return v;
  }
  std::string string() {
    if (s_[p_] != '"') fail("string expected");
    ++p_;
    std::string out;
    while (true) {
      if (p_ >= s_.size()) fail("unterminated string");
      const char c = s_[p_++];
      if (c == '"') return out;
      if (c != '\\') { out.push_back(c); continue; }
      if (p_ >= s_.size()) fail("unterminated escape");
      const char e = s_[p_++];
      switch (e) {
        case '"': out.push_back('"'); break;
        case '\\': out.push_back('\\'); break;
        case '/': out.push_back('/'); break;
        case 'b': out.push_back('\b'); break;
        case 'f': out.push_back('\f'); break;
        case 'n': out.push_back('\n'); break;
        case 'r': out.push_back('\r'); break;
        case 't': out.push_back('\t'); break;
        case 'u': {
          uint32_t cp = hex4();
          if (cp >= 0xD800 && cp < 0xDC00 && p_ + 1 < s_.size() && s_[p_] == '\\' && s_[p_ + 1] == 'u') {   // surrogate pair
            p_ += 2;
            const uint32_t lo = hex4();
            cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
          }
          appendUtf8(out, cp);
          break;
        }
        default: fail("unknown escape");
      }
    }
  }
  Json value(int depth) {
    if (depth > 64) fail("nesting too deep");
    ws();
    if (p_ >= s_.size()) fail("value expected");
    Json v;
    const char c = s_[p_];
    if (c == '{') {
      v.type = Json::Object;
      ++p_;
      ws();
      if (p_ < s_.size() && s_[p_] == '}') { ++p_; return v; }
      while (true) {
        ws();
        std::string k = string();
        ws();
        if (p_ >= s_.size() || s_[p_] != ':') fail("':' expected");
        ++p_;
        v.obj.emplace_back(std::move(k), value(depth + 1));
        ws();
        if (p_ < s_.size() && s_[p_] == ',') { ++p_; continue; }
        if (p_ < s_.size() && s_[p_] == '}') { ++p_; return v; }
        fail("',' or '}' expected");
      }
    }
    if (c == '[') {
      v.type = Json::Array;
      ++p_;
      ws();
      if (p_ < s_.size() && s_[p_] == ']') { ++p_; return v; }
      while (true) {
        v.arr.push_back(value(depth + 1));
        ws();
        if (p_ < s_.size() && s_[p_] == ',') { ++p_; continue; }
        if (p_ < s_.size() && s_[p_] == ']') { ++p_; return v; }
        fail("',' or ']' expected");
      }
    }
    if (c == '"') { v.type = Json::String; v.str = string(); return v; }
    if (s_.compare(p_, 4, "true") == 0) { p_ += 4; v.type = Json::Bool; v.b = true; return v; }
    if (s_.compare(p_, 5, "false") == 0) { p_ += 5; v.type = Json::Bool; return v; }
    if (s_.compare(p_, 4, "null") == 0) { p_ += 4; return v; }
    size_t q = p_;
    while (q < s_.size() && (std::isdigit((unsigned char)s_[q]) || s_[q] == '-' || s_[q] == '+' || s_[q] == '.' || s_[q] == 'e' || s_[q] == 'E')) ++q;
    if (q == p_) fail("unexpected character");
    v.type = Json::Number;
    v.num = std::strtod(s_.substr(p_, q - p_).c_str(), nullptr);
    p_ = q;
    return v;
  }
  const std::string& s_;
  size_t p_ = 0;
};

std::string readAll(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) throw std::runtime_error("cannot open " + path);
  std::stringstream ss;
  ss << f.rdbuf();
  return ss.str();
}
bool isFile(const std::string& p) { struct stat st; return stat(p.c_str(), &st) == 0 && S_ISREG(st.st_mode); }
bool isDir(const std::string& p) { struct stat st; return stat(p.c_str(), &st) == 0 && S_ISDIR(st.st_mode); }

// code point at s[i] and its length in bytes (1 for a stray byte)
uint32_t decodeAt(const std::string& s, size_t i, size_t& len) {
  const uint8_t c = (uint8_t)s[i];
  len = c < 0x80 ? 1 : (c >> 5) == 6 ? 2 : (c >> 4) == 14 ? 3 : (c >> 3) == 30 ? 4 : 1;
  if (i + len > s.size()) len = 1;
  if (len == 1) return c;
  uint32_t cp = c & (0xFF >> (len + 1));
  for (size_t k = 1; k < len; ++k) cp = (cp << 6) | ((uint8_t)s[i + k] & 0x3F);
  return cp;
}

struct Cp { uint32_t cp; size_t pos, len; };
bool isSpace(uint32_t c) { return c == ' ' || c == '\t' || c == '\n' || c == '\r' || c == '\v' || c == '\f'; }
bool isDigit(uint32_t c) { return c >= '0' && c <= '9'; }
bool isLetter(uint32_t c) { return (c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z') || c >= 0x80; }
bool isOther(uint32_t c) { return !isSpace(c) && !isDigit(c) && !isLetter(c); }

}  // namespace

BpeTokenizer::BpeTokenizer(const std::string& path) {
  // GPT-2's byte <-> printable character table: bytes that print keep their code point, the others take 256, 257, ...
  int extra = 0;
  for (int b = 0; b < 256; ++b) {
    const bool keeps = (b >= 33 && b <= 126) || (b >= 161 && b <= 172) || (b >= 174 && b <= 255);
    std::string u;
    appendUtf8(u, keeps ? (uint32_t)b : (uint32_t)(256 + extra++));
    byteToUni_[b] = u;
    uniToByte_[u] = b;
  }
  if (isDir(path)) {
    if (isFile(path + "/tokenizer.json")) loadTokenizerJson(path + "/tokenizer.json");
    else if (isFile(path + "/vocab.json") && isFile(path + "/merges.txt")) loadVocabMerges(path + "/vocab.json", path + "/merges.txt");
    else throw std::runtime_error("no tokenizer.json or vocab.json + merges.txt under " + path);
  } else if (isFile(path)) {
    loadTokenizerJson(path);
  } else {
    throw std::runtime_error("cannot open tokenizer " + path);
  }
  finish();
}

void BpeTokenizer::loadTokenizerJson(const std::string& file) {
  const std::string text = readAll(file);
  const Json root = JsonReader(text).parse();
  const Json* model = root.get("model");
  if (!model || !model->get("vocab") || !model->get("merges")) throw std::runtime_error(file + ": not a BPE tokenizer.json (model.vocab / model.merges missing)");
  if (const Json* t = model->get("type")) if (t->type == Json::String && t->str != "BPE") throw std::runtime_error(file + ": model type " + t->str + " is not BPE");
  for (auto& kv : model->get("vocab")->obj) vocab_[kv.first] = (int)kv.second.num;
  int rank = 0;
  for (auto& m : model->get("merges")->arr) {
    if (m.type == Json::String) mergeRank_.emplace(m.str, rank++);
    else if (m.type == Json::Array && m.arr.size() == 2) mergeRank_.emplace(m.arr[0].str + " " + m.arr[1].str, rank++);
  }
  if (const Json* u = model->get("unk_token")) if (u->type == Json::String && vocab_.count(u->str)) unk_ = vocab_[u->str];
  if (const Json* a = root.get("added_tokens"))
    for (auto& t : a->arr) {
      const Json* c = t.get("content");
      const Json* id = t.get("id");
      if (c && id && c->type == Json::String) special_.emplace_back(c->str, (int)id->num);
    }
  // the pre-tokenizer pattern decides the splitting style: look for the tell-tale fragments anywhere under it
  if (const Json* pre = root.get("pre_tokenizer")) {
    std::string all;
    std::vector<const Json*> stack{pre};
    while (!stack.empty()) {
      const Json* j = stack.back();
      stack.pop_back();
      if (j->type == Json::String) all += j->str + "\n";
      for (auto& x : j->arr) stack.push_back(&x);
      for (auto& kv : j->obj) stack.push_back(&kv.second);
    }
    if (all.find("(?i:") != std::string::npos || all.find("[^\\r\\n\\p{L}\\p{N}]?") != std::string::npos) {
      style_ = 1;
      digitGroup_ = all.find("\\p{N}{1,3}") != std::string::npos ? 3 : 1;
    }
  }
  if (const Json* im = model->get("ignore_merges")) ignoreMerges_ = im->type == Json::Bool && im->b;
}

void BpeTokenizer::loadVocabMerges(const std::string& vocabFile, const std::string& mergesFile) {
  const std::string vt = readAll(vocabFile);
  const Json root = JsonReader(vt).parse();
  if (root.type != Json::Object) throw std::runtime_error(vocabFile + ": an object of token -> id expected");
  for (auto& kv : root.obj) vocab_[kv.first] = (int)kv.second.num;
  std::ifstream f(mergesFile);
  std::string line;
  int rank = 0;
  while (std::getline(f, line)) {
    if (!line.empty() && line.back() == '\r') line.pop_back();
    if (line.empty() || line.rfind("#version", 0) == 0) continue;
    mergeRank_.emplace(line, rank++);
  }
}

void BpeTokenizer::finish() {
  int maxId = -1;
  for (auto& kv : vocab_) maxId = std::max(maxId, kv.second);
  for (auto& sp : special_) maxId = std::max(maxId, sp.second);
  if (maxId < 0) throw std::runtime_error("tokenizer has no vocabulary");
  idToToken_.assign((size_t)maxId + 1, "");
  isSpecial_.assign((size_t)maxId + 1, 0);
  for (auto& kv : vocab_) if (kv.second >= 0) idToToken_[kv.second] = kv.first;
  for (auto& sp : special_) if (sp.second >= 0) { idToToken_[sp.second] = sp.first; isSpecial_[sp.second] = 1; }
  std::stable_sort(special_.begin(), special_.end(), [](auto& a, auto& b) { return a.first.size() > b.first.size(); });
}

int BpeTokenizer::specialId(const std::string& text) const {
  for (auto& sp : special_) if (sp.first == text) return sp.second;
  return -1;
}

std::vector<std::string> BpeTokenizer::split(const std::string& text) const {
  std::vector<Cp> c;
  for (size_t i = 0; i < text.size();) { size_t len; const uint32_t cp = decodeAt(text, i, len); c.push_back({cp, i, len}); i += len; }
  const size_t n = c.size();
  std::vector<std::string> out;
  auto emit = [&](size_t a, size_t b) { out.emplace_back(text, c[a].pos, (b < n ? c[b].pos : text.size()) - c[a].pos); };
  auto lower = [](uint32_t x) { return x >= 'A' && x <= 'Z' ? x + 32 : x; };
  size_t i = 0;
  while (i < n) {
    // 1. contractions
    if (c[i].cp == '\'' && i + 1 < n) {
      static const char* two[] = {"re", "ve", "ll"};
      const uint32_t a = style_ ? lower(c[i + 1].cp) : c[i + 1].cp;
      const uint32_t b = i + 2 < n ? (style_ ? lower(c[i + 2].cp) : c[i + 2].cp) : 0;
      bool hit = false;
      for (const char* t : two)
        if (a == (uint32_t)t[0] && b == (uint32_t)t[1]) { emit(i, i + 3); i += 3; hit = true; break; }
      if (hit) continue;
      if (a == 's' || a == 't' || a == 'm' || a == 'd') { emit(i, i + 2); i += 2; continue; }
    }
    const uint32_t x = c[i].cp;
    const uint32_t y = i + 1 < n ? c[i + 1].cp : 0;
    const bool more = i + 1 < n;
    if (style_ == 0) {
      // GPT-2: ` ?letters+ | ?digits+ | ?others+`
      size_t j = i;
      if (x == ' ' && more && !isSpace(y)) j = i + 1;
      if (j < n && !isSpace(c[j].cp)) {
        bool (*cls)(uint32_t) = isLetter(c[j].cp) ? isLetter : isDigit(c[j].cp) ? isDigit : isOther;
        size_t k = j;
        while (k < n && cls(c[k].cp)) ++k;
        emit(i, k);
        i = k;
        continue;
      }
    } else {
      // tiktoken-style: `[^\r\n letters digits]?letters+ | digits{1,g} | ?others+[\r\n]*`
      if (isLetter(x) || (x != '\r' && x != '\n' && !isDigit(x) && more && isLetter(y))) {
        size_t k = isLetter(x) ? i : i + 1;
        while (k < n && isLetter(c[k].cp)) ++k;
        emit(i, k);
        i = k;
        continue;
      }
      if (isDigit(x)) {
        size_t k = i;
        while (k < n && isDigit(c[k].cp) && (int)(k - i) < digitGroup_) ++k;
        emit(i, k);
        i = k;
        continue;
      }
      size_t j = i;
      if (x == ' ' && more && isOther(y)) j = i + 1;
      if (isOther(c[j].cp)) {
        size_t k = j;
        while (k < n && isOther(c[k].cp)) ++k;
        while (k < n && (c[k].cp == '\r' || c[k].cp == '\n')) ++k;
        emit(i, k);
        i = k;
        continue;
      }
    }
    // whitespace: `\s*[\r\n]+` (tiktoken-style only), `\s+(?!\S)`, `\s+`
    size_t k = i;
    while (k < n && isSpace(c[k].cp)) ++k;
    size_t end = k;
    if (style_ == 1) {
      size_t lastNl = n;
      for (size_t t = i; t < k; ++t) if (c[t].cp == '\r' || c[t].cp == '\n') lastNl = t;
      if (lastNl != n) { emit(i, lastNl + 1); i = lastNl + 1; continue; }
    }
    if (k < n && k - i > 1) end = k - 1;          // leave the last space for the piece that follows
    emit(i, end);
    i = end;
  }
  return out;
}

void BpeTokenizer::bpe(const std::string& piece, std::vector<int32_t>& out) const {
  std::string mapped;
  std::vector<std::string> sym;
  for (unsigned char b : piece) { sym.push_back(byteToUni_[b]); mapped += byteToUni_[b]; }
  if (ignoreMerges_) {
    auto it = vocab_.find(mapped);
    if (it != vocab_.end()) { out.push_back(it->second); return; }
  }
  while (sym.size() > 1) {
    int best = INT_MAX;
    for (size_t i = 0; i + 1 < sym.size(); ++i) {
      auto it = mergeRank_.find(sym[i] + " " + sym[i + 1]);
      if (it != mergeRank_.end() && it->second < best) best = it->second;
    }
    if (best == INT_MAX) break;
    // merge every occurrence of the best pair, left to right
    std::vector<std::string> next;
    for (size_t i = 0; i < sym.size();) {
      if (i + 1 < sym.size()) {
        auto it = mergeRank_.find(sym[i] + " " + sym[i + 1]);
        if (it != mergeRank_.end() && it->second == best) { next.push_back(sym[i] + sym[i + 1]); i += 2; continue; }
      }
      next.push_back(sym[i]);
      ++i;
    }
    sym.swap(next);
  }
  for (const std::string& s : sym) {
    auto it = vocab_.find(s);
    if (it != vocab_.end()) { out.push_back(it->second); continue; }
    // a merged string that is no token (cannot happen with a consistent file): fall back to its characters
    for (size_t i = 0; i < s.size();) {
      size_t len;
      decodeAt(s, i, len);
      auto c1 = vocab_.find(s.substr(i, len));
      if (c1 != vocab_.end()) out.push_back(c1->second);
      else if (unk_ >= 0) out.push_back(unk_);
      i += len;
    }
  }
}

std::vector<int32_t> BpeTokenizer::encode(const std::string& text) const {
  std::vector<int32_t> out;
  size_t start = 0, i = 0;
  auto flush = [&](size_t a, size_t b) {
    if (b > a) for (const std::string& piece : split(text.substr(a, b - a))) bpe(piece, out);
  };
  while (i < text.size()) {
    bool hit = false;
    if (!special_.empty() && text[i] == '<')                    // added tokens all start with '<' in these families
      for (auto& sp : special_)
        if (!sp.first.empty() && text.compare(i, sp.first.size(), sp.first) == 0) {
          flush(start, i);
          out.push_back(sp.second);
          i += sp.first.size();
          start = i;
          hit = true;
          break;
        }
    if (!hit) ++i;
  }
  flush(start, text.size());
  return out;
}

std::string BpeTokenizer::decode(const std::vector<int32_t>& ids) const {
  std::string out;
  for (int32_t id : ids) {
    if (id < 0 || id >= (int)idToToken_.size()) continue;
    const std::string& t = idToToken_[id];
    if (isSpecial_[id]) { out += t; continue; }
    for (size_t i = 0; i < t.size();) {
      size_t len;
      decodeAt(t, i, len);
      auto it = uniToByte_.find(t.substr(i, len));
      if (it != uniToByte_.end()) out.push_back((char)it->second);
      else out += t.substr(i, len);
      i += len;
    }
  }
  return out;
}

}  // namespace xft
