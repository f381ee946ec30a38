#include "ini.h"

#include <algorithm>
#include <cctype>
#include <fstream>

namespace xft {

static std::string trim(const std::string& s) {
  size_t a = 0, b = s.size();
  while (a < b && std::isspace((unsigned char)s[a])) ++a;
  while (b > a && std::isspace((unsigned char)s[b - 1])) --b;
  return s.substr(a, b - a);
}
static std::string lower(std::string s) {
  std::transform(s.begin(), s.end(), s.begin(), [](unsigned char c) { return std::tolower(c); });
  return s;
}

Ini::Ini(const std::string& path) {
  std::ifstream f(path);
  if (!f) return;
  ok_ = true;
  std::string line, sec;
  while (std::getline(f, line)) {
    line = trim(line);
    if (line.empty() || line[0] == ';' || line[0] == '#') continue;
    if (line.front() == '[' && line.back() == ']') {
      sec = trim(line.substr(1, line.size() - 2));
      if (!data_.count(sec)) order_.push_back(sec);
      data_[sec];
      continue;
    }
    size_t eq = line.find_first_of("=:");
    if (eq == std::string::npos) continue;
    data_[sec][lower(trim(line.substr(0, eq)))] = trim(line.substr(eq + 1));
  }
}

bool Ini::has(const std::string& sec, const std::string& key) const {
  auto it = data_.find(sec);
  return it != data_.end() && it->second.count(lower(key));
}
std::string Ini::get(const std::string& sec, const std::string& key, const std::string& def) const {
  auto it = data_.find(sec);
  if (it == data_.end()) return def;
  auto jt = it->second.find(lower(key));
  return jt == it->second.end() || jt->second.empty() ? def : jt->second;
}
long Ini::getInt(const std::string& sec, const std::string& key, long def) const {
  std::string v = get(sec, key);
  if (v.empty()) return def;
  try { return (long)std::stod(v); } catch (...) { return def; }
}
double Ini::getFloat(const std::string& sec, const std::string& key, double def) const {
  std::string v = get(sec, key);
  if (v.empty()) return def;
  try { return std::stod(v); } catch (...) { return def; }
}
bool Ini::getBool(const std::string& sec, const std::string& key, bool def) const {
  std::string v = lower(get(sec, key));
  if (v.empty()) return def;
  if (v == "true" || v == "yes" || v == "on" || v == "1") return true;
  if (v == "false" || v == "no" || v == "off" || v == "0") return false;
  try { return std::stod(v) != 0; } catch (...) { return def; }
}

}  // namespace xft
