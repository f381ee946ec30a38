// Minimal INI reader for config.ini (the reference vendors INIReader.h; semantics kept: first section wins as the
// model type, keys are case-insensitive, `;`/`#` comments, values trimmed).
#pragma once
#include <map>
#include <string>
#include <vector>

namespace xft {

class Ini {
public:
  explicit Ini(const std::string& path);
  bool ok() const { return ok_; }
  const std::vector<std::string>& sections() const { return order_; }
  bool has(const std::string& sec, const std::string& key) const;
  std::string get(const std::string& sec, const std::string& key, const std::string& def = "") const;
  long getInt(const std::string& sec, const std::string& key, long def = 0) const;
  double getFloat(const std::string& sec, const std::string& key, double def = 0.0) const;
  bool getBool(const std::string& sec, const std::string& key, bool def = false) const;

private:
  bool ok_ = false;
  std::vector<std::string> order_;
  std::map<std::string, std::map<std::string, std::string>> data_;
};

}  // namespace xft
