// Stand-in for poplar::OptionFlags: an ordered string -> string map that can be
// filled from an initializer list or a flat JSON object
// (tools/general_matrix_multiply.cpp:305-327 shows the uses).
#ifndef poplar_OptionFlags_hpp
#define poplar_OptionFlags_hpp

#include <initializer_list>
#include <iosfwd>
#include <map>
#include <string>
#include <utility>

namespace poplar {

class OptionFlags {
public:
  using value_type = std::pair<const std::string, std::string>;
  using const_iterator = std::map<std::string, std::string>::const_iterator;
  OptionFlags() = default;
  OptionFlags(std::initializer_list<std::pair<const std::string, std::string>> init) {
    for (const auto &kv : init) flags_[kv.first] = kv.second;
  }
  void set(const std::string &name, const std::string &value) { flags_[name] = value; }
  void set(std::initializer_list<std::pair<const std::string, std::string>> init) {
    for (const auto &kv : init) flags_[kv.first] = kv.second;
  }
  void clear() { flags_.clear(); }
  const_iterator begin() const { return flags_.begin(); }
  const_iterator end() const { return flags_.end(); }
  std::size_t size() const { return flags_.size(); }
  bool empty() const { return flags_.empty(); }
  friend bool operator==(const OptionFlags &a, const OptionFlags &b) { return a.flags_ == b.flags_; }
  friend bool operator<(const OptionFlags &a, const OptionFlags &b) { return a.flags_ < b.flags_; }

private:
  std::map<std::string, std::string> flags_;
};

/// Fills `flags` from a flat JSON object; nested objects are kept as their JSON
/// text (this is how "planConstraints" is passed).  Throws invalid_option.
void readJSON(const std::string &json, OptionFlags &flags);
void readJSON(std::istream &stream, OptionFlags &flags);
std::ostream &operator<<(std::ostream &os, const OptionFlags &flags);

} // namespace poplar

#endif // poplar_OptionFlags_hpp
