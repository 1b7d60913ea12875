// Minimal JSON reader for the two places the poplin surface takes JSON: the
// stream form of ConvParams and the planConstraints option.  Values keep their
// text; objects and arrays keep their children in order (arrays use empty keys).
#pragma once

#include <cctype>
#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "poplar/exceptions.hpp"

namespace poplin {
namespace json {

struct Value {
  enum class Kind { Object, Array, String, Scalar } kind = Kind::Scalar;
  std::string text;                                  // String / Scalar
  std::vector<std::pair<std::string, Value>> items;  // Object / Array

  const Value *find(const std::string &key) const {
    for (const auto &kv : items)
      if (kv.first == key) return &kv.second;
    return nullptr;
  }
  bool isContainer() const { return kind == Kind::Object || kind == Kind::Array; }
};

class Parser {
public:
  explicit Parser(const std::string &s) : s_(s) {}
  Value parse() {
    Value v = value();
    space();
    if (i_ != s_.size()) fail("trailing characters");
    return v;
  }

private:
  [[noreturn]] void fail(const std::string &why) const {
    throw poplar::invalid_option("JSON parse error at offset " + std::to_string(i_) + ": " + why);
  }
  void space() {
    while (i_ < s_.size() && std::isspace(static_cast<unsigned char>(s_[i_]))) ++i_;
  }
  std::string string() {
    if (s_[i_] != '"') fail("expected a string");
    std::string out;
    for (++i_; i_ < s_.size() && s_[i_] != '"'; ++i_) {
      if (s_[i_] == '\\' && i_ + 1 < s_.size()) ++i_;
      out.push_back(s_[i_]);
    }
    if (i_ >= s_.size()) fail("unterminated string");
    ++i_;
    return out;
  }
  Value value() {
    space();
    if (i_ >= s_.size()) fail("unexpected end");
    Value v;
    if (s_[i_] == '{') {
      v.kind = Value::Kind::Object;
      ++i_;
      space();
      if (i_ < s_.size() && s_[i_] == '}') {
        ++i_;
        return v;
      }
      for (;;) {
        space();
        std::string key = string();
        space();
        if (i_ >= s_.size() || s_[i_] != ':') fail("expected ':'");
        ++i_;
        v.items.emplace_back(std::move(key), value());
        space();
        if (i_ < s_.size() && s_[i_] == ',') {
          ++i_;
          continue;
        }
        if (i_ < s_.size() && s_[i_] == '}') {
          ++i_;
          return v;
        }
        fail("expected ',' or '}'");
      }
    }
    if (s_[i_] == '[') {
      v.kind = Value::Kind::Array;
      ++i_;
      space();
      if (i_ < s_.size() && s_[i_] == ']') {
        ++i_;
        return v;
      }
      for (;;) {
        v.items.emplace_back(std::string(), value());
        space();
        if (i_ < s_.size() && s_[i_] == ',') {
          ++i_;
          continue;
        }
        if (i_ < s_.size() && s_[i_] == ']') {
          ++i_;
          return v;
        }
        fail("expected ',' or ']'");
      }
    }
    if (s_[i_] == '"') {
      v.kind = Value::Kind::String;
      v.text = string();
      return v;
    }
    const std::size_t begin = i_;
    while (i_ < s_.size() && s_[i_] != ',' && s_[i_] != '}' && s_[i_] != ']' &&
           !std::isspace(static_cast<unsigned char>(s_[i_])))
      ++i_;
    if (i_ == begin) fail("expected a value");
    v.text = s_.substr(begin, i_ - begin);
    return v;
  }
  const std::string &s_;
  std::size_t i_ = 0;
};

inline Value parse(const std::string &s) { return Parser(s).parse(); }

}  // namespace json
}  // namespace poplin
