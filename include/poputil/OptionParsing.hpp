// Option specification and parsing with the behaviour of the reference's
// include/poputil/OptionParsing.hpp:90-223: an unknown option name, or a value
// its handler rejects, raises poplar::invalid_option with the same wording.
#ifndef poputil_OptionParsing_hpp
#define poputil_OptionParsing_hpp

#include <functional>
#include <initializer_list>
#include <limits>
#include <map>
#include <sstream>
#include <string>
#include <vector>

#include "poplar/exceptions.hpp"

namespace poplibs {

namespace parse {
template <typename T> T asInteger(const std::string &str) {
  std::istringstream iss(str);
  T result;
  if (str.find("0x") != std::string::npos)
    iss >> std::hex >> result;
  else
    iss >> std::dec >> result;
  if (iss.fail() || !iss.eof()) throw poplar::invalid_option("Not a valid integer");
  return result;
}
template <typename T> T asFloatingPoint(const std::string &str) {
  std::istringstream iss(str);
  T result;
  iss >> result;
  if (iss.fail() || !iss.eof()) throw poplar::invalid_option("Not a valid floating point number");
  return result;
}
template <typename T> T asEnum(const std::string &value, const std::map<std::string, T> &map) {
  const auto it = map.find(value);
  if (it != map.end()) return it->second;
  std::stringstream s;
  s << "Unrecognised value. Expected one of: ";
  bool first = true;
  for (const auto &e : map) {
    s << (first ? "" : ", ") << "'" << e.first << "'";
    first = false;
  }
  throw poplar::invalid_option(s.str());
}
} // namespace parse

class OptionHandler {
  std::function<void(const std::string &)> valueHandler;

public:
  template <typename T> OptionHandler(T &&handler) : valueHandler(std::forward<T>(handler)) {}
  void parseValue(const std::string &value) const { valueHandler(value); }

  template <typename T, typename MapT = std::map<std::string, T>>
  static OptionHandler createWithEnum(T &output, MapT &&valueMap) {
    return OptionHandler{[map = std::map<std::string, T>(std::forward<MapT>(valueMap)),
                          &output](const std::string &value) { output = parse::asEnum<T>(value, map); }};
  }
  template <typename T> static OptionHandler createWithInteger(T &output) {
    return OptionHandler{[&output](const std::string &value) { output = parse::asInteger<int>(value); }};
  }
  template <typename T> static OptionHandler createWithBool(T &output) {
    return createWithEnum(output, std::map<std::string, T>{{"true", static_cast<T>(true)},
                                                           {"false", static_cast<T>(false)}});
  }
  template <typename T>
  static void ensureValueIsWithinBounds(T value, const T &lowerBound, bool lowerInclusive,
                                        const T &upperBound, bool upperInclusive) {
    if (value < lowerBound || (!lowerInclusive && value == lowerBound))
      throw poplar::invalid_option("Value must be greater than " +
                                   std::string(lowerInclusive ? "or equal to " : "") +
                                   std::to_string(lowerBound));
    if (value > upperBound || (!upperInclusive && value == upperBound))
      throw poplar::invalid_option("Value must be less than " +
                                   std::string(upperInclusive ? "or equal to " : "") +
                                   std::to_string(upperBound));
  }
  template <typename T>
  static OptionHandler createWithDouble(T &output,
                                        double lowerBound = std::numeric_limits<double>::min(),
                                        bool lowerInclusive = true,
                                        double upperBound = std::numeric_limits<double>::max(),
                                        bool upperInclusive = true) {
    return OptionHandler{[&output, lowerBound, lowerInclusive, upperBound,
                          upperInclusive](const std::string &value) {
      const double v = parse::asFloatingPoint<double>(value);
      ensureValueIsWithinBounds(v, lowerBound, lowerInclusive, upperBound, upperInclusive);
      output = v;
    }};
  }
  static OptionHandler createWithString(std::string &output) {
    return OptionHandler{[&output](const std::string &value) { output = value; }};
  }
};

class OptionSpec {
  std::map<const std::string, OptionHandler> handlers;

public:
  OptionSpec(std::initializer_list<std::pair<const std::string, OptionHandler>> &&h)
      : handlers(std::move(h)) {}

  void parse(const std::string &option, const std::string &value, bool ignoreUnknown = false) const {
    const auto it = handlers.find(option);
    if (it == handlers.end()) {
      if (ignoreUnknown) return;
      throw poplar::invalid_option("Unrecognised option '" + option + "'");
    }
    try {
      it->second.parseValue(value);
    } catch (const poplar::invalid_option &e) {
      throw poplar::invalid_option("Invalid value '" + value + "' for option '" + option +
                                   "': " + e.what());
    }
  }
};

} // namespace poplibs

#endif // poputil_OptionParsing_hpp
