// Helpers shared by the two driver tools: command-line parsing in the style of
// the reference's tools ("--name value" or "--name=value", shapes written
// "{a,b}" or as a scalar that is broadcast, include/poplibs_test/Util.hpp:
// 249-394), conversion of host doubles to the device element types, and tensor
// dumps for external checking.
#pragma once

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <fstream>
#include <map>
#include <random>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "poplar/Type.hpp"

namespace tool {

class Args {
public:
  Args(int argc, char **argv) {
    for (int i = 1; i < argc; ++i) {
      std::string a = argv[i];
      if (a.rfind("--", 0) != 0) throw std::runtime_error("unexpected argument '" + a + "'");
      a = a.substr(2);
      const auto eq = a.find('=');
      if (eq != std::string::npos) {
        values_[a.substr(0, eq)] = a.substr(eq + 1);
      } else if (i + 1 < argc && std::string(argv[i + 1]).rfind("--", 0) != 0) {
        values_[a] = argv[++i];
      } else {
        values_[a] = "";
      }
    }
  }
  bool has(const std::string &name) const {
    used_.insert({name, true});
    return values_.count(name) != 0;
  }
  std::string str(const std::string &name, const std::string &dflt = "") const {
    used_.insert({name, true});
    const auto it = values_.find(name);
    return it == values_.end() ? dflt : it->second;
  }
  template <class T> T get(const std::string &name, T dflt) const {
    if (!has(name)) {
      used_.insert({name, true});
      return dflt;
    }
    std::istringstream iss(str(name));
    T v{};
    if (std::is_same<T, bool>::value) iss >> std::boolalpha;
    iss >> v;
    if (iss.fail()) {
      // "1" / "0" for booleans
      std::istringstream again(str(name));
      again >> std::noboolalpha >> v;
      if (again.fail()) throw std::runtime_error("bad value for --" + name + ": '" + str(name) + "'");
    }
    return v;
  }
  template <class T> T required(const std::string &name) const {
    if (!has(name)) throw std::runtime_error("the option '--" + name + "' is required but missing");
    return get<T>(name, T{});
  }
  /// "{a,b,c}" or a scalar broadcast to `dims` entries.
  template <class T> std::vector<T> shape(const std::string &name, std::size_t dims, T dflt) const {
    if (!has(name)) {
      used_.insert({name, true});
      return std::vector<T>(dims, dflt);
    }
    std::string s = str(name);
    std::vector<T> out;
    if (!s.empty() && s.front() == '{') {
      if (s.back() != '}') throw std::runtime_error("missing '}' in --" + name);
      std::istringstream iss(s.substr(1, s.size() - 2));
      for (std::string item; std::getline(iss, item, ',');) {
        std::istringstream is(item);
        T v{};
        is >> v;
        if (is.fail()) throw std::runtime_error("bad element in --" + name);
        out.push_back(v);
      }
      if (out.size() != dims && dims != 0)
        throw std::runtime_error("--" + name + " needs " + std::to_string(dims) + " values");
    } else {
      std::istringstream is(s);
      T v{};
      is >> v;
      if (is.fail()) throw std::runtime_error("bad value for --" + name);
      out.assign(dims == 0 ? 1 : dims, v);
    }
    return out;
  }
  /// Number of entries of a "{...}" option (1 for a scalar, 0 if absent).
  std::size_t shapeRank(const std::string &name) const {
    if (!has(name)) return 0;
    const std::string s = values_.at(name);
    if (s.empty() || s.front() != '{') return 1;
    return std::size_t(std::count(s.begin(), s.end(), ',')) + 1;
  }
  void rejectUnknown() const {
    for (const auto &kv : values_)
      if (!used_.count(kv.first)) throw std::runtime_error("unrecognised option '--" + kv.first + "'");
  }

private:
  std::map<std::string, std::string> values_;
  mutable std::map<std::string, bool> used_;
};

// ---- element conversion ------------------------------------------------------------
inline uint16_t halfBits(double x) {
  // round to nearest even, overflow to infinity
  const float f = float(x);
  uint32_t u;
  std::memcpy(&u, &f, 4);
  const uint32_t sign = (u >> 16) & 0x8000u;
  const int32_t exp = int32_t((u >> 23) & 0xff) - 127 + 15;
  uint32_t man = u & 0x7fffffu;
  if (((u >> 23) & 0xff) == 0xff) return uint16_t(sign | 0x7c00u | (man ? 0x200u : 0));
  if (exp >= 31) return uint16_t(sign | 0x7c00u);
  if (exp <= 0) {
    if (exp < -10) return uint16_t(sign);
    man |= 0x800000u;
    const int shift = 14 - exp;
    uint32_t half = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1), mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half & 1))) ++half;
    return uint16_t(sign | half);
  }
  uint32_t half = (uint32_t(exp) << 10) | (man >> 13);
  const uint32_t rem = man & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) ++half;
  return uint16_t(sign | half);
}

inline double halfValue(uint16_t h) {
  const int sign = h >> 15, e = (h >> 10) & 31, m = h & 1023;
  double v;
  if (e == 0) v = std::ldexp(double(m), -24);
  else if (e == 31) v = m ? NAN : INFINITY;
  else v = std::ldexp(double(m + 1024), e - 25);
  return sign ? -v : v;
}

// Graphcore F143 (1-4-3, bias 8, largest finite value 240): the encoding whose
// value is half of the E4M3 reading of the same bits.  Round to nearest even,
// saturating at the largest code the tensor core also treats as finite.
inline uint8_t f143Bits(double x) {
  const double y = x * 2.0;  // E4M3 reading of the stored bits
  if (std::isnan(y)) return 0x7f;
  const uint8_t sign = std::signbit(y) ? 0x80 : 0;
  double a = std::fabs(y);
  if (a >= 448.0) return uint8_t(sign | 0x7e);
  if (a == 0.0) return sign;
  int e;
  (void)std::frexp(a, &e);
  int exp2 = std::max(e - 1, -6);
  const double ulp = std::ldexp(1.0, exp2 - 3);
  double q = std::nearbyint(a / ulp) * ulp;
  if (q >= 448.0) return uint8_t(sign | 0x7e);
  if (q == 0.0) return sign;
  (void)std::frexp(q, &e);
  exp2 = e - 1;
  if (exp2 < -6) return uint8_t(sign | uint8_t(q / std::ldexp(1.0, -9)));
  const int m = int((q / std::ldexp(1.0, exp2) - 1.0) * 8.0);
  return uint8_t(sign | ((exp2 + 7) << 3) | m);
}

inline double f143Value(uint8_t b) {
  const int sign = b >> 7, e = (b >> 3) & 15, m = b & 7;
  double v = e == 0 ? std::ldexp(double(m), -9) : std::ldexp(1.0 + m / 8.0, e - 7);
  v *= 0.5;
  return sign ? -v : v;
}

// Graphcore F152 (1-5-2, bias 16): half of the E5M2 reading of the same bits,
// and E5M2 is the upper byte of binary16.  Round to nearest even, saturating at
// the largest finite code.
inline uint8_t f152Bits(double x) {
  const double y = x * 2.0;  // E5M2 reading of the stored bits
  if (std::isnan(y)) return 0x7e;
  const uint16_t h = halfBits(std::max(-57344.0, std::min(57344.0, y)));
  const unsigned lower = h & 0xffu;
  unsigned code = h >> 8;
  if (lower > 0x80u || (lower == 0x80u && (code & 1u))) ++code;
  if ((code & 0x7fu) >= 0x7cu) code = (code & 0x80u) | 0x7bu;
  return uint8_t(code);
}

inline double f152Value(uint8_t b) { return 0.5 * halfValue(uint16_t(uint16_t(b) << 8)); }

/// Converts `values` to the device type (for QUARTER: value = stored * 2^scale)
/// and replaces them by exactly what the device will see.
inline std::vector<uint8_t> toDevice(std::vector<double> &values, const poplar::Type &type, int scale = 0,
                                     bool f152 = false) {
  std::vector<uint8_t> raw(values.size() * type.bytes());
  for (std::size_t i = 0; i < values.size(); ++i) {
    if (type == poplar::HALF) {
      const uint16_t h = halfBits(values[i]);
      std::memcpy(&raw[2 * i], &h, 2);
      values[i] = halfValue(h);
    } else if (type == poplar::FLOAT) {
      const float f = float(values[i]);
      std::memcpy(&raw[4 * i], &f, 4);
      values[i] = f;
    } else if (type == poplar::QUARTER) {
      const double scaled = std::ldexp(values[i], -scale);
      const uint8_t b = f152 ? f152Bits(scaled) : f143Bits(scaled);
      raw[i] = b;
      values[i] = std::ldexp(f152 ? f152Value(b) : f143Value(b), scale);
    } else {
      throw std::runtime_error("unsupported element type " + type.toString());
    }
  }
  return raw;
}

/// "F143" / "F152" (tools' --fp8-format options).
inline poplar::QuarterMetadata::Format quarterFormat(const std::string &name) {
  if (name == "F143") return poplar::QuarterMetadata::Format::F143;
  if (name == "F152") return poplar::QuarterMetadata::Format::F152;
  throw std::runtime_error("unknown quarter format " + name + " (F143 or F152)");
}

inline std::vector<double> fromDevice(const std::vector<uint8_t> &raw, const poplar::Type &type) {
  std::vector<double> out(raw.size() / type.bytes());
  for (std::size_t i = 0; i < out.size(); ++i) {
    if (type == poplar::HALF) {
      uint16_t h;
      std::memcpy(&h, &raw[2 * i], 2);
      out[i] = halfValue(h);
    } else {
      float f;
      std::memcpy(&f, &raw[4 * i], 4);
      out[i] = f;
    }
  }
  return out;
}

/// Uniform doubles in [lo, hi); with `integers` they are whole numbers (exact
/// in every device type), as the reference draws quarter test data
/// (lib/poplibs_test/Util.cpp:140-142).
inline std::vector<double> randomValues(std::size_t n, double lo, double hi, std::mt19937 &rng,
                                        bool integers) {
  std::vector<double> v(n);
  if (integers) {
    std::uniform_int_distribution<int> d(int(std::ceil(lo)), int(std::floor(hi)));
    for (auto &x : v) x = d(rng);
  } else {
    std::uniform_real_distribution<double> d(lo, hi);
    for (auto &x : v) x = d(rng);
  }
  return v;
}

/// Raw little-endian float64 dump: <dir>/<name>.f64, shape recorded in the name's
/// entry of <dir>/manifest.txt ("name d0 d1 ...").
inline void dump(const std::string &dir, const std::string &name, const std::vector<double> &values,
                 const std::vector<std::size_t> &shape) {
  if (dir.empty()) return;
  std::ofstream f(dir + "/" + name + ".f64", std::ios::binary);
  f.write(reinterpret_cast<const char *>(values.data()), std::streamsize(values.size() * 8));
  std::ofstream m(dir + "/manifest.txt", std::ios::app);
  m << name;
  for (auto d : shape) m << ' ' << d;
  m << '\n';
}

inline poplar::Type parseType(const std::string &s) { return poplar::typeFromString(s); }

}  // namespace tool
