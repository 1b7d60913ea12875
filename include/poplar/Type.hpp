// Stand-in for poplar::Type and poplar::QuarterMetadata: the element types the
// poplin contraction path handles (HALF, FLOAT, QUARTER) plus the integer
// types its tools mention.  Value semantics and names follow the Poplar SDK's
// poplar/Type.hpp and poplar/Quarter.hpp as the reference uses them
// (include/poplin/ConvParams.hpp:10, tools/general_matrix_multiply.cpp:124-126).
#ifndef poplar_Type_hpp
#define poplar_Type_hpp

#include <cstddef>
#include <iosfwd>
#include <string>

namespace poplar {

class Type {
public:
  enum class Kind : unsigned char {
    Invalid, Bool, Char, UnsignedChar, Short, UnsignedShort, Int, UnsignedInt,
    Half, Float, Quarter, QuarterMetadata
  };
  constexpr Type() : kind_(Kind::Invalid) {}
  constexpr explicit Type(Kind k) : kind_(k) {}
  std::string toString() const;
  /// Bytes one element occupies in device memory.
  std::size_t bytes() const;
  /// True for QUARTER: values are only meaningful with their QuarterMetadata.
  bool requiresMetadata() const { return kind_ == Kind::Quarter; }
  Kind kind() const { return kind_; }
  friend bool operator==(const Type &a, const Type &b) { return a.kind_ == b.kind_; }
  friend bool operator!=(const Type &a, const Type &b) { return a.kind_ != b.kind_; }
  friend bool operator<(const Type &a, const Type &b) { return a.kind_ < b.kind_; }

private:
  Kind kind_;
};

std::ostream &operator<<(std::ostream &os, const Type &t);
/// Parses "half", "float", "quarter", ... ; throws poplar::invalid_option.
Type typeFromString(const std::string &s);

extern const Type BOOL, CHAR, UNSIGNED_CHAR, SHORT, UNSIGNED_SHORT, INT, UNSIGNED_INT, HALF,
    FLOAT, QUARTER, QUARTER_METADATA;

/// Format and power-of-two scale of a QUARTER tensor: value = stored * 2^scale.
class QuarterMetadata {
public:
  enum class Format : unsigned char { F143, F152 };
  QuarterMetadata() : format_(Format::F143), scale_(0) {}
  QuarterMetadata(Format f, signed char scale) : format_(f), scale_(scale) {}
  Format getFormat() const { return format_; }
  signed char getScale() const { return scale_; }
  friend bool operator==(const QuarterMetadata &a, const QuarterMetadata &b) {
    return a.format_ == b.format_ && a.scale_ == b.scale_;
  }
  friend bool operator!=(const QuarterMetadata &a, const QuarterMetadata &b) { return !(a == b); }

private:
  Format format_;
  signed char scale_;
};

std::ostream &operator<<(std::ostream &os, QuarterMetadata::Format f);

} // namespace poplar

#endif // poplar_Type_hpp
