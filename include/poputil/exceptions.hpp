// poputil::poplibs_error, as include/poputil/exceptions.hpp:17-21 of the reference.
#ifndef poputil_exceptions_hpp
#define poputil_exceptions_hpp

#include <stdexcept>
#include <string>

namespace poputil {

struct poplibs_error : std::runtime_error {
  std::string type;
  explicit poplibs_error(const std::string &s) : std::runtime_error(s), type("poplibs_error") {}
  explicit poplibs_error(const char *s) : std::runtime_error(s), type("poplibs_error") {}
};

} // namespace poputil

#endif // poputil_exceptions_hpp
