// Stand-in for the two index helpers of the reference's poputil/Util.hpp
// (include/poputil/Util.hpp:80-105) that its CPU models call.  The real header
// pulls in the Poplar SDK, which is not available; this one keeps only
// row-major flatten / unflatten.  TEST INFRASTRUCTURE ONLY.
#ifndef ORACLE_SHIM_POPUTIL_UTIL_HPP
#define ORACLE_SHIM_POPUTIL_UTIL_HPP

#include <cassert>
#include <cstddef>
#include <vector>

namespace poputil {

// Row-major coordinates of a flat element index.
template <class T>
std::vector<T> unflattenIndex(const std::vector<T> &shape, std::size_t index) {
  std::vector<T> coord(shape.size());
  std::size_t d = shape.size();
  while (d-- > 0) {
    coord[d] = static_cast<T>(index % shape[d]);
    index /= shape[d];
  }
  assert(index == 0);
  return coord;
}

// Flat row-major element index of a coordinate.
template <class T>
std::size_t flattenIndex(const std::vector<T> &shape,
                         const std::vector<T> &indices) {
  assert(shape.size() == indices.size());
  std::size_t flat = 0;
  for (std::size_t d = 0; d != shape.size(); ++d)
    flat = flat * shape[d] + indices[d];
  return flat;
}

} // namespace poputil

#endif // ORACLE_SHIM_POPUTIL_UTIL_HPP
