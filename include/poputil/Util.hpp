// Index helpers of include/poputil/Util.hpp:80-105 (row-major flatten /
// unflatten); the tile-mapping utilities of that header have no meaning here.
#ifndef poputil_Util_hpp
#define poputil_Util_hpp

#include <cassert>
#include <cstddef>
#include <vector>

namespace poputil {

template <class T> std::vector<T> unflattenIndex(const std::vector<T> &shape, std::size_t index) {
  std::vector<T> coord(shape.size());
  for (std::size_t d = shape.size(); d-- > 0;) {
    coord[d] = static_cast<T>(index % shape[d]);
    index /= shape[d];
  }
  assert(index == 0);
  return coord;
}

template <class T>
std::size_t flattenIndex(const std::vector<T> &shape, const std::vector<T> &indices) {
  assert(shape.size() == indices.size());
  std::size_t flat = 0;
  for (std::size_t d = 0; d != shape.size(); ++d) flat = flat * shape[d] + indices[d];
  return flat;
}

} // namespace poputil

#endif // poputil_Util_hpp
