// Stand-in for poplar::Tensor: a cheap value handle, (storage, element type,
// shape, strides, offset), onto memory owned by a Graph.  As in Poplar,
// reshaping / shuffling / slicing never move data: they make views
// (lib/poplin/MatMul.cpp:385-398 and lib/poplin/Convolution.cpp:3073-3086 rely
// on this).
#ifndef poplar_Tensor_hpp
#define poplar_Tensor_hpp

#include <cstddef>
#include <memory>
#include <string>
#include <vector>

#include "poplar/Type.hpp"

namespace poplar {

namespace detail {
struct Storage;  // one device allocation (+ optional quarter metadata)
}

class Tensor {
public:
  Tensor() = default;
  Tensor(std::shared_ptr<detail::Storage> storage, Type type, std::vector<std::size_t> shape);

  bool valid() const { return static_cast<bool>(storage_); }
  Type elementType() const { return type_; }
  unsigned rank() const { return static_cast<unsigned>(shape_.size()); }
  const std::vector<std::size_t> &shape() const { return shape_; }
  std::size_t dim(unsigned i) const;
  std::size_t numElements() const;
  std::string shapeToString() const;

  // ---- views ------------------------------------------------------------------
  Tensor reshape(const std::vector<std::size_t> &shape) const;
  Tensor flatten() const;
  Tensor flatten(unsigned dimBegin, unsigned dimEnd) const;
  Tensor dimShuffle(const std::vector<unsigned> &permutation) const;
  Tensor dimShufflePartial(const std::vector<unsigned> &source,
                           const std::vector<unsigned> &destination) const;
  Tensor dimRoll(unsigned dimIdx, unsigned newIdx = 0) const;
  Tensor transpose() const;
  Tensor expand(const std::vector<std::size_t> &indices) const;
  Tensor squeeze(const std::vector<std::size_t> &indices) const;
  Tensor slice(std::size_t begin, std::size_t end, unsigned dimension = 0) const;
  Tensor operator[](std::size_t i) const;
  Tensor reverse(unsigned dimension) const;
  /// Splits dimension `dim` into (dim/factor, factor) -- used by group handling.
  Tensor reshapePartial(unsigned beginIndex, unsigned endIndex,
                        const std::vector<std::size_t> &newDims) const;

  /// True if a row-major walk of the view visits memory contiguously.
  bool isContiguous() const;
  /// QUARTER tensors: the metadata attached to the underlying storage.
  bool hasMetadata() const;
  QuarterMetadata getMetadata() const;

  // ---- implementation access (used by the poplin layer and the Engine) -------
  const std::vector<std::ptrdiff_t> &strides() const { return strides_; }
  std::ptrdiff_t offset() const { return offset_; }
  const std::shared_ptr<detail::Storage> &storage() const { return storage_; }
  /// Device address of element (0, 0, ..., 0) of the view.
  void *devicePointer() const;

private:
  std::shared_ptr<detail::Storage> storage_;
  Type type_;
  std::vector<std::size_t> shape_;
  std::vector<std::ptrdiff_t> strides_;  // in elements; may be negative (reverse)
  std::ptrdiff_t offset_ = 0;            // in elements from the start of the storage
};

} // namespace poplar

#endif // poplar_Tensor_hpp
