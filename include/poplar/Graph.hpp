// Stand-in for poplar::Graph: owns the device memory of the variables created
// on it and the C ABI context (device + stream) programs run on.
#ifndef poplar_Graph_hpp
#define poplar_Graph_hpp

#include <cstddef>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "poplar/DebugContext.hpp"
#include "poplar/Target.hpp"
#include "poplar/Tensor.hpp"
#include "poplar/Type.hpp"

struct plb_context;

namespace poplar {

enum class VariableMappingMethod { NONE, LINEAR };
enum class TensorCloneMethod {
  PRESERVE_ORDER_AND_ALIASES,
  CREATE_NEW_ORDER,
  PRESERVE_ORDER_UNLESS_ALIASES,
  GATHER_AND_PRESERVE_TILE_ORDER_AND_ALIASES
};

namespace detail {
struct GraphImpl;
}

class Graph {
public:
  explicit Graph(const Target &target);
  ~Graph();
  Graph(Graph &&) noexcept;
  Graph(const Graph &) = delete;

  const Target &getTarget() const;

  /// A new variable stored row-major (dense) in device memory.
  Tensor addVariable(const Type &type, const std::vector<std::size_t> &shape,
                     const DebugContext &dc = {});
  Tensor addVariable(const Type &type, const std::vector<std::size_t> &shape,
                     VariableMappingMethod, const DebugContext &dc = {});
  /// QUARTER variables carry their metadata with the storage.
  Tensor addVariable(const Type &type, const Tensor *metadata,
                     const std::vector<std::size_t> &shape, const DebugContext &dc = {});
  template <class T>
  Tensor addConstant(const Type &type, const std::vector<std::size_t> &shape, T value,
                     const DebugContext &dc = {}) {
    return addConstantImpl(type, shape, static_cast<double>(value), dc);
  }
  /// Same shape, type and memory layout as `t`, fresh storage.
  Tensor clone(const Tensor &t, const DebugContext &dc = {},
               TensorCloneMethod = TensorCloneMethod::PRESERVE_ORDER_UNLESS_ALIASES);
  Tensor clone(const Type &type, const Tensor &t, const DebugContext &dc = {},
               TensorCloneMethod = TensorCloneMethod::PRESERVE_ORDER_UNLESS_ALIASES);

  /// Tile mapping has no meaning on a GPU; accepted and ignored.
  template <class... A> void setTileMapping(const Tensor &, A &&...) {}

  /// Host access points (Poplar: createHostWrite / createHostRead); the Engine
  /// moves data through them in the tensor's logical (row-major) order.
  void createHostWrite(const std::string &handle, const Tensor &t);
  void createHostRead(const std::string &handle, const Tensor &t);

  /// Sets the metadata of a QUARTER tensor (in Poplar the metadata is a tensor
  /// written like any other; here it lives on the host beside the storage).
  void setQuarterMetadata(const Tensor &t, const QuarterMetadata &md);

  // ---- implementation access --------------------------------------------------
  plb_context *context() const;
  const std::map<std::string, Tensor> &hostWrites() const;
  const std::map<std::string, Tensor> &hostReads() const;
  /// Scratch variable that lives as long as the graph (plan-private buffers).
  Tensor addScratch(const Type &type, const std::vector<std::size_t> &shape);
  /// Gives every variable created so far its device memory (done by the Engine).
  void allocateDeviceMemory();

private:
  Tensor addConstantImpl(const Type &type, const std::vector<std::size_t> &shape, double value,
                         const DebugContext &dc);
  std::unique_ptr<detail::GraphImpl> impl_;
};

} // namespace poplar

#endif // poplar_Graph_hpp
