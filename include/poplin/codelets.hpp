// poplin::addCodelets (include/poplin/codelets.hpp:10): on the IPU this
// registers the vertex code with the graph; the GPU kernels live in the shared
// library, so there is nothing to add.
#ifndef poplin_codelets_hpp
#define poplin_codelets_hpp
#include "poplar/Graph.hpp"
namespace poplin {
inline void addCodelets(poplar::Graph &) {}
} // namespace poplin
#endif // poplin_codelets_hpp
