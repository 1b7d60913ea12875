// popops::addCodelets: nothing to register on this target (see poplin/codelets.hpp).
#ifndef popops_codelets_hpp
#define popops_codelets_hpp
#include "poplar/Graph.hpp"
namespace popops {
inline void addCodelets(poplar::Graph &) {}
} // namespace popops
#endif // popops_codelets_hpp
