// poplin::preplan (include/poplin/ConvPreplan.hpp:36-37): plans a set of
// convolutions and matrix products ahead of graph construction and stores the
// plans in the cache.
#ifndef poplin_ConvPreplan_hpp
#define poplin_ConvPreplan_hpp
#include <set>

#include "poplin/Convolution.hpp"
#include "poplin/MatMul.hpp"

namespace poplin {
void preplan(const std::set<ConvPlanParams> &convs, const std::set<MatMulPlanParams> &matmuls,
             PlanningCache &cache);
} // namespace poplin
#endif // poplin_ConvPreplan_hpp
