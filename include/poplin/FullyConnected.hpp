// poplin::fc::getMatMulPrePlanParameters (include/poplin/FullyConnected.hpp:17-53).
#ifndef poplin_FullyConnected_hpp
#define poplin_FullyConnected_hpp
#include <utility>
#include <vector>

#include "poplin/MatMul.hpp"

namespace poplin {
namespace fc {

struct FullyConnectedParams {
  std::size_t numGroups;
  std::size_t batchSize;
  std::size_t inputSize;
  std::size_t outputSize;
};

/// The forward (and, unless inferenceOnly, backward and weight-update) matrix
/// products of a fully connected layer with their fullyConnectedPass option.
std::vector<std::pair<MatMulParams, poplar::OptionFlags>>
getMatMulPrePlanParameters(FullyConnectedParams parameters, poplar::OptionFlags matmulOptions,
                           poplar::Type type, bool inferenceOnly);

} // namespace fc
} // namespace poplin
#endif // poplin_FullyConnected_hpp
