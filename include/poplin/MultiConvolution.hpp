// poplin::multiconv (include/poplin/MultiConvolution.hpp:62-276): several
// independent convolutions described, created and run together.
//
// On the IPU the point of the interface is to plan the convolutions onto
// disjoint sets of tiles so that they run side by side.  Here every
// convolution is one or more kernel launches on the engine's stream; the
// launches of a multi-convolution are enqueued back to back and, being
// programmatic dependent launches, overlap each other's set-up and tail.  The
// multi-convolution options (planType, perConvReservedTiles, cycleBackOff) are
// validated and otherwise have no effect.
#ifndef poplin_MultiConvolution_hpp
#define poplin_MultiConvolution_hpp
#include <string>
#include <vector>

#include "poplin/Convolution.hpp"

namespace poplin {
namespace multiconv {

struct CreateTensorArgs {
  ConvParams params;
  poplar::OptionFlags options;
  std::string name;
};

poplar::Tensor createWeights(poplar::Graph &graph, const std::vector<CreateTensorArgs> &args,
                             unsigned weightsIndex, const poplar::OptionFlags &options = {},
                             poplin::PlanningCache *cache = nullptr);
poplar::Tensor createInput(poplar::Graph &graph, const std::vector<CreateTensorArgs> &args,
                           unsigned inputIndex, const poplar::OptionFlags &options = {},
                           poplin::PlanningCache *cache = nullptr);

struct ConvolutionArgs {
  poplar::Tensor inputs;
  poplar::Tensor weights;
  ConvParams params;
  poplar::OptionFlags options;
};

/// Fills args[i].weights with the channel-transposed, spatially flipped
/// weightsIn[i] (a new tensor each).
void weightsTransposeChansFlipXY(poplar::Graph &graph, std::vector<ConvolutionArgs> &args,
                                 const std::vector<poplar::Tensor> &weightsIn,
                                 poplar::program::Sequence &prog, const poplar::OptionFlags &options,
                                 const poplar::DebugContext &debugContext,
                                 poplin::PlanningCache *cache);

std::vector<poplar::Tensor> convolution(poplar::Graph &graph,
                                        const std::vector<ConvolutionArgs> &args,
                                        bool transposeAndFlipWeights,
                                        poplar::program::Sequence &prog,
                                        const poplar::DebugContext &debugContext = {},
                                        const poplar::OptionFlags &options = {},
                                        poplin::PlanningCache *cache = nullptr);

struct CalculateWeightDeltasArgs {
  poplar::Tensor zDeltas;
  poplar::Tensor activations;
  ConvParams params;
  poplar::OptionFlags options;
};

std::vector<poplar::Tensor> calculateWeightDeltas(poplar::Graph &graph,
                                                  const std::vector<CalculateWeightDeltasArgs> &args,
                                                  poplar::program::Sequence &prog,
                                                  const poplar::DebugContext &debugContext = {},
                                                  const poplar::OptionFlags &options = {},
                                                  poplin::PlanningCache *cache = nullptr);

struct ConvWeightUpdateArgs {
  poplar::Tensor zDeltas;
  poplar::Tensor weights;
  poplar::Tensor activations;
  poplar::Tensor scale;
  ConvParams params;
  poplar::OptionFlags options;
};

void convolutionWeightUpdate(poplar::Graph &graph, const std::vector<ConvWeightUpdateArgs> &args,
                             poplar::program::Sequence &prog,
                             const poplar::DebugContext &debugContext = {},
                             const poplar::OptionFlags &options = {},
                             poplin::PlanningCache *cache = nullptr);

struct ConvWeightUpdateArgsScalar {
  poplar::Tensor zDeltas;
  poplar::Tensor weights;
  poplar::Tensor activations;
  float scale;
  ConvParams params;
  poplar::OptionFlags options;
};

void convolutionWeightUpdate(poplar::Graph &graph,
                             const std::vector<ConvWeightUpdateArgsScalar> &args,
                             poplar::program::Sequence &prog,
                             const poplar::DebugContext &debugContext = {},
                             const poplar::OptionFlags &options = {},
                             poplin::PlanningCache *cache = nullptr);

} // namespace multiconv
} // namespace poplin
#endif // poplin_MultiConvolution_hpp
