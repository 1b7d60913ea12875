// poplin::multiconv over the single-convolution entry points
// (lib/poplin/MultiConvolution.cpp; options lib/poplin/ConvPlan.cpp:1927-1955).
#include "poplin/MultiConvolution.hpp"

#include <map>

#include "poplar/exceptions.hpp"
#include "poputil/OptionParsing.hpp"
#include "poputil/exceptions.hpp"

namespace poplin {
namespace multiconv {
namespace {

enum class MultiPlanType { PARALLEL, SERIAL };

// Parses (and thereby validates) the options of a multi-convolution.  None of
// them changes what runs: the launches of the individual convolutions follow
// one another on the stream whatever the plan type.
void checkOptions(const poplar::OptionFlags &options) {
  using poplibs::OptionHandler;
  using poplibs::OptionSpec;
  MultiPlanType planType = MultiPlanType::PARALLEL;
  unsigned perConvReservedTiles = 50;
  double cycleBackOff = 0.1;
  const OptionSpec spec{
      {"planType", OptionHandler::createWithEnum(
                       planType, std::map<std::string, MultiPlanType>{{"parallel", MultiPlanType::PARALLEL},
                                                                      {"serial", MultiPlanType::SERIAL}})},
      {"perConvReservedTiles", OptionHandler::createWithInteger(perConvReservedTiles)},
      {"cycleBackOff", OptionHandler::createWithDouble(cycleBackOff)},
  };
  for (const auto &entry : options) spec.parse(entry.first, entry.second);
}

template <typename Args> const typename Args::value_type &at(const Args &args, unsigned index, const char *what) {
  if (index >= args.size())
    throw poputil::poplibs_error(std::string("multiconv::") + what + ": index " + std::to_string(index) +
                                 " is out of range for " + std::to_string(args.size()) + " convolutions");
  return args[index];
}

std::string nameOf(const poplar::DebugContext &dc, std::size_t i) {
  return dc.getPathName() + "/conv" + std::to_string(i);
}

} // namespace

poplar::Tensor createWeights(poplar::Graph &graph, const std::vector<CreateTensorArgs> &args,
                             unsigned weightsIndex, const poplar::OptionFlags &options,
                             PlanningCache *cache) {
  checkOptions(options);
  const auto &a = at(args, weightsIndex, "createWeights");
  return poplin::createWeights(graph, a.params, a.name, a.options, cache);
}

poplar::Tensor createInput(poplar::Graph &graph, const std::vector<CreateTensorArgs> &args,
                           unsigned inputIndex, const poplar::OptionFlags &options,
                           PlanningCache *cache) {
  checkOptions(options);
  const auto &a = at(args, inputIndex, "createInput");
  return poplin::createInput(graph, a.params, a.name, a.options, cache);
}

void weightsTransposeChansFlipXY(poplar::Graph &graph, std::vector<ConvolutionArgs> &args,
                                 const std::vector<poplar::Tensor> &weightsIn,
                                 poplar::program::Sequence &prog, const poplar::OptionFlags &options,
                                 const poplar::DebugContext &debugContext, PlanningCache *cache) {
  checkOptions(options);
  if (weightsIn.size() != args.size())
    throw poputil::poplibs_error("multiconv::weightsTransposeChansFlipXY: " +
                                 std::to_string(weightsIn.size()) + " weight tensors for " +
                                 std::to_string(args.size()) + " convolutions");
  for (std::size_t i = 0; i != args.size(); ++i) {
    args[i].weights =
        poplin::createWeights(graph, args[i].params, nameOf(debugContext, i) + "/bwdWeights",
                              args[i].options, cache);
    poplin::weightsTransposeChansFlipXY(graph, weightsIn[i], args[i].weights, prog,
                                        nameOf(debugContext, i));
  }
}

std::vector<poplar::Tensor> convolution(poplar::Graph &graph,
                                        const std::vector<ConvolutionArgs> &args,
                                        bool transposeAndFlipWeights,
                                        poplar::program::Sequence &prog,
                                        const poplar::DebugContext &debugContext,
                                        const poplar::OptionFlags &options, PlanningCache *cache) {
  checkOptions(options);
  std::vector<poplar::Tensor> out;
  out.reserve(args.size());
  for (std::size_t i = 0; i != args.size(); ++i)
    out.push_back(poplin::convolution(graph, args[i].inputs, args[i].weights, args[i].params,
                                      transposeAndFlipWeights, prog, nameOf(debugContext, i),
                                      args[i].options, cache));
  return out;
}

std::vector<poplar::Tensor> calculateWeightDeltas(poplar::Graph &graph,
                                                  const std::vector<CalculateWeightDeltasArgs> &args,
                                                  poplar::program::Sequence &prog,
                                                  const poplar::DebugContext &debugContext,
                                                  const poplar::OptionFlags &options,
                                                  PlanningCache *cache) {
  checkOptions(options);
  std::vector<poplar::Tensor> out;
  out.reserve(args.size());
  for (std::size_t i = 0; i != args.size(); ++i)
    out.push_back(poplin::calculateWeightDeltas(graph, args[i].zDeltas, args[i].activations,
                                                args[i].params, prog, nameOf(debugContext, i),
                                                args[i].options, cache));
  return out;
}

void convolutionWeightUpdate(poplar::Graph &graph, const std::vector<ConvWeightUpdateArgs> &args,
                             poplar::program::Sequence &prog,
                             const poplar::DebugContext &debugContext,
                             const poplar::OptionFlags &options, PlanningCache *cache) {
  checkOptions(options);
  for (std::size_t i = 0; i != args.size(); ++i)
    poplin::convolutionWeightUpdate(graph, args[i].zDeltas, args[i].weights, args[i].activations,
                                    args[i].params, args[i].scale, prog, nameOf(debugContext, i),
                                    args[i].options, cache);
}

void convolutionWeightUpdate(poplar::Graph &graph,
                             const std::vector<ConvWeightUpdateArgsScalar> &args,
                             poplar::program::Sequence &prog,
                             const poplar::DebugContext &debugContext,
                             const poplar::OptionFlags &options, PlanningCache *cache) {
  checkOptions(options);
  for (std::size_t i = 0; i != args.size(); ++i)
    poplin::convolutionWeightUpdate(graph, args[i].zDeltas, args[i].weights, args[i].activations,
                                    args[i].params, args[i].scale, prog, nameOf(debugContext, i),
                                    args[i].options, cache);
}

} // namespace multiconv
} // namespace poplin
