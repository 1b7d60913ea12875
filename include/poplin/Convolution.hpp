// poplin convolution entry points with the call surface of the reference's
// include/poplin/Convolution.hpp: they append work to a poplar program; nothing
// runs until an Engine runs that program.
//
// Tensor shapes are the reference's external ones: activations
// [N][G*C][field...], weights [G][Co][Ci][kernel...] (a missing leading G of 1 is
// accepted), output [N][G*Co][outField...].  createInput / createWeights /
// createConvOutput return such tensors laid out in memory the way the kernels
// read them (channels innermost), exactly as the reference's create functions
// return plan-friendly layouts; tensors in any other layout are rearranged by
// a copy inside the program.
#ifndef poplin_Convolution_hpp
#define poplin_Convolution_hpp

#include <cstdint>
#include <iosfwd>
#include <istream>
#include <limits>
#include <memory>
#include <set>
#include <tuple>

#include "poplar/DebugContext.hpp"
#include "poplar/Graph.hpp"
#include "poplar/OptionFlags.hpp"
#include "poplar/Program.hpp"
#include "poplar/Tensor.hpp"
#include "poplin/ConvParams.hpp"

namespace poplin {

class PlanningCache;

/// 2 x multiply-accumulates of each pass; products with padding are not counted.
std::uint64_t getFwdFlops(const ConvParams &params);
std::uint64_t getBwdFlops(const ConvParams &params);
std::uint64_t getWuFlops(const ConvParams &params);
/// Time, in seconds, a pass would take at the device's tensor-core peak (the
/// counterpart of the reference's get*PerfectCycleCount).
double getFwdPerfectSeconds(const ConvParams &params, double peakFlopsPerSecond);
/// Cycles of each pass at full use of the target's arithmetic: the
/// multiply-accumulates (padding excluded) / (MACs per SM and cycle x SMs).
/// An optimistic number for judging efficiency, as in the reference.
double getFwdPerfectCycleCount(const poplar::Graph &graph, const ConvParams &params);
double getBwdPerfectCycleCount(const poplar::Graph &graph, const ConvParams &params);
double getWuPerfectCycleCount(const poplar::Graph &graph, const ConvParams &params);

poplar::Tensor createWeights(poplar::Graph &graph, const ConvParams &params,
                             const poplar::DebugContext &debugContext = {},
                             const poplar::OptionFlags &options = {},
                             PlanningCache *cache = nullptr);
poplar::Tensor createBiases(poplar::Graph &graph, const poplar::Tensor &activations,
                            const poplar::DebugContext &debugContext = {});
poplar::Tensor createBiases(poplar::Graph &graph, const poplar::Tensor &activations,
                            const ConvParams &params, const poplar::DebugContext &debugContext = {},
                            const poplar::OptionFlags &options = {},
                            PlanningCache *cache = nullptr);
poplar::Tensor createInput(poplar::Graph &graph, const ConvParams &params,
                           const poplar::DebugContext &debugContext = {},
                           const poplar::OptionFlags &options = {},
                           PlanningCache *cache = nullptr);
poplar::Tensor createConvOutput(poplar::Graph &graph, const ConvParams &params,
                                const poplar::DebugContext &debugContext = {},
                                const poplar::OptionFlags &options = {},
                                PlanningCache *cache = nullptr);

/// out = conv(in, weights).  With transposeAndFlipWeights the weights are the
/// FORWARD pass's [G][Co][Ci][k...] tensor and are used with their channel axes
/// swapped and their spatial axes flipped (the backward pass).
poplar::Tensor convolution(poplar::Graph &graph, const poplar::Tensor &in,
                           const poplar::Tensor &weights, const ConvParams &params,
                           bool transposeAndFlipWeights, poplar::program::Sequence &prog,
                           const poplar::DebugContext &debugContext = {},
                           const poplar::OptionFlags &options = {},
                           PlanningCache *cache = nullptr);
void convolutionWithOutput(poplar::Graph &graph, const poplar::Tensor &in,
                           const poplar::Tensor &weights, const poplar::Tensor &out,
                           const ConvParams &params, bool transposeAndFlipWeights,
                           poplar::program::Sequence &prog,
                           const poplar::DebugContext &debugContext = {},
                           const poplar::OptionFlags &options = {},
                           PlanningCache *cache = nullptr);

using ConvPlanParams =
    std::tuple<const poplar::Target *, const ConvParams, const poplar::OptionFlags *>;
/// \deprecated Use preplan() (poplin/ConvPreplan.hpp).
void preplanConvolutions(const std::set<ConvPlanParams> &convs, PlanningCache &cache);
void preplanConvolutions(poplar::Graph &graph, const std::set<ConvPlanParams> &convs,
                         PlanningCache &cache);

/// weightsOut[g][ci][co][K-1-k...] = weightsIn[g][co][ci][k...].
void weightsTransposeChansFlipXY(poplar::Graph &graph, const poplar::Tensor &weightsIn,
                                 const poplar::Tensor &weightsOut,
                                 poplar::program::Sequence &prog,
                                 const poplar::DebugContext &debugContext = {});

/// Gradient with respect to the weights, [G][Co][Ci][k...], of type params.inputType.
poplar::Tensor calculateWeightDeltas(poplar::Graph &graph, const poplar::Tensor &zDeltas,
                                     const poplar::Tensor &activations, const ConvParams &params,
                                     poplar::program::Sequence &prog,
                                     const poplar::DebugContext &debugContext = {},
                                     const poplar::OptionFlags &options = {},
                                     PlanningCache *cache = nullptr);
/// weights += scale * weightDeltas.
void convolutionWeightUpdate(poplar::Graph &graph, const poplar::Tensor &zDeltas,
                             const poplar::Tensor &weights, const poplar::Tensor &activations,
                             ConvParams params, const poplar::Tensor &scale,
                             poplar::program::Sequence &prog,
                             const poplar::DebugContext &debugContext = {},
                             const poplar::OptionFlags &options = {},
                             PlanningCache *cache = nullptr);
void convolutionWeightUpdate(poplar::Graph &graph, const poplar::Tensor &zDeltas,
                             const poplar::Tensor &weights, const poplar::Tensor &activations,
                             ConvParams params, float scale, poplar::program::Sequence &prog,
                             const poplar::DebugContext &debugContext = {},
                             const poplar::OptionFlags &options = {},
                             PlanningCache *cache = nullptr);
/// biases[c] += scale * sum over batch and field of zDeltas[n][c][...]; sums in fp32.
void convolutionBiasUpdate(poplar::Graph &graph, const poplar::Tensor &zDeltas,
                           const poplar::Tensor &biases, const poplar::Tensor &scale,
                           const poplar::OptionFlags &options, poplar::program::Sequence &prog,
                           const poplar::DebugContext &debugContext = {});
void convolutionBiasUpdate(poplar::Graph &graph, const poplar::Tensor &zDeltas,
                           const poplar::Tensor &biases, float scale,
                           const poplar::OptionFlags &options, poplar::program::Sequence &prog,
                           const poplar::DebugContext &debugContext = {});
/// acts[n][c][...] += biases[c].
void addBias(poplar::Graph &graph, const poplar::Tensor &in, const poplar::Tensor &biases,
             poplar::program::Sequence &prog, const poplar::DebugContext &debugContext = {});

/// Writes the plan chosen for these parameters (CTA tile, pixel box, pipeline
/// depth, split-K, grid) with its algorithmic FLOPs and bytes.
void reportPlanInfo(std::ostream &out, const poplar::Graph &graph, const ConvParams &params,
                    const poplar::OptionFlags &options = {}, PlanningCache *cache = nullptr);
void reportWeightUpdatePlanInfo(std::ostream &out, const poplar::Graph &graph,
                                const ConvParams &fwdParams,
                                const poplar::OptionFlags &fwdOptions = {},
                                PlanningCache *cache = nullptr);

struct PlanCosts {
  constexpr static std::size_t unknown = std::numeric_limits<std::size_t>::max();
  std::size_t cycles = unknown;  ///< estimated SM cycles at the roofline
  std::size_t memory = unknown;  ///< scratch bytes the plan needs
};
PlanCosts reportPlanEstimatedCosts(const poplar::Graph &graph, const ConvParams &params,
                                   const poplar::OptionFlags &options = {},
                                   PlanningCache *cache = nullptr);

namespace internal {
/// Itemised estimate of what the plan costs.  The fields keep the reference's
/// names; on this target a convolution has no exchange, broadcast or dynamic
/// slicing phases, so those stay zero: `rearrangement` is a preparatory pass
/// over the operands where the plan needs one (padded channels, space-to-depth,
/// depth folding), `compute` the contraction kernel at its roofline,
/// `reduction` the kernel that adds split-K partial sums, `outputCast` is part
/// of the kernels' epilogues.  parallelSplit = CTAs launched, serialSplit = 1.
struct DetailedPlanCosts {
  std::size_t parallelSplit = 1;
  std::size_t serialSplit = 1;
  PlanCosts broadcast = {};
  PlanCosts rearrangement = {};
  PlanCosts dynamicSlice = {};
  PlanCosts transform = {};
  PlanCosts exchange = {};
  PlanCosts tileLevelTransform = {};
  PlanCosts inputsCast = {};
  PlanCosts compute = {};
  PlanCosts reduction = {};
  PlanCosts dynamicUpdate = {};
  PlanCosts addInPlace = {};
  PlanCosts outputCast = {};
  PlanCosts total = {};

  template <typename Function>
  void apply(Function fn, bool includeTotal = true, bool serialSplitOnly = false) const {
    const_cast<DetailedPlanCosts *>(this)->apply([&fn](const PlanCosts &c) { fn(c); }, includeTotal,
                                                 serialSplitOnly);
  }
  template <typename Function>
  void apply(Function fn, bool includeTotal = true, bool serialSplitOnly = false) {
    PlanCosts *always[] = {&dynamicSlice, &transform, &exchange, &tileLevelTransform, &inputsCast,
                           &compute, &reduction, &dynamicUpdate};
    if (!serialSplitOnly) {
      fn(broadcast);
      fn(rearrangement);
    }
    for (PlanCosts *c : always) fn(*c);
    if (!serialSplitOnly) {
      fn(addInPlace);
      fn(outputCast);
    }
    if (includeTotal) fn(total);
  }
};
std::ostream &operator<<(std::ostream &os, DetailedPlanCosts const &c);
std::istream &operator>>(std::istream &is, DetailedPlanCosts &c);
DetailedPlanCosts reportDetailedPlanEstimatedCosts(const poplar::Graph &graph, const ConvParams &params,
                                                   const poplar::OptionFlags &options = {},
                                                   PlanningCache *cache = nullptr);
}  // namespace internal

/// The weights of a fully connected layer (a 1-D convolution) arranged for the
/// backward pass described by `params`: [G][Ci][Co][k] from [G][Co][Ci][k].
poplar::Tensor fullyConnectedWeightTranspose(poplar::Graph &graph, poplar::Tensor weights,
                                             const ConvParams &params, poplar::program::Sequence &prog,
                                             const poplar::DebugContext &debugContext = {},
                                             const poplar::OptionFlags &options = {},
                                             PlanningCache *cache = nullptr);

/// Throws poplar::invalid_option for an unknown key or a bad value.
void convolutionValidateOptions(const poplar::OptionFlags &options);

class PlanningCacheImpl;
/// Caller-owned cache of plans keyed by (parameters, options).
class PlanningCache {
public:
  PlanningCache();
  ~PlanningCache();
  std::size_t size() const;
  std::unique_ptr<PlanningCacheImpl> impl;
};

} // namespace poplin

#endif // poplin_Convolution_hpp
