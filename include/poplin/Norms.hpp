// poplin normalisation functions for convolutional layers (the reference's
// include/poplin/Norms.hpp): batch-norm style statistics per channel of an
// activations tensor [N][C][field...], whitening, scale and shift, and the
// three gradients.  Signatures follow the reference; every function appends
// steps to `prog`, nothing runs before the Engine does.  Tensors that are not
// already in the kernels' memory order (N, field..., C) are copied into it.
#ifndef poplin_Norms_hpp
#define poplin_Norms_hpp
#include <functional>
#include <utility>
#include <vector>

#include "poplar/DebugContext.hpp"
#include "poplar/Graph.hpp"
#include "poplar/OptionFlags.hpp"
#include "poplar/Program.hpp"
#include "poplar/Tensor.hpp"

namespace poplin {

/// Per-channel multiplicative parameter (one element per channel of `acts`).
poplar::Tensor createNormGamma(poplar::Graph &graph, const poplar::Tensor &acts,
                               const poplar::Type &type,
                               const poplar::DebugContext &debugContext = {});
poplar::Tensor createNormGamma(poplar::Graph &graph, const poplar::Tensor &acts,
                               const poplar::DebugContext &debugContext = {});
/// Per-channel additive parameter.
poplar::Tensor createNormBeta(poplar::Graph &graph, const poplar::Tensor &acts,
                              const poplar::Type &type,
                              const poplar::DebugContext &debugContext = {});
poplar::Tensor createNormBeta(poplar::Graph &graph, const poplar::Tensor &acts,
                              const poplar::DebugContext &debugContext = {});
/// (gamma, beta).
std::pair<poplar::Tensor, poplar::Tensor>
createNormParams(poplar::Graph &graph, const poplar::Tensor &acts,
                 const poplar::DebugContext &debugContext = {});

/// (mean, 1 / sqrt(variance + eps)) per channel over the batch and the field.
/// With stableAlgo the variance is the mean of squared deviations from the
/// mean, else E[x^2] - mean^2; unbiasedVarEstimate scales it by n / (n - 1).
/// Both results have the activations' type; sums are formed in fp32.
std::pair<poplar::Tensor, poplar::Tensor>
normStatistics(poplar::Graph &graph, const poplar::Tensor &actsUngrouped, float eps,
               poplar::program::Sequence &prog, bool unbiasedVarEstimate, bool stableAlgo = false,
               const poplar::Type &partialsType = poplar::FLOAT,
               const poplar::DebugContext &debugContext = {});

/// Sums the given per-replica tensors over `groupSize` replicas and returns
/// the sums (the caller's all-reduce).
using DistributedNormReduceCallback = std::function<std::vector<poplar::Tensor>(
    poplar::Graph &replicatedGraph, const std::vector<poplar::Tensor> &inputsToReduce,
    poplar::program::Sequence &prog, unsigned groupSize, const poplar::DebugContext &debugContext,
    const poplar::OptionFlags &options)>;

/// normStatistics over `normSize` batch elements spread over replicas that hold
/// acts.dim(0) each: the moments are scaled for the whole batch and handed to
/// the callback before the inverse standard deviation is formed.
std::pair<poplar::Tensor, poplar::Tensor> distributedNormStatistics(
    poplar::Graph &replicatedGraph, const poplar::Tensor &actsUngrouped, float eps,
    poplar::program::Sequence &prog, bool unbiasedVarEstimate,
    DistributedNormReduceCallback allReduceCallback, unsigned normSize, bool stableAlgo = false,
    const poplar::Type &partialsType = poplar::FLOAT, const poplar::DebugContext &debugContext = {});

/// (acts - mean) * iStdDev.
poplar::Tensor normWhiten(poplar::Graph &graph, const poplar::Tensor &acts, const poplar::Tensor &mean,
                          const poplar::Tensor &iStdDev, poplar::program::Sequence &prog,
                          const poplar::DebugContext &debugContext = {});
/// gamma * actsWhitened + beta.
poplar::Tensor normalise(poplar::Graph &graph, const poplar::Tensor &actsWhitened,
                         const poplar::Tensor &gamma, const poplar::Tensor &beta,
                         poplar::program::Sequence &prog,
                         const poplar::DebugContext &debugContext = {});
/// (sum actsWhitened * gradsIn, sum gradsIn) per channel: the gradients of
/// gamma and beta.
std::pair<poplar::Tensor, poplar::Tensor>
normParamGradients(poplar::Graph &graph, const poplar::Tensor &actsWhitened,
                   const poplar::Tensor &gradsIn, poplar::program::Sequence &prog,
                   const poplar::Type &partialsType = poplar::FLOAT,
                   const poplar::DebugContext &debugContext = {});
/// gradsIn * gamma: the gradient through the scale and shift.
poplar::Tensor normGradients(poplar::Graph &graph, const poplar::Tensor &gradsIn,
                             const poplar::Tensor &gamma, poplar::program::Sequence &prog,
                             const poplar::DebugContext &debugContext = {});
/// The gradient through the whitening, given the gradient of its output.
poplar::Tensor normStatisticsGradients(poplar::Graph &graph, const poplar::Tensor &actsWhitened,
                                       const poplar::Tensor &gradsIn, const poplar::Tensor &invStdDev,
                                       poplar::program::Sequence &prog,
                                       const poplar::Type &partialsType = poplar::FLOAT,
                                       const poplar::DebugContext &debugContext = {});
poplar::Tensor distributedNormStatisticsGradients(
    poplar::Graph &replicatedGraph, const poplar::Tensor &actsWhitened, const poplar::Tensor &gradsIn,
    const poplar::Tensor &invStdDev, poplar::program::Sequence &prog,
    poplin::DistributedNormReduceCallback reduceCallback, unsigned normSize,
    const poplar::Type &partialsType = poplar::FLOAT, const poplar::DebugContext &debugContext = {});

} // namespace poplin

#endif // poplin_Norms_hpp
