// Shared helpers of the poplin layer.
#pragma once

#include <string>

#include "poplar/Graph.hpp"
#include "poplar/OptionFlags.hpp"
#include "poplar/Program.hpp"
#include "poplar/Tensor.hpp"
#include "poplin/ConvParams.hpp"
#include "poplibs_b200.h"

namespace poplin {
namespace internal {

/// Flat C ABI form of the parameters; throws poplibs_error for more than three
/// field dimensions or element types the path does not handle.
plb_conv_params toPlb(const ConvParams &p);

// poplin::Pass (lib/poplin/ConvOptions.hpp:13-24)
enum class Pass {
  NONE, NONE_MATMUL, INFERENCE_FWD, TRAINING_FWD, TRAINING_BWD, TRAINING_WU,
  FC_INFERENCE_FWD, FC_TRAINING_FWD, FC_TRAINING_BWD, FC_TRAINING_WU
};

/// Parsed convolution options (lib/poplin/ConvOptions.hpp:26-106).  The keys
/// that steer IPU-specific lowering are accepted, validated and unused.
struct ConvOptions {
  double availableMemoryProportion = 0.6;
  Pass pass = Pass::NONE;
  poplar::Type partialsType = poplar::FLOAT;
  poplar::Type interTilePartialsType = poplar::FLOAT;
  poplar::Type interIpuPartialsType = poplar::FLOAT;
  bool use128BitConvUnitLoad = false;
  std::string planConstraints;  // JSON text, validated
  std::string planConstraintsOutputFilename;
  bool enableMultiStageReduce = true;
  bool enableFastReduce = false;
  bool remapOutputTensor = true;
  bool enableConvDithering = false;
  bool disableTransformations = false;
  bool insertTransformsCycleCountProgs = false;
  bool experimentalConvTransformsEstimates = false;
  bool gatherConvOutput = false;
  bool experimentalSlicVmac16 = false;
  bool disableSRForAMPVertices = false;
  bool enableTileLevelExpandDims = false;

  ConvOptions() = default;
  /// Throws poplar::invalid_option on an unknown key or a bad value.
  explicit ConvOptions(const poplar::OptionFlags &options);
  /// What the options and plan constraints mean for the CUDA planner.
  plb_conv_options toPlb() const;
};

/// Validates the grammar of a planConstraints value
/// (lib/poplin/ConvOptions.cpp:156-329) and returns it unchanged.
std::string validatePlanConstraints(const std::string &jsonText);

/// matMul option set -> equivalent convolution option set
/// (lib/poplin/MatMul.cpp:113-195).
poplar::OptionFlags matMulToConvOptions(const poplar::OptionFlags &matmulOptions);

/// `acts` ([N][C][field...]) in the kernels' memory order (N, field..., C):
/// itself when it already is, else a scratch copy recorded in `prog`.
poplar::Tensor actsInKernelLayout(poplar::Graph &graph, const poplar::Tensor &acts,
                                  poplar::program::Sequence &prog, bool copyValues = true);
/// A new activations tensor of the logical shape of `like` and element type
/// `type`, stored in the kernels' memory order.
poplar::Tensor newActsLike(poplar::Graph &graph, const poplar::Tensor &like, const poplar::Type &type,
                           const std::string &name);

}  // namespace internal
}  // namespace poplin
