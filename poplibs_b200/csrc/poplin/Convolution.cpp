// poplin convolution entry points over the C ABI.  Each call checks its
// arguments, brings the operands into the kernels' memory layouts (views where
// possible, a recorded copy otherwise) and appends one step to the program
// that launches the CUDA kernels when an Engine runs it
// (counterpart of lib/poplin/Convolution.cpp:1445-1725, 3067-3648).
#include "poplin/Convolution.hpp"

#include <algorithm>
#include <fstream>
#include <cmath>
#include <iostream>
#include <map>
#include <numeric>
#include <sstream>

#include "../poplar/standin_impl.hpp"
#include "internal.hpp"
#include "poplar/exceptions.hpp"
#include "poplibs_support/logging.hpp"
#include "poplin/ConvPreplan.hpp"
#include "poplin/ConvUtil.hpp"
#include "poputil/exceptions.hpp"

namespace poplin {

using poplar::Graph;
using poplar::Tensor;
using poplar::program::Sequence;
using poputil::poplibs_error;
namespace logging = poplibs_support::logging;

// ---- planning cache ------------------------------------------------------------
class PlanningCacheImpl {
public:
  std::map<std::string, plb_plan> plans;
};

PlanningCache::PlanningCache() : impl(new PlanningCacheImpl()) {}
PlanningCache::~PlanningCache() = default;
std::size_t PlanningCache::size() const { return impl->plans.size(); }

namespace {

std::string cacheKey(const ConvParams &p, const poplar::OptionFlags &options, int pass) {
  std::ostringstream os;
  os << std::hash<ConvParams>()(p) << '|' << p << '|' << options << '|' << pass;
  return os.str();
}

// The chosen plan as a planConstraints value that reproduces it when fed back
// (option planConstraintsOutputFilename; the reference's
// writePlanConstraintsFile, lib/poplin/ConvPlan.cpp:1574-1664): the K split in
// the reference's own grammar (level 0, inChanSplit.parallel) and this
// planner's knobs under "cuda".
std::string planConstraintsOf(const plb_plan &plan) {
  std::ostringstream os;
  const bool igemm = plan.kernel != 1;
  os << "{\n"
     << "  \"0\": {\"partition\": {\"inChanSplit\": {\"serial\": 1, \"parallel\": "
     << std::max(1, int(plan.split_k)) << "}}},\n"
     << "  \"cuda\": {\"splitK\": " << std::max(1, int(plan.split_k));
  if (igemm)
    os << ", \"tileN\": " << plan.tile_n << ", \"residentWeights\": "
       << (plan.resident_weights ? "true" : "false") << ", \"ctaPair\": "
       << (plan.cta_pair ? "true" : "false");
  os << ", \"halo\": " << (plan.halo_rows > 0 ? "true" : "false") << "}\n}\n";
  return os.str();
}

// <name>_FWD.json / _BWD.json / _WU.json, as getPlanConstraintsOutputFile
// (lib/poplin/ConvPlan.cpp:1631-1658).
void writePlanConstraintsFile(const plb_plan &plan, const internal::ConvOptions &options) {
  std::string path = options.planConstraintsOutputFilename;
  switch (options.pass) {
    case internal::Pass::INFERENCE_FWD:
    case internal::Pass::TRAINING_FWD:
    case internal::Pass::FC_INFERENCE_FWD:
    case internal::Pass::FC_TRAINING_FWD: path += "_FWD"; break;
    case internal::Pass::TRAINING_BWD:
    case internal::Pass::FC_TRAINING_BWD: path += "_BWD"; break;
    case internal::Pass::TRAINING_WU:
    case internal::Pass::FC_TRAINING_WU: path += "_WU"; break;
    default: break;
  }
  path += ".json";
  std::ofstream out(path);
  if (!out) throw poplibs_error("cannot write plan constraints to '" + path + "'");
  out << planConstraintsOf(plan);
}

// Plan for one pass of `params` (PLB_PASS_TRAINING_FWD / _BWD / _WU), cached.
plb_plan planFor(const ConvParams &params, const poplar::OptionFlags &options, int pass,
                 PlanningCache *cache) {
  const internal::ConvOptions parsed(options);
  std::string key;
  if (cache) {
    key = cacheKey(params, options, pass);
    const auto it = cache->impl->plans.find(key);
    if (it != cache->impl->plans.end()) return it->second;
  }
  // A convolution whose input is dilated is the backward pass of a strided
  // layer: it is planned (and run) in that layer's forward terms.
  const bool dilatedInput =
      std::any_of(params.inputTransform.dilation.begin(), params.inputTransform.dilation.end(),
                  [](unsigned d) { return d != 1; });
  const plb_conv_params flat =
      internal::toPlb(dilatedInput ? getGradientParams(params).canonicalize() : params);
  if (dilatedInput && pass != PLB_PASS_TRAINING_WU) pass = PLB_PASS_TRAINING_BWD;
  const plb_conv_options opt = parsed.toPlb();
  plb_plan plan{};
  poplar::detail::check(plb_conv_plan(&flat, &opt, pass, &plan));
  if (cache) cache->impl->plans[key] = plan;
  if (!parsed.planConstraintsOutputFilename.empty()) writePlanConstraintsFile(plan, parsed);
  return plan;
}

std::vector<std::size_t> concat(std::initializer_list<std::vector<std::size_t>> parts) {
  std::vector<std::size_t> out;
  for (const auto &p : parts) out.insert(out.end(), p.begin(), p.end());
  return out;
}

// Logical [N][C][field...] tensor stored [N][field...][C].
Tensor makeActs(Graph &graph, const poplar::Type &type, std::size_t batch, std::size_t chans,
                const std::vector<std::size_t> &field, const std::string &name) {
  Tensor t = graph.addVariable(type, concat({{batch}, field, {chans}}), name);
  return t.dimRoll(unsigned(field.size()) + 1, 1);
}

// Logical [G][Co][Ci][kernel...] tensor stored [G][kernel...][Co][Ci].
Tensor makeWeights(Graph &graph, const poplar::Type &type, std::size_t groups, std::size_t co,
                   std::size_t ci, const std::vector<std::size_t> &kernel,
                   const std::string &name) {
  Tensor t = graph.addVariable(type, concat({{groups}, kernel, {co, ci}}), name);
  const unsigned nd = unsigned(kernel.size());
  // stored dims: 0=G, 1..nd=kernel, nd+1=Co, nd+2=Ci -> logical G, Co, Ci, kernel...
  std::vector<unsigned> perm{0, nd + 1, nd + 2};
  for (unsigned d = 0; d != nd; ++d) perm.push_back(1 + d);
  return t.dimShuffle(perm);
}

// True if `t` is dense in memory with its logical dimensions nested in
// `memoryOrder` (outermost first) and starts on a 16-byte boundary.
bool isDenseInOrder(const Tensor &t, const std::vector<unsigned> &memoryOrder) {
  std::ptrdiff_t expect = 1;
  for (std::size_t i = memoryOrder.size(); i-- > 0;) {
    const unsigned d = memoryOrder[i];
    if (t.shape()[d] != 1 && t.strides()[d] != expect) return false;
    expect *= std::ptrdiff_t(t.shape()[d]);
  }
  return (t.offset() * std::ptrdiff_t(t.elementType().bytes())) % 16 == 0;
}

// `t` itself if it already has the wanted memory order, else a scratch tensor
// of the same logical shape with that order, filled by a recorded copy.
Tensor arranged(Graph &graph, const Tensor &t, const std::vector<unsigned> &memoryOrder,
                Sequence &prog, bool copyValues = true) {
  if (isDenseInOrder(t, memoryOrder)) return t;
  std::vector<std::size_t> physical;
  for (unsigned d : memoryOrder) physical.push_back(t.shape()[d]);
  Tensor base = graph.addScratch(t.elementType(), physical);
  std::vector<unsigned> inverse(memoryOrder.size());
  for (unsigned i = 0; i != memoryOrder.size(); ++i) inverse[memoryOrder[i]] = i;
  Tensor view = base.dimShuffle(inverse);
  if (t.elementType() == poplar::QUARTER && t.hasMetadata())
    graph.setQuarterMetadata(view, t.getMetadata());
  if (copyValues) prog.add(poplar::program::Copy(t, view));
  logging::poplin::debug("rearranging a tensor of shape " + t.shapeToString() +
                         " into the kernel layout");
  return view;
}

std::vector<unsigned> actsOrder(unsigned rank) {  // [N][C][f...] stored N, f..., C
  std::vector<unsigned> order{0};
  for (unsigned d = 2; d < rank; ++d) order.push_back(d);
  order.push_back(1);
  return order;
}

std::vector<unsigned> weightsOrder(unsigned rank) {  // [G][Co][Ci][k...] stored G, k..., Co, Ci
  std::vector<unsigned> order{0};
  for (unsigned d = 3; d < rank; ++d) order.push_back(d);
  order.push_back(1);
  order.push_back(2);
  return order;
}

void checkActsShape(const Tensor &t, std::size_t batch, std::size_t chans,
                    const std::vector<std::size_t> &field, const char *what) {
  const auto expect = concat({{batch, chans}, field});
  if (t.shape() != expect) {
    Tensor probe;
    std::string want = "[";
    for (std::size_t i = 0; i < expect.size(); ++i) want += (i ? "," : "") + std::to_string(expect[i]);
    throw poplibs_error(std::string(what) + " tensor has shape " + t.shapeToString() +
                        " but the convolution parameters need " + want + "]");
  }
}

// Exponent to add for a QUARTER operand: its metadata scale, minus one because
// the F143 / F152 formats (exponent bias 8 / 16) hold half of what the same bits
// mean in the E4M3 / E5M2 encodings (bias 7 / 15) the tensor core decodes.
int quarterExponent(const Tensor &t) {
  if (t.elementType() != poplar::QUARTER) return 0;
  const poplar::QuarterMetadata md = t.hasMetadata() ? t.getMetadata() : poplar::QuarterMetadata();
  return int(md.getScale()) - 1;
}

// plb_quarter_format of a QUARTER operand (PLB_F143 for anything else).
int quarterFormat(const Tensor &t) {
  if (t.elementType() != poplar::QUARTER || !t.hasMetadata()) return PLB_F143;
  return t.getMetadata().getFormat() == poplar::QuarterMetadata::Format::F152 ? PLB_F152 : PLB_F143;
}

void validateTypes(const ConvParams &p) {
  // lib/poplin/ConvValidation.cpp:11-70
  for (const auto &t : {p.inputType, p.outputType})
    if (t != poplar::HALF && t != poplar::FLOAT && t != poplar::QUARTER)
      throw poplibs_error("Unsupported convolution type " + t.toString());
  if (p.inputType == poplar::QUARTER && p.outputType != poplar::HALF)
    throw poplibs_error("Output type must be half when input type is quarter");
}

Tensor withGroupDim(const Tensor &weights, const ConvParams &p) {
  // weights without the leading group dimension are accepted
  // (lib/poplin/Convolution.cpp:3073-3076)
  if (weights.rank() == p.getNumFieldDims() + 2) return weights.expand({0});
  return weights;
}

}  // namespace

namespace internal {
Tensor actsInKernelLayout(Graph &graph, const Tensor &acts, Sequence &prog, bool copyValues) {
  return arranged(graph, acts, actsOrder(acts.rank()), prog, copyValues);
}
Tensor newActsLike(Graph &graph, const Tensor &like, const poplar::Type &type, const std::string &name) {
  const auto shape = like.shape();
  return makeActs(graph, type, shape[0], shape[1],
                  std::vector<std::size_t>(shape.begin() + 2, shape.end()), name);
}
}  // namespace internal

// ---- flops ------------------------------------------------------------------------
std::uint64_t getFwdFlops(const ConvParams &params) {
  const plb_conv_params flat = internal::toPlb(params);
  return 2 * plb_conv_macs(&flat);
}
std::uint64_t getBwdFlops(const ConvParams &params) { return getFwdFlops(params); }
std::uint64_t getWuFlops(const ConvParams &params) { return getFwdFlops(params); }
double getFwdPerfectSeconds(const ConvParams &params, double peakFlopsPerSecond) {
  return double(getFwdFlops(params)) / peakFlopsPerSecond;
}

// MACs / (MACs per SM and cycle x SMs), the reference's getPerfectCycleCount
// (lib/poplin/Convolution.cpp:3227-3248) with this target's arithmetic widths.
static double perfectCycleCount(const Graph &graph, const ConvParams &params) {
  const poplar::Target &target = graph.getTarget();
  const double macs = double(getFwdFlops(params)) / 2.0;
  double perTile;
  if (params.inputType == poplar::FLOAT)
    perTile = target.getFloatVectorWidth();
  else if (params.inputType == poplar::QUARTER)
    perTile = double(target.getFp8InFp16OutConvUnitsPerTile()) * target.getQuarterVectorWidth();
  else
    perTile = double(std::max({target.getFp16InFp16OutConvUnitsPerTile(),
                               target.getFp32InFp32OutConvUnitsPerTile(),
                               target.getFp16InFp32OutConvUnitsPerTile()})) *
              target.getHalfVectorWidth();
  return macs / (perTile * target.getNumTiles());
}
double getFwdPerfectCycleCount(const Graph &graph, const ConvParams &params) {
  return perfectCycleCount(graph, params);
}
double getBwdPerfectCycleCount(const Graph &graph, const ConvParams &params) {
  return perfectCycleCount(graph, params);
}
double getWuPerfectCycleCount(const Graph &graph, const ConvParams &params) {
  return perfectCycleCount(graph, params);
}

// ---- tensor creation -----------------------------------------------------------------
Tensor createInput(Graph &graph, const ConvParams &params, const poplar::DebugContext &dc,
                   const poplar::OptionFlags &options, PlanningCache *) {
  params.validate();
  convolutionValidateOptions(options);
  return makeActs(graph, params.inputType, params.batchSize, params.getNumInputChans(),
                  params.inputFieldShape, dc.getPathName());
}

Tensor createWeights(Graph &graph, const ConvParams &params, const poplar::DebugContext &dc,
                     const poplar::OptionFlags &options, PlanningCache *) {
  params.validate();
  convolutionValidateOptions(options);
  return makeWeights(graph, params.inputType, params.numConvGroups,
                     params.outputChannelsPerConvGroup, params.inputChannelsPerConvGroup,
                     params.kernelShape, dc.getPathName());
}

Tensor createConvOutput(Graph &graph, const ConvParams &params, const poplar::DebugContext &dc,
                        const poplar::OptionFlags &options, PlanningCache *) {
  params.validate();
  convolutionValidateOptions(options);
  return makeActs(graph, params.outputType, params.batchSize, params.getNumOutputChans(),
                  params.getOutputFieldShape(), dc.getPathName());
}

Tensor createBiases(Graph &graph, const Tensor &activations, const poplar::DebugContext &dc) {
  if (activations.rank() < 2) throw poplibs_error("createBiases: activations need a channel dimension");
  return graph.addVariable(activations.elementType(), {activations.dim(1)}, dc);
}

Tensor createBiases(Graph &graph, const Tensor &activations, const ConvParams &,
                    const poplar::DebugContext &dc, const poplar::OptionFlags &, PlanningCache *) {
  return createBiases(graph, activations, dc);
}

// ---- convolution ---------------------------------------------------------------------
void convolutionWithOutput(Graph &graph, const Tensor &in, const Tensor &weights_,
                           const Tensor &out, const ConvParams &params,
                           bool transposeAndFlipWeights, Sequence &prog,
                           const poplar::DebugContext &dc, const poplar::OptionFlags &options,
                           PlanningCache *cache) {
  params.validate();
  validateTypes(params);
  const internal::ConvOptions parsed(options);
  const Tensor weights = withGroupDim(weights_, params);
  const std::size_t G = params.numConvGroups, ci = params.inputChannelsPerConvGroup,
                    co = params.outputChannelsPerConvGroup;
  checkActsShape(in, params.batchSize, G * ci, params.inputFieldShape, "input");
  checkActsShape(out, params.batchSize, G * co, params.getOutputFieldShape(), "output");
  const auto wantW = transposeAndFlipWeights ? concat({{G, ci, co}, params.kernelShape})
                                             : concat({{G, co, ci}, params.kernelShape});
  if (weights.shape() != wantW)
    throw poplibs_error("weights tensor has shape " + weights.shapeToString() +
                        ", which does not match the convolution parameters" +
                        (transposeAndFlipWeights ? " (transposed weights expected)" : ""));
  if (in.elementType() != params.inputType || weights.elementType() != params.inputType)
    throw poplibs_error("input / weights element type does not match params.inputType");
  if (out.elementType() != params.outputType)
    throw poplibs_error("output element type does not match params.outputType");

  const plb_plan plan = planFor(params, options, PLB_PASS_TRAINING_FWD, cache);
  (void)plan;
  const Tensor inA = arranged(graph, in, actsOrder(in.rank()), prog);
  const Tensor wA = arranged(graph, weights, weightsOrder(weights.rank()), prog);
  const bool outDirect = isDenseInOrder(out, actsOrder(out.rank()));
  const Tensor outA = outDirect ? out : arranged(graph, out, actsOrder(out.rank()), prog, false);

  const ConvParams canonical = params.canonicalize();
  plb_conv_options opt = parsed.toPlb();
  const int transpose = transposeAndFlipWeights ? 1 : 0;
  const std::string name = dc.getPathName();
  // The backward pass of a strided layer arrives as a convolution whose input
  // (the output gradients) is dilated by the forward stride
  // (getGradientParams, lib/poplin/ConvUtil.cpp:728-795).  The kernels take that
  // pass in forward terms: getGradientParams is its own inverse up to
  // canonicalisation, and the weights are the forward layer's.
  const bool dilatedInput =
      std::any_of(canonical.inputTransform.dilation.begin(), canonical.inputTransform.dilation.end(),
                  [](unsigned d) { return d != 1; });
  if (dilatedInput) {
    // A dilated input met without the transpose flag is the same computation
    // with this convolution's own weights standing for the transposed, flipped
    // ones: hand the library their channel-transposed, spatially flipped copy.
    Tensor wFwd = wA;
    if (!transposeAndFlipWeights) {
      Tensor t = makeWeights(graph, weights.elementType(), G, ci, co, params.kernelShape,
                             name + "/asForwardWeights");
      if (weights.elementType() == poplar::QUARTER && weights.hasMetadata())
        graph.setQuarterMetadata(t, weights.getMetadata());
      weightsTransposeChansFlipXY(graph, weights, t, prog, name);
      wFwd = t;
    }
    const plb_conv_params fwd = internal::toPlb(getGradientParams(params).canonicalize());
    prog.add([=](plb_context *ctx) mutable {
      opt.scale_in = quarterExponent(inA);
      opt.scale_weights = quarterExponent(wFwd);
      opt.format_in = quarterFormat(inA);
      opt.format_weights = quarterFormat(wFwd);
      logging::poplin::trace("convolution (backward of a strided layer) " + name);
      poplar::detail::check(plb_conv_bwd(ctx, &fwd, &opt, inA.devicePointer(), wFwd.devicePointer(),
                                         outA.devicePointer()));
    });
    if (!outDirect) prog.add(poplar::program::Copy(outA, out));
    return;
  }
  const plb_conv_params flat = internal::toPlb(canonical);
  prog.add([=](plb_context *ctx) mutable {
    opt.scale_in = quarterExponent(inA);
    opt.scale_weights = quarterExponent(wA);
    opt.format_in = quarterFormat(inA);
    opt.format_weights = quarterFormat(wA);
    if (flat.in_chans_per_group == 0 || std::any_of(flat.field, flat.field + flat.num_field_dims,
                                                    [](uint32_t f) { return f == 0; })) {
      // nothing is accumulated: the result is zero
      poplar::detail::check(plb_memset(ctx, outA.devicePointer(), 0,
                                       outA.numElements() * outA.elementType().bytes()));
      return;
    }
    logging::poplin::trace("convolution " + name);
    poplar::detail::check(plb_convolution(ctx, &flat, &opt, inA.devicePointer(),
                                          wA.devicePointer(), nullptr, outA.devicePointer(),
                                          transpose));
  });
  if (!outDirect) prog.add(poplar::program::Copy(outA, out));
}

Tensor convolution(Graph &graph, const Tensor &in, const Tensor &weights, const ConvParams &params,
                   bool transposeAndFlipWeights, Sequence &prog, const poplar::DebugContext &dc,
                   const poplar::OptionFlags &options, PlanningCache *cache) {
  Tensor out = createConvOutput(graph, params, {dc, "out"}, options, cache);
  convolutionWithOutput(graph, in, weights, out, params, transposeAndFlipWeights, prog, dc, options,
                        cache);
  return out;
}

void weightsTransposeChansFlipXY(Graph &graph, const Tensor &weightsIn, const Tensor &weightsOut,
                                 Sequence &prog, const poplar::DebugContext &) {
  if (weightsIn.rank() < 3 || weightsOut.rank() != weightsIn.rank())
    throw poplibs_error("weightsTransposeChansFlipXY: tensors must be [G][Co][Ci][k...]");
  auto expect = weightsIn.shape();
  std::swap(expect[1], expect[2]);
  if (weightsOut.shape() != expect)
    throw poplibs_error("weightsTransposeChansFlipXY: output shape " + weightsOut.shapeToString() +
                        " is not the channel-transposed input shape");
  (void)graph;
  // pure view arithmetic: swap the channel axes, reverse every spatial axis
  Tensor view = weightsIn.dimShufflePartial({1, 2}, {2, 1});
  for (unsigned d = 3; d < view.rank(); ++d) view = view.reverse(d);
  prog.add(poplar::program::Copy(view, weightsOut));
}

// ---- weight update ----------------------------------------------------------------------
namespace {

struct WeightDeltas {
  Tensor deltas;     // [G][Co][Ci][k...], params.inputType, device layout
  Tensor deltasF32;  // same in fp32
};

WeightDeltas weightDeltasImpl(Graph &graph, const Tensor &zDeltas, const Tensor &activations,
                              const ConvParams &params, Sequence &prog,
                              const poplar::DebugContext &dc, const poplar::OptionFlags &options,
                              PlanningCache *cache) {
  params.validate();
  validateTypes(params);
  const internal::ConvOptions parsed(options);
  const std::size_t G = params.numConvGroups, ci = params.inputChannelsPerConvGroup,
                    co = params.outputChannelsPerConvGroup;
  checkActsShape(activations, params.batchSize, G * ci, params.inputFieldShape, "activations");
  checkActsShape(zDeltas, params.batchSize, G * co, params.getOutputFieldShape(), "zDeltas");
  (void)cache;
  const Tensor xA = arranged(graph, activations, actsOrder(activations.rank()), prog);
  const Tensor dyA = arranged(graph, zDeltas, actsOrder(zDeltas.rank()), prog);
  WeightDeltas w;
  // the weight deltas have the type of the forward input
  // (lib/poplin/Convolution.cpp:3537, 3584)
  w.deltas = makeWeights(graph, params.inputType, G, co, ci, params.kernelShape,
                         dc.getPathName() + "/weightDeltas");
  w.deltasF32 = makeWeights(graph, poplar::FLOAT, G, co, ci, params.kernelShape,
                            dc.getPathName() + "/weightDeltasF32");
  const plb_conv_params flat = internal::toPlb(params.canonicalize());
  const plb_conv_options opt = parsed.toPlb();
  const Tensor d16 = w.deltas, d32 = w.deltasF32;
  prog.add([=](plb_context *ctx) {
    // the tensors' storage is [G][k...][Co][Ci]: element (0,0,0,0...) is its start
    poplar::detail::check(plb_conv_wu(ctx, &flat, &opt, xA.devicePointer(), dyA.devicePointer(),
                                      d16.devicePointer(),
                                      static_cast<float *>(d32.devicePointer())));
  });
  return w;
}

}  // namespace

Tensor calculateWeightDeltas(Graph &graph, const Tensor &zDeltas, const Tensor &activations,
                             const ConvParams &params, Sequence &prog,
                             const poplar::DebugContext &dc, const poplar::OptionFlags &options,
                             PlanningCache *cache) {
  return weightDeltasImpl(graph, zDeltas, activations, params, prog, dc, options, cache).deltas;
}

// Reads a scalar float / half tensor from the device (synchronises the stream).
static float fetchScalar(plb_context *ctx, const Tensor &t) {
  float value = 0.f;
  if (t.elementType() == poplar::FLOAT) {
    poplar::detail::check(plb_memcpy_d2h(ctx, &value, t.devicePointer(), sizeof(float)));
    return value;
  }
  uint16_t bits = 0;
  poplar::detail::check(plb_memcpy_d2h(ctx, &bits, t.devicePointer(), sizeof bits));
  // half -> float
  const int sign = bits >> 15, e = (bits >> 10) & 31, m = bits & 1023;
  const float mag = e == 0 ? std::ldexp(float(m), -24)
                           : (e == 31 ? INFINITY : std::ldexp(float(m + 1024), e - 25));
  return sign ? -mag : mag;
}

static void weightUpdateImpl(Graph &graph, const Tensor &zDeltas, const Tensor &weights_,
                             const Tensor &activations, const ConvParams &params,
                             const Tensor *scaleTensor, float scaleValue, Sequence &prog,
                             const poplar::DebugContext &dc, const poplar::OptionFlags &options,
                             PlanningCache *cache) {
  const Tensor weights = withGroupDim(weights_, params);
  const WeightDeltas w =
      weightDeltasImpl(graph, zDeltas, activations, params, prog, dc, options, cache);
  if (weights.shape() != w.deltas.shape())
    throw poplibs_error("weights tensor has shape " + weights.shapeToString() +
                        ", which does not match the convolution parameters");
  const bool direct = isDenseInOrder(weights, weightsOrder(weights.rank()));
  const Tensor wA = direct ? weights : arranged(graph, weights, weightsOrder(weights.rank()), prog);
  const Tensor d32 = w.deltasF32;
  const int dtype = poplar::detail::dtypeOf(weights.elementType());
  Tensor scaleT;
  if (scaleTensor) scaleT = *scaleTensor;
  prog.add([=](plb_context *ctx) {
    const float scale = scaleT.valid() ? fetchScalar(ctx, scaleT) : scaleValue;
    poplar::detail::check(plb_scaled_add_to(ctx, dtype, wA.devicePointer(),
                                            static_cast<const float *>(d32.devicePointer()), scale,
                                            wA.numElements()));
  });
  if (!direct) prog.add(poplar::program::Copy(wA, weights));
}

void convolutionWeightUpdate(Graph &graph, const Tensor &zDeltas, const Tensor &weights,
                             const Tensor &activations, ConvParams params, const Tensor &scale,
                             Sequence &prog, const poplar::DebugContext &dc,
                             const poplar::OptionFlags &options, PlanningCache *cache) {
  if (scale.numElements() != 1) throw poplibs_error("convolutionWeightUpdate: scale must be a scalar");
  weightUpdateImpl(graph, zDeltas, weights, activations, params, &scale, 0.f, prog, dc, options,
                   cache);
}

void convolutionWeightUpdate(Graph &graph, const Tensor &zDeltas, const Tensor &weights,
                             const Tensor &activations, ConvParams params, float scale,
                             Sequence &prog, const poplar::DebugContext &dc,
                             const poplar::OptionFlags &options, PlanningCache *cache) {
  weightUpdateImpl(graph, zDeltas, weights, activations, params, nullptr, scale, prog, dc, options,
                   cache);
}

static void biasUpdateImpl(Graph &graph, const Tensor &zDeltas, const Tensor &biases,
                           const Tensor *scaleTensor, float scaleValue,
                           const poplar::OptionFlags &options, Sequence &prog) {
  const internal::ConvOptions parsed(options);  // validates the keys; sums are always kept in fp32
  (void)parsed;
  if (zDeltas.rank() < 2)
    throw poplibs_error("convolutionBiasUpdate with rank " + std::to_string(zDeltas.rank()) +
                        "; must have at least channel and batch dimensions");
  if (biases.rank() != 1 || biases.dim(0) != zDeltas.dim(1))
    throw poplibs_error("convolutionBiasUpdate: biases must have one element per channel of zDeltas");
  if (scaleTensor && scaleTensor->numElements() != 1)
    throw poplibs_error("convolutionBiasUpdate: scale must be a scalar");
  const Tensor z = arranged(graph, zDeltas, actsOrder(zDeltas.rank()), prog);
  const bool direct = isDenseInOrder(biases, {0});
  const Tensor b = direct ? biases : arranged(graph, biases, {0}, prog);
  const int zType = poplar::detail::dtypeOf(zDeltas.elementType());
  const int bType = poplar::detail::dtypeOf(biases.elementType());
  const std::size_t chans = zDeltas.dim(1);
  const std::size_t pixels = chans ? zDeltas.numElements() / chans : 0;
  Tensor scaleT;
  if (scaleTensor) scaleT = *scaleTensor;
  prog.add([=](plb_context *ctx) {
    const float scale = scaleT.valid() ? fetchScalar(ctx, scaleT) : scaleValue;
    poplar::detail::check(plb_conv_bias_update(ctx, zType, z.devicePointer(), pixels,
                                               uint32_t(chans), bType, b.devicePointer(), scale));
  });
  if (!direct) prog.add(poplar::program::Copy(b, biases));
}

void convolutionBiasUpdate(Graph &graph, const Tensor &zDeltas, const Tensor &biases,
                           const Tensor &scale, const poplar::OptionFlags &options, Sequence &prog,
                           const poplar::DebugContext &) {
  biasUpdateImpl(graph, zDeltas, biases, &scale, 0.f, options, prog);
}

void convolutionBiasUpdate(Graph &graph, const Tensor &zDeltas, const Tensor &biases, float scale,
                           const poplar::OptionFlags &options, Sequence &prog,
                           const poplar::DebugContext &) {
  biasUpdateImpl(graph, zDeltas, biases, nullptr, scale, options, prog);
}

void addBias(Graph &graph, const Tensor &acts, const Tensor &biases, Sequence &prog,
             const poplar::DebugContext &) {
  if (acts.rank() < 2 || biases.rank() != 1 || biases.dim(0) != acts.dim(1))
    throw poplibs_error("addBias: biases must have one element per channel of the activations");
  if (biases.elementType() != acts.elementType())
    throw poplibs_error("addBias: biases and activations must have the same type");
  const bool direct = isDenseInOrder(acts, actsOrder(acts.rank()));
  const Tensor a = direct ? acts : arranged(graph, acts, actsOrder(acts.rank()), prog);
  const Tensor b = arranged(graph, biases, {0}, prog);
  const int dtype = poplar::detail::dtypeOf(acts.elementType());
  const std::size_t chans = acts.dim(1);
  const std::size_t pixels = chans ? acts.numElements() / chans : 0;
  prog.add([=](plb_context *ctx) {
    poplar::detail::check(
        plb_add_bias(ctx, dtype, a.devicePointer(), b.devicePointer(), pixels, uint32_t(chans)));
  });
  if (!direct) prog.add(poplar::program::Copy(a, acts));
}

// ---- plan reporting ------------------------------------------------------------------------
static void printPlan(std::ostream &out, const plb_plan &plan, const char *pass) {
  static const char *kernels[] = {"implicit GEMM (TMA + tcgen05)", "weight update (split-K)",
                                  "small-channel (space-to-depth + implicit GEMM)"};
  out << "  Plan (" << pass << "):\n"
      << "        kernel                     " << kernels[std::min(std::max(plan.kernel, 0), 2)] << "\n"
      << "        CTA tile (pixels x chans)  " << plan.tile_m << " x " << plan.tile_n << "\n"
      << "        pixel box (w, h, n)        {" << plan.box_w << "," << plan.box_h << ","
      << plan.box_n << "}\n"
      << "        K bytes per stage          " << plan.tile_k_bytes << "\n"
      << "        pipeline stages            " << plan.stages << "\n"
      << "        split K                    " << plan.split_k << "\n"
      << "        output tiles               " << plan.tiles << "\n"
      << "        CTAs launched              " << plan.grid << "\n"
      << "        weights resident in SMEM   " << (plan.resident_weights ? "yes" : "no") << "\n"
      << "        halo rows per load         " << plan.halo_rows << "\n"
      << "        CTA pair (256-row MMA)     " << plan.cta_pair << "\n"
      << "        right operand MN-major     " << (plan.b_mn_major ? "yes" : "no") << "\n"
      << "        workspace bytes            " << plan.workspace_bytes << "\n"
      << "        FLOPs (padding excluded)   " << plan.flops << "\n"
      << "        bytes (operands + output)  " << plan.bytes << "\n";
}

void reportPlanInfo(std::ostream &out, const Graph &, const ConvParams &params,
                    const poplar::OptionFlags &options, PlanningCache *cache) {
  const internal::ConvOptions parsed(options);
  const int pass = parsed.pass == internal::Pass::TRAINING_BWD ? PLB_PASS_TRAINING_BWD
                                                               : PLB_PASS_TRAINING_FWD;
  out << params;
  printPlan(out, planFor(params, options, pass, cache),
            pass == PLB_PASS_TRAINING_BWD ? "backward" : "forward");
}

void reportWeightUpdatePlanInfo(std::ostream &out, const Graph &, const ConvParams &fwdParams,
                                const poplar::OptionFlags &fwdOptions, PlanningCache *) {
  const internal::ConvOptions parsed(fwdOptions);
  const plb_conv_params flat = internal::toPlb(fwdParams.canonicalize());
  const plb_conv_options opt = parsed.toPlb();
  plb_plan plan{};
  poplar::detail::check(plb_conv_wu_plan(&flat, &opt, &plan));
  if (!parsed.planConstraintsOutputFilename.empty()) {
    internal::ConvOptions wu = parsed;
    wu.pass = internal::Pass::TRAINING_WU;
    writePlanConstraintsFile(plan, wu);
  }
  out << fwdParams;
  printPlan(out, plan, "weight update");
}

PlanCosts reportPlanEstimatedCosts(const Graph &, const ConvParams &params,
                                   const poplar::OptionFlags &options, PlanningCache *cache) {
  const plb_plan plan = planFor(params, options, PLB_PASS_TRAINING_FWD, cache);
  PlanCosts c;
  // roofline estimate per SM: 8192 dense fp16 FLOPs per cycle per SM, 148 SMs;
  // HBM at roughly 3.5 bytes per SM-cycle
  const double computeCycles = double(plan.flops) / (8192.0 * 148.0);
  const double memoryCycles = double(plan.bytes) / (3.5 * 148.0);
  c.cycles = std::size_t(std::max(computeCycles, memoryCycles));
  c.memory = std::size_t(plan.workspace_bytes);
  return c;
}

namespace internal {

std::ostream &operator<<(std::ostream &os, DetailedPlanCosts const &c) {
  os << c.parallelSplit << " " << c.serialSplit << "\n";
  c.apply([&os](const PlanCosts &x) { os << x.cycles << " " << x.memory << "\n"; });
  return os;
}

std::istream &operator>>(std::istream &is, DetailedPlanCosts &c) {
  is >> c.parallelSplit >> c.serialSplit;
  c.apply([&is](PlanCosts &x) { is >> x.cycles >> x.memory; });
  return is;
}

DetailedPlanCosts reportDetailedPlanEstimatedCosts(const Graph &graph, const ConvParams &params,
                                                   const poplar::OptionFlags &options,
                                                   PlanningCache *cache) {
  const ConvOptions parsed(options);
  const int pass = parsed.pass == Pass::TRAINING_BWD ? PLB_PASS_TRAINING_BWD : PLB_PASS_TRAINING_FWD;
  const plb_plan plan = planFor(params, options, pass, cache);
  // bytes per SM cycle the HBM sustains (about 6.5 TB/s at the 1.965 GHz the cycle counts refer to)
  const double hbmBytesPerCycle = 6.5e12 / graph.getTarget().getTileClockFrequency();
  auto memoryCycles = [&](double bytes) { return bytes / hbmBytesPerCycle; };
  DetailedPlanCosts c;
  c.parallelSplit = std::size_t(std::max(1, plan.grid));
  c.serialSplit = 1;
  auto zero = [](PlanCosts &x) { x.cycles = 0; x.memory = 0; };
  c.apply(zero);
  // compute: the contraction kernel at the slower of its two rooflines
  const double macCycles = getFwdPerfectCycleCount(graph, params);
  c.compute.cycles = std::size_t(std::max(macCycles, memoryCycles(double(plan.bytes))));
  // reduction: split-K partial sums written once and read once by the second kernel
  if (plan.split_k > 1) {
    c.reduction.cycles = std::size_t(memoryCycles(2.0 * double(plan.workspace_bytes)));
    c.reduction.memory = std::size_t(plan.workspace_bytes);
  }
  // rearrangement: the small-channel path rewrites the activations once (space to depth)
  if (plan.kernel == 2) {
    double in_bytes = double(params.getBatchSize()) * double(params.getNumInputChans()) *
                      double(graph.getTarget().getTypeSize(params.inputType));
    for (std::size_t extent : params.inputFieldShape) in_bytes *= double(extent);
    c.rearrangement.cycles = std::size_t(memoryCycles(2.0 * in_bytes));
    c.rearrangement.memory = plan.split_k > 1 ? 0 : std::size_t(plan.workspace_bytes);
  }
  c.total.cycles = c.compute.cycles + c.reduction.cycles + c.rearrangement.cycles;
  c.total.memory = std::size_t(plan.workspace_bytes);
  return c;
}

}  // namespace internal

Tensor fullyConnectedWeightTranspose(Graph &graph, Tensor weights, const ConvParams &params,
                                     Sequence &prog, const poplar::DebugContext &dc,
                                     const poplar::OptionFlags &options, PlanningCache *) {
  // (lib/poplin/Convolution.cpp:3846-3921: the weights' channel axes swapped,
  // in a tensor laid out for the backward-pass convolution `params`)
  convolutionValidateOptions(options);
  if (params.getNumFieldDims() != 1)
    throw poplibs_error("fullyConnectedWeightTranspose() expects a 1-d convolution");
  const Tensor w = withGroupDim(weights, params);
  if (w.rank() != 4 || w.dim(0) != params.numConvGroups ||
      w.dim(1) != params.inputChannelsPerConvGroup || w.dim(2) != params.outputChannelsPerConvGroup)
    throw poplibs_error("fullyConnectedWeightTranspose: weights must be [G][Co][Ci][k] of the forward "
                        "pass, i.e. [G][params.Ci][params.Co][k]");
  Tensor transposed = makeWeights(graph, weights.elementType(), params.numConvGroups,
                                  params.outputChannelsPerConvGroup, params.inputChannelsPerConvGroup,
                                  params.kernelShape, dc.getPathName() + "/transposed");
  if (weights.elementType() == poplar::QUARTER && weights.hasMetadata())
    graph.setQuarterMetadata(transposed, weights.getMetadata());
  prog.add(poplar::program::Copy(w.dimShuffle({0, 2, 1, 3}), transposed));
  return transposed;
}

// ---- pre-planning -------------------------------------------------------------------------
void preplanConvolutions(const std::set<ConvPlanParams> &convs, PlanningCache &cache) {
  preplan(convs, {}, cache);
}

void preplanConvolutions(Graph &, const std::set<ConvPlanParams> &convs, PlanningCache &cache) {
  preplan(convs, {}, cache);
}

void preplan(const std::set<ConvPlanParams> &convs, const std::set<MatMulPlanParams> &matmuls,
             PlanningCache &cache) {
  static const poplar::OptionFlags none;
  for (const auto &c : convs) {
    const poplar::OptionFlags *opts = std::get<2>(c) ? std::get<2>(c) : &none;
    const internal::ConvOptions parsed(*opts);
    int pass = PLB_PASS_TRAINING_FWD;
    if (parsed.pass == internal::Pass::TRAINING_BWD) pass = PLB_PASS_TRAINING_BWD;
    if (parsed.pass == internal::Pass::TRAINING_WU) continue;  // planned when the pass is built
    planFor(std::get<1>(c), *opts, pass, &cache);
  }
  MatMulToConvOptions convOpts;
  for (const auto &c : matMulGetConvPlanParams(matmuls, convOpts))
    planFor(std::get<1>(c), *std::get<2>(c), PLB_PASS_TRAINING_FWD, &cache);
}

}  // namespace poplin
