// Option handling of the poplin surface: the convolution option set
// (lib/poplin/ConvOptions.cpp:105-152), the grammar check of planConstraints
// (lib/poplin/ConvOptions.cpp:156-329), the matMul option set and its
// translation to convolution options (lib/poplin/MatMul.cpp:113-195), and the
// mapping of all of it onto the CUDA planner's few knobs.
#include <cstdint>
#include <map>
#include <set>
#include <sstream>

#include "internal.hpp"
#include "json.hpp"
#include "poplin/Convolution.hpp"
#include "poplin/MatMul.hpp"
#include "poputil/OptionParsing.hpp"

namespace poplin {
namespace internal {

using poplar::invalid_option;

namespace {

const std::map<std::string, Pass> passMap{
    {"NONE", Pass::NONE},
    {"NONE_MATMUL", Pass::NONE_MATMUL},
    {"INFERENCE_FWD", Pass::INFERENCE_FWD},
    {"TRAINING_FWD", Pass::TRAINING_FWD},
    {"TRAINING_BWD", Pass::TRAINING_BWD},
    {"TRAINING_WU", Pass::TRAINING_WU},
    {"FC_INFERENCE_FWD", Pass::FC_INFERENCE_FWD},
    {"FC_TRAINING_FWD", Pass::FC_TRAINING_FWD},
    {"FC_TRAINING_BWD", Pass::FC_TRAINING_BWD},
    {"FC_TRAINING_WU", Pass::FC_TRAINING_WU}};

const std::map<std::string, poplar::Type> partialsTypeMap{{"half", poplar::HALF},
                                                          {"float", poplar::FLOAT}};

// ---- planConstraints grammar ---------------------------------------------------
bool isScalarLeaf(const json::Value &v) { return !v.isContainer(); }

void requireObject(const std::string &path, const json::Value &v) {
  // a bare scalar where an object is expected
  if (isScalarLeaf(v) && !v.text.empty())
    throw invalid_option("'" + path + "': Must be an object");
}

void requireUnsigned(const std::string &path, const json::Value &v) {
  std::istringstream s(v.text);
  long long value;
  s >> value;
  if (v.isContainer() || s.fail() || !s.eof() || value < 0)
    throw invalid_option("'" + path + "': Not a valid unsigned integer");
}

void requireBoolean(const std::string &path, const json::Value &v) {
  if (v.isContainer() || (v.text != "true" && v.text != "false"))
    throw invalid_option("'" + path + "': Not a valid boolean");
}

void requireUnsignedArray(const std::string &path, const json::Value &v) {
  if (!v.isContainer() && !v.text.empty())
    throw invalid_option("'" + path + "': Not a valid array of unsigned integers");
  for (const auto &item : v.items) requireUnsigned(path, item.second);
}

void requireIndex(const std::string &path, const std::string &text) {
  std::stringstream s(text);
  std::int64_t level;
  s >> level;
  if (s.fail()) throw invalid_option("'" + path + "': Index not an integer");
  if (level < 0) throw invalid_option("'" + path + "': Index is negative");
}

void checkTransform(const std::string &path, const json::Value &t) {
  requireObject(path, t);
  for (const auto &child : t.items) {
    const std::string sub = path + "." + child.first;
    if (child.first == "swapOperands")
      requireBoolean(sub, child.second);
    else if (child.first == "expandDims" || child.first == "outChanFlattenDims" ||
             child.first == "combineConvGroupsFactor")
      requireUnsignedArray(sub, child.second);
    else
      throw invalid_option("'" + sub + "': " + child.first +
                           " is not currently handled or does not exist");
  }
}

void checkPartitionVars(const std::string &path, const json::Value &t) {
  requireObject(path, t);
  for (const auto &child : t.items) {
    const std::string sub = path + "." + child.first;
    requireIndex(sub, child.first);
    requireUnsigned(sub, child.second);
  }
}

void checkPartitionSplitVar(const std::string &path, const json::Value &t) {
  requireObject(path, t);
  for (const auto &child : t.items) {
    const std::string sub = path + "." + child.first;
    if (child.first == "parallel" || child.first == "serial")
      requireUnsigned(sub, child.second);
    else
      throw invalid_option("'" + sub + "': " + child.first +
                           " is not either 'parallel' or 'serial'");
  }
}

void checkPartition(const std::string &path, const json::Value &t) {
  requireObject(path, t);
  for (const auto &child : t.items) {
    const std::string sub = path + "." + child.first;
    if (child.first == "convGroupSplit" || child.first == "batchSplit")
      requireUnsigned(sub, child.second);
    else if (child.first == "fieldSplit" || child.first == "kernelSplit")
      checkPartitionVars(sub, child.second);
    else if (child.first == "inChanSplit" || child.first == "outChanSplit")
      checkPartitionSplitVar(sub, child.second);
    else
      throw invalid_option("'" + sub + "': " + child.first +
                           " is not currently handled or does not exist");
  }
}

void checkLevel(const std::string &path, const json::Value &t) {
  requireObject(path, t);
  for (const auto &child : t.items) {
    const std::string sub = path + "." + child.first;
    if (child.first == "transform")
      checkTransform(sub, child.second);
    else if (child.first == "partition")
      checkPartition(sub, child.second);
    else
      throw invalid_option("'" + sub + "': " + child.first +
                           " is not a valid sub-domain of the plan. Must be either "
                           "'transform' or 'partition'");
  }
}

void checkMethod(const std::string &path, const json::Value &t) {
  for (const auto &child : t.items) {
    if (child.first == "type") {
      const std::string &type = child.second.text;
      if (child.second.isContainer()) throw invalid_option("'" + path + "': Not a valid string");
      if (type != "AMP" && type != "SLIC" && type != "HMAC" && type != "VMAC" &&
          type != "OUTER_PRODUCT")
        throw invalid_option("'" + path + "': Not a valid method type");
    } else if (child.first == "useLimitedVersion") {
      requireBoolean(child.first, child.second);
    } else if (child.first == "convUnits" || child.first == "convUnitChainsRequired" ||
               child.first == "windowWidth") {
      requireUnsigned(child.first, child.second);
    }
  }
}

// The CUDA planner's own constraints, an extension of the reference grammar:
//   "cuda": {"tileN": 64|128|256, "splitK": n, "residentWeights": bool, "halo": bool, "ctaPair": bool}
void checkCuda(const std::string &path, const json::Value &t) {
  requireObject(path, t);
  for (const auto &child : t.items) {
    const std::string sub = path + "." + child.first;
    if (child.first == "tileN" || child.first == "splitK")
      requireUnsigned(sub, child.second);
    else if (child.first == "residentWeights" || child.first == "halo" || child.first == "ctaPair")
      requireBoolean(sub, child.second);
    else
      throw invalid_option("'" + sub + "': " + child.first + " is not a CUDA plan constraint");
  }
}

void checkTopLevel(const json::Value &t) {
  if (isScalarLeaf(t) && !t.text.empty())
    throw invalid_option("Plan constraints must be an object");
  for (const auto &child : t.items) {
    if (child.first == "method")
      checkMethod(child.first, child.second);
    else if (child.first == "convGroupsPerGroup" || child.first == "inChansPerGroup" ||
             child.first == "partialChansPerGroup")
      requireUnsigned(child.first, child.second);
    else if (child.first == "cuda")
      checkCuda(child.first, child.second);
    else {
      requireIndex(child.first, child.first);
      checkLevel(child.first, child.second);
    }
  }
}

unsigned asUnsigned(const json::Value &v) {
  std::istringstream s(v.text);
  unsigned u = 0;
  s >> u;
  return u;
}

}  // namespace

std::string validatePlanConstraints(const std::string &jsonText) {
  bool blank = true;
  for (char c : jsonText)
    if (!std::isspace(static_cast<unsigned char>(c))) blank = false;
  if (blank) return jsonText;
  json::Value root;
  try {
    root = json::parse(jsonText);
  } catch (const invalid_option &e) {
    throw invalid_option(std::string("Plan constraints are not valid JSON: ") + e.what());
  }
  checkTopLevel(root);
  return jsonText;
}

ConvOptions::ConvOptions(const poplar::OptionFlags &options) {
  using poplibs::OptionHandler;
  using poplibs::OptionSpec;
  const OptionSpec spec{
      {"availableMemoryProportion", OptionHandler::createWithDouble(availableMemoryProportion, 0.)},
      {"pass", OptionHandler::createWithEnum(pass, passMap)},
      {"partialsType", OptionHandler::createWithEnum(partialsType, partialsTypeMap)},
      {"partialsType.interTile",
       OptionHandler::createWithEnum(interTilePartialsType, partialsTypeMap)},
      {"partialsType.interIPU", OptionHandler::createWithEnum(interIpuPartialsType, partialsTypeMap)},
      {"use128BitConvUnitLoad", OptionHandler::createWithBool(use128BitConvUnitLoad)},
      {"planConstraints", OptionHandler{[this](const std::string &v) {
         planConstraints = validatePlanConstraints(v);
       }}},
      {"planConstraintsOutputFilename",
       OptionHandler::createWithString(planConstraintsOutputFilename)},
      {"enableMultiStageReduce", OptionHandler::createWithBool(enableMultiStageReduce)},
      {"enableFastReduce", OptionHandler::createWithBool(enableFastReduce)},
      {"remapOutputTensor", OptionHandler::createWithBool(remapOutputTensor)},
      {"enableConvDithering", OptionHandler::createWithBool(enableConvDithering)},
      {"disableTransformations", OptionHandler::createWithBool(disableTransformations)},
      {"insertTransformsCycleCountProgs",
       OptionHandler::createWithBool(insertTransformsCycleCountProgs)},
      {"experimental.convTransformsEstimates",
       OptionHandler::createWithBool(experimentalConvTransformsEstimates)},
      {"gatherConvOutput", OptionHandler::createWithBool(gatherConvOutput)},
      {"experimental.slicVmac16", OptionHandler::createWithBool(experimentalSlicVmac16)},
      {"disableSRForAMPVertices", OptionHandler::createWithBool(disableSRForAMPVertices)},
      {"enableTileLevelExpandDims", OptionHandler::createWithBool(enableTileLevelExpandDims)},
  };
  for (const auto &entry : options) spec.parse(entry.first, entry.second);
}

plb_conv_options ConvOptions::toPlb() const {
  plb_conv_options o{};
  switch (pass) {
    case Pass::NONE: o.pass = PLB_PASS_NONE; break;
    case Pass::NONE_MATMUL: o.pass = PLB_PASS_NONE_MATMUL; break;
    case Pass::INFERENCE_FWD: o.pass = PLB_PASS_INFERENCE_FWD; break;
    case Pass::TRAINING_FWD: o.pass = PLB_PASS_TRAINING_FWD; break;
    case Pass::TRAINING_BWD: o.pass = PLB_PASS_TRAINING_BWD; break;
    case Pass::TRAINING_WU: o.pass = PLB_PASS_TRAINING_WU; break;
    case Pass::FC_INFERENCE_FWD: o.pass = PLB_PASS_FC_INFERENCE_FWD; break;
    case Pass::FC_TRAINING_FWD: o.pass = PLB_PASS_FC_TRAINING_FWD; break;
    case Pass::FC_TRAINING_BWD: o.pass = PLB_PASS_FC_TRAINING_BWD; break;
    case Pass::FC_TRAINING_WU: o.pass = PLB_PASS_FC_TRAINING_WU; break;
  }
  o.partials_type = partialsType == poplar::HALF ? PLB_HALF : PLB_FLOAT;
  if (planConstraints.empty()) return o;
  bool blank = true;
  for (char c : planConstraints)
    if (!std::isspace(static_cast<unsigned char>(c))) blank = false;
  if (blank) return o;
  const json::Value root = json::parse(planConstraints);
  // Reference grammar -> CUDA planner: the product of the reduction splits
  // (inChanSplit, kernelSplit) at any level asks for that many CTAs per output
  // tile; outChanSplit.parallel asks for output-channel tiles of 1/n the width.
  unsigned reduction_split = 1;
  for (const auto &level : root.items) {
    if (level.first == "cuda") {
      if (const auto *v = level.second.find("tileN")) o.tile_n = int32_t(asUnsigned(*v));
      if (const auto *v = level.second.find("splitK")) o.split_k = int32_t(asUnsigned(*v));
      if (const auto *v = level.second.find("residentWeights"))
        o.plan_flags |= v->text == "true" ? PLB_PLAN_FORCE_RESIDENT_WEIGHTS
                                          : PLB_PLAN_NO_RESIDENT_WEIGHTS;
      if (const auto *v = level.second.find("halo"))
        if (v->text == "false") o.plan_flags |= PLB_PLAN_NO_HALO;
      if (const auto *v = level.second.find("ctaPair"))
        o.plan_flags |= v->text == "false" ? PLB_PLAN_NO_CTA_PAIR : PLB_PLAN_FORCE_CTA_PAIR;
      continue;
    }
    const json::Value *partition = level.second.find("partition");
    if (!partition) continue;
    if (const auto *in = partition->find("inChanSplit"))
      for (const auto &kv : in->items) reduction_split *= std::max(1u, asUnsigned(kv.second));
    if (const auto *ks = partition->find("kernelSplit"))
      for (const auto &kv : ks->items) reduction_split *= std::max(1u, asUnsigned(kv.second));
  }
  if (o.split_k == 0 && reduction_split > 1) o.split_k = int32_t(reduction_split);
  return o;
}

poplar::OptionFlags matMulToConvOptions(const poplar::OptionFlags &matmulOptions) {
  using poplibs::OptionHandler;
  using poplibs::OptionSpec;
  enum class FcPass { NONE, INFERENCE_FWD, TRAINING_FWD, TRAINING_BWD, TRAINING_WU };
  poplar::Type partialsType = poplar::FLOAT;
  FcPass fcPass = FcPass::NONE;
  bool preArranged = false, use128 = false, multiStage = true, fastReduce = false,
       remapOutput = true, gatherOutput = false, disableSR = false;
  double availableMemoryProportion = 0.6;
  std::string planConstraints;
  const OptionSpec spec{
      {"partialsType", OptionHandler::createWithEnum(partialsType, partialsTypeMap)},
      {"fullyConnectedPass",
       OptionHandler::createWithEnum(
           fcPass, std::map<std::string, FcPass>{{"NONE", FcPass::NONE},
                                                 {"INFERENCE_FWD", FcPass::INFERENCE_FWD},
                                                 {"TRAINING_FWD", FcPass::TRAINING_FWD},
                                                 {"TRAINING_BWD", FcPass::TRAINING_BWD},
                                                 {"TRAINING_WU", FcPass::TRAINING_WU}})},
      {"inputRHSIsPreArranged", OptionHandler::createWithBool(preArranged)},
      {"use128BitConvUnitLoad", OptionHandler::createWithBool(use128)},
      {"enableMultiStageReduce", OptionHandler::createWithBool(multiStage)},
      {"enableFastReduce", OptionHandler::createWithBool(fastReduce)},
      {"remapOutputTensor", OptionHandler::createWithBool(remapOutput)},
      {"availableMemoryProportion",
       OptionHandler::createWithDouble(availableMemoryProportion, 0.)},
      {"planConstraints", OptionHandler::createWithString(planConstraints)},
      {"gatherOutput", OptionHandler::createWithBool(gatherOutput)},
      {"disableSRForAMPVertices", OptionHandler::createWithBool(disableSR)},
  };
  for (const auto &entry : matmulOptions) spec.parse(entry.first, entry.second);
  poplar::OptionFlags conv;
  conv.set("partialsType", partialsType.toString());
  conv.set("availableMemoryProportion", std::to_string(availableMemoryProportion));
  conv.set("use128BitConvUnitLoad", use128 ? "true" : "false");
  conv.set("enableMultiStageReduce", multiStage ? "true" : "false");
  conv.set("enableFastReduce", fastReduce ? "true" : "false");
  conv.set("remapOutputTensor", remapOutput ? "true" : "false");
  conv.set("gatherConvOutput", gatherOutput ? "true" : "false");
  conv.set("disableSRForAMPVertices", disableSR ? "true" : "false");
  conv.set("planConstraints", planConstraints);
  static const char *names[] = {"NONE_MATMUL", "FC_INFERENCE_FWD", "FC_TRAINING_FWD",
                                "FC_TRAINING_BWD", "FC_TRAINING_WU"};
  conv.set("pass", names[int(fcPass)]);
  return conv;
}

}  // namespace internal

void convolutionValidateOptions(const poplar::OptionFlags &options) {
  internal::ConvOptions parsed(options);
  (void)parsed;
}

void matmulValidateOptions(const poplar::OptionFlags &options) {
  internal::ConvOptions parsed(internal::matMulToConvOptions(options));
  (void)parsed;
}

}  // namespace poplin
