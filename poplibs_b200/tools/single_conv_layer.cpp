// single_conv_layer: builds one convolution layer (forward, backward and
// weight-update passes) through the poplin surface, runs it on the GPU and
// reports time and throughput per pass.  A port of the reference driver
// tools/single_conv_layer.cpp with the same option names for the subset that
// has meaning here; instead of linking a CPU model it writes its seeded inputs
// and the device results to --dump-dir for external checking.
#include <fstream>
#include <iostream>
#include <numeric>

#include "poplar/Engine.hpp"
#include "poplar/Graph.hpp"
#include "poplar/exceptions.hpp"
#include "poplin/ConvUtil.hpp"
#include "poplin/Convolution.hpp"
#include "poplin/codelets.hpp"
#include "popops/codelets.hpp"
#include "poputil/exceptions.hpp"
#include "tool_util.hpp"

using namespace poplar;
using namespace poplar::program;

static std::size_t product(const std::vector<std::size_t> &v) {
  return std::accumulate(v.begin(), v.end(), std::size_t(1), std::multiplies<std::size_t>());
}

int main(int argc, char **argv) try {
  const tool::Args args(argc, argv);
  if (args.has("help")) {
    std::cout
        << "Options: --input-channels C --output-channels C --field {h,w} [--kernel-size k]\n"
           "  [--padding p] [--padding-lower p] [--padding-upper p] [--stride s]\n"
           "  [--kernel-dilation d] [--in-dilation d] [--truncation t] [--flip-input b]\n"
           "  [--flip-kernel b] [--batch-size 1] [--conv-groups 1] [--bias 1]\n"
           "  [--data-type half] [--input-type T] [--output-type T]\n"
           "  [--fp8-scale-fwd 1] [--fp8-scale-weights 2] [--fp8-scale-bwd 1]\n"
           "  [--single-phase fwd|bwd|wu|all] [--convolution-options JSON]\n"
           "  [--fwd-plan-constraints JSON] [--report-plan] [--seed 42] [--integer-data]\n"
           "  [--learning-rate 0.05] [--dump-dir DIR] [--compile-only] [--ignore-data]\n"
           "  [--num-executions 1] [--warmup 0] [--device 0] [--profile]\n";
    return 0;
  }
  const unsigned ci = args.required<unsigned>("input-channels");
  const unsigned co = args.required<unsigned>("output-channels");
  if (!args.has("field")) throw std::runtime_error("the option '--field' is required but missing");
  const std::size_t nd = args.shapeRank("field");
  const auto field = args.shape<std::size_t>("field", nd, 1);
  const auto kernel = args.shape<std::size_t>("kernel-size", nd, 1);
  auto padLo = args.shape<unsigned>("padding", nd, 0), padHi = padLo;
  if (args.has("padding-lower")) padLo = args.shape<unsigned>("padding-lower", nd, 0);
  if (args.has("padding-upper")) padHi = args.shape<unsigned>("padding-upper", nd, 0);
  const auto stride = args.shape<unsigned>("stride", nd, 1);
  const auto kernelDilation = args.shape<unsigned>("kernel-dilation", nd, 1);
  const auto inDilation = args.shape<unsigned>("in-dilation", nd, 1);
  auto truncLo = args.shape<unsigned>("truncation", nd, 0), truncHi = truncLo;
  if (args.has("truncation-lower")) truncLo = args.shape<unsigned>("truncation-lower", nd, 0);
  if (args.has("truncation-upper")) truncHi = args.shape<unsigned>("truncation-upper", nd, 0);
  const auto flipInput = args.shape<unsigned>("flip-input", nd, 0);
  const auto flipKernel = args.shape<unsigned>("flip-kernel", nd, 0);
  const unsigned batch = args.get<unsigned>("batch-size", 1);
  const unsigned groups = args.get<unsigned>("conv-groups", 1);
  const bool bias = args.get<unsigned>("bias", 1) != 0;
  Type inputType = tool::parseType(args.str("data-type", "half"));
  Type outputType = inputType;
  if (args.has("input-type")) inputType = tool::parseType(args.str("input-type"));
  if (args.has("output-type")) outputType = tool::parseType(args.str("output-type"));
  else if (inputType == QUARTER) outputType = HALF;
  const int scaleFwd = args.get<int>("fp8-scale-fwd", 1), scaleW = args.get<int>("fp8-scale-weights", 2),
            scaleBwd = args.get<int>("fp8-scale-bwd", 1);
  const auto formatFwd = tool::quarterFormat(args.str("fp8-format-fwd", "F143"));
  const auto formatW = tool::quarterFormat(args.str("fp8-format-weights", "F143"));
  const auto formatBwd = tool::quarterFormat(args.str("fp8-format-bwd", "F143"));
  const std::string phase = args.str("single-phase", "all");
  if (phase != "fwd" && phase != "bwd" && phase != "wu" && phase != "all")
    throw std::runtime_error("--single-phase must be fwd, bwd, wu or all");
  const bool doFwd = phase == "fwd" || phase == "all";
  const bool doBwd = phase == "bwd" || phase == "all";
  // the weight update is never run in quarter (tools/single_conv_layer.cpp:725-733)
  const bool doWu = (phase == "wu" || phase == "all") && inputType != QUARTER;
  const std::string convOptions = args.str("convolution-options");
  const std::string fwdPlanConstraints = args.str("fwd-plan-constraints");
  const unsigned seed = args.get<unsigned>("seed", 42);
  const bool integerData = args.has("integer-data") || inputType == QUARTER;
  const double learningRate = args.get<double>("learning-rate", 0.05);
  const std::string dumpDir = args.str("dump-dir");
  const bool compileOnly = args.has("compile-only"), ignoreData = args.has("ignore-data");
  const bool reportPlan = args.has("report-plan"), profile = args.has("profile");
  const unsigned numExecutions = args.get<unsigned>("num-executions", 1);
  const unsigned warmup = args.get<unsigned>("warmup", 0);  // untimed runs of each pass first
  const int device = args.get<int>("device", 0);
  args.rejectUnknown();

  Graph graph(Target::createGPUTarget(device));
  poplin::addCodelets(graph);
  popops::addCodelets(graph);

  const poplin::ConvParams params(
      inputType, outputType, batch, field, kernel, ci, co, groups,
      poplin::ConvParams::InputTransform(truncLo, truncHi, inDilation, padLo, padHi,
                                         std::vector<bool>(flipInput.begin(), flipInput.end())),
      poplin::ConvParams::InputTransform(std::vector<unsigned>(nd, 0), std::vector<unsigned>(nd, 0),
                                         kernelDilation, std::vector<unsigned>(nd, 0),
                                         std::vector<unsigned>(nd, 0),
                                         std::vector<bool>(flipKernel.begin(), flipKernel.end())),
      poplin::ConvParams::OutputTransform(std::vector<unsigned>(nd, 0), std::vector<unsigned>(nd, 0),
                                          stride, std::vector<unsigned>(nd, 0),
                                          std::vector<unsigned>(nd, 0)));
  params.validate();  // (the constructor does not; sizes below divide by the stride)
  const auto outField = params.getOutputFieldShape();
  const poplin::ConvParams bwdParams = poplin::getGradientParams(params);

  OptionFlags base;
  if (!convOptions.empty()) readJSON(convOptions, base);
  OptionFlags fwdOptions = base, bwdOptions = base, wuOptions = base;
  fwdOptions.set("pass", doBwd || doWu ? "TRAINING_FWD" : "INFERENCE_FWD");
  bwdOptions.set("pass", "TRAINING_BWD");
  wuOptions.set("pass", "TRAINING_WU");
  if (!fwdPlanConstraints.empty()) fwdOptions.set("planConstraints", fwdPlanConstraints);

  poplin::PlanningCache cache;
  if (reportPlan) {
    if (doFwd) poplin::reportPlanInfo(std::cout, graph, params, fwdOptions, &cache);
    if (doBwd) poplin::reportPlanInfo(std::cout, graph, bwdParams, bwdOptions, &cache);
    if (doWu) poplin::reportWeightUpdatePlanInfo(std::cout, graph, params, wuOptions, &cache);
  }

  Tensor prevAct = poplin::createInput(graph, params, "prevAct", fwdOptions, &cache);
  Tensor weights = poplin::createWeights(graph, params, "weights", fwdOptions, &cache);
  if (inputType == QUARTER) {
    graph.setQuarterMetadata(prevAct, QuarterMetadata(formatFwd, (signed char)scaleFwd));
    graph.setQuarterMetadata(weights, QuarterMetadata(formatW, (signed char)scaleW));
  }
  Sequence fwdProg, bwdProg, wuProg;
  Tensor nextAct, biases;
  if (doFwd) {
    Sequence once;
    nextAct = poplin::convolution(graph, prevAct, weights, params, false, once, "fwd", fwdOptions, &cache);
    if (bias) {
      biases = poplin::createBiases(graph, nextAct, "biases");
      poplin::addBias(graph, nextAct, biases, once, "bias");
    }
    fwdProg.add(Repeat(numExecutions, once));
  } else if (bias && doWu) {
    // the weight-update pass also updates the biases (the reference tool
    // always builds the forward pass and takes the biases' layout from it)
    biases = poplin::createBiases(
        graph, poplin::createConvOutput(graph, params, "nextAct", fwdOptions, &cache), "biases");
  }
  Tensor zDeltas, prevDeltas;
  if (doBwd || doWu) {
    // the output gradients are the backward convolution's input
    zDeltas = poplin::createInput(graph, bwdParams, "zDeltas", bwdOptions, &cache);
    if (inputType == QUARTER)
      graph.setQuarterMetadata(zDeltas, QuarterMetadata(formatBwd, (signed char)scaleBwd));
  }
  if (doBwd) {
    Sequence once;
    prevDeltas = poplin::convolution(graph, zDeltas, weights, bwdParams, true, once, "bwd",
                                     bwdOptions, &cache);
    bwdProg.add(Repeat(numExecutions, once));
  }
  Tensor weightDeltas;
  if (doWu) {
    // the gradient first (reported on its own), then weights += -lr * gradient
    weightDeltas = poplin::calculateWeightDeltas(graph, zDeltas, prevAct, params, wuProg, "wu",
                                                 wuOptions, &cache);
    poplin::convolutionWeightUpdate(graph, zDeltas, weights, prevAct, params, float(-learningRate),
                                    wuProg, "wuApply", wuOptions, &cache);
    if (bias)
      poplin::convolutionBiasUpdate(graph, zDeltas, biases, float(-learningRate), wuOptions, wuProg,
                                    "biasUpdate");
  }

  graph.createHostWrite("prevAct", prevAct);
  graph.createHostWrite("weights", weights);
  graph.createHostRead("weights", weights);
  if (biases.valid()) {
    graph.createHostWrite("biases", biases);
    graph.createHostRead("biases", biases);
  }
  if (nextAct.valid()) graph.createHostRead("nextAct", nextAct);
  if (zDeltas.valid()) graph.createHostWrite("zDeltas", zDeltas);
  if (prevDeltas.valid()) graph.createHostRead("prevDeltas", prevDeltas);
  if (weightDeltas.valid()) graph.createHostRead("weightDeltas", weightDeltas);

  if (compileOnly) return 0;  // graph and plans built; no device is touched
  Engine engine(graph, std::vector<Sequence>{fwdProg, bwdProg, wuProg});

  const std::vector<std::size_t> inShape = [&] {
    std::vector<std::size_t> s{batch, std::size_t(groups) * ci};
    s.insert(s.end(), field.begin(), field.end());
    return s;
  }();
  const std::vector<std::size_t> outShape = [&] {
    std::vector<std::size_t> s{batch, std::size_t(groups) * co};
    s.insert(s.end(), outField.begin(), outField.end());
    return s;
  }();
  const std::vector<std::size_t> wShape = [&] {
    std::vector<std::size_t> s{groups, co, ci};
    s.insert(s.end(), kernel.begin(), kernel.end());
    return s;
  }();
  if (!ignoreData) {
    std::mt19937 rng(seed);
    auto hAct = tool::randomValues(product(inShape), -2.0, 2.0, rng, integerData);
    auto hW = tool::randomValues(product(wShape), -1.0, 1.0, rng, integerData);
    auto hBias = tool::randomValues(std::size_t(groups) * co, -2.0, 6.0, rng, integerData);
    auto hDeltas = tool::randomValues(product(outShape), -3.0, 3.0, rng, integerData);
    const auto rAct = tool::toDevice(hAct, inputType, scaleFwd, formatFwd == QuarterMetadata::Format::F152);
    const auto rW = tool::toDevice(hW, inputType, scaleW, formatW == QuarterMetadata::Format::F152);
    engine.writeTensor("prevAct", rAct.data(), rAct.data() + rAct.size());
    engine.writeTensor("weights", rW.data(), rW.data() + rW.size());
    tool::dump(dumpDir, "prevAct", hAct, inShape);
    tool::dump(dumpDir, "weights", hW, wShape);
    if (biases.valid()) {
      const auto rB = tool::toDevice(hBias, outputType);
      engine.writeTensor("biases", rB.data(), rB.data() + rB.size());
      tool::dump(dumpDir, "biases", hBias, {std::size_t(groups) * co});
    }
    if (zDeltas.valid()) {
      const auto rD = tool::toDevice(hDeltas, inputType, scaleBwd, formatBwd == QuarterMetadata::Format::F152);
      engine.writeTensor("zDeltas", rD.data(), rD.data() + rD.size());
      tool::dump(dumpDir, "zDeltas", hDeltas, outShape);
    }
  }
  engine.load(Device());
  const double flops = double(poplin::getFwdFlops(params));
  auto readBack = [&](const char *handle, const Tensor &t, const std::vector<std::size_t> &shape,
                      const char *dumpName = nullptr) {
    if (ignoreData) return;
    std::vector<uint8_t> raw(t.numElements() * t.elementType().bytes());
    engine.readTensor(handle, raw.data(), raw.data() + raw.size());
    tool::dump(dumpDir, dumpName ? dumpName : handle, tool::fromDevice(raw, t.elementType()), shape);
  };
  auto report = [&](const char *pass, unsigned runs) {
    const double ms = engine.lastRunMilliseconds() / runs;
    std::cout << pass << ": " << ms * 1e3 << " us per execution, " << flops / ms / 1e9 << " TFLOP/s\n";
  };
  if (warmup && !ignoreData)
    throw std::runtime_error("--warmup re-runs the passes (the weight update would be applied "
                             "more than once): use it with --ignore-data");
  if (doFwd) {
    for (unsigned i = 0; i < warmup; ++i) engine.run(0);
    engine.run(0);
    report("fwd", numExecutions);
    readBack("nextAct", nextAct, outShape);
  }
  if (doBwd) {
    for (unsigned i = 0; i < warmup; ++i) engine.run(1);
    engine.run(1);
    report("bwd", numExecutions);
    readBack("prevDeltas", prevDeltas, inShape);
  }
  if (doWu) {
    for (unsigned i = 0; i < warmup; ++i) engine.run(2);
    engine.run(2);
    report("wu (gradient + update)", 1);
    readBack("weightDeltas", weightDeltas, wShape);
    readBack("weights", weights, wShape, "weightsUpdated");
    if (biases.valid())
      readBack("biases", biases, {std::size_t(groups) * co}, "biasesUpdated");
  }
  if (profile) engine.printProfileSummary(std::cout);
  return 0;
} catch (const poplar::graph_memory_allocation_error &e) {
  std::cerr << e.what() << "\n";
  return 77;  // out of memory: reported as "skipped", as the reference tools do
} catch (const std::exception &e) {
  std::cerr << "error: " << e.what() << "\n";
  return 1;
}
