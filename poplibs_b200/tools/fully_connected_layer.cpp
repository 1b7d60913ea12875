// fully_connected_layer: forward, backward and weight-update passes of a
// (grouped) fully connected layer through poplin::matMulGrouped,
// transposeGroupedMatrix and matMulAcc / matMulGroupedAcc, with the
// fullyConnectedPass options of each pass.  A port of the reference driver
// tools/fully_connected_layer.cpp (graph construction :274-420) with the same
// option names for the subset that has meaning here; instead of linking a CPU
// model it writes its seeded inputs and the device results to --dump-dir.
//
//   nextAct    [G][B][O] = prevAct [G][B][I] x weights [G][I][O] (+ biases [G][O])
//   prevDeltas [G][B][I] = zDeltas [G][B][O] x weights^T
//   weights   += -lr * prevAct^T x zDeltas;  biases += -lr * sum over the batch of zDeltas
#include <iostream>

#include "poplar/Engine.hpp"
#include "poplar/Graph.hpp"
#include "poplar/exceptions.hpp"
#include "poplibs_b200.h"
#include "poplin/MatMul.hpp"
#include "poplin/codelets.hpp"
#include "popops/codelets.hpp"
#include "poputil/exceptions.hpp"
#include "tool_util.hpp"

using namespace poplar;
using namespace poplar::program;

static void check(int rc) {
  if (rc != 0) throw poputil::poplibs_error(plb_last_error());
}
static int plbType(const Type &t) { return t == FLOAT ? PLB_FLOAT : t == HALF ? PLB_HALF : PLB_QUARTER; }

int main(int argc, char **argv) try {
  const tool::Args args(argc, argv);
  if (args.has("help")) {
    std::cout << "Options: --input-size --output-size [--batch-size 1] [--num-groups 1] [--bias 1]\n"
                 "  [--data-type half] [--input-type T] [--output-type T] [--inference-only]\n"
                 "  [--single-phase all|fwd|bwd|wu] [--learning-rate 0.5] [--matmul-options JSON]\n"
                 "  [--plan-constraints JSON] [--report-plan 0] [--fp8-scale-fwd 0] [--fp8-scale-weights 0]\n"
                 "  [--fp8-scale-bwd 0] [--seed 42] [--integer-data] [--dump-dir DIR] [--compile-only]\n"
                 "  [--ignore-data] [--device 0]\n";
    return 0;
  }
  const std::size_t inputSize = args.required<unsigned>("input-size");
  const std::size_t outputSize = args.required<unsigned>("output-size");
  const std::size_t batchSize = args.get<unsigned>("batch-size", 1);
  const std::size_t numGroups = args.get<unsigned>("num-groups", 1);
  const bool bias = args.get<unsigned>("bias", 1) != 0;
  Type inputType = tool::parseType(args.str("data-type", "half"));
  Type outputType = inputType;
  if (args.has("input-type")) inputType = tool::parseType(args.str("input-type"));
  if (args.has("output-type")) outputType = tool::parseType(args.str("output-type"));
  else if (inputType == QUARTER) outputType = HALF;
  const bool inferenceOnly = args.has("inference-only");
  const std::string phase = args.str("single-phase", "all");
  if (phase != "all" && phase != "fwd" && phase != "bwd" && phase != "wu")
    throw poputil::poplibs_error("--single-phase must be one of all, fwd, bwd, wu");
  const bool doFwd = phase == "all" || phase == "fwd";
  const bool doBwd = !inferenceOnly && (phase == "all" || phase == "bwd");
  // the reference never runs the weight update in quarter
  const bool doWu = !inferenceOnly && inputType != QUARTER && (phase == "all" || phase == "wu");
  const double learningRate = args.get<double>("learning-rate", 0.5);
  const std::string matmulOptions = args.str("matmul-options");
  const std::string planConstraints = args.str("plan-constraints");
  const bool reportPlan = args.get<unsigned>("report-plan", 0) != 0;
  const int scaleFwd = args.get<int>("fp8-scale-fwd", 0), scaleW = args.get<int>("fp8-scale-weights", 0),
            scaleBwd = args.get<int>("fp8-scale-bwd", 0);
  const auto formatFwd = tool::quarterFormat(args.str("fp8-format-fwd", "F143"));
  const auto formatW = tool::quarterFormat(args.str("fp8-format-weights", "F143"));
  const auto formatBwd = tool::quarterFormat(args.str("fp8-format-bwd", "F143"));
  const unsigned seed = args.get<unsigned>("seed", 42);
  const bool integerData = args.has("integer-data") || inputType == QUARTER;
  const std::string dumpDir = args.str("dump-dir");
  const bool compileOnly = args.has("compile-only"), ignoreData = args.has("ignore-data");
  const int device = args.get<int>("device", 0);
  args.str("remap-output-tensor");
  args.str("use-create-input");
  args.str("map-biases-by-use");
  args.str("in-place-update");
  args.rejectUnknown();

  Graph graph(Target::createGPUTarget(device));
  poplin::addCodelets(graph);
  popops::addCodelets(graph);

  OptionFlags fwdOptions;
  if (!matmulOptions.empty()) poplar::readJSON(matmulOptions, fwdOptions);
  fwdOptions.set("fullyConnectedPass", inferenceOnly ? "INFERENCE_FWD" : "TRAINING_FWD");
  if (!planConstraints.empty()) fwdOptions.set("planConstraints", planConstraints);
  poplin::matmulValidateOptions(fwdOptions);
  OptionFlags bwdOptions = fwdOptions, wuOptions = fwdOptions;
  bwdOptions.set("fullyConnectedPass", "TRAINING_BWD");
  wuOptions.set("fullyConnectedPass", "TRAINING_WU");

  poplin::PlanningCache cache;
  const std::vector<std::size_t> actShape{numGroups, batchSize, inputSize},
      wShape{numGroups, inputSize, outputSize}, outShape{numGroups, batchSize, outputSize};
  Tensor prevAct = poplin::createMatMulGroupedInputLHS(graph, inputType, outputType, actShape, wShape,
                                                       "prevAct", fwdOptions, &cache);
  Tensor weights = poplin::createMatMulGroupedInputRHS(graph, inputType, outputType, actShape, wShape,
                                                       "weights", fwdOptions, &cache);
  Tensor biases;
  if (bias) biases = graph.addVariable(outputType, {numGroups, outputSize}, "biases");
  if (inputType == QUARTER) {
    graph.setQuarterMetadata(prevAct, QuarterMetadata(formatFwd, (signed char)scaleFwd));
    graph.setQuarterMetadata(weights, QuarterMetadata(formatW, (signed char)scaleW));
  }

  Sequence fwdProg, bwdProg;
  Tensor nextAct;
  if (doFwd) {
    nextAct = poplin::matMulGrouped(graph, prevAct, weights, fwdProg, outputType, "Fwd", fwdOptions,
                                    &cache);
    if (reportPlan) {
      std::cout << "Forward plan:\n";
      poplin::matMulGroupedReportPlan(std::cout, graph, inputType, outputType, actShape, wShape,
                                      fwdOptions, &cache);
    }
    if (bias) {
      // nextAct[g][b][:] += biases[g][:] on a densely packed [G][B][O] copy (the
      // product's own rows may be padded for alignment)
      const Tensor dense = graph.addVariable(outputType, outShape, "nextActDense");
      fwdProg.add(Copy(nextAct, dense));
      nextAct = dense;
      const Tensor act = nextAct, b = biases;
      const int dtype = plbType(outputType);
      fwdProg.add([=](plb_context *ctx) {
        const std::size_t es = act.elementType().bytes();
        for (std::size_t g = 0; g != numGroups; ++g)
          check(plb_add_bias(ctx, dtype,
                             static_cast<uint8_t *>(act.devicePointer()) + g * batchSize * outputSize * es,
                             static_cast<const uint8_t *>(b.devicePointer()) + g * outputSize * es,
                             batchSize, uint32_t(outputSize)));
      });
    }
  }
  Tensor zDeltas, prevDeltas;
  if (doBwd || doWu) {
    zDeltas = poplin::createMatMulGroupedInputLHS(graph, inputType, outputType, outShape,
                                                  {numGroups, outputSize, inputSize}, "zDeltas",
                                                  bwdOptions, &cache);
    if (inputType == QUARTER)
      graph.setQuarterMetadata(zDeltas, QuarterMetadata(formatBwd, (signed char)scaleBwd));
  }
  if (doBwd) {
    const Tensor weightsTransposed = poplin::transposeGroupedMatrix(weights);
    prevDeltas = poplin::matMulGrouped(graph, zDeltas, weightsTransposed, bwdProg, outputType, "Bwd",
                                       bwdOptions, &cache);
    if (reportPlan) {
      std::cout << "Backward plan:\n";
      poplin::matMulGroupedReportPlan(std::cout, graph, inputType, outputType, zDeltas.shape(),
                                      weightsTransposed.shape(), bwdOptions, &cache);
    }
  }
  if (doWu) {
    const Tensor prevActTransposed = poplin::transposeGroupedMatrix(prevAct);
    // grouped and ungrouped variants of the accumulating product, as the reference tool exercises
    if (numGroups == 1)
      poplin::matMulAcc(graph, weights.squeeze({0}), float(-learningRate), prevActTransposed.squeeze({0}),
                        zDeltas.squeeze({0}), bwdProg, "Wu", wuOptions, &cache);
    else
      poplin::matMulGroupedAcc(graph, weights, float(-learningRate), prevActTransposed, zDeltas, bwdProg,
                               "Wu", wuOptions, &cache);
    if (reportPlan) {
      std::cout << "WU plan:\n";
      poplin::matMulGroupedReportPlan(std::cout, graph, inputType, outputType, prevActTransposed.shape(),
                                      zDeltas.shape(), wuOptions, &cache);
    }
    if (bias) {
      // biases[g][:] += -lr * sum over the batch of zDeltas[g][b][:], on a densely
      // packed copy of the gradients
      const Tensor zDense = graph.addVariable(inputType, outShape, "zDeltasDense");
      bwdProg.add(Copy(zDeltas, zDense));
      const Tensor z = zDense, b = biases;
      const int zType = plbType(inputType), bType = plbType(outputType);
      bwdProg.add([=](plb_context *ctx) {
        const std::size_t zs = z.elementType().bytes(), bs = b.elementType().bytes();
        for (std::size_t g = 0; g != numGroups; ++g)
          check(plb_conv_bias_update(
              ctx, zType, static_cast<const uint8_t *>(z.devicePointer()) + g * batchSize * outputSize * zs,
              batchSize, uint32_t(outputSize), bType,
              static_cast<uint8_t *>(b.devicePointer()) + g * outputSize * bs, float(-learningRate)));
      });
    }
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
  if (compileOnly) return 0;  // graph and plans built; no device is touched
  Engine engine(graph, std::vector<Sequence>{fwdProg, bwdProg});

  if (!ignoreData) {
    std::mt19937 rng(seed);
    auto hAct = tool::randomValues(numGroups * batchSize * inputSize, -4.0, 4.0, rng, integerData);
    auto hW = tool::randomValues(numGroups * inputSize * outputSize, -3.0, 3.0, rng, integerData);
    auto hBias = tool::randomValues(numGroups * outputSize, -4.0, 4.0, rng, integerData);
    auto hDeltas = tool::randomValues(numGroups * batchSize * outputSize, -5.0, 5.0, rng, integerData);
    const auto rAct = tool::toDevice(hAct, inputType, scaleFwd, formatFwd == QuarterMetadata::Format::F152);
    const auto rW = tool::toDevice(hW, inputType, scaleW, formatW == QuarterMetadata::Format::F152);
    engine.writeTensor("prevAct", rAct.data(), rAct.data() + rAct.size());
    engine.writeTensor("weights", rW.data(), rW.data() + rW.size());
    tool::dump(dumpDir, "prevAct", hAct, actShape);
    tool::dump(dumpDir, "weights", hW, wShape);
    if (biases.valid()) {
      const auto rB = tool::toDevice(hBias, outputType);
      engine.writeTensor("biases", rB.data(), rB.data() + rB.size());
      tool::dump(dumpDir, "biases", hBias, {numGroups, outputSize});
    }
    if (zDeltas.valid()) {
      const auto rD = tool::toDevice(hDeltas, inputType, scaleBwd, formatBwd == QuarterMetadata::Format::F152);
      engine.writeTensor("zDeltas", rD.data(), rD.data() + rD.size());
      tool::dump(dumpDir, "zDeltas", hDeltas, outShape);
    }
  }
  engine.load(Device());
  auto readBack = [&](const char *handle, const Tensor &t, const std::vector<std::size_t> &shape,
                      const char *dumpName = nullptr) {
    if (ignoreData) return;
    std::vector<uint8_t> raw(t.numElements() * t.elementType().bytes());
    engine.readTensor(handle, raw.data(), raw.data() + raw.size());
    tool::dump(dumpDir, dumpName ? dumpName : handle, tool::fromDevice(raw, t.elementType()), shape);
  };
  const double flops = 2.0 * numGroups * batchSize * double(inputSize) * outputSize;
  if (doFwd) {
    engine.run(0);
    std::cout << "fwd: " << engine.lastRunMilliseconds() * 1e3 << " us, "
              << flops / engine.lastRunMilliseconds() / 1e9 << " TFLOP/s\n";
    readBack("nextAct", nextAct, outShape);
  }
  if (doBwd || doWu) {
    engine.run(1);
    std::cout << "bwd" << (doWu ? " + wu" : "") << ": " << engine.lastRunMilliseconds() * 1e3 << " us\n";
    if (doBwd) readBack("prevDeltas", prevDeltas, actShape);
    if (doWu) {
      readBack("weights", weights, wShape, "weightsUpdated");
      if (biases.valid()) readBack("biases", biases, {numGroups, outputSize}, "biasesUpdated");
    }
  }
  return 0;
} catch (const poplar::graph_memory_allocation_error &e) {
  std::cerr << e.what() << "\n";
  return 77;  // out of memory: reported as "skipped", as the reference tools do
} catch (const std::exception &e) {
  std::cerr << "error: " << e.what() << "\n";
  return 1;
}
