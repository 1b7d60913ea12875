// general_matrix_multiply: builds D = beta*C + alpha*op(A)*op(B) through the
// poplin::matMulGrouped surface, runs it on the GPU and reports time and
// throughput.  A port of the reference driver tools/general_matrix_multiply.cpp
// with the same option names for the subset that has meaning here; instead of
// linking a CPU model it writes its seeded inputs and the device result to
// --dump-dir for external checking.
#include <chrono>
#include <fstream>
#include <iostream>

#include "poplar/Engine.hpp"
#include "poplar/Graph.hpp"
#include "poplar/exceptions.hpp"
#include "poplin/MatMul.hpp"
#include "poplin/codelets.hpp"
#include "popops/codelets.hpp"
#include "poputil/exceptions.hpp"
#include "tool_util.hpp"

using namespace poplar;
using namespace poplar::program;

int main(int argc, char **argv) try {
  const tool::Args args(argc, argv);
  if (args.has("help")) {
    std::cout << "Options: --m --k --n [--g 1] [--data-type half] [--input-type T] [--output-type T]\n"
                 "  [--partials-type float] [--alpha 1] [--beta 1] [--left-matrix-op normal|transpose]\n"
                 "  [--right-matrix-op normal|transpose] [--fp8-scale-A 0] [--fp8-scale-B 0]\n"
                 "  [--plan-constraints JSON] [--plan-constraints-file F] [--report-plan]\n"
                 "  [--num-executions 1] [--seed 42] [--integer-data] [--dump-dir DIR]\n"
                 "  [--compile-only] [--ignore-data] [--device 0] [--profile]\n";
    return 0;
  }
  const unsigned m = args.required<unsigned>("m"), k = args.required<unsigned>("k"),
                 n = args.required<unsigned>("n"), g = args.get<unsigned>("g", 1);
  Type inputType = tool::parseType(args.str("data-type", "half"));
  Type outputType = inputType;
  if (args.has("input-type")) inputType = tool::parseType(args.str("input-type"));
  if (args.has("output-type")) outputType = tool::parseType(args.str("output-type"));
  else if (inputType == QUARTER) outputType = HALF;
  const std::string partialsType = args.str("partials-type", "float");
  const float alpha = args.get<float>("alpha", 1.f), beta = args.get<float>("beta", 1.f);
  const bool transposeA = args.str("left-matrix-op", "normal") == "transpose";
  const bool transposeB = args.str("right-matrix-op", "normal") == "transpose";
  const int scaleA = args.get<int>("fp8-scale-A", 0), scaleB = args.get<int>("fp8-scale-B", 0);
  const auto formatA = tool::quarterFormat(args.str("fp8-format-A", "F143"));
  const auto formatB = tool::quarterFormat(args.str("fp8-format-B", "F143"));
  std::string planConstraints = args.str("plan-constraints");
  const std::string planConstraintsFile = args.str("plan-constraints-file");
  if (!planConstraints.empty() && !planConstraintsFile.empty())
    throw poputil::poplibs_error("Both plan-constraints and plan-constraints-file were specified");
  if (!planConstraintsFile.empty()) {
    std::ifstream is(planConstraintsFile);
    if (!is.good()) throw poputil::poplibs_error("Plan constraints file doesn't exist");
    planConstraints.assign(std::istreambuf_iterator<char>(is), std::istreambuf_iterator<char>());
  }
  const unsigned numExecutions = args.get<unsigned>("num-executions", 1);
  const unsigned warmup = args.get<unsigned>("warmup", 0);  // untimed runs first (with --ignore-data)
  const unsigned seed = args.get<unsigned>("seed", 42);
  const bool integerData = args.has("integer-data") || inputType == QUARTER;
  const std::string dumpDir = args.str("dump-dir");
  const bool compileOnly = args.has("compile-only"), ignoreData = args.has("ignore-data");
  const bool reportPlan = args.has("report-plan"), profile = args.has("profile");
  const int device = args.get<int>("device", 0);
  args.str("remap-output-tensor");
  args.str("enable-fast-reduce");
  args.str("available-memory-proportion");
  args.rejectUnknown();

  Graph graph(Target::createGPUTarget(device));
  poplin::addCodelets(graph);
  popops::addCodelets(graph);

  poplin::PlanningCache cache;
  OptionFlags mmOpt;
  mmOpt.set("partialsType", partialsType);
  if (!planConstraints.empty()) mmOpt.set("planConstraints", planConstraints);
  if (transposeB) mmOpt.set("fullyConnectedPass", "TRAINING_BWD");
  else if (transposeA) mmOpt.set("fullyConnectedPass", "TRAINING_WU");

  if (reportPlan)
    poplin::matMulGroupedReportPlan(std::cout, graph, inputType, outputType, {g, m, k}, {g, k, n},
                                    mmOpt, &cache);

  // the operands are created for the product and then viewed transposed, as the
  // reference tool does: host data for A' / B' has shape [k][m] / [n][k]
  Tensor matA = poplin::createMatMulGroupedInputLHS(graph, inputType, outputType, {g, m, k},
                                                    {g, k, n}, "matA", mmOpt, &cache);
  if (transposeA) matA = matA.dimShufflePartial({1, 2}, {2, 1});
  Tensor matB = poplin::createMatMulGroupedInputRHS(graph, inputType, outputType, {g, m, k},
                                                    {g, k, n}, "matB", mmOpt, &cache);
  if (transposeB) matB = matB.dimShufflePartial({1, 2}, {2, 1});
  if (inputType == QUARTER) {
    graph.setQuarterMetadata(matA, QuarterMetadata(formatA, (signed char)scaleA));
    graph.setQuarterMetadata(matB, QuarterMetadata(formatB, (signed char)scaleB));
  }
  const Tensor lhs = transposeA ? matA.dimShufflePartial({1, 2}, {2, 1}) : matA;
  const Tensor rhs = transposeB ? matB.dimShufflePartial({1, 2}, {2, 1}) : matB;

  Sequence prog;
  Tensor matC = poplin::createMatMulGroupedOutput(graph, inputType, outputType, {g, m, k},
                                                  {g, k, n}, "matC", mmOpt, &cache);
  // matC = beta * matC + alpha * op(A) op(B): one accumulating product
  Sequence inner;
  if (beta == 0.f) {
    poplin::matMulGroupedWithOutput(graph, lhs, rhs, matC, inner, "op(A) x op(B)", mmOpt, &cache);
    if (alpha != 1.f) throw poputil::poplibs_error("--beta 0 needs --alpha 1");
  } else if (beta == 1.f) {
    poplin::matMulGroupedAcc(graph, matC, alpha, lhs, rhs, inner, "C += alpha op(A) x op(B)", mmOpt,
                             &cache);
  } else {
    throw poputil::poplibs_error("--beta must be 0 or 1 in this port");
  }
  prog.add(Repeat(numExecutions, inner));
  if (numExecutions > 1 && beta != 0.f)
    std::cerr << "note: with beta != 0 every execution accumulates into C\n";

  graph.createHostWrite("matA", matA);
  graph.createHostWrite("matB", matB);
  graph.createHostWrite("matC", matC);
  graph.createHostRead("matC", matC);
  if (compileOnly) return 0;  // graph and plans built; no device is touched
  Engine engine(graph, prog);

  const std::size_t rowsA = transposeA ? k : m, colsA = transposeA ? m : k;
  const std::size_t rowsB = transposeB ? n : k, colsB = transposeB ? k : n;
  std::vector<double> hostA, hostB, hostC;
  if (!ignoreData) {
    std::mt19937 rng(seed);
    hostA = tool::randomValues(std::size_t(g) * rowsA * colsA, -4.0, 4.0, rng, integerData);
    hostB = tool::randomValues(std::size_t(g) * rowsB * colsB, -3.0, 3.0, rng, integerData);
    hostC = tool::randomValues(std::size_t(g) * m * n, -2.0, 2.0, rng, integerData);
    const auto rawA = tool::toDevice(hostA, inputType, scaleA, formatA == QuarterMetadata::Format::F152);
    const auto rawB = tool::toDevice(hostB, inputType, scaleB, formatB == QuarterMetadata::Format::F152);
    const auto rawC = tool::toDevice(hostC, outputType);
    engine.writeTensor("matA", rawA.data(), rawA.data() + rawA.size());
    engine.writeTensor("matB", rawB.data(), rawB.data() + rawB.size());
    engine.writeTensor("matC", rawC.data(), rawC.data() + rawC.size());
    tool::dump(dumpDir, "A", hostA, {g, rowsA, colsA});
    tool::dump(dumpDir, "B", hostB, {g, rowsB, colsB});
    tool::dump(dumpDir, "C", hostC, {g, m, n});
  }
  engine.load(Device());
  if (warmup && !ignoreData && beta != 0.f)
    throw poputil::poplibs_error("--warmup with beta != 0 would accumulate more than once: "
                                 "use it with --ignore-data");
  for (unsigned i = 0; i < warmup; ++i) engine.run(0);
  engine.run(0);
  const double ms = engine.lastRunMilliseconds() / numExecutions;
  const double flops = 2.0 * g * m * double(k) * n;
  std::cout << "gemm " << g << "x" << m << "x" << k << "x" << n << " " << inputType << "->"
            << outputType << ": " << ms * 1e3 << " us per execution, " << flops / ms / 1e9
            << " TFLOP/s\n";
  if (!ignoreData) {
    std::vector<uint8_t> raw(std::size_t(g) * m * n * outputType.bytes());
    engine.readTensor("matC", raw.data(), raw.data() + raw.size());
    tool::dump(dumpDir, "D", tool::fromDevice(raw, outputType), {g, m, n});
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
