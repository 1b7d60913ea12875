// A convolution followed by batch normalisation, forward and backward, through
// the poplin C++ surface on the GPU: convolution -> normStatistics ->
// normWhiten -> normalise, then normGradients -> normParamGradients ->
// normStatisticsGradients on a given output gradient.  Every tensor is dumped
// for the Python test, which checks each stage against the CPU oracle (the
// flow of the reference's norm layer tests: tools/norm_layer.cpp builds the
// same chain after a convolution).
//
//   conv_norm_gpu <dump-dir>
#include <iostream>
#include <random>

#include "poplar/Engine.hpp"
#include "poplar/Graph.hpp"
#include "poplin/Convolution.hpp"
#include "poplin/Norms.hpp"
#include "poplin/codelets.hpp"
#include "tool_util.hpp"

using namespace poplar;
using namespace poplar::program;

int main(int argc, char **argv) try {
  if (argc < 2) {
    std::cerr << "usage: conv_norm_gpu <dump-dir>\n";
    return 2;
  }
  const std::string dir = argv[1];
  Graph graph(Target::createGPUTarget(0));
  poplin::addCodelets(graph);
  const poplin::ConvParams p(HALF, HALF, 4, {10, 10}, {3, 3}, 16, 32, 1,
                             poplin::ConvParams::InputTransform({0, 0}, {0, 0}, {1, 1}, {1, 1}, {1, 1},
                                                                {false, false}),
                             poplin::ConvParams::InputTransform(2), poplin::ConvParams::OutputTransform(2));
  Tensor in = poplin::createInput(graph, p, "in");
  Tensor w = poplin::createWeights(graph, p, "w");
  Sequence fwd, bwd;
  Tensor y = poplin::convolution(graph, in, w, p, false, fwd, "conv");
  auto stats = poplin::normStatistics(graph, y, 1e-3f, fwd, true, false, FLOAT, "bn");
  auto params = poplin::createNormParams(graph, y, "bn");
  Tensor white = poplin::normWhiten(graph, y, stats.first, stats.second, fwd, "bn");
  Tensor out = poplin::normalise(graph, white, params.first, params.second, fwd, "bn");
  // backward: gradient of `out` in, gradients of gamma / beta and of y out
  Tensor gradOut = graph.clone(out, "gradOut");
  Tensor gradWhite = poplin::normGradients(graph, gradOut, params.first, bwd, "bn");
  auto paramGrads = poplin::normParamGradients(graph, white, gradOut, bwd, FLOAT, "bn");
  Tensor gradY = poplin::normStatisticsGradients(graph, white, gradWhite, stats.second, bwd, FLOAT, "bn");

  struct Io { const char *name; Tensor t; bool write; };
  std::vector<Io> ios = {{"in", in, true}, {"w", w, true}, {"gamma", params.first, true},
                         {"beta", params.second, true}, {"gradOut", gradOut, true}, {"y", y, false},
                         {"mean", stats.first, false}, {"iStdDev", stats.second, false},
                         {"white", white, false}, {"out", out, false}, {"gradWhite", gradWhite, false},
                         {"gammaGrad", paramGrads.first, false}, {"betaGrad", paramGrads.second, false},
                         {"gradY", gradY, false}};
  for (const auto &io : ios) {
    if (io.write) graph.createHostWrite(io.name, io.t);
    else graph.createHostRead(io.name, io.t);
  }
  Engine engine(graph, std::vector<Sequence>{fwd, bwd});
  std::mt19937 rng(7);
  for (const auto &io : ios) {
    if (!io.write) continue;
    const bool positive = std::string(io.name) == "gamma";
    auto v = tool::randomValues(io.t.numElements(), positive ? 0.5 : -1.0, positive ? 2.0 : 1.0, rng, false);
    const auto raw = tool::toDevice(v, io.t.elementType());
    engine.writeTensor(io.name, raw.data(), raw.data() + raw.size());
    tool::dump(dir, io.name, v, io.t.shape());
  }
  engine.load(Device());
  engine.run(0);
  engine.run(1);
  for (const auto &io : ios) {
    if (io.write) continue;
    std::vector<uint8_t> raw(io.t.numElements() * io.t.elementType().bytes());
    engine.readTensor(io.name, raw.data(), raw.data() + raw.size());
    tool::dump(dir, io.name, tool::fromDevice(raw, io.t.elementType()), io.t.shape());
  }
  return 0;
} catch (const std::exception &e) {
  std::cerr << "error: " << e.what() << "\n";
  return 1;
}
