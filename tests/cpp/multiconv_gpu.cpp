// Two different convolutions through poplin::multiconv on the GPU: the forward
// pass, the weight gradients and the weight update of both, built as one
// multi-convolution each and run through the Engine.  Inputs are small
// integers (every sum exact); all tensors are dumped for the Python test, which
// compares them with the CPU oracle bit for bit.  The cases follow the
// reference's multi-convolution test (tests/poplin/MultiConvTest.cpp), which
// checks that a multi-convolution equals its member convolutions.
//
//   multiconv_gpu <dump-dir>
#include <cstdio>
#include <iostream>
#include <random>

#include "poplar/Engine.hpp"
#include "poplar/Graph.hpp"
#include "poplin/ConvUtil.hpp"
#include "poplin/MultiConvolution.hpp"
#include "poplin/codelets.hpp"
#include "tool_util.hpp"

using namespace poplar;
using namespace poplar::program;
namespace mc = poplin::multiconv;

int main(int argc, char **argv) try {
  if (argc < 2) {
    std::cerr << "usage: multiconv_gpu <dump-dir>\n";
    return 2;
  }
  const std::string dir = argv[1];
  Graph graph(Target::createGPUTarget(0));
  poplin::addCodelets(graph);
  poplin::PlanningCache cache;

  // a padded 3x3 layer and a grouped, strided pointwise layer
  const poplin::ConvParams pa(HALF, HALF, 3, {12, 12}, {3, 3}, 64, 72, 1,
                              poplin::ConvParams::InputTransform({0, 0}, {0, 0}, {1, 1}, {1, 1}, {1, 1},
                                                                 {false, false}),
                              poplin::ConvParams::InputTransform(2),
                              poplin::ConvParams::OutputTransform(2));
  const poplin::ConvParams pb(HALF, FLOAT, 2, {9, 10}, {1, 1}, 32, 48, 2,
                              poplin::ConvParams::InputTransform(2), poplin::ConvParams::InputTransform(2),
                              poplin::ConvParams::OutputTransform({0, 0}, {0, 0}, {2, 2}, {0, 0}, {0, 0}));
  const std::vector<poplin::ConvParams> params{pa, pb};
  const std::vector<mc::CreateTensorArgs> create{{pa, {}, "a"}, {pb, {}, "b"}};

  std::vector<mc::ConvolutionArgs> fwd;
  for (unsigned i = 0; i < 2; ++i)
    fwd.push_back({mc::createInput(graph, create, i, {}, &cache), mc::createWeights(graph, create, i, {}, &cache),
                   params[i], {}});
  Sequence fwdProg, wuProg;
  const auto outs = mc::convolution(graph, fwd, false, fwdProg, "fwd", {{"planType", "serial"}}, &cache);

  std::vector<Tensor> zDeltas;
  std::vector<mc::CalculateWeightDeltasArgs> wuArgs;
  std::vector<mc::ConvWeightUpdateArgsScalar> updArgs;
  for (unsigned i = 0; i < 2; ++i) {
    // the output gradients have the output's shape and the input's type
    zDeltas.push_back(poplin::createInput(graph, poplin::getGradientParams(params[i]), "zDeltas", {}, &cache));
    wuArgs.push_back({zDeltas[i], fwd[i].inputs, params[i], {}});
    updArgs.push_back({zDeltas[i], fwd[i].weights, fwd[i].inputs, -0.5f, params[i], {}});
  }
  const auto deltas = mc::calculateWeightDeltas(graph, wuArgs, wuProg, "wu", {}, &cache);
  mc::convolutionWeightUpdate(graph, updArgs, wuProg, "upd", {}, &cache);

  for (unsigned i = 0; i < 2; ++i) {
    const std::string n = std::to_string(i);
    graph.createHostWrite("in" + n, fwd[i].inputs);
    graph.createHostWrite("w" + n, fwd[i].weights);
    graph.createHostRead("w" + n, fwd[i].weights);
    graph.createHostWrite("dy" + n, zDeltas[i]);
    graph.createHostRead("out" + n, outs[i]);
    graph.createHostRead("dw" + n, deltas[i]);
  }
  Engine engine(graph, std::vector<Sequence>{fwdProg, wuProg});
  std::mt19937 rng(42);
  for (unsigned i = 0; i < 2; ++i) {
    const std::string n = std::to_string(i);
    auto put = [&](const std::string &name, const Tensor &t, double lo, double hi) {
      auto v = tool::randomValues(t.numElements(), lo, hi, rng, true);
      const auto raw = tool::toDevice(v, t.elementType());
      engine.writeTensor(name, raw.data(), raw.data() + raw.size());
      tool::dump(dir, name, v, t.shape());
    };
    put("in" + n, fwd[i].inputs, -2, 2);
    put("w" + n, fwd[i].weights, -2, 2);
    put("dy" + n, zDeltas[i], -1, 1);
  }
  engine.load(Device());
  engine.run(0);
  engine.run(1);
  for (unsigned i = 0; i < 2; ++i) {
    const std::string n = std::to_string(i);
    auto get = [&](const std::string &name, const Tensor &t, const std::string &as) {
      std::vector<uint8_t> raw(t.numElements() * t.elementType().bytes());
      engine.readTensor(name, raw.data(), raw.data() + raw.size());
      tool::dump(dir, as, tool::fromDevice(raw, t.elementType()), t.shape());
    };
    get("out" + n, outs[i], "out" + n);
    get("dw" + n, deltas[i], "dw" + n);
    get("w" + n, fwd[i].weights, "wUpdated" + n);
  }
  return 0;
} catch (const std::exception &e) {
  std::cerr << "error: " << e.what() << "\n";
  return 1;
}
