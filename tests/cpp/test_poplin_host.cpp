// Host-only checks of the C++ poplar / poplin layer (no GPU is touched: graphs
// are built and programs recorded, but no Engine is created).  The cases are
// the reference's own unit tests restated for this layer: ConvParams JSON
// (tests/poplin/ConvTest.cpp:651-682), option validation (:684-706), the plan
// constraints grammar (tests/poplin/ConvOptionsTest.cpp:12-107), index ranges
// (tests/poplin/RangeTest.cpp, ConvUtilTest.cpp:14-51).
#include <cmath>
#include <cstdio>
#include <fstream>
#include <functional>
#include <iostream>
#include <set>
#include <sstream>
#include <unordered_set>

#include "poplar/Engine.hpp"
#include "poplar/Graph.hpp"
#include "poplar/exceptions.hpp"
#include "poplin/ConvPreplan.hpp"
#include "poplin/ConvUtil.hpp"
#include "poplin/Convolution.hpp"
#include "poplin/FullyConnected.hpp"
#include "poplin/MatMul.hpp"
#include "poplin/MultiConvolution.hpp"
#include "poplin/Norms.hpp"
#include "poplin/codelets.hpp"
#include "poputil/exceptions.hpp"

using namespace poplin;
using poplar::FLOAT;
using poplar::HALF;
using poplar::QUARTER;

static int failures = 0;
#define CHECK(cond)                                                          \
  do {                                                                       \
    if (!(cond)) {                                                           \
      std::printf("FAIL %s:%d: %s\n", __FILE__, __LINE__, #cond);            \
      ++failures;                                                            \
    }                                                                        \
  } while (0)
template <class E, class F> static bool throwsAs(F &&f) {
  try {
    f();
  } catch (const E &) {
    return true;
  } catch (...) {
  }
  return false;
}
template <class F> static bool noThrow(F &&f) {
  try {
    f();
  } catch (const std::exception &e) {
    std::printf("  unexpected exception: %s\n", e.what());
    return false;
  }
  return true;
}

static void testConvParamsJson() {
  std::stringstream is;
  is << R"({
      "dataType": "float", "batchSize": 1, "numConvGroups": 2,
      "inputChannelsPerConvGroup": 3, "outputChannelsPerConvGroup": 4,
      "kernelShape": [50, 60], "inputFieldShape": [70, 80],
      "inputTransform": {"truncationLower": [1, 2], "paddingUpper": [3, 4], "flip": [true, false]},
      "outputTransform": {"stride": [5, 6]}
    })";
  ConvParams uut{};
  is >> uut;
  ConvParams expected(FLOAT, 1, {70, 80}, {50, 60}, 3, 4, 2);
  expected.inputTransform.truncationLower = {1, 2};
  expected.inputTransform.paddingUpper = {3, 4};
  expected.inputTransform.flip = {true, false};
  expected.outputTransform.stride = {5, 6};
  CHECK(uut == expected);
  CHECK(!(uut != expected) && !(uut < expected) && !(expected < uut));
  CHECK(std::hash<ConvParams>()(uut) == std::hash<ConvParams>()(expected));
  std::stringstream bad;
  bad << R"({"inputFieldShape": [3, 3], "kernelShape": [2]})";
  ConvParams q{};
  CHECK((throwsAs<poputil::poplibs_error>([&] { bad >> q; })));
  std::ostringstream text;
  text << expected;
  CHECK(text.str().find("inputFieldShape            {70,80}") != std::string::npos);
  CHECK(text.str().find("stride                     {5,6}") != std::string::npos);
}

static void testValidation() {
  CHECK((throwsAs<poputil::poplibs_error>([&] { ConvParams(HALF, 1, {4, 4}, {3}, 1, 1, 1).validate(); })));
  ConvParams p(HALF, 1, {4, 4}, {3, 3}, 1, 1, 1);
  CHECK(noThrow([&] { p.validate(); }));
  p.outputTransform.stride = {0, 1};
  CHECK((throwsAs<poputil::poplibs_error>([&] { p.validate(); })));
  p.outputTransform.stride = {1, 1};
  p.kernelTransform.dilation = {2, 1};
  try {
    p.validate();
    CHECK(false);
  } catch (const poputil::poplibs_error &e) {
    CHECK(std::string(e.what()) ==
          "Transformed input size for dimension 0 (4) is less than the transformed kernel size (5)");
  }
  // std::set / unordered_set membership as the reference's callers need
  std::set<ConvParams> s;
  s.insert(ConvParams(HALF, 1, {4, 4}, {3, 3}, 1, 1, 1));
  s.insert(ConvParams(HALF, 1, {4, 4}, {3, 3}, 1, 1, 1));
  s.insert(ConvParams(HALF, 2, {4, 4}, {3, 3}, 1, 1, 1));
  CHECK(s.size() == 2);
  std::unordered_set<ConvParams> us(s.begin(), s.end());
  CHECK(us.size() == 2);
}

static ConvParams rangeParams(unsigned stride, unsigned kernel, unsigned padLo, unsigned padHi,
                              unsigned size) {
  ConvParams p(FLOAT, 1, {size, size}, {kernel, kernel}, 1, 1, 1);
  p.inputTransform.paddingLower = {padLo, padLo};
  p.inputTransform.paddingUpper = {padHi, padHi};
  p.outputTransform.stride = {stride, stride};
  return p;
}

static void testRanges() {
  const auto p1 = rangeParams(1, 3, 0, 0, 10);
  CHECK(getInputIndex(0, 0, 0, p1) == 0u && getInputIndex(0, 7, 2, p1) == 9u);
  const auto p5 = rangeParams(2, 3, 1, 0, 10);
  CHECK(getInputIndex(0, 0, 0, p5) == ~0u && getInputIndex(0, 4, 2, p5) == 9u);
  const auto p9 = rangeParams(2, 3, 1, 2, 10);
  CHECK(getInputIndex(0, 5, 0, p9) == 9u && getInputIndex(0, 5, 1, p9) == ~0u);
  CHECK(p9.getOutputSize(0) == 6);
  CHECK(getKernelIndex(0, 4, 9, p9) == 2u && getKernelIndex(0, 0, 9, p9) == ~0u);
  {  // tests/poplin/ConvUtilTest.cpp:14-32
    ConvParams p(FLOAT, 1, {3, 1}, {5, 1}, 1, 1, 1);
    p.inputTransform.paddingLower = {2, 0};
    p.inputTransform.paddingUpper = {2, 0};
    p.inputTransform.flip = {true, false};
    p.kernelTransform.flip = {true, false};
    const auto r = getInputRange(0, {0, 2}, 1, p);
    CHECK(r.first == 0 && r.second == 2);
  }
  {  // tests/poplin/ConvUtilTest.cpp:34-51
    ConvParams p(FLOAT, 1, {3}, {4}, 1, 1, 1);
    p.inputTransform.truncationUpper = {1};
    p.inputTransform.dilation = {2};
    p.inputTransform.paddingLower = {1};
    const auto r = getKernelRange(0, {0, 1}, {0, 3}, p);
    CHECK(r.first == 1 && r.second == 4);
  }
}

static void testCanonicalAndDerivedParams() {
  // 3x3 stride 1 pad 1: already canonical; its gradient convolution is itself
  ConvParams p(HALF, 256, {28, 28}, {3, 3}, 128, 128, 1);
  p.inputTransform.paddingLower = {1, 1};
  p.inputTransform.paddingUpper = {1, 1};
  CHECK(p.canonicalize() == p);
  CHECK(getGradientParams(p) == p);
  const ConvParams wu = getWeightUpdateParams(p);
  CHECK(wu.batchSize == 128 && wu.inputChannelsPerConvGroup == 256 &&
        wu.outputChannelsPerConvGroup == 128);
  CHECK((wu.kernelShape == std::vector<std::size_t>{28, 28}));
  CHECK((wu.getOutputFieldShape() == std::vector<std::size_t>{3, 3}));
  CHECK(getFwdFlops(p) == 56405000192ull && getBwdFlops(p) == getWuFlops(p));
  // stride 2: the gradient convolution dilates its input by the stride
  ConvParams s(HALF, 2, {9, 9}, {3, 3}, 8, 16, 1);
  s.inputTransform.paddingLower = {1, 1};
  s.inputTransform.paddingUpper = {1, 1};
  s.outputTransform.stride = {2, 2};
  const ConvParams g = getGradientParams(s);
  CHECK((g.inputTransform.dilation == std::vector<unsigned>{2, 2}));
  CHECK((g.getOutputFieldShape() == std::vector<std::size_t>{9, 9}));
  CHECK(g.inputChannelsPerConvGroup == 16 && g.outputChannelsPerConvGroup == 8);
  // a stride larger than what a single output needs is dropped
  ConvParams one(HALF, 1, {3}, {3}, 1, 1, 1);
  one.outputTransform.stride = {5};
  CHECK(one.canonicalize().outputTransform.stride[0] == 1);
  // excess input padding that only produces ignored outputs is folded away
  ConvParams pad(HALF, 1, {5}, {3}, 1, 1, 1);
  pad.inputTransform.paddingLower = {2};
  pad.outputTransform.truncationLower = {2};
  const ConvParams c = pad.canonicalize();
  CHECK(c.inputTransform.paddingLower[0] == 0 && c.outputTransform.truncationLower[0] == 0);
  CHECK(c.getOutputSize(0) == pad.getOutputSize(0));
}

static void testOptions() {
  CHECK(noThrow([&] { convolutionValidateOptions({{"partialsType", "half"}}); }));
  CHECK((throwsAs<poplar::invalid_option>([&] { convolutionValidateOptions({{"partialsType", "invalid_value"}}); })));
  CHECK((throwsAs<poplar::invalid_option>([&] { convolutionValidateOptions({{"invalid_key", "half"}}); })));
  CHECK(noThrow([&] { matmulValidateOptions({{"partialsType", "half"}}); }));
  CHECK((throwsAs<poplar::invalid_option>([&] { matmulValidateOptions({{"partialsType", "invalid_value"}}); })));
  CHECK((throwsAs<poplar::invalid_option>([&] { matmulValidateOptions({{"invalid_key", "half"}}); })));
  CHECK(noThrow([&] { convolutionValidateOptions({{"pass", "TRAINING_WU"},
                                             {"availableMemoryProportion", "0.3"},
                                             {"enableFastReduce", "true"},
                                             {"partialsType.interIPU", "float"}}); }));
  CHECK((throwsAs<poplar::invalid_option>([&] { convolutionValidateOptions({{"availableMemoryProportion", "-1"}}); })));
  CHECK((throwsAs<poplar::invalid_option>([&] { convolutionValidateOptions({{"enableFastReduce", "yes"}}); })));
  CHECK(noThrow([&] { matmulValidateOptions({{"fullyConnectedPass", "TRAINING_BWD"},
                                        {"inputRHSIsPreArranged", "true"}}); }));
  try {
    convolutionValidateOptions({{"invalid_key", "half"}});
  } catch (const poplar::invalid_option &e) {
    CHECK(std::string(e.what()) == "Unrecognised option 'invalid_key'");
  }
  // plan constraints grammar
  auto pc = [](const std::string &json) { convolutionValidateOptions({{"planConstraints", json}}); };
  CHECK(noThrow([&] { pc("{}"); }));
  CHECK(noThrow([&] { pc(R"({"0": {}, "2": {}, " 5": {}})"); }));
  CHECK((throwsAs<poplar::invalid_option>([&] { pc(R"({"": {}})"); })));
  CHECK((throwsAs<poplar::invalid_option>([&] { pc(R"({"-1": {}})"); })));
  CHECK((throwsAs<poplar::invalid_option>([&] { pc(R"({"a watched pot never boils": {}})"); })));
  CHECK((throwsAs<poplar::invalid_option>([&] { pc("0"); })));
  CHECK(noThrow([&] { pc(R"({"0": {"partition": {"convGroupSplit": 4, "fieldSplit": {"0": 4, "2": 5},
                                            "inChanSplit": {"serial": 4, "parallel": 5}},
                               "transform": {"swapOperands": false, "expandDims": [0, 1]}},
                        "method": {"type": "AMP", "convUnits": 16}})"); }));
  CHECK((throwsAs<poplar::invalid_option>(
      [&] { pc(R"({"0": {"partition": {"fieldSplit": {"5": "a watched pot never boils"}}}})"); })));
  CHECK((throwsAs<poplar::invalid_option>(
      [&] { pc(R"({"0": {"partition": {"fieldSplit": {"hello": "world"}}}})"); })));
  CHECK((throwsAs<poplar::invalid_option>([&] { pc(R"({"0": {"partition": {"inChanSplit": {"hello": 1}}}})"); })));
  CHECK((throwsAs<poplar::invalid_option>(
      [&] { pc(R"({"0": {"transform": {"swapOperands": "a watched pot never boils"}}})"); })));
  CHECK((throwsAs<poplar::invalid_option>(
      [&] { pc(R"({"0": {"transform": {"a watched pot never boils": {}}}})"); })));
  CHECK((throwsAs<poplar::invalid_option>([&] { pc(R"({"0": {"partition": {"a watched pot never boils": {}}}})"); })));
  CHECK((throwsAs<poplar::invalid_option>([&] { pc(R"({"0": {"somethingElse": {}}})"); })));
  CHECK((throwsAs<poplar::invalid_option>([&] { pc(R"({"method": {"type": "TENSOR_CORE"}})"); })));
  CHECK(noThrow([&] { pc(R"({"cuda": {"tileN": 128, "splitK": 49, "residentWeights": false}})"); }));
  CHECK((throwsAs<poplar::invalid_option>([&] { pc(R"({"cuda": {"tileQ": 1}})"); })));
  // OptionFlags from JSON keeps nested objects as text
  poplar::OptionFlags flags;
  poplar::readJSON(R"({"partialsType": "float", "planConstraints": {"0": {"partition": {"batchSplit": 2}}}})",
                   flags);
  CHECK(flags.size() == 2);
  CHECK(noThrow([&] { convolutionValidateOptions(flags); }));
}

static void testTensorViews() {
  poplar::Graph graph(poplar::Target::createGPUTarget(0));
  poplin::addCodelets(graph);
  auto t = graph.addVariable(HALF, {2, 3, 4, 5}, "t");
  CHECK(t.isContiguous() && t.numElements() == 120 && t.rank() == 4);
  auto s = t.dimShuffle({0, 2, 3, 1});
  CHECK((s.shape() == std::vector<std::size_t>{2, 4, 5, 3}) && !s.isContiguous());
  CHECK((s.strides() == std::vector<std::ptrdiff_t>{60, 5, 1, 20}));
  CHECK((t.dimRoll(3, 1).shape() == std::vector<std::size_t>{2, 5, 3, 4}));
  CHECK((t.dimShufflePartial({1, 2}, {2, 1}).shape() == std::vector<std::size_t>{2, 4, 3, 5}));
  CHECK((t.reshape({6, 20}).strides() == std::vector<std::ptrdiff_t>{20, 1}));
  CHECK((s.reshape({2, 20, 3}).strides() == std::vector<std::ptrdiff_t>{60, 1, 20}));
  CHECK((throwsAs<poputil::poplibs_error>([&] { s.reshape({8, 15}); })));
  CHECK((t.slice(1, 3, 1).shape() == std::vector<std::size_t>{2, 2, 4, 5}) && t.slice(1, 3, 1).offset() == 20);
  CHECK((t[1].shape() == std::vector<std::size_t>{3, 4, 5}) && t[1].offset() == 60);
  CHECK((t.expand({0, 2}).shape() == std::vector<std::size_t>{1, 2, 3, 1, 4, 5}));
  CHECK((t.expand({0}).squeeze({0}).shape() == t.shape()));
  CHECK(t.reverse(3).offset() == 4 && t.reverse(3).strides()[3] == -1);
  CHECK(t.flatten().rank() == 1 && t.flatten(1, 3).dim(1) == 12);
  auto c = graph.clone(s, "clone");
  CHECK(c.shape() == s.shape() && c.strides() == s.strides());
  CHECK((throwsAs<poplar::runtime_error>([&] { t.devicePointer(); })));  // no Engine yet
}

static void testGraphConstructionWithoutDevice() {
  poplar::Graph graph(poplar::Target::createGPUTarget(0));
  PlanningCache cache;
  ConvParams p(HALF, 32, {56, 56}, {3, 3}, 64, 64, 1);
  p.inputTransform.paddingLower = {1, 1};
  p.inputTransform.paddingUpper = {1, 1};
  const poplar::OptionFlags fwdOpts{{"pass", "TRAINING_FWD"}, {"partialsType", "float"}};
  auto in = createInput(graph, p, "in", fwdOpts, &cache);
  auto w = createWeights(graph, p, "weights", fwdOpts, &cache);
  CHECK((in.shape() == std::vector<std::size_t>{32, 64, 56, 56}));
  CHECK((w.shape() == std::vector<std::size_t>{1, 64, 64, 3, 3}));
  // channels innermost in memory
  CHECK(in.strides()[1] == 1 && w.strides()[2] == 1 && w.strides()[1] == 64);
  poplar::program::Sequence prog;
  auto out = convolution(graph, in, w, p, false, prog, "conv", fwdOpts, &cache);
  CHECK((out.shape() == std::vector<std::size_t>{32, 64, 56, 56}));
  CHECK(prog.steps().size() == 1);  // no rearrangement copies were needed
  CHECK(cache.size() == 1);
  // a second identical convolution hits the cache
  convolution(graph, in, w, p, false, prog, "conv2", fwdOpts, &cache);
  CHECK(cache.size() == 1);
  // weights without the group dimension; an input in NCHW memory order needs a copy
  auto plain = graph.addVariable(HALF, {32, 64, 56, 56}, "nchw");
  poplar::program::Sequence prog2;
  convolution(graph, plain, w[0], p, false, prog2, "conv3", fwdOpts, &cache);
  CHECK(prog2.steps().size() == 2);
  // shape and type errors
  CHECK((throwsAs<poputil::poplibs_error>([&] { convolution(graph, in.slice(0, 16, 0), w, p, false, prog, "bad"); })));
  // the weight update pass and its plan report
  auto dw = calculateWeightDeltas(graph, out, in, p, prog, "wu", {{"pass", "TRAINING_WU"}}, &cache);
  CHECK(dw.shape() == w.shape() && dw.elementType() == HALF);
  std::ostringstream report;
  reportPlanInfo(report, graph, p, fwdOpts, &cache);
  reportWeightUpdatePlanInfo(report, graph, p, fwdOpts, &cache);
  CHECK(report.str().find("CTA tile (pixels x chans)  128 x 64") != std::string::npos);
  CHECK(report.str().find("weight update (split-K)") != std::string::npos);
  CHECK(reportPlanEstimatedCosts(graph, p, fwdOpts, &cache).cycles != PlanCosts::unknown);
  // perfect cycle counts: MACs / (4096 fp16 MACs per SM and cycle x 148 SMs)
  {
    const double macs = double(getFwdFlops(p)) / 2.0;
    CHECK(std::abs(getFwdPerfectCycleCount(graph, p) - macs / (4096.0 * 148.0)) < 1e-6 * macs);
    CHECK(getBwdPerfectCycleCount(graph, p) == getFwdPerfectCycleCount(graph, p));
    CHECK(getWuPerfectCycleCount(graph, p) == getFwdPerfectCycleCount(graph, p));
    ConvParams q8 = p;
    q8.inputType = QUARTER;
    CHECK(std::abs(getFwdPerfectCycleCount(graph, q8) * 2.0 - getFwdPerfectCycleCount(graph, p)) < 1e-6 * macs);
  }
  // itemised costs: written and read back in the reference's text form
  {
    const auto d = internal::reportDetailedPlanEstimatedCosts(graph, p, fwdOpts, &cache);
    CHECK(d.total.cycles == d.compute.cycles + d.reduction.cycles + d.rearrangement.cycles);
    CHECK(d.compute.cycles >= std::size_t(getFwdPerfectCycleCount(graph, p)) && d.parallelSplit == 148);
    std::stringstream ss;
    ss << d;
    internal::DetailedPlanCosts back;
    ss >> back;
    CHECK(back.total.cycles == d.total.cycles && back.compute.cycles == d.compute.cycles &&
          back.parallelSplit == d.parallelSplit && back.outputCast.memory == d.outputCast.memory);
    // a long, thin contraction is split over K: the reduction shows up
    ConvParams thin(HALF, HALF, 1, {256}, {1}, 8192, 256, 1);
    const auto dt = internal::reportDetailedPlanEstimatedCosts(graph, thin, fwdOpts);
    CHECK(dt.reduction.cycles > 0 && dt.reduction.memory > 0 && dt.total.memory == dt.reduction.memory);
  }
  // the chosen plan written as planConstraints and fed back reproduces the plan
  {
    const std::string base = "/tmp/plb_plan_constraints_test";
    for (const char *cons : {"", R"({"cuda": {"splitK": 3, "tileN": 128, "halo": false, "ctaPair": true}})"}) {
      poplar::OptionFlags o1 = {{"pass", "TRAINING_FWD"}, {"planConstraintsOutputFilename", base}};
      if (*cons) o1.set("planConstraints", cons);
      std::ostringstream first;
      reportPlanInfo(first, graph, p, o1);
      std::ifstream in(base + "_FWD.json");
      CHECK(bool(in));
      std::stringstream text;
      text << in.rdbuf();
      CHECK(text.str().find("\"inChanSplit\"") != std::string::npos);
      std::ostringstream second;
      reportPlanInfo(second, graph, p, {{"pass", "TRAINING_FWD"}, {"planConstraints", text.str()}});
      CHECK(first.str() == second.str());
      std::remove((base + "_FWD.json").c_str());
    }
    std::ostringstream wu1, wu2;
    reportWeightUpdatePlanInfo(wu1, graph, p, {{"planConstraintsOutputFilename", base}});
    std::ifstream in(base + "_WU.json");
    CHECK(bool(in));
    std::stringstream text;
    text << in.rdbuf();
    reportWeightUpdatePlanInfo(wu2, graph, p, {{"planConstraints", text.str()}});
    CHECK(wu1.str() == wu2.str());
    std::remove((base + "_WU.json").c_str());
  }
  // weights of a fully connected layer rearranged for its backward pass
  {
    ConvParams fcBwd(HALF, HALF, 4, {1}, {1}, 96, 40, 2);   // backward pass: 96 = forward Co, 40 = forward Ci
    auto fcw = graph.addVariable(HALF, {2, 96, 40, 1}, "fcw");   // forward weights [G][Co][Ci][k]
    poplar::program::Sequence fcProg;
    auto t = fullyConnectedWeightTranspose(graph, fcw, fcBwd, fcProg, "fct");
    CHECK((t.shape() == std::vector<std::size_t>{2, 40, 96, 1}) && fcProg.steps().size() == 1);
    ConvParams twoD(HALF, HALF, 4, {2, 2}, {1, 1}, 96, 40, 2);
    CHECK((throwsAs<poputil::poplibs_error>([&] { fullyConnectedWeightTranspose(graph, fcw, twoD, fcProg); })));
  }
  // normalisation after a convolution: shapes, types, recorded steps, errors
  {
    poplar::program::Sequence np_;
    auto acts = createConvOutput(graph, p, "bnActs");
    auto st = normStatistics(graph, acts, 1e-3f, np_, true, false, FLOAT, "bn");
    CHECK(st.first.shape() == std::vector<std::size_t>{64} && st.second.elementType() == HALF);
    auto gb = createNormParams(graph, acts, "bn");
    CHECK(gb.first.numElements() == 64 && gb.second.numElements() == 64);
    CHECK(createNormGamma(graph, acts, FLOAT).elementType() == FLOAT);
    auto wht = normWhiten(graph, acts, st.first, st.second, np_, "bn");
    auto nrm = normalise(graph, wht, gb.first, gb.second, np_, "bn");
    CHECK(wht.shape() == acts.shape() && nrm.shape() == acts.shape());
    auto pg = normParamGradients(graph, wht, nrm, np_);
    CHECK(pg.first.numElements() == 64 && pg.second.elementType() == HALF);
    CHECK(normGradients(graph, nrm, gb.first, np_).shape() == acts.shape());
    CHECK(normStatisticsGradients(graph, wht, nrm, st.second, np_).shape() == acts.shape());
    const std::size_t before = np_.steps().size();
    // the distributed forms call the reduction callback with (mean, power) / the two deltas
    unsigned calls = 0, tensors = 0;
    DistributedNormReduceCallback cb = [&](poplar::Graph &, const std::vector<poplar::Tensor> &in,
                                           poplar::program::Sequence &, unsigned groupSize,
                                           const poplar::DebugContext &, const poplar::OptionFlags &) {
      ++calls;
      tensors += unsigned(in.size());
      CHECK(groupSize == 4);
      return in;
    };
    auto dst = distributedNormStatistics(graph, acts, 1e-3f, np_, false, cb, 128);
    CHECK(calls == 1 && tensors == 2 && dst.first.numElements() == 64);
    distributedNormStatistics(graph, acts, 1e-3f, np_, false, cb, 128, true);
    CHECK(calls == 3 && tensors == 4);   // stable: the mean, then the power
    distributedNormStatisticsGradients(graph, wht, nrm, st.second, np_, cb, 128);
    CHECK(calls == 4 && tensors == 6 && np_.steps().size() > before);
    CHECK((throwsAs<poputil::poplibs_error>([&] { distributedNormStatistics(graph, acts, 1e-3f, np_, false, cb, 100); })));
    CHECK((throwsAs<poputil::poplibs_error>([&] { normWhiten(graph, acts, st.first.slice(0, 8, 0), st.second, np_); })));
    auto q8 = graph.addVariable(QUARTER, {2, 8, 4, 4}, "q8");
    CHECK((throwsAs<poputil::poplibs_error>([&] { normStatistics(graph, q8, 1e-3f, np_, false); })));
  }
  // the full constructor does not validate; validate() does
  {
    CHECK(noThrow([] { ConvParams bad(HALF, HALF, 1, {4, 4}, {3}, 8, 8, 1); (void)bad; }));
    ConvParams bad(HALF, HALF, 1, {4, 4}, {3}, 8, 8, 1);
    CHECK((throwsAs<poputil::poplibs_error>([&] { bad.validate(); })));
  }
  // preplanning fills the cache
  PlanningCache fresh;
  const poplar::Target target = graph.getTarget();
  std::set<ConvPlanParams> convs{std::make_tuple(&target, p, &fwdOpts)};
  const poplar::OptionFlags mmOpts{{"fullyConnectedPass", "TRAINING_FWD"}};
  std::set<MatMulPlanParams> mms{
      std::make_tuple(&target, MatMulParams{HALF, HALF, {1, 512, 1024}, {1, 1024, 1024}}, &mmOpts)};
  preplan(convs, mms, fresh);
  CHECK(fresh.size() == 2);
}

static void testMatMulSurface() {
  poplar::Graph graph(poplar::Target::createGPUTarget(0));
  poplar::program::Sequence prog;
  auto a = createMatMulInputLHS(graph, HALF, {512, 1024}, {1024, 1024}, "a");
  auto b = createMatMulInputRHS(graph, HALF, {512, 1024}, {1024, 1024}, "b");
  CHECK((a.shape() == std::vector<std::size_t>{512, 1024}) && (b.shape() == std::vector<std::size_t>{1024, 1024}));
  CHECK(b.strides()[0] == 1);  // stored [n][k]
  auto c = matMul(graph, a, b, prog, FLOAT, "c", {{"partialsType", "float"}});
  CHECK((c.shape() == std::vector<std::size_t>{512, 1024}) && c.elementType() == FLOAT);
  CHECK(prog.steps().size() == 1);
  matMulAcc(graph, c, 0.5f, a, b, prog, "acc");
  CHECK((throwsAs<poputil::poplibs_error>([&] { matMul(graph, a, a, prog); })));
  CHECK((throwsAs<poputil::poplibs_error>([&] { matMul(graph, a.expand({0}), b, prog); })));
  auto q = graph.addVariable(QUARTER, {8, 16}, "q");
  CHECK((throwsAs<poputil::poplibs_error>(
      [&] { matMul(graph, q, graph.addVariable(QUARTER, {16, 8}, "q2"), prog, FLOAT); })));
  auto g = matMulGrouped(graph, graph.addVariable(HALF, {3, 8, 16}, "ga"),
                         graph.addVariable(HALF, {3, 16, 24}, "gb"), prog, HALF);
  CHECK((g.shape() == std::vector<std::size_t>{3, 8, 24}));
  CHECK((transposeGroupedMatrix(g).shape() == std::vector<std::size_t>{3, 24, 8}));
  std::ostringstream os;
  matMulReportPlan(os, graph, HALF, HALF, {8192, 8192}, {8192, 8192});
  CHECK(os.str().find("CTA tile (rows x cols)     128 x 256") != std::string::npos);
  const auto fcParams = fc::getMatMulPrePlanParameters({2, 16, 32, 64}, {}, HALF, false);
  CHECK(fcParams.size() == 3);
  CHECK((fcParams[1].first.aShape == std::vector<std::size_t>{2, 16, 64}));
  CHECK((fcParams[2].first.bShape == std::vector<std::size_t>{2, 16, 64}));
  CHECK(fc::getMatMulPrePlanParameters({1, 4, 8, 8}, {}, HALF, true).size() == 1);
}

static void testMultiConvAndBiasSurface() {
  poplar::Graph graph(poplar::Target::createGPUTarget(0));
  PlanningCache cache;
  ConvParams p1(HALF, 4, {14, 14}, {3, 3}, 64, 64, 1);
  p1.inputTransform.paddingLower = p1.inputTransform.paddingUpper = {1, 1};
  ConvParams p2(HALF, 4, {12, 12}, {1, 1}, 64, 128, 1);
  p2.outputTransform.stride = {2, 2};
  const std::vector<multiconv::CreateTensorArgs> create{{p1, {}, "a"}, {p2, {}, "b"}};
  std::vector<multiconv::ConvolutionArgs> args;
  for (unsigned i = 0; i != 2; ++i)
    args.push_back({multiconv::createInput(graph, create, i, {}, &cache),
                    multiconv::createWeights(graph, create, i, {}, &cache), create[i].params, {}});
  poplar::program::Sequence prog;
  auto outs = multiconv::convolution(graph, args, false, prog, "mc", {{"planType", "serial"}}, &cache);
  CHECK(outs.size() == 2);
  CHECK((outs[1].shape() == std::vector<std::size_t>{4, 128, 6, 6}));
  CHECK((throwsAs<poplar::invalid_option>(
      [&] { multiconv::convolution(graph, args, false, prog, "mc", {{"planType", "sideways"}}); })));
  CHECK((throwsAs<poplar::invalid_option>(
      [&] { multiconv::convolution(graph, args, false, prog, "mc", {{"noSuchOption", "1"}}); })));
  CHECK((throwsAs<poputil::poplibs_error>([&] { multiconv::createInput(graph, create, 2); })));
  // gradients of both layers; the strided one plans in forward terms
  std::vector<multiconv::CalculateWeightDeltasArgs> wu;
  for (unsigned i = 0; i != 2; ++i) wu.push_back({outs[i], args[i].inputs, args[i].params, {}});
  auto deltas = multiconv::calculateWeightDeltas(graph, wu, prog, "wu", {}, &cache);
  CHECK(deltas.size() == 2 && deltas[1].shape() == args[1].weights.shape());
  std::vector<multiconv::ConvWeightUpdateArgsScalar> upd;
  for (unsigned i = 0; i != 2; ++i)
    upd.push_back({outs[i], args[i].weights, args[i].inputs, -0.5f, args[i].params, {}});
  multiconv::convolutionWeightUpdate(graph, upd, prog, "upd", {}, &cache);
  // backward pass of the strided layer: transposed weights, input dilation in the parameters
  const ConvParams bwd = getGradientParams(p2);
  CHECK(bwd.inputTransform.dilation[0] == 2);
  auto dIn = convolution(graph, outs[1], args[1].weights, bwd, true, prog, "bwd", {}, &cache);
  CHECK(dIn.shape() == args[1].inputs.shape());
  // bias surface
  auto biases = createBiases(graph, outs[0], "biases");
  CHECK((biases.shape() == std::vector<std::size_t>{64}));
  addBias(graph, outs[0], biases, prog, "addBias");
  convolutionBiasUpdate(graph, outs[0], biases, -0.1f, {{"partialsType", "float"}}, prog, "biasUpdate");
  CHECK((throwsAs<poputil::poplibs_error>(
      [&] { convolutionBiasUpdate(graph, outs[1], biases, 1.f, {}, prog); })));
  CHECK((throwsAs<poplar::invalid_option>(
      [&] { convolutionBiasUpdate(graph, outs[0], biases, 1.f, {{"partialsType", "int"}}, prog); })));
}

int main() {
  testConvParamsJson();
  testValidation();
  testRanges();
  testCanonicalAndDerivedParams();
  testOptions();
  testTensorViews();
  testGraphConstructionWithoutDevice();
  testMatMulSurface();
  testMultiConvAndBiasSurface();
  if (failures) {
    std::printf("%d check(s) failed\n", failures);
    return 1;
  }
  std::printf("all host checks passed\n");
  return 0;
}
