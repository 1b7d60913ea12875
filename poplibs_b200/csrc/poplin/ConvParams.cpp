// poplin::ConvParams: construction, validation, sizes, canonical form, ordering,
// hashing, text and JSON IO (behaviour of lib/poplin/ConvParams.cpp:121-751).
#include "poplin/ConvParams.hpp"

#include <algorithm>
#include <functional>
#include <iostream>
#include <sstream>
#include <tuple>

#include "json.hpp"
#include "poplin/ConvUtil.hpp"
#include "poputil/exceptions.hpp"

namespace poplin {

using poputil::poplibs_error;

// ---- transforms -------------------------------------------------------------
ConvParams::InputTransform::InputTransform(std::size_t size)
    : InputTransform(std::vector<unsigned>(size, 0), std::vector<unsigned>(size, 0),
                     std::vector<unsigned>(size, 1), std::vector<unsigned>(size, 0),
                     std::vector<unsigned>(size, 0), std::vector<bool>(size, false)) {}

ConvParams::InputTransform::InputTransform(std::vector<unsigned> truncationLower_,
                                           std::vector<unsigned> truncationUpper_,
                                           std::vector<unsigned> dilation_,
                                           std::vector<unsigned> paddingLower_,
                                           std::vector<unsigned> paddingUpper_,
                                           std::vector<bool> flip_)
    : truncationLower(std::move(truncationLower_)), truncationUpper(std::move(truncationUpper_)),
      dilation(std::move(dilation_)), paddingLower(std::move(paddingLower_)),
      paddingUpper(std::move(paddingUpper_)), flip(std::move(flip_)) {}

ConvParams::OutputTransform::OutputTransform(std::size_t size)
    : OutputTransform(std::vector<unsigned>(size, 0), std::vector<unsigned>(size, 0),
                      std::vector<unsigned>(size, 1), std::vector<unsigned>(size, 0),
                      std::vector<unsigned>(size, 0)) {}

ConvParams::OutputTransform::OutputTransform(std::vector<unsigned> truncationLower_,
                                             std::vector<unsigned> truncationUpper_,
                                             std::vector<unsigned> stride_,
                                             std::vector<unsigned> paddingLower_,
                                             std::vector<unsigned> paddingUpper_)
    : truncationLower(std::move(truncationLower_)), truncationUpper(std::move(truncationUpper_)),
      stride(std::move(stride_)), paddingLower(std::move(paddingLower_)),
      paddingUpper(std::move(paddingUpper_)) {}

static auto tie(const ConvParams::InputTransform &t) {
  return std::tie(t.truncationLower, t.truncationUpper, t.dilation, t.paddingLower, t.paddingUpper,
                  t.flip);
}
static auto tie(const ConvParams::OutputTransform &t) {
  return std::tie(t.truncationLower, t.truncationUpper, t.stride, t.paddingLower, t.paddingUpper);
}
static auto tie(const ConvParams &p) {
  return std::tie(p.inputType, p.outputType, p.batchSize, p.inputFieldShape, p.kernelShape,
                  p.inputChannelsPerConvGroup, p.outputChannelsPerConvGroup, p.numConvGroups,
                  p.inputTransform, p.kernelTransform, p.outputTransform);
}

bool operator<(const ConvParams::InputTransform &a, const ConvParams::InputTransform &b) {
  return tie(a) < tie(b);
}
bool operator==(const ConvParams::InputTransform &a, const ConvParams::InputTransform &b) {
  return tie(a) == tie(b);
}
bool operator!=(const ConvParams::InputTransform &a, const ConvParams::InputTransform &b) {
  return !(a == b);
}
bool operator<(const ConvParams::OutputTransform &a, const ConvParams::OutputTransform &b) {
  return tie(a) < tie(b);
}
bool operator==(const ConvParams::OutputTransform &a, const ConvParams::OutputTransform &b) {
  return tie(a) == tie(b);
}
bool operator!=(const ConvParams::OutputTransform &a, const ConvParams::OutputTransform &b) {
  return !(a == b);
}
bool operator<(const ConvParams &a, const ConvParams &b) { return tie(a) < tie(b); }
bool operator==(const ConvParams &a, const ConvParams &b) { return tie(a) == tie(b); }
bool operator!=(const ConvParams &a, const ConvParams &b) { return !(a == b); }

// ---- construction --------------------------------------------------------------
ConvParams::ConvParams(poplar::Type inputType_, poplar::Type outputType_, std::size_t batchSize_,
                       std::vector<std::size_t> inputFieldShape_,
                       std::vector<std::size_t> kernelShape_, std::size_t inputChannels_,
                       std::size_t outputChannels_, std::size_t numConvGroups_,
                       InputTransform inputTransform_, InputTransform kernelTransform_,
                       OutputTransform outputTransform_)
    : inputType(inputType_), outputType(outputType_), batchSize(batchSize_),
      inputFieldShape(std::move(inputFieldShape_)), kernelShape(std::move(kernelShape_)),
      inputChannelsPerConvGroup(inputChannels_), outputChannelsPerConvGroup(outputChannels_),
      numConvGroups(numConvGroups_), inputTransform(std::move(inputTransform_)),
      kernelTransform(std::move(kernelTransform_)), outputTransform(std::move(outputTransform_)) {
  // not validated here, as in the reference (lib/poplin/ConvParams.cpp:152-170):
  // validate() is called by whatever consumes the parameters
}

ConvParams::ConvParams(poplar::Type inputType_, poplar::Type outputType_, std::size_t batchSize_,
                       std::vector<std::size_t> inputFieldShape_,
                       std::vector<std::size_t> kernelShape_, std::size_t inputChannels_,
                       std::size_t outputChannels_, std::size_t numConvGroups_)
    : inputType(inputType_), outputType(outputType_), batchSize(batchSize_),
      inputFieldShape(std::move(inputFieldShape_)), kernelShape(std::move(kernelShape_)),
      inputChannelsPerConvGroup(inputChannels_), outputChannelsPerConvGroup(outputChannels_),
      numConvGroups(numConvGroups_), inputTransform(inputFieldShape.size()),
      kernelTransform(inputFieldShape.size()), outputTransform(inputFieldShape.size()) {
  // not validated here: callers set the transforms afterwards
  // (tests/poplin/ConvUtilTest.cpp:14-32 builds a 3-wide input with a 5-wide kernel this way)
}

ConvParams::ConvParams(poplar::Type dataType, std::size_t batchSize_,
                       std::vector<std::size_t> inputFieldShape_,
                       std::vector<std::size_t> kernelShape_, std::size_t inputChannels_,
                       std::size_t outputChannels_, std::size_t numConvGroups_)
    : ConvParams(dataType, dataType, batchSize_, std::move(inputFieldShape_),
                 std::move(kernelShape_), inputChannels_, outputChannels_, numConvGroups_) {}

// ---- sizes ---------------------------------------------------------------------
unsigned getDilatedSize(unsigned size, unsigned dilation) {
  return size == 0 ? 0 : 1 + (size - 1) * dilation;
}

static unsigned transformed(std::size_t size, const ConvParams::InputTransform &t, unsigned dim) {
  const unsigned truncated = unsigned(size) - (t.truncationLower[dim] + t.truncationUpper[dim]);
  return t.paddingLower[dim] + getDilatedSize(truncated, t.dilation[dim]) + t.paddingUpper[dim];
}

unsigned ConvParams::getTruncatedInputSize(unsigned dim) const {
  return unsigned(inputFieldShape[dim]) -
         (inputTransform.truncationLower[dim] + inputTransform.truncationUpper[dim]);
}
unsigned ConvParams::getTruncatedKernelSize(unsigned dim) const {
  return unsigned(kernelShape[dim]) -
         (kernelTransform.truncationLower[dim] + kernelTransform.truncationUpper[dim]);
}
unsigned ConvParams::getTransformedInputSize(unsigned dim) const {
  return transformed(inputFieldShape[dim], inputTransform, dim);
}
unsigned ConvParams::getTransformedKernelSize(unsigned dim) const {
  return transformed(kernelShape[dim], kernelTransform, dim);
}
std::size_t ConvParams::getUntransformedOutputSize(unsigned dim) const {
  const unsigned in = getTransformedInputSize(dim), k = getTransformedKernelSize(dim);
  return in < k ? 0 : in - k + 1;  // callers validate() first; this keeps it total
}
std::size_t ConvParams::getOutputSize(unsigned dim) const {
  const std::size_t conv = getUntransformedOutputSize(dim);
  const std::size_t truncated =
      conv - (outputTransform.truncationLower[dim] + outputTransform.truncationUpper[dim]);
  const std::size_t s = outputTransform.stride[dim];
  return outputTransform.paddingLower[dim] + (truncated + s - 1) / s +
         outputTransform.paddingUpper[dim];
}
std::vector<std::size_t> ConvParams::getOutputFieldShape() const {
  std::vector<std::size_t> shape;
  for (unsigned d = 0; d != getNumFieldDims(); ++d) shape.push_back(getOutputSize(d));
  return shape;
}

// ---- validation (messages as lib/poplin/ConvParams.cpp:172-266) -----------------------
void ConvParams::validate() const {
  const auto nd = inputFieldShape.size();
  auto s = [](std::size_t v) { return std::to_string(v); };
  if (kernelShape.size() != nd)
    throw poplibs_error("Number of kernel field dimensions (" + s(kernelShape.size()) +
                        ") does not match the number of input field dimensions (" + s(nd) + ")");
  for (unsigned st : outputTransform.stride)
    if (st == 0) throw poplibs_error("Stride must be non zero");
  for (unsigned d : inputTransform.dilation)
    if (d == 0)
      throw poplibs_error("Input dilation must be non zero. Dilation = 1 results in no dilation");
  for (unsigned d : kernelTransform.dilation)
    if (d == 0)
      throw poplibs_error("Kernel dilation must be non zero. Dilation = 1 results in no dilation");
  const std::pair<std::size_t, const char *> sizes[] = {
      {inputTransform.truncationLower.size(), "input truncation (lower)"},
      {inputTransform.truncationUpper.size(), "input truncation (upper)"},
      {inputTransform.dilation.size(), "input dilation"},
      {inputTransform.paddingLower.size(), "input padding (lower)"},
      {inputTransform.paddingUpper.size(), "input padding (upper)"},
      {inputTransform.flip.size(), "input flip"},
      {kernelTransform.truncationLower.size(), "kernel truncation (lower)"},
      {kernelTransform.truncationUpper.size(), "kernel truncation (upper)"},
      {kernelTransform.dilation.size(), "kernel dilation"},
      {kernelTransform.paddingLower.size(), "kernel padding (lower)"},
      {kernelTransform.paddingUpper.size(), "kernel padding (upper)"},
      {kernelTransform.flip.size(), "kernel flip"},
      {outputTransform.truncationLower.size(), "output truncation (lower)"},
      {outputTransform.truncationUpper.size(), "output truncation (upper)"},
      {outputTransform.stride.size(), "stride"},
      {outputTransform.paddingLower.size(), "output padding (lower)"},
      {outputTransform.paddingUpper.size(), "output padding (upper)"},
  };
  for (const auto &e : sizes)
    if (e.first != nd)
      throw poplibs_error(std::string("Number of ") + e.second + " dimensions (" + s(e.first) +
                          ") does not match the number of field dimensions (" + s(nd) + ")");
  for (unsigned dim = 0; dim != nd; ++dim) {
    const std::size_t inTrunc =
        std::size_t(inputTransform.truncationLower[dim]) + inputTransform.truncationUpper[dim];
    if (inTrunc > inputFieldShape[dim])
      throw poplibs_error("Truncation for dimension " + s(dim) + " (" + s(inTrunc) +
                          ") truncates by more than the size of the field (" +
                          s(inputFieldShape[dim]) + ")");
    const std::size_t kTrunc =
        std::size_t(kernelTransform.truncationLower[dim]) + kernelTransform.truncationUpper[dim];
    if (kTrunc > kernelShape[dim])
      throw poplibs_error("Truncation for dimension " + s(dim) + " (" + s(kTrunc) +
                          ") truncates by more than the size of the kernel (" +
                          s(kernelShape[dim]) + ")");
    const auto in = getTransformedInputSize(dim), k = getTransformedKernelSize(dim);
    if (k == 0) throw poplibs_error("Transformed kernel for dimension " + s(dim) + " has zero size");
    if (in < k)
      throw poplibs_error("Transformed input size for dimension " + s(dim) + " (" + s(in) +
                          ") is less than the transformed kernel size (" + s(k) + ")");
    const std::size_t conv = in - k + 1;
    const std::size_t outTrunc =
        std::size_t(outputTransform.truncationLower[dim]) + outputTransform.truncationUpper[dim];
    if (outTrunc > conv)
      throw poplibs_error("Output truncation for dimension " + s(dim) + " (" + s(outTrunc) +
                          ") truncates by more than the size of the convolution output (" +
                          s(conv) + ")");
  }
}

// ---- canonical form -------------------------------------------------------------
// Parameters of a convolution that produces an all-zero result of the same
// shape (lib/poplin/ConvParams.cpp: getZeroConv).
static ConvParams zeroConv(const ConvParams &p) {
  const auto nd = p.getNumFieldDims();
  std::vector<unsigned> outPad(nd);
  for (unsigned d = 0; d != nd; ++d) outPad[d] = unsigned(p.getOutputSize(d));
  ConvParams z;
  z.inputType = p.inputType;
  z.outputType = p.outputType;
  z.batchSize = p.batchSize;
  z.inputFieldShape = std::vector<std::size_t>(nd, 0);
  z.kernelShape = std::vector<std::size_t>(nd, 0);
  z.inputChannelsPerConvGroup = 0;
  z.outputChannelsPerConvGroup = p.outputChannelsPerConvGroup;
  z.numConvGroups = p.numConvGroups;
  z.inputTransform = ConvParams::InputTransform(nd);
  z.kernelTransform = ConvParams::InputTransform(nd);
  // a zero-sized field convolved with a zero-sized kernel gives one element,
  // which is truncated away; the whole output is padding
  z.outputTransform = ConvParams::OutputTransform(std::vector<unsigned>(nd, 0),
                                                  std::vector<unsigned>(nd, 1),
                                                  std::vector<unsigned>(nd, 1), outPad,
                                                  std::vector<unsigned>(nd, 0));
  return z;
}

ConvParams ConvParams::canonicalize() const {
  validate();
  ConvParams q = *this;
  const auto nd = getNumFieldDims();
  for (unsigned dim = 0; dim != nd; ++dim) {
    const unsigned outSize = unsigned(q.getOutputSize(dim));
    auto &inTruncLo = q.inputTransform.truncationLower[dim];
    auto &inTruncHi = q.inputTransform.truncationUpper[dim];
    auto &inPadLo = q.inputTransform.paddingLower[dim];
    auto &inPadHi = q.inputTransform.paddingUpper[dim];
    auto &kTruncLo = q.kernelTransform.truncationLower[dim];
    auto &kTruncHi = q.kernelTransform.truncationUpper[dim];
    auto &kPadLo = q.kernelTransform.paddingLower[dim];
    auto &kPadHi = q.kernelTransform.paddingUpper[dim];
    auto &outTruncLo = q.outputTransform.truncationLower[dim];
    auto &outTruncHi = q.outputTransform.truncationUpper[dim];
    auto &outPadLo = q.outputTransform.paddingLower[dim];
    auto &outPadHi = q.outputTransform.paddingUpper[dim];
    auto &stride = q.outputTransform.stride[dim];

    // 1. outputs that no (input, kernel) pair reaches are zeros: express them
    //    as output padding
    const auto nonZero =
        getOutputRangeForKernelRange(dim, {0, outSize}, {0, unsigned(q.kernelShape[dim])}, q);
    if (nonZero.first == nonZero.second) return zeroConv(q);
    const unsigned zerosLo = nonZero.first, zerosHi = outSize - nonZero.second;
    if (zerosLo > outPadLo) {
      outTruncLo += (zerosLo - outPadLo) * stride;
      outPadLo = zerosLo;
    }
    if (zerosHi > outPadHi) {
      outTruncHi += (zerosHi - outPadHi) * stride;
      outPadHi = zerosHi;
    }
    // 2. drop the tail the stride skips; a single output needs no stride
    unsigned truncatedConv = unsigned(q.getUntransformedOutputSize(dim)) - (outTruncLo + outTruncHi);
    const unsigned ignored = (truncatedConv - 1) % stride;
    outTruncHi += ignored;
    truncatedConv -= ignored;
    if (truncatedConv == 1) stride = 1;
    // 3. input elements never read become input truncation
    const auto inUsed = getInputRange(dim, {0, outSize}, {0, unsigned(q.kernelShape[dim])}, q);
    const unsigned inIgnoredLo = inUsed.first;
    const unsigned inIgnoredHi = unsigned(q.getInputSize(dim)) - inUsed.second;
    if (inIgnoredLo > inTruncLo) {
      inPadLo += (inIgnoredLo - inTruncLo) * q.inputTransform.dilation[dim];
      inTruncLo = inIgnoredLo;
    }
    if (inIgnoredHi > inTruncHi) {
      inPadHi += (inIgnoredHi - inTruncHi) * q.inputTransform.dilation[dim];
      inTruncHi = inIgnoredHi;
    }
    // 4. kernel elements never used become kernel truncation
    const auto kUsed = getKernelRange(dim, {0, outSize}, {0, unsigned(q.getInputSize(dim))}, q);
    const unsigned kIgnoredLo = kUsed.first;
    const unsigned kIgnoredHi = unsigned(q.kernelShape[dim]) - kUsed.second;
    if (kIgnoredLo > kTruncLo) {
      kPadLo += (kIgnoredLo - kTruncLo) * q.kernelTransform.dilation[dim];
      kTruncLo = kIgnoredLo;
    }
    if (kIgnoredHi > kTruncHi) {
      kPadHi += (kIgnoredHi - kTruncHi) * q.kernelTransform.dilation[dim];
      kTruncHi = kIgnoredHi;
    }
    // 5. padding on both the input and the kernel cancels (seen after flipping)
    const bool kFlip = q.kernelTransform.flip[dim], iFlip = q.inputTransform.flip[dim];
    auto &fkPadLo = kFlip ? kPadHi : kPadLo;
    auto &fkPadHi = kFlip ? kPadLo : kPadHi;
    auto &fiPadLo = iFlip ? inPadHi : inPadLo;
    auto &fiPadHi = iFlip ? inPadLo : inPadHi;
    unsigned excess = std::min({fiPadLo, fkPadLo, q.getTransformedKernelSize(dim) - 1});
    fiPadLo -= excess;
    fkPadLo -= excess;
    excess = std::min({fiPadHi, fkPadHi, q.getTransformedKernelSize(dim) - 1});
    fiPadHi -= excess;
    fkPadHi -= excess;
    // 6. input padding that only feeds truncated outputs cancels too
    excess = std::min({fiPadLo, outTruncLo, unsigned(q.getUntransformedOutputSize(dim) - 1)});
    fiPadLo -= excess;
    outTruncLo -= excess;
    excess = std::min({fiPadHi, outTruncHi, unsigned(q.getUntransformedOutputSize(dim) - 1)});
    fiPadHi -= excess;
    outTruncHi -= excess;
    // 7. a single surviving element needs neither dilation nor flipping
    if (q.inputFieldShape[dim] <= std::size_t(inTruncLo) + 1 + inTruncHi) {
      q.inputTransform.dilation[dim] = 1;
      if (q.inputTransform.flip[dim]) {
        q.inputTransform.flip[dim] = false;
        std::swap(inPadLo, inPadHi);
      }
    }
    if (q.kernelShape[dim] <= std::size_t(kTruncLo) + 1 + kTruncHi) {
      q.kernelTransform.dilation[dim] = 1;
      if (q.kernelTransform.flip[dim]) {
        q.kernelTransform.flip[dim] = false;
        std::swap(kPadLo, kPadHi);
      }
    }
  }
  return q;
}

// ---- text form (layout of lib/poplin/ConvParams.cpp:292-366) ----------------------------
template <class C> static void printList(std::ostream &os, const C &c) {
  os << "{";
  bool first = true;
  for (const auto &e : c) {
    os << (first ? "" : ",") << e;
    first = false;
  }
  os << "}";
}

std::ostream &operator<<(std::ostream &os, const ConvParams &p) {
  auto line = [&](const char *name, const auto &v) {
    os << "        " << name;
    for (std::size_t i = std::char_traits<char>::length(name); i < 27; ++i) os << ' ';
    printList(os, v);
    os << "\n";
  };
  os << "\n  Params:\n";
  os << "        inputType                  " << p.inputType << "\n";
  os << "        outputType                 " << p.outputType << "\n";
  os << "        batchSize                  " << p.batchSize << "\n";
  os << "        numConvGroups              " << p.numConvGroups << "\n";
  line("inputFieldShape", p.inputFieldShape);
  line("kernelShape", p.kernelShape);
  os << "        inputChannelsPerConvGroup  " << p.inputChannelsPerConvGroup << "\n";
  os << "        outputChannelsPerConvGroup " << p.outputChannelsPerConvGroup << "\n";
  line("inputTruncationLower", p.inputTransform.truncationLower);
  line("inputTruncationUpper", p.inputTransform.truncationUpper);
  line("inputDilation", p.inputTransform.dilation);
  line("inputPaddingLower", p.inputTransform.paddingLower);
  line("inputPaddingUpper", p.inputTransform.paddingUpper);
  line("flipInput", p.inputTransform.flip);
  line("kernelTruncationLower", p.kernelTransform.truncationLower);
  line("kernelTruncationUpper", p.kernelTransform.truncationUpper);
  line("kernelDilation", p.kernelTransform.dilation);
  line("kernelPaddingLower", p.kernelTransform.paddingLower);
  line("kernelPaddingUpper", p.kernelTransform.paddingUpper);
  line("flipKernel", p.kernelTransform.flip);
  line("outputTruncationLower", p.outputTransform.truncationLower);
  line("outputTruncationUpper", p.outputTransform.truncationUpper);
  line("stride", p.outputTransform.stride);
  line("outputPaddingLower", p.outputTransform.paddingLower);
  line("outputPaddingUpper", p.outputTransform.paddingUpper);
  line("outputFieldShape", p.getOutputFieldShape());
  return os;
}

// ---- JSON form (keys of lib/poplin/ConvParams.cpp:373-458) --------------------------------
template <class T> static T scalarFrom(const json::Value &v) {
  std::istringstream iss(v.text);
  T out{};
  if (v.text == "true" || v.text == "false")
    out = T(v.text == "true");
  else
    iss >> out;
  return out;
}

template <class Vec> static void readVector(const json::Value &node, const char *name, Vec &field) {
  if (const json::Value *child = node.find(name)) {
    Vec values;
    for (const auto &item : child->items)
      values.push_back(scalarFrom<typename Vec::value_type>(item.second));
    field = std::move(values);
  }
}

static poplar::Type typeFromJson(const std::string &s) {
  if (s == "half") return poplar::HALF;
  if (s == "float") return poplar::FLOAT;
  if (s == "quarter") return poplar::QUARTER;
  throw poplibs_error("Unknown data type '" + s + "' in convolution parameters");
}

std::istream &operator>>(std::istream &is, ConvParams &p) {
  std::stringstream buffer;
  buffer << is.rdbuf();
  const json::Value root = json::parse(buffer.str());
  if (const auto *v = root.find("dataType")) p.inputType = p.outputType = typeFromJson(v->text);
  if (const auto *v = root.find("inputType")) p.inputType = typeFromJson(v->text);
  if (const auto *v = root.find("outputType")) p.outputType = typeFromJson(v->text);
  if (const auto *v = root.find("batchSize")) p.batchSize = scalarFrom<std::size_t>(*v);
  if (const auto *v = root.find("numConvGroups")) p.numConvGroups = scalarFrom<std::size_t>(*v);
  if (const auto *v = root.find("inputChannelsPerConvGroup"))
    p.inputChannelsPerConvGroup = scalarFrom<std::size_t>(*v);
  if (const auto *v = root.find("outputChannelsPerConvGroup"))
    p.outputChannelsPerConvGroup = scalarFrom<std::size_t>(*v);
  readVector(root, "inputFieldShape", p.inputFieldShape);
  readVector(root, "kernelShape", p.kernelShape);
  if (p.inputFieldShape.size() != p.kernelShape.size())
    throw poplibs_error("Input and kernel must have the same number of dimensions");
  const auto readInputTransform = [&](const char *key, ConvParams::InputTransform &t) {
    t = ConvParams::InputTransform(p.inputFieldShape.size());
    if (const json::Value *node = root.find(key)) {
      readVector(*node, "truncationLower", t.truncationLower);
      readVector(*node, "truncationUpper", t.truncationUpper);
      readVector(*node, "dilation", t.dilation);
      readVector(*node, "paddingLower", t.paddingLower);
      readVector(*node, "paddingUpper", t.paddingUpper);
      readVector(*node, "flip", t.flip);
    }
  };
  readInputTransform("inputTransform", p.inputTransform);
  readInputTransform("kernelTransform", p.kernelTransform);
  p.outputTransform = ConvParams::OutputTransform(p.inputFieldShape.size());
  if (const json::Value *node = root.find("outputTransform")) {
    readVector(*node, "truncationLower", p.outputTransform.truncationLower);
    readVector(*node, "truncationUpper", p.outputTransform.truncationUpper);
    readVector(*node, "stride", p.outputTransform.stride);
    readVector(*node, "paddingLower", p.outputTransform.paddingLower);
    readVector(*node, "paddingUpper", p.outputTransform.paddingUpper);
  }
  return is;
}

// ---- hashing -------------------------------------------------------------------
static void mix(std::size_t &seed, std::size_t v) {
  seed ^= v + 0x9e3779b97f4a7c15ull + (seed << 6) + (seed >> 2);
}
template <class C> static void mixRange(std::size_t &seed, const C &c) {
  mix(seed, c.size());
  for (const auto &e : c) mix(seed, std::hash<std::size_t>()(std::size_t(e)));
}

std::size_t hash_value(const ConvParams::InputTransform &it) {
  return std::hash<ConvParams::InputTransform>()(it);
}
std::size_t hash_value(const ConvParams::OutputTransform &ot) {
  return std::hash<ConvParams::OutputTransform>()(ot);
}

}  // namespace poplin

namespace std {
std::size_t hash<poplin::ConvParams::InputTransform>::operator()(
    const poplin::ConvParams::InputTransform &t) const {
  std::size_t seed = 0;
  poplin::mixRange(seed, t.truncationLower);
  poplin::mixRange(seed, t.truncationUpper);
  poplin::mixRange(seed, t.dilation);
  poplin::mixRange(seed, t.paddingLower);
  poplin::mixRange(seed, t.paddingUpper);
  poplin::mixRange(seed, t.flip);
  return seed;
}
std::size_t hash<poplin::ConvParams::OutputTransform>::operator()(
    const poplin::ConvParams::OutputTransform &t) const {
  std::size_t seed = 0;
  poplin::mixRange(seed, t.truncationLower);
  poplin::mixRange(seed, t.truncationUpper);
  poplin::mixRange(seed, t.stride);
  poplin::mixRange(seed, t.paddingLower);
  poplin::mixRange(seed, t.paddingUpper);
  return seed;
}
std::size_t hash<poplin::ConvParams>::operator()(const poplin::ConvParams &p) const {
  std::size_t seed = 0;
  poplin::mix(seed, std::hash<std::string>()(p.inputType.toString()));
  poplin::mix(seed, std::hash<std::string>()(p.outputType.toString()));
  poplin::mix(seed, p.batchSize);
  poplin::mixRange(seed, p.inputFieldShape);
  poplin::mixRange(seed, p.kernelShape);
  poplin::mix(seed, p.inputChannelsPerConvGroup);
  poplin::mix(seed, p.outputChannelsPerConvGroup);
  poplin::mix(seed, p.numConvGroups);
  poplin::mix(seed, std::hash<poplin::ConvParams::InputTransform>()(p.inputTransform));
  poplin::mix(seed, std::hash<poplin::ConvParams::InputTransform>()(p.kernelTransform));
  poplin::mix(seed, std::hash<poplin::ConvParams::OutputTransform>()(p.outputTransform));
  return seed;
}
}  // namespace std
