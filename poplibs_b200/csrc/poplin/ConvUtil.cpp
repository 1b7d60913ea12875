// Range algebra over one spatial dimension and the derived parameter sets of
// the backward and weight-update passes (lib/poplin/ConvUtil.cpp:234-795,
// lib/poplin/Convolution.cpp:3390-3434).
//
// Every range query reduces to the relation
//     input = getInputIndex(dim, output, kernel)      (or "none")
// which the C ABI evaluates; ranges are the tight [first, last+1) interval of
// the qualifying indices, (0, 0) when there are none.
#include "poplin/ConvUtil.hpp"

#include <algorithm>

#include "internal.hpp"
#include "poputil/exceptions.hpp"

namespace poplin {

namespace internal {

plb_conv_params toPlb(const ConvParams &p) {
  const auto nd = p.getNumFieldDims();
  if (nd < 1 || nd > PLB_MAX_FIELD_DIMS)
    throw poputil::poplibs_error("convolutions with " + std::to_string(nd) +
                                 " field dimensions are not supported (1 to 3)");
  auto dtype = [](const poplar::Type &t) {
    if (t == poplar::HALF) return int32_t(PLB_HALF);
    if (t == poplar::FLOAT) return int32_t(PLB_FLOAT);
    if (t == poplar::QUARTER) return int32_t(PLB_QUARTER);
    throw poputil::poplibs_error("Unsupported element type " + t.toString());
  };
  plb_conv_params q{};
  q.input_type = dtype(p.inputType);
  q.output_type = dtype(p.outputType);
  q.num_field_dims = uint32_t(nd);
  q.batch = uint32_t(p.batchSize);
  q.groups = uint32_t(p.numConvGroups);
  q.in_chans_per_group = uint32_t(p.inputChannelsPerConvGroup);
  q.out_chans_per_group = uint32_t(p.outputChannelsPerConvGroup);
  for (unsigned d = 0; d != nd; ++d) {
    q.field[d] = uint32_t(p.inputFieldShape[d]);
    q.kernel[d] = uint32_t(p.kernelShape[d]);
    q.in_trunc_lo[d] = p.inputTransform.truncationLower[d];
    q.in_trunc_hi[d] = p.inputTransform.truncationUpper[d];
    q.in_dilation[d] = p.inputTransform.dilation[d];
    q.in_pad_lo[d] = p.inputTransform.paddingLower[d];
    q.in_pad_hi[d] = p.inputTransform.paddingUpper[d];
    q.in_flip[d] = p.inputTransform.flip[d];
    q.k_trunc_lo[d] = p.kernelTransform.truncationLower[d];
    q.k_trunc_hi[d] = p.kernelTransform.truncationUpper[d];
    q.k_dilation[d] = p.kernelTransform.dilation[d];
    q.k_pad_lo[d] = p.kernelTransform.paddingLower[d];
    q.k_pad_hi[d] = p.kernelTransform.paddingUpper[d];
    q.k_flip[d] = p.kernelTransform.flip[d];
    q.out_trunc_lo[d] = p.outputTransform.truncationLower[d];
    q.out_trunc_hi[d] = p.outputTransform.truncationUpper[d];
    q.stride[d] = p.outputTransform.stride[d];
    q.out_pad_lo[d] = p.outputTransform.paddingLower[d];
    q.out_pad_hi[d] = p.outputTransform.paddingUpper[d];
  }
  return q;
}

}  // namespace internal

namespace {

// One dimension's relation, tabulated once per query.
struct DimRelation {
  unsigned outSize, kSize, inSize;
  plb_conv_params flat;
  unsigned dim;
  DimRelation(unsigned d, const ConvParams &p) : flat(internal::toPlb(p)), dim(d) {
    outSize = unsigned(p.getOutputSize(d));
    kSize = unsigned(p.kernelShape[d]);
    inSize = unsigned(p.inputFieldShape[d]);
  }
  int input(unsigned out, unsigned k) const { return plb_conv_input_index(&flat, dim, out, k); }
};

struct Tight {
  unsigned lo = ~0u, hi = 0;
  void add(unsigned v) {
    lo = std::min(lo, v);
    hi = std::max(hi, v + 1);
  }
  std::pair<unsigned, unsigned> get() const { return lo == ~0u ? std::make_pair(0u, 0u) : std::make_pair(lo, hi); }
};

}  // namespace

unsigned getInputIndex(unsigned dim, unsigned outputIndex, unsigned kernelIndex,
                       const ConvParams &params) {
  const DimRelation r(dim, params);
  const int i = r.input(outputIndex, kernelIndex);
  return i < 0 ? ~0u : unsigned(i);
}

unsigned getKernelIndex(unsigned dim, unsigned outputIndex, unsigned inputIndex,
                        const ConvParams &params) {
  const DimRelation r(dim, params);
  for (unsigned k = 0; k != r.kSize; ++k)
    if (r.input(outputIndex, k) == int(inputIndex)) return k;
  return ~0u;
}

std::pair<unsigned, unsigned> getOutputRangeForKernelRange(unsigned dim,
                                                           std::pair<unsigned, unsigned> outputRange,
                                                           std::pair<unsigned, unsigned> kernelRange,
                                                           const ConvParams &params) {
  const DimRelation r(dim, params);
  Tight t;
  for (unsigned o = outputRange.first; o < outputRange.second; ++o)
    for (unsigned k = kernelRange.first; k < kernelRange.second; ++k)
      if (r.input(o, k) >= 0) {
        t.add(o);
        break;
      }
  return t.get();
}

std::pair<unsigned, unsigned> getOutputRangeForKernelIndex(unsigned dim,
                                                           std::pair<unsigned, unsigned> outputRange,
                                                           unsigned kernelIndex,
                                                           const ConvParams &params) {
  return getOutputRangeForKernelRange(dim, outputRange, {kernelIndex, kernelIndex + 1}, params);
}

std::pair<unsigned, unsigned> getOutputRangeForInputRange(unsigned dim,
                                                          std::pair<unsigned, unsigned> outputRange,
                                                          std::pair<unsigned, unsigned> inputRange,
                                                          const ConvParams &params) {
  const DimRelation r(dim, params);
  Tight t;
  for (unsigned o = outputRange.first; o < outputRange.second; ++o)
    for (unsigned k = 0; k != r.kSize; ++k) {
      const int i = r.input(o, k);
      if (i >= int(inputRange.first) && i < int(inputRange.second)) {
        t.add(o);
        break;
      }
    }
  return t.get();
}

std::pair<unsigned, unsigned> getOutputRangeForInputIndex(unsigned dim,
                                                          std::pair<unsigned, unsigned> outputRange,
                                                          unsigned inputIndex,
                                                          const ConvParams &params) {
  return getOutputRangeForInputRange(dim, outputRange, {inputIndex, inputIndex + 1}, params);
}

std::pair<unsigned, unsigned> getInputRange(unsigned dim, std::pair<unsigned, unsigned> outputRange,
                                            std::pair<unsigned, unsigned> kernelRange,
                                            const ConvParams &params) {
  const DimRelation r(dim, params);
  Tight t;
  for (unsigned o = outputRange.first; o < outputRange.second; ++o)
    for (unsigned k = kernelRange.first; k < kernelRange.second; ++k) {
      const int i = r.input(o, k);
      if (i >= 0) t.add(unsigned(i));
    }
  return t.get();
}

std::pair<unsigned, unsigned> getInputRange(unsigned dim, std::pair<unsigned, unsigned> outputRange,
                                            unsigned kernelIndex, const ConvParams &params) {
  return getInputRange(dim, outputRange, {kernelIndex, kernelIndex + 1}, params);
}

std::pair<unsigned, unsigned> getKernelRange(unsigned dim, std::pair<unsigned, unsigned> outputRange,
                                             std::pair<unsigned, unsigned> inputRange,
                                             const ConvParams &params) {
  const DimRelation r(dim, params);
  Tight t;
  for (unsigned o = outputRange.first; o < outputRange.second; ++o)
    for (unsigned k = 0; k != r.kSize; ++k) {
      const int i = r.input(o, k);
      if (i >= int(inputRange.first) && i < int(inputRange.second)) t.add(k);
    }
  return t.get();
}

std::pair<unsigned, unsigned> getKernelRange(unsigned dim, std::pair<unsigned, unsigned> outputRange,
                                             unsigned inputIndex, const ConvParams &params) {
  return getKernelRange(dim, outputRange, {inputIndex, inputIndex + 1}, params);
}

// The backward pass runs the forward transforms in reverse: what the forward
// pass did to its output (truncate, stride, pad) the backward pass undoes on its
// input (pad, dilate, truncate) and vice versa; the "valid" correlation becomes
// a "full" one, i.e. (transformed kernel size - 1) of extra input padding; the
// kernel is consumed back to front, so its lower / upper truncation and padding
// trade places.  A flipped forward input shows up as a flipped backward output,
// which is the same as flipping both backward operands.
ConvParams getGradientParams(const ConvParams &params) {
  const ConvParams fwd = params.canonicalize();
  const auto nd = fwd.getNumFieldDims();
  auto padLo = fwd.outputTransform.truncationLower;
  auto padHi = fwd.outputTransform.truncationUpper;
  for (unsigned d = 0; d != nd; ++d) {
    const unsigned k = fwd.getTransformedKernelSize(d);
    padLo[d] += k - 1;
    padHi[d] += k - 1;
  }
  std::vector<bool> flipInput(nd, false);
  auto flipKernel = fwd.kernelTransform.flip;
  for (unsigned d = 0; d != nd; ++d)
    if (fwd.inputTransform.flip[d]) {
      flipKernel[d] = !flipKernel[d];
      flipInput[d] = true;
    }
  const ConvParams::InputTransform in{fwd.outputTransform.paddingLower,
                                      fwd.outputTransform.paddingUpper,
                                      fwd.outputTransform.stride,
                                      padLo,
                                      padHi,
                                      flipInput};
  const ConvParams::InputTransform kernel{fwd.kernelTransform.truncationUpper,
                                          fwd.kernelTransform.truncationLower,
                                          fwd.kernelTransform.dilation,
                                          fwd.kernelTransform.paddingUpper,
                                          fwd.kernelTransform.paddingLower,
                                          flipKernel};
  const ConvParams::OutputTransform out{fwd.inputTransform.paddingLower,
                                        fwd.inputTransform.paddingUpper,
                                        fwd.inputTransform.dilation,
                                        fwd.inputTransform.truncationLower,
                                        fwd.inputTransform.truncationUpper};
  const ConvParams bwd(fwd.inputType, fwd.outputType, fwd.batchSize, fwd.getOutputFieldShape(),
                       fwd.kernelShape, fwd.getNumOutputChansPerConvGroup(),
                       fwd.getNumInputChansPerConvGroup(), fwd.getNumConvGroups(), in, kernel, out);
  return bwd.canonicalize();
}

// The weight gradient is itself a convolution: the activations keep their
// transform, the output gradients act as the kernel (so the forward output
// transform becomes the kernel transform, read backwards) and the forward
// kernel transform, read backwards, becomes the output transform.  Batch and
// input channels trade places: the reduction runs over the batch.
ConvParams getWeightUpdateParams(const ConvParams &fwdParams) {
  const ConvParams fwd = fwdParams.canonicalize();
  const auto nd = fwd.getNumFieldDims();
  auto flipInput = fwd.inputTransform.flip;
  std::vector<bool> flipKernel(nd, false);
  for (unsigned d = 0; d != nd; ++d)
    if (fwd.kernelTransform.flip[d]) {
      flipInput[d] = !flipInput[d];
      flipKernel[d] = true;
    }
  auto in = fwd.inputTransform;
  in.flip = flipInput;
  const ConvParams::InputTransform kernel{fwd.outputTransform.paddingLower,
                                          fwd.outputTransform.paddingUpper,
                                          fwd.outputTransform.stride,
                                          fwd.outputTransform.truncationLower,
                                          fwd.outputTransform.truncationUpper,
                                          flipKernel};
  const ConvParams::OutputTransform out{fwd.kernelTransform.paddingLower,
                                        fwd.kernelTransform.paddingUpper,
                                        fwd.kernelTransform.dilation,
                                        fwd.kernelTransform.truncationLower,
                                        fwd.kernelTransform.truncationUpper};
  const ConvParams wu(fwd.inputType, fwd.outputType, fwd.getNumInputChansPerConvGroup(),
                      fwd.inputFieldShape, fwd.getOutputFieldShape(), fwd.getBatchSize(),
                      fwd.getNumOutputChansPerConvGroup(), fwd.numConvGroups, in, kernel, out);
  return wu.canonicalize();
}

}  // namespace poplin
