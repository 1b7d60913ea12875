// Index-range algebra of a convolution and the derived-parameter helpers, with
// the interface of the reference's include/poplin/ConvUtil.hpp:18-104.
#ifndef poplin_ConvUtil_hpp
#define poplin_ConvUtil_hpp

#include <utility>

#include "poplin/ConvParams.hpp"

namespace poplin {

unsigned getDilatedSize(unsigned size, unsigned dilation);

/// Input element multiplied by `kernelIndex` to produce `outputIndex` in
/// dimension `dim`, or ~0U if that product is with padding.
unsigned getInputIndex(unsigned dim, unsigned outputIndex, unsigned kernelIndex,
                       const ConvParams &params);
/// Kernel element multiplied by `inputIndex` to produce `outputIndex`, or ~0U.
unsigned getKernelIndex(unsigned dim, unsigned outputIndex, unsigned inputIndex,
                        const ConvParams &params);

std::pair<unsigned, unsigned> getOutputRangeForKernelIndex(unsigned dim,
                                                           std::pair<unsigned, unsigned> outputRange,
                                                           unsigned kernelIndex,
                                                           const ConvParams &params);
std::pair<unsigned, unsigned> getOutputRangeForInputIndex(unsigned dim,
                                                          std::pair<unsigned, unsigned> outputRange,
                                                          unsigned inputIndex,
                                                          const ConvParams &params);
std::pair<unsigned, unsigned> getOutputRangeForKernelRange(
    unsigned dim, std::pair<unsigned, unsigned> outputRange,
    std::pair<unsigned, unsigned> kernelIndexRange, const ConvParams &params);
std::pair<unsigned, unsigned> getOutputRangeForInputRange(unsigned dim,
                                                          std::pair<unsigned, unsigned> outputRange,
                                                          std::pair<unsigned, unsigned> inputRange,
                                                          const ConvParams &params);
std::pair<unsigned, unsigned> getInputRange(unsigned dim, std::pair<unsigned, unsigned> outputRange,
                                            unsigned kernelIndex, const ConvParams &params);
std::pair<unsigned, unsigned> getKernelRange(unsigned dim, std::pair<unsigned, unsigned> outputRange,
                                             unsigned inputIndex, const ConvParams &params);
std::pair<unsigned, unsigned> getInputRange(unsigned dim, std::pair<unsigned, unsigned> outputRange,
                                            std::pair<unsigned, unsigned> kernelIndexRange,
                                            const ConvParams &params);
std::pair<unsigned, unsigned> getKernelRange(unsigned dim, std::pair<unsigned, unsigned> outputRange,
                                             std::pair<unsigned, unsigned> inputRange,
                                             const ConvParams &params);

inline std::pair<unsigned, unsigned> getInputRange(unsigned dim, unsigned outputIndex,
                                                   std::pair<unsigned, unsigned> kernelIndexRange,
                                                   const ConvParams &params) {
  return getInputRange(dim, {outputIndex, outputIndex + 1}, kernelIndexRange, params);
}
inline std::pair<unsigned, unsigned> getInputRange(unsigned dim, unsigned outputIndex,
                                                   const ConvParams &params) {
  return getInputRange(dim, outputIndex, {0, unsigned(params.kernelShape[dim])}, params);
}
inline std::pair<unsigned, unsigned> getInputRange(unsigned dim,
                                                   std::pair<unsigned, unsigned> outputRange,
                                                   const ConvParams &params) {
  return getInputRange(dim, outputRange, {0, unsigned(params.kernelShape[dim])}, params);
}

/// Parameters of the convolution that maps output gradients to input
/// gradients, given weights transposed in the channel axes and flipped in the
/// spatial axes (lib/poplin/ConvUtil.cpp:728-795).
ConvParams getGradientParams(const ConvParams &params);
/// Parameters of the convolution whose result is the weight gradient
/// (batch and input channels swapped; lib/poplin/Convolution.cpp:3390-3434).
ConvParams getWeightUpdateParams(const ConvParams &fwdParams);

} // namespace poplin

#endif // poplin_ConvUtil_hpp
