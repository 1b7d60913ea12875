// Host-side size and index algebra of a flattened poplin::ConvParams
// (plb_conv_params).  Restates, for one spatial dimension at a time, what
// ConvParams::validate / getTransformedInputSize / getOutputSize
// (lib/poplin/ConvParams.cpp:172-266, 631-698) and poplin::getInputIndex
// (lib/poplin/ConvUtil.cpp:234-292) compute in the reference.
#pragma once

#include <cstdint>
#include <string>

#include "poplibs_b200.h"

namespace plb {

// Size after truncate -> dilate -> pad, or -1 if truncation exceeds the size.
long transformedSize(long size, long truncLo, long truncHi, long dilation, long padLo, long padHi);
long transformedInputSize(const plb_conv_params &p, unsigned dim);
long transformedKernelSize(const plb_conv_params &p, unsigned dim);
// Size of the stride-1 correlation before the output transform.
long untransformedOutputSize(const plb_conv_params &p, unsigned dim);
long outputSize(const plb_conv_params &p, unsigned dim);

// Empty string if valid, else the reference's error message.
std::string validate(const plb_conv_params &p);

// Input element read by (output element, kernel element) in one dimension, or
// -1 when that product is with padding, a dilation hole or a truncated element.
int inputIndex(const plb_conv_params &p, unsigned dim, unsigned outIndex, unsigned kernelIndex);

// Multiply-accumulates against real input elements.
uint64_t numberOfMacs(const plb_conv_params &p);

}  // namespace plb
