#include "conv_geometry.h"

namespace plb {

static long dilatedSize(long size, long dilation) {
  return size == 0 ? 0 : 1 + (size - 1) * dilation;
}

long transformedSize(long size, long truncLo, long truncHi, long dilation, long padLo,
                     long padHi) {
  const long truncated = size - (truncLo + truncHi);
  if (truncated < 0) return -1;
  return padLo + dilatedSize(truncated, dilation) + padHi;
}

long transformedInputSize(const plb_conv_params &p, unsigned d) {
  return transformedSize(p.field[d], p.in_trunc_lo[d], p.in_trunc_hi[d], p.in_dilation[d],
                         p.in_pad_lo[d], p.in_pad_hi[d]);
}

long transformedKernelSize(const plb_conv_params &p, unsigned d) {
  return transformedSize(p.kernel[d], p.k_trunc_lo[d], p.k_trunc_hi[d], p.k_dilation[d],
                         p.k_pad_lo[d], p.k_pad_hi[d]);
}

long untransformedOutputSize(const plb_conv_params &p, unsigned d) {
  const long in = transformedInputSize(p, d), k = transformedKernelSize(p, d);
  if (in < 0 || k <= 0 || in < k) return -1;
  return in - k + 1;
}

long outputSize(const plb_conv_params &p, unsigned d) {
  const long conv = untransformedOutputSize(p, d);
  if (conv < 0 || p.stride[d] == 0) return -1;
  const long truncated = conv - (long(p.out_trunc_lo[d]) + long(p.out_trunc_hi[d]));
  if (truncated < 0) return -1;
  const long strided = (truncated + p.stride[d] - 1) / p.stride[d];
  return long(p.out_pad_lo[d]) + strided + long(p.out_pad_hi[d]);
}

std::string validate(const plb_conv_params &p) {
  auto s = [](long v) { return std::to_string(v); };
  if (p.num_field_dims < 1 || p.num_field_dims > PLB_MAX_FIELD_DIMS)
    return "Number of field dimensions (" + s(p.num_field_dims) + ") is not supported (1 to " +
           s(PLB_MAX_FIELD_DIMS) + ")";
  for (unsigned d = 0; d != p.num_field_dims; ++d)
    if (p.stride[d] == 0) return "Stride must be non zero";
  for (unsigned d = 0; d != p.num_field_dims; ++d)
    if (p.in_dilation[d] == 0)
      return "Input dilation must be non zero. Dilation = 1 results in no dilation";
  for (unsigned d = 0; d != p.num_field_dims; ++d)
    if (p.k_dilation[d] == 0)
      return "Kernel dilation must be non zero. Dilation = 1 results in no dilation";
  for (unsigned d = 0; d != p.num_field_dims; ++d) {
    const long inTrunc = long(p.in_trunc_lo[d]) + p.in_trunc_hi[d];
    if (inTrunc > long(p.field[d]))
      return "Truncation for dimension " + s(d) + " (" + s(inTrunc) +
             ") truncates by more than the size of the field (" + s(p.field[d]) + ")";
    const long kTrunc = long(p.k_trunc_lo[d]) + p.k_trunc_hi[d];
    if (kTrunc > long(p.kernel[d]))
      return "Truncation for dimension " + s(d) + " (" + s(kTrunc) +
             ") truncates by more than the size of the kernel (" + s(p.kernel[d]) + ")";
    const long in = transformedInputSize(p, d), k = transformedKernelSize(p, d);
    if (k == 0) return "Transformed kernel for dimension " + s(d) + " has zero size";
    if (in < k)
      return "Transformed input size for dimension " + s(d) + " (" + s(in) +
             ") is less than the transformed kernel size (" + s(k) + ")";
    const long conv = in - k + 1;
    const long outTrunc = long(p.out_trunc_lo[d]) + p.out_trunc_hi[d];
    if (outTrunc > conv)
      return "Output truncation for dimension " + s(d) + " (" + s(outTrunc) +
             ") truncates by more than the size of the convolution output (" + s(conv) + ")";
  }
  return std::string();
}

int inputIndex(const plb_conv_params &p, unsigned d, unsigned outIndex, unsigned kernelIndex) {
  const long out = outputSize(p, d);
  if (out < 0 || long(outIndex) >= out || kernelIndex >= p.kernel[d]) return -1;
  // output padding holds zeros only
  if (outIndex < p.out_pad_lo[d] || long(outIndex) >= out - long(p.out_pad_hi[d])) return -1;
  const long convIndex =
      long(p.out_trunc_lo[d]) + long(outIndex - p.out_pad_lo[d]) * long(p.stride[d]);
  // where the kernel element sits in the transformed kernel
  if (kernelIndex < p.k_trunc_lo[d] || kernelIndex >= p.kernel[d] - p.k_trunc_hi[d]) return -1;
  const long kSize = transformedKernelSize(p, d);
  long kPos = long(kernelIndex - p.k_trunc_lo[d]) * long(p.k_dilation[d]) + long(p.k_pad_lo[d]);
  if (p.k_flip[d]) kPos = kSize - 1 - kPos;
  // position in the transformed input; undo flip, padding, dilation, truncation
  const long inSize = transformedInputSize(p, d);
  long pos = convIndex + kPos;
  if (pos < 0 || pos >= inSize) return -1;
  if (p.in_flip[d]) pos = inSize - 1 - pos;
  pos -= long(p.in_pad_lo[d]);
  const long truncated = long(p.field[d]) - (long(p.in_trunc_lo[d]) + long(p.in_trunc_hi[d]));
  if (pos < 0 || pos >= dilatedSize(truncated, p.in_dilation[d])) return -1;
  if (pos % long(p.in_dilation[d]) != 0) return -1;
  return int(pos / long(p.in_dilation[d]) + long(p.in_trunc_lo[d]));
}

uint64_t numberOfMacs(const plb_conv_params &p) {
  uint64_t macs = uint64_t(p.batch) * p.groups * p.in_chans_per_group * p.out_chans_per_group;
  for (unsigned d = 0; d != p.num_field_dims; ++d) {
    const long out = outputSize(p, d);
    if (out < 0) return 0;
    uint64_t touching = 0;
    for (unsigned o = 0; o != unsigned(out); ++o)
      for (unsigned k = 0; k != p.kernel[d]; ++k)
        if (inputIndex(p, d, o, k) >= 0) ++touching;
    macs *= touching;
  }
  return macs;
}

}  // namespace plb
