// C ABI entry points of the contraction path: matMul, convolution forward and
// backward-data.  Each maps its poplin-level description onto one or more
// launches of the implicit-GEMM kernel (igemm_sm100.cuh).
#include <cuda_fp16.h>

#include <algorithm>
#include <cmath>
#include <vector>

#include "conv_geometry.h"
#include "runtime.h"

namespace plb {

int launchScaleRows(plb_context *ctx, void *out, const void *c, float beta, bool out_f32,
                    uint32_t rows, uint32_t cols, long long ldo, long long ldc);
int convFwdSmallChannels(plb_context *ctx, const plb_conv_params &p, const plb_conv_options *opt,
                         const void *d_in, const void *d_weights, const float *d_bias,
                         void *d_out, plb_plan *plan_only);

// TMA needs 16-byte pixel strides: 8 half / 16 quarter channels.
static bool channelsFitTma(const plb_conv_params &p, uint32_t chans) {
  return (size_t(chans) * dtypeBytes(p.input_type)) % 16 == 0;
}

namespace {

int checkMatmulDesc(const plb_matmul_desc &d) {
  if (!is16BitFloat(d.input_type) && d.input_type != PLB_QUARTER && d.input_type != PLB_FLOAT)
    return fail(PLB_ERR_INVALID_PARAMS, "matMul input type must be half or quarter");
  if (d.output_type != PLB_HALF && d.output_type != PLB_FLOAT)
    return fail(PLB_ERR_INVALID_PARAMS, "matMul output type must be half or float");
  if (d.input_type == PLB_QUARTER && d.output_type != PLB_HALF)
    // lib/poplin/ConvValidation.cpp:53-69: quarter input requires half output
    return fail(PLB_ERR_INVALID_PARAMS, "Output type must be half when input type is quarter");
  if (d.partials_type != PLB_HALF && d.partials_type != PLB_FLOAT)
    return fail(PLB_ERR_INVALID_OPTION, "partialsType must be half or float");
  if (d.scale_a < -32 || d.scale_a > 31 || d.scale_b < -32 || d.scale_b > 31)
    return fail(PLB_ERR_INVALID_PARAMS, "quarter metadata scale must be in [-32, 31]");
  if ((d.format_a != PLB_F143 && d.format_a != PLB_F152) || (d.format_b != PLB_F143 && d.format_b != PLB_F152))
    return fail(PLB_ERR_INVALID_PARAMS, "quarter format must be PLB_F143 or PLB_F152");
  return PLB_OK;
}

struct Ld {
  long long a, b, c;
};

Ld leadingDims(const plb_matmul_desc &d) {
  Ld l;
  l.a = d.lda ? d.lda : (d.transpose_a ? d.m : d.k);
  l.b = d.ldb ? d.ldb : (d.transpose_b ? d.k : d.n);
  l.c = d.ldc ? d.ldc : d.n;
  return l;
}

// Builds the igemm problem of one group of a matrix product.  `a` is [m][k]
// (row stride lda), `b` either [n][k] (b_is_nk) or [k][n].
IgemmProblem gemmProblem(const plb_matmul_desc &d, const void *a, long long lda, const void *b,
                         long long ldb, bool b_is_nk, const void *c, void *out, long long ldc) {
  IgemmProblem p;
  const size_t es = dtypeBytes(d.input_type);
  p.fp8 = d.input_type == PLB_QUARTER;
  p.bf16 = d.input_type == PLB_BFLOAT16;
  p.fmt_a = d.format_a;
  p.fmt_b = d.format_b;
  p.b_mn = !b_is_nk;
  p.act = a;
  p.act_dims[0] = d.k;
  p.act_dims[1] = d.m;
  p.act_strides[0] = uint64_t(lda) * es;
  p.act_strides[1] = uint64_t(lda) * es * std::max<uint32_t>(d.m, 1);
  p.act_strides[2] = p.act_strides[1];
  p.wgt = b;
  if (b_is_nk) {
    p.wgt_dims[0] = d.k;
    p.wgt_dims[1] = d.n;
    p.wgt_strides[0] = uint64_t(ldb) * es;
    p.wgt_strides[1] = uint64_t(ldb) * es * std::max<uint32_t>(d.n, 1);
  } else {
    p.wgt_dims[0] = d.n;
    p.wgt_dims[1] = d.k;
    p.wgt_strides[0] = uint64_t(ldb) * es;
    p.wgt_strides[1] = uint64_t(ldb) * es * std::max<uint32_t>(d.k, 1);
  }
  p.out_w = int(d.m);
  p.n_total = int(d.n);
  p.k_per_tap = int(d.k);
  p.out = out;
  p.ldc = ldc;
  p.addend = c;
  p.ld_addend = ldc;
  p.alpha = d.alpha;
  if (p.fp8) p.alpha *= std::ldexp(1.0f, d.scale_a + d.scale_b);
  p.beta = d.beta;
  p.out_f32 = d.output_type == PLB_FLOAT;
  return p;
}

uint64_t gemmBytes(const plb_matmul_desc &d) {
  const uint64_t es = dtypeBytes(d.input_type), os = dtypeBytes(d.output_type);
  return uint64_t(d.groups) * (uint64_t(d.m) * d.k * es + uint64_t(d.k) * d.n * es +
                               uint64_t(d.m) * d.n * os * (d.beta != 0.f ? 2 : 1));
}

// ---- convolution --------------------------------------------------------------------

struct ConvShape {
  unsigned nd;
  int H, W, OH, OW;      // input / output field as stored (H = 1 for 1-D)
  int KH, KW;            // filter taps that are used (the kernel after truncation)
  int KHs, KWs;          // filter extent as stored
  int ktH, ktW;          // kernel truncation at the low end
  // padH/padW: input padding minus output truncation minus kernel padding at
  // the low end (the high end's kernel padding for a flipped kernel), i.e.
  // output position o, used tap r reads truncated-input row
  // o*stride + r*dil - pad (may be negative: the first rows are skipped)
  int padH, padW, dilH, dilW, strH, strW, flipH, flipW;
  int tH, tW;            // input truncation at the low end (rows / columns not used)
  int He, We;            // extent of the truncated input
  int opH, opW;          // output padding at the low end (zero rows / columns)
  int OHc, OWc;          // extent of the computed (not padded) output
  bool zero_fill_out;    // the output has padded positions
  bool zero_fill_in;     // the input has truncated positions (backward pass zeroes them)
};

int igemmConvShape(const plb_conv_params &p, ConvShape *s) {
  const std::string err = validate(p);
  if (!err.empty()) return fail(PLB_ERR_INVALID_PARAMS, err);
  if (p.num_field_dims > 2)
    return fail(PLB_ERR_UNSUPPORTED, "3-D convolutions are not implemented on this path yet");
  if (!is16BitFloat(p.input_type) && p.input_type != PLB_QUARTER)
    return fail(PLB_ERR_UNSUPPORTED, "convolution input type must be half, float or quarter");
  if (p.output_type != PLB_HALF && p.output_type != PLB_FLOAT)
    return fail(PLB_ERR_INVALID_PARAMS, "convolution output type must be half or float");
  if (p.input_type == PLB_QUARTER && p.output_type != PLB_HALF)
    return fail(PLB_ERR_INVALID_PARAMS, "Output type must be half when input type is quarter");
  // Input truncation, output truncation and output padding are views and
  // offsets (below).  Input dilation only arrives through the backward pass of
  // a strided layer, which plb_conv_bwd takes in forward terms.
  // Kernel truncation selects a sub-rectangle of the taps (gathered by the
  // entry points), kernel padding only shifts where the taps land.
  for (unsigned d = 0; d != p.num_field_dims; ++d) {
    if (p.in_dilation[d] != 1 || p.in_flip[d])
      return fail(PLB_ERR_UNSUPPORTED,
                  "input dilation/flip are not implemented on this path yet");
  }
  s->nd = p.num_field_dims;
  const unsigned hd = p.num_field_dims == 2 ? 0 : ~0u, wd = p.num_field_dims - 1;
  auto get = [&](const uint32_t *v, unsigned d, int dflt) { return d == ~0u ? dflt : int(v[d]); };
  s->H = get(p.field, hd, 1);
  s->W = get(p.field, wd, 1);
  s->KHs = get(p.kernel, hd, 1);
  s->KWs = get(p.kernel, wd, 1);
  s->ktH = get(p.k_trunc_lo, hd, 0);
  s->ktW = get(p.k_trunc_lo, wd, 0);
  s->KH = s->KHs - s->ktH - get(p.k_trunc_hi, hd, 0);
  s->KW = s->KWs - s->ktW - get(p.k_trunc_hi, wd, 0);
  s->padH = get(p.in_pad_lo, hd, 0);
  s->padW = get(p.in_pad_lo, wd, 0);
  s->dilH = get(p.k_dilation, hd, 1);
  s->dilW = get(p.k_dilation, wd, 1);
  s->strH = get(p.stride, hd, 1);
  s->strW = get(p.stride, wd, 1);
  s->flipH = get(p.k_flip, hd, 0);
  s->flipW = get(p.k_flip, wd, 0);
  s->OH = hd == ~0u ? 1 : int(outputSize(p, hd));
  s->OW = int(outputSize(p, wd));
  s->tH = get(p.in_trunc_lo, hd, 0);
  s->tW = get(p.in_trunc_lo, wd, 0);
  s->He = s->H - s->tH - get(p.in_trunc_hi, hd, 0);
  s->We = s->W - s->tW - get(p.in_trunc_hi, wd, 0);
  s->padH -= get(p.out_trunc_lo, hd, 0) + get(s->flipH ? p.k_pad_hi : p.k_pad_lo, hd, 0);
  s->padW -= get(p.out_trunc_lo, wd, 0) + get(s->flipW ? p.k_pad_hi : p.k_pad_lo, wd, 0);
  s->opH = get(p.out_pad_lo, hd, 0);
  s->opW = get(p.out_pad_lo, wd, 0);
  s->OHc = s->OH - s->opH - get(p.out_pad_hi, hd, 0);
  s->OWc = s->OW - s->opW - get(p.out_pad_hi, wd, 0);
  s->zero_fill_out = s->OHc != s->OH || s->OWc != s->OW;
  s->zero_fill_in = s->He != s->H || s->We != s->W;
  return PLB_OK;
}

uint64_t convBytes(const plb_conv_params &p, const ConvShape &s, int pass) {
  const uint64_t es = dtypeBytes(p.input_type), os = dtypeBytes(p.output_type);
  const uint64_t in = uint64_t(p.batch) * s.H * s.W * p.groups * p.in_chans_per_group;
  const uint64_t out = uint64_t(p.batch) * s.OH * s.OW * p.groups * p.out_chans_per_group;
  const uint64_t w = uint64_t(p.groups) * s.KH * s.KW * p.in_chans_per_group * p.out_chans_per_group;
  // a 1x1 kernel with stride reads only every stride-th pixel
  uint64_t in_read = in;
  if (s.KH == 1 && s.KW == 1) in_read = uint64_t(p.batch) * s.OH * s.OW * p.groups * p.in_chans_per_group;
  switch (pass) {
    case PLB_PASS_TRAINING_BWD: return out * es + w * es + in * os;
    case PLB_PASS_TRAINING_WU: return in * es + out * es + w * es;
    default: return in_read * es + w * es + out * os;
  }
}

// Forward problem of group g.
// With `swapped_weights` the weights are stored [G][tap][Ci][Co] (the forward
// layout of the layer this convolution is the backward pass of) and are used
// with their spatial axes flipped: they are read as a K-by-N (MN-major) operand.
int convFwdProblem(const plb_conv_params &p, const plb_conv_options *opt, const ConvShape &s,
                   unsigned g, const void *in, const void *w, const float *bias, void *out,
                   IgemmProblem *q, bool swapped_weights = false) {
  const size_t es = dtypeBytes(p.input_type), os = dtypeBytes(p.output_type);
  const uint64_t ctot = uint64_t(p.groups) * p.in_chans_per_group;
  const uint64_t cotot = uint64_t(p.groups) * p.out_chans_per_group;
  const uint64_t ci = p.in_chans_per_group, co = p.out_chans_per_group;
  IgemmProblem r;
  r.fp8 = p.input_type == PLB_QUARTER;
  r.bf16 = p.input_type == PLB_BFLOAT16;
  r.fmt_a = opt ? opt->format_in : 0;
  r.fmt_b = opt ? opt->format_weights : 0;
  // the truncated input is a view: same strides, shifted base, smaller extents
  r.act = static_cast<const uint8_t *>(in) +
          ((size_t(s.tH) * s.W + s.tW) * ctot + size_t(g) * ci) * es;
  const bool pointwise = s.KH == 1 && s.KW == 1 && s.padH == 0 && s.padW == 0;
  if (pointwise) {
    // a strided 1x1 convolution reads a sub-lattice: describe only that (its
    // extent is what the input holds; outputs beyond it read zero padding)
    r.act_dims[0] = ci;
    r.act_dims[1] = uint64_t(std::min(s.OWc, (s.We + s.strW - 1) / s.strW));
    r.act_dims[2] = uint64_t(std::min(s.OHc, (s.He + s.strH - 1) / s.strH));
    r.act_dims[3] = p.batch;
    r.act_strides[0] = uint64_t(s.strW) * ctot * es;
    r.act_strides[1] = uint64_t(s.strH) * s.W * ctot * es;
    r.act_strides[2] = uint64_t(s.H) * s.W * ctot * es;
  } else {
    r.act_dims[0] = ci;
    r.act_dims[1] = uint64_t(s.We);
    r.act_dims[2] = uint64_t(s.He);
    r.act_dims[3] = p.batch;
    r.act_strides[0] = ctot * es;
    r.act_strides[1] = uint64_t(s.W) * ctot * es;
    r.act_strides[2] = uint64_t(s.H) * s.W * ctot * es;
    r.stride_h = s.strH;
    r.stride_w = s.strW;
    r.act_elem_strides[1] = uint32_t(s.strW);
    r.act_elem_strides[2] = uint32_t(s.strH);
  }
  r.wgt = static_cast<const uint8_t *>(w) + size_t(g) * s.KH * s.KW * co * ci * es;
  r.b_mn = swapped_weights;
  r.wgt_dims[0] = swapped_weights ? co : ci;
  r.wgt_dims[1] = swapped_weights ? ci : co;
  r.wgt_dims[2] = uint64_t(s.KH) * s.KW;
  r.wgt_strides[0] = (swapped_weights ? co : ci) * es;
  r.wgt_strides[1] = co * ci * es;
  // the computed part of the output is a view of the stored (padded) one
  r.out_w = s.OWc;
  r.out_h = s.OHc;
  r.out_n = int(p.batch);
  r.n_total = int(co);
  r.k_per_tap = int(ci);
  r.taps_h = s.KH;
  r.taps_w = s.KW;
  r.pad_h = s.padH;
  r.pad_w = s.padW;
  r.dil_h = s.dilH;
  r.dil_w = s.dilW;
  r.flip_h = swapped_weights ? !s.flipH : s.flipH;
  r.flip_w = swapped_weights ? !s.flipW : s.flipW;
  r.out = static_cast<uint8_t *>(out) +
          ((size_t(s.opH) * s.OW + s.opW) * cotot + size_t(g) * co) * os;
  r.ldc = (long long)cotot;
  r.out_stride_h = (long long)(cotot * s.OW);
  r.out_stride_n = (long long)(cotot * s.OW * s.OH);
  r.bias = bias ? bias + size_t(g) * co : nullptr;
  r.out_f32 = p.output_type == PLB_FLOAT;
  r.force_tile_n = opt ? opt->tile_n : 0;
  r.force_split_k = opt ? opt->split_k : 0;
  r.plan_flags = opt ? opt->plan_flags : 0;
  if (r.fp8 && opt) r.alpha = std::ldexp(1.0f, opt->scale_in + opt->scale_weights);
  *q = r;
  return PLB_OK;
}

// Backward-data problem of group g (stride 1): the output gradients take the
// activations' role, the taps are traversed in the opposite order, the padding
// becomes (k-1)*dilation - padding, and the stored [tap][Co][Ci] weights are
// read as a K-by-N (MN-major) operand with K = Co, N = Ci.
int convBwdProblem(const plb_conv_params &p, const plb_conv_options *opt, const ConvShape &s,
                   unsigned g, const void *dy, const void *w, void *dx, bool weights_transposed,
                   IgemmProblem *q) {
  const size_t es = dtypeBytes(p.input_type), os = dtypeBytes(p.output_type);
  const uint64_t ctot = uint64_t(p.groups) * p.in_chans_per_group;
  const uint64_t cotot = uint64_t(p.groups) * p.out_chans_per_group;
  const uint64_t ci = p.in_chans_per_group, co = p.out_chans_per_group;
  IgemmProblem r;
  r.fp8 = p.input_type == PLB_QUARTER;
  r.bf16 = p.input_type == PLB_BFLOAT16;
  r.fmt_a = opt ? opt->format_in : 0;
  r.fmt_b = opt ? opt->format_weights : 0;
  // computed part of the output gradients / used part of the input gradients
  r.act = static_cast<const uint8_t *>(dy) +
          ((size_t(s.opH) * s.OW + s.opW) * cotot + size_t(g) * co) * es;
  r.act_dims[0] = co;
  r.act_dims[1] = uint64_t(s.OWc);
  r.act_dims[2] = uint64_t(s.OHc);
  r.act_dims[3] = p.batch;
  r.act_strides[0] = cotot * es;
  r.act_strides[1] = uint64_t(s.OW) * cotot * es;
  r.act_strides[2] = uint64_t(s.OH) * s.OW * cotot * es;
  r.wgt = static_cast<const uint8_t *>(w) + size_t(g) * s.KH * s.KW * co * ci * es;
  if (weights_transposed) {
    // [tap flipped][Ci][Co]: a K-major operand, taps already reversed
    r.wgt_dims[0] = co;
    r.wgt_dims[1] = ci;
    r.wgt_strides[0] = co * es;
    r.flip_h = s.flipH;
    r.flip_w = s.flipW;
  } else {
    r.b_mn = true;
    r.wgt_dims[0] = ci;
    r.wgt_dims[1] = co;
    r.wgt_strides[0] = ci * es;
    r.flip_h = !s.flipH;
    r.flip_w = !s.flipW;
  }
  r.wgt_dims[2] = uint64_t(s.KH) * s.KW;
  r.wgt_strides[1] = co * ci * es;
  r.out_w = s.We;
  r.out_h = s.He;
  r.out_n = int(p.batch);
  r.n_total = int(ci);
  r.k_per_tap = int(co);
  r.taps_h = s.KH;
  r.taps_w = s.KW;
  r.pad_h = (s.KH - 1) * s.dilH - s.padH;
  r.pad_w = (s.KW - 1) * s.dilW - s.padW;
  r.dil_h = s.dilH;
  r.dil_w = s.dilW;
  r.out = static_cast<uint8_t *>(dx) + ((size_t(s.tH) * s.W + s.tW) * ctot + size_t(g) * ci) * os;
  r.ldc = (long long)ctot;
  r.out_stride_h = (long long)(ctot * s.W);
  r.out_stride_n = (long long)(ctot * s.W * s.H);
  r.out_f32 = p.output_type == PLB_FLOAT;
  r.force_tile_n = opt ? opt->tile_n : 0;
  r.force_split_k = opt ? opt->split_k : 0;
  r.plan_flags = opt ? opt->plan_flags : 0;
  if (r.fp8 && opt) r.alpha = std::ldexp(1.0f, opt->scale_in + opt->scale_weights);
  *q = r;
  return PLB_OK;
}

// Filter taps (r0h + jh*sh, r0w + jw*sw), jh < JH, jw < JW, of [G][KH*KW][inner]
// weights gathered into [G][JH*JW][inner]; 16-byte vectors.  With flip_h /
// flip_w the tap indices count from the far end of the stored filter (the
// filter is used spatially flipped).
__global__ void gatherTapsKernel(const uint4 *__restrict__ src, uint4 *__restrict__ dst, int groups,
                                 int KH, int KW, int JH, int JW, int r0h, int r0w, int sh, int sw,
                                 size_t inner_vecs, int flip_h = 0, int flip_w = 0) {
  const size_t total = size_t(groups) * JH * JW * inner_vecs;
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < total;
       i += size_t(gridDim.x) * blockDim.x) {
    const size_t v = i % inner_vecs;
    size_t t = i / inner_vecs;
    const int jw = int(t % JW);
    t /= JW;
    const int jh = int(t % JH);
    const int g = int(t / JH);
    const int th = r0h + jh * sh, tw = r0w + jw * sw;
    const size_t tap = size_t(flip_h ? KH - 1 - th : th) * KW + size_t(flip_w ? KW - 1 - tw : tw);
    dst[i] = src[(size_t(g) * KH * KW + tap) * inner_vecs + v];
  }
}

// out[pixel][c] = bias[c]: what a convolution with a fused bias leaves where
// nothing is accumulated (output padding).
template <typename T>
__global__ void fillBiasKernel(T *out, const float *__restrict__ bias, size_t total, size_t chans) {
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < total;
       i += size_t(gridDim.x) * blockDim.x)
    out[i] = T(bias[i % chans]);
}

// One dimension of the backward pass of a strided convolution, for the input
// positions i*stride + phase: which filter taps reach them and where.  Tap r
// reaches the phase iff (phase + pad - r*dil) is a multiple of the stride; with
// g = gcd(dil, stride) those taps are r0, r0 + stride/g, ... and, from one to the
// next, the output index read at a fixed i moves by dil/g.
struct BwdPhase {
  int first_tap;   // r0: smallest tap with (phase + pad - r*dil) divisible by stride
  int taps;        // J: taps r0, r0 + step, ...
  int step;        // stride / gcd(dil, stride)
  int dil;         // dil / gcd(dil, stride): dilation of the gathered sub-filter
  int offset;      // (phase + pad - r0*dil) / stride: output index read by tap r0 at i = 0
  int extent;      // input positions of this phase
};
void bwdPhase(int phase, int in_size, int kernel, int pad, int dil, int stride, BwdPhase *out) {
  int g = dil, t = stride;
  while (t) {
    const int u = g % t;
    g = t;
    t = u;
  }
  out->extent = phase < in_size ? (in_size - phase + stride - 1) / stride : 0;
  out->first_tap = -1;
  out->taps = 0;
  out->offset = 0;
  out->step = stride / g;
  out->dil = dil / g;
  for (int r = 0; r < kernel; ++r) {
    const int num = phase + pad - r * dil;
    if (((num % stride) + stride) % stride != 0) continue;
    if (out->first_tap < 0) {
      out->first_tap = r;
      out->offset = num / stride;  // exact: num is a multiple of stride (possibly negative)
    }
    ++out->taps;
  }
}

// ---- channel counts TMA cannot address -------------------------------------------
// A pixel must be a multiple of 16 bytes for the tensor maps (8 half / 16 quarter
// channels per group).  Other counts run on zero-padded copies: activations
// [pixels][G][C -> Cp], weights [G][taps][Co -> Cop][Ci -> Cip]; padded input
// channels meet zero weights, padded output channels are dropped.  One arena
// (scratch slot 7) holds the copies.
struct PaddedChans {
  uint32_t ci, co, cip, cop;
  bool needed;
};
PaddedChans paddedChans(const plb_conv_params &p) {
  const uint32_t q = uint32_t(16 / dtypeBytes(p.input_type));
  PaddedChans c{p.in_chans_per_group, p.out_chans_per_group, 0, 0, false};
  c.cip = (c.ci + q - 1) / q * q;
  c.cop = (c.co + q - 1) / q * q;
  c.needed = c.cip != c.ci || c.cop != c.co;
  return c;
}
// [G][taps][rows][cols] -> [G][taps][rows_p][cols_p]
int padWeights(plb_context *ctx, const void *src, void *tmp, void *dst, size_t g_taps, uint32_t rows,
               uint32_t cols, uint32_t rows_p, uint32_t cols_p, size_t es) {
  if (int rc = resizeRows(ctx, src, tmp, g_taps * rows, cols * es, cols_p * es)) return rc;
  return resizeRows(ctx, tmp, dst, g_taps, size_t(rows) * cols_p * es, size_t(rows_p) * cols_p * es);
}
size_t align256(size_t n) { return (n + 255) & ~size_t(255); }

// Weights of a truncated kernel: the used sub-rectangle of taps gathered into
// scratch as a dense [G][KH*KW][Co*Ci] filter.  Returns `w` itself when the
// kernel is not truncated.
int usedTaps(plb_context *ctx, const plb_conv_params &p, const ConvShape &s, const void *w,
             const void **out) {
  *out = w;
  if (s.KH == s.KHs && s.KW == s.KWs) return PLB_OK;
  const size_t es = dtypeBytes(p.input_type);
  const size_t inner = size_t(p.out_chans_per_group) * p.in_chans_per_group * es;
  if (inner % 16 != 0 || (reinterpret_cast<uintptr_t>(w) & 15) != 0)
    return fail(PLB_ERR_UNSUPPORTED, "weights must be 16-byte aligned per tap");
  if (s.KH <= 0 || s.KW <= 0) return PLB_OK;  // nothing is used; callers zero the result
  void *ws = nullptr;
  const size_t bytes = size_t(p.groups) * s.KH * s.KW * inner;
  if (int rc = scratch(ctx, kSlotUsedTaps, bytes + 256, &ws)) return rc;
  const size_t vecs = bytes / 16;
  const int grid = int(std::min<size_t>((vecs + 255) / 256, size_t(ctx->sm_count) * 8));
  gatherTapsKernel<<<grid, 256, 0, ctx->stream>>>(static_cast<const uint4 *>(w),
                                                  static_cast<uint4 *>(ws), int(p.groups), s.KHs,
                                                  s.KWs, s.KH, s.KW, s.ktH, s.ktW, 1, 1, inner / 16);
  PLB_CUDA(cudaGetLastError());
  ctx->launches++;
  *out = ws;
  return PLB_OK;
}

// Backward pass of a strided convolution (the reference's getGradientParams
// gives the output gradients an input dilation equal to the forward stride,
// lib/poplin/ConvUtil.cpp:728-795).  Multiplying the inserted zeros would
// waste stride^2 of the work: instead the input gradient is computed per
// phase (ih mod stride_h, iw mod stride_w).  The positions of one phase see a
// fixed, evenly spaced subset of the filter taps, so each phase is a stride-1
// convolution of the output gradients with the gathered sub-filter, written
// to the strided sub-lattice of the input gradient.
int convBwdStrided(plb_context *ctx, const plb_conv_params &p, const plb_conv_options *opt,
                   const ConvShape &s, const void *dy, const void *w, void *dx) {
  // 8-bit operands have no MN-major form: their gathered sub-filters are
  // transposed per tap ([Co][Ci] -> [Ci][Co]) into a second buffer
  const bool fp8 = p.input_type == PLB_QUARTER;
  const size_t es = dtypeBytes(p.input_type), os = dtypeBytes(p.output_type);
  const uint64_t ci = p.in_chans_per_group, co = p.out_chans_per_group;
  const uint64_t ctot = uint64_t(p.groups) * ci, cotot = uint64_t(p.groups) * co;
  const size_t inner = size_t(co) * ci;  // elements per tap and group
  if ((inner * es) % 16 != 0 || (reinterpret_cast<uintptr_t>(w) & 15) != 0)
    return fail(PLB_ERR_UNSUPPORTED, "weights must be 16-byte aligned per tap");
  // phases and their taps
  std::vector<BwdPhase> ph(size_t(s.strH)), pw(size_t(s.strW));
  for (int a = 0; a < s.strH; ++a) bwdPhase(a, s.He, s.KH, s.padH, s.dilH, s.strH, &ph[size_t(a)]);
  for (int b = 0; b < s.strW; ++b) bwdPhase(b, s.We, s.KW, s.padW, s.dilW, s.strW, &pw[size_t(b)]);
  // positions no tap reaches get zero
  bool any_empty = false;
  size_t scratch_elems = 0;
  for (const auto &a : ph)
    for (const auto &b : pw) {
      if (a.extent == 0 || b.extent == 0) continue;
      if (a.taps == 0 || b.taps == 0) any_empty = true;
      scratch_elems = std::max(scratch_elems, size_t(p.groups) * a.taps * b.taps * inner);
    }
  if (any_empty && !s.zero_fill_in)  // (otherwise the caller has cleared it)
    PLB_CUDA(cudaMemsetAsync(dx, 0, size_t(p.batch) * s.H * s.W * ctot * os, ctx->stream));
  void *ws = nullptr;
  // one buffer per phase: the launches of different phases are in flight together
  const size_t slot = (scratch_elems * es + 255) & ~size_t(255);
  const size_t phases = size_t(s.strH) * s.strW;
  if (int rc = scratch(ctx, kSlotOperands, slot * phases * (fp8 ? 2 : 1) + 256, &ws)) return rc;
  for (int a = 0; a < s.strH; ++a)
    for (int b = 0; b < s.strW; ++b) {
      const BwdPhase &A = ph[size_t(a)], &B = pw[size_t(b)];
      if (A.extent == 0 || B.extent == 0 || A.taps == 0 || B.taps == 0) continue;
      uint8_t *wsub = static_cast<uint8_t *>(ws) + slot * (size_t(a) * s.strW + b);
      const size_t vecs = size_t(p.groups) * A.taps * B.taps * (inner * es / 16);
      const int grid = int(std::min<size_t>((vecs + 255) / 256, size_t(ctx->sm_count) * 8));
      gatherTapsKernel<<<grid, 256, 0, ctx->stream>>>(
          static_cast<const uint4 *>(w), reinterpret_cast<uint4 *>(wsub), int(p.groups), s.KH, s.KW,
          A.taps, B.taps, A.first_tap, B.first_tap, A.step, B.step, inner * es / 16, s.flipH,
          s.flipW);
      PLB_CUDA(cudaGetLastError());
      ctx->launches++;
      if (fp8) {
        uint8_t *wt = static_cast<uint8_t *>(ws) + slot * (phases + size_t(a) * s.strW + b);
        if (int rc = plb_transpose_matrix(ctx, 1, uint32_t(p.groups * A.taps * B.taps), uint32_t(co),
                                          uint32_t(ci), wsub, wt))
          return rc;
        wsub = wt;
      }
      for (unsigned g = 0; g < p.groups; ++g) {
        IgemmProblem r;
        r.fp8 = fp8;
        r.bf16 = p.input_type == PLB_BFLOAT16;
        r.fmt_a = opt ? opt->format_in : 0;
        r.fmt_b = opt ? opt->format_weights : 0;
        r.act = static_cast<const uint8_t *>(dy) +
                ((size_t(s.opH) * s.OW + s.opW) * cotot + size_t(g) * co) * es;
        r.act_dims[0] = co;
        r.act_dims[1] = uint64_t(s.OWc);
        r.act_dims[2] = uint64_t(s.OHc);
        r.act_dims[3] = p.batch;
        r.act_strides[0] = cotot * es;
        r.act_strides[1] = uint64_t(s.OW) * cotot * es;
        r.act_strides[2] = uint64_t(s.OH) * s.OW * cotot * es;
        r.wgt = wsub + size_t(g) * A.taps * B.taps * inner * es;
        if (fp8) {
          // transposed [tap][Ci][Co]: a K-major right operand
          r.wgt_dims[0] = co;
          r.wgt_dims[1] = ci;
          r.wgt_strides[0] = co * es;
          if (opt) r.alpha = std::ldexp(1.0f, opt->scale_in + opt->scale_weights);
        } else {
          // gathered [tap][Co][Ci]: K = co rows of N = ci, an MN-major right operand
          r.b_mn = true;
          r.wgt_dims[0] = ci;
          r.wgt_dims[1] = co;
          r.wgt_strides[0] = ci * es;
        }
        r.wgt_dims[2] = uint64_t(A.taps) * B.taps;
        r.wgt_strides[1] = inner * es;
        r.out_w = B.extent;
        r.out_h = A.extent;
        r.out_n = int(p.batch);
        r.n_total = int(ci);
        r.k_per_tap = int(co);
        r.taps_h = A.taps;
        r.taps_w = B.taps;
        // position i of the phase reads output index i + offset - j*dil for the
        // j-th gathered tap: a correlation with the taps reversed
        r.dil_h = A.dil;
        r.dil_w = B.dil;
        r.pad_h = (A.taps - 1) * A.dil - A.offset;
        r.pad_w = (B.taps - 1) * B.dil - B.offset;
        // (a flipped forward kernel was un-flipped by the gather)
        r.flip_h = 1;
        r.flip_w = 1;
        r.out = static_cast<uint8_t *>(dx) +
                ((size_t(s.tH + a) * s.W + (s.tW + b)) * ctot + size_t(g) * ci) * os;
        r.ldc = (long long)(ctot * s.strW);
        r.out_stride_h = (long long)(ctot * s.W * s.strH);
        r.out_stride_n = (long long)(ctot * s.W * s.H);
        r.out_f32 = p.output_type == PLB_FLOAT;
        r.force_tile_n = opt ? opt->tile_n : 0;
        r.force_split_k = opt ? opt->split_k : 0;
        r.plan_flags = (opt ? opt->plan_flags : 0) | ctx->plan_flags;
        plb_plan plan{};
        if (int rc = planIgemm(r, ctx->sm_count, &plan)) return rc;
        if (int rc = launchIgemm(ctx, r, plan)) return rc;
      }
    }
  return PLB_OK;
}

}  // namespace
}  // namespace plb

using namespace plb;

extern "C" {

int plb_matmul_plan(const plb_matmul_desc *desc, plb_plan *plan) {
  if (!desc || !plan) return fail(PLB_ERR_INVALID_PARAMS, "null argument");
  if (int rc = checkMatmulDesc(*desc)) return rc;
  if (desc->input_type == PLB_FLOAT) {
    // what runs: bfloat16 operands, three terms per product (float_route.cu)
    const plb_matmul_desc q = floatRouteMatmulDesc(*desc);
    if (int rc = plb_matmul_plan(&q, plan)) return rc;
    plan->flops = 2ull * desc->groups * desc->m * desc->k * desc->n;
    plan->bytes = gemmBytes(*desc);
    plan->workspace_bytes += size_t(desc->groups) * desc->k * (size_t(desc->m) + desc->n) * 6 + 768;
    return PLB_OK;
  }
  *plan = plb_plan{};
  plan->flops = 2ull * desc->groups * desc->m * desc->k * desc->n;
  plan->bytes = gemmBytes(*desc);
  if (desc->groups == 0 || desc->m == 0 || desc->n == 0 || desc->k == 0) return PLB_OK;
  const Ld ld = leadingDims(*desc);
  const bool b_is_nk = desc->transpose_b || desc->input_type == PLB_QUARTER;
  IgemmProblem p = gemmProblem(*desc, nullptr, ld.a, nullptr, ld.b, b_is_nk, nullptr, nullptr, ld.c);
  if (int rc = planIgemm(p, 148, plan)) return rc;
  const size_t es = dtypeBytes(desc->input_type);
  if (desc->transpose_a) plan->workspace_bytes += size_t(desc->groups) * desc->m * desc->k * es;
  if (!desc->transpose_b && desc->input_type == PLB_QUARTER)
    plan->workspace_bytes += size_t(desc->groups) * desc->n * desc->k * es;
  return PLB_OK;
}

int plb_matmul(plb_context *ctx, const plb_matmul_desc *desc, const void *d_a, const void *d_b,
               const void *d_c, void *d_d) {
  TraceRange trace_range("plb_matmul");
  if (int rc = activate(ctx)) return rc;
  if (!desc) return fail(PLB_ERR_INVALID_PARAMS, "null descriptor");
  const plb_matmul_desc &d = *desc;
  if (int rc = checkMatmulDesc(d)) return rc;
  if (d.groups == 0 || d.m == 0 || d.n == 0) return PLB_OK;
  if (d.beta != 0.f && d_c == nullptr)
    return fail(PLB_ERR_INVALID_PARAMS, "beta != 0 needs a C matrix");
  if (d_d == nullptr || (d.k != 0 && (d_a == nullptr || d_b == nullptr)))
    return fail(PLB_ERR_INVALID_PARAMS, "null device pointer for a matrix that has elements");
  const Ld ld = leadingDims(d);
  const size_t es = dtypeBytes(d.input_type), os = dtypeBytes(d.output_type);
  if (d.k == 0) {
    // empty reduction: D = beta * C
    for (uint32_t g = 0; g < d.groups; ++g) {
      const size_t off = size_t(g) * d.m * ld.c * os;
      if (int rc = launchScaleRows(ctx, static_cast<uint8_t *>(d_d) + off,
                                   d_c ? static_cast<const uint8_t *>(d_c) + off : nullptr,
                                   d.beta, d.output_type == PLB_FLOAT, d.m, d.n, ld.c, ld.c))
        return rc;
    }
    return PLB_OK;
  }
  if (d.input_type == PLB_FLOAT) return floatMatmul(ctx, d, d_a, d_b, d_c, d_d);
  // operand layouts the kernel takes directly: A as [m][k]; B as [n][k], or
  // (half only) [k][n].  Anything else goes through a transpose into scratch.
  const uint8_t *a = static_cast<const uint8_t *>(d_a);
  const uint8_t *b = static_cast<const uint8_t *>(d_b);
  long long lda = ld.a, ldb = ld.b;
  bool b_is_nk = d.transpose_b != 0;
  size_t scratch_bytes = 0;
  const size_t a_bytes = size_t(d.groups) * d.m * d.k * es, b_bytes = size_t(d.groups) * d.n * d.k * es;
  const bool transpose_b_now = !d.transpose_b && d.input_type == PLB_QUARTER;
  if (d.transpose_a) scratch_bytes += (a_bytes + 255) & ~size_t(255);
  if (transpose_b_now) scratch_bytes += b_bytes;
  if (scratch_bytes) {
    void *ws = nullptr;
    if (int rc = scratch(ctx, kSlotOperands, scratch_bytes, &ws)) return rc;
    uint8_t *cursor = static_cast<uint8_t *>(ws);
    if (d.transpose_a) {
      if (ld.a != (long long)d.m)
        return fail(PLB_ERR_UNSUPPORTED, "transposed A must be densely packed");
      if (int rc = plb_transpose_matrix(ctx, uint32_t(es), d.groups, d.k, d.m, d_a, cursor)) return rc;
      a = cursor;
      lda = d.k;
      cursor += (a_bytes + 255) & ~size_t(255);
    }
    if (transpose_b_now) {
      if (ld.b != (long long)d.n)
        return fail(PLB_ERR_UNSUPPORTED, "quarter B in [k][n] layout must be densely packed");
      if (int rc = plb_transpose_matrix(ctx, uint32_t(es), d.groups, d.k, d.n, d_b, cursor)) return rc;
      b = cursor;
      ldb = d.k;
      b_is_nk = true;
    }
  }
  // Operands whose rows TMA cannot address (base or row pitch not a multiple of
  // 16 bytes: a [k][n] right matrix with n % 8 != 0, odd leading dimensions)
  // are copied once into scratch with the pitch rounded up and the padding
  // zeroed, the way the convolution path pads channel counts.  The output needs
  // no such copy: the epilogue falls back to plain stores.
  {
    const size_t a_rows = size_t(d.groups) * d.m, b_rows = size_t(d.groups) * (b_is_nk ? d.n : d.k);
    const size_t a_cols = d.k, b_cols = b_is_nk ? d.k : d.n;
    auto unaligned = [&](const uint8_t *base, long long pitch) {
      return (reinterpret_cast<uintptr_t>(base) & 15) != 0 || (size_t(pitch) * es) % 16 != 0;
    };
    const bool pad_a = unaligned(a, lda), pad_b = unaligned(b, ldb);
    if (pad_a || pad_b) {
      const size_t per16 = 16 / es;
      const size_t a_pitch = (a_cols + per16 - 1) / per16 * per16, b_pitch = (b_cols + per16 - 1) / per16 * per16;
      const size_t a_pad_bytes = pad_a ? ((a_rows * a_pitch * es + 255) & ~size_t(255)) : 0;
      const size_t b_pad_bytes = pad_b ? b_rows * b_pitch * es : 0;
      void *ws = nullptr;
      if (int rc = scratch(ctx, kSlotPaddedChans, a_pad_bytes + b_pad_bytes + 256, &ws)) return rc;
      uint8_t *cursor = static_cast<uint8_t *>(ws);
      // (all groups' rows are uniformly `pitch` elements apart)
      auto repitch = [&](const uint8_t *src, long long src_pitch, size_t rows, size_t cols,
                         size_t dst_pitch, uint8_t *dst) -> int {
        return copyRowsPitched(ctx, src, size_t(src_pitch) * es, dst, dst_pitch * es, rows, cols * es);
      };
      if (pad_a) {
        if (int rc = repitch(a, lda, a_rows, a_cols, a_pitch, cursor)) return rc;
        a = cursor;
        lda = (long long)a_pitch;
        cursor += a_pad_bytes;
      }
      if (pad_b) {
        if (int rc = repitch(b, ldb, b_rows, b_cols, b_pitch, cursor)) return rc;
        b = cursor;
        ldb = (long long)b_pitch;
      }
    }
  }
  for (uint32_t g = 0; g < d.groups; ++g) {
    const uint8_t *ag = a + size_t(g) * d.m * lda * es;
    const uint8_t *bg = b + size_t(g) * (b_is_nk ? d.n : d.k) * ldb * es;
    const size_t coff = size_t(g) * d.m * ld.c * os;
    IgemmProblem p = gemmProblem(d, ag, lda, bg, ldb, b_is_nk,
                                 d_c ? static_cast<const uint8_t *>(d_c) + coff : nullptr,
                                 static_cast<uint8_t *>(d_d) + coff, ld.c);
    p.plan_flags |= ctx->plan_flags;
    plb_plan plan{};
    if (int rc = planIgemm(p, ctx->sm_count, &plan)) return rc;
    if (int rc = launchIgemm(ctx, p, plan)) return rc;
  }
  return PLB_OK;
}

int plb_matmul_host(plb_context *ctx, const plb_matmul_desc *desc, const void *h_a,
                    const void *h_b, const void *h_c, void *h_d) {
  if (int rc = plb_matmul_host_async(ctx, desc, h_a, h_b, h_c, h_d)) return rc;
  return plb_synchronize(ctx);
}

int plb_matmul_host_async(plb_context *ctx, const plb_matmul_desc *desc, const void *h_a,
                          const void *h_b, const void *h_c, void *h_d) {
  if (int rc = activate(ctx)) return rc;
  if (!desc) return fail(PLB_ERR_INVALID_PARAMS, "null descriptor");
  const plb_matmul_desc &d = *desc;
  if (int rc = checkMatmulDesc(d)) return rc;
  const Ld ld = leadingDims(d);
  const size_t es = dtypeBytes(d.input_type), os = dtypeBytes(d.output_type);
  const size_t a_bytes = size_t(d.groups) * (d.transpose_a ? d.k : d.m) * ld.a * es;
  const size_t b_bytes = size_t(d.groups) * (d.transpose_b ? d.n : d.k) * ld.b * es;
  const size_t c_bytes = size_t(d.groups) * d.m * ld.c * os;
  void *da = nullptr, *db = nullptr, *dc = nullptr, *dd = nullptr;
  if (int rc = scratch(ctx, kSlotHostIn, a_bytes + 16, &da)) return rc;
  if (int rc = scratch(ctx, kSlotHostWeights, b_bytes + 16, &db)) return rc;
  if (int rc = scratch(ctx, kSlotHostOut, c_bytes + 16, &dd)) return rc;
  if (d.beta != 0.f) {
    if (!h_c) return fail(PLB_ERR_INVALID_PARAMS, "beta != 0 needs a C matrix");
    if (int rc = scratch(ctx, kSlotHostBias, c_bytes + 16, &dc)) return rc;
    if (int rc = plb_memcpy_h2d(ctx, dc, h_c, c_bytes)) return rc;
  }
  if (int rc = plb_memcpy_h2d(ctx, da, h_a, a_bytes)) return rc;
  if (int rc = plb_memcpy_h2d(ctx, db, h_b, b_bytes)) return rc;
  if (int rc = plb_matmul(ctx, desc, da, db, dc, dd)) return rc;
  // enqueued only: the caller synchronises (plb_synchronize) before reading h_d
  if (c_bytes) PLB_CUDA(cudaMemcpyAsync(h_d, dd, c_bytes, cudaMemcpyDeviceToHost, ctx->stream));
  return PLB_OK;
}

// ---------------------------------------------------------------------------

int plb_conv_validate(const plb_conv_params *p) {
  if (!p) return fail(PLB_ERR_INVALID_PARAMS, "null params");
  const std::string err = validate(*p);
  return err.empty() ? PLB_OK : fail(PLB_ERR_INVALID_PARAMS, err);
}

int plb_conv_output_field(const plb_conv_params *p, uint32_t out_field[PLB_MAX_FIELD_DIMS]) {
  if (int rc = plb_conv_validate(p)) return rc;
  for (unsigned d = 0; d != p->num_field_dims; ++d) out_field[d] = uint32_t(outputSize(*p, d));
  return PLB_OK;
}

int plb_conv_input_index(const plb_conv_params *p, uint32_t dim, uint32_t out_index,
                         uint32_t kernel_index) {
  if (!p || dim >= p->num_field_dims) return -1;
  return inputIndex(*p, dim, out_index, kernel_index);
}

uint64_t plb_conv_macs(const plb_conv_params *p) { return p ? numberOfMacs(*p) : 0; }

int plb_conv_plan(const plb_conv_params *p_in, const plb_conv_options *opt, int32_t pass,
                  plb_plan *plan) {
  if (!p_in || !plan) return fail(PLB_ERR_INVALID_PARAMS, "null argument");
  if (p_in->input_type == PLB_FLOAT) {
    // what runs: bfloat16 operands, three terms per product (float_route.cu)
    const std::string err = validate(*p_in);
    if (!err.empty()) return fail(PLB_ERR_INVALID_PARAMS, err);
    const plb_conv_params q = floatRouteConvParams(*p_in, pass);
    if (int rc = plb_conv_plan(&q, opt, pass, plan)) return rc;
    plan->flops = 2 * numberOfMacs(*p_in);
    size_t n_in, n_w, n_out;
    convElementCounts(*p_in, &n_in, &n_w, &n_out);
    plan->workspace_bytes += ((pass == PLB_PASS_TRAINING_BWD ? n_out : n_in) + n_w) * 6 + 768;
    return PLB_OK;
  }
  if (p_in->num_field_dims == 3) return conv3dPlan(*p_in, opt, pass, plan);
  // a flipped input runs as the ordinary convolution of the reversed tensor
  plb_conv_params unflipped, undilated;
  const plb_conv_params *p = unflippedInputParams(*p_in, &unflipped) ? &unflipped : p_in;
  DilatedField df;
  // a dilated input runs as the ordinary convolution of the zero-stuffed tensor
  if (undilatedInputParams(*p, &undilated, &df)) p = &undilated;
  ConvShape s;
  if (int rc = igemmConvShape(*p, &s)) return rc;
  *plan = plb_plan{};
  if (pass != PLB_PASS_TRAINING_BWD && !channelsFitTma(*p, p->in_chans_per_group)) {
    const int rc = convFwdSmallChannels(nullptr, *p, opt, nullptr, nullptr, nullptr, nullptr, plan);
    if (rc == PLB_OK) {
      plan->flops = 2 * numberOfMacs(*p);
      plan->bytes = convBytes(*p, s, pass);
      return PLB_OK;
    }
    if (rc != PLB_ERR_UNSUPPORTED) return rc;
  }
  // channel counts TMA cannot address run zero-padded: plan what will run
  plb_conv_params padded = *p;
  const PaddedChans pc = paddedChans(*p);
  if (pc.needed && (pass == PLB_PASS_TRAINING_BWD || !channelsFitTma(*p, pc.ci))) {
    padded.in_chans_per_group = pc.cip;
    padded.out_chans_per_group = pc.cop;
  }
  IgemmProblem q;
  if (pass == PLB_PASS_TRAINING_BWD) {
    if (int rc = convBwdProblem(padded, opt, s, 0, nullptr, nullptr, nullptr,
                                p->input_type == PLB_QUARTER, &q))
      return rc;
  } else {
    if (int rc = convFwdProblem(padded, opt, s, 0, nullptr, nullptr, nullptr, nullptr, &q)) return rc;
  }
  if (q.n_total > 0 && q.out_w > 0 && q.out_h > 0 && q.out_n > 0 && q.k_per_tap > 0)
    if (int rc = planIgemm(q, 148, plan)) return rc;
  plan->flops = 2 * numberOfMacs(*p);
  plan->bytes = convBytes(*p, s, pass);
  return PLB_OK;
}

int plb_convolution(plb_context *ctx, const plb_conv_params *p, const plb_conv_options *opt,
                    const void *d_in, const void *d_weights, const float *d_bias, void *d_out,
                    int transpose_and_flip_weights) {
  TraceRange trace_range("plb_convolution");
  if (int rc = activate(ctx)) return rc;
  if (!p) return fail(PLB_ERR_INVALID_PARAMS, "null params");
  {
    size_t n_in, n_w, n_out;
    convElementCounts(*p, &n_in, &n_w, &n_out);
    if (n_in == 0 || n_w == 0) n_in = n_w = 0;  // nothing is read: the output is zero (or the bias)
    if (int rc = checkConvRequest(*p, false, d_in, n_out ? n_in : 0, d_weights, n_out ? n_w : 0, d_out, n_out))
      return rc;
  }
  if (p->input_type == PLB_FLOAT) {
    const std::string err = validate(*p);
    if (!err.empty()) return fail(PLB_ERR_INVALID_PARAMS, err);
    return floatConvFwd(ctx, *p, opt, d_in, d_weights, d_bias, d_out, transpose_and_flip_weights);
  }
  if (p->num_field_dims == 3)
    return conv3dFwd(ctx, *p, opt, d_in, d_weights, d_bias, d_out, transpose_and_flip_weights);
  {
    // a flipped input: reverse it once (scratch slot 8), then an ordinary convolution
    plb_conv_params q;
    if (unflippedInputParams(*p, &q) && p->num_field_dims <= 2) {
      const std::string err = validate(*p);
      if (!err.empty()) return fail(PLB_ERR_INVALID_PARAMS, err);
      const bool two = p->num_field_dims == 2;
      const uint32_t H = two ? p->field[0] : 1, W = p->field[two ? 1 : 0];
      const size_t px = size_t(p->groups) * p->in_chans_per_group * dtypeBytes(p->input_type);
      void *xf = nullptr;
      if (int rc = scratch(ctx, kSlotFlipped, size_t(p->batch) * H * W * px + 256, &xf)) return rc;
      if (int rc = flipField(ctx, d_in, xf, p->batch, H, W, px, two && p->in_flip[0],
                             p->in_flip[two ? 1 : 0] != 0))
        return rc;
      return plb_convolution(ctx, &q, opt, xf, d_weights, d_bias, d_out, transpose_and_flip_weights);
    }
  }
  {
    // a dilated input: write the zero-stuffed tensor once (scratch slot 12)
    plb_conv_params q;
    DilatedField df;
    if (undilatedInputParams(*p, &q, &df)) {
      const std::string err = validate(*p);
      if (!err.empty()) return fail(PLB_ERR_INVALID_PARAMS, err);
      const size_t px = size_t(p->groups) * p->in_chans_per_group * dtypeBytes(p->input_type);
      void *xd = nullptr;
      if (int rc = scratch(ctx, kSlotDilated, size_t(p->batch) * df.Hd * df.Wd * px + 256, &xd)) return rc;
      if (int rc = dilateField(ctx, d_in, xd, p->batch, df, px, false)) return rc;
      return plb_convolution(ctx, &q, opt, xd, d_weights, d_bias, d_out, transpose_and_flip_weights);
    }
  }
  ConvShape s;
  if (int rc = igemmConvShape(*p, &s)) return rc;
  if (p->batch == 0 || p->groups == 0 || p->out_chans_per_group == 0 || s.OH == 0 || s.OW == 0)
    return PLB_OK;
  if (p->in_chans_per_group == 0)
    return fail(PLB_ERR_UNSUPPORTED, "zero input channels are not implemented on this path yet");
  if (s.zero_fill_out || s.OHc <= 0 || s.OWc <= 0 || s.He <= 0 || s.We <= 0) {
    // padded output positions (and everything, if nothing is computed) hold
    // zero, or the bias alone
    const size_t chans = size_t(p->groups) * p->out_chans_per_group;
    const size_t total = size_t(p->batch) * s.OH * s.OW * chans;
    if (d_bias) {
      const int grid = int(std::min<size_t>((total + 255) / 256, size_t(ctx->sm_count) * 16));
      if (p->output_type == PLB_FLOAT)
        fillBiasKernel<float><<<grid, 256, 0, ctx->stream>>>(static_cast<float *>(d_out), d_bias, total, chans);
      else
        fillBiasKernel<__half><<<grid, 256, 0, ctx->stream>>>(static_cast<__half *>(d_out), d_bias, total, chans);
      PLB_CUDA(cudaGetLastError());
      ctx->launches++;
    } else {
      PLB_CUDA(cudaMemsetAsync(d_out, 0, total * dtypeBytes(p->output_type), ctx->stream));
    }
    if (s.OHc <= 0 || s.OWc <= 0 || s.He <= 0 || s.We <= 0) return PLB_OK;
  }
  if (!channelsFitTma(*p, p->in_chans_per_group) && !transpose_and_flip_weights) {
    // few input channels (a stem): space-to-depth path, where it applies
    const int rc = convFwdSmallChannels(ctx, *p, opt, d_in, d_weights, d_bias, d_out, nullptr);
    if (rc != PLB_ERR_UNSUPPORTED) return rc;
  }
  const PaddedChans pc = paddedChans(*p);
  if (pc.needed && !channelsFitTma(*p, pc.ci)) {
    // run on zero-padded channel counts
    const size_t es = dtypeBytes(p->input_type), os = dtypeBytes(p->output_type);
    const size_t G = p->groups, taps = size_t(s.KHs) * s.KWs;
    const size_t in_px = size_t(p->batch) * s.H * s.W, out_px = size_t(p->batch) * s.OH * s.OW;
    const size_t x_b = align256(in_px * G * pc.cip * es), w_b = align256(G * taps * pc.cop * pc.cip * es),
                 o_b = align256(out_px * G * pc.cop * os), b_b = align256(G * pc.cop * sizeof(float));
    void *arena = nullptr;
    if (int rc = scratch(ctx, kSlotPaddedChans, x_b + 2 * w_b + o_b + b_b, &arena)) return rc;
    uint8_t *xp = static_cast<uint8_t *>(arena), *wp = xp + x_b, *wtmp = wp + w_b, *op = wtmp + w_b,
            *bp = op + o_b;
    if (int rc = resizeRows(ctx, d_in, xp, in_px * G, pc.ci * es, pc.cip * es)) return rc;
    // stored [G][taps][Co][Ci], or [G][taps][Ci][Co] for transposed weights
    if (transpose_and_flip_weights) {
      if (int rc = padWeights(ctx, d_weights, wtmp, wp, G * taps, pc.ci, pc.co, pc.cip, pc.cop, es)) return rc;
    } else {
      if (int rc = padWeights(ctx, d_weights, wtmp, wp, G * taps, pc.co, pc.ci, pc.cop, pc.cip, es)) return rc;
    }
    if (d_bias)
      if (int rc = resizeRows(ctx, d_bias, bp, G, pc.co * sizeof(float), pc.cop * sizeof(float))) return rc;
    plb_conv_params q = *p;
    q.in_chans_per_group = pc.cip;
    q.out_chans_per_group = pc.cop;
    if (int rc = plb_convolution(ctx, &q, opt, xp, wp, d_bias ? reinterpret_cast<const float *>(bp) : nullptr,
                                 op, transpose_and_flip_weights))
      return rc;
    return resizeRows(ctx, op, d_out, out_px * G, pc.cop * os, pc.co * os);
  }
  if (s.strH > 1 || s.strW > 1) {
    const bool pointwise = s.KH == 1 && s.KW == 1 && s.padH == 0 && s.padW == 0;
    if (!pointwise && (s.strH > 8 || s.strW > 8))
      return fail(PLB_ERR_UNSUPPORTED, "strides above 8 are not implemented for k > 1");
  }
  const size_t es = dtypeBytes(p->input_type);
  if (s.KH <= 0 || s.KW <= 0) {
    // every tap is truncated away: the result is zero
    PLB_CUDA(cudaMemsetAsync(d_out, 0,
                             size_t(p->batch) * s.OH * s.OW * p->groups * p->out_chans_per_group *
                                 dtypeBytes(p->output_type),
                             ctx->stream));
    return PLB_OK;
  }
  const void *w = nullptr;
  if (int rc = usedTaps(ctx, *p, s, d_weights, &w)) return rc;
  const void *const w_used = w;
  bool swapped = transpose_and_flip_weights != 0;
  if (swapped && (p->input_type == PLB_QUARTER || !channelsFitTma(*p, p->out_chans_per_group))) {
    // no MN-major path for 8-bit operands (or for rows TMA cannot address):
    // transpose + flip the (small) weights into scratch, then run as usual
    const size_t bytes = size_t(p->groups) * s.KH * s.KW * p->in_chans_per_group *
                         p->out_chans_per_group * es;
    void *ws = nullptr;
    if (int rc = scratch(ctx, kSlotOperands, bytes, &ws)) return rc;
    // stored [G][k][Ci][Co] -> [G][flipped k][Co][Ci]
    if (int rc = plb_weights_transpose_chans_flip_xy(ctx, uint32_t(es), p->groups,
                                                     p->in_chans_per_group, p->out_chans_per_group,
                                                     uint64_t(s.KH) * s.KW, w_used, ws))
      return rc;
    w = ws;
    swapped = false;
  }
  for (unsigned g = 0; g < p->groups; ++g) {
    IgemmProblem q;
    if (int rc = convFwdProblem(*p, opt, s, g, d_in, w, d_bias, d_out, &q, swapped)) return rc;
    q.plan_flags |= ctx->plan_flags;
    plb_plan plan{};
    if (int rc = planIgemm(q, ctx->sm_count, &plan)) return rc;
    if (int rc = launchIgemm(ctx, q, plan)) return rc;
  }
  return PLB_OK;
}

int plb_conv_fwd(plb_context *ctx, const plb_conv_params *p, const plb_conv_options *opt,
                 const void *d_in, const void *d_weights, const float *d_bias, void *d_out) {
  return plb_convolution(ctx, p, opt, d_in, d_weights, d_bias, d_out, 0);
}

int plb_conv_bwd(plb_context *ctx, const plb_conv_params *p, const plb_conv_options *opt,
                 const void *d_out_grads, const void *d_weights, void *d_in_grads) {
  TraceRange trace_range("plb_conv_bwd");
  if (int rc = activate(ctx)) return rc;
  if (!p) return fail(PLB_ERR_INVALID_PARAMS, "null params");
  {
    size_t n_in, n_w, n_out;
    convElementCounts(*p, &n_in, &n_w, &n_out);
    if (n_out == 0 || n_w == 0) n_out = n_w = 0;  // nothing is read: the gradient is zero
    if (int rc = checkConvRequest(*p, false, d_out_grads, n_in ? n_out : 0, d_weights, n_in ? n_w : 0,
                                  d_in_grads, n_in))
      return rc;
  }
  if (p->input_type == PLB_FLOAT) {
    const std::string err = validate(*p);
    if (!err.empty()) return fail(PLB_ERR_INVALID_PARAMS, err);
    return floatConvBwd(ctx, *p, opt, d_out_grads, d_weights, d_in_grads);
  }
  if (p->num_field_dims == 3) return conv3dBwd(ctx, *p, opt, d_out_grads, d_weights, d_in_grads);
  {
    // a flipped input: the gradient of the reversed input, reversed back
    plb_conv_params q;
    if (unflippedInputParams(*p, &q) && p->num_field_dims <= 2) {
      const std::string err = validate(*p);
      if (!err.empty()) return fail(PLB_ERR_INVALID_PARAMS, err);
      const bool two = p->num_field_dims == 2;
      const uint32_t H = two ? p->field[0] : 1, W = p->field[two ? 1 : 0];
      const size_t px = size_t(p->groups) * p->in_chans_per_group * dtypeBytes(p->output_type);
      void *gf = nullptr;
      if (int rc = scratch(ctx, kSlotFlipped, size_t(p->batch) * H * W * px + 256, &gf)) return rc;
      if (int rc = plb_conv_bwd(ctx, &q, opt, d_out_grads, d_weights, gf)) return rc;
      return flipField(ctx, gf, d_in_grads, p->batch, H, W, px, two && p->in_flip[0],
                       p->in_flip[two ? 1 : 0] != 0);
    }
  }
  {
    // a dilated input: the gradient of the zero-stuffed tensor (scratch slot 12),
    // of which the lattice elements are the gradient of the input
    plb_conv_params q;
    DilatedField df;
    if (undilatedInputParams(*p, &q, &df)) {
      const std::string err = validate(*p);
      if (!err.empty()) return fail(PLB_ERR_INVALID_PARAMS, err);
      const size_t px = size_t(p->groups) * p->in_chans_per_group * dtypeBytes(p->output_type);
      void *gd = nullptr;
      if (int rc = scratch(ctx, kSlotDilated, size_t(p->batch) * df.Hd * df.Wd * px + 256, &gd)) return rc;
      if (int rc = plb_conv_bwd(ctx, &q, opt, d_out_grads, d_weights, gd)) return rc;
      return dilateField(ctx, gd, d_in_grads, p->batch, df, px, true);
    }
  }
  ConvShape s;
  if (int rc = igemmConvShape(*p, &s)) return rc;
  if (p->batch == 0 || p->groups == 0 || p->in_chans_per_group == 0 || s.H == 0 || s.W == 0)
    return PLB_OK;
  const size_t es = dtypeBytes(p->input_type);
  if (s.zero_fill_in)  // truncated input positions receive no gradient
    PLB_CUDA(cudaMemsetAsync(d_in_grads, 0,
                             size_t(p->batch) * s.H * s.W * p->groups * p->in_chans_per_group *
                                 dtypeBytes(p->output_type),
                             ctx->stream));
  if (s.OHc <= 0 || s.OWc <= 0 || s.He <= 0 || s.We <= 0) {
    if (!s.zero_fill_in)
      PLB_CUDA(cudaMemsetAsync(d_in_grads, 0,
                               size_t(p->batch) * s.H * s.W * p->groups * p->in_chans_per_group *
                                   dtypeBytes(p->output_type),
                               ctx->stream));
    return PLB_OK;
  }
  const PaddedChans pc = paddedChans(*p);
  if (pc.needed) {
    // run on zero-padded channel counts (see plb_convolution)
    const size_t os = dtypeBytes(p->output_type);
    const size_t G = p->groups, taps = size_t(s.KHs) * s.KWs;
    const size_t in_px = size_t(p->batch) * s.H * s.W, out_px = size_t(p->batch) * s.OH * s.OW;
    const size_t dy_b = align256(out_px * G * pc.cop * es), w_b = align256(G * taps * pc.cop * pc.cip * es),
                 dx_b = align256(in_px * G * pc.cip * os);
    void *arena = nullptr;
    if (int rc = scratch(ctx, kSlotPaddedChans, dy_b + 2 * w_b + dx_b, &arena)) return rc;
    uint8_t *dyp = static_cast<uint8_t *>(arena), *wp = dyp + dy_b, *wtmp = wp + w_b, *dxp = wtmp + w_b;
    if (int rc = resizeRows(ctx, d_out_grads, dyp, out_px * G, pc.co * es, pc.cop * es)) return rc;
    if (int rc = padWeights(ctx, d_weights, wtmp, wp, G * taps, pc.co, pc.ci, pc.cop, pc.cip, es)) return rc;
    plb_conv_params q = *p;
    q.in_chans_per_group = pc.cip;
    q.out_chans_per_group = pc.cop;
    if (int rc = plb_conv_bwd(ctx, &q, opt, dyp, wp, dxp)) return rc;
    return resizeRows(ctx, dxp, d_in_grads, in_px * G, pc.cip * os, pc.ci * os);
  }
  if (s.KH <= 0 || s.KW <= 0) {
    if (!s.zero_fill_in)
      PLB_CUDA(cudaMemsetAsync(d_in_grads, 0,
                               size_t(p->batch) * s.H * s.W * p->groups * p->in_chans_per_group *
                                   dtypeBytes(p->output_type),
                               ctx->stream));
    return PLB_OK;
  }
  const void *w = nullptr;
  if (int rc = usedTaps(ctx, *p, s, d_weights, &w)) return rc;
  if (s.strH != 1 || s.strW != 1) return convBwdStrided(ctx, *p, opt, s, d_out_grads, w, d_in_grads);
  const void *const w_used = w;
  bool transposed = false;
  if (p->input_type == PLB_QUARTER) {
    // no MN-major path for 8-bit operands: transpose + flip the (small) weights
    const size_t bytes = size_t(p->groups) * s.KH * s.KW * p->in_chans_per_group *
                         p->out_chans_per_group * es;
    void *ws = nullptr;
    if (int rc = scratch(ctx, kSlotOperands, bytes, &ws)) return rc;
    if (int rc = plb_weights_transpose_chans_flip_xy(ctx, uint32_t(es), p->groups,
                                                     p->out_chans_per_group, p->in_chans_per_group,
                                                     uint64_t(s.KH) * s.KW, w_used, ws))
      return rc;
    w = ws;
    transposed = true;
  }
  for (unsigned g = 0; g < p->groups; ++g) {
    IgemmProblem q;
    if (int rc = convBwdProblem(*p, opt, s, g, d_out_grads, w, d_in_grads, transposed, &q)) return rc;
    q.plan_flags |= ctx->plan_flags;
    plb_plan plan{};
    if (int rc = planIgemm(q, ctx->sm_count, &plan)) return rc;
    if (int rc = launchIgemm(ctx, q, plan)) return rc;
  }
  return PLB_OK;
}

int plb_conv_fwd_host(plb_context *ctx, const plb_conv_params *p, const plb_conv_options *opt,
                      const void *h_in, const void *h_weights, const float *h_bias, void *h_out) {
  if (int rc = plb_conv_fwd_host_async(ctx, p, opt, h_in, h_weights, h_bias, h_out)) return rc;
  return plb_synchronize(ctx);
}

int plb_conv_fwd_host_async(plb_context *ctx, const plb_conv_params *p,
                            const plb_conv_options *opt, const void *h_in, const void *h_weights,
                            const float *h_bias, void *h_out) {
  if (int rc = activate(ctx)) return rc;
  if (!p) return fail(PLB_ERR_INVALID_PARAMS, "null params");
  const std::string err = validate(*p);
  if (!err.empty()) return fail(PLB_ERR_INVALID_PARAMS, err);
  const size_t es = dtypeBytes(p->input_type), os = dtypeBytes(p->output_type);
  size_t in_px = 1, taps = 1, out_px = 1;
  for (unsigned d = 0; d != p->num_field_dims; ++d) {
    in_px *= p->field[d];
    taps *= p->kernel[d];
    out_px *= size_t(outputSize(*p, d));
  }
  const size_t in_bytes = size_t(p->batch) * in_px * p->groups * p->in_chans_per_group * es;
  const size_t w_bytes = size_t(p->groups) * taps * p->in_chans_per_group * p->out_chans_per_group * es;
  const size_t out_bytes = size_t(p->batch) * out_px * p->groups * p->out_chans_per_group * os;
  const size_t bias_bytes = size_t(p->groups) * p->out_chans_per_group * sizeof(float);
  void *di = nullptr, *dw = nullptr, *dout = nullptr, *dbias = nullptr;
  if (int rc = scratch(ctx, kSlotHostIn, in_bytes + 16, &di)) return rc;
  if (int rc = scratch(ctx, kSlotHostWeights, w_bytes + 16, &dw)) return rc;
  if (int rc = scratch(ctx, kSlotHostOut, out_bytes + 16, &dout)) return rc;
  if (h_bias) {
    if (int rc = scratch(ctx, kSlotHostBias, bias_bytes + 16, &dbias)) return rc;
    if (int rc = plb_memcpy_h2d(ctx, dbias, h_bias, bias_bytes)) return rc;
  }
  if (int rc = plb_memcpy_h2d(ctx, di, h_in, in_bytes)) return rc;
  if (int rc = plb_memcpy_h2d(ctx, dw, h_weights, w_bytes)) return rc;
  if (int rc = plb_conv_fwd(ctx, p, opt, di, dw, static_cast<const float *>(dbias), dout)) return rc;
  // enqueued only: the caller synchronises (plb_synchronize) before reading h_out
  if (out_bytes)
    PLB_CUDA(cudaMemcpyAsync(h_out, dout, out_bytes, cudaMemcpyDeviceToHost, ctx->stream));
  return PLB_OK;
}

}  // extern "C"
