// Float operands (poplar::FLOAT inputs, which the reference accepts next to
// half and quarter: lib/poplin/ConvValidation.cpp:11-70; its tools run
// "--data-type float").  The tensor cores take 16- and 8-bit operands, so a
// float contraction runs as three bfloat16 contractions in one pass:
//
//   x = x_hi + x_lo + O(2^-17 |x|),  x_hi = bf16(x),  x_lo = bf16(x - x_hi)
//   x * w ~= x_hi*w_hi + x_lo*w_hi + x_hi*w_lo         (error O(2^-16 |x w|))
//
// bfloat16 keeps float's exponent range, so no scaling is needed.  The three
// terms are laid side by side along the reduction dimension (x as
// [hi | lo | hi], w as [hi | hi | lo]); what runs is the ordinary kernel on a
// reduction three times as long, with fp32 accumulation as always.  The
// split copies live in one scratch slot.
#include <cuda_bf16.h>

#include <algorithm>

#include "runtime.h"

namespace plb {

namespace {

// in: [outer][mid] rows of `inner` floats, `pitch` elements apart; out: dense
// [outer][3][mid][inner] bfloat16 pieces.  kWeights = false: (hi, lo, hi);
// true: (hi, hi, lo).
template <bool kWeights>
__global__ void __launch_bounds__(256)
splitFloatKernel(const float *__restrict__ in, __nv_bfloat16 *__restrict__ out, size_t outer,
                 size_t mid, size_t inner, size_t pitch) {
  const size_t rows = outer * mid, piece = mid * inner;
  for (size_t row = blockIdx.y * size_t(blockDim.y) + threadIdx.y; row < rows;
       row += size_t(gridDim.y) * blockDim.y) {
    const size_t o = mid == 1 ? row : row / mid, m = row - o * mid;
    const float *src = in + row * pitch;
    __nv_bfloat16 *dst = out + (o * 3 * mid + m) * inner;
    for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < inner;
         i += size_t(gridDim.x) * blockDim.x) {
      const float x = src[i];
      const __nv_bfloat16 hi = __float2bfloat16_rn(x);
      // an infinity or NaN stays in the first piece alone: in the other two it
      // would meet the zero low piece of the other operand and make a NaN of
      // a product that is an infinity
      const bool finite = isfinite(x);
      const __nv_bfloat16 lo = __float2bfloat16_rn(finite ? x - __bfloat162float(hi) : 0.f);
      const __nv_bfloat16 hi2 = finite ? hi : __float2bfloat16_rn(0.f);
      dst[i] = hi;
      dst[piece + i] = kWeights ? hi2 : lo;
      dst[2 * piece + i] = kWeights ? lo : hi2;
    }
  }
}

int splitFloat(plb_context *ctx, const void *in, void *out, size_t outer, size_t mid, size_t inner,
               size_t pitch, bool weights) {
  const size_t rows = outer * mid;
  if (rows == 0 || inner == 0) return PLB_OK;
  // threads along the contiguous dimension, rows across y
  const unsigned bx = inner >= 256 ? 256 : inner >= 128 ? 128 : inner >= 64 ? 64 : 32;
  const unsigned by = 256 / bx;
  const size_t gx = std::min<size_t>((inner + bx - 1) / bx, 2048);
  const size_t gy = std::min<size_t>((rows + by - 1) / by,
                                     std::max<size_t>(1, size_t(ctx->sm_count) * 32 / gx));
  const dim3 grid{unsigned(gx), unsigned(std::min<size_t>(gy, 65535)), 1}, block{bx, by, 1};
  if (weights)
    splitFloatKernel<true><<<grid, block, 0, ctx->stream>>>(
        static_cast<const float *>(in), static_cast<__nv_bfloat16 *>(out), outer, mid, inner, pitch);
  else
    splitFloatKernel<false><<<grid, block, 0, ctx->stream>>>(
        static_cast<const float *>(in), static_cast<__nv_bfloat16 *>(out), outer, mid, inner, pitch);
  PLB_CUDA(cudaGetLastError());
  ctx->launches++;
  return PLB_OK;
}

// Dense [outer][inner] -> [outer][3][inner].
int splitFloat(plb_context *ctx, const void *in, void *out, size_t outer, size_t inner,
               bool weights) {
  return splitFloat(ctx, in, out, outer, 1, inner, inner, weights);
}

size_t align256(size_t n) { return (n + 255) & ~size_t(255); }

// Scratch for two split tensors of n_a and n_b floats.
int splitScratch(plb_context *ctx, size_t n_a, size_t n_b, void **a, void **b) {
  void *arena = nullptr;
  const size_t a_bytes = align256(n_a * 3 * 2);
  if (int rc = scratch(ctx, kSlotFloatSplit, a_bytes + align256(n_b * 3 * 2) + 256, &arena)) return rc;
  *a = arena;
  *b = static_cast<uint8_t *>(arena) + a_bytes;
  return PLB_OK;
}

}  // namespace

plb_conv_params floatRouteConvParams(const plb_conv_params &p, int pass) {
  plb_conv_params q = p;
  q.input_type = PLB_BFLOAT16;
  if (pass == PLB_PASS_TRAINING_BWD)
    q.out_chans_per_group *= 3;
  else if (pass == PLB_PASS_TRAINING_WU)
    q.batch *= 3;
  else
    q.in_chans_per_group *= 3;
  return q;
}

plb_matmul_desc floatRouteMatmulDesc(const plb_matmul_desc &d) {
  plb_matmul_desc q = d;
  q.input_type = PLB_BFLOAT16;
  q.k *= 3;
  q.lda = q.ldb = 0;
  return q;
}

int floatConvFwd(plb_context *ctx, const plb_conv_params &p, const plb_conv_options *opt,
                 const void *d_in, const void *d_weights, const float *d_bias, void *d_out,
                 int transpose_and_flip_weights) {
  size_t n_in, n_w, n_out;
  convElementCounts(p, &n_in, &n_w, &n_out);
  const size_t ci = p.in_chans_per_group, co = p.out_chans_per_group;
  void *x = nullptr, *w = nullptr;
  if (int rc = splitScratch(ctx, n_in, n_w, &x, &w)) return rc;
  if (ci != 0) {
    // activations [pixel][group][ci] -> [pixel][group][hi | lo | hi]
    if (int rc = splitFloat(ctx, d_in, x, n_in / ci, ci, false)) return rc;
    // weights [group][tap][co][ci] -> [..][co][hi | hi | lo]; stored transposed,
    // [group][tap][ci][co] -> [group][tap][hi | hi | lo][co]
    if (transpose_and_flip_weights && co != 0) {
      if (int rc = splitFloat(ctx, d_weights, w, n_w / (ci * co), ci * co, true)) return rc;
    } else {
      if (int rc = splitFloat(ctx, d_weights, w, n_w / ci, ci, true)) return rc;
    }
  }
  const plb_conv_params q = floatRouteConvParams(p, PLB_PASS_TRAINING_FWD);
  return plb_convolution(ctx, &q, opt, x, w, d_bias, d_out, transpose_and_flip_weights);
}

int floatConvBwd(plb_context *ctx, const plb_conv_params &p, const plb_conv_options *opt,
                 const void *d_out_grads, const void *d_weights, void *d_in_grads) {
  size_t n_in, n_w, n_out;
  convElementCounts(p, &n_in, &n_w, &n_out);
  const size_t ci = p.in_chans_per_group, co = p.out_chans_per_group;
  void *dy = nullptr, *w = nullptr;
  if (int rc = splitScratch(ctx, n_out, n_w, &dy, &w)) return rc;
  if (co != 0) {
    // the reduction runs over the output channels
    if (int rc = splitFloat(ctx, d_out_grads, dy, n_out / co, co, false)) return rc;
    if (ci != 0)
      if (int rc = splitFloat(ctx, d_weights, w, n_w / (co * ci), co * ci, true)) return rc;
  }
  const plb_conv_params q = floatRouteConvParams(p, PLB_PASS_TRAINING_BWD);
  return plb_conv_bwd(ctx, &q, opt, dy, w, d_in_grads);
}

int floatConvWu(plb_context *ctx, const plb_conv_params &p, const plb_conv_options *opt,
                const void *d_acts, const void *d_out_grads, void *d_weight_grads,
                float *d_weight_grads_f32) {
  size_t n_in, n_w, n_out;
  convElementCounts(p, &n_in, &n_w, &n_out);
  void *x = nullptr, *dy = nullptr;
  if (int rc = splitScratch(ctx, n_in, n_out, &x, &dy)) return rc;
  // the reduction runs over the batch (and the field): three batches side by side
  if (int rc = splitFloat(ctx, d_acts, x, 1, n_in, false)) return rc;
  if (int rc = splitFloat(ctx, d_out_grads, dy, 1, n_out, true)) return rc;
  const plb_conv_params q = floatRouteConvParams(p, PLB_PASS_TRAINING_WU);
  // a float layer's weight gradient is float either way
  float *result = d_weight_grads_f32 ? d_weight_grads_f32 : static_cast<float *>(d_weight_grads);
  if (int rc = plb_conv_wu(ctx, &q, opt, x, dy, nullptr, result)) return rc;
  if (d_weight_grads && d_weight_grads != static_cast<void *>(result))
    PLB_CUDA(cudaMemcpyAsync(d_weight_grads, result, n_w * sizeof(float), cudaMemcpyDeviceToDevice,
                             ctx->stream));
  return PLB_OK;
}

int floatMatmul(plb_context *ctx, const plb_matmul_desc &d, const void *d_a, const void *d_b,
                const void *d_c, void *d_d) {
  const size_t g = d.groups, m = d.m, k = d.k, n = d.n;
  const size_t lda = d.lda ? size_t(d.lda) : (d.transpose_a ? m : k);
  const size_t ldb = d.ldb ? size_t(d.ldb) : (d.transpose_b ? k : n);
  if (lda < (d.transpose_a ? m : k) || ldb < (d.transpose_b ? k : n))
    return fail(PLB_ERR_INVALID_PARAMS, "leading dimension shorter than a row");
  void *a = nullptr, *b = nullptr;
  if (int rc = splitScratch(ctx, g * m * k, g * k * n, &a, &b)) return rc;
  // A [g][m][k] -> [g][m][hi | lo | hi];  stored [g][k][m] -> [g][hi | lo | hi][m]
  if (d.transpose_a) {
    if (int rc = splitFloat(ctx, d_a, a, g, k, m, lda, false)) return rc;
  } else {
    if (int rc = splitFloat(ctx, d_a, a, g * m, 1, k, lda, false)) return rc;
  }
  // B [g][k][n] -> [g][hi | hi | lo][n];  stored [g][n][k] -> [g][n][hi | hi | lo]
  if (d.transpose_b) {
    if (int rc = splitFloat(ctx, d_b, b, g * n, 1, k, ldb, true)) return rc;
  } else {
    if (int rc = splitFloat(ctx, d_b, b, g, k, n, ldb, true)) return rc;
  }
  // the pieces are densely packed
  const plb_matmul_desc q = floatRouteMatmulDesc(d);
  return plb_matmul(ctx, &q, a, b, d_c, d_d);
}

}  // namespace plb
