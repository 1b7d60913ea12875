// Forward convolution for layers whose input has too few channels for a TMA
// row (the ResNet stem: 3 channels, 7x7, stride 2).  NHWC pixels of 6 bytes
// cannot be addressed by TMA (16-byte granularity), and a 3-channel reduction
// would waste the tensor core's K dimension.  The layer is rewritten as an
// equivalent stride-1 convolution with the horizontal taps folded into K:
//
//  1. space-to-depth: stride s and the padding are absorbed into a rearranged
//     input X2[n][h2][w2][(ph, pw, c)] with C2 = s*s*Cp channels (Cp = channels
//     padded so that a pixel is a multiple of 16 bytes), zero where the
//     original is padding.  The s-strided KHxKW filter becomes a stride-1
//     K2h x K2w filter over X2 (K2 = ceil(K / s)).
//  2. the K2w horizontal taps of one output pixel are K2w consecutive pixels
//     of X2, i.e. one contiguous run of K2w*C2 elements (<= 64): the activation
//     tensor map describes overlapping windows (pixel stride C2 elements,
//     window 64 elements), so each K step is one ordinary 128-byte row per
//     output pixel and the implicit-GEMM kernel runs unchanged with K2h taps.
//
// This is the role the reference gives to its expandDims / outChanFlattenDims
// input transforms for small channel counts (lib/poplin/ConvPlan.cpp:1100-1224,
// lib/poplin/Convolution.cpp:665-978).
#include <cuda_fp16.h>

#include <algorithm>

#include "conv_geometry.h"
#include "runtime.h"

namespace plb {

struct S2dShape {
  int N, H, W, C;       // input
  int s, padH, padW;    // stride (both dims), padding
  int KH, KW;
  int OH, OW;
  int Cp, C2;           // padded channels per original pixel, channels of X2
  int K2h, K2w;         // taps after folding the stride
  int H2, W2;           // extent of X2
};

// X2[n][h2][w2][(ph*s + pw)*Cp + c] = X[n][h2*s + ph - padH][w2*s + pw - padW][c]
__global__ void s2dInputKernel(const __half *__restrict__ x, __half *__restrict__ x2, S2dShape g) {
  // one thread per 8 output halves (16 bytes)
  const size_t vecs_per_pixel = size_t(g.C2) / 8;
  const size_t total = size_t(g.N) * g.H2 * g.W2 * vecs_per_pixel;
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < total;
       i += size_t(gridDim.x) * blockDim.x) {
    const int v = int(i % vecs_per_pixel);
    size_t r = i / vecs_per_pixel;
    const int w2 = int(r % g.W2);
    r /= g.W2;
    const int h2 = int(r % g.H2);
    const int n = int(r / g.H2);
    __align__(16) __half vals[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c2 = v * 8 + j;
      const int sub = c2 / g.Cp, c = c2 - sub * g.Cp;
      const int ph = sub / g.s, pw = sub - ph * g.s;
      const int ih = h2 * g.s + ph - g.padH, iw = w2 * g.s + pw - g.padW;
      __half val = __float2half(0.f);
      if (c < g.C && ih >= 0 && ih < g.H && iw >= 0 && iw < g.W)
        val = x[((size_t(n) * g.H + ih) * g.W + iw) * g.C + c];
      vals[j] = val;
    }
    *reinterpret_cast<uint4 *>(x2 + i * 8) = *reinterpret_cast<const uint4 *>(vals);
  }
}

// The same rearrangement, one (n, h2) row of X2 per block iteration: the s
// input rows that feed it are staged in shared memory with coalesced loads
// (16-byte vectors when the rows are 16-byte aligned), then every thread
// assembles 16-byte output vectors from them.  `lut` maps a channel of X2 to
// (ph, pw, c) once per block instead of dividing per element.
__global__ void __launch_bounds__(128)
s2dInputRowsKernel(const __half *__restrict__ x, __half *__restrict__ x2, S2dShape g,
                   int rows_aligned) {
  extern __shared__ __align__(16) unsigned char s2d_smem[];
  const int row_elems = g.W * g.C;
  const int row_stride = (row_elems + 7) & ~7;  // halves; keeps every staged row 16-byte aligned
  __half *rows = reinterpret_cast<__half *>(s2d_smem);
  int *lut = reinterpret_cast<int *>(s2d_smem + size_t(g.s) * row_stride * 2);
  for (int c2 = threadIdx.x; c2 < g.C2; c2 += blockDim.x) {
    const int sub = c2 / g.Cp, c = c2 - sub * g.Cp;
    const int ph = sub / g.s, pw = sub - ph * g.s;
    lut[c2] = c < g.C ? (ph << 16) | (pw << 8) | c : -1;
  }
  const int vecs_per_pixel = g.C2 / 8;
  const int out_vecs = g.W2 * vecs_per_pixel;
  for (int blk = blockIdx.x; blk < g.N * g.H2; blk += gridDim.x) {
    const int n = blk / g.H2, h2 = blk - n * g.H2;
    __syncthreads();  // previous iteration's readers are done (and the table is written)
    for (int ph = 0; ph < g.s; ++ph) {
      const int ih = h2 * g.s + ph - g.padH;
      if (ih < 0 || ih >= g.H) continue;  // block-uniform
      const __half *src = x + (size_t(n) * g.H + ih) * row_elems;
      __half *dst = rows + ph * row_stride;
      if (rows_aligned) {
        const uint4 *src4 = reinterpret_cast<const uint4 *>(src);
        uint4 *dst4 = reinterpret_cast<uint4 *>(dst);
        for (int v = threadIdx.x; v < row_elems / 8; v += blockDim.x) dst4[v] = src4[v];
      } else {
        for (int e = threadIdx.x; e < row_elems; e += blockDim.x) dst[e] = src[e];
      }
    }
    __syncthreads();
    __half *out_row = x2 + size_t(blk) * g.W2 * g.C2;
    for (int o = threadIdx.x; o < out_vecs; o += blockDim.x) {
      const int w2 = o / vecs_per_pixel, v = o - w2 * vecs_per_pixel;
      __align__(16) __half vals[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int code = lut[v * 8 + j];
        const int ph = code >> 16, pw = (code >> 8) & 0xff, c = code & 0xff;
        const int ih = h2 * g.s + ph - g.padH, iw = w2 * g.s + pw - g.padW;
        __half val = __float2half(0.f);
        if (code >= 0 && ih >= 0 && ih < g.H && iw >= 0 && iw < g.W)
          val = rows[ph * row_stride + iw * g.C + c];
        vals[j] = val;
      }
      *reinterpret_cast<uint4 *>(out_row + size_t(o) * 8) = *reinterpret_cast<const uint4 *>(vals);
    }
  }
}

// W2[a][co][(b*s*s + ph*s + pw)*Cp + c] = W[a*s + ph][b*s + pw][co][c], rows padded to 64:
// element i of the folded weights.
__device__ __forceinline__ __half foldedWeight(const __half *__restrict__ w, const S2dShape &g,
                                               unsigned co_total, unsigned i) {
  const unsigned k = i & 63u;
  const unsigned r = i >> 6;
  const unsigned a = r / co_total, co = r - a * co_total;
  const unsigned b = k / unsigned(g.C2);
  if (b >= unsigned(g.K2w)) return __float2half(0.f);
  const unsigned c2 = k - b * g.C2;
  const unsigned sub = c2 / unsigned(g.Cp), c = c2 - sub * g.Cp;
  const unsigned ph = sub / unsigned(g.s), pw = sub - ph * g.s;
  const unsigned kh = a * g.s + ph, kw = b * g.s + pw;
  if (c < unsigned(g.C) && kh < unsigned(g.KH) && kw < unsigned(g.KW))
    return w[((size_t(kh) * g.KW + kw) * co_total + co) * g.C + c];
  return __float2half(0.f);
}

__global__ void s2dWeightsKernel(const __half *__restrict__ w, __half *__restrict__ w2, S2dShape g,
                                 int co_total) {
  const unsigned total = unsigned(g.K2h) * unsigned(co_total) * 64u;
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x)
    w2[i] = foldedWeight(w, g, unsigned(co_total), i);
}

// The same rearrangement for the common stem shape (3 channels, stride 2, so
// Cp = 4 and one X2 pixel is two 16-byte vectors, one per vertical phase):
// a vector is [X(ih, iw) c0..2, 0, X(ih, iw+1) c0..2, 0], i.e. six consecutive
// halves of one input row.  One block per (n, h2) row of X2, one thread per
// pixel of it (both vectors), so a warp reads one contiguous span of each of
// the two input rows (four aligned 32-bit loads per thread and row,
// overlapping its neighbours' in L1) and writes 1024 contiguous bytes.  No
// shared memory; the only division is one 32-bit one per thread.  The blocks
// past the last row fold the weights and clear the 128 bytes after X2 (they
// only ever meet zero weights, but must be finite), so the layer's
// preparation is one launch.
__global__ void __launch_bounds__(128)
s2dStem3Kernel(const uint32_t *__restrict__ x32, uint4 *__restrict__ x2, S2dShape g,
               const __half *__restrict__ w, __half *__restrict__ w2, int co_total) {
  // the convolution that follows may set itself up meanwhile; it waits for this
  // grid to finish before it reads
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const unsigned rows = unsigned(g.N) * unsigned(g.H2);
  if (blockIdx.x >= rows) {
    const unsigned total = unsigned(g.K2h) * unsigned(co_total) * 64u;
    const unsigned i = (blockIdx.x - rows) * blockDim.x + threadIdx.x;
    if (i < total) w2[i] = foldedWeight(w, g, unsigned(co_total), i);
    if (blockIdx.x == rows && threadIdx.x < 8)
      x2[(size_t(rows) * g.W2 << 1) + threadIdx.x] = make_uint4(0u, 0u, 0u, 0u);
    return;
  }
  const int row_words = g.W * 3 / 2;  // W * 3 is even: rows start on a 32-bit word
  // last rows first: the convolution starts with the first images, which are
  // then the ones most recently written and still in L2
  const unsigned row = rows - 1 - blockIdx.x;
  const unsigned n = row / unsigned(g.H2);
  const int h2 = int(row - n * unsigned(g.H2));
  uint4 *dst = x2 + (size_t(row) * g.W2 << 1);
  for (int w2 = threadIdx.x; w2 < g.W2; w2 += blockDim.x) {
    const int iw = 2 * w2 - g.padW;
    const bool cols = iw + 1 >= 0 && iw < g.W;
    const int h0 = iw * 3;               // first half wanted, relative to the row (may be negative)
    const int odd = h0 & 1;
    const int w0 = (h0 - odd) >> 1;      // first 32-bit word (exact; arithmetic shift)
    const bool left = iw >= 0, right = iw + 1 < g.W;
    uint4 out[2];
#pragma unroll
    for (int ph = 0; ph < 2; ++ph) {
      const int ih = 2 * h2 + ph - g.padH;
      out[ph] = make_uint4(0u, 0u, 0u, 0u);
      if (cols && ih >= 0 && ih < g.H) {
        const uint32_t *row = x32 + (size_t(n) * g.H + ih) * row_words;
        uint32_t w[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) w[k] = (w0 + k >= 0 && w0 + k < row_words) ? row[w0 + k] : 0u;
        // halves h0 .. h0 + 5 of the 8 loaded
        uint32_t a, b, c;  // (h0,h1) (h2,h3) (h4,h5)
        if (odd) {
          a = __funnelshift_r(w[0], w[1], 16);
          b = __funnelshift_r(w[1], w[2], 16);
          c = __funnelshift_r(w[2], w[3], 16);
        } else {
          a = w[0];
          b = w[1];
          c = w[2];
        }
        // pixel iw: h0 h1 h2; pixel iw + 1: h3 h4 h5
        out[ph].x = left ? a : 0u;
        out[ph].y = left ? (b & 0xffffu) : 0u;
        out[ph].z = right ? ((b >> 16) | (c << 16)) : 0u;
        out[ph].w = right ? (c >> 16) : 0u;
      }
    }
    dst[size_t(w2) << 1] = out[0];
    dst[(size_t(w2) << 1) + 1] = out[1];
  }
}


// Returns PLB_ERR_UNSUPPORTED (with a message) when the layer does not fit this path.
int convFwdSmallChannels(plb_context *ctx, const plb_conv_params &p, const plb_conv_options *opt,
                         const void *d_in, const void *d_weights, const float *d_bias,
                         void *d_out, plb_plan *plan_only) {
  if (p.num_field_dims != 2 || p.groups != 1 || !is16BitFloat(p.input_type))
    return fail(PLB_ERR_UNSUPPORTED,
                "input channel count must be a multiple of 8 (half) / 16 (quarter) unless the "
                "layer is a 2-D, ungrouped half convolution");
  for (unsigned d = 0; d != 2; ++d)
    if (p.in_trunc_lo[d] || p.in_trunc_hi[d] || p.in_dilation[d] != 1 || p.in_flip[d] ||
        p.k_trunc_lo[d] || p.k_trunc_hi[d] || p.k_pad_lo[d] || p.k_pad_hi[d] || p.k_flip[d] ||
        p.k_dilation[d] != 1 || p.out_trunc_lo[d] || p.out_trunc_hi[d] || p.out_pad_lo[d] ||
        p.out_pad_hi[d])
      return fail(PLB_ERR_UNSUPPORTED,
                  "small-channel convolutions support padding and stride only");
  if (p.stride[0] != p.stride[1] || p.stride[0] > 2)
    return fail(PLB_ERR_UNSUPPORTED, "small-channel convolutions need equal strides of 1 or 2");
  S2dShape g{};
  g.N = int(p.batch);
  g.H = int(p.field[0]);
  g.W = int(p.field[1]);
  g.C = int(p.in_chans_per_group);
  g.s = int(p.stride[0]);
  g.padH = int(p.in_pad_lo[0]);
  g.padW = int(p.in_pad_lo[1]);
  g.KH = int(p.kernel[0]);
  g.KW = int(p.kernel[1]);
  g.OH = int(outputSize(p, 0));
  g.OW = int(outputSize(p, 1));
  // pixel of X2 must be a multiple of 16 bytes = 8 halves
  g.Cp = g.C;
  while ((g.s * g.s * g.Cp) % 8 != 0) ++g.Cp;
  g.C2 = g.s * g.s * g.Cp;
  g.K2h = (g.KH + g.s - 1) / g.s;
  g.K2w = (g.KW + g.s - 1) / g.s;
  if (g.K2w * g.C2 > 64)
    return fail(PLB_ERR_UNSUPPORTED,
                "small-channel convolution: folded filter row of " +
                    std::to_string(g.K2w * g.C2) + " elements exceeds one 128-byte K step");
  g.H2 = g.OH + g.K2h - 1;
  g.W2 = g.OW + g.K2w - 1;
  const int co = int(p.out_chans_per_group);
  // tail of the last row: the 64-element window of the last pixel may run past
  // the K2w*C2 elements that carry weights; pad the allocation so it stays inside
  const size_t x2_elems = size_t(g.N) * g.H2 * g.W2 * g.C2 + 64;
  const size_t w2_elems = size_t(g.K2h) * co * 64;

  IgemmProblem q;
  q.act_dims[0] = 64;
  q.act_dims[1] = uint64_t(g.OW);
  q.act_dims[2] = uint64_t(g.H2);
  q.act_dims[3] = uint64_t(g.N);
  q.act_strides[0] = uint64_t(g.C2) * 2;
  q.act_strides[1] = uint64_t(g.W2) * g.C2 * 2;
  q.act_strides[2] = uint64_t(g.H2) * g.W2 * g.C2 * 2;
  q.wgt_dims[0] = 64;
  q.wgt_dims[1] = uint64_t(co);
  q.wgt_dims[2] = uint64_t(g.K2h);
  q.wgt_strides[0] = 128;
  q.wgt_strides[1] = uint64_t(co) * 128;
  q.out_w = g.OW;
  q.out_h = g.OH;
  q.out_n = g.N;
  q.n_total = co;
  q.k_per_tap = 64;
  q.taps_h = g.K2h;
  q.taps_w = 1;
  q.ldc = co;
  q.bias = d_bias;
  q.out_f32 = p.output_type == PLB_FLOAT;
  q.force_tile_n = opt ? opt->tile_n : 0;
  q.plan_flags = opt ? opt->plan_flags : 0;
  // The K loop here is short (K2h steps), below the planner's general threshold
  // for CTA pairs, but with 64 output channels the instruction is bound by its
  // activation operand, which a pair splits between two SMs: measured 197 ->
  // 191 us on the 7x7 stride-2 stem of 256 images.  Taken when there are many tiles.
  const int sms = ctx ? ctx->sm_count : 148;
  if ((q.plan_flags & PLB_PLAN_NO_CTA_PAIR) == 0 &&
      uint64_t(g.OW) * g.OH * g.N >= uint64_t(128) * 8 * sms)
    q.plan_flags |= PLB_PLAN_FORCE_CTA_PAIR;
  plb_plan plan{};
  if (int rc = planIgemm(q, sms, &plan)) return rc;
  plan.kernel = 2;
  plan.workspace_bytes = (x2_elems + w2_elems) * 2;
  if (plan_only) {
    *plan_only = plan;
    return PLB_OK;
  }
  void *ws = nullptr;
  if (int rc = scratch(ctx, kSlotOperands, plan.workspace_bytes + 256, &ws)) return rc;
  __half *x2 = static_cast<__half *>(ws);
  __half *w2 = x2 + ((x2_elems + 127) & ~size_t(127));
  {
    bool fused_prep = false;
    const int row_elems = g.W * g.C;
    const size_t smem = size_t(g.s) * ((row_elems + 7) & ~7) * 2 + size_t(g.C2) * sizeof(int);
    if (g.C == 3 && g.s == 2 && g.Cp == 4 && row_elems % 2 == 0 &&
        (reinterpret_cast<uintptr_t>(d_in) & 3) == 0 && size_t(g.N) * g.H2 < (size_t(1) << 31)) {
      const unsigned wblocks = unsigned((w2_elems + 127) / 128);
      s2dStem3Kernel<<<unsigned(g.N) * unsigned(g.H2) + wblocks, 128, 0, ctx->stream>>>(
          static_cast<const uint32_t *>(d_in), reinterpret_cast<uint4 *>(x2), g,
          static_cast<const __half *>(d_weights), w2, co);
      fused_prep = true;
    } else if (smem <= 48 * 1024 && g.C < 256 && g.s < 256) {
      const int rows_aligned =
          (row_elems % 8 == 0 && (reinterpret_cast<uintptr_t>(d_in) & 15) == 0) ? 1 : 0;
      const int grid = int(std::min<size_t>(size_t(g.N) * g.H2, size_t(ctx->sm_count) * 16));
      s2dInputRowsKernel<<<grid, 128, smem, ctx->stream>>>(static_cast<const __half *>(d_in), x2, g,
                                                           rows_aligned);
    } else {
      const size_t vecs = size_t(g.N) * g.H2 * g.W2 * (g.C2 / 8);
      const int grid = int(std::min<size_t>((vecs + 255) / 256, size_t(ctx->sm_count) * 16));
      s2dInputKernel<<<grid, 256, 0, ctx->stream>>>(static_cast<const __half *>(d_in), x2, g);
    }
    PLB_CUDA(cudaGetLastError());
    ctx->launches++;
    if (!fused_prep) {
      // the 64 trailing elements only ever meet zero weights, but must be finite
      PLB_CUDA(cudaMemsetAsync(x2 + size_t(g.N) * g.H2 * g.W2 * g.C2, 0, 128, ctx->stream));
      const int wgrid = int((w2_elems + 255) / 256);
      s2dWeightsKernel<<<wgrid, 256, 0, ctx->stream>>>(static_cast<const __half *>(d_weights), w2, g,
                                                       co);
      PLB_CUDA(cudaGetLastError());
      ctx->launches++;
    }
  }
  q.act = x2;
  q.wgt = w2;
  q.out = d_out;
  return launchIgemm(ctx, q, plan);
}

}  // namespace plb
