// 3-D fields.  The outermost field dimension (depth) is folded into the
// channels so that the 2-D kernels run unchanged, with one rounding of the fp32
// sums as in a native 3-D convolution:
//
//   forward / weight update   X'[n*OD + od][h][w][g][kd*Ci + ci] = x[n][in(od, kd)][h][w][g][ci]
//                             (zero where (od, kd) meets padding, a dilation hole or a truncated
//                             element), then a 2-D convolution with KD*Ci input channels
//   backward                  DY'[n*D + id][oh][ow][g][kd*Co + co] = dy[n][out(id, kd)][oh][ow][g][co],
//                             then the 2-D backward pass with KD*Co output channels
//
// in(o, k) is poplin::getInputIndex for the depth dimension
// (lib/poplin/ConvUtil.cpp:234-292), out(i, k) its inverse, so every input,
// kernel and output transform of the depth dimension (truncation, dilation,
// padding, flips, stride) is absorbed by the gather.  The cost is one extra pass
// that writes and re-reads KD copies of the activations.
#include <algorithm>
#include <string>

#include "conv_geometry.h"
#include "runtime.h"

namespace plb {

namespace {

// The transforms of one dimension, for index arithmetic on the device.
struct DepthMap {
  int in_size, k_size, out_size;
  int in_trunc_lo, in_trunc_hi, in_dil, in_pad_lo, in_flip, in_tsize;
  int k_trunc_lo, k_trunc_hi, k_dil, k_pad_lo, k_flip, k_tsize;
  int out_trunc_lo, stride, out_pad_lo, out_pad_hi;
};

// Position of kernel element k in the transformed kernel, -1 if truncated away.
__host__ __device__ inline int kernelPos(const DepthMap &m, int k) {
  if (k < m.k_trunc_lo || k >= m.k_size - m.k_trunc_hi) return -1;
  const int pos = (k - m.k_trunc_lo) * m.k_dil + m.k_pad_lo;
  return m.k_flip ? m.k_tsize - 1 - pos : pos;
}

// Input element read by (output o, kernel k), or -1.
__host__ __device__ inline int inputOf(const DepthMap &m, int o, int k) {
  if (o < m.out_pad_lo || o >= m.out_size - m.out_pad_hi) return -1;
  const int kpos = kernelPos(m, k);
  if (kpos < 0) return -1;
  int pos = m.out_trunc_lo + (o - m.out_pad_lo) * m.stride + kpos;
  if (pos < 0 || pos >= m.in_tsize) return -1;
  if (m.in_flip) pos = m.in_tsize - 1 - pos;
  pos -= m.in_pad_lo;
  const int truncated = m.in_size - m.in_trunc_lo - m.in_trunc_hi;
  const int dilated = truncated == 0 ? 0 : 1 + (truncated - 1) * m.in_dil;
  if (pos < 0 || pos >= dilated || pos % m.in_dil != 0) return -1;
  return pos / m.in_dil + m.in_trunc_lo;
}

// Output element that reads input i through kernel element k, or -1.
__host__ __device__ inline int outputOf(const DepthMap &m, int i, int k) {
  if (i < m.in_trunc_lo || i >= m.in_size - m.in_trunc_hi) return -1;
  const int kpos = kernelPos(m, k);
  if (kpos < 0) return -1;
  int pos = (i - m.in_trunc_lo) * m.in_dil + m.in_pad_lo;
  if (m.in_flip) pos = m.in_tsize - 1 - pos;
  const int conv = pos - kpos - m.out_trunc_lo;
  if (conv < 0 || conv % m.stride != 0) return -1;
  const int o = conv / m.stride + m.out_pad_lo;
  return o < m.out_size - m.out_pad_hi ? o : -1;
}

template <typename V>
__device__ inline V zeroVec() {
  return V(0);
}
template <>
__device__ inline uint4 zeroVec<uint4>() {
  return make_uint4(0, 0, 0, 0);
}
template <>
__device__ inline uint2 zeroVec<uint2>() {
  return make_uint2(0, 0);
}

// dst[n][dd][pix][g][kd][c] = src[n][map(dd, kd)][pix][g][c], zero where the map has no element.
template <typename V>
__global__ void foldDepthKernel(const V *__restrict__ src, V *__restrict__ dst, DepthMap m,
                                int inverse, uint32_t src_depth, uint32_t dst_depth, uint32_t KD,
                                uint64_t pixels, uint32_t G, uint32_t vecs, uint64_t total) {
  for (uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x; i < total;
       i += uint64_t(gridDim.x) * blockDim.x) {
    uint64_t r = i;
    const uint32_t c = uint32_t(r % vecs);
    r /= vecs;
    const uint32_t kd = uint32_t(r % KD);
    r /= KD;
    const uint32_t g = uint32_t(r % G);
    r /= G;
    const uint64_t pix = r % pixels;
    r /= pixels;
    const uint32_t dd = uint32_t(r % dst_depth);
    const uint64_t n = r / dst_depth;
    const int sd = inverse ? outputOf(m, int(dd), int(kd)) : inputOf(m, int(dd), int(kd));
    V v = zeroVec<V>();
    if (sd >= 0) v = src[(((n * src_depth + uint32_t(sd)) * pixels + pix) * G + g) * vecs + c];
    dst[i] = v;
  }
}

struct Fold3d {
  DepthMap m;
  plb_conv_params p2;  // the two inner dimensions
  uint32_t D, OD, KD;
  uint64_t in_pixels, out_pixels, taps2;  // per depth slice
};

int makeFold(const plb_conv_params &p, Fold3d *f) {
  const std::string err = validate(p);
  if (!err.empty()) return fail(PLB_ERR_INVALID_PARAMS, err);
  if (p.num_field_dims != 3) return fail(PLB_ERR_INVALID_PARAMS, "not a 3-D convolution");
  DepthMap &m = f->m;
  m.in_size = int(p.field[0]);
  m.k_size = int(p.kernel[0]);
  m.out_size = int(outputSize(p, 0));
  m.in_trunc_lo = int(p.in_trunc_lo[0]);
  m.in_trunc_hi = int(p.in_trunc_hi[0]);
  m.in_dil = int(p.in_dilation[0]);
  m.in_pad_lo = int(p.in_pad_lo[0]);
  m.in_flip = int(p.in_flip[0]);
  m.in_tsize = int(transformedInputSize(p, 0));
  m.k_trunc_lo = int(p.k_trunc_lo[0]);
  m.k_trunc_hi = int(p.k_trunc_hi[0]);
  m.k_dil = int(p.k_dilation[0]);
  m.k_pad_lo = int(p.k_pad_lo[0]);
  m.k_flip = int(p.k_flip[0]);
  m.k_tsize = int(transformedKernelSize(p, 0));
  m.out_trunc_lo = int(p.out_trunc_lo[0]);
  m.stride = int(p.stride[0]);
  m.out_pad_lo = int(p.out_pad_lo[0]);
  m.out_pad_hi = int(p.out_pad_hi[0]);
  f->D = p.field[0];
  f->OD = uint32_t(m.out_size);
  f->KD = p.kernel[0];
  // the device arithmetic against the host restatement of getInputIndex
  for (uint32_t o = 0; o < f->OD; ++o)
    for (uint32_t k = 0; k < f->KD; ++k) {
      const int i = inputIndex(p, 0, o, k);
      if (inputOf(m, int(o), int(k)) != i || (i >= 0 && outputOf(m, i, int(k)) != int(o)))
        return fail(PLB_ERR_CUDA, "internal: depth index maps disagree");
    }
  plb_conv_params &q = f->p2;
  q = p;
  q.num_field_dims = 2;
  auto shift = [](uint32_t *v, uint32_t fill) {
    v[0] = v[1];
    v[1] = v[2];
    v[2] = fill;
  };
  shift(q.field, 1);
  shift(q.kernel, 1);
  shift(q.in_trunc_lo, 0);
  shift(q.in_trunc_hi, 0);
  shift(q.in_dilation, 1);
  shift(q.in_pad_lo, 0);
  shift(q.in_pad_hi, 0);
  shift(q.in_flip, 0);
  shift(q.k_trunc_lo, 0);
  shift(q.k_trunc_hi, 0);
  shift(q.k_dilation, 1);
  shift(q.k_pad_lo, 0);
  shift(q.k_pad_hi, 0);
  shift(q.k_flip, 0);
  shift(q.out_trunc_lo, 0);
  shift(q.out_trunc_hi, 0);
  shift(q.stride, 1);
  shift(q.out_pad_lo, 0);
  shift(q.out_pad_hi, 0);
  f->in_pixels = uint64_t(p.field[1]) * p.field[2];
  f->out_pixels = uint64_t(outputSize(p, 1)) * uint64_t(outputSize(p, 2));
  f->taps2 = uint64_t(p.kernel[1]) * p.kernel[2];
  return PLB_OK;
}

// Launches the gather with the widest vector the channel run allows.
int foldDepth(plb_context *ctx, const Fold3d &f, bool inverse, const void *src, void *dst,
              uint64_t n, uint32_t src_depth, uint32_t dst_depth, uint64_t pixels, uint32_t G,
              size_t chan_bytes) {
  size_t vb = 16;
  while (chan_bytes % vb) vb >>= 1;
  const uint32_t vecs = uint32_t(chan_bytes / vb);
  const uint64_t total = n * dst_depth * pixels * G * f.KD * vecs;
  if (total == 0) return PLB_OK;
  const int grid = int(std::min<uint64_t>((total + 255) / 256, uint64_t(ctx->sm_count) * 32));
#define PLB_FOLD(V)                                                                          \
  foldDepthKernel<V><<<grid, 256, 0, ctx->stream>>>(static_cast<const V *>(src),             \
                                                    static_cast<V *>(dst), f.m, inverse ? 1 : 0, \
                                                    src_depth, dst_depth, f.KD, pixels, G, vecs, \
                                                    total)
  switch (vb) {
    case 16: PLB_FOLD(uint4); break;
    case 8: PLB_FOLD(uint2); break;
    case 4: PLB_FOLD(uint32_t); break;
    case 2: PLB_FOLD(uint16_t); break;
    default: PLB_FOLD(uint8_t); break;
  }
#undef PLB_FOLD
  PLB_CUDA(cudaGetLastError());
  ctx->launches++;
  return PLB_OK;
}

// Weights [g][kd][taps2][a][b] -> [g][taps2][a][kd*b_count + b] (fold_last) or
// [g][taps2][kd*a_count + a][b]; reverse_depth stores depth slice kd at KD-1-kd.
int foldWeights(plb_context *ctx, const Fold3d &f, uint32_t elem_bytes, uint32_t G, uint32_t a_count,
                uint32_t b_count, bool fold_last, bool reverse_depth, const void *src, void *dst) {
  const uint64_t shape[5] = {G, f.KD, f.taps2, a_count, b_count};
  const int64_t A = a_count, B = b_count, T = int64_t(f.taps2), K = f.KD;
  const int64_t src_strides[5] = {K * T * A * B, T * A * B, A * B, B, 1};
  int64_t dst_strides[5];
  int64_t offset = 0;
  if (fold_last) {
    const int64_t d[5] = {T * A * K * B, B, A * K * B, K * B, 1};
    std::copy(d, d + 5, dst_strides);
  } else {
    const int64_t d[5] = {T * K * A * B, A * B, K * A * B, B, 1};
    std::copy(d, d + 5, dst_strides);
  }
  if (reverse_depth) {
    offset = (K - 1) * dst_strides[1];
    dst_strides[1] = -dst_strides[1];
  }
  return plb_copy_strided(ctx, elem_bytes, 5, shape, src_strides, dst_strides, src,
                          static_cast<uint8_t *>(dst) + offset * int64_t(elem_bytes));
}

}  // namespace

int conv3dFwd(plb_context *ctx, const plb_conv_params &p, const plb_conv_options *opt,
              const void *d_in, const void *d_weights, const float *d_bias, void *d_out,
              int transpose_and_flip_weights) {
  Fold3d f;
  if (int rc = makeFold(p, &f)) return rc;
  const size_t es = dtypeBytes(p.input_type);
  const uint32_t G = p.groups, Ci = p.in_chans_per_group, Co = p.out_chans_per_group;
  if (p.batch == 0 || G == 0 || Co == 0 || f.OD == 0 || f.out_pixels == 0) return PLB_OK;
  if (Ci == 0) return fail(PLB_ERR_UNSUPPORTED, "zero input channels are not implemented on this path yet");
  void *xf = nullptr, *wf = nullptr;
  if (int rc = scratch(ctx, kSlotDepthFold, size_t(p.batch) * f.OD * f.in_pixels * G * f.KD * Ci * es + 256, &xf)) return rc;
  if (int rc = scratch(ctx, kSlotFoldedWeights, size_t(G) * f.KD * f.taps2 * Co * Ci * es + 256, &wf)) return rc;
  if (int rc = foldDepth(ctx, f, false, d_in, xf, p.batch, f.D, f.OD, f.in_pixels, G, Ci * es)) return rc;
  if (transpose_and_flip_weights) {
    // stored [g][kd][taps][Ci][Co], flipped in every dimension: undo the depth flip here
    if (int rc = foldWeights(ctx, f, uint32_t(es), G, Ci, Co, false, true, d_weights, wf)) return rc;
  } else {
    if (int rc = foldWeights(ctx, f, uint32_t(es), G, Co, Ci, true, false, d_weights, wf)) return rc;
  }
  plb_conv_params q = f.p2;
  q.batch = p.batch * f.OD;
  q.in_chans_per_group = f.KD * Ci;
  return plb_convolution(ctx, &q, opt, xf, wf, d_bias, d_out, transpose_and_flip_weights);
}

int conv3dBwd(plb_context *ctx, const plb_conv_params &p, const plb_conv_options *opt,
              const void *d_out_grads, const void *d_weights, void *d_in_grads) {
  Fold3d f;
  if (int rc = makeFold(p, &f)) return rc;
  const size_t es = dtypeBytes(p.input_type);
  const uint32_t G = p.groups, Ci = p.in_chans_per_group, Co = p.out_chans_per_group;
  if (p.batch == 0 || G == 0 || Ci == 0 || f.D == 0 || f.in_pixels == 0) return PLB_OK;
  if (Co == 0 || f.OD == 0 || f.out_pixels == 0) {
    PLB_CUDA(cudaMemsetAsync(d_in_grads, 0,
                             size_t(p.batch) * f.D * f.in_pixels * G * Ci * dtypeBytes(p.output_type),
                             ctx->stream));
    return PLB_OK;
  }
  void *gf = nullptr, *wf = nullptr;
  if (int rc = scratch(ctx, kSlotDepthFold, size_t(p.batch) * f.D * f.out_pixels * G * f.KD * Co * es + 256, &gf)) return rc;
  if (int rc = scratch(ctx, kSlotFoldedWeights, size_t(G) * f.KD * f.taps2 * Co * Ci * es + 256, &wf)) return rc;
  if (int rc = foldDepth(ctx, f, true, d_out_grads, gf, p.batch, f.OD, f.D, f.out_pixels, G, Co * es)) return rc;
  if (int rc = foldWeights(ctx, f, uint32_t(es), G, Co, Ci, false, false, d_weights, wf)) return rc;
  plb_conv_params q = f.p2;
  q.batch = p.batch * f.D;
  q.out_chans_per_group = f.KD * Co;
  return plb_conv_bwd(ctx, &q, opt, gf, wf, d_in_grads);
}

int conv3dWu(plb_context *ctx, const plb_conv_params &p, const plb_conv_options *opt,
             const void *d_acts, const void *d_out_grads, void *d_weight_grads,
             float *d_weight_grads_f32) {
  Fold3d f;
  if (int rc = makeFold(p, &f)) return rc;
  const size_t es = dtypeBytes(p.input_type);
  const uint32_t G = p.groups, Ci = p.in_chans_per_group, Co = p.out_chans_per_group;
  const size_t w_elems = size_t(G) * f.KD * f.taps2 * Co * Ci;
  if (w_elems == 0) return PLB_OK;
  if (p.batch == 0 || f.OD == 0 || f.out_pixels == 0) {
    if (d_weight_grads) PLB_CUDA(cudaMemsetAsync(d_weight_grads, 0, w_elems * es, ctx->stream));
    if (d_weight_grads_f32)
      PLB_CUDA(cudaMemsetAsync(d_weight_grads_f32, 0, w_elems * sizeof(float), ctx->stream));
    return PLB_OK;
  }
  void *xf = nullptr, *ws = nullptr;
  if (int rc = scratch(ctx, kSlotDepthFold, size_t(p.batch) * f.OD * f.in_pixels * G * f.KD * Ci * es + 256, &xf)) return rc;
  if (int rc = scratch(ctx, kSlotFoldedGrads, 2 * w_elems * sizeof(float) + 512, &ws)) return rc;
  float *folded = static_cast<float *>(ws);
  float *unfolded = d_weight_grads_f32 ? d_weight_grads_f32
                                       : folded + ((w_elems + 63) / 64) * 64;
  if (int rc = foldDepth(ctx, f, false, d_acts, xf, p.batch, f.D, f.OD, f.in_pixels, G, Ci * es)) return rc;
  plb_conv_params q = f.p2;
  q.batch = p.batch * f.OD;
  q.in_chans_per_group = f.KD * Ci;
  if (int rc = plb_conv_wu(ctx, &q, opt, xf, d_out_grads, nullptr, folded)) return rc;
  // [g][taps][Co][kd*Ci + ci] -> [g][kd][taps][Co][ci]
  const uint64_t shape[5] = {G, f.KD, f.taps2, Co, Ci};
  const int64_t T = int64_t(f.taps2), K = f.KD, A = Co, B = Ci;
  const int64_t src_strides[5] = {T * A * K * B, B, A * K * B, K * B, 1};
  const int64_t dst_strides[5] = {K * T * A * B, T * A * B, A * B, B, 1};
  if (int rc = plb_copy_strided(ctx, 4, 5, shape, src_strides, dst_strides, folded, unfolded)) return rc;
  if (d_weight_grads)
    return plb_cast_from_f32(ctx, p.input_type, d_weight_grads, unfolded, w_elems);
  return PLB_OK;
}

// The plan of the folded 2-D problem, with the 3-D layer's own flop count.
int conv3dPlan(const plb_conv_params &p, const plb_conv_options *opt, int32_t pass, plb_plan *plan) {
  Fold3d f;
  if (int rc = makeFold(p, &f)) return rc;
  plb_conv_params q = f.p2;
  int rc;
  if (pass == PLB_PASS_TRAINING_BWD) {
    q.batch = p.batch * f.D;
    q.out_chans_per_group = f.KD * p.out_chans_per_group;
    rc = plb_conv_plan(&q, opt, pass, plan);
  } else {
    q.batch = p.batch * f.OD;
    q.in_chans_per_group = f.KD * p.in_chans_per_group;
    rc = pass == PLB_PASS_TRAINING_WU ? plb_conv_wu_plan(&q, opt, plan) : plb_conv_plan(&q, opt, pass, plan);
  }
  if (rc) return rc;
  plan->flops = 2 * numberOfMacs(p);
  return PLB_OK;
}

}  // namespace plb
