// Weight-update pass: planning and launch of the weight-gradient kernel.
#include <algorithm>
#include <cstdlib>
#include <mutex>
#include <string>

#include "conv_geometry.h"
#include "runtime.h"
#include "wu_sm100.cuh"

namespace plb {
namespace {

struct WuShape {
  int H, W, OH, OW, KH, KW, padH, padW, dilH, dilW, strH, strW;
  // views: input truncation (tH, tW; extent He x We), output padding (opH, opW;
  // computed extent OHc x OWc); padH/padW already include the output truncation
  int tH, tW, He, We, opH, opW, OHc, OWc;
};

int wuShape(const plb_conv_params &p, WuShape *s) {
  const std::string err = validate(p);
  if (!err.empty()) return fail(PLB_ERR_INVALID_PARAMS, err);
  if (p.num_field_dims > 2)
    return fail(PLB_ERR_UNSUPPORTED, "3-D convolutions are not implemented on this path yet");
  if (!is16BitFloat(p.input_type))
    // the reference never runs the weight update in quarter either
    // (tools/single_conv_layer.cpp:725-733)
    return fail(PLB_ERR_UNSUPPORTED, "weight update is implemented for half and float input only");
  for (unsigned d = 0; d != p.num_field_dims; ++d) {
    // (kernel truncation and flip are resolved by plb_conv_wu before it gets here)
    if (p.in_dilation[d] != 1 || p.in_flip[d] || p.k_trunc_lo[d] || p.k_trunc_hi[d] || p.k_flip[d])
      return fail(PLB_ERR_UNSUPPORTED,
                  "input dilation/flip are not implemented on this path yet (kernel truncation "
                  "and flip only through plb_conv_wu)");
    if (p.stride[d] > 8) return fail(PLB_ERR_UNSUPPORTED, "strides above 8 are not implemented");
  }
  const unsigned hd = p.num_field_dims == 2 ? 0 : ~0u, wd = p.num_field_dims - 1;
  auto get = [&](const uint32_t *v, unsigned d, int dflt) { return d == ~0u ? dflt : int(v[d]); };
  s->H = get(p.field, hd, 1);
  s->W = get(p.field, wd, 1);
  s->KH = get(p.kernel, hd, 1);
  s->KW = get(p.kernel, wd, 1);
  s->padH = get(p.in_pad_lo, hd, 0);
  s->padW = get(p.in_pad_lo, wd, 0);
  s->dilH = get(p.k_dilation, hd, 1);
  s->dilW = get(p.k_dilation, wd, 1);
  s->strH = get(p.stride, hd, 1);
  s->strW = get(p.stride, wd, 1);
  s->OH = hd == ~0u ? 1 : int(outputSize(p, hd));
  s->OW = int(outputSize(p, wd));
  s->tH = get(p.in_trunc_lo, hd, 0);
  s->tW = get(p.in_trunc_lo, wd, 0);
  s->He = s->H - s->tH - get(p.in_trunc_hi, hd, 0);
  s->We = s->W - s->tW - get(p.in_trunc_hi, wd, 0);
  // kernel padding only shifts where the taps land
  s->padH -= get(p.out_trunc_lo, hd, 0) + get(p.k_pad_lo, hd, 0);
  s->padW -= get(p.out_trunc_lo, wd, 0) + get(p.k_pad_lo, wd, 0);
  s->opH = get(p.out_pad_lo, hd, 0);
  s->opW = get(p.out_pad_lo, wd, 0);
  s->OHc = s->OH - s->opH - get(p.out_pad_hi, hd, 0);
  s->OWc = s->OW - s->opW - get(p.out_pad_hi, wd, 0);
  return PLB_OK;
}

// Tiling of one group's weight update.
void planWu(const plb_conv_params &p, const WuShape &s, int sm_count, int force_split,
            unsigned plan_flags, WuArgs *a, plb_plan *plan) {
  const int co = int(p.out_chans_per_group), ci = int(p.in_chans_per_group);
  const int taps = s.KH * s.KW;
  a->taps_h = s.KH;
  a->taps_w = s.KW;
  a->pad_h = s.padH;
  a->pad_w = s.padW;
  a->dil_h = s.dilH;
  a->dil_w = s.dilW;
  a->stride_h = s.strH;
  a->stride_w = s.strW;
  a->co_total = co;
  a->ci_total = ci;
  a->co_blocks = (co + 127) / 128;
  a->ci_blk = std::min(256, (ci + 31) / 32 * 32);
  a->ci_blk64 = (a->ci_blk + 63) / 64;
  a->ci_blocks = (ci + a->ci_blk - 1) / a->ci_blk;
  a->taps_per_group = std::max(1, std::min(taps, 512 / a->ci_blk));
  // two pipeline stages of (outGrad tile + one activation box per tap) must fit
  while (a->taps_per_group > 1 &&
         2 * (2 + a->taps_per_group * a->ci_blk64) * kWuBlockBytes > 200 * 1024)
    --a->taps_per_group;
  a->tap_groups = (taps + a->taps_per_group - 1) / a->taps_per_group;
  // even out the groups (9 taps, 4 per group -> 3 groups of 3)
  a->taps_per_group = (taps + a->tap_groups - 1) / a->tap_groups;
  int cols = a->taps_per_group * a->ci_blk, pow2 = 32;
  while (pow2 < cols) pow2 <<= 1;
  a->tmem_cols = pow2;
  // pixel box: 64 pixels, fewest tiles, then widest rows
  long best = -1;
  for (int w = 64; w >= 1; w >>= 1)
    for (int h = 64 / w; h >= 1; h >>= 1) {
      const int n = 64 / (w * h);
      if ((w - 1) * s.strW + 1 > 256 || (h - 1) * s.strH + 1 > 256) continue;
      const long tiles =
          long((s.OWc + w - 1) / w) * ((s.OHc + h - 1) / h) * ((long(p.batch) + n - 1) / n);
      if (best < 0 || tiles < best) {
        best = tiles;
        a->box_w = w;
        a->box_h = h;
        a->box_n = n;
      }
    }
  int stage_bytes = (2 + a->taps_per_group * a->ci_blk64) * kWuBlockBytes;
  // Strip mode: one tap group per filter column, the activations of a K step
  // loaded once for all filter rows.  Needs a unit vertical stride, all filter
  // rows' accumulators in TMEM at once and box_w * box_n a multiple of 8; taken
  // when it costs at most 1/8 more pixel tiles than the best box.
  a->strip_mode = 0;
  // PLB_PLAN_NO_A_COLLECTOR: fetch the outGrad tile for every instruction (A/B timing)
  a->reuse_a = (plan_flags & PLB_PLAN_NO_A_COLLECTOR) ? 0 : 1;
  a->idesc_formats = p.input_type == PLB_BFLOAT16 ? (make_idesc(0, 0, 1, 1, false, false) & ~(1u << 4)) : 0u;
  const int halo = (s.KH - 1) * s.dilH;
  if (s.KH > 1 && s.strH == 1 && s.KH * a->ci_blk <= 512 && (plan_flags & PLB_PLAN_NO_HALO) == 0) {
    long sbest = -1;
    int sw = 0, sh = 0, sn = 0;
    for (int h = 64; h >= 1; h >>= 1)  // tallest first: least halo per row
      for (int w = 64 / h; w >= 1; w >>= 1) {
        const int n = 64 / (w * h);
        if ((w * n) % 8 != 0 || h + halo > 256 || (w - 1) * s.strW + 1 > 256) continue;
        const long tiles =
            long((s.OWc + w - 1) / w) * ((s.OHc + h - 1) / h) * ((long(p.batch) + n - 1) / n);
        if (sbest < 0 || tiles < sbest) {
          sbest = tiles;
          sw = w;
          sh = h;
          sn = n;
        }
      }
    const int strip_rows = sw * sn * (sh + halo);
    const int sbytes = 2 * kWuBlockBytes + a->ci_blk64 * strip_rows * 128;
    if (sbest > 0 && sbest * 8 <= best * 9 && 2 * sbytes <= 200 * 1024) {
      a->strip_mode = 1;
      a->box_w = sw;
      a->box_h = sh;
      a->box_n = sn;
      a->strip_rows = strip_rows;
      a->halo_step_bytes = s.dilH * sw * sn * 128;
      a->taps_per_group = s.KH;
      a->tap_groups = s.KW;
      a->tmem_cols = 32;
      while (a->tmem_cols < s.KH * a->ci_blk) a->tmem_cols <<= 1;
      stage_bytes = sbytes;
      best = sbest;
    }
  }
  a->tiles_w = (s.OWc + a->box_w - 1) / a->box_w;
  a->tiles_h = (s.OHc + a->box_h - 1) / a->box_h;
  a->tiles_n = (int(p.batch) + a->box_n - 1) / a->box_n;
  a->stage_bytes = stage_bytes;
  a->stages = std::max(2, std::min(kWuMaxStages, (200 * 1024) / stage_bytes));
  const int units = a->co_blocks * a->ci_blocks * a->tap_groups;
  int ksplit = force_split > 0 ? force_split : std::max(1, (sm_count > 0 ? sm_count : 148) / units);
  ksplit = int(std::min<long>(ksplit, std::max<long>(best, 1)));
  a->ksplit = ksplit;
  if (plan) {
    plan->kernel = 1;
    plan->tile_m = 128;
    plan->tile_n = a->taps_per_group * a->ci_blk;
    plan->tile_k_bytes = kWuPixelsPerStage * 2;
    plan->box_w = a->box_w;
    plan->box_h = a->box_h;
    plan->box_n = a->box_n;
    plan->stages = a->stages;
    plan->split_k = ksplit;
    plan->tiles = units;
    plan->grid = units * ksplit;
    plan->b_mn_major = 1;
    plan->halo_rows = a->strip_mode ? halo : 0;
    plan->workspace_bytes = size_t(ksplit) * taps * co * ci * sizeof(float);
  }
}

// Gradient of the used taps -> gradient of the stored filter: tap (th, tw) of
// the [G][JH*JW][inner] source goes to tap (r0h + th', r0w + tw') of the
// zero-initialised [G][KH*KW][inner] destination, th' = JH-1-th when the
// kernel is used flipped in that dimension.  `vec_bytes` is 4 or 2.
template <typename T>
__global__ void scatterTapsKernel(const T *__restrict__ src, T *__restrict__ dst, int groups, int KH,
                                  int KW, int JH, int JW, int r0h, int r0w, int flip_h, int flip_w,
                                  size_t inner) {
  const size_t total = size_t(groups) * JH * JW * inner;
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < total;
       i += size_t(gridDim.x) * blockDim.x) {
    const size_t v = i % inner;
    size_t t = i / inner;
    const int tw = int(t % JW);
    t /= JW;
    const int th = int(t % JH);
    const int g = int(t / JH);
    const int oh = r0h + (flip_h ? JH - 1 - th : th), ow = r0w + (flip_w ? JW - 1 - tw : tw);
    dst[(size_t(g) * KH * KW + size_t(oh) * KW + ow) * inner + v] = src[i];
  }
}

// The wu kernel needs more dynamic shared memory than the default limit: raised
// once per device, for every entry point alike.
int configureWuKernel(int device) {
  static std::mutex mutex;
  static bool configured[64] = {};
  if (device < 0 || device >= 64) return fail(PLB_ERR_INVALID_PARAMS, "device ordinal out of range");
  std::lock_guard<std::mutex> lock(mutex);
  if (!configured[device]) {
    // the caller has made `device` current
    PLB_CUDA(cudaFuncSetAttribute(wu_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    configured[device] = true;
  }
  return PLB_OK;
}

// Reduction over the K splits of group g (and, with `peer`, over the ranks).
int launchWuReduce(cudaStream_t stream, const WuArgs &a, size_t w_elems, unsigned g,
                   void *d_weight_grads, float *d_weight_grads_f32, const WuPeerArgs *peer) {
  const size_t es = 2;
  cudaLaunchAttribute pdl[1];
  pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  pdl[0].val.programmaticStreamSerializationAllowed = 1;
  float *out32 = d_weight_grads_f32 ? d_weight_grads_f32 + size_t(g) * w_elems : nullptr;
  uint8_t *out16 =
      d_weight_grads ? static_cast<uint8_t *>(d_weight_grads) + size_t(g) * w_elems * es : nullptr;
  if (peer != nullptr) {
    const size_t count4 = w_elems / 4;
    const unsigned rgrid = unsigned((count4 + kWuFusedChunk - 1) / kWuFusedChunk);
    WuPeerArgs pa = *peer;
    for (int r = 0; r < pa.world; ++r) {
      pa.grads[r] += size_t(g) * count4;
      if (pa.results[r] != nullptr) pa.results[r] += size_t(g) * count4;
    }
    pa.chunk_base = g * rgrid;
    cudaLaunchConfig_t rcfg{};
    rcfg.gridDim = dim3(rgrid);
    rcfg.blockDim = dim3(32, kWuReduceLanes);
    rcfg.stream = stream;
    rcfg.attrs = pdl;
    rcfg.numAttrs = 1;
    PLB_CUDA(cudaLaunchKernelEx(&rcfg, wu_reduce_allreduce_kernel,
                                reinterpret_cast<const float4 *>(a.partial), a.ksplit, count4, pa,
                                reinterpret_cast<float4 *>(out32), reinterpret_cast<uint2 *>(out16)));
  } else if (w_elems % 4 == 0 && (reinterpret_cast<uintptr_t>(out32) & 15) == 0 &&
             (reinterpret_cast<uintptr_t>(out16) & 7) == 0) {
    const size_t count4 = w_elems / 4;
    const unsigned rgrid = unsigned((count4 + 31) / 32);
    cudaLaunchConfig_t rcfg{};
    rcfg.gridDim = dim3(rgrid);
    rcfg.blockDim = dim3(32, kWuReduceLanes);
    rcfg.stream = stream;
    rcfg.attrs = pdl;
    rcfg.numAttrs = 1;
    PLB_CUDA(cudaLaunchKernelEx(&rcfg, wu_reduce4_kernel,
                                reinterpret_cast<const float4 *>(a.partial), a.ksplit, count4,
                                reinterpret_cast<float4 *>(out32), reinterpret_cast<uint2 *>(out16)));
  } else {
    const int rgrid = int(std::min<size_t>((w_elems + 255) / 256, size_t(148) * 8));
    wu_reduce_kernel<<<rgrid, 256, 0, stream>>>(a.partial, a.ksplit, w_elems, out32, out16, 0);
  }
  PLB_CUDA(cudaGetLastError());
  return PLB_OK;
}

// Launches the weight-gradient kernel and the reduction over K splits for every
// group.  `a.partial` and `a.status` are set by the caller.
// With `peer` the reduction also adds the gradients of the other ranks
// (wu_reduce_allreduce_kernel); the caller has checked that the shapes allow it.
int launchWu(cudaStream_t stream, const plb_conv_params &p, const WuShape &s, const WuArgs &a,
             const void *d_acts, const void *d_out_grads, void *d_weight_grads,
             float *d_weight_grads_f32, uint64_t *launches, const WuPeerArgs *peer = nullptr) {
  const int co = int(p.out_chans_per_group), ci = int(p.in_chans_per_group);
  const int taps = s.KH * s.KW;
  const size_t w_elems = size_t(taps) * co * ci;
  const size_t es = 2;
  const uint64_t ctot = uint64_t(p.groups) * ci, cotot = uint64_t(p.groups) * co;
  const int smem = a.stages * a.stage_bytes + 256 + 1024;
  const uint32_t ones[4] = {1, 1, 1, 1};
  CUtensorMap tout;
  {
    // partial sums [ksplit][taps][co][ci] fp32, stored in blocks of 32 x 32
    const uint64_t dims[4] = {uint64_t(ci), uint64_t(co), uint64_t(taps), uint64_t(a.ksplit)};
    const uint64_t strides[3] = {uint64_t(ci) * 4, uint64_t(co) * ci * 4, uint64_t(w_elems) * 4};
    const uint32_t box[4] = {32, 32, 1, 1};
    if (int rc = encodeTensorMap(&tout, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, a.partial, dims,
                                 strides, box, ones))
      return rc;
  }
  for (unsigned g = 0; g < p.groups; ++g) {
    CUtensorMap tdy, tx;
    // pixel dimensions (w, h, n); strip mode orders them (w, n, h)
    const bool strip = a.strip_mode != 0;
    const int halo = strip ? (s.KH - 1) * s.dilH : 0;
    {
      const uint64_t sh = uint64_t(s.OW) * cotot * es, sn = uint64_t(s.OH) * s.OW * cotot * es;
      const uint64_t dims[4] = {uint64_t(co), uint64_t(s.OWc), strip ? p.batch : uint64_t(s.OHc),
                                strip ? uint64_t(s.OHc) : p.batch};
      const uint64_t strides[3] = {cotot * es, strip ? sn : sh, strip ? sh : sn};
      const uint32_t box[4] = {64, uint32_t(a.box_w), uint32_t(strip ? a.box_n : a.box_h),
                               uint32_t(strip ? a.box_h : a.box_n)};
      if (int rc = encodeTensorMap(&tdy, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                                   static_cast<const uint8_t *>(d_out_grads) +
                                       ((size_t(s.opH) * s.OW + s.opW) * cotot + size_t(g) * co) * es,
                                   dims, strides, box, ones))
        return rc;
    }
    {
      const uint64_t sh = uint64_t(s.W) * ctot * es, sn = uint64_t(s.H) * s.W * ctot * es;
      const uint64_t dims[4] = {uint64_t(ci), uint64_t(s.We), strip ? p.batch : uint64_t(s.He),
                                strip ? uint64_t(s.He) : p.batch};
      const uint64_t strides[3] = {ctot * es, strip ? sn : sh, strip ? sh : sn};
      const uint32_t bw = uint32_t((a.box_w - 1) * s.strW + 1);
      const uint32_t bh = strip ? uint32_t(a.box_h + halo) : uint32_t((a.box_h - 1) * s.strH + 1);
      const uint32_t box[4] = {64, bw, strip ? uint32_t(a.box_n) : bh, strip ? bh : uint32_t(a.box_n)};
      const uint32_t estr[4] = {1, uint32_t(s.strW), strip ? 1u : uint32_t(s.strH), 1};
      if (int rc = encodeTensorMap(&tx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                                   static_cast<const uint8_t *>(d_acts) +
                                       ((size_t(s.tH) * s.W + s.tW) * ctot + size_t(g) * ci) * es,
                                   dims, strides, box, estr))
        return rc;
    }
    const int grid = a.co_blocks * a.ci_blocks * a.tap_groups * a.ksplit;
    // programmatic stream serialization: the kernels' set-up overlaps the tail
    // of whatever runs before them; they wait before touching global memory
    cudaLaunchAttribute pdl[1];
    pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    pdl[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(unsigned(grid));
    cfg.blockDim = dim3(kWuThreads);
    cfg.dynamicSmemBytes = size_t(smem);
    cfg.stream = stream;
    cfg.attrs = pdl;
    cfg.numAttrs = 1;
    PLB_CUDA(cudaLaunchKernelEx(&cfg, wu_kernel, tdy, tx, tout, a));
    if (int rc = launchWuReduce(stream, a, w_elems, g, d_weight_grads, d_weight_grads_f32, peer))
      return rc;
    if (launches) *launches += 2;
  }
  return PLB_OK;
}

}  // namespace
}  // namespace plb

using namespace plb;

extern "C" {

int plb_conv_wu_plan(const plb_conv_params *p_in, const plb_conv_options *opt, plb_plan *plan) {
  if (!p_in || !plan) return fail(PLB_ERR_INVALID_PARAMS, "null argument");
  if (p_in->input_type == PLB_FLOAT) {
    // what runs: bfloat16 operands, three batches side by side (float_route.cu)
    const std::string err = validate(*p_in);
    if (!err.empty()) return fail(PLB_ERR_INVALID_PARAMS, err);
    const plb_conv_params q = floatRouteConvParams(*p_in, PLB_PASS_TRAINING_WU);
    if (int rc = plb_conv_wu_plan(&q, opt, plan)) return rc;
    plan->flops = 2 * numberOfMacs(*p_in);
    size_t n_in, n_w, n_out;
    convElementCounts(*p_in, &n_in, &n_w, &n_out);
    plan->workspace_bytes += (n_in + n_out) * 6 + 768;
    return PLB_OK;
  }
  if (p_in->num_field_dims == 3) return conv3dPlan(*p_in, opt, PLB_PASS_TRAINING_WU, plan);
  // plan what plb_conv_wu runs: flipped inputs are reversed first, truncated /
  // flipped kernels are computed as ordinary kernels of the truncated extent
  plb_conv_params q;
  unflippedInputParams(*p_in, &q);
  {
    plb_conv_params undilated;
    DilatedField df;
    if (undilatedInputParams(q, &undilated, &df)) q = undilated;
  }
  for (unsigned d = 0; d != q.num_field_dims && d < PLB_MAX_FIELD_DIMS; ++d) {
    q.kernel[d] -= std::min(q.kernel[d], q.k_trunc_lo[d] + q.k_trunc_hi[d]);
    q.k_trunc_lo[d] = q.k_trunc_hi[d] = 0;
    if (q.k_flip[d]) std::swap(q.k_pad_lo[d], q.k_pad_hi[d]);
    q.k_flip[d] = 0;
  }
  const plb_conv_params *p = &q;
  WuShape s;
  if (int rc = wuShape(*p, &s)) return rc;
  *plan = plb_plan{};
  WuArgs a{};
  planWu(*p, s, 148, opt ? opt->split_k : 0, opt ? opt->plan_flags : 0, &a, plan);
  plan->flops = 2 * numberOfMacs(*p);
  const uint64_t es = dtypeBytes(p->input_type);
  plan->bytes = es * (uint64_t(p->batch) * s.H * s.W * p->groups * p->in_chans_per_group +
                      uint64_t(p->batch) * s.OH * s.OW * p->groups * p->out_chans_per_group +
                      uint64_t(p->groups) * s.KH * s.KW * p->in_chans_per_group *
                          p->out_chans_per_group);
  return PLB_OK;
}

int plb_conv_wu(plb_context *ctx, const plb_conv_params *p, const plb_conv_options *opt,
                const void *d_acts, const void *d_out_grads, void *d_weight_grads,
                float *d_weight_grads_f32) {
  TraceRange trace_range("plb_conv_wu");
  if (int rc = activate(ctx)) return rc;
  if (!p) return fail(PLB_ERR_INVALID_PARAMS, "null params");
  {
    size_t n_in, n_w, n_out;
    convElementCounts(*p, &n_in, &n_w, &n_out);
    if (n_in == 0 || n_out == 0) n_in = n_out = 0;  // nothing is read: the gradient is zero
    const void *result = d_weight_grads ? d_weight_grads : static_cast<const void *>(d_weight_grads_f32);
    if (int rc = checkConvRequest(*p, true, d_acts, n_w ? n_in : 0, d_out_grads, n_w ? n_out : 0, result, n_w))
      return rc;
  }
  if (p->input_type == PLB_FLOAT) {
    const std::string err = validate(*p);
    if (!err.empty()) return fail(PLB_ERR_INVALID_PARAMS, err);
    return floatConvWu(ctx, *p, opt, d_acts, d_out_grads, d_weight_grads, d_weight_grads_f32);
  }
  if (p->input_type == PLB_BFLOAT16 && d_weight_grads)
    return fail(PLB_ERR_UNSUPPORTED, "a bfloat16 layer's weight gradient is returned as fp32 only");
  if (p->num_field_dims == 3)
    return conv3dWu(ctx, *p, opt, d_acts, d_out_grads, d_weight_grads, d_weight_grads_f32);
  {
    // a flipped input: reverse it once (scratch slot 8), then an ordinary weight update
    plb_conv_params q;
    if (unflippedInputParams(*p, &q) && p->num_field_dims <= 2) {
      const std::string err = validate(*p);
      if (!err.empty()) return fail(PLB_ERR_INVALID_PARAMS, err);
      const bool two = p->num_field_dims == 2;
      const uint32_t H = two ? p->field[0] : 1, W = p->field[two ? 1 : 0];
      const size_t px = size_t(p->groups) * p->in_chans_per_group * dtypeBytes(p->input_type);
      void *xf = nullptr;
      if (int rc = scratch(ctx, kSlotFlipped, size_t(p->batch) * H * W * px + 256, &xf)) return rc;
      if (int rc = flipField(ctx, d_acts, xf, p->batch, H, W, px, two && p->in_flip[0],
                             p->in_flip[two ? 1 : 0] != 0))
        return rc;
      return plb_conv_wu(ctx, &q, opt, xf, d_out_grads, d_weight_grads, d_weight_grads_f32);
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
      if (int rc = dilateField(ctx, d_acts, xd, p->batch, df, px, false)) return rc;
      return plb_conv_wu(ctx, &q, opt, xd, d_out_grads, d_weight_grads, d_weight_grads_f32);
    }
  }
  {
    // A truncated and / or flipped kernel: the gradient of the used taps is
    // that of an ordinary kernel of the truncated extent (with the kernel
    // padding of a flipped dimension swapped), scattered back into the stored
    // filter, whose unused taps get zero.
    bool special = false;
    for (unsigned d = 0; d != p->num_field_dims && d < PLB_MAX_FIELD_DIMS; ++d)
      special |= p->k_trunc_lo[d] || p->k_trunc_hi[d] || p->k_flip[d];
    if (special) {
      const std::string err = validate(*p);
      if (!err.empty()) return fail(PLB_ERR_INVALID_PARAMS, err);
      if (p->num_field_dims > 2)
        return fail(PLB_ERR_UNSUPPORTED, "3-D convolutions are not implemented on this path yet");
      plb_conv_params q = *p;
      int K[2] = {1, 1}, J[2] = {1, 1}, r0[2] = {0, 0}, fl[2] = {0, 0};
      for (unsigned d = 0; d != p->num_field_dims; ++d) {
        const unsigned slot = p->num_field_dims == 2 ? d : 1;  // 1-D: the width
        K[slot] = int(p->kernel[d]);
        J[slot] = int(p->kernel[d]) - int(p->k_trunc_lo[d]) - int(p->k_trunc_hi[d]);
        r0[slot] = int(p->k_trunc_lo[d]);
        fl[slot] = p->k_flip[d] ? 1 : 0;
        q.kernel[d] = uint32_t(J[slot]);
        q.k_trunc_lo[d] = q.k_trunc_hi[d] = 0;
        q.k_flip[d] = 0;
        if (p->k_flip[d]) std::swap(q.k_pad_lo[d], q.k_pad_hi[d]);
      }
      const size_t inner = size_t(p->out_chans_per_group) * p->in_chans_per_group;
      const size_t full = size_t(p->groups) * K[0] * K[1] * inner, used = size_t(p->groups) * J[0] * J[1] * inner;
      const size_t es = dtypeBytes(p->input_type);
      if (d_weight_grads) PLB_CUDA(cudaMemsetAsync(d_weight_grads, 0, full * es, ctx->stream));
      if (d_weight_grads_f32) PLB_CUDA(cudaMemsetAsync(d_weight_grads_f32, 0, full * sizeof(float), ctx->stream));
      if (used == 0 || full == 0) return PLB_OK;
      void *tmp = nullptr;
      const size_t used16 = (used * es + 255) & ~size_t(255);
      if (int rc = scratch(ctx, kSlotUsedTaps, used16 + used * sizeof(float) + 256, &tmp)) return rc;
      void *t16 = tmp;
      float *t32 = reinterpret_cast<float *>(static_cast<uint8_t *>(tmp) + used16);
      if (int rc = plb_conv_wu(ctx, &q, opt, d_acts, d_out_grads, d_weight_grads ? t16 : nullptr,
                               d_weight_grads_f32 ? t32 : nullptr))
        return rc;
      const int grid = int(std::min<size_t>((used + 255) / 256, size_t(ctx->sm_count) * 8));
      if (d_weight_grads) {
        scatterTapsKernel<uint16_t><<<grid, 256, 0, ctx->stream>>>(
            static_cast<const uint16_t *>(t16), static_cast<uint16_t *>(d_weight_grads), int(p->groups),
            K[0], K[1], J[0], J[1], r0[0], r0[1], fl[0], fl[1], inner);
        PLB_CUDA(cudaGetLastError());
        ctx->launches++;
      }
      if (d_weight_grads_f32) {
        scatterTapsKernel<float><<<grid, 256, 0, ctx->stream>>>(
            t32, d_weight_grads_f32, int(p->groups), K[0], K[1], J[0], J[1], r0[0], r0[1], fl[0], fl[1],
            inner);
        PLB_CUDA(cudaGetLastError());
        ctx->launches++;
      }
      return PLB_OK;
    }
  }
  WuShape s;
  if (int rc = wuShape(*p, &s)) return rc;
  const int co = int(p->out_chans_per_group), ci = int(p->in_chans_per_group);
  const int taps = s.KH * s.KW;
  const size_t w_elems = size_t(taps) * co * ci;
  if (p->groups == 0 || w_elems == 0) return PLB_OK;
  if (p->batch == 0 || s.OHc <= 0 || s.OWc <= 0 || s.He <= 0 || s.We <= 0) {
    // empty reduction: the gradient is zero
    const size_t n = size_t(p->groups) * w_elems;
    if (d_weight_grads) PLB_CUDA(cudaMemsetAsync(d_weight_grads, 0, n * dtypeBytes(p->input_type), ctx->stream));
    if (d_weight_grads_f32) PLB_CUDA(cudaMemsetAsync(d_weight_grads_f32, 0, n * sizeof(float), ctx->stream));
    return PLB_OK;
  }
  if (ci % 8 != 0 || co % 8 != 0) {
    // Channel counts TMA cannot address (a pixel must be a multiple of 16
    // bytes): run on zero-padded copies and drop the padded rows / columns of
    // the gradient.  Arena in scratch slot 7.
    const size_t es2 = 2, G = p->groups;
    const uint32_t cip = uint32_t((ci + 7) / 8 * 8), cop = uint32_t((co + 7) / 8 * 8);
    const size_t in_px = size_t(p->batch) * s.H * s.W, out_px = size_t(p->batch) * s.OH * s.OW;
    auto al = [](size_t n) { return (n + 255) & ~size_t(255); };
    const size_t x_b = al(in_px * G * cip * es2), dy_b = al(out_px * G * cop * es2);
    const size_t wp_elems = G * size_t(taps) * cop * cip;
    const size_t w16_b = al(wp_elems * es2), w32_b = al(wp_elems * 4);
    void *arena = nullptr;
    if (int rc = scratch(ctx, kSlotPaddedChans, x_b + dy_b + 2 * w16_b + 2 * w32_b, &arena)) return rc;
    uint8_t *xp = static_cast<uint8_t *>(arena), *dyp = xp + x_b, *w16 = dyp + dy_b, *t16 = w16 + w16_b,
            *w32 = t16 + w16_b, *t32 = w32 + w32_b;
    if (int rc = resizeRows(ctx, d_acts, xp, in_px * G, size_t(ci) * es2, cip * es2)) return rc;
    if (int rc = resizeRows(ctx, d_out_grads, dyp, out_px * G, size_t(co) * es2, cop * es2)) return rc;
    plb_conv_params q = *p;
    q.in_chans_per_group = cip;
    q.out_chans_per_group = cop;
    if (int rc = plb_conv_wu(ctx, &q, opt, xp, dyp, d_weight_grads ? w16 : nullptr,
                             d_weight_grads_f32 ? reinterpret_cast<float *>(w32) : nullptr))
      return rc;
    // [G][taps][cop][cip] -> drop rows, then columns
    const size_t gt = G * size_t(taps);
    if (d_weight_grads) {
      if (int rc = resizeRows(ctx, w16, t16, gt, size_t(cop) * cip * es2, size_t(co) * cip * es2)) return rc;
      if (int rc = resizeRows(ctx, t16, d_weight_grads, gt * co, cip * es2, size_t(ci) * es2)) return rc;
    }
    if (d_weight_grads_f32) {
      if (int rc = resizeRows(ctx, w32, t32, gt, size_t(cop) * cip * 4, size_t(co) * cip * 4)) return rc;
      if (int rc = resizeRows(ctx, t32, d_weight_grads_f32, gt * co, cip * 4, size_t(ci) * 4)) return rc;
    }
    return PLB_OK;
  }
  WuArgs a{};
  planWu(*p, s, ctx->sm_count, opt ? opt->split_k : 0, (opt ? opt->plan_flags : 0) | ctx->plan_flags, &a,
         nullptr);
  a.status = ctx->d_status;
  a.trace = ctx->trace;
  void *ws = nullptr;
  if (int rc = scratch(ctx, kSlotOperands, size_t(a.ksplit) * w_elems * sizeof(float), &ws)) return rc;
  a.partial = static_cast<float *>(ws);

  if (int rc = configureWuKernel(ctx->device)) return rc;
  uint64_t launches = 0;
  if (int rc = launchWu(ctx->stream, *p, s, a, d_acts, d_out_grads, d_weight_grads,
                        d_weight_grads_f32, &launches))
    return rc;
  ctx->launches += launches;
  return PLB_OK;
}

// Chunks (= blocks of the fused reduction, = flags per sender) of one call.
static size_t wuPeerChunks(const plb_conv_params &p, const WuShape &s) {
  const size_t w_elems = size_t(s.KH) * s.KW * p.out_chans_per_group * p.in_chans_per_group;
  return size_t(p.groups) * ((w_elems / 4 + kWuFusedChunk - 1) / kWuFusedChunk);
}

uint64_t plb_conv_wu_allreduce_flag_bytes(const plb_conv_params *p) {
  WuShape s;
  if (!p || wuShape(*p, &s)) return 0;
  // per chunk a word per sender, then a word per chunk for the owner's "sum complete"
  return uint64_t(wuPeerChunks(*p, s)) * (kWuPeerMaxWorld + 1) * sizeof(uint32_t);
}

}  // extern "C"

static int wuAllreduce(plb_context *ctx, const plb_conv_params *p, const plb_conv_options *opt,
                       const void *d_acts, const void *d_out_grads, int32_t rank, int32_t world,
                       void *const *d_peer_grads, void *const *d_peer_results,
                       void *const *d_peer_flags, uint32_t epoch, void *d_weight_grads,
                       float *d_weight_grads_f32) {
  TraceRange trace_range("plb_conv_wu_allreduce");
  if (int rc = activate(ctx)) return rc;
  if (!p) return fail(PLB_ERR_INVALID_PARAMS, "null params");
  if (world < 1 || world > kWuPeerMaxWorld || rank < 0 || rank >= world)
    return fail(PLB_ERR_INVALID_PARAMS, "rank / world size out of range (at most " +
                                            std::to_string(kWuPeerMaxWorld) + " ranks)");
  if (!d_peer_grads || !d_peer_flags) return fail(PLB_ERR_INVALID_PARAMS, "null pointer table");
  if (epoch == 0 || (epoch & 0x80000000u))
    return fail(PLB_ERR_INVALID_PARAMS, "steps are numbered from 1 to 2^31 - 1 (flags start at zero)");
  const char *other = "; use plb_conv_wu and plb_allreduce_f32_p2p for this layer";
  if (p->input_type != PLB_HALF)
    return fail(PLB_ERR_UNSUPPORTED, std::string("plb_conv_wu_allreduce takes half operands") + other);
  WuShape s;
  if (int rc = wuShape(*p, &s)) return rc;   // 1-D / 2-D, half, no input dilation / flip, plain kernel
  const int co = int(p->out_chans_per_group), ci = int(p->in_chans_per_group);
  const size_t w_elems = size_t(s.KH) * s.KW * co * ci;
  if (p->groups == 0 || w_elems == 0) return PLB_OK;
  if (ci % 8 != 0 || co % 8 != 0)
    return fail(PLB_ERR_UNSUPPORTED,
                std::string("the fused weight update needs channel counts that are multiples of 8") + other);
  // all blocks of the reduction wait for their peers' blocks: keep the grid resident
  if (wuPeerChunks(*p, s) / p->groups > size_t(ctx->sm_count) * 4)
    return fail(PLB_ERR_UNSUPPORTED,
                std::string("weight gradient too large for the fused reduction over ranks") + other);
  WuPeerArgs pa{};
  for (int r = 0; r < world; ++r) {
    if (!d_peer_grads[r] || !d_peer_flags[r]) return fail(PLB_ERR_INVALID_PARAMS, "null peer pointer");
    if ((reinterpret_cast<uintptr_t>(d_peer_grads[r]) & 15) != 0)
      return fail(PLB_ERR_INVALID_PARAMS, "peer gradient buffers must be 16-byte aligned");
    pa.grads[r] = static_cast<float4 *>(d_peer_grads[r]);
    pa.flags[r] = static_cast<uint32_t *>(d_peer_flags[r]);
    if (d_peer_results) {
      if (!d_peer_results[r] || (reinterpret_cast<uintptr_t>(d_peer_results[r]) & 15) != 0)
        return fail(PLB_ERR_INVALID_PARAMS, "peer result buffers must be non-null and 16-byte aligned");
      pa.results[r] = static_cast<float4 *>(d_peer_results[r]);
    }
  }
  pa.result_flags = uint32_t(wuPeerChunks(*p, s) * kWuPeerMaxWorld);
  if ((reinterpret_cast<uintptr_t>(d_weight_grads_f32) & 15) != 0 ||
      (reinterpret_cast<uintptr_t>(d_weight_grads) & 7) != 0)
    return fail(PLB_ERR_INVALID_PARAMS, "outputs must be 16-byte (fp32) / 8-byte (half) aligned");
  pa.rank = rank;
  pa.world = world;
  pa.epoch = epoch;
  pa.status = ctx->d_status;
  WuArgs a{};
  a.status = ctx->d_status;
  a.trace = ctx->trace;
  if (int rc = configureWuKernel(ctx->device)) return rc;
  uint64_t launches = 0;
  if (p->batch == 0 || s.OHc <= 0 || s.OWc <= 0 || s.He <= 0 || s.We <= 0) {
    // this rank has no share of the batch: it contributes zeros, through one
    // split of zero partial sums, so that the peers still get its flags
    planWu(*p, s, ctx->sm_count, 1, opt ? opt->plan_flags : 0, &a, nullptr);
    a.ksplit = 1;
    void *ws = nullptr;
    if (int rc = scratch(ctx, kSlotOperands, w_elems * sizeof(float), &ws)) return rc;
    PLB_CUDA(cudaMemsetAsync(ws, 0, w_elems * sizeof(float), ctx->stream));
    a.partial = static_cast<float *>(ws);
    for (unsigned g = 0; g < p->groups; ++g) {
      if (int rc = launchWuReduce(ctx->stream, a, w_elems, g, d_weight_grads, d_weight_grads_f32, &pa))
        return rc;
      ++launches;
    }
    ctx->launches += launches;
    return PLB_OK;
  }
  planWu(*p, s, ctx->sm_count, opt ? opt->split_k : 0, opt ? opt->plan_flags : 0, &a, nullptr);
  void *ws = nullptr;
  if (int rc = scratch(ctx, kSlotOperands, size_t(a.ksplit) * w_elems * sizeof(float), &ws)) return rc;
  a.partial = static_cast<float *>(ws);
  if (int rc = launchWu(ctx->stream, *p, s, a, d_acts, d_out_grads, d_weight_grads, d_weight_grads_f32,
                        &launches, &pa))
    return rc;
  ctx->launches += launches;
  return PLB_OK;
}

extern "C" int plb_conv_wu_allreduce(plb_context *ctx, const plb_conv_params *p,
                                     const plb_conv_options *opt, const void *d_acts,
                                     const void *d_out_grads, int32_t rank, int32_t world,
                                     void *const *d_peer_grads, void *const *d_peer_flags,
                                     uint32_t epoch, void *d_weight_grads,
                                     float *d_weight_grads_f32) {
  return wuAllreduce(ctx, p, opt, d_acts, d_out_grads, rank, world, d_peer_grads, nullptr,
                     d_peer_flags, epoch, d_weight_grads, d_weight_grads_f32);
}

extern "C" int plb_conv_wu_allreduce_owners(plb_context *ctx, const plb_conv_params *p,
                                            const plb_conv_options *opt, const void *d_acts,
                                            const void *d_out_grads, int32_t rank, int32_t world,
                                            void *const *d_peer_grads,
                                            void *const *d_peer_results,
                                            void *const *d_peer_flags, uint32_t epoch,
                                            void *d_weight_grads, float *d_weight_grads_f32) {
  if (!d_peer_results) return fail(PLB_ERR_INVALID_PARAMS, "null pointer table");
  return wuAllreduce(ctx, p, opt, d_acts, d_out_grads, rank, world, d_peer_grads, d_peer_results,
                     d_peer_flags, epoch, d_weight_grads, d_weight_grads_f32);
}

// ---------------------------------------------------------------------------
// Weight update for callers that must not allocate device memory
// ---------------------------------------------------------------------------
// Some callers of this library cannot call cudaMalloc when they need a weight
// gradient: code running inside a framework's allocator hooks or under a
// caching allocator that owns all device memory, real-time loops that may not
// take the allocator's global lock, and processes whose memory budget was fixed
// at start-up.  plb_conv_wu grows a scratch buffer with cudaMalloc on demand;
// this entry point instead keeps the split-K partial sums in a fixed array that
// is part of the library's device image.  Every GPU that loads the library
// holds these bytes until the process exits, so the size is kept modest.

namespace {

constexpr size_t kStaticScratchBytes = size_t(32) << 20;  // 32 MiB
static __device__ __align__(256) unsigned char g_wu_static_scratch[kStaticScratchBytes];
static __device__ int g_wu_static_status;

// Device addresses of the two symbols, looked up once per device.  In host code
// the arrays' names are only host-side handles for the symbols, not device
// addresses: kernels must be given what cudaGetSymbolAddress returns.
struct StaticScratch {
  bool ready = false;
  float *partial = nullptr;
  int *status = nullptr;
  int sm_count = 0;
};
StaticScratch g_static_scratch[64];
std::mutex g_static_scratch_mutex;

int staticScratchFor(int device, StaticScratch *out) {
  if (device < 0 || device >= 64) return fail(PLB_ERR_INVALID_PARAMS, "device ordinal out of range");
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  StaticScratch &s = g_static_scratch[device];
  if (!s.ready) {
    // the caller has made `device` current
    void *scratch_ptr = nullptr, *status_ptr = nullptr;
    PLB_CUDA(cudaGetSymbolAddress(&scratch_ptr, g_wu_static_scratch));
    PLB_CUDA(cudaGetSymbolAddress(&status_ptr, g_wu_static_status));
    PLB_CUDA(cudaDeviceGetAttribute(&s.sm_count, cudaDevAttrMultiProcessorCount, device));
    s.partial = static_cast<float *>(scratch_ptr);
    s.status = static_cast<int *>(status_ptr);
    s.ready = true;
  }
  *out = s;
  return PLB_OK;
}

}  // namespace

extern "C" int plb_conv_wu_static_scratch(int device, void *cuda_stream, const plb_conv_params *p,
                                          const plb_conv_options *opt, const void *d_acts,
                                          const void *d_out_grads, void *d_weight_grads,
                                          float *d_weight_grads_f32) {
  if (!p) return fail(PLB_ERR_INVALID_PARAMS, "null params");
  if (int rc = checkConvRequest(*p, true, nullptr, 0, nullptr, 0, nullptr, 0)) return rc;
  if (p->input_type != PLB_HALF)
    // float operands need scratch for their bfloat16 pieces
    return fail(PLB_ERR_UNSUPPORTED, "plb_conv_wu_static_scratch takes half operands; use plb_conv_wu for this layer");
  PLB_CUDA(cudaSetDevice(device));
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  WuShape s;
  if (int rc = wuShape(*p, &s)) return rc;
  const int co = int(p->out_chans_per_group), ci = int(p->in_chans_per_group);
  const int taps = s.KH * s.KW;
  const size_t w_elems = size_t(taps) * co * ci;
  if (p->groups == 0 || w_elems == 0) return PLB_OK;
  if (w_elems * sizeof(float) > kStaticScratchBytes)
    return fail(PLB_ERR_UNSUPPORTED,
                "weight gradient of " + std::to_string(w_elems * sizeof(float)) +
                    " bytes per group exceeds the " + std::to_string(kStaticScratchBytes) +
                    "-byte static scratch of plb_conv_wu_static_scratch; use plb_conv_wu");
  {
    size_t n_in, n_w, n_out;
    convElementCounts(*p, &n_in, &n_w, &n_out);
    if (n_in == 0 || n_out == 0) n_in = n_out = 0;
    const void *result = d_weight_grads ? d_weight_grads : static_cast<const void *>(d_weight_grads_f32);
    if (int rc = checkConvRequest(*p, true, d_acts, n_in, d_out_grads, n_out, result, n_w)) return rc;
  }
  // This entry point runs none of plb_conv_wu's preparatory passes (they need
  // scratch memory of their own): say so instead of failing inside the launch.
  if (ci % 8 != 0 || co % 8 != 0)
    return fail(PLB_ERR_UNSUPPORTED,
                "plb_conv_wu_static_scratch needs channel counts per group that are multiples of 8 "
                "(plb_conv_wu pads other counts in scratch memory); use plb_conv_wu");
  StaticScratch scratch;
  if (int rc = staticScratchFor(device, &scratch)) return rc;
  if (int rc = configureWuKernel(device)) return rc;
  const size_t es = 2;
  if (p->batch == 0 || s.OHc <= 0 || s.OWc <= 0 || s.He <= 0 || s.We <= 0) {
    const size_t n = size_t(p->groups) * w_elems;
    if (d_weight_grads) PLB_CUDA(cudaMemsetAsync(d_weight_grads, 0, n * es, stream));
    if (d_weight_grads_f32) PLB_CUDA(cudaMemsetAsync(d_weight_grads_f32, 0, n * sizeof(float), stream));
    PLB_CUDA(cudaStreamSynchronize(stream));
    return PLB_OK;
  }
  WuArgs a{};
  planWu(*p, s, scratch.sm_count, opt ? opt->split_k : 0, opt ? opt->plan_flags : 0, &a, nullptr);
  // as many K splits as the fixed scratch can hold
  const int max_split = int(kStaticScratchBytes / (w_elems * sizeof(float)));
  a.ksplit = std::max(1, std::min(a.ksplit, max_split));
  a.partial = scratch.partial;
  a.status = scratch.status;
  // the array keeps whatever the previous call left: the status word must start
  // at zero; the partial sums need no clearing, every CTA overwrites its slice
  PLB_CUDA(cudaMemsetAsync(scratch.status, 0, sizeof(int), stream));

  if (int rc = launchWu(stream, *p, s, a, d_acts, d_out_grads, d_weight_grads, d_weight_grads_f32,
                        nullptr))
    return rc;
  // report a kernel that gave up on a bounded wait; this also makes the call
  // complete before it returns, so a second call cannot overlap the first
  PLB_CUDA(cudaStreamSynchronize(stream));
  int status = 0;
  PLB_CUDA(cudaMemcpy(&status, scratch.status, sizeof(int), cudaMemcpyDeviceToHost));
  if (status != 0)
    return fail(PLB_ERR_KERNEL, "weight update kernel reported status " + std::to_string(status));
  return PLB_OK;
}
