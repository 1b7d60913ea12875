// Planning and launch of the implicit-GEMM kernel: CTA tile selection, pixel
// box selection, TMA tensor maps.  This replaces, for the GPU, the search the
// reference's planner does over IPU tile partitions
// (lib/poplin/ConvPlan.cpp:1100-1224, 1674-1768): the quantities chosen here
// are the CTA tile (128 pixels x 64/128/256 channels), the pixel box that makes
// up the 128 rows, the pipeline depth and the number of persistent CTAs.
#include "igemm_sm100.cuh"
#include "runtime.h"

#include <algorithm>
#include <cstdlib>
#include <cstring>

namespace plb {

namespace {

template <int BN, bool kFp8, bool kBMn, bool kResB, bool kHalo, bool k2Cta>
int launchInstance(plb_context *ctx, const CUtensorMap &ta, const CUtensorMap &tb,
                   const CUtensorMap &tout, const IgemmArgs &args, int grid, int resident_bytes,
                   bool pdl) {
  if constexpr (k2Cta && kBMn && BN < 128) {
    return fail(PLB_ERR_INVALID_OPTION, "a CTA pair needs tile_n >= 128 for a row-major B");
  } else {
    using S = IgemmSmem<BN, kResB, k2Cta>;
    static bool configured[64] = {};
    static int max_clusters[64] = {};
    auto kernel = igemm_kernel<BN, kFp8, kBMn, kResB, kHalo, k2Cta>;
    const int dev = ctx->device & 63;
    if (!configured[dev]) {
      PLB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    kIgemmSmemLimit));
      configured[dev] = true;
    }
    const int smem =
        S::totalBytes(args.a_stage_bytes, args.b_tiles_per_stage, args.num_stages, resident_bytes);
    // Launch attributes: programmatic stream serialization (the kernel's set-up
    // may overlap the previous kernel's tail; it waits before touching global
    // memory) and, for CTA pairs, clusters of two.
    cudaLaunchConfig_t cfg{};
    cfg.blockDim = dim3(kIgemmThreads);
    cfg.dynamicSmemBytes = size_t(smem);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    unsigned n_attr = 0;
    if (pdl) {
      attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
      ++n_attr;
    }
    if constexpr (!k2Cta) {
      cfg.gridDim = dim3(unsigned(grid));
    } else {
      // a persistent grid of as many clusters as can be resident at once
      // (pairs of SMs in one GPC), each walking tile pairs
      attr[n_attr].id = cudaLaunchAttributeClusterDimension;
      attr[n_attr].val.clusterDim.x = 2;
      attr[n_attr].val.clusterDim.y = 1;
      attr[n_attr].val.clusterDim.z = 1;
      ++n_attr;
      if (max_clusters[dev] == 0) {
        // queried with the largest shared-memory size, a lower bound for smaller ones
        cudaLaunchConfig_t q = cfg;
        q.gridDim = dim3(unsigned(2 * ctx->sm_count));
        q.dynamicSmemBytes = size_t(kIgemmSmemLimit);
        q.attrs = &attr[n_attr - 1];
        q.numAttrs = 1;
        int n = 0;
        PLB_CUDA(cudaOccupancyMaxActiveClusters(&n, kernel, &q));
        if (n <= 0) return fail(PLB_ERR_CUDA, "no cluster of two CTAs can be resident on this device");
        max_clusters[dev] = n;
      }
      const int clusters = std::max(1, std::min(grid / 2, max_clusters[dev]));
      cfg.gridDim = dim3(unsigned(2 * clusters));
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    PLB_CUDA(cudaLaunchKernelEx(&cfg, kernel, ta, tb, tout, args));
    PLB_CUDA(cudaGetLastError());
    ctx->launches++;
    return PLB_OK;
  }
}

int stagesFor(int bn, int a_stage_bytes, int b_tiles, bool resident, int resident_bytes,
              bool pair) {
  const int a = a_stage_bytes;
#define PLB_STAGES(BN)                                                                         \
  return resident ? (pair ? IgemmSmem<BN, true, true>::stagesFor(a, b_tiles, resident_bytes)   \
                          : IgemmSmem<BN, true, false>::stagesFor(a, b_tiles, resident_bytes)) \
                  : (pair ? IgemmSmem<BN, false, true>::stagesFor(a, b_tiles, 0)               \
                          : IgemmSmem<BN, false, false>::stagesFor(a, b_tiles, 0));
  switch (bn) {
    case 64: PLB_STAGES(64)
    case 128: PLB_STAGES(128)
    default: PLB_STAGES(256)
  }
#undef PLB_STAGES
}

// Weights stay in shared memory when one N tile covers all output channels,
// every CTA gets several pixel tiles to amortise the load over, and the
// weights leave room for a pipeline of at least six activation stages.
constexpr int kMaxResidentBytes = 96 * 1024;

}  // namespace

int planIgemm(const IgemmProblem &p, int sm_count, plb_plan *plan) {
  const int elem = p.fp8 ? 1 : 2;
  if (p.n_total <= 0 || p.out_w <= 0 || p.out_h <= 0 || p.out_n <= 0 || p.k_per_tap <= 0)
    return fail(PLB_ERR_INVALID_PARAMS, "empty contraction reached the kernel planner");
  if (p.fp8 && p.b_mn)
    return fail(PLB_ERR_UNSUPPORTED, "MN-major right operand is only implemented for half");
  // ---- N tile ---------------------------------------------------------------
  // Cost model: waves of tiles over the SMs times the measured duration of a
  // 128 x BN x 16 tensor-core instruction (operand fetch bound: 75 / 95 / 155
  // cycles for BN = 64 / 128 / 256).  Wide tiles win whenever the grid fills
  // the device; a grid of a few tiles (small matrix products) finishes sooner
  // with narrow ones, which also spread it over more SMs.
  int bn = 0;
  if (p.force_tile_n) {
    bn = p.force_tile_n;
    if (bn != 64 && bn != 128 && bn != 256)
      return fail(PLB_ERR_INVALID_OPTION, "tile_n must be 64, 128 or 256");
  } else {
    const long sms = sm_count > 0 ? sm_count : 148;
    const long pixel_tiles = (long(p.out_w) * p.out_h * p.out_n + kTileM - 1) / kTileM;  // lower bound
    long best = -1;
    for (int cand : {256, 128, 64}) {
      const long n_tiles_c = (p.n_total + cand - 1) / cand;
      const long waves = (pixel_tiles * n_tiles_c + sms - 1) / sms;
      const long cost = waves * (cand == 256 ? 155 : cand == 128 ? 95 : 75);
      if (best < 0 || cost < best) {
        best = cost;
        bn = cand;
      }
    }
  }
  // ---- pixel box: bw*bh*bn == 128, fewest tiles, then widest rows ------------
  int bw = 0, bh = 0, bb = 0;
  long best_tiles = -1;
  for (int w = 128; w >= 1; w >>= 1)
    for (int h = 128 / w; h >= 1; h >>= 1) {
      const int n = 128 / (w * h);
      if ((w - 1) * p.stride_w + 1 > 256 || (h - 1) * p.stride_h + 1 > 256) continue;
      const long tiles = long((p.out_w + w - 1) / w) * ((p.out_h + h - 1) / h) *
                         ((p.out_n + n - 1) / n);
      if (best_tiles < 0 || tiles < best_tiles) {
        best_tiles = tiles;
        bw = w;
        bh = h;
        bb = n;
      }
    }
  const int n_tiles = (p.n_total + bn - 1) / bn;
  if (best_tiles * n_tiles > 0x7fffffffL)
    return fail(PLB_ERR_UNSUPPORTED, "too many output tiles for one launch");
  plan->kernel = 0;
  plan->tile_m = kTileM;
  plan->tile_n = bn;
  plan->tile_k_bytes = kStageKBytes;
  plan->box_w = bw;
  plan->box_h = bh;
  plan->box_n = bb;
  plan->split_k = 1;
  plan->tiles = int(best_tiles * n_tiles);
  // CTA pairs: two M tiles share one 256-row MMA, each CTA holding half of the
  // weight tile.  Needs two M tiles and, for a row-major B, a whole 64-column
  // block per CTA.
  // Worth it when every CTA pair gets several tile pairs and a tile's K loop is
  // long: the two SMs advance in lockstep per tile, which costs more than the
  // halved weight traffic saves on short tiles and on grids of a few tiles.
  // With 256-column tiles the weight tile is two thirds of a stage's bytes and
  // half the K length already pays (1x1 stride-2 layer 256 -> 512: 71 -> 67 us).
  const int k_elems_stage = kStageKBytes / elem;
  const long k_steps_per_tile =
      long(p.taps_h) * p.taps_w * ((p.k_per_tap + k_elems_stage - 1) / k_elems_stage);
  const int sms_for_pair = sm_count > 0 ? sm_count : 148;
  const bool pair = (p.plan_flags & PLB_PLAN_NO_CTA_PAIR) == 0 && (!p.b_mn || bn >= 128) &&
                    ((p.plan_flags & PLB_PLAN_FORCE_CTA_PAIR) != 0
                         ? best_tiles >= 2
                         : (k_steps_per_tile >= (bn >= 256 ? 4 : 8) &&
                            best_tiles * n_tiles >= 2L * sms_for_pair));
  plan->cta_pair = pair ? 1 : 0;
  auto grid_for = [&](long m_tiles) {
    const int sms = sm_count > 0 ? sm_count : 148;
    if (!pair) return int(std::min<long>(m_tiles * n_tiles, sms));
    return int(2 * std::min<long>(((m_tiles + 1) / 2) * n_tiles, sms / 2));
  };
  plan->grid = grid_for(best_tiles);
  const int k_elems = kStageKBytes / elem;
  const long k_iters = long(p.taps_h) * p.taps_w * ((p.k_per_tap + k_elems - 1) / k_elems);
  // per CTA
  const long resident_bytes = k_iters * (bn / (pair ? 2 : 1)) * kStageKBytes;
  const bool want_resident = (p.plan_flags & PLB_PLAN_FORCE_RESIDENT_WEIGHTS) != 0 ||
                             plan->tiles >= 2 * plan->grid;
  plan->resident_weights =
      ((p.plan_flags & PLB_PLAN_NO_RESIDENT_WEIGHTS) == 0 && n_tiles == 1 &&
       resident_bytes <= kMaxResidentBytes && want_resident)
          ? 1
          : 0;
  plan->halo_rows = 0;
  plan->stages = stagesFor(bn, kTileM * kStageKBytes, 1, plan->resident_weights != 0,
                           plan->resident_weights ? int(resident_bytes) : 0, pair);
  // Halo mode: with resident weights and a filter taller than one row (unit
  // vertical stride), load (box_h + halo) input rows once per horizontal tap
  // instead of box_h rows per tap.  The tile rows are ordered (w, n, h) so that
  // a vertical shift is a whole number of 8-row groups: box_w * box_n % 8 == 0.
  const int halo = (p.taps_h - 1) * p.dil_h;
  if ((p.plan_flags & PLB_PLAN_NO_HALO) == 0 && p.taps_h > 1 &&
      p.stride_h == 1) {
    // Shared-memory fill per pixel tile and channel chunk, the quantity that
    // bounds a layer whose tensor-core work is short: activation rows plus,
    // unless the weights are resident, one weight tile per filter tap.
    const bool res = plan->resident_weights != 0;
    const long b_tile = res ? 0 : long(bn / (pair ? 2 : 1)) * kStageKBytes;
    const long base_cost =
        best_tiles * p.taps_h * p.taps_w * (long(kTileM) * kStageKBytes + b_tile);
    long best_cost = -1, best_t = -1;
    int hw = 0, hh = 0, hn = 0;
    for (int w = 128; w >= 1; w >>= 1)
      for (int n = 128 / w; n >= 1; n >>= 1) {
        const int h = 128 / (w * n);
        if ((w * n) % 8 != 0 || h + halo > 256 || (w - 1) * p.stride_w + 1 > 256) continue;
        const long tiles = long((p.out_w + w - 1) / w) * ((p.out_h + h - 1) / h) *
                           ((p.out_n + n - 1) / n);
        const long cost =
            tiles * p.taps_w * (long(w) * n * (h + halo) * kStageKBytes + p.taps_h * b_tile);
        if (best_cost < 0 || cost < best_cost || (cost == best_cost && tiles < best_t)) {
          best_cost = cost;
          best_t = tiles;
          hw = w;
          hh = h;
          hn = n;
        }
      }
    if (best_cost > 0) {
      const int a_stage = hw * hn * (hh + halo) * kStageKBytes;
      const int st = stagesFor(bn, a_stage, res ? 1 : p.taps_h, res, res ? int(resident_bytes) : 0,
                               pair);
      // worthwhile only if it really fills less, without much more tensor-core
      // work (padded tiles), and still leaves a pipeline
      if (st >= 3 && best_cost < base_cost && best_t * 8 <= best_tiles * 9) {
        plan->halo_rows = halo;
        plan->box_w = hw;
        plan->box_h = hh;
        plan->box_n = hn;
        plan->stages = st;
        plan->tiles = int(best_t * n_tiles);
        plan->grid = grid_for(best_t);
      }
    }
  }
  plan->b_mn_major = p.b_mn ? 1 : 0;
  plan->workspace_bytes = 0;
  // ---- split-K ---------------------------------------------------------------
  // A product with few output tiles and a long reduction leaves most SMs idle:
  // let several CTAs share a tile, each taking a range of its pipeline steps,
  // and add their fp32 partial sums in a second kernel.  Model (microseconds):
  // a pipeline step of one CTA takes about 0.17 (the producers' issue rate
  // bounds short tiles), the extra kernel about 5 plus its traffic at a few
  // TB/s; the split must save more than it costs.  512 x 1024 x 1024 stays
  // unsplit (16 steps: 2.7 against 1.4 + 5), 256 x 8192 x 256 splits.
  {
    const long units = plan->tiles / (pair ? 2 : 1) + (pair ? plan->tiles % 2 : 0);
    const long steps = plan->halo_rows > 0 ? long(p.taps_w) * ((p.k_per_tap + k_elems - 1) / k_elems)
                                           : k_iters;
    const long sms = sm_count > 0 ? sm_count : 148;
    int split = 1;
    if (p.force_split_k > 0) {
      split = int(std::min<long>(p.force_split_k, steps));
    } else if (units * 2 <= sms && steps >= 16) {
      const double out_mb = double(p.out_w) * p.out_h * p.out_n * p.n_total * 4 / 1e6;
      double best = 0.17 * double(steps);
      for (long sp = 2; sp <= std::min<long>(steps / 4, sms / units); ++sp) {
        const double t = 0.17 * double((steps + sp - 1) / sp) + 5.0 + out_mb * double(sp + 1) / 4000.0;
        if (t < best) {
          best = t;
          split = int(sp);
        }
      }
    }
    if (split > 1 && long(plan->tiles) * split > 0x3fffffffL) split = 1;
    plan->split_k = split;
    if (split > 1) {
      const long units_total = units * split;
      plan->grid = pair ? int(2 * std::min<long>(units_total, sms / 2)) : int(std::min<long>(units_total, sms));
      const size_t ld_p = (size_t(p.n_total) + 31) / 32 * 32;
      plan->workspace_bytes = uint64_t(split) * p.out_w * p.out_h * p.out_n * ld_p * sizeof(float);
    }
  }
  return PLB_OK;
}

namespace {

// Second kernel of a split-K product: adds the splits' partial sums in split
// order (a fixed order, so the result does not depend on timing) and applies
// what the implicit-GEMM kernel's own epilogue would have: alpha, bias, the
// beta-scaled addend, the cast.  One thread per four consecutive channels of
// one output pixel.
struct SplitKReduceArgs {
  const float *partial;
  int split_k;
  long long split_stride;  // elements between splits
  int ld_p;                // elements between pixels in the partial sums
  int n_total, out_w, out_h, out_n;
  void *out;
  long long ldc, out_stride_h, out_stride_n;
  const void *addend;
  long long ld_addend;
  const float *bias;
  float alpha, beta;
  int out_is_f32;
};

__global__ void __launch_bounds__(256) igemm_splitk_reduce_kernel(const SplitKReduceArgs a) {
  pdl_launch_dependents();
  pdl_wait();  // the partial sums come from the previous kernel in the stream
  const int quads = (a.n_total + 3) / 4;
  const long long pixels = (long long)a.out_w * a.out_h * a.out_n;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < pixels * quads;
       i += (long long)gridDim.x * blockDim.x) {
    const long long pixel = i / quads;
    const int c = int(i - pixel * quads) * 4;
    const float *src = a.partial + pixel * a.ld_p + c;
    float4 s = *reinterpret_cast<const float4 *>(src);
    for (int k = 1; k < a.split_k; ++k) {
      const float4 v = *reinterpret_cast<const float4 *>(src + k * a.split_stride);
      s.x += v.x;
      s.y += v.y;
      s.z += v.z;
      s.w += v.w;
    }
    float f[4] = {s.x, s.y, s.z, s.w};
    const int valid = min(4, a.n_total - c);
    if (a.alpha != 1.f)
      for (int j = 0; j < 4; ++j) f[j] *= a.alpha;
    if (a.bias != nullptr)
      for (int j = 0; j < valid; ++j) f[j] += a.bias[c + j];
    if (a.addend != nullptr) {
      if (a.out_is_f32) {
        const float *ad = static_cast<const float *>(a.addend) + pixel * a.ld_addend + c;
        for (int j = 0; j < valid; ++j) f[j] += a.beta * ad[j];
      } else {
        const __half *ad = static_cast<const __half *>(a.addend) + pixel * a.ld_addend + c;
        for (int j = 0; j < valid; ++j) f[j] += a.beta * __half2float(ad[j]);
      }
    }
    const long long ow = pixel % a.out_w, rest = pixel / a.out_w;
    const long long oh = rest % a.out_h, on = rest / a.out_h;
    const long long off = on * a.out_stride_n + oh * a.out_stride_h + ow * a.ldc + c;
    if (a.out_is_f32) {
      float *dst = static_cast<float *>(a.out) + off;
      if (valid == 4 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0)
        *reinterpret_cast<float4 *>(dst) = make_float4(f[0], f[1], f[2], f[3]);
      else
        for (int j = 0; j < valid; ++j) dst[j] = f[j];
    } else {
      __half *dst = static_cast<__half *>(a.out) + off;
      if (valid == 4 && (reinterpret_cast<uintptr_t>(dst) & 7) == 0) {
        const __half2 lo = __floats2half2_rn(f[0], f[1]), hi = __floats2half2_rn(f[2], f[3]);
        *reinterpret_cast<uint2 *>(dst) = make_uint2(*reinterpret_cast<const uint32_t *>(&lo),
                                                     *reinterpret_cast<const uint32_t *>(&hi));
      } else {
        for (int j = 0; j < valid; ++j) dst[j] = __float2half_rn(f[j]);
      }
    }
  }
}

}  // namespace

int launchIgemm(plb_context *ctx, const IgemmProblem &p, const plb_plan &plan) {
  const int elem = p.fp8 ? 1 : 2;
  const int k_elems_per_stage = kStageKBytes / elem;
  const CUtensorMapDataType dt =
      p.fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;

  const bool halo = plan.halo_rows > 0;
  // In halo mode the pixel dimensions are ordered (w, n, h) in every tensor map.
  auto order = [&](uint64_t w, uint64_t h, uint64_t n, uint64_t *out3) {
    out3[0] = w;
    out3[1] = halo ? n : h;
    out3[2] = halo ? h : n;
  };
  CUtensorMap ta, tb;
  {
    uint64_t dims[4] = {p.act_dims[0], 0, 0, 0}, strides[3];
    order(p.act_dims[1], p.act_dims[2], p.act_dims[3], dims + 1);
    strides[0] = p.act_strides[0];
    strides[1] = halo ? p.act_strides[2] : p.act_strides[1];
    strides[2] = halo ? p.act_strides[1] : p.act_strides[2];
    uint64_t b3[3];
    order(uint64_t((plan.box_w - 1) * p.stride_w + 1),
          uint64_t((plan.box_h + plan.halo_rows - 1) * p.stride_h + 1), uint64_t(plan.box_n), b3);
    const uint32_t box[4] = {uint32_t(k_elems_per_stage), uint32_t(b3[0]), uint32_t(b3[1]),
                             uint32_t(b3[2])};
    uint64_t e3[3];
    order(uint64_t(p.stride_w), uint64_t(p.stride_h), 1, e3);
    const uint32_t es[4] = {1, uint32_t(e3[0]), uint32_t(e3[1]), uint32_t(e3[2])};
    if (int rc = encodeTensorMap(&ta, dt, 4, p.act, dims, strides, box, es)) return rc;
  }
  {
    uint32_t box[3];
    if (p.b_mn) {
      box[0] = 64;
      box[1] = 64;
      box[2] = 1;
    } else {
      box[0] = uint32_t(k_elems_per_stage);
      box[1] = uint32_t(plan.tile_n / (plan.cta_pair ? 2 : 1));
      box[2] = 1;
    }
    const uint32_t es[3] = {1, 1, 1};
    if (int rc = encodeTensorMap(&tb, dt, 3, p.wgt, p.wgt_dims, p.wgt_strides, box, es)) return rc;
  }

  IgemmArgs a{};
  a.split_k = std::max(1, int(plan.split_k));
  a.fd_split = make_fastdiv(uint32_t(a.split_k));
  const bool split = a.split_k > 1;
  const size_t ld_p = (size_t(p.n_total) + 31) / 32 * 32;
  float *partial = nullptr;
  if (split) {
    void *ws = nullptr;
    a.split_stride = (long long)p.out_w * p.out_h * p.out_n * (long long)ld_p;
    if (int rc = scratch(ctx, kSlotSplitK, size_t(a.split_k) * size_t(a.split_stride) * sizeof(float), &ws))
      return rc;
    partial = static_cast<float *>(ws);
  }
  // Output through TMA when the tensor can be described to it: 16-byte aligned
  // base and pixel stride.  Each epilogue warp stores a (columns, w, h, n) box
  // holding its 32 pixels and 32 columns: 128-byte rows of fp32, 64-byte rows
  // (64-byte swizzle) of half.
  CUtensorMap tout;
  std::memset(&tout, 0, sizeof tout);
  const size_t out_es = p.out_f32 ? 4 : 2;
  const long long out_stride_h = p.out_stride_h ? p.out_stride_h : (long long)p.out_w * p.ldc;
  const long long out_stride_n =
      p.out_stride_n ? p.out_stride_n : (long long)p.out_h * p.out_w * p.ldc;
  // the 32 rows of one epilogue warp as a box over the tile's row order
  const int d2 = halo ? plan.box_n : plan.box_h;
  a.sub_w = std::min(plan.box_w, 32);
  a.sub_h = std::min(d2, 32 / a.sub_w);  // extent along the second row dimension
  const int sub_3 = 32 / (a.sub_w * a.sub_h);
  a.use_tma_store = 0;
  if (!split && (p.plan_flags & PLB_PLAN_NO_TMA_STORE) == 0 &&
      (reinterpret_cast<uintptr_t>(p.out) & 15) == 0 &&
      (size_t(p.ldc) * out_es) % 16 == 0 && (size_t(out_stride_h) * out_es) % 16 == 0 &&
      (size_t(out_stride_n) * out_es) % 16 == 0) {
    uint64_t dims[4] = {uint64_t(p.n_total), 0, 0, 0}, strides[3];
    order(uint64_t(p.out_w), uint64_t(p.out_h), uint64_t(p.out_n), dims + 1);
    const uint64_t sw = uint64_t(p.ldc) * out_es, sh = uint64_t(out_stride_h) * out_es,
                   sn = uint64_t(out_stride_n) * out_es;
    strides[0] = sw;
    strides[1] = halo ? sn : sh;
    strides[2] = halo ? sh : sn;
    const uint32_t box[4] = {32u, uint32_t(a.sub_w), uint32_t(a.sub_h), uint32_t(sub_3)};
    const uint32_t es[4] = {1, 1, 1, 1};
    if (int rc = encodeTensorMap(&tout,
                                 p.out_f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                           : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                                 4, p.out, dims, strides, box, es, p.out_f32 ? 128 : 64))
      return rc;
    a.use_tma_store = 1;
  }
  a.box_w = plan.box_w;
  a.box_h = plan.box_h;
  a.box_n = plan.box_n;
  a.tiles_w = (p.out_w + plan.box_w - 1) / plan.box_w;
  a.tiles_h = (p.out_h + plan.box_h - 1) / plan.box_h;
  a.tiles_n = (p.out_n + plan.box_n - 1) / plan.box_n;
  a.out_w = p.out_w;
  a.out_h = p.out_h;
  a.out_n = p.out_n;
  a.n_tiles = (p.n_total + plan.tile_n - 1) / plan.tile_n;
  a.n_total = p.n_total;
  a.taps_h = p.taps_h;
  a.taps_w = p.taps_w;
  a.k_chunks = (p.k_per_tap + k_elems_per_stage - 1) / k_elems_per_stage;
  a.pad_h = p.pad_h;
  a.pad_w = p.pad_w;
  a.dil_h = p.dil_h;
  a.dil_w = p.dil_w;
  a.stride_h = p.stride_h;
  a.stride_w = p.stride_w;
  a.flip_h = p.flip_h;
  a.flip_w = p.flip_w;
  a.group_m = plan.cta_pair ? 8 : 16;  // M tiles (pairs of them) per band
  a.h_outer = halo ? 1 : 0;
  a.fd_band = make_fastdiv(uint32_t(std::max(1, a.group_m * a.n_tiles)));
  a.fd_gm = make_fastdiv(uint32_t(std::max(1, a.group_m)));
  a.fd_tw = make_fastdiv(uint32_t(std::max(1, a.tiles_w)));
  a.fd_inner = make_fastdiv(uint32_t(std::max(1, a.h_outer ? a.tiles_n : a.tiles_h)));
  a.a_stage_bytes = plan.box_w * plan.box_n * (plan.box_h + plan.halo_rows) * kStageKBytes;
  a.b_tiles_per_stage = (halo && !plan.resident_weights) ? p.taps_h : 1;
  a.halo_step_bytes = p.dil_h * plan.box_w * plan.box_n * kStageKBytes;
  a.num_stages = plan.stages;
  // Short tiles (few tensor-core instructions each) are bound by what one
  // thread can issue and wait for per tile: let two issuers take alternate tiles.
  {
    const int steps_per_tile = halo ? a.taps_w * a.k_chunks : a.taps_h * a.taps_w * a.k_chunks;
    const int mmas_per_tile = a.taps_h * a.taps_w * a.k_chunks * 4;
    // (only with CTA pairs and 64-column tiles, the case it was built and
    // verified for: weights resident or streamed, halo strips)
    a.dual_issue = ((p.plan_flags & PLB_PLAN_NO_DUAL_ISSUE) == 0 && steps_per_tile <= 4 && mmas_per_tile <= 48 &&
                    plan.tiles >= 2 * plan.grid && plan.cta_pair && plan.tile_n == 64)
                       ? 1
                       : 0;
  }
  const int resident_bytes =
      plan.resident_weights ? a.taps_h * a.taps_w * a.k_chunks *
                                  (plan.tile_n / (plan.cta_pair ? 2 : 1)) * kStageKBytes
                            : 0;
  a.out = p.out;
  a.ldc = p.ldc;
  a.out_stride_h = out_stride_h;
  a.out_stride_n = out_stride_n;
  a.addend = p.beta != 0.f ? p.addend : nullptr;
  a.ld_addend = p.ld_addend;
  a.bias = p.bias;
  if (split) {
    // raw fp32 sums, dense in pixels, into this split's slice of the scratch
    a.out = partial;
    a.ldc = (long long)ld_p;
    a.out_stride_h = (long long)p.out_w * a.ldc;
    a.out_stride_n = (long long)p.out_h * a.out_stride_h;
    a.addend = nullptr;
    a.bias = nullptr;
  }
  a.idesc_formats = p.bf16 ? make_idesc(0, 0, 1, 1, false, false) & ~(1u << 4)
                    : p.fp8 ? make_idesc(0, 0, uint32_t(p.fmt_a & 1), uint32_t(p.fmt_b & 1), false, false) & ~(1u << 4)
                          : 0u;
  a.alpha = split ? 1.f : p.alpha;
  a.beta = split ? 0.f : p.beta;
  a.out_is_f32 = split || p.out_f32 ? 1 : 0;
  a.status = ctx->d_status;
  a.trace = ctx->trace;

  const int grid = plan.grid;
  const bool pdl = (p.plan_flags & PLB_PLAN_NO_PDL) == 0;
  auto dispatch = [&]() -> int {
#define PLB_DISPATCH3(BN, RES, HALO, PAIR)                                                            \
  if (p.fp8)                                                                                          \
    return launchInstance<BN, true, false, RES, HALO, PAIR>(ctx, ta, tb, tout, a, grid,               \
                                                            resident_bytes, pdl);                          \
  if (p.b_mn)                                                                                         \
    return launchInstance<BN, false, true, RES, HALO, PAIR>(ctx, ta, tb, tout, a, grid,               \
                                                            resident_bytes, pdl);                          \
  return launchInstance<BN, false, false, RES, HALO, PAIR>(ctx, ta, tb, tout, a, grid, resident_bytes, pdl);
#define PLB_DISPATCH2(BN, RES, HALO)     \
  if (plan.cta_pair) {                   \
    PLB_DISPATCH3(BN, RES, HALO, true)   \
  } else {                               \
    PLB_DISPATCH3(BN, RES, HALO, false)  \
  }
#define PLB_DISPATCH(BN)                       \
  if (halo && plan.resident_weights) {         \
    PLB_DISPATCH2(BN, true, true)              \
  } else if (halo) {                           \
    PLB_DISPATCH2(BN, false, true)             \
  } else if (plan.resident_weights) {          \
    PLB_DISPATCH2(BN, true, false)             \
  } else {                                     \
    PLB_DISPATCH2(BN, false, false)            \
  }
  switch (plan.tile_n) {
    case 64: PLB_DISPATCH(64)
    case 128: PLB_DISPATCH(128)
    case 256: PLB_DISPATCH(256)
    default: break;
  }
#undef PLB_DISPATCH
#undef PLB_DISPATCH2
#undef PLB_DISPATCH3
    return fail(PLB_ERR_INVALID_OPTION, "unsupported tile_n in plan");
  };
  if (int rc = dispatch()) return rc;
  if (!split) return PLB_OK;
  SplitKReduceArgs r{};
  r.partial = partial;
  r.split_k = a.split_k;
  r.split_stride = a.split_stride;
  r.ld_p = int(ld_p);
  r.n_total = p.n_total;
  r.out_w = p.out_w;
  r.out_h = p.out_h;
  r.out_n = p.out_n;
  r.out = p.out;
  r.ldc = p.ldc;
  r.out_stride_h = out_stride_h;
  r.out_stride_n = out_stride_n;
  r.addend = p.beta != 0.f ? p.addend : nullptr;
  r.ld_addend = p.ld_addend;
  r.bias = p.bias;
  r.alpha = p.alpha;
  r.beta = p.beta;
  r.out_is_f32 = p.out_f32 ? 1 : 0;
  const long long work = (long long)p.out_w * p.out_h * p.out_n * ((p.n_total + 3) / 4);
  cudaLaunchAttribute pdl_attr[1];
  pdl_attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  pdl_attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(unsigned(std::max<long long>(1, std::min<long long>((work + 255) / 256,
                                                                         (long long)ctx->sm_count * 8))));
  cfg.blockDim = dim3(256);
  cfg.stream = ctx->stream;
  cfg.attrs = pdl_attr;
  cfg.numAttrs = pdl ? 1 : 0;
  PLB_CUDA(cudaLaunchKernelEx(&cfg, igemm_splitk_reduce_kernel, r));
  PLB_CUDA(cudaGetLastError());
  ctx->launches++;
  return PLB_OK;
}

}  // namespace plb
