// Planning and launch of the implicit-GEMM kernel: CTA tile selection, pixel
// box selection, TMA tensor maps.  This replaces, for the GPU, the search the
// reference's planner does over IPU tile partitions
// (lib/poplin/ConvPlan.cpp:1100-1224, 1674-1768): the quantities chosen here
// are the CTA tile (128 pixels x 64/128/256 channels), the pixel box that makes
// up the 128 rows, the pipeline depth and the number of persistent CTAs.
#include "igemm_sm100.cuh"
#include "runtime.h"

#include <algorithm>

namespace plb {

namespace {

template <int BN, bool kFp8, bool kBMn>
int launchInstance(plb_context *ctx, const CUtensorMap &ta, const CUtensorMap &tb,
                   const IgemmArgs &args, int grid) {
  using S = IgemmSmem<BN>;
  static bool configured[64] = {};
  auto kernel = igemm_kernel<BN, kFp8, kBMn>;
  if (!configured[ctx->device & 63]) {
    PLB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
    configured[ctx->device & 63] = true;
  }
  kernel<<<grid, kIgemmThreads, S::kTotal, ctx->stream>>>(ta, tb, args);
  PLB_CUDA(cudaGetLastError());
  ctx->launches++;
  return PLB_OK;
}

template <int BN>
int stagesFor() {
  return IgemmSmem<BN>::kStages;
}

}  // namespace

int planIgemm(const IgemmProblem &p, int sm_count, plb_plan *plan) {
  const int elem = p.fp8 ? 1 : 2;
  if (p.n_total <= 0 || p.out_w <= 0 || p.out_h <= 0 || p.out_n <= 0 || p.k_per_tap <= 0)
    return fail(PLB_ERR_INVALID_PARAMS, "empty contraction reached the kernel planner");
  if (p.fp8 && p.b_mn)
    return fail(PLB_ERR_UNSUPPORTED, "MN-major right operand is only implemented for half");
  // ---- N tile: smallest padded width, ties to the wider tile ----------------
  int bn = 0;
  if (p.force_tile_n) {
    bn = p.force_tile_n;
    if (bn != 64 && bn != 128 && bn != 256)
      return fail(PLB_ERR_INVALID_OPTION, "tile_n must be 64, 128 or 256");
  } else {
    long best = -1;
    for (int cand : {256, 128, 64}) {
      const long padded = long((p.n_total + cand - 1) / cand) * cand;
      if (best < 0 || padded < best) {
        best = padded;
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
  plan->stages = bn == 64 ? stagesFor<64>() : bn == 128 ? stagesFor<128>() : stagesFor<256>();
  plan->split_k = 1;
  plan->tiles = int(best_tiles * n_tiles);
  plan->grid = std::min(plan->tiles, sm_count > 0 ? sm_count : 148);
  plan->b_mn_major = p.b_mn ? 1 : 0;
  plan->workspace_bytes = 0;
  (void)elem;
  return PLB_OK;
}

int launchIgemm(plb_context *ctx, const IgemmProblem &p, const plb_plan &plan) {
  const int elem = p.fp8 ? 1 : 2;
  const int k_elems_per_stage = kStageKBytes / elem;
  const CUtensorMapDataType dt =
      p.fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;

  CUtensorMap ta, tb;
  {
    const uint32_t box[4] = {uint32_t(k_elems_per_stage),
                             uint32_t((plan.box_w - 1) * p.stride_w + 1),
                             uint32_t((plan.box_h - 1) * p.stride_h + 1), uint32_t(plan.box_n)};
    const uint32_t es[4] = {1, uint32_t(p.stride_w), uint32_t(p.stride_h), 1};
    if (int rc = encodeTensorMap(&ta, dt, 4, p.act, p.act_dims, p.act_strides, box, es)) return rc;
  }
  {
    uint32_t box[3];
    if (p.b_mn) {
      box[0] = 64;
      box[1] = 64;
      box[2] = 1;
    } else {
      box[0] = uint32_t(k_elems_per_stage);
      box[1] = uint32_t(plan.tile_n);
      box[2] = 1;
    }
    const uint32_t es[3] = {1, 1, 1};
    if (int rc = encodeTensorMap(&tb, dt, 3, p.wgt, p.wgt_dims, p.wgt_strides, box, es)) return rc;
  }

  IgemmArgs a{};
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
  a.group_m = 16;
  a.out = p.out;
  a.ldc = p.ldc;
  a.addend = p.beta != 0.f ? p.addend : nullptr;
  a.ld_addend = p.ld_addend;
  a.bias = p.bias;
  a.alpha = p.alpha;
  a.beta = p.beta;
  a.out_is_f32 = p.out_f32 ? 1 : 0;
  a.status = ctx->d_status;

  const int grid = plan.grid;
#define PLB_DISPATCH(BN)                                                      \
  if (p.fp8) return launchInstance<BN, true, false>(ctx, ta, tb, a, grid);    \
  if (p.b_mn) return launchInstance<BN, false, true>(ctx, ta, tb, a, grid);   \
  return launchInstance<BN, false, false>(ctx, ta, tb, a, grid);
  switch (plan.tile_n) {
    case 64: PLB_DISPATCH(64)
    case 128: PLB_DISPATCH(128)
    case 256: PLB_DISPATCH(256)
    default: break;
  }
#undef PLB_DISPATCH
  return fail(PLB_ERR_INVALID_OPTION, "unsupported tile_n in plan");
}

}  // namespace plb
