// Implicit-GEMM contraction kernel for sm_100a.
//
// One kernel serves poplin::matMul and the forward / backward-data passes of
// poplin::convolution (the roles of the reference's ConvPartial1x1Out and
// ConvPartialnx1 codelets, lib/poplin/codelets/ConvPartial1x1Out.cpp:100-180,
// lib/poplin/codelets/ConvPartialnx1.cpp:115-245, together with the partial
// reduction and the cast to the output type that follow them,
// lib/poplin/Convolution.cpp:2762-2816):
//
//   out[pixel, co] = alpha * sum_{tap, ci} act[pixel + offset(tap), ci] * w[tap, co, ci]
//                    (+ beta * addend[pixel, co]) (+ bias[co])
//
// Data layout in HBM: activations NHWC (channels innermost), weights
// [tap][Co][Ci]; a matrix product is the 1x1 case with pixels = rows of A.
//
// Structure: a persistent CTA per SM walks output tiles of 128 pixels x BN
// channels.  Warp 0 is the TMA producer (one 4-D box of the activations and
// one box of the weights per K step, 128-byte swizzle, zero fill outside the
// tensor, which is what implements the padding), warp 1 issues tcgen05.mma
// with fp32 accumulators in tensor memory, warps 2-5 drain finished
// accumulators (tcgen05.ld), scale / add / cast and store them.  Two
// accumulators alternate so the epilogue of one tile overlaps the main loop
// of the next.
#pragma once

#include "sm100_prims.cuh"

namespace plb {

constexpr int kTileM = 128;        // pixels (rows) per tile = TMEM lanes
constexpr int kStageKBytes = 128;  // bytes of K per pipeline stage row (one swizzle span)
constexpr int kIgemmThreads = 192;

struct IgemmArgs {
  // ---- M side: output pixels, tiled by a (w, h, n) box of 128 pixels ------
  int box_w, box_h, box_n;
  int tiles_w, tiles_h, tiles_n;
  int out_w, out_h, out_n;  // extents of the output (matrix product: rows, 1, 1)
  // ---- N side ---------------------------------------------------------------
  int n_tiles;  // tiles of BN output channels
  int n_total;  // valid output channels
  // ---- K side ---------------------------------------------------------------
  int taps_h, taps_w;  // filter extent (1 x 1 for a matrix product)
  int k_chunks;        // stages per tap = ceil(bytes of K per tap / 128)
  int pad_h, pad_w;    // tap (r, s) reads input pixel (oh*stride_h + r*dil_h - pad_h, ...)
  int dil_h, dil_w;
  int stride_h, stride_w;  // output pixel oh starts at input row oh*stride_h (TMA traversal stride)
  int flip_h, flip_w;  // tap (r, s) uses the weights stored at (R-1-r, ...) / (..., S-1-s)
  int group_m;    // tile rasterisation: M tiles per band
  // ---- epilogue ---------------------------------------------------------------
  void *out;
  long long ldc;  // elements between consecutive output pixels
  const void *addend;
  long long ld_addend;
  const float *bias;
  float alpha, beta;
  int out_is_f32;
  int *status;
};

template <int BN>
struct IgemmSmem {
  static constexpr int kABytes = kTileM * kStageKBytes;
  static constexpr int kBBytes = BN * kStageKBytes;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBudget = 200 * 1024;
  static constexpr int kStages = (kBudget / kStageBytes) > 8 ? 8 : (kBudget / kStageBytes);
  static constexpr int kBarrierBytes = 256;
  static constexpr int kTotal = kStages * kStageBytes + kBarrierBytes + 1024;  // + alignment slack
};

// kFp8: operands are E4M3 bytes (kind::f8f6f4, 128 elements per stage row,
//       K = 32 per instruction); otherwise fp16 (64 per row, K = 16).
// kBMn: the B operand is stored K-by-N with N contiguous (a row-major right-hand
//       matrix); it is loaded as 64-column blocks and fed to the tensor core as
//       an MN-major operand.  fp16 only.
template <int BN, bool kFp8, bool kBMn>
__global__ void __launch_bounds__(kIgemmThreads, 1)
igemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
             const IgemmArgs args) {
  using S = IgemmSmem<BN>;
  constexpr int kStages = S::kStages;
  constexpr uint32_t kTmemCols = 2 * BN;  // two accumulators
  static_assert(kTmemCols >= 32 && kTmemCols <= 512 && (kTmemCols & (kTmemCols - 1)) == 0, "");
  static_assert(!(kFp8 && kBMn), "MN-major B is implemented for fp16 only");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + kStages * S::kStageBytes;
  // barrier words: full[kStages], empty[kStages], tmem_full[2], tmem_empty[2], drain
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tmem_full_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
  auto tmem_empty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
  const uint32_t drain_bar = bar_base + 8u * (2 * kStages + 4);
  const uint32_t tmem_slot = bar_base + 8u * (2 * kStages + 5);
  uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t *tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t *>(smem_gen + kStages * S::kStageBytes + 8 * (2 * kStages + 5));
  volatile int *abort_flag =
      reinterpret_cast<volatile int *>(smem_gen + kStages * S::kStageBytes + 8 * (2 * kStages + 6));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tmem_full_bar(a), 1);
      mbar_init(tmem_empty_bar(a), 128);
    }
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_ptr;

  const int m_tiles = args.tiles_w * args.tiles_h * args.tiles_n;
  const int total_tiles = m_tiles * args.n_tiles;
  const int taps = args.taps_h * args.taps_w;
  const int k_iters = taps * args.k_chunks;
  constexpr int kElemsPerStage = kFp8 ? 128 : 64;

  // tile index -> (m tile, n tile): bands of group_m M tiles, M fastest inside a band
  auto tile_coords = [&](int tile, int &m_idx, int &n_idx) {
    const int band_tiles = args.group_m * args.n_tiles;
    const int band = tile / band_tiles;
    const int within = tile - band * band_tiles;
    const int m0 = band * args.group_m;
    const int gm = min(args.group_m, m_tiles - m0);
    m_idx = m0 + within % gm;
    n_idx = within / gm;
  };

  if (warp == 0) {
    // ===================== TMA producer =====================
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        int m_idx, n_idx;
        tile_coords(tile, m_idx, n_idx);
        const int tw = m_idx % args.tiles_w;
        const int th = (m_idx / args.tiles_w) % args.tiles_h;
        const int tn = m_idx / (args.tiles_w * args.tiles_h);
        const int w0 = tw * args.box_w, h0 = th * args.box_h, n0 = tn * args.box_n;
        for (int it = 0; it < k_iters; ++it) {
          const int tap = it / args.k_chunks;
          const int kc = it - tap * args.k_chunks;
          const int r = tap / args.taps_w, s = tap - r * args.taps_w;
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
            atomicCAS(args.status, kStatusOk, kStatusProducerTimeout);
            ok = false;
            break;
          }
          const uint32_t a_dst = smem_base + stage * S::kStageBytes;
          const uint32_t b_dst = a_dst + S::kABytes;
          mbar_expect_tx(full_bar(stage), S::kStageBytes);
          tma_load_4d(a_dst, &tm_a, full_bar(stage), kc * kElemsPerStage,
                      w0 * args.stride_w + s * args.dil_w - args.pad_w,
                      h0 * args.stride_h + r * args.dil_h - args.pad_h, n0);
          const int b_tap = (args.flip_h ? args.taps_h - 1 - r : r) * args.taps_w +
                            (args.flip_w ? args.taps_w - 1 - s : s);
          if constexpr (kBMn) {
            // K rows x 64 columns per block; blocks of 64 columns are kStageKBytes*64 apart
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(b_dst + j * (64 * kStageKBytes), &tm_b, full_bar(stage),
                          n_idx * BN + j * 64, kc * 64, b_tap);
          } else {
            tma_load_3d(b_dst, &tm_b, full_bar(stage), kc * kElemsPerStage, n_idx * BN, b_tap);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      // Teardown: every copy this thread issued must have landed before the CTA
      // may exit.  In a run without errors the consumer has already waited for
      // them, so this costs one try_wait per stage.  Stages below `stage` were
      // last filled in the current round (parity `phase`), the others in the
      // previous round (parity `phase ^ 1`); a barrier that was never used
      // reports the phase before its first one as complete.
      for (int s = 0; s < kStages; ++s) {
        const uint32_t last = (s < stage) ? phase : (phase ^ 1u);
        long long start = clock64();
        while (!mbar_try_wait(full_bar(s), last)) {
          if (clock64() - start > kWaitCycleLimit) {
            atomicCAS(args.status, kStatusOk, kStatusDrainTimeout);
            break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc(kTileM, BN, 0, 0, false, kBMn);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase[2] = {0, 0};
      int local_tile = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local_tile) {
        const int acc = local_tile & 1;
        // wait for the epilogue to have drained this accumulator
        if (!mbar_wait(tmem_empty_bar(acc), acc_phase[acc] ^ 1u, abort_flag)) {
          atomicCAS(args.status, kStatusOk, kStatusMmaTimeout);
          ok = false;
          break;
        }
        acc_phase[acc] ^= 1u;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int it = 0; it < k_iters; ++it) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
            atomicCAS(args.status, kStatusOk, kStatusMmaTimeout);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_base + stage * S::kStageBytes;
          const uint32_t b_addr = a_addr + S::kABytes;
          const uint64_t a_desc = make_smem_desc(a_addr, 16, 1024);
          const uint64_t b_desc = kBMn ? make_smem_desc(b_addr, 64 * kStageKBytes, 1024)
                                       : make_smem_desc(b_addr, 16, 1024);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            // one instruction consumes 32 bytes of K: advance the start address
            // inside the swizzle span (K-major) or by 16 rows (MN-major B)
            const uint64_t a_k = a_desc + uint64_t(k * 2);
            const uint64_t b_k = b_desc + uint64_t(kBMn ? k * ((16 * kStageKBytes) >> 4) : k * 2);
            umma_ss<kFp8>(d_tmem, a_k, b_k, idesc, (it | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));  // frees the stage when these MMAs retire
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) umma_commit(tmem_full_bar(acc));
      }
      // make sure nothing is still executing before TMEM is released
      umma_commit(drain_bar);
      long long start = clock64();
      while (!mbar_try_wait(drain_bar, 0)) {
        if (clock64() - start > kWaitCycleLimit) {
          atomicCAS(args.status, kStatusOk, kStatusDrainTimeout);
          break;
        }
      }
    }
  } else {
    // ===================== epilogue (warps 2..5) =====================
    const int quarter = warp & 3;            // TMEM lanes [32*quarter, 32*quarter+32)
    const int row = quarter * 32 + lane;     // tile row handled by this thread
    uint32_t acc_phase[2] = {0, 0};
    int local_tile = 0;
    const int box_wh = args.box_w * args.box_h;
    const int rw = row % args.box_w;
    const int rh = (row / args.box_w) % args.box_h;
    const int rn = row / box_wh;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local_tile) {
      int m_idx, n_idx;
      tile_coords(tile, m_idx, n_idx);
      const int tw = m_idx % args.tiles_w;
      const int th = (m_idx / args.tiles_w) % args.tiles_h;
      const int tn = m_idx / (args.tiles_w * args.tiles_h);
      const int ow = tw * args.box_w + rw, oh = th * args.box_h + rh, on = tn * args.box_n + rn;
      const bool row_ok = (rn < args.box_n) && ow < args.out_w && oh < args.out_h && on < args.out_n;
      const long long pixel = (static_cast<long long>(on) * args.out_h + oh) * args.out_w + ow;
      const int acc = local_tile & 1;
      if (!mbar_wait(tmem_full_bar(acc), acc_phase[acc], abort_flag)) {
        atomicCAS(args.status, kStatusOk, kStatusEpilogueTimeout);
        break;
      }
      acc_phase[acc] ^= 1u;
      tc_fence_after_sync();
      const uint32_t t_addr = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
      const int col_base = n_idx * BN;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t v[32];
        __syncwarp();
        tmem_ld_32x32(t_addr + c, v);
        tmem_ld_wait();
        if (c + 32 >= BN) {
          // the accumulator is fully read: hand it back before the stores
          tc_fence_before_sync();
          mbar_arrive(tmem_empty_bar(acc));
        }
        const int col0 = col_base + c;
        if (row_ok && col0 < args.n_total) {
        float f[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]) * args.alpha;
        const int valid = min(32, args.n_total - col0);
        if (args.bias != nullptr) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j < valid) f[j] += args.bias[col0 + j];
        }
        if (args.out_is_f32) {
          float *dst = static_cast<float *>(args.out) + pixel * args.ldc + col0;
          if (args.addend != nullptr) {
            const float *src = static_cast<const float *>(args.addend) + pixel * args.ld_addend + col0;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < valid) f[j] += args.beta * src[j];
          }
          if (valid == 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              *reinterpret_cast<float4 *>(dst + j) = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < valid) dst[j] = f[j];
          }
        } else {
          __half *dst = static_cast<__half *>(args.out) + pixel * args.ldc + col0;
          if (args.addend != nullptr) {
            const __half *src = static_cast<const __half *>(args.addend) + pixel * args.ld_addend + col0;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < valid) f[j] += args.beta * __half2float(src[j]);
          }
          if (valid == 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 pk;
              __half2 h0 = __floats2half2_rn(f[j], f[j + 1]);
              __half2 h1 = __floats2half2_rn(f[j + 2], f[j + 3]);
              __half2 h2 = __floats2half2_rn(f[j + 4], f[j + 5]);
              __half2 h3 = __floats2half2_rn(f[j + 6], f[j + 7]);
              pk.x = *reinterpret_cast<uint32_t *>(&h0);
              pk.y = *reinterpret_cast<uint32_t *>(&h1);
              pk.z = *reinterpret_cast<uint32_t *>(&h2);
              pk.w = *reinterpret_cast<uint32_t *>(&h3);
              *reinterpret_cast<uint4 *>(dst + j) = pk;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < valid) dst[j] = __float2half_rn(f[j]);
          }
        }
        }  // row_ok
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace plb
