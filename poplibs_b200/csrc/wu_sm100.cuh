// Weight-update (weight-gradient) kernel for sm_100a.
//
//   dW[tap][co][ci] = sum over pixels (n, oh, ow) of
//                     outGrad[n, oh, ow, co] * act[n, oh*stride + tap offset, ..., ci]
//
// This is the contraction poplin::calculateWeightDeltas builds by swapping the
// batch and input-channel axes of the forward convolution
// (lib/poplin/Convolution.cpp:3390-3507); its reduction runs over the whole
// batch and output field.  Both operands are NHWC, i.e. the reduction index
// (pixels) is the slow axis of both: the tensor core reads them as MN-major
// operands straight from the TMA-written tiles, no transposition anywhere.
//
// Work split: the grid is (Co blocks of 128) x (Ci blocks) x (groups of filter
// taps whose accumulators fit the 512 TMEM columns) x (K splits over pixel
// tiles).  Every CTA leaves its partial sums in a global fp32 scratch buffer;
// a second kernel adds the K splits in a fixed order (the role of the
// reference's ReduceAdd codelet, lib/poplin/codelets/ReduceAdd.cpp) and casts.
#pragma once

#include "sm100_prims.cuh"

namespace plb {

constexpr int kWuThreads = 192;
constexpr int kWuPixelsPerStage = 64;   // K per pipeline stage
constexpr int kWuBlockBytes = kWuPixelsPerStage * 128;  // one 64-channel block of one stage
constexpr int kWuMaxStages = 8;

struct WuArgs {
  int box_w, box_h, box_n;        // pixel box of one stage (product 64)
  int tiles_w, tiles_h, tiles_n;  // pixel tiles over the output field and batch
  int taps_h, taps_w;
  int pad_h, pad_w, dil_h, dil_w, stride_h, stride_w;
  int taps_per_group, tap_groups;
  int co_blocks, ci_blocks;
  int ci_blk;     // accumulator columns per tap (multiple of 16, <= 256)
  int ci_blk64;   // 64-channel blocks loaded per tap = ceil(ci_blk / 64)
  int co_total, ci_total;
  int ksplit;
  int stages;
  int tmem_cols;
  float *partial;  // [ksplit][taps][co_total][ci_total]
  int *status;
};

__global__ void __launch_bounds__(kWuThreads, 1)
wu_kernel(const __grid_constant__ CUtensorMap tm_dy, const __grid_constant__ CUtensorMap tm_x,
          const WuArgs args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int a_bytes = 2 * kWuBlockBytes;  // 128 output channels
  const int b_bytes = args.taps_per_group * args.ci_blk64 * kWuBlockBytes;
  const int stage_bytes = a_bytes + b_bytes;
  const int stages = args.stages;
  const uint32_t bar_base = smem_base + stages * stage_bytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kWuMaxStages + s); };
  const uint32_t acc_bar = bar_base + 8u * (2 * kWuMaxStages);
  const uint32_t tmem_slot = bar_base + 8u * (2 * kWuMaxStages + 1);
  uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t *tmem_slot_ptr = reinterpret_cast<volatile uint32_t *>(
      smem_gen + stages * stage_bytes + 8 * (2 * kWuMaxStages + 1));
  volatile int *abort_flag = reinterpret_cast<volatile int *>(
      smem_gen + stages * stage_bytes + 8 * (2 * kWuMaxStages + 2));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(acc_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_dy);
    tma_prefetch_desc(&tm_x);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, uint32_t(args.tmem_cols));
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_ptr;

  // ---- which unit of work is this CTA's ------------------------------------
  int unit = blockIdx.x;
  const int split = unit % args.ksplit;
  unit /= args.ksplit;
  const int tap_group = unit % args.tap_groups;
  unit /= args.tap_groups;
  const int ci_block = unit % args.ci_blocks;
  const int co_block = unit / args.ci_blocks;
  const int taps = args.taps_h * args.taps_w;
  const int tap0 = tap_group * args.taps_per_group;
  const int ntaps = min(args.taps_per_group, taps - tap0);
  const int pixel_tiles = args.tiles_w * args.tiles_h * args.tiles_n;
  const int t_begin = int((long long)pixel_tiles * split / args.ksplit);
  const int t_end = int((long long)pixel_tiles * (split + 1) / args.ksplit);
  const int k_iters = t_end - t_begin;

  if (warp == 0) {
    // ===================== TMA producer =====================
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      for (int it = 0; it < k_iters; ++it) {
        const int tile = t_begin + it;
        const int tw = tile % args.tiles_w;
        const int th = (tile / args.tiles_w) % args.tiles_h;
        const int tn = tile / (args.tiles_w * args.tiles_h);
        const int w0 = tw * args.box_w, h0 = th * args.box_h, n0 = tn * args.box_n;
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
          atomicCAS(args.status, kStatusOk, kStatusProducerTimeout);
          break;
        }
        const uint32_t a_dst = smem_base + stage * stage_bytes;
        const uint32_t b_dst = a_dst + a_bytes;
        mbar_expect_tx(full_bar(stage), uint32_t(a_bytes + ntaps * args.ci_blk64 * kWuBlockBytes));
#pragma unroll
        for (int j = 0; j < 2; ++j)
          tma_load_4d(a_dst + j * kWuBlockBytes, &tm_dy, full_bar(stage),
                      co_block * 128 + j * 64, w0, h0, n0);
        for (int t = 0; t < ntaps; ++t) {
          const int tap = tap0 + t;
          const int r = tap / args.taps_w, s = tap - r * args.taps_w;
          const int iw = w0 * args.stride_w + s * args.dil_w - args.pad_w;
          const int ih = h0 * args.stride_h + r * args.dil_h - args.pad_h;
          for (int j = 0; j < args.ci_blk64; ++j)
            tma_load_4d(b_dst + (t * args.ci_blk64 + j) * kWuBlockBytes, &tm_x, full_bar(stage),
                        ci_block * args.ci_blk + j * 64, iw, ih, n0);
        }
        if (++stage == stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      // all copies issued by this thread must have landed before the CTA exits
      for (int s = 0; s < stages; ++s) {
        const uint32_t last = (s < stage) ? phase : (phase ^ 1u);
        const long long start = clock64();
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
      const uint32_t idesc = make_idesc(128, uint32_t(args.ci_blk), 0, 0, true, true);
      int stage = 0;
      uint32_t phase = 0;
      for (int it = 0; it < k_iters; ++it) {
        if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
          atomicCAS(args.status, kStatusOk, kStatusMmaTimeout);
          break;
        }
        tc_fence_after_sync();
        const uint32_t a_addr = smem_base + stage * stage_bytes;
        const uint32_t b_addr = a_addr + a_bytes;
#pragma unroll
        for (int k = 0; k < kWuPixelsPerStage / 16; ++k) {
          // 16 pixels = 16 rows of 128 bytes
          const uint64_t a_desc = make_smem_desc(a_addr + k * 2048, kWuBlockBytes, 1024);
          for (int t = 0; t < ntaps; ++t) {
            const uint64_t b_desc = make_smem_desc(
                b_addr + t * args.ci_blk64 * kWuBlockBytes + k * 2048, kWuBlockBytes, 1024);
            umma_ss<false>(tmem_base + t * args.ci_blk, a_desc, b_desc, idesc,
                           (it | k) != 0 ? 1u : 0u);
          }
        }
        umma_commit(empty_bar(stage));
        if (++stage == stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      umma_commit(acc_bar);
      // also keeps the TMEM release below behind the last MMA
      const long long start = clock64();
      while (!mbar_try_wait(acc_bar, 0)) {
        if (clock64() - start > kWaitCycleLimit) {
          atomicCAS(args.status, kStatusOk, kStatusDrainTimeout);
          break;
        }
      }
    }
  } else {
    // ===================== epilogue (warps 2..5) =====================
    const int quarter = warp & 3;
    const int co = co_block * 128 + quarter * 32 + lane;
    if (mbar_wait(acc_bar, 0, abort_flag)) {
      tc_fence_after_sync();
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
      for (int t = 0; t < ntaps; ++t) {
        const int tap = tap0 + t;
        float *row = args.partial +
                     ((size_t(split) * taps + tap) * args.co_total + co) * size_t(args.ci_total) +
                     size_t(ci_block) * args.ci_blk;
        for (int c = 0; c < args.ci_blk; c += 32) {
          uint32_t v[32];
          __syncwarp();
          if (k_iters > 0) {
            // ci_blk is a multiple of 16: the last chunk may be half valid
            tmem_ld_32x32(t_addr + t * args.ci_blk + c, v);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0u;
          }
          if (co < args.co_total) {
            const int ci0 = ci_block * args.ci_blk + c;
            const int valid = min(min(32, args.ci_blk - c), args.ci_total - ci0);
            if (valid == 32 && (reinterpret_cast<uintptr_t>(row + c) & 15) == 0) {
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<float4 *>(row + c + j) =
                    make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (j < valid) row[c + j] = __uint_as_float(v[j]);
            }
          }
        }
      }
    } else {
      atomicCAS(args.status, kStatusOk, kStatusEpilogueTimeout);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, uint32_t(args.tmem_cols));
  }
}

// Adds the K splits in order and writes the fp32 sums and/or their cast.
__global__ void wu_reduce_kernel(const float *__restrict__ partial, int ksplit, size_t count,
                                 float *__restrict__ out_f32, void *__restrict__ out_cast,
                                 int cast_is_f32) {
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < count;
       i += size_t(gridDim.x) * blockDim.x) {
    float s = 0.f;
    for (int k = 0; k < ksplit; ++k) s += partial[size_t(k) * count + i];
    if (out_f32) out_f32[i] = s;
    if (out_cast) {
      if (cast_is_f32)
        static_cast<float *>(out_cast)[i] = s;
      else
        static_cast<__half *>(out_cast)[i] = __float2half_rn(s);
    }
  }
}

}  // namespace plb
