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
// channels.
//   warps 0..P-1  TMA producers.  One thread each; K step g is issued by
//                 producer g mod P (one 4-D box of the activations and one box
//                 of the weights per step, 128-byte swizzle, zero fill outside
//                 the tensor, which is what implements the padding).  Issuing a
//                 tensor copy costs a thread a few hundred cycles, so a single
//                 producer cannot keep the tensor core fed on narrow tiles.
//   warp 3        issues tcgen05.mma with fp32 accumulators in tensor memory.
//   warp 20       a second issuer for short tiles: issuing an MMA costs its
//                 thread about 28 cycles and every tile a few hundred more in
//                 barrier waits and commits, which on a tile of 16 instructions
//                 exceeds the 46 cycles the tensor core needs per instruction.
//                 The two issuers take alternate tiles (and so always the
//                 same accumulator each).
//   warps 4..19   epilogue, two groups of eight warps: drain a finished
//                 accumulator (tcgen05.ld), scale / add / cast, stage 32 rows
//                 x 128 bytes per pair of warps in shared memory and hand them
//                 to a TMA store (coalesced, clipped to the tensor by the
//                 hardware); plain vector stores are the fallback when the
//                 output cannot be described to TMA.  The per-warp chain
//                 load -> convert -> stage -> store is latency bound, so the
//                 epilogue's throughput comes from the number of warps.
// Two accumulators alternate so the epilogue of one tile overlaps the main loop
// of the next; accumulator g is always drained by epilogue group g, so a group
// has two tile periods for its tile.
#pragma once

#include "sm100_prims.cuh"

#ifndef PLB_IGEMM_PRODUCERS
#define PLB_IGEMM_PRODUCERS 3
#endif

namespace plb {

constexpr int kTileM = 128;        // pixels (rows) per tile = TMEM lanes
constexpr int kStageKBytes = 128;  // bytes of K per pipeline stage row (one swizzle span)
constexpr int kIgemmThreads = 672;
constexpr int kIgemmProducers = PLB_IGEMM_PRODUCERS;
constexpr int kIgemmMmaWarp = 3;
constexpr int kIgemmMmaWarp2 = 20;  // second MMA issuer (short tiles), after the 16 epilogue warps
constexpr int kEpiStagingBytes = 8 * 4096;  // 8 pairs of epilogue warps x (32 rows x 128 B)
static_assert(kIgemmProducers >= 1 && kIgemmProducers <= 3, "producer warps are warps 0..2");

struct IgemmArgs {
  // ---- M side: output pixels, tiled by a (w, h, n) box of 128 pixels ------
  int box_w, box_h, box_n;
  int tiles_w, tiles_h, tiles_n;
  int out_w, out_h, out_n;  // extents of the output (matrix product: rows, 1, 1)
  int h_outer;              // rows of a tile are ordered (w, n, h) instead of (w, h, n)
  // Halo mode: one stage holds a strip of box_h + (taps_h-1)*dil_h input rows and
  // serves all taps_h vertical taps (row r starts halo_step_bytes * r further on).
  int halo_step_bytes;
  int a_stage_bytes;        // bytes of activations per stage
  int b_tiles_per_stage;    // streamed weight tiles per stage (taps_h with a halo strip, else 1)
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
  // division by group_m * n_tiles, group_m, tiles_w and (h_outer ? tiles_n : tiles_h)
  FastDiv fd_band, fd_gm, fd_tw, fd_inner;
  int num_stages;  // pipeline depth (<= kIgemmMaxStages)
  // Split-K: split_k CTAs share one output tile, each taking a contiguous range
  // of the tile's pipeline steps and leaving raw fp32 sums in its own slice of
  // a scratch tensor (`out`, split_stride elements apart), which a second
  // kernel adds in split order before the scale / add / cast.  The role of the
  // reference's inChanSplit / kernelSplit partitions and the reduction that
  // follows them (lib/poplin/ConvPlan.hpp:28-77, lib/poplin/ConvReduce.cpp:316-362).
  int split_k;
  FastDiv fd_split;
  long long split_stride;
  int dual_issue;  // two MMA-issuing threads take alternate tiles
  uint32_t idesc_formats;  // operand format bits of the instruction descriptor (8-bit operands: 1 = E5M2)
  // ---- epilogue ---------------------------------------------------------------
  void *out;
  long long ldc;  // elements between consecutive output pixels (along w)
  long long out_stride_h, out_stride_n;  // elements between output rows / images
  const void *addend;
  long long ld_addend;
  const float *bias;
  float alpha, beta;
  int out_is_f32;
  int use_tma_store;        // tm_out is valid: stage through shared memory + TMA store
  int sub_w, sub_h;         // pixel box of one epilogue warp's 32 rows: (sub_w, sub_h, 32/(sub_w*sub_h))
  int *status;
  // Optional timeline (only written by builds with -DPLB_TRACE): CTA 0 stores
  // clock64() stamps, 4096 slots per role (producer 0, MMA issuer, epilogue).
  long long *trace;
};

#ifdef PLB_TRACE
#define PLB_TRACE_STAMP(role, slot)                                            \
  do {                                                                         \
    if (args.trace != nullptr && blockIdx.x == 0 && (slot) < 4096)             \
      args.trace[(role)*4096 + (slot)] = clock64();                            \
  } while (0)
#else
#define PLB_TRACE_STAMP(role, slot) do { } while (0)
#endif

constexpr int kIgemmMaxStages = 8;
constexpr int kIgemmBarrierBytes = 384;
constexpr int kIgemmSmemLimit = 227 * 1024;

// Shared memory: [stages][resident weights][epilogue staging][barriers], after
// up to 1023 bytes of alignment slack.  A stage holds the 128 x 128-byte
// activation tile and, unless the weights are resident, the BN x 128-byte
// weight tile of one K step.
// With a CTA pair (k2Cta) each CTA holds half of the weight tile's rows.
template <int BN, bool kResB, bool k2Cta = false>
struct IgemmSmem {
  static constexpr int kABytes = kTileM * kStageKBytes;  // without a halo
  static constexpr int kBBytes = (BN / (k2Cta ? 2 : 1)) * kStageKBytes;
  static constexpr int kFixedBytes = kEpiStagingBytes + kIgemmBarrierBytes + 1024;
  // b_tiles: streamed weight tiles per stage (1, or with a halo strip one per
  // vertical filter tap)
  __host__ __device__ static constexpr int stageBytes(int a_stage_bytes, int b_tiles) {
    return a_stage_bytes + (kResB ? 0 : b_tiles * kBBytes);
  }
  // deepest pipeline that fits beside `resident` bytes of weights
  static constexpr int stagesFor(int a_stage_bytes, int b_tiles, int resident) {
    const int n =
        (kIgemmSmemLimit - kFixedBytes - resident) / stageBytes(a_stage_bytes, b_tiles);
    return n > kIgemmMaxStages ? kIgemmMaxStages : n;
  }
  static constexpr int totalBytes(int a_stage_bytes, int b_tiles, int stages, int resident) {
    return stages * stageBytes(a_stage_bytes, b_tiles) + resident + kFixedBytes;
  }
};

// kFp8: operands are E4M3 bytes (kind::f8f6f4, 128 elements per stage row,
//       K = 32 per instruction); otherwise fp16 (64 per row, K = 16).
// kBMn: the B operand is stored K-by-N with N contiguous (a row-major right-hand
//       matrix); it is loaded as 64-column blocks and fed to the tensor core as
//       an MN-major operand.  fp16 only.
// kResB: weight-stationary.  All K steps' weight tiles are loaded once per CTA
//       and stay in shared memory; the pipeline then streams activations only.
//       Used when there is a single N tile and the weights fit (small filters
//       with few channels), where re-fetching them per pixel tile would cost
//       as much shared-memory fill bandwidth as the activations themselves.
// kHalo: one activation strip per (horizontal tap, channel chunk) feeds all
//       vertical taps: the strip of tap row r is the same shared memory shifted
//       by whole 8-row groups, which the descriptor's start address can express.
//       Cuts the activation traffic of a KxK filter K-fold.  Streamed weights
//       (no kResB) then travel as taps_h tiles per stage.
// k2Cta: the kernel is launched in clusters of two CTAs that share one
//       tcgen05.mma of 256 rows (cta_group::2): the CTA of rank r works on M
//       tile 2 * pair + r, loads its own activations and rows
//       [r * BN/2, (r+1) * BN/2) of the weight tile, and drains its own
//       accumulator.  Rank 0 issues the MMAs; its "full" barriers count the
//       bytes of both CTAs' copies, its "accumulator free" barriers the
//       epilogue threads of both, and its commits release the stages and
//       publish the accumulators in both CTAs.  Halving the weight rows per
//       CTA halves their shared-memory fill and operand fetch per FLOP, and
//       the instruction is twice as large, which matters because a
//       128-row instruction is bound by operand fetch, not by arithmetic.
template <int BN, bool kFp8, bool kBMn, bool kResB, bool kHalo, bool k2Cta>
__global__ void __launch_bounds__(kIgemmThreads, 1)
igemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
             const __grid_constant__ CUtensorMap tm_out, const IgemmArgs args) {
  using S = IgemmSmem<BN, kResB, k2Cta>;
  static_assert(!k2Cta || !kBMn || BN >= 128, "a CTA needs a whole 64-column block of MN-major B");
  const uint32_t cta_rank = k2Cta ? cluster_cta_rank() : 0u;
  const bool leader = cta_rank == 0;
  constexpr int kMaxStages = kIgemmMaxStages;
  const int kStages = args.num_stages;
  constexpr int P = kIgemmProducers;
  constexpr uint32_t kTmemCols = 2 * BN;  // two accumulators
  static_assert(kTmemCols >= 32 && kTmemCols <= 512 && (kTmemCols & (kTmemCols - 1)) == 0, "");
  static_assert(!(kFp8 && kBMn), "MN-major B is implemented for fp16 only");

  extern __shared__ uint8_t smem_raw[];
  if (threadIdx.x == 0) PLB_TRACE_STAMP(2, 4000);
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  // K steps: every (r, s, kc); pipeline steps: in halo mode one per (s, kc)
  const int k_iters = args.taps_h * args.taps_w * args.k_chunks;
  const int p_iters = kHalo ? args.taps_w * args.k_chunks : k_iters;
  const int stage_bytes = S::stageBytes(args.a_stage_bytes, args.b_tiles_per_stage);
  const uint32_t resb_base = smem_base + kStages * stage_bytes;
  const uint32_t staging_base = resb_base + (kResB ? k_iters * S::kBBytes : 0);
  const uint32_t bar_base = staging_base + kEpiStagingBytes;
  // barrier words: full[8], empty[8], tmem_full[2], tmem_empty[2], drain, resident-B
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kMaxStages + s); };
  auto tmem_full_bar = [&](int a) { return bar_base + 8u * (2 * kMaxStages + a); };
  auto tmem_empty_bar = [&](int a) { return bar_base + 8u * (2 * kMaxStages + 2 + a); };
  const uint32_t drain_bar = bar_base + 8u * (2 * kMaxStages + 4);
  const uint32_t drain_bar2 = bar_base + 8u * (2 * kMaxStages + 8);
  const uint32_t resb_bar = bar_base + 8u * (2 * kMaxStages + 5);
  const uint32_t tmem_slot = bar_base + 8u * (2 * kMaxStages + 6);
  uint8_t *bar_gen = smem_raw + (bar_base - smem_u32(smem_raw));
  volatile uint32_t *tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t *>(bar_gen + 8 * (2 * kMaxStages + 6));
  volatile int *abort_flag = reinterpret_cast<volatile int *>(bar_gen + 8 * (2 * kMaxStages + 7));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // Set-up is spread over the warps: the lanes of warp 0 initialise the barrier
  // words (one each), a thread of warp 1 asks for the tensor maps, warp 3
  // allocates tensor memory.
  if (warp == 0) {
    // barrier slots: full[8], empty[8], tmem_full[2], tmem_empty[2], drain, resident-B;
    // slot 24: the second issuer's drain
    if (lane == 22) mbar_init(bar_base + 8u * (2 * kMaxStages + 8), 1u);
    if (lane < 2 * kMaxStages + 6) {
      // tmem_empty counts a group's epilogue threads (of both CTAs of a pair)
      const bool acc_free = lane == 2 * kMaxStages + 2 || lane == 2 * kMaxStages + 3;
      mbar_init(bar_base + 8u * lane, acc_free ? (k2Cta ? 512u : 256u) : 1u);
    }
    if (lane == 0) *abort_flag = 0;
    mbar_fence_init();
    if (lane == 0) PLB_TRACE_STAMP(2, 4010);
  } else if (threadIdx.x == 32) {
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
    if (args.use_tma_store) tma_prefetch_desc(&tm_out);
  }
  if (warp == kIgemmMmaWarp) {
    if constexpr (k2Cta) {
      tmem_alloc_pair(tmem_slot, kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, kTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0) PLB_TRACE_STAMP(2, 4011);
  // the other CTA's copies and arrivals must find initialised barriers
  // (published by fence.mbarrier_init above)
  if constexpr (k2Cta) cluster_sync_relaxed();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_ptr;
  // Everything above touched only this SM (barriers, tensor memory): with a
  // programmatic launch it overlaps the tail of the previous kernel in the
  // stream.  Each role goes on preparing what it can without reading or writing
  // global memory (tile coordinates, descriptors, L2 prefetches of the first
  // operands, which have no architectural effect) and calls pdl_wait() itself
  // right before its first access.
  if (threadIdx.x == 0) PLB_TRACE_STAMP(2, 4001);
  pdl_launch_dependents();

  // Work units: output tiles, or with a CTA pair, pairs of M tiles (the odd
  // last one is padded: its copies read zeros and its stores are clipped).
  const int m_tiles = args.tiles_w * args.tiles_h * args.tiles_n;
  const int m_units = k2Cta ? (m_tiles + 1) / 2 : m_tiles;
  const int total_tiles = m_units * args.n_tiles;
  // a unit of work is an output tile, or with split-K one of its K ranges
  // (the splits of a tile are consecutive units, i.e. run on different CTAs)
  const int total_units = total_tiles * args.split_k;
  const int first_unit = k2Cta ? int(blockIdx.x >> 1) : int(blockIdx.x);
  const int unit_stride = k2Cta ? int(gridDim.x >> 1) : int(gridDim.x);
  // barriers of the CTA that issues the MMAs, as cluster addresses
  auto lead_bar = [&](uint32_t bar) { return k2Cta ? map_to_cta(bar, 0) : bar; };
  constexpr int kElemsPerStage = kFp8 ? 128 : 64;

  // Tile coordinates are needed once per tile by every producer and epilogue
  // thread; a chain of hardware integer divisions there costs more than a
  // thousand cycles per tile (measured: it paced the producers of short tiles).
  // The divisors are fixed for the launch: divide by multiplication instead.
  // (the multipliers come with the launch arguments: computing them here would
  // put four 64-bit divisions into every thread's prologue)
  const FastDiv fd_band = args.fd_band, fd_gm = args.fd_gm, fd_tw = args.fd_tw, fd_inner = args.fd_inner;

  // unit -> (tile, range [it_begin, it_end) of the tile's pipeline steps)
  auto unit_coords = [&](int unit, int &tile, int &split, int &it_begin, int &it_end) {
    if (args.split_k == 1) {
      tile = unit;
      split = 0;
      it_begin = 0;
      it_end = p_iters;
    } else {
      tile = int(fast_div(uint32_t(unit), args.fd_split));
      split = unit - tile * args.split_k;
      it_begin = int(fast_div(uint32_t(p_iters * split), args.fd_split));
      it_end = int(fast_div(uint32_t(p_iters * (split + 1)), args.fd_split));
    }
  };
  // tile index -> (m tile, n tile): bands of group_m M tiles, M fastest inside a band
  auto tile_coords = [&](int tile, int &m_idx, int &n_idx) {
    const int band_tiles = args.group_m * args.n_tiles;
    const int band = int(fast_div(uint32_t(tile), fd_band));
    const int within = tile - band * band_tiles;
    const int m0 = band * args.group_m;
    const int gm = min(args.group_m, m_units - m0);
    // (only the last band can be narrower)
    const int q = gm == args.group_m ? int(fast_div(uint32_t(within), fd_gm)) : within / gm;
    m_idx = m0 + within - q * gm;
    n_idx = q;
    if constexpr (k2Cta) m_idx = 2 * m_idx + int(cta_rank);
  };

  // M tile index -> first pixel of the tile; tile row -> pixel inside the tile
  auto tile_origin = [&](int m_idx, int &w0, int &h0, int &n0) {
    const int rest = int(fast_div(uint32_t(m_idx), fd_tw));
    const int tw = m_idx - rest * args.tiles_w;
    const int outer = int(fast_div(uint32_t(rest), fd_inner));
    const int inner = rest - outer * (args.h_outer ? args.tiles_n : args.tiles_h);
    int th, tn;
    if (args.h_outer) {
      tn = inner;
      th = outer;
    } else {
      th = inner;
      tn = outer;
    }
    w0 = tw * args.box_w;
    h0 = th * args.box_h;
    n0 = tn * args.box_n;
  };
  auto row_pixel = [&](int row, int &rw, int &rh, int &rn) {
    rw = row % args.box_w;
    const int rest = row / args.box_w;
    if (args.h_outer) {
      rn = rest % args.box_n;
      rh = rest / args.box_n;
    } else {
      rh = rest % args.box_h;
      rn = rest / args.box_h;
    }
  };

  // B tile of K step (r, s, kc) -> shared memory at `dst`; with kPrefetch the
  // same box is only pulled towards L2
  auto load_b = [&](uint32_t dst, uint32_t bar, int r, int s, int kc, int n_col, bool prefetch) {
    const int b_tap = (args.flip_h ? args.taps_h - 1 - r : r) * args.taps_w +
                      (args.flip_w ? args.taps_w - 1 - s : s);
    // a CTA of a pair loads its half of the tile's N rows / columns
    constexpr int kMyN = k2Cta ? BN / 2 : BN;
    const int my_col = n_col + int(cta_rank) * kMyN;
    if constexpr (kBMn) {
      // K rows x 64 columns per block; blocks of 64 columns are 64 rows apart
#pragma unroll
      for (int j = 0; j < kMyN / 64; ++j) {
        if (prefetch)
          tma_prefetch_l2_3d(&tm_b, my_col + j * 64, kc * 64, b_tap);
        else if constexpr (k2Cta)
          tma_load_3d_pair(dst + j * (64 * kStageKBytes), &tm_b, bar, my_col + j * 64, kc * 64,
                           b_tap);
        else
          tma_load_3d(dst + j * (64 * kStageKBytes), &tm_b, bar, my_col + j * 64, kc * 64, b_tap);
      }
    } else {
      if (prefetch)
        tma_prefetch_l2_3d(&tm_b, kc * kElemsPerStage, my_col, b_tap);
      else if constexpr (k2Cta)
        tma_load_3d_pair(dst, &tm_b, bar, kc * kElemsPerStage, my_col, b_tap);
      else
        tma_load_3d(dst, &tm_b, bar, kc * kElemsPerStage, my_col, b_tap);
    }
  };
  // pipeline step index inside a tile -> (filter row, filter column, channel chunk)
  auto step_coords = [&](int it, int &r, int &s, int &kc) {
    kc = it % args.k_chunks;
    const int t = it / args.k_chunks;
    s = t % args.taps_w;
    r = t / args.taps_w;
  };
  // the barriers that count copied bytes are those of the MMA-issuing CTA,
  // which alone announces the byte count (both CTAs' shares)
  constexpr uint32_t kPairFactor = k2Cta ? 2u : 1u;

  if (warp < P) {
    // ===================== TMA producers =====================
    if (elect_one()) {
      const int me = warp;
      int stage = me;          // stage of this producer's next K step
      uint32_t phase = 0;
      int turn = 0;            // (global K step) mod P
      bool ok = true;
      [[maybe_unused]] int trace_slot = 0;
      // One pipeline step: the activation box and, unless the weights are
      // resident, the weight tile(s) of step (r, s, kc) -> stage memory at a_dst
      // (or, before the predecessor kernel is known to have finished, only
      // towards L2).
      auto issue_step = [&](bool prefetch, uint32_t a_dst, uint32_t full, int r, int s, int kc,
                            int w_base, int h_base, int n0, int n_col) {
        const int cw = w_base + s * args.dil_w, ch = h_base + r * args.dil_h;
        const int c2 = args.h_outer ? n0 : ch, c3 = args.h_outer ? ch : n0;
        if (prefetch)
          tma_prefetch_l2_4d(&tm_a, kc * kElemsPerStage, cw, c2, c3);
        else if constexpr (k2Cta)
          tma_load_4d_pair(a_dst, &tm_a, full, kc * kElemsPerStage, cw, c2, c3);
        else
          tma_load_4d(a_dst, &tm_a, full, kc * kElemsPerStage, cw, c2, c3);
        if constexpr (!kResB) {
          // with a halo strip the stage carries the weight tiles of every filter row
          const int row_taps = kHalo ? args.taps_h : 1;
          for (int rr = 0; rr < row_taps; ++rr)
            load_b(a_dst + args.a_stage_bytes + rr * S::kBBytes, full, kHalo ? rr : r, s, kc, n_col,
                   prefetch);
        }
      };
      // While the predecessor kernel may still be running: pull the boxes of
      // this producer's first steps towards L2.
      if (first_unit < total_units) {
        int tile, split, it_begin, it_end;
        unit_coords(first_unit, tile, split, it_begin, it_end);
        int m_idx, n_idx;
        tile_coords(tile, m_idx, n_idx);
        int w0, h0, n0;
        tile_origin(m_idx, w0, h0, n0);
        const int steps = min(it_end, it_begin + kStages);
        for (int it = it_begin + me; it < steps; it += P) {
          int r, s, kc;
          step_coords(it, r, s, kc);
          issue_step(true, 0u, 0u, r, s, kc, w0 * args.stride_w - args.pad_w,
                     h0 * args.stride_h - args.pad_h, n0, n_idx * BN);
        }
      }
      pdl_wait();
      if (me == 0) PLB_TRACE_STAMP(2, 4002);
      for (int unit = first_unit; unit < total_units && ok; unit += unit_stride) {
        if (me == 0) { PLB_TRACE_STAMP(0, trace_slot); ++trace_slot; }
        int tile, split, it_begin, it_end;
        unit_coords(unit, tile, split, it_begin, it_end);
        int m_idx, n_idx;
        tile_coords(tile, m_idx, n_idx);
        int w0, h0, n0;
        tile_origin(m_idx, w0, h0, n0);
        if (me == 0) { PLB_TRACE_STAMP(0, trace_slot); ++trace_slot; }
        const int w_base = w0 * args.stride_w - args.pad_w;
        const int h_base = h0 * args.stride_h - args.pad_h;
        const int n_col = n_idx * BN;
        int r = 0, s = 0, kc = 0;
        if (it_begin != 0) step_coords(it_begin, r, s, kc);
        for (int it = it_begin; it < it_end; ++it) {
          if (turn == me) {
            if (me == 0) { PLB_TRACE_STAMP(0, trace_slot); ++trace_slot; }
            if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
              atomicCAS(args.status, kStatusOk, kStatusProducerTimeout);
              ok = false;
              break;
            }
            if (me == 0) { PLB_TRACE_STAMP(0, trace_slot); ++trace_slot; }
            const uint32_t a_dst = smem_base + stage * stage_bytes;
            if (leader) mbar_expect_tx(full_bar(stage), kPairFactor * uint32_t(stage_bytes));
            const uint32_t full = lead_bar(full_bar(stage));
            issue_step(false, a_dst, full, r, s, kc, w_base, h_base, n0, n_col);
            if (me == 0) { PLB_TRACE_STAMP(0, trace_slot); ++trace_slot; }
            stage += P;
            if (stage >= kStages) {
              stage -= kStages;
              phase ^= 1u;
            }
          }
          if (++turn == P) turn = 0;
          // next pipeline step: kc fastest, then s, then (without a halo) r
          if (++kc == args.k_chunks) {
            kc = 0;
            if (++s == args.taps_w) {
              s = 0;
              ++r;
            }
          }
        }
      }
      if (me == 0) PLB_TRACE_STAMP(2, 4014);
    }
  } else if (warp == kIgemmMmaWarp || warp == kIgemmMmaWarp2) {
    // ===================== MMA issuer(s) =====================
    // (with a CTA pair only the CTA of rank 0 issues)
    const int mi = warp == kIgemmMmaWarp ? 0 : 1;
    const int n_issuers = args.dual_issue ? 2 : 1;
    if (mi < n_issuers && leader && elect_one()) {
      const uint32_t idesc =
          make_idesc(k2Cta ? 2 * kTileM : kTileM, BN, 0, 0, false, kBMn) | args.idesc_formats;
      // completion of the MMAs issued so far -> barrier (in both CTAs of a pair)
      auto commit = [&](uint32_t bar) {
        if constexpr (k2Cta)
          umma_commit_pair(bar, uint16_t(3));
        else
          umma_commit(bar);
      };
      const uint64_t a_desc0 = make_smem_desc(smem_base, 16, 1024);
      // B tiles: resident ones start at resb_base, streamed ones follow the
      // activations inside their stage
      const uint64_t b_desc0 =
          kBMn ? make_smem_desc(kResB ? resb_base : smem_base + uint32_t(args.a_stage_bytes),
                                64 * kStageKBytes, 1024)
               : make_smem_desc(kResB ? resb_base : smem_base + uint32_t(args.a_stage_bytes), 16,
                                1024);
      [[maybe_unused]] const uint64_t halo_step16 = uint64_t(uint32_t(args.halo_step_bytes) >> 4);
      // weight tile of the next filter row: resident tiles are indexed (r, s, kc),
      // streamed ones follow one another inside the stage
      [[maybe_unused]] const uint64_t b_row_step16 =
          uint64_t(uint32_t(kResB ? args.taps_w * args.k_chunks : 1) * (S::kBBytes >> 4));
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase[2] = {0, 0};
      int local_tile = 0;
      bool ok = true;
      [[maybe_unused]] int trace_slot = 0;
      if (kResB && first_unit < total_units) {
        if (!mbar_wait(resb_bar, 0, abort_flag)) {
          atomicCAS(args.status, kStatusOk, kStatusMmaTimeout);
          ok = false;
        }
      }
      for (int unit = first_unit; unit < total_units && ok; unit += unit_stride, ++local_tile) {
        int tile, split, it_begin, it_end;
        unit_coords(unit, tile, split, it_begin, it_end);
        if (n_issuers == 2 && (local_tile & 1) != mi) {
          // the other issuer's tile: step over its pipeline stages
          stage += it_end - it_begin;
          while (stage >= kStages) {
            stage -= kStages;
            phase ^= 1u;
          }
          continue;
        }
        const int acc = local_tile & 1;
        if (mi == 0) { PLB_TRACE_STAMP(1, trace_slot); ++trace_slot; }
        // wait for the epilogue to have drained this accumulator
        if (!mbar_wait(tmem_empty_bar(acc), acc_phase[acc] ^ 1u, abort_flag)) {
          atomicCAS(args.status, kStatusOk, kStatusMmaTimeout);
          ok = false;
          break;
        }
        acc_phase[acc] ^= 1u;
        tc_fence_after_sync();
        if (mi == 0) { PLB_TRACE_STAMP(1, trace_slot); ++trace_slot; }
        const uint32_t d_tmem = tmem_base + acc * BN;
        int s_tap = 0, kc = 0;  // halo mode: pipeline step = (s_tap, kc), kc fastest
        if (kHalo && it_begin != 0) {
          kc = it_begin % args.k_chunks;
          s_tap = it_begin / args.k_chunks;
        }
        for (int it = it_begin; it < it_end; ++it) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
            atomicCAS(args.status, kStatusOk, kStatusMmaTimeout);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          if (mi == 0) { PLB_TRACE_STAMP(1, trace_slot); ++trace_slot; }
          // Descriptors are advanced by adding to their start-address field
          // (16-byte units, cannot overflow for shared-memory addresses): the
          // issuing thread's own instruction count bounds the MMA rate on
          // narrow tiles.
          const uint32_t stage_off16 = uint32_t(stage * stage_bytes) >> 4;
          uint64_t a_desc = a_desc0 + stage_off16;
          uint64_t b_desc;
          if constexpr (kHalo && kResB)
            b_desc = b_desc0 + uint64_t((s_tap * args.k_chunks + kc) * (S::kBBytes >> 4));
          else if constexpr (kResB)
            b_desc = b_desc0 + uint64_t(it * (S::kBBytes >> 4));
          else
            b_desc = b_desc0 + stage_off16;
          const int row_taps = kHalo ? args.taps_h : 1;
          for (int r = 0; r < row_taps; ++r) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              // one instruction consumes 32 bytes of K: advance the start address
              // inside the swizzle span (K-major) or by 16 rows (MN-major B)
              const uint64_t a_k = a_desc + uint64_t(k * 2);
              const uint64_t b_k =
                  b_desc + uint64_t(kBMn ? k * ((16 * kStageKBytes) >> 4) : k * 2);
              if constexpr (k2Cta)
                umma_ss_pair<kFp8>(d_tmem, a_k, b_k, idesc, ((it - it_begin) | r | k) != 0 ? 1u : 0u);
              else
                umma_ss<kFp8>(d_tmem, a_k, b_k, idesc, ((it - it_begin) | r | k) != 0 ? 1u : 0u);
            }
            if constexpr (kHalo) {
              // next filter row: the strip shifted by whole 8-row groups; its
              // resident weight tile is taps_w * k_chunks tiles further on
              a_desc += halo_step16;
              b_desc += b_row_step16;
            }
          }
          commit(empty_bar(stage));  // frees the stage when these MMAs retire
          if (mi == 0) { PLB_TRACE_STAMP(1, trace_slot); ++trace_slot; }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
          if (++kc == args.k_chunks) {
            kc = 0;
            ++s_tap;
          }
        }
        if (ok) commit(tmem_full_bar(acc));
      }
      // make sure nothing is still executing before TMEM is released
      const uint32_t my_drain = mi == 0 ? drain_bar : drain_bar2;
      if constexpr (k2Cta)
        umma_commit_pair(my_drain, uint16_t(1));
      else
        umma_commit(my_drain);
      const long long start = clock64();
      while (!mbar_try_wait(my_drain, 0)) {
        if (clock64() - start > kWaitCycleLimit) {
          atomicCAS(args.status, kStatusOk, kStatusDrainTimeout);
          break;
        }
      }
      if (mi == 0) PLB_TRACE_STAMP(2, 4015);
    }
  } else if (warp >= 4 && warp < 20) {
    // ===================== epilogue (warps 4..19) =====================
    // Accumulator g is drained by the eight warps of group g.  A warp can read
    // the 32 TMEM lanes (tile rows) [32*(warp%4), +32); the two warps that share
    // a lane quarter split every block of 64 columns between them (columns
    // [0,32) and [32,64) of the block) and stage their halves of the same
    // 32-row x 128-byte buffer, which one of them then hands to a tensor store.
    // The two synchronise through two mbarriers (bounded waits, like every wait
    // in this kernel): "buffer free" before writing, "buffer staged" before the
    // store; the storing role alternates so that both wait for their own stores
    // in turn.
    const int group = (warp - 4) >> 3;       // drains accumulator `group`
    const int half = ((warp - 4) >> 2) & 1;  // which 32 columns of each 64-column block
    const int quarter = warp & 3;            // TMEM lanes [32*quarter, 32*quarter+32)
    const int row = quarter * 32 + lane;     // tile row handled by this thread
    uint32_t acc_phase = 0;
    int rw, rh, rn;
    row_pixel(row, rw, rh, rn);
    // origin of this warp's 32 rows inside the tile's pixel box
    int qw, qh, qn;
    row_pixel(quarter * 32, qw, qh, qn);
    // fp32 output: one 32-row x 128-byte staging buffer per lane quarter of a
    // group (a second one was measured: it costs a pipeline stage and hides
    // nothing, the chain below is bound by its own instructions, not by the
    // store reading the buffer)
    const uint32_t buf = staging_base + uint32_t(group * 4 + quarter) * 4096u;
    const uint32_t row_addr = buf + uint32_t(lane) * 128u;
    const bool tma_store = args.use_tma_store != 0;
    const bool out_f32 = args.out_is_f32 != 0;
    // fp32 rows fill the 128-byte staged row with 32 columns: the `half == 1`
    // warps then leave the work to their partners
    const bool idle = tma_store && out_f32 && half == 1;
    const bool stamp = threadIdx.x == 128;
    const int acc = group;
    int local_tile = group;
    const uint32_t acc_free_bar = lead_bar(tmem_empty_bar(acc));
    if constexpr (kResB) {
      // Resident weights: a single N tile, so every tile of this CTA uses the
      // same weights.  The epilogue warps have nothing to do until the first
      // accumulator is complete, so one lane of each issues a share of the
      // copies (a copy costs its issuing thread some hundred cycles, and the
      // first MMA waits for all of them), leaving the producers free to start
      // on the activations at once.
      if (lane == 0 && first_unit < total_units) {
        for (int it = warp - 4; it < k_iters; it += 16) {
          int r, s, kc;
          step_coords(it, r, s, kc);
          load_b(0u, 0u, r, s, kc, 0, true);
        }
        pdl_wait();
        if (warp == 4 && leader)
          mbar_expect_tx(resb_bar, kPairFactor * uint32_t(k_iters) * S::kBBytes);
        const uint32_t resb_bar_lead = lead_bar(resb_bar);
        for (int it = warp - 4; it < k_iters; it += 16) {
          int r, s, kc;
          step_coords(it, r, s, kc);
          load_b(resb_base + it * S::kBBytes, resb_bar_lead, r, s, kc, 0, false);
        }
        if (warp == 4) PLB_TRACE_STAMP(2, 4012);
      }
      __syncwarp();
    }
    pdl_wait();
    for (int unit = first_unit + group * unit_stride; unit < total_units;
         unit += 2 * unit_stride, local_tile += 2) {
      int tile, split, it_begin, it_end;
      unit_coords(unit, tile, split, it_begin, it_end);
      int m_idx, n_idx;
      tile_coords(tile, m_idx, n_idx);
      int w0, h0, n0;
      tile_origin(m_idx, w0, h0, n0);
      const int ow = w0 + rw, oh = h0 + rh, on = n0 + rn;
      const bool row_ok = ow < args.out_w && oh < args.out_h && on < args.out_n;
      // element offset of this row's output pixel; the addend is dense in pixels
      const long long pixel = (static_cast<long long>(on) * args.out_h + oh) * args.out_w + ow;
      const long long out_off = static_cast<long long>(on) * args.out_stride_n +
                                static_cast<long long>(oh) * args.out_stride_h +
                                static_cast<long long>(ow) * args.ldc;
      if (stamp) PLB_TRACE_STAMP(2, local_tile * 4 + 0);
      if (!mbar_wait(tmem_full_bar(acc), acc_phase, abort_flag)) {
        atomicCAS(args.status, kStatusOk, kStatusEpilogueTimeout);
        break;
      }
      acc_phase ^= 1u;
      tc_fence_after_sync();
      if (stamp) PLB_TRACE_STAMP(2, local_tile * 4 + 1);
      const uint32_t t_addr = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
      const int col_base = n_idx * BN;
      const bool box_ok = w0 + qw < args.out_w && h0 + qh < args.out_h && n0 + qn < args.out_n;
      auto release_accumulator = [&]() {
        tc_fence_before_sync();
        if constexpr (k2Cta)
          mbar_arrive_cluster(acc_free_bar);
        else
          mbar_arrive(acc_free_bar);
      };
      if (idle) {
        release_accumulator();
        continue;
      }

      // 32 accumulator columns [c, c + 32) of this thread's row: scale / add / cast
      auto finish = [&](const uint32_t (&v)[32], float (&f)[32], const int c) {
        const int col0 = col_base + c;
        const int valid = min(32, args.n_total - col0);  // may be <= 0 on a padded N tile
        if (args.alpha != 1.f) {
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]) * args.alpha;
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
        }
        if (args.bias != nullptr) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j < valid) f[j] += args.bias[col0 + j];
        }
        if (args.addend != nullptr && row_ok) {
          if (out_f32) {
            const float *src = static_cast<const float *>(args.addend) + pixel * args.ld_addend + col0;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < valid) f[j] += args.beta * src[j];
          } else {
            const __half *src = static_cast<const __half *>(args.addend) + pixel * args.ld_addend + col0;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < valid) f[j] += args.beta * __half2float(src[j]);
          }
        }
      };
      // plain vector stores of 32 finished columns (output not describable to TMA)
      auto store_direct = [&](const float (&f)[32], const int c) {
        const int col0 = col_base + c;
        const int valid = min(32, args.n_total - col0);
        if (!row_ok || valid <= 0) return;
        if (out_f32) {
          // (with split-K: this split's slice of the partial sums)
          float *dst = static_cast<float *>(args.out) + split * args.split_stride + out_off + col0;
          if (valid == 32 && (reinterpret_cast<uintptr_t>(dst) & 31) == 0) {
            // whole 32-byte sectors per lane
#pragma unroll
            for (int j = 0; j < 32; j += 8)
              st_global_v8(dst + j, __float_as_uint(f[j]), __float_as_uint(f[j + 1]),
                           __float_as_uint(f[j + 2]), __float_as_uint(f[j + 3]),
                           __float_as_uint(f[j + 4]), __float_as_uint(f[j + 5]),
                           __float_as_uint(f[j + 6]), __float_as_uint(f[j + 7]));
          } else if (valid == 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              *reinterpret_cast<float4 *>(dst + j) = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < valid) dst[j] = f[j];
          }
        } else {
          __half *dst = static_cast<__half *>(args.out) + out_off + col0;
          if (valid == 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
            uint32_t pk[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              __half2 h = __floats2half2_rn(f[2 * j], f[2 * j + 1]);
              pk[j] = *reinterpret_cast<uint32_t *>(&h);
            }
            if ((reinterpret_cast<uintptr_t>(dst) & 31) == 0) {
              st_global_v8(dst, pk[0], pk[1], pk[2], pk[3], pk[4], pk[5], pk[6], pk[7]);
              st_global_v8(dst + 16, pk[8], pk[9], pk[10], pk[11], pk[12], pk[13], pk[14], pk[15]);
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j)
                *reinterpret_cast<uint4 *>(dst + 8 * j) =
                    make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < valid) dst[j] = __float2half_rn(f[j]);
          }
        }
      };
      // issue (lane 0) the tensor store of the staged buffer: columns [store_col, +128 bytes)
      auto store_staged = [&](const uint32_t buf, const int store_col) {
        if (lane == 0) {
          // a box that starts outside the tensor has nothing to write
          if (store_col < args.n_total && box_ok) {
            if (args.h_outer)
              tma_store_4d(&tm_out, buf, store_col, w0 + qw, n0 + qn, h0 + qh);
            else
              tma_store_4d(&tm_out, buf, store_col, w0 + qw, h0 + qh, n0 + qn);
          }
          tma_store_commit();
        }
      };

      uint32_t v[32];
      float f[32];
      if (!tma_store) {
        // each warp stores its own 32 columns of every 64-column block
#pragma unroll 1
        for (int c = half * 32; c < BN; c += 64) {
          __syncwarp();
          tmem_ld_32x32(t_addr + c, v);
          tmem_ld_wait_for(v);
          if (c + 64 >= BN) release_accumulator();
          finish(v, f, c);
          store_direct(f, c);
        }
      } else if (out_f32) {
        // (half == 0 warps only) one 32-column chunk per staged buffer and store
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          __syncwarp();
          tmem_ld_32x32(t_addr + c, v);
          tmem_ld_wait_for(v);
          if (c + 32 >= BN) release_accumulator();
          finish(v, f, c);
          if (lane == 0) tma_store_wait_read<0>();  // the previous store has read the buffer
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 8; ++j)
            st_shared_v4(row_addr + (uint32_t(j ^ (lane & 7)) << 4), __float_as_uint(f[4 * j]),
                         __float_as_uint(f[4 * j + 1]), __float_as_uint(f[4 * j + 2]),
                         __float_as_uint(f[4 * j + 3]));
          fence_proxy_async_smem();
          __syncwarp();
          store_staged(buf, col_base + c);
        }
      } else {
        // half output: each warp stages its own 32 rows x 32 columns (64-byte
        // rows; 16-byte pieces XOR-swizzled with bits 1-2 of the row index, the
        // tensor map's 64-byte swizzle, which also keeps the stores free of bank
        // conflicts) and hands them to a tensor store of its own, so no barrier
        // between warps lies on the chain load -> convert -> stage -> store.
        const uint32_t wbuf = staging_base + uint32_t(warp - 4) * 2048u;
        const uint32_t wrow = wbuf + uint32_t(lane) * 64u;
        const uint32_t sw = (uint32_t(lane) >> 1) & 3u;
#pragma unroll 1
        for (int c = half * 32; c < BN; c += 64) {
          __syncwarp();
          tmem_ld_32x32(t_addr + c, v);
          tmem_ld_wait_for(v);
          if (c + 64 >= BN) release_accumulator();
          finish(v, f, c);
          if (lane == 0) tma_store_wait_read<0>();  // this warp's previous store has read the buffer
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            __half2 h0 = __floats2half2_rn(f[8 * j], f[8 * j + 1]);
            __half2 h1 = __floats2half2_rn(f[8 * j + 2], f[8 * j + 3]);
            __half2 h2 = __floats2half2_rn(f[8 * j + 4], f[8 * j + 5]);
            __half2 h3 = __floats2half2_rn(f[8 * j + 6], f[8 * j + 7]);
            st_shared_v4(wrow + ((uint32_t(j) ^ sw) << 4), *reinterpret_cast<uint32_t *>(&h0),
                         *reinterpret_cast<uint32_t *>(&h1), *reinterpret_cast<uint32_t *>(&h2),
                         *reinterpret_cast<uint32_t *>(&h3));
          }
          fence_proxy_async_smem();
          __syncwarp();
          store_staged(wbuf, col_base + c);
        }
      }
      if (stamp) PLB_TRACE_STAMP(2, local_tile * 4 + 2);
      if (stamp) PLB_TRACE_STAMP(2, local_tile * 4 + 3);
    }
    // this thread's stores must have read their staging buffers before the CTA
    // gives up its shared memory (the writes themselves complete with the grid)
    if (tma_store && lane == 0) tma_store_wait_read<0>();
    if (stamp) PLB_TRACE_STAMP(2, 4016);
  }

  if (threadIdx.x == 0) PLB_TRACE_STAMP(2, 4003);
  tc_fence_before_sync();
  // Every tensor copy must have landed before the CTA gives up its shared
  // memory.  In a run without errors the MMA issuer has waited for every
  // stage it consumed, i.e. for all of them; only after an aborted wait can
  // copies still be in flight, and then they are waited for here (bounded).
  // Stage s was last filled by pipeline step g = the largest g < total with
  // g mod kStages == s, in phase (g / kStages) & 1.  With a CTA pair the
  // barriers live in the MMA-issuing CTA, which waits for both CTAs' copies;
  // the other CTA cannot leave before the rendezvous below.
  __syncthreads();
  if (*abort_flag != 0 && threadIdx.x == 0 && leader) {
    int my_tiles = 0;
    long long total_steps = 0;
    for (int unit = first_unit; unit < total_units; unit += unit_stride, ++my_tiles) {
      int tile, split, it_begin, it_end;
      unit_coords(unit, tile, split, it_begin, it_end);
      total_steps += it_end - it_begin;
    }
    const long long start = clock64();
    auto drain = [&](uint32_t bar, uint32_t parity) {
      while (!mbar_try_wait(bar, parity)) {
        if (clock64() - start > kWaitCycleLimit) {
          atomicCAS(args.status, kStatusOk, kStatusDrainTimeout);
          break;
        }
      }
    };
    if (kResB && my_tiles > 0) drain(resb_bar, 0);
    for (int st = 0; st < kStages; ++st) {
      if (total_steps <= st) continue;
      const long long g = st + ((total_steps - 1 - st) / kStages) * kStages;
      drain(full_bar(st), uint32_t((g / kStages) & 1));
    }
  }
  // Neither CTA of a pair may go away while the other can still touch its
  // barriers, shared memory or tensor memory: the rendezvous of all threads of
  // the cluster (which is also this CTA's own barrier) orders that.
  if constexpr (k2Cta)
    cluster_sync_relaxed();
  else
    __syncthreads();
  if (threadIdx.x == 0) PLB_TRACE_STAMP(2, 4004);
  if (warp == kIgemmMmaWarp) {
    tc_fence_after_sync();
    if constexpr (k2Cta)
      tmem_dealloc_pair(tmem_base, kTmemCols);
    else
      tmem_dealloc(tmem_base, kTmemCols);
  }
#ifdef PLB_TRACE
  if (threadIdx.x == 0) {
    PLB_TRACE_STAMP(2, 4005);
    uint32_t smid;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
    if (args.trace != nullptr && blockIdx.x == 0) args.trace[2 * 4096 + 4006] = smid;
  }
#endif
}

}  // namespace plb
