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
//   warps 4..11   epilogue, two groups of four warps: drain a finished
//                 accumulator (tcgen05.ld, the next 32 columns in flight while
//                 the current ones are processed), scale / add / cast, stage
//                 32 rows x 128 bytes per warp in shared memory and hand them
//                 to a TMA store (coalesced, clipped to the tensor by the
//                 hardware); plain vector stores are the fallback when the
//                 output cannot be described to TMA.
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
constexpr int kIgemmThreads = 384;
constexpr int kIgemmProducers = PLB_IGEMM_PRODUCERS;
constexpr int kIgemmMmaWarp = 3;
constexpr int kEpiStagingBytes = 8 * 4096;  // 8 epilogue warps x (32 rows x 128 B)
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
  int num_stages;  // pipeline depth (<= kIgemmMaxStages)
  // ---- epilogue ---------------------------------------------------------------
  void *out;
  long long ldc;  // elements between consecutive output pixels
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
constexpr int kIgemmBarrierBytes = 256;
constexpr int kIgemmSmemLimit = 227 * 1024;

// Shared memory: [stages][resident weights][epilogue staging][barriers], after
// up to 1023 bytes of alignment slack.  A stage holds the 128 x 128-byte
// activation tile and, unless the weights are resident, the BN x 128-byte
// weight tile of one K step.
template <int BN, bool kResB>
struct IgemmSmem {
  static constexpr int kABytes = kTileM * kStageKBytes;  // without a halo
  static constexpr int kBBytes = BN * kStageKBytes;
  static constexpr int kFixedBytes = kEpiStagingBytes + kIgemmBarrierBytes + 1024;
  __host__ __device__ static constexpr int stageBytes(int a_stage_bytes) {
    return a_stage_bytes + (kResB ? 0 : kBBytes);
  }
  // deepest pipeline that fits beside `resident` bytes of weights
  static constexpr int stagesFor(int a_stage_bytes, int resident) {
    const int n = (kIgemmSmemLimit - kFixedBytes - resident) / stageBytes(a_stage_bytes);
    return n > kIgemmMaxStages ? kIgemmMaxStages : n;
  }
  static constexpr int totalBytes(int a_stage_bytes, int stages, int resident) {
    return stages * stageBytes(a_stage_bytes) + resident + kFixedBytes;
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
// kHalo: (with kResB) one activation strip per (horizontal tap, channel chunk)
//       feeds all vertical taps: the strip of tap row r is the same shared
//       memory shifted by whole 8-row groups, which the descriptor's start
//       address can express.  Cuts the activation traffic of a KxK filter K-fold.
template <int BN, bool kFp8, bool kBMn, bool kResB, bool kHalo>
__global__ void __launch_bounds__(kIgemmThreads, 1)
igemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
             const __grid_constant__ CUtensorMap tm_out, const IgemmArgs args) {
  using S = IgemmSmem<BN, kResB>;
  constexpr int kMaxStages = kIgemmMaxStages;
  const int kStages = args.num_stages;
  constexpr int P = kIgemmProducers;
  constexpr uint32_t kTmemCols = 2 * BN;  // two accumulators
  static_assert(kTmemCols >= 32 && kTmemCols <= 512 && (kTmemCols & (kTmemCols - 1)) == 0, "");
  static_assert(!(kFp8 && kBMn), "MN-major B is implemented for fp16 only");
  static_assert(!kHalo || kResB, "halo mode keeps the weights resident");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  // K steps: every (r, s, kc); pipeline steps: in halo mode one per (s, kc)
  const int k_iters = args.taps_h * args.taps_w * args.k_chunks;
  const int p_iters = kHalo ? args.taps_w * args.k_chunks : k_iters;
  const int stage_bytes = S::stageBytes(args.a_stage_bytes);
  const uint32_t resb_base = smem_base + kStages * stage_bytes;
  const uint32_t staging_base = resb_base + (kResB ? k_iters * S::kBBytes : 0);
  const uint32_t bar_base = staging_base + kEpiStagingBytes;
  // barrier words: full[8], empty[8], tmem_full[2], tmem_empty[2], drain, resident-B
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kMaxStages + s); };
  auto tmem_full_bar = [&](int a) { return bar_base + 8u * (2 * kMaxStages + a); };
  auto tmem_empty_bar = [&](int a) { return bar_base + 8u * (2 * kMaxStages + 2 + a); };
  const uint32_t drain_bar = bar_base + 8u * (2 * kMaxStages + 4);
  const uint32_t resb_bar = bar_base + 8u * (2 * kMaxStages + 5);
  const uint32_t tmem_slot = bar_base + 8u * (2 * kMaxStages + 6);
  uint8_t *bar_gen = smem_raw + (bar_base - smem_u32(smem_raw));
  volatile uint32_t *tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t *>(bar_gen + 8 * (2 * kMaxStages + 6));
  volatile int *abort_flag = reinterpret_cast<volatile int *>(bar_gen + 8 * (2 * kMaxStages + 7));

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
    mbar_init(resb_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
    if (args.use_tma_store) tma_prefetch_desc(&tm_out);
  }
  if (warp == kIgemmMmaWarp) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_ptr;

  const int m_tiles = args.tiles_w * args.tiles_h * args.tiles_n;
  const int total_tiles = m_tiles * args.n_tiles;
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

  // M tile index -> first pixel of the tile; tile row -> pixel inside the tile
  auto tile_origin = [&](int m_idx, int &w0, int &h0, int &n0) {
    const int tw = m_idx % args.tiles_w;
    const int rest = m_idx / args.tiles_w;
    int th, tn;
    if (args.h_outer) {
      tn = rest % args.tiles_n;
      th = rest / args.tiles_n;
    } else {
      th = rest % args.tiles_h;
      tn = rest / args.tiles_h;
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

  if (warp < P) {
    // ===================== TMA producers =====================
    if (elect_one()) {
      const int me = warp;
      int stage = me;          // stage of this producer's next K step
      uint32_t phase = 0;
      int turn = 0;            // (global K step) mod P
      bool ok = true;
      [[maybe_unused]] int trace_slot = 0;
      // B tile of K step (r, s, kc) -> shared memory at `dst`
      auto load_b = [&](uint32_t dst, uint32_t bar, int r, int s, int kc, int n_col) {
        const int b_tap = (args.flip_h ? args.taps_h - 1 - r : r) * args.taps_w +
                          (args.flip_w ? args.taps_w - 1 - s : s);
        if constexpr (kBMn) {
          // K rows x 64 columns per block; blocks of 64 columns are 64 rows apart
#pragma unroll
          for (int j = 0; j < BN / 64; ++j)
            tma_load_3d(dst + j * (64 * kStageKBytes), &tm_b, bar, n_col + j * 64, kc * 64, b_tap);
        } else {
          tma_load_3d(dst, &tm_b, bar, kc * kElemsPerStage, n_col, b_tap);
        }
      };
      if constexpr (kResB) {
        if (me == 0 && int(blockIdx.x) < total_tiles) {
          // single N tile: every tile of this CTA uses the same weights
          mbar_expect_tx(resb_bar, uint32_t(k_iters) * S::kBBytes);
          int r = 0, s = 0, kc = 0;
          for (int it = 0; it < k_iters; ++it) {
            load_b(resb_base + it * S::kBBytes, resb_bar, r, s, kc, 0);
            if (++kc == args.k_chunks) {
              kc = 0;
              if (++s == args.taps_w) {
                s = 0;
                ++r;
              }
            }
          }
        }
      }
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        int m_idx, n_idx;
        tile_coords(tile, m_idx, n_idx);
        int w0, h0, n0;
        tile_origin(m_idx, w0, h0, n0);
        const int w_base = w0 * args.stride_w - args.pad_w;
        const int h_base = h0 * args.stride_h - args.pad_h;
        const int n_col = n_idx * BN;
        int r = 0, s = 0, kc = 0;
        for (int it = 0; it < p_iters; ++it) {
          if (turn == me) {
            if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
              atomicCAS(args.status, kStatusOk, kStatusProducerTimeout);
              ok = false;
              break;
            }
            if (me == 0) { PLB_TRACE_STAMP(0, trace_slot); ++trace_slot; }
            const uint32_t a_dst = smem_base + stage * stage_bytes;
            mbar_expect_tx(full_bar(stage), uint32_t(stage_bytes));
            const int cw = w_base + s * args.dil_w, ch = h_base + r * args.dil_h;
            if (args.h_outer)
              tma_load_4d(a_dst, &tm_a, full_bar(stage), kc * kElemsPerStage, cw, n0, ch);
            else
              tma_load_4d(a_dst, &tm_a, full_bar(stage), kc * kElemsPerStage, cw, ch, n0);
            if constexpr (!kResB)
              load_b(a_dst + args.a_stage_bytes, full_bar(stage), r, s, kc, n_col);
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
      // Teardown (producer 0): every copy must have landed before the CTA may
      // exit.  In a run without errors the consumer has already waited for
      // them, so this costs one try_wait per stage.  Stage s was last filled
      // by K step g = the largest g < total with g mod kStages == s, in phase
      // (g / kStages) & 1; a stage that was never used is skipped.
      if (me == 0) {
        const int my_tiles = (total_tiles > int(blockIdx.x))
                                 ? (total_tiles - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x)
                                 : 0;
        const long long total_steps = (long long)my_tiles * p_iters;
        if (kResB && my_tiles > 0) {
          const long long start = clock64();
          while (!mbar_try_wait(resb_bar, 0)) {
            if (*abort_flag != 0 || clock64() - start > kWaitCycleLimit) {
              atomicCAS(args.status, kStatusOk, kStatusDrainTimeout);
              break;
            }
          }
        }
        for (int st = 0; st < kStages; ++st) {
          if (total_steps <= st) continue;
          const long long g = st + ((total_steps - 1 - st) / kStages) * kStages;
          const uint32_t last = uint32_t((g / kStages) & 1);
          const long long start = clock64();
          while (!mbar_try_wait(full_bar(st), last)) {
            if (*abort_flag != 0 || clock64() - start > kWaitCycleLimit) {
              atomicCAS(args.status, kStatusOk, kStatusDrainTimeout);
              break;
            }
          }
        }
      }
    }
  } else if (warp == kIgemmMmaWarp) {
    // ===================== MMA issuer =====================
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc(kTileM, BN, 0, 0, false, kBMn);
      const uint64_t a_desc0 = make_smem_desc(smem_base, 16, 1024);
      // B tiles: resident ones start at resb_base, streamed ones follow the
      // activations inside their stage
      const uint64_t b_desc0 =
          kBMn ? make_smem_desc(kResB ? resb_base : smem_base + uint32_t(args.a_stage_bytes),
                                64 * kStageKBytes, 1024)
               : make_smem_desc(kResB ? resb_base : smem_base + uint32_t(args.a_stage_bytes), 16,
                                1024);
      [[maybe_unused]] const uint64_t halo_step16 = uint64_t(uint32_t(args.halo_step_bytes) >> 4);
      [[maybe_unused]] const uint64_t b_row_step16 =
          uint64_t(uint32_t(args.taps_w * args.k_chunks) * (S::kBBytes >> 4));
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase[2] = {0, 0};
      int local_tile = 0;
      bool ok = true;
      [[maybe_unused]] int trace_slot = 0;
      if (kResB && int(blockIdx.x) < total_tiles) {
        if (!mbar_wait(resb_bar, 0, abort_flag)) {
          atomicCAS(args.status, kStatusOk, kStatusMmaTimeout);
          ok = false;
        }
      }
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local_tile) {
        const int acc = local_tile & 1;
        PLB_TRACE_STAMP(1, trace_slot); ++trace_slot;
        // wait for the epilogue to have drained this accumulator
        if (!mbar_wait(tmem_empty_bar(acc), acc_phase[acc] ^ 1u, abort_flag)) {
          atomicCAS(args.status, kStatusOk, kStatusMmaTimeout);
          ok = false;
          break;
        }
        acc_phase[acc] ^= 1u;
        tc_fence_after_sync();
        PLB_TRACE_STAMP(1, trace_slot); ++trace_slot;
        const uint32_t d_tmem = tmem_base + acc * BN;
        int s_tap = 0, kc = 0;  // halo mode: pipeline step = (s_tap, kc), kc fastest
        for (int it = 0; it < p_iters; ++it) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
            atomicCAS(args.status, kStatusOk, kStatusMmaTimeout);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          PLB_TRACE_STAMP(1, trace_slot); ++trace_slot;
          // Descriptors are advanced by adding to their start-address field
          // (16-byte units, cannot overflow for shared-memory addresses): the
          // issuing thread's own instruction count bounds the MMA rate on
          // narrow tiles.
          const uint32_t stage_off16 = uint32_t(stage * stage_bytes) >> 4;
          uint64_t a_desc = a_desc0 + stage_off16;
          uint64_t b_desc;
          if constexpr (kHalo)
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
              umma_ss<kFp8>(d_tmem, a_k, b_k, idesc, (it | r | k) != 0 ? 1u : 0u);
            }
            if constexpr (kHalo) {
              // next filter row: the strip shifted by whole 8-row groups; its
              // resident weight tile is taps_w * k_chunks tiles further on
              a_desc += halo_step16;
              b_desc += b_row_step16;
            }
          }
          umma_commit(empty_bar(stage));  // frees the stage when these MMAs retire
          PLB_TRACE_STAMP(1, trace_slot); ++trace_slot;
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
          if (++kc == args.k_chunks) {
            kc = 0;
            ++s_tap;
          }
        }
        if (ok) umma_commit(tmem_full_bar(acc));
      }
      // make sure nothing is still executing before TMEM is released
      umma_commit(drain_bar);
      const long long start = clock64();
      while (!mbar_try_wait(drain_bar, 0)) {
        if (clock64() - start > kWaitCycleLimit) {
          atomicCAS(args.status, kStatusOk, kStatusDrainTimeout);
          break;
        }
      }
    }
  } else if (warp >= 4) {
    // ===================== epilogue (warps 4..11) =====================
    const int group = (warp - 4) >> 2;       // drains accumulator `group`
    const int quarter = warp & 3;            // TMEM lanes [32*quarter, 32*quarter+32)
    const int row = quarter * 32 + lane;     // tile row handled by this thread
    uint32_t acc_phase = 0;
    int rw, rh, rn;
    row_pixel(row, rw, rh, rn);
    // origin of this warp's 32 rows inside the tile's pixel box
    int qw, qh, qn;
    row_pixel(quarter * 32, qw, qh, qn);
    const uint32_t buf = staging_base + uint32_t(warp - 4) * 4096u;  // this warp's staged rows
    const uint32_t row_addr = buf + uint32_t(lane) * 128u;
    const bool tma_store = args.use_tma_store != 0;
    const bool out_f32 = args.out_is_f32 != 0;
    const bool stamp = threadIdx.x == 128;
    const int acc = group;
    int local_tile = group;
    for (int tile = int(blockIdx.x) + group * int(gridDim.x); tile < total_tiles;
         tile += 2 * int(gridDim.x), local_tile += 2) {
      int m_idx, n_idx;
      tile_coords(tile, m_idx, n_idx);
      int w0, h0, n0;
      tile_origin(m_idx, w0, h0, n0);
      const int ow = w0 + rw, oh = h0 + rh, on = n0 + rn;
      const bool row_ok = ow < args.out_w && oh < args.out_h && on < args.out_n;
      const long long pixel = (static_cast<long long>(on) * args.out_h + oh) * args.out_w + ow;
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

      // 32 accumulator columns [c, c + 32) of this thread's row: scale / add /
      // cast and store (or stage for the tensor store)
      auto process = [&](const uint32_t (&v)[32], const int c) {
        [[maybe_unused]] const bool fine = stamp && local_tile == 2;
        if (fine) PLB_TRACE_STAMP(2, 2048 + (c >> 5) * 8 + 0);
        const int col0 = col_base + c;
        const int valid = min(32, args.n_total - col0);  // may be <= 0 on a padded N tile
        float f[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]) * args.alpha;
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
        if (tma_store) {
          // 32 columns of this row go to its 128-byte staged row: fp32 fills the
          // row, half fills half of it (two passes per store).  16-byte pieces
          // are XOR-swizzled with the row index, the pattern the tensor map uses.
          const int pass = out_f32 ? 0 : ((c >> 5) & 1);
          if (pass == 0) {
            // the previous store from this buffer must have read it
            if (fine) PLB_TRACE_STAMP(2, 2048 + (c >> 5) * 8 + 1);
            if (lane == 0) tma_store_wait_read<0>();
            __syncwarp();
          }
          if (fine) PLB_TRACE_STAMP(2, 2048 + (c >> 5) * 8 + 2);
          if (out_f32) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              st_shared_v4(row_addr + (uint32_t(j ^ (lane & 7)) << 4), __float_as_uint(f[4 * j]),
                           __float_as_uint(f[4 * j + 1]), __float_as_uint(f[4 * j + 2]),
                           __float_as_uint(f[4 * j + 3]));
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              __half2 h0 = __floats2half2_rn(f[8 * j], f[8 * j + 1]);
              __half2 h1 = __floats2half2_rn(f[8 * j + 2], f[8 * j + 3]);
              __half2 h2 = __floats2half2_rn(f[8 * j + 4], f[8 * j + 5]);
              __half2 h3 = __floats2half2_rn(f[8 * j + 6], f[8 * j + 7]);
              st_shared_v4(row_addr + (uint32_t((pass * 4 + j) ^ (lane & 7)) << 4),
                           *reinterpret_cast<uint32_t *>(&h0), *reinterpret_cast<uint32_t *>(&h1),
                           *reinterpret_cast<uint32_t *>(&h2), *reinterpret_cast<uint32_t *>(&h3));
            }
          }
          const bool last_pass = out_f32 || pass == 1 || c + 32 >= BN;
          if (fine) PLB_TRACE_STAMP(2, 2048 + (c >> 5) * 8 + 3);
          if (last_pass) {
            fence_proxy_async_smem();
            __syncwarp();
            if (fine) PLB_TRACE_STAMP(2, 2048 + (c >> 5) * 8 + 4);
            if (lane == 0) {
              const int store_col = col_base + (out_f32 ? c : (c & ~63));
              // a box that starts outside the tensor has nothing to write
              if (store_col < args.n_total && box_ok) {
                if (args.h_outer)
                  tma_store_4d(&tm_out, buf, store_col, w0 + qw, n0 + qn, h0 + qh);
                else
                  tma_store_4d(&tm_out, buf, store_col, w0 + qw, h0 + qh, n0 + qn);
              }
              tma_store_commit();
            }
            if (fine) PLB_TRACE_STAMP(2, 2048 + (c >> 5) * 8 + 5);
          }
        } else if (row_ok && valid > 0) {
          if (out_f32) {
            float *dst = static_cast<float *>(args.out) + pixel * args.ldc + col0;
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
            __half *dst = static_cast<__half *>(args.out) + pixel * args.ldc + col0;
            if (valid == 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
              uint32_t pk[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                __half2 h = __floats2half2_rn(f[2 * j], f[2 * j + 1]);
                pk[j] = *reinterpret_cast<uint32_t *>(&h);
              }
              if ((reinterpret_cast<uintptr_t>(dst) & 31) == 0) {
                // whole 32-byte sectors per lane
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
        }
      };

      // Two register buffers: while one block of 32 columns is processed the
      // load of the next is in flight (tcgen05.wait::ld covers all loads issued
      // so far, so it is only executed between a load and the use of its data).
      uint32_t va[32], vb[32];
      __syncwarp();
      tmem_ld_32x32(t_addr, va);
#pragma unroll
      for (int c = 0; c < BN; c += 64) {
        tmem_ld_wait_for(va);
        tmem_ld_32x32(t_addr + c + 32, vb);
        process(va, c);
        tmem_ld_wait_for(vb);
        if (c + 64 < BN) {
          tmem_ld_32x32(t_addr + c + 64, va);
        } else {
          // the accumulator is fully read: hand it back before the last stores
          tc_fence_before_sync();
          mbar_arrive(tmem_empty_bar(acc));
          if (stamp) PLB_TRACE_STAMP(2, local_tile * 4 + 2);
        }
        process(vb, c + 32);
      }
      if (stamp) PLB_TRACE_STAMP(2, local_tile * 4 + 3);
    }
    // all of this thread's stores must be complete before the CTA exits
    if (tma_store && lane == 0) tma_store_wait_all<0>();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == kIgemmMmaWarp) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace plb
