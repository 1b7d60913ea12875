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
// tiles).  With a unit vertical stride a group is one filter column: the
// activations of a K step are loaded once, as a strip of box_h + halo input
// rows, and serve all taps_h vertical taps.  The pixels of a tile are then
// ordered (w, n, h), h slowest, and box_w * box_n is a multiple of 8, so that
// moving down one filter row moves the operand's start by whole 1024-byte
// swizzle atoms.  Every CTA leaves its partial sums in a global fp32 scratch buffer;
// a second kernel adds the K splits in a fixed order (the role of the
// reference's ReduceAdd codelet, lib/poplin/codelets/ReduceAdd.cpp) and casts.
//
// Roles inside a CTA: warps 0..2 issue the tensor copies of every K step
// between them (a copy costs its issuing thread on the order of a hundred
// cycles, a K step needs 2 + taps * ci_blk64 copies), warp 3 issues the MMAs
// (neighbouring taps share one instruction when their accumulators and
// operand blocks are contiguous, which halves the reads of the outGrad tile),
// warps 4..7 move the accumulators TMEM -> registers -> swizzled shared memory
// -> global with tensor stores.
#pragma once

#include "sm100_prims.cuh"

namespace plb {

constexpr int kWuThreads = 256;
constexpr int kWuProducers = 3;  // warps 0..2 issue TMA, warp 3 issues MMA, warps 4..7 drain
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
  int stage_bytes;  // host-side copy of the kernel's stage size
  int tmem_cols;
  // Strip mode (halo_rows > 0, or a filter of height 1 handled the same way):
  // tap group g = filter column g, local tap t = filter row t.
  int strip_mode;
  int strip_rows;       // pixels of one strip: box_w * box_n * (box_h + halo)
  int halo_step_bytes;  // operand offset from one filter row to the next
  // The instructions of one 16-pixel step all read the same outGrad tile: keep
  // it in the tensor core's collector buffer between them (0 = fetch it each time).
  int reuse_a;
  uint32_t idesc_formats;  // operand format bits of the instruction descriptor (bfloat16 operands)
  float *partial;  // [ksplit][taps][co_total][ci_total]
  int *status;
  long long *trace;  // optional timeline of CTA 0 (builds with -DPLB_TRACE only)
};

#ifdef PLB_TRACE
#define PLB_WU_STAMP(role, slot)                                               \
  do {                                                                         \
    if (args.trace != nullptr && blockIdx.x == 0 && (slot) < 4096)             \
      args.trace[(role)*4096 + (slot)] = clock64();                            \
  } while (0)
#else
#define PLB_WU_STAMP(role, slot) do { } while (0)
#endif

__global__ void __launch_bounds__(kWuThreads, 1)
wu_kernel(const __grid_constant__ CUtensorMap tm_dy, const __grid_constant__ CUtensorMap tm_x,
          const __grid_constant__ CUtensorMap tm_out, const WuArgs args) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int a_bytes = 2 * kWuBlockBytes;  // 128 output channels
  const bool strip = args.strip_mode != 0;
  // one 64-channel block of the activations of a stage
  const int b_block_bytes = strip ? args.strip_rows * 128 : kWuBlockBytes;
  const int b_bytes = (strip ? 1 : args.taps_per_group) * args.ci_blk64 * b_block_bytes;
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
      mbar_init(full_bar(s), kWuProducers);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(acc_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_dy);
    tma_prefetch_desc(&tm_x);
    tma_prefetch_desc(&tm_out);
  }
  if (warp == 3) {
    tmem_alloc(tmem_slot, uint32_t(args.tmem_cols));
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_ptr;
  // set-up done: with a programmatic launch everything above overlapped the
  // previous kernel's tail; global memory is touched only from here on
  pdl_launch_dependents();
  pdl_wait();

  // ---- which unit of work is this CTA's ------------------------------------
  int unit = blockIdx.x;
  const int split = unit % args.ksplit;
  unit /= args.ksplit;
  const int tap_group = unit % args.tap_groups;
  unit /= args.tap_groups;
  const int ci_block = unit % args.ci_blocks;
  const int co_block = unit / args.ci_blocks;
  const int taps = args.taps_h * args.taps_w;
  // local tap t of this CTA is filter tap tap0 + t * tap_step
  const int tap0 = strip ? tap_group : tap_group * args.taps_per_group;
  const int tap_step = strip ? args.taps_w : 1;
  const int ntaps = strip ? args.taps_h : min(args.taps_per_group, taps - tap0);
  const int pixel_tiles = args.tiles_w * args.tiles_h * args.tiles_n;
  const int t_begin = int((long long)pixel_tiles * split / args.ksplit);
  const int t_end = int((long long)pixel_tiles * (split + 1) / args.ksplit);
  const int k_iters = t_end - t_begin;

  if (warp < kWuProducers) {
    // ===================== TMA producers =====================
    // Copy c of a K step (0, 1: the two 64-channel halves of the outGrad tile;
    // then the 64-channel blocks of the activations, per tap or per strip) is
    // issued by producer c mod kWuProducers; each producer arrives once per
    // stage with the byte count of its own copies.
    if (elect_one()) {
      const int me = warp;
      const int copies = 2 + (strip ? 1 : ntaps) * args.ci_blk64;
      uint32_t my_bytes = 0;
      for (int c = me; c < copies; c += kWuProducers)
        my_bytes += uint32_t(c < 2 ? kWuBlockBytes : b_block_bytes);
      int stage = 0;
      uint32_t phase = 0;
      // pixel tile of the current K step, advanced without divisions
      int tw = t_begin % args.tiles_w;
      int th = (t_begin / args.tiles_w) % args.tiles_h;
      int tn = t_begin / (args.tiles_w * args.tiles_h);
      [[maybe_unused]] int trace_slot = 0;
      for (int it = 0; it < k_iters; ++it) {
        const int w0 = tw * args.box_w, h0 = th * args.box_h, n0 = tn * args.box_n;
        if (me == 0) { PLB_WU_STAMP(0, trace_slot); ++trace_slot; }
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
          atomicCAS(args.status, kStatusOk, kStatusProducerTimeout);
          break;
        }
        if (me == 0) { PLB_WU_STAMP(0, trace_slot); ++trace_slot; }
        const uint32_t a_dst = smem_base + stage * stage_bytes;
        const uint32_t b_dst = a_dst + a_bytes;
        mbar_expect_tx(full_bar(stage), my_bytes);
        for (int c = me; c < copies; c += kWuProducers) {
          if (c < 2) {
            // tensor dimensions are (channel, w, h, n), in strip mode (channel, w, n, h)
            tma_load_4d(a_dst + c * kWuBlockBytes, &tm_dy, full_bar(stage),
                        co_block * 128 + c * 64, w0, strip ? n0 : h0, strip ? h0 : n0);
          } else if (strip) {
            const int j = c - 2;
            const int iw = w0 * args.stride_w + tap0 * args.dil_w - args.pad_w;
            const int ih = h0 - args.pad_h;
            tma_load_4d(b_dst + j * b_block_bytes, &tm_x, full_bar(stage),
                        ci_block * args.ci_blk + j * 64, iw, n0, ih);
          } else {
            const int t = (c - 2) / args.ci_blk64, j = (c - 2) - t * args.ci_blk64;
            const int tap = tap0 + t;
            const int r = tap / args.taps_w, sx = tap - r * args.taps_w;
            const int iw = w0 * args.stride_w + sx * args.dil_w - args.pad_w;
            const int ih = h0 * args.stride_h + r * args.dil_h - args.pad_h;
            tma_load_4d(b_dst + (c - 2) * kWuBlockBytes, &tm_x, full_bar(stage),
                        ci_block * args.ci_blk + j * 64, iw, ih, n0);
          }
        }
        if (me == 0) { PLB_WU_STAMP(0, trace_slot); ++trace_slot; }
        if (++stage == stages) {
          stage = 0;
          phase ^= 1u;
        }
        if (++tw == args.tiles_w) {
          tw = 0;
          if (++th == args.tiles_h) {
            th = 0;
            ++tn;
          }
        }
      }
      // producer 0: all copies must have landed before the CTA exits.  Stage st
      // was last filled by K step g = the largest g < k_iters with g mod stages
      // == st, in phase (g / stages) & 1.
      if (me == 0) {
        for (int st = 0; st < stages; ++st) {
          if (k_iters <= st) continue;
          const int g = st + ((k_iters - 1 - st) / stages) * stages;
          const uint32_t last = uint32_t((g / stages) & 1);
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
  } else if (warp == 3) {
    // ===================== MMA issuer =====================
    if (elect_one()) {
      // taps whose accumulator columns and operand blocks follow one another
      // without a gap go into one instruction of up to 256 columns
      const int merge =
          !strip && args.ci_blk == args.ci_blk64 * 64 ? max(1, 256 / args.ci_blk) : 1;
      const int tap_bytes = strip ? args.halo_step_bytes : args.ci_blk64 * kWuBlockBytes;
      const uint32_t idesc_full =
          make_idesc(128, uint32_t(merge * args.ci_blk), 0, 0, true, true) | args.idesc_formats;
      const uint32_t idesc_rest =
          make_idesc(128, uint32_t(max(1, ntaps % merge) * args.ci_blk), 0, 0, true, true) |
          args.idesc_formats;
      const uint32_t d_step = uint32_t(merge * args.ci_blk);
      const uint64_t b_step16 = uint64_t(merge * tap_bytes) >> 4;
      const uint64_t a_desc0 = make_smem_desc(smem_base, kWuBlockBytes, 1024);
      const uint64_t b_desc0 = make_smem_desc(smem_base + a_bytes, uint32_t(b_block_bytes), 1024);
      // at least two instructions per step, all of the same shape
      const bool reuse_a = args.reuse_a != 0 && ntaps % merge == 0 && ntaps / merge >= 2;
      int stage = 0;
      uint32_t phase = 0;
      [[maybe_unused]] int trace_slot = 0;
      for (int it = 0; it < k_iters; ++it) {
        PLB_WU_STAMP(1, trace_slot); ++trace_slot;
        if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
          atomicCAS(args.status, kStatusOk, kStatusMmaTimeout);
          break;
        }
        tc_fence_after_sync();
        PLB_WU_STAMP(1, trace_slot); ++trace_slot;
        // The issuing thread's own instructions bound the MMA rate when an MMA
        // is short, so descriptors are advanced with one addition each: the
        // start-address field counts 16-byte units and never overflows.
        const uint32_t stage_off16 = uint32_t(stage * stage_bytes) >> 4;
        const uint64_t a_stage = a_desc0 + stage_off16;
        const uint64_t b_stage = b_desc0 + stage_off16;
#pragma unroll
        for (int k = 0; k < kWuPixelsPerStage / 16; ++k) {
          // 16 pixels = 16 rows of 128 bytes
          const uint64_t a_desc = a_stage + uint64_t(k * (2048 >> 4));
          uint64_t b_desc = b_stage + uint64_t(k * (2048 >> 4));
          uint32_t d_col = tmem_base;
          const uint32_t accumulate = (it | k) != 0 ? 1u : 0u;
          int t = 0;
          if (reuse_a) {
            // same A tile and shape for all of them: fill, use ..., lastuse
            umma_ss_f16_collect_a<1>(d_col, a_desc, b_desc, idesc_full, accumulate);
            for (t = merge; t + 2 * merge <= ntaps; t += merge) {
              d_col += d_step;
              b_desc += b_step16;
              umma_ss_f16_collect_a<2>(d_col, a_desc, b_desc, idesc_full, accumulate);
            }
            d_col += d_step;
            b_desc += b_step16;
            umma_ss_f16_collect_a<3>(d_col, a_desc, b_desc, idesc_full, accumulate);
            continue;
          }
          for (; t + merge <= ntaps; t += merge) {
            umma_ss<false>(d_col, a_desc, b_desc, idesc_full, accumulate);
            d_col += d_step;
            b_desc += b_step16;
          }
          if (t < ntaps) umma_ss<false>(d_col, a_desc, b_desc, idesc_rest, accumulate);
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
  } else if (warp >= 4) {
    // ===================== epilogue (warps 4..7) =====================
    // Each warp owns 32 output channels (its TMEM lanes).  A 32 x 32 block of
    // fp32 sums goes through a 4 KB staging buffer in the (now idle) pipeline
    // memory, written with the 128-byte swizzle the tensor map expects, and
    // leaves with one tensor store; two buffers per warp overlap the store of
    // one block with the TMEM read of the next.  The store clips rows and
    // columns beyond the tensor's extents.
    const int quarter = warp & 3;
    const int co0 = co_block * 128 + quarter * 32;
    if (mbar_wait(acc_bar, 0, abort_flag)) {
      tc_fence_after_sync();
      if (threadIdx.x == 128) PLB_WU_STAMP(2, 0);
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
      const uint32_t stage_buf = smem_base + uint32_t(quarter) * 8192u;
      int buf = 0;
      for (int t = 0; t < ntaps; ++t) {
        for (int c = 0; c < args.ci_blk; c += 32) {
          const int ci0 = ci_block * args.ci_blk + c;
          if (co0 >= args.co_total || ci0 >= args.ci_total) continue;  // warp-uniform
          uint32_t v[32];
          if (k_iters > 0) {
            tmem_ld_32x32(t_addr + t * args.ci_blk + c, v);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0u;
          }
          // the store issued from this buffer two blocks ago must have read it
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
          const uint32_t row_addr = stage_buf + uint32_t(buf) * 4096u + uint32_t(lane) * 128u;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            st_shared_v4(row_addr + (uint32_t(j ^ (lane & 7)) << 4), v[4 * j], v[4 * j + 1],
                         v[4 * j + 2], v[4 * j + 3]);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_4d(&tm_out, stage_buf + uint32_t(buf) * 4096u, ci0, co0,
                         tap0 + t * tap_step, split);
            tma_store_commit();
          }
          buf ^= 1;
        }
      }
      // the stores must have read their staging buffers before the CTA gives up
      // its shared memory; the writes themselves complete with the grid
      if (lane == 0) tma_store_wait_read<0>();
      __syncwarp();
      if (threadIdx.x == 128) PLB_WU_STAMP(2, 1);
    } else {
      atomicCAS(args.status, kStatusOk, kStatusEpilogueTimeout);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 3) {
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

// The same over four consecutive sums per thread (count is a multiple of 4
// and the pointers are 16-byte / 8-byte aligned), with the K splits of one
// output spread over kWuReduceLanes threads so that enough loads are in
// flight: lane y adds splits y, y + lanes, ... in order, then the lanes'
// sums are added in lane order.  The order of additions is fixed, so the
// result does not depend on timing.
constexpr int kWuReduceLanes = 8;
__global__ void __launch_bounds__(32 * kWuReduceLanes)
wu_reduce4_kernel(const float4 *__restrict__ partial, int ksplit, size_t count4,
                  float4 *__restrict__ out_f32, uint2 *__restrict__ out_half) {
  __shared__ float4 part[kWuReduceLanes][32];
  pdl_launch_dependents();
  pdl_wait();  // the partial sums come from the previous kernel in the stream
  const size_t i = blockIdx.x * size_t(32) + threadIdx.x;
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  if (i < count4) {
#pragma unroll 4
    for (int k = threadIdx.y; k < ksplit; k += kWuReduceLanes) {
      const float4 v = partial[size_t(k) * count4 + i];
      s.x += v.x;
      s.y += v.y;
      s.z += v.z;
      s.w += v.w;
    }
  }
  part[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && i < count4) {
#pragma unroll
    for (int y = 1; y < kWuReduceLanes; ++y) {
      const float4 v = part[y][threadIdx.x];
      s.x += v.x;
      s.y += v.y;
      s.z += v.z;
      s.w += v.w;
    }
    if (out_f32) out_f32[i] = s;
    if (out_half) {
      const __half2 lo = __floats2half2_rn(s.x, s.y), hi = __floats2half2_rn(s.z, s.w);
      out_half[i] = make_uint2(*reinterpret_cast<const uint32_t *>(&lo),
                               *reinterpret_cast<const uint32_t *>(&hi));
    }
  }
}

// ---- split-K reduction fused with the sum over ranks -------------------------------
// Batch-sharded weight update on several GPUs: the split-K reduction above and
// the all-reduce of the per-rank gradients in ONE kernel.  A block reduces the
// K splits of a chunk of kWuFusedChunk float4 sums exactly as wu_reduce4_kernel
// does, writes them into this rank's peer-addressable gradient buffer and at
// once tells every peer "chunk b of rank r is complete" (a flag per chunk and
// sender in the receiver's flag area, carrying the step number).  It then
// waits, with a cycle budget, for the same chunk's flag from every peer, reads
// the peers' chunk with plain peer loads, adds the ranks' sums in rank order
// (every rank forms identical bits) and writes the fp32 gradient of the whole
// batch and / or its cast.  The exchange of a chunk overlaps the reduction of
// the following ones, so the collective costs little more than one NVLink
// round trip after the last chunk instead of a kernel launch, a flag round
// for the whole vector and the transfer.
//
// Block b of a rank waits only for block b of the peers, and only after it has
// sent its own flag; blocks are dispatched in index order, so a block's
// predecessors on every GPU have all sent theirs.  The host caps the grid at
// what is resident at once anyway.  No multicast, no TMA on peer memory.
constexpr int kWuFusedGroups = 4;                     // groups of 32 float4 per block
constexpr int kWuFusedChunk = 32 * kWuFusedGroups;    // float4 sums per block
constexpr int kWuPeerMaxWorld = 16;
constexpr int kStatusWuPeerTimeout = 5;  // a peer's chunk flag did not arrive within the budget

struct WuPeerArgs {
  float4 *grads[kWuPeerMaxWorld];      // every rank's gradient buffer (this group's part)
  // Owner mode (results[rank] != nullptr): chunk c is added by rank c mod world
  // alone, which leaves the sum in its result buffer for the others to fetch.
  float4 *results[kWuPeerMaxWorld];    // every rank's result buffer (this group's part), or null
  uint32_t *flags[kWuPeerMaxWorld];    // every rank's flag area: [chunk][sender] words, then [chunk] result flags
  uint32_t result_flags;               // word offset of the result flags in a flag area
  int rank, world;
  uint32_t epoch;       // step number, 1, 2, 3, ...; flags only grow
  uint32_t chunk_base;  // first chunk index of this launch (groups follow one another)
  int *status;
};

__global__ void __launch_bounds__(32 * kWuReduceLanes)
wu_reduce_allreduce_kernel(const float4 *__restrict__ partial, int ksplit, size_t count4,
                           const WuPeerArgs pa, float4 *__restrict__ out_f32,
                           uint2 *__restrict__ out_half) {
  __shared__ float4 part[kWuReduceLanes][kWuFusedGroups][32];
  __shared__ int ok;
  const int tid = threadIdx.y * 32 + threadIdx.x;
  if (tid == 0) ok = 1;
  pdl_launch_dependents();
  pdl_wait();  // the partial sums come from the previous kernel in the stream
  float4 *mine = pa.grads[pa.rank];
  // Lane y adds splits y, y + lanes, ... of the block's kWuFusedGroups groups of
  // 32 sums side by side (one accumulator per group, so that the loads of all
  // groups are in flight together); then thread (x, j) adds the lanes' sums of
  // group j in lane order: the same order of additions as wu_reduce4_kernel.
  const size_t i0 = blockIdx.x * size_t(kWuFusedChunk) + threadIdx.x;
  float4 s[kWuFusedGroups];
#pragma unroll
  for (int j = 0; j < kWuFusedGroups; ++j) s[j] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 2
  for (int k = threadIdx.y; k < ksplit; k += kWuReduceLanes) {
    float4 v[kWuFusedGroups];
#pragma unroll
    for (int j = 0; j < kWuFusedGroups; ++j) {
      const size_t i = i0 + size_t(j) * 32;
      v[j] = i < count4 ? partial[size_t(k) * count4 + i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < kWuFusedGroups; ++j) {
      s[j].x += v[j].x;
      s[j].y += v[j].y;
      s[j].z += v[j].z;
      s[j].w += v[j].w;
    }
  }
#pragma unroll
  for (int j = 0; j < kWuFusedGroups; ++j) part[threadIdx.y][j][threadIdx.x] = s[j];
  __syncthreads();
  if (threadIdx.y < kWuFusedGroups) {
    const int j = threadIdx.y;
    const size_t i = i0 + size_t(j) * 32;
    float4 t = part[0][j][threadIdx.x];
#pragma unroll
    for (int y = 1; y < kWuReduceLanes; ++y) {
      const float4 v = part[y][j][threadIdx.x];
      t.x += v.x;
      t.y += v.y;
      t.z += v.z;
      t.w += v.w;
    }
    if (i < count4) mine[i] = t;
  }
  __syncthreads();
  // This rank's chunk is complete; the barrier above orders every thread's
  // stores before the flag-sending threads.  Publishing: the chunk lies in THIS
  // GPU's memory and the peers read it through this GPU's L2, the point of
  // coherence for that memory, so it is enough that the stores have reached L2
  // before the flag leaves: a device-scope fence (cumulative over the barrier),
  // then a plain system-scope store of the flag into the peer's memory.  A
  // system-scope release instead also waits for every access this SM has in
  // flight over NVLink (other blocks' peer loads and flag stores): measured at
  // 1.5 to 7.7 us per block against 0.6 us, 63.4 against 56.9 us per step on
  // two GPUs.  -DPLB_STRICT_SYSTEM_FENCE builds the formally scoped form.
  const uint32_t chunk = pa.chunk_base + blockIdx.x;
  if (pa.results[pa.rank] != nullptr) {
    // ---- owner mode: per rank (world - 1) / world of the gradient comes in
    // twice (the owners' inputs, the others' results) instead of world - 1 times
    const int owner = int(chunk % uint32_t(pa.world));
    const size_t i = blockIdx.x * size_t(kWuFusedChunk) + tid;
    auto publish = [&](uint32_t *flag) {
#ifdef PLB_STRICT_SYSTEM_FENCE
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(pa.epoch) : "memory");
#else
      __threadfence();
      asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(pa.epoch) : "memory");
#endif
    };
    auto await = [&](const uint32_t *flag) {
      const long long start = clock64();
      while (true) {
        uint32_t seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
        if (int32_t(seen - pa.epoch) >= 0) break;
        if (clock64() - start > kWaitCycleLimit) {
          atomicCAS(pa.status, kStatusOk, kStatusWuPeerTimeout);
          ok = 0;
          break;
        }
      }
    };
    auto write_out = [&](const float4 &t) {
      if (out_f32) out_f32[i] = t;
      if (out_half) {
        const __half2 lo = __floats2half2_rn(t.x, t.y), hi = __floats2half2_rn(t.z, t.w);
        out_half[i] = make_uint2(*reinterpret_cast<const uint32_t *>(&lo),
                                 *reinterpret_cast<const uint32_t *>(&hi));
      }
    };
    if (pa.rank != owner) {
      if (tid == 0) {
        // "my chunk is complete" to the owner, then wait for "the sum is complete"
        publish(pa.flags[owner] + size_t(chunk) * kWuPeerMaxWorld + pa.rank);
        await(pa.flags[pa.rank] + pa.result_flags + chunk);
      }
      __syncthreads();
      if (!ok) return;
      if (tid < kWuFusedChunk && i < count4) {
        float4 t;
        const float4 *src = pa.results[owner] + i;
        asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
                     : "=f"(t.x), "=f"(t.y), "=f"(t.z), "=f"(t.w)
                     : "l"(src)
                     : "memory");
        write_out(t);
      }
      return;
    }
    if (tid < pa.world && tid != pa.rank)
      await(pa.flags[pa.rank] + size_t(chunk) * kWuPeerMaxWorld + tid);
    __syncthreads();
    if (!ok) return;
    if (tid < kWuFusedChunk && i < count4) {
      float4 v[kWuPeerMaxWorld];
#pragma unroll
      for (int r = 0; r < kWuPeerMaxWorld; ++r) {
        if (r < pa.world) {
          const float4 *src = pa.grads[r] + i;
          if (r == pa.rank) {
            v[r] = *src;
          } else {
            asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
                         : "=f"(v[r].x), "=f"(v[r].y), "=f"(v[r].z), "=f"(v[r].w)
                         : "l"(src)
                         : "memory");
          }
        }
      }
      float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int r = 0; r < kWuPeerMaxWorld; ++r) {
        if (r < pa.world) {
          t.x += v[r].x;
          t.y += v[r].y;
          t.z += v[r].z;
          t.w += v[r].w;
        }
      }
      pa.results[pa.rank][i] = t;
      write_out(t);
    }
    __syncthreads();
    if (tid < pa.world && tid != pa.rank) publish(pa.flags[tid] + pa.result_flags + chunk);
    return;
  }
  if (tid < pa.world && tid != pa.rank) {
    uint32_t *theirs = pa.flags[tid] + size_t(chunk) * kWuPeerMaxWorld + pa.rank;
#ifdef PLB_STRICT_SYSTEM_FENCE
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(pa.epoch) : "memory");
#else
    __threadfence();
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(pa.epoch) : "memory");
#endif
    const uint32_t *from = pa.flags[pa.rank] + size_t(chunk) * kWuPeerMaxWorld + tid;
    const long long start = clock64();

    // (acquire loads: a relaxed poll followed by a system-scope fence was
    // measured slower, the fence also waits for the flag store just sent to be
    // acknowledged by the peer)
    while (true) {
      uint32_t seen;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(from) : "memory");
      if (int32_t(seen - pa.epoch) >= 0) break;
      if (clock64() - start > kWaitCycleLimit) {
        atomicCAS(pa.status, kStatusOk, kStatusWuPeerTimeout);
        ok = 0;
        break;
      }
    }
  }
  __syncthreads();
  if (!ok) return;
  // sum over ranks, rank order; a thread's peer loads are all in flight together
  if (tid < kWuFusedChunk) {
    const size_t i = blockIdx.x * size_t(kWuFusedChunk) + tid;
    if (i < count4) {
      float4 v[kWuPeerMaxWorld];
#pragma unroll
      for (int r = 0; r < kWuPeerMaxWorld; ++r) {
        if (r < pa.world) {
          const float4 *src = pa.grads[r] + i;
          if (r == pa.rank) {
            v[r] = *src;
          } else {
            // from the peer, never from a stale line of this GPU's caches
            asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
                         : "=f"(v[r].x), "=f"(v[r].y), "=f"(v[r].z), "=f"(v[r].w)
                         : "l"(src)
                         : "memory");
          }
        }
      }
      float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int r = 0; r < kWuPeerMaxWorld; ++r) {
        if (r < pa.world) {
          s.x += v[r].x;
          s.y += v[r].y;
          s.z += v[r].z;
          s.w += v[r].w;
        }
      }
      if (out_f32) out_f32[i] = s;
      if (out_half) {
        const __half2 lo = __floats2half2_rn(s.x, s.y), hi = __floats2half2_rn(s.z, s.w);
        out_half[i] = make_uint2(*reinterpret_cast<const uint32_t *>(&lo),
                                 *reinterpret_cast<const uint32_t *>(&hi));
      }
    }
  }
}

}  // namespace plb
