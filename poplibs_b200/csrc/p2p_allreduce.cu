// All-reduce of the fp32 weight gradient over NVLink peer memory, fused with
// the cast to the weights' type.
//
// The weight-update pass of a batch-sharded convolution leaves one full-size
// fp32 gradient per GPU (a few hundred KB); the gradient of the whole batch is
// their sum.  For a message this small a library all-reduce is dominated by
// its launch and protocol latency.  Here every rank keeps its gradient in a
// buffer that all peers can address (symmetric memory, one process per GPU),
// and ONE kernel per rank
//   1. tells every peer that this rank's buffer is complete (block 0: a flag
//      written into each peer's signal pad over NVLink),
//   2. waits, with a cycle budget, for the same flag from every peer, then
//      releases the kernel's other blocks through a word in local memory,
//   3. reads all ranks' buffers with plain peer loads (one 16-byte load per
//      rank per thread, all in flight together: the message is small, so the
//      time is a few NVLink round trips, not bandwidth), adds them in rank
//      order (so every rank computes bit-identical sums) and writes the fp32
//      sum and/or its cast to local memory.
// No multicast objects and no TMA are involved: plain loads and stores to peer
// pointers.  The kernels of different ranks wait on one another, which is only
// sound because each runs on its own GPU.
//
// Re-use of the buffers: the caller alternates between two halves of its
// symmetric buffer by the parity of `epoch`.  A rank can start step e + 2
// (which overwrites the half read in step e) only after every peer has sent
// its flag of step e + 1, i.e. after that peer's kernel of step e has retired.
//
// The reference has no counterpart (it spreads one convolution over IPU tiles
// inside a single graph); this replaces the ncclAllReduce + cast that the
// multi-GPU weight update would otherwise use.
#include <cuda_fp16.h>

#include <algorithm>
#include <string>

#include "runtime.h"
#include "sm100_prims.cuh"

namespace plb {
namespace {

constexpr int kP2pMaxWorld = 16;
constexpr int kP2pThreads = 256;
constexpr int kStatusPeerTimeout = 5;  // a peer's flag did not arrive within the cycle budget

// Signal pad of a rank, 32-bit words: [r] = latest epoch announced by rank r,
// [kP2pMaxWorld] = latest epoch this rank's own block 0 has seen from everyone.
constexpr int kP2pGoSlot = kP2pMaxWorld;

struct P2pArgs {
  const float *buffers[kP2pMaxWorld];   // every rank's gradient (this step's half)
  uint32_t *signal_pads[kP2pMaxWorld];  // every rank's signal pad
  int rank, world;
  uint32_t epoch;
  size_t count4;  // float4 elements
  float4 *out_f32;
  uint2 *out_half;
  int *status;
};

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// peer data must come from the peer, not from a stale line of this GPU's caches
__device__ __forceinline__ float4 ld_peer_f4(const float4 *p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
// epochs only grow; compare modulo 2^32
__device__ __forceinline__ bool reached(uint32_t seen, uint32_t epoch) {
  return int32_t(seen - epoch) >= 0;
}

__global__ void __launch_bounds__(kP2pThreads)
p2pAllReduceKernel(const P2pArgs a) {
  __shared__ int ok;
  if (threadIdx.x == 0) ok = 1;
  // launched with programmatic stream serialization: the kernel that produced
  // this rank's gradient must have completed before the flag says so
  pdl_wait();
  __syncthreads();
  uint32_t *my_pad = a.signal_pads[a.rank];
  if (blockIdx.x == 0) {
    // 1 + 2: flags.  Thread r handles peer r.
    if (threadIdx.x < unsigned(a.world) && int(threadIdx.x) != a.rank) {
      const int peer = int(threadIdx.x);
      st_release_sys(a.signal_pads[peer] + a.rank, a.epoch);
      const long long start = clock64();
      while (!reached(ld_acquire_sys(my_pad + peer), a.epoch)) {
        if (clock64() - start > kWaitCycleLimit) {
          atomicCAS(a.status, kStatusOk, kStatusPeerTimeout);
          ok = 0;
          break;
        }
      }
    }
    __syncthreads();
    // release the other blocks (also after a timeout, so that they return)
    if (threadIdx.x == 0) st_release_sys(my_pad + kP2pGoSlot, ok ? a.epoch : a.epoch | 0x80000000u);
  } else {
    if (threadIdx.x == 0) {
      const long long start = clock64();
      uint32_t seen;
      while (true) {
        seen = ld_acquire_sys(my_pad + kP2pGoSlot);
        if ((seen & 0x7fffffffu) == (a.epoch & 0x7fffffffu)) break;
        if (clock64() - start > 2 * kWaitCycleLimit) {
          atomicCAS(a.status, kStatusOk, kStatusPeerTimeout);
          seen = 0x80000000u;
          break;
        }
      }
      if (seen & 0x80000000u) ok = 0;
    }
    __syncthreads();
  }
  if (!ok) return;
  // 3: sum in rank order; all of a thread's peer loads are issued before the adds
  for (size_t i = blockIdx.x * size_t(kP2pThreads) + threadIdx.x; i < a.count4;
       i += size_t(gridDim.x) * kP2pThreads) {
    float4 v[kP2pMaxWorld];
#pragma unroll
    for (int r = 0; r < kP2pMaxWorld; ++r) {
      if (r < a.world) {
        const float4 *src = reinterpret_cast<const float4 *>(a.buffers[r]) + i;
        v[r] = r == a.rank ? *src : ld_peer_f4(src);
      }
    }
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < kP2pMaxWorld; ++r) {
      if (r < a.world) {
        s.x += v[r].x;
        s.y += v[r].y;
        s.z += v[r].z;
        s.w += v[r].w;
      }
    }
    if (a.out_f32) a.out_f32[i] = s;
    if (a.out_half) {
      const __half2 lo = __floats2half2_rn(s.x, s.y), hi = __floats2half2_rn(s.z, s.w);
      a.out_half[i] = make_uint2(*reinterpret_cast<const uint32_t *>(&lo),
                                 *reinterpret_cast<const uint32_t *>(&hi));
    }
  }
}

// ---- reduce-scatter + all-gather form ------------------------------------------
// The one-shot kernel above has every rank read all N buffers: (N - 1) x the
// message over NVLink per rank.  Here rank r owns slice r of the vector:
//   1. flags, round 1: "my input is complete" to every peer; wait for theirs;
//   2. the owner reads its slice from every rank's input (peer loads), adds in
//      rank order and writes the fp32 sums into every rank's result buffer
//      (peer stores): (N - 1) / N of the message in and the same out per rank;
//   3. a counter in local memory tells the last block of this rank that all
//      of the rank's stores are fenced; that block sends flags, round 2: "my
//      slice is in your result buffer", waits for the peers' and releases the
//      rank's other blocks;
//   4. every rank reads its own result buffer, writes the fp32 sum and / or
//      its cast.
// Each sum is formed once, by its owner, in rank order: all ranks end up with
// identical bits, the same bits as the one-shot kernel's.  Flag round 2 also
// tells a rank that every peer has finished reading its input of this step,
// and round 1 of the next step that every peer has consumed its results.
// Words of a rank's signal pad used here (disjoint from the one-shot kernel's):
constexpr int kRsFlag1 = 32;                  // [32 + r]: rank r's input of `epoch` is complete
constexpr int kRsFlag2 = 32 + kP2pMaxWorld;   // [48 + r]: rank r's slice of `epoch` is stored here
constexpr int kRsGo1 = 32 + 2 * kP2pMaxWorld;  // block 0 -> the rank's other blocks
constexpr int kRsGo2 = kRsGo1 + 1;             // last block -> the rank's other blocks
constexpr int kRsCounter = kRsGo1 + 2;         // blocks of this rank that finished step 2
constexpr int kRsWords = kRsGo1 + 3;
constexpr int kRsThreads = 128;

struct P2pRsArgs {
  const float *inputs[kP2pMaxWorld];    // every rank's gradient
  float *results[kP2pMaxWorld];         // every rank's result buffer (same size)
  uint32_t *signal_pads[kP2pMaxWorld];
  int rank, world;
  uint32_t epoch;
  size_t count4;   // float4 elements of the vector
  size_t slice4;   // float4 elements per owner (the last slice may be shorter)
  float4 *out_f32;
  uint2 *out_half;
  int *status;
};

__device__ __forceinline__ void st_peer_f4(float4 *p, const float4 v) {
  asm volatile("st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(v.x), "f"(v.y),
               "f"(v.z), "f"(v.w)
               : "memory");
}

// bounded wait for `word` to reach `epoch`; false (and the status word set) when it does not.
// A set top bit means "the sender gave up".
__device__ __forceinline__ bool wait_word(const uint32_t *word, uint32_t epoch, int *status,
                                          long long budget) {
  const long long start = clock64();
  while (true) {
    const uint32_t seen = ld_acquire_sys(word);
    if ((seen & 0x7fffffffu) == (epoch & 0x7fffffffu) || reached(seen & 0x7fffffffu, epoch))
      return (seen & 0x80000000u) == 0;
    if (clock64() - start > budget) {
      atomicCAS(status, kStatusOk, kStatusPeerTimeout);
      return false;
    }
  }
}

__global__ void __launch_bounds__(kRsThreads)
p2pReduceScatterAllGatherKernel(const P2pRsArgs a) {
  __shared__ int ok;
  __shared__ int last;
  if (threadIdx.x == 0) ok = 1;
  // the kernel that produced this rank's gradient must have completed before
  // the flag says so
  pdl_wait();
  __syncthreads();
  uint32_t *my_pad = a.signal_pads[a.rank];
  // ---- 1: input-complete flags --------------------------------------------------
  if (blockIdx.x == 0) {
    if (threadIdx.x < unsigned(a.world) && int(threadIdx.x) != a.rank) {
      const int peer = int(threadIdx.x);
      st_release_sys(a.signal_pads[peer] + kRsFlag1 + a.rank, a.epoch);
      if (!wait_word(my_pad + kRsFlag1 + peer, a.epoch, a.status, kWaitCycleLimit)) ok = 0;
    }
    __syncthreads();
    if (threadIdx.x == 0) st_release_sys(my_pad + kRsGo1, ok ? a.epoch : a.epoch | 0x80000000u);
  } else {
    if (threadIdx.x == 0 && !wait_word(my_pad + kRsGo1, a.epoch, a.status, 2 * kWaitCycleLimit))
      ok = 0;
    __syncthreads();
  }
  // ---- 2: this rank's slice: sum in rank order, store to every rank ---------------
  if (ok) {
    const size_t begin = min(a.count4, size_t(a.rank) * a.slice4);
    const size_t end = min(a.count4, begin + a.slice4);
    for (size_t i = begin + blockIdx.x * size_t(kRsThreads) + threadIdx.x; i < end;
         i += size_t(gridDim.x) * kRsThreads) {
      float4 v[kP2pMaxWorld];
#pragma unroll
      for (int r = 0; r < kP2pMaxWorld; ++r) {
        if (r < a.world) {
          const float4 *src = reinterpret_cast<const float4 *>(a.inputs[r]) + i;
          v[r] = r == a.rank ? *src : ld_peer_f4(src);
        }
      }
      float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int r = 0; r < kP2pMaxWorld; ++r) {
        if (r < a.world) {
          s.x += v[r].x;
          s.y += v[r].y;
          s.z += v[r].z;
          s.w += v[r].w;
        }
      }
#pragma unroll
      for (int r = 0; r < kP2pMaxWorld; ++r)
        if (r < a.world) st_peer_f4(reinterpret_cast<float4 *>(a.results[r]) + i, s);
    }
  }
  // ---- 3: all of this rank's stores fenced -> result flags ------------------------
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(my_pad + kRsCounter, 1u);
    last = prev == gridDim.x - 1 ? 1 : 0;
    if (last) atomicExch(my_pad + kRsCounter, 0u);  // for the next call
  }
  __syncthreads();
  if (last) {
    __threadfence_system();
    if (threadIdx.x < unsigned(a.world) && int(threadIdx.x) != a.rank) {
      const int peer = int(threadIdx.x);
      st_release_sys(a.signal_pads[peer] + kRsFlag2 + a.rank, ok ? a.epoch : a.epoch | 0x80000000u);
      if (!wait_word(my_pad + kRsFlag2 + peer, a.epoch, a.status, kWaitCycleLimit)) ok = 0;
    }
    __syncthreads();
    if (threadIdx.x == 0) st_release_sys(my_pad + kRsGo2, ok ? a.epoch : a.epoch | 0x80000000u);
  } else {
    if (threadIdx.x == 0 && !wait_word(my_pad + kRsGo2, a.epoch, a.status, 3 * kWaitCycleLimit))
      ok = 0;
    __syncthreads();
  }
  if (!ok) return;
  // ---- 4: the whole vector from this rank's result buffer ----------------------------
  const float4 *res = reinterpret_cast<const float4 *>(a.results[a.rank]);
  for (size_t i = blockIdx.x * size_t(kRsThreads) + threadIdx.x; i < a.count4;
       i += size_t(gridDim.x) * kRsThreads) {
    const float4 s = ld_peer_f4(res + i);  // written by peers: not from a stale cache line
    if (a.out_f32) a.out_f32[i] = s;
    if (a.out_half) {
      const __half2 lo = __floats2half2_rn(s.x, s.y), hi = __floats2half2_rn(s.z, s.w);
      a.out_half[i] = make_uint2(*reinterpret_cast<const uint32_t *>(&lo),
                                 *reinterpret_cast<const uint32_t *>(&hi));
    }
  }
}

}  // namespace
}  // namespace plb

using namespace plb;

extern "C" int plb_allreduce_f32_p2p(plb_context *ctx, int32_t rank, int32_t world,
                                     const void *const *d_buffers, void *const *d_signal_pads,
                                     uint32_t epoch, size_t count, float *d_out_f32,
                                     void *d_out_half) {
  if (int rc = activate(ctx)) return rc;
  if (world < 1 || world > kP2pMaxWorld || rank < 0 || rank >= world)
    return fail(PLB_ERR_INVALID_PARAMS, "rank / world size out of range (at most " +
                                            std::to_string(kP2pMaxWorld) + " ranks)");
  if (!d_buffers || !d_signal_pads) return fail(PLB_ERR_INVALID_PARAMS, "null pointer table");
  if (count % 4 != 0) return fail(PLB_ERR_INVALID_PARAMS, "element count must be a multiple of 4");
  if (epoch == 0) return fail(PLB_ERR_INVALID_PARAMS, "epochs start at 1 (pads are zero-initialised)");
  if (count == 0) return PLB_OK;
  P2pArgs a{};
  for (int r = 0; r < world; ++r) {
    if (!d_buffers[r] || !d_signal_pads[r]) return fail(PLB_ERR_INVALID_PARAMS, "null peer pointer");
    if ((reinterpret_cast<uintptr_t>(d_buffers[r]) & 15) != 0)
      return fail(PLB_ERR_INVALID_PARAMS, "peer buffers must be 16-byte aligned");
    a.buffers[r] = static_cast<const float *>(d_buffers[r]);
    a.signal_pads[r] = static_cast<uint32_t *>(d_signal_pads[r]);
  }
  if ((reinterpret_cast<uintptr_t>(d_out_f32) & 15) != 0 ||
      (reinterpret_cast<uintptr_t>(d_out_half) & 7) != 0)
    return fail(PLB_ERR_INVALID_PARAMS, "outputs must be 16-byte (fp32) / 8-byte (half) aligned");
  a.rank = rank;
  a.world = world;
  a.epoch = epoch;
  a.count4 = count / 4;
  a.out_f32 = reinterpret_cast<float4 *>(d_out_f32);
  a.out_half = static_cast<uint2 *>(d_out_half);
  a.status = ctx->d_status;
  if (epoch & 0x80000000u) return fail(PLB_ERR_INVALID_PARAMS, "epoch must be below 2^31");
  // one thread per 16 bytes, at most two blocks' worth per SM: block 0 (always
  // among the first scheduled) exchanges the flags, the others wait for it
  const size_t want = (a.count4 + kP2pThreads - 1) / kP2pThreads;
  const unsigned blocks = unsigned(std::max<size_t>(1, std::min<size_t>(want, size_t(ctx->sm_count) * 2)));
  // the launch overlaps the tail of the kernel that writes this rank's gradient
  cudaLaunchAttribute pdl[1];
  pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  pdl[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(blocks);
  cfg.blockDim = dim3(kP2pThreads);
  cfg.stream = ctx->stream;
  cfg.attrs = pdl;
  cfg.numAttrs = 1;
  PLB_CUDA(cudaLaunchKernelEx(&cfg, p2pAllReduceKernel, a));
  PLB_CUDA(cudaGetLastError());
  ctx->launches++;
  return PLB_OK;
}

extern "C" int plb_allreduce_f32_p2p_rs(plb_context *ctx, int32_t rank, int32_t world,
                                        const void *const *d_inputs, void *const *d_results,
                                        void *const *d_signal_pads, uint32_t epoch, size_t count,
                                        float *d_out_f32, void *d_out_half) {
  if (int rc = activate(ctx)) return rc;
  if (world < 1 || world > kP2pMaxWorld || rank < 0 || rank >= world)
    return fail(PLB_ERR_INVALID_PARAMS, "rank / world size out of range (at most " +
                                            std::to_string(kP2pMaxWorld) + " ranks)");
  if (!d_inputs || !d_results || !d_signal_pads)
    return fail(PLB_ERR_INVALID_PARAMS, "null pointer table");
  if (count % 4 != 0) return fail(PLB_ERR_INVALID_PARAMS, "element count must be a multiple of 4");
  if (epoch == 0 || (epoch & 0x80000000u))
    return fail(PLB_ERR_INVALID_PARAMS, "epochs run from 1 to 2^31 - 1 (pads are zero-initialised)");
  if (count == 0) return PLB_OK;
  P2pRsArgs a{};
  for (int r = 0; r < world; ++r) {
    if (!d_inputs[r] || !d_results[r] || !d_signal_pads[r])
      return fail(PLB_ERR_INVALID_PARAMS, "null peer pointer");
    if (((reinterpret_cast<uintptr_t>(d_inputs[r]) | reinterpret_cast<uintptr_t>(d_results[r])) & 15) != 0)
      return fail(PLB_ERR_INVALID_PARAMS, "peer buffers must be 16-byte aligned");
    a.inputs[r] = static_cast<const float *>(d_inputs[r]);
    a.results[r] = static_cast<float *>(d_results[r]);
    a.signal_pads[r] = static_cast<uint32_t *>(d_signal_pads[r]);
  }
  if ((reinterpret_cast<uintptr_t>(d_out_f32) & 15) != 0 ||
      (reinterpret_cast<uintptr_t>(d_out_half) & 7) != 0)
    return fail(PLB_ERR_INVALID_PARAMS, "outputs must be 16-byte (fp32) / 8-byte (half) aligned");
  a.rank = rank;
  a.world = world;
  a.epoch = epoch;
  a.count4 = count / 4;
  a.slice4 = (a.count4 + size_t(world) - 1) / size_t(world);
  a.out_f32 = reinterpret_cast<float4 *>(d_out_f32);
  a.out_half = static_cast<uint2 *>(d_out_half);
  a.status = ctx->d_status;
  // All blocks of a rank wait for one another (counter, go words), so the grid
  // must be resident at once: at most one block per SM.
  const size_t want = (a.count4 + 2 * kRsThreads - 1) / (2 * kRsThreads);
  const unsigned blocks = unsigned(std::max<size_t>(1, std::min<size_t>(want, size_t(ctx->sm_count))));
  cudaLaunchAttribute pdl[1];
  pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  pdl[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(blocks);
  cfg.blockDim = dim3(kRsThreads);
  cfg.stream = ctx->stream;
  cfg.attrs = pdl;
  cfg.numAttrs = 1;
  PLB_CUDA(cudaLaunchKernelEx(&cfg, p2pReduceScatterAllGatherKernel, a));
  PLB_CUDA(cudaGetLastError());
  ctx->launches++;
  return PLB_OK;
}

extern "C" uint32_t plb_allreduce_p2p_signal_bytes(int32_t world) {
  (void)world;
  return uint32_t(kRsWords) * uint32_t(sizeof(uint32_t));
}
