// Batch normalisation after a convolution: the kernels behind poplin's Norms
// API (include/poplin/Norms.hpp:33-334, lib/poplin/Norms.cpp), on device-layout
// activations [pixels][chans] (NHWC: the channels of a pixel are contiguous),
// statistics per channel over all pixels.
//
// Every operation here moves each activation once or twice and does a handful
// of flops on it: HBM bound.  The per-channel sums are column reductions of a
// row-major matrix: a block covers 64 channels x a slab of rows, a thread
// accumulates two adjacent channels (one 4-byte load per row for half) in fp32
// down its rows, the block's eight row lanes are added in a fixed order in
// shared memory, and each block leaves one partial per channel; a second
// kernel adds the blocks' partials in block order.  The order of additions is
// fixed, so results do not depend on timing (the reference's reductions are
// deterministic too).  The element-wise kernels read their per-channel
// operands from fp32 arrays and round once, in the output type.
#include <cuda_fp16.h>

#include <algorithm>
#include <string>

#include "runtime.h"
#include "sm100_prims.cuh"

namespace plb {
namespace {

constexpr int kNormChansPerBlock = 64;   // 32 threads x 2 channels
constexpr int kNormRowLanes = 8;

template <typename T> __device__ __forceinline__ float toFloat(T v);
template <> __device__ __forceinline__ float toFloat<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float toFloat<float>(float v) { return v; }
template <typename T> __device__ __forceinline__ T fromFloat(float v);
template <> __device__ __forceinline__ __half fromFloat<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ float fromFloat<float>(float v) { return v; }

// What a column reduction adds up per channel (two sums at once).
enum NormSums : int {
  kSumXAndXX = 0,      // sum x, sum x^2
  kSumCentredXX = 1,   // -, sum (x - centre[c])^2          (centre in the activations' type)
  kSumXYAndY = 2,      // sum x * y, sum y                  (whitened activations x gradients)
};

template <typename T, int kMode>
__global__ void __launch_bounds__(32 * kNormRowLanes)
normColumnPartialsKernel(const T *__restrict__ x, const T *__restrict__ y,
                         const T *__restrict__ centre, size_t rows, int chans,
                         float *__restrict__ partial_a, float *__restrict__ partial_b) {
  pdl_launch_dependents();
  pdl_wait();  // inputs may come from the previous kernel in the stream
  __shared__ float sa[kNormRowLanes][kNormChansPerBlock], sb[kNormRowLanes][kNormChansPerBlock];
  const int c0 = blockIdx.x * kNormChansPerBlock + 2 * threadIdx.x;
  const bool ok0 = c0 < chans, ok1 = c0 + 1 < chans;
  float m0 = 0.f, m1 = 0.f;
  if (kMode == kSumCentredXX) {
    if (ok0) m0 = toFloat(centre[c0]);
    if (ok1) m1 = toFloat(centre[c0 + 1]);
  }
  float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
  for (size_t r = blockIdx.y * size_t(kNormRowLanes) + threadIdx.y; r < rows;
       r += size_t(gridDim.y) * kNormRowLanes) {
    const T *px = x + r * chans + c0;
    float x0 = ok0 ? toFloat(px[0]) : 0.f, x1 = ok1 ? toFloat(px[1]) : 0.f;
    if (kMode == kSumXAndXX) {
      a0 += x0;
      a1 += x1;
      b0 += x0 * x0;
      b1 += x1 * x1;
    } else if (kMode == kSumCentredXX) {
      // the deviation is formed in the activations' type, as the reference's
      // "acts - cast(mean)" map does (lib/poplin/Norms.cpp:216-219)
      const float d0 = toFloat(fromFloat<T>(x0 - m0)), d1 = toFloat(fromFloat<T>(x1 - m1));
      b0 += ok0 ? d0 * d0 : 0.f;
      b1 += ok1 ? d1 * d1 : 0.f;
    } else {
      const T *py = y + r * chans + c0;
      const float y0 = ok0 ? toFloat(py[0]) : 0.f, y1 = ok1 ? toFloat(py[1]) : 0.f;
      a0 += x0 * y0;
      a1 += x1 * y1;
      b0 += y0;
      b1 += y1;
    }
  }
  sa[threadIdx.y][2 * threadIdx.x] = a0;
  sa[threadIdx.y][2 * threadIdx.x + 1] = a1;
  sb[threadIdx.y][2 * threadIdx.x] = b0;
  sb[threadIdx.y][2 * threadIdx.x + 1] = b1;
  __syncthreads();
  const int t = threadIdx.y * 32 + threadIdx.x;
  if (t < kNormChansPerBlock) {
    const int c = blockIdx.x * kNormChansPerBlock + t;
    if (c < chans) {
      float ta = sa[0][t], tb = sb[0][t];
#pragma unroll
      for (int l = 1; l < kNormRowLanes; ++l) {
        ta += sa[l][t];
        tb += sb[l][t];
      }
      partial_a[size_t(blockIdx.y) * chans + c] = ta;
      partial_b[size_t(blockIdx.y) * chans + c] = tb;
    }
  }
}


// The same sums over 16-byte vectors for channel counts whose vectors per row
// divide the block size (powers of two from 8 halves / 4 floats up): thread t
// of the grid walks vectors t, t + T, t + 2T, ... of the whole [rows x chans]
// array with T a multiple of the vectors per row, so it always meets the same
// kVec channels and keeps their sums in registers.  Threads of a block that
// share a channel group are added in thread order in shared memory.
template <typename T> struct NormVec;
template <> struct NormVec<__half> {
  static constexpr int kVec = 8;
  static __device__ __forceinline__ void load(const __half *p, float (&f)[8]) {
    const uint4 v = *reinterpret_cast<const uint4 *>(p);
    const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 t = __half22float2(h[j]);
      f[2 * j] = t.x;
      f[2 * j + 1] = t.y;
    }
  }
  static __device__ __forceinline__ void store(__half *p, const float (&f)[8]) {
    uint4 v;
    __half2 *h = reinterpret_cast<__half2 *>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __floats2half2_rn(f[2 * j], f[2 * j + 1]);
    *reinterpret_cast<uint4 *>(p) = v;
  }
};
template <> struct NormVec<float> {
  static constexpr int kVec = 4;
  static __device__ __forceinline__ void load(const float *p, float (&f)[4]) {
    const float4 v = *reinterpret_cast<const float4 *>(p);
    f[0] = v.x;
    f[1] = v.y;
    f[2] = v.z;
    f[3] = v.w;
  }
  static __device__ __forceinline__ void store(float *p, const float (&f)[4]) {
    *reinterpret_cast<float4 *>(p) = make_float4(f[0], f[1], f[2], f[3]);
  }
};

constexpr int kNormVecThreads = 256;

template <typename T, int kMode>
__global__ void __launch_bounds__(kNormVecThreads)
normColumnPartialsVecKernel(const T *__restrict__ x, const T *__restrict__ y,
                            const T *__restrict__ centre, size_t vectors, int chans,
                            float *__restrict__ partial_a, float *__restrict__ partial_b) {
  pdl_launch_dependents();
  pdl_wait();  // inputs may come from the previous kernel in the stream
  constexpr int kVec = NormVec<T>::kVec;
  extern __shared__ float red[];   // [2][kNormVecThreads][kVec]
  const int per_row = chans / kVec;              // divides kNormVecThreads
  const int group = threadIdx.x % per_row;       // this thread's channels: [group * kVec, +kVec)
  float m[kVec], a[kVec], b[kVec];
#pragma unroll
  for (int j = 0; j < kVec; ++j) a[j] = b[j] = m[j] = 0.f;
  if (kMode == kSumCentredXX) NormVec<T>::load(centre + group * kVec, m);
  for (size_t v = blockIdx.x * size_t(kNormVecThreads) + threadIdx.x; v < vectors;
       v += size_t(gridDim.x) * kNormVecThreads) {
    float xv[kVec];
    NormVec<T>::load(x + v * kVec, xv);
    if (kMode == kSumXAndXX) {
#pragma unroll
      for (int j = 0; j < kVec; ++j) {
        a[j] += xv[j];
        b[j] += xv[j] * xv[j];
      }
    } else if (kMode == kSumCentredXX) {
#pragma unroll
      for (int j = 0; j < kVec; ++j) {
        const float d = toFloat(fromFloat<T>(xv[j] - m[j]));
        b[j] += d * d;
      }
    } else {
      float yv[kVec];
      NormVec<T>::load(y + v * kVec, yv);
#pragma unroll
      for (int j = 0; j < kVec; ++j) {
        a[j] += xv[j] * yv[j];
        b[j] += yv[j];
      }
    }
  }
  float *ra = red, *rb = red + kNormVecThreads * kVec;
#pragma unroll
  for (int j = 0; j < kVec; ++j) {
    ra[threadIdx.x * kVec + j] = a[j];
    rb[threadIdx.x * kVec + j] = b[j];
  }
  __syncthreads();
  // thread c < chans adds channel c over the block's threads that share its group, in thread order
  for (int c = threadIdx.x; c < chans; c += kNormVecThreads) {
    const int g = c / kVec, j = c - g * kVec;
    float ta = 0.f, tb = 0.f;
    for (int t = g; t < kNormVecThreads; t += per_row) {
      ta += ra[t * kVec + j];
      tb += rb[t * kVec + j];
    }
    partial_a[size_t(blockIdx.x) * chans + c] = ta;
    partial_b[size_t(blockIdx.x) * chans + c] = tb;
  }
}

// Sums over the blocks' partials, times `scale`: a warp per channel, lane l
// adds blocks l, l + 32, ... in order, then the lanes' sums are added by a
// fixed tree of shuffles (the order of additions never depends on timing).
template <typename TA, typename TB>
__global__ void __launch_bounds__(256)
normColumnFinishKernel(const float *__restrict__ partial_a, const float *__restrict__ partial_b,
                       int blocks, int chans, float scale, TA *__restrict__ out_a,
                       TB *__restrict__ out_b, TA *__restrict__ inv_std, float eps, float scale_var) {
  pdl_launch_dependents();
  pdl_wait();  // inputs may come from the previous kernel in the stream
  const int c = blockIdx.x * 8 + threadIdx.y;
  if (c >= chans) return;   // (whole warps leave together)
  float a = 0.f, b = 0.f;
  for (int k = threadIdx.x; k < blocks; k += 32) {
    a += partial_a[size_t(k) * chans + c];
    b += partial_b[size_t(k) * chans + c];
  }
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) {
    a += __shfl_xor_sync(0xffffffffu, a, d);
    b += __shfl_xor_sync(0xffffffffu, b, d);
  }
  if (threadIdx.x == 0) {
    const float mean = __fmul_rn(a, scale), power = __fmul_rn(b, scale);
    if (out_a) out_a[c] = fromFloat<TA>(mean);
    if (out_b) out_b[c] = fromFloat<TB>(power);
    if (inv_std) {
      // normInvStdDevKernel's arithmetic on the values as stored: the mean
      // rounded to its type, the power in fp32
      const float m = toFloat(fromFloat<TA>(mean));
      float var = power - m * m;
      if (var < 0.f) var = 0.f;
      var = (var + eps) * scale_var;
      inv_std[c] = fromFloat<TA>(1.0f / sqrtf(var));
    }
  }
}

// iStdDev from mean and power: the reference's InverseStdDeviation vertex
// (lib/poplin/codelets/InverseStdDeviation.cpp:33-55), in fp32.
template <typename T>
__global__ void normInvStdDevKernel(const T *__restrict__ mean, const float *__restrict__ power,
                                    int chans, float eps, float scale_var, int stable,
                                    T *__restrict__ inv_std) {
  pdl_launch_dependents();
  pdl_wait();  // inputs may come from the previous kernel in the stream
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= chans) return;
  float var;
  if (stable) {
    var = (power[c] + eps) * scale_var;
  } else {
    const float m = toFloat(mean[c]);
    var = power[c] - m * m;
    if (var < 0.f) var = 0.f;   // rounding can make the estimate negative
    var = (var + eps) * scale_var;
  }
  inv_std[c] = fromFloat<T>(1.0f / sqrtf(var));
}

// Element-wise forms, one thread per element, channel = index mod chans.
enum NormMap : int {
  kWhiten = 0,          // (x - p[c]) * q[c]
  kScaleShift = 1,      // x * p[c] + q[c]
  kScale = 2,           // x * p[c]
  kStatsGrad = 3,       // (y + x * p[c] + q[c]) * r[c]     x = whitened, y = gradient
};

template <typename T, int kMode>
__global__ void normMapKernel(const T *__restrict__ x, const T *__restrict__ y,
                              const T *__restrict__ p, const T *__restrict__ q,
                              const T *__restrict__ r, const float *__restrict__ pf,
                              const float *__restrict__ qf, size_t count, int chans,
                              T *__restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();  // inputs may come from the previous kernel in the stream
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < count;
       i += size_t(gridDim.x) * blockDim.x) {
    const int c = int(i % size_t(chans));
    const float v = toFloat(x[i]);
    float o;
    if (kMode == kWhiten)
      o = (v - toFloat(p[c])) * toFloat(q[c]);
    else if (kMode == kScaleShift)
      o = v * toFloat(p[c]) + toFloat(q[c]);
    else if (kMode == kScale)
      o = v * toFloat(p[c]);
    else
      o = (toFloat(y[i]) + v * (pf ? pf[c] : toFloat(p[c])) + (qf ? qf[c] : toFloat(q[c]))) * toFloat(r[c]);
    out[i] = fromFloat<T>(o);
  }
}

// The element-wise forms over 16-byte vectors (channel count a multiple of the
// vector length, all pointers 16-byte aligned).
template <typename T, int kMode>
__global__ void normMapVecKernel(const T *__restrict__ x, const T *__restrict__ y,
                                 const T *__restrict__ p, const T *__restrict__ q,
                                 const T *__restrict__ r, const float *__restrict__ pf,
                                 const float *__restrict__ qf, size_t vectors, int chans,
                                 T *__restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();  // inputs may come from the previous kernel in the stream
  constexpr int kVec = NormVec<T>::kVec;
  const int per_row = chans / kVec;
  for (size_t v = blockIdx.x * size_t(blockDim.x) + threadIdx.x; v < vectors;
       v += size_t(gridDim.x) * blockDim.x) {
    const int c0 = int(v % size_t(per_row)) * kVec;
    float xv[kVec], yv[kVec], pv[kVec], qv[kVec], rv[kVec], o[kVec];
    NormVec<T>::load(x + v * kVec, xv);
    if (kMode == kStatsGrad) {
      NormVec<T>::load(y + v * kVec, yv);
      NormVec<T>::load(r + c0, rv);
      if (pf) {
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
          pv[j] = pf[c0 + j];
          qv[j] = qf[c0 + j];
        }
      } else {
        NormVec<T>::load(p + c0, pv);
        NormVec<T>::load(q + c0, qv);
      }
    } else {
      NormVec<T>::load(p + c0, pv);
      if (kMode != kScale) NormVec<T>::load(q + c0, qv);
    }
#pragma unroll
    for (int j = 0; j < kVec; ++j) {
      if (kMode == kWhiten)
        o[j] = (xv[j] - pv[j]) * qv[j];
      else if (kMode == kScaleShift)
        o[j] = xv[j] * pv[j] + qv[j];
      else if (kMode == kScale)
        o[j] = xv[j] * pv[j];
      else
        o[j] = (yv[j] + xv[j] * pv[j] + qv[j]) * rv[j];
    }
    NormVec<T>::store(out + v * kVec, o);
  }
}

// Whiten, then scale and shift, in one pass: the whitened value is rounded to
// the activations' type (and stored, if asked for) before it is scaled, so both
// outputs are the bits that normMapVecKernel<kWhiten> followed by
// normMapVecKernel<kScaleShift> leave.
template <typename T>
__global__ void normNormaliseVecKernel(const T *__restrict__ x, const T *__restrict__ mean,
                                       const T *__restrict__ inv_std, const T *__restrict__ gamma,
                                       const T *__restrict__ beta, size_t vectors, int chans,
                                       T *__restrict__ whitened, T *__restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();  // inputs may come from the previous kernel in the stream
  constexpr int kVec = NormVec<T>::kVec;
  const int per_row = chans / kVec;
  for (size_t v = blockIdx.x * size_t(blockDim.x) + threadIdx.x; v < vectors;
       v += size_t(gridDim.x) * blockDim.x) {
    const int c0 = int(v % size_t(per_row)) * kVec;
    float xv[kVec], mv[kVec], sv[kVec], gv[kVec], bv[kVec], w[kVec], o[kVec];
    NormVec<T>::load(x + v * kVec, xv);
    NormVec<T>::load(mean + c0, mv);
    NormVec<T>::load(inv_std + c0, sv);
    NormVec<T>::load(gamma + c0, gv);
    NormVec<T>::load(beta + c0, bv);
#pragma unroll
    for (int j = 0; j < kVec; ++j) {
      w[j] = toFloat(fromFloat<T>((xv[j] - mv[j]) * sv[j]));
      o[j] = w[j] * gv[j] + bv[j];
    }
    if (whitened) NormVec<T>::store(whitened + v * kVec, w);
    NormVec<T>::store(out + v * kVec, o);
  }
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Launch with programmatic stream serialization: the kernel may become
// resident while its predecessor drains; it waits before touching memory.
template <typename... KArgs, typename... Args>
int launchPdl(plb_context *ctx, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, Args... args) {
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cfg.attrs = attr;
  cfg.numAttrs = (ctx->plan_flags & PLB_PLAN_NO_PDL) ? 0 : 1;
  PLB_CUDA(cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...));
  PLB_CUDA(cudaGetLastError());
  ctx->launches++;
  return PLB_OK;
}

int rowBlocks(const plb_context *ctx, size_t rows, int chans) {
  const int chan_blocks = (chans + kNormChansPerBlock - 1) / kNormChansPerBlock;
  const size_t want = (rows + 4 * kNormRowLanes - 1) / (4 * kNormRowLanes);   // >= 4 rows per thread
  const size_t cap = std::max<size_t>(1, size_t(ctx->sm_count) * 8 / size_t(chan_blocks));
  return int(std::max<size_t>(1, std::min(want, cap)));
}

// Column sums of mode kMode -> out_a, out_b (either may be null), times scale.
template <typename T, int kMode, typename TA, typename TB>
int columnSums(plb_context *ctx, const T *x, const T *y, const T *centre, size_t rows, int chans,
               float scale, TA *out_a, TB *out_b, TA *inv_std = nullptr, float eps = 0.f,
               float scale_var = 1.f) {
  constexpr int kVec = NormVec<T>::kVec;
  const bool vec = chans % kVec == 0 && kNormVecThreads % (chans / kVec) == 0 && aligned16(x) &&
                   (y == nullptr || aligned16(y)) && (centre == nullptr || aligned16(centre));
  int blocks;
  float *pa, *pb;
  void *ws = nullptr;
  if (vec) {
    const size_t vectors = rows * size_t(chans / kVec);
    blocks = int(std::max<size_t>(1, std::min<size_t>((vectors + 4 * kNormVecThreads - 1) / (4 * kNormVecThreads),
                                                      size_t(ctx->sm_count) * 2)));
    if (int rc = scratch(ctx, kSlotBiasUpdate, size_t(2) * blocks * chans * sizeof(float), &ws)) return rc;
    pa = static_cast<float *>(ws);
    pb = pa + size_t(blocks) * chans;
    if (int rc = launchPdl(ctx, normColumnPartialsVecKernel<T, kMode>, dim3(unsigned(blocks)),
                           dim3(kNormVecThreads), 2 * kNormVecThreads * kVec * sizeof(float), x, y, centre,
                           vectors, chans, pa, pb))
      return rc;
  } else {
    blocks = rowBlocks(ctx, rows, chans);
    if (int rc = scratch(ctx, kSlotBiasUpdate, size_t(2) * blocks * chans * sizeof(float), &ws)) return rc;
    pa = static_cast<float *>(ws);
    pb = pa + size_t(blocks) * chans;
    const dim3 grid(unsigned((chans + kNormChansPerBlock - 1) / kNormChansPerBlock), unsigned(blocks));
    if (int rc = launchPdl(ctx, normColumnPartialsKernel<T, kMode>, grid, dim3(32, kNormRowLanes), 0, x, y,
                           centre, rows, chans, pa, pb))
      return rc;
  }
  return launchPdl(ctx, normColumnFinishKernel<TA, TB>, dim3(unsigned((chans + 7) / 8)), dim3(32, 8), 0,
                   (const float *)pa, (const float *)pb, blocks, chans, scale, out_a, out_b, inv_std, eps,
                   scale_var);
}

template <typename T, int kMode>
int mapLaunch(plb_context *ctx, const T *x, const T *y, const T *p, const T *q, const T *r,
              const float *pf, const float *qf, size_t count, int chans, T *out) {
  if (count == 0) return PLB_OK;
  constexpr int kVec = NormVec<T>::kVec;
  if (chans % kVec == 0 && aligned16(x) && aligned16(out) && (y == nullptr || aligned16(y)) &&
      (p == nullptr || aligned16(p)) && (q == nullptr || aligned16(q)) && (r == nullptr || aligned16(r))) {
    const size_t vectors = count / kVec;
    const int grid = int(std::min<size_t>((vectors + 255) / 256, size_t(ctx->sm_count) * 16));
    return launchPdl(ctx, normMapVecKernel<T, kMode>, dim3(unsigned(grid)), dim3(256), 0, x, y, p, q, r, pf, qf,
                     vectors, chans, out);
  }
  const int grid = int(std::min<size_t>((count + 255) / 256, size_t(ctx->sm_count) * 16));
  return launchPdl(ctx, normMapKernel<T, kMode>, dim3(unsigned(grid)), dim3(256), 0, x, y, p, q, r, pf, qf, count,
                   chans, out);
}

template <typename T>
int normaliseFused(plb_context *ctx, const T *x, const T *mean, const T *inv, const T *gamma,
                          const T *beta, uint64_t pixels, uint32_t chans, T *whitened, T *out) {
  constexpr int kVec = NormVec<T>::kVec;
  const size_t n = size_t(pixels) * chans;
  if (n == 0) return PLB_OK;
  if (chans % kVec == 0 && aligned16(x) && aligned16(out) && aligned16(mean) && aligned16(inv) &&
      aligned16(gamma) && aligned16(beta) && (whitened == nullptr || aligned16(whitened))) {
    const size_t vectors = n / kVec;
    const int grid = int(std::min<size_t>((vectors + 255) / 256, size_t(ctx->sm_count) * 16));
    return launchPdl(ctx, normNormaliseVecKernel<T>, dim3(unsigned(grid)), dim3(256), 0, x, mean, inv, gamma,
                     beta, vectors, int(chans), whitened, out);
  }
  return -1;   // not vectorisable: the caller takes the two-pass route
}

int checkNorm(int32_t dtype, uint64_t pixels, uint32_t chans) {
  if (dtype != PLB_HALF && dtype != PLB_FLOAT)
    return fail(PLB_ERR_UNSUPPORTED, "normalisation is implemented for half and float activations");
  if (chans == 0 || chans > (1u << 30) || pixels > (uint64_t(1) << 40))
    return fail(PLB_ERR_INVALID_PARAMS, "normalisation: channel or pixel count out of range");
  return PLB_OK;
}

}  // namespace
}  // namespace plb

using namespace plb;

#define PLB_NORM_DISPATCH(dtype, CALL_HALF, CALL_FLOAT) \
  ((dtype) == PLB_HALF ? (CALL_HALF) : (CALL_FLOAT))

extern "C" {

int plb_norm_moments(plb_context *ctx, int32_t dtype, const void *d_acts, uint64_t pixels,
                     uint32_t chans, float scale, const void *d_centre, void *d_mean,
                     float *d_power) {
  TraceRange trace_range("plb_norm_moments");
  if (int rc = activate(ctx)) return rc;
  if (int rc = checkNorm(dtype, pixels, chans)) return rc;
  if (!d_acts && pixels) return fail(PLB_ERR_INVALID_PARAMS, "null activations");
  if (d_centre) {
    // mean of squared deviations from a given centre (the "stable" estimator)
    return PLB_NORM_DISPATCH(
        dtype,
        (columnSums<__half, kSumCentredXX, __half, float>(
            ctx, static_cast<const __half *>(d_acts), nullptr, static_cast<const __half *>(d_centre),
            pixels, int(chans), scale, nullptr, d_power)),
        (columnSums<float, kSumCentredXX, float, float>(
            ctx, static_cast<const float *>(d_acts), nullptr, static_cast<const float *>(d_centre),
            pixels, int(chans), scale, nullptr, d_power)));
  }
  return PLB_NORM_DISPATCH(
      dtype,
      (columnSums<__half, kSumXAndXX, __half, float>(ctx, static_cast<const __half *>(d_acts), nullptr,
                                                     nullptr, pixels, int(chans), scale,
                                                     static_cast<__half *>(d_mean), d_power)),
      (columnSums<float, kSumXAndXX, float, float>(ctx, static_cast<const float *>(d_acts), nullptr,
                                                   nullptr, pixels, int(chans), scale,
                                                   static_cast<float *>(d_mean), d_power)));
}

int plb_norm_statistics(plb_context *ctx, int32_t dtype, const void *d_acts, uint64_t pixels,
                        uint32_t chans, float eps, float scale_var, void *d_mean, void *d_inv_std,
                        float *d_power) {
  TraceRange trace_range("plb_norm_statistics");
  if (int rc = activate(ctx)) return rc;
  if (int rc = checkNorm(dtype, pixels, chans)) return rc;
  if ((!d_acts && pixels) || !d_mean || !d_inv_std)
    return fail(PLB_ERR_INVALID_PARAMS, "normalisation: null pointer");
  const float scale = pixels > 0 ? 1.0f / float(pixels) : 1.0f;
  return PLB_NORM_DISPATCH(
      dtype,
      (columnSums<__half, kSumXAndXX, __half, float>(ctx, static_cast<const __half *>(d_acts), nullptr,
                                                     nullptr, pixels, int(chans), scale,
                                                     static_cast<__half *>(d_mean), d_power,
                                                     static_cast<__half *>(d_inv_std), eps, scale_var)),
      (columnSums<float, kSumXAndXX, float, float>(ctx, static_cast<const float *>(d_acts), nullptr,
                                                   nullptr, pixels, int(chans), scale,
                                                   static_cast<float *>(d_mean), d_power,
                                                   static_cast<float *>(d_inv_std), eps, scale_var)));
}

int plb_norm_normalise(plb_context *ctx, int32_t dtype, const void *d_acts, const void *d_mean,
                       const void *d_inv_std, const void *d_gamma, const void *d_beta, uint64_t pixels,
                       uint32_t chans, void *d_whitened, void *d_out) {
  TraceRange trace_range("plb_norm_normalise");
  if (int rc = activate(ctx)) return rc;
  if (int rc = checkNorm(dtype, pixels, chans)) return rc;
  if (!d_mean || !d_inv_std || !d_gamma || !d_beta || ((!d_acts || !d_out) && pixels))
    return fail(PLB_ERR_INVALID_PARAMS, "normalisation: null pointer");
  const int rc = PLB_NORM_DISPATCH(
      dtype,
      (normaliseFused<__half>(ctx, static_cast<const __half *>(d_acts), static_cast<const __half *>(d_mean),
                              static_cast<const __half *>(d_inv_std), static_cast<const __half *>(d_gamma),
                              static_cast<const __half *>(d_beta), pixels, chans,
                              static_cast<__half *>(d_whitened), static_cast<__half *>(d_out))),
      (normaliseFused<float>(ctx, static_cast<const float *>(d_acts), static_cast<const float *>(d_mean),
                             static_cast<const float *>(d_inv_std), static_cast<const float *>(d_gamma),
                             static_cast<const float *>(d_beta), pixels, chans,
                             static_cast<float *>(d_whitened), static_cast<float *>(d_out))));
  if (rc != -1) return rc;
  // channel counts or addresses the vector kernel cannot take: whiten (into the
  // output if the whitened activations are not wanted), then scale and shift
  void *w = d_whitened ? d_whitened : d_out;
  if (int rc2 = plb_norm_whiten(ctx, dtype, d_acts, d_mean, d_inv_std, pixels, chans, w)) return rc2;
  return plb_norm_scale_shift(ctx, dtype, w, d_gamma, d_beta, pixels, chans, d_out);
}

int plb_norm_inv_std_dev(plb_context *ctx, int32_t dtype, const void *d_mean, const float *d_power,
                         uint32_t chans, float eps, float scale_var, int stable, void *d_inv_std) {
  if (int rc = activate(ctx)) return rc;
  if (int rc = checkNorm(dtype, 0, chans)) return rc;
  if (!d_power || !d_inv_std || (!stable && !d_mean))
    return fail(PLB_ERR_INVALID_PARAMS, "normalisation: null statistics pointer");
  const dim3 grid(unsigned((chans + 127) / 128));
  if (dtype == PLB_HALF)
    return launchPdl(ctx, normInvStdDevKernel<__half>, grid, dim3(128), 0, static_cast<const __half *>(d_mean),
                     d_power, int(chans), eps, scale_var, stable, static_cast<__half *>(d_inv_std));
  return launchPdl(ctx, normInvStdDevKernel<float>, grid, dim3(128), 0, static_cast<const float *>(d_mean),
                   d_power, int(chans), eps, scale_var, stable, static_cast<float *>(d_inv_std));
}

int plb_norm_whiten(plb_context *ctx, int32_t dtype, const void *d_acts, const void *d_mean,
                    const void *d_inv_std, uint64_t pixels, uint32_t chans, void *d_out) {
  TraceRange trace_range("plb_norm_whiten");
  if (int rc = activate(ctx)) return rc;
  if (int rc = checkNorm(dtype, pixels, chans)) return rc;
  const size_t n = size_t(pixels) * chans;
  return PLB_NORM_DISPATCH(
      dtype,
      (mapLaunch<__half, kWhiten>(ctx, static_cast<const __half *>(d_acts), nullptr,
                                  static_cast<const __half *>(d_mean),
                                  static_cast<const __half *>(d_inv_std), nullptr, nullptr, nullptr, n,
                                  int(chans), static_cast<__half *>(d_out))),
      (mapLaunch<float, kWhiten>(ctx, static_cast<const float *>(d_acts), nullptr,
                                 static_cast<const float *>(d_mean),
                                 static_cast<const float *>(d_inv_std), nullptr, nullptr, nullptr, n,
                                 int(chans), static_cast<float *>(d_out))));
}

int plb_norm_scale_shift(plb_context *ctx, int32_t dtype, const void *d_acts, const void *d_scale,
                         const void *d_shift, uint64_t pixels, uint32_t chans, void *d_out) {
  TraceRange trace_range("plb_norm_scale_shift");
  if (int rc = activate(ctx)) return rc;
  if (int rc = checkNorm(dtype, pixels, chans)) return rc;
  const size_t n = size_t(pixels) * chans;
  if (d_shift)
    return PLB_NORM_DISPATCH(
        dtype,
        (mapLaunch<__half, kScaleShift>(ctx, static_cast<const __half *>(d_acts), nullptr,
                                        static_cast<const __half *>(d_scale),
                                        static_cast<const __half *>(d_shift), nullptr, nullptr, nullptr,
                                        n, int(chans), static_cast<__half *>(d_out))),
        (mapLaunch<float, kScaleShift>(ctx, static_cast<const float *>(d_acts), nullptr,
                                       static_cast<const float *>(d_scale),
                                       static_cast<const float *>(d_shift), nullptr, nullptr, nullptr, n,
                                       int(chans), static_cast<float *>(d_out))));
  return PLB_NORM_DISPATCH(
      dtype,
      (mapLaunch<__half, kScale>(ctx, static_cast<const __half *>(d_acts), nullptr,
                                 static_cast<const __half *>(d_scale), nullptr, nullptr, nullptr, nullptr,
                                 n, int(chans), static_cast<__half *>(d_out))),
      (mapLaunch<float, kScale>(ctx, static_cast<const float *>(d_acts), nullptr,
                                static_cast<const float *>(d_scale), nullptr, nullptr, nullptr, nullptr, n,
                                int(chans), static_cast<float *>(d_out))));
}

int plb_norm_param_gradients(plb_context *ctx, int32_t dtype, const void *d_whitened,
                             const void *d_grads, uint64_t pixels, uint32_t chans, float scale,
                             void *d_gamma_delta, void *d_beta_delta, float *d_gamma_delta_f32,
                             float *d_beta_delta_f32) {
  TraceRange trace_range("plb_norm_param_gradients");
  if (int rc = activate(ctx)) return rc;
  if (int rc = checkNorm(dtype, pixels, chans)) return rc;
  if (d_gamma_delta_f32 || d_beta_delta_f32) {
    // fp32 sums (what the statistics gradient consumes)
    if (int rc = PLB_NORM_DISPATCH(
            dtype,
            (columnSums<__half, kSumXYAndY, float, float>(
                ctx, static_cast<const __half *>(d_whitened), static_cast<const __half *>(d_grads),
                nullptr, pixels, int(chans), scale, d_gamma_delta_f32, d_beta_delta_f32)),
            (columnSums<float, kSumXYAndY, float, float>(
                ctx, static_cast<const float *>(d_whitened), static_cast<const float *>(d_grads),
                nullptr, pixels, int(chans), scale, d_gamma_delta_f32, d_beta_delta_f32))))
      return rc;
  }
  if (d_gamma_delta || d_beta_delta)
    return PLB_NORM_DISPATCH(
        dtype,
        (columnSums<__half, kSumXYAndY, __half, __half>(
            ctx, static_cast<const __half *>(d_whitened), static_cast<const __half *>(d_grads), nullptr,
            pixels, int(chans), scale, static_cast<__half *>(d_gamma_delta),
            static_cast<__half *>(d_beta_delta))),
        (columnSums<float, kSumXYAndY, float, float>(
            ctx, static_cast<const float *>(d_whitened), static_cast<const float *>(d_grads), nullptr,
            pixels, int(chans), scale, static_cast<float *>(d_gamma_delta),
            static_cast<float *>(d_beta_delta))));
  return PLB_OK;
}

int plb_norm_statistics_gradients(plb_context *ctx, int32_t dtype, const void *d_whitened,
                                  const void *d_grads, const void *d_inv_std, const void *d_var_delta,
                                  const void *d_mean_delta, uint64_t pixels, uint32_t chans,
                                  void *d_out) {
  TraceRange trace_range("plb_norm_statistics_gradients");
  if (int rc = activate(ctx)) return rc;
  if (int rc = checkNorm(dtype, pixels, chans)) return rc;
  if (pixels == 0) return PLB_OK;
  if ((d_var_delta == nullptr) != (d_mean_delta == nullptr))
    return fail(PLB_ERR_INVALID_PARAMS, "give both per-channel deltas or neither");
  if (d_var_delta) {
    // the two per-channel means come from the caller (already reduced over replicas)
    const size_t n = size_t(pixels) * chans;
    return PLB_NORM_DISPATCH(
        dtype,
        (mapLaunch<__half, kStatsGrad>(ctx, static_cast<const __half *>(d_whitened),
                                       static_cast<const __half *>(d_grads),
                                       static_cast<const __half *>(d_var_delta),
                                       static_cast<const __half *>(d_mean_delta),
                                       static_cast<const __half *>(d_inv_std), nullptr, nullptr, n,
                                       int(chans), static_cast<__half *>(d_out))),
        (mapLaunch<float, kStatsGrad>(ctx, static_cast<const float *>(d_whitened),
                                      static_cast<const float *>(d_grads),
                                      static_cast<const float *>(d_var_delta),
                                      static_cast<const float *>(d_mean_delta),
                                      static_cast<const float *>(d_inv_std), nullptr, nullptr, n,
                                      int(chans), static_cast<float *>(d_out))));
  }
  // -mean(whitened * grads) and -mean(grads) per channel, kept in fp32, then
  // out = (grads + whitened * varDelta + meanDelta) * invStdDev
  // (lib/poplin/Norms.cpp:447-512, without its split of the scale in two
  // factors, which only serves half-precision intermediates)
  void *ws = nullptr;
  if (int rc = scratch(ctx, kSlotUsedTaps, size_t(2) * chans * sizeof(float) + 256, &ws)) return rc;
  float *var_delta = static_cast<float *>(ws), *mean_delta = var_delta + chans;
  if (int rc = plb_norm_param_gradients(ctx, dtype, d_whitened, d_grads, pixels, chans,
                                        -1.0f / float(pixels), nullptr, nullptr, var_delta, mean_delta))
    return rc;
  const size_t n = size_t(pixels) * chans;
  return PLB_NORM_DISPATCH(
      dtype,
      (mapLaunch<__half, kStatsGrad>(ctx, static_cast<const __half *>(d_whitened),
                                     static_cast<const __half *>(d_grads), nullptr, nullptr,
                                     static_cast<const __half *>(d_inv_std), var_delta, mean_delta, n,
                                     int(chans), static_cast<__half *>(d_out))),
      (mapLaunch<float, kStatsGrad>(ctx, static_cast<const float *>(d_whitened),
                                    static_cast<const float *>(d_grads), nullptr, nullptr,
                                    static_cast<const float *>(d_inv_std), var_delta, mean_delta, n,
                                    int(chans), static_cast<float *>(d_out))));
}

}  // extern "C"
