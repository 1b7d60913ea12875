// Context, memory and error plumbing of the C ABI, TMA tensor-map encoding and
// the small data-movement kernels (layout changes, casts, scaled add).
#include "conv_geometry.h"
#include "runtime.h"

#include <cuda_fp16.h>
#include <cudaTypedefs.h>

#include <cstdio>
#include <cstring>
#include <mutex>

namespace plb {

static thread_local std::string g_last_error;

int fail(int code, const std::string &message) {
  g_last_error = message;
  return code;
}

int cudaFail(cudaError_t err, const char *what) {
  g_last_error = std::string("CUDA error: ") + cudaGetErrorString(err) + " in " + what;
  return err == cudaErrorMemoryAllocation ? PLB_ERR_OUT_OF_MEMORY : PLB_ERR_CUDA;
}

int activate(plb_context *ctx) {
  if (ctx == nullptr) return fail(PLB_ERR_INVALID_PARAMS, "null context");
  PLB_CUDA(cudaSetDevice(ctx->device));
  return PLB_OK;
}

int scratch(plb_context *ctx, int slot, size_t bytes, void **ptr) {
  if (slot < 0 || slot >= plb_context::kScratchSlots)
    return fail(PLB_ERR_INVALID_PARAMS, "bad scratch slot");
  if (ctx->scratch_bytes[slot] < bytes) {
    // work already enqueued may still read the old buffer
    PLB_CUDA(cudaStreamSynchronize(ctx->stream));
    if (ctx->scratch[slot]) PLB_CUDA(cudaFree(ctx->scratch[slot]));
    ctx->scratch[slot] = nullptr;
    ctx->scratch_bytes[slot] = 0;
    const size_t rounded = (bytes + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
    PLB_CUDA(cudaMalloc(&ctx->scratch[slot], rounded));
    ctx->scratch_bytes[slot] = rounded;
  }
  *ptr = ctx->scratch[slot];
  return PLB_OK;
}

int encodeTensorMap(CUtensorMap *tm, CUtensorMapDataType type, int rank, const void *base,
                    const uint64_t *dims, const uint64_t *strides_bytes, const uint32_t *box,
                    const uint32_t *elem_strides, int swizzle_bytes) {
  static PFN_cuTensorMapEncodeTiled_v12000 encode = nullptr;
  static std::once_flag once;
  static cudaError_t lookup_err = cudaSuccess;
  std::call_once(once, [] {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    lookup_err = cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &fn, 12000,
                                                  cudaEnableDefault, &qres);
    if (lookup_err == cudaSuccess && qres == cudaDriverEntryPointSuccess)
      encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
  });
  if (encode == nullptr)
    return fail(PLB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the CUDA driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0)
    return fail(PLB_ERR_UNSUPPORTED, "tensor base address must be 16-byte aligned for TMA");
  for (int i = 0; i + 1 < rank; ++i)
    if (strides_bytes[i] % 16 != 0)
      return fail(PLB_ERR_UNSUPPORTED,
                  "tensor stride of " + std::to_string(strides_bytes[i]) +
                      " bytes is not a multiple of 16 (TMA requirement)");
  cuuint64_t gdims[5], gstrides[4];
  cuuint32_t gbox[5], gestr[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    gestr[i] = elem_strides[i];
    if (i + 1 < rank) gstrides[i] = strides_bytes[i];
  }
  const CUresult res = encode(tm, type, cuuint32_t(rank), const_cast<void *>(base), gdims,
                              gstrides, gbox, gestr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                                  : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (res != CUDA_SUCCESS) {
    std::string msg = "cuTensorMapEncodeTiled failed with CUresult " + std::to_string(int(res)) +
                      " (rank " + std::to_string(rank) + ", dims";
    for (int i = 0; i < rank; ++i) msg += " " + std::to_string(dims[i]);
    msg += ", box";
    for (int i = 0; i < rank; ++i) msg += " " + std::to_string(box[i]);
    msg += ")";
    return fail(PLB_ERR_CUDA, msg);
  }
  return PLB_OK;
}

// ---------------------------------------------------------------------------
// Data-movement kernels
// ---------------------------------------------------------------------------

// Batched transpose src[b][rows][cols] -> dst[b][cols][rows] through a padded
// shared-memory tile so that both sides are coalesced.
template <typename T>
__global__ void transposeKernel(const T *__restrict__ src, T *__restrict__ dst, uint32_t rows,
                                uint32_t cols) {
  __shared__ T tile[32][33];
  const size_t batch_off = size_t(blockIdx.z) * rows * cols;
  const uint32_t c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (uint32_t i = threadIdx.y; i < 32; i += blockDim.y) {
    const uint32_t r = r0 + i, c = c0 + threadIdx.x;
    if (r < rows && c < cols) tile[i][threadIdx.x] = src[batch_off + size_t(r) * cols + c];
  }
  __syncthreads();
  for (uint32_t i = threadIdx.y; i < 32; i += blockDim.y) {
    const uint32_t c = c0 + i, r = r0 + threadIdx.x;
    if (r < rows && c < cols) dst[batch_off + size_t(c) * rows + r] = tile[threadIdx.x][i];
  }
}

static int launchTranspose(plb_context *ctx, uint32_t elem_bytes, uint64_t batch, uint64_t rows,
                           uint64_t cols, const void *src, void *dst) {
  if (batch == 0 || rows == 0 || cols == 0) return PLB_OK;
  if (rows > 0xffffffffull || cols > 0xffffffffull)
    return fail(PLB_ERR_UNSUPPORTED, "matrix too large to transpose");
  const dim3 block(32, 8);
  const uint64_t gy = (rows + 31) / 32, gx = (cols + 31) / 32;
  if (gy > 65535 || batch > 65535) {
    // fold: process batches one launch at a time / split rows
    if (gy > 65535) return fail(PLB_ERR_UNSUPPORTED, "matrix too tall to transpose");
  }
  for (uint64_t b0 = 0; b0 < batch; b0 += 65535) {
    const uint32_t nb = uint32_t(std::min<uint64_t>(65535, batch - b0));
    const dim3 grid(uint32_t(gx), uint32_t(gy), nb);
    const size_t off = size_t(b0) * rows * cols;
    switch (elem_bytes) {
      case 1:
        transposeKernel<uint8_t><<<grid, block, 0, ctx->stream>>>(
            static_cast<const uint8_t *>(src) + off, static_cast<uint8_t *>(dst) + off,
            uint32_t(rows), uint32_t(cols));
        break;
      case 2:
        transposeKernel<uint16_t><<<grid, block, 0, ctx->stream>>>(
            static_cast<const uint16_t *>(src) + off, static_cast<uint16_t *>(dst) + off,
            uint32_t(rows), uint32_t(cols));
        break;
      case 4:
        transposeKernel<uint32_t><<<grid, block, 0, ctx->stream>>>(
            static_cast<const uint32_t *>(src) + off, static_cast<uint32_t *>(dst) + off,
            uint32_t(rows), uint32_t(cols));
        break;
      default:
        return fail(PLB_ERR_INVALID_PARAMS, "element size must be 1, 2 or 4 bytes");
    }
    PLB_CUDA(cudaGetLastError());
    ctx->launches++;
  }
  return PLB_OK;
}

// [G][K][Co][Ci] -> [G][K flipped][Ci][Co]; weights are small, one element per thread.
template <typename T>
__global__ void transposeFlipKernel(const T *__restrict__ src, T *__restrict__ dst,
                                    uint32_t groups, uint32_t kelems, uint32_t co, uint32_t ci) {
  const size_t total = size_t(groups) * kelems * co * ci;
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < total;
       i += size_t(gridDim.x) * blockDim.x) {
    const uint32_t o = uint32_t(i % co);
    size_t r = i / co;
    const uint32_t c = uint32_t(r % ci);
    r /= ci;
    const uint32_t k = uint32_t(r % kelems);
    const uint32_t g = uint32_t(r / kelems);
    dst[i] = src[((size_t(g) * kelems + (kelems - 1 - k)) * co + o) * ci + c];
  }
}

template <typename T>
__global__ void castFromF32Kernel(T *__restrict__ dst, const float *__restrict__ src, size_t n);
template <>
__global__ void castFromF32Kernel<__half>(__half *__restrict__ dst, const float *__restrict__ src,
                                          size_t n) {
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n;
       i += size_t(gridDim.x) * blockDim.x)
    dst[i] = __float2half_rn(src[i]);
}
template <>
__global__ void castFromF32Kernel<float>(float *__restrict__ dst, const float *__restrict__ src,
                                         size_t n) {
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n;
       i += size_t(gridDim.x) * blockDim.x)
    dst[i] = src[i];
}

template <typename T>
__global__ void scaledAddKernel(T *__restrict__ w, const float *__restrict__ d, float scale,
                                size_t n);
template <>
__global__ void scaledAddKernel<__half>(__half *__restrict__ w, const float *__restrict__ d,
                                        float scale, size_t n) {
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n;
       i += size_t(gridDim.x) * blockDim.x)
    w[i] = __float2half_rn(__half2float(w[i]) + scale * d[i]);
}
template <>
__global__ void scaledAddKernel<float>(float *__restrict__ w, const float *__restrict__ d,
                                       float scale, size_t n) {
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n;
       i += size_t(gridDim.x) * blockDim.x)
    w[i] = w[i] + scale * d[i];
}

// out = beta * c (matrix product with an empty reduction dimension)
__global__ void scaleRowsKernel(void *out, const void *c, float beta, int out_f32, uint32_t rows,
                                uint32_t cols, long long ldo, long long ldc) {
  const size_t total = size_t(rows) * cols;
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < total;
       i += size_t(gridDim.x) * blockDim.x) {
    const size_t r = i / cols, col = i % cols;
    if (out_f32) {
      const float v = c ? beta * static_cast<const float *>(c)[r * ldc + col] : 0.f;
      static_cast<float *>(out)[r * ldo + col] = v;
    } else {
      const float v = c ? beta * __half2float(static_cast<const __half *>(c)[r * ldc + col]) : 0.f;
      static_cast<__half *>(out)[r * ldo + col] = __float2half_rn(v);
    }
  }
}

struct StridedCopyArgs {
  uint32_t rank;
  uint64_t shape[PLB_MAX_VIEW_RANK];
  long long src_strides[PLB_MAX_VIEW_RANK];
  long long dst_strides[PLB_MAX_VIEW_RANK];
};

template <typename T>
__global__ void stridedCopyKernel(const T *__restrict__ src, T *__restrict__ dst,
                                  StridedCopyArgs a, size_t total) {
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < total;
       i += size_t(gridDim.x) * blockDim.x) {
    size_t r = i;
    long long so = 0, dof = 0;
    for (int d = int(a.rank) - 1; d >= 0; --d) {
      const size_t idx = r % a.shape[d];
      r /= a.shape[d];
      so += (long long)idx * a.src_strides[d];
      dof += (long long)idx * a.dst_strides[d];
    }
    dst[dof] = src[so];
  }
}

template <typename T>
__global__ void addBiasKernel(T *acts, const T *__restrict__ biases, size_t total, uint32_t chans);
template <>
__global__ void addBiasKernel<__half>(__half *acts, const __half *__restrict__ biases, size_t total,
                                      uint32_t chans) {
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < total;
       i += size_t(gridDim.x) * blockDim.x)
    acts[i] = __float2half_rn(__half2float(acts[i]) + __half2float(biases[i % chans]));
}
template <>
__global__ void addBiasKernel<float>(float *acts, const float *__restrict__ biases, size_t total,
                                     uint32_t chans) {
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < total;
       i += size_t(gridDim.x) * blockDim.x)
    acts[i] += biases[i % chans];
}

template <typename T>
__global__ void fillKernel(T *dst, T value, size_t n) {
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n;
       i += size_t(gridDim.x) * blockDim.x)
    dst[i] = value;
}

// Column sums of a [rows][chans] matrix (device-layout activations: one row per
// pixel), first stage: block (x, y) adds the rows y, y + gridDim.y, ... of the
// 8-channel vectors it owns into fp32 and leaves one partial row per slab.
// Threads are arranged as (vector of 8 channels, row lane).
template <typename T>
__global__ void __launch_bounds__(256)
columnSumPartialKernel(const T *__restrict__ in, float *__restrict__ partial, uint64_t rows,
                       uint32_t chans, uint32_t vec_lanes) {
  constexpr int kVec = 16 / int(sizeof(T));  // elements per 16-byte load
  __shared__ float red[256 * 8];
  const uint32_t vx = threadIdx.x % vec_lanes, ry = threadIdx.x / vec_lanes;
  const uint32_t row_lanes = blockDim.x / vec_lanes;
  const uint32_t vec = blockIdx.x * vec_lanes + vx;
  const uint32_t vecs = chans / kVec;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  if (vec < vecs) {
    for (uint64_t r = uint64_t(blockIdx.y) * row_lanes + ry; r < rows;
         r += uint64_t(gridDim.y) * row_lanes) {
      const uint4 v = *reinterpret_cast<const uint4 *>(in + r * chans + size_t(vec) * kVec);
      if constexpr (sizeof(T) == 2) {
        const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __half22float2(h[j]);
          acc[2 * j] += f.x;
          acc[2 * j + 1] += f.y;
        }
      } else {
        const float *f = reinterpret_cast<const float *>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[j] += f[j];
      }
    }
  }
#pragma unroll
  for (int j = 0; j < kVec; ++j) red[threadIdx.x * 8 + j] = acc[j];
  __syncthreads();
  // row lane 0 adds the lanes in order
  if (ry == 0 && vec < vecs) {
    for (uint32_t y = 1; y < row_lanes; ++y)
#pragma unroll
      for (int j = 0; j < kVec; ++j) acc[j] += red[(y * vec_lanes + vx) * 8 + j];
#pragma unroll
    for (int j = 0; j < kVec; ++j)
      partial[size_t(blockIdx.y) * chans + size_t(vec) * kVec + j] = acc[j];
  }
}
// Generic first stage (any channel count / alignment): one thread per channel.
template <typename T>
__global__ void columnSumPartialScalarKernel(const T *__restrict__ in, float *__restrict__ partial,
                                             uint64_t rows, uint32_t chans) {
  const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= chans) return;
  float acc = 0.f;
  for (uint64_t r = blockIdx.y; r < rows; r += gridDim.y) acc += float(in[r * chans + c]);
  partial[size_t(blockIdx.y) * chans + c] = acc;
}
// Second stage: biases[c] += scale * (sum of the slabs' partial rows, in order).
template <typename T>
__global__ void biasUpdateKernel(const float *__restrict__ partial, uint32_t slabs, uint32_t chans,
                                 T *__restrict__ biases, float scale) {
  const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= chans) return;
  float s = 0.f;
  for (uint32_t k = 0; k < slabs; ++k) s += partial[size_t(k) * chans + c];
  biases[c] = T(float(biases[c]) + scale * s);
}

// Copies rows of `c_src` elements into rows of `c_dst` elements (same row
// count), zero-filling the tail when the destination rows are longer and
// dropping it when they are shorter: channel padding / un-padding.
__global__ void resizeRowsKernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst,
                                 size_t rows, uint32_t src_bytes, uint32_t dst_bytes) {
  // 2-byte granularity covers half and quarter-pairs; odd byte counts use bytes
  const size_t total = rows * dst_bytes;
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < total;
       i += size_t(gridDim.x) * blockDim.x) {
    const size_t r = i / dst_bytes;
    const uint32_t b = uint32_t(i - r * dst_bytes);
    dst[i] = b < src_bytes ? src[r * src_bytes + b] : uint8_t(0);
  }
}

int resizeRows(plb_context *ctx, const void *src, void *dst, size_t rows, size_t src_bytes,
               size_t dst_bytes) {
  if (rows == 0 || dst_bytes == 0) return PLB_OK;
  const size_t total = rows * dst_bytes;
  const int grid = int(std::min<size_t>((total + 255) / 256, size_t(ctx->sm_count) * 16));
  resizeRowsKernel<<<grid, 256, 0, ctx->stream>>>(static_cast<const uint8_t *>(src),
                                                  static_cast<uint8_t *>(dst), rows,
                                                  uint32_t(src_bytes), uint32_t(dst_bytes));
  PLB_CUDA(cudaGetLastError());
  ctx->launches++;
  return PLB_OK;
}

// The same for source rows `src_pitch` bytes apart: dst row r = the first
// `row_bytes` bytes of source row r, zero-filled up to `dst_pitch`.
__global__ void copyRowsPitchedKernel(const uint8_t *__restrict__ src, size_t src_pitch,
                                      uint8_t *__restrict__ dst, uint32_t dst_pitch, size_t rows,
                                      uint32_t row_bytes) {
  const size_t total = rows * dst_pitch;
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < total;
       i += size_t(gridDim.x) * blockDim.x) {
    const size_t r = i / dst_pitch;
    const uint32_t b = uint32_t(i - r * dst_pitch);
    dst[i] = b < row_bytes ? src[r * src_pitch + b] : uint8_t(0);
  }
}

int copyRowsPitched(plb_context *ctx, const void *src, size_t src_pitch, void *dst, size_t dst_pitch,
                    size_t rows, size_t row_bytes) {
  if (rows == 0 || dst_pitch == 0) return PLB_OK;
  const size_t total = rows * dst_pitch;
  const int grid = int(std::min<size_t>((total + 255) / 256, size_t(ctx->sm_count) * 16));
  copyRowsPitchedKernel<<<grid, 256, 0, ctx->stream>>>(static_cast<const uint8_t *>(src), src_pitch,
                                                       static_cast<uint8_t *>(dst), uint32_t(dst_pitch),
                                                       rows, uint32_t(row_bytes));
  PLB_CUDA(cudaGetLastError());
  ctx->launches++;
  return PLB_OK;
}

// dst[n][h][w][:] = src[n][flip_h ? H-1-h : h][flip_w ? W-1-w : w][:], pixels of
// `pixel_bytes` bytes: the spatial flip of the reference's input transform.
__global__ void flipFieldKernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst,
                                size_t n_images, uint32_t H, uint32_t W, uint32_t pixel_bytes,
                                int flip_h, int flip_w) {
  const size_t total = n_images * H * W * pixel_bytes;
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < total;
       i += size_t(gridDim.x) * blockDim.x) {
    const uint32_t b = uint32_t(i % pixel_bytes);
    size_t r = i / pixel_bytes;
    const uint32_t w = uint32_t(r % W);
    r /= W;
    const uint32_t h = uint32_t(r % H);
    const size_t n = r / H;
    const uint32_t sh = flip_h ? H - 1 - h : h, sw = flip_w ? W - 1 - w : w;
    dst[i] = src[((n * H + sh) * W + sw) * size_t(pixel_bytes) + b];
  }
}

bool unflippedInputParams(const plb_conv_params &p, plb_conv_params *q) {
  bool any = false;
  *q = p;
  for (unsigned d = 0; d != p.num_field_dims && d < PLB_MAX_FIELD_DIMS; ++d) {
    if (!p.in_flip[d]) continue;
    any = true;
    q->in_flip[d] = 0;
    std::swap(q->in_pad_lo[d], q->in_pad_hi[d]);
    std::swap(q->in_trunc_lo[d], q->in_trunc_hi[d]);
  }
  return any;
}

int flipField(plb_context *ctx, const void *src, void *dst, size_t n_images, uint32_t H, uint32_t W,
              size_t pixel_bytes, bool flip_h, bool flip_w) {
  const size_t total = n_images * H * W * pixel_bytes;
  if (total == 0) return PLB_OK;
  const int grid = int(std::min<size_t>((total + 255) / 256, size_t(ctx->sm_count) * 16));
  flipFieldKernel<<<grid, 256, 0, ctx->stream>>>(static_cast<const uint8_t *>(src),
                                                 static_cast<uint8_t *>(dst), n_images, H, W,
                                                 uint32_t(pixel_bytes), flip_h ? 1 : 0, flip_w ? 1 : 0);
  PLB_CUDA(cudaGetLastError());
  ctx->launches++;
  return PLB_OK;
}

void convElementCounts(const plb_conv_params &p, size_t *in, size_t *weights, size_t *out) {
  size_t in_px = 1, taps = 1, out_px = 1;
  for (unsigned d = 0; d != p.num_field_dims && d < PLB_MAX_FIELD_DIMS; ++d) {
    in_px *= p.field[d];
    taps *= p.kernel[d];
    const long o = outputSize(p, d);
    out_px *= o > 0 ? size_t(o) : 0;
  }
  *in = size_t(p.batch) * in_px * p.groups * p.in_chans_per_group;
  *weights = size_t(p.groups) * taps * p.in_chans_per_group * p.out_chans_per_group;
  *out = size_t(p.batch) * out_px * p.groups * p.out_chans_per_group;
}

int checkConvRequest(const plb_conv_params &p, bool wu, const void *first, size_t first_elems,
                     const void *second, size_t second_elems, const void *result,
                     size_t result_elems) {
  const std::string err = validate(p);
  if (!err.empty()) return fail(PLB_ERR_INVALID_PARAMS, err);
  if (wu && !is16BitFloat(p.input_type) && p.input_type != PLB_FLOAT)
    // the reference never runs the weight update in quarter either
    // (tools/single_conv_layer.cpp:725-733)
    return fail(PLB_ERR_UNSUPPORTED, "weight update is implemented for half and float input only");
  if (!is16BitFloat(p.input_type) && p.input_type != PLB_QUARTER && p.input_type != PLB_FLOAT)
    return fail(PLB_ERR_UNSUPPORTED, "convolution input type must be half, float or quarter");
  if (p.output_type != PLB_HALF && p.output_type != PLB_FLOAT)
    return fail(PLB_ERR_INVALID_PARAMS, "convolution output type must be half or float");
  if (p.input_type == PLB_QUARTER && p.output_type != PLB_HALF)
    return fail(PLB_ERR_INVALID_PARAMS, "Output type must be half when input type is quarter");
  if ((first_elems && !first) || (second_elems && !second) || (result_elems && !result))
    return fail(PLB_ERR_INVALID_PARAMS, "null device pointer for a tensor that has elements");
  return PLB_OK;
}

// ---- input dilation as data ---------------------------------------------------
// dst = dilate(truncate(src)): [n][Hd][Wd] with the truncated field's elements
// dH / dW apart and zeros between them; or (adjoint) the gradient of that
// operation: dst[n][h][w] = src[n][(h - tH)*dH][(w - tW)*dW] inside the
// truncated range, zero outside.
template <typename V>
__device__ inline V dilateZero() {
  return V(0);
}
template <>
__device__ inline uint4 dilateZero<uint4>() {
  return make_uint4(0, 0, 0, 0);
}

template <typename V>
__global__ void dilateFieldKernel(const V *__restrict__ src, V *__restrict__ dst, size_t n_images,
                                  DilatedField s, uint32_t vecs, int adjoint) {
  const uint32_t OH = adjoint ? s.H : s.Hd, OW = adjoint ? s.W : s.Wd;
  const size_t total = n_images * OH * OW * vecs;
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < total;
       i += size_t(gridDim.x) * blockDim.x) {
    const uint32_t v = uint32_t(i % vecs);
    size_t r = i / vecs;
    const uint32_t w = uint32_t(r % OW);
    r /= OW;
    const uint32_t h = uint32_t(r % OH);
    const size_t n = r / OH;
    V val = dilateZero<V>();
    if (adjoint) {
      if (h >= s.tH && h < s.tH + s.TH && w >= s.tW && w < s.tW + s.TW)
        val = src[((n * s.Hd + size_t(h - s.tH) * s.dH) * s.Wd + size_t(w - s.tW) * s.dW) * vecs + v];
    } else if (h % s.dH == 0 && w % s.dW == 0) {
      val = src[((n * s.H + s.tH + h / s.dH) * s.W + s.tW + w / s.dW) * vecs + v];
    }
    dst[i] = val;
  }
}

bool undilatedInputParams(const plb_conv_params &p, plb_conv_params *q, DilatedField *f) {
  *q = p;
  if (p.num_field_dims < 1 || p.num_field_dims > 2) return false;
  bool any = false;
  uint32_t size[2] = {1, 1}, trunc_lo[2] = {0, 0}, kept[2] = {1, 1}, dil[2] = {1, 1}, dilated[2] = {1, 1};
  for (unsigned d = 0; d != p.num_field_dims; ++d) {
    const unsigned slot = p.num_field_dims == 2 ? d : 1;
    const uint32_t cut = p.in_trunc_lo[d] + p.in_trunc_hi[d];
    size[slot] = p.field[d];
    if (p.in_dilation[d] == 0 || cut > p.field[d]) return false;  // invalid: reported by validate()
    if (p.in_dilation[d] != 1) any = true;
    trunc_lo[slot] = p.in_trunc_lo[d];
    kept[slot] = p.field[d] - cut;
    dil[slot] = p.in_dilation[d];
    dilated[slot] = kept[slot] == 0 ? 0 : 1 + (kept[slot] - 1) * dil[slot];
  }
  if (!any) return false;
  for (unsigned d = 0; d != p.num_field_dims; ++d) {
    const unsigned slot = p.num_field_dims == 2 ? d : 1;
    q->field[d] = dilated[slot];
    q->in_trunc_lo[d] = q->in_trunc_hi[d] = 0;
    q->in_dilation[d] = 1;
  }
  *f = DilatedField{size[0], size[1], trunc_lo[0], trunc_lo[1], kept[0], kept[1], dil[0], dil[1],
                    dilated[0], dilated[1]};
  return true;
}

int dilateField(plb_context *ctx, const void *src, void *dst, size_t n_images, const DilatedField &f,
                size_t pixel_bytes, bool adjoint) {
  size_t vb = 16;
  while (pixel_bytes % vb) vb >>= 1;
  const uint32_t vecs = uint32_t(pixel_bytes / vb);
  const size_t total = n_images * (adjoint ? size_t(f.H) * f.W : size_t(f.Hd) * f.Wd) * vecs;
  if (total == 0) return PLB_OK;
  const int grid = int(std::min<size_t>((total + 255) / 256, size_t(ctx->sm_count) * 16));
#define PLB_DILATE(V)                                                                        \
  dilateFieldKernel<V><<<grid, 256, 0, ctx->stream>>>(static_cast<const V *>(src),           \
                                                      static_cast<V *>(dst), n_images, f, vecs, \
                                                      adjoint ? 1 : 0)
  switch (vb) {
    case 16: PLB_DILATE(uint4); break;
    case 8: PLB_DILATE(uint64_t); break;
    case 4: PLB_DILATE(uint32_t); break;
    case 2: PLB_DILATE(uint16_t); break;
    default: PLB_DILATE(uint8_t); break;
  }
#undef PLB_DILATE
  PLB_CUDA(cudaGetLastError());
  ctx->launches++;
  return PLB_OK;
}

int launchScaleRows(plb_context *ctx, void *out, const void *c, float beta, bool out_f32,
                    uint32_t rows, uint32_t cols, long long ldo, long long ldc) {
  if (rows == 0 || cols == 0) return PLB_OK;
  const size_t total = size_t(rows) * cols;
  const int grid = int(std::min<size_t>((total + 255) / 256, 148 * 8));
  scaleRowsKernel<<<grid, 256, 0, ctx->stream>>>(out, c, beta, out_f32 ? 1 : 0, rows, cols, ldo,
                                                 ldc);
  PLB_CUDA(cudaGetLastError());
  ctx->launches++;
  return PLB_OK;
}

}  // namespace plb

using namespace plb;

// ---------------------------------------------------------------------------
// C ABI: context and memory
// ---------------------------------------------------------------------------
namespace plb {
// Streams of 16-byte accesses: reads one (optional), writes up to four.
__global__ void __launch_bounds__(512)
memoryMixKernel(const uint4 *__restrict__ in, uint4 *__restrict__ out, size_t n, int reads, int writes) {
  uint32_t sink = 0;
  for (size_t i = blockIdx.x * size_t(blockDim.x) + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) {
    uint4 v = reads ? in[i] : make_uint4(uint32_t(i), uint32_t(i >> 3), uint32_t(i) * 2654435761u, 7u);
    for (int w = 0; w < writes; ++w) {
      out[size_t(w) * n + i] = v;
      v.x ^= 1u;
    }
    sink ^= v.x ^ v.y ^ v.z ^ v.w;
  }
  // a read-only run keeps its loads alive through a store that never happens
  if (writes == 0 && sink == 0x9e3779b9u && n == 1) out[0] = make_uint4(sink, 0, 0, 0);
}
}  // namespace plb

extern "C" {

const char *plb_last_error(void) { return g_last_error.c_str(); }

const char *plb_version(void) { return "poplibs_b200 0.1 (sm_100a)"; }

int plb_context_create_on_stream(int device, void *cuda_stream, plb_context **out) {
  if (out == nullptr) return fail(PLB_ERR_INVALID_PARAMS, "null output pointer");
  *out = nullptr;
  int count = 0;
  PLB_CUDA(cudaGetDeviceCount(&count));
  if (device < 0 || device >= count)
    return fail(PLB_ERR_CUDA, "CUDA device " + std::to_string(device) + " not present (" +
                                  std::to_string(count) + " visible)");
  PLB_CUDA(cudaSetDevice(device));
  cudaDeviceProp prop;
  PLB_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10)
    return fail(PLB_ERR_CUDA, std::string("device '") + prop.name + "' is compute capability " +
                                  std::to_string(prop.major) + "." + std::to_string(prop.minor) +
                                  "; this library only carries sm_100a kernels");
  plb_context *ctx = new plb_context();
  ctx->device = device;
  ctx->sm_count = prop.multiProcessorCount;
  if (cuda_stream != nullptr) {
    ctx->stream = static_cast<cudaStream_t>(cuda_stream);
    ctx->owns_stream = false;
  } else {
    cudaError_t e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) {
      delete ctx;
      return cudaFail(e, "cudaStreamCreateWithFlags");
    }
    ctx->owns_stream = true;
  }
  void *host_word = nullptr, *dev_word = nullptr;
  cudaError_t e = cudaHostAlloc(&host_word, sizeof(int), cudaHostAllocMapped);
  if (e == cudaSuccess) {
    ctx->h_status = static_cast<volatile int *>(host_word);
    *ctx->h_status = 0;
    e = cudaHostGetDevicePointer(&dev_word, host_word, 0);
    ctx->d_status = static_cast<int *>(dev_word);
  }
  if (e != cudaSuccess) {
    plb_context_destroy(ctx);
    return cudaFail(e, "status word allocation");
  }
  *out = ctx;
  return PLB_OK;
}

int plb_context_create(int device, plb_context **out) {
  return plb_context_create_on_stream(device, nullptr, out);
}

int plb_device_pci_address(int device, char *buf, size_t len) {
  if (buf == nullptr || len < 16) return fail(PLB_ERR_INVALID_PARAMS, "buffer of at least 16 bytes needed");
  PLB_CUDA(cudaDeviceGetPCIBusId(buf, int(len), device));
  for (size_t i = 0; i < len && buf[i]; ++i)
    if (buf[i] >= 'A' && buf[i] <= 'F') buf[i] = char(buf[i] - 'A' + 'a');  // sysfs spells it in lower case
  return PLB_OK;
}

void plb_context_destroy(plb_context *ctx) {
  if (ctx == nullptr) return;
  cudaSetDevice(ctx->device);
  if (ctx->stream) cudaStreamSynchronize(ctx->stream);
  for (int i = 0; i < plb_context::kScratchSlots; ++i)
    if (ctx->scratch[i]) cudaFree(ctx->scratch[i]);
  if (ctx->h_status) cudaFreeHost(const_cast<int *>(ctx->h_status));
  if (ctx->timer_start) cudaEventDestroy(ctx->timer_start);
  if (ctx->timer_stop) cudaEventDestroy(ctx->timer_stop);
  if (ctx->owns_stream && ctx->stream) cudaStreamDestroy(ctx->stream);
  delete ctx;
}

void *plb_context_stream(plb_context *ctx) { return ctx ? ctx->stream : nullptr; }

uint64_t plb_launch_count(const plb_context *ctx) { return ctx ? ctx->launches : 0; }

void plb_context_set_plan_flags(plb_context *ctx, int32_t plan_flags) {
  if (ctx) ctx->plan_flags = plan_flags;
}

int plb_synchronize(plb_context *ctx) {
  if (int rc = activate(ctx)) return rc;
  PLB_CUDA(cudaStreamSynchronize(ctx->stream));
  const int status = *ctx->h_status;
  if (status != 0) {
    *ctx->h_status = 0;
    static const char *names[] = {"ok", "TMA producer wait ran out", "MMA issuer wait ran out",
                                  "epilogue wait ran out", "teardown could not see copies complete",
                                  "a peer's flag did not arrive (all-reduce over peer memory)"};
    return fail(PLB_ERR_KERNEL, std::string("kernel status ") + std::to_string(status) + ": " +
                                    (status > 0 && status < 6 ? names[status] : "unknown"));
  }
  return PLB_OK;
}

int plb_malloc(plb_context *ctx, size_t bytes, void **d_ptr) {
  if (int rc = activate(ctx)) return rc;
  if (d_ptr == nullptr) return fail(PLB_ERR_INVALID_PARAMS, "null output pointer");
  *d_ptr = nullptr;
  if (bytes == 0) bytes = 16;
  PLB_CUDA(cudaMalloc(d_ptr, bytes));
  return PLB_OK;
}

int plb_free(plb_context *ctx, void *d_ptr) {
  if (int rc = activate(ctx)) return rc;
  if (d_ptr) {
    PLB_CUDA(cudaStreamSynchronize(ctx->stream));
    PLB_CUDA(cudaFree(d_ptr));
  }
  return PLB_OK;
}

int plb_memcpy_h2d(plb_context *ctx, void *d_dst, const void *h_src, size_t bytes) {
  if (int rc = activate(ctx)) return rc;
  if (bytes) PLB_CUDA(cudaMemcpyAsync(d_dst, h_src, bytes, cudaMemcpyHostToDevice, ctx->stream));
  return PLB_OK;
}

int plb_memcpy_d2h(plb_context *ctx, void *h_dst, const void *d_src, size_t bytes) {
  if (int rc = activate(ctx)) return rc;
  if (bytes) PLB_CUDA(cudaMemcpyAsync(h_dst, d_src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
  PLB_CUDA(cudaStreamSynchronize(ctx->stream));
  return PLB_OK;
}

int plb_memset(plb_context *ctx, void *d_dst, int value, size_t bytes) {
  if (int rc = activate(ctx)) return rc;
  if (bytes) PLB_CUDA(cudaMemsetAsync(d_dst, value, bytes, ctx->stream));
  return PLB_OK;
}

// ---------------------------------------------------------------------------
// C ABI: layout changes, casts
// ---------------------------------------------------------------------------

int plb_rearrange_acts_to_device(plb_context *ctx, uint32_t elem_bytes, uint32_t batch,
                                 uint32_t chans, uint64_t field_elems, const void *d_src,
                                 void *d_dst) {
  if (int rc = activate(ctx)) return rc;
  return launchTranspose(ctx, elem_bytes, batch, chans, field_elems, d_src, d_dst);
}

int plb_rearrange_acts_from_device(plb_context *ctx, uint32_t elem_bytes, uint32_t batch,
                                   uint32_t chans, uint64_t field_elems, const void *d_src,
                                   void *d_dst) {
  if (int rc = activate(ctx)) return rc;
  return launchTranspose(ctx, elem_bytes, batch, field_elems, chans, d_src, d_dst);
}

int plb_rearrange_weights_to_device(plb_context *ctx, uint32_t elem_bytes, uint32_t groups,
                                    uint32_t out_chans, uint32_t in_chans, uint64_t kernel_elems,
                                    const void *d_src, void *d_dst) {
  if (int rc = activate(ctx)) return rc;
  return launchTranspose(ctx, elem_bytes, groups, uint64_t(out_chans) * in_chans, kernel_elems,
                         d_src, d_dst);
}

int plb_rearrange_weights_from_device(plb_context *ctx, uint32_t elem_bytes, uint32_t groups,
                                      uint32_t out_chans, uint32_t in_chans,
                                      uint64_t kernel_elems, const void *d_src, void *d_dst) {
  if (int rc = activate(ctx)) return rc;
  return launchTranspose(ctx, elem_bytes, groups, kernel_elems, uint64_t(out_chans) * in_chans,
                         d_src, d_dst);
}

int plb_weights_transpose_chans_flip_xy(plb_context *ctx, uint32_t elem_bytes, uint32_t groups,
                                        uint32_t out_chans, uint32_t in_chans,
                                        uint64_t kernel_elems, const void *d_src, void *d_dst) {
  if (int rc = activate(ctx)) return rc;
  const size_t total = size_t(groups) * kernel_elems * out_chans * in_chans;
  if (total == 0) return PLB_OK;
  const int grid = int(std::min<size_t>((total + 255) / 256, 148 * 16));
  switch (elem_bytes) {
    case 1:
      transposeFlipKernel<uint8_t><<<grid, 256, 0, ctx->stream>>>(
          static_cast<const uint8_t *>(d_src), static_cast<uint8_t *>(d_dst), groups,
          uint32_t(kernel_elems), out_chans, in_chans);
      break;
    case 2:
      transposeFlipKernel<uint16_t><<<grid, 256, 0, ctx->stream>>>(
          static_cast<const uint16_t *>(d_src), static_cast<uint16_t *>(d_dst), groups,
          uint32_t(kernel_elems), out_chans, in_chans);
      break;
    case 4:
      transposeFlipKernel<uint32_t><<<grid, 256, 0, ctx->stream>>>(
          static_cast<const uint32_t *>(d_src), static_cast<uint32_t *>(d_dst), groups,
          uint32_t(kernel_elems), out_chans, in_chans);
      break;
    default:
      return fail(PLB_ERR_INVALID_PARAMS, "element size must be 1, 2 or 4 bytes");
  }
  PLB_CUDA(cudaGetLastError());
  ctx->launches++;
  return PLB_OK;
}

int plb_transpose_matrix(plb_context *ctx, uint32_t elem_bytes, uint32_t groups, uint32_t rows,
                         uint32_t cols, const void *d_src, void *d_dst) {
  if (int rc = activate(ctx)) return rc;
  return launchTranspose(ctx, elem_bytes, groups, rows, cols, d_src, d_dst);
}

int plb_copy_strided(plb_context *ctx, uint32_t elem_bytes, uint32_t rank, const uint64_t *shape,
                     const int64_t *src_strides, const int64_t *dst_strides, const void *d_src,
                     void *d_dst) {
  if (int rc = activate(ctx)) return rc;
  if (rank > PLB_MAX_VIEW_RANK) return fail(PLB_ERR_UNSUPPORTED, "tensor rank above 8");
  StridedCopyArgs a{};
  a.rank = rank ? rank : 1;
  size_t total = 1;
  a.shape[0] = 1;
  for (uint32_t d = 0; d < rank; ++d) {
    a.shape[d] = shape[d];
    a.src_strides[d] = src_strides[d];
    a.dst_strides[d] = dst_strides[d];
    total *= shape[d];
  }
  if (total == 0) return PLB_OK;
  const int grid = int(std::min<size_t>((total + 255) / 256, size_t(148) * 32));
  switch (elem_bytes) {
    case 1:
      stridedCopyKernel<uint8_t><<<grid, 256, 0, ctx->stream>>>(
          static_cast<const uint8_t *>(d_src), static_cast<uint8_t *>(d_dst), a, total);
      break;
    case 2:
      stridedCopyKernel<uint16_t><<<grid, 256, 0, ctx->stream>>>(
          static_cast<const uint16_t *>(d_src), static_cast<uint16_t *>(d_dst), a, total);
      break;
    case 4:
      stridedCopyKernel<uint32_t><<<grid, 256, 0, ctx->stream>>>(
          static_cast<const uint32_t *>(d_src), static_cast<uint32_t *>(d_dst), a, total);
      break;
    default:
      return fail(PLB_ERR_INVALID_PARAMS, "element size must be 1, 2 or 4 bytes");
  }
  PLB_CUDA(cudaGetLastError());
  ctx->launches++;
  return PLB_OK;
}

int plb_fill(plb_context *ctx, int32_t dtype, void *d_dst, float value, size_t count) {
  if (int rc = activate(ctx)) return rc;
  if (count == 0) return PLB_OK;
  const int grid = int(std::min<size_t>((count + 255) / 256, size_t(148) * 16));
  if (dtype == PLB_HALF)
    fillKernel<__half><<<grid, 256, 0, ctx->stream>>>(static_cast<__half *>(d_dst),
                                                      __float2half_rn(value), count);
  else if (dtype == PLB_FLOAT)
    fillKernel<float><<<grid, 256, 0, ctx->stream>>>(static_cast<float *>(d_dst), value, count);
  else
    return fail(PLB_ERR_INVALID_PARAMS, "fill type must be half or float");
  PLB_CUDA(cudaGetLastError());
  ctx->launches++;
  return PLB_OK;
}

int plb_add_bias(plb_context *ctx, int32_t dtype, void *d_acts, const void *d_biases,
                 uint64_t pixels, uint32_t chans) {
  if (int rc = activate(ctx)) return rc;
  const size_t total = size_t(pixels) * chans;
  if (total == 0) return PLB_OK;
  const int grid = int(std::min<size_t>((total + 255) / 256, size_t(148) * 16));
  if (dtype == PLB_HALF)
    addBiasKernel<__half><<<grid, 256, 0, ctx->stream>>>(
        static_cast<__half *>(d_acts), static_cast<const __half *>(d_biases), total, chans);
  else if (dtype == PLB_FLOAT)
    addBiasKernel<float><<<grid, 256, 0, ctx->stream>>>(
        static_cast<float *>(d_acts), static_cast<const float *>(d_biases), total, chans);
  else
    return fail(PLB_ERR_INVALID_PARAMS, "bias add needs half or float activations");
  PLB_CUDA(cudaGetLastError());
  ctx->launches++;
  return PLB_OK;
}

int plb_conv_bias_update(plb_context *ctx, int32_t acts_dtype, const void *d_out_grads,
                         uint64_t pixels, uint32_t chans, int32_t bias_dtype, void *d_biases,
                         float scale) {
  if (int rc = activate(ctx)) return rc;
  if ((acts_dtype != PLB_HALF && acts_dtype != PLB_FLOAT) ||
      (bias_dtype != PLB_HALF && bias_dtype != PLB_FLOAT))
    return fail(PLB_ERR_INVALID_PARAMS, "bias update needs half or float gradients and biases");
  if (chans == 0) return PLB_OK;
  // slabs of rows, enough blocks to fill the device; partial sums in fp32
  const size_t es = dtypeBytes(acts_dtype);
  const uint32_t vec = uint32_t(16 / es);
  const bool vector_ok = chans % vec == 0 && (reinterpret_cast<uintptr_t>(d_out_grads) & 15) == 0;
  uint32_t vec_lanes = 1, col_blocks = 1, slabs = 1;
  if (vector_ok) {
    const uint32_t vecs = chans / vec;
    vec_lanes = 1;
    while (vec_lanes < 32 && vec_lanes < vecs) vec_lanes <<= 1;
    col_blocks = (vecs + vec_lanes - 1) / vec_lanes;
    const uint32_t row_lanes = 256 / vec_lanes;
    const uint64_t want = std::max<uint64_t>(1, uint64_t(ctx->sm_count) * 8 / col_blocks);
    slabs = uint32_t(std::max<uint64_t>(1, std::min<uint64_t>(want, (pixels + row_lanes - 1) / row_lanes)));
  } else {
    col_blocks = (chans + 127) / 128;
    slabs = uint32_t(std::max<uint64_t>(1, std::min<uint64_t>(pixels, uint64_t(ctx->sm_count) * 16 / col_blocks)));
  }
  void *ws = nullptr;
  if (int rc = scratch(ctx, kSlotBiasUpdate, size_t(slabs) * chans * sizeof(float), &ws)) return rc;
  float *partial = static_cast<float *>(ws);
  if (vector_ok) {
    if (acts_dtype == PLB_HALF)
      columnSumPartialKernel<__half><<<dim3(col_blocks, slabs), 256, 0, ctx->stream>>>(
          static_cast<const __half *>(d_out_grads), partial, pixels, chans, vec_lanes);
    else
      columnSumPartialKernel<float><<<dim3(col_blocks, slabs), 256, 0, ctx->stream>>>(
          static_cast<const float *>(d_out_grads), partial, pixels, chans, vec_lanes);
  } else {
    if (acts_dtype == PLB_HALF)
      columnSumPartialScalarKernel<__half><<<dim3(col_blocks, slabs), 128, 0, ctx->stream>>>(
          static_cast<const __half *>(d_out_grads), partial, pixels, chans);
    else
      columnSumPartialScalarKernel<float><<<dim3(col_blocks, slabs), 128, 0, ctx->stream>>>(
          static_cast<const float *>(d_out_grads), partial, pixels, chans);
  }
  PLB_CUDA(cudaGetLastError());
  ctx->launches++;
  const uint32_t ugrid = (chans + 127) / 128;
  if (bias_dtype == PLB_HALF)
    biasUpdateKernel<__half><<<ugrid, 128, 0, ctx->stream>>>(partial, slabs, chans,
                                                            static_cast<__half *>(d_biases), scale);
  else
    biasUpdateKernel<float><<<ugrid, 128, 0, ctx->stream>>>(partial, slabs, chans,
                                                           static_cast<float *>(d_biases), scale);
  PLB_CUDA(cudaGetLastError());
  ctx->launches++;
  return PLB_OK;
}

int plb_timer_start(plb_context *ctx) {
  if (int rc = activate(ctx)) return rc;
  if (!ctx->timer_start) {
    PLB_CUDA(cudaEventCreate(&ctx->timer_start));
    PLB_CUDA(cudaEventCreate(&ctx->timer_stop));
  }
  PLB_CUDA(cudaEventRecord(ctx->timer_start, ctx->stream));
  return PLB_OK;
}

int plb_memory_mix_probe(plb_context *ctx, int32_t reads, int32_t writes, size_t bytes,
                         const void *d_in, void *d_out) {
  if (int rc = activate(ctx)) return rc;
  if (reads < 0 || reads > 1 || writes < 0 || writes > 4 || reads + writes == 0 || bytes % 16 != 0)
    return fail(PLB_ERR_INVALID_PARAMS, "memory probe: 0-1 read and 0-4 write streams of a multiple of 16 bytes");
  if ((reads && !d_in) || (writes && !d_out) || (reinterpret_cast<uintptr_t>(d_in) & 15) ||
      (reinterpret_cast<uintptr_t>(d_out) & 15))
    return fail(PLB_ERR_INVALID_PARAMS, "memory probe: null or unaligned buffer");
  const size_t n = bytes / 16;
  if (n == 0) return PLB_OK;
  const int grid = ctx->sm_count * 16;
  plb::memoryMixKernel<<<grid, 512, 0, ctx->stream>>>(static_cast<const uint4 *>(d_in),
                                                      static_cast<uint4 *>(d_out), n, reads, writes);
  PLB_CUDA(cudaGetLastError());
  ctx->launches++;
  return PLB_OK;
}

int plb_timer_stop(plb_context *ctx, float *milliseconds) {
  if (int rc = activate(ctx)) return rc;
  if (!ctx->timer_start) return fail(PLB_ERR_INVALID_PARAMS, "timer was not started");
  PLB_CUDA(cudaEventRecord(ctx->timer_stop, ctx->stream));
  PLB_CUDA(cudaEventSynchronize(ctx->timer_stop));
  float ms = 0.f;
  PLB_CUDA(cudaEventElapsedTime(&ms, ctx->timer_start, ctx->timer_stop));
  if (milliseconds) *milliseconds = ms;
  return PLB_OK;
}

int plb_cast_from_f32(plb_context *ctx, int32_t dtype, void *d_dst, const float *d_src,
                      size_t count) {
  if (int rc = activate(ctx)) return rc;
  if (count == 0) return PLB_OK;
  const int grid = int(std::min<size_t>((count + 255) / 256, 148 * 16));
  if (dtype == PLB_HALF)
    castFromF32Kernel<__half><<<grid, 256, 0, ctx->stream>>>(static_cast<__half *>(d_dst), d_src,
                                                             count);
  else if (dtype == PLB_FLOAT)
    castFromF32Kernel<float><<<grid, 256, 0, ctx->stream>>>(static_cast<float *>(d_dst), d_src,
                                                            count);
  else
    return fail(PLB_ERR_INVALID_PARAMS, "cast target must be half or float");
  PLB_CUDA(cudaGetLastError());
  ctx->launches++;
  return PLB_OK;
}

int plb_scaled_add_to(plb_context *ctx, int32_t dtype, void *d_weights, const float *d_deltas_f32,
                      float scale, size_t count) {
  if (int rc = activate(ctx)) return rc;
  if (count == 0) return PLB_OK;
  const int grid = int(std::min<size_t>((count + 255) / 256, 148 * 16));
  if (dtype == PLB_HALF)
    scaledAddKernel<__half><<<grid, 256, 0, ctx->stream>>>(static_cast<__half *>(d_weights),
                                                           d_deltas_f32, scale, count);
  else if (dtype == PLB_FLOAT)
    scaledAddKernel<float><<<grid, 256, 0, ctx->stream>>>(static_cast<float *>(d_weights),
                                                          d_deltas_f32, scale, count);
  else
    return fail(PLB_ERR_INVALID_PARAMS, "weights must be half or float");
  PLB_CUDA(cudaGetLastError());
  ctx->launches++;
  return PLB_OK;
}

}  // extern "C"

#ifdef PLB_TRACE
// Development builds only: attach a device buffer of 3*4096 clock stamps.
extern "C" __attribute__((visibility("default"))) void plb_debug_set_trace(plb_context *ctx,
                                                                            long long *d_trace) {
  ctx->trace = d_trace;
}
#endif
