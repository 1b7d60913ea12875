// Internal host-side runtime shared by the C ABI entry points: the context
// (device, stream, kernel status word, scratch memory), error reporting and
// TMA tensor-map construction.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <string>
#include <vector>

#include "poplibs_b200.h"

// Grow-only scratch buffers of a context, by use.  Entry points call one
// another (3-D -> 2-D -> flipped -> dilated -> padded channels ...), so every
// pre-pass has a slot of its own.
enum plb_scratch_slot {
  kSlotOperands = 0,    // rearranged operands, split-K partial sums, gathered sub-filters
  kSlotHostIn,          // staging of the host-buffer entry points
  kSlotHostWeights,
  kSlotHostOut,
  kSlotHostBias,
  kSlotBiasUpdate,      // column sums of the bias update
  kSlotUsedTaps,        // taps of a truncated / flipped kernel
  kSlotPaddedChans,     // zero-padded channel counts
  kSlotFlipped,         // reversed input (input flip)
  kSlotDepthFold,       // depth taps of a 3-D field gathered into the channels
  kSlotFoldedWeights,
  kSlotFoldedGrads,
  kSlotDilated,         // zero-stuffed input (input dilation)
  kSlotSplitK,          // fp32 partial sums of a split-K forward / backward / matrix product
  kSlotFloatSplit,      // bfloat16 pieces of float operands
  kSlotCount
};

struct plb_context {
  int device = 0;
  int sm_count = 0;
  cudaStream_t stream = nullptr;
  bool owns_stream = false;
  // Kernel status word (0 = OK): page-locked host memory mapped into the device,
  // written by kernels only when a bounded wait runs out, read by the host
  // without a copy (a copy would queue behind other streams' transfers).
  int *d_status = nullptr;        // device address
  volatile int *h_status = nullptr;  // host address of the same word
  uint64_t launches = 0;          // kernels launched through this context
  int plan_flags = 0;             // PLB_PLAN_* bits added to every plan made through this context
  long long *trace = nullptr;     // device timeline buffer for builds with -DPLB_TRACE
  cudaEvent_t timer_start = nullptr, timer_stop = nullptr;
  // grow-only scratch buffers, one per use (plb_scratch_slot)
  static constexpr int kScratchSlots = kSlotCount;
  void *scratch[kScratchSlots] = {};
  size_t scratch_bytes[kScratchSlots] = {};
};

#include <nvtx3/nvToolsExt.h>

namespace plb {

// A named range around a public entry point, visible to profilers that hook
// NVTX (the role of POPLIN_TRACEPOINT at the reference's entry points,
// include/poplibs_support/Tracepoint.hpp:69-78).  Header-only: without a
// profiler attached the calls are a null-pointer test each.
struct TraceRange {
  explicit TraceRange(const char *name) { nvtxRangePushA(name); }
  ~TraceRange() { nvtxRangePop(); }
  TraceRange(const TraceRange &) = delete;
  TraceRange &operator=(const TraceRange &) = delete;
};

// Records the message for plb_last_error() and returns `code`.
int fail(int code, const std::string &message);
int cudaFail(cudaError_t err, const char *what);

#define PLB_CUDA(expr)                                         \
  do {                                                         \
    cudaError_t plb_err__ = (expr);                            \
    if (plb_err__ != cudaSuccess) return ::plb::cudaFail(plb_err__, #expr); \
  } while (0)

// Makes the context's device current.
int activate(plb_context *ctx);
// Returns a scratch buffer of at least `bytes` (grows, synchronising first, if needed).
int scratch(plb_context *ctx, int slot, size_t bytes, void **ptr);

// cuTensorMapEncodeTiled with 128-byte swizzle and zero fill outside the
// tensor.  dims[0] is the contiguous dimension; strides_bytes[i] is the byte
// stride of dims[i + 1].
int encodeTensorMap(CUtensorMap *tm, CUtensorMapDataType type, int rank, const void *base,
                    const uint64_t *dims, const uint64_t *strides_bytes, const uint32_t *box,
                    const uint32_t *elem_strides, int swizzle_bytes = 128);

inline size_t dtypeBytes(int dtype) {
  return dtype == PLB_FLOAT ? 4 : (dtype == PLB_HALF || dtype == PLB_BFLOAT16) ? 2 : 1;
}
// 16-bit floating-point operands (the kind::f16 instruction takes either)
inline bool is16BitFloat(int dtype) { return dtype == PLB_HALF || dtype == PLB_BFLOAT16; }

// Row resize (runtime.cu): rows of src_bytes -> rows of dst_bytes, zero fill / drop of the tail.
int resizeRows(plb_context *ctx, const void *src, void *dst, size_t rows, size_t src_bytes,
               size_t dst_bytes);
int copyRowsPitched(plb_context *ctx, const void *src, size_t src_pitch, void *dst, size_t dst_pitch,
                    size_t rows, size_t row_bytes);

// Input flip of the reference's input transform: the convolution of a flipped
// input equals the convolution of the reversed tensor with the input padding and
// truncation of the flipped dimensions swapped.  Returns true and fills `q` if
// `p` flips its input in some dimension.
bool unflippedInputParams(const plb_conv_params &p, plb_conv_params *q);
// Spatial flip of an [n][H][W][pixel] tensor (runtime.cu).
int flipField(plb_context *ctx, const void *src, void *dst, size_t n_images, uint32_t H, uint32_t W,
              size_t pixel_bytes, bool flip_h, bool flip_w);

// First check of every convolution entry point, before any pre-pass is
// launched: the reference's parameter validation, the element types this path
// implements (wu: the weight update takes half only) and that no tensor with
// elements is passed as a null pointer.  `in` / `weights` / `out` follow the
// forward naming; pass the tensors of the pass in that order
// (backward: out grads, weights, in grads; weight update: acts, out grads, any
// of the two gradient outputs).
int checkConvRequest(const plb_conv_params &p, bool wu, const void *in_like, size_t in_elems,
                     const void *second, size_t second_elems, const void *result,
                     size_t result_elems);
// Element counts of the activations, weights and output of `p` (any rank).
void convElementCounts(const plb_conv_params &p, size_t *in, size_t *weights, size_t *out);

// Input dilation of the reference's input transform, as data: the convolution of
// a dilated input equals the ordinary convolution of the zero-stuffed tensor
// dilate(truncate(x)).  A fallback (the inserted zeros are multiplied); the
// backward pass of a strided layer does not come this way (plb_conv_bwd takes
// it in forward terms).  [n][H][W] field (H = 1 for 1-D), tH/tW lower truncation,
// TH/TW kept extent, dH/dW dilation, Hd/Wd dilated extent.
struct DilatedField {
  uint32_t H, W, tH, tW, TH, TW, dH, dW, Hd, Wd;
};
// Returns true and fills `q` (field = dilated extent, no truncation, dilation 1)
// and `f` if `p` (1-D or 2-D) dilates its input.
bool undilatedInputParams(const plb_conv_params &p, plb_conv_params *q, DilatedField *f);
// dst = dilate(truncate(src)) ([n][Hd][Wd]); adjoint: dst ([n][H][W]) = the
// elements of src ([n][Hd][Wd]) on the lattice, zero in the truncated margins.
int dilateField(plb_context *ctx, const void *src, void *dst, size_t n_images, const DilatedField &f,
                size_t pixel_bytes, bool adjoint);

// ---- 3-D fields (conv3d.cu): depth folded into the channels of a 2-D problem ----
int conv3dFwd(plb_context *ctx, const plb_conv_params &p, const plb_conv_options *opt,
              const void *d_in, const void *d_weights, const float *d_bias, void *d_out,
              int transpose_and_flip_weights);
int conv3dBwd(plb_context *ctx, const plb_conv_params &p, const plb_conv_options *opt,
              const void *d_out_grads, const void *d_weights, void *d_in_grads);
int conv3dWu(plb_context *ctx, const plb_conv_params &p, const plb_conv_options *opt,
             const void *d_acts, const void *d_out_grads, void *d_weight_grads,
             float *d_weight_grads_f32);
int conv3dPlan(const plb_conv_params &p, const plb_conv_options *opt, int32_t pass, plb_plan *plan);

// ---- contraction launch (igemm_launch.cu) -----------------------------------

// A fully resolved implicit-GEMM problem: one launch of the igemm kernel.
struct IgemmProblem {
  bool fp8 = false;      // 8-bit operands (else 16-bit)
  bool bf16 = false;     // 16-bit operands are bfloat16 (else half)
  int fmt_a = 0, fmt_b = 0;  // plb_quarter_format of the activations / weights when fp8
  bool b_mn = false;     // right operand stored [tap][K][N], N contiguous
  // activations: 4-D tensor (C, W, H, N) with byte strides of W, H, N
  const void *act = nullptr;
  uint64_t act_dims[4] = {1, 1, 1, 1};
  uint64_t act_strides[3] = {16, 16, 16};
  uint32_t act_elem_strides[4] = {1, 1, 1, 1};  // traversal strides (conv stride on W, H)
  // weights: (K, N, taps) K-major or (N, K, taps) MN-major, byte strides of dims 1, 2
  const void *wgt = nullptr;
  uint64_t wgt_dims[3] = {1, 1, 1};
  uint64_t wgt_strides[2] = {16, 16};
  // output
  int out_w = 1, out_h = 1, out_n = 1;  // pixels
  int n_total = 0;                      // output channels
  int k_per_tap = 0;                    // reduction length per tap (elements)
  int taps_h = 1, taps_w = 1, pad_h = 0, pad_w = 0, dil_h = 1, dil_w = 1;
  int flip_h = 0, flip_w = 0;
  int stride_h = 1, stride_w = 1;
  void *out = nullptr;
  long long ldc = 0;  // elements between output pixels along w
  // elements between output rows / images; 0 = dense (out_w * ldc, out_h * out_w * ldc)
  long long out_stride_h = 0, out_stride_n = 0;
  const void *addend = nullptr;
  long long ld_addend = 0;
  const float *bias = nullptr;
  float alpha = 1.f, beta = 0.f;
  bool out_f32 = false;
  int force_tile_n = 0;  // 0 = planner's choice
  int force_split_k = 0; // 0 = planner's choice; n = n CTAs per output tile (clamped to the K steps)
  int plan_flags = 0;    // PLB_PLAN_* bits
};

// Fills the tiling part of `plan` for a problem; returns non-zero if the
// problem cannot be run by the igemm kernel (message recorded).
int planIgemm(const IgemmProblem &p, int sm_count, plb_plan *plan);

// ---- float operands (float_route.cu) ------------------------------------------
// The layer / product that runs for float operands: bfloat16, the reduction
// dimension of the pass three times as long.
plb_conv_params floatRouteConvParams(const plb_conv_params &p, int pass);
plb_matmul_desc floatRouteMatmulDesc(const plb_matmul_desc &d);
int floatConvFwd(plb_context *ctx, const plb_conv_params &p, const plb_conv_options *opt,
                 const void *d_in, const void *d_weights, const float *d_bias, void *d_out,
                 int transpose_and_flip_weights);
int floatConvBwd(plb_context *ctx, const plb_conv_params &p, const plb_conv_options *opt,
                 const void *d_out_grads, const void *d_weights, void *d_in_grads);
int floatConvWu(plb_context *ctx, const plb_conv_params &p, const plb_conv_options *opt,
                const void *d_acts, const void *d_out_grads, void *d_weight_grads,
                float *d_weight_grads_f32);
int floatMatmul(plb_context *ctx, const plb_matmul_desc &d, const void *d_a, const void *d_b,
                const void *d_c, void *d_d);

int launchIgemm(plb_context *ctx, const IgemmProblem &p, const plb_plan &plan);

}  // namespace plb
