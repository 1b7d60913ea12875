/*
 * poplibs_b200 -- C ABI of the B200 (sm_100a) implementation of the poplin
 * dense-contraction path: poplin::matMul and poplin::convolution (forward,
 * backward-data and weight-update passes).
 *
 * The reference exposes this path only as deferred C++ graph construction
 * (include/poplin/MatMul.hpp, include/poplin/Convolution.hpp: calls take
 * poplar::Graph / Tensor / program::Sequence and nothing runs until
 * poplar::Engine::run).  This header is the layer underneath the C++ drop-in
 * (include/poplin/ *.hpp of this repository): plain pointers and sizes, device
 * buffers owned by the caller, every call enqueues its kernels on the
 * context's CUDA stream.  It is also what a foreign-language binding (ctypes,
 * cgo, JNI) would bind.
 *
 * Conventions
 *  - Every function returns 0 on success and a non-zero plb_status otherwise;
 *    plb_last_error() gives the message for the calling thread (the C++ layer
 *    rethrows it as poputil::poplibs_error / poplar::invalid_option, the
 *    exception types of include/poputil/exceptions.hpp:17-21 and
 *    include/poputil/OptionParsing.hpp:204-221).
 *  - Pointers named d_* are device pointers, h_* host pointers.
 *  - Device layouts (they mirror poplin's internal channels-innermost shapes,
 *    lib/poplin/ConvUtilInternal.cpp:147-175):
 *      activations  [N][field...][G*C]           ("NHWC")
 *      weights      [G][kernel...][Co][Ci]
 *    plb_rearrange_* convert from / to the external shapes of
 *    include/poplin/Convolution.hpp:81-82, 323-328 ([N][G*C][field...],
 *    [G][Co][Ci][kernel...]).
 *  - There is no CPU fallback: if no CUDA device / sm_100a kernel image is
 *    available the calls fail with PLB_ERR_CUDA.
 */
#ifndef POPLIBS_B200_H
#define POPLIBS_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define PLB_API __attribute__((visibility("default")))
#else
#define PLB_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define PLB_MAX_FIELD_DIMS 3

typedef enum plb_status {
  PLB_OK = 0,
  PLB_ERR_INVALID_PARAMS = 1, /* poputil::poplibs_error in the C++ layer      */
  PLB_ERR_INVALID_OPTION = 2, /* poplar::invalid_option                       */
  PLB_ERR_UNSUPPORTED = 3,    /* valid poplin request this build cannot run   */
  PLB_ERR_CUDA = 4,           /* CUDA runtime / driver failure                */
  PLB_ERR_KERNEL = 5,         /* a kernel reported a non-zero status word     */
  PLB_ERR_OUT_OF_MEMORY = 6   /* poplar::graph_memory_allocation_error        */
} plb_status;

/* poplar::Type values used on this path (HALF, FLOAT, QUARTER).  PLB_BFLOAT16
 * is not a poplar type: it is the operand type a float contraction runs in
 * (three bfloat16 terms per product, fp32 accumulation) and is accepted as an
 * input type in its own right; results are PLB_HALF or PLB_FLOAT as for half. */
typedef enum plb_dtype { PLB_HALF = 0, PLB_FLOAT = 1, PLB_QUARTER = 2, PLB_BFLOAT16 = 3 } plb_dtype;

/* poplin::Pass (lib/poplin/ConvOptions.hpp:13-24). */
typedef enum plb_pass {
  PLB_PASS_NONE = 0,
  PLB_PASS_NONE_MATMUL,
  PLB_PASS_INFERENCE_FWD,
  PLB_PASS_TRAINING_FWD,
  PLB_PASS_TRAINING_BWD,
  PLB_PASS_TRAINING_WU,
  PLB_PASS_FC_INFERENCE_FWD,
  PLB_PASS_FC_TRAINING_FWD,
  PLB_PASS_FC_TRAINING_BWD,
  PLB_PASS_FC_TRAINING_WU
} plb_pass;

PLB_API const char *plb_last_error(void);
/* Library version and the GPU architecture the kernels were compiled for. */
PLB_API const char *plb_version(void);

/* ------------------------------------------------------------------------ */
/* Context: one CUDA device + stream + kernel status word + scratch memory.  */
/* Stands in for the poplar::Graph / Engine pair a poplin call is made on    */
/* (tools/single_conv_layer.cpp:585-587, 1169, 1326-1340).                   */
/* ------------------------------------------------------------------------ */
/* Every call that takes a context makes the context's device the calling     */
/* thread's current CUDA device (cudaSetDevice) and leaves it so; so does     */
/* plb_conv_wu_static_scratch with its `device` argument.                     */
typedef struct plb_context plb_context;

PLB_API int plb_context_create(int device, plb_context **out);
/* Same, on a CUDA stream the caller owns (cudaStream_t passed as void*). */
PLB_API int plb_context_create_on_stream(int device, void *cuda_stream, plb_context **out);
PLB_API void plb_context_destroy(plb_context *ctx);
PLB_API void *plb_context_stream(plb_context *ctx);
/* Blocks until all enqueued work is done, then checks the kernel status word:
 * returns PLB_ERR_KERNEL if any kernel gave up on a bounded wait. */
PLB_API int plb_synchronize(plb_context *ctx);
/* PCI address of a device ("0000:1b:00.0") into buf (at least 16 bytes): what
 * a host uses to find the CPUs and memory next to the GPU
 * (/sys/bus/pci/devices/<address>/local_cpulist) before it allocates the
 * page-locked buffers of the *_host entry points. */
PLB_API int plb_device_pci_address(int device, char *buf, size_t len);
/* Number of kernels this context has launched so far. */
PLB_API uint64_t plb_launch_count(const plb_context *ctx);
/* PLB_PLAN_* bits (below) that are added to every plan made for a call through
 * this context, also for calls that take no options (plb_matmul): the role of
 * the per-graph option flags a poplin user sets once
 * (lib/poplin/ConvOptions.cpp:40-150).  Used by the tests and for A/B timing. */
PLB_API void plb_context_set_plan_flags(plb_context *ctx, int32_t plan_flags);

/* Device memory helpers for callers without an allocator of their own. */
PLB_API int plb_malloc(plb_context *ctx, size_t bytes, void **d_ptr);
PLB_API int plb_free(plb_context *ctx, void *d_ptr);
PLB_API int plb_memcpy_h2d(plb_context *ctx, void *d_dst, const void *h_src, size_t bytes);
PLB_API int plb_memcpy_d2h(plb_context *ctx, void *h_dst, const void *d_src, size_t bytes);
PLB_API int plb_memset(plb_context *ctx, void *d_dst, int value, size_t bytes);

/* ------------------------------------------------------------------------ */
/* poplin::matMul / matMulGrouped / matMulAcc                                */
/* (include/poplin/MatMul.hpp:110-420, lib/poplin/MatMul.cpp:368-404,        */
/*  782-856; tools/general_matrix_multiply.cpp:355-370)                      */
/* ------------------------------------------------------------------------ */
/* Bit layout of a QUARTER element (poplar::QuarterMetadata::Format,
 * lib/poplin/codelets/convCastSupport.hpp:8-31).  The tensor core decodes the
 * OCP encodings: PLB_F143 = E4M3 (bias 7, largest finite 448), PLB_F152 = E5M2
 * (bias 15, infinities and NaNs as in binary16).  Graphcore's F143 / F152 use
 * a bias one higher: the C++ layer folds that factor 1/2 into the scale. */
typedef enum plb_quarter_format { PLB_F143 = 0, PLB_F152 = 1 } plb_quarter_format;

typedef struct plb_matmul_desc {
  uint32_t groups, m, k, n;
  int32_t input_type;   /* plb_dtype: PLB_HALF, PLB_QUARTER or PLB_FLOAT (each
                           product of float operands is formed from three
                           bfloat16 terms: relative error about 2^-16,
                           accumulation in fp32)                            */
  int32_t output_type;  /* plb_dtype: PLB_HALF or PLB_FLOAT                */
  int32_t partials_type;/* plb_dtype: option "partialsType"; accumulation is
                           always fp32 on this hardware, PLB_HALF is accepted
                           and widened (lib/poplin/ConvValidation.cpp:28-51) */
  int32_t transpose_a;  /* A is stored [g][k][m] ("--left-matrix-op transpose") */
  int32_t transpose_b;  /* B is stored [g][n][k] ("--right-matrix-op transpose",
                           also the layout preArrangeMatMulInputRHS produces) */
  float alpha, beta;    /* D = beta*C + alpha*A*B (matMulAcc: beta=1, alpha=k) */
  int32_t scale_a, scale_b; /* QUARTER metadata exponents: value = stored*2^scale
                               (poplar::QuarterMetadata), range [-32, 31]  */
  int64_t lda, ldb, ldc;/* row strides in elements; 0 = densely packed     */
  int32_t format_a, format_b; /* plb_quarter_format of QUARTER operands
                                 (poplar::QuarterMetadata::Format)          */
} plb_matmul_desc;

/* d_c may be NULL when beta == 0; d_c may alias d_d.  A, B, C, D are
 * [groups][rows][cols] row-major with the leading dimensions above. */
PLB_API int plb_matmul(plb_context *ctx, const plb_matmul_desc *desc, const void *d_a,
               const void *d_b, const void *d_c, void *d_d);
/* Same through host buffers: uploads A, B (and C), runs, downloads D and
 * synchronises.  This is the end-to-end call the benchmark times. */
PLB_API int plb_matmul_host(plb_context *ctx, const plb_matmul_desc *desc, const void *h_a,
                    const void *h_b, const void *h_c, void *h_d);
/* plb_matmul_host without the final synchronisation: copies and kernel are
 * enqueued on the context's stream and the call returns.  The host buffers
 * must be page-locked for the copies to overlap anything, and must stay valid
 * (and h_d unread) until plb_synchronize(ctx).  Successive calls on one
 * context reuse its staging buffers in stream order; alternate between two
 * contexts to overlap one call's download with the next one's upload. */
PLB_API int plb_matmul_host_async(plb_context *ctx, const plb_matmul_desc *desc, const void *h_a,
                          const void *h_b, const void *h_c, void *h_d);

/* ------------------------------------------------------------------------ */
/* poplin::ConvParams (include/poplin/ConvParams.hpp:16-224), flattened.     */
/* Channel counts are per group, as in the reference.                        */
/* ------------------------------------------------------------------------ */
typedef struct plb_conv_params {
  int32_t input_type;  /* plb_dtype */
  int32_t output_type; /* plb_dtype */
  uint32_t num_field_dims; /* 1..3 */
  uint32_t batch;
  uint32_t groups;
  uint32_t in_chans_per_group;
  uint32_t out_chans_per_group;
  uint32_t field[PLB_MAX_FIELD_DIMS];
  uint32_t kernel[PLB_MAX_FIELD_DIMS];
  /* InputTransform of the activations */
  uint32_t in_trunc_lo[PLB_MAX_FIELD_DIMS], in_trunc_hi[PLB_MAX_FIELD_DIMS];
  uint32_t in_dilation[PLB_MAX_FIELD_DIMS];
  uint32_t in_pad_lo[PLB_MAX_FIELD_DIMS], in_pad_hi[PLB_MAX_FIELD_DIMS];
  uint32_t in_flip[PLB_MAX_FIELD_DIMS];
  /* InputTransform of the kernel */
  uint32_t k_trunc_lo[PLB_MAX_FIELD_DIMS], k_trunc_hi[PLB_MAX_FIELD_DIMS];
  uint32_t k_dilation[PLB_MAX_FIELD_DIMS];
  uint32_t k_pad_lo[PLB_MAX_FIELD_DIMS], k_pad_hi[PLB_MAX_FIELD_DIMS];
  uint32_t k_flip[PLB_MAX_FIELD_DIMS];
  /* OutputTransform */
  uint32_t out_trunc_lo[PLB_MAX_FIELD_DIMS], out_trunc_hi[PLB_MAX_FIELD_DIMS];
  uint32_t stride[PLB_MAX_FIELD_DIMS];
  uint32_t out_pad_lo[PLB_MAX_FIELD_DIMS], out_pad_hi[PLB_MAX_FIELD_DIMS];
} plb_conv_params;

/* ConvParams::validate (lib/poplin/ConvParams.cpp:172-266). */
PLB_API int plb_conv_validate(const plb_conv_params *p);
/* ConvParams::getOutputSize (lib/poplin/ConvParams.cpp:670-698). */
PLB_API int plb_conv_output_field(const plb_conv_params *p, uint32_t out_field[PLB_MAX_FIELD_DIMS]);
/* poplin::getInputIndex (lib/poplin/ConvUtil.cpp:234-292): index of the input
 * element read by (output, kernel) in one dimension, or -1 for padding. */
PLB_API int plb_conv_input_index(const plb_conv_params *p, uint32_t dim, uint32_t out_index,
                         uint32_t kernel_index);
/* getNumberOfMACs (lib/poplin/PerformanceEstimation.hpp:1641-1666): products
 * with padding are not counted.  getFwdFlops = 2 * this
 * (lib/poplin/Convolution.cpp:3217-3225). */
PLB_API uint64_t plb_conv_macs(const plb_conv_params *p);

/* Options that change what is computed or how it is planned
 * (lib/poplin/ConvOptions.cpp:105-152).  Zero-initialise for the defaults. */
typedef struct plb_conv_options {
  int32_t pass;          /* plb_pass */
  int32_t partials_type; /* plb_dtype; see plb_matmul_desc.partials_type */
  /* plan constraints this implementation understands; 0 = planner's choice */
  int32_t tile_n;        /* output channels per CTA tile: 64, 128 or 256     */
  int32_t split_k;       /* CTAs that share one output tile (weight update)  */
  int32_t plan_flags;    /* PLB_PLAN_* bits                                   */
  int32_t scale_in;      /* QUARTER metadata exponents of the activations and  */
  int32_t scale_weights; /* the weights: value = stored * 2^scale              */
  int32_t format_in;      /* plb_quarter_format of the activations (or, in the   */
  int32_t format_weights; /* backward pass, the output gradients) and the weights */
  int32_t reserved;
} plb_conv_options;

/* plb_conv_options.plan_flags */
#define PLB_PLAN_FORCE_RESIDENT_WEIGHTS 1 /* keep weights in shared memory even for few tiles */
#define PLB_PLAN_NO_RESIDENT_WEIGHTS 2    /* always stream the weights                        */
#define PLB_PLAN_NO_HALO 4                /* one activation load per filter tap               */
#define PLB_PLAN_NO_CTA_PAIR 8            /* every CTA issues its own 128-row MMAs            */
#define PLB_PLAN_FORCE_CTA_PAIR 16        /* CTA pairs whenever the shape allows them         */
#define PLB_PLAN_NO_TMA_STORE 32          /* plain vector stores in the epilogue              */
#define PLB_PLAN_NO_PDL 64                /* launch without programmatic stream serialization */
#define PLB_PLAN_NO_A_COLLECTOR 128       /* weight update: fetch the outGrad tile per MMA    */
#define PLB_PLAN_NO_DUAL_ISSUE 256        /* one MMA-issuing thread also on short tiles       */

/* out = conv(in, weights) (+ bias), poplin::convolution
 * (include/poplin/Convolution.hpp:345-384, lib/poplin/Convolution.cpp:3128-3215).
 * d_bias may be NULL (poplin::addBias fused, include/poplin/Convolution.hpp:536-544). */
PLB_API int plb_conv_fwd(plb_context *ctx, const plb_conv_params *p, const plb_conv_options *opt,
                 const void *d_in, const void *d_weights, const float *d_bias, void *d_out);
/* The general form behind poplin::convolution(..., transposeAndFlipWeights, ...)
 * (lib/poplin/Convolution.cpp:3067-3126): with transpose_and_flip_weights != 0
 * d_weights holds [G][kernel...][Ci][Co] -- the device layout of the weights of
 * the layer this convolution is the backward pass of -- and is used with its
 * channel axes swapped and its spatial axes flipped, without being rearranged
 * in memory (half; quarter weights are transposed into scratch first). */
PLB_API int plb_convolution(plb_context *ctx, const plb_conv_params *p, const plb_conv_options *opt,
                    const void *d_in, const void *d_weights, const float *d_bias, void *d_out,
                    int transpose_and_flip_weights);
/* Gradient w.r.t. the input from the FORWARD pass's params and weights:
 * what convolution(zDeltas, weights, getGradientParams(p), true) computes
 * (lib/poplin/ConvUtil.cpp:728-795, lib/poplin/Convolution.cpp:3077-3086). */
PLB_API int plb_conv_bwd(plb_context *ctx, const plb_conv_params *p, const plb_conv_options *opt,
                 const void *d_out_grads, const void *d_weights, void *d_in_grads);
/* Weight gradient of the FORWARD pass's params, poplin::calculateWeightDeltas
 * (include/poplin/Convolution.hpp:460-466, lib/poplin/Convolution.cpp:3436-3507).
 * d_weight_grads has the device weights layout and type p->input_type
 * (lib/poplin/Convolution.cpp:3537); if d_weight_grads_f32 is not NULL the
 * fp32 sums are also left there (what a multi-GPU caller all-reduces). */
PLB_API int plb_conv_wu(plb_context *ctx, const plb_conv_params *p, const plb_conv_options *opt,
                const void *d_acts, const void *d_out_grads, void *d_weight_grads,
                float *d_weight_grads_f32);
/* The weight update of a batch-sharded layer on several GPUs of one box, with the
 * sum over the ranks fused into the split-K reduction: every rank passes its
 * batch slice, and d_weight_grads / d_weight_grads_f32 receive the gradient of
 * the WHOLE batch on every rank (bit-identical on all of them: the ranks' sums
 * are added in rank order).  The reduction kernel writes this rank's gradient
 * chunk by chunk into a peer-addressable buffer, flags each chunk to the peers
 * and adds the peers' chunks with NVLink peer loads as their flags arrive, so the
 * exchange overlaps the reduction instead of following it as a second kernel.
 * This replaces plb_conv_wu + plb_allreduce_f32_p2p; the reference has no
 * counterpart (it spreads one convolution over IPU tiles inside one graph,
 * lib/poplin/ConvPlan.hpp:28-77).
 *   d_peer_grads[r]  rank r's gradient buffer: groups * kernel elements * Co * Ci
 *                    floats, 16-byte aligned, addressable from this GPU; the
 *                    caller alternates between two such buffers on successive
 *                    steps (a peer may still be reading the previous step's);
 *   d_peer_flags[r]  rank r's flag area, plb_conv_wu_allreduce_flag_bytes(p)
 *                    bytes, zero before the first step, used only by this call;
 *   epoch            1, 2, 3, ... the same on every rank for the same step.
 * Every rank must make the call (a rank with an empty slice contributes zeros).
 * Waits are bounded: a peer that never signals is reported through the context's
 * status word (plb_synchronize), nothing hangs.  Layers that plb_conv_wu runs
 * through a preparatory pass (channel counts not a multiple of 8, input dilation
 * or flip, truncated or flipped kernels, 3-D fields) and gradients larger than
 * 4 chunks of 2 KiB per SM return PLB_ERR_UNSUPPORTED: use the two-call form. */
PLB_API int plb_conv_wu_allreduce(plb_context *ctx, const plb_conv_params *p,
                          const plb_conv_options *opt, const void *d_acts, const void *d_out_grads,
                          int32_t rank, int32_t world, void *const *d_peer_grads,
                          void *const *d_peer_flags, uint32_t epoch, void *d_weight_grads,
                          float *d_weight_grads_f32);
PLB_API uint64_t plb_conv_wu_allreduce_flag_bytes(const plb_conv_params *p);
/* The same with the sum shared out: chunk c of the gradient is added (in rank
 * order) by rank c mod world alone, which leaves it in its result buffer and
 * flags it; the other ranks fetch the finished chunk from there.  Per rank
 * 2 * (world - 1) / world of the gradient crosses NVLink instead of world - 1
 * times, at the price of a second flag per chunk: the form for many ranks.
 *   d_peer_results[r]  rank r's result buffer, the size of a gradient buffer,
 *                      16-byte aligned, addressable from this GPU (one buffer:
 *                      a rank's next step cannot begin before the others have
 *                      fetched this step's sums from it).
 * Flags: the same area as plb_conv_wu_allreduce (its size covers both forms). */
PLB_API int plb_conv_wu_allreduce_owners(plb_context *ctx, const plb_conv_params *p,
                          const plb_conv_options *opt, const void *d_acts, const void *d_out_grads,
                          int32_t rank, int32_t world, void *const *d_peer_grads,
                          void *const *d_peer_results, void *const *d_peer_flags, uint32_t epoch,
                          void *d_weight_grads, float *d_weight_grads_f32);
/* The same weight gradient for callers that cannot allocate device memory when
 * they need it (code running under an allocator that owns all device memory or
 * inside its hooks, loops that may not take the allocator's lock, processes with
 * a memory budget fixed at start-up).  This entry point has no counterpart in the
 * reference.  It calls no cudaMalloc / cudaFree: the split-K partial sums live in
 * a 32 MiB array that is part of the library's device image (every GPU that loads
 * the library holds it until the process exits), the caller passes the device
 * ordinal, the CUDA stream (cudaStream_t as void*) and all input / output
 * buffers.  Limits and rules:
 *  - one group's fp32 gradient (kernel elements * Co * Ci * 4 bytes) must fit in
 *    32 MiB, else PLB_ERR_UNSUPPORTED; fewer K splits are used than plb_conv_wu
 *    would choose when only fewer fit;
 *  - it runs none of the preparatory passes plb_conv_wu has (each needs scratch
 *    memory of its own): channel counts per group must be multiples of 8, and
 *    float operands, 3-D fields, input dilation or flip, and truncated or
 *    flipped kernels are refused with PLB_ERR_UNSUPPORTED and a message naming
 *    plb_conv_wu;
 *  - the first call on a device looks up the array's device address (and sets a
 *    kernel attribute): make that first call before any stream capture;
 *  - all calls share the one array: calls that overlap on the GPU (different
 *    streams or threads) race.  The call synchronises the stream before it
 *    returns and reports a kernel failure as PLB_ERR_KERNEL. */
PLB_API int plb_conv_wu_static_scratch(int device, void *cuda_stream, const plb_conv_params *p,
                               const plb_conv_options *opt, const void *d_acts,
                               const void *d_out_grads, void *d_weight_grads,
                               float *d_weight_grads_f32);
/* All-reduce (sum) of `count` fp32 values over NVLink peer memory, fused with
 * the cast to half: the multi-GPU step of the weight update.  No counterpart in
 * the reference (which spreads one convolution over IPU tiles in one graph);
 * it replaces ncclAllReduce + cast for this small message.
 *   d_buffers[r]     rank r's input, addressable from this GPU (symmetric /
 *                    IPC-mapped memory, one process per GPU), 16-byte aligned;
 *   d_signal_pads[r] rank r's signal pad: plb_allreduce_p2p_signal_bytes(world)
 *                    bytes, zero before the first call, used only by this call;
 *   epoch            1, 2, 3, ... the same on every rank for the same step.
 * The caller must alternate between two input buffers on successive epochs (a
 * peer may still be reading the previous one).  Every rank must make the call:
 * the kernel waits, with a cycle budget, for all peers' flags and reports a
 * missing peer through the context's status word (plb_synchronize).  Sums are
 * formed in rank order, so all ranks get identical bits.  Either output may be
 * null. */
PLB_API int plb_allreduce_f32_p2p(plb_context *ctx, int32_t rank, int32_t world,
                          const void *const *d_buffers, void *const *d_signal_pads,
                          uint32_t epoch, size_t count, float *d_out_f32, void *d_out_half);
/* The same sum as a reduce-scatter followed by an all-gather inside one kernel
 * per rank: rank r adds slice r of every rank's input (peer loads, rank order)
 * and stores the sums into every rank's result buffer (peer stores); after a
 * second round of flags every rank reads its own result buffer and writes the
 * fp32 sum and / or its cast.  Per rank (N - 1) / N of the vector crosses
 * NVLink in each direction instead of N - 1 times the vector inbound, which
 * is what pays from about four ranks on; results are bit-identical to
 * plb_allreduce_f32_p2p's.  No counterpart in the reference (see above).
 *   d_inputs[r]   rank r's fp32 vector, `count` elements, peer-addressable;
 *   d_results[r]  rank r's result buffer, `count` elements, peer-addressable,
 *                 distinct from the inputs;
 *   d_signal_pads, epoch as above (the same pads may serve both calls).
 * One input and one result buffer suffice: the second flag round tells a rank
 * that all peers have read its input, the next call's first round that all
 * have consumed their results.  Calls on one set of buffers must not overlap. */
PLB_API int plb_allreduce_f32_p2p_rs(plb_context *ctx, int32_t rank, int32_t world,
                             const void *const *d_inputs, void *const *d_results,
                             void *const *d_signal_pads, uint32_t epoch, size_t count,
                             float *d_out_f32, void *d_out_half);
PLB_API uint32_t plb_allreduce_p2p_signal_bytes(int32_t world);
/* weights += scale * weight_grads_f32, cast to the weights' type
 * (popops::scaledAddTo in convolutionWeightUpdate, lib/poplin/Convolution.cpp:3509-3522). */
PLB_API int plb_scaled_add_to(plb_context *ctx, int32_t dtype, void *d_weights,
                      const float *d_deltas_f32, float scale, size_t count);
/* biases[c] += scale * sum over pixels of out_grads[pixel][c] on device-layout
 * output gradients, sums in fp32 (poplin::convolutionBiasUpdate,
 * include/poplin/Convolution.hpp:536-561; a reduce with update = true and the
 * given scale, lib/poplin/Convolution.cpp:3601-3637). */
PLB_API int plb_conv_bias_update(plb_context *ctx, int32_t acts_dtype, const void *d_out_grads,
                         uint64_t pixels, uint32_t chans, int32_t bias_dtype, void *d_biases,
                         float scale);
/* acts[pixel][c] += biases[c] on device-layout activations (poplin::addBias,
 * include/poplin/Convolution.hpp:570-572); biases have the activations' type. */
PLB_API int plb_add_bias(plb_context *ctx, int32_t dtype, void *d_acts, const void *d_biases,
                 uint64_t pixels, uint32_t chans);
/* fp32 -> half/float cast of a buffer (popops::cast after a reduction). */
PLB_API int plb_cast_from_f32(plb_context *ctx, int32_t dtype, void *d_dst, const float *d_src,
                      size_t count);

/* ------------------------------------------------------------------------ */
/* Batch normalisation of a convolution's output (include/poplin/Norms.hpp:   */
/* 33-334, lib/poplin/Norms.cpp).  Activations are in the device layout        */
/* [pixels][chans]; statistics and parameters are per channel; dtype is        */
/* PLB_HALF or PLB_FLOAT; sums are formed in fp32 in a fixed order.            */
/* ------------------------------------------------------------------------ */
/* First and second moments per channel, times `scale` (1 / pixels, or
 * 1 / (pixels of all replicas) before a caller's own all-reduce):
 *   d_centre == NULL: d_mean[c] (dtype) = scale * sum x, d_power[c] (fp32) =
 *                     scale * sum x^2  (popops::reduceMany ADD / SQUARE_ADD,
 *                     lib/poplin/Norms.cpp:225-242);
 *   d_centre != NULL: d_power[c] = scale * sum (x - d_centre[c])^2, the
 *                     "stable" estimator (:205-223); d_mean is not written. */
PLB_API int plb_norm_moments(plb_context *ctx, int32_t dtype, const void *d_acts, uint64_t pixels,
                     uint32_t chans, float scale, const void *d_centre, void *d_mean,
                     float *d_power);
/* d_inv_std[c] = 1 / sqrt((power - mean^2 + eps) * scale_var), or with `stable`
 * 1 / sqrt((power + eps) * scale_var): the InverseStdDeviation vertex
 * (lib/poplin/codelets/InverseStdDeviation.cpp:33-55). */
PLB_API int plb_norm_inv_std_dev(plb_context *ctx, int32_t dtype, const void *d_mean,
                         const float *d_power, uint32_t chans, float eps, float scale_var,
                         int stable, void *d_inv_std);
/* Mean and inverse standard deviation in one call (poplin::normStatistics with
 * the default estimator, Norms.hpp:64-72): plb_norm_moments with scale =
 * 1 / pixels, and plb_norm_inv_std_dev's arithmetic applied by the kernel that
 * finishes the sums; the same bits as the two calls.  d_power may be NULL. */
PLB_API int plb_norm_statistics(plb_context *ctx, int32_t dtype, const void *d_acts, uint64_t pixels,
                        uint32_t chans, float eps, float scale_var, void *d_mean, void *d_inv_std,
                        float *d_power);
/* Whitening followed by scale and shift in one pass over the activations
 * (poplin::normWhiten then poplin::normalise): out = w * gamma[c] + beta[c] with
 * w = (acts - mean[c]) * inv_std[c] rounded to the activations' type, as the two
 * calls would store it; d_whitened (may be NULL) receives w. */
PLB_API int plb_norm_normalise(plb_context *ctx, int32_t dtype, const void *d_acts, const void *d_mean,
                       const void *d_inv_std, const void *d_gamma, const void *d_beta,
                       uint64_t pixels, uint32_t chans, void *d_whitened, void *d_out);
/* out = (acts - mean[c]) * inv_std[c]  (poplin::normWhiten, Norms.hpp:212-216). */
PLB_API int plb_norm_whiten(plb_context *ctx, int32_t dtype, const void *d_acts, const void *d_mean,
                    const void *d_inv_std, uint64_t pixels, uint32_t chans, void *d_out);
/* out = acts * scale[c] + shift[c]; d_shift == NULL: out = acts * scale[c]
 * (poplin::normalise with gamma / beta, Norms.hpp:229-234; poplin::normGradients
 * with gamma alone, :266-270). */
PLB_API int plb_norm_scale_shift(plb_context *ctx, int32_t dtype, const void *d_acts,
                         const void *d_scale, const void *d_shift, uint64_t pixels,
                         uint32_t chans, void *d_out);
/* gamma_delta[c] = scale * sum whitened * grads, beta_delta[c] = scale * sum grads
 * (poplin::normParamGradients, Norms.hpp:249-254), in dtype and / or in fp32;
 * any of the four outputs may be NULL. */
PLB_API int plb_norm_param_gradients(plb_context *ctx, int32_t dtype, const void *d_whitened,
                             const void *d_grads, uint64_t pixels, uint32_t chans, float scale,
                             void *d_gamma_delta, void *d_beta_delta, float *d_gamma_delta_f32,
                             float *d_beta_delta_f32);
/* out = (grads - whitened * mean_c(whitened * grads) - mean_c(grads)) * inv_std[c]
 * (poplin::normStatisticsGradients, Norms.hpp:289-294).  With d_var_delta and
 * d_mean_delta (dtype, per channel; both or neither) the two means are taken
 * from the caller instead, already negated and reduced over the replicas:
 * out = (grads + whitened * var_delta[c] + mean_delta[c]) * inv_std[c]
 * (distributedNormStatisticsGradients, Norms.hpp:324-330). */
PLB_API int plb_norm_statistics_gradients(plb_context *ctx, int32_t dtype, const void *d_whitened,
                                  const void *d_grads, const void *d_inv_std,
                                  const void *d_var_delta, const void *d_mean_delta,
                                  uint64_t pixels, uint32_t chans, void *d_out);

/* Host-buffer variants (device layouts, host memory): upload, run, download,
 * synchronise. */
PLB_API int plb_conv_fwd_host(plb_context *ctx, const plb_conv_params *p, const plb_conv_options *opt,
                      const void *h_in, const void *h_weights, const float *h_bias, void *h_out);
/* Without the final synchronisation (see plb_matmul_host_async). */
PLB_API int plb_conv_fwd_host_async(plb_context *ctx, const plb_conv_params *p,
                            const plb_conv_options *opt, const void *h_in, const void *h_weights,
                            const float *h_bias, void *h_out);

/* ------------------------------------------------------------------------ */
/* Layout changes between poplin's external shapes and the device layouts.   */
/* ------------------------------------------------------------------------ */
/* [N][C][field...] -> [N][field...][C] and back; elem_bytes is 1, 2 or 4. */
PLB_API int plb_rearrange_acts_to_device(plb_context *ctx, uint32_t elem_bytes, uint32_t batch,
                                 uint32_t chans, uint64_t field_elems, const void *d_src,
                                 void *d_dst);
PLB_API int plb_rearrange_acts_from_device(plb_context *ctx, uint32_t elem_bytes, uint32_t batch,
                                   uint32_t chans, uint64_t field_elems, const void *d_src,
                                   void *d_dst);
/* [G][Co][Ci][kernel...] -> [G][kernel...][Co][Ci] and back. */
PLB_API int plb_rearrange_weights_to_device(plb_context *ctx, uint32_t elem_bytes, uint32_t groups,
                                    uint32_t out_chans, uint32_t in_chans, uint64_t kernel_elems,
                                    const void *d_src, void *d_dst);
PLB_API int plb_rearrange_weights_from_device(plb_context *ctx, uint32_t elem_bytes, uint32_t groups,
                                      uint32_t out_chans, uint32_t in_chans,
                                      uint64_t kernel_elems, const void *d_src, void *d_dst);
/* poplin::weightsTransposeChansFlipXY on device-layout weights
 * (include/poplin/Convolution.hpp:434-439): [G][k...][Co][Ci] ->
 * [G][flipped k...][Ci][Co]. */
PLB_API int plb_weights_transpose_chans_flip_xy(plb_context *ctx, uint32_t elem_bytes, uint32_t groups,
                                        uint32_t out_chans, uint32_t in_chans,
                                        uint64_t kernel_elems, const void *d_src, void *d_dst);
/* Row-major matrix transpose [rows][cols] -> [cols][rows] per group
 * (poplin::transposeGroupedMatrix, include/poplin/MatMul.hpp:600-606). */
PLB_API int plb_transpose_matrix(plb_context *ctx, uint32_t elem_bytes, uint32_t groups, uint32_t rows,
                         uint32_t cols, const void *d_src, void *d_dst);

/* General strided element copy dst[i0..] = src[i0..] over a common logical
 * shape (rank <= 8); strides are in elements and may be zero (broadcast source)
 * or negative.  This is what a poplar::program::Copy between two tensor views
 * lowers to, and how host data in logical order reaches a device layout. */
#define PLB_MAX_VIEW_RANK 8
PLB_API int plb_copy_strided(plb_context *ctx, uint32_t elem_bytes, uint32_t rank, const uint64_t *shape,
                     const int64_t *src_strides, const int64_t *dst_strides, const void *d_src,
                     void *d_dst);
/* Fills `count` elements of type `dtype` (PLB_HALF / PLB_FLOAT) with `value`. */
PLB_API int plb_fill(plb_context *ctx, int32_t dtype, void *d_dst, float value, size_t count);
/* Streaming probe of the memory system, for roofline denominators that match a
 * kernel's mix of reads and writes: one grid-stride kernel of 16-byte accesses
 * that reads `reads` (0 or 1) and writes `writes` (0..4) streams of `bytes`
 * bytes each (d_in: `bytes`; d_out: writes * bytes; both 16-byte aligned).
 * Timed by the caller (plb_timer_start / plb_timer_stop). */
PLB_API int plb_memory_mix_probe(plb_context *ctx, int32_t reads, int32_t writes, size_t bytes,
                         const void *d_in, void *d_out);
/* Device-side stopwatch on the context's stream (CUDA events). */
PLB_API int plb_timer_start(plb_context *ctx);
PLB_API int plb_timer_stop(plb_context *ctx, float *milliseconds);

/* ------------------------------------------------------------------------ */
/* Planner: the CTA-level plan chosen for a contraction (the role of         */
/* poplin::getPlan, lib/poplin/ConvPlan.cpp:1877-1923, and what               */
/* poplin::reportPlanInfo prints, include/poplin/Convolution.hpp:584-594).    */
/* ------------------------------------------------------------------------ */
typedef struct plb_plan {
  int32_t kernel;      /* 0 = implicit GEMM (fwd/bwd/matmul), 1 = weight update, 2 = small-channel */
  int32_t tile_m;      /* output pixels (rows) per CTA tile                  */
  int32_t tile_n;      /* output channels (columns) per CTA tile             */
  int32_t tile_k_bytes;/* bytes of K per pipeline stage                      */
  int32_t box_w, box_h, box_n; /* pixel box of one activation TMA load       */
  int32_t stages;      /* shared-memory pipeline depth                       */
  int32_t split_k;     /* CTAs per output tile                               */
  int32_t grid;        /* CTAs launched                                      */
  int32_t tiles;       /* output tiles                                       */
  int32_t b_mn_major;  /* right operand fed as an MN-major matrix            */
  int32_t resident_weights; /* weights loaded once per CTA and kept in shared memory */
  int32_t halo_rows;   /* extra input rows per activation load that let one load
                          serve every vertical filter tap (0 = one load per tap) */
  int32_t cta_pair;    /* 1 = clusters of two CTAs share 256-row tensor-core instructions */
  int32_t reserved;
  uint64_t flops;      /* 2 * MACs (padding excluded)                        */
  uint64_t bytes;      /* operands read once + output written once           */
  uint64_t workspace_bytes;
} plb_plan;

PLB_API int plb_matmul_plan(const plb_matmul_desc *desc, plb_plan *plan);
PLB_API int plb_conv_plan(const plb_conv_params *p, const plb_conv_options *opt, int32_t pass,
                  plb_plan *plan);
/* Plan of the weight-update pass of the FORWARD parameters `p`
 * (poplin::reportWeightUpdatePlanInfo, include/poplin/Convolution.hpp:690-694). */
PLB_API int plb_conv_wu_plan(const plb_conv_params *p, const plb_conv_options *opt, plb_plan *plan);

#ifdef __cplusplus
}
#endif
#endif /* POPLIBS_B200_H */
