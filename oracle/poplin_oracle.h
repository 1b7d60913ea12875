/*
 * CPU oracle for the poplin dense-contraction path.  TEST INFRASTRUCTURE ONLY.
 *
 * This is a plain-C restatement of the reference's double-precision CPU models
 * (poplibs_test::conv::{convolution, convolutionBackward, weightUpdate},
 * lib/poplibs_test/Convolution.cpp:455-895; poplibs_test::gemm::
 * generalMatrixMultiply, lib/poplibs_test/GeneralMatrixMultiply.cpp:190-283)
 * and of the element comparison rule poplibs_test::checkIsClose
 * (lib/poplibs_test/Util.cpp:198-217, 316-348).  Nothing on the product path
 * may link, load or call it: it is the checker for the GPU kernels and the
 * timed CPU baseline, never the thing shipped.
 *
 * Parity status: pinned.  The restatement is checked (tests/test_oracle.py)
 * against the reference's own sources compiled from where they lie
 * (oracle/_ref, see oracle/Makefile) on randomised parameter sets, and against
 * the golden vectors under tests/golden/ that were produced by that build.
 */
#ifndef POPLIN_ORACLE_H
#define POPLIN_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ORACLE_MAX_FIELD_DIMS 3

/* One spatial dimension's worth of poplin::ConvParams transforms
 * (include/poplin/ConvParams.hpp:16-140), flattened to plain integers. */
typedef struct oracle_conv_params {
  uint32_t num_field_dims; /* 1..3 */
  uint32_t batch;
  uint32_t groups;
  uint32_t in_chans_per_group;
  uint32_t out_chans_per_group;
  uint32_t field[ORACLE_MAX_FIELD_DIMS];
  uint32_t kernel[ORACLE_MAX_FIELD_DIMS];
  /* input transform: truncate, dilate, pad, flip */
  uint32_t in_trunc_lo[ORACLE_MAX_FIELD_DIMS];
  uint32_t in_trunc_hi[ORACLE_MAX_FIELD_DIMS];
  uint32_t in_dilation[ORACLE_MAX_FIELD_DIMS];
  uint32_t in_pad_lo[ORACLE_MAX_FIELD_DIMS];
  uint32_t in_pad_hi[ORACLE_MAX_FIELD_DIMS];
  uint32_t in_flip[ORACLE_MAX_FIELD_DIMS];
  /* kernel transform */
  uint32_t k_trunc_lo[ORACLE_MAX_FIELD_DIMS];
  uint32_t k_trunc_hi[ORACLE_MAX_FIELD_DIMS];
  uint32_t k_dilation[ORACLE_MAX_FIELD_DIMS];
  uint32_t k_pad_lo[ORACLE_MAX_FIELD_DIMS];
  uint32_t k_pad_hi[ORACLE_MAX_FIELD_DIMS];
  uint32_t k_flip[ORACLE_MAX_FIELD_DIMS];
  /* output transform: truncate, stride, pad */
  uint32_t out_trunc_lo[ORACLE_MAX_FIELD_DIMS];
  uint32_t out_trunc_hi[ORACLE_MAX_FIELD_DIMS];
  uint32_t stride[ORACLE_MAX_FIELD_DIMS];
  uint32_t out_pad_lo[ORACLE_MAX_FIELD_DIMS];
  uint32_t out_pad_hi[ORACLE_MAX_FIELD_DIMS];
} oracle_conv_params;

/* Output field size of one dimension; returns -1 if the parameters describe
 * no valid convolution (negative intermediate size). */
int oracle_conv_out_size(const oracle_conv_params *p, uint32_t dim);

/* Index of the input element that output element `out_idx` reads through
 * kernel element `k_idx` in dimension `dim`, or -1 when that product is with
 * padding / a dilation hole / a truncated element.  Restates
 * poplin::getInputIndex (lib/poplin/ConvUtil.cpp:234-292) for one dimension
 * and agrees with the materialise-then-convolve model of the reference. */
int oracle_conv_input_index(const oracle_conv_params *p, uint32_t dim,
                            uint32_t out_idx, uint32_t k_idx);

/* Layouts are the reference model's: activations [batch][G*C][prod(field)],
 * weights [G][Co][Ci][prod(kernel)], biases [G*Co] (may be NULL => zero).
 * All return 0 on success, non-zero on bad parameters.  `threads` <= 0 means
 * "all host cores". */
int oracle_conv_fwd(const oracle_conv_params *p, const double *in,
                    const double *weights, const double *biases, double *out,
                    int threads);
int oracle_conv_bwd(const oracle_conv_params *p, const double *out_grads,
                    const double *weights, double *in_grads, int threads);
/* Weight gradient dW (no learning-rate update): dW[g][oc][ic][k] and, when
 * bias_grads != NULL, bias_grads[oc] = sum of out_grads over batch and field.
 * The reference's weightUpdate computes weights += lr * -dW; callers get dW
 * itself from it with weights = 0, lr = -1. */
int oracle_conv_wu(const oracle_conv_params *p, const double *acts,
                   const double *out_grads, double *weight_grads,
                   double *bias_grads, int threads);

/* D[g] = beta*C[g] + alpha*op(A[g])*op(B[g]); op(A) is m x k, op(B) is k x n,
 * all row-major; C may be NULL when beta == 0.  alpha and beta are float in
 * the reference's signature and are widened to double here the same way. */
int oracle_gemm(uint32_t groups, uint32_t m, uint32_t k, uint32_t n,
                const double *a, const double *b, const double *c, double *d,
                float alpha, float beta, int transpose_a, int transpose_b,
                int threads);

/* poplibs_test::checkIsClose for one pair. */
int oracle_is_close(double actual, double expected, double rel_tol,
                    double abs_tol);
/* Array form: returns the number of failing elements; *first_bad (optional)
 * receives the index of the first one, *max_rel (optional) the largest
 * |actual-expected|/|expected| seen over elements with expected != 0. */
size_t oracle_check_is_close(const double *actual, const double *expected,
                             size_t n, double rel_tol, double abs_tol,
                             size_t *first_bad, double *max_rel);

/* IEEE binary16 and E4M3 (OCP "FN": bias 7, no infinities, max 448) helpers
 * used to condition test data exactly as the device sees it. */
double oracle_round_to_half(double x);
uint8_t oracle_e4m3_from_double(double x); /* RNE, saturating to +-448 */
double oracle_e4m3_to_double(uint8_t bits);

/* Batch normalisation over activations [batch][chans][field]
 * (lib/poplibs_test/Norms.cpp, NormType::BatchNorm: statistics per channel
 * over the batch and the field).
 * Statistics: mean[c] and inv_std[c] = 1 / sqrt(var[c] + eps), var biased or
 * (unbiased != 0) scaled by n / (n - 1); with stable != 0 the variance is the
 * mean of squared deviations, else E[x^2] - mean^2 (:38-85). */
void oracle_norm_statistics(const double *acts, uint32_t batch, uint32_t chans,
                            uint32_t field, double eps, int unbiased,
                            int stable, double *mean, double *inv_std);
/* whitened = (acts - mean[c]) * inv_std[c]; out = gamma[c] * whitened + beta[c]
 * (:147-176). */
void oracle_norm_normalise(const double *acts, const double *gamma,
                           const double *beta, const double *mean,
                           const double *inv_std, uint32_t batch,
                           uint32_t chans, uint32_t field, double *out,
                           double *whitened);
/* grads_out = (g - w * mean_c(w * g) - mean_c(g)) * gamma[c] * inv_std[c]
 * (:226-262). */
void oracle_norm_gradients(const double *whitened, const double *grads_in,
                           const double *inv_std, const double *gamma,
                           uint32_t batch, uint32_t chans, uint32_t field,
                           double *grads_out);
/* beta[c] -= lr * sum_c(g); gamma[c] -= lr * sum_c(w * g) (:346-375). */
void oracle_norm_param_update(const double *whitened, const double *grads_in,
                              double learning_rate, uint32_t batch,
                              uint32_t chans, uint32_t field, double *gamma,
                              double *beta);

int oracle_num_threads(void);

#ifdef __cplusplus
}
#endif
#endif /* POPLIN_ORACLE_H */
