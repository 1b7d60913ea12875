/*
 * CPU oracle for the poplin dense-contraction path.  TEST INFRASTRUCTURE ONLY;
 * see poplin_oracle.h for what it restates and how it is pinned.
 *
 * The reference model (lib/poplibs_test/Convolution.cpp) materialises the
 * truncated -> dilated -> padded -> flipped copies of input and kernel
 * (:125-195), runs a stride-1 "valid" correlation over them (:536-559), and
 * then applies the inverse of an activations transform to truncate / stride /
 * pad the result (:561-564).  Here the same arithmetic is expressed through a
 * per-dimension index table
 *     input_index(out, k)  in  {-1, 0 .. field-1}
 * so that no padded copies are built and stride-s layers do not pay for the
 * s*s outputs the reference computes and throws away.  The forward, backward
 * (:577-722) and weight-update (:724-895) passes all walk the same
 * (output element, kernel element) -> input element relation.
 *
 * Everything is double precision, like the reference.
 */
#include "poplin_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>
#include <unistd.h>

int oracle_num_threads(void) {
  long n = sysconf(_SC_NPROCESSORS_ONLN);
  const char *env = getenv("ORACLE_NUM_THREADS");
  if (env && atoi(env) > 0)
    n = atoi(env);
  return n < 1 ? 1 : (n > 256 ? 256 : (int)n);
}

/* Minimal fork-join helper: body(tid, nthreads, ctx) on nthreads threads. */
typedef void (*par_body)(int tid, int nthreads, void *ctx);
typedef struct {
  par_body body;
  void *ctx;
  int tid, nthreads;
} par_arg;

static void *par_trampoline(void *v) {
  par_arg *a = v;
  a->body(a->tid, a->nthreads, a->ctx);
  return NULL;
}

static void parallel_run(int nthreads, par_body body, void *ctx) {
  if (nthreads <= 1) {
    body(0, 1, ctx);
    return;
  }
  pthread_t *th = malloc(sizeof(pthread_t) * (size_t)nthreads);
  par_arg *args = malloc(sizeof(par_arg) * (size_t)nthreads);
  char *started = calloc((size_t)nthreads, 1);
  for (int t = 0; t < nthreads; ++t) {
    args[t].body = body;
    args[t].ctx = ctx;
    args[t].tid = t;
    args[t].nthreads = nthreads;
  }
  for (int t = 1; t < nthreads; ++t) {
    if (pthread_create(&th[t], NULL, par_trampoline, &args[t]) == 0)
      started[t] = 1;
    else
      par_trampoline(&args[t]); /* could not spawn: run it here */
  }
  par_trampoline(&args[0]);
  for (int t = 1; t < nthreads; ++t)
    if (started[t])
      pthread_join(th[t], NULL);
  free(started);
  free(th);
  free(args);
}

static int pick_threads(int threads) {
  int max = oracle_num_threads();
  if (threads <= 0 || threads > max)
    return max;
  return threads;
}

/* ---- per-dimension size algebra (Convolution.cpp:21-75) ---------------- */

static long dilated_size(long size, long dilation) {
  return size == 0 ? 0 : 1 + (size - 1) * dilation;
}

static long transformed_size(long size, long trunc_lo, long trunc_hi,
                             long dilation, long pad_lo, long pad_hi) {
  long truncated = size - (trunc_lo + trunc_hi);
  if (truncated < 0)
    return -1;
  return pad_lo + dilated_size(truncated, dilation) + pad_hi;
}

static long padded_in_size(const oracle_conv_params *p, uint32_t d) {
  return transformed_size(p->field[d], p->in_trunc_lo[d], p->in_trunc_hi[d],
                          p->in_dilation[d], p->in_pad_lo[d], p->in_pad_hi[d]);
}

static long padded_kernel_size(const oracle_conv_params *p, uint32_t d) {
  return transformed_size(p->kernel[d], p->k_trunc_lo[d], p->k_trunc_hi[d],
                          p->k_dilation[d], p->k_pad_lo[d], p->k_pad_hi[d]);
}

int oracle_conv_out_size(const oracle_conv_params *p, uint32_t d) {
  if (d >= p->num_field_dims || p->stride[d] == 0 || p->in_dilation[d] == 0 ||
      p->k_dilation[d] == 0)
    return -1;
  long in = padded_in_size(p, d), k = padded_kernel_size(p, d);
  if (in < 0 || k < 0 || k > in || k == 0)
    return -1;
  long conv_out = in - k + 1;
  long truncated = conv_out - ((long)p->out_trunc_lo[d] + p->out_trunc_hi[d]);
  if (truncated < 0)
    return -1;
  long strided = (truncated + p->stride[d] - 1) / p->stride[d];
  return (int)(p->out_pad_lo[d] + strided + p->out_pad_hi[d]);
}

int oracle_conv_input_index(const oracle_conv_params *p, uint32_t d,
                            uint32_t out_idx, uint32_t k_idx) {
  int out_size = oracle_conv_out_size(p, d);
  if (out_size < 0 || (int)out_idx >= out_size || k_idx >= p->kernel[d])
    return -1;
  long in_padded = padded_in_size(p, d);
  long k_padded = padded_kernel_size(p, d);
  /* output padding contributes zeros only */
  if (out_idx < p->out_pad_lo[d] ||
      (long)out_idx >= (long)out_size - (long)p->out_pad_hi[d])
    return -1;
  long conv_idx =
      (long)p->out_trunc_lo[d] + (long)(out_idx - p->out_pad_lo[d]) * p->stride[d];
  /* kernel element -> position in the transformed kernel */
  if (k_idx < p->k_trunc_lo[d] || k_idx >= p->kernel[d] - p->k_trunc_hi[d])
    return -1;
  long kq = (long)(k_idx - p->k_trunc_lo[d]) * p->k_dilation[d] + p->k_pad_lo[d];
  if (p->k_flip[d])
    kq = k_padded - 1 - kq;
  /* position in the transformed input, then undo flip / pad / dilate / trunc */
  long pos = conv_idx + kq;
  if (pos < 0 || pos >= in_padded)
    return -1;
  if (p->in_flip[d])
    pos = in_padded - 1 - pos;
  pos -= p->in_pad_lo[d];
  long truncated = (long)p->field[d] - ((long)p->in_trunc_lo[d] + p->in_trunc_hi[d]);
  long dil = dilated_size(truncated, p->in_dilation[d]);
  if (pos < 0 || pos >= dil || pos % p->in_dilation[d] != 0)
    return -1;
  return (int)(pos / p->in_dilation[d] + p->in_trunc_lo[d]);
}

/* ---- shared geometry --------------------------------------------------- */

typedef struct {
  uint32_t nd;
  size_t in_elems, k_elems, out_elems;
  uint32_t out_size[ORACLE_MAX_FIELD_DIMS];
  /* link[o * k_elems + k] = flat input element or -1 */
  int32_t *link;
} geometry;

static int build_geometry(const oracle_conv_params *p, geometry *g) {
  memset(g, 0, sizeof *g);
  if (p->num_field_dims < 1 || p->num_field_dims > ORACLE_MAX_FIELD_DIMS)
    return 1;
  g->nd = p->num_field_dims;
  g->in_elems = g->k_elems = g->out_elems = 1;
  int32_t *tab[ORACLE_MAX_FIELD_DIMS] = {0};
  for (uint32_t d = 0; d < g->nd; ++d) {
    int os = oracle_conv_out_size(p, d);
    if (os < 0)
      return 2;
    g->out_size[d] = (uint32_t)os;
    g->in_elems *= p->field[d];
    g->k_elems *= p->kernel[d];
    g->out_elems *= (size_t)os;
  }
  if (g->out_elems * g->k_elems == 0) {
    g->link = NULL;
    return 0;
  }
  for (uint32_t d = 0; d < g->nd; ++d) {
    tab[d] = malloc(sizeof(int32_t) * (size_t)g->out_size[d] * p->kernel[d]);
    for (uint32_t o = 0; o < g->out_size[d]; ++o)
      for (uint32_t k = 0; k < p->kernel[d]; ++k)
        tab[d][(size_t)o * p->kernel[d] + k] =
            oracle_conv_input_index(p, d, o, k);
  }
  g->link = malloc(sizeof(int32_t) * g->out_elems * g->k_elems);
  for (size_t o = 0; o < g->out_elems; ++o) {
    uint32_t oc[ORACLE_MAX_FIELD_DIMS];
    size_t r = o;
    for (uint32_t d = g->nd; d-- > 0;) {
      oc[d] = (uint32_t)(r % g->out_size[d]);
      r /= g->out_size[d];
    }
    for (size_t k = 0; k < g->k_elems; ++k) {
      size_t rk = k;
      uint32_t kc[ORACLE_MAX_FIELD_DIMS];
      for (uint32_t d = g->nd; d-- > 0;) {
        kc[d] = (uint32_t)(rk % p->kernel[d]);
        rk /= p->kernel[d];
      }
      long flat = 0;
      for (uint32_t d = 0; d < g->nd; ++d) {
        int i = tab[d][(size_t)oc[d] * p->kernel[d] + kc[d]];
        if (i < 0) {
          flat = -1;
          break;
        }
        flat = flat * p->field[d] + i;
      }
      g->link[o * g->k_elems + k] = (int32_t)flat;
    }
  }
  for (uint32_t d = 0; d < g->nd; ++d)
    free(tab[d]);
  return 0;
}

static void free_geometry(geometry *g) { free(g->link); }

/* [b][C][e] <-> [b][e][C] */
static double *to_channels_last(const double *src, size_t batch, size_t chans,
                                size_t elems) {
  double *dst = malloc(sizeof(double) * (batch * chans * elems + 1));
  for (size_t b = 0; b < batch; ++b)
    for (size_t c = 0; c < chans; ++c)
      for (size_t e = 0; e < elems; ++e)
        dst[(b * elems + e) * chans + c] = src[(b * chans + c) * elems + e];
  return dst;
}

static void from_channels_last(const double *src, double *dst, size_t batch,
                               size_t chans, size_t elems) {
  for (size_t b = 0; b < batch; ++b)
    for (size_t c = 0; c < chans; ++c)
      for (size_t e = 0; e < elems; ++e)
        dst[(b * chans + c) * elems + e] = src[(b * elems + e) * chans + c];
}

/* ---- forward ----------------------------------------------------------- */

typedef struct {
  const geometry *g;
  size_t G, Ci, Co, B;
  const double *x, *w, *dy, *biases;
  double *y, *dx, *part;
} conv_ctx;

static void fwd_body(int tid, int nt, void *v) {
  const conv_ctx *c = v;
  const geometry *g = c->g;
  const size_t G = c->G, Ci = c->Ci, Co = c->Co;
  const size_t ke = g->k_elems, oe = g->out_elems, ie = g->in_elems;
  const size_t work = c->B * oe;
  const size_t lo = work * (size_t)tid / (size_t)nt,
               hi = work * ((size_t)tid + 1) / (size_t)nt;
  for (size_t idx = lo; idx < hi; ++idx) {
    const size_t b = idx / oe, o = idx % oe;
    double *acc = c->y + idx * G * Co;
    for (size_t ch = 0; ch < G * Co; ++ch)
      acc[ch] = 0.0;
    for (size_t k = 0; k < ke; ++k) {
      const int32_t i = g->link[o * ke + k];
      if (i < 0)
        continue;
      for (size_t gi = 0; gi < G; ++gi) {
        const double *xv = c->x + (b * ie + (size_t)i) * G * Ci + gi * Ci;
        const double *wk = c->w + (gi * ke + k) * Ci * Co;
        double *a = acc + gi * Co;
        for (size_t ic = 0; ic < Ci; ++ic) {
          const double xi = xv[ic];
          const double *wr = wk + ic * Co;
          for (size_t oc = 0; oc < Co; ++oc)
            a[oc] += wr[oc] * xi;
        }
      }
    }
    if (c->biases)
      for (size_t ch = 0; ch < G * Co; ++ch)
        acc[ch] += c->biases[ch];
  }
}

int oracle_conv_fwd(const oracle_conv_params *p, const double *in,
                    const double *weights, const double *biases, double *out,
                    int threads) {
  geometry g;
  int rc = build_geometry(p, &g);
  if (rc)
    return rc;
  const size_t G = p->groups, Ci = p->in_chans_per_group,
               Co = p->out_chans_per_group, B = p->batch;
  const size_t ke = g.k_elems, oe = g.out_elems, ie = g.in_elems;
  /* weights [g][oc][ic][k] -> [g][k][ic][oc]: inner loop runs over oc */
  double *w = malloc(sizeof(double) * (G * ke * Ci * Co + 1));
  for (size_t gi = 0; gi < G; ++gi)
    for (size_t oc = 0; oc < Co; ++oc)
      for (size_t ic = 0; ic < Ci; ++ic)
        for (size_t k = 0; k < ke; ++k)
          w[((gi * ke + k) * Ci + ic) * Co + oc] =
              weights[((gi * Co + oc) * Ci + ic) * ke + k];
  double *x = to_channels_last(in, B, G * Ci, ie);
  double *y = malloc(sizeof(double) * (B * oe * G * Co + 1));
  conv_ctx c = {&g, G, Ci, Co, B, x, w, NULL, biases, y, NULL, NULL};
  parallel_run(pick_threads(threads), fwd_body, &c);
  from_channels_last(y, out, B, G * Co, oe);
  free(w);
  free(x);
  free(y);
  free_geometry(&g);
  return 0;
}

/* ---- backward (gradient w.r.t. the input) ------------------------------ */

static void bwd_body(int tid, int nt, void *v) {
  const conv_ctx *c = v;
  const geometry *g = c->g;
  const size_t G = c->G, Ci = c->Ci, Co = c->Co;
  const size_t ke = g->k_elems, oe = g->out_elems, ie = g->in_elems;
  const size_t b0 = c->B * (size_t)tid / (size_t)nt,
               b1 = c->B * ((size_t)tid + 1) / (size_t)nt;
  for (size_t b = b0; b < b1; ++b)
    for (size_t o = 0; o < oe; ++o) {
      const double *dyv = c->dy + (b * oe + o) * G * Co;
      for (size_t k = 0; k < ke; ++k) {
        const int32_t i = g->link[o * ke + k];
        if (i < 0)
          continue;
        for (size_t gi = 0; gi < G; ++gi) {
          double *a = c->dx + (b * ie + (size_t)i) * G * Ci + gi * Ci;
          const double *wk = c->w + (gi * ke + k) * Co * Ci;
          for (size_t oc = 0; oc < Co; ++oc) {
            const double d = dyv[gi * Co + oc];
            const double *wr = wk + oc * Ci;
            for (size_t ic = 0; ic < Ci; ++ic)
              a[ic] += wr[ic] * d;
          }
        }
      }
    }
}

int oracle_conv_bwd(const oracle_conv_params *p, const double *out_grads,
                    const double *weights, double *in_grads, int threads) {
  geometry g;
  int rc = build_geometry(p, &g);
  if (rc)
    return rc;
  const size_t G = p->groups, Ci = p->in_chans_per_group,
               Co = p->out_chans_per_group, B = p->batch;
  const size_t ke = g.k_elems, oe = g.out_elems, ie = g.in_elems;
  /* weights -> [g][k][oc][ic]: inner loop runs over ic */
  double *w = malloc(sizeof(double) * (G * ke * Ci * Co + 1));
  for (size_t gi = 0; gi < G; ++gi)
    for (size_t oc = 0; oc < Co; ++oc)
      for (size_t ic = 0; ic < Ci; ++ic)
        for (size_t k = 0; k < ke; ++k)
          w[((gi * ke + k) * Co + oc) * Ci + ic] =
              weights[((gi * Co + oc) * Ci + ic) * ke + k];
  double *dy = to_channels_last(out_grads, B, G * Co, oe);
  double *dx = calloc(B * ie * G * Ci + 1, sizeof(double));
  conv_ctx c = {&g, G, Ci, Co, B, NULL, w, dy, NULL, NULL, dx, NULL};
  int nt = pick_threads(threads);
  if ((size_t)nt > B)
    nt = B ? (int)B : 1;
  parallel_run(nt, bwd_body, &c);
  from_channels_last(dx, in_grads, B, G * Ci, ie);
  free(w);
  free(dy);
  free(dx);
  free_geometry(&g);
  return 0;
}

/* ---- weight update (gradient w.r.t. the weights) ----------------------- */

static void wu_body(int tid, int nt, void *v) {
  const conv_ctx *c = v;
  const geometry *g = c->g;
  const size_t G = c->G, Ci = c->Ci, Co = c->Co;
  const size_t ke = g->k_elems, oe = g->out_elems, ie = g->in_elems;
  const size_t wn = G * ke * Co * Ci;
  double *dw = c->part + (size_t)tid * wn;
  const size_t b0 = c->B * (size_t)tid / (size_t)nt,
               b1 = c->B * ((size_t)tid + 1) / (size_t)nt;
  for (size_t b = b0; b < b1; ++b)
    for (size_t o = 0; o < oe; ++o) {
      const double *dyv = c->dy + (b * oe + o) * G * Co;
      for (size_t k = 0; k < ke; ++k) {
        const int32_t i = g->link[o * ke + k];
        if (i < 0)
          continue;
        const double *xv = c->x + (b * ie + (size_t)i) * G * Ci;
        for (size_t gi = 0; gi < G; ++gi) {
          double *wk = dw + (gi * ke + k) * Co * Ci;
          const double *xr = xv + gi * Ci;
          for (size_t oc = 0; oc < Co; ++oc) {
            const double d = dyv[gi * Co + oc];
            double *wr = wk + oc * Ci;
            for (size_t ic = 0; ic < Ci; ++ic)
              wr[ic] += xr[ic] * d;
          }
        }
      }
    }
}

int oracle_conv_wu(const oracle_conv_params *p, const double *acts,
                   const double *out_grads, double *weight_grads,
                   double *bias_grads, int threads) {
  geometry g;
  int rc = build_geometry(p, &g);
  if (rc)
    return rc;
  const size_t G = p->groups, Ci = p->in_chans_per_group,
               Co = p->out_chans_per_group, B = p->batch;
  const size_t ke = g.k_elems, oe = g.out_elems, ie = g.in_elems;
  const size_t wn = G * ke * Co * Ci;
  double *x = to_channels_last(acts, B, G * Ci, ie);
  double *dy = to_channels_last(out_grads, B, G * Co, oe);
  int nt = pick_threads(threads);
  if ((size_t)nt > B)
    nt = B ? (int)B : 1;
  /* one partial dW per thread, each [g][k][oc][ic]; summed in thread order */
  double *part = calloc((size_t)nt * wn + 1, sizeof(double));
  conv_ctx c = {&g, G, Ci, Co, B, x, NULL, dy, NULL, NULL, NULL, part};
  parallel_run(nt, wu_body, &c);
  for (size_t gi = 0; gi < G; ++gi)
    for (size_t oc = 0; oc < Co; ++oc)
      for (size_t ic = 0; ic < Ci; ++ic)
        for (size_t k = 0; k < ke; ++k) {
          double s = 0.0;
          for (int t = 0; t < nt; ++t)
            s += part[(size_t)t * wn + ((gi * ke + k) * Co + oc) * Ci + ic];
          weight_grads[((gi * Co + oc) * Ci + ic) * ke + k] = s;
        }
  if (bias_grads) {
    for (size_t ch = 0; ch < G * Co; ++ch) {
      double s = 0.0;
      for (size_t b = 0; b < B; ++b)
        for (size_t o = 0; o < oe; ++o)
          s += out_grads[(b * G * Co + ch) * oe + o];
      bias_grads[ch] = s;
    }
  }
  free(part);
  free(x);
  free(dy);
  free_geometry(&g);
  return 0;
}

/* ---- GEMM (GeneralMatrixMultiply.cpp:190-283) --------------------------- */

typedef struct {
  size_t groups, M, K, N;
  const double *a, *bp, *c;
  double *d;
  double alpha, beta;
  int transpose_a;
} gemm_ctx;

static void gemm_body(int tid, int nt, void *v) {
  const gemm_ctx *c = v;
  const size_t M = c->M, K = c->K, N = c->N;
  const size_t rows = c->groups * M;
  const size_t lo = rows * (size_t)tid / (size_t)nt,
               hi = rows * ((size_t)tid + 1) / (size_t)nt;
  for (size_t r = lo; r < hi; ++r) {
    const size_t g = r / M, i = r % M;
    double *drow = c->d + (g * M + i) * N;
    for (size_t j = 0; j < N; ++j)
      drow[j] = 0.0;
    for (size_t kk = 0; kk < K; ++kk) {
      const double av = c->transpose_a ? c->a[(g * K + kk) * M + i]
                                       : c->a[(g * M + i) * K + kk];
      const double *br = c->bp + (g * K + kk) * N;
      for (size_t j = 0; j < N; ++j)
        drow[j] += av * br[j];
    }
    for (size_t j = 0; j < N; ++j)
      drow[j] = (c->c ? c->beta * c->c[(g * M + i) * N + j] : 0.0) +
                c->alpha * drow[j];
  }
}

int oracle_gemm(uint32_t groups, uint32_t m, uint32_t k, uint32_t n,
                const double *a, const double *b, const double *c, double *d,
                float alpha, float beta, int transpose_a, int transpose_b,
                int threads) {
  if (beta != 0.0f && c == NULL)
    return 1;
  const size_t K = k, N = n;
  /* B is repacked row-major k x n so that the inner loop is contiguous */
  double *bp = malloc(sizeof(double) * ((size_t)groups * K * N + 1));
  for (size_t g = 0; g < groups; ++g)
    for (size_t kk = 0; kk < K; ++kk)
      for (size_t j = 0; j < N; ++j)
        bp[(g * K + kk) * N + j] = transpose_b ? b[(g * N + j) * K + kk]
                                               : b[(g * K + kk) * N + j];
  gemm_ctx ctx = {groups, m, K, N, a, bp, beta != 0.0f ? c : NULL, d,
                  alpha,  beta, transpose_a};
  parallel_run(pick_threads(threads), gemm_body, &ctx);
  free(bp);
  return 0;
}

/* ---- comparison (Util.cpp:198-217, 316-348) ----------------------------- */

/* Boost.Test 1.70 close_at_tolerance with the default "strong" check and a
 * fractional tolerance: |a-b|/|a| <= tol and |a-b|/|b| <= tol, with the
 * library's guarded division (overflow -> max, underflow -> 0). */
static double safe_div(double f1, double f2) {
  const double max = 1.7976931348623157e308, min = 2.2250738585072014e-308;
  if (f2 < 1.0 && f1 > f2 * max)
    return max;
  if (fabs(f1) <= min || (f2 > 1.0 && f1 < f2 * min))
    return 0.0;
  return f1 / f2;
}

int oracle_is_close(double actual, double expected, double rel_tol,
                    double abs_tol) {
  if (isnan(actual) || isnan(expected))
    return isnan(actual) && isnan(expected);
  if (actual == expected)
    return 1;
  if (fabs(actual) <= rel_tol && fabs(expected) <= rel_tol)
    return 1; /* small_with_tolerance on both sides */
  const double diff = fabs(actual - expected);
  const double f1 = safe_div(diff, fabs(expected));
  const double f2 = safe_div(diff, fabs(actual));
  if ((f1 > f2 ? f1 : f2) <= rel_tol)
    return 1;
  return diff <= abs_tol;
}

size_t oracle_check_is_close(const double *actual, const double *expected,
                             size_t n, double rel_tol, double abs_tol,
                             size_t *first_bad, double *max_rel) {
  size_t bad = 0;
  double worst = 0.0;
  for (size_t i = 0; i < n; ++i) {
    if (!oracle_is_close(actual[i], expected[i], rel_tol, abs_tol)) {
      if (bad == 0 && first_bad)
        *first_bad = i;
      ++bad;
    }
    if (expected[i] != 0.0 && !isnan(actual[i]) && !isnan(expected[i])) {
      const double r = fabs(actual[i] - expected[i]) / fabs(expected[i]);
      if (r > worst)
        worst = r;
    }
  }
  if (max_rel)
    *max_rel = worst;
  return bad;
}

/* ---- number formats ----------------------------------------------------- */

/* Round a double to the nearest IEEE binary16 value (ties to even), overflow
 * to infinity, like a conversion double -> half -> double
 * (lib/poplibs_test/Util.cpp:20-33 rounds test data the same way). */
double oracle_round_to_half(double x) {
  if (isnan(x) || isinf(x) || x == 0.0)
    return x;
  const double ax = fabs(x);
  int e;
  (void)frexp(ax, &e); /* ax = f * 2^e, f in [0.5, 1) */
  int exp2 = e - 1;    /* ax in [2^exp2, 2^(exp2+1)) */
  if (exp2 < -14)
    exp2 = -14; /* subnormal spacing */
  const double ulp = ldexp(1.0, exp2 - 10);
  double q = nearbyint(ax / ulp) * ulp; /* default mode: ties to even */
  if (q >= 65520.0)
    q = INFINITY;
  return x < 0 ? -q : q;
}

/* E4M3 "FN": 1 sign, 4 exponent (bias 7), 3 mantissa bits; no infinities,
 * S.1111.111 is NaN, largest finite 448. */
double oracle_e4m3_to_double(uint8_t bits) {
  const int sign = bits >> 7, e = (bits >> 3) & 0xF, m = bits & 7;
  double v;
  if (e == 0xF && m == 7)
    return NAN;
  if (e == 0)
    v = ldexp((double)m, -9); /* subnormal: m/8 * 2^-6 */
  else
    v = ldexp(1.0 + m / 8.0, e - 7);
  return sign ? -v : v;
}

uint8_t oracle_e4m3_from_double(double x) {
  if (isnan(x))
    return 0x7F;
  const uint8_t sign = signbit(x) ? 0x80 : 0;
  double ax = fabs(x);
  if (ax >= 448.0)
    return sign | 0x7E; /* saturate */
  if (ax == 0.0)
    return sign;
  int e;
  (void)frexp(ax, &e);
  int exp2 = e - 1;
  if (exp2 < -6)
    exp2 = -6;
  const double ulp = ldexp(1.0, exp2 - 3);
  double q = nearbyint(ax / ulp) * ulp;
  if (q >= 448.0)
    return sign | 0x7E;
  if (q == 0.0)
    return sign;
  (void)frexp(q, &e);
  exp2 = e - 1;
  if (exp2 < -6) { /* subnormal */
    const int m = (int)(q / ldexp(1.0, -9));
    return sign | (uint8_t)m;
  }
  const int m = (int)((q / ldexp(1.0, exp2) - 1.0) * 8.0);
  return sign | (uint8_t)(((exp2 + 7) << 3) | m);
}


/* ---- batch normalisation (lib/poplibs_test/Norms.cpp, BatchNorm) ----------- */
/* Element (b, c, f) of a [batch][chans][field] array. */
#define NORM_AT(a, b, c, f) ((a)[((size_t)(b) * chans + (c)) * field + (f)])

void oracle_norm_statistics(const double *acts, uint32_t batch, uint32_t chans,
                            uint32_t field, double eps, int unbiased,
                            int stable, double *mean, double *inv_std) {
  const double n = (double)batch * (double)field;
  for (uint32_t c = 0; c < chans; ++c) {
    double sum = 0.0, squares = 0.0;
    for (uint32_t b = 0; b < batch; ++b)
      for (uint32_t f = 0; f < field; ++f) {
        const double x = NORM_AT(acts, b, c, f);
        sum += x;
        squares += x * x;
      }
    const double m = sum / n;
    if (stable) {
      squares = 0.0;
      for (uint32_t b = 0; b < batch; ++b)
        for (uint32_t f = 0; f < field; ++f) {
          const double d = NORM_AT(acts, b, c, f) - m;
          squares += d * d;
        }
    }
    const double biased = squares / n - (stable ? 0.0 : m * m);
    const double var = n == 1.0 ? 1.0 : (unbiased ? biased * n / (n - 1.0) : biased);
    mean[c] = m;
    inv_std[c] = 1.0 / sqrt(var + eps);
  }
}

void oracle_norm_normalise(const double *acts, const double *gamma,
                           const double *beta, const double *mean,
                           const double *inv_std, uint32_t batch,
                           uint32_t chans, uint32_t field, double *out,
                           double *whitened) {
  for (uint32_t b = 0; b < batch; ++b)
    for (uint32_t c = 0; c < chans; ++c)
      for (uint32_t f = 0; f < field; ++f) {
        const double w = (NORM_AT(acts, b, c, f) - mean[c]) * inv_std[c];
        if (whitened) NORM_AT(whitened, b, c, f) = w;
        if (out) NORM_AT(out, b, c, f) = gamma[c] * w + beta[c];
      }
}

void oracle_norm_gradients(const double *whitened, const double *grads_in,
                           const double *inv_std, const double *gamma,
                           uint32_t batch, uint32_t chans, uint32_t field,
                           double *grads_out) {
  const double n = (double)batch * (double)field;
  for (uint32_t c = 0; c < chans; ++c) {
    double sum_g = 0.0, sum_wg = 0.0;
    for (uint32_t b = 0; b < batch; ++b)
      for (uint32_t f = 0; f < field; ++f) {
        sum_g += NORM_AT(grads_in, b, c, f);
        sum_wg += NORM_AT(whitened, b, c, f) * NORM_AT(grads_in, b, c, f);
      }
    for (uint32_t b = 0; b < batch; ++b)
      for (uint32_t f = 0; f < field; ++f) {
        const double t = NORM_AT(grads_in, b, c, f) -
                         NORM_AT(whitened, b, c, f) * sum_wg / n - sum_g / n;
        NORM_AT(grads_out, b, c, f) = t * gamma[c] * inv_std[c];
      }
  }
}

void oracle_norm_param_update(const double *whitened, const double *grads_in,
                              double learning_rate, uint32_t batch,
                              uint32_t chans, uint32_t field, double *gamma,
                              double *beta) {
  for (uint32_t c = 0; c < chans; ++c) {
    double d_beta = 0.0, d_gamma = 0.0;
    for (uint32_t b = 0; b < batch; ++b)
      for (uint32_t f = 0; f < field; ++f) {
        d_beta += NORM_AT(grads_in, b, c, f);
        d_gamma += NORM_AT(whitened, b, c, f) * NORM_AT(grads_in, b, c, f);
      }
    beta[c] -= learning_rate * d_beta;
    gamma[c] -= learning_rate * d_gamma;
  }
}
#undef NORM_AT
