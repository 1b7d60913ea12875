// C entry points over the REFERENCE's own CPU models, compiled unmodified from
// the reference tree (lib/poplibs_test/Convolution.cpp,
// lib/poplibs_test/GeneralMatrixMultiply.cpp and lib/poplibs_test/Norms.cpp) against the stand-in headers in
// oracle/shim.  TEST INFRASTRUCTURE ONLY: the resulting library
// (oracle/_ref/libpoplibs_test_ref.so) validates the C restatement in
// poplin_oracle.c, generates the golden vectors under tests/golden/, and is
// the "reference" arm of the benchmark.  Nothing on the product path uses it.
#include "poplin_oracle.h"

#include <poplibs_test/Convolution.hpp>
#include <poplibs_test/GeneralMatrixMultiply.hpp>
#include <poplibs_test/Norms.hpp>

#include <cstring>
#include <exception>
#include <string>
#include <vector>

namespace {

thread_local std::string lastError;

struct Vecs {
  std::vector<unsigned> field, kernel, inTruncLo, inTruncHi, inDil, inPadLo,
      inPadHi, kTruncLo, kTruncHi, kDil, kPadLo, kPadHi, outTruncLo,
      outTruncHi, stride, outPadLo, outPadHi;
  std::vector<bool> inFlip, kFlip;
  std::size_t inElems = 1, kElems = 1, outElems = 1;
};

std::vector<unsigned> vec(const uint32_t *p, unsigned n) {
  return std::vector<unsigned>(p, p + n);
}
std::vector<bool> vecb(const uint32_t *p, unsigned n) {
  std::vector<bool> v(n);
  for (unsigned i = 0; i != n; ++i)
    v[i] = p[i] != 0;
  return v;
}

bool unpack(const oracle_conv_params *p, Vecs &v) {
  const unsigned n = p->num_field_dims;
  v.field = vec(p->field, n);
  v.kernel = vec(p->kernel, n);
  v.inTruncLo = vec(p->in_trunc_lo, n);
  v.inTruncHi = vec(p->in_trunc_hi, n);
  v.inDil = vec(p->in_dilation, n);
  v.inPadLo = vec(p->in_pad_lo, n);
  v.inPadHi = vec(p->in_pad_hi, n);
  v.inFlip = vecb(p->in_flip, n);
  v.kTruncLo = vec(p->k_trunc_lo, n);
  v.kTruncHi = vec(p->k_trunc_hi, n);
  v.kDil = vec(p->k_dilation, n);
  v.kPadLo = vec(p->k_pad_lo, n);
  v.kPadHi = vec(p->k_pad_hi, n);
  v.kFlip = vecb(p->k_flip, n);
  v.outTruncLo = vec(p->out_trunc_lo, n);
  v.outTruncHi = vec(p->out_trunc_hi, n);
  v.stride = vec(p->stride, n);
  v.outPadLo = vec(p->out_pad_lo, n);
  v.outPadHi = vec(p->out_pad_hi, n);
  for (unsigned d = 0; d != n; ++d) {
    int os = oracle_conv_out_size(p, d);
    if (os < 0)
      return false;
    v.inElems *= p->field[d];
    v.kElems *= p->kernel[d];
    v.outElems *= static_cast<std::size_t>(os);
  }
  return true;
}

template <class F> int guarded(F &&f) {
  try {
    f();
    return 0;
  } catch (const std::exception &e) {
    lastError = e.what();
    return 1;
  }
}

} // namespace

extern "C" {

const char *ref_last_error(void) { return lastError.c_str(); }

int ref_conv_fwd(const oracle_conv_params *p, const double *in,
                 const double *weights, const double *biases, double *out) {
  Vecs v;
  if (!unpack(p, v)) {
    lastError = "invalid convolution parameters";
    return 2;
  }
  const std::size_t inC = std::size_t(p->groups) * p->in_chans_per_group;
  const std::size_t outC = std::size_t(p->groups) * p->out_chans_per_group;
  std::vector<double> zeroBias(outC, 0.0);
  return guarded([&] {
    boost::const_multi_array_ref<double, 3> inRef(
        in, boost::extents[p->batch][inC][v.inElems]);
    boost::const_multi_array_ref<double, 4> wRef(
        weights, boost::extents[p->groups][p->out_chans_per_group]
                               [p->in_chans_per_group][v.kElems]);
    boost::const_multi_array_ref<double, 1> bRef(
        biases ? biases : zeroBias.data(), boost::extents[outC]);
    boost::multi_array_ref<double, 3> outRef(
        out, boost::extents[p->batch][outC][v.outElems]);
    poplibs_test::conv::convolution(
        v.field, v.inTruncLo, v.inTruncHi, v.inDil, v.inPadLo, v.inPadHi,
        v.inFlip, v.kernel, v.kTruncLo, v.kTruncHi, v.kDil, v.kPadLo, v.kPadHi,
        v.kFlip, v.outTruncLo, v.outTruncHi, v.stride, v.outPadLo, v.outPadHi,
        inRef, wRef, bRef, outRef);
  });
}

int ref_conv_bwd(const oracle_conv_params *p, const double *outGrads,
                 const double *weights, double *inGrads) {
  Vecs v;
  if (!unpack(p, v)) {
    lastError = "invalid convolution parameters";
    return 2;
  }
  const std::size_t inC = std::size_t(p->groups) * p->in_chans_per_group;
  const std::size_t outC = std::size_t(p->groups) * p->out_chans_per_group;
  return guarded([&] {
    boost::const_multi_array_ref<double, 3> dyRef(
        outGrads, boost::extents[p->batch][outC][v.outElems]);
    boost::const_multi_array_ref<double, 4> wRef(
        weights, boost::extents[p->groups][p->out_chans_per_group]
                               [p->in_chans_per_group][v.kElems]);
    boost::multi_array_ref<double, 3> dxRef(
        inGrads, boost::extents[p->batch][inC][v.inElems]);
    poplibs_test::conv::convolutionBackward(
        v.field, v.inTruncLo, v.inTruncHi, v.inDil, v.inPadLo, v.inPadHi,
        v.inFlip, v.kernel, v.kTruncLo, v.kTruncHi, v.kDil, v.kPadLo, v.kPadHi,
        v.kFlip, v.outTruncLo, v.outTruncHi, v.stride, v.outPadLo, v.outPadHi,
        dyRef, wRef, dxRef);
  });
}

// dW and bias gradient, read out of the reference's in-place update
// (weights += lr * -dW, Convolution.cpp:873, 893) by starting from zero
// weights with lr = -1.
int ref_conv_wu(const oracle_conv_params *p, const double *acts,
                const double *outGrads, double *weightGrads,
                double *biasGrads) {
  Vecs v;
  if (!unpack(p, v)) {
    lastError = "invalid convolution parameters";
    return 2;
  }
  const std::size_t inC = std::size_t(p->groups) * p->in_chans_per_group;
  const std::size_t outC = std::size_t(p->groups) * p->out_chans_per_group;
  std::vector<double> bias(outC, 0.0);
  const std::size_t wElems = std::size_t(p->groups) * p->out_chans_per_group *
                             p->in_chans_per_group * v.kElems;
  std::memset(weightGrads, 0, sizeof(double) * wElems);
  int rc = guarded([&] {
    boost::const_multi_array_ref<double, 3> xRef(
        acts, boost::extents[p->batch][inC][v.inElems]);
    boost::const_multi_array_ref<double, 3> dyRef(
        outGrads, boost::extents[p->batch][outC][v.outElems]);
    boost::multi_array_ref<double, 4> wRef(
        weightGrads, boost::extents[p->groups][p->out_chans_per_group]
                                   [p->in_chans_per_group][v.kElems]);
    boost::multi_array_ref<double, 1> bRef(bias.data(), boost::extents[outC]);
    poplibs_test::conv::weightUpdate(
        v.field, v.inTruncLo, v.inTruncHi, v.inDil, v.inPadLo, v.inPadHi,
        v.inFlip, v.kernel, v.kTruncLo, v.kTruncHi, v.kDil, v.kPadLo, v.kPadHi,
        v.kFlip, v.outTruncLo, v.outTruncHi, v.stride, v.outPadLo, v.outPadHi,
        -1.0, xRef, dyRef, wRef, bRef);
  });
  if (rc == 0 && biasGrads)
    std::memcpy(biasGrads, bias.data(), sizeof(double) * outC);
  return rc;
}

int ref_gemm(uint32_t groups, uint32_t m, uint32_t k, uint32_t n,
             const double *a, const double *b, const double *c, double *d,
             float alpha, float beta, int transposeA, int transposeB) {
  return guarded([&] {
    const std::size_t aR = transposeA ? k : m, aC = transposeA ? m : k;
    const std::size_t bR = transposeB ? n : k, bC = transposeB ? k : n;
    std::vector<double> zeros;
    if (!c) {
      zeros.assign(std::size_t(groups) * m * n, 0.0);
      c = zeros.data();
    }
    boost::multi_array_ref<double, 3> aRef(const_cast<double *>(a),
                                           boost::extents[groups][aR][aC]);
    boost::multi_array_ref<double, 3> bRef(const_cast<double *>(b),
                                           boost::extents[groups][bR][bC]);
    boost::multi_array_ref<double, 3> cRef(const_cast<double *>(c),
                                           boost::extents[groups][m][n]);
    boost::multi_array_ref<double, 3> dRef(d, boost::extents[groups][m][n]);
    poplibs_test::gemm::generalGroupedMatrixMultiply(
        aRef, bRef, cRef, dRef, alpha, beta, transposeA != 0, transposeB != 0);
  });
}

// ---- the reference's batch-norm models (lib/poplibs_test/Norms.cpp) ------------
using Ref3 = boost::multi_array_ref<double, 3>;
using Ref1 = boost::multi_array_ref<double, 1>;
static Ref3 r3(const double *p, uint32_t b, uint32_t c, uint32_t f) {
  return Ref3(const_cast<double *>(p), boost::extents[b][c][f]);
}
static Ref1 r1(const double *p, uint32_t c) {
  return Ref1(const_cast<double *>(p), boost::extents[c]);
}
constexpr auto kBatchNorm = poplibs_test::norm::NormType::BatchNorm;

int ref_norm_statistics(const double *acts, uint32_t batch, uint32_t chans, uint32_t field,
                        double eps, int unbiased, int stable, double *mean, double *inv_std) {
  return guarded([&] {
    poplibs_test::norm::normStatistics(r3(acts, batch, chans, field), eps, unbiased != 0, stable != 0,
                                       r1(mean, chans), r1(inv_std, chans), kBatchNorm, false);
  });
}

int ref_norm_normalise(const double *acts, const double *gamma, const double *beta, const double *mean,
                       const double *inv_std, uint32_t batch, uint32_t chans, uint32_t field,
                       double *out, double *whitened) {
  return guarded([&] {
    poplibs_test::norm::normalise(r3(acts, batch, chans, field), r1(gamma, chans), r1(beta, chans),
                                  r1(mean, chans), r1(inv_std, chans), r3(out, batch, chans, field),
                                  r3(whitened, batch, chans, field), kBatchNorm, false);
  });
}

int ref_norm_gradients(const double *whitened, const double *grads_in, const double *inv_std,
                       const double *gamma, uint32_t batch, uint32_t chans, uint32_t field,
                       double *grads_out) {
  return guarded([&] {
    poplibs_test::norm::normGradients(r3(whitened, batch, chans, field), r3(grads_in, batch, chans, field),
                                      r1(inv_std, chans), r1(gamma, chans),
                                      r3(grads_out, batch, chans, field), kBatchNorm, false);
  });
}

int ref_norm_param_update(const double *whitened, const double *grads_in, double learning_rate,
                          uint32_t batch, uint32_t chans, uint32_t field, double *gamma, double *beta) {
  return guarded([&] {
    poplibs_test::norm::normParamUpdate(r3(whitened, batch, chans, field),
                                        r3(grads_in, batch, chans, field), learning_rate,
                                        r1(gamma, chans), r1(beta, chans), kBatchNorm);
  });
}

} // extern "C"
