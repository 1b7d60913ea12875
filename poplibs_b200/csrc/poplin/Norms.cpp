// poplin::Norms over the C ABI (plb_norm_*).  Follows the data flow of the
// reference's lib/poplin/Norms.cpp: moments (mean and power) -> optional
// caller-supplied all-reduce -> inverse standard deviation; whitening; scale
// and shift; parameter gradients as one joint column reduction; the gradient
// through the statistics.
#include "poplin/Norms.hpp"

#include <cmath>

#include "../poplar/standin_impl.hpp"
#include "internal.hpp"
#include "poplibs_support/logging.hpp"
#include "poputil/exceptions.hpp"

namespace poplin {

using poplar::Graph;
using poplar::Tensor;
using poplar::program::Sequence;
using poputil::poplibs_error;
namespace logging = poplibs_support::logging;

namespace {

struct ActsInfo {
  int dtype;
  std::size_t chans, pixels;
};

ActsInfo describe(const Tensor &acts, const char *what) {
  if (acts.rank() < 2)
    throw poplibs_error(std::string(what) + ": activations of rank " + std::to_string(acts.rank()) +
                        ", expected >= 2");
  if (acts.elementType() != poplar::HALF && acts.elementType() != poplar::FLOAT)
    throw poplibs_error(std::string(what) + ": activations must be half or float");
  ActsInfo a;
  a.dtype = poplar::detail::dtypeOf(acts.elementType());
  a.chans = acts.dim(1);
  a.pixels = a.chans ? acts.numElements() / a.chans : 0;
  return a;
}

void requirePerChannel(const Tensor &t, const Tensor &acts, const char *name) {
  if (t.numElements() != acts.dim(1))
    throw poplibs_error(std::string(name) + " must have one element per channel of the activations");
  if (t.elementType() != acts.elementType())
    throw poplibs_error(std::string(name) + " must have the activations' element type");
}

// a per-channel vector in contiguous memory (copied if it is a strided view)
Tensor flatDense(Graph &graph, const Tensor &t, Sequence &prog) {
  const Tensor f = t.flatten();
  if (f.numElements() <= 1 || f.strides()[0] == 1) return f;
  Tensor d = graph.addScratch(t.elementType(), {f.numElements()});
  prog.add(poplar::program::Copy(f, d));
  return d;
}

Tensor perChannel(Graph &graph, const Tensor &acts, const poplar::Type &type, const std::string &name) {
  return graph.addVariable(type, {acts.dim(1)}, name);
}

std::pair<Tensor, Tensor> statisticsImpl(Graph &graph, const Tensor &acts, float eps, Sequence &prog,
                                         bool unbiased, bool stable,
                                         const DistributedNormReduceCallback &callback, unsigned normSize,
                                         const poplar::DebugContext &dc) {
  const ActsInfo a = describe(acts, "normStatistics");
  const std::size_t replicaSize = acts.dim(0);
  const bool distributed = callback != nullptr && normSize > replicaSize && replicaSize > 0;
  if (distributed && normSize % replicaSize)
    throw poplibs_error("Norm batch size must be an integer multiple of replica batch size");
  std::size_t n = a.pixels * (distributed ? normSize / replicaSize : 1);
  float scale = 1.0f, scaleVar = 1.0f;
  if (n > 1) {
    scale /= float(n);
    if (unbiased) scaleVar = float(n) / float(n - 1);
  }
  logging::poplin::info("normStatistics acts=" + acts.shapeToString() + " eps=" + std::to_string(eps) +
                        " unbiased=" + std::to_string(unbiased) + " name=" + dc.getPathName());
  const Tensor x = internal::actsInKernelLayout(graph, acts, prog);
  Tensor mean = perChannel(graph, acts, acts.elementType(), dc.getPathName() + "/mean");
  Tensor power = perChannel(graph, acts, poplar::FLOAT, dc.getPathName() + "/power");
  const unsigned group = distributed ? unsigned(normSize / replicaSize) : 1;
  auto moments = [=](const Tensor &centre, const Tensor &meanOut, const Tensor &powerOut) {
    return [=](plb_context *ctx) {
      poplar::detail::check(plb_norm_moments(
          ctx, a.dtype, x.devicePointer(), a.pixels, uint32_t(a.chans), scale,
          centre.valid() ? centre.devicePointer() : nullptr, meanOut.valid() ? meanOut.devicePointer() : nullptr,
          static_cast<float *>(powerOut.devicePointer())));
    };
  };
  if (!stable && !distributed) {
    // the common case in one call: the kernel that finishes the sums also forms 1 / sigma
    Tensor iStdDev = perChannel(graph, acts, acts.elementType(), dc.getPathName() + "/iStdDev");
    prog.add([=](plb_context *ctx) {
      poplar::detail::check(plb_norm_statistics(ctx, a.dtype, x.devicePointer(), a.pixels, uint32_t(a.chans), eps,
                                                scaleVar, mean.devicePointer(), iStdDev.devicePointer(),
                                                static_cast<float *>(power.devicePointer())));
    });
    return {mean, iStdDev};
  }
  if (stable) {
    // mean first (reduced over the replicas), then the squared deviations from it
    Tensor unusedPower = perChannel(graph, acts, poplar::FLOAT, dc.getPathName() + "/rawPower");
    prog.add(moments(Tensor(), mean, unusedPower));
    if (distributed) mean = callback(graph, {mean}, prog, group, dc, {}).at(0);
    prog.add(moments(mean, Tensor(), power));
    if (distributed) power = callback(graph, {power}, prog, group, dc, {}).at(0);
  } else {
    prog.add(moments(Tensor(), mean, power));
    if (distributed) {
      const auto reduced = callback(graph, {mean, power}, prog, group, dc, {});
      mean = reduced.at(0);
      power = reduced.at(1);
    }
  }
  Tensor iStdDev = perChannel(graph, acts, acts.elementType(), dc.getPathName() + "/iStdDev");
  const Tensor meanF = flatDense(graph, mean, prog), powerF = flatDense(graph, power, prog);
  prog.add([=](plb_context *ctx) {
    poplar::detail::check(plb_norm_inv_std_dev(ctx, a.dtype, meanF.devicePointer(),
                                               static_cast<const float *>(powerF.devicePointer()),
                                               uint32_t(a.chans), eps, scaleVar, stable ? 1 : 0,
                                               iStdDev.devicePointer()));
  });
  return {mean, iStdDev};
}

std::pair<Tensor, Tensor> paramGradientsImpl(Graph &graph, const Tensor &whitened, const Tensor &grads,
                                             float scale, Sequence &prog, const poplar::DebugContext &dc) {
  const ActsInfo a = describe(whitened, "normParamGradients");
  if (grads.shape() != whitened.shape() || grads.elementType() != whitened.elementType())
    throw poplibs_error("normParamGradients: gradients must match the whitened activations");
  const Tensor w = internal::actsInKernelLayout(graph, whitened, prog);
  const Tensor g = internal::actsInKernelLayout(graph, grads, prog);
  Tensor gammaDelta = perChannel(graph, whitened, grads.elementType(), dc.getPathName() + "/gammaDelta");
  Tensor betaDelta = perChannel(graph, whitened, grads.elementType(), dc.getPathName() + "/betaDelta");
  prog.add([=](plb_context *ctx) {
    poplar::detail::check(plb_norm_param_gradients(ctx, a.dtype, w.devicePointer(), g.devicePointer(),
                                                   a.pixels, uint32_t(a.chans), scale,
                                                   gammaDelta.devicePointer(), betaDelta.devicePointer(),
                                                   nullptr, nullptr));
  });
  return {gammaDelta, betaDelta};
}

}  // namespace

Tensor createNormGamma(Graph &graph, const Tensor &acts, const poplar::Type &type,
                       const poplar::DebugContext &dc) {
  describe(acts, "createNormGamma");
  return perChannel(graph, acts, type, dc.getPathName() + "/gamma");
}
Tensor createNormGamma(Graph &graph, const Tensor &acts, const poplar::DebugContext &dc) {
  return createNormGamma(graph, acts, acts.elementType(), dc);
}
Tensor createNormBeta(Graph &graph, const Tensor &acts, const poplar::Type &type,
                      const poplar::DebugContext &dc) {
  describe(acts, "createNormBeta");
  return perChannel(graph, acts, type, dc.getPathName() + "/beta");
}
Tensor createNormBeta(Graph &graph, const Tensor &acts, const poplar::DebugContext &dc) {
  return createNormBeta(graph, acts, acts.elementType(), dc);
}
std::pair<Tensor, Tensor> createNormParams(Graph &graph, const Tensor &acts, const poplar::DebugContext &dc) {
  return {createNormGamma(graph, acts, dc), createNormBeta(graph, acts, dc)};
}

std::pair<Tensor, Tensor> normStatistics(Graph &graph, const Tensor &acts, float eps, Sequence &prog,
                                         bool unbiasedVarEstimate, bool stableAlgo, const poplar::Type &,
                                         const poplar::DebugContext &dc) {
  return statisticsImpl(graph, acts, eps, prog, unbiasedVarEstimate, stableAlgo, nullptr,
                        unsigned(acts.rank() ? acts.dim(0) : 0), dc);
}

std::pair<Tensor, Tensor> distributedNormStatistics(Graph &graph, const Tensor &acts, float eps,
                                                    Sequence &prog, bool unbiasedVarEstimate,
                                                    DistributedNormReduceCallback callback, unsigned normSize,
                                                    bool stableAlgo, const poplar::Type &,
                                                    const poplar::DebugContext &dc) {
  return statisticsImpl(graph, acts, eps, prog, unbiasedVarEstimate, stableAlgo, callback, normSize, dc);
}

Tensor normWhiten(Graph &graph, const Tensor &acts, const Tensor &mean, const Tensor &iStdDev,
                  Sequence &prog, const poplar::DebugContext &dc) {
  const ActsInfo a = describe(acts, "normWhiten");
  requirePerChannel(mean, acts, "mean");
  requirePerChannel(iStdDev, acts, "iStdDev");
  const Tensor x = internal::actsInKernelLayout(graph, acts, prog);
  const Tensor m = flatDense(graph, mean, prog), s = flatDense(graph, iStdDev, prog);
  Tensor out = internal::newActsLike(graph, acts, acts.elementType(), dc.getPathName() + "/whitened");
  const Tensor o = internal::actsInKernelLayout(graph, out, prog, false);
  prog.add([=](plb_context *ctx) {
    poplar::detail::check(plb_norm_whiten(ctx, a.dtype, x.devicePointer(), m.devicePointer(),
                                          s.devicePointer(), a.pixels, uint32_t(a.chans), o.devicePointer()));
  });
  return out;
}

static Tensor scaleShift(Graph &graph, const Tensor &acts, const Tensor &scale, const Tensor *shift,
                         Sequence &prog, const std::string &name, const char *what) {
  const ActsInfo a = describe(acts, what);
  requirePerChannel(scale, acts, "the per-channel scale");
  if (shift) requirePerChannel(*shift, acts, "the per-channel shift");
  const Tensor x = internal::actsInKernelLayout(graph, acts, prog);
  const Tensor sc = flatDense(graph, scale, prog);
  const Tensor sh = shift ? flatDense(graph, *shift, prog) : Tensor();
  Tensor out = internal::newActsLike(graph, acts, acts.elementType(), name);
  const Tensor o = internal::actsInKernelLayout(graph, out, prog, false);
  prog.add([=](plb_context *ctx) {
    poplar::detail::check(plb_norm_scale_shift(ctx, a.dtype, x.devicePointer(), sc.devicePointer(),
                                               sh.valid() ? sh.devicePointer() : nullptr, a.pixels,
                                               uint32_t(a.chans), o.devicePointer()));
  });
  return out;
}

Tensor normalise(Graph &graph, const Tensor &actsWhitened, const Tensor &gamma, const Tensor &beta,
                 Sequence &prog, const poplar::DebugContext &dc) {
  return scaleShift(graph, actsWhitened, gamma, &beta, prog, dc.getPathName() + "/normalised", "normalise");
}

std::pair<Tensor, Tensor> normParamGradients(Graph &graph, const Tensor &actsWhitened, const Tensor &gradsIn,
                                             Sequence &prog, const poplar::Type &,
                                             const poplar::DebugContext &dc) {
  return paramGradientsImpl(graph, actsWhitened, gradsIn, 1.0f, prog, dc);
}

Tensor normGradients(Graph &graph, const Tensor &gradsIn, const Tensor &gamma, Sequence &prog,
                     const poplar::DebugContext &dc) {
  return scaleShift(graph, gradsIn, gamma, nullptr, prog, dc.getPathName() + "/normGrad", "normGradients");
}

static Tensor statisticsGradientsImpl(Graph &graph, const Tensor &whitened, const Tensor &gradsIn,
                                      const Tensor &invStdDev, Sequence &prog,
                                      const DistributedNormReduceCallback &callback, unsigned normSize,
                                      const poplar::DebugContext &dc) {
  const ActsInfo a = describe(whitened, "normStatisticsGradients");
  if (gradsIn.shape() != whitened.shape() || gradsIn.elementType() != whitened.elementType())
    throw poplibs_error("normStatisticsGradients: gradients must match the whitened activations");
  requirePerChannel(invStdDev, whitened, "invStdDev");
  const std::size_t replicaSize = whitened.dim(0);
  const bool distributed = callback != nullptr && normSize > replicaSize && replicaSize > 0;
  if (distributed && normSize % replicaSize)
    throw poplibs_error("Norm batch size must be an integer multiple of replica batch size");
  const Tensor w = internal::actsInKernelLayout(graph, whitened, prog);
  const Tensor g = internal::actsInKernelLayout(graph, gradsIn, prog);
  const Tensor s = flatDense(graph, invStdDev, prog);
  Tensor out = internal::newActsLike(graph, whitened, whitened.elementType(), dc.getPathName() + "/gradient");
  const Tensor o = internal::actsInKernelLayout(graph, out, prog, false);
  if (!distributed) {
    prog.add([=](plb_context *ctx) {
      poplar::detail::check(plb_norm_statistics_gradients(ctx, a.dtype, w.devicePointer(), g.devicePointer(),
                                                          s.devicePointer(), nullptr, nullptr, a.pixels,
                                                          uint32_t(a.chans), o.devicePointer()));
    });
    return out;
  }
  // distributed: -mean(w * g) and -mean(g) over the whole batch through the
  // caller's all-reduce, then (g + w * varDelta + meanDelta) * invStdDev
  const float rScale = 1.0f / float(a.pixels * (normSize / replicaSize));
  auto deltas = paramGradientsImpl(graph, whitened, gradsIn, -rScale, prog, dc);
  const auto reduced =
      callback(graph, {deltas.first, deltas.second}, prog, unsigned(normSize / replicaSize), dc, {});
  const Tensor varDelta = flatDense(graph, reduced.at(0), prog), meanDelta = flatDense(graph, reduced.at(1), prog);
  prog.add([=](plb_context *ctx) {
    poplar::detail::check(plb_norm_statistics_gradients(
        ctx, a.dtype, w.devicePointer(), g.devicePointer(), s.devicePointer(), varDelta.devicePointer(),
        meanDelta.devicePointer(), a.pixels, uint32_t(a.chans), o.devicePointer()));
  });
  return out;
}

Tensor normStatisticsGradients(Graph &graph, const Tensor &actsWhitened, const Tensor &gradsIn,
                               const Tensor &invStdDev, Sequence &prog, const poplar::Type &,
                               const poplar::DebugContext &dc) {
  return statisticsGradientsImpl(graph, actsWhitened, gradsIn, invStdDev, prog, nullptr,
                                 unsigned(actsWhitened.rank() ? actsWhitened.dim(0) : 0), dc);
}

Tensor distributedNormStatisticsGradients(Graph &graph, const Tensor &actsWhitened, const Tensor &gradsIn,
                                          const Tensor &invStdDev, Sequence &prog,
                                          DistributedNormReduceCallback reduceCallback, unsigned normSize,
                                          const poplar::Type &, const poplar::DebugContext &dc) {
  return statisticsGradientsImpl(graph, actsWhitened, gradsIn, invStdDev, prog, reduceCallback, normSize, dc);
}

}  // namespace poplin
