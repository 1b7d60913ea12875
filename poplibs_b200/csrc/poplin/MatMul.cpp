// poplin matrix-multiplication entry points over the C ABI (counterpart of
// lib/poplin/MatMul.cpp:236-1035 and lib/poplin/FullyConnected.cpp:39-97).
#include "poplin/MatMul.hpp"

#include <algorithm>
#include <iostream>
#include <sstream>

#include "../poplar/standin_impl.hpp"
#include "internal.hpp"
#include "poplin/FullyConnected.hpp"
#include "poputil/exceptions.hpp"

namespace poplin {

using poplar::Graph;
using poplar::Tensor;
using poplar::program::Sequence;
using poputil::poplibs_error;

namespace {

std::string shapeText(const std::vector<std::size_t> &s) {
  std::string t = "[";
  for (std::size_t i = 0; i < s.size(); ++i) t += (i ? "," : "") + std::to_string(s[i]);
  return t + "]";
}

// lib/poplin/MatMul.cpp:406-418
void dimChecks(const std::vector<std::size_t> &a, const std::vector<std::size_t> &b) {
  if (a.size() != 3 || b.size() != 3)
    throw poplibs_error("Operand to matrix multiplication is not a grouped matrix");
  if (a[0] != b[0])
    throw poplibs_error("Number of matrix multiplication groups must be the same for both operands");
  if (a[2] != b[1])
    throw poplibs_error("Second dimension of first operand to matrix multiplication does not match "
                        "first dimension of second operand: " + shapeText(a) + " x " + shapeText(b));
}

void typeChecks(const poplar::Type &in, const poplar::Type &out) {
  if (in != poplar::HALF && in != poplar::FLOAT && in != poplar::QUARTER)
    throw poplibs_error("matMul input type " + in.toString() +
                        " is not supported on this target (half, float and quarter are)");
  if (out != poplar::HALF && out != poplar::FLOAT)
    throw poplibs_error("matMul output type must be half or float");
  if (in == poplar::QUARTER && out != poplar::HALF)
    throw poplibs_error("Output type must be half when input type is quarter");
}

// How a [g][rows][cols] view sits in memory, as the C ABI can take it.
struct MatrixLayout {
  bool ok = false;         // directly usable
  bool transposed = false; // memory is [g][cols][rows]
  long long ld = 0;        // leading dimension in elements
};

MatrixLayout layoutOf(const Tensor &t) {
  MatrixLayout l;
  const auto &s = t.strides();
  const std::size_t g = t.dim(0), rows = t.dim(1), cols = t.dim(2);
  const std::size_t es = t.elementType().bytes();
  if ((t.offset() * std::ptrdiff_t(es)) % 16 != 0) return l;
  auto aligned = [&](long long ld) { return ld > 0 && (std::size_t(ld) * es) % 16 == 0; };
  if ((cols == 1 || s[2] == 1) && (rows == 1 || (s[1] >= std::ptrdiff_t(cols) && aligned(s[1])))) {
    const long long ld = rows == 1 ? std::max<long long>(cols, 1) : s[1];
    if (aligned(ld) && (g == 1 || s[0] == std::ptrdiff_t(rows) * ld)) {
      l.ok = true;
      l.ld = ld;
      return l;
    }
  }
  if ((rows == 1 || s[1] == 1) && (cols == 1 || (s[2] >= std::ptrdiff_t(rows) && aligned(s[2])))) {
    const long long ld = cols == 1 ? std::max<long long>(rows, 1) : s[2];
    if (aligned(ld) && (g == 1 || s[0] == std::ptrdiff_t(cols) * ld)) {
      l.ok = true;
      l.transposed = true;
      l.ld = ld;
      return l;
    }
  }
  return l;
}

int quarterExponent(const Tensor &t) {
  if (t.elementType() != poplar::QUARTER) return 0;
  const poplar::QuarterMetadata md = t.hasMetadata() ? t.getMetadata() : poplar::QuarterMetadata();
  // F143 / F152 values are half the E4M3 / E5M2 reading of the same bits
  return int(md.getScale()) - 1;
}

// Dense row-major copy of a grouped matrix whose row length is padded to a
// multiple of 16 elements, so that every row starts 16-byte aligned.
Tensor denseCopy(Graph &graph, const Tensor &t, Sequence &prog) {
  const std::size_t cols = t.dim(2), padded = (cols + 15) / 16 * 16;
  Tensor base = graph.addScratch(t.elementType(), {t.dim(0), t.dim(1), padded});
  Tensor view = base.slice(0, cols, 2);
  if (t.elementType() == poplar::QUARTER && t.hasMetadata())
    graph.setQuarterMetadata(view, t.getMetadata());
  prog.add(poplar::program::Copy(t, view));
  return view;
}

// out (+)= alpha * A * B.  A [g][m][k], B [g][k][n], out [g][m][n].
void matMulImpl(Graph &graph, const Tensor &A_, const Tensor &B_, const Tensor &out, float alpha,
                float beta, Sequence &prog, const poplar::OptionFlags &options) {
  dimChecks(A_.shape(), B_.shape());
  const std::size_t g = A_.dim(0), m = A_.dim(1), k = A_.dim(2), n = B_.dim(2);
  if (out.shape() != std::vector<std::size_t>{g, m, n})
    throw poplibs_error("matMul output has shape " + out.shapeToString() + ", expected " +
                        shapeText({g, m, n}));
  if (A_.elementType() != B_.elementType())
    throw poplibs_error("matMul operands must have the same element type");
  typeChecks(A_.elementType(), out.elementType());
  const internal::ConvOptions parsed(internal::matMulToConvOptions(options));

  Tensor A = A_, B = B_;
  MatrixLayout la = layoutOf(A), lb = layoutOf(B);
  // a transposed left operand is transposed into scratch by the library, which
  // takes it densely packed only: a padded one is copied like any other layout
  if (la.ok && la.transposed && la.ld != (long long)m) la.ok = false;
  if (!la.ok && k > 0 && m > 0) {
    A = denseCopy(graph, A_, prog);
    la = layoutOf(A);
  }
  // a row-major [k][n] right operand is taken as it is (half, float); otherwise (and for
  // quarter, where it would be transposed at every call anyway) keep a [n][k] copy
  const bool bRowMajorUsable = lb.ok && !lb.transposed &&
                               (A.elementType() == poplar::HALF || A.elementType() == poplar::FLOAT);
  if (k > 0 && n > 0 && !(lb.ok && lb.transposed) && !bRowMajorUsable) {
    B = denseCopy(graph, B_.dimShufflePartial({1, 2}, {2, 1}), prog).dimShufflePartial({1, 2}, {2, 1});
    lb = layoutOf(B);
  }
  MatrixLayout lo = layoutOf(out);
  const bool outDirect = lo.ok && !lo.transposed;
  Tensor O = out;
  if (!outDirect) {
    const std::size_t padded = (n + 15) / 16 * 16;
    O = graph.addScratch(out.elementType(), {g, m, padded}).slice(0, n, 2);
    if (beta != 0.f) prog.add(poplar::program::Copy(out, O));
    lo = layoutOf(O);
  }

  plb_matmul_desc d{};
  d.groups = uint32_t(g);
  d.m = uint32_t(m);
  d.k = uint32_t(k);
  d.n = uint32_t(n);
  d.input_type = poplar::detail::dtypeOf(A.elementType());
  d.output_type = poplar::detail::dtypeOf(out.elementType());
  d.partials_type = parsed.partialsType == poplar::HALF ? PLB_HALF : PLB_FLOAT;
  d.transpose_a = la.transposed;
  d.transpose_b = lb.transposed;
  d.alpha = alpha;
  d.beta = beta;
  d.lda = la.ld;
  d.ldb = lb.ld;
  d.ldc = lo.ld;
  prog.add([=](plb_context *ctx) mutable {
    d.scale_a = quarterExponent(A);
    d.scale_b = quarterExponent(B);
    auto format = [](const Tensor &t) {
      return t.elementType() == poplar::QUARTER && t.hasMetadata() &&
                     t.getMetadata().getFormat() == poplar::QuarterMetadata::Format::F152
                 ? PLB_F152
                 : PLB_F143;
    };
    d.format_a = format(A);
    d.format_b = format(B);
    if (d.scale_a < -32) d.scale_a = -32;
    if (d.scale_b < -32) d.scale_b = -32;
    const void *c = d.beta != 0.f ? O.devicePointer() : nullptr;
    poplar::detail::check(plb_matmul(ctx, &d, k && m ? A.devicePointer() : nullptr,
                                     k && n ? B.devicePointer() : nullptr, c, O.devicePointer()));
  });
  if (!outDirect) prog.add(poplar::program::Copy(O, out));
}

Tensor allocMatrix(Graph &graph, const poplar::Type &type, const std::vector<std::size_t> &shape,
                   const poplar::DebugContext &dc) {
  // rows padded to a multiple of 16 elements keep every row TMA-addressable
  const std::size_t cols = shape.back(), padded = std::max<std::size_t>((cols + 15) / 16 * 16, 16);
  std::vector<std::size_t> phys(shape);
  phys.back() = padded;
  Tensor base = graph.addVariable(type, phys, dc);
  return padded == cols ? base : base.slice(0, cols, unsigned(shape.size() - 1));
}

std::vector<std::size_t> grouped(const std::vector<std::size_t> &s) {
  if (s.size() != 2) throw poplibs_error("Operand to matrix multiplication is not a matrix");
  return {1, s[0], s[1]};
}

}  // namespace

// ---- products ------------------------------------------------------------------
Tensor matMulGrouped(Graph &graph, const Tensor &A, const Tensor &B, Sequence &prog,
                     const poplar::Type &outputType, const poplar::DebugContext &dc,
                     const poplar::OptionFlags &options, PlanningCache *) {
  dimChecks(A.shape(), B.shape());
  Tensor out = allocMatrix(graph, outputType, {A.dim(0), A.dim(1), B.dim(2)}, {dc, "out"});
  matMulImpl(graph, A, B, out, 1.f, 0.f, prog, options);
  return out;
}

void matMulGroupedWithOutput(Graph &graph, const Tensor &A, const Tensor &B, Tensor &out,
                             Sequence &prog, const poplar::DebugContext &,
                             const poplar::OptionFlags &options, PlanningCache *) {
  matMulImpl(graph, A, B, out, 1.f, 0.f, prog, options);
}

Tensor matMul(Graph &graph, const Tensor &A, const Tensor &B, Sequence &prog,
              const poplar::Type &outputType, const poplar::DebugContext &dc,
              const poplar::OptionFlags &options, PlanningCache *cache) {
  if (A.rank() != 2 || B.rank() != 2)
    throw poplibs_error("Operand to matrix multiplication is not a matrix");
  return matMulGrouped(graph, A.expand({0}), B.expand({0}), prog, outputType, dc, options, cache)[0];
}

Tensor matMul(Graph &graph, const Tensor &A, const Tensor &B, Sequence &prog,
              const poplar::DebugContext &dc, const poplar::OptionFlags &options,
              PlanningCache *cache) {
  return matMul(graph, A, B, prog, A.elementType(), dc, options, cache);
}

void matMulWithOutput(Graph &graph, const Tensor &A, const Tensor &B, Tensor &out, Sequence &prog,
                      const poplar::DebugContext &, const poplar::OptionFlags &options,
                      PlanningCache *) {
  if (A.rank() != 2 || B.rank() != 2 || out.rank() != 2)
    throw poplibs_error("Operand to matrix multiplication is not a matrix");
  matMulImpl(graph, A.expand({0}), B.expand({0}), out.expand({0}), 1.f, 0.f, prog, options);
}

void matMulGroupedAcc(Graph &graph, const Tensor &C, float k, const Tensor &A, const Tensor &B,
                      Sequence &prog, const poplar::DebugContext &,
                      const poplar::OptionFlags &options, PlanningCache *) {
  matMulImpl(graph, A, B, C, k, 1.f, prog, options);
}

void matMulAcc(Graph &graph, const Tensor &C, float k, const Tensor &A, const Tensor &B,
               Sequence &prog, const poplar::DebugContext &, const poplar::OptionFlags &options,
               PlanningCache *) {
  if (A.rank() != 2 || B.rank() != 2 || C.rank() != 2)
    throw poplibs_error("Operand to matrix multiplication is not a matrix");
  matMulImpl(graph, A.expand({0}), B.expand({0}), C.expand({0}), k, 1.f, prog, options);
}

// ---- operand creation ------------------------------------------------------------
Tensor createMatMulGroupedInputLHS(Graph &graph, const poplar::Type &inputType,
                                   const poplar::Type &outputType,
                                   const std::vector<std::size_t> &aShape,
                                   const std::vector<std::size_t> &bShape,
                                   const poplar::DebugContext &dc,
                                   const poplar::OptionFlags &options, PlanningCache *) {
  dimChecks(aShape, bShape);
  typeChecks(inputType, outputType);
  matmulValidateOptions(options);
  return allocMatrix(graph, inputType, aShape, dc);
}

Tensor createMatMulGroupedInputRHS(Graph &graph, const poplar::Type &inputType,
                                   const poplar::Type &outputType,
                                   const std::vector<std::size_t> &aShape,
                                   const std::vector<std::size_t> &bShape,
                                   const poplar::DebugContext &dc,
                                   const poplar::OptionFlags &options, PlanningCache *) {
  dimChecks(aShape, bShape);
  typeChecks(inputType, outputType);
  matmulValidateOptions(options);
  // stored [g][n][k] (K contiguous: the layout both operand types read without
  // any rearrangement), presented as [g][k][n]
  return allocMatrix(graph, inputType, {bShape[0], bShape[2], bShape[1]}, dc)
      .dimShufflePartial({1, 2}, {2, 1});
}

Tensor createMatMulGroupedOutput(Graph &graph, const poplar::Type &inputType,
                                 const poplar::Type &outputType,
                                 const std::vector<std::size_t> &aShape,
                                 const std::vector<std::size_t> &bShape,
                                 const poplar::DebugContext &dc, const poplar::OptionFlags &options,
                                 PlanningCache *) {
  dimChecks(aShape, bShape);
  typeChecks(inputType, outputType);
  matmulValidateOptions(options);
  return allocMatrix(graph, outputType, {aShape[0], aShape[1], bShape[2]}, dc);
}

Tensor createMatMulInputLHS(Graph &graph, const poplar::Type &inputType,
                            const poplar::Type &outputType, const std::vector<std::size_t> &aShape,
                            const std::vector<std::size_t> &bShape, const poplar::DebugContext &dc,
                            const poplar::OptionFlags &options, PlanningCache *cache) {
  return createMatMulGroupedInputLHS(graph, inputType, outputType, grouped(aShape), grouped(bShape),
                                     dc, options, cache)[0];
}
Tensor createMatMulInputLHS(Graph &graph, const poplar::Type &dataType,
                            const std::vector<std::size_t> &aShape,
                            const std::vector<std::size_t> &bShape, const poplar::DebugContext &dc,
                            const poplar::OptionFlags &options, PlanningCache *cache) {
  return createMatMulInputLHS(graph, dataType, dataType, aShape, bShape, dc, options, cache);
}
Tensor createMatMulInputRHS(Graph &graph, const poplar::Type &inputType,
                            const poplar::Type &outputType, const std::vector<std::size_t> &aShape,
                            const std::vector<std::size_t> &bShape, const poplar::DebugContext &dc,
                            const poplar::OptionFlags &options, PlanningCache *cache) {
  return createMatMulGroupedInputRHS(graph, inputType, outputType, grouped(aShape), grouped(bShape),
                                     dc, options, cache)[0];
}
Tensor createMatMulInputRHS(Graph &graph, const poplar::Type &dataType,
                            const std::vector<std::size_t> &aShape,
                            const std::vector<std::size_t> &bShape, const poplar::DebugContext &dc,
                            const poplar::OptionFlags &options, PlanningCache *cache) {
  return createMatMulInputRHS(graph, dataType, dataType, aShape, bShape, dc, options, cache);
}
Tensor createMatMulOutput(Graph &graph, const poplar::Type &inputType,
                          const poplar::Type &outputType, const std::vector<std::size_t> &aShape,
                          const std::vector<std::size_t> &bShape, const poplar::DebugContext &dc,
                          const poplar::OptionFlags &options, PlanningCache *cache) {
  return createMatMulGroupedOutput(graph, inputType, outputType, grouped(aShape), grouped(bShape),
                                   dc, options, cache)[0];
}
Tensor createMatMulOutput(Graph &graph, const poplar::Type &dataType,
                          const std::vector<std::size_t> &aShape,
                          const std::vector<std::size_t> &bShape, const poplar::DebugContext &dc,
                          const poplar::OptionFlags &options, PlanningCache *cache) {
  return createMatMulOutput(graph, dataType, dataType, aShape, bShape, dc, options, cache);
}

Tensor preArrangeMatMulGroupedInputRHS(Graph &graph, const std::vector<std::size_t> &aShape,
                                       const Tensor &B, Sequence &prog,
                                       const poplar::Type &outputType,
                                       const poplar::DebugContext &dc,
                                       const poplar::OptionFlags &options, PlanningCache *cache) {
  Tensor arranged = createMatMulGroupedInputRHS(graph, B.elementType(), outputType, aShape,
                                                B.shape(), dc, options, cache);
  prog.add(poplar::program::Copy(B, arranged));
  return arranged;
}
Tensor preArrangeMatMulInputRHS(Graph &graph, const std::vector<std::size_t> &aShape,
                                const Tensor &B, Sequence &prog, const poplar::Type &outputType,
                                const poplar::DebugContext &dc, const poplar::OptionFlags &options,
                                PlanningCache *cache) {
  return preArrangeMatMulGroupedInputRHS(graph, grouped(aShape), B.expand({0}), prog, outputType,
                                         dc, options, cache)[0];
}
Tensor preArrangeMatMulInputRHS(Graph &graph, const std::vector<std::size_t> &aShape,
                                const Tensor &B, Sequence &prog, const poplar::DebugContext &dc,
                                const poplar::OptionFlags &options, PlanningCache *cache) {
  return preArrangeMatMulInputRHS(graph, aShape, B, prog, B.elementType(), dc, options, cache);
}

Tensor transposeGroupedMatrix(const Tensor &A) {
  if (A.rank() != 3) throw poplibs_error("transposeGroupedMatrix needs a [g][a][b] tensor");
  return A.dimShufflePartial({1, 2}, {2, 1});
}

// ---- planning ----------------------------------------------------------------------
bool operator<(const MatMulParams &a, const MatMulParams &b) {
  return std::tie(a.inputType, a.outputType, a.aShape, a.bShape) <
         std::tie(b.inputType, b.outputType, b.aShape, b.bShape);
}

// The convolution a grouped product is planned as (lib/poplin/MatMul.cpp:236-273):
// batch = m, 1-element field and kernel, input channels = k, output channels = n.
static ConvParams convParamsOf(const poplar::Type &inputType, const poplar::Type &outputType,
                               const std::vector<std::size_t> &aShape,
                               const std::vector<std::size_t> &bShape) {
  dimChecks(aShape, bShape);
  return ConvParams(inputType, outputType, aShape[1], {1}, {1}, aShape[2], bShape[2], aShape[0]);
}

std::set<ConvPlanParams> matMulGetConvPlanParams(const std::set<MatMulPlanParams> &matmuls,
                                                 MatMulToConvOptions &matmulToConvOpts) {
  std::set<ConvPlanParams> convs;
  static const poplar::OptionFlags none;
  for (const auto &mm : matmuls) {
    const poplar::OptionFlags *opts = std::get<2>(mm) ? std::get<2>(mm) : &none;
    auto it = matmulToConvOpts.find(opts);
    if (it == matmulToConvOpts.end())
      it = matmulToConvOpts.emplace(opts, internal::matMulToConvOptions(*opts)).first;
    const MatMulParams &p = std::get<1>(mm);
    auto a = p.aShape, b = p.bShape;
    if (a.size() == 2) a = grouped(a);
    if (b.size() == 2) b = grouped(b);
    convs.emplace(std::get<0>(mm), convParamsOf(p.inputType, p.outputType, a, b), &it->second);
  }
  return convs;
}

void preplanMatMuls(const std::set<MatMulPlanParams> &matmuls, matmul::PlanningCache &cache) {
  MatMulToConvOptions convOpts;
  const auto convs = matMulGetConvPlanParams(matmuls, convOpts);
  preplanConvolutions(convs, cache.getImpl());
}

void matMulGroupedReportPlan(std::ostream &out, const Graph &, const poplar::Type &inputType,
                             const poplar::Type &outputType, const std::vector<std::size_t> &aShape,
                             const std::vector<std::size_t> &bShape,
                             const poplar::OptionFlags &options, PlanningCache *) {
  dimChecks(aShape, bShape);
  typeChecks(inputType, outputType);
  matmulValidateOptions(options);
  plb_matmul_desc d{};
  d.groups = uint32_t(aShape[0]);
  d.m = uint32_t(aShape[1]);
  d.k = uint32_t(aShape[2]);
  d.n = uint32_t(bShape[2]);
  d.input_type = poplar::detail::dtypeOf(inputType);
  d.output_type = poplar::detail::dtypeOf(outputType);
  d.partials_type = PLB_FLOAT;
  d.transpose_b = 1;  // operands from createMatMulGroupedInputRHS are [n][k] in memory
  d.alpha = 1.f;
  plb_plan plan{};
  poplar::detail::check(plb_matmul_plan(&d, &plan));
  out << "  Matrix product " << shapeText(aShape) << " x " << shapeText(bShape) << " ("
      << inputType << " -> " << outputType << "), planned as the convolution\n"
      << convParamsOf(inputType, outputType, aShape, bShape)
      << "  Plan:\n"
      << "        CTA tile (rows x cols)     " << plan.tile_m << " x " << plan.tile_n << "\n"
      << "        K bytes per stage          " << plan.tile_k_bytes << "\n"
      << "        pipeline stages            " << plan.stages << "\n"
      << "        output tiles               " << plan.tiles << "\n"
      << "        CTAs launched              " << plan.grid << "\n"
      << "        FLOPs                      " << plan.flops << "\n"
      << "        bytes (operands + output)  " << plan.bytes << "\n";
}

void matMulReportPlan(std::ostream &out, const Graph &graph, const poplar::Type &inputType,
                      const poplar::Type &outputType, const std::vector<std::size_t> &aShape,
                      const std::vector<std::size_t> &bShape, const poplar::OptionFlags &options,
                      PlanningCache *cache) {
  matMulGroupedReportPlan(out, graph, inputType, outputType, grouped(aShape), grouped(bShape),
                          options, cache);
}

// ---- fully connected layers ------------------------------------------------------------
namespace fc {

std::vector<std::pair<MatMulParams, poplar::OptionFlags>>
getMatMulPrePlanParameters(FullyConnectedParams p, poplar::OptionFlags matmulOptions,
                           poplar::Type type, bool inferenceOnly) {
  // forward: [batch x in] . [in x out]; backward swaps in and out; the weight
  // update swaps in and batch
  auto make = [&](std::size_t batch, std::size_t in, std::size_t out) {
    return MatMulParams{type, type, {p.numGroups, batch, in}, {p.numGroups, in, out}};
  };
  std::vector<std::pair<MatMulParams, poplar::OptionFlags>> result;
  poplar::OptionFlags fwd = matmulOptions;
  fwd.set("fullyConnectedPass", inferenceOnly ? "INFERENCE_FWD" : "TRAINING_FWD");
  result.emplace_back(make(p.batchSize, p.inputSize, p.outputSize), fwd);
  if (!inferenceOnly) {
    poplar::OptionFlags bwd = matmulOptions, wu = matmulOptions;
    bwd.set("fullyConnectedPass", "TRAINING_BWD");
    wu.set("fullyConnectedPass", "TRAINING_WU");
    result.emplace_back(make(p.batchSize, p.outputSize, p.inputSize), bwd);
    result.emplace_back(make(p.inputSize, p.batchSize, p.outputSize), wu);
  }
  return result;
}

}  // namespace fc
}  // namespace poplin
