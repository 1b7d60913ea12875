// poplin matrix-multiplication entry points with the call surface of the
// reference's include/poplin/MatMul.hpp:110-694.  A product is planned and run
// as the 1x1 convolution the reference maps it to (lib/poplin/MatMul.cpp:
// 236-273, 368-404): batch = m, input channels = k, output channels = n.
//
// Options (lib/poplin/MatMul.cpp:113-157): partialsType, fullyConnectedPass,
// inputRHSIsPreArranged, use128BitConvUnitLoad, enableMultiStageReduce,
// enableFastReduce, remapOutputTensor, availableMemoryProportion,
// planConstraints, gatherOutput, disableSRForAMPVertices.  The IPU-only ones
// are parsed and have no effect here.
#ifndef poplin_MatMul_hpp
#define poplin_MatMul_hpp

#include <iosfwd>
#include <set>
#include <tuple>
#include <unordered_map>
#include <vector>

#include "poplin/Convolution.hpp"

namespace poplin {

poplar::Tensor matMul(poplar::Graph &graph, const poplar::Tensor &A, const poplar::Tensor &B,
                      poplar::program::Sequence &prog, const poplar::Type &outputType,
                      const poplar::DebugContext &debugContext = {},
                      const poplar::OptionFlags &options = {}, PlanningCache *cache = nullptr);
poplar::Tensor matMul(poplar::Graph &graph, const poplar::Tensor &A, const poplar::Tensor &B,
                      poplar::program::Sequence &prog, const poplar::DebugContext &debugContext = {},
                      const poplar::OptionFlags &options = {}, PlanningCache *cache = nullptr);
void matMulWithOutput(poplar::Graph &graph, const poplar::Tensor &A, const poplar::Tensor &B,
                      poplar::Tensor &out, poplar::program::Sequence &prog,
                      const poplar::DebugContext &debugContext = {},
                      const poplar::OptionFlags &options = {}, PlanningCache *cache = nullptr);
void matMulReportPlan(std::ostream &out, const poplar::Graph &graph, const poplar::Type &inputType,
                      const poplar::Type &outputType, const std::vector<std::size_t> &aShape,
                      const std::vector<std::size_t> &bShape,
                      const poplar::OptionFlags &options = {}, PlanningCache *cache = nullptr);

/// Grouped forms: A [g][m][k], B [g][k][n], result [g][m][n].
poplar::Tensor matMulGrouped(poplar::Graph &graph, const poplar::Tensor &A,
                             const poplar::Tensor &B, poplar::program::Sequence &prog,
                             const poplar::Type &outputType,
                             const poplar::DebugContext &debugContext = {},
                             const poplar::OptionFlags &options = {},
                             PlanningCache *cache = nullptr);
void matMulGroupedWithOutput(poplar::Graph &graph, const poplar::Tensor &A,
                             const poplar::Tensor &B, poplar::Tensor &out,
                             poplar::program::Sequence &prog,
                             const poplar::DebugContext &debugContext = {},
                             const poplar::OptionFlags &options = {},
                             PlanningCache *cache = nullptr);
void matMulGroupedReportPlan(std::ostream &out, const poplar::Graph &graph,
                             const poplar::Type &inputType, const poplar::Type &outputType,
                             const std::vector<std::size_t> &aShape,
                             const std::vector<std::size_t> &bShape,
                             const poplar::OptionFlags &options = {},
                             PlanningCache *cache = nullptr);

/// C += k * A * B.
void matMulAcc(poplar::Graph &graph, const poplar::Tensor &C, float k, const poplar::Tensor &A,
               const poplar::Tensor &B, poplar::program::Sequence &prog,
               const poplar::DebugContext &debugContext = {},
               const poplar::OptionFlags &options = {}, PlanningCache *cache = nullptr);
void matMulGroupedAcc(poplar::Graph &graph, const poplar::Tensor &C, float k,
                      const poplar::Tensor &A, const poplar::Tensor &B,
                      poplar::program::Sequence &prog,
                      const poplar::DebugContext &debugContext = {},
                      const poplar::OptionFlags &options = {}, PlanningCache *cache = nullptr);

poplar::Tensor createMatMulInputLHS(poplar::Graph &graph, const poplar::Type &inputType,
                                    const poplar::Type &outputType,
                                    const std::vector<std::size_t> &aShape,
                                    const std::vector<std::size_t> &bShape,
                                    const poplar::DebugContext &debugContext,
                                    const poplar::OptionFlags &options = {},
                                    PlanningCache *cache = nullptr);
poplar::Tensor createMatMulInputLHS(poplar::Graph &graph, const poplar::Type &dataType,
                                    const std::vector<std::size_t> &aShape,
                                    const std::vector<std::size_t> &bShape,
                                    const poplar::DebugContext &debugContext,
                                    const poplar::OptionFlags &options = {},
                                    PlanningCache *cache = nullptr);
poplar::Tensor createMatMulGroupedInputLHS(poplar::Graph &graph, const poplar::Type &inputType,
                                           const poplar::Type &outputType,
                                           const std::vector<std::size_t> &aShape,
                                           const std::vector<std::size_t> &bShape,
                                           const poplar::DebugContext &debugContext,
                                           const poplar::OptionFlags &options = {},
                                           PlanningCache *cache = nullptr);
poplar::Tensor createMatMulInputRHS(poplar::Graph &graph, const poplar::Type &inputType,
                                    const poplar::Type &outputType,
                                    const std::vector<std::size_t> &aShape,
                                    const std::vector<std::size_t> &bShape,
                                    const poplar::DebugContext &debugContext,
                                    const poplar::OptionFlags &options = {},
                                    PlanningCache *cache = nullptr);
poplar::Tensor createMatMulInputRHS(poplar::Graph &graph, const poplar::Type &dataType,
                                    const std::vector<std::size_t> &aShape,
                                    const std::vector<std::size_t> &bShape,
                                    const poplar::DebugContext &debugContext,
                                    const poplar::OptionFlags &options = {},
                                    PlanningCache *cache = nullptr);
poplar::Tensor createMatMulGroupedInputRHS(poplar::Graph &graph, const poplar::Type &inputType,
                                           const poplar::Type &outputType,
                                           const std::vector<std::size_t> &aShape,
                                           const std::vector<std::size_t> &bShape,
                                           const poplar::DebugContext &debugContext,
                                           const poplar::OptionFlags &options = {},
                                           PlanningCache *cache = nullptr);
poplar::Tensor createMatMulOutput(poplar::Graph &graph, const poplar::Type &inputType,
                                  const poplar::Type &outputType,
                                  const std::vector<std::size_t> &aShape,
                                  const std::vector<std::size_t> &bShape,
                                  const poplar::DebugContext &debugContext,
                                  const poplar::OptionFlags &options = {},
                                  PlanningCache *cache = nullptr);
poplar::Tensor createMatMulOutput(poplar::Graph &graph, const poplar::Type &dataType,
                                  const std::vector<std::size_t> &aShape,
                                  const std::vector<std::size_t> &bShape,
                                  const poplar::DebugContext &debugContext,
                                  const poplar::OptionFlags &options = {},
                                  PlanningCache *cache = nullptr);
poplar::Tensor createMatMulGroupedOutput(poplar::Graph &graph, const poplar::Type &inputType,
                                         const poplar::Type &outputType,
                                         const std::vector<std::size_t> &aShape,
                                         const std::vector<std::size_t> &bShape,
                                         const poplar::DebugContext &debugContext,
                                         const poplar::OptionFlags &options = {},
                                         PlanningCache *cache = nullptr);

/// Copies B into the layout the kernel reads fastest ([n][k], K contiguous) and
/// returns a [k][n]-shaped view of it, for use with inputRHSIsPreArranged.
poplar::Tensor preArrangeMatMulInputRHS(poplar::Graph &graph,
                                        const std::vector<std::size_t> &aShape,
                                        const poplar::Tensor &B, poplar::program::Sequence &prog,
                                        const poplar::Type &outputType,
                                        const poplar::DebugContext &debugContext = {},
                                        const poplar::OptionFlags &options = {},
                                        PlanningCache *cache = nullptr);
poplar::Tensor preArrangeMatMulInputRHS(poplar::Graph &graph,
                                        const std::vector<std::size_t> &aShape,
                                        const poplar::Tensor &B, poplar::program::Sequence &prog,
                                        const poplar::DebugContext &debugContext = {},
                                        const poplar::OptionFlags &options = {},
                                        PlanningCache *cache = nullptr);
poplar::Tensor preArrangeMatMulGroupedInputRHS(poplar::Graph &graph,
                                               const std::vector<std::size_t> &aShape,
                                               const poplar::Tensor &B,
                                               poplar::program::Sequence &prog,
                                               const poplar::Type &outputType,
                                               const poplar::DebugContext &debugContext = {},
                                               const poplar::OptionFlags &options = {},
                                               PlanningCache *cache = nullptr);
/// [g][a][b] -> [g][b][a] view.
poplar::Tensor transposeGroupedMatrix(const poplar::Tensor &A);

struct MatMulParams {
  poplar::Type inputType;
  poplar::Type outputType;
  std::vector<std::size_t> aShape;
  std::vector<std::size_t> bShape;
  friend bool operator<(const MatMulParams &a, const MatMulParams &b);
};
using MatMulPlanParams =
    std::tuple<const poplar::Target *, const MatMulParams, const poplar::OptionFlags *>;
using MatMulToConvOptions = std::unordered_map<const poplar::OptionFlags *, poplar::OptionFlags>;
std::set<ConvPlanParams> matMulGetConvPlanParams(const std::set<MatMulPlanParams> &matmuls,
                                                 MatMulToConvOptions &matmulToConvOpts);
void matmulValidateOptions(const poplar::OptionFlags &options);

namespace matmul {
class PlanningCache : public poplin::PlanningCache {
public:
  poplin::PlanningCache &getImpl() { return *this; }
};
} // namespace matmul
/// \deprecated Use preplan().
void preplanMatMuls(const std::set<MatMulPlanParams> &matmuls, matmul::PlanningCache &cache);

} // namespace poplin

#endif // poplin_MatMul_hpp
