// Stand-in for poplar::Engine: replays recorded programs on the graph's CUDA
// stream and moves host data in and out (tools/single_conv_layer.cpp:1169,
// 1326-1340 show the protocol: construct, load, run(i), read back).
#ifndef poplar_Engine_hpp
#define poplar_Engine_hpp

#include <iosfwd>
#include <string>
#include <vector>

#include "poplar/Graph.hpp"
#include "poplar/OptionFlags.hpp"
#include "poplar/Program.hpp"

namespace poplar {

class Device {
public:
  Device() = default;
};

class Engine {
public:
  Engine(Graph &graph, const program::Program &prog, const OptionFlags &opt = {});
  Engine(Graph &graph, const std::vector<program::Sequence> &progs, const OptionFlags &opt = {});

  void load(const Device &) {}
  /// Runs program `index` and waits for it; throws poplar::runtime_error if a
  /// kernel reported a failure.
  void run(unsigned index = 0);
  /// Device time of the last run() in milliseconds (CUDA events).
  double lastRunMilliseconds() const { return last_ms_; }

  /// Host -> tensor registered with Graph::createHostWrite, logical row-major
  /// order, elements in the tensor's device type.
  void writeTensor(const std::string &handle, const void *begin, const void *end);
  void writeTensor(const std::string &handle, const void *begin) { writeTensor(handle, begin, nullptr); }
  void readTensor(const std::string &handle, void *begin, void *end);
  void readTensor(const std::string &handle, void *begin) { readTensor(handle, begin, nullptr); }

  void printProfileSummary(std::ostream &os, const OptionFlags &opt = {}) const;

private:
  Graph *graph_;
  std::vector<std::vector<program::Step>> programs_;
  double last_ms_ = 0.0;
  unsigned long long launches_ = 0;
};

/// Copies `t` (any view) to / from a dense row-major staging buffer on the
/// device; shared by the Engine and by program::Copy.
void copyViewToDense(plb_context *ctx, const Tensor &t, void *denseDevice);
void copyDenseToView(plb_context *ctx, const void *denseDevice, const Tensor &t);

} // namespace poplar

#endif // poplar_Engine_hpp
