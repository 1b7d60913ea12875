// Stand-in for poplar::program: a Sequence is a recorded list of steps that the
// Engine replays on the graph's CUDA stream.  poplin entry points append steps
// and compute nothing themselves, as in the reference (every public call there
// appends to a poplar::program::Sequence; lib/poplin/Convolution.cpp:2208-2290).
#ifndef poplar_Program_hpp
#define poplar_Program_hpp

#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "poplar/DebugContext.hpp"
#include "poplar/Tensor.hpp"

struct plb_context;

namespace poplar {

class Graph;

namespace program {

/// One replayable step; it enqueues work on the context's stream.
using Step = std::function<void(plb_context *)>;

class Program {
public:
  virtual ~Program() = default;
  const std::vector<Step> &steps() const { return *steps_; }

protected:
  Program() : steps_(std::make_shared<std::vector<Step>>()) {}
  std::shared_ptr<std::vector<Step>> steps_;
};

class Sequence : public Program {
public:
  Sequence() = default;
  Sequence(const DebugContext &) {}
  template <class... Ps> explicit Sequence(const Program &first, const Ps &...rest) {
    add(first);
    (add(rest), ...);
  }
  void add(const Program &p) {
    // a Sequence added to itself would recurse forever; Poplar forbids it too
    if (p.steps().data() == steps_->data() && !steps_->empty()) return;
    steps_->insert(steps_->end(), p.steps().begin(), p.steps().end());
  }
  void add(Step s) { steps_->push_back(std::move(s)); }
  bool isEmpty() const { return steps_->empty(); }
};

/// dst = src, element by element over the logical shapes (any strides).
class Copy : public Program {
public:
  Copy(const Tensor &src, const Tensor &dst, bool dontOutline = false,
       const DebugContext &dc = {});
};

/// Runs `body` `count` times.
class Repeat : public Program {
public:
  Repeat(unsigned count, const Program &body, const DebugContext &dc = {});
};

/// No-op on this target (liveness hint in Poplar).
class WriteUndef : public Program {
public:
  explicit WriteUndef(const Tensor &, const DebugContext & = {}) {}
};

} // namespace program
} // namespace poplar

#endif // poplar_Program_hpp
