// Stand-in for poplar::DebugContext / DebugNameAndId: a name that poplin entry
// points carry for logging (include/poplin/Convolution.hpp:345-384).
#ifndef poplar_DebugContext_hpp
#define poplar_DebugContext_hpp

#include <string>

namespace poplar {

class DebugContext {
public:
  DebugContext() = default;
  DebugContext(const char *name) : name_(name ? name : "") {}
  DebugContext(const std::string &name) : name_(name) {}
  DebugContext(const DebugContext &parent, const std::string &name)
      : name_(parent.name_.empty() ? name : parent.name_ + "/" + name) {}
  const std::string &getPathName() const { return name_; }

private:
  std::string name_;
};

using DebugNameAndId = DebugContext;

} // namespace poplar

#endif // poplar_DebugContext_hpp
