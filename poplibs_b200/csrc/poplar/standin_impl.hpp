// Internals shared by the poplar stand-in and the poplin layer.
#pragma once

#include <cstddef>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "poplar/Graph.hpp"
#include "poplar/Tensor.hpp"
#include "poplibs_b200.h"

namespace poplar {
namespace detail {

// One allocation.  Device memory is attached when the Engine is built (graph
// construction itself needs no GPU), and released with the last handle.
struct Storage {
  std::size_t elements = 0;
  Type type;
  std::string name;
  void *device = nullptr;
  plb_context *ctx = nullptr;
  bool hasMetadata = false;
  QuarterMetadata metadata;
  bool isConstant = false;
  double constantValue = 0.0;
  ~Storage();
};

struct GraphImpl {
  Target target;
  plb_context *ctx = nullptr;  // created on first use
  std::vector<std::weak_ptr<Storage>> storages;
  std::map<std::string, Tensor> hostWrites, hostReads;
  ~GraphImpl();
};

// Throws the exception type that corresponds to a C ABI status.
[[noreturn]] void throwStatus(int status);
inline void check(int status) {
  if (status != 0) throwStatus(status);
}

int dtypeOf(const Type &t);  // plb_dtype; throws for unsupported element types

}  // namespace detail
}  // namespace poplar
