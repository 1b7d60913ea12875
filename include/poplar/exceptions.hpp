// Exception types of the Poplar SDK that the poplin path throws or documents
// (include/poputil/OptionParsing.hpp:204-221; tools/single_conv_layer.cpp:1532).
#ifndef poplar_exceptions_hpp
#define poplar_exceptions_hpp

#include <stdexcept>
#include <string>

namespace poplar {

struct poplar_error : std::runtime_error {
  explicit poplar_error(const std::string &s) : std::runtime_error(s) {}
};
/// Unknown option name or unparsable option value.
struct invalid_option : poplar_error {
  explicit invalid_option(const std::string &s) : poplar_error(s) {}
};
/// The device cannot hold the tensors the program needs.
struct graph_memory_allocation_error : poplar_error {
  explicit graph_memory_allocation_error(const std::string &s) : poplar_error(s) {}
};
/// Runtime (CUDA) failure while a program runs.
struct runtime_error : poplar_error {
  explicit runtime_error(const std::string &s) : poplar_error(s) {}
};

} // namespace poplar

#endif // poplar_exceptions_hpp
