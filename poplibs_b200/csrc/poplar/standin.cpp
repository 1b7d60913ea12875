// Implementation of the poplar stand-in: types, option flags, tensor views,
// graph storage, recorded programs and the replaying Engine.  Everything that
// touches the GPU goes through the C ABI (include/poplibs_b200.h).
#include <algorithm>
#include <cctype>
#include <cstring>
#include <iostream>
#include <numeric>
#include <sstream>

#include "poplar/Engine.hpp"
#include "poplar/Graph.hpp"
#include "poplar/OptionFlags.hpp"
#include "poplar/Program.hpp"
#include "poplar/Tensor.hpp"
#include "poplar/Type.hpp"
#include "poplar/exceptions.hpp"
#include "poputil/exceptions.hpp"
#include "standin_impl.hpp"

namespace poplar {

// ---------------------------------------------------------------- Type -------
const Type BOOL(Type::Kind::Bool), CHAR(Type::Kind::Char), UNSIGNED_CHAR(Type::Kind::UnsignedChar),
    SHORT(Type::Kind::Short), UNSIGNED_SHORT(Type::Kind::UnsignedShort), INT(Type::Kind::Int),
    UNSIGNED_INT(Type::Kind::UnsignedInt), HALF(Type::Kind::Half), FLOAT(Type::Kind::Float),
    QUARTER(Type::Kind::Quarter), QUARTER_METADATA(Type::Kind::QuarterMetadata);

std::string Type::toString() const {
  switch (kind_) {
    case Kind::Bool: return "bool";
    case Kind::Char: return "char";
    case Kind::UnsignedChar: return "unsigned char";
    case Kind::Short: return "short";
    case Kind::UnsignedShort: return "unsigned short";
    case Kind::Int: return "int";
    case Kind::UnsignedInt: return "unsigned int";
    case Kind::Half: return "half";
    case Kind::Float: return "float";
    case Kind::Quarter: return "quarter";
    case Kind::QuarterMetadata: return "quarter_metadata";
    default: return "invalid";
  }
}

std::size_t Type::bytes() const {
  switch (kind_) {
    case Kind::Bool:
    case Kind::Char:
    case Kind::UnsignedChar:
    case Kind::Quarter:
    case Kind::QuarterMetadata: return 1;
    case Kind::Short:
    case Kind::UnsignedShort:
    case Kind::Half: return 2;
    case Kind::Int:
    case Kind::UnsignedInt:
    case Kind::Float: return 4;
    default: return 0;
  }
}

std::ostream &operator<<(std::ostream &os, const Type &t) { return os << t.toString(); }

Type typeFromString(const std::string &s) {
  for (const Type *t : {&BOOL, &CHAR, &UNSIGNED_CHAR, &SHORT, &UNSIGNED_SHORT, &INT, &UNSIGNED_INT,
                        &HALF, &FLOAT, &QUARTER})
    if (t->toString() == s) return *t;
  throw invalid_option("Unknown type '" + s + "'");
}

std::ostream &operator<<(std::ostream &os, QuarterMetadata::Format f) {
  return os << (f == QuarterMetadata::Format::F143 ? "F143" : "F152");
}

// --------------------------------------------------------- OptionFlags -------
namespace {

void skipSpace(const std::string &s, std::size_t &i) {
  while (i < s.size() && std::isspace(static_cast<unsigned char>(s[i]))) ++i;
}

std::string parseJsonString(const std::string &s, std::size_t &i) {
  if (s[i] != '"') throw invalid_option("JSON: expected a string");
  std::string out;
  for (++i; i < s.size() && s[i] != '"'; ++i) {
    if (s[i] == '\\' && i + 1 < s.size()) ++i;
    out.push_back(s[i]);
  }
  if (i >= s.size()) throw invalid_option("JSON: unterminated string");
  ++i;
  return out;
}

// Text of the JSON value starting at i (object, array, string or scalar).
std::string parseJsonValueText(const std::string &s, std::size_t &i) {
  skipSpace(s, i);
  if (i >= s.size()) throw invalid_option("JSON: unexpected end");
  if (s[i] == '"') return parseJsonString(s, i);
  const std::size_t begin = i;
  if (s[i] == '{' || s[i] == '[') {
    int depth = 0;
    bool inString = false;
    for (; i < s.size(); ++i) {
      const char c = s[i];
      if (inString) {
        if (c == '\\') ++i;
        else if (c == '"') inString = false;
      } else if (c == '"') inString = true;
      else if (c == '{' || c == '[') ++depth;
      else if (c == '}' || c == ']') {
        if (--depth == 0) {
          ++i;
          return s.substr(begin, i - begin);
        }
      }
    }
    throw invalid_option("JSON: unbalanced brackets");
  }
  while (i < s.size() && s[i] != ',' && s[i] != '}' && !std::isspace(static_cast<unsigned char>(s[i])))
    ++i;
  return s.substr(begin, i - begin);
}

}  // namespace

void readJSON(const std::string &json, OptionFlags &flags) {
  std::size_t i = 0;
  skipSpace(json, i);
  if (i >= json.size() || json[i] != '{') throw invalid_option("JSON: expected an object");
  ++i;
  skipSpace(json, i);
  if (i < json.size() && json[i] == '}') return;
  for (;;) {
    skipSpace(json, i);
    const std::string key = parseJsonString(json, i);
    skipSpace(json, i);
    if (i >= json.size() || json[i] != ':') throw invalid_option("JSON: expected ':'");
    ++i;
    flags.set(key, parseJsonValueText(json, i));
    skipSpace(json, i);
    if (i < json.size() && json[i] == ',') {
      ++i;
      continue;
    }
    if (i < json.size() && json[i] == '}') return;
    throw invalid_option("JSON: expected ',' or '}'");
  }
}

void readJSON(std::istream &stream, OptionFlags &flags) {
  std::stringstream ss;
  ss << stream.rdbuf();
  readJSON(ss.str(), flags);
}

std::ostream &operator<<(std::ostream &os, const OptionFlags &flags) {
  os << "{";
  bool first = true;
  for (const auto &kv : flags) {
    os << (first ? "" : ", ") << kv.first << ": " << kv.second;
    first = false;
  }
  return os << "}";
}

// --------------------------------------------------------------- detail -------
namespace detail {

Storage::~Storage() {
  if (device && ctx) plb_free(ctx, device);
}

GraphImpl::~GraphImpl() {
  // storages may outlive the graph through tensor handles; detach them first
  for (auto &w : storages)
    if (auto s = w.lock()) {
      if (s->device && s->ctx) plb_free(s->ctx, s->device);
      s->device = nullptr;
      s->ctx = nullptr;
    }
  if (ctx) plb_context_destroy(ctx);
}

void throwStatus(int status) {
  const std::string msg = plb_last_error();
  switch (status) {
    case PLB_ERR_INVALID_PARAMS: throw poputil::poplibs_error(msg);
    case PLB_ERR_INVALID_OPTION: throw invalid_option(msg);
    case PLB_ERR_OUT_OF_MEMORY: throw graph_memory_allocation_error(msg);
    case PLB_ERR_UNSUPPORTED: throw poputil::poplibs_error("not supported on this target: " + msg);
    default: throw runtime_error(msg);
  }
}

int dtypeOf(const Type &t) {
  if (t == HALF) return PLB_HALF;
  if (t == FLOAT) return PLB_FLOAT;
  if (t == QUARTER) return PLB_QUARTER;
  throw poputil::poplibs_error("element type " + t.toString() + " is not supported on this path");
}

}  // namespace detail

// --------------------------------------------------------------- Tensor -------
Tensor::Tensor(std::shared_ptr<detail::Storage> storage, Type type, std::vector<std::size_t> shape)
    : storage_(std::move(storage)), type_(type), shape_(std::move(shape)) {
  strides_.resize(shape_.size());
  std::ptrdiff_t stride = 1;
  for (std::size_t i = shape_.size(); i-- > 0;) {
    strides_[i] = stride;
    stride *= static_cast<std::ptrdiff_t>(shape_[i]);
  }
}

std::size_t Tensor::dim(unsigned i) const {
  if (i >= shape_.size()) throw poputil::poplibs_error("Tensor::dim: index out of range");
  return shape_[i];
}

std::size_t Tensor::numElements() const {
  return std::accumulate(shape_.begin(), shape_.end(), std::size_t(1), std::multiplies<std::size_t>());
}

std::string Tensor::shapeToString() const {
  std::string s = "[";
  for (std::size_t i = 0; i < shape_.size(); ++i) s += (i ? "," : "") + std::to_string(shape_[i]);
  return s + "]";
}

bool Tensor::isContiguous() const {
  std::ptrdiff_t expect = 1;
  for (std::size_t i = shape_.size(); i-- > 0;) {
    if (shape_[i] != 1 && strides_[i] != expect) return false;
    expect *= static_cast<std::ptrdiff_t>(shape_[i]);
  }
  return true;
}

Tensor Tensor::reshape(const std::vector<std::size_t> &shape) const {
  const std::size_t n = std::accumulate(shape.begin(), shape.end(), std::size_t(1),
                                        std::multiplies<std::size_t>());
  if (n != numElements())
    throw poputil::poplibs_error("reshape from " + shapeToString() + " changes the element count");
  Tensor out = *this;
  out.shape_ = shape;
  out.strides_.assign(shape.size(), 0);
  if (n == 0) return out;
  // Merge the old dimensions into maximal contiguous runs, then split each run
  // across the new dimensions; a new dimension must not straddle two runs.
  std::vector<std::size_t> oshape;
  std::vector<std::ptrdiff_t> ostride;
  for (std::size_t i = 0; i < shape_.size(); ++i) {
    if (shape_[i] == 1) continue;
    if (!oshape.empty() &&
        ostride.back() == strides_[i] * static_cast<std::ptrdiff_t>(shape_[i])) {
      oshape.back() *= shape_[i];
      ostride.back() = strides_[i];
    } else {
      oshape.push_back(shape_[i]);
      ostride.push_back(strides_[i]);
    }
  }
  std::size_t run = 0, left = oshape.empty() ? 1 : oshape[0];
  for (std::size_t j = 0; j < shape.size(); ++j) {
    const std::size_t d = shape[j];
    if (d == 1) {
      out.strides_[j] = 1;
      continue;
    }
    if (run >= oshape.size() || left % d != 0)
      throw poputil::poplibs_error("reshape of a non-contiguous view from " + shapeToString() +
                                   " would need a copy");
    left /= d;
    out.strides_[j] = ostride[run] * static_cast<std::ptrdiff_t>(left);
    if (left == 1) {
      ++run;
      left = run < oshape.size() ? oshape[run] : 1;
    }
  }
  return out;
}

Tensor Tensor::flatten() const { return reshape({numElements()}); }

Tensor Tensor::flatten(unsigned dimBegin, unsigned dimEnd) const {
  if (dimBegin > dimEnd || dimEnd > rank()) throw poputil::poplibs_error("flatten: bad range");
  std::vector<std::size_t> s(shape_.begin(), shape_.begin() + dimBegin);
  std::size_t n = 1;
  for (unsigned i = dimBegin; i < dimEnd; ++i) n *= shape_[i];
  s.push_back(n);
  s.insert(s.end(), shape_.begin() + dimEnd, shape_.end());
  return reshape(s);
}

Tensor Tensor::reshapePartial(unsigned beginIndex, unsigned endIndex,
                              const std::vector<std::size_t> &newDims) const {
  if (beginIndex > endIndex || endIndex > rank())
    throw poputil::poplibs_error("reshapePartial: bad range");
  std::vector<std::size_t> s(shape_.begin(), shape_.begin() + beginIndex);
  s.insert(s.end(), newDims.begin(), newDims.end());
  s.insert(s.end(), shape_.begin() + endIndex, shape_.end());
  return reshape(s);
}

Tensor Tensor::dimShuffle(const std::vector<unsigned> &permutation) const {
  if (permutation.size() != shape_.size())
    throw poputil::poplibs_error("dimShuffle: permutation has the wrong rank");
  Tensor out = *this;
  std::vector<bool> seen(shape_.size(), false);
  for (std::size_t i = 0; i < permutation.size(); ++i) {
    const unsigned p = permutation[i];
    if (p >= shape_.size() || seen[p]) throw poputil::poplibs_error("dimShuffle: not a permutation");
    seen[p] = true;
    out.shape_[i] = shape_[p];
    out.strides_[i] = strides_[p];
  }
  return out;
}

Tensor Tensor::dimShufflePartial(const std::vector<unsigned> &source,
                                 const std::vector<unsigned> &destination) const {
  if (source.size() != destination.size())
    throw poputil::poplibs_error("dimShufflePartial: size mismatch");
  std::vector<int> perm(shape_.size(), -1);
  std::vector<bool> used(shape_.size(), false);
  for (std::size_t i = 0; i < source.size(); ++i) {
    if (source[i] >= rank() || destination[i] >= rank() || perm[destination[i]] != -1 ||
        used[source[i]])
      throw poputil::poplibs_error("dimShufflePartial: bad indices");
    perm[destination[i]] = int(source[i]);
    used[source[i]] = true;
  }
  unsigned next = 0;
  for (auto &p : perm) {
    if (p != -1) continue;
    while (used[next]) ++next;
    p = int(next);
    used[next] = true;
  }
  return dimShuffle(std::vector<unsigned>(perm.begin(), perm.end()));
}

Tensor Tensor::dimRoll(unsigned dimIdx, unsigned newIdx) const {
  std::vector<unsigned> perm;
  for (unsigned i = 0; i < rank(); ++i)
    if (i != dimIdx) perm.push_back(i);
  if (dimIdx >= rank() || newIdx >= rank()) throw poputil::poplibs_error("dimRoll: bad index");
  perm.insert(perm.begin() + newIdx, dimIdx);
  return dimShuffle(perm);
}

Tensor Tensor::transpose() const {
  if (rank() != 2) throw poputil::poplibs_error("transpose needs a rank-2 tensor");
  return dimShuffle({1, 0});
}

Tensor Tensor::expand(const std::vector<std::size_t> &indices) const {
  Tensor out = *this;
  for (std::size_t k = 0; k < indices.size(); ++k) {
    const std::size_t at = indices[k] + k;  // indices refer to the original rank
    if (at > out.shape_.size()) throw poputil::poplibs_error("expand: index out of range");
    out.shape_.insert(out.shape_.begin() + at, 1);
    out.strides_.insert(out.strides_.begin() + at, 1);
  }
  return out;
}

Tensor Tensor::squeeze(const std::vector<std::size_t> &indices) const {
  Tensor out = *this;
  std::vector<std::size_t> sorted = indices;
  std::sort(sorted.rbegin(), sorted.rend());
  for (std::size_t at : sorted) {
    if (at >= out.shape_.size() || out.shape_[at] != 1)
      throw poputil::poplibs_error("squeeze: dimension is not of size 1");
    out.shape_.erase(out.shape_.begin() + at);
    out.strides_.erase(out.strides_.begin() + at);
  }
  return out;
}

Tensor Tensor::slice(std::size_t begin, std::size_t end, unsigned dimension) const {
  if (dimension >= rank() || begin > end || end > shape_[dimension])
    throw poputil::poplibs_error("slice: range out of bounds");
  Tensor out = *this;
  out.offset_ += static_cast<std::ptrdiff_t>(begin) * strides_[dimension];
  out.shape_[dimension] = end - begin;
  return out;
}

Tensor Tensor::operator[](std::size_t i) const {
  if (rank() == 0) throw poputil::poplibs_error("operator[] on a scalar tensor");
  return slice(i, i + 1, 0).squeeze({0});
}

Tensor Tensor::reverse(unsigned dimension) const {
  if (dimension >= rank()) throw poputil::poplibs_error("reverse: bad dimension");
  Tensor out = *this;
  if (shape_[dimension] > 0)
    out.offset_ += static_cast<std::ptrdiff_t>(shape_[dimension] - 1) * strides_[dimension];
  out.strides_[dimension] = -strides_[dimension];
  return out;
}

bool Tensor::hasMetadata() const { return storage_ && storage_->hasMetadata; }

QuarterMetadata Tensor::getMetadata() const {
  if (!storage_ || type_ != QUARTER)
    throw poputil::poplibs_error("getMetadata: tensor is not of type quarter");
  return storage_->metadata;
}

void *Tensor::devicePointer() const {
  if (!storage_ || !storage_->device)
    throw runtime_error("tensor has no device memory yet (no Engine has been built for its graph)");
  return static_cast<char *>(storage_->device) + offset_ * static_cast<std::ptrdiff_t>(type_.bytes());
}

// ---------------------------------------------------------------- Graph -------
Graph::Graph(const Target &target) : impl_(new detail::GraphImpl()) { impl_->target = target; }
Graph::~Graph() = default;
Graph::Graph(Graph &&) noexcept = default;

const Target &Graph::getTarget() const { return impl_->target; }

static Tensor makeVariable(detail::GraphImpl &g, const Type &type,
                           const std::vector<std::size_t> &shape, const std::string &name) {
  auto st = std::make_shared<detail::Storage>();
  st->type = type;
  st->name = name;
  st->elements = std::accumulate(shape.begin(), shape.end(), std::size_t(1),
                                 std::multiplies<std::size_t>());
  g.storages.push_back(st);
  return Tensor(st, type, shape);
}

Tensor Graph::addVariable(const Type &type, const std::vector<std::size_t> &shape,
                          const DebugContext &dc) {
  return makeVariable(*impl_, type, shape, dc.getPathName());
}

Tensor Graph::addVariable(const Type &type, const std::vector<std::size_t> &shape,
                          VariableMappingMethod, const DebugContext &dc) {
  return addVariable(type, shape, dc);
}

Tensor Graph::addVariable(const Type &type, const Tensor *metadata,
                          const std::vector<std::size_t> &shape, const DebugContext &dc) {
  Tensor t = addVariable(type, shape, dc);
  if (metadata && metadata->valid() && metadata->storage()->hasMetadata)
    setQuarterMetadata(t, metadata->storage()->metadata);
  return t;
}

Tensor Graph::addConstantImpl(const Type &type, const std::vector<std::size_t> &shape, double value,
                              const DebugContext &dc) {
  Tensor t = addVariable(type, shape, dc);
  t.storage()->isConstant = true;
  t.storage()->constantValue = value;
  return t;
}

Tensor Graph::addScratch(const Type &type, const std::vector<std::size_t> &shape) {
  return addVariable(type, shape, DebugContext("scratch"));
}

Tensor Graph::clone(const Tensor &t, const DebugContext &dc, TensorCloneMethod m) {
  return clone(t.elementType(), t, dc, m);
}

Tensor Graph::clone(const Type &type, const Tensor &t, const DebugContext &dc, TensorCloneMethod) {
  // same memory order as the source view: allocate in order of decreasing
  // stride, then permute back to the logical dimension order
  const unsigned r = t.rank();
  std::vector<unsigned> order(r);
  std::iota(order.begin(), order.end(), 0u);
  std::stable_sort(order.begin(), order.end(), [&](unsigned a, unsigned b) {
    const auto sa = std::abs(t.strides()[a]), sb = std::abs(t.strides()[b]);
    return sa > sb;
  });
  std::vector<std::size_t> physical(r);
  for (unsigned i = 0; i < r; ++i) physical[i] = t.shape()[order[i]];
  Tensor base = addVariable(type, physical, dc);
  std::vector<unsigned> inverse(r);
  for (unsigned i = 0; i < r; ++i) inverse[order[i]] = i;
  Tensor out = base.dimShuffle(inverse);
  if (t.valid() && t.storage()->hasMetadata && type == QUARTER)
    setQuarterMetadata(out, t.storage()->metadata);
  return out;
}

void Graph::createHostWrite(const std::string &handle, const Tensor &t) {
  impl_->hostWrites[handle] = t;
}
void Graph::createHostRead(const std::string &handle, const Tensor &t) {
  impl_->hostReads[handle] = t;
}

void Graph::setQuarterMetadata(const Tensor &t, const QuarterMetadata &md) {
  if (!t.valid() || t.elementType() != QUARTER)
    throw poputil::poplibs_error("setQuarterMetadata: tensor is not of type quarter");
  t.storage()->hasMetadata = true;
  t.storage()->metadata = md;
}

plb_context *Graph::context() const {
  if (!impl_->ctx) detail::check(plb_context_create(impl_->target.getDeviceOrdinal(), &impl_->ctx));
  return impl_->ctx;
}

const std::map<std::string, Tensor> &Graph::hostWrites() const { return impl_->hostWrites; }
const std::map<std::string, Tensor> &Graph::hostReads() const { return impl_->hostReads; }

// Attaches device memory to every variable that has none yet.
void Graph::allocateDeviceMemory() {
  plb_context *ctx = context();
  for (auto &w : impl_->storages) {
    auto s = w.lock();
    if (!s || s->device) continue;
    const std::size_t bytes = std::max<std::size_t>(s->elements * s->type.bytes(), 16);
    detail::check(plb_malloc(ctx, bytes, &s->device));
    s->ctx = ctx;
    if (s->isConstant) {
      if (s->type == HALF || s->type == FLOAT)
        detail::check(plb_fill(ctx, detail::dtypeOf(s->type), s->device,
                               static_cast<float>(s->constantValue), s->elements));
      else
        detail::check(plb_memset(ctx, s->device, 0, bytes));
    }
  }
}

// -------------------------------------------------------------- Program -------
void copyViewToDense(plb_context *ctx, const Tensor &t, void *dense) {
  const unsigned r = t.rank();
  std::vector<uint64_t> shape(std::max(r, 1u), 1);
  std::vector<int64_t> ss(std::max(r, 1u), 1), ds(std::max(r, 1u), 1);
  int64_t stride = 1;
  for (unsigned i = r; i-- > 0;) {
    shape[i] = t.shape()[i];
    ss[i] = t.strides()[i];
    ds[i] = stride;
    stride *= int64_t(t.shape()[i]);
  }
  detail::check(plb_copy_strided(ctx, uint32_t(t.elementType().bytes()), std::max(r, 1u),
                                 shape.data(), ss.data(), ds.data(), t.devicePointer(), dense));
}

void copyDenseToView(plb_context *ctx, const void *dense, const Tensor &t) {
  const unsigned r = t.rank();
  std::vector<uint64_t> shape(std::max(r, 1u), 1);
  std::vector<int64_t> ss(std::max(r, 1u), 1), ds(std::max(r, 1u), 1);
  int64_t stride = 1;
  for (unsigned i = r; i-- > 0;) {
    shape[i] = t.shape()[i];
    ds[i] = t.strides()[i];
    ss[i] = stride;
    stride *= int64_t(t.shape()[i]);
  }
  detail::check(plb_copy_strided(ctx, uint32_t(t.elementType().bytes()), std::max(r, 1u),
                                 shape.data(), ss.data(), ds.data(), dense, t.devicePointer()));
}

namespace program {

Copy::Copy(const Tensor &src, const Tensor &dst, bool, const DebugContext &) {
  if (src.shape() != dst.shape())
    throw poputil::poplibs_error("Copy: shapes differ: " + src.shapeToString() + " vs " +
                                 dst.shapeToString());
  if (src.elementType().bytes() != dst.elementType().bytes())
    throw poputil::poplibs_error("Copy: element sizes differ");
  steps_->push_back([src, dst](plb_context *ctx) {
    const unsigned r = std::max(src.rank(), 1u);
    std::vector<uint64_t> shape(r, 1);
    std::vector<int64_t> ss(r, 1), ds(r, 1);
    for (unsigned i = 0; i < src.rank(); ++i) {
      shape[i] = src.shape()[i];
      ss[i] = src.strides()[i];
      ds[i] = dst.strides()[i];
    }
    detail::check(plb_copy_strided(ctx, uint32_t(src.elementType().bytes()), r, shape.data(),
                                   ss.data(), ds.data(), src.devicePointer(), dst.devicePointer()));
    if (src.elementType() == QUARTER && src.storage()->hasMetadata) {
      dst.storage()->hasMetadata = true;
      dst.storage()->metadata = src.storage()->metadata;
    }
  });
}

Repeat::Repeat(unsigned count, const Program &body, const DebugContext &) {
  auto steps = body.steps();
  steps_->push_back([count, steps](plb_context *ctx) {
    for (unsigned i = 0; i < count; ++i)
      for (const auto &s : steps) s(ctx);
  });
}

}  // namespace program

// --------------------------------------------------------------- Engine -------
Engine::Engine(Graph &graph, const program::Program &prog, const OptionFlags &)
    : graph_(&graph) {
  programs_.push_back(prog.steps());
  graph.allocateDeviceMemory();
}

Engine::Engine(Graph &graph, const std::vector<program::Sequence> &progs, const OptionFlags &)
    : graph_(&graph) {
  for (const auto &p : progs) programs_.push_back(p.steps());
  graph.allocateDeviceMemory();
}

void Engine::run(unsigned index) {
  if (index >= programs_.size()) throw poputil::poplibs_error("Engine::run: no such program");
  plb_context *ctx = graph_->context();
  const unsigned long long before = plb_launch_count(ctx);
  detail::check(plb_timer_start(ctx));
  for (const auto &step : programs_[index]) step(ctx);
  float ms = 0.f;
  detail::check(plb_timer_stop(ctx, &ms));
  last_ms_ = ms;
  launches_ = plb_launch_count(ctx) - before;
  detail::check(plb_synchronize(ctx));
}

void Engine::writeTensor(const std::string &handle, const void *begin, const void *end) {
  const auto it = graph_->hostWrites().find(handle);
  if (it == graph_->hostWrites().end())
    throw poputil::poplibs_error("Engine::writeTensor: unknown handle '" + handle + "'");
  const Tensor &t = it->second;
  const std::size_t bytes = t.numElements() * t.elementType().bytes();
  if (end && static_cast<const char *>(end) - static_cast<const char *>(begin) !=
                 static_cast<std::ptrdiff_t>(bytes))
    throw poputil::poplibs_error("Engine::writeTensor: size mismatch for '" + handle + "'");
  plb_context *ctx = graph_->context();
  if (bytes == 0) return;
  if (t.isContiguous()) {
    detail::check(plb_memcpy_h2d(ctx, t.devicePointer(), begin, bytes));
  } else {
    void *staging = nullptr;
    detail::check(plb_malloc(ctx, bytes, &staging));
    detail::check(plb_memcpy_h2d(ctx, staging, begin, bytes));
    copyDenseToView(ctx, staging, t);
    detail::check(plb_free(ctx, staging));
  }
  detail::check(plb_synchronize(ctx));
}

void Engine::readTensor(const std::string &handle, void *begin, void *end) {
  const auto it = graph_->hostReads().find(handle);
  if (it == graph_->hostReads().end())
    throw poputil::poplibs_error("Engine::readTensor: unknown handle '" + handle + "'");
  const Tensor &t = it->second;
  const std::size_t bytes = t.numElements() * t.elementType().bytes();
  if (end && static_cast<char *>(end) - static_cast<char *>(begin) != static_cast<std::ptrdiff_t>(bytes))
    throw poputil::poplibs_error("Engine::readTensor: size mismatch for '" + handle + "'");
  plb_context *ctx = graph_->context();
  if (bytes == 0) return;
  if (t.isContiguous()) {
    detail::check(plb_memcpy_d2h(ctx, begin, t.devicePointer(), bytes));
  } else {
    void *staging = nullptr;
    detail::check(plb_malloc(ctx, bytes, &staging));
    copyViewToDense(ctx, t, staging);
    detail::check(plb_memcpy_d2h(ctx, begin, staging, bytes));
    detail::check(plb_free(ctx, staging));
  }
}

void Engine::printProfileSummary(std::ostream &os, const OptionFlags &) const {
  os << "Execution summary: last program took " << last_ms_ << " ms on the device, " << launches_
     << " kernel launches\n";
}

}  // namespace poplar
