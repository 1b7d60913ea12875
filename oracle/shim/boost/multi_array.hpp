// Stand-in for the small part of Boost.MultiArray that the reference's CPU
// models (lib/poplibs_test/Convolution.cpp, GeneralMatrixMultiply.cpp) use.
// TEST INFRASTRUCTURE ONLY: it exists so that those two reference sources can
// be compiled, unmodified and from where they lie, into the checker library.
// Row-major ("C") storage order only, zero index bases only.
#ifndef ORACLE_SHIM_BOOST_MULTI_ARRAY_HPP
#define ORACLE_SHIM_BOOST_MULTI_ARRAY_HPP

#include <algorithm>
#include <array>
#include <cassert>
#include <cmath>  // (the real header brings it in; the reference's models rely on that)
#include <cstddef>
#include <numeric>
#include <type_traits>
#include <vector>

namespace boost {

namespace detail_ma {

// extents[a][b][c] builder.
template <std::size_t N> struct extent_gen {
  std::array<std::size_t, N> ext{};
  extent_gen<N + 1> operator[](std::size_t e) const {
    extent_gen<N + 1> r;
    for (std::size_t i = 0; i != N; ++i)
      r.ext[i] = ext[i];
    r.ext[N] = e;
    return r;
  }
};

// A view of the trailing N dimensions starting at some element.
template <class T, std::size_t N> class sub_array {
public:
  using element = typename std::remove_const<T>::type;
  sub_array(T *base, const std::size_t *shape, const std::size_t *strides)
      : base_(base), shape_(shape), strides_(strides) {}
  sub_array<T, N - 1> operator[](std::size_t i) const {
    assert(i < shape_[0]);
    return sub_array<T, N - 1>(base_ + i * strides_[0], shape_ + 1,
                               strides_ + 1);
  }
  const std::size_t *shape() const { return shape_; }
  std::size_t size() const { return shape_[0]; }

private:
  T *base_;
  const std::size_t *shape_;
  const std::size_t *strides_;
};

template <class T> class sub_array<T, 1> {
public:
  sub_array(T *base, const std::size_t *shape, const std::size_t *strides)
      : base_(base), shape_(shape), strides_(strides) {}
  T &operator[](std::size_t i) const {
    assert(i < shape_[0]);
    return base_[i * strides_[0]];
  }
  // The innermost dimension is contiguous (stride 1) in row-major storage.
  T *begin() const { return base_; }
  T *end() const { return base_ + shape_[0]; }
  const std::size_t *shape() const { return shape_; }
  std::size_t size() const { return shape_[0]; }

private:
  T *base_;
  const std::size_t *shape_;
  const std::size_t *strides_;
};

template <class T, std::size_t N> struct indexer {
  using type = sub_array<T, N - 1>;
  static type get(T *base, const std::size_t *shape,
                  const std::size_t *strides, std::size_t i) {
    assert(i < shape[0]);
    return type(base + i * strides[0], shape + 1, strides + 1);
  }
};
template <class T> struct indexer<T, 1> {
  using type = T &;
  static type get(T *base, const std::size_t *shape,
                  const std::size_t *strides, std::size_t i) {
    assert(i < shape[0]);
    return base[i * strides[0]];
  }
};

} // namespace detail_ma

static const detail_ma::extent_gen<0> extents{};

template <class T, std::size_t N> class const_multi_array_ref {
public:
  using element = T;
  using size_type = std::size_t;
  const_multi_array_ref(const T *data, const detail_ma::extent_gen<N> &e)
      : data_(const_cast<T *>(data)) {
    set_shape(e.ext);
  }
  const size_type *shape() const { return shape_.data(); }
  size_type num_elements() const { return num_elements_; }
  size_type size() const { return shape_[0]; }
  static constexpr size_type num_dimensions() { return N; }
  const T *data() const { return data_; }
  const T *origin() const { return data_; }
  typename detail_ma::indexer<const T, N>::type
  operator[](std::size_t i) const {
    return detail_ma::indexer<const T, N>::get(data_, shape_.data(),
                                               strides_.data(), i);
  }

protected:
  const_multi_array_ref() : data_(nullptr) {}
  void set_shape(const std::array<std::size_t, N> &s) {
    shape_ = s;
    std::size_t stride = 1;
    for (std::size_t i = N; i > 0; --i) {
      strides_[i - 1] = stride;
      stride *= shape_[i - 1];
    }
    num_elements_ = stride;
  }
  T *data_;
  std::array<std::size_t, N> shape_{};
  std::array<std::size_t, N> strides_{};
  std::size_t num_elements_ = 0;
};

template <class T, std::size_t N>
class multi_array_ref : public const_multi_array_ref<T, N> {
  using base = const_multi_array_ref<T, N>;

public:
  multi_array_ref(T *data, const detail_ma::extent_gen<N> &e)
      : base(data, e) {}
  multi_array_ref(const multi_array_ref &) = default;
  // Assignment copies elements (shapes must match), as in Boost.
  multi_array_ref &operator=(const multi_array_ref &o) {
    copy_from(o);
    return *this;
  }
  template <class Other> multi_array_ref &operator=(const Other &o) {
    copy_from(o);
    return *this;
  }
  using base::data;
  using base::origin;
  using base::operator[];
  T *data() const { return this->data_; }
  T *origin() const { return this->data_; }
  typename detail_ma::indexer<T, N>::type operator[](std::size_t i) const {
    return detail_ma::indexer<T, N>::get(this->data_, this->shape_.data(),
                                         this->strides_.data(), i);
  }

protected:
  multi_array_ref() = default;
  template <class Other> void copy_from(const Other &o) {
    assert(o.num_elements() == this->num_elements_);
    for (std::size_t i = 0; i != N; ++i)
      assert(o.shape()[i] == this->shape_[i]);
    if (static_cast<const void *>(o.data()) !=
        static_cast<const void *>(this->data_))
      std::copy(o.data(), o.data() + o.num_elements(), this->data_);
  }
};

template <class T, std::size_t N>
class multi_array : public multi_array_ref<T, N> {
  using base = multi_array_ref<T, N>;

public:
  multi_array() { rebind(); }
  explicit multi_array(const detail_ma::extent_gen<N> &e) {
    this->set_shape(e.ext);
    storage_.assign(this->num_elements_, T());
    rebind();
  }
  multi_array(const multi_array &o) : base() {
    this->set_shape(o.shape_);
    storage_ = o.storage_;
    rebind();
  }
  multi_array(multi_array &&o) noexcept : base() {
    this->set_shape(o.shape_);
    storage_ = std::move(o.storage_);
    rebind();
  }
  multi_array(const const_multi_array_ref<T, N> &o) : base() {
    std::array<std::size_t, N> s;
    for (std::size_t i = 0; i != N; ++i)
      s[i] = o.shape()[i];
    this->set_shape(s);
    storage_.assign(o.data(), o.data() + o.num_elements());
    rebind();
  }
  multi_array &operator=(const multi_array &o) {
    if (this != &o) {
      // Boost requires equal shapes here; the reference only assigns
      // same-shaped arrays, so a plain element copy (with resize for a
      // default-constructed target) is enough.
      this->set_shape(o.shape_);
      storage_ = o.storage_;
      rebind();
    }
    return *this;
  }
  multi_array &operator=(multi_array &&o) noexcept {
    this->set_shape(o.shape_);
    storage_ = std::move(o.storage_);
    rebind();
    return *this;
  }
  void resize(const detail_ma::extent_gen<N> &e) {
    this->set_shape(e.ext);
    storage_.assign(this->num_elements_, T());
    rebind();
  }

private:
  void rebind() { this->data_ = storage_.data(); }
  std::vector<T> storage_;
};

} // namespace boost

#endif // ORACLE_SHIM_BOOST_MULTI_ARRAY_HPP
