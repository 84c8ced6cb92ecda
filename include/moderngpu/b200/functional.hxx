// Binary functors, the read-only load helper and the iterator adaptors that
// appear in the signatures of segreduce / transform_lbs and their callers
// (reference: src/moderngpu/operators.hxx:34-124 functors and ldg,
// :129-343 iterators).
#pragma once
#include "base.hxx"

BEGIN_MGPU_NAMESPACE

////////////////////////////////////////////////////////////////////////////////
// ldg(p): read through the read-only path when p is a raw pointer to an
// arithmetic type, plain dereference otherwise.

namespace detail {
template<typename it_t>
struct is_arith_pointer {
  typedef typename std::iterator_traits<it_t>::value_type value_t;
  enum { value = std::is_pointer<it_t>::value &&
    std::is_arithmetic<value_t>::value };
};
} // namespace detail

template<typename it_t>
MGPU_HOST_DEVICE typename std::iterator_traits<it_t>::value_type ldg(it_t it) {
#ifdef __CUDA_ARCH__
  if constexpr (detail::is_arith_pointer<it_t>::value) return __ldg(it);
  else return *it;
#else
  return *it;
#endif
}

template<typename real_t>
MGPU_HOST_DEVICE real_t sq(real_t x) { return x * x; }

template<typename type_t>
MGPU_HOST_DEVICE void swap(type_t& a, type_t& b) {
  type_t t = a; a = b; b = t;
}

////////////////////////////////////////////////////////////////////////////////
// Comparison and arithmetic functors.

#define MGPU_B200_BINARY_FUNCTOR(name, result_t, expr)                        \
  template<typename type_t>                                                   \
  struct name {                                                               \
    MGPU_HOST_DEVICE result_t operator()(type_t a, type_t b) const {          \
      return expr;                                                            \
    }                                                                         \
  };

MGPU_B200_BINARY_FUNCTOR(less_t,          bool,   a < b)
MGPU_B200_BINARY_FUNCTOR(less_equal_t,    bool,   a <= b)
MGPU_B200_BINARY_FUNCTOR(greater_t,       bool,   a > b)
MGPU_B200_BINARY_FUNCTOR(greater_equal_t, bool,   a >= b)
MGPU_B200_BINARY_FUNCTOR(equal_to_t,      bool,   a == b)
MGPU_B200_BINARY_FUNCTOR(not_equal_to_t,  bool,   a != b)
MGPU_B200_BINARY_FUNCTOR(plus_t,          type_t, a + b)
MGPU_B200_BINARY_FUNCTOR(minus_t,         type_t, a - b)
MGPU_B200_BINARY_FUNCTOR(multiplies_t,    type_t, a * b)
MGPU_B200_BINARY_FUNCTOR(maximum_t,       type_t, max(a, b))
MGPU_B200_BINARY_FUNCTOR(minimum_t,       type_t, min(a, b))

#undef MGPU_B200_BINARY_FUNCTOR

////////////////////////////////////////////////////////////////////////////////
// Index-generating iterators. Each models "operator[](i) -> value" plus
// iterator +/- so kernels may rebase them, and publishes value_type through
// std::iterator_traits.

template<typename derived_t, typename value_t, typename int_t = int>
struct generator_iterator_t {
  typedef value_t value_type;
  typedef int_t difference_type;
  typedef const value_t* pointer;
  typedef const value_t& reference;
  typedef std::random_access_iterator_tag iterator_category;

  int_t index;

  generator_iterator_t() = default;
  MGPU_HOST_DEVICE explicit generator_iterator_t(int_t i) : index(i) { }

  MGPU_HOST_DEVICE value_t operator[](int_t i) const {
    return static_cast<const derived_t&>(*this)(index + i);
  }
  MGPU_HOST_DEVICE value_t operator*() const { return (*this)[0]; }

  MGPU_HOST_DEVICE derived_t operator+(int_t d) const {
    derived_t r = static_cast<const derived_t&>(*this);
    r.index += d;
    return r;
  }
  MGPU_HOST_DEVICE derived_t operator-(int_t d) const {
    derived_t r = static_cast<const derived_t&>(*this);
    r.index -= d;
    return r;
  }
  MGPU_HOST_DEVICE derived_t& operator+=(int_t d) {
    index += d;
    return static_cast<derived_t&>(*this);
  }
  MGPU_HOST_DEVICE derived_t& operator-=(int_t d) {
    index -= d;
    return static_cast<derived_t&>(*this);
  }
};

// counting_iterator_t<T>(k)[i] == T(k + i).
template<typename type_t, typename int_t = int>
struct counting_iterator_t :
  generator_iterator_t<counting_iterator_t<type_t, int_t>, type_t, int_t> {
  typedef generator_iterator_t<counting_iterator_t, type_t, int_t> base_t;
  counting_iterator_t() = default;
  MGPU_HOST_DEVICE counting_iterator_t(type_t first) : base_t((int_t)first) { }
  MGPU_HOST_DEVICE type_t operator()(int_t i) const { return (type_t)i; }
};

// strided_iterator_t<T>(offset, stride)[i] == offset + i * stride.
template<typename type_t, typename int_t = int>
struct strided_iterator_t :
  generator_iterator_t<strided_iterator_t<type_t, int_t>, type_t, int_t> {
  typedef generator_iterator_t<strided_iterator_t, type_t, int_t> base_t;
  type_t offset, stride;
  strided_iterator_t() = default;
  MGPU_HOST_DEVICE strided_iterator_t(type_t offset_, type_t stride_) :
    base_t(0), offset(offset_), stride(stride_) { }
  MGPU_HOST_DEVICE type_t operator()(int_t i) const {
    return offset + (type_t)i * stride;
  }
};

// constant_iterator_t<T>(v)[i] == v.
template<typename type_t>
struct constant_iterator_t :
  generator_iterator_t<constant_iterator_t<type_t>, type_t, int> {
  typedef generator_iterator_t<constant_iterator_t, type_t, int> base_t;
  type_t value;
  MGPU_HOST_DEVICE constant_iterator_t(type_t v) : base_t(0), value(v) { }
  MGPU_HOST_DEVICE type_t operator()(int) const { return value; }
};

// Output iterator that drops what is stored to it.
template<typename value_t>
struct discard_iterator_t {
  typedef value_t value_type;
  typedef int difference_type;
  typedef const value_t* pointer;
  typedef const value_t& reference;
  typedef std::random_access_iterator_tag iterator_category;

  struct sink_t {
    MGPU_HOST_DEVICE value_t operator=(value_t) { return value_t(); }
  };
  MGPU_HOST_DEVICE sink_t operator[](int) const { return sink_t(); }
  MGPU_HOST_DEVICE sink_t operator*() const { return sink_t(); }
  MGPU_HOST_DEVICE discard_iterator_t operator+(int) const { return *this; }
  MGPU_HOST_DEVICE discard_iterator_t operator-(int) const { return *this; }
};

#ifdef __CUDACC__

////////////////////////////////////////////////////////////////////////////////
// lambda_iterator_t wraps a device lambda as a load and/or store iterator:
//   make_load_iterator<T>([=]MGPU_DEVICE(int i) { return ...; })
//   make_store_iterator<T>([=]MGPU_DEVICE(T v, int i) { ... })

template<typename load_t, typename store_t, typename value_t, typename int_t>
struct lambda_iterator_t {
  typedef value_t value_type;
  typedef int_t difference_type;
  typedef const value_t* pointer;
  typedef const value_t& reference;
  typedef std::random_access_iterator_tag iterator_category;

  load_t load;
  store_t store;
  int_t base;

  lambda_iterator_t(load_t l, store_t s, int_t b) :
    load(l), store(s), base(b) { }

  // Proxy: converts to value_t by calling load, assigns by calling store.
  struct proxy_t {
    load_t load;
    store_t store;
    int_t index;

    MGPU_LAMBDA proxy_t& operator=(value_t rhs) {
      static_assert(!std::is_same<store_t, empty_t>::value,
        "this lambda iterator has no store function");
      store(rhs, index);
      return *this;
    }
    MGPU_LAMBDA operator value_t() const {
      static_assert(!std::is_same<load_t, empty_t>::value,
        "this lambda iterator has no load function");
      return load(index);
    }
  };

  MGPU_LAMBDA proxy_t operator[](int_t i) const {
    return proxy_t { load, store, base + i };
  }
  MGPU_LAMBDA proxy_t operator*() const {
    return proxy_t { load, store, base };
  }
  MGPU_HOST_DEVICE lambda_iterator_t operator+(int_t d) const {
    lambda_iterator_t r = *this; r.base += d; return r;
  }
  MGPU_HOST_DEVICE lambda_iterator_t operator-(int_t d) const {
    lambda_iterator_t r = *this; r.base -= d; return r;
  }
  MGPU_HOST_DEVICE lambda_iterator_t& operator+=(int_t d) {
    base += d; return *this;
  }
  MGPU_HOST_DEVICE lambda_iterator_t& operator-=(int_t d) {
    base -= d; return *this;
  }
};

template<typename value_t, typename int_t = int, typename load_t,
  typename store_t>
lambda_iterator_t<load_t, store_t, value_t, int_t>
make_load_store_iterator(load_t load, store_t store, int_t base = 0) {
  return lambda_iterator_t<load_t, store_t, value_t, int_t>(load, store, base);
}

template<typename value_t, typename int_t = int, typename load_t>
lambda_iterator_t<load_t, empty_t, value_t, int_t>
make_load_iterator(load_t load, int_t base = 0) {
  return lambda_iterator_t<load_t, empty_t, value_t, int_t>(load, empty_t(),
    base);
}

template<typename value_t, typename int_t = int, typename store_t>
lambda_iterator_t<empty_t, store_t, value_t, int_t>
make_store_iterator(store_t store, int_t base = 0) {
  return lambda_iterator_t<empty_t, store_t, value_t, int_t>(empty_t(), store,
    base);
}

#endif // __CUDACC__

END_MGPU_NAMESPACE
