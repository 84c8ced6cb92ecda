// Foundation of the B200 build of the moderngpu segmented-reduction path:
// qualifier macros, small integer helpers, value types shared by every header.
//
// The names below are the ones user code written against moderngpu 2.x sees
// (reference: src/moderngpu/meta.hxx:13-30,87-98,140-172 and
// src/moderngpu/types.hxx:9-138). Only what the load-balanced
// segmented-reduction path and its callers need is provided.
#pragma once

#include <cstdint>
#include <cstddef>
#include <cstdio>
#include <cstring>
#include <cassert>
#include <cfloat>
#include <exception>
#include <iterator>
#include <type_traits>
#include <utility>
#include <cuda_runtime.h>

#ifdef __CUDACC__
  #ifndef MGPU_HOST_DEVICE
    #define MGPU_HOST_DEVICE __forceinline__ __host__ __device__
  #endif
  #ifndef MGPU_DEVICE
    #define MGPU_DEVICE __device__
  #endif
  #ifndef MGPU_LAMBDA
    #define MGPU_LAMBDA __device__
  #endif
#else
  #ifndef MGPU_HOST_DEVICE
    #define MGPU_HOST_DEVICE inline
  #endif
#endif

#define BEGIN_MGPU_NAMESPACE namespace mgpu {
#define END_MGPU_NAMESPACE }

#define MGPU_ALIGN(x) __attribute__((aligned(x)))

BEGIN_MGPU_NAMESPACE

enum { warp_size = 32 };

// Tag meaning "argument not supplied"; also the default of the leading
// launch_arg_t template slot of every entry point.
struct empty_t { };

template<bool cond, typename type_t = void>
using enable_if_t = typename std::enable_if<cond, type_t>::type;

// conditional_typedef_t<a, b>::type_t is a unless a is empty_t.
template<typename first_t, typename second_t>
struct conditional_typedef_t {
  typedef typename std::conditional<std::is_same<first_t, empty_t>::value,
    second_t, first_t>::type type_t;
};

MGPU_HOST_DEVICE constexpr bool is_pow2(int x) { return (x & (x - 1)) == 0; }

MGPU_HOST_DEVICE constexpr int div_up(int num, int den) {
  return (num + den - 1) / den;
}
MGPU_HOST_DEVICE constexpr int64_t div_up(int64_t num, int64_t den) {
  return (num + den - 1) / den;
}
MGPU_HOST_DEVICE constexpr size_t div_up(size_t num, size_t den) {
  return (num + den - 1) / den;
}

// Unqualified min/max inside namespace mgpu resolve here (user functors such
// as maximum_t call max(a, b) on arbitrary arithmetic types).
template<typename real_t>
MGPU_HOST_DEVICE constexpr real_t min(real_t a, real_t b) {
  return b < a ? b : a;
}
template<typename real_t>
MGPU_HOST_DEVICE constexpr real_t max(real_t a, real_t b) {
  return a < b ? b : a;
}

template<typename... args_t>
MGPU_HOST_DEVICE void swallow(args_t...) { }

// Compile-time unrolled loop: f(0), f(1), ... f(count - 1).
namespace detail {
template<int i, int end>
struct unroll_t {
  template<typename func_t>
  MGPU_HOST_DEVICE static void run(func_t& f) {
    f(i);
    unroll_t<i + 1, end>::run(f);
  }
};
template<int end>
struct unroll_t<end, end> {
  template<typename func_t>
  MGPU_HOST_DEVICE static void run(func_t&) { }
};
} // namespace detail

template<int begin, int end, typename func_t>
MGPU_HOST_DEVICE void iterate(func_t f) {
  detail::unroll_t<begin, (end > begin ? end : begin)>::run(f);
}
template<int count, typename func_t>
MGPU_HOST_DEVICE void iterate(func_t f) {
  iterate<0, count>(f);
}

// Errors surface as C++ exceptions carrying the CUDA status
// (reference: src/moderngpu/types.hxx:9-16).
struct cuda_exception_t : std::exception {
  cudaError_t result;
  explicit cuda_exception_t(cudaError_t status) : result(status) { }
  const char* what() const noexcept override {
    return cudaGetErrorString(result);
  }
};

// Raised when a kernel of this library reported a device-side status other
// than success: a bounded wait ran out (status 1: a look-back, 2: a staged
// copy), so the outputs of that call are incomplete. It is a
// cuda_exception_t (cudaErrorLaunchTimeout), which is what callers of the
// reference already catch.
struct status_exception_t : cuda_exception_t {
  int status;
  explicit status_exception_t(int s) :
    cuda_exception_t(cudaErrorLaunchTimeout), status(s) { }
  const char* what() const noexcept override {
    return "mgpu: a kernel's bounded wait ran out (device-side status)";
  }
};

template<typename type_t, int size>
struct array_t {
  type_t data[size];
  MGPU_HOST_DEVICE type_t operator[](int i) const { return data[i]; }
  MGPU_HOST_DEVICE type_t& operator[](int i) { return data[i]; }
};

enum bounds_t { bounds_lower, bounds_upper };

struct MGPU_ALIGN(8) range_t {
  int begin, end;
  MGPU_HOST_DEVICE int size() const { return end - begin; }
  MGPU_HOST_DEVICE int count() const { return end - begin; }
  MGPU_HOST_DEVICE bool valid() const { return begin < end; }
};

MGPU_HOST_DEVICE range_t get_tile(int cta, int nv, int count) {
  int lo = nv * cta;
  int hi = lo + nv;
  return range_t { lo, hi < count ? hi : count };
}

// One tile of a merge of items (a) with segment starts (b).
struct MGPU_ALIGN(16) merge_range_t {
  int a_begin, a_end, b_begin, b_end;
  MGPU_HOST_DEVICE int a_count() const { return a_end - a_begin; }
  MGPU_HOST_DEVICE int b_count() const { return b_end - b_begin; }
  MGPU_HOST_DEVICE int total() const { return a_count() + b_count(); }
  MGPU_HOST_DEVICE range_t a_range() const { return range_t { a_begin, a_end }; }
  MGPU_HOST_DEVICE range_t b_range() const { return range_t { b_begin, b_end }; }
  MGPU_HOST_DEVICE bool a_valid() const { return a_begin < a_end; }
  MGPU_HOST_DEVICE bool b_valid() const { return b_begin < b_end; }
};

// Tile k of a merge cut every `spacing` merged elements, given the item
// counts mp0/mp1 on its two bounding diagonals
// (reference: src/moderngpu/cta_merge.hxx:52-59).
MGPU_HOST_DEVICE merge_range_t compute_merge_range(int a_count, int b_count,
  int partition, int spacing, int mp0, int mp1) {
  int d0 = spacing * partition;
  int d1 = d0 + spacing;
  if(d1 > a_count + b_count) d1 = a_count + b_count;
  return merge_range_t { mp0, mp1, d0 - mp0, d1 - mp1 };
}

END_MGPU_NAMESPACE
