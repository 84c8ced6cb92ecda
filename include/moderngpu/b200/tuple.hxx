// mgpu::tuple and the helpers that transform_lbs / lbs_segreduce functors see.
//
// The reference carries its own device-capable tuple
// (src/moderngpu/tuple.hxx:226-300) because CUDA had none in 2016. The CUDA
// toolkit now ships one (libcu++), so mgpu::tuple is an alias of it; functor
// parameters spelled `tuple<int, float> desc` and calls `get<0>(desc)` compile
// unchanged. The per-segment cached load (reference:
// src/moderngpu/cpp11.hxx:6-59) is restated on top of it.
#pragma once
#include "base.hxx"
#include <cuda/std/tuple>
#include <cuda/std/utility>

BEGIN_MGPU_NAMESPACE

using ::cuda::std::tuple;
using ::cuda::std::get;
using ::cuda::std::make_tuple;
using ::cuda::std::forward_as_tuple;
using ::cuda::std::tie;
using ::cuda::std::tuple_size;
using ::cuda::std::tuple_element;
using ::cuda::std::index_sequence;
using ::cuda::std::make_index_sequence;
using ::cuda::std::integer_sequence;

// tuple<it0, it1, ...> -> tuple<value_type of it0, value_type of it1, ...>
template<typename tpl_t>
struct tuple_iterator_value;

template<typename... its_t>
struct tuple_iterator_value<tuple<its_t...> > {
  typedef tuple<typename std::iterator_traits<its_t>::value_type...> type;
};

template<typename tpl_t>
using tuple_iterator_value_t = typename tuple_iterator_value<tpl_t>::type;

namespace detail {
template<typename int_t, typename... its_t, size_t... idx>
MGPU_HOST_DEVICE tuple_iterator_value_t<tuple<its_t...> >
gather_tuple(const tuple<its_t...>& its, int_t index, index_sequence<idx...>) {
  typedef tuple_iterator_value_t<tuple<its_t...> > value_t;
  return value_t(get<idx>(its)[index]...);
}

template<typename int_t, typename... its_t, size_t... idx>
MGPU_HOST_DEVICE void scatter_tuple(const tuple<its_t...>& its,
  const tuple_iterator_value_t<tuple<its_t...> >& values, int_t index,
  index_sequence<idx...>) {
  swallow((get<idx>(its)[index] = get<idx>(values))...);
}
} // namespace detail

// load(tuple_of_iterators, i) reads element i through every iterator.
template<typename int_t, typename... its_t>
MGPU_HOST_DEVICE tuple_iterator_value_t<tuple<its_t...> >
load(tuple<its_t...> its, int_t index) {
  return detail::gather_tuple(its, index,
    make_index_sequence<sizeof...(its_t)>());
}

// store(tuple_of_iterators, values, i) writes element i through every iterator.
template<typename int_t, typename... its_t>
MGPU_HOST_DEVICE void store(tuple<its_t...> its,
  tuple_iterator_value_t<tuple<its_t...> > values, int_t index) {
  detail::scatter_tuple(its, values, index,
    make_index_sequence<sizeof...(its_t)>());
}

END_MGPU_NAMESPACE
