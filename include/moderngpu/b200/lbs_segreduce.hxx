// lbs_segreduce: segmented reduction of f(index, seg, rank, cached...) —
// signature-compatible with the reference
// (src/moderngpu/kernel_segreduce.hxx:303-308 and the overload without
// cached iterators :390-395). Empty segments yield `init`.
//
// The reference fuses the load-balancing search into its reduction tile
// kernel. Here the functor is evaluated by transform_lbs into a temporary
// array of count values (from context.alloc), which the single-pass
// segmented reduction then folds; results are identical, at the cost of one
// extra write and read of the values.
#pragma once
#include "segreduce.hxx"
#include "load_balance.hxx"

#ifdef __CUDACC__

BEGIN_MGPU_NAMESPACE

template<typename launch_arg_t = empty_t, typename func_t,
  typename segments_it, typename pointers_t, typename output_it,
  typename op_t, typename type_t, typename... args_t>
void lbs_segreduce(func_t f, int count, segments_it segments,
  int num_segments, pointers_t caching_iterators, output_it output, op_t op,
  type_t init, context_t& context, args_t... args) {
  typedef tuple_iterator_value_t<pointers_t> value_t;
  mem_t<type_t> values(count, context);
  type_t* values_data = values.data();
  transform_lbs<launch_arg_t>(
    [=]MGPU_DEVICE(int index, int seg, int rank, value_t cached,
      args_t... rest) {
      values_data[index] = f(index, seg, rank, cached, rest...);
    }, count, segments, num_segments, caching_iterators, context, args...);
  segreduce<launch_arg_t>((const type_t*)values_data, count, segments,
    num_segments, output, op, init, context);
}

template<typename launch_arg_t = empty_t, typename func_t,
  typename segments_it, typename output_it, typename op_t, typename type_t,
  typename... args_t>
void lbs_segreduce(func_t f, int count, segments_it segments,
  int num_segments, output_it output, op_t op, type_t init,
  context_t& context, args_t... args) {
  lbs_segreduce<launch_arg_t>(
    [=]MGPU_DEVICE(int index, int seg, int rank, tuple<>, args_t... rest) {
      return f(index, seg, rank, rest...);
    }, count, segments, num_segments, tuple<>(), output, op, init, context,
    args...);
}

END_MGPU_NAMESPACE

#endif // __CUDACC__
