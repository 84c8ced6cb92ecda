// lbs_segreduce: segmented reduction of f(index, seg, rank, cached...) —
// signature-compatible with the reference
// (src/moderngpu/kernel_segreduce.hxx:303-308 and the overload without
// cached iterators :390-395). Empty segments yield `init`.
//
// As in the reference, the load-balancing search is fused into the reduction
// kernel: the consumers of a tile work out the segment and rank of every item
// in shared memory, evaluate the functor in striped order (so that its loads
// from index-addressed arrays coalesce) and fold the values in place.
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
  typedef typename detail::pick_segreduce_tuning<launch_arg_t, type_t,
    typename detail::lbs_segreduce_default_tuning<type_t>::type>::type
    tuning_t;
  typedef detail::lbs_source_t<func_t, pointers_t, type_t, args_t...>
    source_t;
  detail::throw_on_device_status();
  detail::check_merged_size(count, num_segments);
  detail::segreduce_plan_t<tuning_t, type_t> plan(count, num_segments);
  if(!plan.num_tiles) return;
  mem_t<char> workspace(plan.bytes, context);
  source_t source { f, caching_iterators, tuple<args_t...>(args...) };
  detail::segreduce_enqueue<tuning_t>(source, count, segments, num_segments,
    output, op, init, workspace.data(), context.stream());
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
