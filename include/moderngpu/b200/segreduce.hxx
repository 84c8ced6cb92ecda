// Entry points of the segmented-reduction family, signature-compatible with
// the reference (src/moderngpu/kernel_segreduce.hxx:193-197 segreduce,
// :272-276 transform_segreduce, :285-290 spmv).
//
// segments[] holds num_segments START offsets (segments[0] == 0,
// non-decreasing, every value <= count); segment s covers
// [segments[s], segments[s+1]) and the last one ends at count. An empty
// segment yields `init`; a non-empty one yields the left-to-right fold of its
// items, `init` not included. count + num_segments must be below 2^31.
//
// Temporaries (one block: partition table and tile-status words) come from
// context.alloc and are handed back with context.free before returning; all
// work is enqueued on context.stream() and nothing waits for the device.
#pragma once
#include "segreduce_kernel.hxx"

#ifdef __CUDACC__

BEGIN_MGPU_NAMESPACE

namespace detail {

// A caller may pass segreduce_tuning_t<...> in the launch_arg_t slot to pick
// the tile shape; launch boxes written for other architectures are accepted
// and replaced by the Blackwell default.
template<typename launch_arg_t, typename type_t,
  typename default_t = typename segreduce_default_tuning<type_t>::type>
struct pick_segreduce_tuning {
  typedef default_t type;
};
template<int nt, int vt, int stages, int occ, typename type_t,
  typename default_t>
struct pick_segreduce_tuning<segreduce_tuning_t<nt, vt, stages, occ>, type_t,
  default_t> {
  typedef segreduce_tuning_t<nt, vt, stages, occ> type;
};

inline void check_merged_size(int count, int num_segments) {
  if(count < 0 || num_segments < 0 ||
    (int64_t)count + num_segments > (int64_t)0x7fffffff - 65536)
    throw cuda_exception_t(cudaErrorInvalidValue);
}

} // namespace detail

template<typename launch_arg_t = empty_t, typename input_it,
  typename segments_it, typename output_it, typename op_t, typename type_t>
void segreduce(input_it input, int count, segments_it segments,
  int num_segments, output_it output, op_t op, type_t init,
  context_t& context) {

  typedef typename detail::pick_segreduce_tuning<launch_arg_t, type_t>::type
    tuning_t;
  typedef typename detail::source_for<input_it, type_t>::type source_t;

  detail::throw_on_device_status();
  detail::check_merged_size(count, num_segments);
  detail::segreduce_plan_t<tuning_t, type_t> plan(count, num_segments);
  if(!plan.num_tiles) return;

  mem_t<char> workspace(plan.bytes, context);
  detail::segreduce_enqueue<tuning_t>(source_t { input }, count, segments,
    num_segments, output, op, init, workspace.data(), context.stream());
}

// Reduce f(index) for index in [0, count) by segment.
template<typename launch_arg_t = empty_t, typename func_t,
  typename segments_it, typename output_it, typename op_t, typename type_t>
void transform_segreduce(func_t f, int count, segments_it segments,
  int num_segments, output_it output, op_t op, type_t init,
  context_t& context) {
  segreduce<launch_arg_t>(make_load_iterator<type_t>(f), count, segments,
    num_segments, output, op, init, context);
}

// y = A * x for a CSR matrix: `matrix` and `columns` hold the count non-zeros
// row after row, segments[] the first non-zero of each of num_segments rows.
template<typename launch_arg_t = empty_t, typename matrix_it,
  typename columns_it, typename vector_it, typename segments_it,
  typename output_it>
void spmv(matrix_it matrix, columns_it columns, vector_it vector, int count,
  segments_it segments, int num_segments, output_it output,
  context_t& context) {
  typedef typename std::iterator_traits<matrix_it>::value_type type_t;
  typedef typename std::iterator_traits<columns_it>::value_type col_t;
  typedef typename std::iterator_traits<vector_it>::value_type vec_t;
  constexpr bool arrays = std::is_pointer<matrix_it>::value &&
    std::is_pointer<columns_it>::value && std::is_pointer<vector_it>::value &&
    std::is_floating_point<type_t>::value &&
    std::is_same<typename std::remove_cv<vec_t>::type, type_t>::value &&
    std::is_same<typename std::remove_cv<col_t>::type, int>::value &&
    std::is_same<launch_arg_t, empty_t>::value;
  if constexpr (arrays) {
    detail::throw_on_device_status();
    // Plain CSR arrays: matrix values and column indices are staged by bulk
    // copies, x is gathered through the read-only path.
    typedef typename detail::spmv_default_tuning<type_t>::type tuning_t;
    detail::check_merged_size(count, num_segments);
    detail::segreduce_plan_t<tuning_t, type_t> plan(count, num_segments);
    if(!plan.num_tiles) return;
    mem_t<char> workspace(plan.bytes, context);
    detail::spmv_source_t<type_t> source { matrix, columns, vector };
    detail::segreduce_enqueue<tuning_t>(source, count, segments, num_segments,
      output, plus_t<type_t>(), (type_t)0, workspace.data(), context.stream());
    return;
  }
  transform_segreduce<launch_arg_t>([=]MGPU_DEVICE(int index) {
    return matrix[index] * ldg(vector + columns[index]);
  }, count, segments, num_segments, output, plus_t<type_t>(), (type_t)0,
    context);
}

END_MGPU_NAMESPACE

#endif // __CUDACC__
