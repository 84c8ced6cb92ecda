// Vectorised sorted search and the relational inner join built on it, for
// sm_100a.
//
// Interface parity (reference): sorted_search
// src/moderngpu/kernel_sortedsearch.hxx:7-62 -- for every needle (sorted) the
// lower or upper bound of its position in the haystack (sorted);
// merge_path_partitions src/moderngpu/search.hxx:12-27; inner_join
// src/moderngpu/kernel_join.hxx:9-48 -- all pairs (i, j) with
// a[i] equivalent to b[j], as int2, ordered by i then j.
//
// These are callers of the load-balancing search: inner_join turns the
// per-needle match counts into segment starts with a scan and lets
// transform_lbs write one pair per output slot.
//
// A tile (cut by the merge-path partition, so that tiles carry equal work
// whatever the key distribution) stages its needles and its haystack range in
// shared memory with coalesced loads; every thread finds its own diagonal and
// merges vt elements serially, noting for each needle it meets how many
// haystack keys came before; the bounds leave through shared memory in
// coalesced stores. (A binary search per needle over the staged haystack
// range, the first version: 0.77 ms for 2^27 + 2^27 int32 keys; this one
// 0.63 ms = 2.5 TB/s. What is left is the unhidden load-merge-store sequence
// of one small tile per CTA; the kernel does not prefetch.)
#pragma once
#include "partition.hxx"
#include "scan.hxx"
#include "load_balance.hxx"

#ifdef __CUDACC__

BEGIN_MGPU_NAMESPACE

template<int nt_, int vt_>
struct search_tuning_t {
  enum { nt = nt_, vt = vt_, nv = nt_ * vt_ };
};

namespace detail {

// 256 x 15 measured best of nine shapes (2^27 + 2^27 int32 keys: 632 us).
typedef search_tuning_t<256, 15> search_default_tuning;

template<typename launch_arg_t>
struct pick_search_tuning { typedef search_default_tuning type; };
template<int nt, int vt>
struct pick_search_tuning<search_tuning_t<nt, vt> > {
  typedef search_tuning_t<nt, vt> type;
};

// partitions[k] = number of `a` keys among the first min(k * spacing, total)
// elements of merge(a, b).
template<bounds_t bounds, typename a_it, typename b_it, typename comp_t>
__global__ void merge_path_partitions_k(a_it a, int a_count, b_it b,
  int b_count, int spacing, int num_partitions, comp_t comp, int* partitions) {
  int k = (int)(blockIdx.x * blockDim.x + threadIdx.x);
  if(k >= num_partitions) return;
  long long diag = (long long)k * spacing;
  long long total = (long long)a_count + b_count;
  if(diag > total) diag = total;
  partitions[k] = merge_path<bounds>(a, a_count, b, b_count, (int)diag, comp);
}

template<bounds_t bounds, typename tuning_t, typename type_t,
  typename needles_it, typename haystack_it, typename indices_it,
  typename comp_t>
__global__ void __launch_bounds__(tuning_t::nt)
sorted_search_k(needles_it needles, int num_needles, haystack_it haystack,
  int num_haystack, indices_it indices, comp_t comp, const int* partitions) {
  enum { nt = tuning_t::nt, vt = tuning_t::vt, nv = tuning_t::nv };
  __shared__ type_t keys[nv];     // the tile's needles, then its haystack keys
  __shared__ int found[nv];       // per needle of the tile

  const int tid = (int)threadIdx.x;
  const int tile = (int)blockIdx.x;
  const long long total = (long long)num_needles + num_haystack;
  const long long d0 = (long long)tile * nv;
  const long long d1 = d0 + nv < total ? d0 + nv : total;
  const int a0 = partitions[tile], a1 = partitions[tile + 1];
  const int b0 = (int)(d0 - a0), b1 = (int)(d1 - a1);
  const int na = a1 - a0, nb = b1 - b0;

  for(int i = tid; i < na; i += nt) keys[i] = needles[a0 + i];
  for(int i = tid; i < nb; i += nt) keys[na + i] = haystack[b0 + i];
  __syncthreads();
  const type_t* ka = keys;
  const type_t* kb = keys + na;

  // Needles go first among equal keys for the lower bound, last for the
  // upper bound: when a needle is merged, the haystack keys merged before it
  // are exactly those its bound counts.
  auto needle_first = [&](const type_t& a, const type_t& b) {
    return (bounds_upper == bounds) ? comp(a, b) : !comp(b, a);
  };

  // This thread merges elements [diag, diag + vt) of the tile: find where
  // they start in each sequence, then walk.
  const int diag = min(tid * vt, na + nb);
  int lo = diag > nb ? diag - nb : 0, hi = diag < na ? diag : na;
  while(lo < hi) {
    int mid = (lo + hi) >> 1;
    if(needle_first(ka[mid], kb[diag - 1 - mid])) lo = mid + 1;
    else hi = mid;
  }
  int ai = lo, bi = diag - lo;
  type_t a_key = ai < na ? ka[ai] : type_t();
  type_t b_key = bi < nb ? kb[bi] : type_t();
  #pragma unroll
  for(int i = 0; i < vt; ++i) {
    if(diag + i < na + nb) {
      bool take_needle = bi >= nb || (ai < na && needle_first(a_key, b_key));
      if(take_needle) {
        found[ai] = b0 + bi;
        ++ai;
        if(ai < na) a_key = ka[ai];
      } else {
        ++bi;
        if(bi < nb) b_key = kb[bi];
      }
    }
  }
  __syncthreads();
  for(int i = tid; i < na; i += nt) indices[a0 + i] = found[i];
}

// Ints of scratch the search needs for its partition table.
template<typename tuning_t = search_default_tuning>
inline size_t sorted_search_partitions(int num_needles, int num_haystack) {
  return (size_t)div_up((int64_t)num_needles + num_haystack,
    (int64_t)tuning_t::nv) + 1;
}

// Partition + search kernel on `stream`; `partitions` holds
// sorted_search_partitions<tuning_t>(...) ints.
template<bounds_t bounds, typename tuning_t, typename needles_it,
  typename haystack_it, typename indices_it, typename comp_t>
void sorted_search_enqueue(needles_it needles, int num_needles,
  haystack_it haystack, int num_haystack, indices_it indices, comp_t comp,
  int* partitions, cudaStream_t stream) {
  typedef typename std::iterator_traits<needles_it>::value_type type_t;
  if(!num_needles) return;
  int num_tiles = (int)div_up((int64_t)num_needles + num_haystack,
    (int64_t)tuning_t::nv);
  int num_partitions = num_tiles + 1;
  merge_path_partitions_k<bounds><<<div_up(num_partitions, 128), 128, 0,
    stream>>>(needles, num_needles, haystack, num_haystack, (int)tuning_t::nv,
    num_partitions, comp, partitions);
  sorted_search_k<bounds, tuning_t, type_t><<<num_tiles, (int)tuning_t::nt, 0,
    stream>>>(needles, num_needles, haystack, num_haystack, indices, comp,
    partitions);
}

} // namespace detail

// The merge-path partition table of two sorted sequences, one entry per
// `spacing` merged elements plus the closing one.
template<bounds_t bounds, typename a_keys_it, typename b_keys_it,
  typename comp_t>
mem_t<int> merge_path_partitions(a_keys_it a, int64_t a_count, b_keys_it b,
  int64_t b_count, int64_t spacing, comp_t comp, context_t& context) {
  int num_partitions = (int)div_up(a_count + b_count, spacing) + 1;
  mem_t<int> partitions(num_partitions, context);
  detail::merge_path_partitions_k<bounds><<<div_up(num_partitions, 128), 128,
    0, context.stream()>>>(a, (int)a_count, b, (int)b_count, (int)spacing,
    num_partitions, comp, partitions.data());
  return partitions;
}

template<bounds_t bounds, typename launch_arg_t = empty_t,
  typename needles_it, typename haystack_it, typename indices_it,
  typename comp_it>
void sorted_search(needles_it needles, int num_needles, haystack_it haystack,
  int num_haystack, indices_it indices, comp_it comp, context_t& context) {
  typedef typename detail::pick_search_tuning<launch_arg_t>::type tuning_t;
  if(num_needles < 0 || num_haystack < 0 ||
    (int64_t)num_needles + num_haystack > (int64_t)0x7fffffff - 65536)
    throw cuda_exception_t(cudaErrorInvalidValue);
  if(!num_needles) return;
  mem_t<int> partitions(detail::sorted_search_partitions<tuning_t>(
    num_needles, num_haystack), context);
  detail::sorted_search_enqueue<bounds, tuning_t>(needles, num_needles,
    haystack, num_haystack, indices, comp, partitions.data(),
    context.stream());
}

// All pairs (a_index, b_index) whose keys are equivalent under `comp`; both
// inputs sorted by `comp`. The size of the result is known only after the
// match counts have been scanned, so the call reads one int back from the
// device (as the reference does) before it allocates the output.
template<typename launch_arg_t = empty_t, typename a_it, typename b_it,
  typename comp_t>
mem_t<int2> inner_join(a_it a, int a_count, b_it b, int b_count, comp_t comp,
  context_t& context) {
  if(a_count <= 0 || b_count <= 0) return mem_t<int2>(0, context);

  mem_t<int> lower(a_count, context);
  mem_t<int> upper(a_count, context);
  sorted_search<bounds_lower, launch_arg_t>(a, a_count, b, b_count,
    lower.data(), comp, context);
  sorted_search<bounds_upper, launch_arg_t>(a, a_count, b, b_count,
    upper.data(), comp, context);

  // Start of every a-key's run of pairs = exclusive scan of its match count.
  mem_t<int> pair_start(a_count, context);
  mem_t<int> pair_count(1, context);
  const int* lower_data = lower.data();
  const int* upper_data = upper.data();
  transform_scan<int>([=]MGPU_DEVICE(int index) {
    return upper_data[index] - lower_data[index];
  }, a_count, pair_start.data(), plus_t<int>(), pair_count.data(), context);
  int join_count = from_mem(pair_count)[0];

  mem_t<int2> output(join_count, context);
  int2* output_data = output.data();
  transform_lbs([=]MGPU_DEVICE(int index, int seg, int rank,
    tuple<int> first_match) {
    output_data[index] = make_int2(seg, get<0>(first_match) + rank);
  }, join_count, pair_start.data(), a_count, make_tuple(lower_data), context);
  return output;
}

END_MGPU_NAMESPACE

#endif // __CUDACC__
