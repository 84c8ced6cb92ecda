// Merge-path partitioner for load-balancing search.
//
// Items 0..count-1 are merged with the segment start offsets; a segment start
// sorts before the item with the same index. partition[k] is the number of
// ITEMS among the first min(k * spacing, count + num_segments) merged
// elements, which cuts the merged sequence into tiles of `spacing` elements
// no matter how items and segment starts are distributed.
//
// Interface parity (reference): merge_path src/moderngpu/cta_merge.hxx:8-29,
// load_balance_partitions src/moderngpu/search.hxx:29-37 (via
// merge_path_partitions<bounds_upper> :12-27). Results are bit-identical.
//
// The reference runs one thread per diagonal with a binary search of
// ~log2(count) dependent global loads. Here one warp owns a diagonal and
// probes 32 pivots per round, so a diagonal resolves in ~log33 rounds of
// independent loads; the kernel can also clear the per-tile status words the
// segmented-reduction kernel needs, saving a memset launch.
#pragma once
#include "runtime.hxx"

BEGIN_MGPU_NAMESPACE

// Serial merge path, host or device. Returns how many keys of `a` lie among
// the first `diag` elements of merge(a, b).
template<bounds_t bounds = bounds_lower, typename a_keys_it,
  typename b_keys_it, typename int_t, typename comp_t>
MGPU_HOST_DEVICE int_t merge_path(a_keys_it a_keys, int_t a_count,
  b_keys_it b_keys, int_t b_count, int_t diag, comp_t comp) {
  int_t lo = diag > b_count ? diag - b_count : (int_t)0;
  int_t hi = diag < a_count ? diag : a_count;
  while(lo < hi) {
    int_t mid = lo + (hi - lo) / 2;
    auto a_key = a_keys[mid];
    auto b_key = b_keys[diag - 1 - mid];
    bool take_a = (bounds_upper == bounds) ? comp(a_key, b_key) :
      !comp(b_key, a_key);
    if(take_a) lo = mid + 1;
    else hi = mid;
  }
  return lo;
}

#ifdef __CUDACC__

namespace detail {

// Items among the first `diag` merged elements, found by one warp.
// The predicate "item mid sorts before segment start diag-1-mid", i.e.
// mid < segments[diag-1-mid], is true for a prefix of mid values; the answer
// is the length of that prefix within [lo, hi).
template<typename segments_it>
MGPU_DEVICE int warp_lbs_diagonal(segments_it segments, int count,
  int num_segments, int64_t diag, int lane) {
  int64_t lo = diag > num_segments ? diag - num_segments : 0;
  int64_t hi = diag < count ? diag : count;
  const unsigned full = 0xffffffffu;
  while(hi - lo > 32) {
    int64_t width = hi - lo;
    int64_t stride = (width + 32) / 33;
    int64_t mid = lo + (int64_t)(lane + 1) * stride - 1;
    bool before = false;
    if(mid < hi) before = mid < (int64_t)segments[diag - 1 - mid];
    unsigned votes = __ballot_sync(full, before);
    int taken = __popc(votes);            // probes 0..taken-1 are true
    int64_t new_lo = lo + (int64_t)taken * stride;
    int64_t probe_next = lo + (int64_t)(taken + 1) * stride - 1;
    if(taken < 32 && probe_next < hi) hi = probe_next;
    lo = new_lo < hi ? new_lo : hi;
  }
  int64_t mid = lo + lane;
  bool before = false;
  if(mid < hi) before = mid < (int64_t)segments[diag - 1 - mid];
  unsigned votes = __ballot_sync(full, before);
  return (int)(lo + __popc(votes));
}

template<int nt, typename segments_it, typename int_t>
__global__ void __launch_bounds__(nt)
lbs_partition_k(segments_it segments, int count, int num_segments,
  int64_t spacing, int num_partitions, int_t* partitions,
  uint32_t* clear_head, int clear_head_words,
  uint32_t* clear_tiles, int words_per_tile) {

  int lane = (int)(threadIdx.x & 31);
  int k = (int)((blockIdx.x * (unsigned)nt + threadIdx.x) >> 5);
  if(k >= num_partitions) return;

  int64_t total = (int64_t)count + num_segments;
  int64_t diag = spacing * k;
  if(diag > total) diag = total;
  int mp = warp_lbs_diagonal(segments, count, num_segments, diag, lane);
  if(!lane) partitions[k] = (int_t)mp;

  // Optional: reset the consumer kernel's header and tile k's status words.
  if(clear_tiles && k + 1 < num_partitions)
    for(int i = lane; i < words_per_tile; i += 32)
      clear_tiles[(size_t)k * words_per_tile + i] = 0;
  if(clear_head && 0 == k)
    for(int i = lane; i < clear_head_words; i += 32) clear_head[i] = 0;
}

// Enqueue the partition kernel. `partitions` holds num_partitions entries.
template<typename segments_it, typename int_t>
void launch_lbs_partition(segments_it segments, int count, int num_segments,
  int64_t spacing, int num_partitions, int_t* partitions, cudaStream_t stream,
  uint32_t* clear_head = nullptr, int clear_head_words = 0,
  uint32_t* clear_tiles = nullptr, int words_per_tile = 0) {
  enum { nt = 256, warps = nt / 32 };
  int num_ctas = div_up(num_partitions, (int)warps);
  if(num_ctas > 0)
    lbs_partition_k<nt><<<num_ctas, nt, 0, stream>>>(segments, count,
      num_segments, spacing, num_partitions, partitions, clear_head,
      clear_head_words, clear_tiles, words_per_tile);
}

} // namespace detail

// Public partitioner with the reference's signature. Returns
// div_up(dest_count + num_segments, spacing) + 1 entries.
template<typename segments_it>
auto load_balance_partitions(int64_t dest_count, segments_it segments,
  int num_segments, int spacing, context_t& context) ->
  mem_t<typename std::iterator_traits<segments_it>::value_type> {
  typedef typename std::iterator_traits<segments_it>::value_type int_t;
  int num_partitions =
    (int)div_up(dest_count + num_segments, (int64_t)spacing) + 1;
  mem_t<int_t> mem(num_partitions, context);
  detail::launch_lbs_partition(segments, (int)dest_count, num_segments,
    (int64_t)spacing, num_partitions, mem.data(), context.stream());
  return mem;
}

#endif // __CUDACC__

END_MGPU_NAMESPACE
