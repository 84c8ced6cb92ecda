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
// The reference runs one thread per diagonal, each doing a binary search of
// ~log2(count) dependent, uncoalesced global loads. Here the search is turned
// inside out. Segment start j sits at merged position key[j] = segments[j] + j
// (segments[j] items and j starts precede it), and key[] is strictly
// increasing, so the number of starts before diagonal d is the number of keys
// below d. One coalesced, 128-bit-vectorised pass over segments[] finds, for
// each j, the diagonals that fall between key[j-1] and key[j] and writes
// their entries; every diagonal is written exactly once. The same pass can
// clear the per-tile status words the segmented-reduction kernel needs, which
// saves a memset launch.
#pragma once
#include "runtime.hxx"
#include "ptx.hxx"

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

template<typename segments_it>
struct is_int_array {
  typedef typename std::iterator_traits<segments_it>::value_type value_t;
  enum { value = std::is_pointer<segments_it>::value &&
    std::is_same<typename std::remove_cv<value_t>::type, int>::value };
};

// Each thread owns `per_thread` consecutive segment indices j (128-bit loads
// when segments[] is an aligned int array) and walks their keys in order,
// keeping `bound`, the merged position of the first diagonal not yet written.
// A key below `bound` (the common case: one compare) crosses no diagonal.
// Otherwise the diagonals k with bound <= k * spacing <= key[j] have exactly
// j starts before them. The virtual index j == num_segments closes the array
// and takes every remaining diagonal. Short runs of diagonals are written by
// the thread itself; a long run (one segment spanning many tiles) is handed
// to the whole warp at the end so it does not serialise on one thread.
// A partitioner launch can carry a few extra CTAs that do unrelated work which
// must precede the dependent kernel anyway (the multi-GPU layer posts a
// shard's boundary record this way instead of in a launch of its own):
// the grid's first tail_t::ctas CTAs run tail(k), k = 0 .. ctas - 1, with the
// partitioner's nt threads (first, so that they are done long before the
// partitioner's last CTA).
struct no_partition_tail_t {
  enum { ctas = 0 };
  MGPU_DEVICE void operator()(int) const { }
};

template<int nt, int per_thread, typename segments_it, typename int_t,
  typename tail_t>
__global__ void __launch_bounds__(nt)
lbs_partition_k(segments_it segments, int count, int num_segments,
  uint32_t step, int num_partitions, int_t* partitions,
  uint32_t* clear_head, int clear_head_words,
  uint32_t* clear_tiles, int words_per_tile, int tile_stride, tail_t tail) {

  // Let a dependent kernel (the reduction) set itself up meanwhile.
  ptx::grid_launch_dependents();
  if constexpr (tail_t::ctas > 0) {
    if((int)blockIdx.x < (int)tail_t::ctas) {
      tail((int)blockIdx.x);
      return;
    }
  }
  const int cta = (int)blockIdx.x - (int)tail_t::ctas;
  const unsigned full = 0xffffffffu;
  const int lane = (int)(threadIdx.x & 31);
  const uint32_t total = (uint32_t)count + (uint32_t)num_segments;
  const int64_t j0 = ((int64_t)cta * nt + threadIdx.x) * per_thread;
  const uint32_t last = (uint32_t)(num_partitions - 1);

  if(clear_head && 0 == cta)
    for(int i = (int)threadIdx.x; i < clear_head_words; i += nt)
      clear_head[i] = 0;

  auto write_entry = [&](uint32_t k, uint32_t starts) {
    uint64_t diag = (uint64_t)k * step;
    if(diag > total) diag = total;
    partitions[k] = (int_t)((uint32_t)diag - starts);
    if(clear_tiles && k < last)
      for(int w = 0; w < words_per_tile; ++w)
        clear_tiles[(size_t)k * tile_stride + w] = 0;
  };

  // Pending long run of this thread: diagonals [run_lo, run_hi], all with
  // `run_starts` segment starts before them.
  uint32_t run_lo = 1, run_hi = 0, run_starts = 0;

  if(j0 <= num_segments) {
    int offs[per_thread];
    bool vector_ok = false;
    if constexpr (is_int_array<segments_it>::value)
      vector_ok = 0 == ((uintptr_t)segments & 15) &&
        j0 + per_thread <= num_segments;
    if(vector_ok) {
      if constexpr (is_int_array<segments_it>::value) {
        #pragma unroll
        for(int q = 0; q < per_thread / 4; ++q) {
          int4 v = *reinterpret_cast<const int4*>(segments + j0 + 4 * q);
          offs[4 * q] = v.x; offs[4 * q + 1] = v.y;
          offs[4 * q + 2] = v.z; offs[4 * q + 3] = v.w;
        }
      }
    } else {
      #pragma unroll
      for(int i = 0; i < per_thread; ++i)
        offs[i] = (j0 + i < num_segments) ? (int)segments[j0 + i] : 0;
    }

    uint32_t k_next = 0;
    if(j0 > 0)
      k_next = ((uint32_t)segments[j0 - 1] + (uint32_t)(j0 - 1)) / step + 1;
    uint64_t bound = (uint64_t)k_next * step;

    // Keys increase with j, so the indices that reach `bound` form a suffix.
    // Count the ones below it with straight-line code; the rest of the work
    // happens in a compact loop that most threads never enter.
    auto key_of = [&](uint32_t j, int off) -> uint32_t {
      // Indices past the virtual closing start never cross anything.
      return j < (uint32_t)num_segments ? (uint32_t)off + j :
        (j == (uint32_t)num_segments ? 0xffffffffu : 0u);
    };
    int below = 0;
    #pragma unroll
    for(int i = 0; i < per_thread; ++i) {
      uint32_t j = (uint32_t)j0 + i;
      below += (j <= (uint32_t)num_segments && key_of(j, offs[i]) < bound) ?
        1 : 0;
    }
    const uint32_t key_last = key_of((uint32_t)j0 + per_thread - 1,
      offs[per_thread - 1]);

    for(int i = below; i < per_thread; ++i) {
      uint32_t j = (uint32_t)j0 + i;
      if(j > (uint32_t)num_segments) break;
      uint32_t key = key_of(j, j < (uint32_t)num_segments ?
        (int)segments[j] : 0);
      if(key >= bound) {
        uint32_t k_hi = k_next;
        if(j == (uint32_t)num_segments) k_hi = last;
        else if(key - bound >= step) k_hi = key / step;
        if(k_hi > last) k_hi = last;
        if(k_hi - k_next >= 16) {
          // Keep one long run for the warp; flush an older one serially.
          for(uint32_t k = run_lo; k <= run_hi && run_lo <= run_hi; ++k)
            write_entry(k, run_starts);
          run_lo = k_next; run_hi = k_hi; run_starts = j;
        } else {
          for(uint32_t k = k_next; k <= k_hi; ++k) write_entry(k, j);
        }
        k_next = k_hi + 1;
        bound = (uint64_t)k_next * step;
      }
      if(key_last < bound && (uint32_t)j0 + per_thread - 1 <
        (uint32_t)num_segments) break;
    }
  }

  unsigned busy = __ballot_sync(full, run_lo <= run_hi);
  while(busy) {
    int src = __ffs(busy) - 1;
    busy &= busy - 1;
    uint32_t lo = __shfl_sync(full, run_lo, src);
    uint32_t hi = __shfl_sync(full, run_hi, src);
    uint32_t starts = __shfl_sync(full, run_starts, src);
    for(uint64_t k = (uint64_t)lo + lane; k <= hi; k += 32)
      write_entry((uint32_t)k, starts);
  }
}

// Enqueue the partition kernel. `partitions` holds num_partitions entries.
enum { lbs_partition_threads = 128 };

template<typename segments_it, typename int_t,
  typename tail_t = no_partition_tail_t>
void launch_lbs_partition(segments_it segments, int count, int num_segments,
  int64_t spacing, int num_partitions, int_t* partitions, cudaStream_t stream,
  uint32_t* clear_head = nullptr, int clear_head_words = 0,
  uint32_t* clear_tiles = nullptr, int words_per_tile = 0,
  int tile_stride = 0, tail_t tail = tail_t()) {
  enum { nt = lbs_partition_threads, per_thread = 16 };
  // One more index than there are segments: the virtual closing start.
  int num_ctas = (int)div_up((int64_t)num_segments + 1,
    (int64_t)(nt * per_thread));
  uint32_t step = (uint32_t)(spacing < 0x7fffffff ? spacing : 0x7fffffff);
  if(num_partitions > 0)
    lbs_partition_k<nt, per_thread><<<num_ctas + (int)tail_t::ctas, nt, 0,
      stream>>>(segments, count, num_segments, step, num_partitions,
      partitions, clear_head, clear_head_words, clear_tiles, words_per_tile,
      tile_stride ? tile_stride : words_per_tile, tail);
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
