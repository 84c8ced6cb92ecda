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
// 0.63 ms, 0.55 ms in the streaming variant below, which prefetches, and
// 0.48 ms = 3.3 TB/s once the merge walk was written without branches.)
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

// 256 x 15: 2^27 + 2^27 int32 keys in 483 us with the streaming kernel
// (256 x 23: 467 us, but its tiles of 8-byte keys no longer fit the 48 KB of
// static shared memory of the one-CTA-per-tile kernel).
typedef search_tuning_t<256, 15> search_default_tuning;

// 4-byte keys take the larger tile (47 KB of static shared memory in the
// one-CTA-per-tile kernel, just under its limit). Scratch is always sized for
// the default, smaller tile, which needs the longer partition table.
template<typename type_t, int size = (int)sizeof(type_t)>
struct search_tuning_for { typedef search_default_tuning type; };
template<typename type_t>
struct search_tuning_for<type_t, 4> { typedef search_tuning_t<256, 23> type; };

template<typename launch_arg_t, typename type_t>
struct pick_search_tuning {
  typedef typename search_tuning_for<type_t>::type type;
};
template<int nt, int vt, typename type_t>
struct pick_search_tuning<search_tuning_t<nt, vt>, type_t> {
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

// One thread's share of a tile's merge: vt steps from (ai, diag - ai). The
// walk is written without branches -- which side is taken only selects
// addresses and values -- because the threads of a warp take different sides
// at every step (with branches a third of the issue slots went to divergence
// and the kernel was bound by instruction issue). Both key runs live in one
// shared array, so the one reload per step is a single load from a selected
// address; a load one element past a run reads a neighbour or padding and is
// never used.
template<int vt, typename type_t, typename first_t>
MGPU_DEVICE void serial_search_merge(const type_t* ka, int na,
  const type_t* kb, int nb, int ai, int diag, int b0, int* found,
  first_t needle_first) {
  int bi = diag - ai;
  int steps = na + nb - diag;
  type_t a_key = ka[ai < na ? ai : 0];
  type_t b_key = kb[bi < nb ? bi : 0];
  #pragma unroll
  for(int i = 0; i < vt; ++i) {
    bool active = i < steps;
    bool take_needle = bi >= nb || (ai < na && needle_first(a_key, b_key));
    if(active && take_needle) found[ai] = b0 + bi;
    ai += active && take_needle;
    bi += active && !take_needle;
    const type_t* next = take_needle ? ka + ai : kb + bi;
    type_t key = *next;
    a_key = take_needle ? key : a_key;
    b_key = take_needle ? b_key : key;
  }
}

template<bounds_t bounds, typename tuning_t, typename type_t,
  typename needles_it, typename haystack_it, typename indices_it,
  typename comp_t>
__global__ void __launch_bounds__(tuning_t::nt)
sorted_search_k(needles_it needles, int num_needles, haystack_it haystack,
  int num_haystack, indices_it indices, comp_t comp, const int* partitions) {
  enum { nt = tuning_t::nt, vt = tuning_t::vt, nv = tuning_t::nv };
  __shared__ type_t keys[nv + 1]; // the tile's needles, then its haystack
                                  // keys, and one slot the merge may read past
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
  serial_search_merge<vt>(ka, na, kb, nb, lo, diag, b0, found, needle_first);
  __syncthreads();
  for(int i = tid; i < na; i += nt) indices[a0 + i] = found[i];
}

////////////////////////////////////////////////////////////////////////////////
// Streaming variant for 4- and 8-byte arithmetic keys behind 16-byte aligned
// raw pointers. The kernel above loads, merges and stores one small tile per
// CTA in sequence, so most of a CTA's life is spent waiting for its loads.
// Here a persistent CTA walks its tiles while one producer lane stages the
// needle and haystack windows of the tiles ahead with bulk asynchronous
// copies; the consumers only ever wait for shared memory.

struct search_window_t {
  int a0, a1, b0, b1;          // needles [a0, a1), haystack keys [b0, b1)
  int a_slot, b_slot;          // shared-memory element index of a0 and of b0
  int a_bulk, b_bulk;          // first needle / key index NOT delivered by
                               // the bulk copies (the ragged end of an array)
};

template<typename tuning_t, int stages, typename type_t>
struct search_stream_smem_t {
  enum { nv = tuning_t::nv, per16 = 16 / (int)sizeof(type_t),
    key_slots = nv + 4 * per16 };
  alignas(128) type_t keys[stages][key_slots];
  int found[2][nv];
  search_window_t window[stages];
  uint64_t full[stages], empty[stages];
};

template<bounds_t bounds, typename tuning_t, int stages, typename type_t,
  typename indices_it, typename comp_t>
__global__ void __launch_bounds__(tuning_t::nt + 32)
sorted_search_stream_k(const type_t* needles, int num_needles,
  const type_t* haystack, int num_haystack, indices_it indices, comp_t comp,
  const int* partitions, int num_tiles, uint64_t timeout_ns,
  uint32_t* status) {
  enum { nt = tuning_t::nt, vt = tuning_t::vt, nv = tuning_t::nv,
    warps = nt / 32, per16 = 16 / (int)sizeof(type_t) };
  typedef search_stream_smem_t<tuning_t, stages, type_t> smem_t;
  extern __shared__ __align__(128) char search_raw[];
  smem_t& shared = *reinterpret_cast<smem_t*>(search_raw);

  const int tid = (int)threadIdx.x;
  if(0 == tid) {
    for(int s = 0; s < stages; ++s) {
      ptx::mbar_init(&shared.full[s], 1);
      ptx::mbar_init(&shared.empty[s], nt);
    }
    ptx::fence_proxy_async();
  }
  __syncthreads();

  const int first_tile = (int)blockIdx.x, step = (int)gridDim.x;
  const int my_tiles = first_tile < num_tiles ?
    (num_tiles - first_tile + step - 1) / step : 0;
  const long long total = (long long)num_needles + num_haystack;

  if(tid >= nt) {
    //////////////////////////////////////////////////////////////////////////
    // Producer lane.
    if(tid > nt || !my_tiles) return;
    // Window of array elements [x0, x1): the whole 16-byte granules inside
    // the array that cover it. c_lo: first element copied; bytes: size of the
    // copy (0: none); bulk_end: first index the copy does not deliver.
    auto plan_window = [&](int n, int x0, int x1, int& c_lo, uint32_t& bytes,
      int& bulk_end) {
      c_lo = x0 / per16 * per16;
      int c_hi = (x1 + per16 - 1) / per16 * per16;
      int inner = n / per16 * per16;
      if(c_hi > inner) c_hi = inner;
      bytes = 0;
      bulk_end = x0;
      if(x1 > x0 && c_hi > c_lo) {
        bytes = (uint32_t)(c_hi - c_lo) * (uint32_t)sizeof(type_t);
        bulk_end = c_hi < x1 ? c_hi : x1;
      }
    };
    int p0 = partitions[first_tile], p1 = partitions[first_tile + 1];
    for(int k = 0; k < my_tiles; ++k) {
      const int tile = first_tile + k * step;
      const int s = k % stages;
      int q0 = 0, q1 = 0;
      if(k + 1 < my_tiles) {
        q0 = partitions[tile + step];
        q1 = partitions[tile + step + 1];
      }
      if(k >= stages &&
        !ptx::mbar_wait(&shared.empty[s], ((k / stages) - 1) & 1, timeout_ns)) {
        // The stage was never released: give up and say so.
        raise_status(status, (uint32_t)status_copy_timeout);
        return;
      }
      const long long d0 = (long long)tile * nv;
      const long long d1 = d0 + nv < total ? d0 + nv : total;
      search_window_t w;
      w.a0 = p0; w.a1 = p1;
      w.b0 = (int)(d0 - p0); w.b1 = (int)(d1 - p1);
      int a_lo, b_lo;
      uint32_t a_bytes, b_bytes;
      plan_window(num_needles, w.a0, w.a1, a_lo, a_bytes, w.a_bulk);
      plan_window(num_haystack, w.b0, w.b1, b_lo, b_bytes, w.b_bulk);
      type_t* a_dst = shared.keys[s];
      // The haystack window follows the needles' slots, on a 16-byte line.
      int a_span = (w.a0 - a_lo) + (w.a1 - w.a0);
      type_t* b_dst = a_dst + (a_span + per16 - 1) / per16 * per16;
      w.a_slot = w.a0 - a_lo;
      w.b_slot = (int)(b_dst - a_dst) + (w.b0 - b_lo);
      // The consumers read the descriptor after the barrier: write it first.
      shared.window[s] = w;
      ptx::fence_proxy_async();
      if(a_bytes + b_bytes) {
        ptx::mbar_arrive_expect_tx(&shared.full[s], a_bytes + b_bytes);
        if(a_bytes)
          ptx::bulk_load(a_dst, needles + a_lo, a_bytes, &shared.full[s]);
        if(b_bytes)
          ptx::bulk_load(b_dst, haystack + b_lo, b_bytes, &shared.full[s]);
      } else
        ptx::mbar_arrive(&shared.full[s]);
      p0 = q0; p1 = q1;
    }
    return;
  }

  ////////////////////////////////////////////////////////////////////////////
  // Consumers.
  auto needle_first = [&](const type_t& a, const type_t& b) {
    return (bounds_upper == bounds) ? comp(a, b) : !comp(b, a);
  };
  for(int k = 0; k < my_tiles; ++k) {
    const int s = k % stages;
    bool arrived = ptx::mbar_wait(&shared.full[s], (k / stages) & 1, timeout_ns);
    const search_window_t w = shared.window[s];
    type_t* ka = shared.keys[s] + w.a_slot;
    type_t* kb = shared.keys[s] + w.b_slot;
    const int na = w.a1 - w.a0, nb = w.b1 - w.b0;
    // The ragged ends of the arrays (at most per16 - 1 elements each) come
    // by plain loads.
    for(int i = w.a_bulk - w.a0 + tid; i < na; i += nt) ka[i] = needles[w.a0 + i];
    for(int i = w.b_bulk - w.b0 + tid; i < nb; i += nt) kb[i] = haystack[w.b0 + i];
    if(!ptx::named_all<1, nt>(arrived)) {
      // A staged copy did not complete in time: the remaining bounds stay
      // unwritten and the status word tells the host.
      if(0 == tid) raise_status(status, (uint32_t)status_copy_timeout);
      return;
    }

    int* found = shared.found[k & 1];
    const int diag = min(tid * vt, na + nb);
    int lo = diag > nb ? diag - nb : 0, hi = diag < na ? diag : na;
    while(lo < hi) {
      int mid = (lo + hi) >> 1;
      if(needle_first(ka[mid], kb[diag - 1 - mid])) lo = mid + 1;
      else hi = mid;
    }
    serial_search_merge<vt>(ka, na, kb, nb, lo, diag, w.b0, found,
      needle_first);
    // The keys are no longer needed: the producer may refill the stage while
    // the bounds are being written out.
    ptx::mbar_arrive(&shared.empty[s]);
    ptx::named_sync<1, nt>();
    for(int i = tid; i < na; i += nt) indices[w.a0 + i] = found[i];
  }
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
  int* partitions, cudaStream_t stream,
  uint64_t timeout_ns = 2000000000ull, uint32_t* status = nullptr) {
  typedef typename std::iterator_traits<needles_it>::value_type type_t;
  if(!num_needles) return;
  int num_tiles = (int)div_up((int64_t)num_needles + num_haystack,
    (int64_t)tuning_t::nv);
  int num_partitions = num_tiles + 1;
  merge_path_partitions_k<bounds><<<div_up(num_partitions, 128), 128, 0,
    stream>>>(needles, num_needles, haystack, num_haystack, (int)tuning_t::nv,
    num_partitions, comp, partitions);
  constexpr bool streamable =
    std::is_pointer<needles_it>::value && std::is_pointer<haystack_it>::value &&
    std::is_arithmetic<type_t>::value &&
    (4 == sizeof(type_t) || 8 == sizeof(type_t)) &&
    std::is_same<typename std::remove_cv<typename std::remove_pointer<
      haystack_it>::type>::type, type_t>::value;
  if constexpr (streamable) {
    if(0 == ((uintptr_t)needles | (uintptr_t)haystack) % 16) {
      enum { stages = 2 };
      typedef search_stream_smem_t<tuning_t, stages, type_t> smem_t;
      auto kernel = sorted_search_stream_k<bounds, tuning_t, stages, type_t,
        indices_it, comp_t>;
      const int threads = (int)tuning_t::nt + 32;
      const int smem = (int)sizeof(smem_t);
      static int resident[64] = { };
      int device = 0;
      throw_on_error(cudaGetDevice(&device));
      int grid = device < 64 ? resident[device] : 0;
      if(!grid) {
        throw_on_error(cudaFuncSetAttribute(kernel,
          cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        int per_sm = 0, sms = 0;
        throw_on_error(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm,
          kernel, threads, smem));
        throw_on_error(cudaDeviceGetAttribute(&sms,
          cudaDevAttrMultiProcessorCount, device));
        grid = per_sm * sms > 0 ? per_sm * sms : 1;
        if(device < 64) resident[device] = grid;
      }
      if(grid > num_tiles) grid = num_tiles;
      kernel<<<grid, threads, smem, stream>>>((const type_t*)needles,
        num_needles, (const type_t*)haystack, num_haystack, indices, comp,
        partitions, num_tiles, timeout_ns, status);
      return;
    }
  }
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
  typedef typename std::iterator_traits<needles_it>::value_type key_t;
  typedef typename detail::pick_search_tuning<launch_arg_t, key_t>::type
    tuning_t;
  detail::throw_on_device_status();
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
