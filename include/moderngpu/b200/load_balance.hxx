// Load-balancing search for sm_100a: transform_lbs, load_balance_search and
// the interval_* family built on it.
//
// Interface parity (reference): transform_lbs
// src/moderngpu/kernel_load_balance.hxx:8-76, load_balance_search :78-86,
// interval_expand / gather / scatter / move
// src/moderngpu/kernel_intervalmove.hxx:7-65. The functor is called exactly
// once per item index in [0, count) as
//   f(index, seg, rank, tuple_of_cached_values, args...)
// with seg = (number of segment starts <= index) - 1 and
// rank = index - segments[seg]; the order of calls is unspecified.
//
// The reference materialises (seg, rank) with a per-thread merge-path search
// and a serial merge over shared memory (src/moderngpu/cta_load_balance.hxx:
// 107-184). Here a tile (cut by the same merge-path partition) stages its
// segment starts in shared memory with one bulk asynchronous copy, scatters
// one head bit and one segment id per NON-EMPTY segment, and turns them into
// per-item segment ids with a register-blocked running maximum plus a
// warp-shuffle max-scan; items are then visited in striped order so that the
// functor's loads and stores to index-addressed arrays coalesce.
#pragma once
#include "partition.hxx"
#include "ptx.hxx"
#include "tile_state.hxx"

#ifdef __CUDACC__

BEGIN_MGPU_NAMESPACE

// Tile shape of the load-balancing kernels: nt threads x vt items each.
template<int nt_, int vt_, int occ_ = 0>
struct lbs_tuning_t {
  enum { nt = nt_, vt = vt_, occ = occ_, nv = nt_ * vt_ };
  static_assert(nt_ % 32 == 0 && vt_ % 4 == 0 && vt_ <= 32, "unsupported tile");
};

namespace detail {

// 256 x 20: the int4 stores of a thread's 20 ids are bank-conflict free
// (20 = 4 mod 8) and five 41 KB CTAs fit on an SM; measured best on B200.
typedef lbs_tuning_t<256, 20, 4> lbs_default_tuning;

template<typename launch_arg_t>
struct pick_lbs_tuning { typedef lbs_default_tuning type; };
template<int nt, int vt, int occ>
struct pick_lbs_tuning<lbs_tuning_t<nt, vt, occ> > {
  typedef lbs_tuning_t<nt, vt, occ> type;
};

template<typename tuning_t>
struct lbs_smem_t {
  enum { nt = tuning_t::nt, vt = tuning_t::vt, nv = tuning_t::nv,
    warps = nt / 32, flag_words = nv / 32 + 1 };
  alignas(16) int seg_of[nv];        // head segment ids, then per-item ids
  alignas(16) int offs[nv + 12];     // staged segment starts
  uint32_t flags[flag_words];
  int warp_max[warps];
  uint64_t bar;
};

// Computes, for the tile `tile`, the segment of every item into
// shared.seg_of[] (indexed by item - a0) and leaves the tile's segment starts
// in shared.offs[] (indexed by seg - ob). Returns the tile geometry.
struct lbs_tile_t {
  int a0, a1, b0, b1;   // items [a0, a1), segment starts [b0, b1)
  int ob, oe;           // segment indices staged in shared.offs
};

template<typename tuning_t, typename segments_it>
MGPU_DEVICE lbs_tile_t lbs_tile_segments(int tile, int count,
  segments_it segments, int num_segments, const int* partitions,
  lbs_smem_t<tuning_t>& shared, uint64_t timeout_ns, uint32_t* status) {

  enum { nt = tuning_t::nt, vt = tuning_t::vt, nv = tuning_t::nv,
    warps = nt / 32, flag_words = lbs_smem_t<tuning_t>::flag_words,
    seg_bulk = is_int_array<segments_it>::value };
  const int tid = (int)threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const unsigned full = 0xffffffffu;

  lbs_tile_t t;
  const int64_t total = (int64_t)count + num_segments;
  int64_t d0 = (int64_t)tile * nv;
  int64_t d1 = d0 + nv < total ? d0 + nv : total;
  t.a0 = partitions[tile];
  t.a1 = partitions[tile + 1];
  t.a0 = t.a0 < 0 ? 0 : (t.a0 > count ? count : t.a0);
  t.a1 = t.a1 < t.a0 ? t.a0 : (t.a1 > count ? count : t.a1);
  if(t.a1 - t.a0 > nv) t.a1 = t.a0 + nv;
  int64_t b0 = d0 - t.a0, b1 = d1 - t.a1;
  b0 = b0 < 0 ? 0 : (b0 > num_segments ? num_segments : b0);
  b1 = b1 < b0 ? b0 : (b1 > num_segments ? num_segments : b1);
  if(b1 - b0 > nv) b1 = b0 + nv;
  t.b0 = (int)b0;
  t.b1 = (int)b1;
  const int na = t.a1 - t.a0;

  // Stage segment starts [b0 - 1, b1): whole 16-byte granules by bulk copy
  // when segments[] is an int array, element loads otherwise.
  const int jlo = t.b0 > 0 ? t.b0 - 1 : 0;
  const int jhi = t.b1;
  if constexpr (seg_bulk) {
    const int* seg = segments;
    int mis = (int)(((uintptr_t)seg / 4) % 4);
    int64_t inner_lo = mis ? 4 : 0;
    int64_t inner_hi = ((int64_t)num_segments + mis) / 4 * 4;
    int64_t c_lo = ((int64_t)jlo + mis) / 4 * 4;
    if(c_lo < inner_lo) c_lo = inner_lo;
    int64_t c_hi = ((int64_t)jhi + mis + 3) / 4 * 4;
    if(c_hi > inner_hi) c_hi = inner_hi;
    t.ob = t.oe = 0;
    if(jhi > jlo && c_hi > c_lo) {
      t.ob = (int)(c_lo - mis);
      t.oe = (int)(c_hi - mis);
    }
    if(0 == tid) {
      ptx::mbar_init(&shared.bar, 1);
      ptx::fence_proxy_async();
      if(t.oe > t.ob) {
        uint32_t bytes = (uint32_t)(t.oe - t.ob) * 4;
        ptx::mbar_arrive_expect_tx(&shared.bar, bytes);
        ptx::bulk_load(shared.offs, seg + t.ob, bytes, &shared.bar);
      } else {
        ptx::mbar_arrive(&shared.bar);
      }
    }
  } else {
    t.ob = jlo;
    t.oe = jhi;
    for(int j = jlo + tid; j < jhi; j += nt)
      shared.offs[j - jlo] = (int)segments[j];
  }
  for(int i = tid; i < flag_words; i += nt) shared.flags[i] = 0;
  __syncthreads();
  if constexpr (seg_bulk) {
    if(!ptx::mbar_wait(&shared.bar, 0, timeout_ns) && status)
      atomicMax(status, (uint32_t)status_copy_timeout);
  }

  const int ob = t.ob, oe = t.oe;
  auto seg_start = [&](int j) -> int {
    if(j >= num_segments) return count;
    if(j >= ob && j < oe) return shared.offs[j - ob];
    return (int)segments[j];
  };

  // One head bit and one id per distinct start inside the tile; among equal
  // starts the last segment owns the items.
  for(int j = t.b0 + tid; j < t.b1; j += nt) {
    int p = seg_start(j);
    bool owner = j + 1 >= t.b1 || seg_start(j + 1) != p;
    int w = p - t.a0;
    if(owner && w >= 0 && w < na) {
      shared.seg_of[w] = j;
      atomicOr(&shared.flags[w >> 5], 1u << (w & 31));
    }
  }
  __syncthreads();

  // Running maximum of head ids: within the thread, then across the CTA.
  const int w0 = tid * vt;
  uint32_t bits = __funnelshift_r(shared.flags[w0 >> 5],
    (w0 >> 5) + 1 < flag_words ? shared.flags[(w0 >> 5) + 1] : 0u, w0 & 31);
  if(vt < 32) bits &= (1u << vt) - 1;
  int mine = -1;
  if(bits) mine = shared.seg_of[w0 + 31 - __clz(bits)];
  int incl = mine;
  #pragma unroll
  for(int delta = 1; delta < 32; delta *= 2) {
    int y = __shfl_up_sync(full, incl, delta);
    if(lane >= delta) incl = max(incl, y);
  }
  int before = __shfl_up_sync(full, incl, 1);
  if(0 == lane) before = -1;
  if(31 == lane) shared.warp_max[warp] = incl;
  __syncthreads();
  int cur = t.b0 - 1;
  for(int k = 0; k < warp; ++k) cur = max(cur, shared.warp_max[k]);
  cur = max(cur, before);

  if(w0 < na) {
    int ids[vt];
    #pragma unroll
    for(int i = 0; i < vt; ++i) {
      if((bits >> i) & 1) cur = shared.seg_of[w0 + i];
      ids[i] = cur;
    }
    #pragma unroll
    for(int i = 0; i < vt; i += 4)
      *reinterpret_cast<int4*>(&shared.seg_of[w0 + i]) =
        make_int4(ids[i], ids[i + 1], ids[i + 2], ids[i + 3]);
  }
  __syncthreads();
  return t;
}

template<typename tuning_t, typename func_t, typename segments_it,
  typename pointers_t, typename... args_t>
__global__ void __launch_bounds__(tuning_t::nt, tuning_t::occ)
transform_lbs_k(func_t f, int count, segments_it segments, int num_segments,
  const int* partitions, pointers_t caching_iterators, uint64_t timeout_ns,
  uint32_t* status, args_t... args) {

  enum { nt = tuning_t::nt, vt = tuning_t::vt };
  extern __shared__ __align__(128) char lbs_smem_raw[];
  lbs_smem_t<tuning_t>& shared =
    *reinterpret_cast<lbs_smem_t<tuning_t>*>(lbs_smem_raw);

  lbs_tile_t t = lbs_tile_segments<tuning_t>((int)blockIdx.x, count, segments,
    num_segments, partitions, shared, timeout_ns, status);
  const int tid = (int)threadIdx.x;
  const int na = t.a1 - t.a0;
  const int ob = t.ob, oe = t.oe;

  // Usual case: every segment start the tile refers to is staged and no item
  // precedes the first segment, so the per-item work is two shared loads.
  const bool simple = t.b0 > 0 && (t.b0 - 1) >= ob && t.b1 <= oe;
  if(simple) {
    const int* offs_by_seg = shared.offs - ob;
    const int full_rounds = na / nt;        // rounds in which no thread idles
    #pragma unroll
    for(int i = 0; i < vt; ++i) {
      if(i < full_rounds) {
        int w = i * nt + tid;
        int seg = shared.seg_of[w];
        int index = t.a0 + w;
        f(index, seg, index - offs_by_seg[seg],
          mgpu::load(caching_iterators, seg), args...);
      }
    }
    int w = full_rounds * nt + tid;
    if(w < na) {
      int seg = shared.seg_of[w];
      int index = t.a0 + w;
      f(index, seg, index - offs_by_seg[seg],
        mgpu::load(caching_iterators, seg), args...);
    }
    return;
  }

  #pragma unroll
  for(int i = 0; i < vt; ++i) {
    int w = i * nt + tid;
    if(w < na) {
      int seg = shared.seg_of[w];
      if(seg >= 0) {
        int index = t.a0 + w;
        int start = (seg >= ob && seg < oe) ? shared.offs[seg - ob] :
          (int)segments[seg];
        f(index, seg, index - start, mgpu::load(caching_iterators, seg),
          args...);
      }
    }
  }
}

// Partition + kernel, enqueued on `stream`. `partitions` must hold
// div_up(count + num_segments, tuning_t::nv) + 1 ints.
template<typename tuning_t, typename func_t, typename segments_it,
  typename pointers_t, typename... args_t>
void transform_lbs_enqueue(func_t f, int count, segments_it segments,
  int num_segments, pointers_t caching_iterators, int* partitions,
  cudaStream_t stream, uint64_t timeout_ns, uint32_t* status,
  args_t... args) {
  int64_t total = (int64_t)count + num_segments;
  int num_tiles = (int)div_up(total, (int64_t)tuning_t::nv);
  if(!num_tiles) return;
  launch_lbs_partition(segments, count, num_segments, (int64_t)tuning_t::nv,
    num_tiles + 1, partitions, stream);
  auto kernel = transform_lbs_k<tuning_t, func_t, segments_it, pointers_t,
    args_t...>;
  int smem_bytes = (int)sizeof(lbs_smem_t<tuning_t>);
  // More than 48 KB of shared memory per CTA has to be opted into, once per
  // kernel and device.
  static bool opted_in[64] = { };
  int device = 0;
  throw_on_error(cudaGetDevice(&device));
  if(device < 64 && !opted_in[device]) {
    throw_on_error(cudaFuncSetAttribute(kernel,
      cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    opted_in[device] = true;
  }
  kernel<<<num_tiles, (int)tuning_t::nt, smem_bytes, stream>>>(f, count,
    segments, num_segments, partitions, caching_iterators, timeout_ns, status,
    args...);
}

inline size_t lbs_partition_bytes(int count, int num_segments, int nv) {
  int64_t total = (int64_t)count + num_segments;
  return (size_t)(div_up(total, (int64_t)nv) + 1) * sizeof(int);
}

} // namespace detail

////////////////////////////////////////////////////////////////////////////////
// Public entry points.

template<typename launch_arg_t = empty_t, typename func_t,
  typename segments_it, typename pointers_t, typename... args_t>
void transform_lbs(func_t f, int count, segments_it segments,
  int num_segments, pointers_t caching_iterators, context_t& context,
  args_t... args) {
  typedef typename detail::pick_lbs_tuning<launch_arg_t>::type tuning_t;
  if(count < 0 || num_segments < 0 ||
    (int64_t)count + num_segments > (int64_t)0x7fffffff - 65536)
    throw cuda_exception_t(cudaErrorInvalidValue);
  if(0 == count + num_segments) return;
  mem_t<int> partitions(
    detail::lbs_partition_bytes(count, num_segments, tuning_t::nv) /
      sizeof(int), context);
  detail::transform_lbs_enqueue<tuning_t>(f, count, segments, num_segments,
    caching_iterators, partitions.data(), context.stream(),
    (uint64_t)2000000000ull, (uint32_t*)nullptr, args...);
}

// Without per-segment cached values: f(index, seg, rank, args...).
template<typename launch_arg_t = empty_t, typename func_t,
  typename segments_it, typename... args_t>
void transform_lbs(func_t f, int count, segments_it segments,
  int num_segments, context_t& context, args_t... args) {
  transform_lbs<launch_arg_t>(
    [=]MGPU_DEVICE(int index, int seg, int rank, tuple<>, args_t... rest) {
      f(index, seg, rank, rest...);
    }, count, segments, num_segments, tuple<>(), context, args...);
}

// output[index] = segment of item index.
template<typename launch_arg_t = empty_t, typename segments_it,
  typename output_it>
void load_balance_search(int count, segments_it segments, int num_segments,
  output_it output, context_t& context) {
  transform_lbs<launch_arg_t>([=]MGPU_DEVICE(int index, int seg, int rank) {
    output[index] = seg;
  }, count, segments, num_segments, context);
}

// output[index] = input[segment of item index].
template<typename launch_arg_t = empty_t, typename input_it,
  typename segments_it, typename output_it>
void interval_expand(input_it input, int count, segments_it segments,
  int num_segments, output_it output, context_t& context) {
  typedef typename std::iterator_traits<input_it>::value_type type_t;
  transform_lbs<launch_arg_t>(
    []MGPU_DEVICE(int index, int seg, int rank, tuple<type_t> desc,
      output_it output) {
      output[index] = get<0>(desc);
    }, count, segments, num_segments, make_tuple(input), context, output);
}

// output[index] = input[gather[seg] + rank].
template<typename launch_arg_t = empty_t, typename input_it,
  typename segments_it, typename gather_it, typename output_it>
void interval_gather(input_it input, int count, segments_it segments,
  int num_segments, gather_it gather, output_it output, context_t& context) {
  transform_lbs<launch_arg_t>(
    []MGPU_DEVICE(int index, int seg, int rank, tuple<int> desc,
      input_it input, output_it output) {
      output[index] = input[get<0>(desc) + rank];
    }, count, segments, num_segments, make_tuple(gather), context, input,
    output);
}

// output[scatter[seg] + rank] = input[index].
template<typename launch_arg_t = empty_t, typename input_it,
  typename segments_it, typename scatter_it, typename output_it>
void interval_scatter(input_it input, int count, segments_it segments,
  int num_segments, scatter_it scatter, output_it output,
  context_t& context) {
  transform_lbs<launch_arg_t>(
    []MGPU_DEVICE(int index, int seg, int rank, tuple<int> desc,
      input_it input, output_it output) {
      output[get<0>(desc) + rank] = input[index];
    }, count, segments, num_segments, make_tuple(scatter), context, input,
    output);
}

// output[scatter[seg] + rank] = input[gather[seg] + rank].
template<typename launch_arg_t = empty_t, typename input_it,
  typename segments_it, typename scatter_it, typename gather_it,
  typename output_it>
void interval_move(input_it input, int count, segments_it segments,
  int num_segments, scatter_it scatter, gather_it gather, output_it output,
  context_t& context) {
  transform_lbs<launch_arg_t>(
    []MGPU_DEVICE(int index, int seg, int rank, tuple<int, int> desc,
      input_it input, output_it output) {
      output[get<0>(desc) + rank] = input[get<1>(desc) + rank];
    }, count, segments, num_segments, make_tuple(scatter, gather), context,
    input, output);
}

END_MGPU_NAMESPACE

#endif // __CUDACC__
