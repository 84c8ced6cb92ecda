// Dynamic work creation on top of the load-balancing search, for sm_100a.
//
// Interface parity (reference): expt::lbs_workcreate / expt::workcreate_t
// src/moderngpu/kernel_workcreate.hxx:14-268 -- the engine the reference's
// breadth-first-search demos (demo/bfs2.cu:27-58) expand a frontier with.
//
//   auto engine = expt::lbs_workcreate(count, segments, num_segments, context);
//   auto n = engine.upsweep(f[, caching_iterators]);
//     f(index, seg, rank[, cached]) -> number of work items this item creates;
//     n.num_segments = items that create work, n.count = work items in all.
//   mem_t<int> next = engine.downsweep(g[, caching_iterators], args...);
//     g(dest_seg, index, seg, rank[, cached], args...) is called for the
//     creating items only, in index order, dest_seg = 0, 1, 2, ...; it
//     returns the same number again, and next[dest_seg] is the exclusive
//     prefix sum of those numbers: the segment starts of the next round.
//
// Both sweeps run the tile machinery of transform_lbs (bulk-staged segment
// starts, head ids, max-scan). The upsweep leaves one bit per item (does it
// create work?) and one (creators, work) pair per tile; a single-pass scan
// turns the pairs into tile offsets; the downsweep compacts each tile's
// creators from the bits and scans their counts inside the CTA.
#pragma once
#include "load_balance.hxx"
#include "scan.hxx"

#ifdef __CUDACC__

BEGIN_MGPU_NAMESPACE

namespace detail {

struct add_int2_t {
  MGPU_HOST_DEVICE int2 operator()(int2 a, int2 b) const {
    return make_int2(a.x + b.x, a.y + b.y);
  }
};

// Exclusive prefix sum of one int per thread over the CTA; `total` receives
// the sum. Two barriers; `warp_sums` holds nt / 32 ints.
template<int nt>
MGPU_DEVICE int cta_exclusive_sum(int x, int* warp_sums, int& total) {
  const int tid = (int)threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int incl = x;
  #pragma unroll
  for(int delta = 1; delta < 32; delta *= 2) {
    int y = __shfl_up_sync(0xffffffffu, incl, delta);
    if(lane >= delta) incl += y;
  }
  __syncthreads();                        // warp_sums free for reuse
  if(31 == lane) warp_sums[warp] = incl;
  __syncthreads();
  int before = 0, sum = 0;
  #pragma unroll
  for(int w = 0; w < nt / 32; ++w) {
    int s = warp_sums[w];
    if(w < warp) before += s;
    sum += s;
  }
  total = sum;
  return before + incl - x;
}

template<typename tuning_t>
struct workcreate_smem_t {
  enum { nv = tuning_t::nv, words = nv / 32, warps = tuning_t::nt / 32 };
  lbs_smem_t<tuning_t> lbs;
  int targets[nv];            // downsweep: tile positions of the creators
  uint32_t mask[words];       // one bit per item of the tile
  int warp_sums[2][warps];
};

template<typename tuning_t, typename func_t, typename segments_it,
  typename pointers_t>
__global__ void __launch_bounds__(tuning_t::nt, tuning_t::occ)
workcreate_upsweep_k(func_t f, int count, segments_it segments,
  int num_segments, const int* partitions, pointers_t caching_iterators,
  uint32_t* bits, int2* tile_counts) {
  enum { nt = tuning_t::nt, vt = tuning_t::vt, nv = tuning_t::nv,
    words = nv / 32 };
  extern __shared__ __align__(128) char workcreate_raw[];
  workcreate_smem_t<tuning_t>& shared =
    *reinterpret_cast<workcreate_smem_t<tuning_t>*>(workcreate_raw);
  const int tid = (int)threadIdx.x;
  const int tile = (int)blockIdx.x;

  for(int i = tid; i < words; i += nt) shared.mask[i] = 0;
  lbs_tile_t t = lbs_tile_segments<tuning_t>(tile, count, segments,
    num_segments, partitions, shared.lbs, (uint64_t)2000000000ull,
    (uint32_t*)nullptr);
  const int na = t.a1 - t.a0;

  int creators = 0, work = 0;
  #pragma unroll
  for(int i = 0; i < vt; ++i) {
    int w = i * nt + tid;
    if(w < na) {
      int seg = shared.lbs.seg_of[w];
      if(seg >= 0) {
        int index = t.a0 + w;
        int start = (seg >= t.ob && seg < t.oe) ? shared.lbs.offs[seg - t.ob] :
          (int)segments[seg];
        int n = f(index, seg, index - start,
          mgpu::load(caching_iterators, seg));
        if(n > 0) {
          atomicOr(&shared.mask[w >> 5], 1u << (w & 31));
          ++creators;
          work += n;
        }
      }
    }
  }
  int all_creators = 0, all_work = 0;
  cta_exclusive_sum<nt>(creators, shared.warp_sums[0], all_creators);
  cta_exclusive_sum<nt>(work, shared.warp_sums[1], all_work);
  if(0 == tid) tile_counts[tile] = make_int2(all_creators, all_work);
  // The barriers inside the sums also order the atomicOr's before this.
  for(int i = tid; i < words; i += nt)
    bits[(size_t)tile * words + i] = shared.mask[i];
}

template<typename tuning_t, typename func_t, typename segments_it,
  typename pointers_t, typename... args_t>
__global__ void __launch_bounds__(tuning_t::nt, tuning_t::occ)
workcreate_downsweep_k(func_t f, int count, segments_it segments,
  int num_segments, const int* partitions, pointers_t caching_iterators,
  const uint32_t* bits, const int2* tile_offsets, int* segments_output,
  args_t... args) {
  enum { nt = tuning_t::nt, vt = tuning_t::vt, nv = tuning_t::nv,
    words = nv / 32 };
  static_assert(words <= nt, "one thread per word of the tile's bit mask");
  extern __shared__ __align__(128) char workcreate_raw[];
  workcreate_smem_t<tuning_t>& shared =
    *reinterpret_cast<workcreate_smem_t<tuning_t>*>(workcreate_raw);
  const int tid = (int)threadIdx.x;
  const int tile = (int)blockIdx.x;

  for(int i = tid; i < words; i += nt)
    shared.mask[i] = bits[(size_t)tile * words + i];
  lbs_tile_t t = lbs_tile_segments<tuning_t>(tile, count, segments,
    num_segments, partitions, shared.lbs, (uint64_t)2000000000ull,
    (uint32_t*)nullptr);

  // Compact the tile positions of the creators, in item order.
  uint32_t m = tid < words ? shared.mask[tid] : 0u;
  int num_items = 0;
  int at = cta_exclusive_sum<nt>(__popc(m), shared.warp_sums[0], num_items);
  while(m) {
    int b = __ffs(m) - 1;
    shared.targets[at++] = 32 * tid + b;
    m &= m - 1;
  }
  __syncthreads();

  const int2 offset = tile_offsets[tile];
  int work_dest = offset.y;
  for(int round = 0; round * nt < num_items; ++round) {
    int j = round * nt + tid;
    int n = 0;
    if(j < num_items) {
      int w = shared.targets[j];
      int seg = shared.lbs.seg_of[w];
      int index = t.a0 + w;
      int start = (seg >= t.ob && seg < t.oe) ? shared.lbs.offs[seg - t.ob] :
        (int)segments[seg];
      n = f(offset.x + j, index, seg, index - start,
        mgpu::load(caching_iterators, seg), args...);
    }
    int round_total = 0;
    int before = cta_exclusive_sum<nt>(n, shared.warp_sums[1], round_total);
    if(j < num_items) segments_output[offset.x + j] = work_dest + before;
    work_dest += round_total;
  }
}

} // namespace detail

// experimental feature (as in the reference)
namespace expt {

template<typename launch_arg_t, typename segments_it>
struct workcreate_t {
  typedef typename mgpu::detail::pick_lbs_tuning<launch_arg_t>::type tuning_t;
  enum { nv = tuning_t::nv, words = nv / 32 };

  segments_it segments;
  int num_segments;
  int count;
  context_t& context;
  int num_tiles;

  mem_t<int> partitions;
  mem_t<uint32_t> bits;          // one bit per item: does it create work?
  mem_t<int2> tile_offsets;      // (creators, work) per tile, then scanned
  int2 total;

  struct count_t {
    int count;
    int num_segments;
  };

  workcreate_t(int count_, segments_it segments_, int num_segments_,
    context_t& context_) : segments(segments_), num_segments(num_segments_),
    count(count_), context(context_), total(make_int2(0, 0)) {
    if(count < 0 || num_segments < 0 ||
      (int64_t)count + num_segments > (int64_t)0x7fffffff - 65536)
      throw cuda_exception_t(cudaErrorInvalidValue);
    num_tiles = (int)div_up((int64_t)count + num_segments, (int64_t)nv);
    partitions = mem_t<int>(num_tiles + 1, context);
    if(num_tiles)
      mgpu::detail::launch_lbs_partition(segments, count, num_segments,
        (int64_t)nv, num_tiles + 1, partitions.data(), context.stream());
    bits = mem_t<uint32_t>((size_t)num_tiles * words, context);
    tile_offsets = mem_t<int2>(num_tiles, context);
  }

  static int smem_bytes() {
    return (int)sizeof(mgpu::detail::workcreate_smem_t<tuning_t>);
  }
  template<typename kernel_t>
  static void opt_in(kernel_t kernel) {
    mgpu::detail::throw_on_error(cudaFuncSetAttribute(kernel,
      cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes()));
  }

  // f(int index, int seg, int rank, tuple<...> cached) returns the number of
  // work items to create.
  template<typename func_t, typename pointers_t>
  count_t upsweep(func_t f, pointers_t caching_iterators) {
    total = make_int2(0, 0);
    if(!num_tiles) return count_t { 0, 0 };
    auto kernel = mgpu::detail::workcreate_upsweep_k<tuning_t, func_t,
      segments_it, pointers_t>;
    opt_in(kernel);
    kernel<<<num_tiles, (int)tuning_t::nt, smem_bytes(), context.stream()>>>(
      f, count, segments, num_segments, partitions.data(), caching_iterators,
      bits.data(), tile_offsets.data());

    // Tile offsets = exclusive scan of the per-tile pairs; the grand total
    // comes back to the host, which must size the next round's arrays.
    mem_t<int2> total_device(1, context);
    scan(tile_offsets.data(), num_tiles, tile_offsets.data(),
      mgpu::detail::add_int2_t(), total_device.data(), context);
    total = from_mem(total_device)[0];
    return count_t { total.y, total.x };
  }

  template<typename func_t>
  count_t upsweep(func_t f) {
    return upsweep([=]MGPU_DEVICE(int index, int seg, int rank, tuple<>) {
      return f(index, seg, rank);
    }, tuple<>());
  }

  // f(int dest_seg, int index, int source_seg, int rank, tuple<...> cached,
  // args...) returns the number of work items to create (as in the upsweep).
  template<typename func_t, typename pointers_t, typename... args_t>
  mem_t<int> downsweep(func_t f, pointers_t caching_iterators,
    args_t... args) {
    mem_t<int> segments_result(total.x, context);
    if(!num_tiles || !total.x) return segments_result;
    auto kernel = mgpu::detail::workcreate_downsweep_k<tuning_t, func_t,
      segments_it, pointers_t, args_t...>;
    opt_in(kernel);
    kernel<<<num_tiles, (int)tuning_t::nt, smem_bytes(), context.stream()>>>(
      f, count, segments, num_segments, partitions.data(), caching_iterators,
      bits.data(), tile_offsets.data(), segments_result.data(), args...);
    return segments_result;
  }

  template<typename func_t, typename... args_t>
  mem_t<int> downsweep(func_t f, args_t... args) {
    return downsweep(
      [=]MGPU_DEVICE(int dest_seg, int index, int seg, int rank, tuple<>,
        args_t... rest) {
        return f(dest_seg, index, seg, rank, rest...);
      }, tuple<>(), args...);
  }
};

// Use lbs_workcreate to construct an engine, then call upsweep and downsweep.
template<typename launch_arg_t = empty_t, typename segments_it>
workcreate_t<launch_arg_t, segments_it>
lbs_workcreate(int count, segments_it segments, int num_segments,
  context_t& context) {
  return workcreate_t<launch_arg_t, segments_it>(count, segments,
    num_segments, context);
}

} // namespace expt

END_MGPU_NAMESPACE

#endif // __CUDACC__
