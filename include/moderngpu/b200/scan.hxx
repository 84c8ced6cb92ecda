// Single-pass prefix scan for sm_100a: scan, scan_event, transform_scan.
//
// Interface parity (reference): src/moderngpu/kernel_scan.hxx:11-196 —
// scan<scan_type>(input, count, output, op, reduction, context), the
// plus/discard shorthand, scan_event and transform_scan(_event);
// scan_type_exc / scan_type_inc as in src/moderngpu/cta_scan.hxx:8-11. An
// exclusive scan starts with type_t() (the reference's `init`), `*reduction`
// receives the fold of all items (type_t() when count is 0). This is the
// step that turns segment lengths into the start offsets the segmented
// reduction and the load-balancing search consume.
//
// The reference runs three passes (upsweep, recursive spine, downsweep:
// 2 reads + 1 write of the data). Here a tile is read once and written once:
// tiles take a ticket, scan locally (register-blocked through a padded
// shared-memory transpose, warp shuffles across threads), publish their
// aggregate in the same per-tile status words the segmented reduction uses
// and obtain their carry-in by a decoupled look-back (tile_state.hxx).
#pragma once
#include "runtime.hxx"
#include "tile_state.hxx"

BEGIN_MGPU_NAMESPACE

enum scan_type_t {
  scan_type_exc,
  scan_type_inc
};

#ifdef __CUDACC__

template<int nt_, int vt_, int occ_ = 0>
struct scan_tuning_t {
  enum { nt = nt_, vt = vt_, occ = occ_, nv = nt_ * vt_ };
};

namespace detail {

template<typename type_t, int size = (int)sizeof(type_t)>
struct scan_default_tuning { typedef scan_tuning_t<128, 4, 4> type; };
template<typename type_t>
struct scan_default_tuning<type_t, 4> { typedef scan_tuning_t<512, 20, 2> type; };
template<typename type_t>
struct scan_default_tuning<type_t, 8> { typedef scan_tuning_t<256, 8, 4> type; };

template<typename launch_arg_t, typename type_t>
struct pick_scan_tuning { typedef typename scan_default_tuning<type_t>::type type; };
template<int nt, int vt, int occ, typename type_t>
struct pick_scan_tuning<scan_tuning_t<nt, vt, occ>, type_t> {
  typedef scan_tuning_t<nt, vt, occ> type;
};

// Shared-memory index with one pad word per 32: a thread's vt consecutive
// items and a warp's striped items both spread over the banks.
MGPU_HOST_DEVICE int scan_pad(int j) { return j + (j >> 5); }

template<typename tuning_t, scan_type_t scan_type, typename type_t,
  typename input_it, typename output_it, typename op_t, typename reduction_it>
__global__ void __launch_bounds__(tuning_t::nt, tuning_t::occ)
scan_k(input_it input, int count, output_it output, op_t op,
  reduction_it reduction, uint32_t* header, void* tile_state, int num_tiles,
  uint64_t timeout_ns) {

  enum { nt = tuning_t::nt, vt = tuning_t::vt, nv = tuning_t::nv,
    warps = nt / 32 };
  __shared__ type_t values[nv + nv / 32 + 1];
  __shared__ type_t warp_total[warps];
  __shared__ type_t carry_slot;
  __shared__ int carry_have;
  __shared__ int tile_slot;

  const int tid = (int)threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const unsigned full = 0xffffffffu;

  // Tiles are handed out in order, so a tile's predecessors are running or
  // finished whenever it looks back.
  if(0 == tid) tile_slot = (int)atomicAdd(header, 1u);
  __syncthreads();
  const int tile = tile_slot;
  if(tile >= num_tiles) return;
  const int begin = tile * nv;
  const int n = count - begin < nv ? count - begin : nv;

  tile_state_t<type_t> state;
  state.bind(tile_state, num_tiles);

  // Coalesced (striped) loads, transposed through shared memory.
  #pragma unroll
  for(int i = 0; i < vt; ++i) {
    int j = i * nt + tid;
    if(j < n) values[scan_pad(j)] = (type_t)input[begin + j];
  }
  __syncthreads();

  // Thread-local inclusive scan of items [tid * vt, tid * vt + mine).
  const int first = tid * vt;
  const int mine = n - first < 0 ? 0 : (n - first < vt ? n - first : vt);
  type_t y[vt];
  type_t total = type_t();
  #pragma unroll
  for(int i = 0; i < vt; ++i) {
    if(i < mine) {
      type_t x = values[scan_pad(first + i)];
      y[i] = i ? op(y[i - 1], x) : x;
      total = y[i];
    }
  }
  bool have = mine > 0;

  // Inclusive scan of the thread totals across the warp (threads without
  // items sit at the end and contribute nothing).
  type_t incl = total;
  bool incl_have = have;
  #pragma unroll
  for(int delta = 1; delta < 32; delta *= 2) {
    type_t left = shfl_up_any(incl, delta);
    bool left_have = __shfl_up_sync(full, incl_have, delta);
    if(lane >= delta && left_have) {
      incl = incl_have ? op(left, incl) : left;
      incl_have = true;
    }
  }
  type_t before = shfl_up_any(incl, 1);
  bool before_have = __shfl_up_sync(full, incl_have, 1) && lane > 0;
  if(31 == lane) warp_total[warp] = incl;
  // A warp has items iff its first thread has.
  __syncthreads();
  const int warps_used = (n + 32 * vt - 1) / (32 * vt);

  // Fold of the warps before this one, and the tile's aggregate.
  type_t warp_before = type_t();
  bool warp_before_have = false;
  for(int k = 0; k < warp && k < warps_used; ++k) {
    warp_before = warp_before_have ? op(warp_before, warp_total[k]) :
      warp_total[k];
    warp_before_have = true;
  }

  if(0 == warp) {
    type_t aggregate = warp_total[0];
    for(int k = 1; k < warps_used; ++k) aggregate = op(aggregate, warp_total[k]);
    if(0 == lane)
      state.publish(tile, tile ? tile_partial : tile_inclusive, aggregate);
    type_t carry = aggregate;
    bool carry_ok = false;
    if(tile > 0) {
      carry_ok = lookback(state, tile, op, carry, timeout_ns, header + 1);
      if(0 == lane && carry_ok)
        state.publish(tile, tile_inclusive, op(carry, aggregate));
    }
    if(0 == lane) {
      carry_slot = carry;
      carry_have = carry_ok;
      if(tile == num_tiles - 1)
        *reduction = carry_ok ? op(carry, aggregate) : aggregate;
    }
  }
  __syncthreads();

  // What precedes this thread's first item: earlier tiles, earlier warps,
  // earlier lanes -- folded in that order.
  type_t prefix = type_t();
  bool prefix_have = false;
  if(carry_have) { prefix = carry_slot; prefix_have = true; }
  if(warp_before_have) {
    prefix = prefix_have ? op(prefix, warp_before) : warp_before;
    prefix_have = true;
  }
  if(before_have) {
    prefix = prefix_have ? op(prefix, before) : before;
    prefix_have = true;
  }

  // Results back through shared memory for coalesced stores.
  #pragma unroll
  for(int i = 0; i < vt; ++i) {
    if(i < mine) {
      type_t inclusive = prefix_have ? op(prefix, y[i]) : y[i];
      type_t result;
      if(scan_type_inc == scan_type) result = inclusive;
      else if(0 == i) result = prefix_have ? prefix : type_t();
      else result = prefix_have ? op(prefix, y[i - 1]) : y[i - 1];
      values[scan_pad(first + i)] = result;
    }
  }
  __syncthreads();
  #pragma unroll
  for(int i = 0; i < vt; ++i) {
    int j = i * nt + tid;
    if(j < n) output[begin + j] = values[scan_pad(j)];
  }
}

template<typename type_t, typename reduction_it>
__global__ void scan_empty_k(reduction_it reduction) {
  if(0 == threadIdx.x && 0 == blockIdx.x) *reduction = type_t();
}

// Bytes of scratch a scan over `count` items needs.
template<typename tuning_t, typename type_t>
size_t scan_workspace_bytes(int count) {
  int num_tiles = div_up(count, (int)tuning_t::nv);
  return 128 + tile_state_bytes<type_t>(num_tiles) + 128;
}

template<typename tuning_t, scan_type_t scan_type, typename type_t,
  typename input_it, typename output_it, typename op_t, typename reduction_it>
void scan_enqueue(input_it input, int count, output_it output, op_t op,
  reduction_it reduction, void* workspace, cudaStream_t stream,
  uint64_t timeout_ns = 2000000000ull) {
  if(count <= 0) {
    scan_empty_k<type_t><<<1, 32, 0, stream>>>(reduction);
    return;
  }
  int num_tiles = div_up(count, (int)tuning_t::nv);
  char* base = (char*)workspace;
  // Ticket counter, status word and every tile's status start at zero.
  throw_on_error(cudaMemsetAsync(base, 0,
    128 + tile_state_bytes<type_t>(num_tiles), stream));
  scan_k<tuning_t, scan_type, type_t><<<num_tiles, (int)tuning_t::nt, 0,
    stream>>>(input, count, output, op, reduction, (uint32_t*)base,
    base + 128, num_tiles, timeout_ns);
}

} // namespace detail

////////////////////////////////////////////////////////////////////////////////
// Public entry points.

template<scan_type_t scan_type = scan_type_exc,
  typename launch_arg_t = empty_t, typename input_it,
  typename output_it, typename op_t, typename reduction_it>
void scan_event(input_it input, int count, output_it output, op_t op,
  reduction_it reduction, context_t& context, cudaEvent_t event) {
  typedef typename std::iterator_traits<input_it>::value_type type_t;
  typedef typename detail::pick_scan_tuning<launch_arg_t, type_t>::type
    tuning_t;
  mem_t<char> workspace(
    detail::scan_workspace_bytes<tuning_t, type_t>(count), context);
  detail::scan_enqueue<tuning_t, scan_type, type_t>(input, count, output, op,
    reduction, workspace.data(), context.stream());
  // The reduction is complete when the kernel is.
  if(event) cudaEventRecord(event, context.stream());
}

template<scan_type_t scan_type = scan_type_exc,
  typename launch_arg_t = empty_t, typename input_it,
  typename output_it, typename op_t, typename reduction_it>
void scan(input_it input, int count, output_it output, op_t op,
  reduction_it reduction, context_t& context) {
  scan_event<scan_type, launch_arg_t>(input, count, output, op, reduction,
    context, 0);
}

template<scan_type_t scan_type = scan_type_exc,
  typename launch_arg_t = empty_t, typename input_it, typename output_it>
void scan(input_it input, int count, output_it output, context_t& context) {
  typedef typename std::iterator_traits<input_it>::value_type type_t;
  scan<scan_type, launch_arg_t>(input, count, output, plus_t<type_t>(),
    discard_iterator_t<type_t>(), context);
}

template<typename type_t, scan_type_t scan_type = scan_type_exc,
  typename launch_arg_t = empty_t, typename func_t, typename output_it,
  typename op_t, typename reduction_it>
void transform_scan_event(func_t f, int count, output_it output, op_t op,
  reduction_it reduction, context_t& context, cudaEvent_t event) {
  scan_event<scan_type, launch_arg_t>(make_load_iterator<type_t>(f), count,
    output, op, reduction, context, event);
}

template<typename type_t, scan_type_t scan_type = scan_type_exc,
  typename launch_arg_t = empty_t, typename func_t, typename output_it,
  typename op_t, typename reduction_it>
void transform_scan(func_t f, int count, output_it output, op_t op,
  reduction_it reduction, context_t& context) {
  transform_scan_event<type_t, scan_type, launch_arg_t>(f, count, output, op,
    reduction, context, 0);
}

#endif // __CUDACC__

END_MGPU_NAMESPACE
