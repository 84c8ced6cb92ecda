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
//
// Two kernels. scan_k takes any iterators and any value type: one CTA per
// tile, plain loads and stores. scan_stream_k serves the common case -- 4- or
// 8-byte arithmetic values behind 16-byte aligned raw pointers -- with a
// persistent grid in which no thread ever waits for global memory: a producer
// lane moves whole tiles between global and shared memory with bulk
// asynchronous copies (in AND out), 256 consumer threads work on shared
// memory only, and a carry warp does the look-back while the consumers are
// already busy with the next tile.
#pragma once
#include "runtime.hxx"
#include "ptx.hxx"
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

// Windows of 32 tiles a look-back reads per round trip. In a scan every tile
// depends on the whole chain before it, and the chain's front moves by one
// window per L2 round trip, so the number of tiles in flight decides: the
// generic kernel (hundreds of small tiles in flight) reads two windows at a
// time, the streaming kernel keeps one large tile per SM in flight and is
// served best by one.
enum { scan_lookback_rows = 2, scan_stream_lookback_rows = 1 };

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
      carry_ok = lookback_wide<scan_lookback_rows>(state, tile, op, carry,
        timeout_ns, header + 1);
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

////////////////////////////////////////////////////////////////////////////////
// Streaming kernel.

template<int nt_, int vt_, int stages_ = 3, int occ_ = 1>
struct scan_stream_tuning_t {
  enum { nt = nt_, vt = vt_, stages = stages_, occ = occ_, nv = nt_ * vt_ };
};

// vt is chosen so that a thread's run of items is a whole number of 16-byte
// words whose 128-bit shared loads do not collide (run length = 4 mod 8
// 32-bit words). Tiles are as large as three stages of shared memory allow
// (72 KB each, one CTA per SM): the fewer tiles, the shorter the chain of
// look-backs. Measured on 2^28 int32: 256 x 20 tiles, two CTAs per SM:
// 1,117 us; 512 x 36: 359 us.
template<typename type_t, int size = (int)sizeof(type_t)>
struct scan_stream_default_tuning { typedef scan_stream_tuning_t<512, 36> type; };
template<typename type_t>
struct scan_stream_default_tuning<type_t, 8> {
  typedef scan_stream_tuning_t<512, 18> type;
};

template<typename tuning_t, scan_type_t scan_type, typename type_t,
  typename op_t, typename reduction_it>
__global__ void __launch_bounds__(tuning_t::nt + 64, tuning_t::occ)
scan_stream_k(const type_t* input, int count, type_t* output, op_t op,
  reduction_it reduction, uint32_t* header, void* tile_state, int num_tiles,
  uint64_t timeout_ns) {

  enum { nt = tuning_t::nt, vt = tuning_t::vt, nv = tuning_t::nv,
    stages = tuning_t::stages, warps = nt / 32,
    words = vt * (int)sizeof(type_t) / 16,      // 16-byte words per thread
    producer_warp = warps, carry_warp = warps + 1 };
  static_assert(0 == (vt * sizeof(type_t)) % 16, "whole 16-byte words");

  extern __shared__ __align__(128) char scan_shared[];
  type_t* data = (type_t*)scan_shared;           // [stages][nv]
  __shared__ uint64_t full[stages], store_ready[stages], agg_ready[stages],
    carry_ready[stages];
  __shared__ int tile_of[stages], count_of[stages], carry_have[stages];
  __shared__ type_t agg[stages], carry_slot[stages];
  __shared__ type_t warp_total[2][warps];

  const int tid = (int)threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const unsigned all_lanes = 0xffffffffu;

  if(0 == tid) {
    for(int s = 0; s < stages; ++s) {
      ptx::mbar_init(&full[s], 1);
      ptx::mbar_init(&store_ready[s], nt);
      ptx::mbar_init(&agg_ready[s], 1);
      ptx::mbar_init(&carry_ready[s], 1);
      tile_of[s] = -1;
      count_of[s] = 0;
    }
    ptx::fence_proxy_async();
  }
  __syncthreads();

  if(warp == producer_warp) {
    //////////////////////////////////////////////////////////////////////////
    // Producer: results out of a stage, then the next tile into it.
    if(lane) return;
    const uint64_t policy = ptx::l2_policy_evict_first();
    auto store_stage = [&](int s) {
      uint32_t bytes = (uint32_t)(count_of[s] * (int)sizeof(type_t)) & ~15u;
      if(bytes)
        ptx::bulk_store(output + (size_t)tile_of[s] * nv, data + s * nv, bytes);
      ptx::bulk_commit();
    };
    for(int j = 0; ; ++j) {
      const int s = j % stages;
      if(j >= stages) {
        if(!ptx::mbar_wait(&store_ready[s], ((j / stages) - 1) & 1, timeout_ns)) {
          raise_status(header + 1, (uint32_t)status_copy_timeout);
          break;
        }
        store_stage(s);
        ptx::bulk_wait_read<0>();
      }
      const int tile = (int)atomicAdd(header, 1u);
      if(tile >= num_tiles) {
        tile_of[s] = -1;
        ptx::mbar_arrive(&full[s]);
        for(int j2 = j - stages + 1 > 0 ? j - stages + 1 : 0; j2 < j; ++j2) {
          const int s2 = j2 % stages;
          if(!ptx::mbar_wait(&store_ready[s2], (j2 / stages) & 1, timeout_ns)) {
            raise_status(header + 1, (uint32_t)status_copy_timeout);
            break;
          }
          store_stage(s2);
        }
        break;
      }
      const int begin = tile * nv;
      const int n = count - begin < nv ? count - begin : nv;
      tile_of[s] = tile;
      count_of[s] = n;
      const uint32_t bytes = (uint32_t)(n * (int)sizeof(type_t)) & ~15u;
      if(bytes) {
        ptx::fence_proxy_async();
        ptx::mbar_arrive_expect_tx(&full[s], bytes);
        ptx::bulk_load_hint(data + s * nv, input + begin, bytes, &full[s],
          policy);
      } else
        ptx::mbar_arrive(&full[s]);
    }
    // The shared memory must outlive the reads of the last stores.
    ptx::bulk_wait_read<0>();
    return;
  }

  tile_state_t<type_t> state;
  state.bind(tile_state, num_tiles);

  if(warp == carry_warp) {
    //////////////////////////////////////////////////////////////////////////
    // Carry warp: one look-back per tile, off the consumers' critical path.
    for(int k = 0; ; ++k) {
      const int s = k % stages;
      if(!ptx::mbar_wait(&agg_ready[s], (k / stages) & 1, timeout_ns)) {
        if(!lane) raise_status(header + 1, (uint32_t)status_copy_timeout);
        return;
      }
      const int tile = tile_of[s];
      if(tile < 0) return;
      const type_t aggregate = agg[s];
      if(0 == lane)
        state.publish(tile, tile ? tile_partial : tile_inclusive, aggregate);
      type_t carry = aggregate;
      bool carry_ok = false;
      if(tile > 0) {
        carry_ok = lookback_wide<scan_lookback_rows>(state, tile, op, carry,
        timeout_ns, header + 1);
        if(0 == lane && carry_ok)
          state.publish(tile, tile_inclusive, op(carry, aggregate));
      }
      if(0 == lane) {
        carry_slot[s] = carry;
        carry_have[s] = carry_ok;
        if(tile == num_tiles - 1)
          *reduction = carry_ok ? op(carry, aggregate) : aggregate;
        ptx::mbar_arrive(&carry_ready[s]);
      }
      __syncwarp();
    }
  }

  ////////////////////////////////////////////////////////////////////////////
  // Consumers. Iteration k: the local scan of tile k, then the finish of tile
  // k - 1, whose carry the carry warp has produced in the meantime.
  struct alignas(16) run_t { type_t x[vt]; };
  auto load_run = [&](int s, run_t& r) {
    const uint4* from = (const uint4*)(data + s * nv + tid * vt);
    #pragma unroll
    for(int w = 0; w < words; ++w) ((uint4*)r.x)[w] = from[w];
  };
  auto store_run = [&](int s, const run_t& r) {
    uint4* to = (uint4*)(data + s * nv + tid * vt);
    #pragma unroll
    for(int w = 0; w < words; ++w) to[w] = ((const uint4*)r.x)[w];
  };

  int prev_s = -1, prev_n = 0, prev_tile = 0;
  type_t prev_prefix = type_t();
  bool prev_prefix_have = false;

  for(int k = 0; ; ++k) {
    const int s = k % stages;
    bool arrived = ptx::mbar_wait(&full[s], (k / stages) & 1, timeout_ns);
    const int tile = tile_of[s];
    const int n = count_of[s];
    const int first = tid * vt;
    const int mine = n - first < 0 ? 0 : (n - first < vt ? n - first : vt);

    type_t prefix = type_t();
    bool prefix_have = false;
    if(tile >= 0) {
      // Items beyond the last whole 16-byte word of the array come by plain
      // loads, into the shared-memory slots of the thread that owns them.
      const int bulk_items = (int)(((uint32_t)(n * (int)sizeof(type_t)) & ~15u) /
        sizeof(type_t));
      if(first + mine > bulk_items)
        for(int i = bulk_items > first ? bulk_items - first : 0; i < mine; ++i)
          data[s * nv + first + i] = input[(size_t)tile * nv + first + i];

      run_t r;
      load_run(s, r);
      type_t total = r.x[0];
      #pragma unroll
      for(int i = 1; i < vt; ++i)
        if(i < mine) total = op(total, r.x[i]);
      bool have = mine > 0;

      // Inclusive scan of the thread totals across the warp (threads without
      // items sit at the end and contribute nothing).
      type_t incl = total;
      bool incl_have = have;
      #pragma unroll
      for(int delta = 1; delta < 32; delta *= 2) {
        type_t left = shfl_up_any(incl, delta);
        bool left_have = __shfl_up_sync(all_lanes, incl_have, delta);
        if(lane >= delta && left_have) {
          incl = incl_have ? op(left, incl) : left;
          incl_have = true;
        }
      }
      type_t before = shfl_up_any(incl, 1);
      bool before_have = __shfl_up_sync(all_lanes, incl_have, 1) && lane > 0;
      if(31 == lane) warp_total[k & 1][warp] = incl;
      arrived = ptx::named_all<1, nt>(arrived);

      const int warps_used = (n + 32 * vt - 1) / (32 * vt);
      type_t aggregate = warp_total[k & 1][0];
      for(int w = 1; w < warps_used; ++w) {
        if(w == warp) { prefix = aggregate; prefix_have = true; }
        aggregate = op(aggregate, warp_total[k & 1][w]);
      }
      if(before_have) {
        prefix = prefix_have ? op(prefix, before) : before;
        prefix_have = true;
      }
      if(0 == tid) {
        agg[s] = aggregate;
        ptx::mbar_arrive(&agg_ready[s]);
      }
    } else {
      arrived = ptx::named_all<1, nt>(arrived);
      if(0 == tid) ptx::mbar_arrive(&agg_ready[s]);     // lets the carry warp leave
    }
    if(!arrived) {
      if(0 == tid) raise_status(header + 1, (uint32_t)status_copy_timeout);
      return;
    }

    if(prev_s >= 0) {
      // Finish tile k - 1.
      const int ps = prev_s;
      if(!ptx::mbar_wait(&carry_ready[ps], ((k - 1) / stages) & 1, timeout_ns))
        raise_status(header + 1, (uint32_t)status_copy_timeout);
      type_t pre = prev_prefix;
      bool pre_have = prev_prefix_have;
      if(carry_have[ps]) {
        pre = pre_have ? op(carry_slot[ps], pre) : carry_slot[ps];
        pre_have = true;
      }
      const int pfirst = tid * vt;
      const int pmine = prev_n - pfirst < 0 ? 0 :
        (prev_n - pfirst < vt ? prev_n - pfirst : vt);
      run_t r;
      load_run(ps, r);
      type_t running = pre;
      bool running_have = pre_have;
      #pragma unroll
      for(int i = 0; i < vt; ++i) {
        type_t inclusive = running_have ? op(running, r.x[i]) : r.x[i];
        if(scan_type_inc == scan_type) r.x[i] = inclusive;
        else r.x[i] = running_have ? running : type_t();
        running = inclusive;
        running_have = true;
      }
      store_run(ps, r);
      const int bulk_items = (int)(((uint32_t)(prev_n * (int)sizeof(type_t)) &
        ~15u) / sizeof(type_t));
      if(pfirst + pmine > bulk_items)
        for(int i = bulk_items > pfirst ? bulk_items - pfirst : 0; i < pmine; ++i)
          output[(size_t)prev_tile * nv + pfirst + i] =
            data[ps * nv + pfirst + i];
      ptx::fence_proxy_async();
      ptx::mbar_arrive(&store_ready[ps]);
    }
    if(tile < 0) return;
    prev_s = s;
    prev_n = n;
    prev_tile = tile;
    prev_prefix = prefix;
    prev_prefix_have = prefix_have;
  }
}

template<typename type_t, typename reduction_it>
__global__ void scan_empty_k(reduction_it reduction) {
  if(0 == threadIdx.x && 0 == blockIdx.x) *reduction = type_t();
}

// Which kernel serves a call: the streaming kernel needs raw pointers to the
// same 4- or 8-byte arithmetic type on both sides (and, at run time, 16-byte
// aligned addresses); a scan_tuning_t in the launch_arg_t slot asks for the
// generic kernel, a scan_stream_tuning_t picks the streaming tile shape.
template<typename launch_arg_t, typename type_t, typename input_it,
  typename output_it>
struct scan_route_t {
  enum { streamable =
    std::is_pointer<input_it>::value && std::is_pointer<output_it>::value &&
    std::is_arithmetic<type_t>::value &&
    (4 == sizeof(type_t) || 8 == sizeof(type_t)) &&
    std::is_same<typename std::remove_cv<
      typename std::remove_pointer<input_it>::type>::type, type_t>::value &&
    std::is_same<typename std::remove_pointer<output_it>::type, type_t>::value };
  typedef typename pick_scan_tuning<launch_arg_t, type_t>::type tuning_t;
  typedef typename scan_stream_default_tuning<type_t>::type stream_tuning_t;
};
template<int nt, int vt, int occ, typename type_t, typename input_it,
  typename output_it>
struct scan_route_t<scan_tuning_t<nt, vt, occ>, type_t, input_it, output_it> {
  enum { streamable = 0 };
  typedef scan_tuning_t<nt, vt, occ> tuning_t;
  typedef typename scan_stream_default_tuning<type_t>::type stream_tuning_t;
};
template<int nt, int vt, int stages, int occ, typename type_t,
  typename input_it, typename output_it>
struct scan_route_t<scan_stream_tuning_t<nt, vt, stages, occ>, type_t,
  input_it, output_it> :
  scan_route_t<empty_t, type_t, input_it, output_it> {
  typedef scan_stream_tuning_t<nt, vt, stages, occ> stream_tuning_t;
};

// Bytes of scratch a scan over `count` items needs (enough for either kernel).
template<typename tuning_t, typename type_t,
  typename stream_tuning_t = typename scan_stream_default_tuning<type_t>::type>
size_t scan_workspace_bytes(int count) {
  int nv = (int)tuning_t::nv < (int)stream_tuning_t::nv ? (int)tuning_t::nv :
    (int)stream_tuning_t::nv;
  int num_tiles = div_up(count, nv);
  return 128 + tile_state_bytes<type_t>(num_tiles) + 128;
}

template<typename tag_t, typename kernel_t>
int scan_resident_ctas(kernel_t kernel, int threads, int smem_bytes) {
  int device = 0;
  throw_on_error(cudaGetDevice(&device));
  static int cached[64] = { };
  if(device < 64 && cached[device]) return cached[device];
  throw_on_error(cudaFuncSetAttribute(kernel,
    cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
  int per_sm = 0, sms = 0;
  throw_on_error(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm,
    kernel, threads, smem_bytes));
  throw_on_error(cudaDeviceGetAttribute(&sms,
    cudaDevAttrMultiProcessorCount, device));
  int n = per_sm * sms;
  if(n < 1) n = 1;
  if(device < 64) cached[device] = n;
  return n;
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

template<typename tuning_t, scan_type_t scan_type, typename type_t,
  typename op_t, typename reduction_it>
void scan_stream_enqueue(const type_t* input, int count, type_t* output,
  op_t op, reduction_it reduction, void* workspace, cudaStream_t stream,
  uint64_t timeout_ns = 2000000000ull) {
  int num_tiles = div_up(count, (int)tuning_t::nv);
  char* base = (char*)workspace;
  throw_on_error(cudaMemsetAsync(base, 0,
    128 + tile_state_bytes<type_t>(num_tiles), stream));
  auto kernel = scan_stream_k<tuning_t, scan_type, type_t, op_t, reduction_it>;
  const int threads = (int)tuning_t::nt + 64;
  const int smem = (int)tuning_t::stages * (int)tuning_t::nv *
    (int)sizeof(type_t);
  int resident = scan_resident_ctas<
    tuple<tuning_t, type_t, op_t, reduction_it,
      std::integral_constant<int, (int)scan_type> > >(kernel, threads, smem);
  int grid = num_tiles < resident ? num_tiles : resident;
  kernel<<<grid, threads, smem, stream>>>(input, count, output, op, reduction,
    (uint32_t*)base, base + 128, num_tiles, timeout_ns);
}

// Picks the kernel. Both share the workspace layout.
template<typename route_t, scan_type_t scan_type, typename type_t,
  typename input_it, typename output_it, typename op_t, typename reduction_it>
void scan_dispatch(input_it input, int count, output_it output, op_t op,
  reduction_it reduction, void* workspace, cudaStream_t stream,
  uint64_t timeout_ns = 2000000000ull) {
  if constexpr (route_t::streamable) {
    if(count > 0 && 0 == ((uintptr_t)input | (uintptr_t)output) % 16) {
      scan_stream_enqueue<typename route_t::stream_tuning_t, scan_type, type_t>(
        (const type_t*)input, count, (type_t*)output, op, reduction, workspace,
        stream, timeout_ns);
      return;
    }
  }
  scan_enqueue<typename route_t::tuning_t, scan_type, type_t>(input, count,
    output, op, reduction, workspace, stream, timeout_ns);
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
  typedef detail::scan_route_t<launch_arg_t, type_t, input_it, output_it>
    route_t;
  detail::throw_on_device_status();
  mem_t<char> workspace(detail::scan_workspace_bytes<
    typename route_t::tuning_t, type_t, typename route_t::stream_tuning_t>(
      count), context);
  detail::scan_dispatch<route_t, scan_type, type_t>(input, count, output, op,
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
