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
    if(!ptx::mbar_wait(&shared.bar, 0, timeout_ns) )
      raise_status(status, (uint32_t)status_copy_timeout);
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

////////////////////////////////////////////////////////////////////////////////
// Fill kernels. load_balance_search, the (segment, rank) recorder and
// interval_expand with raw pointers write, for every item, values that are
// contiguous in the item index, so a tile's output is one contiguous piece of
// each output array. Instead of visiting the items a second time in striped
// order (one dependent shared-memory lookup per item and output), every
// thread expands its vt consecutive items in registers -- a segment's rank
// restarts at a head bit, so nothing has to be looked up per item -- writes
// them to shared memory with 128-bit stores, and one thread hands the tile to
// the copy engine (bulk asynchronous copy shared -> global). Items are placed
// in shared memory so that 16-byte granules of the output array are 16-byte
// granules there; the up to three items of a ragged first or last granule
// are stored by ordinary stores.
//
// The kernel is persistent: CTAs take tiles from a ticket counter. A
// producer lane fetches tickets and partition values a few tiles ahead, and
// every consumer thread requests the segment start it will scatter for the
// NEXT tile before it works on the current one, so that no tile waits for a
// global load; the copy engine writes tile k out while tile k + 1 is worked
// on (head ids are scattered into an array of their own, the only one tile
// k + 1 writes before the copy engine is known to be done with tile k).

enum { lbs_fill_ids = 0, lbs_fill_ids_ranks = 1, lbs_fill_values = 2 };

template<int kind, typename value_t>
struct lbs_fill_args_t {
  int* ids;                 // kinds ids, ids_ranks: segment of every item
  int* ranks;               // kind ids_ranks: rank of every item
  const value_t* values;    // kind values: one value per segment,
  value_t* expanded;        //   copied to every item of the segment
};

template<int nt_, int vt_, int occ_>
struct lbs_fill_tuning_t {
  // A tile holds nt * vt slots; four are kept free so that the tile's first
  // item can sit anywhere in a 16-byte granule.
  enum { nt = nt_, vt = vt_, occ = occ_, slots = nt_ * vt_, nv = slots - 4 };
  static_assert(nt_ % 32 == 0 && vt_ % 4 == 0 && vt_ <= 28 &&
    nt_ * vt_ <= 8192, "unsupported tile");
};
typedef lbs_fill_tuning_t<256, 20, 4> lbs_fill_default_tuning;
// Per kind of output. Measured on 2^28 items over 2^22 segments (ids only /
// ids + ranks): 256 x 20 at 4 CTAs per SM 186.9 / 335.5 us; 256 x 28 at 3:
// 174.9 / 334.4; 256 x 28 at 2: 175.1 / 324.5; 192 x 28 at 4: 174.4 / 337.9;
// 384 x 20 at 2: 228.8 / 323.8; 320 x 20 at 3: 198.9 / 331.8; tile heights that
// are a multiple of 8 lose to bank conflicts on the 16-byte stores (256 x 16
// at 5: 286.8 / 533.5; 256 x 24 at 4: 192.8 / 346.7).
// Expanded values (interval_expand; the per-segment values of the next tile
// are requested ahead like its segment starts: 237.7 -> 199.4 us for 2^28
// 4-byte values, 290.6 -> 231.6 us for 2^27 8-byte values at 256 x 20 x 4):
// 4-byte values 256 x 20 at 2 - 4 CTAs 198.8 - 199.9 us, 256 x 28: 201.2 -
// 201.8, 256 x 12: 292; 8-byte values 256 x 12 at 4: 179.5 us, at 3: 212.8,
// 256 x 20: 231 - 232, 256 x 28: 263 - 264.
template<int kind, int value_bytes = 4>
struct lbs_fill_tuning_for { typedef lbs_fill_default_tuning type; };
template<int value_bytes>
struct lbs_fill_tuning_for<lbs_fill_ids, value_bytes> { typedef lbs_fill_tuning_t<256, 28, 3> type; };
template<int value_bytes>
struct lbs_fill_tuning_for<lbs_fill_ids_ranks, value_bytes> { typedef lbs_fill_tuning_t<256, 28, 2> type; };
template<>
struct lbs_fill_tuning_for<lbs_fill_values, 8> { typedef lbs_fill_tuning_t<256, 12, 4> type; };

struct lbs_fill_desc_t { int tile, a0, a1, pad; };

template<typename tuning_t, int kind, typename value_t>
struct lbs_fill_smem_t {
  typedef typename std::conditional<lbs_fill_values == kind, value_t,
    int>::type second_t;
  enum { slots = tuning_t::slots, warps = tuning_t::nt / 32,
    flag_words = slots / 32 + 2, ring = 4,
    ids_slots = lbs_fill_values == kind ? 4 : slots,
    second_slots = lbs_fill_ids == kind ? 4 : slots,
    head_value_slots = lbs_fill_values == kind ? slots : 4 };
  alignas(128) int ids[ids_slots];                // per-item ids
  alignas(128) second_t second[second_slots];     // ranks or expanded values
  alignas(16) second_t head_values[head_value_slots];   // value at each head
  alignas(16) uint16_t heads[slots];    // id - b0 of the segment at each head
  uint32_t flags[2][flag_words];
  int warp_max[warps];
  lbs_fill_desc_t desc[ring];
  uint64_t full[ring], empty[ring];
};

template<typename tuning_t, int kind, typename value_t, typename segments_it>
__global__ void __launch_bounds__(tuning_t::nt + 32, tuning_t::occ)
lbs_fill_k(lbs_fill_args_t<kind, value_t> out, int count,
  segments_it segments, int num_segments, const int* partitions,
  int num_tiles, uint32_t* header, uint64_t timeout_ns) {

  typedef lbs_fill_smem_t<tuning_t, kind, value_t> smem_t;
  typedef typename smem_t::second_t second_t;
  // The array that decides where item a0 sits in shared memory.
  typedef typename std::conditional<lbs_fill_values == kind, value_t,
    int>::type first_t;
  enum { nt = tuning_t::nt, vt = tuning_t::vt, nv = tuning_t::nv,
    warps = nt / 32, ring = smem_t::ring, flag_words = smem_t::flag_words,
    per16 = 16 / (int)sizeof(first_t) };
  extern __shared__ __align__(128) char lbs_fill_raw[];
  smem_t& shared = *reinterpret_cast<smem_t*>(lbs_fill_raw);

  const int tid = (int)threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const unsigned full = 0xffffffffu;
  uint32_t* status = header + 1;

  if(0 == tid) {
    for(int r = 0; r < ring; ++r) {
      ptx::mbar_init(&shared.full[r], 1);
      ptx::mbar_init(&shared.empty[r], nt);
    }
  }
  for(int i = tid; i < 2 * flag_words; i += nt + 32)
    (&shared.flags[0][0])[i] = 0;
  __syncthreads();
  // The partitioner (the preceding launch) wrote the table and cleared the
  // ticket counter.
  ptx::grid_dependency_wait();

  //////////////////////////////////////////////////////////////////////////////
  // Producer lane: tickets and partition values, up to `ring` tiles ahead.

  if(warp == warps) {
    if(lane) return;
    for(int k = 0; ; ++k) {
      const int r = k % ring;
      if(k >= ring &&
        !ptx::mbar_wait(&shared.empty[r], (k / ring - 1) & 1, timeout_ns)) {
        raise_status(status, (uint32_t)status_copy_timeout);
        return;
      }
      lbs_fill_desc_t d;
      d.tile = (int)atomicAdd(header, 1u);
      d.a0 = d.a1 = d.pad = 0;
      if(d.tile < num_tiles) {
        d.a0 = partitions[d.tile];
        d.a1 = partitions[d.tile + 1];
      } else {
        d.tile = -1;
      }
      shared.desc[r] = d;
      ptx::mbar_arrive(&shared.full[r]);    // release: the record is visible
      if(d.tile < 0) return;
    }
  }

  //////////////////////////////////////////////////////////////////////////////
  // Consumers.

  first_t* first_out = nullptr;
  if constexpr (lbs_fill_values == kind) first_out = out.expanded;
  else first_out = out.ids;
  const int64_t total = (int64_t)count + num_segments;

  struct tile_t { int tile, a0, a1, b0, b1, na, shift; };
  // Tile k of this CTA, from the producer's record. False: no more tiles (or
  // the record never came).
  auto fetch = [&](int k, tile_t& t) -> bool {
    const int r = k % ring;
    bool arrived = ptx::mbar_wait(&shared.full[r], (k / ring) & 1, timeout_ns);
    lbs_fill_desc_t d = shared.desc[r];
    ptx::mbar_arrive(&shared.empty[r]);
    if(!arrived) {
      raise_status(status, (uint32_t)status_copy_timeout);
      d.tile = -1;
    }
    t.tile = d.tile;
    if(d.tile < 0) return false;
    int64_t d0 = (int64_t)d.tile * nv;
    int64_t d1 = d0 + nv < total ? d0 + nv : total;
    int a0 = d.a0, a1 = d.a1;
    a0 = a0 < 0 ? 0 : (a0 > count ? count : a0);
    a1 = a1 < a0 ? a0 : (a1 > count ? count : a1);
    if(a1 - a0 > nv) a1 = a0 + nv;
    int64_t b0 = d0 - a0, b1 = d1 - a1;
    b0 = b0 < 0 ? 0 : (b0 > num_segments ? num_segments : b0);
    b1 = b1 < b0 ? b0 : (b1 > num_segments ? num_segments : b1);
    if(b1 - b0 > nv) b1 = b0 + nv;
    t.a0 = a0; t.a1 = a1; t.b0 = (int)b0; t.b1 = (int)b1; t.na = a1 - a0;
    // Slot of item a0: its position within a 16-byte granule of the output.
    t.shift = (int)(((uintptr_t)first_out / sizeof(first_t) + (uintptr_t)a0) %
      per16);
    return true;
  };
  auto start_of = [&](int j) -> int {
    return j < num_segments ? (int)segments[j] : count;
  };
  // What a thread needs from global memory for a tile: the start it scatters
  // (segment b0 + tid) and the next one, and what describes the segment that
  // is open at the tile's left edge.
  struct wanted_t {
    int p, p_next, open_start;
    second_t open_value, head_value;
  };
  auto request = [&](const tile_t& t, wanted_t& w) {
    const int j = t.b0 + tid;
    w.p = w.p_next = 0;
    w.head_value = second_t();
    if(j < t.b1) {
      w.p = start_of(j);
      if(j + 1 < t.b1) w.p_next = start_of(j + 1);
      if constexpr (lbs_fill_values == kind) w.head_value = out.values[j];
    }
    w.open_start = 0;
    w.open_value = second_t();
    if(t.b0 > 0) {
      if constexpr (lbs_fill_ids_ranks == kind) w.open_start = start_of(t.b0 - 1);
      if constexpr (lbs_fill_values == kind) w.open_value = out.values[t.b0 - 1];
    }
  };

  tile_t cur, next;
  wanted_t cur_w, next_w;
  bool have = fetch(0, cur);
  if(have) request(cur, cur_w);
  for(int k = 0; have; ++k) {
    const bool more = fetch(k + 1, next);
    if(more) request(next, next_w);

    uint32_t* flags = shared.flags[k & 1];
    const int a0 = cur.a0, b0 = cur.b0, b1 = cur.b1, na = cur.na,
      shift = cur.shift;

    // One head bit and one id (and, for values, the segment's value) per
    // distinct start inside the tile; among equal starts the last segment
    // owns the items.
    auto scatter = [&](int j, int p, int p_next, second_t head_value) {
      bool owner = j + 1 >= b1 || p_next != p;
      int w = p - a0;
      if(owner && w >= 0 && w < na) {
        int u = shift + w;
        shared.heads[u] = (uint16_t)(j - b0);
        if constexpr (lbs_fill_values == kind)
          shared.head_values[u] = head_value;
        atomicOr(&flags[u >> 5], 1u << (u & 31));
      }
    };
    if(b0 + tid < b1)
      scatter(b0 + tid, cur_w.p, cur_w.p_next, cur_w.head_value);
    for(int j = b0 + tid + nt; j < b1; j += nt) {    // rare: many starts
      second_t head_value = second_t();
      if constexpr (lbs_fill_values == kind) head_value = out.values[j];
      scatter(j, start_of(j), j + 1 < b1 ? start_of(j + 1) : 0, head_value);
    }
    ptx::named_sync<1, nt>();

    // The other flag buffer served the previous tile, which is done with it.
    {
      uint32_t* other = shared.flags[(k + 1) & 1];
      for(int i = tid; i < flag_words; i += nt) other[i] = 0;
    }
    // Running maximum of (head slot, head id): within the thread, then
    // across the CTA. Both grow together, so one key carries both.
    const int u0 = tid * vt;
    uint32_t bits = __funnelshift_r(flags[u0 >> 5], flags[(u0 >> 5) + 1],
      u0 & 31) & ((1u << vt) - 1);
    int mine = -1;
    if(bits) {
      int u = u0 + 31 - __clz(bits);
      mine = (u << 16) | (int)shared.heads[u];
    }
    int incl = mine;
    #pragma unroll
    for(int delta = 1; delta < 32; delta *= 2) {
      int y = __shfl_up_sync(full, incl, delta);
      if(lane >= delta) incl = max(incl, y);
    }
    int before = __shfl_up_sync(full, incl, 1);
    if(0 == lane) before = -1;
    if(31 == lane) shared.warp_max[warp] = incl;
    // Before this tile's values overwrite the previous tile's, the copy
    // engine must have read those.
    if(0 == tid) ptx::bulk_wait_read<0>();
    ptx::named_sync<1, nt>();
    int key = before;
    for(int w = 0; w < warp; ++w) key = max(key, shared.warp_max[w]);

    // Expansion of the thread's vt slots in registers. At a head slot the
    // segment starts right there, so ranks need no lookup either.
    const int hi = shift + na;
    if(u0 < hi) {
      const int index0 = a0 + u0 - shift;     // item index of slot u0
      int seg = b0 - 1;
      int start = cur_w.open_start;
      second_t value = cur_w.open_value;
      if(key >= 0) {
        seg = b0 + (key & 0xffff);
        start = a0 + (key >> 16) - shift;
        if constexpr (lbs_fill_values == kind)
          value = shared.head_values[key >> 16];
      }
      int id[vt];
      second_t second[vt];
      #pragma unroll
      for(int i = 0; i < vt; ++i) {
        if((bits >> i) & 1) {
          seg = b0 + (int)shared.heads[u0 + i];
          start = index0 + i;
          if constexpr (lbs_fill_values == kind)
            value = shared.head_values[u0 + i];
        }
        id[i] = seg;
        if constexpr (lbs_fill_ids_ranks == kind) second[i] = index0 + i - start;
        if constexpr (lbs_fill_values == kind) second[i] = value;
      }
      if constexpr (lbs_fill_values != kind) {
        #pragma unroll
        for(int i = 0; i < vt; i += 4)
          *reinterpret_cast<int4*>(&shared.ids[u0 + i]) =
            make_int4(id[i], id[i + 1], id[i + 2], id[i + 3]);
      }
      if constexpr (lbs_fill_ids != kind) {
        enum { per_quad = 16 / (int)sizeof(second_t) };
        #pragma unroll
        for(int i = 0; i < vt; i += per_quad) {
          uint4 q;
          memcpy(&q, &second[i], 16);
          *reinterpret_cast<uint4*>(&shared.second[u0 + i]) = q;
        }
      }
    }
    // The copy engine reads what the threads wrote.
    ptx::fence_proxy_async();
    ptx::named_sync<1, nt>();

    // Whole granules go out by bulk copy; slots [shift, g_lo) and [g_hi, hi)
    // by ordinary stores. An array whose granules do not line up with the
    // first array's (a second output pointer of different alignment) is
    // stored by the threads, coalesced.
    if(na) {
      auto put = [&](auto* array, const auto* staged) {
        typedef typename std::remove_pointer<decltype(array)>::type elem_t;
        enum { per = 16 / (int)sizeof(elem_t) };
        auto* dst = array + a0;                 // item a0 + i at dst[i]
        const bool lined_up =
          (int)(((uintptr_t)array / sizeof(elem_t) + (uintptr_t)a0) % per) ==
          shift % per;
        int g_lo = (shift + per - 1) / per * per;
        int g_hi = hi / per * per;
        if(!lined_up || g_hi <= g_lo) { g_lo = hi; g_hi = hi; }
        if(0 == tid && g_hi > g_lo)
          ptx::bulk_store(dst + (g_lo - shift), staged + g_lo,
            (uint32_t)(g_hi - g_lo) * (uint32_t)sizeof(elem_t));
        const int head_end = g_lo < hi ? g_lo : hi;
        for(int u = shift + tid; u < head_end; u += nt)
          dst[u - shift] = staged[u];
        for(int u = g_hi + tid; u < hi; u += nt) dst[u - shift] = staged[u];
      };
      if constexpr (lbs_fill_values == kind) put(out.expanded, shared.second);
      else put(out.ids, shared.ids);
      if constexpr (lbs_fill_ids_ranks == kind) put(out.ranks, shared.second);
      if(0 == tid) ptx::bulk_commit();
    }
    // Ordinary stores of the ragged ends read shared memory too: they must
    // be done before the next tile's expansion, which the barriers of the
    // next tile see to (two lie between here and there).
    cur = next;
    cur_w = next_w;
    have = more;
  }
  // The shared memory must outlive the copy engine's reads.
  if(0 == tid) ptx::bulk_wait_read<0>();
}

inline size_t lbs_partition_bytes(int count, int num_segments, int nv);

// Ints of scratch a fill call needs: a 32-word header (ticket counter, status
// word) followed by the partition table.
template<typename tuning_t>
inline size_t lbs_fill_scratch_ints(int count, int num_segments) {
  return 32 + (size_t)div_up((int64_t)count + num_segments,
    (int64_t)tuning_t::nv) + 1;
}

// Partition + fill kernel on `stream`. `header` (32 words, [0] the ticket
// counter, [1] the status word; cleared by the partitioner) and `partitions`
// (div_up(count + num_segments, tuning_t::nv) + 1 ints) are scratch.
template<typename tuning_t, int kind, typename value_t, typename segments_it>
void lbs_fill_enqueue(lbs_fill_args_t<kind, value_t> out, int count,
  segments_it segments, int num_segments, uint32_t* header, int* partitions,
  cudaStream_t stream, uint64_t timeout_ns) {
  int64_t total = (int64_t)count + num_segments;
  int num_tiles = (int)div_up(total, (int64_t)tuning_t::nv);
  if(!num_tiles) return;
  launch_lbs_partition(segments, count, num_segments, (int64_t)tuning_t::nv,
    num_tiles + 1, partitions, stream, header, 32);
  auto kernel = lbs_fill_k<tuning_t, kind, value_t, segments_it>;
  const int threads = (int)tuning_t::nt + 32;
  const int smem_bytes = (int)sizeof(lbs_fill_smem_t<tuning_t, kind, value_t>);
  // CTAs that fit on the device at once, found once per kernel and device.
  static int resident[64] = { };
  int device = 0;
  throw_on_error(cudaGetDevice(&device));
  int grid = device < 64 ? resident[device] : 0;
  if(!grid) {
    throw_on_error(cudaFuncSetAttribute(kernel,
      cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    int per_sm = 0, sms = 0;
    throw_on_error(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm,
      kernel, threads, smem_bytes));
    throw_on_error(cudaDeviceGetAttribute(&sms,
      cudaDevAttrMultiProcessorCount, device));
    grid = per_sm * sms > 0 ? per_sm * sms : 1;
    if(device < 64) resident[device] = grid;
  }
  if(grid > num_tiles) grid = num_tiles;
  // A programmatic dependent of the partitioner: its CTAs set themselves up
  // while the partitioner's last CTAs run.
  cudaLaunchConfig_t config = { };
  config.gridDim = dim3(grid);
  config.blockDim = dim3(threads);
  config.dynamicSmemBytes = smem_bytes;
  config.stream = stream;
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  throw_on_error(cudaLaunchKernelEx(&config, kernel, out, count, segments,
    num_segments, (const int*)partitions, num_tiles, header, timeout_ns));
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
  detail::throw_on_device_status();
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

namespace detail {

// Checks shared by the entry points that run a fill kernel.
inline bool lbs_fill_sizes(int count, int num_segments) {
  if(count < 0 || num_segments < 0 ||
    (int64_t)count + num_segments > (int64_t)0x7fffffff - 65536)
    throw cuda_exception_t(cudaErrorInvalidValue);
  return 0 != count + num_segments;
}

template<int kind, typename value_t, typename segments_it>
void lbs_fill(lbs_fill_args_t<kind, value_t> out, int count,
  segments_it segments, int num_segments, context_t& context) {
  typedef typename lbs_fill_tuning_for<kind, (int)sizeof(value_t)>::type
    tuning_t;
  throw_on_device_status();
  if(!lbs_fill_sizes(count, num_segments)) return;
  mem_t<int> scratch(lbs_fill_scratch_ints<tuning_t>(count, num_segments),
    context);
  lbs_fill_enqueue<tuning_t>(out, count, segments, num_segments,
    (uint32_t*)scratch.data(), scratch.data() + 32, context.stream(),
    (uint64_t)2000000000ull);
}

} // namespace detail

// output[index] = segment of item index.
template<typename launch_arg_t = empty_t, typename segments_it,
  typename output_it>
void load_balance_search(int count, segments_it segments, int num_segments,
  output_it output, context_t& context) {
  if constexpr (std::is_same<launch_arg_t, empty_t>::value &&
    std::is_same<output_it, int*>::value) {
    // A plain int array: the tile's ids leave through the copy engine.
    detail::lbs_fill_args_t<detail::lbs_fill_ids, int> out = { };
    out.ids = output;
    detail::lbs_fill(out, count, segments, num_segments, context);
  } else {
    transform_lbs<launch_arg_t>([=]MGPU_DEVICE(int index, int seg, int rank) {
      output[index] = seg;
    }, count, segments, num_segments, context);
  }
}

// output[index] = input[segment of item index].
template<typename launch_arg_t = empty_t, typename input_it,
  typename segments_it, typename output_it>
void interval_expand(input_it input, int count, segments_it segments,
  int num_segments, output_it output, context_t& context) {
  typedef typename std::iterator_traits<input_it>::value_type type_t;
  constexpr bool arrays = std::is_same<launch_arg_t, empty_t>::value &&
    std::is_pointer<input_it>::value &&
    std::is_same<output_it, type_t*>::value &&
    std::is_trivially_copyable<type_t>::value &&
    (4 == sizeof(type_t) || 8 == sizeof(type_t)) &&
    alignof(type_t) == sizeof(type_t);
  if constexpr (arrays) {
    detail::lbs_fill_args_t<detail::lbs_fill_values, type_t> out = { };
    out.values = input;
    out.expanded = output;
    detail::lbs_fill(out, count, segments, num_segments, context);
  } else {
    transform_lbs<launch_arg_t>(
      []MGPU_DEVICE(int index, int seg, int rank, tuple<type_t> desc,
        output_it output) {
        output[index] = get<0>(desc);
      }, count, segments, num_segments, make_tuple(input), context, output);
  }
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
