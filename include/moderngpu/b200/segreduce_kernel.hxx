// Single-pass load-balanced segmented reduction for sm_100a.
//
// Replaces the reference's tile kernel plus recursive fix-up
// (src/moderngpu/kernel_segreduce.hxx:17-100 cta_segreduce_t, :105-185
// segreduce_fixup, :219-263 k_reduce) and its CTA segmented scan
// (src/moderngpu/cta_segscan.hxx:16-104) with one persistent kernel.
//
// Work decomposition. Items and segment starts are merged (a start sorts
// before the item with the same index) and cut into tiles of `nv` merged
// elements by the partitioner, so a tile never holds more than nv items nor
// more than nv segment starts. Tile t owns items [a0, a1) and segment starts
// [b0, b1). The tile that holds the START of segment j is the one that writes
// output[j-1]: every item of segment j-1 lies in that tile or in earlier
// ones. The last tile also writes the last segment.
//
// A CTA is nt consumer threads plus one producer warp and one carry warp.
//  * Producer (one lane): takes the next tile from a global ticket counter,
//    reads its two partition values, and issues bulk asynchronous copies of
//    the tile's item window and segment-start window from HBM into one of
//    `stages` shared-memory buffers, completion counted on an mbarrier.
//    Several tiles are in flight per CTA at any time.
//  * Consumers, per tile:
//      1. scatter a head-flag bit for every segment start of the tile into a
//         shared bitmask; write `init` for empty segments;
//      2. each thread folds vt consecutive items taken from shared memory
//         with 128-bit loads, restarting at head flags;
//      3. warp-shuffle segmented scan of the per-thread partials, one
//         shared-memory hop across warps;
//      4. second sweep over the registers: values at segment ends are stored
//         in place; a second pass over the segment starts copies them to
//         output[] (coalesced);
//      5. two threads leave a small record for the CTA's carry warps, which
//         publish the value of the segment open at the tile's right edge in
//         the tile-status array and finish the one output that needs items
//         of earlier tiles by looking back through that array
//         (tile_state.hxx).
//
// Results: each segment is folded strictly left to right within a thread and
// combined as op(earlier, later) everywhere else; `init` is written for empty
// segments and never folded into a non-empty one (reference behaviour,
// tests/test_segreduce.cu:40-49). Integer results are exact; floating-point
// sums differ from a serial sum only by association.
#pragma once
#include "partition.hxx"
#include "tile_state.hxx"

#ifdef __CUDACC__

BEGIN_MGPU_NAMESPACE

// Tile shape: nt consumer threads x vt items per thread, `stages` buffers per
// CTA, at least `occ` CTAs per SM.
template<int nt_, int vt_, int stages_, int occ_>
struct segreduce_tuning_t {
  enum { nt = nt_, vt = vt_, stages = stages_, occ = occ_,
    nv = nt_ * vt_ - 8 };
  static_assert(nt_ % 32 == 0 && nt_ >= 128 && vt_ >= 4 && vt_ <= 31,
    "unsupported tile");
};

namespace detail {

// Blackwell defaults, chosen from measurements on B200: vt is picked so that
// a thread's run of vt values starts on a 16-byte boundary and the 128-bit
// shared-memory loads of a quarter warp hit distinct banks.
template<typename type_t, int size = (int)sizeof(type_t)>
struct segreduce_default_tuning { typedef segreduce_tuning_t<128, 4, 2, 4> type; };
template<typename type_t>
struct segreduce_default_tuning<type_t, 1> { typedef segreduce_tuning_t<256, 16, 3, 3> type; };
template<typename type_t>
struct segreduce_default_tuning<type_t, 2> { typedef segreduce_tuning_t<256, 16, 3, 3> type; };
template<typename type_t>
struct segreduce_default_tuning<type_t, 4> { typedef segreduce_tuning_t<256, 28, 2, 3> type; };
template<typename type_t>
struct segreduce_default_tuning<type_t, 8> { typedef segreduce_tuning_t<256, 26, 2, 2> type; };
template<typename type_t>
struct segreduce_default_tuning<type_t, 16> { typedef segreduce_tuning_t<256, 5, 3, 3> type; };

// spmv stages 4 more bytes per item, and what bounds it is the number of
// gathers from x in flight, i.e. resident warps, not tile size: ncu on
// 2^24 rows x 16 non-zeros showed 256 x 20 tiles (2 CTAs per SM) at 31 % of
// the warp slots, 58 % of them waiting for a load, DRAM at a third of its
// bandwidth (1.87 ms; the reference's kernel, at 96 % of the warp slots:
// 1.62 ms). Measured on the same matrix: 256 x 20 x 2 stages, 2 CTAs: 1.86 ms;
// 256 x 12, 3 CTAs: 1.39; 384 x 12, 2 CTAs: 1.45; 256 x 8, 4 CTAs: 1.47;
// 256 x 12, 4 CTAs: 3.6 (the streams of so many CTAs push x out of the L2).
// With one stage buffer per CTA four CTAs do fit beside x: 256 x 12 x 1 stage
// at 4 CTAs 1.363 ms against 1.388 for 2 stages at 3 (same run); at 5 or 6:
// 2.76 - 2.79; 256 x 20 x 1 at 3 / 4: 1.47 / 1.86; 128 x 12 x 2 at 6: 1.87.
template<typename type_t, int size = (int)sizeof(type_t)>
struct spmv_default_tuning { typedef segreduce_tuning_t<256, 12, 1, 4> type; };
template<typename type_t>
struct spmv_default_tuning<type_t, 8> { typedef segreduce_tuning_t<256, 14, 2, 2> type; };

// lbs_segreduce keeps 4 more bytes per item in shared memory as well, and its
// consumers compute the values themselves (search + functor), so nothing but
// the few segment starts is staged ahead: one stage buffer and many small
// CTAs hide the functor's loads and the extra barriers best. What its time
// follows is the number of trips to memory a tile makes, i.e. how its whole
// rounds split into straight-line batches (see functor_batch). Measured on
// 2^28 fp32 items in 2^23 segments, functor values[index] * weight[seg]
// (per-segment tuples in the tile's slots, 32-bit segment ids per item):
// 128 x 28 x 1 stage at 6 CTAs per SM 0.61 ms; 128 x 20 at 8: 0.70; 192 x 28 at 4: 0.63; 256 x 28 at 3: 0.64;
// 256 x 24 at 4: 0.74; 384 x 20 at 3: 0.71; 256 x 28 x 2 stages at 3: 1.40.
// Segments of 16 / 100 items on average: 0.67 / 0.58 ms. fp64 (2^27 items):
// 128 x 18 at 5: 0.54 ms; 128 x 28 at 3: 0.61; 256 x 26 x 2 stages at 2: 0.90.
// With 16-bit ids per item (relative to the segment open at the tile's left
// edge) a CTA's shared memory drops from 34.7 to 27.7 KB and more CTAs fit:
// 128 x 28 at 6 / 7 / 8 CTAs per SM 0.558 / 0.524 / 0.491 ms (0.561 with
// 32-bit ids at 6); 128 x 30 at 8: 0.539; 128 x 20 at 8: 0.625; segments of
// 12 items on average 0.749 -> 0.636 ms. fp64: 128 x 18 at 5 / 6 / 7: 0.512 /
// 0.448 / 0.513 ms (7: spills at 40 registers); 128 x 14 at 8: 0.503.
// ncu (128 x 20 at 8): 37 thread instructions per item (the plain reduction:
// 13), 18 warps waiting on a global load per instruction issued, DRAM at a
// fifth of its bandwidth. Tried and measured no better: two batches in
// flight per thread (the next batch's loads issued before this batch's
// stores: 0.63 against 0.61 ms), batches of 12 or 20 rounds at 40 registers
// (0.83 / 1.24 ms), the tile's last rounds as a predicated batch (1.2 ms),
// a software pipeline that keeps the next tile's values in registers while
// this tile is folded (2 CTAs of 256 x 20: 1.2 ms), and a group of evaluator
// warps of its own (as many threads as consumers) that searches and
// evaluates tile k + 1 while the consumers fold tile k (0.73 - 1.05 ms over
// six tile shapes: the search and the functor are two thirds of the work,
// and taking the fold away from the threads that wait on the loads only
// halves the number of threads that have loads in flight).
template<typename type_t, int size = (int)sizeof(type_t)>
struct lbs_segreduce_default_tuning {
  typedef typename segreduce_default_tuning<type_t>::type type;
};
template<typename type_t>
struct lbs_segreduce_default_tuning<type_t, 4> { typedef segreduce_tuning_t<128, 28, 1, 8> type; };
template<typename type_t>
struct lbs_segreduce_default_tuning<type_t, 8> { typedef segreduce_tuning_t<128, 18, 1, 6> type; };

////////////////////////////////////////////////////////////////////////////////
// Value sources.

// Contiguous array of type_t in global memory: staged by bulk copies.
template<typename type_t>
struct array_source_t {
  enum { bulk = 1 };
  const type_t* data;
  MGPU_DEVICE type_t load(int index) const { return data[index]; }
};

// CSR spmv: the value of item i is matrix[i] * x[columns[i]]. matrix and
// columns are staged by bulk copies like an array source; the consumers then
// gather x and overwrite the staged matrix values with the products.
template<typename type_t>
struct spmv_source_t {
  enum { bulk = 2 };
  const type_t* data;       // matrix values
  const int* columns;
  const type_t* x;
  MGPU_DEVICE type_t load(int index) const {
    return data[index] * __ldg(x + columns[index]);
  }
};

// lbs_segreduce: the value of item i is f(i, seg, rank, cached..., args...)
// where seg and rank come from a load-balancing search over the tile. The
// consumers work the segment of every item out in shared memory (head ids +
// running maximum, as the load-balancing kernels do) and evaluate f in
// striped order; nothing is staged for the items themselves.
template<typename func_t, typename pointers_t, typename type_t,
  typename... args_t>
struct lbs_source_t {
  enum { bulk = 3 };
  func_t f;
  pointers_t caching;
  tuple<args_t...> args;

  // What the caching iterators yield for one segment. A tile keeps these in
  // shared memory, loaded once per segment, when it has no more segments than
  // consumer threads and the tuple is small (the reference stages them the
  // same way, cta_load_balance.hxx:216-244); the functor's per-item gather
  // from global memory becomes a shared-memory read.
  typedef tuple_iterator_value_t<pointers_t> cached_t;
  enum {
    cached_bytes = (tuple_size<pointers_t>::value > 0 &&
      sizeof(cached_t) <= 16 &&
      std::is_trivially_copyable<cached_t>::value) ?
      (int)sizeof(cached_t) : 0
  };

  template<size_t... idx>
  MGPU_DEVICE type_t call(int index, int seg, int rank,
    const cached_t& cached, index_sequence<idx...>) const {
    return (type_t)f(index, seg, rank, cached, get<idx>(args)...);
  }
  MGPU_DEVICE cached_t fetch(int seg) const {
    return mgpu::load(caching, seg);
  }
  MGPU_DEVICE type_t eval_with(int index, int seg, int rank,
    const cached_t& cached) const {
    return call(index, seg, rank, cached,
      make_index_sequence<sizeof...(args_t)>());
  }
  MGPU_DEVICE type_t eval(int index, int seg, int rank) const {
    return eval_with(index, seg, rank, fetch(seg));
  }
};

// Bytes per consumer thread that a source wants in every stage buffer on top
// of the values (the per-segment tuples of lbs_source_t).
template<typename source_t, typename = void>
struct source_slot_bytes { enum { value = 0 }; };
template<typename source_t>
struct source_slot_bytes<source_t,
  typename std::enable_if<(source_t::cached_bytes >= 0)>::type> {
  enum { value = source_t::cached_bytes };
};

// Anything with operator[]: evaluated by the consumer threads.
template<typename input_it, typename type_t>
struct iterator_source_t {
  enum { bulk = 0 };
  input_it input;
  MGPU_DEVICE type_t load(int index) const { return (type_t)input[index]; }
};

template<typename input_it, typename type_t>
struct source_for {
  typedef typename std::iterator_traits<input_it>::value_type value_t;
  enum { bulk = std::is_pointer<input_it>::value &&
    std::is_same<typename std::remove_cv<value_t>::type, type_t>::value &&
    std::is_arithmetic<type_t>::value &&
    (sizeof(type_t) == 4 || sizeof(type_t) == 8) };
  typedef typename std::conditional<bulk, array_source_t<type_t>,
    iterator_source_t<input_it, type_t> >::type type;
};

template<typename segments_it>
struct segments_are_int_array {
  typedef typename std::iterator_traits<segments_it>::value_type value_t;
  enum { value = std::is_pointer<segments_it>::value &&
    std::is_same<typename std::remove_cv<value_t>::type, int>::value };
};

////////////////////////////////////////////////////////////////////////////////

// What the producer tells the consumers about a staged tile. Positions
// ("w") index the stage buffer's value array; item a0 sits at w == lo.
struct tile_desc_t {
  int tile;             // -1: no more tiles
  int a0, a1, b0, b1;   // items [a0, a1), segment starts [b0, b1)
  int lo;               // position of item a0
  int src_lo, src_hi;   // positions delivered by the bulk copy
  int ob, oe;           // segment indices whose offsets are staged
  int offs_byte;        // byte offset of the staged offsets in the stage
  int cols_byte;        // spmv: byte offset of the staged column indices,
  int cols_lo;          //   position of item a0 among them,
  int cols_src_lo, cols_src_hi;   // positions delivered by the bulk copy
  int pad;
};

// The call's LAST output is stored by the carry warp of the last tile, not by
// the consumers (which keeps the end of the array out of their loop over the
// tile's segment starts: 1.3 us of 196 on 2^28 items), and passes through
// finish_t first: finish(value) returns what is stored. The multi-GPU layer
// folds the following shards' boundary partials into a shard's last output
// this way, instead of in a launch of its own. Called once per launch, by one
// thread.
struct no_finish_t {
  template<typename type_t>
  MGPU_DEVICE type_t operator()(type_t value) const { return value; }
};

template<typename type_t, typename source_t, typename segments_it,
  typename output_it, typename op_t, typename finish_t = no_finish_t>
struct segreduce_args_t {
  source_t source;
  segments_it segments;
  output_it output;
  op_t op;
  type_t init;
  int count, num_segments, num_tiles;
  const int* partitions;
  uint32_t* header;       // [0] ticket counter, [1] status
  void* tile_state;
  uint64_t timeout_ns;    // bound on every device-side wait
  finish_t finish;
};

// What a finished tile leaves for the CTA's carry warp: enough to finish the
// one output that may depend on earlier tiles (the segment open at the tile's
// left edge) and to publish the inclusive value of a tile without segment
// starts. Two consumer threads of different warps fill it, so that no warp
// carries a long serial tail; the decisions are taken by the carry warp.
template<typename type_t>
struct tile_edge_t {
  int tile;
  int a0, na;        // first item and number of items of the tile
  int b0, nb;        // first segment start and number of starts of the tile
  int has_first;     // the end marker of segment b0 - 1 lies in this tile
  int prev0, p0;     // start offsets of segments b0 - 1 and b0
  int closed;        // a segment start sits exactly on the tile's right edge
  int pad;
  alignas(8) char lead[sizeof(type_t)];   // fold of items [a0, p0) of the tile
  alignas(8) char tail[sizeof(type_t)];   // fold of the run ending at a1 - 1
};

// Carry warps per CTA; tile k of a CTA goes to warp k % segreduce_carry_warps.
enum { segreduce_carry_warps = 1 };

template<typename tuning_t, typename type_t, int source_kind = 1,
  int slot_bytes_ = 0>
struct segreduce_smem_t {
  enum {
    nt = tuning_t::nt, vt = tuning_t::vt, stages = tuning_t::stages,
    nv = tuning_t::nv, warps = nt / 32,
    flag_words = nt * vt / 32 + 2,
    elem = (int)sizeof(type_t),
    slot_bytes = slot_bytes_,
    wide = elem > 4 ? elem : 4,
    // spmv stages one int32 column index per item on top of everything else.
    // lbs_segreduce keeps one int32 segment id per item there instead.
    // (spmv: an int32 column index per item; lbs sources: a 16-bit segment id
    // per item, relative to the segment open at the tile's left edge.)
    cols_bytes = 2 == source_kind ? nv * 4 + 48 :
      (3 == source_kind ? nv * 2 + 48 : 0),
    // Slots in front of the values that shifted run ends may use (see the
    // fold): nt - 1 of them, arithmetic types only.
    pad_bytes = std::is_arithmetic<type_t>::value ?
      (nt * elem + 127) / 128 * 128 : 0,
    // Slots at the end of the stage for lbs_source_t's per-segment tuples:
    // 16 bytes per consumer thread.
    slots_offset = (nv * wide + 8 * elem + 64 + cols_bytes + 15) / 16 * 16,
    slots = nt * (slot_bytes_ <= 4 ? 4 : (slot_bytes_ <= 8 ? 2 : 1)),
    stage_bytes = pad_bytes +
      (slots_offset + slots * slot_bytes + 127) / 128 * 128,
    ring = 32
  };
  struct fixed_t {
    uint64_t full[stages];
    uint64_t empty[stages];
    uint64_t edge_full[ring];   // consumers -> carry warp
    uint64_t edge_free[ring];   // carry warp -> consumers
    tile_desc_t desc[stages];
    tile_edge_t<type_t> edge[ring];
    uint32_t flags[2][flag_words];
    int warp_head[warps];
    alignas(16) char warp_agg[warps * elem];
  };
  enum {
    fixed_bytes = ((int)sizeof(fixed_t) + 127) / 128 * 128,
    total_bytes = fixed_bytes + stages * stage_bytes
  };
};

// Functor values are evaluated round by round (one item per consumer thread
// and round), whole rounds in straight-line batches so that a thread's loads
// are in flight together: every batch is one trip to memory for the CTA, and
// the trips per tile are what a functor source's time follows (measured:
// 128 x 28 tiles, usually 27 whole rounds: batches of 7 / 8 / 9 / 10 rounds,
// i.e. 9 / 6 / 3 / 9 trips: 0.79 / 0.69 / 0.64 / 0.81 ms on 2^28 items). So
// the batch divides vt - 1 (a tile of nt x vt merged elements with fewer
// segment starts than threads has vt - 1 whole rounds) where 9 does, and
// what is left over goes in batches of 4 and 2 before single rounds.
template<int vt>
struct functor_batch {
  enum { value = vt < 8 ? vt : ((vt - 1) % 9 == 0 ? 9 : 8) };
};
template<int batch, typename run_t>
MGPU_DEVICE void for_whole_rounds(int& round, int full_rounds, run_t run) {
  while(round + batch <= full_rounds)
    run(std::integral_constant<int, batch>());
  if constexpr (batch > 4) {
    while(round + 4 <= full_rounds)
      run(std::integral_constant<int, 4>());
  }
  if constexpr (batch > 2) {
    if(round + 2 <= full_rounds)
      run(std::integral_constant<int, 2>());
  }
}

// vt consecutive values from shared memory into registers.
template<int vt, typename type_t>
MGPU_DEVICE void load_chunk(const type_t* src, type_t (&v)[vt]) {
  if constexpr ((vt * sizeof(type_t)) % 16 == 0 &&
    std::is_trivially_copyable<type_t>::value) {
    enum { quads = vt * sizeof(type_t) / 16 };
    uint4 q[quads];
    const uint4* p = reinterpret_cast<const uint4*>(src);
    #pragma unroll
    for(int i = 0; i < quads; ++i) q[i] = p[i];
    memcpy(v, q, sizeof(q));
  } else {
    #pragma unroll
    for(int i = 0; i < vt; ++i) v[i] = src[i];
  }
}

template<typename tuning_t, typename type_t, typename source_t,
  typename segments_it, typename output_it, typename op_t,
  typename finish_t = no_finish_t>
__global__ void __launch_bounds__(tuning_t::nt + 32 + 32 * segreduce_carry_warps,
  tuning_t::occ)
segreduce_k(const segreduce_args_t<type_t, source_t, segments_it, output_it,
  op_t, finish_t> args) {

  typedef segreduce_smem_t<tuning_t, type_t, source_t::bulk,
    source_slot_bytes<source_t>::value> layout_t;
  typedef typename layout_t::fixed_t fixed_t;
  enum { nt = tuning_t::nt, vt = tuning_t::vt, stages = tuning_t::stages,
    nv = tuning_t::nv, warps = nt / 32, flag_words = layout_t::flag_words,
    elem = layout_t::elem, stage_bytes = layout_t::stage_bytes,
    pad_bytes = layout_t::pad_bytes, ring = layout_t::ring,
    src_bulk = source_t::bulk,
    seg_bulk = segments_are_int_array<segments_it>::value };

  extern __shared__ __align__(128) char smem_raw[];
  fixed_t& fixed = *reinterpret_cast<fixed_t*>(smem_raw);
  char* stage_base = smem_raw + layout_t::fixed_bytes;

  const int tid = (int)threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int count = args.count;
  const int num_segments = args.num_segments;
  const int num_tiles = args.num_tiles;

  if(0 == tid) {
    for(int s = 0; s < stages; ++s) {
      ptx::mbar_init(&fixed.full[s], 1);
      ptx::mbar_init(&fixed.empty[s], nt);
      fixed.desc[s].tile = -1;
    }
    for(int r = 0; r < ring; ++r) {
      ptx::mbar_init(&fixed.edge_full[r], 2);
      ptx::mbar_init(&fixed.edge_free[r], 1);
    }
    ptx::fence_proxy_async();
  }
  for(int i = tid; i < 2 * flag_words; i += nt + 32 + 32 * segreduce_carry_warps)
    (&fixed.flags[0][0])[i] = 0;
  __syncthreads();
  // Everything above ran while the partitioner was still at work; what
  // follows reads its output.
  ptx::grid_dependency_wait();

  //////////////////////////////////////////////////////////////////////////////
  // Producer warp: tickets, partition lookups, bulk copies.

  if(warp == warps) {
    if(lane) return;
    const int64_t total = (int64_t)count + num_segments;
    // Items (and spmv's matrix and column arrays) are read exactly once.
    const uint64_t stream_policy = ptx::l2_policy_evict_first();
    // The next ticket and its two partition values are fetched one
    // iteration ahead, so their latency hides behind the wait for a free
    // stage buffer.
    int next_tile = (int)atomicAdd(args.header, 1u);
    int next_a0 = 0, next_a1 = 0;
    if(next_tile < num_tiles) {
      next_a0 = args.partitions[next_tile];
      next_a1 = args.partitions[next_tile + 1];
    }
    for(int it = 0; ; ++it) {
      int s = it % stages;
      int use = it / stages;
      if(use > 0 &&
        !ptx::mbar_wait(&fixed.empty[s], (use - 1) & 1, args.timeout_ns))
        raise_status(args.header + 1, (uint32_t)status_copy_timeout);
      // The consumers wrote into this stage with ordinary stores; order those
      // (observed through the barrier) before the bulk copy's writes. Doing
      // it here rather than in every consumer keeps their pending global
      // stores out of the stage's release.
      ptx::fence_proxy_async();

      tile_desc_t d;
      d.tile = next_tile;
      if(d.tile >= num_tiles) {
        fixed.desc[s].tile = -1;
        ptx::mbar_arrive(&fixed.full[s]);
        break;
      }
      d.a0 = next_a0;
      d.a1 = next_a1;
      int64_t d0 = (int64_t)d.tile * nv;
      int64_t d1 = d0 + nv < total ? d0 + nv : total;
      // No-ops for valid input; offsets that are not sorted or exceed count
      // give wrong results but must never index outside the arrays.
      d.a0 = d.a0 < 0 ? 0 : (d.a0 > count ? count : d.a0);
      d.a1 = d.a1 < d.a0 ? d.a0 : (d.a1 > count ? count : d.a1);
      if(d.a1 - d.a0 > nv) d.a1 = d.a0 + nv;
      int64_t b0 = d0 - d.a0, b1 = d1 - d.a1;
      b0 = b0 < 0 ? 0 : (b0 > num_segments ? num_segments : b0);
      b1 = b1 < b0 ? b0 : (b1 > num_segments ? num_segments : b1);
      if(b1 - b0 > nv) b1 = b0 + nv;
      d.b0 = (int)b0;
      d.b1 = (int)b1;
      d.pad = 0;
      char* stage = stage_base + s * stage_bytes + pad_bytes;
      int na = d.a1 - d.a0;

      // Item window: whole 16-byte granules of the input array.
      uint32_t item_bytes = 0;
      const char* item_src = nullptr;
      char* item_dst = nullptr;
      int items_end;
      if constexpr (1 == src_bulk || 2 == src_bulk) {
        enum { per16 = 16 / elem };
        const type_t* data = args.source.data;
        int mis = (int)(((uintptr_t)data / elem) % per16);
        int64_t u0 = (int64_t)d.a0 + mis;
        int64_t ubase = u0 / per16 * per16;
        d.lo = (int)(u0 - ubase);
        int64_t inner_lo = mis ? per16 : 0;
        int64_t inner_hi = ((int64_t)count + mis) / per16 * per16;
        int64_t c_lo = ubase > inner_lo ? ubase : inner_lo;
        int64_t c_hi = ((int64_t)d.a1 + mis + per16 - 1) / per16 * per16;
        if(c_hi > inner_hi) c_hi = inner_hi;
        d.src_lo = d.src_hi = 0;
        if(na > 0 && c_hi > c_lo) {
          item_bytes = (uint32_t)((c_hi - c_lo) * elem);
          item_src = (const char*)(data + (c_lo - mis));
          item_dst = stage + (c_lo - ubase) * elem;
          d.src_lo = (int)(c_lo - ubase);
          d.src_hi = (int)(c_hi - ubase);
        }
        items_end = (d.lo + na + per16 - 1) / per16 * per16;
      } else {
        d.lo = 0;
        d.src_lo = 0;
        d.src_hi = na;
        items_end = na;
      }
      d.offs_byte = (items_end * elem + 15) / 16 * 16;

      // Segment-start window [b0 - 1, b1), again whole granules.
      int jlo = d.b0 > 0 ? d.b0 - 1 : 0;
      int jhi = d.b1;
      uint32_t offs_bytes = 0;
      const char* offs_src = nullptr;
      if constexpr (seg_bulk) {
        const int* seg = args.segments;
        int mis = (int)(((uintptr_t)seg / 4) % 4);
        int64_t inner_lo = mis ? 4 : 0;
        int64_t inner_hi = ((int64_t)num_segments + mis) / 4 * 4;
        int64_t c_lo = ((int64_t)jlo + mis) / 4 * 4;
        if(c_lo < inner_lo) c_lo = inner_lo;
        int64_t c_hi = ((int64_t)jhi + mis + 3) / 4 * 4;
        if(c_hi > inner_hi) c_hi = inner_hi;
        d.ob = d.oe = 0;
        if(jhi > jlo && c_hi > c_lo) {
          offs_bytes = (uint32_t)((c_hi - c_lo) * 4);
          offs_src = (const char*)(seg + (c_lo - mis));
          d.ob = (int)(c_lo - mis);
          d.oe = (int)(c_hi - mis);
        }
      } else {
        d.ob = jlo;
        d.oe = jhi;
      }

      // spmv: the tile's column indices, whole granules of columns[].
      uint32_t cols_bytes = 0;
      const char* cols_src = nullptr;
      char* cols_dst = nullptr;
      d.cols_byte = d.cols_lo = d.cols_src_lo = d.cols_src_hi = 0;
      if constexpr (3 == src_bulk) {
        int offs_count = (jhi > jlo ? jhi - jlo : 0) + 8;
        d.cols_byte = (d.offs_byte + offs_count * 4 + 15) / 16 * 16;
      }
      if constexpr (2 == src_bulk) {
        const int* cols = args.source.columns;
        int mis = (int)(((uintptr_t)cols / 4) % 4);
        int64_t u0 = (int64_t)d.a0 + mis;
        int64_t ubase = u0 / 4 * 4;
        d.cols_lo = (int)(u0 - ubase);
        int64_t inner_lo = mis ? 4 : 0;
        int64_t inner_hi = ((int64_t)count + mis) / 4 * 4;
        int64_t c_lo = ubase > inner_lo ? ubase : inner_lo;
        int64_t c_hi = ((int64_t)d.a1 + mis + 3) / 4 * 4;
        if(c_hi > inner_hi) c_hi = inner_hi;
        int offs_count = (jhi > jlo ? jhi - jlo : 0) + 8;
        d.cols_byte = (d.offs_byte + offs_count * 4 + 15) / 16 * 16;
        if(na > 0 && c_hi > c_lo) {
          cols_bytes = (uint32_t)((c_hi - c_lo) * 4);
          cols_src = (const char*)(cols + (c_lo - mis));
          cols_dst = stage + d.cols_byte + (c_lo - ubase) * 4;
          d.cols_src_lo = (int)(c_lo - ubase);
          d.cols_src_hi = (int)(c_hi - ubase);
        }
      }

      fixed.desc[s] = d;
      if(item_bytes + offs_bytes + cols_bytes) {
        ptx::mbar_arrive_expect_tx(&fixed.full[s],
          item_bytes + offs_bytes + cols_bytes);
        if(cols_bytes)
          ptx::bulk_load_hint(cols_dst, cols_src, cols_bytes, &fixed.full[s],
            stream_policy);
        if(item_bytes)
          ptx::bulk_load_hint(item_dst, item_src, item_bytes, &fixed.full[s],
            stream_policy);
        if(offs_bytes)
          ptx::bulk_load(stage + d.offs_byte, offs_src, offs_bytes,
            &fixed.full[s]);
      } else {
        ptx::mbar_arrive(&fixed.full[s]);
      }

      next_tile = (int)atomicAdd(args.header, 1u);
      if(next_tile < num_tiles) {
        next_a0 = args.partitions[next_tile];
        next_a1 = args.partitions[next_tile + 1];
      }
    }
    return;
  }

  op_t op = args.op;
  const type_t init = args.init;
  tile_state_t<type_t> state;
  state.bind(args.tile_state, num_tiles);

  //////////////////////////////////////////////////////////////////////////////
  // Carry warp: finishes, off the consumers' critical path, whatever needs
  // values of earlier tiles. One record per tile arrives through a small
  // ring; a record whose tile is -1 ends the loop.

  if(warp > warps) {
    for(int n = warp - warps - 1; ; n += segreduce_carry_warps) {
      int r = n % ring;
      if(!ptx::mbar_wait(&fixed.edge_full[r], (n / ring) & 1,
        args.timeout_ns)) {
        // Never act on a record that was not delivered.
        raise_status(args.header + 1, (uint32_t)status_copy_timeout);
        break;
      }
      const tile_edge_t<type_t> e = fixed.edge[r];
      __syncwarp();
      if(0 == lane) ptx::mbar_arrive(&fixed.edge_free[r]);
      if(e.tile < 0) break;

      type_t lead, tail;
      memcpy(&lead, e.lead, sizeof(type_t));
      memcpy(&tail, e.tail, sizeof(type_t));
      // Segment b0 - 1 is written here unless it is empty (then the
      // consumers wrote `init`); it needs earlier tiles when it began
      // before a0. A tile without starts also owes its inclusive value.
      const bool need_out = e.has_first && e.prev0 != e.p0;
      const bool has_lead = e.p0 > e.a0 && e.na > 0;
      const bool need_left = need_out && e.prev0 < e.a0 && e.tile > 0;
      const bool partial = 0 == e.nb && e.tile > 0;
      // First of all tell later tiles what this tile contributes to the
      // segment open at its right edge. Publishing from here keeps the
      // store's completion off the consumers' barriers.
      if(0 == lane) {
        if(e.closed) state.publish(e.tile, tile_closed);
        else state.publish(e.tile, partial ? tile_partial : tile_inclusive,
          tail);
      }
      bool have = false;
      type_t carry = init;
      if(need_left || partial)
        have = lookback(state, e.tile, op, carry, args.timeout_ns,
          args.header + 1);
      if(0 == lane) {
        if(partial)
          state.publish(e.tile, tile_inclusive,
            have ? op(carry, tail) : tail);
        if(need_out && e.b0 <= num_segments) {
          type_t result = lead;
          if(need_left && have) result = has_lead ? op(carry, lead) : carry;
          if(e.b0 == num_segments) result = args.finish(result);
          args.output[e.b0 - 1] = result;
        }
        // The last segment starts inside the last tile: its value is the
        // tile's last run (or `init` when a start sits on the array's end).
        if(e.tile == num_tiles - 1 && e.nb > 0 && num_segments > 0)
          args.output[num_segments - 1] =
            args.finish(e.closed ? init : tail);
      }
    }
    return;
  }

  //////////////////////////////////////////////////////////////////////////////
  // Consumers.

  type_t* warp_agg = reinterpret_cast<type_t*>(fixed.warp_agg);
  const unsigned full_mask = 0xffffffffu;
  const uint32_t vt_mask = (1u << vt) - 1;
  const int edge_thread_a = nt / 2, edge_thread_b = nt / 2 + 32;
  // One tile. The body exists in two forms, chosen once per CTA (below): the
  // plain one keeps every run end in place; the shifting one (staged arrays
  // of arithmetic values only) takes the values into registers early and
  // keeps run ends in shifted slots. Returns false when there are no more
  // tiles.
  auto consume_tile = [&](auto shifting_tag, const int it) -> bool {
    constexpr bool shifting = decltype(shifting_tag)::value;
    int s = it % stages;
    if(!ptx::mbar_wait(&fixed.full[s], (it / stages) & 1, args.timeout_ns))
      raise_status(args.header + 1, (uint32_t)status_copy_timeout);
    const tile_desc_t d = fixed.desc[s];
    if(d.tile < 0) return false;

    char* stage = stage_base + s * stage_bytes + pad_bytes;
    type_t* vals = reinterpret_cast<type_t*>(stage);
    int* offs = reinterpret_cast<int*>(stage + d.offs_byte);
    uint32_t* flags = fixed.flags[it & 1];
    uint32_t* flags_next = fixed.flags[(it + 1) & 1];

    const int a0 = d.a0, a1 = d.a1, b0 = d.b0, b1 = d.b1, lo = d.lo;
    const int na = a1 - a0;
    const int nb = b1 - b0;
    const int hi = lo + na;
    const bool is_last = d.tile == num_tiles - 1;
    const int jend = b1 + (is_last ? 1 : 0);
    // Outputs the consumers look up: the call's last output (whose end marker
    // is the end of the array) is the carry warp's.
    const int jend_lookup = b1;
    const int ob = d.ob, oe = d.oe;

    // Start offset of segment j; j == num_segments is the end of the array.
    auto seg_start = [&](int j) -> int {
      if(j >= num_segments) return count;
      if(j >= ob && j < oe) return offs[j - ob];
      return (int)args.segments[j];
    };
    // Same, when every offset this tile touches is staged (the usual case).
    const int* offs_by_seg = offs - ob;
    auto seg_start_staged = [&](int j) -> int { return offs_by_seg[j]; };
    const bool all_staged = !is_last && (b0 > 0 ? b0 - 1 : 0) >= ob &&
      b1 <= oe;

    // Positions whose value is already in the stage buffer.
    int src_lo = d.src_lo, src_hi = d.src_hi;
    if constexpr (0 == src_bulk) {
      // Whole rounds in batches of straight-line loads (all in flight
      // together), the ragged rest one by one.
      const int full_rounds = na / nt;
      int round = 0;
      auto run_batch = [&](auto n_tag) {
        constexpr int n = decltype(n_tag)::value;
        type_t r[n];
        #pragma unroll
        for(int k = 0; k < n; ++k)
          r[k] = args.source.load(a0 + (round + k) * nt + tid);
        #pragma unroll
        for(int k = 0; k < n; ++k)
          vals[(round + k) * nt + tid] = r[k];
        round += n;
      };
      for_whole_rounds<functor_batch<vt>::value>(round, full_rounds,
        run_batch);
      for(int i = round * nt + tid; i < na; i += nt)
        vals[i] = args.source.load(a0 + i);
    }
    if constexpr (2 == src_bulk) {
      // Products in place: staged matrix value times the gathered x entry.
      const int* cols_s = reinterpret_cast<const int*>(stage + d.cols_byte);
      const uint64_t keep_policy = ptx::l2_policy_evict_last();
      // Batches of `batch` items per thread: all column indices first, then
      // all gathers (independent loads in flight together), then the stores.
      // The gathers go round the L1 (they never hit there) and ask the L2 to
      // keep x. Three or four in flight per thread measured best (2^24 rows
      // x 16 non-zeros, random columns, 256 x 12 tiles: 2 -> 1.44 ms,
      // 3 -> 1.38, 4 -> 1.39, 6 -> 1.45): more only queue up in front of
      // the L2.
      enum { batch = vt < 4 ? vt : 4 };
      for(int first = tid; first < na; first += nt * batch) {
        int c[batch];
        type_t m[batch], xv[batch];
        #pragma unroll
        for(int k = 0; k < batch; ++k) {
          int i = first + k * nt;
          if(i < na) {
            int w = lo + i;
            int wc = d.cols_lo + i;
            m[k] = (w >= src_lo && w < src_hi) ? vals[w] :
              args.source.data[a0 + i];
            c[k] = (wc >= d.cols_src_lo && wc < d.cols_src_hi) ? cols_s[wc] :
              args.source.columns[a0 + i];
          }
        }
        #pragma unroll
        for(int k = 0; k < batch; ++k)
          if(first + k * nt < na)
            xv[k] = ptx::ld_no_l1_hint(args.source.x + c[k], keep_policy);
        #pragma unroll
        for(int k = 0; k < batch; ++k)
          if(first + k * nt < na) vals[lo + first + k * nt] = m[k] * xv[k];
      }
      src_lo = lo;
      src_hi = hi;
    }
    if constexpr (!seg_bulk) {
      for(int j = ob + tid; j < oe; j += nt)
        offs[j - ob] = (int)args.segments[j];
      ptx::named_sync<1, nt>();
    }

    // 1. Head flags.
    auto mark_heads = [&](auto start_of) {
      for(int j = b0 + tid; j < b1; j += nt) {
        unsigned rel = (unsigned)(start_of(j) - a0);
        int w = lo + (int)(rel < (unsigned)na ? rel : (unsigned)na);
        atomicOr(&flags[w >> 5], 1u << (w & 31));
      }
    };
    auto start_any = [&](int j) -> int {
      return all_staged ? offs_by_seg[j] : seg_start(j);
    };
    mark_heads(start_any);
    // lbs sources: ids are kept relative to segment b0 - 1, the one open at
    // the tile's left edge (0), so that 16 bits hold them.
    [[maybe_unused]] uint16_t* ids =
      reinterpret_cast<uint16_t*>(stage + d.cols_byte);
    [[maybe_unused]] const int seg_base = b0 - 1;
    // Segments b0 - 1 .. b1 - 1 have items in this tile. Their cached tuples
    // go to the stage's slots (one per consumer thread) when they fit; the
    // barriers of the id pass below order these stores before the functor
    // rounds, and their latency hides behind that pass.
    [[maybe_unused]] const int seg_first = b0 > 0 ? b0 - 1 : 0;
    [[maybe_unused]] bool tuples_staged = false;
    if constexpr (3 == src_bulk && layout_t::slot_bytes > 0) {
      typedef typename source_t::cached_t cached_t;
      tuples_staged = b1 - seg_first <= layout_t::slots;
      if(tuples_staged) {
        #pragma unroll
        for(int k = 0; k < layout_t::slots / nt; ++k) {
          int j = k * nt + tid;
          if(seg_first + j < b1)
            reinterpret_cast<cached_t*>(stage + layout_t::slots_offset)[j] =
              args.source.fetch(seg_first + j);
        }
      }
    }
    if constexpr (3 == src_bulk) {
      // Among equal starts the last segment owns the items: its id is left
      // at the head position.
      for(int j = b0 + tid; j < b1; j += nt) {
        int p = start_any(j);
        bool owner = j + 1 >= b1 || start_any(j + 1) != p;
        int w = p - a0;
        if(owner && w >= 0 && w < na) ids[w] = (uint16_t)(j - seg_base);
      }
    }
    if(0 == tid) {
      // Sentinels: the tile's right edge always ends a run, and a head at
      // the first item keeps padding to its left out of every fold.
      atomicOr(&flags[hi >> 5], 1u << (hi & 31));
      if(lo) atomicOr(&flags[lo >> 5], 1u << (lo & 31));
    }
    // The thread's range of positions, [w0 + i_lo, w0 + i_hi) of
    // [w0, w0 + vt), and whether the unrolled fold serves it. For arithmetic
    // types that path also serves the threads that straddle the tile's
    // edges: padding positions hold arbitrary bits whose folds are never
    // stored or propagated, thanks to the sentinels.
    const int w0 = tid * vt;
    const int i_lo = lo > w0 ? lo - w0 : 0;
    const int i_hi = hi - w0 < vt ? hi - w0 : vt;
    const bool inside = w0 + i_lo >= src_lo && w0 + i_hi <= src_hi;
    const bool fast = std::is_arithmetic<type_t>::value ?
      (i_lo < i_hi && inside) : (inside && 0 == i_lo && vt == i_hi);
    // The shifting form takes the values into registers BEFORE the barrier:
    // after it no thread of a fully staged tile still needs its range of the
    // stage, so a run end may be stored anywhere in it (see below).
    enum { early_load = shifting };
    type_t v[vt];
    if constexpr (early_load) { if(fast) load_chunk<vt>(vals + w0, v); }
    ptx::named_sync<1, nt>();
    // The shifting form of the body: in a tile that is whole in its stage the
    // run end at position e, which thread e / vt produces, is kept
    // nt - 1 - e / vt slots to the left of e. The shift shrinks from thread to
    // thread, so no two run ends share a slot; it spreads ends that are a
    // multiple of 8 apart over all banks; and since it is constant within a
    // thread the fold's stores keep their immediate offsets. Slots lie in
    // other threads' ranges (or in the pad in front of the values): every
    // thread took its values into registers before the barrier above.
    const bool shifted = early_load && all_staged && src_lo <= lo &&
      src_hi >= hi;
    const int my_shift = shifted ? nt - 1 - tid : 0;
    auto slot_of = [&](int e) -> int {
      return shifted ? e - (nt - 1 - e / vt) : e;
    };

    if constexpr (3 == src_bulk) {
      // Segment of every item (running maximum of head ids: thread, warp,
      // CTA), then the functor in striped order. lo is 0 for this source.
      const int w0 = tid * vt;
      uint32_t bits = __funnelshift_r(flags[w0 >> 5], flags[(w0 >> 5) + 1],
        w0 & 31) & ((1u << vt) - 1);
      if(w0 >= na) bits = 0;
      else if(w0 + vt > na) bits &= (1u << (na - w0)) - 1;
      int mine = bits ? (int)ids[w0 + 31 - __clz(bits)] : 0;
      int incl = mine;
      #pragma unroll
      for(int delta = 1; delta < 32; delta *= 2) {
        int y = __shfl_up_sync(0xffffffffu, incl, delta);
        if(lane >= delta) incl = max(incl, y);
      }
      int before = __shfl_up_sync(0xffffffffu, incl, 1);
      if(0 == lane) before = 0;
      if(31 == lane) fixed.warp_head[warp] = incl;
      ptx::named_sync<1, nt>();
      int cur = 0;
      for(int k = 0; k < warp; ++k) cur = max(cur, fixed.warp_head[k]);
      cur = max(cur, before);
      if(w0 < na) {
        // The thread's vt ids in registers, then out in 8- or 4-byte stores
        // of four or two ids (slots past the tile's last item take ids as
        // well: they are never read).
        int id[vt];
        #pragma unroll
        for(int i = 0; i < vt; ++i) {
          if((bits >> i) & 1) cur = (int)ids[w0 + i];
          id[i] = cur;
        }
        if constexpr (0 == vt % 4) {
          #pragma unroll
          for(int i = 0; i < vt; i += 4)
            *reinterpret_cast<uint2*>(ids + w0 + i) = make_uint2(
              (uint32_t)id[i] | ((uint32_t)id[i + 1] << 16),
              (uint32_t)id[i + 2] | ((uint32_t)id[i + 3] << 16));
        } else if constexpr (0 == vt % 2) {
          #pragma unroll
          for(int i = 0; i < vt; i += 2)
            *reinterpret_cast<uint32_t*>(ids + w0 + i) =
              (uint32_t)id[i] | ((uint32_t)id[i + 1] << 16);
        } else {
          #pragma unroll
          for(int i = 0; i < vt; ++i) ids[w0 + i] = (uint16_t)id[i];
        }
      }
      ptx::named_sync<1, nt>();
      // The functor usually loads from arrays addressed by index or segment.
      // Whole rounds (every thread has an item) are evaluated `batch` at a
      // time in straight-line code, results stored afterwards, so that a
      // thread's loads are in flight together instead of one round trip after
      // the other; only the ragged last rounds, and the one tile in which an
      // item may precede the first segment, take the item-by-item path.
      // evaluate(index, seg): the functor's value, the segment's tuple taken
      // from the stage's slots or gathered from global memory.
      auto functor_rounds = [&](auto evaluate) {
        int round = 0;
        // n whole rounds in straight-line code.
        auto run_batch = [&](auto n_tag) {
          constexpr int n = decltype(n_tag)::value;
          type_t r[n];
          #pragma unroll
          for(int k = 0; k < n; ++k) {
            int i = (round + k) * nt + tid;
            r[k] = evaluate(a0 + i, seg_base + (int)ids[i]);
          }
          #pragma unroll
          for(int k = 0; k < n; ++k)
            vals[(round + k) * nt + tid] = r[k];
          round += n;
        };
        if(b0 > 0)
          for_whole_rounds<functor_batch<vt>::value>(round, na / nt,
            run_batch);
        for(int i = round * nt + tid; i < na; i += nt) {
          int seg = seg_base + (int)ids[i];
          vals[i] = seg >= 0 ? evaluate(a0 + i, seg) : init;
        }
      };
      if constexpr (layout_t::slot_bytes > 0) {
        typedef typename source_t::cached_t cached_t;
        const cached_t* by_seg = reinterpret_cast<const cached_t*>(
          stage + layout_t::slots_offset) - seg_first;
        if(tuples_staged)
          functor_rounds([&](int index, int seg) {
            return args.source.eval_with(index, seg,
              index - start_any(seg), by_seg[seg]);
          });
        else
          functor_rounds([&](int index, int seg) {
            return args.source.eval(index, seg, index - start_any(seg));
          });
      } else {
        functor_rounds([&](int index, int seg) {
          return args.source.eval(index, seg, index - start_any(seg));
        });
      }
      ptx::named_sync<1, nt>();
    }

    if(na > 0) {
      // 2. Per-thread fold of positions [w0, w0 + vt). The value of every
      // run that ends inside the thread's range is stored in place (shifted
      // tiles: in its shifted slot); the first of them still lacks what
      // precedes the thread (step 4).
      uint32_t bits = __funnelshift_r(flags[w0 >> 5], flags[(w0 >> 5) + 1],
        w0 & 31);
      uint32_t ends = bits >> 1;

      type_t x = init;
      bool head = true;
      type_t* own = vals + w0 - my_shift;   // where this thread's run ends go
      if(fast) {
        if constexpr (!early_load) load_chunk<vt>(vals + w0, v);
        x = v[0];
        if(ends & 1) own[0] = x;
        #pragma unroll
        for(int i = 1; i < vt; ++i) {
          x = ((bits >> i) & 1) ? v[i] : op(x, v[i]);
          if((ends >> i) & 1) own[i] = x;
        }
        head = 0 != (bits & vt_mask);
        ends &= vt_mask;
      } else if(i_lo < i_hi) {
        if constexpr (1 == src_bulk) {
          // Array elements outside the 16-byte-aligned interior.
          for(int i = i_lo; i < i_hi; ++i) {
            int w = w0 + i;
            if(w < src_lo || w >= src_hi)
              vals[w] = args.source.load(a0 + (w - lo));
          }
        }
        x = vals[w0 + i_lo];
        if((ends >> i_lo) & 1) vals[w0 + i_lo] = x;
        for(int i = i_lo + 1; i < i_hi; ++i) {
          type_t y = vals[w0 + i];
          x = ((bits >> i) & 1) ? y : op(x, y);
          if((ends >> i) & 1) vals[w0 + i] = x;
        }
        uint32_t range = ((1u << i_hi) - 1) & ~((1u << i_lo) - 1);
        head = 0 != (bits & range);
        ends &= range;
      } else {
        ends = 0;
      }
      // Does the thread's first run start at a head of its own?
      const int first_item = fast ? 0 : i_lo;
      const bool first_is_head = (bits >> first_item) & 1;

      // 3. Segmented scan of (head, x) across the CTA.
      unsigned head_mask = __ballot_sync(full_mask, head);
      unsigned at_or_below = head_mask & (full_mask >> (31 - lane));
      int run_start = at_or_below ? 31 - __clz(at_or_below) : 0;
      type_t incl = x;
      #pragma unroll
      for(int delta = 1; delta < 32; delta *= 2) {
        type_t y = shfl_up_any(incl, delta);
        if(lane - delta >= run_start) incl = op(y, incl);
      }
      type_t c = shfl_up_any(incl, 1);
      if(31 == lane) {
        warp_agg[warp] = incl;
        fixed.warp_head[warp] = 0 != head_mask;
      }
      ptx::named_sync<1, nt>();

      // 4. Complete the first run end of each thread with what precedes it:
      // the lanes before it in the warp (c) and, for the lanes in front of
      // the warp's first head, what the earlier warps carry in (cw, the same
      // for every lane: no divergence).
      type_t cw = init;
      if(warp > 0) {
        cw = warp_agg[warp - 1];
        for(int k = warp - 1; k > 0 && !fixed.warp_head[k]; --k)
          cw = op(warp_agg[k - 1], cw);
      }
      const bool use_cw = warp > 0 && 0 == (head_mask & ((1u << lane) - 1));
      if(ends && !first_is_head && (lane > 0 || use_cw)) {
        type_t carry = lane > 0 ? (use_cw ? op(cw, c) : c) : cw;
        int e1 = __ffs(ends) - 1;
        own[e1] = op(carry, own[e1]);
      }
    }

    for(int i = tid; i < flag_words; i += nt) flags_next[i] = 0;
    ptx::named_sync<1, nt>();

    // 5. Outputs of the segments whose end marker (the next segment's start)
    // lies in this tile: `init` for empty ones, the stored run end otherwise.
    // The first one may need items of earlier tiles: the carry warp's job.
    {
      // Two threads of different warps fill the tile's edge record.
      const int r = it % ring;
      tile_edge_t<type_t>& e = fixed.edge[r];
      if(edge_thread_a == tid || edge_thread_b == tid) {
        if(it >= ring &&
          !ptx::mbar_wait(&fixed.edge_free[r], (it / ring - 1) & 1,
            args.timeout_ns))
          raise_status(args.header + 1, (uint32_t)status_copy_timeout);
      }
      if(edge_thread_a == tid) {
        const bool has_first = b0 >= 1 && b0 < jend;
        int prev0 = 0, p0 = 0;
        type_t lead = init;
        if(has_first) {
          prev0 = start_any(b0 - 1);
          p0 = start_any(b0);
          unsigned q0 = (unsigned)(p0 - a0);
          if(q0 > (unsigned)na) q0 = p0 < a0 ? 0u : (unsigned)na;
          if(q0 > 0) lead = vals[slot_of(lo + (int)q0 - 1)];
        }
        e.tile = d.tile; e.a0 = a0; e.na = na; e.b0 = b0; e.nb = nb;
        e.has_first = has_first; e.prev0 = prev0; e.p0 = p0;
        memcpy(e.lead, &lead, sizeof(type_t));
        ptx::mbar_arrive(&fixed.edge_full[r]);
      }
      if(edge_thread_b == tid) {
        type_t tail = init;
        if(na > 0) tail = vals[slot_of(hi - 1)];
        int p_last = a1 - 1;
        if(nb > 0)
          p_last = start_any(b1 - 1);
        e.closed = p_last == a1;
        memcpy(e.tail, &tail, sizeof(type_t));
        ptx::mbar_arrive(&fixed.edge_full[r]);
      }
    }
    // Each thread looks up at most one output per pass: the value is read
    // from the stage first, so that in the usual case (no more segment
    // starts than threads) the stage is released before the global stores.
    // (Straight-line: the stored run end is read whether or not it is used;
    // its slot always lies inside the stage.)
    auto lookup_output = [&](auto start_of, int j, type_t& value) -> bool {
      const int p = start_of(j);
      const bool empty = j > 0 && start_of(j > 0 ? j - 1 : 0) == p;
      unsigned rel = (unsigned)(p - a0);
      if(rel > (unsigned)na) rel = (unsigned)na;
      if(rel < 1u) rel = 1u;
      const type_t stored = vals[slot_of(lo + (int)rel - 1)];
      value = empty ? init : stored;
      // Segment b0 - 1, when it has items, is the carry warp's.
      return j > 0 && (empty || j != b0);
    };
    // (More than one trip only when the tile has more starts than threads.)
    for(int j = b0 + tid; ; j += nt) {
      const bool more = j + nt < jend_lookup;
      type_t value;
      bool write = false;
      if(j < jend_lookup) write = lookup_output(start_any, j, value);
      if(!more) ptx::mbar_arrive(&fixed.empty[s]);
      if(write) args.output[j - 1] = value;
      if(!more) break;
    }
    return true;
  };

  // Rows of one fixed width whose length is a multiple of 8 (the usual shape
  // of a dense-ish matrix or a batched reduction) put every run end of a tile
  // into one or two shared-memory banks when the ends are kept in place: a
  // third more time on rows of 16 or 32 fp32 items. The shifting form has no
  // such shape but costs ~2 % elsewhere, so a CTA picks by looking at the
  // segment starts of its first tile: all at the same position modulo 8 (and
  // at least 64 of them) means fixed-width rows.
  int tiles_done = 0;
  bool shifting = false;
  if constexpr (1 == src_bulk && seg_bulk && std::is_arithmetic<type_t>::value) {
    if(!ptx::mbar_wait(&fixed.full[0], 0, args.timeout_ns))
      raise_status(args.header + 1, (uint32_t)status_copy_timeout);
    const tile_desc_t d = fixed.desc[0];
    bool aligned = d.tile >= 0 && d.b1 - d.b0 >= 64;
    if(aligned) {
      const int* offs = reinterpret_cast<const int*>(
        stage_base + pad_bytes + d.offs_byte);
      // Staged starts of segments [ob, oe); compare those of the tile.
      int j = d.b0 + tid, j0 = d.b0;
      if(j < d.b1 && j >= d.ob && j < d.oe && j0 >= d.ob)
        aligned = 0 == ((offs[j - d.ob] ^ offs[j0 - d.ob]) & 7);
    }
    shifting = ptx::named_all<1, nt>(aligned);
  }
  // With two stages, two tiles per trip of the loop: the stage, the flag
  // buffer and the barrier parities alternate between constants (~1 % of the
  // kernel's time against a loop that derives them from the counter).
  auto consume_all = [&](auto shifting_tag) {
    #pragma unroll (2 == stages ? 2 : 1)
    for(int it = 0; ; ++it) {
      if(!consume_tile(shifting_tag, it)) break;
      ++tiles_done;
    }
  };
  if(shifting) consume_all(std::true_type());
  else consume_all(std::false_type());
  if(edge_thread_a == tid || edge_thread_b == tid) {
    // One end-of-work record for each carry warp.
    for(int n = tiles_done; n < tiles_done + segreduce_carry_warps; ++n) {
      const int r = n % ring;
      if(n >= ring &&
        !ptx::mbar_wait(&fixed.edge_free[r], (n / ring - 1) & 1,
          args.timeout_ns))
        raise_status(args.header + 1, (uint32_t)status_copy_timeout);
      if(edge_thread_a == tid) fixed.edge[r].tile = -1;
      ptx::mbar_arrive(&fixed.edge_full[r]);
    }
  }
}

////////////////////////////////////////////////////////////////////////////////
// Host side.

// Workspace layout: [header 128 B][partitions][tile status].
template<typename tuning_t, typename type_t>
struct segreduce_plan_t {
  int num_tiles;
  size_t partitions_offset, state_offset, bytes;

  segreduce_plan_t(int count, int num_segments) {
    int64_t total = (int64_t)count + num_segments;
    num_tiles = (int)div_up(total, (int64_t)tuning_t::nv);
    partitions_offset = 128;
    size_t part_bytes = ((size_t)(num_tiles + 1) * 4 + 127) / 128 * 128;
    state_offset = partitions_offset + part_bytes;
    bytes = state_offset + tile_state_bytes<type_t>(num_tiles) + 128;
  }
};

// CTAs of `kernel` that fit on the current device at once. `tag_t` must be
// unique per kernel instantiation: the answer is cached per (tag, device).
template<typename tag_t, typename kernel_t>
int resident_ctas(kernel_t kernel, int threads, int smem_bytes) {
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

// Default bound on device-side waits: two seconds.
constexpr uint64_t default_timeout_ns = 2000000000ull;

// Enqueue partitioner + reduction on `stream`. `workspace` must hold
// segreduce_plan_t<...>(count, num_segments).bytes bytes, 128-byte aligned.
// `after_partition`, when given, is recorded between the two kernels.
// `tail` rides in the partitioner's launch and `finish` ends the reduction
// (see no_partition_tail_t, no_finish_t). `parts`: 1 enqueues the partitioner
// only, 2 the reduction only (the partitioner of the same call must precede
// it in the stream), 3 both.
enum { segreduce_partition_part = 1, segreduce_reduce_part = 2,
  segreduce_both_parts = 3 };

template<typename tuning_t, typename type_t, typename source_t,
  typename segments_it, typename output_it, typename op_t,
  typename tail_t = no_partition_tail_t, typename finish_t = no_finish_t>
void segreduce_enqueue(source_t source, int count, segments_it segments,
  int num_segments, output_it output, op_t op, type_t init, void* workspace,
  cudaStream_t stream, uint64_t timeout_ns = default_timeout_ns,
  cudaEvent_t after_partition = nullptr, tail_t tail = tail_t(),
  finish_t finish = finish_t(), int parts = segreduce_both_parts) {

  typedef segreduce_smem_t<tuning_t, type_t, source_t::bulk,
    source_slot_bytes<source_t>::value> layout_t;
  typedef segreduce_args_t<type_t, source_t, segments_it, output_it, op_t,
    finish_t> args_t;
  segreduce_plan_t<tuning_t, type_t> plan(count, num_segments);
  if(!plan.num_tiles) return;

  char* base = (char*)workspace;
  uint32_t* header = (uint32_t*)base;
  int* partitions = (int*)(base + plan.partitions_offset);
  void* state = base + plan.state_offset;

  if(parts & segreduce_partition_part)
    launch_lbs_partition(segments, count, num_segments,
      (int64_t)tuning_t::nv, plan.num_tiles + 1, partitions, stream,
      header, 32, (uint32_t*)state,
      (int)tile_state_traits<type_t>::clear_words,
      (int)tile_state_traits<type_t>::stride_words, tail);
  if(after_partition) cudaEventRecord(after_partition, stream);
  if(!(parts & segreduce_reduce_part)) return;

  auto kernel = segreduce_k<tuning_t, type_t, source_t, segments_it,
    output_it, op_t, finish_t>;
  int threads = tuning_t::nt + 32 + 32 * segreduce_carry_warps;
  int resident = resident_ctas<tuple<tuning_t, args_t> >(kernel, threads,
    (int)layout_t::total_bytes);
  int grid = plan.num_tiles < resident ? plan.num_tiles : resident;

  args_t args { source, segments, output, op, init, count, num_segments,
    plan.num_tiles, partitions, header, state, timeout_ns, finish };
  // Launched as a programmatic dependent of the partitioner: its CTAs start,
  // initialise their barriers and wait inside the kernel.
  cudaLaunchConfig_t config = { };
  config.gridDim = dim3(grid);
  config.blockDim = dim3(threads);
  config.dynamicSmemBytes = layout_t::total_bytes;
  config.stream = stream;
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  throw_on_error(cudaLaunchKernelEx(&config, kernel, args));
}

} // namespace detail

END_MGPU_NAMESPACE

#endif // __CUDACC__
