// Per-tile status words for the single-pass ("decoupled look-back") carry
// between tiles of a segmented reduction.
//
// The reference finishes a segmented reduction with a second, recursive
// fix-up pass over per-CTA carry-outs (src/moderngpu/kernel_segreduce.hxx:
// 105-185). Here every tile publishes, as soon as it knows it, the value of
// the segment still open at its right edge, and a later tile that needs the
// part of its first segment lying to its left reads those words backwards
// until it meets a tile whose value no longer depends on anything earlier.
//
// A tile's word is one of
//   tile_empty          nothing published yet
//   tile_partial        fold of ALL items of the tile; the tile holds no
//                       segment start, so earlier tiles still contribute
//   tile_inclusive      fold of the open segment up to the tile's right edge,
//                       everything to the left already included
//   tile_closed         a segment start sits exactly on the tile's right
//                       edge: the open segment has no items yet
// Readers stop at the first tile_inclusive or tile_closed word.
#pragma once
#include "ptx.hxx"

#ifdef __CUDACC__

BEGIN_MGPU_NAMESPACE
namespace detail {

enum : uint32_t {
  tile_empty = 0,
  tile_partial = 1,
  tile_inclusive = 2,
  tile_closed = 3
};

// Status codes reported through the workspace header.
enum : uint32_t {
  status_ok = 0,
  status_lookback_timeout = 1,   // a predecessor tile never published
  status_copy_timeout = 2        // a staged copy never completed
};

template<typename type_t>
struct tile_state_traits {
  // Value and code travel in one 64-bit word when the value fits in 32 bits,
  // in one aligned 16-byte access when it fits in 64 bits; otherwise the code
  // is made visible after the value has been written.
  enum { packed = sizeof(type_t) <= 8 &&
    std::is_trivially_copyable<type_t>::value };
  // Wide layout of one tile: [code:4, pad:12][partial value][inclusive value],
  // each value slot rounded up to 16 bytes.
  enum { slot_bytes = ((int)sizeof(type_t) + 15) / 16 * 16 };
  // Each tile's status lives in 128-byte lines of its own: tiles that are in
  // flight together belong to different SMs (and dies), which would otherwise
  // write and poll one shared line.
  enum { tile_bytes = packed ? 128 : (16 + 2 * slot_bytes + 127) / 128 * 128 };
  // 32-bit words per tile that must read zero before a launch, and the
  // distance in 32-bit words between consecutive tiles.
  enum { clear_words = packed ? (sizeof(type_t) <= 4 ? 2 : 4) : 1,
    stride_words = tile_bytes / 4 };
};

// Bytes of tile-status storage for num_tiles tiles.
template<typename type_t>
inline size_t tile_state_bytes(int num_tiles) {
  return (size_t)num_tiles * tile_state_traits<type_t>::tile_bytes;
}

// layout: 1 = one 64-bit word, 2 = one 16-byte word, 0 = code + value slots.
template<typename type_t, int layout = !tile_state_traits<type_t>::packed ? 0 :
  (sizeof(type_t) <= 4 ? 1 : 2)>
struct tile_state_t;

template<typename type_t>
struct tile_state_t<type_t, 1> {
  enum { stride = tile_state_traits<type_t>::stride_words / 2 };
  uint64_t* words;

  MGPU_DEVICE void bind(void* base, int) { words = (uint64_t*)base; }

  MGPU_DEVICE void publish(int tile, uint32_t code, type_t value) const {
    uint32_t bits = 0;
    memcpy(&bits, &value, sizeof(type_t));
    ptx::st_relaxed_u64(words + (size_t)tile * stride, ((uint64_t)code << 32) | bits);
  }
  MGPU_DEVICE void publish(int tile, uint32_t code) const {
    ptx::st_relaxed_u64(words + (size_t)tile * stride, (uint64_t)code << 32);
  }
  MGPU_DEVICE uint32_t peek(int tile, type_t& value) const {
    uint64_t w = ptx::ld_relaxed_u64(words + (size_t)tile * stride);
    uint32_t bits = (uint32_t)w;
    memcpy(&value, &bits, sizeof(type_t));
    return (uint32_t)(w >> 32);
  }
};

template<typename type_t>
struct tile_state_t<type_t, 2> {
  enum { tile_bytes = tile_state_traits<type_t>::tile_bytes };
  char* base;

  MGPU_DEVICE void bind(void* base_, int) { base = (char*)base_; }

  MGPU_DEVICE void publish(int tile, uint32_t code, type_t value) const {
    uint64_t bits = 0;
    memcpy(&bits, &value, sizeof(type_t));
    ptx::st_relaxed_v2u64(base + (size_t)tile * tile_bytes, bits, code);
  }
  MGPU_DEVICE void publish(int tile, uint32_t code) const {
    ptx::st_relaxed_v2u64(base + (size_t)tile * tile_bytes, 0, code);
  }
  MGPU_DEVICE uint32_t peek(int tile, type_t& value) const {
    uint64_t bits, code;
    ptx::ld_relaxed_v2u64(base + (size_t)tile * tile_bytes, bits, code);
    memcpy(&value, &bits, sizeof(type_t));
    return (uint32_t)code;
  }
};

template<typename type_t>
struct tile_state_t<type_t, 0> {
  enum { slot_bytes = tile_state_traits<type_t>::slot_bytes,
    tile_bytes = tile_state_traits<type_t>::tile_bytes };
  char* base;

  MGPU_DEVICE void bind(void* base_, int) { base = (char*)base_; }

  MGPU_DEVICE uint32_t* code_of(int tile) const {
    return (uint32_t*)(base + (size_t)tile * tile_bytes);
  }
  MGPU_DEVICE char* slot_of(int tile, uint32_t code) const {
    return base + (size_t)tile * tile_bytes + 16 +
      (tile_partial == code ? 0 : slot_bytes);
  }

  static MGPU_DEVICE void put(char* slot, const type_t& value) {
    uint32_t tmp[slot_bytes / 4] = { };
    memcpy(tmp, &value, sizeof(type_t));
    volatile uint32_t* dst = (volatile uint32_t*)slot;
    #pragma unroll
    for(int i = 0; i < slot_bytes / 4; ++i) dst[i] = tmp[i];
  }
  static MGPU_DEVICE void take(const char* slot, type_t& value) {
    uint32_t tmp[slot_bytes / 4];
    const volatile uint32_t* src = (const volatile uint32_t*)slot;
    #pragma unroll
    for(int i = 0; i < slot_bytes / 4; ++i) tmp[i] = src[i];
    memcpy(&value, tmp, sizeof(type_t));
  }

  MGPU_DEVICE void publish(int tile, uint32_t code, type_t value) const {
    put(slot_of(tile, code), value);
    ptx::st_release_u32(code_of(tile), code);
  }
  MGPU_DEVICE void publish(int tile, uint32_t code) const {
    ptx::st_release_u32(code_of(tile), code);
  }
  // Polls stay cheap (a relaxed load); the fence that orders the value loads
  // after the code is paid only once the code says a value is there.
  MGPU_DEVICE uint32_t peek(int tile, type_t& value) const {
    uint32_t code = ptx::ld_relaxed_u32(code_of(tile));
    if(tile_partial == code || tile_inclusive == code) {
      __threadfence();
      take(slot_of(tile, code), value);
    }
    return code;
  }
};

// Lane-to-lane copy of a value of any size.
template<typename type_t>
MGPU_DEVICE type_t shfl_any(const type_t& x, int src_lane) {
  enum { words = (sizeof(type_t) + 3) / 4 };
  uint32_t w[words] = { };
  memcpy(w, &x, sizeof(type_t));
  #pragma unroll
  for(int i = 0; i < words; ++i)
    w[i] = __shfl_sync(0xffffffffu, w[i], src_lane);
  type_t y;
  memcpy(&y, w, sizeof(type_t));
  return y;
}
template<typename type_t>
MGPU_DEVICE type_t shfl_up_any(const type_t& x, int delta) {
  enum { words = (sizeof(type_t) + 3) / 4 };
  uint32_t w[words] = { };
  memcpy(w, &x, sizeof(type_t));
  #pragma unroll
  for(int i = 0; i < words; ++i)
    w[i] = __shfl_up_sync(0xffffffffu, w[i], delta);
  type_t y;
  memcpy(&y, w, sizeof(type_t));
  return y;
}

template<typename type_t>
MGPU_DEVICE type_t shfl_down_any(const type_t& x, int delta) {
  int lane = (int)(threadIdx.x & 31);
  return shfl_any(x, lane + delta < 32 ? lane + delta : lane);
}

// Executed by one full warp of tile `tile` (> 0): fold what tiles
// tile-1, tile-2, ... contribute to the segment that is open at this tile's
// left edge. Returns true and sets `carry` when there is a contribution.
// `timeout_ns` bounds every wait; on expiry *status is set and false returned.
template<typename type_t, typename op_t>
MGPU_DEVICE bool lookback(const tile_state_t<type_t>& state, int tile,
  op_t op, type_t& carry, uint64_t timeout_ns, uint32_t* status) {
  const unsigned full = 0xffffffffu;
  int lane = (int)(threadIdx.x & 31);
  bool have = false;
  type_t acc = carry;
  int base = tile - 1;

  // Common case: the tile just before has a segment start of its own, so its
  // word is final as soon as it appears. Every lane reads the same word.
  {
    type_t value = carry;
    uint32_t code = tile_empty;
    uint64_t start = 0;
    for(uint32_t spin = 0; ; ++spin) {
      code = state.peek(base, value);
      // Lane 0's view decides for the whole warp, so that every lane leaves
      // the loop in the same iteration and the shuffles below stay converged.
      code = __shfl_sync(full, code, 0);
      if(tile_empty != code) break;
      if(spin > 16) __nanosleep(100);
      if(31 == (spin & 31)) {
        uint64_t now = __shfl_sync(full, ptx::global_timer_ns(), 0);
        if(!start) start = now;
        else if(now - start > timeout_ns) break;
      }
    }
    value = shfl_any(value, 0);
    if(tile_empty == code) {
      if(!lane) raise_status(status, (uint32_t)status_lookback_timeout);
      return false;
    }
    if(tile_closed == code) return false;
    if(tile_inclusive == code) { carry = value; return true; }
  }

  while(true) {
    int idx = base - lane;
    uint32_t code = tile_closed;      // before tile 0: nothing to add
    type_t value = carry;
    int stop = 32;
    bool ready = false;
    uint64_t start = 0;
    for(uint32_t spin = 0; ; ++spin) {
      if(idx >= 0) code = state.peek(idx, value);
      unsigned final_mask = __ballot_sync(full, code >= tile_inclusive);
      unsigned empty_mask = __ballot_sync(full, tile_empty == code);
      stop = final_mask ? __ffs(final_mask) - 1 : 32;
      unsigned needed = stop >= 31 ? full : ((2u << stop) - 1);
      if(0 == (empty_mask & needed)) { ready = true; break; }
      if(spin > 16) __nanosleep(100);
      if(31 == (spin & 31)) {
        // Lane 0's clock decides for the whole warp.
        uint64_t now = __shfl_sync(full, ptx::global_timer_ns(), 0);
        if(!start) start = now;
        else if(now - start > timeout_ns) break;
      }
    }
    if(!ready) {
      if(!lane) raise_status(status, (uint32_t)status_lookback_timeout);
      return false;
    }
    // Fold lanes last..0 (earliest tile first).
    int last = stop < 31 ? stop : 31;
    bool w_have = false;
    type_t w = value;
    for(int l = last; l >= 0; --l) {
      type_t v = shfl_any(value, l);
      uint32_t c = __shfl_sync(full, code, l);
      if(tile_closed != c) {
        w = w_have ? op(w, v) : v;
        w_have = true;
      }
    }
    if(w_have) {
      acc = have ? op(w, acc) : w;
      have = true;
    }
    if(stop < 32) break;
    base -= 32;
  }
  if(have) carry = acc;
  return have;
}

// Look-back for a chain in which EVERY tile depends on all earlier ones (a
// prefix scan: no tile_closed words, few tile_inclusive words near the
// front). The inclusive front advances by at most one window per round trip
// to the L2, so the window is `rows` x 32 tiles wide: lane l reads tiles
// base - l - 32 r for r < rows, all loads in flight together, and the rows
// are folded with a shuffle tree. Executed by one full warp of tile `tile`
// (> 0). Returns true and sets `carry` (the fold of all earlier tiles); on
// expiry of `timeout_ns` sets *status and returns false.
template<int rows, typename type_t, typename op_t>
MGPU_DEVICE bool lookback_wide(const tile_state_t<type_t>& state, int tile,
  op_t op, type_t& carry, uint64_t timeout_ns, uint32_t* status) {
  const unsigned full = 0xffffffffu;
  const int lane = (int)(threadIdx.x & 31);
  bool have = false;
  type_t acc = carry;
  int base = tile - 1;
  uint64_t start = 0;
  uint32_t spin = 0;

  while(true) {
    uint32_t code[rows];
    type_t value[rows];
    #pragma unroll
    for(int r = 0; r < rows; ++r) {
      int idx = base - lane - 32 * r;
      code[r] = tile_inclusive;         // before tile 0: the chain ends here
      value[r] = carry;
      if(idx >= 0) code[r] = state.peek(idx, value[r]);
    }
    // Rows are used front to back until one holds a final word or a gap.
    bool done = false, gap = false;
    #pragma unroll
    for(int r = 0; r < rows; ++r) {
      if(done || gap) continue;
      bool before_zero = base - lane - 32 * r < 0;
      unsigned final_mask = __ballot_sync(full, code[r] >= tile_inclusive);
      unsigned empty_mask = __ballot_sync(full, tile_empty == code[r]);
      int stop = final_mask ? __ffs(final_mask) - 1 : 32;
      unsigned needed = stop >= 31 ? full : ((2u << stop) - 1);
      if(empty_mask & needed) {
        // Use the published words in front of the first gap, then poll again
        // from the gap on.
        int first_gap = __ffs(empty_mask & needed) - 1;
        stop = first_gap - 1;            // last usable lane (may be -1)
        gap = true;
        needed = first_gap ? ((1u << first_gap) - 1) : 0u;
      }
      // Fold lanes [0, min(stop, 31)], the earliest tile (highest lane) first.
      int last = stop < 31 ? stop : 31;
      bool mine = lane <= last && !(before_zero);
      type_t x = value[r];
      #pragma unroll
      for(int delta = 1; delta < 32; delta *= 2) {
        type_t up = shfl_down_any(x, delta);
        bool up_have = __shfl_down_sync(full, mine, delta) && lane + delta < 32;
        if(up_have) { x = mine ? op(up, x) : up; mine = true; }
      }
      x = shfl_any(x, 0);
      bool row_have = __shfl_sync(full, mine, 0);
      if(row_have) {
        acc = have ? op(x, acc) : x;
        have = true;
      }
      if(gap) base -= 32 * r + (stop + 1);
      else if(stop < 32) done = true;
    }
    if(done) break;
    if(!gap) { base -= 32 * rows; continue; }
    // Tile `base` had not published anything yet: poll that one word (every
    // lane the same address) until it has, then read the window again.
    while(true) {
      type_t ignored = carry;
      uint32_t c = state.peek(base, ignored);
      if(tile_empty != __shfl_sync(full, c, 0)) break;
      if(spin > 8) __nanosleep(32);
      if(15 == (spin & 15)) {
        uint64_t now = __shfl_sync(full, ptx::global_timer_ns(), 0);
        if(!start) start = now;
        else if(now - start > timeout_ns) {
          if(!lane) raise_status(status, (uint32_t)status_lookback_timeout);
          return false;
        }
      }
      ++spin;
    }
  }
  if(have) carry = acc;
  return have;
}

} // namespace detail
END_MGPU_NAMESPACE

#endif // __CUDACC__
