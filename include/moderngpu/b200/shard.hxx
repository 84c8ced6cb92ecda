// Multi-GPU segmented reduction: mgpu::sharded_segreduce.
//
// The reference is a single-device library (one stream on the current
// device, src/moderngpu/context.hxx:85,109-110; `int count` and a
// `mem_t<int>` partition table, src/moderngpu/kernel_segreduce.hxx:195,
// 207-215, limit one call to 2^31 items). This layer has no counterpart
// there: it reduces ONE array that is cut into consecutive shards held by
// several GPUs of one machine (or by one GPU, when the array is only too
// long for a single call), with the semantics of mgpu::segreduce over the
// whole array (tests/test_segreduce.cu:40-49).
//
// How it works. Shard v holds items [count * v / V, count * (v + 1) / V) and
// a shard-local start table: entry 0 is 0 and stands for the segment carried
// in from the left, the other entries are the local offsets of the segments
// that START inside the shard. Each shard runs the single-GPU reduction on
// (items, table); out[0] of a shard is then its boundary partial -- the fold
// of its leading items, which belong to a segment owned by an earlier shard
// -- and its last output may lack the leading items of the following shards.
// One 16-byte boundary record per shard and step settles both:
//  * the partitioner launch of a shard's reduction carries a few extra CTAs
//    that fold the shard's leading items (a few dozen in the usual case) and
//    store the record {value, flags} into the mailbox of every GPU that holds
//    this or an earlier shard -- peer-to-peer stores over NVLink, three
//    8-byte words that each carry the step number, so the reader needs no
//    fence;
//  * the thread of the reduction kernel that stores the shard's last output
//    first reads, in ITS OWN GPU's memory, the records of the following
//    shards and folds them into that value, in shard order.
// No collective, no extra launch, no kernel that polls another GPU's memory;
// every wait is bounded and reports through the mailbox's status word.
#pragma once
#include "segreduce.hxx"

#ifdef __CUDACC__
#include <vector>

BEGIN_MGPU_NAMESPACE

namespace detail {

enum : uint32_t {
  shard_has_partial = 1,   // the record's value folds at least one item
  shard_has_start = 2,     // at least one segment starts inside the shard
  shard_last_empty = 4     // the last local segment has no local item
};

struct shard_record_t {
  unsigned long long value;   // the partial's bits, zero-padded to 8 bytes
  uint32_t flags;
  uint32_t seq;               // mailbox only: the step the record belongs to
};

// Mailbox: one block of device memory per GPU that the other GPUs of the box
// map (peer access within a process, CUDA IPC across processes) and write
// into over NVLink. Fixed layout:
//   [0, 256)        status word (0 = fine, 3 = a record did not arrive in
//                   time, 4 = a ring slot was not released in time)
//   [256, 1280)     scratch of the leading-items reduction
//   [1280, 9472)    acks: shard v's last finished step, one 128-byte line each,
//                   written by the GPU that holds shard v
//   [9472, ...)     slots[shard][step % ring]: 32-byte records written by the
//                   GPU that holds the shard
enum {
  mailbox_ring = 64, mailbox_max_shards = 64,
  mailbox_scratch_offset = 256, mailbox_ack_offset = 1280,
  mailbox_slot_offset = mailbox_ack_offset + 128 * mailbox_max_shards,
  mailbox_slot_bytes = 32,
  mailbox_used_bytes = mailbox_slot_offset +
    mailbox_slot_bytes * mailbox_ring * mailbox_max_shards,
  mailbox_alloc_bytes = 2 << 20,   // a whole allocation block of its own
  status_record_timeout = 3, status_slot_timeout = 4
};

struct mailbox_t {
  char* base;
  MGPU_DEVICE uint32_t* status() const { return (uint32_t*)base; }
  MGPU_DEVICE volatile uint32_t* ack(int shard) const {
    return (volatile uint32_t*)(base + mailbox_ack_offset + 128 * shard);
  }
  MGPU_DEVICE volatile unsigned long long* slot(int shard,
    uint32_t step) const {
    return (volatile unsigned long long*)(base + mailbox_slot_offset +
      mailbox_slot_bytes * (shard * mailbox_ring + step % mailbox_ring));
  }
};

// What a posting / collecting kernel needs to know about the chain of shards.
// peers[p] is GPU p's mailbox as mapped into this GPU's address space (this
// GPU's own mailbox at its own index). Shard v lives on GPU v / per_gpu.
struct shard_chain_t {
  char* const* peers;
  int shard, num_shards, per_gpu;
  uint32_t step;
  unsigned long long timeout_ns;
};

// How long a kernel waits for another GPU's record or ack before it gives up.
constexpr unsigned long long default_mailbox_wait_ns = 10000000000ull;

// Waits, for at most timeout_ns, until this GPU's copy of the record of
// (shard, step) is complete. Returns false when time ran out.
inline MGPU_DEVICE bool mailbox_wait_record(const mailbox_t& box, int shard,
  uint32_t step, unsigned long long timeout_ns, shard_record_t& got) {
  volatile unsigned long long* word = box.slot(shard, step);
  unsigned long long begin = 0;
  for(unsigned spin = 0; ; ++spin) {
    unsigned long long w0 = word[0], w1 = word[1], w2 = word[2];
    if((uint32_t)(w0 >> 32) == step && (uint32_t)(w1 >> 32) == step &&
      (uint32_t)(w2 >> 32) == step) {
      got.value = (w0 & 0xffffffffull) | (w1 << 32);
      got.flags = (uint32_t)w2;
      got.seq = step;
      return true;
    }
    if(0 == (spin & 63)) {
      unsigned long long now = ptx::global_timer_ns();
      if(!begin) begin = now;
      else if(now - begin > timeout_ns) return false;
    }
  }
}

// Waits until every shard held by GPU `gpu` has finished step `step - ring`,
// i.e. until the ring slot about to be overwritten there is no longer read.
inline MGPU_DEVICE bool mailbox_wait_slot_free(const mailbox_t& box,
  const shard_chain_t& chain, int gpu) {
  if(chain.step <= (uint32_t)mailbox_ring) return true;
  const uint32_t need = chain.step - mailbox_ring;
  const int v_end = min((gpu + 1) * chain.per_gpu, chain.num_shards);
  unsigned long long begin = 0;
  for(int v = gpu * chain.per_gpu; v < v_end; ++v) {
    for(unsigned spin = 0; ; ++spin) {
      if((int)(*box.ack(v) - need) >= 0) break;
      if(0 == (spin & 63)) {
        unsigned long long now = ptx::global_timer_ns();
        if(!begin) begin = now;
        else if(now - begin > chain.timeout_ns) return false;
      }
    }
  }
  return true;
}

// The post, as extra CTAs of the partitioner's launch: the fold of the
// shard's leading items (those before its first real segment start) goes,
// with the shard's flags, into the mailbox of every GPU that holds this or
// an earlier shard. Few leading items (the usual case): the first CTA does it
// alone; otherwise `ctas` CTAs fold one contiguous chunk each and the last
// one to finish folds the chunk results in order. The same CTA also tells the
// GPUs that hold later shards that this shard is done with the previous step
// (its collect ran in the previous reduction): they may reuse that slot.
template<typename type_t, typename op_t>
struct shard_post_tail_t {
  enum { ctas = 64, threads = lbs_partition_threads, small = 8192,
    warps = threads / 32 };
  static_assert(std::is_trivially_copyable<type_t>::value &&
    sizeof(type_t) <= 8, "boundary records carry values of up to 8 bytes");
  const type_t* input;
  const int* starts;
  int num_starts, count;
  op_t op;
  shard_chain_t chain;
  char* mailbox;            // this GPU's own mailbox

  // Fold of (value, has) pairs over the CTA, earlier threads first; the
  // total ends up in thread 0.
  MGPU_DEVICE void cta_fold(type_t& acc, bool& has, type_t* warp_value,
    int* warp_has) const {
    const int tid = (int)threadIdx.x;
    const int lane = tid & 31;
    for(int delta = 1; delta < 32; delta *= 2) {
      type_t other = shfl_down_any(acc, delta);
      int other_has = __shfl_down_sync(0xffffffffu, (int)has, delta);
      if(other_has && lane + delta < 32) {
        acc = has ? op(acc, other) : other;
        has = true;
      }
    }
    if(0 == lane) { warp_value[tid >> 5] = acc; warp_has[tid >> 5] = has; }
    __syncthreads();
    if(tid < 32) {
      bool h = tid < warps && warp_has[tid];
      type_t v = h ? warp_value[tid] : type_t();
      for(int delta = 1; delta < warps; delta *= 2) {
        type_t other = shfl_down_any(v, delta);
        int other_has = __shfl_down_sync(0xffffffffu, (int)h, delta);
        if(other_has && tid + delta < 32) {
          v = h ? op(v, other) : other;
          h = true;
        }
      }
      acc = v;
      has = h;
    }
    __syncthreads();
  }

  // Called by every thread of the CTA that holds the shard's total (in
  // thread 0): thread p serves GPU p.
  MGPU_DEVICE void finish(type_t total, int lead, bool real) const {
    __shared__ shard_record_t posted;
    const int tid = (int)threadIdx.x;
    if(0 == tid) {
      uint32_t flags = 0;
      if(lead > 0) flags |= shard_has_partial;
      if(real) flags |= shard_has_start;
      if(real && starts[num_starts - 1] >= count) flags |= shard_last_empty;
      unsigned long long bits = 0;
      memcpy(&bits, &total, sizeof(type_t));
      posted.value = bits;
      posted.flags = flags;
      posted.seq = chain.step;
    }
    __syncthreads();
    const int own_gpu = chain.shard / chain.per_gpu;
    const int gpus = (chain.num_shards + chain.per_gpu - 1) / chain.per_gpu;
    mailbox_t mine = { mailbox };
    for(int p = tid; p <= own_gpu; p += threads) {
      if(mailbox_wait_slot_free(mine, chain, p)) {
        mailbox_t theirs = { chain.peers[p] };
        volatile unsigned long long* word =
          theirs.slot(chain.shard, chain.step);
        const unsigned long long tag = (unsigned long long)chain.step << 32;
        word[0] = (posted.value & 0xffffffffull) | tag;
        word[1] = (posted.value >> 32) | tag;
        word[2] = (unsigned long long)posted.flags | tag;
      } else
        atomicMax(mine.status(), (uint32_t)status_slot_timeout);
    }
    // Every launch on this stream follows the previous step's reduction and
    // with it that step's collect.
    if(chain.step > 1)
      for(int p = own_gpu + tid; p < gpus; p += threads) {
        mailbox_t theirs = { chain.peers[p] };
        *theirs.ack(chain.shard) = chain.step - 1;
      }
  }

  MGPU_DEVICE void operator()(int cta) const {
    __shared__ type_t warp_value[warps];
    __shared__ int warp_has[warps];
    __shared__ bool last_cta;
    unsigned long long* chunk_value =
      (unsigned long long*)(mailbox + mailbox_scratch_offset);
    uint32_t* chunk_has = (uint32_t*)(chunk_value + ctas);
    uint32_t* ticket = chunk_has + ctas;

    const bool real = num_starts > 1;
    const int lead = real ? min(max(starts[1], 0), count) : count;
    const int tid = (int)threadIdx.x;
    const bool alone = lead <= small;
    if(alone && cta) return;
    const long long lo = alone ? 0 : (long long)lead * cta / ctas;
    const long long hi = alone ? lead : (long long)lead * (cta + 1) / ctas;

    // Thread t folds a contiguous slice, so that thread order is item order.
    const long long span = hi - lo;
    const long long t_lo = lo + span * tid / threads;
    const long long t_hi = lo + span * (tid + 1) / threads;
    type_t acc = type_t();
    bool has = false;
    for(long long i = t_lo; i < t_hi; ++i) {
      type_t v = input[i];
      acc = has ? op(acc, v) : v;
      has = true;
    }
    cta_fold(acc, has, warp_value, warp_has);
    if(alone) {
      finish(acc, lead, real);
      return;
    }
    if(0 == tid) {
      unsigned long long bits = 0;
      memcpy(&bits, &acc, sizeof(type_t));
      chunk_value[cta] = bits;
      chunk_has[cta] = has;
      __threadfence();
      last_cta = (ctas - 1 == atomicAdd(ticket, 1u));
    }
    __syncthreads();
    if(!last_cta) return;
    __threadfence();
    has = tid < ctas && ((volatile uint32_t*)chunk_has)[tid];
    acc = type_t();
    if(has) {
      unsigned long long bits =
        ((volatile unsigned long long*)chunk_value)[tid];
      memcpy(&acc, &bits, sizeof(type_t));
    }
    cta_fold(acc, has, warp_value, warp_has);
    if(0 == tid) *ticket = 0;
    finish(acc, lead, real);
  }
};

// The collect, inside the shard's reduction: the thread that is about to
// store the shard's last output passes the value through here first. The
// partials of the following shards belong to the segment that is open at
// this shard's right edge, up to and including the first shard that holds a
// segment start of its own. The records are read from THIS GPU's mailbox
// (they were posted before the following shards' reductions even began, so
// they have normally long arrived); a record that does not arrive in time
// leaves the value as it is and sets the mailbox's status word.
template<typename type_t, typename op_t>
struct shard_collect_finish_t {
  char* mailbox;
  shard_chain_t chain;
  op_t op;

  MGPU_DEVICE type_t operator()(type_t current) const {
    mailbox_t box = { mailbox };
    shard_record_t r;
    if(!mailbox_wait_record(box, chain.shard, chain.step, chain.timeout_ns,
      r)) {
      atomicMax(box.status(), (uint32_t)status_record_timeout);
      return current;
    }
    const uint32_t mine = r.flags;
    if(!(mine & shard_has_start)) return current;      // owns nothing
    bool have = false;
    type_t acc = current;
    for(int k = chain.shard + 1; k < chain.num_shards; ++k) {
      if(!mailbox_wait_record(box, k, chain.step, chain.timeout_ns, r)) {
        atomicMax(box.status(), (uint32_t)status_record_timeout);
        return current;
      }
      if(r.flags & shard_has_partial) {
        type_t x;
        memcpy(&x, &r.value, sizeof(type_t));
        acc = have ? op(acc, x) : x;
        have = true;
      }
      if(r.flags & shard_has_start) break;
    }
    if(!have) return current;
    return (mine & shard_last_empty) ? acc : op(current, acc);
  }
};

// Shard-local start tables from ONE global table of 64-bit start offsets.
// bounds[v] = first segment that starts at or after the first item of shard
// v (lower bound); bounds[num_shards] = num_segments, so that the last shard
// also takes the trailing empty segments that start at `count`.
static __global__ void shard_bounds_k(const long long* segments,
  long long num_segments, long long count, int num_shards,
  long long* bounds) {
  int v = (int)(blockIdx.x * blockDim.x + threadIdx.x);
  if(v > num_shards) return;
  if(v == num_shards) { bounds[v] = num_segments; return; }
  long long begin = count * v / num_shards;
  long long lo = 0, hi = num_segments;
  while(lo < hi) {
    long long mid = lo + (hi - lo) / 2;
    if(segments[mid] < begin) lo = mid + 1;
    else hi = mid;
  }
  bounds[v] = lo;
}

// table[0] = 0 (the virtual start), table[1 + j] = segments[first + j] - begin.
static __global__ void shard_cut_k(const long long* segments, long long first,
  int n, long long begin, int* table) {
  int j = (int)(blockIdx.x * blockDim.x + threadIdx.x);
  if(0 == j) table[0] = 0;
  if(j < n) table[1 + j] = (int)(segments[first + j] - begin);
}

} // namespace detail

////////////////////////////////////////////////////////////////////////////////
// Host side.

// The GPUs of one process that share an array, shards_per_device consecutive
// shards on each, with their mailboxes, streams and scratch. Construct once;
// a group serves one sharded call at a time.
class shard_group_t {
  std::vector<int> devices_;
  int per_device_;
  std::vector<char*> mailboxes_;          // one per device
  std::vector<char**> peers_;             // per device: device array of them
  std::vector<cudaStream_t> streams_;     // one per device
  std::vector<void*> workspaces_;         // one per shard, grown on demand
  std::vector<size_t> workspace_bytes_;
  uint32_t step_ = 0;

  static void check(cudaError_t e) { detail::throw_on_error(e); }

public:
  shard_group_t(const shard_group_t&) = delete;
  shard_group_t& operator=(const shard_group_t&) = delete;

  explicit shard_group_t(const std::vector<int>& devices,
    int shards_per_device = 1) :
    devices_(devices), per_device_(shards_per_device) {
    const int gpus = (int)devices_.size();
    if(!gpus || shards_per_device < 1 ||
      gpus * shards_per_device > (int)detail::mailbox_max_shards)
      throw cuda_exception_t(cudaErrorInvalidValue);
    int before = 0;
    check(cudaGetDevice(&before));
    mailboxes_.assign(gpus, nullptr);
    peers_.assign(gpus, nullptr);
    streams_.assign(gpus, nullptr);
    workspaces_.assign(num_shards(), nullptr);
    workspace_bytes_.assign(num_shards(), 0);
    for(int g = 0; g < gpus; ++g) {
      check(cudaSetDevice(devices_[g]));
      for(int h = 0; h < gpus; ++h) {
        if(devices_[h] == devices_[g]) continue;
        int can = 0;
        check(cudaDeviceCanAccessPeer(&can, devices_[g], devices_[h]));
        if(!can) throw cuda_exception_t(cudaErrorPeerAccessUnsupported);
        cudaError_t e = cudaDeviceEnablePeerAccess(devices_[h], 0);
        if(cudaErrorPeerAccessAlreadyEnabled == e) cudaGetLastError();
        else check(e);
      }
      check(cudaMalloc((void**)&mailboxes_[g], detail::mailbox_alloc_bytes));
      check(cudaMemset(mailboxes_[g], 0, detail::mailbox_alloc_bytes));
      check(cudaStreamCreateWithFlags(&streams_[g], cudaStreamNonBlocking));
    }
    for(int g = 0; g < gpus; ++g) {
      check(cudaSetDevice(devices_[g]));
      check(cudaMalloc((void**)&peers_[g], sizeof(char*) * gpus));
      check(cudaMemcpy(peers_[g], mailboxes_.data(), sizeof(char*) * gpus,
        cudaMemcpyHostToDevice));
      check(cudaDeviceSynchronize());
    }
    check(cudaSetDevice(before));
  }

  ~shard_group_t() {
    int before = 0;
    cudaGetDevice(&before);
    for(size_t g = 0; g < devices_.size(); ++g) {
      cudaSetDevice(devices_[g]);
      cudaDeviceSynchronize();
    }
    for(size_t g = 0; g < devices_.size(); ++g) {
      cudaSetDevice(devices_[g]);
      if(peers_[g]) cudaFree(peers_[g]);
      if(mailboxes_[g]) cudaFree(mailboxes_[g]);
      if(streams_[g]) cudaStreamDestroy(streams_[g]);
      for(int j = 0; j < per_device_; ++j)
        if(workspaces_[g * per_device_ + j])
          cudaFree(workspaces_[g * per_device_ + j]);
    }
    cudaSetDevice(before);
  }

  int num_devices() const { return (int)devices_.size(); }
  int shards_per_device() const { return per_device_; }
  int num_shards() const { return num_devices() * per_device_; }
  int device_of(int shard) const { return devices_[shard / per_device_]; }
  cudaStream_t stream_of(int shard) const {
    return streams_[shard / per_device_];
  }
  char* mailbox_of(int shard) const { return mailboxes_[shard / per_device_]; }
  char* const* peers_of(int shard) const { return peers_[shard / per_device_]; }
  uint32_t next_step() { return ++step_; }

  // Scratch of shard `shard` (on its device), at least `bytes` large.
  void* workspace(int shard, size_t bytes) {
    if(workspace_bytes_[shard] < bytes) {
      check(cudaSetDevice(device_of(shard)));
      check(cudaStreamSynchronize(stream_of(shard)));
      if(workspaces_[shard]) check(cudaFree(workspaces_[shard]));
      workspaces_[shard] = nullptr;
      workspace_bytes_[shard] = 0;
      check(cudaMalloc(&workspaces_[shard], bytes + bytes / 4 + 256));
      workspace_bytes_[shard] = bytes + bytes / 4 + 256;
    }
    return workspaces_[shard];
  }

  // Waits for every device of the group, then throws cuda_exception_t
  // (cudaErrorLaunchTimeout) if a bounded wait of a post or a collect ran out
  // on any of them since the last call; the status words are cleared.
  void synchronize() {
    int before = 0;
    check(cudaGetDevice(&before));
    uint32_t worst = 0;
    for(int g = 0; g < num_devices(); ++g) {
      check(cudaSetDevice(devices_[g]));
      check(cudaStreamSynchronize(streams_[g]));
      uint32_t word = 0;
      check(cudaMemcpy(&word, mailboxes_[g], sizeof(word),
        cudaMemcpyDeviceToHost));
      if(word) {
        worst = word > worst ? word : worst;
        check(cudaMemset(mailboxes_[g], 0, sizeof(word)));
      }
    }
    check(cudaSetDevice(before));
    if(worst) throw cuda_exception_t(cudaErrorLaunchTimeout);
  }
};

// How one array of `count` items and its global start table are cut over the
// shards of a group. Owns the shard-local tables (device memory).
class shard_plan_t {
public:
  long long count = 0;
  std::vector<long long> item_begin, item_end;  // per shard: [begin, end)
  std::vector<long long> first_segment;   // first segment starting inside
  std::vector<int> num_starts;            // entries of the local table
  std::vector<int*> tables;               // device arrays, on the shard's GPU
  std::vector<int> devices;

  shard_plan_t() = default;
  shard_plan_t(const shard_plan_t&) = delete;
  shard_plan_t& operator=(const shard_plan_t&) = delete;
  shard_plan_t(shard_plan_t&& rhs) { *this = std::move(rhs); }
  shard_plan_t& operator=(shard_plan_t&& rhs) {
    release();
    count = rhs.count;
    item_begin.swap(rhs.item_begin); item_end.swap(rhs.item_end);
    first_segment.swap(rhs.first_segment); num_starts.swap(rhs.num_starts);
    tables.swap(rhs.tables); devices.swap(rhs.devices);
    return *this;
  }
  ~shard_plan_t() { release(); }

  int num_shards() const { return (int)tables.size(); }
  // Items of shard v, and outputs it produces (entry 0 is its boundary
  // partial, entries 1.. are segments first_segment[v], first_segment[v]+1, ..).
  int items(int v) const { return (int)(item_end[v] - item_begin[v]); }
  int outputs(int v) const { return num_starts[v]; }

private:
  void release() {
    int before = 0;
    cudaGetDevice(&before);
    for(size_t v = 0; v < tables.size(); ++v)
      if(tables[v]) { cudaSetDevice(devices[v]); cudaFree(tables[v]); }
    tables.clear();
    cudaSetDevice(before);
  }
};

// Cuts [0, count) evenly over the group's shards and derives every shard's
// local start table from the global one ON THE DEVICES: `segments` holds
// num_segments 64-bit start offsets (segments[0] == 0, non-decreasing, every
// value <= count) in device memory that every GPU of the group can read (for
// example on one of them: the group enables peer access). A segment belongs
// to the shard in which it starts; the last shard also takes the empty
// segments that start at `count`. Reads one small array back (this call
// synchronises); the per-step call below does not.
inline shard_plan_t sharded_partition(const long long* segments,
  long long num_segments, long long count, shard_group_t& group) {
  const int shards = group.num_shards();
  shard_plan_t plan;
  plan.count = count;
  int before = 0;
  detail::throw_on_error(cudaGetDevice(&before));

  detail::throw_on_error(cudaSetDevice(group.device_of(0)));
  long long* bounds_device = nullptr;
  detail::throw_on_error(cudaMalloc((void**)&bounds_device,
    sizeof(long long) * (shards + 1)));
  detail::shard_bounds_k<<<1, 128, 0, group.stream_of(0)>>>(segments,
    num_segments, count, shards, bounds_device);
  std::vector<long long> bounds(shards + 1);
  detail::throw_on_error(cudaMemcpyAsync(bounds.data(), bounds_device,
    sizeof(long long) * (shards + 1), cudaMemcpyDeviceToHost,
    group.stream_of(0)));
  detail::throw_on_error(cudaStreamSynchronize(group.stream_of(0)));
  detail::throw_on_error(cudaFree(bounds_device));

  for(int v = 0; v < shards; ++v) {
    long long begin = count * v / shards, end = count * (v + 1) / shards;
    long long n = bounds[v + 1] - bounds[v];
    // What a single call can index (as in mgpu::segreduce).
    if(n < 0 || end - begin + n + 1 > (long long)0x7fffffff - 65536) {
      detail::throw_on_error(cudaSetDevice(before));
      throw cuda_exception_t(cudaErrorInvalidValue);
    }
    plan.item_begin.push_back(begin);
    plan.item_end.push_back(end);
    plan.first_segment.push_back(bounds[v]);
    plan.num_starts.push_back((int)n + 1);
    plan.devices.push_back(group.device_of(v));
    plan.tables.push_back(nullptr);
    detail::throw_on_error(cudaSetDevice(group.device_of(v)));
    detail::throw_on_error(cudaMalloc((void**)&plan.tables[v],
      sizeof(int) * (size_t)(n + 1)));
    int blocks = (int)((n + 256) / 256);
    detail::shard_cut_k<<<blocks, 256, 0, group.stream_of(v)>>>(segments,
      bounds[v], (int)n, begin, plan.tables[v]);
  }
  for(int v = 0; v < shards; ++v) {
    detail::throw_on_error(cudaSetDevice(group.device_of(v)));
    detail::throw_on_error(cudaStreamSynchronize(group.stream_of(v)));
  }
  detail::throw_on_error(cudaSetDevice(before));
  return plan;
}

// mgpu::segreduce over one array held as the shards of `plan`:
//   inputs[v]   the items of shard v (plan.items(v) of them), on its GPU;
//   outputs[v]  plan.outputs(v) results, on its GPU: entry 0 is the shard's
//               boundary partial (part of a segment that an earlier shard
//               owns and has folded in), entry 1 + j the result of global
//               segment plan.first_segment[v] + j.
// op must be associative and commutative over type_t (arithmetic, at most 8
// bytes); init as in segreduce. Everything is enqueued on the group's
// streams, two launches per shard, and nothing waits for a device:
// group.synchronize() does, and reports waits that ran out.
template<typename type_t, typename op_t>
void sharded_segreduce(const type_t* const* inputs, const shard_plan_t& plan,
  type_t* const* outputs, op_t op, type_t init, shard_group_t& group,
  uint64_t wait_ns = 0) {
  typedef typename detail::segreduce_default_tuning<type_t>::type tuning_t;
  typedef detail::array_source_t<type_t> source_t;
  typedef detail::shard_post_tail_t<type_t, op_t> tail_t;
  typedef detail::shard_collect_finish_t<type_t, op_t> finish_t;
  detail::throw_on_device_status();
  const int shards = plan.num_shards();
  if(shards != group.num_shards())
    throw cuda_exception_t(cudaErrorInvalidValue);
  const uint32_t step = group.next_step();
  const unsigned long long wait =
    wait_ns ? wait_ns : detail::default_mailbox_wait_ns;
  int before = 0;
  detail::throw_on_error(cudaGetDevice(&before));

  // Every shard's partitioner (with its post) first, then every reduction
  // (with its collect): a collect may need the post of a later shard of the
  // same GPU, which must therefore precede it in the stream.
  for(int pass = 0; pass < 2; ++pass) {
    for(int v = 0; v < shards; ++v) {
      detail::throw_on_error(cudaSetDevice(group.device_of(v)));
      const int count = plan.items(v), num_starts = plan.num_starts[v];
      detail::segreduce_plan_t<tuning_t, type_t> sizes(count, num_starts);
      void* workspace = group.workspace(v, sizes.bytes);
      detail::shard_chain_t chain = { group.peers_of(v), v, shards,
        group.shards_per_device(), step, wait };
      tail_t tail = { inputs[v], plan.tables[v], num_starts, count, op, chain,
        group.mailbox_of(v) };
      finish_t finish = { group.mailbox_of(v), chain, op };
      detail::segreduce_enqueue<tuning_t>(source_t { inputs[v] }, count,
        (const int*)plan.tables[v], num_starts, outputs[v], op, init,
        workspace, group.stream_of(v), detail::default_timeout_ns, nullptr,
        tail, finish, pass ? detail::segreduce_reduce_part :
          detail::segreduce_partition_part);
    }
  }
  detail::throw_on_error(cudaSetDevice(before));
}

END_MGPU_NAMESPACE

#endif // __CUDACC__
