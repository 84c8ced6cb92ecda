// Multi-GPU layer of the segmented reduction: the item range is cut evenly
// across GPUs, each GPU reduces its shard with the single-GPU kernel, and the
// one value per shard that belongs to a segment owned by an earlier GPU (the
// fold of the shard's leading items) is exchanged and folded in by the owner.
// The reference has no multi-GPU layer; contracts are in
// include/moderngpu_b200.h.
//
// Shard-local convention: starts[0] == 0 is a virtual segment that stands for
// the segment carried in from the left; starts[1..] are the segments that
// START inside the shard. out[0] is therefore the shard's boundary partial
// (or `init` when the shard's first real segment starts at item 0).
#include <moderngpu_b200.h>
#include <moderngpu/kernel_sharded.hxx>
#include <cstring>

namespace {

// Record format, mailbox layout and the bounded waits: include/moderngpu/
// b200/shard.hxx, shared with the C++ entry point mgpu::sharded_segreduce.
using mgpu::detail::shard_has_partial;
using mgpu::detail::shard_has_start;
using mgpu::detail::shard_last_empty;
using mgpu::detail::shard_record_t;
using mgpu::detail::mailbox_t;
using mgpu::detail::mailbox_ring;
using mgpu::detail::mailbox_max_shards;
using mgpu::detail::mailbox_scratch_offset;
using mgpu::detail::mailbox_used_bytes;
using mgpu::detail::mailbox_alloc_bytes;
using mgpu::detail::status_record_timeout;
using mgpu::detail::status_slot_timeout;
typedef mgpu::detail::shard_chain_t chain_t;

__device__ bool wait_record(const mailbox_t& box, int shard, uint32_t step,
  unsigned long long timeout_ns, shard_record_t& got) {
  return mgpu::detail::mailbox_wait_record(box, shard, step, timeout_ns, got);
}
__device__ bool wait_slot_free(const mailbox_t& box, const chain_t& chain,
  int gpu) {
  return mgpu::detail::mailbox_wait_slot_free(box, chain, gpu);
}

template<typename type_t>
__global__ void shard_pack_k(const type_t* out, const int* starts,
  int num_starts, int count, shard_record_t* record) {
  if(threadIdx.x || blockIdx.x) return;
  uint32_t flags = 0;
  bool real = num_starts > 1;
  int first = real ? starts[1] : count;
  if(first > 0) flags |= shard_has_partial;
  if(real) flags |= shard_has_start;
  if(real && starts[num_starts - 1] >= count) flags |= shard_last_empty;
  unsigned long long bits = 0;
  type_t v = out[0];
  memcpy(&bits, &v, sizeof(type_t));
  record->value = bits;
  record->flags = flags;
  record->seq = 0;
}

template<typename type_t>
__device__ type_t apply(int op, type_t a, type_t b) {
  if(MGPU_B200_PLUS == op) return a + b;
  if(MGPU_B200_MAX == op) return a < b ? b : a;
  return b < a ? b : a;
}

// Rank `rank` owns the segment that is open at its right edge. The partials
// of the following shards belong to it, up to and including the first shard
// that holds a segment start of its own.
template<typename type_t>
__global__ void shard_fold_k(const shard_record_t* records, int rank,
  int world, int op, type_t* out, int num_starts, type_t init) {
  if(threadIdx.x || blockIdx.x) return;
  uint32_t mine = records[rank].flags;
  if(!(mine & shard_has_start)) return;
  bool have = false;
  type_t acc = init;
  for(int k = rank + 1; k < world; ++k) {
    uint32_t f = records[k].flags;
    if(f & shard_has_partial) {
      type_t v;
      unsigned long long bits = records[k].value;
      memcpy(&v, &bits, sizeof(type_t));
      acc = have ? apply(op, acc, v) : v;
      have = true;
    }
    if(f & shard_has_start) break;
  }
  if(!have) return;
  type_t& last = out[num_starts - 1];
  last = (mine & shard_last_empty) ? acc : apply(op, last, acc);
}

// Boundary record computed directly from the shard's leading items (those
// before its first real segment start), without waiting for the shard's
// reduction: the exchange of the records can then overlap that reduction.
// `lead_ctas` CTAs fold one contiguous chunk each; the last one to finish
// folds the chunk results in order, writes the record and leaves the ticket
// counter at zero for the next call. scratch: lead_ctas values of 8 bytes, a
// uint32 "chunk has items" word each, and the ticket counter.
enum { lead_ctas = 64, lead_threads = 256, lead_small = 8192 };

// Fold of (value, has) pairs over the CTA, earlier threads first. Returns the
// total in thread 0.
template<typename type_t>
__device__ void lead_cta_fold(int op, type_t& acc, bool& has,
  type_t* warp_value, int* warp_has) {
  const int tid = (int)threadIdx.x;
  for(int delta = 1; delta < 32; delta *= 2) {
    unsigned long long bits = 0;
    memcpy(&bits, &acc, sizeof(type_t));
    bits = __shfl_down_sync(0xffffffffu, bits, delta);
    int other_has = __shfl_down_sync(0xffffffffu, (int)has, delta);
    type_t other;
    memcpy(&other, &bits, sizeof(type_t));
    if(other_has && (tid & 31) + delta < 32) {
      acc = has ? apply(op, acc, other) : other;
      has = true;
    }
  }
  if(0 == (tid & 31)) { warp_value[tid >> 5] = acc; warp_has[tid >> 5] = has; }
  __syncthreads();
  if(tid < 32) {
    bool h = tid < lead_threads / 32 && warp_has[tid];
    type_t v = h ? warp_value[tid] : type_t();
    for(int delta = 1; delta < lead_threads / 32; delta *= 2) {
      unsigned long long bits = 0;
      memcpy(&bits, &v, sizeof(type_t));
      bits = __shfl_down_sync(0xffffffffu, bits, delta);
      int other_has = __shfl_down_sync(0xffffffffu, (int)h, delta);
      type_t other;
      memcpy(&other, &bits, sizeof(type_t));
      if(other_has && tid + delta < 32) {
        v = h ? apply(op, v, other) : other;
        h = true;
      }
    }
    acc = v;
    has = h;
  }
  __syncthreads();
}

// Called by every thread of the CTA that holds the shard's total (in thread
// 0): writes the record locally and, with a mailbox, into the mailbox of every
// GPU that holds this shard or an earlier one -- thread p serves GPU p.
template<typename type_t>
__device__ void lead_finish(shard_record_t* record, type_t total, int lead,
  bool real, const int* starts, int num_starts, int count,
  const chain_t& chain, char* mailbox) {
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
    if(record) *record = posted;
  }
  if(!chain.peers) return;
  __syncthreads();
  const int last_gpu = chain.shard / chain.per_gpu;
  if(tid <= last_gpu) {
    mailbox_t mine = { mailbox };
    if(wait_slot_free(mine, chain, tid)) {
      mailbox_t theirs = { chain.peers[tid] };
      volatile unsigned long long* word = theirs.slot(chain.shard, chain.step);
      const unsigned long long tag = (unsigned long long)chain.step << 32;
      word[0] = (posted.value & 0xffffffffull) | tag;
      word[1] = (posted.value >> 32) | tag;
      word[2] = (unsigned long long)posted.flags | tag;
    } else
      atomicMax(mine.status(), (uint32_t)status_slot_timeout);
  }
}

template<typename type_t>
__global__ void __launch_bounds__(lead_threads)
shard_lead_k(const type_t* input, const int* starts, int num_starts, int count,
  int op, shard_record_t* record, unsigned long long* chunk_value,
  uint32_t* chunk_has, uint32_t* ticket, chain_t chain, char* mailbox) {
  __shared__ type_t warp_value[lead_threads / 32];
  __shared__ int warp_has[lead_threads / 32];
  __shared__ bool last_cta;

  const bool real = num_starts > 1;
  const int lead = real ? min(max(starts[1], 0), count) : count;
  const int cta = (int)blockIdx.x, tid = (int)threadIdx.x;

  // Few leading items (the usual case): the first CTA does it alone.
  const bool alone = lead <= lead_small;
  if(alone && cta) return;
  const long long lo = alone ? 0 : (long long)lead * cta / lead_ctas;
  const long long hi = alone ? lead : (long long)lead * (cta + 1) / lead_ctas;

  // Thread t folds a contiguous slice, so that thread order is item order.
  const long long span = hi - lo;
  const long long t_lo = lo + span * tid / lead_threads;
  const long long t_hi = lo + span * (tid + 1) / lead_threads;
  type_t acc = type_t();
  bool has = false;
  for(long long i = t_lo; i < t_hi; ++i) {
    type_t v = input[i];
    acc = has ? apply(op, acc, v) : v;
    has = true;
  }
  lead_cta_fold(op, acc, has, warp_value, warp_has);
  if(alone) {
    lead_finish(record, acc, lead, real, starts, num_starts, count, chain,
      mailbox);
    return;
  }

  if(0 == tid) {
    unsigned long long bits = 0;
    memcpy(&bits, &acc, sizeof(type_t));
    chunk_value[cta] = bits;
    chunk_has[cta] = has;
    __threadfence();
    last_cta = (lead_ctas - 1 == atomicAdd(ticket, 1u));
  }
  __syncthreads();
  if(!last_cta) return;
  __threadfence();
  has = tid < lead_ctas && ((volatile uint32_t*)chunk_has)[tid];
  acc = type_t();
  if(has) {
    unsigned long long bits = ((volatile unsigned long long*)chunk_value)[tid];
    memcpy(&acc, &bits, sizeof(type_t));
  }
  lead_cta_fold(op, acc, has, warp_value, warp_has);
  if(0 == tid) *ticket = 0;
  lead_finish(record, acc, lead, real, starts, num_starts, count, chain,
    mailbox);
}

// The owner's side: shard `chain.shard` folds the partials of the following
// shards into its last output (same rule as shard_fold_k), reading the records
// from this GPU's own mailbox as they arrive, then tells the GPUs that hold
// later shards that it is done with the step.
template<typename type_t>
__global__ void shard_collect_k(char* mailbox, chain_t chain, int op,
  type_t* out, int num_starts, type_t init) {
  const int lane = (int)threadIdx.x;
  const unsigned full = 0xffffffffu;
  mailbox_t box = { mailbox };

  // Everything the warp may need is requested at once: lane l looks (once,
  // without waiting) at the record of shard `shard + l`, lane 0 also at the
  // output it may update, and every lane at the mailbox it will ack to.
  const int first_gpu = chain.shard / chain.per_gpu;
  const int gpus = (chain.num_shards + chain.per_gpu - 1) / chain.per_gpu;
  char* ack_to = first_gpu + lane < gpus ? chain.peers[first_gpu + lane] : nullptr;
  shard_record_t seen = shard_record_t();
  bool seen_ok = false;
  if(chain.shard + lane < chain.num_shards) {
    volatile unsigned long long* word = box.slot(chain.shard + lane, chain.step);
    unsigned long long w0 = word[0], w1 = word[1], w2 = word[2];
    seen_ok = (uint32_t)(w0 >> 32) == chain.step &&
      (uint32_t)(w1 >> 32) == chain.step && (uint32_t)(w2 >> 32) == chain.step;
    seen.value = (w0 & 0xffffffffull) | (w1 << 32);
    seen.flags = (uint32_t)w2;
  }
  type_t last = type_t();
  if(0 == lane) last = out[num_starts - 1];

  // The warp walks the chain together; a record that had not arrived at the
  // first look is waited for (bounded) by lane 0.
  bool ok = true, have = false, stop = false;
  type_t acc = init;
  uint32_t mine = 0;
  for(int i = 0; ok && !stop && chain.shard + i < chain.num_shards; ++i) {
    shard_record_t r = shard_record_t();
    bool got = false;
    if(i < 32) {
      got = __shfl_sync(full, (int)seen_ok, i);
      r.value = __shfl_sync(full, seen.value, i);
      r.flags = __shfl_sync(full, seen.flags, i);
    }
    if(!got) {
      int fine = 0;
      if(0 == lane)
        fine = wait_record(box, chain.shard + i, chain.step, chain.timeout_ns, r);
      ok = __shfl_sync(full, fine, 0);
      r.value = __shfl_sync(full, r.value, 0);
      r.flags = __shfl_sync(full, r.flags, 0);
      if(!ok) break;
    }
    if(0 == i) {
      mine = r.flags;
      stop = !(mine & shard_has_start);      // owns nothing
      continue;
    }
    if(r.flags & shard_has_partial) {
      type_t x;
      memcpy(&x, &r.value, sizeof(type_t));
      acc = have ? apply(op, acc, x) : x;
      have = true;
    }
    stop = 0 != (r.flags & shard_has_start);
  }
  if(0 == lane) {
    if(!ok) atomicMax(box.status(), (uint32_t)status_record_timeout);
    else if(have)
      out[num_starts - 1] = (mine & shard_last_empty) ? acc : apply(op, last, acc);
  }
  // Done reading this step's records (also after a timeout: the writers must
  // not be held up by a reader that has given up).
  if(ack_to) { mailbox_t theirs = { ack_to }; *theirs.ack(chain.shard) = chain.step; }
  for(int p = first_gpu + 32 + lane; p < gpus; p += 32) {
    mailbox_t theirs = { chain.peers[p] };
    *theirs.ack(chain.shard) = chain.step;
  }
}

using mgpu::detail::default_mailbox_wait_ns;

inline int code_of(cudaError_t e) {
  return cudaSuccess == e ? MGPU_B200_OK : MGPU_B200_E_CUDA + (int)e;
}

} // namespace

namespace {

// The fused step (mgpu_b200_shard_begin / _finish): the shard's partitioner
// with the post riding in its launch, and the shard's reduction with the
// collect inside it -- the same kernels mgpu::sharded_segreduce runs.
template<typename type_t, typename op_t>
int fused_typed(int parts, const void* input, int count, const int* starts,
  int num_starts, void* out, const void* init_host, void* workspace,
  void* mailbox, const void* const* peers, int shard, int num_shards,
  int per_gpu, unsigned step, uint64_t timeout_ns, cudaStream_t stream) {
  using namespace mgpu;
  typedef typename detail::segreduce_default_tuning<type_t>::type tuning_t;
  type_t init = type_t();
  if(init_host) memcpy(&init, init_host, sizeof(type_t));
  chain_t chain = { (char* const*)peers, shard, num_shards, per_gpu, step,
    timeout_ns ? timeout_ns : default_mailbox_wait_ns };
  detail::shard_post_tail_t<type_t, op_t> tail = { (const type_t*)input,
    starts, num_starts, count, op_t(), chain, (char*)mailbox };
  detail::shard_collect_finish_t<type_t, op_t> finish = { (char*)mailbox,
    chain, op_t() };
  try {
    detail::segreduce_enqueue<tuning_t>(
      detail::array_source_t<type_t> { (const type_t*)input }, count, starts,
      num_starts, (type_t*)out, op_t(), init, workspace, stream,
      detail::default_timeout_ns, nullptr, tail, finish, parts);
  } catch(cuda_exception_t& e) {
    return MGPU_B200_E_CUDA + (int)e.result;
  }
  cudaError_t e = cudaGetLastError();
  return cudaSuccess == e ? MGPU_B200_OK : MGPU_B200_E_CUDA + (int)e;
}

template<typename type_t>
int fused_op(int op, int parts, const void* input, int count,
  const int* starts, int num_starts, void* out, const void* init_host,
  void* workspace, void* mailbox, const void* const* peers, int shard,
  int num_shards, int per_gpu, unsigned step, uint64_t timeout_ns,
  cudaStream_t stream) {
  switch(op) {
    case MGPU_B200_PLUS: return fused_typed<type_t, mgpu::plus_t<type_t> >(
      parts, input, count, starts, num_starts, out, init_host, workspace,
      mailbox, peers, shard, num_shards, per_gpu, step, timeout_ns, stream);
    case MGPU_B200_MAX: return fused_typed<type_t, mgpu::maximum_t<type_t> >(
      parts, input, count, starts, num_starts, out, init_host, workspace,
      mailbox, peers, shard, num_shards, per_gpu, step, timeout_ns, stream);
    case MGPU_B200_MIN: return fused_typed<type_t, mgpu::minimum_t<type_t> >(
      parts, input, count, starts, num_starts, out, init_host, workspace,
      mailbox, peers, shard, num_shards, per_gpu, step, timeout_ns, stream);
  }
  return MGPU_B200_E_UNSUPPORTED;
}

int fused_dispatch(int dtype, int op, int parts, const void* input, int count,
  const int* starts, int num_starts, void* out, const void* init_host,
  void* workspace, size_t workspace_bytes, void* mailbox,
  const void* const* peers, int shard, int num_shards, int per_gpu,
  unsigned step, uint64_t timeout_ns, void* stream);

} // namespace

extern "C" {

size_t mgpu_b200_shard_lead_scratch_bytes(void) {
  return (size_t)lead_ctas * 12 + 64;
}

int mgpu_b200_shard_lead(int dtype, int op, const void* input_device,
  int count, const int* starts_device, int num_starts, void* record_device,
  void* scratch_device, void* stream) {
  if(!starts_device || !record_device || !scratch_device || num_starts < 1 ||
    count < 0 || (count && !input_device) || (uintptr_t)scratch_device % 8)
    return MGPU_B200_E_INVALID;
  if(op < MGPU_B200_PLUS || op > MGPU_B200_MIN) return MGPU_B200_E_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  shard_record_t* rec = (shard_record_t*)record_device;
  unsigned long long* values = (unsigned long long*)scratch_device;
  uint32_t* has = (uint32_t*)(values + lead_ctas);
  uint32_t* ticket = has + lead_ctas;
  switch(dtype) {
    case MGPU_B200_F32: shard_lead_k<<<lead_ctas, lead_threads, 0, s>>>(
      (const float*)input_device, starts_device, num_starts, count, op, rec,
      values, has, ticket, chain_t(), nullptr); break;
    case MGPU_B200_F64: shard_lead_k<<<lead_ctas, lead_threads, 0, s>>>(
      (const double*)input_device, starts_device, num_starts, count, op, rec,
      values, has, ticket, chain_t(), nullptr); break;
    case MGPU_B200_I32: shard_lead_k<<<lead_ctas, lead_threads, 0, s>>>(
      (const int*)input_device, starts_device, num_starts, count, op, rec,
      values, has, ticket, chain_t(), nullptr); break;
    case MGPU_B200_I64: shard_lead_k<<<lead_ctas, lead_threads, 0, s>>>(
      (const long long*)input_device, starts_device, num_starts, count, op,
      rec, values, has, ticket, chain_t(), nullptr); break;
    default: return MGPU_B200_E_UNSUPPORTED;
  }
  return code_of(cudaGetLastError());
}

size_t mgpu_b200_mailbox_bytes(void) { return mailbox_alloc_bytes; }

int mgpu_b200_mailbox_create(void** mailbox_device, void* handle_out) {
  if(!mailbox_device || !handle_out) return MGPU_B200_E_INVALID;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  static_assert(mailbox_used_bytes <= mailbox_alloc_bytes, "mailbox size");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, mailbox_alloc_bytes);
  if(cudaSuccess != e) return code_of(e);
  e = cudaMemset(p, 0, mailbox_alloc_bytes);
  if(cudaSuccess == e) e = cudaDeviceSynchronize();
  cudaIpcMemHandle_t handle;
  if(cudaSuccess == e) e = cudaIpcGetMemHandle(&handle, p);
  if(cudaSuccess != e) { cudaFree(p); return code_of(e); }
  memcpy(handle_out, &handle, sizeof(handle));
  *mailbox_device = p;
  return MGPU_B200_OK;
}

int mgpu_b200_mailbox_open(const void* handle_in, void** peer_device) {
  if(!handle_in || !peer_device) return MGPU_B200_E_INVALID;
  cudaIpcMemHandle_t handle;
  memcpy(&handle, handle_in, sizeof(handle));
  return code_of(cudaIpcOpenMemHandle(peer_device, handle,
    cudaIpcMemLazyEnablePeerAccess));
}

int mgpu_b200_mailbox_close(void* peer_device) {
  if(!peer_device) return MGPU_B200_E_INVALID;
  return code_of(cudaIpcCloseMemHandle(peer_device));
}

int mgpu_b200_mailbox_destroy(void* mailbox_device) {
  if(!mailbox_device) return MGPU_B200_E_INVALID;
  return code_of(cudaFree(mailbox_device));
}

int mgpu_b200_mailbox_status(const void* mailbox_device, void* stream,
  int* status_host) {
  if(!mailbox_device || !status_host) return MGPU_B200_E_INVALID;
  uint32_t word = 0;
  cudaError_t e = cudaMemcpyAsync(&word, mailbox_device, 4,
    cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if(cudaSuccess == e) e = cudaStreamSynchronize((cudaStream_t)stream);
  *status_host = (int)word;
  return code_of(e);
}

static bool chain_ok(const void* mailbox, const void* peers, int shard,
  int num_shards, int per_gpu, unsigned step) {
  return mailbox && peers && per_gpu >= 1 && num_shards >= 1 &&
    num_shards <= mailbox_max_shards && 0 == num_shards % per_gpu &&
    num_shards / per_gpu <= lead_threads &&
    shard >= 0 && shard < num_shards && step >= 1;
}

int mgpu_b200_shard_post(int dtype, int op, const void* input_device,
  int count, const int* starts_device, int num_starts, void* mailbox_device,
  const void* const* peers_device, int shard, int num_shards,
  int shards_per_gpu, unsigned step, uint64_t timeout_ns, void* stream) {
  if(!starts_device || num_starts < 1 || count < 0 ||
    (count && !input_device) ||
    !chain_ok(mailbox_device, peers_device, shard, num_shards, shards_per_gpu,
      step))
    return MGPU_B200_E_INVALID;
  if(op < MGPU_B200_PLUS || op > MGPU_B200_MIN) return MGPU_B200_E_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  char* box = (char*)mailbox_device;
  unsigned long long* values =
    (unsigned long long*)(box + mailbox_scratch_offset);
  uint32_t* has = (uint32_t*)(values + lead_ctas);
  uint32_t* ticket = has + lead_ctas;
  chain_t chain = { (char* const*)peers_device, shard, num_shards,
    shards_per_gpu, step, timeout_ns ? timeout_ns : default_mailbox_wait_ns };
  switch(dtype) {
    case MGPU_B200_F32: shard_lead_k<<<lead_ctas, lead_threads, 0, s>>>(
      (const float*)input_device, starts_device, num_starts, count, op,
      nullptr, values, has, ticket, chain, box); break;
    case MGPU_B200_F64: shard_lead_k<<<lead_ctas, lead_threads, 0, s>>>(
      (const double*)input_device, starts_device, num_starts, count, op,
      nullptr, values, has, ticket, chain, box); break;
    case MGPU_B200_I32: shard_lead_k<<<lead_ctas, lead_threads, 0, s>>>(
      (const int*)input_device, starts_device, num_starts, count, op,
      nullptr, values, has, ticket, chain, box); break;
    case MGPU_B200_I64: shard_lead_k<<<lead_ctas, lead_threads, 0, s>>>(
      (const long long*)input_device, starts_device, num_starts, count, op,
      nullptr, values, has, ticket, chain, box); break;
    default: return MGPU_B200_E_UNSUPPORTED;
  }
  return code_of(cudaGetLastError());
}

int mgpu_b200_shard_collect(int dtype, int op, void* mailbox_device,
  const void* const* peers_device, int shard, int num_shards,
  int shards_per_gpu, unsigned step, void* out_device, int num_starts,
  const void* init_host, uint64_t timeout_ns, void* stream) {
  if(!out_device || !init_host || num_starts < 1 ||
    !chain_ok(mailbox_device, peers_device, shard, num_shards, shards_per_gpu,
      step))
    return MGPU_B200_E_INVALID;
  if(op < MGPU_B200_PLUS || op > MGPU_B200_MIN) return MGPU_B200_E_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  char* box = (char*)mailbox_device;
  chain_t chain = { (char* const*)peers_device, shard, num_shards,
    shards_per_gpu, step, timeout_ns ? timeout_ns : default_mailbox_wait_ns };
  switch(dtype) {
    case MGPU_B200_F32: { float i; memcpy(&i, init_host, 4);
      shard_collect_k<<<1, 32, 0, s>>>(box, chain, op, (float*)out_device,
        num_starts, i); break; }
    case MGPU_B200_F64: { double i; memcpy(&i, init_host, 8);
      shard_collect_k<<<1, 32, 0, s>>>(box, chain, op, (double*)out_device,
        num_starts, i); break; }
    case MGPU_B200_I32: { int i; memcpy(&i, init_host, 4);
      shard_collect_k<<<1, 32, 0, s>>>(box, chain, op, (int*)out_device,
        num_starts, i); break; }
    case MGPU_B200_I64: { long long i; memcpy(&i, init_host, 8);
      shard_collect_k<<<1, 32, 0, s>>>(box, chain, op, (long long*)out_device,
        num_starts, i); break; }
    default: return MGPU_B200_E_UNSUPPORTED;
  }
  return code_of(cudaGetLastError());
}

int mgpu_b200_shard_pack(int dtype, const void* out_device,
  const int* starts_device, int num_starts, int count, void* record_device,
  void* stream) {
  if(!out_device || !starts_device || !record_device || num_starts < 1 ||
    count < 0)
    return MGPU_B200_E_INVALID;
  cudaStream_t s = (cudaStream_t)stream;
  shard_record_t* rec = (shard_record_t*)record_device;
  switch(dtype) {
    case MGPU_B200_F32: shard_pack_k<<<1, 32, 0, s>>>((const float*)out_device,
      starts_device, num_starts, count, rec); break;
    case MGPU_B200_F64: shard_pack_k<<<1, 32, 0, s>>>((const double*)out_device,
      starts_device, num_starts, count, rec); break;
    case MGPU_B200_I32: shard_pack_k<<<1, 32, 0, s>>>((const int*)out_device,
      starts_device, num_starts, count, rec); break;
    case MGPU_B200_I64: shard_pack_k<<<1, 32, 0, s>>>(
      (const long long*)out_device, starts_device, num_starts, count, rec);
      break;
    default: return MGPU_B200_E_UNSUPPORTED;
  }
  return code_of(cudaGetLastError());
}

int mgpu_b200_shard_fold(int dtype, int op, const void* records_device,
  int rank, int world, void* out_device, int num_starts,
  const void* init_host, void* stream) {
  if(!records_device || !out_device || !init_host || rank < 0 ||
    rank >= world || num_starts < 1)
    return MGPU_B200_E_INVALID;
  if(op < MGPU_B200_PLUS || op > MGPU_B200_MIN) return MGPU_B200_E_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  const shard_record_t* rec = (const shard_record_t*)records_device;
  switch(dtype) {
    case MGPU_B200_F32: { float i; memcpy(&i, init_host, 4);
      shard_fold_k<<<1, 32, 0, s>>>(rec, rank, world, op, (float*)out_device,
        num_starts, i); break; }
    case MGPU_B200_F64: { double i; memcpy(&i, init_host, 8);
      shard_fold_k<<<1, 32, 0, s>>>(rec, rank, world, op, (double*)out_device,
        num_starts, i); break; }
    case MGPU_B200_I32: { int i; memcpy(&i, init_host, 4);
      shard_fold_k<<<1, 32, 0, s>>>(rec, rank, world, op, (int*)out_device,
        num_starts, i); break; }
    case MGPU_B200_I64: { long long i; memcpy(&i, init_host, 8);
      shard_fold_k<<<1, 32, 0, s>>>(rec, rank, world, op,
        (long long*)out_device, num_starts, i); break; }
    default: return MGPU_B200_E_UNSUPPORTED;
  }
  return code_of(cudaGetLastError());
}

int mgpu_b200_shard_begin(int dtype, int op, const void* input_device,
  int count, const int* starts_device, int num_starts, void* workspace_device,
  size_t workspace_bytes, void* mailbox_device,
  const void* const* peers_device, int shard, int num_shards,
  int shards_per_gpu, unsigned step, uint64_t timeout_ns, void* stream) {
  return fused_dispatch(dtype, op, mgpu::detail::segreduce_partition_part,
    input_device, count, starts_device, num_starts, nullptr, nullptr,
    workspace_device, workspace_bytes, mailbox_device, peers_device, shard,
    num_shards, shards_per_gpu, step, timeout_ns, stream);
}

int mgpu_b200_shard_finish(int dtype, int op, const void* input_device,
  int count, const int* starts_device, int num_starts, void* out_device,
  const void* init_host, void* workspace_device, size_t workspace_bytes,
  void* mailbox_device, const void* const* peers_device, int shard,
  int num_shards, int shards_per_gpu, unsigned step, uint64_t timeout_ns,
  void* stream) {
  if(!out_device || !init_host) return MGPU_B200_E_INVALID;
  return fused_dispatch(dtype, op, mgpu::detail::segreduce_reduce_part,
    input_device, count, starts_device, num_starts, out_device, init_host,
    workspace_device, workspace_bytes, mailbox_device, peers_device, shard,
    num_shards, shards_per_gpu, step, timeout_ns, stream);
}

int mgpu_b200_mailbox_clear_status(void* mailbox_device, void* stream) {
  if(!mailbox_device) return MGPU_B200_E_INVALID;
  return code_of(cudaMemsetAsync(mailbox_device, 0, 4, (cudaStream_t)stream));
}

} // extern "C"

namespace {
int fused_dispatch(int dtype, int op, int parts, const void* input, int count,
  const int* starts, int num_starts, void* out, const void* init_host,
  void* workspace, size_t workspace_bytes, void* mailbox,
  const void* const* peers, int shard, int num_shards, int per_gpu,
  unsigned step, uint64_t timeout_ns, void* stream) {
  if(!starts || num_starts < 1 || count < 0 || (count && !input) ||
    !workspace || (uintptr_t)workspace % 128 ||
    !chain_ok(mailbox, peers, shard, num_shards, per_gpu, step))
    return MGPU_B200_E_INVALID;
  size_t need = mgpu_b200_segreduce_workspace_bytes(dtype, count, num_starts);
  if(!need) return MGPU_B200_E_UNSUPPORTED;
  if(workspace_bytes < need) return MGPU_B200_E_WORKSPACE;
  cudaStream_t s = (cudaStream_t)stream;
  switch(dtype) {
    case MGPU_B200_F32: return fused_op<float>(op, parts, input, count,
      starts, num_starts, out, init_host, workspace, mailbox, peers, shard,
      num_shards, per_gpu, step, timeout_ns, s);
    case MGPU_B200_F64: return fused_op<double>(op, parts, input, count,
      starts, num_starts, out, init_host, workspace, mailbox, peers, shard,
      num_shards, per_gpu, step, timeout_ns, s);
    case MGPU_B200_I32: return fused_op<int>(op, parts, input, count, starts,
      num_starts, out, init_host, workspace, mailbox, peers, shard,
      num_shards, per_gpu, step, timeout_ns, s);
    case MGPU_B200_I64: return fused_op<long long>(op, parts, input, count,
      starts, num_starts, out, init_host, workspace, mailbox, peers, shard,
      num_shards, per_gpu, step, timeout_ns, s);
  }
  return MGPU_B200_E_UNSUPPORTED;
}
} // namespace
