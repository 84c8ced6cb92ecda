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
#include <cuda_runtime.h>
#include <cstring>

namespace {

enum : uint32_t {
  shard_has_partial = 1,   // out[0] folds at least one item
  shard_has_start = 2,     // at least one segment starts inside the shard
  shard_last_empty = 4     // the last local segment has no local item
};

struct shard_record_t {
  unsigned long long value;   // the partial's bits, zero-padded to 8 bytes
  uint32_t flags;
  uint32_t pad;
};

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
  record->pad = 0;
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

template<typename type_t>
__device__ void lead_write_record(shard_record_t* record, type_t total,
  int lead, bool real, const int* starts, int num_starts, int count) {
  uint32_t flags = 0;
  if(lead > 0) flags |= shard_has_partial;
  if(real) flags |= shard_has_start;
  if(real && starts[num_starts - 1] >= count) flags |= shard_last_empty;
  unsigned long long bits = 0;
  memcpy(&bits, &total, sizeof(type_t));
  record->value = bits;
  record->flags = flags;
  record->pad = 0;
}

template<typename type_t>
__global__ void __launch_bounds__(lead_threads)
shard_lead_k(const type_t* input, const int* starts, int num_starts, int count,
  int op, shard_record_t* record, unsigned long long* chunk_value,
  uint32_t* chunk_has, uint32_t* ticket) {
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
    if(0 == tid)
      lead_write_record(record, acc, lead, real, starts, num_starts, count);
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
  if(0 == tid) {
    lead_write_record(record, acc, lead, real, starts, num_starts, count);
    *ticket = 0;
  }
}

inline int code_of(cudaError_t e) {
  return cudaSuccess == e ? MGPU_B200_OK : MGPU_B200_E_CUDA + (int)e;
}

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
      values, has, ticket); break;
    case MGPU_B200_F64: shard_lead_k<<<lead_ctas, lead_threads, 0, s>>>(
      (const double*)input_device, starts_device, num_starts, count, op, rec,
      values, has, ticket); break;
    case MGPU_B200_I32: shard_lead_k<<<lead_ctas, lead_threads, 0, s>>>(
      (const int*)input_device, starts_device, num_starts, count, op, rec,
      values, has, ticket); break;
    case MGPU_B200_I64: shard_lead_k<<<lead_ctas, lead_threads, 0, s>>>(
      (const long long*)input_device, starts_device, num_starts, count, op,
      rec, values, has, ticket); break;
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

} // extern "C"
