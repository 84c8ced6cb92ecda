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

inline int code_of(cudaError_t e) {
  return cudaSuccess == e ? MGPU_B200_OK : MGPU_B200_E_CUDA + (int)e;
}

} // namespace

extern "C" {

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
