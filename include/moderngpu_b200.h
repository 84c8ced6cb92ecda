/*
 * C ABI of the B200 build of moderngpu's load-balanced segmented-reduction
 * path. Plain pointers and sizes only; every pointer named "device" must be
 * device memory of the current CUDA device, every call is enqueued on the
 * given stream (a cudaStream_t passed as void*, NULL = default stream) and
 * returns without waiting for the device unless stated otherwise.
 *
 * The reference is a header-only C++ template library; it has no FFI of its
 * own. Each entry point below is the pre-instantiated form of one template
 * entry point of the reference, which a binding (ctypes, cgo, JNI ...) would
 * otherwise have to instantiate itself; the C++ templates with the reference's
 * exact signatures live in include/moderngpu/ and accept user functors.
 *
 * Return value: 0 on success, MGPU_B200_E_* below, or 1000 + cudaError_t.
 *
 * Common conventions (reference: tests/test_segreduce.cu:16-22,41-42):
 * `segments` holds num_segments START offsets, segments[0] == 0,
 * non-decreasing, every value <= count; segment s is
 * [segments[s], segments[s+1]) and the last one ends at count.
 * count + num_segments must be below 2^31 - 65536.
 */
#ifndef MODERNGPU_B200_H
#define MODERNGPU_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  MGPU_B200_OK = 0,
  MGPU_B200_E_INVALID = 1,        /* bad argument (null pointer, negative size, size limit) */
  MGPU_B200_E_WORKSPACE = 2,      /* workspace smaller than *_workspace_bytes() */
  MGPU_B200_E_UNSUPPORTED = 3,    /* dtype / op combination not instantiated */
  MGPU_B200_E_DEVICE_STATUS = 4,  /* a kernel recorded a failure, see mgpu_b200_workspace_status */
  MGPU_B200_E_CUDA = 1000         /* 1000 + cudaError_t */
};

/* Element types. */
enum { MGPU_B200_F32 = 0, MGPU_B200_F64 = 1, MGPU_B200_I32 = 2, MGPU_B200_I64 = 3 };

/* Reduction operators: mgpu::plus_t, maximum_t, minimum_t
 * (reference: src/moderngpu/operators.hxx:94-124). */
enum { MGPU_B200_PLUS = 0, MGPU_B200_MAX = 1, MGPU_B200_MIN = 2 };

/* Device-side status words a kernel can record in its workspace. */
enum {
  MGPU_B200_STATUS_OK = 0,
  MGPU_B200_STATUS_LOOKBACK_TIMEOUT = 1,
  MGPU_B200_STATUS_COPY_TIMEOUT = 2
};

/* Library version: major * 10000 + minor * 100 + patch. */
int mgpu_b200_version(void);

/* Static string for a return value of this API. */
const char* mgpu_b200_error_string(int code);

/*
 * mgpu::segreduce (reference: src/moderngpu/kernel_segreduce.hxx:193-268) for
 * a device array of `dtype` elements and one of the built-in operators.
 *   output[s] = fold_op(input[segments[s] .. end of segment s)), or *init for
 *   an empty segment (init is never folded into a non-empty segment).
 * `init` is a HOST pointer to one element of `dtype`.
 * `workspace` is device scratch of at least
 * mgpu_b200_segreduce_workspace_bytes(dtype, count, num_segments) bytes,
 * 128-byte aligned; its contents need not be initialised and are overwritten.
 * Two calls that overlap on the device must not share a workspace.
 */
size_t mgpu_b200_segreduce_workspace_bytes(int dtype, int count, int num_segments);

int mgpu_b200_segreduce(int dtype, int op, const void* input_device, int count,
  const int* segments_device, int num_segments, void* output_device,
  const void* init_host, void* workspace_device, size_t workspace_bytes,
  void* stream);

/*
 * mgpu_b200_segreduce for callers that cannot allocate device memory (no
 * counterpart in the reference, whose temporaries always come from
 * context_t::alloc). Same arguments and results as mgpu_b200_segreduce minus
 * the workspace: the scratch is a fixed block of
 * mgpu_b200_static_scratch_bytes() bytes (4 MiB) of device memory that is
 * part of the loaded library, so every GPU that loads the library holds it
 * until the process exits. The call allocates and frees nothing.
 *  - A problem whose scratch exceeds the block is refused with
 *    MGPU_B200_E_WORKSPACE before anything is launched. The scratch is about
 *    132 bytes per tile (one 128-byte status line + one partition entry), so
 *    the block serves 31,773 tiles: count + num_segments up to 227,494,680
 *    for 4-byte types (tiles of 7,160) and 211,226,904 for 8-byte types
 *    (tiles of 6,648). 2^27 items with 2^22 segments fit; 2^28 items do not.
 *    mgpu_b200_segreduce_workspace_bytes(dtype, count, num_segments) <=
 *    mgpu_b200_static_scratch_bytes() is the exact test.
 *  - All calls on one GPU share the block, which keeps the previous call's
 *    contents; the kernels clear what must start at zero. Calls that overlap
 *    on a GPU (two streams, two host threads) race on it: run them one after
 *    the other, or use mgpu_b200_segreduce with a workspace per stream.
 *  - The block's address is looked up on the first call made with a given
 *    GPU current; make that first call outside any stream capture.
 */
size_t mgpu_b200_static_scratch_bytes(void);

int mgpu_b200_segreduce_static(int dtype, int op, const void* input_device,
  int count, const int* segments_device, int num_segments,
  void* output_device, const void* init_host, void* stream);

/*
 * Diagnostic form of mgpu_b200_segreduce: same arguments and result, but the
 * call waits for the device and reports how long its two kernels ran, as
 * measured by CUDA events on `stream`: the merge-path partitioner
 * (*partition_ms) and the reduction kernel (*reduce_ms). No counterpart in
 * the reference; it exists so that a benchmark can attribute time to the
 * dominant kernel. Either pointer may be NULL. Not safe to call from two
 * host threads at once.
 */
int mgpu_b200_segreduce_profile(int dtype, int op, const void* input_device,
  int count, const int* segments_device, int num_segments, void* output_device,
  const void* init_host, void* workspace_device, size_t workspace_bytes,
  void* stream, float* partition_ms, float* reduce_ms);

/*
 * Reads back the status word of the most recent call that used `workspace`
 * (waits for `stream`). *status receives MGPU_B200_STATUS_*; the return value
 * is MGPU_B200_E_DEVICE_STATUS when it is not MGPU_B200_STATUS_OK.
 */
int mgpu_b200_workspace_status(const void* workspace_device, void* stream,
  int* status);

/*
 * mgpu::load_balance_partitions (reference: src/moderngpu/search.hxx:29-37).
 * Writes div_up(count + num_segments, spacing) + 1 int32 values:
 * partitions[k] = number of items among the first
 * min(k * spacing, count + num_segments) elements of the merge of item
 * indices with segment starts (a start precedes the item of equal index).
 */
int mgpu_b200_load_balance_partitions(int count, const int* segments_device,
  int num_segments, int spacing, int* partitions_device, void* stream);

/*
 * mgpu::spmv (reference: src/moderngpu/kernel_segreduce.hxx:285-298):
 *   y[r] = sum over the non-zeros i of row r of matrix[i] * vector[columns[i]]
 * for a CSR matrix with nnz non-zeros and `rows` rows; row_starts plays the
 * part of `segments` (first non-zero of each row), rows without non-zeros
 * give 0. dtype is MGPU_B200_F32 or MGPU_B200_F64; columns are int32 and are
 * not range-checked. Workspace as for mgpu_b200_segreduce.
 */
size_t mgpu_b200_spmv_workspace_bytes(int dtype, int nnz, int rows);

int mgpu_b200_spmv(int dtype, const void* matrix_device,
  const int* columns_device, const void* vector_device, int nnz,
  const int* row_starts_device, int rows, void* y_device,
  void* workspace_device, size_t workspace_bytes, void* stream);

/*
 * mgpu::lbs_segreduce (reference: src/moderngpu/kernel_segreduce.hxx:303-387)
 * with the functor f(index, seg, rank, tuple<weight>) = values[index] * weight,
 * the weight cached per segment (caching_iterators = tuple<weights>), op plus,
 * init 0:  output[s] = sum over the items i of segment s of
 * values[i] * weights[s]; 0 for an empty segment. The load-balancing search
 * that finds every item's segment is fused into the reduction. dtype is
 * MGPU_B200_F32 or MGPU_B200_F64. Other functors: the C++ header.
 */
size_t mgpu_b200_lbs_segreduce_weighted_workspace_bytes(int dtype, int count,
  int num_segments);

int mgpu_b200_lbs_segreduce_weighted(int dtype, const void* values_device,
  int count, const int* segments_device, int num_segments,
  const void* weights_device, void* output_device, void* workspace_device,
  size_t workspace_bytes, void* stream);

/*
 * mgpu::transform_lbs (reference: src/moderngpu/kernel_load_balance.hxx:8-76)
 * with the functor that records its arguments: for every item index in
 * [0, count), seg_out[index] = (number of segment starts <= index) - 1 and,
 * when rank_out is not NULL, rank_out[index] = index - segments[seg].
 * With rank_out == NULL this is mgpu::load_balance_search (:78-86).
 * Workspace: mgpu_b200_lbs_workspace_bytes(count, num_segments) bytes,
 * 128-byte aligned, contents overwritten.
 */
size_t mgpu_b200_lbs_workspace_bytes(int count, int num_segments);

int mgpu_b200_load_balance_search(int count, const int* segments_device,
  int num_segments, int* seg_out_device, int* rank_out_device,
  void* workspace_device, size_t workspace_bytes, void* stream);

/*
 * mgpu::interval_expand (reference: src/moderngpu/kernel_intervalmove.hxx:
 * 7-20): output[index] = input[segment of index], elements of elem_bytes
 * bytes (1, 2, 4 or 8) copied bit for bit. Workspace as for
 * mgpu_b200_load_balance_search.
 */
int mgpu_b200_interval_expand(int elem_bytes, const void* input_device,
  int count, const int* segments_device, int num_segments,
  void* output_device, void* workspace_device, size_t workspace_bytes,
  void* stream);

/*
 * mgpu::segreduce on HOST arrays: what a caller of the reference does with
 * to_mem / segreduce / from_mem (reference: src/moderngpu/memory.hxx:61-75,
 * tests/test_segreduce.cu:24-38), as one call. input, segments and output
 * are host pointers (pinned memory copies fastest). The call cuts the problem
 * at segment boundaries into chunks of about 32 Mi items and overlaps the
 * copy-in, the reduction and the copy-out of successive chunks on three
 * internal streams of the current device; it returns when output_host holds
 * every result. Device buffers are kept and reused by later calls.
 * `reserved` must be NULL.
 */
int mgpu_b200_segreduce_host(int dtype, int op, const void* input_host,
  int count, const int* segments_host, int num_segments, void* output_host,
  const void* init_host, void* reserved);

/*
 * mgpu::sorted_search (reference: src/moderngpu/kernel_sortedsearch.hxx:7-62)
 * with less-than: for every one of num_needles SORTED keys, the lower bound
 * (upper == 0: number of haystack keys less than it) or the upper bound
 * (upper != 0: number of haystack keys not greater than it) in the SORTED
 * haystack. dtype is MGPU_B200_I32, _I64, _F32 or _F64. Workspace:
 * mgpu_b200_sorted_search_workspace_bytes(num_needles, num_haystack),
 * 128-byte aligned. inner_join and the other callers that need user types
 * are in the C++ headers.
 */
size_t mgpu_b200_sorted_search_workspace_bytes(int num_needles,
  int num_haystack);

int mgpu_b200_sorted_search(int dtype, int upper, const void* needles_device,
  int num_needles, const void* haystack_device, int num_haystack,
  int* indices_device, void* workspace_device, size_t workspace_bytes,
  void* stream);

/*
 * Optional L2 residency for an array that later calls on `stream` gather from
 * at random -- the vector of mgpu_b200_spmv. No counterpart in the reference.
 * mgpu_b200_l2_pin sets aside min(bytes, the device's maximum) of this
 * context's L2 for persisting lines and attaches an access-policy window over
 * the array to the stream; kernels launched on the stream afterwards keep the
 * array's lines in preference to everything they stream through.
 * mgpu_b200_l2_unpin removes the window, releases the persisting lines and
 * returns the set-aside to zero. Both are settings of the calling process's
 * CUDA context only; nothing outlasts the process. A caller that manages the
 * set-aside itself should not use these.
 */
int mgpu_b200_l2_pin(const void* array_device, size_t bytes, void* stream);
int mgpu_b200_l2_unpin(void* stream);

/*
 * mgpu::scan with plus (reference: src/moderngpu/kernel_scan.hxx:159-175):
 * exclusive (inclusive == 0: output[i] = sum of input[0 .. i), output[0] = 0)
 * or inclusive prefix sums of `count` elements of `dtype`; the usual way to
 * turn segment lengths into the start offsets the calls above take.
 * total_device, when not NULL, receives the sum of all elements (0 for
 * count == 0). input and output may be the same array. Workspace:
 * mgpu_b200_scan_workspace_bytes(dtype, count), 128-byte aligned.
 */
size_t mgpu_b200_scan_workspace_bytes(int dtype, int count);

int mgpu_b200_scan(int dtype, int inclusive, const void* input_device,
  int count, void* output_device, void* total_device, void* workspace_device,
  size_t workspace_bytes, void* stream);

/*
 * Multi-GPU layer (no counterpart in the reference, which is single-device).
 * The item range of a large problem is cut across GPUs; GPU r holds count_r
 * items and a shard-local start table `starts` whose entry 0 is always 0 and
 * stands for the segment carried in from the left, followed by the local
 * offsets of the segments that START inside the shard. Each GPU runs
 * mgpu_b200_segreduce on (items, starts): out[0] is then its boundary
 * partial, out[1..] its own segments, the last of which may continue on later
 * GPUs.
 *
 * mgpu_b200_shard_pack writes one 16-byte record {value bits, flags} that
 * describes the shard's boundary: what out[0] holds and whether the shard
 * contains a segment start. The caller exchanges the records of all GPUs
 * (16 bytes per GPU: an all-gather, or peer-to-peer copies into every GPU's
 * own memory) into `records_device`, ordered by shard.
 *
 * mgpu_b200_shard_fold then makes the GPU that owns a straddling segment fold
 * in the partials of the following shards, in shard order:
 *   out[num_starts - 1] = op(out[num_starts - 1], partial_{r+1}, ...)
 * up to and including the first later shard that holds a start of its own.
 * `init_host` is the same init that the reduction used.
 */
int mgpu_b200_shard_pack(int dtype, const void* out_device,
  const int* starts_device, int num_starts, int count, void* record_device,
  void* stream);

/*
 * mgpu_b200_shard_lead writes the same 16-byte record as mgpu_b200_shard_pack,
 * but computes the boundary partial itself from the shard's leading items
 * (those before its first real segment start) instead of reading out[0]. It
 * can therefore run BEFORE the shard's reduction, and the exchange of the
 * records can overlap that reduction. `scratch_device`: at least
 * mgpu_b200_shard_lead_scratch_bytes() bytes, 8-byte aligned, zeroed once
 * before first use (the call leaves it ready for the next one); one scratch
 * per stream. Built-in operators only (they commute).
 */
size_t mgpu_b200_shard_lead_scratch_bytes(void);

int mgpu_b200_shard_lead(int dtype, int op, const void* input_device,
  int count, const int* starts_device, int num_starts, void* record_device,
  void* scratch_device, void* stream);

/*
 * Peer-to-peer exchange of the boundary records (no collective library).
 *
 * Every GPU owns one mailbox: a block of device memory that the other GPUs of
 * the box map into their address space (CUDA IPC) and write into over NVLink.
 * mgpu_b200_mailbox_create allocates and zeroes it on the current device and
 * returns a 64-byte handle; the caller hands the handle to the other
 * processes by whatever means it has, and each of them maps it with
 * mgpu_b200_mailbox_open (close with mgpu_b200_mailbox_close before the
 * owner destroys it). A process must not open its own handle; it uses the
 * pointer mgpu_b200_mailbox_create returned.
 *
 * The array is a chain of num_shards consecutive shards (at most 64),
 * shards_per_gpu of them on each GPU in order; peers_device is a DEVICE array
 * of num_shards / shards_per_gpu mailbox pointers, indexed by GPU, this GPU's
 * own mailbox at its own index. `step` counts the calls: 1 for the first
 * step, one more for each following step, the same on every GPU.
 *
 * mgpu_b200_shard_post reduces the shard's leading items (as
 * mgpu_b200_shard_lead) and stores the record into the mailbox of every GPU
 * that holds this or an earlier shard. mgpu_b200_shard_collect, enqueued
 * after the shard's mgpu_b200_segreduce, waits in THIS GPU's memory for the
 * records of the following shards and folds them into out[num_starts - 1]
 * (as mgpu_b200_shard_fold), then releases the records' slots. Slots are
 * reused after 64 steps; a GPU that runs 64 steps ahead of a reader waits
 * for it. Every wait is bounded: after timeout_ns (0 = 10 s) the kernel
 * gives up, leaves the output untouched and sets the mailbox's status word,
 * which mgpu_b200_mailbox_status reads back (0 fine, 3 = a record did not
 * arrive, 4 = a slot was not released). One mailbox serves one stream.
 */
size_t mgpu_b200_mailbox_bytes(void);
int mgpu_b200_mailbox_create(void** mailbox_device, void* handle_out);
int mgpu_b200_mailbox_open(const void* handle_in, void** peer_device);
int mgpu_b200_mailbox_close(void* peer_device);
int mgpu_b200_mailbox_destroy(void* mailbox_device);
int mgpu_b200_mailbox_status(const void* mailbox_device, void* stream,
  int* status_host);

int mgpu_b200_shard_post(int dtype, int op, const void* input_device,
  int count, const int* starts_device, int num_starts, void* mailbox_device,
  const void* const* peers_device, int shard, int num_shards,
  int shards_per_gpu, unsigned step, uint64_t timeout_ns, void* stream);

int mgpu_b200_shard_collect(int dtype, int op, void* mailbox_device,
  const void* const* peers_device, int shard, int num_shards,
  int shards_per_gpu, unsigned step, void* out_device, int num_starts,
  const void* init_host, uint64_t timeout_ns, void* stream);

int mgpu_b200_shard_fold(int dtype, int op, const void* records_device,
  int rank, int world, void* out_device, int num_starts,
  const void* init_host, void* stream);

/*
 * The fused step: what mgpu_b200_shard_post + mgpu_b200_segreduce +
 * mgpu_b200_shard_collect do in four launches, in two (no counterpart in the
 * reference; the C++ form is mgpu::sharded_segreduce, include/moderngpu/
 * kernel_sharded.hxx).
 *
 * mgpu_b200_shard_begin enqueues the merge-path partitioner of the shard's
 * reduction; a few extra CTAs of the same launch fold the shard's leading
 * items and store the boundary record into the mailboxes (as
 * mgpu_b200_shard_post), and tell the GPUs that hold later shards that this
 * shard is done with step - 1. mgpu_b200_shard_finish enqueues the reduction
 * kernel; the thread that stores out[num_starts - 1] first folds the
 * following shards' records into it (as mgpu_b200_shard_collect, same
 * bounded wait and status word). The two calls of a shard take the same arguments, stream and
 * workspace (mgpu_b200_segreduce_workspace_bytes(dtype, count, num_starts)
 * bytes, 128-byte aligned, one per shard). A GPU that holds several shards
 * calls _begin for all of them, in shard order, before the first _finish: a
 * shard's collect may need the record of a later shard of the same GPU.
 * `step` counts from 1, the same on every GPU; a GPU may run at most 63 steps
 * ahead of a GPU that reads its records.
 */
int mgpu_b200_shard_begin(int dtype, int op, const void* input_device,
  int count, const int* starts_device, int num_starts, void* workspace_device,
  size_t workspace_bytes, void* mailbox_device,
  const void* const* peers_device, int shard, int num_shards,
  int shards_per_gpu, unsigned step, uint64_t timeout_ns, void* stream);

int mgpu_b200_shard_finish(int dtype, int op, const void* input_device,
  int count, const int* starts_device, int num_starts, void* out_device,
  const void* init_host, void* workspace_device, size_t workspace_bytes,
  void* mailbox_device, const void* const* peers_device, int shard,
  int num_shards, int shards_per_gpu, unsigned step, uint64_t timeout_ns,
  void* stream);

/* Returns a mailbox's status word to 0 (enqueued on `stream`), so that a
 * later wait that runs out can be told from an earlier one. */
int mgpu_b200_mailbox_clear_status(void* mailbox_device, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* MODERNGPU_B200_H */
