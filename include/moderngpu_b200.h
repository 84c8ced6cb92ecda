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

#ifdef __cplusplus
}
#endif

#endif /* MODERNGPU_B200_H */
