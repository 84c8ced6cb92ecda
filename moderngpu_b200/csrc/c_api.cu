// C ABI over pre-instantiated fast paths of the template library in
// include/moderngpu/. Declarations and contracts: include/moderngpu_b200.h.
#include <moderngpu_b200.h>
#include <moderngpu/kernel_segreduce.hxx>

using namespace mgpu;

namespace {

inline int cuda_code(cudaError_t e) {
  return cudaSuccess == e ? MGPU_B200_OK : MGPU_B200_E_CUDA + (int)e;
}

inline int last_launch_code() { return cuda_code(cudaGetLastError()); }

// Bound on every device-side wait, in nanoseconds. Adjustable so that tests
// can make a wait run out quickly without hanging anything.
uint64_t g_timeout_ns = detail::default_timeout_ns;

template<typename type_t>
struct type_tuning { typedef typename detail::segreduce_default_tuning<type_t>::type type; };

template<typename type_t>
size_t segreduce_bytes(int count, int num_segments) {
  detail::segreduce_plan_t<typename type_tuning<type_t>::type, type_t>
    plan(count, num_segments);
  return plan.bytes;
}

template<typename type_t, typename op_t>
int segreduce_typed(const void* input, int count, const int* segments,
  int num_segments, void* output, const void* init_host, void* workspace,
  cudaStream_t stream) {
  typedef typename type_tuning<type_t>::type tuning_t;
  type_t init;
  memcpy(&init, init_host, sizeof(type_t));
  detail::array_source_t<type_t> source { (const type_t*)input };
  try {
    detail::segreduce_enqueue<tuning_t>(source, count, segments, num_segments,
      (type_t*)output, op_t(), init, workspace, stream, g_timeout_ns);
  } catch(cuda_exception_t& e) {
    return cuda_code(e.result);
  }
  return last_launch_code();
}

template<typename type_t>
int segreduce_op(int op, const void* input, int count, const int* segments,
  int num_segments, void* output, const void* init_host, void* workspace,
  cudaStream_t stream) {
  switch(op) {
    case MGPU_B200_PLUS:
      return segreduce_typed<type_t, plus_t<type_t> >(input, count, segments,
        num_segments, output, init_host, workspace, stream);
    case MGPU_B200_MAX:
      return segreduce_typed<type_t, maximum_t<type_t> >(input, count,
        segments, num_segments, output, init_host, workspace, stream);
    case MGPU_B200_MIN:
      return segreduce_typed<type_t, minimum_t<type_t> >(input, count,
        segments, num_segments, output, init_host, workspace, stream);
  }
  return MGPU_B200_E_UNSUPPORTED;
}

inline bool sizes_ok(int count, int num_segments) {
  return count >= 0 && num_segments >= 0 &&
    (int64_t)count + num_segments <= (int64_t)0x7fffffff - 65536;
}

} // namespace

extern "C" {

int mgpu_b200_version(void) { return 100; }

const char* mgpu_b200_error_string(int code) {
  switch(code) {
    case MGPU_B200_OK: return "success";
    case MGPU_B200_E_INVALID: return "invalid argument";
    case MGPU_B200_E_WORKSPACE: return "workspace too small";
    case MGPU_B200_E_UNSUPPORTED: return "unsupported dtype or operator";
    case MGPU_B200_E_DEVICE_STATUS: return "a kernel recorded a failure status";
  }
  if(code >= MGPU_B200_E_CUDA)
    return cudaGetErrorString((cudaError_t)(code - MGPU_B200_E_CUDA));
  return "unknown error";
}

// Test hook: bound, in nanoseconds, on every device-side wait of later calls
// (0 restores the default). Returns the previous value. Not part of the
// stable interface.
uint64_t mgpu_b200_debug_set_wait_limit_ns(uint64_t ns) {
  uint64_t old = g_timeout_ns;
  g_timeout_ns = ns ? ns : detail::default_timeout_ns;
  return old;
}

size_t mgpu_b200_segreduce_workspace_bytes(int dtype, int count,
  int num_segments) {
  if(!sizes_ok(count, num_segments)) return 0;
  switch(dtype) {
    case MGPU_B200_F32: return segreduce_bytes<float>(count, num_segments);
    case MGPU_B200_F64: return segreduce_bytes<double>(count, num_segments);
    case MGPU_B200_I32: return segreduce_bytes<int32_t>(count, num_segments);
    case MGPU_B200_I64: return segreduce_bytes<int64_t>(count, num_segments);
  }
  return 0;
}

int mgpu_b200_segreduce(int dtype, int op, const void* input_device, int count,
  const int* segments_device, int num_segments, void* output_device,
  const void* init_host, void* workspace_device, size_t workspace_bytes,
  void* stream) {
  if(!sizes_ok(count, num_segments) || !init_host) return MGPU_B200_E_INVALID;
  if(0 == count + num_segments) return MGPU_B200_OK;
  if((count && !input_device) || (num_segments && !segments_device) ||
    (num_segments && !output_device) || !workspace_device)
    return MGPU_B200_E_INVALID;
  if((uintptr_t)workspace_device % 128) return MGPU_B200_E_INVALID;
  size_t need = mgpu_b200_segreduce_workspace_bytes(dtype, count, num_segments);
  if(!need) return MGPU_B200_E_UNSUPPORTED;
  if(workspace_bytes < need) return MGPU_B200_E_WORKSPACE;

  cudaStream_t s = (cudaStream_t)stream;
  switch(dtype) {
    case MGPU_B200_F32:
      return segreduce_op<float>(op, input_device, count, segments_device,
        num_segments, output_device, init_host, workspace_device, s);
    case MGPU_B200_F64:
      return segreduce_op<double>(op, input_device, count, segments_device,
        num_segments, output_device, init_host, workspace_device, s);
    case MGPU_B200_I32:
      return segreduce_op<int32_t>(op, input_device, count, segments_device,
        num_segments, output_device, init_host, workspace_device, s);
    case MGPU_B200_I64:
      return segreduce_op<int64_t>(op, input_device, count, segments_device,
        num_segments, output_device, init_host, workspace_device, s);
  }
  return MGPU_B200_E_UNSUPPORTED;
}

int mgpu_b200_workspace_status(const void* workspace_device, void* stream,
  int* status) {
  if(!workspace_device || !status) return MGPU_B200_E_INVALID;
  uint32_t word = 0;
  cudaError_t e = cudaMemcpyAsync(&word, (const uint32_t*)workspace_device + 1,
    sizeof(word), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if(cudaSuccess == e) e = cudaStreamSynchronize((cudaStream_t)stream);
  if(cudaSuccess != e) return cuda_code(e);
  *status = (int)word;
  return word ? MGPU_B200_E_DEVICE_STATUS : MGPU_B200_OK;
}

int mgpu_b200_load_balance_partitions(int count, const int* segments_device,
  int num_segments, int spacing, int* partitions_device, void* stream) {
  if(!sizes_ok(count, num_segments) || spacing <= 0 || !partitions_device ||
    (num_segments && !segments_device))
    return MGPU_B200_E_INVALID;
  int num_partitions =
    (int)div_up((int64_t)count + num_segments, (int64_t)spacing) + 1;
  detail::launch_lbs_partition(segments_device, count, num_segments,
    (int64_t)spacing, num_partitions, partitions_device,
    (cudaStream_t)stream);
  return last_launch_code();
}

} // extern "C"
