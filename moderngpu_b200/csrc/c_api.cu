// C ABI over pre-instantiated fast paths of the template library in
// include/moderngpu/. Declarations and contracts: include/moderngpu_b200.h.
#include <atomic>
#include <moderngpu_b200.h>
#include <moderngpu/kernel_segreduce.hxx>
#include <moderngpu/kernel_load_balance.hxx>
#include <moderngpu/kernel_intervalmove.hxx>
#include <moderngpu/kernel_scan.hxx>
#include <moderngpu/kernel_sortedsearch.hxx>
#include <moderngpu/b200/lbs_segreduce.hxx>
#include <mutex>
#include <vector>
#include <algorithm>

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

// Event recorded between the partition kernel and the reduction kernel of the
// next segreduce call (diagnostic entry point only).
cudaEvent_t g_between = nullptr;

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
      (type_t*)output, op_t(), init, workspace, stream, g_timeout_ns,
      g_between);
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

////////////////////////////////////////////////////////////////////////////////
// spmv: matrix values and column indices staged by bulk copies, products
// matrix[i] * x[columns[i]] formed in shared memory by the reduction kernel's
// consumer threads (reference: src/moderngpu/kernel_segreduce.hxx:285-298).

template<typename type_t>
size_t spmv_bytes(int nnz, int rows) {
  detail::segreduce_plan_t<typename detail::spmv_default_tuning<type_t>::type,
    type_t> plan(nnz, rows);
  return plan.bytes;
}

// Set while mgpu_b200_l2_pin is in effect (process-wide, like the set-aside).
std::atomic<int> g_l2_pinned(0);

template<typename type_t>
int spmv_typed(const void* matrix, const int* columns, const void* x, int nnz,
  const int* row_starts, int rows, void* y, void* workspace,
  cudaStream_t stream) {
  typedef typename detail::spmv_default_tuning<type_t>::type tuning_t;
  // While the caller holds x in the L2 (mgpu_b200_l2_pin) the matrix's streams
  // cannot push it out, and two stage buffers per CTA pay again (2^24 rows x
  // 16 non-zeros, fp32: 1.28 ms against 1.36 ms with the default shape). The
  // two shapes have the same tile size, hence the same workspace.
  typedef segreduce_tuning_t<tuning_t::nt, tuning_t::vt, 2,
    (tuning_t::occ < 3 ? tuning_t::occ : 3)> pinned_tuning_t;
  static_assert((int)pinned_tuning_t::nv == (int)tuning_t::nv, "same tiles");
  detail::spmv_source_t<type_t> source { (const type_t*)matrix, columns,
    (const type_t*)x };
  try {
    if(g_l2_pinned.load())
      detail::segreduce_enqueue<pinned_tuning_t>(source, nnz, row_starts, rows,
        (type_t*)y, plus_t<type_t>(), (type_t)0, workspace, stream,
        g_timeout_ns);
    else
      detail::segreduce_enqueue<tuning_t>(source, nnz, row_starts, rows,
        (type_t*)y, plus_t<type_t>(), (type_t)0, workspace, stream,
        g_timeout_ns);
  } catch(cuda_exception_t& e) {
    return cuda_code(e.result);
  }
  return last_launch_code();
}

// lbs_segreduce with a cached per-segment weight:
// f(index, seg, rank, tuple<weight>) = values[index] * weight.
template<typename type_t>
struct weighted_item_t {
  const type_t* values;
  MGPU_DEVICE type_t operator()(int index, int seg, int rank,
    tuple<type_t> weight) const {
    // Every value is read once: a streaming load (evict-first).
    return __ldcs(values + index) * get<0>(weight);
  }
};

template<typename type_t>
struct weighted_types {
  typedef typename detail::lbs_segreduce_default_tuning<type_t>::type tuning_t;
  typedef detail::lbs_source_t<weighted_item_t<type_t>,
    tuple<const type_t*>, type_t> source_t;
};

template<typename type_t>
size_t weighted_bytes(int count, int num_segments) {
  detail::segreduce_plan_t<typename weighted_types<type_t>::tuning_t, type_t>
    plan(count, num_segments);
  return plan.bytes;
}

template<typename type_t>
int weighted_typed(const void* values, int count, const int* segments,
  int num_segments, const void* weights, void* output, void* workspace,
  cudaStream_t stream) {
  typedef weighted_types<type_t> types;
  typename types::source_t source { weighted_item_t<type_t> {
    (const type_t*)values }, make_tuple((const type_t*)weights),
    tuple<>() };
  try {
    detail::segreduce_enqueue<typename types::tuning_t>(source, count,
      segments, num_segments, (type_t*)output, plus_t<type_t>(), (type_t)0,
      workspace, stream, g_timeout_ns);
  } catch(cuda_exception_t& e) {
    return cuda_code(e.result);
  }
  return last_launch_code();
}

////////////////////////////////////////////////////////////////////////////////
// Load-balancing search functors.

template<typename elem_t>
struct expand_t {
  elem_t* output;
  MGPU_DEVICE void operator()(int index, int seg, int rank,
    tuple<elem_t> value) const {
    output[index] = get<0>(value);
  }
};

typedef detail::lbs_default_tuning lbs_tuning;
// The smallest fill tile (interval_expand of 8-byte values): lbs_bytes sizes
// the partition table for it, which serves every larger tile too.
typedef detail::lbs_fill_tuning_for<detail::lbs_fill_values, 8>::type
  fill_tuning;
static_assert((int)fill_tuning::nv <=
  (int)detail::lbs_fill_tuning_for<detail::lbs_fill_values, 4>::type::nv &&
  (int)fill_tuning::nv <=
  (int)detail::lbs_fill_tuning_for<detail::lbs_fill_ids>::type::nv &&
  (int)fill_tuning::nv <=
  (int)detail::lbs_fill_tuning_for<detail::lbs_fill_ids_ranks>::type::nv,
  "lbs_bytes sizes the partition table for the smallest tile");

// 4- and 8-byte elements go through the fill kernel (tile output by bulk
// copy), 1- and 2-byte elements through the generic functor path.
template<typename elem_t>
int expand_fill(const void* input, int count, const int* segments,
  int num_segments, void* output, void* workspace, cudaStream_t stream) {
  // The header (ticket counter, status word) is cleared by the partitioner.
  int* partitions = (int*)((char*)workspace + 128);
  detail::lbs_fill_args_t<detail::lbs_fill_values, elem_t> out = { };
  out.values = (const elem_t*)input;
  out.expanded = (elem_t*)output;
  try {
    detail::lbs_fill_enqueue<typename detail::lbs_fill_tuning_for<
      detail::lbs_fill_values, (int)sizeof(elem_t)>::type>(out, count, segments,
      num_segments, (uint32_t*)workspace, partitions, stream, g_timeout_ns);
  } catch(cuda_exception_t& e) {
    return cuda_code(e.result);
  }
  return last_launch_code();
}

template<typename elem_t>
int expand_typed(const void* input, int count, const int* segments,
  int num_segments, void* output, void* workspace, cudaStream_t stream) {
  uint32_t* status = (uint32_t*)workspace + 1;
  int* partitions = (int*)((char*)workspace + 128);
  cudaError_t cleared = cudaMemsetAsync(workspace, 0, 128, stream);
  if(cudaSuccess != cleared) return cuda_code(cleared);
  try {
    detail::transform_lbs_enqueue<lbs_tuning>(
      expand_t<elem_t> { (elem_t*)output }, count, segments, num_segments,
      make_tuple((const elem_t*)input), partitions, stream, g_timeout_ns,
      status);
  } catch(cuda_exception_t& e) {
    return cuda_code(e.result);
  }
  return last_launch_code();
}

inline size_t lbs_bytes(int count, int num_segments) {
  // Serves the generic tiles and the (slightly smaller) fill tiles.
  enum { nv = (int)fill_tuning::nv < (int)lbs_tuning::nv ?
    (int)fill_tuning::nv : (int)lbs_tuning::nv };
  return 128 + (detail::lbs_partition_bytes(count, num_segments, nv) + 127) /
    128 * 128;
}

////////////////////////////////////////////////////////////////////////////////
// Host-buffer segreduce: the arrays live in host memory; the call cuts the
// problem at segment boundaries into chunks, and pipelines
// copy-in / reduce / copy-out of successive chunks over three streams.

template<typename type_t>
__global__ void rebase_offsets_k(int* offsets, int n, int base) {
  int i = (int)(blockIdx.x * blockDim.x + threadIdx.x);
  if(i < n) offsets[i] -= base;
}

struct host_slot_t {
  cudaStream_t stream = nullptr;
  void* items = nullptr;
  int* offsets = nullptr;
  void* output = nullptr;
  void* workspace = nullptr;
  size_t items_cap = 0, offsets_cap = 0, output_cap = 0, workspace_cap = 0;
};

struct host_pipeline_t {
  enum { slots = 3 };
  host_slot_t slot[slots];
  int device = -1;
};

std::mutex g_host_mutex;
host_pipeline_t g_host_pipeline[16];

cudaError_t grow(void** p, size_t* cap, size_t need) {
  if(*cap >= need) return cudaSuccess;
  if(*p) cudaFree(*p);
  *p = nullptr;
  *cap = 0;
  size_t want = need + need / 4 + 256;
  cudaError_t e = cudaMalloc(p, want);
  if(cudaSuccess == e) *cap = want;
  return e;
}

int segreduce_dispatch(int dtype, int op, const void* input, int count,
  const int* segments, int num_segments, void* output, const void* init_host,
  void* workspace, cudaStream_t stream);

size_t elem_size(int dtype) {
  switch(dtype) {
    case MGPU_B200_F32: case MGPU_B200_I32: return 4;
    case MGPU_B200_F64: case MGPU_B200_I64: return 8;
  }
  return 0;
}

int segreduce_host_impl(int dtype, int op, const char* input, int count,
  const int* segments, int num_segments, char* output,
  const void* init_host) {
  const size_t es = elem_size(dtype);
  if(!es) return MGPU_B200_E_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_host_mutex);

  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if(cudaSuccess != e) return cuda_code(e);
  if(device < 0 || device >= 16) return MGPU_B200_E_UNSUPPORTED;
  host_pipeline_t& pipe = g_host_pipeline[device];
  if(pipe.device != device) {
    for(auto& s : pipe.slot) {
      e = cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking);
      if(cudaSuccess != e) return cuda_code(e);
    }
    pipe.device = device;
  }

  // Chunks of about 32 Mi items, cut where a segment starts.
  const int target = 32 << 20;
  std::vector<int> cut;        // first segment of each chunk, then the end
  cut.push_back(0);
  while(cut.back() < num_segments) {
    int s0 = cut.back();
    int64_t want = (int64_t)segments[s0] + target;
    const int* hit = std::lower_bound(segments + s0 + 1,
      segments + num_segments, want > count ? count : (int)want);
    int s1 = (int)(hit - segments);
    if(s1 <= s0) s1 = s0 + 1;
    // Keep trailing empty segments at the array's end in the last chunk.
    if(want >= count) s1 = num_segments;
    cut.push_back(s1);
  }

  int code = MGPU_B200_OK;
  for(size_t c = 0; c + 1 < cut.size() && MGPU_B200_OK == code; ++c) {
    host_slot_t& s = pipe.slot[c % host_pipeline_t::slots];
    int s0 = cut[c], s1 = cut[c + 1];
    int item0 = segments[s0];
    int item1 = s1 < num_segments ? segments[s1] : count;
    int n_items = item1 - item0, n_segs = s1 - s0;
    size_t ws_need = mgpu_b200_segreduce_workspace_bytes(dtype, n_items,
      n_segs);
    // The slot's previous chunk must be finished before its buffers change.
    e = cudaStreamSynchronize(s.stream);
    if(cudaSuccess == e) e = grow(&s.items, &s.items_cap, (size_t)n_items * es + 64);
    if(cudaSuccess == e) e = grow((void**)&s.offsets, &s.offsets_cap, (size_t)n_segs * 4 + 64);
    if(cudaSuccess == e) e = grow(&s.output, &s.output_cap, (size_t)n_segs * es + 64);
    if(cudaSuccess == e) e = grow(&s.workspace, &s.workspace_cap, ws_need + 256);
    if(cudaSuccess == e && n_items)
      e = cudaMemcpyAsync(s.items, input + (size_t)item0 * es,
        (size_t)n_items * es, cudaMemcpyHostToDevice, s.stream);
    if(cudaSuccess == e)
      e = cudaMemcpyAsync(s.offsets, segments + s0, (size_t)n_segs * 4,
        cudaMemcpyHostToDevice, s.stream);
    if(cudaSuccess != e) { code = cuda_code(e); break; }
    if(item0)
      rebase_offsets_k<int><<<div_up(n_segs, 256), 256, 0, s.stream>>>(
        s.offsets, n_segs, item0);
    code = segreduce_dispatch(dtype, op, s.items, n_items, s.offsets, n_segs,
      s.output, init_host, s.workspace, s.stream);
    if(MGPU_B200_OK != code) break;
    e = cudaMemcpyAsync(output + (size_t)s0 * es, s.output,
      (size_t)n_segs * es, cudaMemcpyDeviceToHost, s.stream);
    if(cudaSuccess != e) code = cuda_code(e);
  }
  for(auto& s : pipe.slot) {
    e = cudaStreamSynchronize(s.stream);
    if(cudaSuccess != e && MGPU_B200_OK == code) code = cuda_code(e);
  }
  return code;
}


// Diagnostic kernel: one warp looks back from tile `tile` over a tile-status
// array in which nothing was ever published, so its bounded wait must run out
// and leave status_lookback_timeout in *status. Nothing spins forever and
// nothing faults; the context stays usable.
__global__ void lookback_probe_k(void* state_words, int tile,
  uint64_t timeout_ns, uint32_t* status, int* returned) {
  detail::tile_state_t<float> state;
  state.bind(state_words, tile + 1);
  float carry = 0;
  bool have = detail::lookback(state, tile, plus_t<float>(), carry, timeout_ns,
    status);
  if(0 == threadIdx.x) *returned = have ? 1 : 0;
}

template<typename type_t>
int scan_typed(int inclusive, const void* input, int count, void* output,
  void* total, void* workspace, cudaStream_t stream) {
  typedef detail::scan_route_t<empty_t, type_t, const type_t*, type_t*> route_t;
  try {
    if(total) {
      if(inclusive)
        detail::scan_dispatch<route_t, scan_type_inc, type_t>(
          (const type_t*)input, count, (type_t*)output, plus_t<type_t>(),
          (type_t*)total, workspace, stream, g_timeout_ns);
      else
        detail::scan_dispatch<route_t, scan_type_exc, type_t>(
          (const type_t*)input, count, (type_t*)output, plus_t<type_t>(),
          (type_t*)total, workspace, stream, g_timeout_ns);
    } else {
      discard_iterator_t<type_t> nowhere;
      if(inclusive)
        detail::scan_dispatch<route_t, scan_type_inc, type_t>(
          (const type_t*)input, count, (type_t*)output, plus_t<type_t>(),
          nowhere, workspace, stream, g_timeout_ns);
      else
        detail::scan_dispatch<route_t, scan_type_exc, type_t>(
          (const type_t*)input, count, (type_t*)output, plus_t<type_t>(),
          nowhere, workspace, stream, g_timeout_ns);
    }
  } catch(cuda_exception_t& e) {
    return cuda_code(e.result);
  }
  return last_launch_code();
}

template<typename type_t>
size_t scan_bytes(int count) {
  return detail::scan_workspace_bytes<
    typename detail::scan_default_tuning<type_t>::type, type_t>(count);
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

  return segreduce_dispatch(dtype, op, input_device, count, segments_device,
    num_segments, output_device, init_host, workspace_device,
    (cudaStream_t)stream);
}

int mgpu_b200_segreduce_profile(int dtype, int op, const void* input_device,
  int count, const int* segments_device, int num_segments, void* output_device,
  const void* init_host, void* workspace_device, size_t workspace_bytes,
  void* stream, float* partition_ms, float* reduce_ms) {
  cudaStream_t s = (cudaStream_t)stream;
  cudaEvent_t ev[3];
  for(auto& e : ev) {
    cudaError_t c = cudaEventCreate(&e);
    if(cudaSuccess != c) return cuda_code(c);
  }
  cudaEventRecord(ev[0], s);
  g_between = ev[1];
  int code = mgpu_b200_segreduce(dtype, op, input_device, count,
    segments_device, num_segments, output_device, init_host, workspace_device,
    workspace_bytes, stream);
  g_between = nullptr;
  cudaEventRecord(ev[2], s);
  cudaError_t c = cudaEventSynchronize(ev[2]);
  if(MGPU_B200_OK == code && cudaSuccess != c) code = cuda_code(c);
  if(MGPU_B200_OK == code) {
    float a = 0, b = 0;
    if(cudaSuccess != cudaEventElapsedTime(&a, ev[0], ev[1])) a = 0;
    if(cudaSuccess != cudaEventElapsedTime(&b, ev[1], ev[2])) b = 0;
    if(partition_ms) *partition_ms = a;
    if(reduce_ms) *reduce_ms = b;
  }
  for(auto& e : ev) cudaEventDestroy(e);
  return code;
}

// Test hook (not part of the stable interface): runs the look-back of a
// single warp against `tiles` unpublished tile-status words held in
// workspace_device (at least 128 * tiles + 256 bytes, 128-byte aligned) with
// the given bound on its wait, waits for it, and returns the status word the
// kernel recorded (MGPU_B200_STATUS_LOOKBACK_TIMEOUT is the expected answer).
int mgpu_b200_debug_lookback_timeout(void* workspace_device, int tiles,
  uint64_t timeout_ns, int* status_host, void* stream) {
  if(!workspace_device || !status_host || tiles < 1 || tiles > 1024 ||
    (uintptr_t)workspace_device % 128)
    return MGPU_B200_E_INVALID;
  cudaStream_t s = (cudaStream_t)stream;
  size_t bytes = (size_t)tiles * 128 + 256;
  cudaError_t e = cudaMemsetAsync(workspace_device, 0, bytes, s);
  if(cudaSuccess != e) return cuda_code(e);
  char* base = (char*)workspace_device;
  uint32_t* status = (uint32_t*)base;
  int* returned = (int*)(base + 64);
  lookback_probe_k<<<1, 32, 0, s>>>(base + 256, tiles, timeout_ns, status,
    returned);
  uint32_t word[17] = { };
  e = cudaMemcpyAsync(word, base, sizeof(word), cudaMemcpyDeviceToHost, s);
  if(cudaSuccess == e) e = cudaStreamSynchronize(s);
  if(cudaSuccess != e) return cuda_code(e);
  *status_host = (int)word[0];
  return word[16] ? MGPU_B200_E_DEVICE_STATUS : MGPU_B200_OK;
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

namespace {
int segreduce_dispatch(int dtype, int op, const void* input, int count,
  const int* segments, int num_segments, void* output, const void* init_host,
  void* workspace, cudaStream_t s) {
  switch(dtype) {
    case MGPU_B200_F32:
      return segreduce_op<float>(op, input, count, segments, num_segments,
        output, init_host, workspace, s);
    case MGPU_B200_F64:
      return segreduce_op<double>(op, input, count, segments, num_segments,
        output, init_host, workspace, s);
    case MGPU_B200_I32:
      return segreduce_op<int32_t>(op, input, count, segments, num_segments,
        output, init_host, workspace, s);
    case MGPU_B200_I64:
      return segreduce_op<int64_t>(op, input, count, segments, num_segments,
        output, init_host, workspace, s);
  }
  return MGPU_B200_E_UNSUPPORTED;
}
} // namespace

extern "C" {

size_t mgpu_b200_spmv_workspace_bytes(int dtype, int nnz, int rows) {
  if(!sizes_ok(nnz, rows)) return 0;
  if(MGPU_B200_F32 == dtype) return spmv_bytes<float>(nnz, rows);
  if(MGPU_B200_F64 == dtype) return spmv_bytes<double>(nnz, rows);
  return 0;
}

int mgpu_b200_spmv(int dtype, const void* matrix_device,
  const int* columns_device, const void* vector_device, int nnz,
  const int* row_starts_device, int rows, void* y_device,
  void* workspace_device, size_t workspace_bytes, void* stream) {
  if(!sizes_ok(nnz, rows)) return MGPU_B200_E_INVALID;
  if(0 == nnz + rows) return MGPU_B200_OK;
  if((nnz && (!matrix_device || !columns_device || !vector_device)) ||
    (rows && (!row_starts_device || !y_device)) || !workspace_device ||
    (uintptr_t)workspace_device % 128)
    return MGPU_B200_E_INVALID;
  if(MGPU_B200_F32 != dtype && MGPU_B200_F64 != dtype)
    return MGPU_B200_E_UNSUPPORTED;
  if(workspace_bytes < mgpu_b200_spmv_workspace_bytes(dtype, nnz, rows))
    return MGPU_B200_E_WORKSPACE;
  cudaStream_t s = (cudaStream_t)stream;
  if(MGPU_B200_F32 == dtype)
    return spmv_typed<float>(matrix_device, columns_device, vector_device,
      nnz, row_starts_device, rows, y_device, workspace_device, s);
  return spmv_typed<double>(matrix_device, columns_device, vector_device, nnz,
    row_starts_device, rows, y_device, workspace_device, s);
}

size_t mgpu_b200_lbs_segreduce_weighted_workspace_bytes(int dtype, int count,
  int num_segments) {
  if(!sizes_ok(count, num_segments)) return 0;
  if(MGPU_B200_F32 == dtype) return weighted_bytes<float>(count, num_segments);
  if(MGPU_B200_F64 == dtype) return weighted_bytes<double>(count, num_segments);
  return 0;
}

int mgpu_b200_lbs_segreduce_weighted(int dtype, const void* values_device,
  int count, const int* segments_device, int num_segments,
  const void* weights_device, void* output_device, void* workspace_device,
  size_t workspace_bytes, void* stream) {
  if(!sizes_ok(count, num_segments)) return MGPU_B200_E_INVALID;
  if(0 == count + num_segments) return MGPU_B200_OK;
  if((count && !values_device) ||
    (num_segments && (!segments_device || !weights_device || !output_device)) ||
    !workspace_device || (uintptr_t)workspace_device % 128)
    return MGPU_B200_E_INVALID;
  if(MGPU_B200_F32 != dtype && MGPU_B200_F64 != dtype)
    return MGPU_B200_E_UNSUPPORTED;
  if(workspace_bytes <
    mgpu_b200_lbs_segreduce_weighted_workspace_bytes(dtype, count, num_segments))
    return MGPU_B200_E_WORKSPACE;
  cudaStream_t s = (cudaStream_t)stream;
  if(MGPU_B200_F32 == dtype)
    return weighted_typed<float>(values_device, count, segments_device,
      num_segments, weights_device, output_device, workspace_device, s);
  return weighted_typed<double>(values_device, count, segments_device,
    num_segments, weights_device, output_device, workspace_device, s);
}

size_t mgpu_b200_lbs_workspace_bytes(int count, int num_segments) {
  if(!sizes_ok(count, num_segments)) return 0;
  return lbs_bytes(count, num_segments);
}

int mgpu_b200_load_balance_search(int count, const int* segments_device,
  int num_segments, int* seg_out_device, int* rank_out_device,
  void* workspace_device, size_t workspace_bytes, void* stream) {
  if(!sizes_ok(count, num_segments)) return MGPU_B200_E_INVALID;
  if(0 == count + num_segments) return MGPU_B200_OK;
  if((count && !seg_out_device) || (num_segments && !segments_device) ||
    !workspace_device || (uintptr_t)workspace_device % 128)
    return MGPU_B200_E_INVALID;
  if(workspace_bytes < lbs_bytes(count, num_segments))
    return MGPU_B200_E_WORKSPACE;
  cudaStream_t s = (cudaStream_t)stream;
  // The header (ticket counter, status word) is cleared by the partitioner.
  uint32_t* header = (uint32_t*)workspace_device;
  int* partitions = (int*)((char*)workspace_device + 128);
  try {
    if(rank_out_device) {
      detail::lbs_fill_args_t<detail::lbs_fill_ids_ranks, int> out = { };
      out.ids = seg_out_device;
      out.ranks = rank_out_device;
      detail::lbs_fill_enqueue<
        detail::lbs_fill_tuning_for<detail::lbs_fill_ids_ranks>::type>(out,
        count, segments_device, num_segments, header, partitions, s,
        g_timeout_ns);
    } else {
      detail::lbs_fill_args_t<detail::lbs_fill_ids, int> out = { };
      out.ids = seg_out_device;
      detail::lbs_fill_enqueue<
        detail::lbs_fill_tuning_for<detail::lbs_fill_ids>::type>(out, count,
        segments_device, num_segments, header, partitions, s, g_timeout_ns);
    }
  } catch(cuda_exception_t& e) {
    return cuda_code(e.result);
  }
  return last_launch_code();
}

int mgpu_b200_interval_expand(int elem_bytes, const void* input_device,
  int count, const int* segments_device, int num_segments,
  void* output_device, void* workspace_device, size_t workspace_bytes,
  void* stream) {
  if(!sizes_ok(count, num_segments)) return MGPU_B200_E_INVALID;
  if(0 == count + num_segments) return MGPU_B200_OK;
  if((count && !output_device) ||
    (num_segments && (!segments_device || !input_device)) ||
    !workspace_device || (uintptr_t)workspace_device % 128)
    return MGPU_B200_E_INVALID;
  if(workspace_bytes < lbs_bytes(count, num_segments))
    return MGPU_B200_E_WORKSPACE;
  cudaStream_t s = (cudaStream_t)stream;
  switch(elem_bytes) {
    case 1: return expand_typed<uint8_t>(input_device, count, segments_device,
      num_segments, output_device, workspace_device, s);
    case 2: return expand_typed<uint16_t>(input_device, count, segments_device,
      num_segments, output_device, workspace_device, s);
    case 4: return expand_fill<uint32_t>(input_device, count, segments_device,
      num_segments, output_device, workspace_device, s);
    case 8: return expand_fill<uint64_t>(input_device, count, segments_device,
      num_segments, output_device, workspace_device, s);
  }
  return MGPU_B200_E_UNSUPPORTED;
}

int mgpu_b200_segreduce_host(int dtype, int op, const void* input_host,
  int count, const int* segments_host, int num_segments, void* output_host,
  const void* init_host, void* reserved) {
  (void)reserved;
  if(!sizes_ok(count, num_segments) || !init_host) return MGPU_B200_E_INVALID;
  if(0 == num_segments) return MGPU_B200_OK;
  if((count && !input_host) || !segments_host || !output_host)
    return MGPU_B200_E_INVALID;
  return segreduce_host_impl(dtype, op, (const char*)input_host, count,
    segments_host, num_segments, (char*)output_host, init_host);
}

size_t mgpu_b200_sorted_search_workspace_bytes(int num_needles,
  int num_haystack) {
  if(num_needles < 0 || num_haystack < 0) return 0;
  // 128-byte header (status word, as in the other calls) + partition table.
  return 128 + (detail::sorted_search_partitions<>(num_needles, num_haystack) *
    sizeof(int) + 127) / 128 * 128;
}

int mgpu_b200_sorted_search(int dtype, int upper, const void* needles_device,
  int num_needles, const void* haystack_device, int num_haystack,
  int* indices_device, void* workspace_device, size_t workspace_bytes,
  void* stream) {
  if(!sizes_ok(num_needles, num_haystack)) return MGPU_B200_E_INVALID;
  if(0 == num_needles) return MGPU_B200_OK;
  if(!needles_device || !indices_device ||
    (num_haystack && !haystack_device) || !workspace_device)
    return MGPU_B200_E_INVALID;
  if(workspace_bytes <
    mgpu_b200_sorted_search_workspace_bytes(num_needles, num_haystack))
    return MGPU_B200_E_WORKSPACE;
  if((uintptr_t)workspace_device % 128) return MGPU_B200_E_INVALID;
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t cleared = cudaMemsetAsync(workspace_device, 0, 128, s);
  if(cudaSuccess != cleared) return cuda_code(cleared);
  uint32_t* status = (uint32_t*)workspace_device + 1;
  int* partitions = (int*)((char*)workspace_device + 128);
  #define MGPU_B200_SEARCH(type_t) \
    if(upper) detail::sorted_search_enqueue<bounds_upper, \
      detail::search_tuning_for<type_t>::type>( \
      (const type_t*)needles_device, num_needles, \
      (const type_t*)haystack_device, num_haystack, indices_device, \
      less_t<type_t>(), partitions, s, g_timeout_ns, status); \
    else detail::sorted_search_enqueue<bounds_lower, \
      detail::search_tuning_for<type_t>::type>( \
      (const type_t*)needles_device, num_needles, \
      (const type_t*)haystack_device, num_haystack, indices_device, \
      less_t<type_t>(), partitions, s, g_timeout_ns, status);
  try {
    switch(dtype) {
      case MGPU_B200_I32: MGPU_B200_SEARCH(int) break;
      case MGPU_B200_I64: MGPU_B200_SEARCH(long long) break;
      case MGPU_B200_F32: MGPU_B200_SEARCH(float) break;
      case MGPU_B200_F64: MGPU_B200_SEARCH(double) break;
      default: return MGPU_B200_E_UNSUPPORTED;
    }
  } catch(cuda_exception_t& e) {
    return cuda_code(e.result);
  }
  #undef MGPU_B200_SEARCH
  return last_launch_code();
}

int mgpu_b200_l2_pin(const void* array_device, size_t bytes, void* stream) {
  if(!array_device || !bytes) return MGPU_B200_E_INVALID;
  int device = 0, max_persisting = 0, max_window = 0;
  cudaError_t e = cudaGetDevice(&device);
  if(cudaSuccess == e) e = cudaDeviceGetAttribute(&max_persisting,
    cudaDevAttrMaxPersistingL2CacheSize, device);
  if(cudaSuccess == e) e = cudaDeviceGetAttribute(&max_window,
    cudaDevAttrMaxAccessPolicyWindowSize, device);
  if(cudaSuccess != e) return cuda_code(e);
  if(max_persisting <= 0 || max_window <= 0) return MGPU_B200_E_UNSUPPORTED;
  size_t set_aside = bytes < (size_t)max_persisting ? bytes :
    (size_t)max_persisting;
  e = cudaDeviceSetLimit(cudaLimitPersistingL2CacheSize, set_aside);
  if(cudaSuccess != e) return cuda_code(e);
  cudaStreamAttrValue value = { };
  value.accessPolicyWindow.base_ptr = const_cast<void*>(array_device);
  value.accessPolicyWindow.num_bytes = bytes < (size_t)max_window ? bytes :
    (size_t)max_window;
  // Only as large a share of the window as the set-aside can hold is marked
  // persisting; the rest streams, so the persisting lines do not evict each
  // other.
  value.accessPolicyWindow.hitRatio =
    (float)((double)set_aside / (double)value.accessPolicyWindow.num_bytes);
  if(value.accessPolicyWindow.hitRatio > 1.0f)
    value.accessPolicyWindow.hitRatio = 1.0f;
  value.accessPolicyWindow.hitProp = cudaAccessPropertyPersisting;
  value.accessPolicyWindow.missProp = cudaAccessPropertyStreaming;
  e = cudaStreamSetAttribute((cudaStream_t)stream,
    cudaStreamAttributeAccessPolicyWindow, &value);
  if(cudaSuccess == e) g_l2_pinned.store(1);
  return cuda_code(e);
}

int mgpu_b200_l2_unpin(void* stream) {
  g_l2_pinned.store(0);
  cudaStreamAttrValue value = { };
  value.accessPolicyWindow.num_bytes = 0;
  cudaError_t e = cudaStreamSetAttribute((cudaStream_t)stream,
    cudaStreamAttributeAccessPolicyWindow, &value);
  if(cudaSuccess == e) e = cudaCtxResetPersistingL2Cache();
  if(cudaSuccess == e) e = cudaDeviceSetLimit(cudaLimitPersistingL2CacheSize, 0);
  return cuda_code(e);
}

size_t mgpu_b200_scan_workspace_bytes(int dtype, int count) {
  if(count < 0) return 0;
  switch(dtype) {
    case MGPU_B200_F32: return scan_bytes<float>(count);
    case MGPU_B200_F64: return scan_bytes<double>(count);
    case MGPU_B200_I32: return scan_bytes<int32_t>(count);
    case MGPU_B200_I64: return scan_bytes<int64_t>(count);
  }
  return 0;
}

int mgpu_b200_scan(int dtype, int inclusive, const void* input_device,
  int count, void* output_device, void* total_device, void* workspace_device,
  size_t workspace_bytes, void* stream) {
  if(count < 0 || (count && (!input_device || !output_device)) ||
    !workspace_device || (uintptr_t)workspace_device % 128)
    return MGPU_B200_E_INVALID;
  size_t need = mgpu_b200_scan_workspace_bytes(dtype, count);
  if(!need) return MGPU_B200_E_UNSUPPORTED;
  if(workspace_bytes < need) return MGPU_B200_E_WORKSPACE;
  if(0 == count && !total_device) return MGPU_B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  switch(dtype) {
    case MGPU_B200_F32: return scan_typed<float>(inclusive, input_device,
      count, output_device, total_device, workspace_device, s);
    case MGPU_B200_F64: return scan_typed<double>(inclusive, input_device,
      count, output_device, total_device, workspace_device, s);
    case MGPU_B200_I32: return scan_typed<int32_t>(inclusive, input_device,
      count, output_device, total_device, workspace_device, s);
    case MGPU_B200_I64: return scan_typed<int64_t>(inclusive, input_device,
      count, output_device, total_device, workspace_device, s);
  }
  return MGPU_B200_E_UNSUPPORTED;
}

} // extern "C"
