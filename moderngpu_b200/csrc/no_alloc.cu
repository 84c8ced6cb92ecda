// mgpu_b200_segreduce_static: segmented reduction for callers that cannot
// allocate device memory.
//
// Who needs it. mgpu_b200_segreduce takes its scratch block (partition table
// and tile-status words) from the caller, which normally obtains it from
// cudaMalloc or a framework allocator. Some callers cannot do that at the
// point of the call: code running inside a region where the CUDA allocator is
// off limits (a stream capture in progress, a real-time loop that must not
// take the allocator's lock, a plug-in whose host forbids allocation after
// start-up), or a binding that can only pass the input and output pointers it
// was given. For them the scratch lives inside the library: a fixed block of
// device memory that comes with the loaded module.
//
// What it costs. Every GPU on which this library is loaded holds
// mgpu_b200_static_scratch_bytes() bytes (4 MiB) for the life of the process,
// used or not. Problems whose scratch does not fit are refused with
// MGPU_B200_E_WORKSPACE; nothing is ever allocated or freed here.
//
// Sharing. There is ONE block per GPU, shared by every call on that GPU, and
// it still holds what the previous call left there. The kernels clear the
// words that must start at zero (ticket counter, status word, tile status)
// themselves at the start of each call, so back-to-back calls on one stream
// are fine. Two calls that overlap on the same GPU (different streams, or
// different host threads) race on the block and give wrong results: serialise
// them, or use mgpu_b200_segreduce with one workspace per stream.
//
// First call. The block's device address is looked up once per GPU, on the
// first call made with that GPU current (cudaGetSymbolAddress). Make that
// first call outside any stream capture.
#include <moderngpu_b200.h>
#include <cuda_runtime.h>
#include <mutex>

namespace {

constexpr size_t kScratchBytes = 4u << 20;

// The name below is a host-side handle in host code, not a device address:
// host code must go through cudaGetSymbolAddress before handing it to a
// kernel or to another entry point.
static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_address[kMaxDevices] = { };

// Device address of the scratch block on the current GPU, looked up on first
// use with that GPU current.
int scratch_for_current_device(void** address) {
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if(cudaSuccess != e) return MGPU_B200_E_CUDA + (int)e;
  if(device < 0 || device >= kMaxDevices) return MGPU_B200_E_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if(!g_scratch_address[device]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if(cudaSuccess != e) return MGPU_B200_E_CUDA + (int)e;
    if(!p) return MGPU_B200_E_CUDA + (int)cudaErrorInvalidSymbol;
    g_scratch_address[device] = p;
  }
  *address = g_scratch_address[device];
  return MGPU_B200_OK;
}

} // namespace

extern "C" {

size_t mgpu_b200_static_scratch_bytes(void) { return kScratchBytes; }

int mgpu_b200_segreduce_static(int dtype, int op, const void* input_device,
  int count, const int* segments_device, int num_segments,
  void* output_device, const void* init_host, void* stream) {
  // Size first: a problem that does not fit is refused before any pointer is
  // looked at.
  if(count < 0 || num_segments < 0) return MGPU_B200_E_INVALID;
  if(dtype < MGPU_B200_F32 || dtype > MGPU_B200_I64)
    return MGPU_B200_E_UNSUPPORTED;
  if(0 == count && 0 == num_segments) return MGPU_B200_OK;
  // 0 means the sizes are beyond what any call of this library accepts.
  size_t need = mgpu_b200_segreduce_workspace_bytes(dtype, count,
    num_segments);
  if(!need || need > kScratchBytes) return MGPU_B200_E_WORKSPACE;

  void* scratch = nullptr;
  int code = scratch_for_current_device(&scratch);
  if(MGPU_B200_OK != code) return code;
  return mgpu_b200_segreduce(dtype, op, input_device, count, segments_device,
    num_segments, output_device, init_host, scratch, kScratchBytes, stream);
}

} // extern "C"
