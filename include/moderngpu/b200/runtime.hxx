// Host runtime behind the entry points: the context interface the caller
// hands in, RAII device memory, host<->device copies, and the generic
// "run this functor over a grid" launchers.
//
// Interface parity (reference): context_t src/moderngpu/context.hxx:53-75,
// standard_context_t :81-168, mem_t :173-225, copies and fills
// src/moderngpu/memory.hxx:11-129, launch_params_t / launch_box_t
// src/moderngpu/launch_params.hxx:98-156 and launch_box.hxx:18-80,
// cta_launch / cta_transform / transform src/moderngpu/transform.hxx:14-102.
//
// Differences that a caller can observe:
//  * standard_context_t serves device memory from the stream-ordered CUDA
//    pool (cudaMallocAsync / cudaFreeAsync on the context's stream) with the
//    pool's release threshold raised, so temporaries of back-to-back calls
//    are recycled without a device-wide synchronisation. The reference calls
//    cudaMalloc / cudaFree for every temporary.
//  * launch boxes are accepted wherever the reference accepts them, but this
//    library targets one architecture: a box resolves to its entry for the
//    newest architecture it lists, and the segmented-reduction and
//    load-balancing kernels use their own Blackwell tile shapes regardless.
#pragma once
#include "base.hxx"
#include "functional.hxx"
#include "tuple.hxx"

#include <algorithm>
#include <memory>
#include <mutex>
#include <random>
#include <string>
#include <vector>
#include <cstdarg>

BEGIN_MGPU_NAMESPACE

////////////////////////////////////////////////////////////////////////////////
// Launch parameters.

struct MGPU_ALIGN(8) cta_dim_t {
  int nt, vt;
  int nv() const { return nt * vt; }
  int num_ctas(int count) const { return div_up(count, nv()); }
};

template<int nt_, int vt_ = 1, int vt0_ = vt_, int occ_ = 0>
struct launch_cta_t {
  enum { nt = nt_, vt = vt_, vt0 = vt0_, occ = occ_ };
};

struct context_t;

// Fixed launch parameters.
template<int nt_, int vt_ = 1, int vt0_ = vt_, int occ_ = 0>
struct launch_params_t : launch_cta_t<nt_, vt_, vt0_, occ_> {
  typedef launch_params_t sm_ptx;
  static cta_dim_t cta_dim() { return cta_dim_t { nt_, vt_ }; }
  static cta_dim_t cta_dim(int) { return cta_dim(); }
  static cta_dim_t cta_dim(const context_t&) { return cta_dim(); }
  static int nv(const context_t&) { return nt_ * vt_; }
};

// arch_NN<params> tags a parameter set with the architecture it was tuned
// for; launch_box_t<...> selects among them.
template<int version_, typename params_t>
struct arch_tagged_t {
  enum { version = version_ };
  typedef params_t params;
};

#define MGPU_B200_ARCH(ver)                                                   \
  template<typename params_t>                                                 \
  using arch_##ver = arch_tagged_t<ver, params_t>;                            \
  template<int nt, int vt = 1, int vt0 = vt, int occ = 0>                     \
  using arch_##ver##_cta = arch_tagged_t<ver, launch_cta_t<nt, vt, vt0, occ> >;

MGPU_B200_ARCH(20) MGPU_B200_ARCH(21) MGPU_B200_ARCH(30) MGPU_B200_ARCH(32)
MGPU_B200_ARCH(35) MGPU_B200_ARCH(37) MGPU_B200_ARCH(50) MGPU_B200_ARCH(52)
MGPU_B200_ARCH(53) MGPU_B200_ARCH(60) MGPU_B200_ARCH(61) MGPU_B200_ARCH(62)
MGPU_B200_ARCH(70) MGPU_B200_ARCH(75) MGPU_B200_ARCH(80) MGPU_B200_ARCH(86)
MGPU_B200_ARCH(90) MGPU_B200_ARCH(100)
#undef MGPU_B200_ARCH

namespace detail {
template<typename... tagged_t>
struct newest_arch_t;
template<typename only_t>
struct newest_arch_t<only_t> { typedef only_t type; };
template<typename first_t, typename... rest_t>
struct newest_arch_t<first_t, rest_t...> {
  typedef typename newest_arch_t<rest_t...>::type tail_t;
  typedef typename std::conditional<
    ((int)first_t::version >= (int)tail_t::version), first_t, tail_t>::type type;
};
} // namespace detail

template<typename... tagged_t>
struct launch_box_t {
  typedef typename detail::newest_arch_t<tagged_t...>::type::params sm_ptx;
  static cta_dim_t cta_dim() { return cta_dim_t { sm_ptx::nt, sm_ptx::vt }; }
  static cta_dim_t cta_dim(int) { return cta_dim(); }
  static cta_dim_t cta_dim(const context_t&) { return cta_dim(); }
  static int nv(const context_t&) { return sm_ptx::nt * sm_ptx::vt; }
};

////////////////////////////////////////////////////////////////////////////////
// context_t: what every entry point takes by reference. Derive it to route
// temporaries through a custom allocator or to run on a custom stream.

enum memory_space_t {
  memory_space_device = 0,
  memory_space_host = 1
};

struct context_t {
  context_t() = default;
  context_t(const context_t&) = delete;
  context_t& operator=(const context_t&) = delete;
  virtual ~context_t() = default;

  virtual const cudaDeviceProp& props() const = 0;
  virtual int ptx_version() const = 0;
  virtual cudaStream_t stream() = 0;

  virtual void* alloc(size_t size, memory_space_t space) = 0;
  virtual void free(void* p, memory_space_t space) = 0;

  virtual void synchronize() = 0;

  virtual cudaEvent_t event() = 0;
  virtual void timer_begin() = 0;
  virtual double timer_end() = 0;
};

namespace detail {

inline void throw_on_error(cudaError_t status) {
  if(cudaSuccess != status) throw cuda_exception_t(status);
}

inline std::string stringprintf(const char* format, ...) {
  va_list args;
  va_start(args, format);
  int len = vsnprintf(nullptr, 0, format, args);
  va_end(args);
  std::string text((size_t)(len > 0 ? len : 0), '\0');
  va_start(args, format);
  vsnprintf(&text[0], text.size() + 1, format, args);
  va_end(args);
  return text;
}

template<int unused>
__global__ void arch_probe_k() { }

#ifdef __CUDACC__
////////////////////////////////////////////////////////////////////////////////
// Device-side status, made visible to the host without a synchronisation.
//
// A kernel whose bounded wait runs out records a code in its call's scratch
// (which the C++ entry points hand back to the context before anyone could
// read it) AND in one word of pinned host memory per device. Every mgpu::
// entry point looks at that word when it is called and
// standard_context_t::synchronize() looks at it after waiting: a call that
// failed surfaces as a status_exception_t (a cuda_exception_t, as for every
// other error: reference src/moderngpu/types.hxx:9-16) at the next of these.
// The word's device address lives in a variable of the translation unit's
// own module, set on first use per device; code that never calls
// throw_on_device_status() (the C ABI, which reports through its workspaces)
// never allocates it.

static __device__ uint32_t* device_sticky_status = nullptr;

// Device side of every failure report.
MGPU_DEVICE inline void raise_status(uint32_t* word, uint32_t code) {
  if(word) atomicMax(word, code);
  uint32_t* sticky = device_sticky_status;
  if(sticky) *(volatile uint32_t*)sticky = code;
}

// The current device's word (host address), created on first use.
static inline volatile uint32_t* sticky_status_word() {
  enum { max_devices = 64 };
  static std::mutex lock;
  static uint32_t* words[max_devices] = { };
  int device = 0;
  throw_on_error(cudaGetDevice(&device));
  if(device < 0 || device >= max_devices) return nullptr;
  std::lock_guard<std::mutex> guard(lock);
  if(!words[device]) {
    uint32_t* host = nullptr;
    uint32_t* mapped = nullptr;
    throw_on_error(cudaHostAlloc((void**)&host, 64,
      cudaHostAllocMapped | cudaHostAllocPortable));
    *host = 0;
    throw_on_error(cudaHostGetDevicePointer((void**)&mapped, host, 0));
    throw_on_error(cudaMemcpyToSymbol(device_sticky_status, &mapped,
      sizeof(mapped)));
    words[device] = host;
  }
  return words[device];
}

// Throws status_exception_t if a kernel of an earlier call on this device
// reported a failure (and forgets it). Does not wait for the device.
static inline void throw_on_device_status() {
  volatile uint32_t* word = sticky_status_word();
  if(!word) return;
  uint32_t code = *word;
  if(code) {
    *word = 0;
    throw status_exception_t((int)code);
  }
}
#else
static inline void throw_on_device_status() { }
#endif

} // namespace detail

// One-paragraph description of the current device, printed by
// standard_context_t when asked to.
inline std::string device_prop_string(const cudaDeviceProp& prop) {
  int ordinal = 0;
  cudaGetDevice(&ordinal);
  size_t free_bytes = 0, total_bytes = 0;
  detail::throw_on_error(cudaMemGetInfo(&free_bytes, &total_bytes));
  int mem_khz = 0, sm_khz = 0, bus_bits = 0;
  cudaDeviceGetAttribute(&mem_khz, cudaDevAttrMemoryClockRate, ordinal);
  cudaDeviceGetAttribute(&sm_khz, cudaDevAttrClockRate, ordinal);
  cudaDeviceGetAttribute(&bus_bits, cudaDevAttrGlobalMemoryBusWidth, ordinal);
  double gbs = 2.0 * mem_khz * 1.0e3 * (bus_bits / 8) / 1.0e9;
  return detail::stringprintf(
    "%s (device %d): sm_%d%d, %d SMs at %.0f MHz\n"
    "memory: %zu MiB free of %zu MiB, %d-bit bus at %.0f MHz (%.0f GB/s)\n",
    prop.name, ordinal, prop.major, prop.minor, prop.multiProcessorCount,
    sm_khz / 1.0e3, free_bytes >> 20, total_bytes >> 20, bus_bits,
    mem_khz / 1.0e3, gbs);
}

class standard_context_t : public context_t {
protected:
  cudaDeviceProp _props;
  int _ptx_version;
  int _device;
  cudaStream_t _stream;
  cudaEvent_t _timer[2];
  cudaEvent_t _event;

  void init() {
    cudaFuncAttributes attr;
    detail::throw_on_error(
      cudaFuncGetAttributes(&attr, detail::arch_probe_k<0>));
    _ptx_version = attr.ptxVersion;
    detail::throw_on_error(cudaGetDevice(&_device));
    detail::throw_on_error(cudaGetDeviceProperties(&_props, _device));
    cudaEventCreate(&_timer[0]);
    cudaEventCreate(&_timer[1]);
    cudaEventCreateWithFlags(&_event, cudaEventDisableTiming);

    // Keep freed temporaries in the stream-ordered pool instead of handing
    // them back to the driver at every synchronisation.
    cudaMemPool_t pool;
    if(cudaSuccess == cudaDeviceGetDefaultMemPool(&pool, _device)) {
      uint64_t keep = ~(uint64_t)0;
      cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
    } else {
      cudaGetLastError();
    }
  }

public:
  standard_context_t(bool print_prop = true, cudaStream_t stream_ = 0) :
    _stream(stream_) {
    init();
    if(print_prop) printf("%s\n", device_prop_string(_props).c_str());
  }
  ~standard_context_t() override {
    cudaEventDestroy(_timer[0]);
    cudaEventDestroy(_timer[1]);
    cudaEventDestroy(_event);
  }

  const cudaDeviceProp& props() const override { return _props; }
  int ptx_version() const override { return _ptx_version; }
  cudaStream_t stream() override { return _stream; }

  void* alloc(size_t size, memory_space_t space) override {
    void* p = nullptr;
    if(!size) return p;
    cudaError_t status = (memory_space_device == space) ?
      cudaMallocAsync(&p, size, _stream) : cudaMallocHost(&p, size);
    detail::throw_on_error(status);
    return p;
  }

  void free(void* p, memory_space_t space) override {
    if(!p) return;
    cudaError_t status = (memory_space_device == space) ?
      cudaFreeAsync(p, _stream) : cudaFreeHost(p);
    detail::throw_on_error(status);
  }

  // Also the point at which a kernel's failed wait surfaces for certain.
  void synchronize() override {
    detail::throw_on_error(_stream ? cudaStreamSynchronize(_stream) :
      cudaDeviceSynchronize());
    detail::throw_on_device_status();
  }

  cudaEvent_t event() override { return _event; }
  void timer_begin() override { cudaEventRecord(_timer[0], _stream); }
  double timer_end() override {
    cudaEventRecord(_timer[1], _stream);
    cudaEventSynchronize(_timer[1]);
    float ms = 0;
    cudaEventElapsedTime(&ms, _timer[0], _timer[1]);
    return ms / 1.0e3;
  }
};

////////////////////////////////////////////////////////////////////////////////
// mem_t<T>: move-only array owned through a context.

template<typename type_t>
class mem_t {
  context_t* _context;
  type_t* _pointer;
  size_t _size;
  memory_space_t _space;

public:
  mem_t() : _context(nullptr), _pointer(nullptr), _size(0),
    _space(memory_space_device) { }

  mem_t(size_t size, context_t& context,
    memory_space_t space = memory_space_device) :
    _context(&context), _pointer(nullptr), _size(size), _space(space) {
    _pointer = (type_t*)context.alloc(sizeof(type_t) * size, space);
  }

  mem_t(const mem_t&) = delete;
  mem_t& operator=(const mem_t&) = delete;

  mem_t(mem_t&& rhs) : mem_t() { swap(rhs); }
  mem_t& operator=(mem_t&& rhs) { swap(rhs); return *this; }

  ~mem_t() {
    if(_context && _pointer) _context->free(_pointer, _space);
    _pointer = nullptr;
    _size = 0;
  }

  void swap(mem_t& rhs) {
    std::swap(_context, rhs._context);
    std::swap(_pointer, rhs._pointer);
    std::swap(_size, rhs._size);
    std::swap(_space, rhs._space);
  }

  context_t& context() { return *_context; }
  size_t size() const { return _size; }
  type_t* data() const { return _pointer; }
  memory_space_t space() const { return _space; }

  mem_t clone() {
    mem_t copy(_size, *_context, _space);
    if(_size) {
      cudaMemcpyKind kind = (memory_space_device == _space) ?
        cudaMemcpyDeviceToDevice : cudaMemcpyHostToHost;
      detail::throw_on_error(cudaMemcpyAsync(copy._pointer, _pointer,
        sizeof(type_t) * _size, kind, _context->stream()));
    }
    return copy;
  }
};

////////////////////////////////////////////////////////////////////////////////
// Generic grid launchers.

namespace detail {

template<typename params_t, typename func_t, typename... args_t>
__global__ void __launch_bounds__(params_t::nt)
cta_entry_k(func_t f, int num_ctas, args_t... args) {
  int tid = (int)threadIdx.x;
  int cta = (int)blockIdx.x;
  if(cta < num_ctas) f(tid, cta, args...);
}

template<typename params_t>
struct index_transform_t {
  template<typename func_t, typename... args_t>
  MGPU_DEVICE void operator()(int tid, int cta, func_t f, size_t count,
    args_t... args) const {
    enum { nt = params_t::nt, vt = params_t::vt };
    size_t first = (size_t)cta * (nt * vt);
    #pragma unroll
    for(int i = 0; i < vt; ++i) {
      size_t index = first + (size_t)i * nt + tid;
      if(index < count) f((int)index, args...);
    }
  }
};

} // namespace detail

// f(tid, cta, args...) on num_ctas CTAs of launch_t::nt threads.
template<typename launch_t, typename func_t, typename... args_t>
void cta_launch(func_t f, int num_ctas, context_t& context, args_t... args) {
  typedef typename launch_t::sm_ptx params_t;
  if(num_ctas > 0)
    detail::cta_entry_k<params_t, func_t, args_t...>
      <<<num_ctas, (int)params_t::nt, 0, context.stream()>>>(
        f, num_ctas, args...);
}
template<int nt, int vt = 1, typename func_t, typename... args_t>
void cta_launch(func_t f, int num_ctas, context_t& context, args_t... args) {
  cta_launch<launch_params_t<nt, vt> >(f, num_ctas, context, args...);
}

// As cta_launch, with the grid sized to cover `count` work items.
template<typename launch_t, typename func_t, typename... args_t>
void cta_transform(func_t f, int count, context_t& context, args_t... args) {
  int num_ctas = launch_t::cta_dim(context).num_ctas(count);
  cta_launch<launch_t>(f, num_ctas, context, args...);
}
template<int nt, int vt = 1, typename func_t, typename... args_t>
void cta_transform(func_t f, int count, context_t& context, args_t... args) {
  cta_transform<launch_params_t<nt, vt> >(f, count, context, args...);
}

// f(index, args...) for every index in [0, count).
template<typename launch_t, typename func_t, typename... args_t>
void transform(func_t f, size_t count, context_t& context, args_t... args) {
  typedef typename launch_t::sm_ptx params_t;
  cta_transform<launch_t>(detail::index_transform_t<params_t>(), (int)count,
    context, f, count, args...);
}
template<size_t nt = 128, int vt = 1, typename func_t, typename... args_t>
void transform(func_t f, size_t count, context_t& context, args_t... args) {
  transform<launch_params_t<(int)nt, vt> >(f, count, context, args...);
}

////////////////////////////////////////////////////////////////////////////////
// Copies between host and device.

#define MGPU_B200_COPY(name, kind)                                            \
  template<typename type_t>                                                   \
  cudaError_t name(type_t* dest, const type_t* source, size_t count) {        \
    return count ? cudaMemcpy(dest, source, sizeof(type_t) * count, kind) :   \
      cudaSuccess;                                                            \
  }
MGPU_B200_COPY(htoh, cudaMemcpyHostToHost)
MGPU_B200_COPY(dtoh, cudaMemcpyDeviceToHost)
MGPU_B200_COPY(htod, cudaMemcpyHostToDevice)
MGPU_B200_COPY(dtod, cudaMemcpyDeviceToDevice)
#undef MGPU_B200_COPY

template<typename type_t>
cudaError_t dtoh(std::vector<type_t>& dest, const type_t* source,
  size_t count) {
  dest.resize(count);
  return dtoh(dest.data(), source, count);
}
template<typename type_t>
cudaError_t htod(type_t* dest, const std::vector<type_t>& source) {
  return htod(dest, source.data(), source.size());
}

template<typename type_t>
mem_t<type_t> to_mem(const std::vector<type_t>& data, context_t& context) {
  mem_t<type_t> mem(data.size(), context);
  detail::throw_on_error(htod(mem.data(), data));
  return mem;
}

template<typename type_t>
std::vector<type_t> from_mem(const mem_t<type_t>& mem) {
  std::vector<type_t> host;
  detail::throw_on_error(dtoh(host, mem.data(), mem.size()));
  return host;
}

#ifdef __CUDACC__

template<typename type_t, typename func_t>
mem_t<type_t> fill_function(func_t f, size_t count, context_t& context) {
  mem_t<type_t> mem(count, context);
  type_t* p = mem.data();
  transform([=]MGPU_DEVICE(int index) { p[index] = f(index); }, count,
    context);
  return mem;
}

template<typename type_t>
mem_t<type_t> fill(type_t value, size_t count, context_t& context) {
  mem_t<type_t> mem(count, context);
  type_t* p = mem.data();
  transform([=]MGPU_DEVICE(int index) { p[index] = value; }, count, context);
  return mem;
}

template<typename it_t>
auto copy_to_mem(it_t input, size_t count, context_t& context) ->
  mem_t<typename std::iterator_traits<it_t>::value_type> {
  typedef typename std::iterator_traits<it_t>::value_type type_t;
  mem_t<type_t> mem(count, context);
  type_t* p = mem.data();
  transform([=]MGPU_DEVICE(int index) { p[index] = input[index]; }, count,
    context);
  return mem;
}

#endif // __CUDACC__

inline std::mt19937& get_mt19937() {
  static std::mt19937 engine;
  return engine;
}

inline mem_t<int> fill_random(int a, int b, size_t count, bool sorted,
  context_t& context) {
  std::uniform_int_distribution<int> dist(a, b);
  std::vector<int> host(count);
  for(size_t i = 0; i < count; ++i) host[i] = dist(get_mt19937());
  if(sorted) std::sort(host.begin(), host.end());
  return to_mem(host, context);
}

END_MGPU_NAMESPACE
