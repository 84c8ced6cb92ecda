// Thin wrappers over the sm_100a instructions the kernels use directly:
// shared-memory transaction barriers (mbarrier), bulk asynchronous copies
// from global to this CTA's shared memory (the TMA engine's untiled form,
// always to the issuing CTA only), named barriers for a subset of a CTA,
// and scoped loads/stores for the cross-CTA tile-status protocol.
//
// Every wait is bounded by wall-clock time (the %globaltimer register): it
// returns false once `timeout_ns` has passed, so the caller can record a
// status and carry on instead of spinning forever.
#pragma once
#include "base.hxx"

#ifdef __CUDACC__

BEGIN_MGPU_NAMESPACE
namespace ptx {

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

////////////////////////////////////////////////////////////////////////////////
// mbarrier

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;"
    :: "r"(smem_addr(bar)), "r"(arrivals) : "memory");
}

// Makes barrier initialisation and earlier generic-proxy shared-memory
// accesses visible to the asynchronous (bulk copy) proxy.
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];"
    :: "r"(smem_addr(bar)) : "memory");
}

// One arrival that also announces `bytes` of bulk-copy traffic to wait for.
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar,
  uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;"
    :: "r"(smem_addr(bar)), "r"(bytes) : "memory");
}

// One poll; the thread may stay suspended in hardware for up to ~20 us
// (a hint) before the instruction reports "not yet".
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
    "{\n"
    "  .reg .pred p;\n"
    "  mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
    "  selp.u32 %0, 1, 0, p;\n"
    "}\n"
    : "=r"(done) : "r"(smem_addr(bar)), "r"(parity), "r"(20000u) : "memory");
  return done != 0;
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait for the phase with the given parity to complete.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity,
  uint64_t timeout_ns) {
  if(mbar_try_wait(bar, parity)) return true;
  uint64_t start = global_timer_ns();
  while(true) {
    // Kept rolled: unrolled, the 32 polls are ~1.7 KB of code at every wait,
    // and the reduction's tile loop is instruction-cache-sensitive (2 us of
    // 195 on 2^28 items).
    #pragma unroll 1
    for(int spin = 0; spin < 32; ++spin)
      if(mbar_try_wait(bar, parity)) return true;
    if(global_timer_ns() - start > timeout_ns) return false;
  }
}

////////////////////////////////////////////////////////////////////////////////
// Bulk copy global -> shared memory of the issuing CTA, completion counted
// in bytes on an mbarrier. Source, destination and size must be multiples of
// 16 bytes.

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src,
  uint32_t bytes, uint64_t* bar) {
  asm volatile(
    "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes "
    "[%0], [%1], %2, [%3];"
    :: "r"(smem_addr(smem_dst)), "l"(gmem_src), "r"(bytes),
       "r"(smem_addr(bar)) : "memory");
}

// Bulk copy shared memory of the issuing CTA -> global. The issuing thread
// groups its copies (commit) and waits either until their source has been
// read (the shared memory may be reused) or until they are complete. These
// waits concern the thread's own copies only and always end.
__device__ __forceinline__ void bulk_store(void* gmem_dst, const void* smem_src,
  uint32_t bytes) {
  asm volatile(
    "cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
    :: "l"(gmem_dst), "r"(smem_addr(smem_src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template<int pending>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" :: "n"(pending) : "memory");
}
template<int pending>
__device__ __forceinline__ void bulk_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" :: "n"(pending) : "memory");
}

// Programmatic dependent launch: a kernel launched with the programmatic
// stream-serialization attribute may start while its predecessor in the
// stream is still running; it must call grid_dependency_wait() before it
// touches anything the predecessor writes. The predecessor calls
// grid_launch_dependents() once it no longer minds company on the SMs.
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void grid_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// L2 residency hints. Streaming inputs are read once: marking their copies
// evict-first leaves the L2 to data that is reused (the x vector of spmv,
// which is gathered with evict-last).
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;"
    : "=l"(policy));
  return policy;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;"
    : "=l"(policy));
  return policy;
}

__device__ __forceinline__ void bulk_load_hint(void* smem_dst,
  const void* gmem_src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
  asm volatile(
    "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes"
    ".L2::cache_hint [%0], [%1], %2, [%3], %4;"
    :: "r"(smem_addr(smem_dst)), "l"(gmem_src), "r"(bytes),
       "r"(smem_addr(bar)), "l"(policy) : "memory");
}

// Read-only load of a 4- or 8-byte value with an L2 policy.
template<typename type_t>
__device__ __forceinline__ type_t ld_nc_hint(const type_t* p, uint64_t policy) {
  static_assert(sizeof(type_t) == 4 || sizeof(type_t) == 8, "4 or 8 bytes");
  type_t v;
  if constexpr (sizeof(type_t) == 4) {
    uint32_t bits;
    asm volatile("ld.global.nc.L2::cache_hint.b32 %0, [%1], %2;"
      : "=r"(bits) : "l"(p), "l"(policy));
    memcpy(&v, &bits, 4);
  } else {
    uint64_t bits;
    asm volatile("ld.global.nc.L2::cache_hint.b64 %0, [%1], %2;"
      : "=l"(bits) : "l"(p), "l"(policy));
    memcpy(&v, &bits, 8);
  }
  return v;
}

// The same without a line in the L1: for gathers that never hit there.
template<typename type_t>
__device__ __forceinline__ type_t ld_no_l1_hint(const type_t* p, uint64_t policy) {
  static_assert(sizeof(type_t) == 4 || sizeof(type_t) == 8, "4 or 8 bytes");
  type_t v;
  if constexpr (sizeof(type_t) == 4) {
    uint32_t bits;
    asm volatile("ld.global.L1::no_allocate.L2::cache_hint.b32 %0, [%1], %2;"
      : "=r"(bits) : "l"(p), "l"(policy));
    memcpy(&v, &bits, 4);
  } else {
    uint64_t bits;
    asm volatile("ld.global.L1::no_allocate.L2::cache_hint.b64 %0, [%1], %2;"
      : "=l"(bits) : "l"(p), "l"(policy));
    memcpy(&v, &bits, 8);
  }
  return v;
}

////////////////////////////////////////////////////////////////////////////////
// Named barrier over `count` threads (a multiple of 32) of the CTA.

template<int id, int count>
__device__ __forceinline__ void named_sync() {
  asm volatile("bar.sync %0, %1;" :: "n"(id), "n"(count) : "memory");
}

// The same barrier with a vote: true for all `count` threads iff `mine` is
// true for all of them. Lets a subset of a CTA agree to leave a loop together
// after a bounded wait has run out for some of its threads.
template<int id, int count>
__device__ __forceinline__ bool named_all(bool mine) {
  uint32_t out;
  asm volatile(
    "{\n"
    "  .reg .pred p, q;\n"
    "  setp.ne.u32 q, %1, 0;\n"
    "  bar.red.and.pred p, %2, %3, q;\n"
    "  selp.u32 %0, 1, 0, p;\n"
    "}\n"
    : "=r"(out) : "r"((uint32_t)mine), "n"(id), "n"(count) : "memory");
  return out != 0;
}

////////////////////////////////////////////////////////////////////////////////
// Device-scope loads and stores for flags shared between CTAs.

__device__ __forceinline__ uint64_t ld_relaxed_u64(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p)
    : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_u64(uint64_t* p, uint64_t v) {
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" :: "l"(p), "l"(v)
    : "memory");
}
// 16-byte accesses. ASSUMPTION the tile-status protocol makes for 8-byte
// values (value and code travel together): a 16-byte aligned .v2.u64 access
// is performed as ONE transaction, so a reader never sees the value of one
// store with the code of another. The PTX memory model does not promise this
// (it treats a vector access as its scalar parts); the hardware this library
// targets performs aligned 128-bit global accesses as single 16-byte sector
// transactions, the same property CUB's decoupled look-back relies on for
// 16-byte status words. tests/cpp/test_template_api.cu stresses it: tiles of
// 504 fp64 items, segments spanning hundreds of tiles, maximum over distinct
// values, 50 runs compared bit for bit (a torn word would surface as a wrong
// maximum). A port to hardware without the property has to publish through
// atom.exch.b128 / atom.cas.b128 instead.
__device__ __forceinline__ void ld_relaxed_v2u64(const void* p, uint64_t& a,
  uint64_t& b) {
  asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];"
    : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
__device__ __forceinline__ void st_relaxed_v2u64(void* p, uint64_t a,
  uint64_t b) {
  asm volatile("st.relaxed.gpu.global.v2.u64 [%0], {%1, %2};"
    :: "l"(p), "l"(a), "l"(b) : "memory");
}
__device__ __forceinline__ uint32_t ld_relaxed_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p)
    : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p)
    : "memory");
  return v;
}
__device__ __forceinline__ void st_release_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" :: "l"(p), "r"(v)
    : "memory");
}

} // namespace ptx
END_MGPU_NAMESPACE

#endif // __CUDACC__
