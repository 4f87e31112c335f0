// Shared device helpers of the KV-cache data-movement kernels (sm_100a only).
//
// Everything here moves opaque bytes: 16-byte and 32-byte global loads/stores
// with explicit cache policy, bulk (TMA) copies between global and shared
// memory completed through an mbarrier with a bounded wait, and the per-device
// error record the debug checks write instead of trapping.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace lms {

// ---------------------------------------------------------------- error record
// One per device, in device memory.  A kernel that meets an out-of-range index
// (debug checks on) or a wait that ran out writes the FIRST such event here and
// skips the access; the host reads it back in lms_check_device_errors.
struct ErrRecord {
  unsigned int code;   // 0 = clean
  unsigned int where;  // kernel id
  long long index;     // position in the index table
  long long value;     // offending value
  long long reserved;  // pads the record to 32 bytes
};

enum : unsigned int {
  kErrNone = 0,
  kErrBadSlot = 1,
  kErrBadSrcBlock = 2,
  kErrBadDstBlock = 3,
  kErrWaitTimeout = 4,
  kErrBadPosition = 5,
};

__device__ __forceinline__ void report(ErrRecord* e, unsigned int code,
                                       unsigned int where, long long index,
                                       long long value) {
  if (e == nullptr) return;
  if (atomicCAS(&e->code, 0u, code) == 0u) {
    e->where = where;
    e->index = index;
    e->value = value;
  }
}

// ---------------------------------------------------------------- cache policy
// L2 policies: streaming data that will not be re-read by this kernel leaves
// L2 first; fan-out sources (one block copied to many) stay.
__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}

// A hint that brings the 128-byte line of `p` into L2.  It returns nothing and orders nothing,
// so it may be issued for memory another kernel is still writing: L2 is the point of coherence,
// a later load sees whatever was written last.
__device__ __forceinline__ void prefetch_l2(const void* p) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

// ---------------------------------------------------------------- 16-byte path
struct V16 {
  uint4 v;
  static constexpr int kBytes = 16;
};
__device__ __forceinline__ void ld(V16& r, const char* p) {
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.v.x), "=r"(r.v.y), "=r"(r.v.z), "=r"(r.v.w)
               : "l"(p));
}
__device__ __forceinline__ void ld_hint(V16& r, const char* p, uint64_t pol) {
  asm volatile(
      "ld.global.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
      : "=r"(r.v.x), "=r"(r.v.y), "=r"(r.v.z), "=r"(r.v.w)
      : "l"(p), "l"(pol));
}
__device__ __forceinline__ void st(char* p, const V16& r) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(r.v.x),
               "r"(r.v.y), "r"(r.v.z), "r"(r.v.w)
               : "memory");
}
__device__ __forceinline__ void st_hint(char* p, const V16& r, uint64_t pol) {
  asm volatile(
      "st.global.L1::no_allocate.L2::cache_hint.v4.u32 [%0], {%1,%2,%3,%4}, %5;" ::"l"(p),
      "r"(r.v.x), "r"(r.v.y), "r"(r.v.z), "r"(r.v.w), "l"(pol)
      : "memory");
}

// ---------------------------------------------------------------- 32-byte path
// 256-bit global accesses exist from sm_100 on; they halve the instruction
// count per byte.  Addresses must be 32-byte aligned.
struct V32 {
  uint32_t a[8];
  static constexpr int kBytes = 32;
};
__device__ __forceinline__ void ld(V32& r, const char* p) {
  asm volatile(
      "ld.global.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
      : "=r"(r.a[0]), "=r"(r.a[1]), "=r"(r.a[2]), "=r"(r.a[3]), "=r"(r.a[4]),
        "=r"(r.a[5]), "=r"(r.a[6]), "=r"(r.a[7])
      : "l"(p));
}
__device__ __forceinline__ void ld_hint(V32& r, const char* p, uint64_t pol) {
  asm volatile(
      "ld.global.L1::no_allocate.L2::cache_hint.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8], %9;"
      : "=r"(r.a[0]), "=r"(r.a[1]), "=r"(r.a[2]), "=r"(r.a[3]), "=r"(r.a[4]),
        "=r"(r.a[5]), "=r"(r.a[6]), "=r"(r.a[7])
      : "l"(p), "l"(pol));
}
__device__ __forceinline__ void st(char* p, const V32& r) {
  asm volatile(
      "st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(r.a[0]),
      "r"(r.a[1]), "r"(r.a[2]), "r"(r.a[3]), "r"(r.a[4]), "r"(r.a[5]),
      "r"(r.a[6]), "r"(r.a[7])
      : "memory");
}
__device__ __forceinline__ void st_hint(char* p, const V32& r, uint64_t pol) {
  asm volatile(
      "st.global.L1::no_allocate.L2::cache_hint.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8}, %9;" ::"l"(p),
      "r"(r.a[0]), "r"(r.a[1]), "r"(r.a[2]), "r"(r.a[3]), "r"(r.a[4]),
      "r"(r.a[5]), "r"(r.a[6]), "r"(r.a[7]), "l"(pol)
      : "memory");
}

// ---------------------------------------------------------------- bulk copies
// cp.async.bulk (the untiled TMA path): both addresses 16-byte aligned, size a
// multiple of 16.  Loads complete on an mbarrier; stores complete through the
// issuing thread's bulk async-group.
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
  asm volatile(
      "mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
      "r"(bytes)
      : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: polls until the phase completes or `limit_ns` of wall time have
// passed (default one second, far beyond any healthy copy).  Returns false when
// it gave up; the caller then reports kErrWaitTimeout and stops issuing work.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, unsigned parity,
                                                  unsigned long long limit_ns = 1000000000ull) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (global_ns() - t0 > limit_ns) return false;
  }
}
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc,
                                         unsigned bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(smem_dst)),
      "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* gdst, const void* smem_src,
                                         unsigned bytes) {
  asm volatile(
      "cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst),
      "r"(smem_u32(smem_src)), "r"(bytes)
      : "memory");
}
__device__ __forceinline__ void bulk_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Source shared memory of all committed stores has been read (safe to reuse).
__device__ __forceinline__ void bulk_wait_read_all() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
// All committed stores are complete (written).
__device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

}  // namespace lms
