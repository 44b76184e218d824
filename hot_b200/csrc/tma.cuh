// mbarrier and TMA (cp.async.bulk.tensor) wrappers shared by the kernels, and the host-side
// tensor-map builder.  Every wait is bounded in time.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace hot {

// Tensor map over a [rows, row_bytes] byte matrix with pitch ld, box = box_bytes x box_rows.
int make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t row_bytes, int64_t ld, int box_bytes,
             int box_rows, int swizzle_bytes);  // swizzle_bytes: 0, 64 or 128

// The time limit of every device-side wait: 1.5 s unless hot_set_wait_limit_ns changed it; the launchers copy it
// into the kernel parameters (host side: common.cu).
uint64_t wait_limit_ns();

#ifdef __CUDACC__

// ---- PTX wrappers ------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// CLUSTER: acquire at cluster scope, for a barrier that threads of the partner CTA arrive on
template <bool CLUSTER = false>
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  if (CLUSTER) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
  }
  return ok != 0;
}
// try_wait that lets the hardware park the thread for up to `hint_ns` while the phase is incomplete (it is
// woken as soon as the phase completes), so that a waiting warp does not spend issue slots on polling
__device__ __forceinline__ bool mbar_try_wait_parked(uint64_t* bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait.  Returns false when it gave up (time limit, or another role already aborted).
template <bool CLUSTER = false>
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, uint64_t limit_ns) {
  if (mbar_try_wait<CLUSTER>(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait<CLUSTER>(bar, parity)) return true;
    if ((it & 63u) == 0) {
      if (*abort_flag) return false;
      if (global_timer_ns() - t0 > limit_ns) {
        *abort_flag = 1u;
        return false;
      }
    }
  }
}

// The same bounded wait for roles that wait long and often (a whole tile's worth of work by another role):
// each poll parks the thread for up to 2 us, so a waiting warp issues a handful of instructions per wait.
__device__ __forceinline__ bool mbar_wait_parked(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, uint64_t limit_ns) {
  if (mbar_try_wait<false>(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait_parked(bar, parity, 2000u)) return true;
    if ((it & 7u) == 0) {
      if (*abort_flag) return false;
      if (global_timer_ns() - t0 > limit_ns) {
        *abort_flag = 1u;
        return false;
      }
    }
  }
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
// tiled store shared -> global (bulk-group completion); x in elements of the map (16-byte aligned in bytes)
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(reinterpret_cast<uint64_t>(map)),
               "r"(x), "r"(y), "r"(smem_u32(src))
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// at most N of this thread's most recent bulk groups are still reading their shared-memory source
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// at most N of this thread's most recent bulk groups are incomplete
template <int N>
__device__ __forceinline__ void bulk_wait_group() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// untiled bulk copy global -> shared; both addresses 16-byte aligned, bytes a multiple of 16
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
               "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}


#endif  // __CUDACC__

}  // namespace hot
