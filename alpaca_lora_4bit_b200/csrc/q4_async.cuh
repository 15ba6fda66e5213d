// mbarrier / TMA / programmatic-dependent-launch helpers (inline PTX, sm_100a) and the host side
// tensor-map encoder.  Every CTA fetches its own tiles with copies of its own.
#pragma once

#include <cuda.h>

#include "q4_common.cuh"

namespace q4 {

// ---- host: tensor maps ----------------------------------------------------------------------
// 2-D row-major tensor of `elem_bytes`-wide elements, box = box_cols x box_rows.
// swizzle: 0 none, 1 32B, 2 64B, 3 128B (CUtensorMapSwizzle values).
int make_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elem_bytes,
                 uint64_t cols, uint64_t rows, uint64_t row_pitch_bytes, uint32_t box_cols, uint32_t box_rows,
                 CUtensorMapSwizzle swizzle);

#ifdef __CUDACC__

// Device-visible status word values written when a bounded wait expires.
constexpr unsigned Q4_STATUS_OK = 0u;
constexpr unsigned Q4_STATUS_WAIT_EXPIRED = 0xDEAD0001u;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}

// Non-blocking test of the phase.  (mbarrier.try_wait is compiled into a polling loop of its own -
// try, short sleep, retry until an internal time limit - whose instructions compete for issue
// slots with working warps on the same scheduler; test_wait is a single instruction, so the
// caller decides how often a waiting thread polls.)
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// The same on a barrier that CTAs of the whole cluster arrive on (acquire at cluster scope).
__device__ __forceinline__ bool mbar_test_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}

// Bounded wait.  Returns false if the phase did not complete within `limit` polls; the caller
// then records Q4_STATUS_WAIT_EXPIRED and carries on without waiting (results are garbage but
// every thread still reaches the end of the kernel, so nothing can hang).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t limit) {
  for (uint32_t i = 0; i < limit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}

// Sleeping variant: the hardware may suspend the thread for up to `ns` nanoseconds per try, so a
// waiting warp does not compete for issue slots with the warps that have work.
__device__ __forceinline__ bool mbar_try_wait_sleep(uint64_t* bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(ns) : "memory");
  return ok != 0;
}

// Warp-wide bounded wait: lane 0 sleeps on the barrier, then every lane confirms the phase with
// one try of its own (which returns at once) so that each thread has acquired the data.
// All 32 lanes must call it.  Returns false (on every lane) if the phase never completed.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, uint32_t limit) {
  bool ok = true;
  if ((threadIdx.x & 31) == 0) {
    ok = false;
    for (uint32_t i = 0; i < limit && !ok; ++i) ok = mbar_try_wait_sleep(bar, parity, 2000u);
  }
  ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
  if (ok) ok = mbar_try_wait(bar, parity);
  return __all_sync(0xffffffffu, ok ? 1 : 0) != 0;
}

// 2-D tiled TMA load global -> shared, completion signalled on `bar` (no multicast).
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar)) : "memory");
}
// expect_tx + 2-D tile load as one predicated pair: the lanes with `pred` false issue nothing, and no
// divergent region (with its reconvergence bookkeeping) is opened around the two instructions
__device__ __forceinline__ void tma_expect_load_2d_if(bool pred, void* dst, const CUtensorMap* map, int c0, int c1,
                                                      uint64_t* bar, uint32_t bytes) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.u32 p, %6, 0;\n\t"
      "@p mbarrier.arrive.expect_tx.shared::cta.b64 _, [%4], %5;\n\t"
      "@p cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n\t"
      "}"
      ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar)), "r"(bytes), "r"((uint32_t)pred) : "memory");
}
// ---- thread-block cluster helpers (CTA pairs) ---------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t mapa_u32(uint32_t cta_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(cta_addr), "r"(rank));
  return r;
}
// all threads of all CTAs of the cluster
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on an mbarrier of any CTA of the cluster (address from mapa_u32).  Default semantics
// (release at CTA scope): what the arriving thread published is shared memory of its own CTA,
// made visible to the async proxy by a proxy fence before the arrive; a cluster-scope release
// would add a device-wide memory barrier to every arrive.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// one try on an own mbarrier that CTAs of the whole cluster arrive on (acquire at cluster scope)
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// sleeping try on an own mbarrier that CTAs of the whole cluster arrive on (acquire at cluster scope)
__device__ __forceinline__ bool mbar_try_wait_sleep_cluster(uint64_t* bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(ns) : "memory");
  return ok != 0;
}
// 2-D tiled TMA load into this CTA's shared memory whose completion bytes are counted on an
// mbarrier of either CTA of the pair (`bar_cluster_addr` from mapa_u32).
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int c0, int c1, uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(bar_cluster_addr) : "memory");
}

// Ask for a 2-D tile to be brought into L2 (no shared-memory destination, no completion signal).
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap* map, int c0, int c1) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(map), "r"(c0), "r"(c1) : "memory");
}

__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// Programmatic dependent launch: let the next kernel in the stream start early / wait for the
// previous kernel's memory to be visible.  Both are no-ops when the launch has no such edge.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

#endif  // __CUDACC__

}  // namespace q4
