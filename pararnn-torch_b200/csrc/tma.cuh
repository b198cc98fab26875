// TMA (cp.async.bulk.tensor) and mbarrier helpers for sm_100a, plus the host-side
// tensor-map builder.  Loads are plain tile loads from this GPU's own memory into the
// issuing CTA's shared memory; no multicast is used anywhere.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace prb {

// ---------------------------------------------------------------- device side
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: returns false when the limit ran out (the caller records an error status
// and leaves the kernel; nothing spins for ever).
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint32_t limit) {
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    return false;
}
// Same wait with a suspend-time hint on the polls after the first: the waiting thread sleeps in
// hardware (and wakes when the phase completes) instead of spinning, which leaves the issue slots
// to the warps that have work.  Measured: the per-pass sLSTM Newton sweep 1.05 -> 0.92 ms, the
// Picard sweep 0.43 -> 0.40 ms; the reverse sweep gets slower with it and keeps the plain wait.
__device__ __forceinline__ bool mbar_try_wait_hint(uint64_t* bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}
// A hinted poll may sleep up to the hint (20 us), so the poll count is capped: 2^16 polls are at most
// 1.3 s, the same order as the 2^24 plain polls of mbar_wait_bounded.
__device__ __forceinline__ bool mbar_wait_bounded_sleepy(uint64_t* bar, uint32_t parity, uint32_t limit) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint32_t n = limit > (1u << 16) ? (1u << 16) : limit;
    for (uint32_t i = 0; i < n; ++i) {
        if (mbar_try_wait_hint(bar, parity, 20000u)) return true;
    }
    return false;
}
// Once a thread has seen one of its bounded waits run out it passes this limit to its later waits
// (`timed_out ? kWaitLimitAfterTimeout : limit`): a CTA whose input stalled then leaves after about
// one full limit per warp, not one per remaining wait, and the normal path pays nothing for it.
constexpr uint32_t kWaitLimitAfterTimeout = 64;
constexpr uint32_t kDrainLimit = 1u << 20;
// After a time-out: the thread that issued the bulk loads waits (bounded) until the loads already
// issued into the ring have landed, so the CTA does not exit with copies in flight into its
// shared memory.  `n_issued` = number of stages issued so far (round r went to stage r % nstage).
__device__ __forceinline__ void drain_ring(uint64_t* full, int nstage, int n_issued, uint32_t limit) {
    for (int s = 0; s < nstage; ++s) {
        if (n_issued <= s) continue;
        const int last = ((n_issued - 1 - s) / nstage) * nstage + s;  // last round issued into stage s
        mbar_wait_bounded(&full[s], (last / nstage) & 1, limit);
    }
}
// Orders earlier generic-proxy accesses to shared memory before later async-proxy (TMA) ones.
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x,
                                            int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_u32(smem_dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
        : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x,
                                            int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(smem_dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---------------------------------------------------------------- host side
// Tensor map of a (rows, mid, inner) row-major array (mid may be 1): box = (box_rows, mid, 32)
// elements, no swizzle, out-of-range elements read as zero.  Returns false when the array does
// not meet TMA's rules (16-byte aligned base, strides multiple of 16 bytes) or the driver entry
// point is missing; the caller then uses the non-TMA kernels.
bool make_tile_map(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint32_t mid,
                   uint64_t inner, uint32_t box_rows);

}  // namespace prb
