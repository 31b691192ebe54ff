// Asynchronous-copy building blocks: mbarriers with bounded waits, bulk (TMA) copies between global and
// shared memory, tensor-map tile loads.  No multicast anywhere.
#pragma once

#include <cuda.h>

#include "tkq_common.cuh"

namespace tkq {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

// Bounded wait: returns false if the phase did not complete within `limit` polls (the default is seconds long).
// A kernel whose wait fails raises its failure flag and returns; what it has written by then is undefined.
constexpr uint32_t kDefaultPollLimit = 1u << 22;

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t limit = kDefaultPollLimit) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i < limit; ++i) {
        uint32_t done;
        asm volatile(
            "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}

// Orders this thread's earlier generic-proxy accesses to shared memory before later async-proxy (TMA)
// accesses to it.  Needed in both directions: before a TMA load refills a buffer the thread has read, and
// before a TMA store reads a buffer the thread has written.
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// One-dimensional bulk copy global -> shared, completing on `bar`.  Both addresses 16-byte aligned, bytes a
// multiple of 16.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// An L2 policy for data that is read exactly once: evict first, so that streaming input does not push the kernel's
// own output (still dirty in L2) out to DRAM early.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}

// bulk_load with an L2 cache policy
__device__ __forceinline__ void bulk_load_hint(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
                 : "memory");
}

// One-dimensional bulk copy shared -> global, tracked by the issuing thread's bulk async-group.
__device__ __forceinline__ void bulk_store(void* gmem_dst, const void* smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst), "r"(smem_u32(smem_src)), "r"(bytes)
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// Waits until all but the `kPending` most recent bulk stores of this thread have finished *reading* shared memory.
template <int kPending>
__device__ __forceinline__ void bulk_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kPending) : "memory");
}

// Waits until all bulk stores of this thread are complete (needed before the block exits).
__device__ __forceinline__ void bulk_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// One TMA tile load: the box at column `x`, row `y` of the tensor described by `tmap` lands in shared memory;
// elements outside the tensor arrive as zeros and count towards the barrier's byte count.  x * element size
// must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_tile(void* smem_dst, const CUtensorMap* tmap, int32_t x, int32_t y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}

// Each translation unit with waiting kernels keeps its own failure flag; these read and clear them.
int tile_wait_flag();
int row_wait_flag();
int swiglu_wait_flag();

}  // namespace tkq
