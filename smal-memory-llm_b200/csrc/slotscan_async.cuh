// Bulk asynchronous copies into shared memory and the mbarrier that counts their bytes (sm_90 and later): the staging
// path of the kernels that stream token chunks or snapshot tiles.  Every wait is bounded.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace slotscan {

// ---- bulk asynchronous copy global -> shared with an mbarrier that counts the bytes (sm_90 and later) ----
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// both addresses 16-byte aligned, bytes a multiple of 16
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, unsigned bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// ---- bulk asynchronous copy shared -> global, tracked by bulk groups of the issuing thread ----
// make shared-memory writes of this thread visible to the asynchronous proxy before a bulk copy reads them
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void bulk_s2g(void* dst, const void* src, unsigned bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(smem_u32(src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// at most PENDING of this thread's bulk groups still in flight (writes complete, not only the reads of the source)
template <int PENDING>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(PENDING) : "memory"); }
template <int PENDING>
__device__ __forceinline__ void bulk_wait() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(PENDING) : "memory"); }

// Bounded wait: a copy that never lands must not hang the GPU.  Returns false after ~0.2 s of polling.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, unsigned parity) {
    for (int it = 0; it < (1 << 22); it++) {
        if (mbar_try_wait(bar, parity)) return true;
        if (it > 64) __nanosleep(40);
    }
    return false;
}

}  // namespace slotscan
