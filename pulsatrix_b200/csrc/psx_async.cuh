// mbarrier and bulk asynchronous copy (TMA, global -> this CTA's shared memory) as inline PTX for
// sm_100a, shared by the kernels that stage rows in shared memory.  No multicast anywhere: every
// copy lands in the shared memory of the CTA that asked for it.
#pragma once

#include <stdint.h>

namespace psx {

__device__ __forceinline__ uint32_t smem_address(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void barrier_init(uint64_t* bar, uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_address(bar)), "r"(arrivals) : "memory");
}

// Makes freshly initialised barriers visible to the asynchronous proxy (the copy engine).
__device__ __forceinline__ void barrier_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

// One arrival that also announces `bytes` bytes of copies that will complete on the barrier.
__device__ __forceinline__ void barrier_expect_bytes(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_address(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void barrier_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_address(bar)) : "memory");
}

// dst and src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_copy_to_shared(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_address(dst)),
                 "l"(src), "r"(bytes), "r"(smem_address(bar))
                 : "memory");
}

__device__ __forceinline__ unsigned long long global_nanoseconds() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Waits for the phase of parity `parity` to complete, but not for ever: a try blocks in the
// hardware for a short, implementation-defined time only; every 32 failed tries the global timer is
// read, and `limit_ns` nanoseconds after its first reading the wait gives up and returns false.
// `give_up` (shared memory, may be null) is looked at too: once another warp of the CTA has set it,
// this wait gives up at once as well.
__device__ __forceinline__ bool barrier_wait_bounded(uint64_t* bar, uint32_t parity, unsigned long long limit_ns,
                                                     const volatile uint32_t* give_up = nullptr) {
    const uint32_t addr = smem_address(bar);
    unsigned long long started = 0;
    for (uint32_t tries = 1;; ++tries) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
        if ((tries & 31u) == 0) {
            if (give_up && *give_up) return false;
            const unsigned long long now = global_nanoseconds();
            if (started == 0) started = now;
            else if (now - started > limit_ns) return false;
        }
    }
}

}  // namespace psx
