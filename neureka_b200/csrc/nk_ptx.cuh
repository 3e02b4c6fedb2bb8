// Inline-PTX wrappers shared by the pipelined kernels: cp.async, mbarrier (every wait bounded), proxy fences.
#pragma once
#include <cstdint>

#define NK_WAIT_LIMIT_NS 2000000000ull   // bounded mbarrier wait: two seconds by the global timer, then the kernel gives up and reports

__device__ __forceinline__ void nk_cp_async_16(void* smem, const void* gmem, int src_bytes) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void nk_cp_async_8(void* smem, const void* gmem, int src_bytes) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;\n" ::"r"(s), "l"(gmem), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void nk_cp_async_4(void* smem, const void* gmem, int src_bytes) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(s), "l"(gmem), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void nk_cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void nk_cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

__device__ __forceinline__ void nk_mbar_init(uint64_t* bar, unsigned count) {
    unsigned a = (unsigned)__cvta_generic_to_shared(bar);
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(a), "r"(count) : "memory");
}
__device__ __forceinline__ void nk_mbar_expect_tx(uint64_t* bar, unsigned bytes) {
    unsigned a = (unsigned)__cvta_generic_to_shared(bar);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(a), "r"(bytes) : "memory");
}
__device__ __forceinline__ void nk_mbar_arrive(uint64_t* bar) {
    unsigned a = (unsigned)__cvta_generic_to_shared(bar);
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(a) : "memory");
}
__device__ __forceinline__ unsigned nk_mbar_try_wait(uint64_t* bar, unsigned parity) {
    unsigned a = (unsigned)__cvta_generic_to_shared(bar), ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(a), "r"(parity) : "memory");
    return ok;
}
__device__ __forceinline__ unsigned long long nk_globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
    return t;
}
// Waits for a phase of an mbarrier, but never longer than limit_ns (nor past a raised abort word, if one is given):
// the first poll costs nothing extra; only a blocked waiter reads the timer, once per 64 polls.
// Returns 1 = phase complete, 0 = somebody else aborted, -1 = this wait ran out.
__device__ __forceinline__ int nk_mbar_wait_bounded(uint64_t* bar, unsigned parity, unsigned long long limit_ns, volatile int* abort_word) {
    if (nk_mbar_try_wait(bar, parity)) return 1;
    const unsigned long long t0 = nk_globaltimer_ns();
    unsigned spins = 0;
    while (!nk_mbar_try_wait(bar, parity)) {
        if ((++spins & 63u) == 0) {
            if (abort_word && *abort_word) return 0;
            if (nk_globaltimer_ns() - t0 > limit_ns) return -1;
        }
    }
    return 1;
}
__device__ __forceinline__ void nk_fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }
__device__ __forceinline__ void nk_fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }


// One 2-D tile load (c0 = innermost coordinate in elements, a multiple of 16 bytes' worth; c1 = row). The tensor map must
// describe memory of the launching GPU; no multicast.
__device__ __forceinline__ void nk_tma_load_2d(void* smem, const void* tensor_map, uint64_t* bar, int c0, int c1) {
    unsigned d = (unsigned)__cvta_generic_to_shared(smem), b = (unsigned)__cvta_generic_to_shared(bar);
    unsigned long long m = reinterpret_cast<unsigned long long>(tensor_map);
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
                 ::"r"(d), "l"(m), "r"(c0), "r"(c1), "r"(b) : "memory");
}
