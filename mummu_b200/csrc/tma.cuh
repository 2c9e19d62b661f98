// mbarrier and TMA (cp.async.bulk.tensor) PTX wrappers shared by the kernels that stage
// operands in shared memory with the copy engine, plus the host-side tensor-map encoder.
// Plain tiled loads only: no cluster multicast anywhere.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace mummu {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
// make freshly initialised barriers visible to the copy engine
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}

// One suspending probe: the thread may sleep in hardware for up to about `ns` nanoseconds
// waiting for the phase, instead of burning issue slots in a polling loop.
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(ns)
        : "memory");
    return ok;
}

// Bounded wait.  Returns false when `limit` probes (each suspending for at most a microsecond or
// so) ran out (the abort flag is raised) or another role of the CTA already gave up.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                  uint32_t limit) {
    if (mbar_test(bar, parity)) return true;
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity, 1000u)) return true;
        if ((i & 63u) == 63u && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}

// generic-proxy writes to shared memory -> visible to the async proxy (TMA, tcgen05.mma operands)
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
}

// one 2-D tile, global -> this CTA's shared memory, completion counted in bytes on `bar`
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c_inner, int c_outer,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n" ::
            "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c_inner), "r"(c_outer)
        : "memory");
}

// Host: encode a row-major 2-D view [outer, inner] (inner contiguous) with the given box.
// Returns MUMMU_OK or MUMMU_ERR_DEVICE with the error text set.
int encode_tiled_2d(CUtensorMap* map, const void* base, CUtensorMapDataType dtype, uint32_t elem_bytes,
                    uint64_t inner, uint64_t outer, uint32_t box_inner, uint32_t box_outer,
                    CUtensorMapSwizzle swizzle);

}  // namespace mummu
