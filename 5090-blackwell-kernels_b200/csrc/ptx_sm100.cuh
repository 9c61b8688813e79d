// Inline-PTX wrappers for sm_100a: mbarrier, bulk asynchronous copies (the TMA engine's
// untiled form), legacy warp-level mma, and the bounded waits every spin in this library uses.
//
// Rule of this library: no unbounded spin on the device. mbar_wait() polls for a limited time;
// when the limit is hit it records SPK_TIMEOUT in the device status word and returns false, and
// the caller drains what it has in flight (again bounded) and returns.
#pragma once

#include <cuda_bf16.h>

#include <cstdint>

namespace spk::ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier --------------------------------------------------------------------------------

__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

// Makes mbarrier initialisation visible to the asynchronous proxy (the TMA engine).
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// One try: the thread is suspended until the phase completes or a time slice has passed (the hint, in
// nanoseconds, asks for a long slice: a waiting warp should cost no issue slots, the SM's schedulers are
// shared with warps that have work). True if the phase has completed.
constexpr unsigned kSuspendHintNs = 1000000u;

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(kSuspendHintNs)
        : "memory");
    return ok != 0;
}

// Non-blocking probe: true if the phase has completed. Its result comes back through the scoreboard, so
// a probe issued before a stretch of arithmetic costs nothing if the answer is used only afterwards.
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Limit of one wait, in SM clock cycles: about a second at 2 GHz, far beyond any healthy copy or MMA
// (and beyond a chained launch's wait for the kernel in front), and short enough that a broken
// pipeline returns instead of hanging the GPU. The limit is a time, not a number of tries, because
// how long one try stays suspended is up to the hardware.
constexpr long long kWaitCycles = 2000000000ll;

// Bounded wait for phase `parity` of `bar`. On timeout writes SPK_TIMEOUT (3) to *status
// (first writer wins) and returns false.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity, int* status) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    do {
        if (mbar_try_wait(bar, parity)) return true;
    } while (clock64() - t0 < kWaitCycles);
    if (status != nullptr) atomicCAS(status, 0, 3);
    return false;
}

// ---- bulk asynchronous copy global -> shared (TMA, untiled) -----------------------------------
// dst and src 16-byte aligned, bytes a multiple of 16. Completion is signalled on `bar` as
// `bytes` of transaction count.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, unsigned bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// ---- loads -------------------------------------------------------------------------------------

// 16-byte read-only load that does not allocate in L1 (streamed once).
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// 16-byte read-only load through L1 (activations re-read by neighbouring warps).
__device__ __forceinline__ uint4 ldg_cached(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// ---- bf16 helpers ------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));  // (a & b) | c
    return d;
}
__device__ __forceinline__ uint32_t bf16x2_sub(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// D += A(16x16, row) * B(16x8, col), bf16 in, fp32 accumulate (warp-level legacy MMA).
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

}  // namespace spk::ptx
