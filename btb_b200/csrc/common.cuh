// Shared device helpers of the sm_100a decode kernels: bf16 conversions, the error convention, bounded mbarrier
// waits and 1-D bulk (TMA) copies into shared memory.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

typedef __nv_bfloat16 bf16;

// ---- the C-ABI's return codes: the reference's (native/src/lib.rs:17-33) plus two for the device --------------
#define B2_OK 0
#define B2_ERR_NULL (-1)
#define B2_ERR_DOMAIN (-6)
#define B2_ERR_CUDA (-10)
#define B2_ERR_TIMEOUT (-11)

#define NEG_INF (__int_as_float(0xff800000))

__device__ __forceinline__ float bf2f(bf16 v) { return __bfloat162float(v); }
__device__ __forceinline__ bf16 f2bf(float v) { return __float2bfloat16_rn(v); }
__device__ __forceinline__ float bfround(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
// the two bf16 of a 32-bit word as f32: the low half is the earlier element
__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// Two bf16 times two bf16 into an f32 chain: acc = fma(w_lo, x_lo, acc), then acc = fma(w_hi, x_hi, acc), the
// operands bf16 as they lie in their packed words and the sum f32 - sm_100's mixed-precision fma. A bf16 product is
// exact in f32, so each step is fmaf(float(w), float(x), acc) to the bit, without the two widening instructions.
__device__ __forceinline__ float fma2_bf16(uint32_t w, uint32_t x, float acc) {
    asm("{\n.reg .b16 wl, wh, xl, xh;\nmov.b32 {wl, wh}, %1;\nmov.b32 {xl, xh}, %2;\nfma.rn.f32.bf16 %0, wl, xl, %0;\n"
        "fma.rn.f32.bf16 %0, wh, xh, %0;\n}\n"
        : "+f"(acc)
        : "r"(w), "r"(x));
    return acc;
}

// one step of such a chain with the operands' halves named: HW, HX 0 the low half (the earlier element), 1 the high
#define B2_FMA1(WH, XH)                                                                                              \
    asm("{\n.reg .b16 wl, wh, xl, xh;\nmov.b32 {wl, wh}, %1;\nmov.b32 {xl, xh}, %2;\nfma.rn.f32.bf16 %0, " WH ", " XH \
        ", %0;\n}\n"                                                                                                 \
        : "+f"(acc)                                                                                                  \
        : "r"(w), "r"(x))
template <int HW, int HX>
__device__ __forceinline__ float fma1_bf16(uint32_t w, uint32_t x, float acc) {
    if (HW == 0 && HX == 0) B2_FMA1("wl", "xl");
    else if (HW == 0 && HX == 1) B2_FMA1("wl", "xh");
    else if (HW == 1 && HX == 0) B2_FMA1("wh", "xl");
    else B2_FMA1("wh", "xh");
    return acc;
}

// the same with the operands as 16-bit values: a packed word's halves (free: they name the word's register halves) and one step
__device__ __forceinline__ void split_bf16(uint32_t w, unsigned short& lo, unsigned short& hi) {
    asm("mov.b32 {%0, %1}, %2;" : "=h"(lo), "=h"(hi) : "r"(w));
}
__device__ __forceinline__ float fma_bf16(unsigned short w, unsigned short x, float acc) {
    asm("fma.rn.f32.bf16 %0, %1, %2, %0;" : "+f"(acc) : "h"(w), "h"(x));
    return acc;
}

// two e4m3fn bytes (the low 16 bits of `two`) times an f32 scale, each product rounded to f32 and then to the nearest
// bf16 (ties to even), as the packed pair (first byte in the low half): the weight btb's FP8 codec holds
// (btb/fp8.py:36-46, 97-100). e4m3 -> f16 is one conversion a pair; f16 -> f32 goes through the fma pipe
// (fma.rn.f32.f16 with 1 and -0: exact, the sign of a zero kept) instead of the narrower conversion unit; the pair is
// packed by one cvt.rn.bf16x2.f32.
__device__ __forceinline__ uint32_t e4m3x2_held_pair(uint32_t two, float scale) {
    uint32_t h, p;
    float f0, f1;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h) : "h"((unsigned short)(two & 0xffffu)));
    asm("{\n.reg .b16 lo, hi, one;\nmov.b32 {lo, hi}, %2;\nmov.b16 one, 0x3C00;\nfma.rn.f32.f16 %0, lo, one, %3;\n"
        "fma.rn.f32.f16 %1, hi, one, %3;\n}\n"
        : "=f"(f0), "=f"(f1)
        : "r"(h), "f"(-0.0f));
    f0 = __fmul_rn(f0, scale);
    f1 = __fmul_rn(f1, scale);
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(p) : "f"(f1), "f"(f0));
    return p;
}

// the butterfly every card reduction ends with (xor 16, 8, 4, 2, 1): the order is part of the result's bits
__device__ __forceinline__ float warp_sum(float a) {
    a += __shfl_xor_sync(0xffffffffu, a, 16);
    a += __shfl_xor_sync(0xffffffffu, a, 8);
    a += __shfl_xor_sync(0xffffffffu, a, 4);
    a += __shfl_xor_sync(0xffffffffu, a, 2);
    a += __shfl_xor_sync(0xffffffffu, a, 1);
    return a;
}

// ---- device status word -----------------------------------------------------------------------------------------
// A kernel that gives up a bounded wait records where in this word and returns; the host reads it with
// btb_b200_status(). Kernels never trap.
// Each translation unit holds its own word (no relocatable device code needed) and exposes a host function that
// reads and clears it; btb_b200_status() asks every unit.
static __device__ int g_b2_status = 0;
__device__ __forceinline__ void b2_fail(int code) { atomicCAS(&g_b2_status, 0, code); }
#define B2_DEFINE_STATUS(unit)                                                                              \
    int b2_status_take_##unit(int* v) {                                                                     \
        *v = 0;                                                                                             \
        if (cudaMemcpyFromSymbol(v, g_b2_status, sizeof(int)) != cudaSuccess) return B2_ERR_CUDA;           \
        if (*v != 0) {                                                                                      \
            const int zero = 0;                                                                             \
            if (cudaMemcpyToSymbol(g_b2_status, &zero, sizeof(int)) != cudaSuccess) return B2_ERR_CUDA;     \
        }                                                                                                   \
        return B2_OK;                                                                                       \
    }

// ---- mbarrier + bulk copy ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    // makes the barriers' initial state visible to the async proxy that will complete transactions on them
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// a wait that gives up: each try suspends the thread for a hardware-bounded time, so the limit is of the order of
// a second, far past any healthy copy
#define B2_WAIT_LIMIT (1u << 22)
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    for (uint32_t it = 0; it < B2_WAIT_LIMIT; ++it)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// global -> shared bulk copy (the TMA unit's untiled form): both addresses 16-byte aligned, bytes a multiple of
// 16; completion is counted in bytes on the barrier. No cluster multicast anywhere in this library.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
// the same with an L2 evict-first policy: weights are read once a step and must not push the cache's rows and the
// activations out of L2
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_g2s_hint(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar,
                                              uint64_t pol) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::
            "r"(dst),
        "l"(src), "r"(bytes), "r"(bar), "l"(pol)
        : "memory");
}
// orders this thread's earlier generic-proxy accesses to shared memory before later async-proxy ones (a stage is
// read by the lanes, then refilled by a bulk copy)
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- programmatic dependent launch ------------------------------------------------------------------------------
// wait: everything the grids before this one wrote is visible after it (a no-op without the launch attribute).
// launch_dependents: the next grid in the stream may start its prologue now.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
