// Device-side building blocks of the MoE decode kernels (sm_100a).
//
// Arithmetic notes. Every float step that the CPU path of the reference performs as a single
// IEEE operation is written here with a rounding-mode intrinsic, so neither the compiler nor
// -use_fast_math can contract or reassociate it; results are then bit-identical to the
// reference's host code (src/qwen38_cpu_moe.cuh) and not merely close.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace wd {

// Error bits a kernel can raise in the engine's device status word.
enum : unsigned {
    kErrBarrierTimeout = 1u,   // a grid barrier wait ran out
    kErrCopyTimeout = 2u,      // a bulk copy never completed
    kErrExpertMiss = 4u,       // a selected expert has no slot
    kErrGeometry = 8u,         // launch geometry does not match the parameters
};

constexpr unsigned kSpinLimit = 1u << 22;   // polls before a wait gives up (well under a second)

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------------------------------------
// mbarrier + 1-D bulk copy (TMA unit, no tensor map, no multicast)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// global -> this CTA's shared memory; dst, src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_load(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait; on timeout raises kErrCopyTimeout and returns false (the caller carries on with
// whatever is in shared memory so that the kernel still terminates).
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, unsigned *err) {
    for (unsigned i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    atomicOr(err, kErrCopyTimeout);
    return false;
}

// ---------------------------------------------------------------------------------------------
// grid barrier (all CTAs co-resident: cooperative launch). Sense = generation counter.
// ---------------------------------------------------------------------------------------------
// One 64-bit counter that only ever grows: a CTA arrives with a release add and waits until the
// counter reaches the next multiple of the grid size. No reset, no second word, no full fence: one
// atomic and a few polling loads per barrier. (The host zeroes the counter after a reported error.)
// `target` is the counter value at which this barrier opens; the host hands every launch the value
// the counter had before it, so the kernel needs no returned value: the arrival is a fire-and-forget
// release reduction, the wait polls with relaxed loads and takes one acquire fence at the end.
__device__ __forceinline__ void grid_barrier(unsigned long long *ctr, unsigned long long target, unsigned *err) {
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long now;
        asm volatile("red.release.gpu.global.add.u64 [%0], 1;" ::"l"(ctr) : "memory");
        unsigned i = 0;
        for (;;) {
            asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(now) : "l"(ctr) : "memory");
            if (now >= target) break;
            if (++i > kSpinLimit) {
                atomicOr(err, kErrBarrierTimeout);
                break;
            }
        }
        asm volatile("fence.acquire.gpu;" ::: "memory");
    }
    __syncthreads();
}

// Order-preserving map float -> u32 for selection: larger float = larger key, NaN = 0 (never wins).
__device__ __forceinline__ uint32_t order_key(float v) {
    const uint32_t b = __float_as_uint(v);
    if (v != v) return 0u;
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
constexpr uint32_t kKeyNegInf = 0x007fffffu;   // order_key(-inf): nothing at or below it is selectable

// ---------------------------------------------------------------------------------------------
// scalar math in the reference's order
// ---------------------------------------------------------------------------------------------
// One lane of ggml's AVX2 ggml_v_expf (src/qwen38_exact_math.cuh:94-115, src/qwen38_cpu_moe.cuh:816-834).
__device__ __noinline__ float exp_ggml(float x) {
    const float r = 0x1.8p23f;
    const float z = __fmaf_rn(x, 0x1.715476p+0f, r);
    const float n = __fsub_rn(z, r);
    const float b = __fmaf_rn(-n, 0x1.7f7d1cp-20f, __fmaf_rn(-n, 0x1.62e4p-1f, x));
    const uint32_t e = __float_as_uint(z) << 23;
    const float k = __uint_as_float(e + 0x3f800000u);
    const float u = __fmul_rn(b, b);
    const float t0 = __fmaf_rn(0x1.0e4020p-7f, b, 0x1.573e2ep-5f);
    const float t1 = __fmaf_rn(t0, u, __fmaf_rn(0x1.555e66p-3f, b, 0x1.fffdb6p-2f));
    const float j = __fmaf_rn(t1, u, __fmul_rn(0x1.ffffecp-1f, b));
    if (!(fabsf(n) > 126.0f)) return __fmaf_rn(j, k, k);
    const uint32_t g = n <= 0.0f ? 0x82000000u : 0u;
    const float s1 = __uint_as_float(g + 0x7f000000u);
    const float s2 = __uint_as_float(e - g);
    if (fabsf(n) > 192.0f) return __fmul_rn(s1, s1);
    return __fmul_rn(__fmaf_rn(s2, j, s2), s1);
}
// src/qwen38_cpu_moe.cuh:836-842
__device__ __forceinline__ float silu_ggml(float x) { return __fdiv_rn(x, __fadd_rn(1.0f, exp_ggml(-x))); }
__device__ __forceinline__ float sigmoid_ggml(float x) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, exp_ggml(-x))); }

// Closing reduction of ggml's 8-lane accumulator across 8 consecutive lanes (lane & 7 = chunk-lane):
// (v0+v4, v1+v5, v2+v6, v3+v7) then (r0+r2) + (r1+r3) (src/qwen38_cpu_moe.cuh:290-296). Every
// lane of the group ends with the sum.
__device__ __forceinline__ float hsum8_lanes(float v) {
    v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 4));
    v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 2));
    v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 1));
    return v;
}

__device__ __forceinline__ float half_bits_to_float(uint16_t h) { return __half2float(__ushort_as_half(h)); }

// 4 x int8 dot with accumulate.
__device__ __forceinline__ int dp4a_s8(int a, int b, int c) { return __dp4a(a, b, c); }

}  // namespace wd
