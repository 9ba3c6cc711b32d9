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
    kErrBarrierTimeout = 1u,   // a wait for another CTA's (or GPU's) value ran out
    kErrCopyTimeout = 2u,      // a bulk copy never completed
    kErrExpertMiss = 4u,       // a selected expert has no slot
    kErrGeometry = 8u,         // launch geometry does not match the parameters
    kErrOverrun = 16u,         // a polled word carried a LATER layer's tag: it was overwritten before it was read
};

constexpr unsigned kSpinLimit = 1u << 20;   // polls before a copy wait gives up
constexpr unsigned long long kWaitLimitNs = 1000000000ull;   // a wait for another CTA or GPU gives up after one second

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t) : : "memory");
    return t;
}

// Programmatic dependent launch: a kernel launched with the programmatic-serialization attribute may start while its
// predecessor in the stream still runs. grid_dep_launch() lets the successor be scheduled from now on;
// grid_dep_wait() returns once the predecessor has completed and its memory is visible (at once for an ordinary launch).
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

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
// Bounded wait: one second of the global timer (checked every 64 polls; a poll can itself suspend the thread for a
// while), or 64 more polls once another wait of this launch has failed, so that a broken launch ends quickly. On
// timeout raises kErrCopyTimeout, leaves the barrier's shared-memory address in err[2] (first failure only, for
// diagnosis) and returns false; the caller carries on with whatever is in shared memory so that the kernel terminates.
__device__ __noinline__ bool mbar_wait_slow(uint64_t *bar, uint32_t parity, unsigned *err) {
    const unsigned long long t0 = global_timer_ns();
#pragma unroll 1
    for (unsigned i = 0;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63u) == 63u) {
            const bool others = (*reinterpret_cast<volatile unsigned *>(err) & (kErrBarrierTimeout | kErrCopyTimeout)) != 0u;
            if (others || global_timer_ns() - t0 > kWaitLimitNs) break;
        }
    }
    if ((atomicOr(err, kErrCopyTimeout) & kErrCopyTimeout) == 0u) err[2] = smem_u32(bar);
    return false;
}
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, unsigned *err) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, err);
}

// Integer atomics on this CTA's shared memory, addressed in the shared window (an atomic through a generic
// pointer has to find out at run time which memory it targets).
__device__ __forceinline__ void red_add_shared(int *p, int v) {
    asm volatile("red.shared.add.s32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}
__device__ __forceinline__ void red_or_shared(uint32_t *p, uint32_t v) {
    asm volatile("red.shared.or.b32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}
__device__ __forceinline__ int atom_add_shared(int *p, int v) {
    int old;
    asm volatile("atom.shared.add.s32 %0, [%1], %2;" : "=r"(old) : "r"(smem_u32(p)), "r"(v) : "memory");
    return old;
}

// with acquire-release ordering at CTA scope: what the thread wrote before is visible to whoever reads the new count
__device__ __forceinline__ int atom_add_shared_acq_rel(int *p, int v) {
    int old;
    asm volatile("atom.acq_rel.cta.shared.add.s32 %0, [%1], %2;" : "=r"(old) : "r"(smem_u32(p)), "r"(v) : "memory");
    return old;
}
__device__ __forceinline__ int atom_cas_shared(int *p, int expect, int v) {
    int old;
    asm volatile("atom.shared.cas.b32 %0, [%1], %2, %3;" : "=r"(old) : "r"(smem_u32(p)), "r"(expect), "r"(v) : "memory");
    return old;
}

// ---------------------------------------------------------------------------------------------
// Tagged words: a float and the tag of the layer that produced it, published with ONE 8-byte store.
// A consumer polls the word itself until the tag matches, so no fence and no separate flag is needed
// (an aligned 8-byte access is single-copy atomic). Tags grow monotonically over layers and launches.
// ---------------------------------------------------------------------------------------------
typedef unsigned long long tagged_t;

// True when a polling loop should give up: one second of the global timer has passed since its 1024th
// poll (a time limit, so that it does not depend on how long one poll takes: local L2 or another GPU
// over NVLink), or some other wait of this launch already failed (then the remaining waits end after
// 1024 polls, so that a broken launch still terminates quickly). Raises kErrBarrierTimeout. `t0` is
// the caller's loop-local start time, 0 before the loop.
__device__ __noinline__ bool wait_expired_slow(unsigned it, unsigned long long &t0, unsigned *err);
__device__ __forceinline__ bool wait_expired(unsigned it, unsigned long long &t0, unsigned *err) {
    if ((it & 0x3ffu) != 0x3ffu) return false;
    return wait_expired_slow(it, t0, err);
}
__device__ __noinline__ bool wait_expired_slow(unsigned it, unsigned long long &t0, unsigned *err) {
    const unsigned long long now = global_timer_ns();
    if (t0 == 0ull) t0 = now;
    if (now - t0 > kWaitLimitNs || it >= 0xfffffc00u ||
        (*reinterpret_cast<volatile unsigned *>(err) & (kErrBarrierTimeout | kErrCopyTimeout)) != 0u) {
        atomicOr(err, kErrBarrierTimeout);
        return true;
    }
    return false;
}

// Tags are compared as a wrapping sequence. A word whose tag is still behind the wanted one has not been
// written yet; one whose tag is ahead was overwritten by a later layer before this reader got to it,
// which the exchange protocol must never allow: it is reported (kErrOverrun) instead of waited for.
__device__ __forceinline__ unsigned tag_behind(tagged_t w, uint32_t tag) {
    return static_cast<int32_t>(static_cast<uint32_t>(w >> 32) - tag) < 0;
}
__device__ __forceinline__ unsigned tag_ahead(tagged_t w, uint32_t tag) {
    return static_cast<int32_t>(static_cast<uint32_t>(w >> 32) - tag) > 0;
}
__device__ __noinline__ void report_overrun_slow(unsigned *err) { atomicOr(err, kErrOverrun); }
__device__ __forceinline__ void report_overrun(unsigned over, unsigned *err) {
    if (over) report_overrun_slow(err);
}

__device__ __forceinline__ tagged_t make_tagged(float v, uint32_t tag) {
    return (static_cast<unsigned long long>(tag) << 32) | __float_as_uint(v);
}
__device__ __forceinline__ void st_tagged(tagged_t *p, float v, uint32_t tag) {
    asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(p), "l"(make_tagged(v, tag)) : "memory");
}
// same, to memory that may belong to another GPU
__device__ __forceinline__ void st_tagged_sys(tagged_t *p, float v, uint32_t tag) {
    asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(p), "l"(make_tagged(v, tag)) : "memory");
}
// same, ordered after this thread's earlier loads and stores (a progress word that tells another GPU that
// this one has finished READING something must not pass those reads)
__device__ __forceinline__ void st_tagged_sys_release(tagged_t *p, float v, uint32_t tag) {
    asm volatile("st.release.sys.global.b64 [%0], %1;" ::"l"(p), "l"(make_tagged(v, tag)) : "memory");
}
__device__ __forceinline__ tagged_t ld_tagged(const tagged_t *p) {
    tagged_t w;
    asm volatile("ld.relaxed.gpu.global.b64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return w;
}
// Polls up to N words (word i at p[i * stride], i < n) until every tag has reached `tag`; values to out[].
// Bounded: on timeout raises kErrBarrierTimeout and returns what it has; a tag beyond `tag` raises kErrOverrun.
template <int N>
__device__ __forceinline__ void wait_tagged(const tagged_t *p, int stride, int n, uint32_t tag, float out[N],
                                            unsigned *err) {
    tagged_t w[N] = {};
    unsigned long long t0 = 0ull;
    for (unsigned it = 0;; ++it) {
        // all loads first, then the checks, so that the loads are in flight together
#pragma unroll
        for (int i = 0; i < N; ++i)
            if (i < n) w[i] = ld_tagged(p + static_cast<size_t>(i) * stride);
        unsigned bad = 0;
#pragma unroll
        for (int i = 0; i < N; ++i) bad |= (i < n) & tag_behind(w[i], tag);
        if (!bad) break;
        if (wait_expired(it, t0, err)) break;
    }
    unsigned over = 0;
#pragma unroll
    for (int i = 0; i < N; ++i) over |= (i < n) & tag_ahead(w[i], tag);
    report_overrun(over, err);
#pragma unroll
    for (int i = 0; i < N; ++i) out[i] = i < n ? __uint_as_float(static_cast<uint32_t>(w[i])) : 0.0f;
}

// Same with one address per word.
template <int N>
__device__ __forceinline__ void wait_tagged_at(const tagged_t *const p[N], int n, uint32_t tag, float out[N],
                                               unsigned *err) {
    tagged_t w[N] = {};
    unsigned long long t0 = 0ull;
    for (unsigned it = 0;; ++it) {
#pragma unroll
        for (int i = 0; i < N; ++i)
            if (i < n) w[i] = ld_tagged(p[i]);
        unsigned bad = 0;
#pragma unroll
        for (int i = 0; i < N; ++i) bad |= (i < n) & tag_behind(w[i], tag);
        if (!bad) break;
        if (wait_expired(it, t0, err)) break;
    }
    unsigned over = 0;
#pragma unroll
    for (int i = 0; i < N; ++i) over |= (i < n) & tag_ahead(w[i], tag);
    report_overrun(over, err);
#pragma unroll
    for (int i = 0; i < N; ++i) out[i] = i < n ? __uint_as_float(static_cast<uint32_t>(w[i])) : 0.0f;
}
// Waits until the tag of *p has reached `tag` (tags compared as a wrapping sequence).
__device__ __forceinline__ void wait_tag_reached(const tagged_t *p, uint32_t tag, unsigned *err) {
    unsigned long long t0 = 0ull;
    for (unsigned it = 0;; ++it) {
        const uint32_t t = static_cast<uint32_t>(ld_tagged(p) >> 32);
        if (static_cast<int32_t>(t - tag) >= 0) break;
        if (wait_expired(it, t0, err)) break;
    }
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
__device__ __forceinline__ float exp_ggml(float x) {
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
