// Block-parallel router of the fused MoE layer kernel.
#pragma once

#include "wd_blocks.cuh"

namespace wd {

// ---------------------------------------------------------------------------------------------
// router: softmax over all experts + top-k by the whole CTA (src/qwen38_moe.cuh:711-818).
// Thread t owns experts t and t + kThreads (E <= 1024). Every float step is the reference's:
// running max; exp_ggml(x - max); groups of eight summed in the AVX2 lane order; the group sums
// accumulated ascending into a double by one thread; p * (float)(1 / sum); k rungs of "largest
// remaining probability, ties to the lower index, NaN never, nothing above -inf gives id 0";
// weights = picked / max((float)double_sum, 2^-14), times w_scale unless it is 0 or 1.
// The rungs run as a tournament: each warp keeps its champion (key, index) in shared memory, all
// warps read the 16 champions and agree on the winner with two redux steps, and only the winner's
// warp recomputes its champion. One __syncthreads per rung.
// Shared scratch: probs[E], gsum[E/8], champ[2][kWarps][2] u32, dsum[2] double, top[kMaxK].
// ---------------------------------------------------------------------------------------------
struct RouterScratch {
    float *probs;       // [E]
    float *gsum;        // [E/8]
    uint32_t *champ;    // [2][kWarps][2]
    double *dsum;       // [2]
    float *red;         // [kWarps]
    float *top;         // [kMaxK]
};

__device__ __noinline__ void router_select_cta(const float *logits, int E, int K, float w_scale,
                                                  const RouterScratch &S, int *ids_out, float *w_out) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int e0 = tid, e1 = tid + kThreads;
    const bool h0 = e0 < E, h1 = e1 < E;
    const float l0 = h0 ? logits[e0] : -INFINITY, l1 = h1 ? logits[e1] : -INFINITY;
    float mx = fmaxf(l0, l1);
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
    if (lane == 0) S.red[warp] = mx;
    __syncthreads();
    mx = S.red[0];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) mx = fmaxf(mx, S.red[w]);
    float p0 = h0 ? exp_ggml(__fsub_rn(l0, mx)) : 0.0f;
    float p1 = h1 ? exp_ggml(__fsub_rn(l1, mx)) : 0.0f;
    const float g0 = hsum8_lanes(p0), g1 = hsum8_lanes(p1);   // the reference's 8-lane tree
    if ((lane & 7) == 0) {
        if (h0) S.gsum[e0 >> 3] = g0;
        if (h1) S.gsum[e1 >> 3] = g1;
    }
    __syncthreads();
    if (warp == 0) {
        // The reference adds the group sums one by one, ascending, into a double. When every partial
        // sum is exactly representable the order cannot matter, and a shuffle tree gives the same bits:
        // all terms are non-negative multiples of the smallest term's last bit q, so any partial sum is
        // a multiple of q below the total; it is exact if total < 2^53 * q, i.e. if the exponent span
        // between the total and the smallest non-zero term (minus its 23 mantissa bits) stays under 53.
        // Otherwise (and for inf/nan/denormal terms) one lane replays the reference's order.
        const int ng = E >> 3;
        double part = 0.0;
        int min_exp = 0x7fffffff, bad = 0;
        for (int g = lane; g < ng; g += 32) {
            const float v = S.gsum[g];
            const int ex = static_cast<int>((__float_as_uint(v) >> 23) & 0xffu);
            if (v != 0.0f) {
                if (ex == 0 || ex == 255 || v < 0.0f) bad = 1;
                min_exp = min(min_exp, ex);
            }
            part = __dadd_rn(part, static_cast<double>(v));
        }
#pragma unroll
        for (int s = 1; s < 32; s <<= 1) part = __dadd_rn(part, __shfl_xor_sync(0xffffffffu, part, s));
        min_exp = __reduce_min_sync(0xffffffffu, min_exp);
        bad = __any_sync(0xffffffffu, bad);
        const int tot_exp = static_cast<int>((__double_as_longlong(part) >> 52) & 0x7ff) - 1023 + 127;   // float-biased
        double sum = part;
        if (bad || (min_exp != 0x7fffffff && tot_exp + 1 - (min_exp - 23) > 52)) {
            sum = 0.0;
            if (lane == 0)
                for (int g = 0; g < ng; ++g) sum = __dadd_rn(sum, static_cast<double>(S.gsum[g]));
        }
        if (lane == 0) {
            S.dsum[0] = sum;
            S.dsum[1] = sum == 0.0 ? 0.0 : static_cast<double>(__double2float_rn(__ddiv_rn(1.0, sum)));
        }
    }
    __syncthreads();
    const double sum = S.dsum[0];
    if (sum == 0.0) {
        p0 = p1 = -INFINITY;
    } else {
        const float inv = static_cast<float>(S.dsum[1]);
        p0 = __fmul_rn(p0, inv);
        p1 = __fmul_rn(p1, inv);
    }
    if (h0) S.probs[e0] = p0;
    if (h1) S.probs[e1] = p1;
    uint32_t k0 = h0 ? order_key(p0) : 0u, k1 = h1 ? order_key(p1) : 0u;
    bool dirty = true;
    for (int j = 0; j < K; ++j) {
        uint32_t *cw = S.champ + (j & 1) * kWarps * 2;
        if (dirty) {
            const uint32_t mine = max(k0, k1);
            const uint32_t m = __reduce_max_sync(0xffffffffu, mine);
            const uint32_t cand = (k0 == m) ? static_cast<uint32_t>(e0) : ((k1 == m) ? static_cast<uint32_t>(e1) : 0xffffffffu);
            const uint32_t mi = __reduce_min_sync(0xffffffffu, cand);
            if (lane == 0) {
                cw[warp * 2] = m;
                cw[warp * 2 + 1] = mi;
            }
            dirty = false;
        } else if (lane == 0) {
            const uint32_t *pw = S.champ + ((j & 1) ^ 1) * kWarps * 2;
            cw[warp * 2] = pw[warp * 2];
            cw[warp * 2 + 1] = pw[warp * 2 + 1];
        }
        __syncthreads();
        const uint32_t cm = lane < kWarps ? cw[lane * 2] : 0u;
        const uint32_t ci = lane < kWarps ? cw[lane * 2 + 1] : 0xffffffffu;
        const uint32_t M = __reduce_max_sync(0xffffffffu, cm);
        uint32_t win = __reduce_min_sync(0xffffffffu, cm == M ? ci : 0xffffffffu);
        if (M <= kKeyNegInf) win = 0u;                 // nothing selectable: the rung keeps expert 0
        else {
            if (win == static_cast<uint32_t>(e0)) k0 = 0u;
            if (win == static_cast<uint32_t>(e1)) k1 = 0u;
            if (((win & (kThreads - 1)) >> 5) == static_cast<uint32_t>(warp)) dirty = true;
        }
        if (tid == 0) {
            ids_out[j] = static_cast<int>(win);
            S.top[j] = S.probs[win];
        }
    }
    __syncthreads();
    if (tid == 0) {
        double wsum = 0.0;
        for (int j = 0; j < K; ++j) wsum = __dadd_rn(wsum, static_cast<double>(S.top[j]));
        const float denom = fmaxf(__double2float_rn(wsum), 6.103515625e-5f);
        for (int j = 0; j < K; ++j) {
            float w = __fdiv_rn(S.top[j], denom);
            if (w_scale != 0.0f && w_scale != 1.0f) w = __fmul_rn(w, w_scale);
            w_out[j] = w;
        }
    }
    __syncthreads();
}

}  // namespace wd
