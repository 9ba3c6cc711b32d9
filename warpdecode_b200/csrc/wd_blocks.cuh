// Building blocks of the fused MoE layer kernel: activation quantisers, the Q8_0 row task, the
// F32 dot, the float side of an IQ3_S tile, and the block-parallel router.
#pragma once

#include "wd_formats.cuh"

namespace wd {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxK = 16;
constexpr int kMaxExperts = 1024;

// ---------------------------------------------------------------------------------------------
// phase 0: activation quantisers (bit-exact twins of src/qwen38_cpu_moe.cuh:220-263)
// ---------------------------------------------------------------------------------------------
// Q8_0 of n floats (n multiple of 128) held in shared `xf`; output: quants in task layout
// [g][l][16 B] (word i = values 4l..4l+3 of block 4g+i) and per-block scales as the f16-rounded float.
__device__ __forceinline__ void quantize_q8_0_cta(const float *xf, int n, uint8_t *q_out, float *d_out) {
    const int nchunks = n >> 2;    // groups of four values; 8 chunks form a block
    for (int ch = threadIdx.x; ch < ((nchunks + 31) & ~31); ch += blockDim.x) {
        const bool live = ch < nchunks;
        float4 v = live ? *reinterpret_cast<const float4 *>(xf + 4 * ch) : make_float4(0, 0, 0, 0);
        float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
        if (!live) continue;
        const int b = ch >> 3, l = ch & 7;
        const __half dh = __float2half_rn(__fdiv_rn(amax, 127.0f));
        uint32_t packed = 0;
        if (amax != 0.0f) {
            const float inv = __fdiv_rn(127.0f, amax);
            const float f[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                int q = __float2int_rn(__fmul_rn(f[j], inv));
                q = max(-128, min(127, q));
                packed |= static_cast<uint32_t>(q & 0xff) << (8 * j);
            }
        }
        *reinterpret_cast<uint32_t *>(q_out + (((b >> 2) * 8 + l) * 16 + (b & 3) * 4)) = packed;
        if (l == 0) d_out[b] = __half2float(dh);
    }
}

// Q8_K of one 256-value superblock by one warp: lane holds values 8*lane .. 8*lane+7.
__device__ __forceinline__ void quantize_q8_K_warp(const float v[8], int lane, uint8_t *q_out_sb, float *d_out) {
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, s));
    uint32_t w0 = 0, w1 = 0;
    float d = 0.0f;
    if (amax != 0.0f) {
        const float iscale = __fdiv_rn(-127.0f, amax);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int q = min(127, __float2int_rn(__fmul_rn(v[j], iscale)));
            if (j < 4) w0 |= static_cast<uint32_t>(q & 0xff) << (8 * j);
            else w1 |= static_cast<uint32_t>(q & 0xff) << (8 * (j - 4));
        }
        d = __fdiv_rn(1.0f, iscale);
    }
    *reinterpret_cast<uint2 *>(q_out_sb + lane * 8) = make_uint2(w0, w1);
    if (lane == 0) *d_out = d;
}

// ---------------------------------------------------------------------------------------------
// Q8_0 x Q8_0 row task: 4 rows per warp, lane = (row r = lane / 8, chunk-lane l = lane & 7).
// One fmaf(d_w * d_x, int_dot, lane_acc) per block, blocks ascending, then the 8-lane reduction
// (src/qwen38_cpu_moe.cuh:424-440, device twin src/qwen38_hc.cuh:420).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float q8_task_row(const uint8_t *task, int nb, const uint8_t *xq, const float *xd,
                                             int lane) {
    const int r = lane >> 3, l = lane & 7;
    const uint8_t *wq = task + r * 128 + l * 16;
    const uint8_t *wd = task + nb * 128 + r * nb * 2;
    float acc = 0.0f;
    for (int g = 0; g < (nb >> 2); ++g) {
        const uint4 w = *reinterpret_cast<const uint4 *>(wq + g * 512);
        const uint4 a = *reinterpret_cast<const uint4 *>(xq + (g * 8 + l) * 16);
        const uint2 dw = *reinterpret_cast<const uint2 *>(wd + g * 8);
        const float4 dx = *reinterpret_cast<const float4 *>(xd + g * 4);
        const float s0 = __fmul_rn(half_bits_to_float(dw.x & 0xffffu), dx.x);
        const float s1 = __fmul_rn(half_bits_to_float(dw.x >> 16), dx.y);
        const float s2 = __fmul_rn(half_bits_to_float(dw.y & 0xffffu), dx.z);
        const float s3 = __fmul_rn(half_bits_to_float(dw.y >> 16), dx.w);
        acc = __fmaf_rn(s0, static_cast<float>(dp4a_s8(w.x, a.x, 0)), acc);
        acc = __fmaf_rn(s1, static_cast<float>(dp4a_s8(w.y, a.y, 0)), acc);
        acc = __fmaf_rn(s2, static_cast<float>(dp4a_s8(w.z, a.z, 0)), acc);
        acc = __fmaf_rn(s3, static_cast<float>(dp4a_s8(w.w, a.w, 0)), acc);
    }
    return hsum8_lanes(acc);
}

// ggml_vec_dot_f32 in its AVX2 order by one warp: lane t owns elements = t (mod 32)
// (src/qwen38_cpu_moe.cuh:847-871; n is a multiple of 32 here).
__device__ __forceinline__ float dot_f32_warp(const float *a, const float *b, int n, int lane) {
    float s = 0.0f;
    for (int i = lane; i < n; i += 32) s = __fmaf_rn(a[i], b[i], s);
    s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 16));
    s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 8));
    s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 4));
    s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 1));
    s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 2));
    return s;
}

// ---------------------------------------------------------------------------------------------
// float side of an IQ3_S tile: lanes hold (row, sb) integer partials; chains over sb are run per
// (row, chunk-lane) in superblock order with one fmaf each, then the 8-lane reduction
// (src/qwen38_cpu_moe.cuh:337-375). nsb in {1,2,4,8,16,32}; rows per tile R = 32 / nsb.
// Returns, in every lane, the finished row sums of rows r = (lane >> 3) + 4*it for it < nit.
// ---------------------------------------------------------------------------------------------
template <int MAXIT>
__device__ __forceinline__ void iq_tile_rows(const int partial[8], float scale, int nsb, int lane, float *scr,
                                             float rows_out[MAXIT]) {
    // scr layout: per tile row r a stripe of (nsb*8 + 8) floats: [sb][c], then after all stripes
    // the scales [r][sb]
    const int R = 32 / nsb;
    const int stripe = nsb * 8 + 8;
    const int r = lane / nsb, sb = lane % nsb;
    float *dst = scr + r * stripe + sb * 8;
    *reinterpret_cast<float4 *>(dst) = make_float4(static_cast<float>(partial[0]), static_cast<float>(partial[1]),
                                                   static_cast<float>(partial[2]), static_cast<float>(partial[3]));
    *reinterpret_cast<float4 *>(dst + 4) = make_float4(static_cast<float>(partial[4]), static_cast<float>(partial[5]),
                                                       static_cast<float>(partial[6]), static_cast<float>(partial[7]));
    float *sc = scr + R * stripe;
    sc[r * nsb + sb] = scale;
    __syncwarp();
    const int nit = (R * 8 + 31) / 32;
#pragma unroll
    for (int it = 0; it < MAXIT; ++it) {
        float acc = 0.0f;
        if (it < nit) {
            const int ch = it * 32 + lane;          // chain index = row * 8 + c
            const int rr = ch >> 3, c = ch & 7;
            if (rr < R) {
                for (int s = 0; s < nsb; ++s) acc = __fmaf_rn(sc[rr * nsb + s], scr[rr * stripe + s * 8 + c], acc);
            }
        }
        rows_out[it] = hsum8_lanes(acc);
    }
    __syncwarp();
}

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

__device__ __forceinline__ void router_select_cta(const float *logits, int E, int K, float w_scale,
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
