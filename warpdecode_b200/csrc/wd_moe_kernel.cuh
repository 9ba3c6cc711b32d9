// The fused MoE layer kernel: one persistent cooperative launch per layer (batch 1).
//
//   phase 0  every CTA: x (optionally RMSNorm(residual) * w) -> Q8_0 and Q8_K blocks in shared memory
//   phase 1  Q8_0 row tasks spread over the grid: router logits, shared-expert gate/up + SiLU,
//            shared gate scalar                                     -> grid barrier
//   phase 1b every CTA: softmax / top-k (one warp), shared activation -> Q8_0; then ALL bulk copies
//            of this CTA's share of the selected experts' gate/up/down tiles are issued at once
//   phase 2  gate+up tiles -> SiLU(g)*u per expert row                -> grid barrier
//   phase 3  expert activations -> Q8_K; down tiles and shared-down rows; the warp that delivers
//            the last contribution of a 16-row output tile performs the ordered combine
//
// Reference call sites this replaces: q38_moe_select_experts_f32_x (src/qwen38_moe.cuh:2323),
// q38_moe_run_batched_experts (:3312, five launches), run_qwen38_shared_expert_f32_x (:3963, nine
// launches), q38_finish_moe_f32 (:2442) and the per-layer ids D2H + stream sync (:2363-2379).
#pragma once

#include "wd_formats.cuh"

namespace wd {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxK = 16;
constexpr int kMaxExperts = 1024;
constexpr int kMaxBars = 96;

struct MoeParams {
    // geometry
    int H, F, SF, E, K;
    int nsb_h, nsb_f;            // superblocks per row of gate/up and of down
    int e_first, e_count;        // owned expert range
    float w_scale, eps;
    // layer weights (device, repacked)
    const uint8_t *router_w;     // Q8_0 tasks [E/4]
    const float *router_bias;    // nullable
    const float *sh_gate_vec;    // F32 [H]
    const uint8_t *sh_gate, *sh_up, *sh_down;   // Q8_0 tasks
    const float *norm_w;         // nullable
    const int *slot_of_expert;   // [E] slot index or -1
    const uint8_t *pool;         // slot pool base
    unsigned long long slot_bytes;
    unsigned gate_off, up_off, down_off;        // offsets of the three matrices inside a slot
    const uint16_t *grid_packed; // packed codebook in global memory
    // activations
    const float *x;              // [H] (used when residual == nullptr)
    float *residual;             // nullable: x = RMSNorm(residual) * norm_w, residual += out
    float *out;                  // [H]
    // scratch (global)
    float *logits;               // [E]
    int *ids;                    // [K]
    float *weights;              // [K]
    float *act;                  // [K][F]
    float *expert_out;           // [K][H]
    float *routed;               // [H]
    float *shared_act;           // [SF]
    float *shared_down;          // [H]
    float *shared_gate;          // [1]
    unsigned long long *stamps;  // nullable: [cta][16] globaltimer values at phase boundaries (profiling)
    unsigned *sync;              // [0] barrier count, [1] generation, [2] error word, [16..] tile counters
    // shared memory plan (byte offsets from the dynamic shared base; all 16-byte aligned)
    unsigned off_tab, off_xq0, off_xd0, off_xk, off_xdk, off_actk, off_actd, off_shq, off_shd,
        off_misc, off_scr, off_bar, off_stage_a, off_stage_b;
    unsigned scr_bytes;          // per-warp transposition scratch
    unsigned n1r, n1s, n2, n3, nsd;   // staging slots per CTA: router tasks, shared g/u tasks, phase-2 units,
                                      // phase-3 tiles, shared-down tasks
};

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
// router: softmax over all experts + top-k by one warp (src/qwen38_moe.cuh:711-818).
// Lane L owns the groups of eight g = L, L+32, ...; at most 4 groups (E <= 1024).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void router_topk_warp(const float *logits, int E, int K, float w_scale, int lane,
                                                 float *gsum_smem, float *top_smem, int *ids_out,
                                                 float *w_out, float *probs_out) {
    const int ngroups = E >> 3;
    float p[32];
    float mx = -INFINITY;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
        const int g = lane + 32 * t;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            p[t * 8 + j] = g < ngroups ? logits[g * 8 + j] : -INFINITY;
            if (g < ngroups) mx = fmaxf(mx, p[t * 8 + j]);
        }
    }
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
#pragma unroll
    for (int t = 0; t < 4; ++t) {
        const int g = lane + 32 * t;
        if (g < ngroups) {
#pragma unroll
            for (int j = 0; j < 8; ++j) p[t * 8 + j] = exp_ggml(__fsub_rn(p[t * 8 + j], mx));
            const float *v = &p[t * 8];
            const float lo = __fadd_rn(v[0], v[4]), lh = __fadd_rn(v[2], v[6]);
            const float hi = __fadd_rn(v[1], v[5]), hh = __fadd_rn(v[3], v[7]);
            gsum_smem[g] = __fadd_rn(__fadd_rn(lo, lh), __fadd_rn(hi, hh));
        }
    }
    __syncwarp();
    double sum = 0.0;
    if (lane == 0) {
        for (int g = 0; g < ngroups; ++g) sum = __dadd_rn(sum, static_cast<double>(gsum_smem[g]));
    }
    sum = __shfl_sync(0xffffffffu, sum, 0);
    if (sum == 0.0) {
#pragma unroll
        for (int i = 0; i < 32; ++i) p[i] = -INFINITY;
    } else {
        const float inv = __double2float_rn(__ddiv_rn(1.0, sum));
#pragma unroll
        for (int i = 0; i < 32; ++i) p[i] = __fmul_rn(p[i], inv);
    }
    if (probs_out) {
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const int g = lane + 32 * t;
            if (g < ngroups) {
#pragma unroll
                for (int j = 0; j < 8; ++j) probs_out[g * 8 + j] = p[t * 8 + j];
            }
        }
    }
    // k rungs of a descending argsort: higher probability wins, equal falls to the lower index,
    // a NaN is never promoted, nothing above -inf leaves (value of expert 0, id 0).
    unsigned taken = 0;
    const float p0 = __shfl_sync(0xffffffffu, p[0], 0);   // probability of expert 0
    for (int j = 0; j < K; ++j) {
        float best = -INFINITY;
        int best_id = 0x7fffffff;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const int g = lane + 32 * t;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int slot = t * 8 + i;
                if (g < ngroups && !((taken >> slot) & 1u) && p[slot] > best) {
                    best = p[slot];
                    best_id = g * 8 + i;
                }
            }
        }
#pragma unroll
        for (int s = 1; s < 32; s <<= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, s);
            const int oi = __shfl_xor_sync(0xffffffffu, best_id, s);
            if (ov > best || (ov == best && oi < best_id)) {
                best = ov;
                best_id = oi;
            }
        }
        float val = best;
        if (best_id == 0x7fffffff) {   // no candidate anywhere: the reference's rung keeps id 0
            best_id = 0;
            val = p0;
        } else {
            const int g = best_id >> 3;
            if ((g & 31) == lane) taken |= 1u << (((g >> 5) << 3) | (best_id & 7));
        }
        if (lane == 0) {
            ids_out[j] = best_id;
            top_smem[j] = val;
        }
    }
    __syncwarp();
    if (lane == 0) {
        double wsum = 0.0;
        for (int j = 0; j < K; ++j) wsum = __dadd_rn(wsum, static_cast<double>(top_smem[j]));
        const float denom = fmaxf(__double2float_rn(wsum), 6.103515625e-5f);
        for (int j = 0; j < K; ++j) {
            float w = __fdiv_rn(top_smem[j], denom);
            if (w_scale != 0.0f && w_scale != 1.0f) w = __fmul_rn(w, w_scale);
            w_out[j] = w;
        }
    }
    __syncwarp();
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
// the kernel
// ---------------------------------------------------------------------------------------------
extern __shared__ __align__(128) uint8_t wd_smem[];

__global__ void __launch_bounds__(kThreads, 1) moe_layer_kernel(const __grid_constant__ MoeParams P) {
    uint8_t *sm = wd_smem;
    uint8_t *tab = sm + P.off_tab;
    uint8_t *xq0 = sm + P.off_xq0;                                   // Q8_0 quants of x
    float *xd0 = reinterpret_cast<float *>(sm + P.off_xd0);          // Q8_0 scales of x
    uint8_t *xk = sm + P.off_xk;                                     // Q8_K quants of x, kActSbStride per superblock
    float *xdk = reinterpret_cast<float *>(sm + P.off_xdk);
    uint8_t *actk = sm + P.off_actk;                                 // per selected expert: Q8_K act
    float *actd = reinterpret_cast<float *>(sm + P.off_actd);
    uint8_t *shq = sm + P.off_shq;                                   // Q8_0 quants of the shared activation
    float *shd = reinterpret_cast<float *>(sm + P.off_shd);
    float *misc = reinterpret_cast<float *>(sm + P.off_misc);        // x as float, later logits etc.
    uint64_t *bars = reinterpret_cast<uint64_t *>(sm + P.off_bar);
    uint8_t *stage_a = sm + P.off_stage_a;
    uint8_t *stage_b = sm + P.off_stage_b;
    unsigned *err = P.sync + 2;
    unsigned *tile_cnt = P.sync + 16;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cta = blockIdx.x, ncta = gridDim.x;
    const int nbh = P.H >> 5, nbs = P.SF >> 5;
    const uint32_t lane4x2 = static_cast<uint32_t>(lane * 4) * 0x0101u;
    float *scr = reinterpret_cast<float *>(sm + P.off_scr + warp * P.scr_bytes);

    // ---- shared memory carve inside misc: xf[H] first, reused after phase 1 -------------------
    float *xf = misc;                                   // [H]
    float *gsum = misc;                                 // [E/8]   (after the barrier)
    float *topv = misc + 128;                           // [K]
    int *sel_ids = reinterpret_cast<int *>(misc + 160); // [K]
    float *sel_w = misc + 192;                          // [K]
    int *loc_j = reinterpret_cast<int *>(misc + 224);   // [K] rank-order index of each owned selected expert
    int *loc_slot = reinterpret_cast<int *>(misc + 256);// [K]
    int *loc_n = reinterpret_cast<int *>(misc + 288);   // [1]
    float *red = misc + 320;                            // [64] reduction scratch (as double pairs)

#define WD_STAMP(i)                                                                            \
    if (P.stamps != nullptr && tid == 0) {                                                     \
        unsigned long long t__;                                                                \
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__));                                \
        P.stamps[cta * 16 + (i)] = t__;                                                        \
    }
    WD_STAMP(0);
    const int n_bars = P.n1r + P.n1s + P.n2 + P.n3 + P.nsd;
    if (tid == 0) {
        for (int i = 0; i < n_bars; ++i) mbar_init(&bars[i], 1);
        mbar_fence_init();
    }
    build_grid_table(tab, P.grid_packed);
    __syncthreads();
    WD_STAMP(1);   // table built

    // ---- issue phase-1 copies: router tasks and shared gate/up tasks of this CTA --------------
    const int n_rt = P.E >> 2;                     // router tasks (4 rows each)
    const int n_st = P.SF >> 2;                    // shared gate/up tasks (4 row pairs each)
    const unsigned rt_bytes = static_cast<unsigned>(nbh) * 136u;
    const unsigned a1_slot = 2u * rt_bytes;        // staging slot of phase 1
    if (tid == 0) {
        int s = 0;
        for (int t = cta; t < n_rt; t += ncta, ++s) {
            mbar_expect_tx(&bars[s], rt_bytes);
            bulk_load(stage_a + s * a1_slot, P.router_w + static_cast<size_t>(t) * rt_bytes, rt_bytes, &bars[s]);
        }
        s = P.n1r;
        for (int t = ncta - 1 - cta; t < n_st; t += ncta, ++s) {
            mbar_expect_tx(&bars[s], 2u * rt_bytes);
            bulk_load(stage_a + s * a1_slot, P.sh_gate + static_cast<size_t>(t) * rt_bytes, rt_bytes, &bars[s]);
            bulk_load(stage_a + s * a1_slot + rt_bytes, P.sh_up + static_cast<size_t>(t) * rt_bytes, rt_bytes, &bars[s]);
        }
    }

    // ---- phase 0: x -> shared (with the optional RMSNorm prologue), then both quantisations --
    if (P.residual != nullptr) {
        // sum of squares as a perfect binary tree over consecutive elements, in double
        const int epl = P.H >= kThreads ? P.H / kThreads : 1;
        double ss = 0.0;
        if (tid * epl < P.H) {
            double loc[16];
            for (int i = 0; i < epl; ++i) {
                const double v = static_cast<double>(P.residual[tid * epl + i]);
                loc[i] = __dmul_rn(v, v);
            }
            for (int w = 1; w < epl; w <<= 1)
                for (int i = 0; i + w < epl; i += 2 * w) loc[i] = __dadd_rn(loc[i], loc[i + w]);
            ss = loc[0];
        }
#pragma unroll
        for (int s = 1; s < 32; s <<= 1) ss = __dadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, s));
        double *redd = reinterpret_cast<double *>(red);
        if (lane == 0) redd[warp] = ss;
        __syncthreads();
        double tot[kWarps];
#pragma unroll
        for (int i = 0; i < kWarps; ++i) tot[i] = redd[i];
#pragma unroll
        for (int w = 1; w < kWarps; w <<= 1)
#pragma unroll
            for (int i = 0; i + w < kWarps; i += 2 * w) tot[i] = __dadd_rn(tot[i], tot[i + w]);
        const float scale = __double2float_rn(
            __ddiv_rn(1.0, __dsqrt_rn(__dadd_rn(__ddiv_rn(tot[0], static_cast<double>(P.H)), static_cast<double>(P.eps)))));
        __syncthreads();   // red is about to be covered by xf
        for (int i = tid; i < P.H; i += kThreads) {
            float v = __fmul_rn(P.residual[i], scale);
            if (P.norm_w) v = __fmul_rn(v, P.norm_w[i]);
            xf[i] = v;
        }
    } else {
        for (int i = tid; i < P.H; i += kThreads) xf[i] = P.x[i];
    }
    __syncthreads();
    quantize_q8_0_cta(xf, P.H, xq0, xd0);
    for (int sb = warp; sb < P.nsb_h; sb += kWarps) {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = xf[sb * 256 + lane * 8 + j];
        quantize_q8_K_warp(v, lane, xk + sb * kActSbStride, &xdk[sb]);
    }
    __syncthreads();
    WD_STAMP(2);   // x quantised

    // ---- phase 1: Q8_0 row tasks ------------------------------------------------------------
    {
        // local task list: [0, n1r) router, [n1r, n1r+n1s) shared gate/up; one warp per task
        const int my_rt = cta < n_rt ? (n_rt - cta + ncta - 1) / ncta : 0;
        const int first_st = ncta - 1 - cta;
        const int my_st = first_st < n_st ? (n_st - first_st + ncta - 1) / ncta : 0;
        for (int lt = warp; lt < my_rt + my_st; lt += kWarps) {
            if (lt < my_rt) {
                const int t = cta + lt * ncta;
                mbar_wait(&bars[lt], 0, err);
                float v = q8_task_row(stage_a + lt * a1_slot, nbh, xq0, xd0, lane);
                const int row = t * 4 + (lane >> 3);
                if ((lane & 7) == 0) {
                    if (P.router_bias) v = __fadd_rn(v, P.router_bias[row]);
                    P.logits[row] = v;
                }
            } else {
                const int ls = lt - my_rt;
                const int t = first_st + ls * ncta;
                mbar_wait(&bars[P.n1r + ls], 0, err);
                const uint8_t *base = stage_a + (P.n1r + ls) * a1_slot;
                const float g = q8_task_row(base, nbh, xq0, xd0, lane);
                const float u = q8_task_row(base + rt_bytes, nbh, xq0, xd0, lane);
                if ((lane & 7) == 0) P.shared_act[t * 4 + (lane >> 3)] = __fmul_rn(silu_ggml(g), u);
            }
        }
        if (P.SF > 0 && cta == ncta / 2 && warp == kWarps - 1) {
            const float d = dot_f32_warp(P.sh_gate_vec, xf, P.H, lane);
            if (lane == 0) *P.shared_gate = sigmoid_ggml(d);
        }
    }
    WD_STAMP(3);   // phase 1 done (before barrier 1)
    grid_barrier(P.sync, P.sync + 1, ncta, err);
    WD_STAMP(4);   // after barrier 1

    // ---- phase 1b: selection (warp 0) and shared activation -> Q8_0 (all threads) ------------
    if (warp == 0) {
        float *lg = misc + 512;     // logits copy [E] behind the small arrays
        for (int i = lane; i < P.E; i += 32) lg[i] = __ldcg(P.logits + i);
        __syncwarp();
        router_topk_warp(lg, P.E, P.K, P.w_scale, lane, gsum, topv, sel_ids, sel_w, nullptr);
        if (lane == 0) {
            int n = 0;
            for (int j = 0; j < P.K; ++j) {
                const int e = sel_ids[j];
                if (e >= P.e_first && e < P.e_first + P.e_count) {
                    const int slot = P.slot_of_expert[e];
                    if (slot < 0) atomicOr(err, kErrExpertMiss);
                    loc_j[n] = j;
                    loc_slot[n] = slot < 0 ? 0 : slot;
                    ++n;
                }
            }
            *loc_n = n;
            if (cta == 0) {
                for (int j = 0; j < P.K; ++j) {
                    P.ids[j] = sel_ids[j];
                    P.weights[j] = sel_w[j];
                }
            }
        }
    }
    if (P.SF > 0) {
        float *sf = misc + 512 + kMaxExperts;     // shared activation as float [SF]
        for (int i = tid; i < P.SF; i += kThreads) sf[i] = __ldcg(P.shared_act + i);
        __syncthreads();
        quantize_q8_0_cta(sf, P.SF, shq, shd);
    }
    fence_proxy_async();
    __syncthreads();
    WD_STAMP(5);   // selection done

    // ---- issue every remaining copy of this CTA: gate/up units, down tiles, shared-down tasks -
    const int n_loc = *loc_n;
    const int T2 = P.F / (32 / P.nsb_h);           // gate/up tiles per expert
    const int T3 = P.H / (32 / P.nsb_f);           // down tiles per expert
    const int n_u2 = n_loc * T2, n_u3 = n_loc * T3;
    const int n_sd = P.SF > 0 ? (P.H >> 2) : 0;    // shared-down tasks (4 rows each)
    const unsigned sd_bytes = static_cast<unsigned>(nbs) * 136u;
    const int bar2 = P.n1r + P.n1s, bar3 = bar2 + P.n2, bar_sd = bar3 + P.n3;
    const int n_t3_local = n_u3 > cta ? (n_u3 - cta + ncta - 1) / ncta : 0;   // down tiles of this CTA
    if (warp == 0) {
        for (int s = lane; cta + s * ncta < n_u2; s += 32) {
            const int u = cta + s * ncta;
            const int jl = u / T2, t = u % T2;
            const uint8_t *slot = P.pool + static_cast<size_t>(loc_slot[jl]) * P.slot_bytes;
            mbar_expect_tx(&bars[bar2 + s], 2u * kIq3TileBytes);
            bulk_load(stage_a + s * 2 * kIq3TileBytes, slot + P.gate_off + static_cast<size_t>(t) * kIq3TileBytes,
                      kIq3TileBytes, &bars[bar2 + s]);
            bulk_load(stage_a + s * 2 * kIq3TileBytes + kIq3TileBytes,
                      slot + P.up_off + static_cast<size_t>(t) * kIq3TileBytes, kIq3TileBytes, &bars[bar2 + s]);
        }
        for (int li = lane; cta + li * ncta < n_u3 + n_sd; li += 32) {
            const int v = cta + li * ncta;
            if (v < n_u3) {
                const int jl = v / T3, t = v % T3;
                const uint8_t *slot = P.pool + static_cast<size_t>(loc_slot[jl]) * P.slot_bytes;
                mbar_expect_tx(&bars[bar3 + li], kIq3TileBytes);
                bulk_load(stage_b + li * kIq3TileBytes, slot + P.down_off + static_cast<size_t>(t) * kIq3TileBytes,
                          kIq3TileBytes, &bars[bar3 + li]);
            } else {
                const int t = v - n_u3, sd = li - n_t3_local;
                mbar_expect_tx(&bars[bar_sd + sd], sd_bytes);
                bulk_load(stage_b + P.n3 * kIq3TileBytes + sd * sd_bytes,
                          P.sh_down + static_cast<size_t>(t) * sd_bytes, sd_bytes, &bars[bar_sd + sd]);
            }
        }
    }

    WD_STAMP(6);   // copies issued
    // ---- phase 2: gate + up tiles -> act ---------------------------------------------------------
    {
        const int R = 32 / P.nsb_h;
        int s = warp;
        for (int u = cta + warp * ncta; u < n_u2; u += kWarps * ncta, s += kWarps) {
            const int jl = u / T2, t = u % T2;
            mbar_wait(&bars[bar2 + s], 0, err);
            const uint8_t *tg = stage_a + s * 2 * kIq3TileBytes;
            const uint8_t *tu = tg + kIq3TileBytes;
            Iq3Regs rg, ru;
            iq3_load(tg, lane, rg);
            iq3_load(tu, lane, ru);
            const int sb = lane % P.nsb_h;
            int pg[8], pu[8];
            iq3_block_partials2(rg, ru, xk + sb * kActSbStride, lane4x2, tab, pg, pu);
            const float dx = xdk[sb];
            const float dg = half_bits_to_float(*reinterpret_cast<const uint16_t *>(tg + kIq3OffD + lane * 2));
            const float du = half_bits_to_float(*reinterpret_cast<const uint16_t *>(tu + kIq3OffD + lane * 2));
            float gr[8], ur[8];
            iq_tile_rows<8>(pg, __fmul_rn(dg, dx), P.nsb_h, lane, scr, gr);
            iq_tile_rows<8>(pu, __fmul_rn(du, dx), P.nsb_h, lane, scr, ur);
            const int nit = (R * 8 + 31) / 32;
            float *act_j = P.act + static_cast<size_t>(loc_j[jl]) * P.F;
#pragma unroll
            for (int it = 0; it < 8; ++it) {
                const int rr = it * 4 + (lane >> 3);
                if (it < nit && rr < R && (lane & 7) == 0) act_j[t * R + rr] = __fmul_rn(silu_ggml(gr[it]), ur[it]);
            }
        }
    }
    WD_STAMP(7);   // phase 2 done (before barrier 2)
    grid_barrier(P.sync, P.sync + 1, ncta, err);
    WD_STAMP(8);   // after barrier 2

    // ---- phase 3: act -> Q8_K, down tiles, shared-down rows, ordered combine ----------------------
    for (int w = warp; w < n_loc * P.nsb_f; w += kWarps) {
        const int jl = w / P.nsb_f, sb = w % P.nsb_f;
        const float *src = P.act + static_cast<size_t>(loc_j[jl]) * P.F + sb * 256 + lane * 8;
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __ldcg(src + j);
        quantize_q8_K_warp(v, lane, actk + (jl * P.nsb_f + sb) * kActSbStride, &actd[jl * P.nsb_f + sb]);
    }
    __syncthreads();
    WD_STAMP(9);   // activations quantised
    {
        const int R = 32 / P.nsb_f;                 // rows per down tile
        const int expected = n_loc + (P.SF > 0 ? R / 4 : 0);
        const float sgate = P.SF > 0 ? __ldcg(P.shared_gate) : 0.0f;
        int li = warp;
        for (int v = cta + warp * ncta; v < n_u3 + n_sd; v += kWarps * ncta, li += kWarps) {
            const bool is_tile = v < n_u3;
            const int my_s3 = li, my_sd = li - n_t3_local;
            int out_tile;
            if (is_tile) {
                const int jl = v / T3, t = v % T3;
                mbar_wait(&bars[bar3 + my_s3], 0, err);
                const uint8_t *td = stage_b + my_s3 * kIq3TileBytes;
                Iq3Regs rd;
                iq3_load(td, lane, rd);
                const int sb = lane % P.nsb_f;
                int pd[8];
                iq3_block_partials(rd, actk + (jl * P.nsb_f + sb) * kActSbStride, lane4x2, tab, pd);
                const float dd = half_bits_to_float(*reinterpret_cast<const uint16_t *>(td + kIq3OffD + lane * 2));
                float dr[8];
                iq_tile_rows<8>(pd, __fmul_rn(dd, actd[jl * P.nsb_f + sb]), P.nsb_f, lane, scr, dr);
                const int nit = (R * 8 + 31) / 32;
                float *eo = P.expert_out + static_cast<size_t>(loc_j[jl]) * P.H;
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                    const int rr = it * 4 + (lane >> 3);
                    if (it < nit && rr < R && (lane & 7) == 0) eo[t * R + rr] = dr[it];
                }
                out_tile = t;
            } else {
                const int t = v - n_u3;
                mbar_wait(&bars[bar_sd + my_sd], 0, err);
                const float d = q8_task_row(stage_b + P.n3 * kIq3TileBytes + my_sd * sd_bytes, nbs, shq, shd, lane);
                if ((lane & 7) == 0) P.shared_down[t * 4 + (lane >> 3)] = d;
                out_tile = (t * 4) / R;
            }
            // hand in this contribution; the last one of the tile combines its rows
            __threadfence();
            __syncwarp();
            unsigned old = 0;
            if (lane == 0) old = atomicAdd(&tile_cnt[out_tile], 1u);
            old = __shfl_sync(0xffffffffu, old, 0);
            if (old == static_cast<unsigned>(expected - 1)) {
                __threadfence();
                if (lane == 0) tile_cnt[out_tile] = 0;
                for (int rr = lane; rr < R; rr += 32) {
                    const int row = out_tile * R + rr;
                    float acc = 0.0f;
                    for (int jl = 0; jl < n_loc; ++jl) {
                        const int j = loc_j[jl];
                        acc = __fadd_rn(acc, __fmul_rn(__ldcg(P.expert_out + static_cast<size_t>(j) * P.H + row), sel_w[j]));
                    }
                    P.routed[row] = acc;
                    float o = acc;
                    if (P.SF > 0) o = __fadd_rn(acc, __fmul_rn(__ldcg(P.shared_down + row), sgate));
                    P.out[row] = o;
                    if (P.residual) P.residual[row] = __fadd_rn(P.residual[row], o);
                }
            }
        }
        if (expected == 0) {
            for (int row = cta * kThreads + tid; row < P.H; row += ncta * kThreads) {
                P.routed[row] = 0.0f;
                P.out[row] = 0.0f;
            }
        }
    }
    WD_STAMP(10);   // done
#undef WD_STAMP
}

}  // namespace wd
