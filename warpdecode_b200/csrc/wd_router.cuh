// Block-parallel router of the fused MoE layer kernel.
#pragma once

#include "wd_blocks.cuh"

namespace wd {

// ---------------------------------------------------------------------------------------------
// router: softmax over all experts + top-k by the whole CTA (src/qwen38_moe.cuh:711-818).
// Thread t owns experts t and t + kThreads (E <= 1024) and receives their logits in registers. Every
// float step is the reference's: running max; exp_ggml(x - max); groups of eight summed in the AVX2
// lane order; the group sums accumulated ascending into a double; p * (float)(1 / sum); k rungs of
// "largest remaining probability, ties to the lower index, NaN never, nothing above -inf gives id 0";
// weights = picked / max((float)double_sum, 2^-14), times w_scale unless it is 0 or 1.
// The rungs run in two stages with one __syncthreads between them: every warp lists its own k best
// (key, index) pairs in rung order with two redux steps per rung; warp 0 then merges the 16 sorted
// lists, one head per lane. The order (larger key, then lower index) is total, so the merged rungs are
// exactly the rungs over all experts. The lists are first cut at kShortList entries; when the merge decides a
// rung while a cut list has run out and something that list left out could have won, both stages are repeated
// with lists of k entries.
// Shared scratch: gsum[E/8], red[kWarps] (unused), cand[2][kWarps][kMaxK] u32, first[2];
// probs[E] is optional (nullptr: not stored).
// ---------------------------------------------------------------------------------------------
struct RouterScratch {
    float *probs;       // [E] or nullptr
    float *gsum;        // [E/8]
    uint32_t *cand;     // [2][kWarps][kMaxK]: keys, then indices
    float *red;         // [kWarps]
    float *first;       // [2] probability of expert 0 (what a rung reports when nothing is selectable); repeat flag
};

constexpr int kShortList = 4;    // entries per warp list in the first attempt of the rungs

// inverse of order_key for keys above kKeyNegInf
__device__ __forceinline__ float key_to_float(uint32_t key) {
    return __uint_as_float((key & 0x80000000u) ? (key ^ 0x80000000u) : ~key);
}

__device__ __forceinline__ void router_softmax_given_max(float l0, float l1, float mx, int E, const RouterScratch &S,
                                                         float &p0_out, float &p1_out,
                                                         unsigned long long *stage_stamps = nullptr, float *inv_out = nullptr);

// Softmax of the whole row (the first half of router_select_cta): thread t holds the logits of experts t and
// t + kThreads and receives their probabilities (-inf in every place when the sum is zero).
__device__ __forceinline__ void router_softmax_cta(float l0, float l1, int E, const RouterScratch &S, float &p0_out,
                                                   float &p1_out, unsigned long long *stage_stamps = nullptr) {
#define WD_RSTAMP(i)                                                       \
    if (stage_stamps != nullptr && threadIdx.x == 0) {                     \
        unsigned long long t__;                                            \
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__) : : "memory");            \
        stage_stamps[i] = t__;                                             \
    }
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int e0 = tid, e1 = tid + kThreads;
    const bool h0 = e0 < E, h1 = e1 < E;
    if (!h0) l0 = -INFINITY;
    if (!h1) l1 = -INFINITY;
    // running max through the order-preserving integer key (one redux per level instead of a shuffle tree). NaN maps
    // to key 0 and is passed over as fmaxf would; if every logit is NaN the result is a NaN, as with fmaxf.
    uint32_t mk = __reduce_max_sync(0xffffffffu, max(order_key(l0), order_key(l1)));
    if (lane == 0) S.cand[warp] = mk;
    __syncthreads();
    mk = __reduce_max_sync(0xffffffffu, lane < kWarps ? S.cand[lane] : 0u);
    const float mx = __uint_as_float((mk & 0x80000000u) ? (mk ^ 0x80000000u) : ~mk);
    router_softmax_given_max(l0, l1, mx, E, S, p0_out, p1_out, stage_stamps);
#undef WD_RSTAMP
}

// The softmax once the row maximum is known (one block-wide synchronisation inside). `inv_out`, optional: the factor
// (float)(1 / sum) every exponential was multiplied with, 0 when the sum was zero (then every probability is -inf).
__device__ __forceinline__ void router_softmax_given_max(float l0, float l1, float mx, int E, const RouterScratch &S,
                                                         float &p0_out, float &p1_out, unsigned long long *stage_stamps,
                                                         float *inv_out) {
#define WD_RSTAMP(i)                                                       \
    if (stage_stamps != nullptr && threadIdx.x == 0) {                     \
        unsigned long long t__;                                            \
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__) : : "memory");            \
        stage_stamps[i] = t__;                                             \
    }
    const int tid = threadIdx.x, lane = tid & 31;
    const int e0 = tid, e1 = tid + kThreads;
    const bool h0 = e0 < E, h1 = e1 < E;
    WD_RSTAMP(0)
    float p0 = h0 ? exp_ggml(__fsub_rn(l0, mx)) : 0.0f;
    float p1 = h1 ? exp_ggml(__fsub_rn(l1, mx)) : 0.0f;
    const float g0 = hsum8_lanes(p0), g1 = hsum8_lanes(p1);   // the reference's 8-lane tree
    if ((lane & 7) == 0) {
        if (h0) S.gsum[e0 >> 3] = g0;
        if (h1) S.gsum[e1 >> 3] = g1;
    }
    __syncthreads();
    WD_RSTAMP(1)
    {
        // The reference adds the group sums one by one, ascending, into a double. When every partial
        // sum is exactly representable the order cannot matter, and a shuffle tree gives the same bits:
        // all terms are non-negative multiples of the smallest term's last bit q, so any partial sum is
        // a multiple of q below the total; it is exact if total < 2^53 * q, i.e. if the exponent span
        // between the total and the smallest non-zero term (minus its 23 mantissa bits) stays under 53.
        // Otherwise (and for inf/nan/denormal terms) one lane replays the reference's order.
        // Every warp computes the sum for itself: cheaper than one more block-wide hand-over.
        const int ng = E >> 3;
        double part = 0.0;
        int min_exp = 0x7fffffff, bad = 0;
#pragma unroll 1
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
#pragma unroll 1
            for (int g = 0; g < ng; ++g) sum = __dadd_rn(sum, static_cast<double>(S.gsum[g]));
        }
        if (sum == 0.0) {
            p0 = p1 = -INFINITY;
            if (inv_out) *inv_out = 0.0f;
        } else {
            const float inv = __double2float_rn(__ddiv_rn(1.0, sum));
            p0 = __fmul_rn(p0, inv);
            p1 = __fmul_rn(p1, inv);
            if (inv_out) *inv_out = inv;
        }
    }
    p0_out = p0;
    p1_out = p1;
#undef WD_RSTAMP
}

// Closing step of the selection by one warp: lane j < K holds the j-th picked probability; returns its weight
// = picked / max((float) sum of the K picked, 2^-14) (times w_scale unless it is 0 or 1). The reference adds the
// picked probabilities one by one into a double; as for the softmax sum, a shuffle tree gives the same bits
// whenever every partial sum is exact, else the serial order is replayed.
__device__ __forceinline__ float router_weights_warp(float my_p, int K, float w_scale, int lane) {
    const float tp = lane < K ? my_p : 0.0f;
    const int ex = static_cast<int>((__float_as_uint(tp) >> 23) & 0xffu);
    const bool nz = tp != 0.0f;
    const int bad = __any_sync(0xffffffffu, nz && (ex == 0 || ex == 255 || tp < 0.0f));
    const int min_exp = __reduce_min_sync(0xffffffffu, nz ? ex : 0x7fffffff);
    double wsum = static_cast<double>(tp);
#pragma unroll
    for (int sft = 1; sft < 32; sft <<= 1) wsum = __dadd_rn(wsum, __shfl_xor_sync(0xffffffffu, wsum, sft));
    const int tot_exp = static_cast<int>((__double_as_longlong(wsum) >> 52) & 0x7ff) - 1023 + 127;
    if (bad || (min_exp != 0x7fffffff && tot_exp + 1 - (min_exp - 23) > 52)) {
        wsum = 0.0;
#pragma unroll 1
        for (int j = 0; j < K; ++j) wsum = __dadd_rn(wsum, static_cast<double>(__shfl_sync(0xffffffffu, my_p, j)));
    }
    const float denom = fmaxf(__double2float_rn(wsum), 6.103515625e-5f);
    float w = __fdiv_rn(my_p, denom);
    if (w_scale != 0.0f && w_scale != 1.0f) w = __fmul_rn(w, w_scale);
    return w;
}

// The k rungs over the probabilities (the second half of router_select_cta).
__device__ __forceinline__ void router_rungs_cta(float p0, float p1, int E, int K, float w_scale, const RouterScratch &S,
                                                 int *ids_out, float *w_out, unsigned long long *stage_stamps = nullptr) {
#define WD_RSTAMP(i)                                                       \
    if (stage_stamps != nullptr && threadIdx.x == 0) {                     \
        unsigned long long t__;                                            \
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__) : : "memory");            \
        stage_stamps[i] = t__;                                             \
    }
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int e0 = tid, e1 = tid + kThreads;
    const bool h0 = e0 < E, h1 = e1 < E;
    WD_RSTAMP(2)
    if (S.probs) {
        if (h0) S.probs[e0] = p0;
        if (h1) S.probs[e1] = p1;
    }
    if (tid == 0) *S.first = p0;
    // stage 1: this warp's best, in rung order. The lists are first cut at kShortList entries: ten rungs over 512
    // experts rarely take more than that from one warp, and the merge notices when it would have needed more
    // (then everything is repeated with full lists).
    const uint32_t key0 = h0 ? order_key(p0) : 0u, key1 = h1 ? order_key(p1) : 0u;
    uint32_t *ck = S.cand, *ci = S.cand + kWarps * kMaxK;
    uint32_t my_id = 0u;
    float my_p = 0.0f;
    int depth = min(K, kShortList);
#pragma unroll 1
    for (;;) {
        uint32_t k0 = key0, k1 = key1;
#pragma unroll 1
        for (int j = 0; j < depth; ++j) {
            const uint32_t m = __reduce_max_sync(0xffffffffu, max(k0, k1));
            const uint32_t cand = (k0 == m) ? static_cast<uint32_t>(e0) : ((k1 == m) ? static_cast<uint32_t>(e1) : 0xffffffffu);
            const uint32_t mi = __reduce_min_sync(0xffffffffu, cand);
            if (lane == 0) {
                ck[warp * kMaxK + j] = m;
                ci[warp * kMaxK + j] = mi;
            }
            if (m <= kKeyNegInf) {          // nothing selectable is left in this warp: the rest of its list is empty
                if (lane == 0)
#pragma unroll 1
                    for (int q = j + 1; q < depth; ++q) ck[warp * kMaxK + q] = 0u;
                break;
            }
            if (mi == static_cast<uint32_t>(e0)) k0 = 0u;
            if (mi == static_cast<uint32_t>(e1)) k1 = 0u;
        }
        __syncthreads();
        WD_RSTAMP(3)
        // stage 2: warp 0 merges the lists; lane w holds the head of warp w's list
        if (warp == 0) {
            int ptr = 0;
            bool starved = false;       // a rung was decided while this lane's (cut) list had run out
            const float p_first = *S.first;
            // key of the last entry of a list that was cut while it still had selectable entries (else 0): what
            // the warp did not list is at most this
            const uint32_t last_key = (lane < kWarps && depth < K) ? ck[lane * kMaxK + depth - 1] : 0u;
            const bool cut = last_key > kKeyNegInf;
#pragma unroll 1
            for (int j = 0; j < K; ++j) {
                const bool live = lane < kWarps && ptr < depth;
                const uint32_t hk = live ? ck[lane * kMaxK + ptr] : 0u;
                const uint32_t hi = live ? ci[lane * kMaxK + ptr] : 0xffffffffu;
                const uint32_t M = __reduce_max_sync(0xffffffffu, hk);
                uint32_t win = __reduce_min_sync(0xffffffffu, hk == M ? hi : 0xffffffffu);
                starved = starved || (cut && ptr == depth && M <= last_key);    // an unlisted entry could have won
                float p;
                if (M <= kKeyNegInf) {      // nothing selectable: the rung keeps expert 0
                    win = 0u;
                    p = p_first;
                } else {
                    p = key_to_float(M);
                    if (static_cast<uint32_t>(lane) == ((win & (kThreads - 1)) >> 5)) ++ptr;
                }
                if (lane == j) {
                    my_id = win;
                    my_p = p;
                }
            }
            const int again = __any_sync(0xffffffffu, starved);
            if (lane == 0) S.first[1] = again ? 1.0f : 0.0f;
        }
        __syncthreads();
        if (depth == K || S.first[1] == 0.0f) break;
        depth = K;
        __syncthreads();        // everyone has read the flag before the lists are rewritten
    }
    if (warp == 0) {
        if (lane == 0) { WD_RSTAMP(4) }
        const float w = router_weights_warp(my_p, K, w_scale, lane);
        if (lane < K) {
            ids_out[lane] = static_cast<int>(my_id);
            w_out[lane] = w;
        }
    }
    __syncthreads();
    WD_RSTAMP(5)
#undef WD_RSTAMP
}

__device__ __forceinline__ void router_select_cta(float l0, float l1, int E, int K, float w_scale, const RouterScratch &S,
                                                  int *ids_out, float *w_out, unsigned long long *stage_stamps = nullptr) {
    float p0, p1;
    router_softmax_cta(l0, l1, E, S, p0, p1, stage_stamps);
    router_rungs_cta(p0, p1, E, K, w_scale, S, ids_out, w_out, stage_stamps);
}

}  // namespace wd

namespace wd {

// ---------------------------------------------------------------------------------------------
// Expert ids from a threshold on the LOGITS, proven afterwards against the probabilities.
//
// The rungs of the reference pick by probability (larger first, ties to the lower index). Probabilities are a
// non-decreasing function of the logits, so the k largest logits are the k rungs unless probabilities tie or fall
// out of order at the last bit, a sum degenerates, or non-finite values are involved. The ids therefore come from
// the logits at once (the tile copies can start), and while the tiles are in flight the softmax and a proof run:
// nothing outside the picked set may beat its weakest member by PROBABILITY, and inside it the probabilities must
// fall in exactly the picked order, every one an ordinary number. A row that fails the proof (or has more than 32
// candidates above the threshold, or fewer than k groups with a finite logit) takes the exact rungs.
//
// Stages, with one __syncthreads by the caller after each of the first three:
//   a  16 group maxima of the order keys
//   b  threshold = k-th best group maximum (at least k experts reach it); candidates above it into a list
//   c  warp 0 ranks the candidates: sel_ids / sel_keys in rank order, a bit mask of the picked
//   proof (router_threshold_proof): softmax with the known maximum, the test above, the weights
// Thread t owns experts t and t + kThreads (E <= 1024), as in router_select_cta.
// ---------------------------------------------------------------------------------------------
struct ThresholdScratch {
    uint32_t *gm;        // [16]
    int *cnt;            // [1]
    uint2 *cand;         // [64] (key, expert)
    uint32_t *sel_keys;  // [kMaxK]
    uint32_t *selmask;   // [kMaxExperts / 32]
};
constexpr int kThresholdMaxCand = 64;

__device__ __forceinline__ void router_threshold_stage_a(uint32_t key0, uint32_t key1, int E, const ThresholdScratch &T) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint32_t m = max(key0, key1);
    if (E >= kThreads) {
        m = __reduce_max_sync(0xffffffffu, m);
        if (lane == 0) T.gm[warp] = m;
    } else {
        int group = 1;                          // lanes per group: the power of two that lets 16 groups cover E experts
        while (16 * group < E) group <<= 1;
#pragma unroll 1
        for (int s = 1; s < group; s <<= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, s));
        if (tid < 16 * group) {
            if ((tid % group) == 0) T.gm[tid / group] = tid < E ? m : 0u;
        }
    }
    if (tid == 0) *T.cnt = 0;
    if (tid < kMaxExperts / 32) T.selmask[tid] = 0u;
}

// Returns true when the row must take the exact rungs already (fewer than K groups hold a selectable logit).
__device__ __forceinline__ bool router_threshold_stage_b(uint32_t key0, uint32_t key1, bool h0, bool h1, int K,
                                                         const ThresholdScratch &T) {
    const int tid = threadIdx.x, lane = tid & 31;
    const uint32_t mine = T.gm[lane & 15];
    int rank = 0;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const uint32_t o = T.gm[j];
        rank += (o > mine) || (o == mine && j < (lane & 15));
    }
    const uint32_t thr = T.gm[__ffs(__ballot_sync(0xffffffffu, lane < 16 && rank == K - 1)) - 1];
    const bool c0 = h0 && key0 >= thr, c1 = h1 && key1 >= thr;
    const unsigned b0 = __ballot_sync(0xffffffffu, c0), b1 = __ballot_sync(0xffffffffu, c1);
    int base = 0;
    if (lane == 0 && (b0 | b1)) base = atom_add_shared(T.cnt, __popc(b0) + __popc(b1));
    base = __shfl_sync(0xffffffffu, base, 0);
    const unsigned lt = (1u << lane) - 1u;
    if (c0) {
        const int pos = base + __popc(b0 & lt);
        if (pos < kThresholdMaxCand) T.cand[pos] = make_uint2(key0, static_cast<uint32_t>(tid));
    }
    if (c1) {
        const int pos = base + __popc(b0) + __popc(b1 & lt);
        if (pos < kThresholdMaxCand) T.cand[pos] = make_uint2(key1, static_cast<uint32_t>(tid + kThreads));
    }
    return thr <= kKeyNegInf;
}

// Warp 0 only, when the candidate count is in [K, 32]: ranks by (larger key, then lower index), a total order.
__device__ __forceinline__ void router_threshold_rank_warp(int nc, int K, const ThresholdScratch &T, int *sel_ids, int lane) {
    const uint2 me = lane < nc ? T.cand[lane] : make_uint2(0u, 0xffffffffu);
    int rank = 0;
#pragma unroll 8
    for (int j = 0; j < nc; ++j) {          // the loads do not depend on one another
        const uint2 o = T.cand[j];
        rank += (o.x > me.x) || (o.x == me.x && o.y < me.y);
    }
    if (lane < nc && rank < K) {
        sel_ids[rank] = static_cast<int>(me.y);
        T.sel_keys[rank] = me.x;
        red_or_shared(&T.selmask[me.y >> 5], 1u << (me.y & 31u));
    }
    __syncwarp();
}

__device__ __noinline__ float exp_ggml_call(float x) { return exp_ggml(x); }

// The proof (all threads; one __syncthreads inside the softmax and one vote). `slow`: the row already failed an
// earlier stage. Returns true when sel_ids are the reference's rungs; sel_w then holds their weights. p0 / p1: this
// thread's probabilities, for router_rungs_cta when the proof fails.
__device__ __forceinline__ bool router_threshold_proof(float l0, float l1, bool h0, bool h1, int E, int K, float w_scale,
                                                       bool slow, const ThresholdScratch &T, const RouterScratch &S,
                                                       const int *sel_ids, float *sel_w, float &p0, float &p1) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t mk = __reduce_max_sync(0xffffffffu, lane < 16 ? T.gm[lane] : 0u);     // row maximum = best group maximum
    const float mx = __uint_as_float((mk & 0x80000000u) ? (mk ^ 0x80000000u) : ~mk);
    float inv = 0.0f;
    router_softmax_given_max(l0, l1, mx, E, S, p0, p1, nullptr, &inv);
    bool bad = slow;
    if (!slow) {
        // every thread forms the weakest member's probability itself, with the operations its owner used
        const float pb = __fmul_rn(exp_ggml_call(__fsub_rn(key_to_float(T.sel_keys[K - 1]), mx)), inv);
        const int eb = sel_ids[K - 1];
        const bool s0 = h0 && ((T.selmask[tid >> 5] >> (tid & 31)) & 1u);
        const bool s1 = h1 && ((T.selmask[(tid + kThreads) >> 5] >> (tid & 31)) & 1u);
        bad = (h0 && !s0 && (p0 > pb || (p0 == pb && tid < eb))) || (h1 && !s1 && (p1 > pb || (p1 == pb && tid + kThreads < eb)));
        bad = bad || !(inv > 0.0f && inv < INFINITY);
        if (warp == 0) {
            const float pj = lane < K ? __fmul_rn(exp_ggml_call(__fsub_rn(key_to_float(T.sel_keys[lane]), mx)), inv) : 0.0f;
            const int ej = lane < K ? sel_ids[lane] : 0x7fffffff;
            const float pn = __shfl_down_sync(0xffffffffu, pj, 1);
            const int en = __shfl_down_sync(0xffffffffu, ej, 1);
            const bool fine = lane >= K || (pj == pj && pj > -INFINITY && (lane == K - 1 || pj > pn || (pj == pn && ej < en)));
            // the vote first, on its own: `bad || !vote` would let the lanes whose `bad` is already set skip it
            const bool all_fine = __all_sync(0xffffffffu, fine);
            bad = bad || !all_fine;
            const float w = router_weights_warp(pj, K, w_scale, lane);
            if (lane < K) sel_w[lane] = w;
        }
    }
    return !__syncthreads_or(bad);
}

}  // namespace wd
