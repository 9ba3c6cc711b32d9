// The layer kernel for geometries known at compile time (IQ3_S experts, a Q8_0 shared expert).
//
// Same dataflow idea as moe_layer_kernel (one cooperative launch runs a range of layers; values that cross
// CTAs travel as tagged words; no grid barrier), with a shorter dependency chain per layer:
//
//   phase 0   one warp per 256-value superblock of x: waits for the residual rows, RMSNorm, Q8_0 and Q8_K
//             straight from registers (two block-wide synchronisations in all)
//   phase 1   ONE ROW PER WARP: a router row, or a gate/up row pair of the shared expert, with the 64-block
//             float chain handed from lane group to lane group (the integer work of a row runs 4-wide)
//   phase 1b  expert ids from the LOGITS: k-th best of 16 group maxima as a threshold, the few candidates above
//             it ranked by every warp for itself. The tile copies are issued from these ids at once; the
//             softmax, the weights and the proof that ranking by probability gives the same rungs run while
//             the tiles are in flight. A row where the proof fails (ties between probabilities, zero or
//             non-finite sums, more than 32 candidates) takes the exact rungs and re-issues its copies.
//   phase 2   gate and up tiles, cut into sub-block units that are spread evenly over the 16 warps; the
//             integer partials of a tile meet in shared memory (exact, so their order is free); one float
//             chain per (row, chunk-lane); act = SiLU(g) * u published
//   phase 3   ROW BANDS: a CTA owns the rows of one down tile position (32 / nsb_f output rows) for ALL selected
//             experts and for the shared expert: it gathers every expert's act (Q8_K), decodes its tiles and
//             performs the ordered weighted combine for its rows itself; the new residual rows are published
//             for the next layer. No exchange between the down products and the combine.
//
// Reference call sites this replaces: q38_moe_select_experts_f32_x (src/qwen38_moe.cuh:2323),
// q38_moe_run_batched_experts (:3312, five launches), run_qwen38_shared_expert_f32_x (:3963, nine
// launches), q38_finish_moe_f32 (:2442) and the per-layer ids D2H + stream sync (:2363-2379).
#pragma once

#include "wd_moe_kernel.cuh"

namespace wd {

template <int H_, int F_, int E_, int K_, int SF_>
struct FastGeo {
    static constexpr int H = H_, F = F_, E = E_, K = K_, SF = SF_;
    static constexpr int NSB_H = H / 256, NSB_F = F / 256;      // superblocks per gate/up row and per down row
    static constexpr int NBH = H / 32, NBS = SF / 32;           // Q8_0 blocks per row over H and over SF columns
    static constexpr int R2 = 32 / NSB_H, R3 = 32 / NSB_F;      // rows per gate/up tile and per down tile (= band)
    static constexpr int T2 = F / R2;                           // tile pairs (gate + up) per expert
    static constexpr int T3 = H / R3;                           // down tiles per expert = row bands
    static constexpr int ROW_H = NBH * 34, ROW_S = NBS * 34;    // bytes of a Q8_0 row
    static constexpr int EPT = (E + kThreads - 1) / kThreads;   // experts per thread of the selection
    static constexpr int GROUP = E >= 512 ? 32 : (E / 16 > 0 ? E / 16 : 1);   // lanes per group maximum: 16 groups
    static_assert(H % 256 == 0 && (NSB_H & (NSB_H - 1)) == 0 && NSB_H >= 1 && NSB_H <= 16, "hidden");
    static_assert(F % 256 == 0 && (NSB_F & (NSB_F - 1)) == 0 && NSB_F >= 1 && NSB_F <= 8, "expert_ffn");
    static_assert(SF % 256 == 0 && SF >= 256 && SF <= 2048, "shared_ffn");
    static_assert(E % 32 == 0 && E >= 32 && E <= kMaxExperts && (E & (E - 1)) == 0, "n_experts");
    static_assert(K >= 1 && K <= kMaxK && K <= 16, "top_k");
};

constexpr int kFastAccStride = 288;     // ints per tile in the shared accumulator: [lane * 9 + chunk-lane]
constexpr int kFastMaxCand = 64;
// mbarriers: 0 router rows, 1 shared gate/up rows, 2 shared gate vector, 3 slot table, 4 shared down rows,
// 8.. one per gate/up tile, then one per down tile
constexpr int kFbRows = 0, kFbShared = 1, kFbGateVec = 2, kFbSlots = 3, kFbSharedDown = 4, kFbTiles = 8;

struct FastParams {
    int e_first, e_count;        // owned expert range
    float w_scale, eps;
    const LayerDev *layers;      // router / shared tensors in the one-row layout (repack_q8_0_rows_kernel)
    int layer_begin, layer_end;
    int stamp_layer, select_only;
    const uint8_t *pool;
    unsigned long long slot_bytes;
    unsigned gate_off, up_off, down_off;
    const uint16_t *grid_packed;
    const float *x;              // [H] (used when residual == nullptr)
    float *residual;             // nullable: x = RMSNorm(residual) * norm_w, residual += out
    float *out;                  // [H]
    // Exchange between CTAs: a producer PUSHES its values (tagged words, in whole 128-byte lines) into every mailbox,
    // and a consumer polls only the mailbox of its own group of `mbox_group` neighbouring CTAs. One copy that all
    // 148 SMs poll while it is being written comes back microseconds late (the line is hot in L2); one copy per CTA
    // costs 148 stores per line and producer. A mailbox per 16 CTAs measured best. Mailbox d (words): [2][E] logits | [2][SF] shared act | [2][16] shared gate |
    // [2][H] residual | [2][K][F] act values (row jl = the jl-th owned selected expert).
    tagged_t *xbuf;
    unsigned long long xstride;  // words per mailbox
    int mbox_group;              // CTAs per mailbox: a mailbox is shared by this many neighbouring CTAs (they all poll it)
    tagged_t *t_expert_out;      // [2][K][H]  rows that expert-parallel peers push (unused on one GPU)
    tagged_t *t_progress;        // [grid]   tag of the last layer each CTA has left
    tagged_t *peer_expert_out[8];
    int n_peers;
    tagged_t *t_peer_left;       // [8] see MoeParams
    tagged_t *peer_left_out[8];
    int peer_rank[8];
    int *ids;                    // [K] plain copies for inspection (CTA 0)
    float *weights;              // [K]
    float *routed;               // [H]
    float *expert_out;           // [K][H] plain: every selected expert's down rows (inspection)
    float *shared_down;          // [H] plain: the shared expert's down rows
    unsigned long long *stamps;
    unsigned *host_status;
    unsigned *sync;              // as MoeParams::sync
    unsigned *fallbacks;         // nullable: counts layers that took the exact rungs (CTA 0)
    // shared memory plan (byte offsets, 128-byte aligned)
    unsigned off_tab, off_xq0, off_xd0, off_xk, off_xdk, off_xf, off_actk, off_actd, off_shq, off_shd, off_misc, off_bar,
        off_slots, off_acc, off_rowbuf, off_rows3, off_push, off_a, off_b, off_c;
    unsigned n_sp;               // shared row pairs per CTA (most)
    unsigned act_pad;            // words per CTA in t_act: p2_max * rows per tile, rounded up to whole 128-byte lines
    unsigned p2_max;             // gate/up tile pairs per CTA (most)
    unsigned b3_max;             // row bands per CTA (most)
};

// float offsets inside `misc`
constexpr int kFmGsum = 0, kFmCand = 128, kFmFirst = 640, kFmRed = 648, kFmGm = 664, kFmCnt = 680, kFmCk = 688,
              kFmCi = 752, kFmIds = 816, kFmW = 832, kFmSelP = 848, kFmFlag = 864, kFmLocJ = 872, kFmLocSlot = 888,
              kFmLocN = 904, kFmSelMask = 912, kFmShRow = 944, kFmEnd = 1024;

// One Q8_0 row of NB blocks against the Q8_0 activation by one warp. Lane = (chunk-lane c = lane & 7, group
// q = lane >> 3); group q owns blocks [q * NB/Q, (q+1) * NB/Q): it forms their integer dots and scale products
// on its own, then the float chain fmaf(d_w * d_x, dot, acc) runs over the blocks in ascending order, handed from
// group to group. The same operations in the same order as q8_task_row. Row layout: quants [g][c][16 B] (word i
// = values 4c..4c+3 of block 4g+i), then NB f16 scales.
template <int NB>
__device__ __noinline__ float q8_row_warp(const uint8_t *row, const uint8_t *xq, const float *xd, int lane) {
    constexpr int Q = NB / 4 >= 4 ? 4 : NB / 4;       // lane groups at work
    constexpr int GPL = NB / 4 / Q;                   // 4-block groups per lane
    static_assert(NB % 8 == 0 && GPL * Q * 4 == NB, "blocks per row");
    const int c = lane & 7, q = lane >> 3;
    float sc[GPL * 4], fd[GPL * 4];
    if (q < Q) {
#pragma unroll
        for (int i = 0; i < GPL; ++i) {
            const int g = q * GPL + i;
            const uint4 w = *reinterpret_cast<const uint4 *>(row + (g * 8 + c) * 16);
            const uint4 a = *reinterpret_cast<const uint4 *>(xq + (g * 8 + c) * 16);
            const uint2 dw = *reinterpret_cast<const uint2 *>(row + NB * 32 + g * 8);
            const float4 dx = *reinterpret_cast<const float4 *>(xd + g * 4);
            sc[4 * i + 0] = __fmul_rn(half_bits_to_float(dw.x & 0xffffu), dx.x);
            sc[4 * i + 1] = __fmul_rn(half_bits_to_float(dw.x >> 16), dx.y);
            sc[4 * i + 2] = __fmul_rn(half_bits_to_float(dw.y & 0xffffu), dx.z);
            sc[4 * i + 3] = __fmul_rn(half_bits_to_float(dw.y >> 16), dx.w);
            fd[4 * i + 0] = static_cast<float>(dp4a_s8(w.x, a.x, 0));
            fd[4 * i + 1] = static_cast<float>(dp4a_s8(w.y, a.y, 0));
            fd[4 * i + 2] = static_cast<float>(dp4a_s8(w.z, a.z, 0));
            fd[4 * i + 3] = static_cast<float>(dp4a_s8(w.w, a.w, 0));
        }
    }
    float acc = 0.0f;
#pragma unroll
    for (int s = 0; s < Q; ++s) {
        if (s > 0) acc = __shfl_up_sync(0xffffffffu, acc, 8);
        if (q == s) {
#pragma unroll
            for (int i = 0; i < GPL * 4; ++i) acc = __fmaf_rn(sc[i], fd[i], acc);
        }
    }
    // the last group holds the eight chunk-lane sums
    acc = hsum8_lanes(acc);
    return __shfl_sync(0xffffffffu, acc, (Q - 1) * 8);
}

// Integer partials of this warp's share [u0, u1) of a list of IQ3_S tiles, in units of one sub-block (of all 32
// blocks of a tile), added into the shared accumulator (ints [list index][lane * 9 + c]). List index d lives in staging
// slot s = d (nl == 0: gate/up tiles, one activation for all) or s = (d / nl) * K + d % nl (down tiles of nl experts:
// band, expert; the expert's activation is act + (d % nl) * act_stride). The one copy of the decoder in the kernel.
template <int K>
__device__ __noinline__ void fast_tile_units(int u0, int u1, const uint8_t *tiles, uint64_t *bars, int *acc, const uint8_t *act,
                                             int act_stride, int nl, int lane, const uint8_t *tab, uint32_t tpar, unsigned *err) {
    const uint32_t lane4x2 = static_cast<uint32_t>(lane * 4) * 0x0101u;
    int cur = -1;
    int p[8];
    Iq3Head h;
    const uint8_t *tile = tiles;
    const uint4 *av = reinterpret_cast<const uint4 *>(act);
#ifndef WD_FAST_PAIRED_UNITS
#define WD_FAST_PAIRED_UNITS 1
#endif
#pragma unroll 1
    for (int u = u0; u < u1; ++u) {
        const int d = u >> 3, i = u & 7;
        if (d != cur) {
            if (cur >= 0) {
                int *dst = acc + cur * kFastAccStride + lane * 9;
#pragma unroll
                for (int c = 0; c < 8; ++c) red_add_shared(dst + c, p[c]);
            }
            cur = d;
            int s = d, jl = 0;
            if (nl > 0) {
                const int bi = d / nl;
                jl = d - bi * nl;
                s = bi * K + jl;
            }
            tile = tiles + s * kIq3TileBytes;
            mbar_wait(&bars[s], tpar, err);
            iq3_head(tile, lane, h);
            av = reinterpret_cast<const uint4 *>(act + jl * act_stride);
#pragma unroll
            for (int c = 0; c < 8; ++c) p[c] = 0;
        }
        if (WD_FAST_PAIRED_UNITS && i < 7 && u + 1 < u1) {
            // two sub-blocks of the same tile at once: sixteen independent chunk chains in flight
            iq3_subblock(tile, h, i, lane, av[2 * i], av[2 * i + 1], lane4x2, tab, p);
            iq3_subblock(tile, h, i + 1, lane, av[2 * i + 2], av[2 * i + 3], lane4x2, tab, p);
            ++u;
        } else {
            iq3_subblock(tile, h, i, lane, av[2 * i], av[2 * i + 1], lane4x2, tab, p);
        }
    }
    if (cur >= 0) {
        int *dst = acc + cur * kFastAccStride + lane * 9;
#pragma unroll
        for (int c = 0; c < 8; ++c) red_add_shared(dst + c, p[c]);
    }
}

// Q8_K of 256 values held eight per lane (src/qwen38_cpu_moe.cuh:239): quants to q_out_sb, scale to *d_out.
__device__ __noinline__ void q8k_from_regs(const float v[8], int lane, uint8_t *q_out_sb, float *d_out) {
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

__device__ __noinline__ float silu_mul(float g, float u) { return __fmul_rn(silu_ggml(g), u); }

// out-of-line copies of the two halves of the router (the second one is the rare, exact path)
__device__ __noinline__ void fast_softmax(float l0, float l1, float mx, int E, const RouterScratch &S, float &p0, float &p1,
                                          float *inv) {
    router_softmax_given_max(l0, l1, mx, E, S, p0, p1, nullptr, inv);
}
__device__ __noinline__ float exp_noinline(float x) { return exp_ggml(x); }
__device__ __noinline__ void fast_rungs(float p0, float p1, int E, int K, float w_scale, const RouterScratch &S, int *ids,
                                        float *w) {
    router_rungs_cta(p0, p1, E, K, w_scale, S, ids, w);
}

// Float side of a list of tiles: one chain per (tile, row, chunk-lane) over the NSB superblocks of the row,
// fmaf(d_w * d_x, (float) partial, acc) ascending, then ggml's 8-lane tree (src/qwen38_cpu_moe.cuh:337-375).
// Chains are spread over the whole CTA. List index d -> staging slot and expert as in fast_tile_units; the
// activation scales of d are dx + (d % nl) * NSB (nl == 0: dx). Returns this thread's chains through `emit`.
// The chains of list indices [d0, d1) are spread over `nthr` threads (a whole number of warps), this one being `t`.
template <int NSB, int K, class Emit>
__device__ __forceinline__ void fast_float_stage(int d0, int d1, const uint8_t *tiles, const int *acc, const float *dx, int nl,
                                                 int t, int nthr, Emit emit) {
    constexpr int R = 32 / NSB;
#pragma unroll 1
    for (int ch = t; ch < (((d1 - d0) * R * 8 + 31) & ~31); ch += nthr) {
        const int d = d0 + ch / (R * 8), rr = (ch >> 3) % R, c = ch & 7;
        const bool live = d < d1;
        float a = 0.0f;
        int bi = 0, jl = 0;
        if (live) {
            int s = d;
            if (nl > 0) {
                bi = d / nl;
                jl = d - bi * nl;
                s = bi * K + jl;
            }
            const uint8_t *tile = tiles + s * kIq3TileBytes;
            const float *dxs = dx + jl * NSB;
            const int *src = acc + d * kFastAccStride;
#pragma unroll
            for (int sb = 0; sb < NSB; ++sb) {
                const int blk = rr * NSB + sb;
                const float dw = half_bits_to_float(*reinterpret_cast<const uint16_t *>(tile + kIq3OffD + blk * 2));
                a = __fmaf_rn(__fmul_rn(dw, dxs[sb]), static_cast<float>(src[blk * 9 + c]), a);
            }
        }
        a = hsum8_lanes(a);
        if (live && c == 0) emit(d, bi, jl, rr, a);
    }
}

// Pushes the n tagged words at `src` (shared memory) to word offset `off` of the mailboxes of CTAs [0, n_dest), the
// destinations spread over the warps of the CTA, a line (16 words) per store instruction.
__device__ __forceinline__ void push_words(const tagged_t *src, int n, tagged_t *xbuf, unsigned long long xstride, size_t off,
                                           int n_dest, int warp, int lane) {
#pragma unroll 1
    for (int d = warp; d < n_dest; d += kWarps) {
        tagged_t *dst = xbuf + static_cast<size_t>(d) * xstride + off;
#pragma unroll 1
        for (int i = lane; i < n; i += 32)
            asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(dst + i), "l"(src[i]) : "memory");
    }
}

extern __shared__ __align__(128) uint8_t wd_fast_smem[];

template <class G>
__global__ void __launch_bounds__(kThreads, 1) moe_fast_kernel(const __grid_constant__ FastParams P) {
    constexpr int H = G::H, F = G::F, E = G::E, K = G::K, SF = G::SF;
    constexpr int NSB_H = G::NSB_H, NSB_F = G::NSB_F, R2 = G::R2, R3 = G::R3, T2 = G::T2, T3 = G::T3;
    uint8_t *sm = wd_fast_smem;
    uint8_t *tab = sm + P.off_tab;
    uint8_t *xq0 = sm + P.off_xq0;
    float *xd0 = reinterpret_cast<float *>(sm + P.off_xd0);
    uint8_t *xk = sm + P.off_xk;
    float *xdk = reinterpret_cast<float *>(sm + P.off_xdk);
    float *xf = reinterpret_cast<float *>(sm + P.off_xf);
    uint8_t *actk = sm + P.off_actk;
    float *actd = reinterpret_cast<float *>(sm + P.off_actd);
    uint8_t *shq = sm + P.off_shq;
    float *shd = reinterpret_cast<float *>(sm + P.off_shd);
    float *misc = reinterpret_cast<float *>(sm + P.off_misc);
    uint64_t *bars = reinterpret_cast<uint64_t *>(sm + P.off_bar);
    int *slot_tab = reinterpret_cast<int *>(sm + P.off_slots);
    int *acc = reinterpret_cast<int *>(sm + P.off_acc);
    float *rowbuf = reinterpret_cast<float *>(sm + P.off_rowbuf);     // [gate/up tile][R2]
    float *rows3 = reinterpret_cast<float *>(sm + P.off_rows3);       // [band][K][R3] down rows, then [band][R3] old residual
    uint8_t *reg_a = sm + P.off_a;       // phase-1 rows + gate vector, then gate/up tiles
    uint8_t *reg_b = sm + P.off_b;       // down tiles
    uint8_t *reg_c = sm + P.off_c;       // shared-expert down rows of this CTA's bands
    unsigned *err = P.sync + 2;
    uint32_t epoch;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(epoch) : "l"(P.sync + 8) : "memory");

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cta = blockIdx.x, ncta = gridDim.x;

    uint32_t *gm = reinterpret_cast<uint32_t *>(misc + kFmGm);
    int *cnt = reinterpret_cast<int *>(misc + kFmCnt);
    uint2 *cand = reinterpret_cast<uint2 *>(misc + kFmCk);         // candidates above the threshold: (key, expert)
    int *sel_ids = reinterpret_cast<int *>(misc + kFmIds);
    float *sel_w = misc + kFmW;
    uint32_t *sel_keys = reinterpret_cast<uint32_t *>(misc + kFmSelP);   // order keys of the picked logits, rank order
    int *loc_j = reinterpret_cast<int *>(misc + kFmLocJ), *loc_slot = reinterpret_cast<int *>(misc + kFmLocSlot);
    int *loc_n = reinterpret_cast<int *>(misc + kFmLocN);
    uint32_t *selmask = reinterpret_cast<uint32_t *>(misc + kFmSelMask);
    float *shrow = misc + kFmShRow;                                 // shared-expert down rows of this CTA's bands
    tagged_t *pushbuf = reinterpret_cast<tagged_t *>(sm + P.off_push);   // tagged words on their way to the mailboxes

    // this CTA's fixed shares
    // Router rows in runs of 16 on the first E / 16 CTAs (one row per warp; a CTA's 16 logits are one 128-byte line of
    // the exchange buffer, written by nobody else); the shared expert's gate/up row pairs in contiguous runs on the
    // other CTAs. Words that many CTAs poll while many others write into the same line come back late.
    constexpr int NR = E / 16;
    const int NP = ncta - NR;
    const bool router_cta = cta < NR;
    const int my_rr = router_cta ? 16 : 0, rr0 = 16 * cta;
    const int sp0 = router_cta ? 0 : (cta - NR) * SF / NP;
    const int my_sp = router_cta ? 0 : (cta - NR + 1) * SF / NP - sp0;
    const int my_b3 = cta < T3 ? (T3 - cta + ncta - 1) / ncta : 0;                       // row bands cta, cta + ncta, ..
    const int gcta = ncta - 1;                                                           // computes the shared gate scalar
    const unsigned a_gv = max(16u, 2u * P.n_sp) * G::ROW_H;                               // gate vector inside region A

    // Profiling stamps are SM cycle counts (cheap to read; a global-timer read takes long enough to disturb what it
    // measures). Slots 30 and 31 hold the global timer and the cycle count at the top of the stamped layer, slot 29 the
    // global timer at its end, so that the host can put all CTAs on one time axis.
#define WD_DSTAMP(i, cond)                                                                     \
    if (P.stamps != nullptr && layer == P.stamp_layer && (cond)) {                             \
        long long c__;                                                                         \
        asm volatile("mov.u64 %0, %%clock64;" : "=l"(c__) : : "memory");                       \
        P.stamps[cta * kStampStride + (i)] = static_cast<unsigned long long>(c__);             \
    }
#define WD_STAMP(i) WD_DSTAMP(i, tid == 0)
#define WD_GSTAMP(i)                                                                           \
    if (P.stamps != nullptr && layer == P.stamp_layer && tid == 0) {                           \
        unsigned long long t__;                                                                \
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__) : : "memory");                   \
        P.stamps[cta * kStampStride + (i)] = t__;                                              \
    }
    if (tid < kMaxBars) {
        mbar_init(&bars[tid], 1);
        mbar_fence_init();
    }
    if (cta == 0 && tid == 0) P.sync[5] = smem_u32(bars);      // so that a copy timeout can be reported by barrier index
    build_grid_table(tab, P.grid_packed);
    __syncthreads();

    // copies of one layer's phase-1 weights into region A, and of its slot table (one warp): each CTA's rows are
    // contiguous in the one-row layout, so a run of rows is one copy
    auto issue_phase1 = [&](const LayerDev &L) {
        if (lane == 0) {
            mbar_expect_tx(&bars[kFbRows], static_cast<uint32_t>(my_rr) * G::ROW_H);
            mbar_expect_tx(&bars[kFbShared], static_cast<uint32_t>(my_sp) * 2u * G::ROW_H);
            mbar_expect_tx(&bars[kFbSlots], E * 4u);
            if (cta == gcta) mbar_expect_tx(&bars[kFbGateVec], H * 4u);
            else mbar_arrive(&bars[kFbGateVec]);
        }
        __syncwarp();
        if (lane == 0 && my_rr > 0)
            bulk_load(reg_a, L.router_w + static_cast<size_t>(rr0) * G::ROW_H, static_cast<uint32_t>(my_rr) * G::ROW_H, &bars[kFbRows]);
        if (lane == 1 && my_sp > 0)
            bulk_load(reg_a, L.sh_gate + static_cast<size_t>(sp0) * G::ROW_H, static_cast<uint32_t>(my_sp) * G::ROW_H, &bars[kFbShared]);
        if (lane == 2 && my_sp > 0)
            bulk_load(reg_a + P.n_sp * G::ROW_H, L.sh_up + static_cast<size_t>(sp0) * G::ROW_H, static_cast<uint32_t>(my_sp) * G::ROW_H,
                      &bars[kFbShared]);
        if (lane == 3) bulk_load(slot_tab, L.slot_of_expert, E * 4u, &bars[kFbSlots]);
        if (lane == 4 && cta == gcta) bulk_load(reg_a + a_gv, L.sh_gate_vec, H * 4u, &bars[kFbGateVec]);
    };
    // the shared expert's down rows of this CTA's bands into region C (its own buffer: requested at the top of the
    // layer that uses them, when the previous layer is done with it)
    auto issue_shared_down = [&](const LayerDev &L) {
        if (lane == 0) {
            if (P.select_only) mbar_arrive(&bars[kFbSharedDown]);
            else mbar_expect_tx(&bars[kFbSharedDown], static_cast<uint32_t>(my_b3) * R3 * G::ROW_S);
        }
        __syncwarp();
        if (lane < my_b3 && !P.select_only)
            bulk_load(reg_c + lane * R3 * G::ROW_S, L.sh_down + static_cast<size_t>(cta + lane * ncta) * R3 * G::ROW_S,
                      R3 * G::ROW_S, &bars[kFbSharedDown]);
    };

    uint32_t tflip = 0;         // flips when a layer issued its tile copies twice (the exact rungs disagreed)
#pragma unroll 1
    for (int layer = P.layer_begin; layer < P.layer_end; ++layer) {
    const LayerDev L = P.layers[layer];
    const uint32_t mpar = static_cast<uint32_t>(layer - P.layer_begin) & 1u;      // mbarriers complete once per layer
    const uint32_t tag = epoch + static_cast<uint32_t>(layer - P.layer_begin) + 1u;
    const uint32_t par = tag & 1u;                                                // halves of the exchange buffers
        const bool first = layer == P.layer_begin;
    // word offsets inside a mailbox (this layer's halves), and this CTA's own mailbox
    const size_t o_logits = par * E, o_shact = 2 * E + par * SF, o_shgate = 2 * E + 2 * SF + par * 16,
                 o_res = 2 * E + 2 * SF + 32 + par * H, o_res_prev = 2 * E + 2 * SF + 32 + (par ^ 1u) * H,
                 o_act = 2 * E + 2 * SF + 32 + 2 * H + static_cast<size_t>(par) * K * F;
    tagged_t *mbox = P.xbuf + static_cast<size_t>(cta / P.mbox_group) * P.xstride;
    const int n_band_ctas = min(T3, ncta);          // the CTAs that own row bands (the first ones)
    const int n_mbox = (ncta + P.mbox_group - 1) / P.mbox_group;                 // mailboxes in all
    const int n_band_mbox = (n_band_ctas + P.mbox_group - 1) / P.mbox_group;     // mailboxes that band CTAs read
    tagged_t *t_eo = P.t_expert_out + static_cast<size_t>(par) * K * H;
    WD_GSTAMP(30);
    WD_DSTAMP(31, tid == 0);
    WD_STAMP(0);
    if (P.stamps != nullptr && tid == 0 && layer == P.stamp_layer + 1) {
        long long c__;
        asm volatile("mov.u64 %0, %%clock64;" : "=l"(c__) : : "memory");
        P.stamps[cta * kStampStride + 14] = static_cast<unsigned long long>(c__);
    }
    // (No proxy fence anywhere in this kernel: a buffer that receives a bulk copy has only ever been READ by ordinary
    // loads since its last copy, and those reads are complete before the block-wide synchronisation that precedes
    // the new copy.)
    if (warp == kWarps - 1) {
        if (first) issue_phase1(L);         // later layers' copies were requested by the layer before
        issue_shared_down(L);
    }

    // ---- phase 0: x (optionally RMSNorm(residual) * w) -> Q8_0 and Q8_K, one warp per superblock ------------------
    {
        float v[8];
        const bool mine = warp < NSB_H;
        const int e0 = warp * 256 + lane * 8;
        float nw[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) nw[i] = (mine && L.norm_w != nullptr) ? L.norm_w[e0 + i] : 1.0f;
        if (P.residual != nullptr) {
            if (first) {
                if (mine) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) v[i] = P.residual[e0 + i];
                }
            } else {
                // The previous layer's combine publishes the residual in runs of one 128-byte line per row band, each
                // written by one CTA. Words that are there are not read again. No check against CTAs that lag two
                // layers behind is needed: every CTA publishes logits or shared activations in phase 1 of every layer,
                // and a layer cannot end before all of those are read, so nobody is ever more than one layer ahead
                // of the slowest CTA.
                const tagged_t *src = mbox + o_res_prev + e0;
                tagged_t w[8] = {};
                unsigned long long t0 = 0ull;
                for (unsigned it = 0;; ++it) {
                    unsigned bad = 0;
                    if (mine) {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            if (it == 0 || tag_behind(w[i], tag - 1u)) w[i] = ld_tagged(src + i);
#pragma unroll
                        for (int i = 0; i < 8; ++i) bad |= tag_behind(w[i], tag - 1u);
                    }
                    if (!bad) break;
                    if (wait_expired(it, t0, err)) break;
                }
                unsigned over = 0;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    over |= mine & tag_ahead(w[i], tag - 1u);
                    v[i] = __uint_as_float(static_cast<uint32_t>(w[i]));
                }
                report_overrun(over, err);
            }
            // sum of squares: a perfect binary tree over consecutive elements, in double
            double sq[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) sq[i] = mine ? __dmul_rn(static_cast<double>(v[i]), static_cast<double>(v[i])) : 0.0;
#pragma unroll
            for (int w = 1; w < 8; w <<= 1)
#pragma unroll
                for (int i = 0; i + w < 8; i += 2 * w) sq[i] = __dadd_rn(sq[i], sq[i + w]);
            double ss = sq[0];
#pragma unroll
            for (int s = 1; s < 32; s <<= 1) ss = __dadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, s));
            double *redd = reinterpret_cast<double *>(misc + kFmGsum);
            if (lane == 0 && mine) redd[warp] = ss;
            __syncthreads();
            // every residual row of the previous layer is here: every CTA of this rank has finished reading that
            // layer's expert rows (a combine publishes its rows after it has read them)
            if (cta == 0 && !first && tid < P.n_peers) st_tagged_sys_release(P.peer_left_out[tid], 0.0f, tag - 1u);
            if (mine) {
                double tot[NSB_H];
#pragma unroll
                for (int i = 0; i < NSB_H; ++i) tot[i] = redd[i];
#pragma unroll
                for (int w = 1; w < NSB_H; w <<= 1)
#pragma unroll
                    for (int i = 0; i + w < NSB_H; i += 2 * w) tot[i] = __dadd_rn(tot[i], tot[i + w]);
                const float scale = __double2float_rn(__ddiv_rn(
                    1.0, __dsqrt_rn(__dadd_rn(__dmul_rn(tot[0], 1.0 / static_cast<double>(H)), static_cast<double>(P.eps)))));
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    v[i] = __fmul_rn(v[i], scale);
                    if (L.norm_w != nullptr) v[i] = __fmul_rn(v[i], nw[i]);
                }
            }
        } else {
            if (layer >= P.layer_begin + 2 && tid < ncta) wait_tag_reached(P.t_progress + tid, tag - 2u, err);
            if (mine) {
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = P.x[e0 + i];
            }
            if (P.n_peers > 0 && cta == 0 && layer >= P.layer_begin + 2) {
                __syncthreads();
                if (tid < P.n_peers) st_tagged_sys_release(P.peer_left_out[tid], 0.0f, tag - 2u);
            }
        }
        if (mine) {
            // Q8_0 (src/qwen38_cpu_moe.cuh:220): a block is four lanes
            float a0 = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) a0 = fmaxf(a0, fabsf(v[i]));
            a0 = fmaxf(a0, __shfl_xor_sync(0xffffffffu, a0, 1));
            a0 = fmaxf(a0, __shfl_xor_sync(0xffffffffu, a0, 2));
            const int b = warp * 8 + (lane >> 2), c0 = (lane & 3) * 2;
            uint32_t w0 = 0, w1 = 0;
            if (a0 != 0.0f) {
                const float inv = __fdiv_rn(127.0f, a0);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    int q = __float2int_rn(__fmul_rn(v[i], inv));
                    q = max(-128, min(127, q));
                    if (i < 4) w0 |= static_cast<uint32_t>(q & 0xff) << (8 * i);
                    else w1 |= static_cast<uint32_t>(q & 0xff) << (8 * (i - 4));
                }
            }
            uint8_t *qdst = xq0 + ((b >> 2) * 8 + c0) * 16 + (b & 3) * 4;
            *reinterpret_cast<uint32_t *>(qdst) = w0;
            *reinterpret_cast<uint32_t *>(qdst + 16) = w1;
            if ((lane & 3) == 0) xd0[b] = __half2float(__float2half_rn(__fdiv_rn(a0, 127.0f)));
            // Q8_K: the warp's 256 values
            q8k_from_regs(v, lane, xk + warp * kActSbStride, &xdk[warp]);
            if (cta == gcta) {
                *reinterpret_cast<float4 *>(xf + e0) = make_float4(v[0], v[1], v[2], v[3]);
                *reinterpret_cast<float4 *>(xf + e0 + 4) = make_float4(v[4], v[5], v[6], v[7]);
            }
        }
        __syncthreads();
    }
    WD_STAMP(1);
    WD_DSTAMP(27, tid == kThreads - 1);

    // ---- phase 1: one row (or shared row pair) per warp -------------------------------------------------------------
    {
        const int n_tasks = router_cta ? my_rr : 2 * my_sp;     // a pair CTA: gate rows [0, my_sp), then the up rows
        float *rowres = shrow;                                   // row results of a pair CTA (free until phase 3)
#pragma unroll 1
        for (int t = warp; t < n_tasks; t += kWarps) {
            if (router_cta) {
                const int row = rr0 + t;
                const float bias = L.router_bias ? L.router_bias[row] : 0.0f;      // fetched before the wait
                mbar_wait(&bars[kFbRows], mpar, err);
                float l = q8_row_warp<G::NBH>(reg_a + t * G::ROW_H, xq0, xd0, lane);
                if (lane == 0) {
                    if (L.router_bias) l = __fadd_rn(l, bias);
                    pushbuf[t] = make_tagged(l, tag);
                }
            } else {
                mbar_wait(&bars[kFbShared], mpar, err);
                const int r = t < my_sp ? t : static_cast<int>(P.n_sp) + t - my_sp;
                const float v = q8_row_warp<G::NBH>(reg_a + r * G::ROW_H, xq0, xd0, lane);
                if (lane == 0) rowres[t] = v;
            }
        }
        if (cta == gcta && warp == kWarps - 1) {
            mbar_wait(&bars[kFbGateVec], mpar, err);
            const float d = dot_f32_warp(reinterpret_cast<const float *>(reg_a + a_gv), xf, H, lane);
            // the gate scalar goes to the CTAs that combine: one word each
            const tagged_t w = make_tagged(sigmoid_ggml(d), tag);
#pragma unroll 1
            for (int dd = lane; dd < n_band_mbox; dd += 32)
                asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(P.xbuf + static_cast<size_t>(dd) * P.xstride + o_shgate), "l"(w)
                             : "memory");
        }
        __syncthreads();
        if (router_cta) {
            // a router CTA's 16 logits are one line of every mailbox
            push_words(pushbuf, my_rr, P.xbuf, P.xstride, o_logits + rr0, n_mbox, warp, lane);
        } else {
            // a pair CTA's shared activations: every warp forms them itself (lane = pair) and carries them to its share
            // of the band CTAs' mailboxes
            tagged_t w = 0ull;
            if (lane < my_sp) w = make_tagged(silu_mul(rowres[lane], rowres[my_sp + lane]), tag);
#pragma unroll 1
            for (int d = warp; d < n_band_mbox; d += kWarps)
                if (lane < my_sp)
                    asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(P.xbuf + static_cast<size_t>(d) * P.xstride + o_shact + sp0 + lane),
                                 "l"(w)
                                 : "memory");
        }
    }
    WD_STAMP(2);

    // ---- phase 1b: logits -> ids (threshold on the logits), tile copies issued from them ---------------------------
    float lg[2] = {-INFINITY, -INFINITY};
    {
        constexpr int EPT = G::EPT;
        tagged_t w[2] = {};
        unsigned long long t0 = 0ull;
        const bool h0 = tid < E, h1 = EPT > 1 && tid + kThreads < E;
        for (unsigned it = 0;; ++it) {
            unsigned bad = 0;
            if (h0) {
                w[0] = ld_tagged(mbox + o_logits + tid);
                bad |= tag_behind(w[0], tag);
            }
            if (h1) {
                w[1] = ld_tagged(mbox + o_logits + tid + kThreads);
                bad |= tag_behind(w[1], tag);
            }
            if (!bad) break;
            if (wait_expired(it, t0, err)) break;
        }
        report_overrun((h0 & tag_ahead(w[0], tag)) | (h1 & tag_ahead(w[1], tag)), err);
        if (h0) lg[0] = __uint_as_float(static_cast<uint32_t>(w[0]));
        if (h1) lg[1] = __uint_as_float(static_cast<uint32_t>(w[1]));
    }
    WD_STAMP(3);
    WD_DSTAMP(16, tid == kThreads - 1);
    WD_DSTAMP(21, tid == 4 * 32);
    const bool h0 = tid < E, h1 = G::EPT > 1 && tid + kThreads < E;
    const uint32_t key0 = h0 ? order_key(lg[0]) : 0u, key1 = h1 ? order_key(lg[1]) : 0u;
    {
        // 16 group maxima (a group is GROUP lanes, or a whole warp's two keys per thread)
        uint32_t m = max(key0, key1);
        if (G::GROUP >= 32) {
            m = __reduce_max_sync(0xffffffffu, m);
            if (lane == 0) gm[warp] = m;
        } else {
#pragma unroll
            for (int s = 1; s < G::GROUP; s <<= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, s));
            if (tid < E && (tid % G::GROUP) == 0) gm[tid / G::GROUP] = m;
        }
        if (tid == 0) *cnt = 0;
        if (tid < E / 32) selmask[tid] = 0u;
    }
    __syncthreads();
    WD_DSTAMP(18, tid == 0);
    bool slow;
    {
        // threshold: the K-th best group maximum (at least K experts reach it). Every lane ranks one of the 16 maxima
        // against all of them, read from shared memory (no shuffle loops: the shuffle unit is one per SM).
        const uint32_t mine = gm[lane & 15];
        int rank = 0;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const uint32_t o = gm[j];
            rank += (o > mine) || (o == mine && j < (lane & 15));
        }
        const uint32_t thr = gm[__ffs(__ballot_sync(0xffffffffu, lane < 16 && rank == K - 1)) - 1];
        const bool c0 = h0 && key0 >= thr, c1 = h1 && key1 >= thr;
        const unsigned b0 = __ballot_sync(0xffffffffu, c0), b1 = __ballot_sync(0xffffffffu, c1);
        int base = 0;
        if (lane == 0 && (b0 | b1)) base = atom_add_shared(cnt, __popc(b0) + __popc(b1));
        base = __shfl_sync(0xffffffffu, base, 0);
        const unsigned lt = (1u << lane) - 1u;
        if (c0) {
            const int pos = base + __popc(b0 & lt);
            if (pos < kFastMaxCand) cand[pos] = make_uint2(key0, static_cast<uint32_t>(tid));
        }
        if (c1) {
            const int pos = base + __popc(b0) + __popc(b1 & lt);
            if (pos < kFastMaxCand) cand[pos] = make_uint2(key1, static_cast<uint32_t>(tid + kThreads));
        }
        slow = thr <= kKeyNegInf;      // fewer than K groups hold a finite logit: leave it to the exact rungs
    }
    __syncthreads();
    WD_DSTAMP(19, tid == 0);
    const int p2_max = static_cast<int>(P.p2_max), n_dslots = static_cast<int>(P.b3_max) * K;
    uint64_t *bar_gu = bars + kFbTiles, *bar_dn = bars + kFbTiles + 2 * p2_max;
    // warp 0: the owned picked experts in rank order with their slots, from sel_ids
    auto build_loc = [&]() {
        const int e = lane < K ? sel_ids[lane] : -1;
        const bool owned = lane < K && e >= P.e_first && e < P.e_first + P.e_count;
        int slot = owned ? slot_tab[e] : 0;
        if (owned && slot < 0) {
            if (!P.select_only) atomicOr(err, kErrExpertMiss);
            slot = 0;
        }
        const unsigned mask = __ballot_sync(0xffffffffu, owned);
        if (owned) {
            const int pos = __popc(mask & ((1u << lane) - 1u));
            loc_j[pos] = lane;
            loc_slot[pos] = slot;
        }
        if (lane == 0) *loc_n = __popc(mask);
    };
    {
        const int nc = *cnt;
        slow = slow || nc > 32 || nc < K;
        if (!slow && warp == 0) {
            // warp 0 ranks the candidates: (larger key, then lower index) is a total order
            const uint2 me = lane < nc ? cand[lane] : make_uint2(0u, 0xffffffffu);
            int rank = 0;
#pragma unroll 8
            for (int j = 0; j < nc; ++j) {      // the loads do not depend on one another
                const uint2 o = cand[j];
                rank += (o.x > me.x) || (o.x == me.x && o.y < me.y);
            }
            if (lane < nc && rank < K) {
                sel_ids[rank] = static_cast<int>(me.y);
                sel_keys[rank] = me.x;
                red_or_shared(&selmask[me.y >> 5], 1u << (me.y & 31u));
            }
            __syncwarp();
            mbar_wait(&bars[kFbSlots], mpar, err);
            build_loc();
        }
    }
    __syncthreads();
    WD_STAMP(4);

    int n_loc = 0;
    // this warp's share of the tile copies of the owned picked experts (loc_*)
    auto issue_tiles = [&]() {
        const int nl = *loc_n;
        const int n_pairs = nl * T2;
#pragma unroll 1
        for (int s = warp; s < max(p2_max, n_dslots); s += kWarps) {
            // lanes 0, 1: gate and up tile of pair slot s; lane 2: down tile slot s
            const int u = cta + s * ncta;
            const bool pair_ok = s < p2_max, pair_live = pair_ok && u < n_pairs;
            const int jl = pair_live ? u / T2 : 0, t = u % T2;
            const int bi = s / K, jj = s % K;
            const bool dn_ok = s < n_dslots, dn_live = dn_ok && bi < my_b3 && jj < nl;
            const int sl_p = loc_slot[jl], sl_d = loc_slot[dn_live ? jj : 0];
            if (lane <= 1 && pair_ok) {
                uint64_t *bar = &bar_gu[2 * s + lane];
                if (pair_live) {
                    mbar_expect_tx(bar, kIq3TileBytes);
                    bulk_load(reg_a + (2 * s + lane) * kIq3TileBytes,
                              P.pool + static_cast<size_t>(sl_p) * P.slot_bytes + (lane ? P.up_off : P.gate_off) +
                                  static_cast<size_t>(t) * kIq3TileBytes,
                              kIq3TileBytes, bar);
                } else {
                    mbar_arrive(bar);
                }
            } else if (lane == 2 && dn_ok) {
                uint64_t *bar = &bar_dn[s];
                if (dn_live) {
                    mbar_expect_tx(bar, kIq3TileBytes);
                    bulk_load(reg_b + s * kIq3TileBytes,
                              P.pool + static_cast<size_t>(sl_d) * P.slot_bytes + P.down_off +
                                  static_cast<size_t>(cta + bi * ncta) * kIq3TileBytes,
                              kIq3TileBytes, bar);
                } else {
                    mbar_arrive(bar);
                }
            }
        }
        return nl;
    };
    bool issued = false;
    if (!slow && !P.select_only) {
        n_loc = issue_tiles();
        issued = true;
    }
    WD_STAMP(5);

    // ---- while the tiles fly: softmax, weights, and the proof that the rungs by probability are these ids ------------
    {
        RouterScratch rs;
        rs.probs = nullptr;
        rs.gsum = misc + kFmGsum;
        rs.red = misc + kFmRed;
        rs.first = misc + kFmFirst;
        rs.cand = reinterpret_cast<uint32_t *>(misc + kFmCand);
        // the row maximum is the largest group maximum of the selection
        uint32_t mk = __reduce_max_sync(0xffffffffu, lane < 16 ? gm[lane] : 0u);
        const float mx = __uint_as_float((mk & 0x80000000u) ? (mk ^ 0x80000000u) : ~mk);
        float p0, p1, inv = 0.0f;
        fast_softmax(lg[0], lg[1], mx, E, rs, p0, p1, &inv);      // one block-wide synchronisation inside
        bool bad = slow;
        if (!slow) {
            // The picked set must be the rungs by PROBABILITY: nothing outside it may beat its weakest member (larger
            // probability, or the same with a lower index), and inside it the probabilities must fall in exactly this
            // order with every one an ordinary number. Every thread forms the weakest member's probability itself,
            // with the operations its owner used.
            const float pb = __fmul_rn(exp_noinline(__fsub_rn(key_to_float(sel_keys[K - 1]), mx)), inv);
            const int eb = sel_ids[K - 1];
            const bool s0 = h0 && ((selmask[tid >> 5] >> (tid & 31)) & 1u);
            const bool s1 = h1 && ((selmask[(tid + kThreads) >> 5] >> (tid & 31)) & 1u);
            bad = (h0 && !s0 && (p0 > pb || (p0 == pb && tid < eb))) || (h1 && !s1 && (p1 > pb || (p1 == pb && tid + kThreads < eb)));
            bad = bad || !(inv > 0.0f && inv < INFINITY);
            if (warp == 0) {
                const float pj = lane < K ? __fmul_rn(exp_noinline(__fsub_rn(key_to_float(sel_keys[lane]), mx)), inv) : 0.0f;
                const int ej = lane < K ? sel_ids[lane] : 0x7fffffff;
                const float pn = __shfl_down_sync(0xffffffffu, pj, 1);
                const int en = __shfl_down_sync(0xffffffffu, ej, 1);
                const bool fine = lane >= K || (pj == pj && pj > -INFINITY && (lane == K - 1 || pj > pn || (pj == pn && ej < en)));
                const bool all_fine = __all_sync(0xffffffffu, fine);   // the vote on its own: every lane must take part
                bad = bad || !all_fine;
                const float w = router_weights_warp(pj, K, P.w_scale, lane);
                if (lane < K) sel_w[lane] = w;
            }
        }
        const bool ok = !__syncthreads_or(bad);
        if (!ok) {
            // the exact rungs (rare): ids and weights as the reference computes them, and the copies once more
            fast_rungs(p0, p1, E, K, P.w_scale, rs, sel_ids, sel_w);
            if (cta == 0 && tid == 0 && P.fallbacks != nullptr) atomicAdd(P.fallbacks, 1u);
            if (warp == 0) {
                mbar_wait(&bars[kFbSlots], mpar, err);
                build_loc();
            }
            __syncthreads();
            if (!P.select_only) {
                if (issued) {
                    // the copies issued from the first ids must land before their buffers and barriers are reused
                    for (int s = tid; s < 2 * p2_max + n_dslots; s += kThreads) mbar_wait(&bar_gu[s], mpar ^ tflip, err);
                    __syncthreads();
                    tflip ^= 1u;
                }
                n_loc = issue_tiles();
            }
        }
        if (cta == 0 && tid < K) {
            P.ids[tid] = sel_ids[tid];
            P.weights[tid] = sel_w[tid];
        }
    }
    const uint32_t tpar = mpar ^ tflip;
    WD_STAMP(6);
    if (P.select_only) break;       // every copy this CTA issued has been waited for

    // ---- shared activation -> Q8_0 (needed by the shared down rows of phase 3); zero the tile accumulator ------------
    const int my_pairs = (n_loc * T2 > cta) ? (n_loc * T2 - cta + ncta - 1) / ncta : 0;
    const int n_t2 = 2 * my_pairs;
    {
        if (my_b3 > 0 && tid < SF / 4) {
            float sv[4];
            wait_tagged<4>(mbox + o_shact + tid * 4, 1, 4, tag, sv, err);
            float amax = fmaxf(fmaxf(fabsf(sv[0]), fabsf(sv[1])), fmaxf(fabsf(sv[2]), fabsf(sv[3])));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
            const int b = tid >> 3, l = tid & 7;
            uint32_t packed = 0;
            if (amax != 0.0f) {
                const float inv = __fdiv_rn(127.0f, amax);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    int q = __float2int_rn(__fmul_rn(sv[j], inv));
                    q = max(-128, min(127, q));
                    packed |= static_cast<uint32_t>(q & 0xff) << (8 * j);
                }
            }
            *reinterpret_cast<uint32_t *>(shq + (((b >> 2) * 8 + l) * 16 + (b & 3) * 4)) = packed;
            if (l == 0) shd[b] = __half2float(__float2half_rn(__fdiv_rn(amax, 127.0f)));
        }
        for (int i = tid; i < n_t2 * kFastAccStride; i += kThreads) acc[i] = 0;
        __syncthreads();
    }

    // ---- phase 2: gate and up tiles in sub-block units, evenly over the warps ---------------------------------------
    {
        const uint8_t *a_lane = xk + (lane % NSB_H) * kActSbStride;
        auto to_rowbuf = [&](int d, int, int, int rr, float a) { rowbuf[d * R2 + rr] = a; };
        if (n_t2 >= kWarps) {
            // A whole tile per warp first: its partials never leave the warp (they pass through the warp's own slot of
            // the accumulator only to change hands between lanes), and the warp runs the tile's float chains at once.
            // The tiles beyond 16 are cut into sub-block units, one or two per warp.
            fast_tile_units<K>(warp * 8, warp * 8 + 8, reg_a, bar_gu, acc, a_lane, 0, 0, lane, tab, tpar, err);
            __syncwarp();
            fast_float_stage<NSB_H, K>(warp, warp + 1, reg_a, acc, xdk, 0, lane, 32, to_rowbuf);
            const int n_left = (n_t2 - kWarps) * 8, per = (n_left + kWarps - 1) / kWarps;
            const int u0 = kWarps * 8 + min(warp * per, n_left), u1 = min(u0 + per, kWarps * 8 + n_left);
            fast_tile_units<K>(u0, u1, reg_a, bar_gu, acc, a_lane, 0, 0, lane, tab, tpar, err);
            __syncthreads();
            WD_STAMP(7);
            fast_float_stage<NSB_H, K>(kWarps, n_t2, reg_a, acc, xdk, 0, tid, kThreads, to_rowbuf);
        } else {
            // less than one tile per warp (few owned experts): everything in sub-block units, evenly over the warps
            const int n_units = n_t2 * 8, per = (n_units + kWarps - 1) / kWarps;
            const int u0 = min(warp * per, n_units), u1 = min(u0 + per, n_units);
            fast_tile_units<K>(u0, u1, reg_a, bar_gu, acc, a_lane, 0, 0, lane, tab, tpar, err);
            __syncthreads();
            WD_STAMP(7);
            fast_float_stage<NSB_H, K>(0, n_t2, reg_a, acc, xdk, 0, tid, kThreads, to_rowbuf);
        }
        __syncthreads();
        if (tid < my_pairs * R2) {
            const int s2 = tid / R2, rr = tid % R2;
            const int u = cta + s2 * ncta, jl = u / T2, t = u % T2;
            const float g = rowbuf[(2 * s2) * R2 + rr], up = rowbuf[(2 * s2 + 1) * R2 + rr];
            (void)jl;
            (void)t;
            pushbuf[s2 * R2 + rr] = make_tagged(silu_mul(g, up), tag);
        }
        const int n_t3 = my_b3 * n_loc;
        for (int i = tid; i < n_t3 * kFastAccStride; i += kThreads) acc[i] = 0;
        __syncthreads();            // region A is free: it receives the next layer's phase-1 rows during the down phase
        // this CTA's act values into every band CTA's mailbox, each tile pair's rows at their place in [expert][F]
        {
            const int n_w = my_pairs * R2;
#pragma unroll 1
            for (int i0 = 0; i0 < n_w; i0 += 32) {
                const int i = i0 + lane;
                const bool live = i < n_w;
                const int s2 = i / R2, u = cta + s2 * ncta;
                const size_t off = o_act + static_cast<size_t>(u / T2) * F + (u % T2) * R2 + i % R2;
                const tagged_t w = live ? pushbuf[i] : 0ull;
#pragma unroll 1
                for (int d = warp; d < n_band_mbox; d += kWarps)
                    if (live)
                        asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(P.xbuf + static_cast<size_t>(d) * P.xstride + off), "l"(w)
                                     : "memory");
            }
        }
    }
    WD_STAMP(8);
    // the next layer's phase-1 weights travel during the down phase
    if (warp == kWarps - 1 && layer + 1 < P.layer_end) issue_phase1(P.layers[layer + 1]);

    // ---- phase 3: this CTA's row bands ----------------------------------------------------------------------------------
    if (my_b3 > 0) {
        const int n_t3 = my_b3 * n_loc;
        // expert parallel: this layer's rows go into the half of every peer's row buffer that layer tag - 2 used; the
        // peer must have left that layer (the synchronisation after the gather below hands the result to every warp)
        if (warp == 1 && lane < P.n_peers) wait_tag_reached(P.t_peer_left + P.peer_rank[lane], tag - 2u, err);
        // the shared gate scalar (published in phase 1 by one CTA) for the combine threads
        float sg = 0.0f;
        if (tid < my_b3 * R3) {
            float one[1];
            wait_tagged<1>(mbox + o_shgate, 1, 1, tag, one, err);
            sg = one[0];
        }
        // Every owned expert's activation -> Q8_K, one warp per superblock (256 consecutive words of the mailbox). A warp
        // with two superblocks (more than 16 in all) polls both at once, so that the second costs no round trip.
        const int n_sb = n_loc * NSB_F;
#pragma unroll 1
        for (int sb0 = warp; sb0 < n_sb; sb0 += 2 * kWarps) {
            const int sb1 = sb0 + kWarps;
            const bool two = sb1 < n_sb;
            const tagged_t *src0 = mbox + o_act + static_cast<size_t>(sb0 / NSB_F) * F + (sb0 % NSB_F) * 256 + lane * 8;
            const tagged_t *src1 = mbox + o_act + static_cast<size_t>((two ? sb1 : sb0) / NSB_F) * F + ((two ? sb1 : sb0) % NSB_F) * 256 + lane * 8;
            tagged_t w[16] = {};
            unsigned long long t0 = 0ull;
            for (unsigned it = 0;; ++it) {
                unsigned bad = 0;
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (it == 0 || tag_behind(w[i], tag)) w[i] = ld_tagged(src0 + i);
                if (two) {
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        if (it == 0 || tag_behind(w[8 + i], tag)) w[8 + i] = ld_tagged(src1 + i);
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) bad |= tag_behind(w[i], tag) | (two & tag_behind(w[8 + i], tag));
                if (!bad) break;
                if (wait_expired(it, t0, err)) break;
            }
            float v[8];
            unsigned over = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                over |= tag_ahead(w[i], tag) | (two & tag_ahead(w[8 + i], tag));
                v[i] = __uint_as_float(static_cast<uint32_t>(w[i]));
            }
            report_overrun(over, err);
            WD_DSTAMP(24, tid == 0 && sb0 == 0);
            q8k_from_regs(v, lane, actk + sb0 * kActSbStride, &actd[sb0]);
            if (two) {
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(static_cast<uint32_t>(w[8 + i]));
                q8k_from_regs(v, lane, actk + sb1 * kActSbStride, &actd[sb1]);
            }
        }
        WD_DSTAMP(26, tid == 0);
        __syncthreads();
        WD_STAMP(9);
        {
            // down tile list of this CTA: index d = bi * n_loc + jl lives in staging slot bi * K + jl
            const int n_units = n_t3 * 8, per = (n_units + kWarps - 1) / kWarps;
            const int u0 = min(warp * per, n_units), u1 = min(u0 + per, n_units);
            fast_tile_units<K>(u0, u1, reg_b, bar_dn, acc, actk + (lane % NSB_F) * kActSbStride, NSB_F * kActSbStride, n_loc,
                               lane, tab, tpar, err);
        }
        // the shared expert's down rows of the bands: one row per warp
        mbar_wait(&bars[kFbSharedDown], mpar, err);
#pragma unroll 1
        for (int r = warp; r < my_b3 * R3; r += kWarps) {
            const float d = q8_row_warp<G::NBS>(reg_c + r * G::ROW_S, shq, shd, lane);
            if (lane == 0) shrow[r] = d;
        }
        __syncthreads();
        WD_STAMP(10);
        // float chains of the down tiles; expert parallel: the peers combine these rows too
        fast_float_stage<NSB_F, K>(0, n_t3, reg_b, acc, actd, n_loc, tid, kThreads, [&](int, int bi, int jl, int rr, float a) {
            const int j = loc_j[jl], row = (cta + bi * ncta) * R3 + rr;
            rows3[(bi * K + j) * R3 + rr] = a;
            P.expert_out[static_cast<size_t>(j) * H + row] = a;
#pragma unroll 1
            for (int pr = 0; pr < P.n_peers; ++pr)
                st_tagged_sys(P.peer_expert_out[pr] + static_cast<size_t>(par) * K * H + static_cast<size_t>(j) * H + row, a, tag);
        });
        __syncthreads();
        // ---- combine: one thread per row of the bands -------------------------------------------------------------------
        if (tid < my_b3 * R3) {
            const int bi = tid / R3, rr = tid % R3, row = (cta + bi * ncta) * R3 + rr;
            float accf = 0.0f;
            if (P.n_peers == 0 && n_loc == K) {
                // one GPU: every picked expert's row is in shared memory; rank-ordered add_rn(mul_rn())
                float ev[K];
#pragma unroll
                for (int j = 0; j < K; ++j) ev[j] = rows3[(bi * K + j) * R3 + rr];
#pragma unroll
                for (int j = 0; j < K; ++j) accf = __fadd_rn(accf, __fmul_rn(ev[j], sel_w[j]));
            } else if (P.n_peers == 0) {
                // an unconnected rank's partial sum: its own experts, in rank order
#pragma unroll 1
                for (int q = 0; q < n_loc; ++q) {
                    const int j = loc_j[q];
                    accf = __fadd_rn(accf, __fmul_rn(rows3[(bi * K + j) * R3 + rr], sel_w[j]));
                }
            } else {
                // rows of the experts other ranks own arrive in this rank's row buffer
                float ev[K];
                unsigned ownedmask = 0;
                for (int q = 0; q < n_loc; ++q) ownedmask |= 1u << loc_j[q];
                tagged_t w[K] = {};
                unsigned long long t0 = 0ull;
                for (unsigned it = 0;; ++it) {
                    unsigned bad = 0;
#pragma unroll
                    for (int j = 0; j < K; ++j)
                        if (!((ownedmask >> j) & 1u)) {
                            w[j] = ld_tagged(t_eo + static_cast<size_t>(j) * H + row);
                            bad |= tag_behind(w[j], tag);
                        }
                    if (!bad) break;
                    if (wait_expired(it, t0, err)) break;
                }
                unsigned over = 0;
#pragma unroll
                for (int j = 0; j < K; ++j) {
                    const bool mine_j = (ownedmask >> j) & 1u;
                    over |= !mine_j & tag_ahead(w[j], tag);
                    ev[j] = mine_j ? rows3[(bi * K + j) * R3 + rr] : __uint_as_float(static_cast<uint32_t>(w[j]));
                    if (!mine_j) P.expert_out[static_cast<size_t>(j) * H + row] = ev[j];
                }
                report_overrun(over, err);
#pragma unroll
                for (int j = 0; j < K; ++j) accf = __fadd_rn(accf, __fmul_rn(ev[j], sel_w[j]));
            }
            const float sd = shrow[tid];
            P.routed[row] = accf;
            P.shared_down[row] = sd;
            const float o = __fadd_rn(accf, __fmul_rn(sd, sg));
            P.out[row] = o;
            if (P.residual != nullptr) {
                float *oldr = rows3 + P.b3_max * K * R3;
                const float old = first ? P.residual[row] : oldr[tid];
                const float nr = __fadd_rn(old, o);
                oldr[tid] = nr;
                pushbuf[tid] = make_tagged(nr, tag);
                if (layer + 1 == P.layer_end) P.residual[row] = nr;
            }
        }
        if (P.residual != nullptr) {
            // the new residual rows of this CTA's bands into every mailbox: a band is whole lines
            __syncthreads();
#pragma unroll 1
            for (int bi = 0; bi < my_b3; ++bi)
                push_words(pushbuf + bi * R3, R3, P.xbuf, P.xstride, o_res + static_cast<size_t>(cta + bi * ncta) * R3, n_mbox, warp, lane);
        }
    }
    WD_STAMP(11);
    WD_GSTAMP(29);
    __syncthreads();    // the next layer reuses this CTA's shared memory
    if (tid == 0) st_tagged(P.t_progress + cta, 0.0f, tag);
    }   // layers
#undef WD_STAMP
#undef WD_DSTAMP
#undef WD_GSTAMP
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(P.sync + 9, 1u) == static_cast<unsigned>(ncta) - 1u) {
            P.sync[9] = 0u;
            P.sync[8] = epoch + static_cast<uint32_t>(P.layer_end - P.layer_begin);
            __threadfence();
            for (int p = 0; p < P.n_peers; ++p)
                st_tagged_sys_release(P.peer_left_out[p], 0.0f, epoch + static_cast<uint32_t>(P.layer_end - P.layer_begin));
            if (P.host_status) *P.host_status = *reinterpret_cast<volatile unsigned *>(err);
        }
    }
}

}  // namespace wd
