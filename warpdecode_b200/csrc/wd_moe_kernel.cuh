// The fused MoE layer kernel: one persistent cooperative launch runs a range of layers (batch 1).
//
// Values that cross CTAs travel as tagged words (value + layer tag in one 8-byte store) that the consumer
// polls; there is no grid barrier and no fence anywhere in the layer loop.
//
//   phase 0  every CTA: x (optionally RMSNorm(residual) * w) -> Q8_0 and Q8_K blocks in shared memory
//   phase 1  Q8_0 row tasks spread over the grid: router logits, shared-expert gate/up + SiLU,
//            shared gate scalar                                        -> published
//   phase 1b every CTA gathers the logits and the shared activation: softmax / top-k (whole CTA), shared
//            activation -> Q8_0; then ALL bulk copies of this CTA's share of the selected experts'
//            gate/up/down tiles are issued at once
//   phase 2  gate+up tiles -> SiLU(g)*u per expert row; shared-expert down rows on the warps that have
//            no tile                                                    -> published
//   phase 3  gather the owned experts' activations -> Q8_K; down tiles   -> published (also to peers)
//   combine  each CTA owns a band of output rows: ordered weighted sum + shared expert + residual update,
//            the new residual published for the next layer's phase 0
//
// Reference call sites this replaces: q38_moe_select_experts_f32_x (src/qwen38_moe.cuh:2323),
// q38_moe_run_batched_experts (:3312, five launches), run_qwen38_shared_expert_f32_x (:3963, nine
// launches), q38_finish_moe_f32 (:2442) and the per-layer ids D2H + stream sync (:2363-2379).
#pragma once

#include "wd_router.cuh"

namespace wd {

constexpr int kMaxBars = 96;
constexpr int kStampStride = 32;    // profiling stamps per CTA: 0..15 phases of the layer, 16..23 stages of the selection

// Weights of one layer (device pointers, repacked layouts).
struct LayerDev {
    const uint8_t *router_w;     // Q8_0 tasks [E/4]
    const float *router_bias;    // nullable
    const float *sh_gate_vec;    // F32 [H]
    const uint8_t *sh_gate, *sh_up, *sh_down;   // Q8_0 tasks
    const float *norm_w;         // nullable
    const int *slot_of_expert;   // [E] slot index or -1
};

struct MoeParams {
    // geometry
    int H, F, SF, E, K;
    int nsb_h, nsb_f;            // superblocks per row of gate/up and of down
    int t2_log2, t3_log2;        // log2 of the tiles per expert: gate/up (F*nsb_h/32) and down (H*nsb_f/32)
    int e_first, e_count;        // owned expert range
    float w_scale, eps;
    double inv_h;                // 1 / H when H is a power of two (the division is then an exact multiply), else 0
    // layers [layer_begin, layer_end) run back to back inside one launch, so that after the first layer
    // every instruction comes from the instruction cache
    const LayerDev *layers;      // device array, one entry per layer of the stack
    int layer_begin, layer_end;
    // A batch of tokens through ONE layer (speculative verify): n_tokens > 1 runs layer_begin once per token inside one
    // launch, token t reading x + t * H and writing out + t * H, ids + t * K, weights + t * K (no residual mode). The
    // tokens take the place of the layers in the launch's sequence of tags and mbarrier phases, and the copies of the
    // layer's phase-1 weights for token t + 1 travel during token t's down phase.
    int n_tokens;
    int stamp_layer;             // the layer whose phase timestamps are recorded
    int select_only;             // 1: stop after the selection (ids and weights written); nothing else changes
    // Capped expert cache, optimistic: layers run on as long as every selected expert has a slot. A layer that meets
    // an expert without one stops the launch there (every CTA computes the same selection, so all of them stop at
    // the same layer without talking to one another): the residual as of that layer's input goes back to `residual`,
    // miss_info[0] receives the layer's index (-1: the launch ran through) and the host places the experts and
    // launches again from that layer. miss_info[1 + l * K + j] logs every finished layer's picks (for the cache's
    // recency order); miss_info lives in page-locked host memory.
    int stop_on_miss;
    int *miss_info;
    int threshold_select;        // 1: expert ids from a threshold on the logits, proven afterwards (wd_router.cuh); 0: the rungs
    unsigned *fallbacks;         // nullable: counts the rows whose proof failed and that took the exact rungs (CTA 0)
    const uint8_t *pool;         // slot pool base
    unsigned long long slot_bytes;
    unsigned gate_off, up_off, down_off;        // offsets of the three matrices inside a slot
    const uint16_t *grid_packed; // packed IQ3_S codebook in global memory
    const uint16_t *grid2_packed;// packed IQ2_S codebook
    int gu_type, d_type;         // ggml type of the gate/up tensors and of the down tensor (IQ3_S or IQ2_S)
    unsigned gu_tile, d_tile;    // bytes of one tile of 32 blocks of each
    // activations
    const float *x;              // [H] (used when residual == nullptr)
    float *residual;             // nullable: x = RMSNorm(residual) * norm_w, residual += out
    float *out;                  // [H]
    // exchange buffers (global): every value travels as a tagged word (value + layer tag, one 8-byte
    // store) that its consumers poll; there is no grid barrier and no fence. Each buffer exists twice,
    // indexed by layer parity, so that a CTA one layer ahead never overwrites words still being read.
    tagged_t *t_logits;          // [2][E]
    tagged_t *t_shared_act;      // [2][SF]
    tagged_t *t_shared_gate;     // [2][1]
    tagged_t *t_act;             // [2][K][F]
    tagged_t *t_expert_out;      // [2][K][H]
    tagged_t *t_shared_down;     // [2][H]
    tagged_t *t_residual;        // [2][H]   updated residual = next layer's input
    tagged_t *t_progress;        // [grid]   tag of the last layer each CTA has completely left
    tagged_t *peer_expert_out[8];// expert-parallel peers' t_expert_out buffers (n_peers entries)
    int n_peers;                 // 0: single GPU (or partial sums only); else every rank combines all K experts
    // Flow control between ranks: word [r] of t_peer_left holds the tag of the last layer whose expert rows rank r
    // has finished reading. Rank r writes it into every peer (peer_left_out[p] = that peer's word for this rank);
    // a rank stores layer t's rows into a peer only after that peer has left layer t - 2, the previous user of the
    // same half of its row buffer.
    tagged_t *t_peer_left;       // [8]
    tagged_t *peer_left_out[8];
    int peer_rank[8];            // global rank of peer p
    int *ids;                    // [K]   (plain copies for inspection, written by CTA 0)
    float *weights;              // [K]
    float *routed;               // [H]
    unsigned long long *stamps;  // nullable: [cta][kStampStride] globaltimer values at phase boundaries (profiling)
    unsigned *host_status;       // nullable, host memory: receives the error word when the launch ends
    unsigned *sync;              // [2] error word, [8] tag epoch (tag of layer `layer_begin` is epoch + 1; the
                                 // last CTA to leave advances it by the layers run), [9] count of CTAs that left
    // shared memory plan (byte offsets from the dynamic shared base; all 128-byte aligned)
    unsigned off_tab, off_tab2, off_xq0, off_xd0, off_xk, off_xdk, off_actk, off_actd, off_shq, off_shd,
        off_misc, off_scr, off_bar, off_slots, off_rowbuf, off_stage_a, off_stage_b;
    unsigned scr_bytes;          // per-warp transposition scratch
    unsigned scr_rows;           // float offset of the two 32-float row buffers inside it
    unsigned n1r, n1s, n2, n3, nsd;   // staging slots per CTA: router tasks, shared g/u tasks, phase-2 units,
                                      // phase-3 tiles, shared-down tasks
};

// float offsets inside the `misc` region once phase 1 is over (before that it holds x as floats)
#ifndef WD_MAX_SLICES
#define WD_MAX_SLICES 2
#endif
constexpr int kMaxSlices = WD_MAX_SLICES;   // slices per gate/up tile left over after a whole round (measured: 2 beats 4 beats 8)
constexpr int kLeftInts = 2048;     // = kMiscGsum: the x floats / router candidates region, reused in phase 2
constexpr int kMiscLogits = 0, kMiscProbs = 1024, kMiscGsum = 2048, kMiscRed = 2176, kMiscTop = 2192,
              kMiscChamp = 2208, kMiscDsum = 2272, kMiscIds = 2288, kMiscW = 2304, kMiscLocJ = 2320,
              kMiscLocSlot = 2336, kMiscLocN = 2352, kMiscMiss = 2353, kMiscSlots = 2368, kMiscSharedAct = 2400;

// Phase 0 of one thread: its EPL consecutive residual values (plain memory in the first layer of a launch, the
// previous layer's tagged words otherwise, polled together with the progress word), the norm weights, and the
// binary-tree sum of their squares in double.
template <int EPL>
__device__ __forceinline__ double p0_gather(const float *plain, const float *norm_w, const tagged_t *src, const tagged_t *progress,
                                            bool mine, bool first, bool chk, uint32_t tag, unsigned *err, float rv[16],
                                            float nw[16]) {
#pragma unroll
    for (int i = 0; i < EPL; ++i) nw[i] = (norm_w && mine) ? norm_w[i] : 1.0f;      // fetched before the wait, used after it
    if (!mine) return 0.0;
    if (first) {
#pragma unroll
        for (int i = 0; i < EPL; ++i) rv[i] = plain[i];
    } else {
        tagged_t w[EPL];
        unsigned long long t0 = 0ull;
        for (unsigned it = 0;; ++it) {
#pragma unroll
            for (int i = 0; i < EPL; ++i) w[i] = ld_tagged(src + i);
            const tagged_t wp = chk ? ld_tagged(progress) : 0;
            unsigned bad = chk & tag_behind(wp, tag - 2u);
#pragma unroll
            for (int i = 0; i < EPL; ++i) bad |= tag_behind(w[i], tag - 1u);
            if (!bad) break;
            if (wait_expired(it, t0, err)) break;
        }
        unsigned over = 0;
#pragma unroll
        for (int i = 0; i < EPL; ++i) over |= tag_ahead(w[i], tag - 1u);
        report_overrun(over, err);
#pragma unroll
        for (int i = 0; i < EPL; ++i) rv[i] = __uint_as_float(static_cast<uint32_t>(w[i]));
    }
    double loc[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) loc[i] = __dmul_rn(static_cast<double>(rv[i]), static_cast<double>(rv[i]));
#pragma unroll
    for (int w = 1; w < EPL; w <<= 1)
#pragma unroll
        for (int i = 0; i + w < EPL; i += 2 * w) loc[i] = __dadd_rn(loc[i], loc[i + w]);
    return loc[0];
}

// The bulk copies of phase 1 of one layer, issued by the lanes of one warp together: lanes 0-7 router tasks,
// 8-15 shared gate tasks, 16-23 their up halves (same barrier), 24 the slot table, 25 the shared gate vector (one
// CTA); eight slots of each kind per round. `tasks`: the row tasks and the slot table (their buffers are free from
// the previous layer's down phase on); `gate_vec`: the shared gate vector, whose buffer (stage B) is not.
__device__ __forceinline__ void issue_phase1_copies(const MoeParams &P, const LayerDev &L, int lane, int cta, int ncta,
                                                    unsigned rt_bytes, uint8_t *stage_a, uint8_t *stage_b, int *slot_tab,
                                                    uint64_t *bars, bool tasks, bool gate_vec) {
    const int n_rt = P.E >> 2, n_st = P.SF >> 2;
    const unsigned a1_slot = 2u * rt_bytes;
    const int k = lane & 7, grp = lane >> 3;
    const int rounds = tasks ? (max(static_cast<int>(P.n1r), static_cast<int>(P.n1s)) + 7) >> 3 : 1;
#pragma unroll 1
    for (int r = 0; r < max(rounds, 1); ++r) {
        const int s = r * 8 + k;
        bool copy = false, expect = false;
        uint8_t *dst = stage_a;
        const uint8_t *src = L.router_w;
        unsigned bytes = rt_bytes, tx = rt_bytes;
        uint64_t *bar = bars;
        if (grp == 0) {
            const int t = cta + s * ncta;
            copy = expect = tasks && s < static_cast<int>(P.n1r) && t < n_rt;
            dst = stage_a + s * a1_slot;
            src = L.router_w + static_cast<size_t>(copy ? t : 0) * rt_bytes;
            bar = &bars[s];
        } else if (grp <= 2) {
            const int t = ncta - 1 - cta + s * ncta;
            copy = tasks && s < static_cast<int>(P.n1s) && t < n_st;
            expect = copy && grp == 1;
            dst = stage_a + (P.n1r + s) * a1_slot + (grp == 2 ? rt_bytes : 0u);
            src = (grp == 1 ? L.sh_gate : L.sh_up) + static_cast<size_t>(copy ? t : 0) * rt_bytes;
            tx = 2u * rt_bytes;
            bar = &bars[P.n1r + s];
        } else if (r == 0 && k == 0) {
            copy = expect = tasks;
            dst = reinterpret_cast<uint8_t *>(slot_tab);
            src = reinterpret_cast<const uint8_t *>(L.slot_of_expert);
            bytes = tx = static_cast<unsigned>(P.E) * 4u;
            bar = &bars[kMaxBars - 2];
        } else if (r == 0 && k == 1) {
            // the one CTA that computes the shared gate scalar brings the F32 gate vector into stage B
            copy = expect = gate_vec && P.SF > 0 && cta == ncta / 2;
            dst = stage_b;
            src = reinterpret_cast<const uint8_t *>(L.sh_gate_vec);
            bytes = tx = static_cast<unsigned>(P.H) * 4u;
            bar = &bars[kMaxBars - 1];
        }
        if (expect) mbar_expect_tx(bar, tx);
        if (copy) bulk_load(dst, src, bytes, bar);
    }
}

extern __shared__ __align__(128) uint8_t wd_smem[];

__global__ void __launch_bounds__(kThreads, 1) moe_layer_kernel(const __grid_constant__ MoeParams P) {
    uint8_t *sm = wd_smem;
    uint8_t *tab = sm + P.off_tab;                                   // IQ3_S codebook, lane-private copies
    uint8_t *tab2 = sm + P.off_tab2;                                 // IQ2_S codebook
    uint8_t *xq0 = sm + P.off_xq0;                                   // Q8_0 quants of x
    float *xd0 = reinterpret_cast<float *>(sm + P.off_xd0);          // Q8_0 scales of x
    uint8_t *xk = sm + P.off_xk;                                     // Q8_K quants of x, kActSbStride per superblock
    float *xdk = reinterpret_cast<float *>(sm + P.off_xdk);
    uint8_t *actk = sm + P.off_actk;                                 // per selected expert: Q8_K act
    float *actd = reinterpret_cast<float *>(sm + P.off_actd);
    uint8_t *shq = sm + P.off_shq;                                   // Q8_0 quants of the shared activation
    float *shd = reinterpret_cast<float *>(sm + P.off_shd);
    float *misc = reinterpret_cast<float *>(sm + P.off_misc);
    uint64_t *bars = reinterpret_cast<uint64_t *>(sm + P.off_bar);
    int *slot_tab = reinterpret_cast<int *>(sm + P.off_slots);      // this layer's slot of every expert
    float *rowbuf = reinterpret_cast<float *>(sm + P.off_rowbuf);    // row sums of this CTA's gate and up tiles
    int *left_ints = reinterpret_cast<int *>(misc);                  // integer partials of sliced tile tasks: the
                                                                     // first kLeftInts words of misc, free in phase 2
    uint8_t *stage_a = sm + P.off_stage_a;
    uint8_t *stage_b = sm + P.off_stage_b;
    unsigned *err = P.sync + 2;
    uint32_t epoch;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(epoch) : "l"(P.sync + 8) : "memory");

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cta = blockIdx.x, ncta = gridDim.x;
    const int nbh = P.H >> 5, nbs = P.SF >> 5;
    const uint32_t lane4x2 = static_cast<uint32_t>(lane * 4) * 0x0101u;
    float *scr = reinterpret_cast<float *>(sm + P.off_scr + warp * P.scr_bytes);
    float *rows_a = scr + P.scr_rows;                               // per-warp row results of a tile

    float *xf = misc;                                               // [H], phases 0 and 1 only
    int *sel_ids = reinterpret_cast<int *>(misc + kMiscIds);
    float *sel_w = misc + kMiscW;
    int *loc_j = reinterpret_cast<int *>(misc + kMiscLocJ);         // rank-order index of each owned selected expert
    int *loc_slot = reinterpret_cast<int *>(misc + kMiscLocSlot);
    int *loc_n = reinterpret_cast<int *>(misc + kMiscLocN);

#define WD_STAMP(i)                                                                            \
    if (stamp_on) {                                                                            \
        unsigned long long t__;                                                                \
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__) : : "memory");                                \
        P.stamps[cta * kStampStride + (i)] = t__;                                                        \
        if ((i) == 0 || (i) == 10) P.stamps[cta * kStampStride + 24 + (i) / 10] = clock64();   /* SM clock rate */ \
    }
    if (tid < kMaxBars) {       // the last two belong to the shared gate vector and the slot table
        mbar_init(&bars[tid], 1);
        mbar_fence_init();
    }
    if (cta == 0 && tid == 0) P.sync[5] = smem_u32(bars);      // so that a copy timeout can be reported by barrier index
    if (P.gu_type == kTypeIq3s || P.d_type == kTypeIq3s) build_grid_table(tab, P.grid_packed);   // first needed in phase 2
    if (P.gu_type == kTypeIq2s || P.d_type == kTypeIq2s) build_iq2_table(tab2, P.grid2_packed);
    __syncthreads();

    const int seq_end = P.n_tokens > 1 ? P.layer_begin + P.n_tokens : P.layer_end;   // end of the launch's sequence
    int seq_done = seq_end - P.layer_begin;             // positions that consumed a tag (less when a miss stops the launch)
    int *miss_flag = reinterpret_cast<int *>(misc + kMiscMiss);
    uint32_t tflip = 0;         // flips when a layer issued its tile copies twice (the proof of the picked set failed)
#pragma unroll 1
    for (int layer = P.layer_begin; layer < seq_end; ++layer) {     // position in the sequence: a layer, or a token
    const int tok = P.n_tokens > 1 ? layer - P.layer_begin : 0;
    const LayerDev L = P.layers[P.n_tokens > 1 ? P.layer_begin : layer];
    const uint32_t mpar = static_cast<uint32_t>(layer - P.layer_begin) & 1u;  // every mbarrier completes once per layer
    const uint32_t tag = epoch + static_cast<uint32_t>(layer - P.layer_begin) + 1u;
    // The half of every exchange buffer follows the TAG, not the position in the launch: consecutive layers then
    // alternate halves across launches too (a peer may still be one launch behind).
    const uint32_t par = tag & 1u;
    const bool stamp_on = P.stamps != nullptr && tid == 0 && layer == P.stamp_layer;
    // this layer's halves of the exchange buffers
    tagged_t *t_logits = P.t_logits + par * P.E;
    tagged_t *t_shact = P.t_shared_act + par * (P.SF > 0 ? P.SF : 1);
    tagged_t *t_shgate = P.t_shared_gate + par;
    tagged_t *t_act = P.t_act + static_cast<size_t>(par) * P.K * P.F;
    tagged_t *t_eo = P.t_expert_out + static_cast<size_t>(par) * P.K * P.H;
    tagged_t *t_shdown = P.t_shared_down + par * P.H;
    tagged_t *t_res = P.t_residual + par * P.H;
    WD_STAMP(0);
    if (P.stamps != nullptr && tid == 0 && layer == P.stamp_layer + 1) {   // start of the next layer: the layer period
        unsigned long long t__;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__) : : "memory");
        P.stamps[cta * kStampStride + 14] = t__;
    }

    // ---- issue phase-1 copies: router tasks and shared gate/up tasks of this CTA --------------
    const int n_rt = P.E >> 2;                     // router tasks (4 rows each)
    const int n_st = P.SF >> 2;                    // shared gate/up tasks (4 row pairs each)
    const unsigned rt_bytes = static_cast<unsigned>(nbh) * 136u;
    const unsigned a1_slot = 2u * rt_bytes;        // staging slot of phase 1
    // Phase-1 weights do not depend on data: from the second layer of a launch on they were requested by the
    // previous layer (see the down phase), so only the first layer asks for them here.
    if (warp == 0) {
        fence_proxy_async();        // the staging buffers were last read by ordinary loads (previous layer)
        issue_phase1_copies(P, L, lane, cta, ncta, rt_bytes, stage_a, stage_b, slot_tab, bars, layer == P.layer_begin, true);
    }
    WD_STAMP(1);

    // ---- phase 0: x -> shared (with the optional RMSNorm prologue), then both quantisations --
    if (P.residual != nullptr) {
        // sum of squares as a perfect binary tree over consecutive elements, in double
        const int epl = P.H >= kThreads ? P.H / kThreads : 1;       // 1, 2, 4, 8 or 16 (H = 256 * 2^n)
        const bool mine = tid * epl < P.H;
        const bool first = layer == P.layer_begin;
        // the previous layer's combine publishes the updated residual row by row; the same round trips check that
        // no CTA is still inside the layer whose exchange buffers this layer overwrites
        const bool chk = layer >= P.layer_begin + 2 && tid < ncta;
        const tagged_t *src = P.t_residual + (par ^ 1u) * P.H + tid * epl;
        float rv[16], nw[16];
        double ss;
        switch (epl) {      // the element count per thread as a compile-time constant: no predicated-off work
            case 1: ss = p0_gather<1>(P.residual + tid * epl, L.norm_w ? L.norm_w + tid * epl : nullptr, src, P.t_progress + tid, mine, first, chk, tag, err, rv, nw); break;
            case 2: ss = p0_gather<2>(P.residual + tid * epl, L.norm_w ? L.norm_w + tid * epl : nullptr, src, P.t_progress + tid, mine, first, chk, tag, err, rv, nw); break;
            case 4: ss = p0_gather<4>(P.residual + tid * epl, L.norm_w ? L.norm_w + tid * epl : nullptr, src, P.t_progress + tid, mine, first, chk, tag, err, rv, nw); break;
            case 8: ss = p0_gather<8>(P.residual + tid * epl, L.norm_w ? L.norm_w + tid * epl : nullptr, src, P.t_progress + tid, mine, first, chk, tag, err, rv, nw); break;
            default: ss = p0_gather<16>(P.residual + tid * epl, L.norm_w ? L.norm_w + tid * epl : nullptr, src, P.t_progress + tid, mine, first, chk, tag, err, rv, nw); break;
        }
#pragma unroll
        for (int s = 1; s < 32; s <<= 1) ss = __dadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, s));
        double *redd = reinterpret_cast<double *>(sm + P.off_scr);
        if (lane == 0) redd[warp] = ss;
        __syncthreads();
        // Every residual row of the previous layer is here, so every CTA of this rank has finished reading that
        // layer's expert rows (a combine publishes its residual rows after it has read them): tell the peers.
        if (cta == 0 && !first && tid < P.n_peers) st_tagged_sys_release(P.peer_left_out[tid], 0.0f, tag - 1u);
        double tot[kWarps];
#pragma unroll
        for (int i = 0; i < kWarps; ++i) tot[i] = redd[i];
#pragma unroll
        for (int w = 1; w < kWarps; w <<= 1)
#pragma unroll
            for (int i = 0; i + w < kWarps; i += 2 * w) tot[i] = __dadd_rn(tot[i], tot[i + w]);
        const float scale = __double2float_rn(
            __ddiv_rn(1.0, __dsqrt_rn(__dadd_rn(P.inv_h != 0.0 ? __dmul_rn(tot[0], P.inv_h)
                                                               : __ddiv_rn(tot[0], static_cast<double>(P.H)),
                                                static_cast<double>(P.eps)))));
        if (mine) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                if (i >= epl) break;
                float v = __fmul_rn(rv[i], scale);
                if (L.norm_w) v = __fmul_rn(v, nw[i]);
                xf[tid * epl + i] = v;
            }
        }
    } else {
        if (layer >= P.layer_begin + 2 && tid < ncta) wait_tag_reached(P.t_progress + tid, tag - 2u, err);
#pragma unroll 1
        for (int i = tid; i < P.H; i += kThreads) xf[i] = P.x[static_cast<size_t>(tok) * P.H + i];
        if (P.n_peers > 0 && cta == 0 && layer >= P.layer_begin + 2) {      // every CTA has left layer tag - 2
            __syncthreads();
            if (tid < P.n_peers) st_tagged_sys_release(P.peer_left_out[tid], 0.0f, tag - 2u);
        }
    }
    const float *gate_vec_s = reinterpret_cast<const float *>(stage_b);
    __syncthreads();
    quantize_q8_0_cta(xf, P.H, xq0, xd0);
#pragma unroll 1
    for (int sb = warp; sb < P.nsb_h; sb += kWarps)
        quantize_q8_K_warp(xf + sb * 256, lane, xk + sb * kActSbStride, &xdk[sb]);
    __syncthreads();
    WD_STAMP(2);

#include "wd_moe_kernel_phases.inc"

    WD_STAMP(10);
    __syncthreads();    // the next layer reuses this CTA's shared memory
    if (tid == 0) st_tagged(P.t_progress + cta, 0.0f, tag);
    }   // layers
#undef WD_STAMP
    if (tid == 0) {
        // every CTA read the epoch before it got here, so the last one to leave may advance it
        __threadfence();        // this CTA's reads of the last layers' rows come before its arrival below
        if (atomicAdd(P.sync + 9, 1u) == static_cast<unsigned>(ncta) - 1u) {
            P.sync[9] = 0u;
            P.sync[8] = epoch + static_cast<uint32_t>(seq_done);
            // every CTA of this rank has left the launch: the peers may overwrite both halves of its row buffer
            __threadfence();
            for (int p = 0; p < P.n_peers; ++p)
                st_tagged_sys_release(P.peer_left_out[p], 0.0f, epoch + static_cast<uint32_t>(seq_done));
            if (P.host_status) *P.host_status = *reinterpret_cast<volatile unsigned *>(err);
        }
    }
}

}  // namespace wd
