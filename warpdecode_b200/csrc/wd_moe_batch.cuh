// The MoE block for a batch of up to four tokens (speculative verify) as ONE pass over the layer.
//
// Reference: Qwen38MoeTokenBatch::run (src/qwen38_moe.cuh:2955-3107) runs M tokens x k experts as pairs
// p = t * k + j through one grouped launch per matrix (pair kernels :1317-1412); the caller is the MTP verify
// loop (src/qwen38_mtp.cuh:704-797). Here the whole batch is one cooperative launch:
//
//   front   every CTA quantises the T activations; the router rows and the shared expert's gate/up rows are
//           staged ONCE and applied to all T activations; the logits of all tokens travel together; T selections
//   tiles   the T * k pairs' gate/up tiles and then their down tiles form one task list per CTA that the
//           sixteen warps walk round-robin, one tile per task, through a ring of staging slots: the warp that
//           has consumed a slot asks for the tile `ring` tasks ahead at once, so copies, decoding and the
//           publication of results overlap without any block-wide synchronisation. A gate tile and its up tile
//           sit on neighbouring warps, which meet at a named barrier; the activations a CTA's down tiles need
//           are gathered (and quantised to Q8_K) by warps that have run out of gate/up tiles, and handed over
//           through mbarriers. Only the pairs at the end of the list wait for their activations: the exchange
//           latency of a layer is paid once per batch, not once per token.
//   combine every token's rows in its own rank order (pair (t, j) weighs with weights[t][j]), plus the shared expert
//
// Arithmetic is the single-token kernel's (same decoders, same quantisers, same router), so every token's ids,
// weights and output are bit-identical to a single-token call. Single GPU, every expert resident.
#pragma once

#include "wd_moe_kernel.cuh"

namespace wd {

constexpr int kMaxTokens = 4;
constexpr int kBatchMaxBars = 128;
constexpr int kBatchMaxRing = 48;

struct BatchParams {
    int H, F, SF, E, K, T;
    int nsb_h, nsb_f, t2_log2, t3_log2;
    float w_scale;
    const LayerDev *layers;
    int layer;
    const uint8_t *pool;
    unsigned long long slot_bytes;
    unsigned gate_off, up_off, down_off;
    const uint16_t *grid_packed, *grid2_packed;
    int gu_type, d_type;
    unsigned gu_tile, d_tile;
    int threshold_select;
    const float *x;              // [T][H]
    float *out;                  // [T][H]
    int *ids;                    // [T][K]
    float *weights;              // [T][K]
    float *routed;               // [H], of the last token
    // exchange words, written once per launch and told apart from earlier launches by the tag
    tagged_t *t_logits;          // [T][E]
    tagged_t *t_shact;           // [T][SF]
    tagged_t *t_shgate;          // [T]
    tagged_t *t_act;             // [T * K][F]
    tagged_t *t_eo;              // [T * K][H]
    tagged_t *t_shdown;          // [T][H]
    tagged_t *t_sel;             // [T][2 * kMaxK] picked ids (as bits), then weights
    unsigned *sync;              // the engine's status / epoch words (see MoeParams::sync)
    unsigned *host_status;
    unsigned *fallbacks;
    // Capped expert cache: when a picked expert has no slot the launch stops before any tile is touched (every CTA
    // sees the same picks and the same slot table, so all of them stop), miss_info[0] = 1, and the host places the
    // experts and launches again. miss_info (page-locked host memory, nullable): [0] missed, then the picks [T][K].
    int stop_on_miss;
    int *miss_info;
    unsigned long long *stamps;  // nullable: [cta][kStampStride] SM clock counter of thread 0 at the steps of the launch (profiling)
    // shared memory plan (byte offsets, 128-byte aligned)
    unsigned off_tab, off_tab2, off_tok, tok_stride, tok_xd0, tok_xk, tok_xdk, tok_shq, tok_shd, tok_sel;
    unsigned off_misc, off_scr, scr_bytes, scr_rows, off_bar, off_slots, off_seq, off_seg, off_tasks, off_pairbuf, off_actk,
        off_actd, off_ring, off_sd;
    unsigned ring, ring_slot;    // staging slots of the ring and bytes of one
    unsigned max_tasks;          // tile tasks of one CTA at most
    unsigned n1r, n1s, nsd, n_act;   // router tasks, shared gate/up tasks, shared-down tasks, activation superblocks per CTA (maxima)
};

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ int ld_acquire_shared(const int *p) {
    int v;
    asm volatile("ld.acquire.cta.shared.s32 %0, [%1];" : "=r"(v) : "r"(smem_u32(p)) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_shared(int *p, int v) {
    asm volatile("st.release.cta.shared.s32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}
// value t of a register array of kMaxTokens entries, without indexing it (which would move it to local memory)
__device__ __forceinline__ float pick4(const float (&a)[kMaxTokens], int t) {
    return t == 0 ? a[0] : t == 1 ? a[1] : t == 2 ? a[2] : a[3];
}

__global__ void __launch_bounds__(kThreads, 1) moe_batch_kernel(const __grid_constant__ BatchParams P) {
    uint8_t *sm = wd_smem;
    uint8_t *tab = sm + P.off_tab, *tab2 = sm + P.off_tab2;
    float *misc = reinterpret_cast<float *>(sm + P.off_misc);
    uint64_t *bars = reinterpret_cast<uint64_t *>(sm + P.off_bar);
    int *slot_tab = reinterpret_cast<int *>(sm + P.off_slots);
    int *ring_seq = reinterpret_cast<int *>(sm + P.off_seq);         // [ring] how often each slot has been asked for again
    float *pairbuf = reinterpret_cast<float *>(sm + P.off_pairbuf);  // [32][2][R] row sums of gate/up tile pairs in flight
    int *unit_cnt = reinterpret_cast<int *>(sm + P.off_seg) + 64;    // [32] halves of a pair that are done
    int *act_state = reinterpret_cast<int *>(sm + P.off_seg) + 96;   // [n_act] 0: nobody has asked for this superblock yet
    uint8_t *actk = sm + P.off_actk;
    float *actd = reinterpret_cast<float *>(sm + P.off_actd);
    uint8_t *ring = sm + P.off_ring;
    uint8_t *stage_sd = sm + P.off_sd;
    unsigned *err = P.sync + 2;
    uint32_t epoch;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(epoch) : "l"(P.sync + 8) : "memory");
    const uint32_t tag = epoch + 1u;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cta = blockIdx.x, ncta = gridDim.x;
    const int T = P.T;
    const int nbh = P.H >> 5, nbs = P.SF >> 5;
    const uint32_t lane4x2 = static_cast<uint32_t>(lane * 4) * 0x0101u;
    float *scr = reinterpret_cast<float *>(sm + P.off_scr + warp * P.scr_bytes);
    float *rows_a = scr + P.scr_rows;
    const LayerDev L = P.layers[P.layer];
#define WD_BSTAMP(i)                                                                   \
    if (P.stamps != nullptr && lane == 0) {                                            \
        unsigned long long c__;                                                        \
        asm volatile("mov.u64 %0, %%clock64;" : "=l"(c__) : : "memory");               \
        if (warp == 0) P.stamps[cta * kStampStride + (i)] = c__;                       \
        if (warp == kWarps - 1) P.stamps[cta * kStampStride + 16 + (i)] = c__;         \
    }
    WD_BSTAMP(0);

    // per-token regions
    auto tok_base = [&](int t) { return sm + P.off_tok + static_cast<size_t>(t) * P.tok_stride; };
    auto xq0_of = [&](int t) { return tok_base(t); };
    auto xd0_of = [&](int t) { return reinterpret_cast<float *>(tok_base(t) + P.tok_xd0); };
    auto xk_of = [&](int t) { return tok_base(t) + P.tok_xk; };
    auto xdk_of = [&](int t) { return reinterpret_cast<float *>(tok_base(t) + P.tok_xdk); };
    auto shq_of = [&](int t) { return tok_base(t) + P.tok_shq; };
    auto shd_of = [&](int t) { return reinterpret_cast<float *>(tok_base(t) + P.tok_shd); };
    auto ids_of = [&](int t) { return reinterpret_cast<int *>(tok_base(t) + P.tok_sel); };
    auto w_of = [&](int t) { return reinterpret_cast<float *>(tok_base(t) + P.tok_sel + kMaxK * 4); };

    // barriers: [0, ring) ring slots; then router tasks, shared gate/up tasks, slot table, gate vector, the activations,
    // shared-down tasks, the tokens' quantised shared activations, activation superblocks. Every one of them outside the ring completes at most once per launch.
    const int bar_rt = P.ring, bar_st = bar_rt + P.n1r, bar_tab = bar_st + P.n1s, bar_gv = bar_tab + 1, bar_x = bar_gv + 1,
              bar_sd = bar_x + 1, bar_shq = bar_sd + P.nsd, bar_act = bar_shq + kMaxTokens, n_bars = bar_act + P.n_act;
    if (tid < n_bars) {
        mbar_init(&bars[tid], 1);
        mbar_fence_init();
    }
    if (tid < static_cast<int>(P.ring)) ring_seq[tid] = 0;
    if (tid < 32) unit_cnt[tid] = 0;
    if (tid < static_cast<int>(P.n_act)) act_state[tid] = 0;
    if (cta == 0 && tid == 0) P.sync[5] = smem_u32(bars);
    const int u_tok = P.K << P.t2_log2, v_tok = P.K << P.t3_log2;      // gate/up units and down tiles of one token
    const int n_exp_tok = static_cast<int>(P.n_act) / (kMaxTokens * P.nsb_f);     // pairs a run may touch (planned maximum)
    // The tile tasks of a CTA form one list of segments: gate/up(token 0), gate/up(1), then for every token t
    // gate/up(t + 2) (while there is one) followed by down(t). The down tiles of a token thus come two segments after
    // its gate/up tiles, when the activations they need have long been published, and nobody waits for them.
    // Per token the gate/up units go round the CTAs (rotated by token, so that the odd units even out) and the down
    // tiles are cut into one contiguous run per CTA (a run needs the activations of one or two pairs only).
    int *seg_begin = reinterpret_cast<int *>(sm + P.off_seg);          // [2T + 1] first task of every segment
    int *seg_info = seg_begin + 9;                                     // [2T] token * 2 + (1: down tiles)
    int *tok_cta = seg_begin + 17, *tok_vb = seg_begin + 21, *tok_jl0 = seg_begin + 25, *tok_ng = seg_begin + 29;
    __syncthreads();
    if (tid == 32) {         // the list does not depend on the picks: laid out while the front's copies travel
        int c2[kMaxTokens], c3[kMaxTokens];
        for (int t = 0; t < T; ++t) {
            int ct = cta + t * (ncta / kMaxTokens);
            if (ct >= ncta) ct -= ncta;
            tok_cta[t] = ct;
            c2[t] = u_tok > ct ? (u_tok - ct + ncta - 1) / ncta : 0;
            const int vb = static_cast<int>(static_cast<unsigned>(ct) * static_cast<unsigned>(v_tok) / static_cast<unsigned>(ncta));
            const int ve = static_cast<int>(static_cast<unsigned>(ct + 1) * static_cast<unsigned>(v_tok) / static_cast<unsigned>(ncta));
            tok_vb[t] = vb;
            tok_jl0[t] = vb >> P.t3_log2;
            c3[t] = ve - vb;
            tok_ng[t] = ve > vb ? (((ve - 1) >> P.t3_log2) - (vb >> P.t3_log2) + 1) * P.nsb_f : 0;   // activation superblocks of the run
        }
        int at = 0, k = 0;
        auto add = [&](int t, int down) {
            seg_begin[k] = at;
            seg_info[k] = t * 2 + down;
            at += down ? c3[t] : 2 * c2[t];
            ++k;
        };
        add(0, 0);
        if (T > 1) add(1, 0);
        for (int t = 0; t < T; ++t) {
            if (t + 2 < T) add(t + 2, 0);
            add(t, 1);
        }
        seg_begin[k] = at;
    }
    // ---- the copies of the front (into the ring's memory): the T activations, the router tasks and shared gate/up
    // tasks of this CTA, the slot table, the shared gate vector (one CTA) ----
    const int n_rt = P.E >> 2, n_st = P.SF >> 2;
    const unsigned rt_bytes = static_cast<unsigned>(nbh) * 136u, a1_slot = 2u * rt_bytes;
    uint8_t *gate_vec_stage = ring + static_cast<size_t>(P.n1r + P.n1s) * a1_slot;
    const float *xs = reinterpret_cast<const float *>(gate_vec_stage + static_cast<size_t>(P.H) * 4);   // [T][H]
    if (warp == 0) {
        if (lane == 2) {
            const unsigned xb = static_cast<unsigned>(T) * static_cast<unsigned>(P.H) * 4u;
            mbar_expect_tx(&bars[bar_x], xb);
            bulk_load(const_cast<float *>(xs), P.x, xb, &bars[bar_x]);
        }
        for (int s = lane; s < static_cast<int>(P.n1r); s += 32) {
            const int t = cta + s * ncta;
            if (t < n_rt) {
                mbar_expect_tx(&bars[bar_rt + s], rt_bytes);
                bulk_load(ring + s * a1_slot, L.router_w + static_cast<size_t>(t) * rt_bytes, rt_bytes, &bars[bar_rt + s]);
            }
        }
        for (int s = lane; s < static_cast<int>(P.n1s); s += 32) {
            const int t = ncta - 1 - cta + s * ncta;
            if (t < n_st) {
                uint8_t *dst = ring + (P.n1r + s) * a1_slot;
                mbar_expect_tx(&bars[bar_st + s], 2u * rt_bytes);
                bulk_load(dst, L.sh_gate + static_cast<size_t>(t) * rt_bytes, rt_bytes, &bars[bar_st + s]);
                bulk_load(dst + rt_bytes, L.sh_up + static_cast<size_t>(t) * rt_bytes, rt_bytes, &bars[bar_st + s]);
            }
        }
        if (lane == 0) {
            mbar_expect_tx(&bars[bar_tab], static_cast<unsigned>(P.E) * 4u);
            bulk_load(slot_tab, L.slot_of_expert, static_cast<unsigned>(P.E) * 4u, &bars[bar_tab]);
        }
        if (lane == 1 && P.SF > 0 && cta == ncta / 2) {
            mbar_expect_tx(&bars[bar_gv], static_cast<unsigned>(P.H) * 4u);
            bulk_load(gate_vec_stage, L.sh_gate_vec, static_cast<unsigned>(P.H) * 4u, &bars[bar_gv]);
        }
    }
    if (P.gu_type == kTypeIq3s || P.d_type == kTypeIq3s) build_grid_table(tab, P.grid_packed);      // first needed by the tiles
    if (P.gu_type == kTypeIq2s || P.d_type == kTypeIq2s) build_iq2_table(tab2, P.grid2_packed);

    WD_BSTAMP(1);
    // ---- the T activations: Q8_0 (router, shared expert) and Q8_K (routed experts) ----------------------------
    mbar_wait(&bars[bar_x], 0, err);
    if ((tid >> 7) < T)     // 128 threads per token
        quantize_q8_0_part(xs + static_cast<size_t>(tid >> 7) * P.H, P.H, xq0_of(tid >> 7), xd0_of(tid >> 7), tid & 127, 128);
#pragma unroll 1
    for (int w = warp; w < T * P.nsb_h; w += kWarps) {
        const int t = w / P.nsb_h, sb = w - t * P.nsb_h;
        quantize_q8_K_warp(xs + static_cast<size_t>(t) * P.H + sb * 256, lane, xk_of(t) + sb * kActSbStride, &xdk_of(t)[sb]);
    }
    __syncthreads();

    WD_BSTAMP(2);
    // ---- row tasks: every staged row task meets all T activations, one warp per (task, token) ------------------
    {
        const int my_rt = cta < n_rt ? (n_rt - cta + ncta - 1) / ncta : 0;
        const int first_st = ncta - 1 - cta;
        const int my_st = first_st < n_st ? (n_st - first_st + ncta - 1) / ncta : 0;
#pragma unroll 1
        for (int it = warp; it < (my_rt + my_st) * T; it += kWarps) {
            const int lt = it / T, t = it - lt * T;
            if (lt < my_rt) {
                const int row = (cta + lt * ncta) * 4 + (lane >> 3);
                mbar_wait(&bars[bar_rt + lt], 0, err);
                float v = q8_task_row(ring + lt * a1_slot, nbh, xq0_of(t), xd0_of(t), lane);
                if ((lane & 7) == 0) {
                    if (L.router_bias) v = __fadd_rn(v, L.router_bias[row]);
                    st_tagged(P.t_logits + static_cast<size_t>(t) * P.E + row, v, tag);
                }
            } else {
                const int ls = lt - my_rt;
                const int row = (first_st + ls * ncta) * 4 + (lane >> 3);
                mbar_wait(&bars[bar_st + ls], 0, err);
                const uint8_t *base = ring + (P.n1r + ls) * a1_slot;
                float g, u;
                q8_task_row2(base, base + rt_bytes, nbh, xq0_of(t), xd0_of(t), lane, g, u);
                if ((lane & 7) == 0) st_tagged(P.t_shact + static_cast<size_t>(t) * P.SF + row, __fmul_rn(silu_ggml(g), u), tag);
            }
        }
        if (P.SF > 0 && cta == ncta / 2 && warp >= kWarps - T) {         // one warp per token: the shared gate scalar
            const int t = kWarps - 1 - warp;
            mbar_wait(&bars[bar_gv], 0, err);
            const float d = dot_f32_warp(reinterpret_cast<const float *>(gate_vec_stage), xs + static_cast<size_t>(t) * P.H, P.H, lane);
            if (lane == 0) st_tagged(P.t_shgate + t, sigmoid_ggml(d), tag);
        }
    }

    WD_BSTAMP(3);
    __syncthreads();        // the staged rows are not read any more: their memory becomes the ring
    WD_BSTAMP(4);

    // ---- the selections: CTA t picks token t's experts (the whole CTA, as in the single-token kernel) and publishes
    // ids and weights; every CTA then gathers the picks of all tokens ----
    {
        if (cta < T) {
            const bool h0 = tid < P.E, h1 = tid + kThreads < P.E;
            float lg[2];
            wait_tagged<2>(P.t_logits + static_cast<size_t>(cta) * P.E + tid, kThreads, (h0 ? 1 : 0) + (h1 ? 1 : 0), tag, lg, err);
            const float l0 = lg[0], l1 = lg[1];
            RouterScratch rs;
            rs.probs = nullptr;
            rs.gsum = misc + kMiscGsum;
            rs.red = misc + kMiscRed;
            rs.first = misc + kMiscTop;
            rs.cand = reinterpret_cast<uint32_t *>(misc + kMiscProbs);
            int *sel_ids = ids_of(cta);
            float *sel_w = w_of(cta);
            if (P.threshold_select) {
                ThresholdScratch ts;
                ts.gm = reinterpret_cast<uint32_t *>(misc);
                ts.cnt = reinterpret_cast<int *>(misc + 16);
                ts.selmask = reinterpret_cast<uint32_t *>(misc + 32);
                ts.sel_keys = reinterpret_cast<uint32_t *>(misc + 64);
                ts.cand = reinterpret_cast<uint2 *>(misc + 128);
                const uint32_t key0 = h0 ? order_key(l0) : 0u, key1 = h1 ? order_key(l1) : 0u;
                router_threshold_stage_a(key0, key1, P.E, ts);
                __syncthreads();
                bool slow = router_threshold_stage_b(key0, key1, h0, h1, P.K, ts);
                __syncthreads();
                const int nc = *ts.cnt;
                slow = slow || nc > 32 || nc < P.K;
                if (!slow && warp == 0) router_threshold_rank_warp(nc, P.K, ts, sel_ids, lane);
                __syncthreads();
                float p0, p1;
                const bool ok = router_threshold_proof(l0, l1, h0, h1, P.E, P.K, P.w_scale, slow, ts, rs, sel_ids, sel_w, p0, p1);
                if (!ok) {
                    router_rungs_cta(p0, p1, P.E, P.K, P.w_scale, rs, sel_ids, sel_w);
                    if (tid == 0 && P.fallbacks != nullptr) atomicAdd(P.fallbacks, 1u);
                }
            } else {
                router_select_cta(l0, l1, P.E, P.K, P.w_scale, rs, sel_ids, sel_w);
            }
            if (tid < P.K) {
                st_tagged(P.t_sel + cta * 2 * kMaxK + tid, __int_as_float(sel_ids[tid]), tag);
                st_tagged(P.t_sel + cta * 2 * kMaxK + kMaxK + tid, sel_w[tid], tag);
            }
            __syncthreads();
        }
    }
    int n_tiles = seg_begin[2 * T];
    const int n_sd = P.SF > 0 ? (P.H >> 2) : 0;
    int my_sd = n_sd > cta ? (n_sd - cta + ncta - 1) / ncta : 0;
    bool stopped = false;
    const unsigned sd_bytes = static_cast<unsigned>(nbs) * 136u;
    const int ns = static_cast<int>(P.ring);
    const int act_per_tok = n_exp_tok * P.nsb_f;
    // Every task's description, worked out once (the walk further down runs while the integer pipes are saturated by
    // the decoders, so it must be short), here while the picks travel: the offset of its tile inside an expert's
    // slot (the slot's address is added once the picks are known), and
    //   desc: bit 0 down tile, 1-2 token, 3-8 pair, 9-20 tile inside the pair's matrix, 21 up tile (else gate),
    //         22-27 one more than the activation superblock this task's warp gathers afterwards (0: none)
    //   aux : gate/up tile: entry of the pair buffer; down tile: first activation superblock of its pair
    unsigned long long *task_src = reinterpret_cast<unsigned long long *>(sm + P.off_tasks);
    uint32_t *task_desc = reinterpret_cast<uint32_t *>(task_src + P.max_tasks);
    int *task_aux = reinterpret_cast<int *>(task_desc + P.max_tasks);
#pragma unroll 1
    for (int i = tid; i < n_tiles; i += kThreads) {
        int k = 0;
        while (k + 1 < 2 * T && i >= seg_begin[k + 1]) ++k;
        const int t = seg_info[k] >> 1, down = seg_info[k] & 1, li = i - seg_begin[k];
        uint32_t d;
        unsigned long long src;
        int aux;
        if (!down) {
            const int u = tok_cta[t] + (li >> 1) * ncta;
            const int pair = t * P.K + (u >> P.t2_log2), tile = u & ((1 << P.t2_log2) - 1);
            src = ((li & 1) ? P.up_off : P.gate_off) + static_cast<unsigned long long>(tile) * P.gu_tile;
            d = static_cast<uint32_t>(t << 1) | static_cast<uint32_t>(pair << 3) | static_cast<uint32_t>(tile << 9) |
                static_cast<uint32_t>((li & 1) << 21);
            aux = ((i - (li & 1)) >> 1) & 31;
        } else {
            const int v = tok_vb[t] + li;
            const int pl = v >> P.t3_log2, tile = v & ((1 << P.t3_log2) - 1);
            const int pair = t * P.K + pl;
            src = P.down_off + static_cast<unsigned long long>(tile) * P.d_tile;
            d = 1u | static_cast<uint32_t>(t << 1) | static_cast<uint32_t>(pair << 3) | static_cast<uint32_t>(tile << 9);
            aux = t * act_per_tok + (pl - tok_jl0[t]) * P.nsb_f;
        }
        // the gathers of a down segment are handed to the tasks that end a round (16 tasks) before it starts
#pragma unroll 1
        for (int kd = 0; kd < 2 * T; ++kd) {
            if (!(seg_info[kd] & 1)) continue;
            const int td = seg_info[kd] >> 1;
            const int base = max(0, seg_begin[kd] - kWarps - tok_ng[td]);
            // at most one per task (short segments overlap); a gather nobody was handed is done by the first tile that needs it
            if (i >= base && i < base + tok_ng[td] && (d >> 22) == 0u) d |= static_cast<uint32_t>(td * act_per_tok + (i - base) + 1) << 22;
        }
        task_src[i] = src;
        task_desc[i] = d;
        task_aux[i] = aux;
    }
    {
        if (tid < T * 2 * kMaxK) {
            const int t = tid / (2 * kMaxK), j = tid - t * 2 * kMaxK;
            if ((j & (kMaxK - 1)) < P.K) {
                float v[1];
                wait_tagged<1>(P.t_sel + tid, 1, 1, tag, v, err);
                if (j < kMaxK) {
                    ids_of(t)[j] = __float_as_int(v[0]);
                    if (cta == 0) P.ids[t * P.K + j] = __float_as_int(v[0]);
                } else {
                    w_of(t)[j - kMaxK] = v[0];
                    if (cta == 0) P.weights[t * P.K + j - kMaxK] = v[0];
                }
            }
        }
        mbar_wait(&bars[bar_tab], 0, err);
        __syncthreads();
        if (P.miss_info != nullptr) {
            int miss = 0, e = 0;
            if (tid < T * P.K) {
                e = ids_of(tid / P.K)[tid % P.K];
                miss = slot_tab[e] < 0;
            }
            miss = __syncthreads_or(miss);
            if (cta == 0) {
                if (tid < T * P.K) P.miss_info[1 + tid] = e;
                if (tid == 0) P.miss_info[0] = miss ? 1 : 0;
            }
            if (miss && P.stop_on_miss) {       // nothing of the tile phase runs; the front's copies have all been waited for
                stopped = true;
                n_tiles = 0;
                my_sd = 0;
            }
        }
        // the picked experts' slots complete the tile addresses
#pragma unroll 1
        for (int i = tid; i < n_tiles; i += kThreads) {
            const int pair = static_cast<int>((task_desc[i] >> 3) & 63u), t = static_cast<int>((task_desc[i] >> 1) & 3u);
            int slot = slot_tab[ids_of(t)[pair - t * P.K]];
            if (slot < 0) {
                atomicOr(err, kErrExpertMiss);
                slot = 0;
            }
            task_src[i] += reinterpret_cast<unsigned long long>(P.pool) + static_cast<unsigned long long>(slot) * P.slot_bytes;
        }
    }

    WD_BSTAMP(5);
    // ---- the tile tasks of this CTA ---------------------------------------------------------------------------
    // A warp walks its tasks i = warp, warp + 16, ...; task i sits in slot i % ring during round i / ring of that slot.
    // A consumed slot is asked for again by lane 0 of the warp that read it; the count of requests tells a warp that
    // is ahead of that one which phase of the slot's barrier it may wait for.
    auto issue = [&](int i, int slot) {
        const unsigned bytes = (task_desc[i] & 1u) ? P.d_tile : P.gu_tile;
        mbar_expect_tx(&bars[slot], bytes);
        bulk_load(ring + static_cast<size_t>(slot) * P.ring_slot, reinterpret_cast<const void *>(task_src[i]), bytes, &bars[slot]);
    };
    int i = warp, slot = warp, round = 0;
    auto reissue = [&]() {
        __syncwarp();
        if (lane == 0 && i + ns < n_tiles) {
            issue(i + ns, slot);
            st_release_shared(&ring_seq[slot], round + 1);
        }
    };
    auto wait_slot = [&]() {
        if (round > 0) {
            unsigned long long t0 = 0ull;
            for (unsigned it = 0; ld_acquire_shared(&ring_seq[slot]) < round; ++it)
                if (wait_expired(it, t0, err)) break;
        }
        mbar_wait(&bars[slot], static_cast<uint32_t>(round & 1), err);
    };
    // activation superblock g (token g / act_per_tok, then pair of the run, then superblock): whoever asks first polls
    // the published values, quantises them to Q8_K and opens the superblock's barrier
    auto gather = [&](int g) {
        int won = 0;
        if (lane == 0) won = atom_cas_shared(&act_state[g], 0, 1) == 0;
        won = __shfl_sync(0xffffffffu, won, 0);
        if (!won) return;
        const int t = g / act_per_tok, r = g - t * act_per_tok;
        const int pl = r / P.nsb_f, sbk = r - pl * P.nsb_f;
        float av[8];
        wait_tagged<8>(P.t_act + static_cast<size_t>(t * P.K + tok_jl0[t] + pl) * P.F + sbk * 256 + lane, 32, 8, tag, av, err);
#pragma unroll
        for (int k = 0; k < 8; ++k) scr[lane + 32 * k] = av[k];
        __syncwarp();
        quantize_q8_K_warp(scr, lane, actk + g * kActSbStride, &actd[g]);
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[bar_act + g]);
    };
    fence_proxy_async();
    __syncthreads();
    if (tid < min(ns, n_tiles)) issue(tid, tid);
    if (tid >= 64 && tid < 64 + my_sd) {
        const int k = tid - 64;
        mbar_expect_tx(&bars[bar_sd + k], sd_bytes);
        bulk_load(stage_sd + k * sd_bytes, L.sh_down + static_cast<size_t>(cta + k * ncta) * sd_bytes, sd_bytes, &bars[bar_sd + k]);
    }

    WD_BSTAMP(6);
    // The shared expert's activation of token t (published by the row tasks long ago) -> Q8_0, by warp 15 - t while the
    // first tiles are on their way; the floats pass through the memory of the token's Q8_0 quants of x, which only
    // the row tasks read. The shared-down tasks at the end of the list wait on the token's barrier.
    if (P.SF > 0 && warp >= kWarps - T) {
        const int t = kWarps - 1 - warp;
        float *sf = reinterpret_cast<float *>(xq0_of(t));
#pragma unroll 1
        for (int base = 0; base < P.SF; base += 256) {
            float v[8];
            wait_tagged<8>(P.t_shact + static_cast<size_t>(t) * P.SF + base + lane, 32, min(8, (P.SF - base) >> 5), tag, v, err);
#pragma unroll
            for (int k = 0; k < 8; ++k)
                if (base + 32 * k < P.SF) sf[base + lane + 32 * k] = v[k];
        }
        __syncwarp();
        quantize_q8_0_part(sf, P.SF, shq_of(t), shd_of(t), lane, 32);
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[bar_shq + t]);
    }
    {
        const int R2 = 32 / P.nsb_h, R3 = 32 / P.nsb_f;
        const int sb2 = lane % P.nsb_h, sb3 = lane % P.nsb_f;
#pragma unroll 1
        for (; i < n_tiles; i += kWarps, slot += kWarps) {
            if (slot >= ns) {
                slot -= ns;
                ++round;
            }
            const uint32_t d = task_desc[i];
            const int aux = task_aux[i];
            const int t = (d >> 1) & 3, pair = (d >> 3) & 63, tile = (d >> 9) & 4095;
            const uint8_t *tile_mem = ring + static_cast<size_t>(slot) * P.ring_slot;
            if (!(d & 1u)) {
                // a gate tile or its up tile: row sums into the pair's buffer; whichever of the two warps finishes second
                // forms SiLU(g) * u and publishes the rows
                const int up = (d >> 21) & 1;
                float *buf = pairbuf + aux * 2 * R2;
                wait_slot();
                iq_tile_to_rows_any<8>(P.gu_type, tile_mem, xk_of(t) + sb2 * kActSbStride, xdk_of(t)[sb2], P.nsb_h, lane, lane4x2, tab,
                                    tab2, scr, buf + up * R2, nullptr);
                reissue();
                int second = 0;
                if (lane == 0) {
                    second = atom_add_shared_acq_rel(&unit_cnt[aux], 1);
                    if (second) unit_cnt[aux] = 0;
                }
                second = __shfl_sync(0xffffffffu, second, 0);
                __syncwarp();       // orders the other lanes' reads of the buffer after lane 0's acquire
                if (second && lane < R2)
                    st_tagged(P.t_act + static_cast<size_t>(pair) * P.F + tile * R2 + lane, __fmul_rn(silu_ggml(buf[lane]), buf[R2 + lane]), tag);
            } else {
                // the pair's activations: normally gathered a round ago; else the first warp to need a superblock does it
#pragma unroll 1
                for (int sk = 0; sk < P.nsb_f; ++sk) {
                    if (!mbar_try_wait(&bars[bar_act + aux + sk], 0)) {
                        gather(aux + sk);
                        mbar_wait(&bars[bar_act + aux + sk], 0, err);
                    }
                }
                const int ab = aux + sb3;
                wait_slot();
                iq_tile_to_rows_any<8>(P.d_type, tile_mem, actk + ab * kActSbStride, actd[ab], P.nsb_f, lane, lane4x2, tab, tab2, scr,
                                    rows_a, nullptr);
                reissue();
#pragma unroll 1
                for (int rr = lane; rr < R3; rr += 32)
                    st_tagged(P.t_eo + static_cast<size_t>(pair) * P.H + tile * R3 + rr, rows_a[rr], tag);
                __syncwarp();
            }
            const int job = static_cast<int>((d >> 22) & 63u);
            if (job) gather(job - 1);
        }
    }
    WD_BSTAMP(9);
    // shared-expert down rows, on the warps that come next in the round
#pragma unroll 1
    for (int k = (warp - n_tiles % kWarps + kWarps) % kWarps; k < my_sd; k += kWarps) {
        const int row = (cta + k * ncta) * 4 + (lane >> 3);
        mbar_wait(&bars[bar_sd + k], 0, err);
#pragma unroll 1
        for (int t = 0; t < T; ++t) {
            mbar_wait(&bars[bar_shq + t], 0, err);
            const float d = q8_task_row(stage_sd + k * sd_bytes, nbs, shq_of(t), shd_of(t), lane);
            if ((lane & 7) == 0) st_tagged(P.t_shdown + static_cast<size_t>(t) * P.H + row, d, tag);
        }
    }

    WD_BSTAMP(10);
    // ---- combine: this CTA's band of output rows, for every token ----------------------------------------------
    {
        const int rpc = (P.H + ncta - 1) / ncta;
        const int t = tid / rpc, r = tid - t * rpc;
        const int row = cta * rpc + r;
        if (t < T && row < P.H && !stopped) {
            const float *sel_w = w_of(t);
            tagged_t w[kMaxK] = {}, wsd = 0, wsg = 0;
            const tagged_t *src = P.t_eo + static_cast<size_t>(t) * P.K * P.H + row;
            unsigned long long t0 = 0ull;
            for (unsigned it = 0;; ++it) {
#pragma unroll
                for (int q = 0; q < kMaxK; ++q)
                    if (q < P.K) w[q] = ld_tagged(src + static_cast<size_t>(q) * P.H);
                if (P.SF > 0) {
                    wsd = ld_tagged(P.t_shdown + static_cast<size_t>(t) * P.H + row);
                    wsg = ld_tagged(P.t_shgate + t);
                }
                unsigned bad = (P.SF > 0) & (tag_behind(wsd, tag) | tag_behind(wsg, tag));
#pragma unroll
                for (int q = 0; q < kMaxK; ++q) bad |= (q < P.K) & tag_behind(w[q], tag);
                if (!bad) break;
                if (wait_expired(it, t0, err)) break;
            }
            float acc = 0.0f;
#pragma unroll
            for (int q = 0; q < kMaxK; ++q)
                if (q < P.K) acc = __fadd_rn(acc, __fmul_rn(__uint_as_float(static_cast<uint32_t>(w[q])), sel_w[q]));
            if (t == T - 1) P.routed[row] = acc;
            float o = acc;
            if (P.SF > 0) o = __fadd_rn(acc, __fmul_rn(__uint_as_float(static_cast<uint32_t>(wsd)), __uint_as_float(static_cast<uint32_t>(wsg))));
            P.out[static_cast<size_t>(t) * P.H + row] = o;
        }
    }
    WD_BSTAMP(11);
    __syncthreads();
    WD_BSTAMP(12);
#undef WD_BSTAMP
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(P.sync + 9, 1u) == static_cast<unsigned>(ncta) - 1u) {
            P.sync[9] = 0u;
            P.sync[8] = epoch + 1u;
            __threadfence();
            if (P.host_status) *P.host_status = *reinterpret_cast<volatile unsigned *>(err);
        }
    }
}

}  // namespace wd
