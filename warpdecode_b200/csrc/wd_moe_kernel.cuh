// The fused MoE layer kernel: one persistent cooperative launch per layer (batch 1).
//
//   phase 0  every CTA: x (optionally RMSNorm(residual) * w) -> Q8_0 and Q8_K blocks in shared memory
//   phase 1  Q8_0 row tasks spread over the grid: router logits, shared-expert gate/up + SiLU,
//            shared gate scalar                                        -> grid barrier
//   phase 1b every CTA: softmax / top-k (whole CTA), shared activation -> Q8_0; then ALL bulk copies of
//            this CTA's share of the selected experts' gate/up/down tiles are issued at once
//   phase 2  gate+up tiles -> SiLU(g)*u per expert row (+ running max per superblock);
//            shared-expert down rows on the warps that have no tile      -> grid barrier
//   phase 3  expert activations -> Q8_K; down tiles; the warp that delivers the last contribution
//            of an output tile performs the ordered combine and the finish
//
// Reference call sites this replaces: q38_moe_select_experts_f32_x (src/qwen38_moe.cuh:2323),
// q38_moe_run_batched_experts (:3312, five launches), run_qwen38_shared_expert_f32_x (:3963, nine
// launches), q38_finish_moe_f32 (:2442) and the per-layer ids D2H + stream sync (:2363-2379).
#pragma once

#include "wd_router.cuh"

namespace wd {

constexpr int kMaxBars = 96;

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
    // layers [layer_begin, layer_end) run back to back inside one launch (a grid barrier between them),
    // so that after the first layer every instruction comes from the instruction cache
    const LayerDev *layers;      // device array, one entry per layer of the stack
    int layer_begin, layer_end;
    int stamp_layer;             // the layer whose phase timestamps are recorded
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
    unsigned *act_amax;          // [K][nsb_f] bit pattern of max |act| per superblock
    float *expert_out;           // [K][H]
    float *routed;               // [H]
    float *shared_act;           // [SF]
    float *shared_down;          // [H]
    float *shared_gate;          // [1]
    unsigned long long *stamps;  // nullable: [cta][16] globaltimer values at phase boundaries (profiling)
    unsigned long long *barrier; // grid barrier counter (only ever grows)
    unsigned long long barrier_base;   // its value when this launch starts
    unsigned *sync;              // [2] error word, [16..] output-tile counters
    // shared memory plan (byte offsets from the dynamic shared base; all 128-byte aligned)
    unsigned off_tab, off_xq0, off_xd0, off_xk, off_xdk, off_actk, off_actd, off_shq, off_shd,
        off_misc, off_scr, off_bar, off_stage_a, off_stage_b;
    unsigned scr_bytes;          // per-warp transposition scratch
    unsigned scr_rows;           // float offset of the two 32-float row buffers inside it
    unsigned n1r, n1s, n2, n3, nsd;   // staging slots per CTA: router tasks, shared g/u tasks, phase-2 units,
                                      // phase-3 tiles, shared-down tasks
};

// float offsets inside the `misc` region once phase 1 is over (before that it holds x as floats)
constexpr int kMiscLogits = 0, kMiscProbs = 1024, kMiscGsum = 2048, kMiscRed = 2176, kMiscTop = 2192,
              kMiscChamp = 2208, kMiscDsum = 2272, kMiscIds = 2288, kMiscW = 2304, kMiscLocJ = 2320,
              kMiscLocSlot = 2336, kMiscLocN = 2352, kMiscSlots = 2368, kMiscSharedAct = 2400;

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
    float *misc = reinterpret_cast<float *>(sm + P.off_misc);
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
    float *rows_a = scr + P.scr_rows, *rows_b = rows_a + 32;       // per-warp row results of a tile

    float *xf = misc;                                               // [H], phases 0 and 1 only
    int *sel_ids = reinterpret_cast<int *>(misc + kMiscIds);
    float *sel_w = misc + kMiscW;
    int *loc_j = reinterpret_cast<int *>(misc + kMiscLocJ);         // rank-order index of each owned selected expert
    int *loc_slot = reinterpret_cast<int *>(misc + kMiscLocSlot);
    int *loc_n = reinterpret_cast<int *>(misc + kMiscLocN);

#define WD_STAMP(i)                                                                            \
    if (stamp_on) {                                                                            \
        unsigned long long t__;                                                                \
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__));                                \
        P.stamps[cta * 16 + (i)] = t__;                                                        \
    }
    const int n_bars = P.n1r + P.n1s + P.n2 + P.n3 + P.nsd;
    if (tid < n_bars) {
        mbar_init(&bars[tid], 1);
        mbar_fence_init();
    }
    build_grid_table(tab, P.grid_packed);          // first needed in phase 2
    __syncthreads();
    unsigned long long bar_target = P.barrier_base;

#pragma unroll 1
    for (int layer = P.layer_begin; layer < P.layer_end; ++layer) {
    const LayerDev L = P.layers[layer];
    const uint32_t par = static_cast<uint32_t>(layer - P.layer_begin) & 1u;   // every mbarrier completes once per layer
    const bool stamp_on = P.stamps != nullptr && tid == 0 && layer == P.stamp_layer;
    WD_STAMP(0);
    if (cta == 0 && tid < P.K * P.nsb_f) P.act_amax[tid] = 0u;

    // ---- issue phase-1 copies: router tasks and shared gate/up tasks of this CTA --------------
    const int n_rt = P.E >> 2;                     // router tasks (4 rows each)
    const int n_st = P.SF >> 2;                    // shared gate/up tasks (4 row pairs each)
    const unsigned rt_bytes = static_cast<unsigned>(nbh) * 136u;
    const unsigned a1_slot = 2u * rt_bytes;        // staging slot of phase 1
    if (tid == 0) {
        fence_proxy_async();        // the staging buffers were last read by ordinary loads (previous layer)
        int s = 0;
        for (int t = cta; t < n_rt; t += ncta, ++s) {
            mbar_expect_tx(&bars[s], rt_bytes);
            bulk_load(stage_a + s * a1_slot, L.router_w + static_cast<size_t>(t) * rt_bytes, rt_bytes, &bars[s]);
        }
        s = P.n1r;
        for (int t = ncta - 1 - cta; t < n_st; t += ncta, ++s) {
            mbar_expect_tx(&bars[s], 2u * rt_bytes);
            bulk_load(stage_a + s * a1_slot, L.sh_gate + static_cast<size_t>(t) * rt_bytes, rt_bytes, &bars[s]);
            bulk_load(stage_a + s * a1_slot + rt_bytes, L.sh_up + static_cast<size_t>(t) * rt_bytes, rt_bytes, &bars[s]);
        }
    }
    WD_STAMP(1);

    // ---- phase 0: x -> shared (with the optional RMSNorm prologue), then both quantisations --
    if (P.residual != nullptr) {
        // sum of squares as a perfect binary tree over consecutive elements, in double
        const int epl = P.H >= kThreads ? P.H / kThreads : 1;
        double ss = 0.0;
        float rv[16];
        if (tid * epl < P.H) {
            double loc[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                rv[i] = i < epl ? P.residual[tid * epl + i] : 0.0f;
                loc[i] = __dmul_rn(static_cast<double>(rv[i]), static_cast<double>(rv[i]));
            }
#pragma unroll
            for (int w = 1; w < 16; w <<= 1)
#pragma unroll
                for (int i = 0; i + w < 16; i += 2 * w) loc[i] = __dadd_rn(loc[i], loc[i + w]);
            ss = loc[0];
        }
#pragma unroll
        for (int s = 1; s < 32; s <<= 1) ss = __dadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, s));
        double *redd = reinterpret_cast<double *>(sm + P.off_scr);
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
        if (tid * epl < P.H) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                if (i < epl) {
                    float v = __fmul_rn(rv[i], scale);
                    if (L.norm_w) v = __fmul_rn(v, L.norm_w[tid * epl + i]);
                    xf[tid * epl + i] = v;
                }
            }
        }
    } else {
        for (int i = tid; i < P.H; i += kThreads) xf[i] = P.x[i];
    }
    // the one CTA that computes the shared gate scalar brings the gate vector in with one round trip
    float *gate_vec_s = reinterpret_cast<float *>(stage_b);
    if (P.SF > 0 && cta == ncta / 2)
        for (int i = tid; i < P.H; i += kThreads) gate_vec_s[i] = L.sh_gate_vec[i];
    __syncthreads();
    quantize_q8_0_cta(xf, P.H, xq0, xd0);
    for (int sb = warp; sb < P.nsb_h; sb += kWarps)
        quantize_q8_K_warp(xf + sb * 256, lane, xk + sb * kActSbStride, &xdk[sb]);
    __syncthreads();
    WD_STAMP(2);

#include "wd_moe_kernel_phases.inc"

    WD_STAMP(10);
    // the next layer reads the residual and reuses every shared and global scratch buffer
    if (layer + 1 < P.layer_end) grid_barrier(P.barrier, bar_target += ncta, err);
    }   // layers
#undef WD_STAMP
}

}  // namespace wd
