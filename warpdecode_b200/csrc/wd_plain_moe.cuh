// The MoE block on tensors that stay in ggml block layout: the path for geometries the tiled kernels do not take.
//
// The tiled kernels (wd_moe_kernel.cuh, wd_moe_batch.cuh) want a power-of-two number of superblocks per row and
// IQ3_S / IQ2_S tensors throughout. The reference's own model has hidden 2560 (ten superblocks), expert_ffn 640,
// IQ4_NL down tensors fed by a Q8_0 activation, and an F32 router (src/qwen38_moe.cuh:2181-2211, :2252-2258). Here
// every row product is one warp (IQ4_NL: half a warp) reading the ggml blocks where they lie, so any hidden that is a
// multiple of 256 and any expert_ffn that is a multiple of 64 runs. The arithmetic contract is the same as everywhere
// else in this library: integer sums per (superblock or block, chunk-lane), one fmaf per block and chunk-lane in
// block order, ggml's 8-lane closing tree (src/qwen38_cpu_moe.cuh:290-440).
//
// One call is seven small kernels on the caller's stream (quantise, router + shared gate/up rows, selection, expert
// gate/up rows, activation quantiser, down rows, ordered combine); blockIdx.y is the token of a verify batch.
#pragma once

#include "wd_blocks.cuh"
#include "wd_router.cuh"

namespace wd {

constexpr int kTypeIq4nl = 20;

struct PlainParams {
    int H, F, SF, E, K;
    int gate_type, up_type, down_type;      // ggml ids: IQ3_S / IQ2_S; down also IQ4_NL
    float w_scale;
    // weights of the layer
    const uint8_t *router_tasks;            // Q8_0 in 4-row tasks (wd_formats.cuh), or null when
    const float *router_f32;                // the router is F32 [E][H]
    const float *bias, *gate_vec;
    const uint8_t *sh_gate, *sh_up, *sh_down;       // Q8_0 tasks
    const uint8_t *gate, *up, *down;                // ggml layout, experts contiguous
    const uint16_t *grid3, *grid2;                  // packed codebooks (wd_grids.h)
    // activations and scratch, all [token][...]
    const float *x;
    float *out;
    uint8_t *xq0;       // Q8_0 of x in task layout [H]
    float *xd0;         // [H / 32]
    int8_t *xk;         // Q8_K of x [H]
    float *xdk;         // [H / 256]
    float *logits, *probs, *weights;
    int *ids;
    float *shact;       // [SF]
    uint8_t *shq0;      // its Q8_0, task layout
    float *shd0;
    float *sgate;       // [1]
    float *act;         // [K][F]
    int8_t *actq;       // [K][F] quants of act (Q8_0 blocks of 32 or Q8_K superblocks of 256)
    float *actd;        // [K][F / 32]
    float *eo;          // [K][H]
    float *shdown;      // [H]
    float *routed;      // [H]
};

// 0xff in byte j where bit j of the nibble is set
__device__ __forceinline__ uint32_t nibble_to_byte_mask(uint32_t nib) {
    return ((nib * 0x00204081u) & 0x01010101u) * 0xffu;
}

// four magnitudes (each >= 1) with the signs of a nibble applied, as packed int8
__device__ __forceinline__ int apply_signs(uint32_t mags, uint32_t nib) {
    const uint32_t m = nibble_to_byte_mask(nib);
    const uint32_t neg = 0x01010100u - mags;            // per-byte two's complement
    return static_cast<int>((mags & ~m) | (neg & m));
}

// The closing tree when lane p (0..3) holds chunk-lanes 2p (even) and 2p + 1 (odd): (v0+v4, v1+v5, v2+v6, v3+v7),
// then (r0 + r2) + (r1 + r3) (src/qwen38_cpu_moe.cuh:290-296).
__device__ __forceinline__ float hsum8_pairs(float even, float odd) {
    even = __fadd_rn(even, __shfl_xor_sync(0xffffffffu, even, 2));
    odd = __fadd_rn(odd, __shfl_xor_sync(0xffffffffu, odd, 2));
    even = __fadd_rn(even, __shfl_xor_sync(0xffffffffu, even, 1));
    odd = __fadd_rn(odd, __shfl_xor_sync(0xffffffffu, odd, 1));
    return __fadd_rn(even, odd);
}

__device__ __forceinline__ int sum_over_subblocks(int v) {
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    v += __shfl_xor_sync(0xffffffffu, v, 8);
    v += __shfl_xor_sync(0xffffffffu, v, 16);
    return v;
}

// One IQ3_S row (ggml blocks: d(2) qs(64) qh(8) signs(32) scales(4)) against a Q8_K activation, by one warp.
// Lane = (sub-block ib = lane / 4, pair p = lane % 4) takes chunk-lanes 2p and 2p + 1 of sub-block ib of every
// superblock; the integer sums over the eight sub-blocks meet by shuffles (src/qwen38_cpu_moe.cuh:337-375).
__device__ __forceinline__ float plain_row_iq3s(const uint8_t *row, int nsb, const int8_t *a, const float *da,
                                                const uint16_t *grid, int lane) {
    const int ib = lane >> 2, p = lane & 3;
    float even = 0.0f, odd = 0.0f;
#pragma unroll 2
    for (int sb = 0; sb < nsb; ++sb) {
        const uint8_t *blk = row + sb * 110;
        const uint32_t q2 = *reinterpret_cast<const uint16_t *>(blk + 2 + ib * 8 + 2 * p);
        const uint32_t h = blk[66 + ib] >> (2 * p);
        const uint32_t sg = blk[74 + ib * 4 + p];
        const uint32_t scb = blk[106 + (ib >> 1)];
        const int ls = 1 + 2 * static_cast<int>((ib & 1) ? (scb >> 4) : (scb & 15u));
        const int2 av = *reinterpret_cast<const int2 *>(a + sb * 256 + ib * 32 + p * 8);
        const uint32_t p0 = grid[(q2 & 0xffu) | ((h & 1u) << 8)], p1 = grid[(q2 >> 8) | ((h & 2u) << 7)];
        uint32_t g0 = 0, g1 = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            g0 |= (2u * ((p0 >> (3 * j)) & 7u) + 1u) << (8 * j);
            g1 |= (2u * ((p1 >> (3 * j)) & 7u) + 1u) << (8 * j);
        }
        const int s0 = sum_over_subblocks(dp4a_s8(av.x, apply_signs(g0, sg & 15u), 0) * ls);
        const int s1 = sum_over_subblocks(dp4a_s8(av.y, apply_signs(g1, sg >> 4), 0) * ls);
        const float d = __fmul_rn(half_bits_to_float(*reinterpret_cast<const uint16_t *>(blk)), da[sb]);
        even = __fmaf_rn(d, static_cast<float>(s0), even);
        odd = __fmaf_rn(d, static_cast<float>(s1), odd);
    }
    return hsum8_pairs(even, odd);
}

// One IQ2_S row (d(2) qs(32) signs(32) qh(8) scales(8)): a ten-bit index picks eight magnitudes, the low four for the
// even chunk-lane of the pair and the high four for the odd one; result * 0.125 (src/qwen38_cpu_moe.cuh:298-335).
__device__ __forceinline__ float plain_row_iq2s(const uint8_t *row, int nsb, const int8_t *a, const float *da,
                                                const uint16_t *grid, int lane) {
    const int ib = lane >> 2, p = lane & 3;
    float even = 0.0f, odd = 0.0f;
#pragma unroll 2
    for (int sb = 0; sb < nsb; ++sb) {
        const uint8_t *blk = row + sb * 82;
        const uint32_t idx = blk[2 + ib * 4 + p] | (((static_cast<uint32_t>(blk[66 + ib]) >> (2 * p)) & 3u) << 8);
        const uint32_t sg = blk[34 + ib * 4 + p];
        const uint32_t scb = blk[74 + ib];
        const int ls = 1 + 2 * static_cast<int>(p < 2 ? (scb & 15u) : (scb >> 4));
        const int2 av = *reinterpret_cast<const int2 *>(a + sb * 256 + ib * 32 + p * 8);
        const uint64_t g = wd_iq2s_unpack(grid[idx]);
        const int s0 = sum_over_subblocks(dp4a_s8(av.x, apply_signs(static_cast<uint32_t>(g), sg & 15u), 0) * ls);
        const int s1 = sum_over_subblocks(dp4a_s8(av.y, apply_signs(static_cast<uint32_t>(g >> 32), sg >> 4), 0) * ls);
        const float d = __fmul_rn(half_bits_to_float(*reinterpret_cast<const uint16_t *>(blk)), da[sb]);
        even = __fmaf_rn(d, static_cast<float>(s0), even);
        odd = __fmaf_rn(d, static_cast<float>(s1), odd);
    }
    return __fmul_rn(0.125f, hsum8_pairs(even, odd));
}

__device__ __forceinline__ float plain_row_iq(int type, const uint8_t *row, int nsb, const int8_t *a, const float *da,
                                              const uint16_t *grid3, const uint16_t *grid2, int lane) {
    return type == kTypeIq2s ? plain_row_iq2s(row, nsb, a, da, grid2, lane) : plain_row_iq3s(row, nsb, a, da, grid3, lane);
}

// One IQ4_NL row (blocks of 32: d(2), sixteen bytes, value j in the low nibble and j + 16 in the high one) against a
// Q8_0 activation, by HALF a warp: lane % 16 = (parity of the block, chunk-lane l). Even and odd blocks keep separate
// fmaf chains per chunk-lane, which are added before the closing tree (src/qwen38_cpu_moe.cuh:377-422; nb is even).
__device__ __forceinline__ float plain_row_iq4nl_half(const uint8_t *row, int nb, const int8_t *aq, const float *ad,
                                                      const uint8_t *lut, int lane) {
    const int par = (lane >> 3) & 1, l = lane & 7, hi = l >> 2, k = 4 * (l & 3);
    float acc = 0.0f;
#pragma unroll 2
    for (int b = par; b < nb; b += 2) {
        const uint8_t *wb = row + b * 18;
        const uint32_t w = *reinterpret_cast<const uint16_t *>(wb + 2 + k) |
                           (static_cast<uint32_t>(*reinterpret_cast<const uint16_t *>(wb + 4 + k)) << 16);
        const uint32_t nib = (hi ? (w >> 4) : w) & 0x0f0f0f0fu;
        const uint32_t v = lut[nib & 15u] | (lut[(nib >> 8) & 15u] << 8) | (lut[(nib >> 16) & 15u] << 16) |
                           (static_cast<uint32_t>(lut[nib >> 24]) << 24);
        const int aw = *reinterpret_cast<const int *>(aq + b * 32 + 16 * hi + k);
        const float d = __fmul_rn(half_bits_to_float(*reinterpret_cast<const uint16_t *>(wb)), ad[b]);
        acc = __fmaf_rn(d, static_cast<float>(dp4a_s8(aw, static_cast<int>(v), 0)), acc);
    }
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 8));
    return hsum8_lanes(acc);
}

// Q8_0 of 32 floats held one per lane, plain layout (same rule as quantize_q8_0_part).
__device__ __forceinline__ void plain_q8_0_block(float v, int lane, int8_t *q_out, float *d_out) {
    float amax = fabsf(v);
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, s));
    int q = 0;
    if (amax != 0.0f) {
        q = __float2int_rn(__fmul_rn(v, __fdiv_rn(127.0f, amax)));
        q = max(-128, min(127, q));
    }
    q_out[lane] = static_cast<int8_t>(q);
    if (lane == 0) *d_out = __half2float(__float2half_rn(__fdiv_rn(amax, 127.0f)));
}

// ---- 1: x -> Q8_0 (task layout) and Q8_K --------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) plain_quant_kernel(const PlainParams P) {
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float *x = P.x + static_cast<size_t>(t) * P.H;
    quantize_q8_0_cta(x, P.H, P.xq0 + static_cast<size_t>(t) * P.H, P.xd0 + static_cast<size_t>(t) * (P.H / 32));
    for (int sb = warp; sb < P.H / 256; sb += kWarps)
        quantize_q8_K_warp(x + sb * 256, lane, reinterpret_cast<uint8_t *>(P.xk) + static_cast<size_t>(t) * P.H + sb * 256,
                           P.xdk + static_cast<size_t>(t) * (P.H / 256) + sb);
}

// ---- 2: router logits, shared expert gate/up rows with SiLU * up, the shared expert's sigmoid gate ------------------
// one warp per task: [router tasks | shared gate/up 4-row tasks | the gate dot]
__global__ void __launch_bounds__(kThreads) plain_rows_kernel(const PlainParams P) {
    extern __shared__ __align__(16) uint8_t psm[];
    const int t = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nbh = P.H / 32;
    uint8_t *xq = psm;
    float *xd = reinterpret_cast<float *>(psm + P.H);
    for (int i = threadIdx.x; i < P.H / 16; i += kThreads)
        reinterpret_cast<uint4 *>(xq)[i] = reinterpret_cast<const uint4 *>(P.xq0 + static_cast<size_t>(t) * P.H)[i];
    for (int i = threadIdx.x; i < nbh; i += kThreads) xd[i] = P.xd0[static_cast<size_t>(t) * nbh + i];
    __syncthreads();
    const float *x = P.x + static_cast<size_t>(t) * P.H;
    const int n_router = P.router_f32 ? P.E : P.E / 4, n_sh = P.SF / 4;
    const int task = blockIdx.x * kWarps + warp;
    if (task < n_router) {
        if (P.router_f32) {
            float v = dot_f32_warp(P.router_f32 + static_cast<size_t>(task) * P.H, x, P.H, lane);
            if (P.bias) v = __fadd_rn(v, P.bias[task]);
            if (lane == 0) P.logits[static_cast<size_t>(t) * P.E + task] = v;
        } else {
            float v = q8_task_row(P.router_tasks + static_cast<size_t>(task) * nbh * 136, nbh, xq, xd, lane);
            const int e = task * 4 + (lane >> 3);
            if (P.bias) v = __fadd_rn(v, P.bias[e]);
            if ((lane & 7) == 0) P.logits[static_cast<size_t>(t) * P.E + e] = v;
        }
    } else if (task < n_router + n_sh) {
        const int i = task - n_router;
        float g, u;
        q8_task_row2(P.sh_gate + static_cast<size_t>(i) * nbh * 136, P.sh_up + static_cast<size_t>(i) * nbh * 136, nbh, xq, xd, lane, g, u);
        if ((lane & 7) == 0) P.shact[static_cast<size_t>(t) * P.SF + i * 4 + (lane >> 3)] = __fmul_rn(silu_ggml(g), u);
    } else if (task == n_router + n_sh && P.SF > 0) {
        const float v = dot_f32_warp(P.gate_vec, x, P.H, lane);
        if (lane == 0) P.sgate[t] = sigmoid_ggml(v);
    }
}

// ---- 3: softmax / top-k of one token's logits; the shared expert's activation -> Q8_0 -------------------------------
__global__ void __launch_bounds__(kThreads) plain_select_kernel(const PlainParams P) {
    __shared__ float pr[kMaxExperts];
    __shared__ float gsum[kMaxExperts / 8];
    __shared__ float red[kWarps];
    __shared__ float first[2];
    __shared__ uint32_t cand[2 * kWarps * kMaxK];
    __shared__ int sid[kMaxK];
    __shared__ float sw[kMaxK];
    const int t = blockIdx.x, tid = threadIdx.x;
    const float *logits = P.logits + static_cast<size_t>(t) * P.E;
    RouterScratch rs;
    rs.probs = pr; rs.gsum = gsum; rs.red = red; rs.first = first; rs.cand = cand;
    router_select_cta(tid < P.E ? logits[tid] : 0.0f, tid + kThreads < P.E ? logits[tid + kThreads] : 0.0f, P.E, P.K, P.w_scale,
                      rs, sid, sw);
    __syncthreads();
    for (int j = tid; j < P.K; j += kThreads) {
        P.ids[t * P.K + j] = sid[j];
        P.weights[t * P.K + j] = sw[j];
    }
    for (int i = tid; i < P.E; i += kThreads) P.probs[static_cast<size_t>(t) * P.E + i] = pr[i];
    if (P.SF > 0)
        quantize_q8_0_cta(P.shact + static_cast<size_t>(t) * P.SF, P.SF, P.shq0 + static_cast<size_t>(t) * P.SF,
                          P.shd0 + static_cast<size_t>(t) * (P.SF / 32));
}

// ---- 4: gate and up rows of the selected experts, act = SiLU(gate) * up ---------------------------------------------
// one warp per (slot j, row r)
__global__ void __launch_bounds__(kThreads) plain_gate_up_kernel(const PlainParams P) {
    const int t = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int task = blockIdx.x * kWarps + warp;
    if (task >= P.K * P.F) return;
    const int j = task / P.F, r = task - j * P.F, nsb = P.H / 256;
    const int e = P.ids[t * P.K + j];
    const int8_t *a = P.xk + static_cast<size_t>(t) * P.H;
    const float *da = P.xdk + static_cast<size_t>(t) * nsb;
    const size_t grb = static_cast<size_t>(nsb) * iq_block_bytes(P.gate_type), urb = static_cast<size_t>(nsb) * iq_block_bytes(P.up_type);
    const float g = plain_row_iq(P.gate_type, P.gate + (static_cast<size_t>(e) * P.F + r) * grb, nsb, a, da, P.grid3, P.grid2, lane);
    const float u = plain_row_iq(P.up_type, P.up + (static_cast<size_t>(e) * P.F + r) * urb, nsb, a, da, P.grid3, P.grid2, lane);
    if (lane == 0) P.act[(static_cast<size_t>(t) * P.K + j) * P.F + r] = __fmul_rn(silu_ggml(g), u);
}

// ---- 5: the activation of every (token, slot) in the format the down tensor's type takes ----------------------------
__global__ void __launch_bounds__(256) plain_act_quant_kernel(const PlainParams P) {
    const int j = blockIdx.x, t = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t row = static_cast<size_t>(t) * P.K + j;
    const float *act = P.act + row * P.F;
    int8_t *q = P.actq + row * P.F;
    float *d = P.actd + row * (P.F / 32);
    if (P.down_type == kTypeIq4nl) {
        for (int b = warp; b < P.F / 32; b += 8) plain_q8_0_block(act[b * 32 + lane], lane, q + b * 32, d + b);
    } else {
        for (int sb = warp; sb < P.F / 256; sb += 8)
            quantize_q8_K_warp(act + sb * 256, lane, reinterpret_cast<uint8_t *>(q) + sb * 256, d + sb);
    }
}

// ---- 6: down rows of the selected experts and of the shared expert ---------------------------------------------------
// warp tasks: [K * H rows (IQ4_NL: two rows per warp) | H / 4 shared-expert tasks]
__global__ void __launch_bounds__(kThreads) plain_down_kernel(const PlainParams P) {
    __shared__ uint8_t lut[16];
    if (threadIdx.x < 16) {
        const int v[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};
        lut[threadIdx.x] = static_cast<uint8_t>(v[threadIdx.x]);
    }
    __syncthreads();
    const int t = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int task = blockIdx.x * kWarps + warp;
    const bool nl = P.down_type == kTypeIq4nl;
    const int n_rows = nl ? P.K * P.H / 2 : P.K * P.H;
    if (task < n_rows) {
        if (nl) {
            const int idx = task * 2 + (lane >> 4);                 // (slot, row) of this half of the warp
            const int j = idx / P.H, h = idx - j * P.H, nb = P.F / 32;
            const int e = P.ids[t * P.K + j];
            const size_t arow = static_cast<size_t>(t) * P.K + j;
            const float v = plain_row_iq4nl_half(P.down + (static_cast<size_t>(e) * P.H + h) * nb * 18, nb, P.actq + arow * P.F,
                                                 P.actd + arow * nb, lut, lane);
            if ((lane & 15) == 0) P.eo[arow * P.H + h] = v;
        } else {
            const int j = task / P.H, h = task - j * P.H, nsb = P.F / 256;
            const int e = P.ids[t * P.K + j];
            const size_t arow = static_cast<size_t>(t) * P.K + j;
            const size_t rb = static_cast<size_t>(nsb) * iq_block_bytes(P.down_type);
            const float v = plain_row_iq(P.down_type, P.down + (static_cast<size_t>(e) * P.H + h) * rb, nsb, P.actq + arow * P.F,
                                         P.actd + arow * (P.F / 32), P.grid3, P.grid2, lane);
            if (lane == 0) P.eo[arow * P.H + h] = v;
        }
    } else if (P.SF > 0 && task - n_rows < P.H / 4) {
        const int i = task - n_rows, nbs = P.SF / 32;
        const float v = q8_task_row(P.sh_down + static_cast<size_t>(i) * nbs * 136, nbs, P.shq0 + static_cast<size_t>(t) * P.SF,
                                    P.shd0 + static_cast<size_t>(t) * nbs, lane);
        if ((lane & 7) == 0) P.shdown[static_cast<size_t>(t) * P.H + i * 4 + (lane >> 3)] = v;
    }
}

// ---- 7: out = sum over slots in rank order of mul_rn(expert row, weight), + shared * gate ----------------------------
// (src/qwen38_cpu_moe.cuh:1281-1290, src/qwen38_precision.hpp:32-34)
__global__ void __launch_bounds__(256) plain_combine_kernel(const PlainParams P) {
    const int t = blockIdx.y, h = blockIdx.x * 256 + threadIdx.x;
    if (h >= P.H) return;
    float r = 0.0f;
    for (int j = 0; j < P.K; ++j)
        r = __fadd_rn(r, __fmul_rn(P.eo[(static_cast<size_t>(t) * P.K + j) * P.H + h], P.weights[t * P.K + j]));
    P.routed[static_cast<size_t>(t) * P.H + h] = r;
    P.out[static_cast<size_t>(t) * P.H + h] =
        P.SF > 0 ? __fadd_rn(r, __fmul_rn(P.shdown[static_cast<size_t>(t) * P.H + h], P.sgate[t])) : r;
}

}  // namespace wd
