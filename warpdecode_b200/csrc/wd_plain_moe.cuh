// The MoE block on tensors that stay in ggml block layout: the path for geometries the tiled kernels do not take.
//
// The tiled kernels (wd_moe_kernel.cuh, wd_moe_batch.cuh) want a power-of-two number of superblocks per row and
// IQ3_S / IQ2_S tensors throughout. The reference's own model has hidden 2560 (ten superblocks), expert_ffn 640,
// IQ4_NL down tensors fed by a Q8_0 activation, and an F32 router (src/qwen38_moe.cuh:2181-2211, :2252-2258). Here
// a warp computes whole rows (a gate and an up row together, four IQ4_NL rows, or one IQ3_S / IQ2_S down row) from the
// ggml blocks as they lie, so any hidden that is a multiple of 256 and any expert_ffn that is a multiple of 64 runs.
// The arithmetic contract is the same as everywhere
// else in this library: integer sums per (superblock or block, chunk-lane), one fmaf per block and chunk-lane in
// block order, ggml's 8-lane closing tree (src/qwen38_cpu_moe.cuh:290-440).
//
// One call is four kernels on the caller's stream, launched with programmatic stream serialization so that each one's
// start-up (and every weight copy that does not depend on its predecessor) overlaps the kernel before it:
//   rows     x -> Q8_0; router logits, the shared expert's gate/up rows with SiLU * up, its sigmoid gate
//   select   softmax / top-k; x -> Q8_K
//   gate_up  gate and up rows of the selected experts, SiLU * up
//   down     activation quantisers, down rows of the selected experts and of the shared expert, ordered combine
// Every CTA brings the weight bytes it will read into shared memory with bulk copies issued at once (a chunk of
// sixteen consecutive rows is contiguous and a multiple of 16 bytes in every format), so no row product waits on
// HBM in its dependent chain. Each kernel first waits for its predecessor, then releases its successor: whatever a
// kernel reads before that wait was written at least two kernels earlier.
#pragma once

#include "wd_blocks.cuh"
#include "wd_router.cuh"

namespace wd {

constexpr int kTypeIq4nl = 20;

struct PlainParams {
    int H, F, SF, E, K, T;                  // T: tokens of this call
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
    int8_t *xk;         // Q8_K of x [H]
    float *xdk;         // [H / 256]
    float *logits, *probs, *weights;
    int *ids;
    float *shact;       // [SF]
    float *sgate;       // [1]
    float *act;         // [K][F]
    float *eo;          // [K][H]
    float *shdown;      // [H]
    float *routed;      // [H]
    unsigned *status;   // error word of the engine (a copy that never arrives raises kErrCopyTimeout there)
    unsigned long long *stamps;     // optional [2][CTA][8] step times (ns) of the gate/up and down kernels of token 0
};

#define WD_PSTAMP(kernel, i)                                                                                   \
    if (P.stamps != nullptr && threadIdx.x == 0 && blockIdx.y == 0)                                            \
        P.stamps[((kernel) * 512 + (blockIdx.x & 511)) * 8 + (i)] = global_timer_ns();

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

// Four consecutive IQ4_NL rows (blocks of 32: d(2), sixteen bytes, value j in the low nibble and j + 16 in the high one)
// against a Q8_0 activation, by one warp: lane = (row = lane / 8, parity of the block = (lane / 4) % 2, l = lane % 4).
// A weight word holds chunk-lane l in its low nibbles and chunk-lane l + 4 in its high ones, so one lane carries both
// fmaf chains of its blocks. Even and odd blocks keep separate chains per chunk-lane, which are added before the
// closing tree (src/qwen38_cpu_moe.cuh:377-422; nb is even). Every lane of a row's eight ends with the row's sum.
__device__ __forceinline__ float plain_rows4_iq4nl(const uint8_t *rows, size_t row_bytes, int nb, const int8_t *aq, const float *ad,
                                                   const uint8_t *lut, int lane) {
    const uint8_t *row = rows + (lane >> 3) * row_bytes;
    const int par = (lane >> 2) & 1, k = 4 * (lane & 3);
    float lo = 0.0f, hi = 0.0f;
#pragma unroll 5
    for (int b = par; b < nb; b += 2) {
        const uint8_t *wb = row + b * 18;
        const uint32_t w = *reinterpret_cast<const uint16_t *>(wb + 2 + k) |
                           (static_cast<uint32_t>(*reinterpret_cast<const uint16_t *>(wb + 4 + k)) << 16);
        const uint32_t n0 = w & 0x0f0f0f0fu, n1 = (w >> 4) & 0x0f0f0f0fu;
        const uint32_t v0 = lut[n0 & 15u] | (lut[(n0 >> 8) & 15u] << 8) | (lut[(n0 >> 16) & 15u] << 16) |
                            (static_cast<uint32_t>(lut[n0 >> 24]) << 24);
        const uint32_t v1 = lut[n1 & 15u] | (lut[(n1 >> 8) & 15u] << 8) | (lut[(n1 >> 16) & 15u] << 16) |
                            (static_cast<uint32_t>(lut[n1 >> 24]) << 24);
        const int a0 = *reinterpret_cast<const int *>(aq + b * 32 + k), a1 = *reinterpret_cast<const int *>(aq + b * 32 + 16 + k);
        const float d = __fmul_rn(half_bits_to_float(*reinterpret_cast<const uint16_t *>(wb)), ad[b]);
        lo = __fmaf_rn(d, static_cast<float>(dp4a_s8(a0, static_cast<int>(v0), 0)), lo);
        hi = __fmaf_rn(d, static_cast<float>(dp4a_s8(a1, static_cast<int>(v1), 0)), hi);
    }
    lo = __fadd_rn(lo, __shfl_xor_sync(0xffffffffu, lo, 4));        // even + odd blocks, chunk-lane l
    hi = __fadd_rn(hi, __shfl_xor_sync(0xffffffffu, hi, 4));        // chunk-lane l + 4
    float r = __fadd_rn(lo, hi);                                    // v[l] + v[l + 4]
    r = __fadd_rn(r, __shfl_xor_sync(0xffffffffu, r, 2));           // r0 + r2, r1 + r3
    return __fadd_rn(r, __shfl_xor_sync(0xffffffffu, r, 1));
}

// Q8_0 of n floats in shared memory, plain layout (quants [n], one f16-rounded scale per 32), by the whole CTA: a thread
// takes four values, eight neighbouring lanes a block (the rule of quantize_q8_0_part).
__device__ __forceinline__ void plain_quantize_q8_0_cta(const float *xf, int n, int8_t *q_out, float *d_out) {
    const int nchunks = n >> 2;
#pragma unroll 1
    for (int ch = threadIdx.x; ch < ((nchunks + 31) & ~31); ch += blockDim.x) {
        const bool live = ch < nchunks;
        const float4 v = live ? *reinterpret_cast<const float4 *>(xf + 4 * ch) : make_float4(0, 0, 0, 0);
        float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
        if (!live) continue;
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
        *reinterpret_cast<uint32_t *>(q_out + 4 * ch) = packed;
        if ((ch & 7) == 0) d_out[ch >> 3] = __half2float(__float2half_rn(__fdiv_rn(amax, 127.0f)));
    }
}

// ---- gate and up row of one expert row index in one pass -------------------------------------------------------------
// The rows above spend most of their instructions on meeting the integer sums of the eight sub-blocks by shuffles. Here
// a lane keeps a whole superblock to itself: unit u in [0, 2 nsb) is superblock u of the gate row or superblock u - nsb
// of the up row; lane (grp = lane / 4, p = lane % 4) takes chunk-lanes 2p and 2p + 1 of units grp, grp + 8, ..., all
// eight sub-blocks, so its two integer sums per unit are complete. The float chains (one fmaf per superblock in
// superblock order for each row and chunk-lane) then run on every lane from values handed round by shuffles.
// Codebooks are read expanded from shared memory: IQ3_S 512 x 4 magnitudes, IQ2_S 1024 x 8.
constexpr int kPlainActStride = 272;        // bytes between superblocks of the activation: groups hit different banks

__device__ __forceinline__ void plain_build_tables(uint32_t *t3, uint64_t *t2, const uint16_t *grid3, const uint16_t *grid2,
                                                   bool need3, bool need2) {
    if (need3)
        for (int i = threadIdx.x; i < 512; i += blockDim.x) {
            const uint32_t pk = grid3[i];
            uint32_t g = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) g |= (2u * ((pk >> (3 * j)) & 7u) + 1u) << (8 * j);
            t3[i] = g;
        }
    if (need2)
        for (int i = threadIdx.x; i < 1024; i += blockDim.x) t2[i] = wd_iq2s_unpack(grid2[i]);
}

__device__ __forceinline__ void plain_unit_iq3s(const uint8_t *blk, const int8_t *a, int p, const uint32_t *t3, int &s0, int &s1) {
    uint32_t qh[4], sc[2];
#pragma unroll
    for (int i = 0; i < 4; ++i) qh[i] = *reinterpret_cast<const uint16_t *>(blk + 66 + 2 * i);
#pragma unroll
    for (int i = 0; i < 2; ++i) sc[i] = *reinterpret_cast<const uint16_t *>(blk + 106 + 2 * i);
    s0 = s1 = 0;
#pragma unroll
    for (int ib = 0; ib < 8; ++ib) {
        const uint32_t q2 = *reinterpret_cast<const uint16_t *>(blk + 2 + ib * 8 + 2 * p);
        const uint32_t sg = blk[74 + ib * 4 + p];
        const uint32_t h = (qh[ib >> 1] >> (8 * (ib & 1) + 2 * p));
        const int ls = 1 + 2 * static_cast<int>((sc[ib >> 2] >> (4 * (ib & 3))) & 15u);
        const int2 av = *reinterpret_cast<const int2 *>(a + ib * 32 + p * 8);
        const uint32_t g0 = t3[(q2 & 0xffu) | ((h & 1u) << 8)], g1 = t3[(q2 >> 8) | ((h & 2u) << 7)];
        s0 += dp4a_s8(av.x, apply_signs(g0, sg & 15u), 0) * ls;
        s1 += dp4a_s8(av.y, apply_signs(g1, sg >> 4), 0) * ls;
    }
}

__device__ __forceinline__ void plain_unit_iq2s(const uint8_t *blk, const int8_t *a, int p, const uint64_t *t2, int &s0, int &s1) {
    uint32_t qh[4], sc[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        qh[i] = *reinterpret_cast<const uint16_t *>(blk + 66 + 2 * i);
        sc[i] = *reinterpret_cast<const uint16_t *>(blk + 74 + 2 * i);
    }
    s0 = s1 = 0;
#pragma unroll
    for (int ib = 0; ib < 8; ++ib) {
        const uint32_t hb = (qh[ib >> 1] >> (8 * (ib & 1))) & 0xffu, scb = (sc[ib >> 1] >> (8 * (ib & 1))) & 0xffu;
        const uint32_t idx = blk[2 + ib * 4 + p] | (((hb >> (2 * p)) & 3u) << 8);
        const uint32_t sg = blk[34 + ib * 4 + p];
        const int ls = 1 + 2 * static_cast<int>(p < 2 ? (scb & 15u) : (scb >> 4));
        const int2 av = *reinterpret_cast<const int2 *>(a + ib * 32 + p * 8);
        const uint2 g = *reinterpret_cast<const uint2 *>(t2 + idx);
        s0 += dp4a_s8(av.x, apply_signs(g.x, sg & 15u), 0) * ls;
        s1 += dp4a_s8(av.y, apply_signs(g.y, sg >> 4), 0) * ls;
    }
}

// a: the Q8_K activation in shared memory with kPlainActStride bytes per superblock; da: its scales. nsb <= 16.
__device__ __forceinline__ void plain_gate_up_pair(int gtype, int utype, const uint8_t *grow, const uint8_t *urow, int nsb,
                                                   const int8_t *a, const float *da, const uint32_t *t3, const uint64_t *t2,
                                                   int lane, float &g_out, float &u_out) {
    const int grp = lane >> 2, p = lane & 3, total = 2 * nsb;
    int s0[4], s1[4];
    float dd[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        s0[k] = s1[k] = 0;
        dd[k] = 0.0f;
        const int unit = k * 8 + grp;
        if (k * 8 < total && unit < total) {
            const bool is_up = unit >= nsb;
            const int sb = is_up ? unit - nsb : unit, type = is_up ? utype : gtype;
            const uint8_t *blk = (is_up ? urow : grow) + sb * iq_block_bytes(type);
            if (type == kTypeIq2s) plain_unit_iq2s(blk, a + sb * kPlainActStride, p, t2, s0[k], s1[k]);
            else plain_unit_iq3s(blk, a + sb * kPlainActStride, p, t3, s0[k], s1[k]);
            dd[k] = __fmul_rn(half_bits_to_float(*reinterpret_cast<const uint16_t *>(blk)), da[sb]);
        }
    }
    float ge = 0.0f, go = 0.0f, ue = 0.0f, uo = 0.0f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        if (k * 8 >= total) break;
#pragma unroll
        for (int gq = 0; gq < 8; ++gq) {
            const int unit = k * 8 + gq;
            if (unit >= total) break;
            const int src = gq * 4 + p;
            const float v0 = static_cast<float>(__shfl_sync(0xffffffffu, s0[k], src));
            const float v1 = static_cast<float>(__shfl_sync(0xffffffffu, s1[k], src));
            const float d = __shfl_sync(0xffffffffu, dd[k], src);
            if (unit < nsb) {
                ge = __fmaf_rn(d, v0, ge);
                go = __fmaf_rn(d, v1, go);
            } else {
                ue = __fmaf_rn(d, v0, ue);
                uo = __fmaf_rn(d, v1, uo);
            }
        }
    }
    g_out = hsum8_pairs(ge, go);
    u_out = hsum8_pairs(ue, uo);
    if (gtype == kTypeIq2s) g_out = __fmul_rn(0.125f, g_out);
    if (utype == kTypeIq2s) u_out = __fmul_rn(0.125f, u_out);
}

// Shared-memory plans (bytes); the host sizes the launches with the same functions.
__host__ __device__ inline size_t plain_rows_stage_bytes(int H) { return static_cast<size_t>(H / 32) * 272; }   // two 4-row Q8_0 tasks
__host__ __device__ inline size_t plain_rows_fixed_bytes(int H, int T) {
    return 128 + static_cast<size_t>(T) * H * 4 + static_cast<size_t>(T) * H + static_cast<size_t>(T) * (H / 32) * 4;
}
__host__ __device__ inline size_t plain_iq_row_bytes(int type, int cols) {
    return type == kTypeIq4nl ? static_cast<size_t>(cols / 32) * 18 : static_cast<size_t>(cols / 256) * iq_block_bytes(type);
}
__host__ __device__ inline size_t plain_gate_up_chunks_off(int H) {       // header, padded activation, both codebooks
    return (256 + static_cast<size_t>(H / 256) * 272 + 2048 + 8192 + 127) / 128 * 128;
}
__host__ __device__ inline size_t plain_gate_up_smem(int H, int gate_type, int up_type) {
    return plain_gate_up_chunks_off(H) + 16 * (plain_iq_row_bytes(gate_type, H) + plain_iq_row_bytes(up_type, H));
}
// offset of the staged weight chunks of the down kernel: after the header, the quantised activations and their scales
__host__ __device__ inline size_t plain_down_chunks_off(int F, int K) {
    return (256 + 16 * 64 + static_cast<size_t>(K) * F + static_cast<size_t>(K) * (F / 32) * 4 + 127) / 128 * 128;
}
__host__ __device__ inline size_t plain_down_smem(int F, int SF, int K, int down_type) {
    const size_t act_floats = static_cast<size_t>(K) * F > static_cast<size_t>(SF) ? static_cast<size_t>(K) * F : static_cast<size_t>(SF);
    return plain_down_chunks_off(F, K) + static_cast<size_t>(K) * 16 * plain_iq_row_bytes(down_type, F) + static_cast<size_t>(4) * (SF / 32) * 136 +
           SF + (SF / 32 + 3) / 4 * 16 + act_floats * 4;
}

// ---- 0 (stack step only): x = RMSNorm(residual) * w -----------------------------------------------------------------
// The sum of squares is the perfect binary tree in double over consecutive elements, zero-padded to `width` (the power
// of two at or above n), that defines the RMSNorm between the blocks of the stack on the CPU side as well; one CTA of
// min(512, width) threads, a thread owns width / blockDim consecutive leaves. `prev_out`: the block output of the layer
// before, still to be added to the residual stream (residual += out, one rounded addition), or null.
__global__ void __launch_bounds__(kThreads) plain_norm_kernel(float *residual, const float *prev_out, const float *w, int n, int width,
                                                              float eps, float *x_out) {
    __shared__ double red[kWarps];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5, per = width / blockDim.x;
    grid_dep_wait();
    grid_dep_launch();
    double acc[16];       // width <= 8192 with 512 threads
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        acc[i] = 0.0;
        const int e = tid * per + i;
        if (i < per && e < n) {
            float v = residual[e];
            if (prev_out != nullptr) {
                v = __fadd_rn(v, prev_out[e]);
                residual[e] = v;
            }
            acc[i] = __dmul_rn(static_cast<double>(v), static_cast<double>(v));
        }
    }
#pragma unroll
    for (int s = 1; s < 16; s <<= 1)
#pragma unroll
        for (int i = 0; i + s < 16; i += 2 * s) acc[i] = __dadd_rn(acc[i], acc[i + s]);     // zeros beyond `per` add nothing
    double ss = acc[0];
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) ss = __dadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, s));
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    double tot[kWarps];
#pragma unroll
    for (int i = 0; i < kWarps; ++i) tot[i] = i < nwarps ? red[i] : 0.0;
#pragma unroll
    for (int s = 1; s < kWarps; s <<= 1)
#pragma unroll
        for (int i = 0; i + s < kWarps; i += 2 * s) tot[i] = __dadd_rn(tot[i], tot[i + s]);
    const float scale = __double2float_rn(
        __ddiv_rn(1.0, __dsqrt_rn(__dadd_rn(__ddiv_rn(tot[0], static_cast<double>(n)), static_cast<double>(eps)))));
    for (int i = 0; i < per; ++i) {
        const int e = tid * per + i;
        if (e < n) {
            const float v = __fmul_rn(residual[e], scale);
            x_out[e] = w != nullptr ? __fmul_rn(v, w[e]) : v;
        }
    }
}

// residual += out after the last layer of a stack step
__global__ void plain_add_kernel(float *residual, const float *out, int n) {
    grid_dep_wait();
    grid_dep_launch();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) residual[i] = __fadd_rn(residual[i], out[i]);
}

// ---- 1: x -> Q8_0; router logits, shared expert gate/up rows with SiLU * up, the shared expert's sigmoid gate -------
// One warp per task, [router tasks | shared gate/up pairs of 4-row tasks | the gate dot]; the task's weights are staged
// by one bulk copy and applied to every token of the call.
__global__ void __launch_bounds__(256) plain_rows_kernel(const PlainParams P) {
    extern __shared__ __align__(128) uint8_t psm[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, W = blockDim.x >> 5;
    const int H = P.H, nbh = H / 32, T = P.T;
    uint64_t *bars = reinterpret_cast<uint64_t *>(psm);
    float *xf = reinterpret_cast<float *>(psm + 128);
    uint8_t *xq = reinterpret_cast<uint8_t *>(xf + static_cast<size_t>(T) * H);
    float *xd = reinterpret_cast<float *>(xq + static_cast<size_t>(T) * H);
    uint8_t *stage = reinterpret_cast<uint8_t *>(xd + static_cast<size_t>(T) * nbh) + warp * plain_rows_stage_bytes(H);
    const int n_router = P.router_f32 ? P.E : P.E / 4, n_sh = P.SF / 4;
    const int task = blockIdx.x * W + warp;
    const bool is_router = task < n_router, is_pair = !is_router && task < n_router + n_sh;
    const bool is_gate = task == n_router + n_sh && P.SF > 0;
    if (lane == 0 && (is_router || is_pair || is_gate)) {
        mbar_init(&bars[warp], 1);
        mbar_fence_init();
        const uint32_t tb = static_cast<uint32_t>(nbh) * 136u;
        if (is_gate || (is_router && P.router_f32)) {
            mbar_expect_tx(&bars[warp], static_cast<uint32_t>(H) * 4u);
            bulk_load(stage, is_gate ? P.gate_vec : P.router_f32 + static_cast<size_t>(task) * H, static_cast<uint32_t>(H) * 4u, &bars[warp]);
        } else if (is_router) {
            mbar_expect_tx(&bars[warp], tb);
            bulk_load(stage, P.router_tasks + static_cast<size_t>(task) * tb, tb, &bars[warp]);
        } else {
            const size_t i = static_cast<size_t>(task - n_router);
            mbar_expect_tx(&bars[warp], 2u * tb);
            bulk_load(stage, P.sh_gate + i * tb, tb, &bars[warp]);
            bulk_load(stage + tb, P.sh_up + i * tb, tb, &bars[warp]);
        }
    }
    __syncwarp();
    grid_dep_wait();
    grid_dep_launch();
    for (int i = threadIdx.x; i < T * H / 4; i += blockDim.x) reinterpret_cast<float4 *>(xf)[i] = reinterpret_cast<const float4 *>(P.x)[i];
    __syncthreads();
    for (int t = 0; t < T; ++t) quantize_q8_0_part(xf + t * H, H, xq + t * H, xd + t * nbh, threadIdx.x, blockDim.x);
    __syncthreads();
    if (is_router || is_pair || is_gate) mbar_wait(&bars[warp], 0, P.status);
    for (int t = 0; t < T; ++t) {
        const float *x = xf + t * H;
        if (is_router && P.router_f32) {
            float v = dot_f32_warp(reinterpret_cast<const float *>(stage), x, H, lane);
            if (P.bias) v = __fadd_rn(v, P.bias[task]);
            if (lane == 0) P.logits[static_cast<size_t>(t) * P.E + task] = v;
        } else if (is_router) {
            float v = q8_task_row(stage, nbh, xq + t * H, xd + t * nbh, lane);
            const int e = task * 4 + (lane >> 3);
            if (P.bias) v = __fadd_rn(v, P.bias[e]);
            if ((lane & 7) == 0) P.logits[static_cast<size_t>(t) * P.E + e] = v;
        } else if (is_pair) {
            float g, u;
            q8_task_row2(stage, stage + nbh * 136, nbh, xq + t * H, xd + t * nbh, lane, g, u);
            if ((lane & 7) == 0)
                P.shact[static_cast<size_t>(t) * P.SF + (task - n_router) * 4 + (lane >> 3)] = __fmul_rn(silu_ggml(g), u);
        } else if (is_gate) {
            const float v = dot_f32_warp(reinterpret_cast<const float *>(stage), x, H, lane);
            if (lane == 0) P.sgate[t] = sigmoid_ggml(v);
        }
    }
}

// ---- 2: x -> Q8_K; softmax / top-k of one token's logits ------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) plain_select_kernel(const PlainParams P) {
    __shared__ float pr[kMaxExperts];
    __shared__ float gsum[kMaxExperts / 8];
    __shared__ float red[kWarps];
    __shared__ float first[2];
    __shared__ uint32_t cand[2 * kWarps * kMaxK];
    __shared__ int sid[kMaxK];
    __shared__ float sw[kMaxK];
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // x is older than the kernel before this one: its Q8_K form does not wait
    const float *x = P.x + static_cast<size_t>(t) * P.H;
    for (int sb = warp; sb < P.H / 256; sb += kWarps)
        quantize_q8_K_warp(x + sb * 256, lane, reinterpret_cast<uint8_t *>(P.xk) + static_cast<size_t>(t) * P.H + sb * 256,
                           P.xdk + static_cast<size_t>(t) * (P.H / 256) + sb);
    grid_dep_wait();
    grid_dep_launch();
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
}

// ---- 3: gate and up rows of the selected experts, act = SiLU(gate) * up ---------------------------------------------
// CTA = (slot j, sixteen consecutive rows) of token blockIdx.y; one warp per row
__global__ void __launch_bounds__(kThreads) plain_gate_up_kernel(const PlainParams P) {
    extern __shared__ __align__(128) uint8_t psm[];
    const int t = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int chunks = P.F / 16, j = blockIdx.x / chunks, r0 = (blockIdx.x - j * chunks) * 16, nsb = P.H / 256;
    uint64_t *bar = reinterpret_cast<uint64_t *>(psm);
    float *da = reinterpret_cast<float *>(psm + 128);
    int8_t *a = reinterpret_cast<int8_t *>(psm + 256);
    uint32_t *t3 = reinterpret_cast<uint32_t *>(psm + 256 + nsb * kPlainActStride);
    uint64_t *t2 = reinterpret_cast<uint64_t *>(reinterpret_cast<uint8_t *>(t3) + 2048);
    const size_t grb = plain_iq_row_bytes(P.gate_type, P.H), urb = plain_iq_row_bytes(P.up_type, P.H);
    uint8_t *gs = psm + plain_gate_up_chunks_off(P.H), *us = gs + 16 * grb;
    // the codebooks do not depend on anything this call computes
    WD_PSTAMP(0, 0)
    plain_build_tables(t3, t2, P.grid3, P.grid2, P.gate_type != kTypeIq2s || P.up_type != kTypeIq2s,
                       P.gate_type == kTypeIq2s || P.up_type == kTypeIq2s);
    WD_PSTAMP(0, 1)
    grid_dep_wait();
    grid_dep_launch();
    WD_PSTAMP(0, 2)
    if (threadIdx.x == 0) {
        const size_t e = static_cast<size_t>(P.ids[t * P.K + j]);
        mbar_init(bar, 1);
        mbar_fence_init();
        mbar_expect_tx(bar, static_cast<uint32_t>(16 * (grb + urb)));
        bulk_load(gs, P.gate + (e * P.F + r0) * grb, static_cast<uint32_t>(16 * grb), bar);
        bulk_load(us, P.up + (e * P.F + r0) * urb, static_cast<uint32_t>(16 * urb), bar);
    }
    for (int i = threadIdx.x; i < P.H / 16; i += kThreads)       // sixteen bytes at a time, superblock i / 16
        *reinterpret_cast<uint4 *>(a + (i >> 4) * kPlainActStride + (i & 15) * 16) =
            reinterpret_cast<const uint4 *>(P.xk + static_cast<size_t>(t) * P.H)[i];
    if (threadIdx.x < nsb) da[threadIdx.x] = P.xdk[static_cast<size_t>(t) * nsb + threadIdx.x];
    __syncthreads();
    WD_PSTAMP(0, 3)
    mbar_wait(bar, 0, P.status);
    WD_PSTAMP(0, 4)
    float g, u;
    plain_gate_up_pair(P.gate_type, P.up_type, gs + warp * grb, us + warp * urb, nsb, a, da, t3, t2, lane, g, u);
    if (lane == 0) P.act[(static_cast<size_t>(t) * P.K + j) * P.F + r0 + warp] = __fmul_rn(silu_ggml(g), u);
    WD_PSTAMP(0, 5)
}

// ---- 4: activation quantisers, down rows of the selected experts and of the shared expert, ordered combine ----------
// CTA = sixteen consecutive output rows of token blockIdx.y, all K slots, 16 warps. Warp tasks: (slot, group of four rows)
// for IQ4_NL, (slot, row) for IQ3_S / IQ2_S, then the four 4-row tasks of the shared expert. The rows land in shared
// memory; sixteen threads then form out = sum over slots in rank order of mul_rn(row, weight), + shared * gate
// (src/qwen38_cpu_moe.cuh:1281-1290, src/qwen38_precision.hpp:32-34).
__global__ void __launch_bounds__(kThreads) plain_down_kernel(const PlainParams P) {
    extern __shared__ __align__(128) uint8_t psm[];
    const int t = blockIdx.y, h0 = blockIdx.x * 16, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const bool nl = P.down_type == kTypeIq4nl;
    const int K = P.K, F = P.F, SF = P.SF, nbs = SF / 32;
    uint64_t *bar = reinterpret_cast<uint64_t *>(psm);
    uint8_t *lut = psm + 64;
    float *shd_s = reinterpret_cast<float *>(psm + 128);                    // [16] shared expert rows
    float *eo_s = reinterpret_cast<float *>(psm + 256);                     // [K][16] expert rows
    int8_t *actq = reinterpret_cast<int8_t *>(psm + 256 + kMaxK * 64);
    float *actd = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(actq) + static_cast<size_t>(K) * F);
    const size_t drb = plain_iq_row_bytes(P.down_type, F);
    uint8_t *chunks = psm + plain_down_chunks_off(F, K);
    uint8_t *shs = chunks + static_cast<size_t>(K) * 16 * drb;             // the shared expert's four tasks
    uint8_t *shq = shs + 4 * static_cast<size_t>(nbs) * 136;               // its activation, Q8_0 in task layout
    float *shd = reinterpret_cast<float *>(shq + SF);
    float *actf = reinterpret_cast<float *>(shq + SF + (nbs + 3) / 4 * 16); // F32 staging of the activations
    WD_PSTAMP(1, 0)
    // The ids come from the selection, two kernels back: the weight copies leave before the wait for the gate/up rows.
    if (warp == 0) {        // lane j fetches slot j's expert id and issues its copy; the loads of the ids overlap
        const uint32_t shb = SF > 0 ? 4u * static_cast<uint32_t>(nbs) * 136u : 0u;
        const size_t e = lane < K ? static_cast<size_t>(P.ids[t * K + lane]) : 0;
        if (lane == 0) {
            mbar_init(bar, 1);
            mbar_fence_init();
            mbar_expect_tx(bar, static_cast<uint32_t>(K * 16 * drb) + shb);
        }
        __syncwarp();
        if (lane < K) bulk_load(chunks + static_cast<size_t>(lane) * 16 * drb, P.down + (e * P.H + h0) * drb, static_cast<uint32_t>(16 * drb), bar);
        if (lane == K && shb) bulk_load(shs, P.sh_down + static_cast<size_t>(h0 / 4) * nbs * 136, shb, bar);
    }
    if (threadIdx.x < 16) {
        const int v[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};
        lut[threadIdx.x] = static_cast<uint8_t>(v[threadIdx.x]);
    }
    // the shared expert's activation is older than the kernel before this one
    for (int i = threadIdx.x; i < SF / 4; i += kThreads)
        reinterpret_cast<float4 *>(actf)[i] = reinterpret_cast<const float4 *>(P.shact + static_cast<size_t>(t) * SF)[i];
    __syncthreads();
    if (SF > 0) quantize_q8_0_cta(actf, SF, shq, shd);
    __syncthreads();
    WD_PSTAMP(1, 1)
    grid_dep_wait();
    grid_dep_launch();
    WD_PSTAMP(1, 2)
    // the activations of all slots arrive in one round of loads
    const float *act = P.act + static_cast<size_t>(t) * K * F;
#pragma unroll 4
    for (int i = threadIdx.x; i < K * F / 4; i += kThreads) reinterpret_cast<float4 *>(actf)[i] = reinterpret_cast<const float4 *>(act)[i];
    __syncthreads();
    WD_PSTAMP(1, 3)
    if (nl) {
        plain_quantize_q8_0_cta(actf, K * F, actq, actd);
    } else {
        for (int s = warp; s < K * F / 256; s += kWarps) {
            const int j = s / (F / 256), q = s - j * (F / 256);
            quantize_q8_K_warp(actf + s * 256, lane, reinterpret_cast<uint8_t *>(actq) + s * 256, actd + j * (F / 32) + q);
        }
    }
    __syncthreads();
    WD_PSTAMP(1, 4)
    mbar_wait(bar, 0, P.status);
    WD_PSTAMP(1, 5)
    const int n_exp = nl ? K * 4 : K * 16, n_tasks = n_exp + (SF > 0 ? 4 : 0);
    for (int task = warp; task < n_tasks; task += kWarps) {
        if (task >= n_exp) {
            const int i = task - n_exp;
            const float v = q8_task_row(shs + static_cast<size_t>(i) * nbs * 136, nbs, shq, shd, lane);
            if ((lane & 7) == 0) shd_s[i * 4 + (lane >> 3)] = v;
        } else if (nl) {
            const int j = task >> 2, rg = task & 3;
            const float v = plain_rows4_iq4nl(chunks + (static_cast<size_t>(j) * 16 + rg * 4) * drb, drb, F / 32, actq + j * F,
                                              actd + j * (F / 32), lut, lane);
            if ((lane & 7) == 0) eo_s[j * 16 + rg * 4 + (lane >> 3)] = v;
        } else {
            const int j = task >> 4, row = task & 15;
            const float v = plain_row_iq(P.down_type, chunks + (static_cast<size_t>(j) * 16 + row) * drb, F / 256, actq + j * F,
                                         actd + j * (F / 32), P.grid3, P.grid2, lane);
            if (lane == 0) eo_s[j * 16 + row] = v;
        }
    }
    __syncthreads();
    WD_PSTAMP(1, 6)
    for (int i = threadIdx.x; i < K * 16; i += kThreads)
        P.eo[(static_cast<size_t>(t) * K + (i >> 4)) * P.H + h0 + (i & 15)] = eo_s[i];
    if (threadIdx.x < 16) {
        const size_t o = static_cast<size_t>(t) * P.H + h0 + threadIdx.x;
        float r = 0.0f;
        for (int j = 0; j < K; ++j) r = __fadd_rn(r, __fmul_rn(eo_s[j * 16 + threadIdx.x], P.weights[t * K + j]));
        P.routed[o] = r;
        if (SF > 0) {
            P.shdown[o] = shd_s[threadIdx.x];
            P.out[o] = __fadd_rn(r, __fmul_rn(shd_s[threadIdx.x], P.sgate[t]));
        } else {
            P.out[o] = r;
        }
    }
    WD_PSTAMP(1, 7)
}

}  // namespace wd
