// Building blocks of the fused MoE layer kernel: activation quantisers, the Q8_0 row task, the
// F32 dot and the float side of an IQ3_S tile.
//
// Code size matters here as much as instruction count: the layer kernel runs each instruction only a
// few times per launch, so instruction fetch is part of its critical path. Which helpers are real
// functions (__noinline__: the tile decoders, used from three places) and which are inlined, and how far
// each loop is unrolled, was settled by same-device A/B timing of the whole layer stack, not by rule;
// loops that do not need unrolling carry `#pragma unroll 1`.
#pragma once

#include "wd_formats.cuh"

namespace wd {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxK = 16;
constexpr int kMaxExperts = 1024;

// ---------------------------------------------------------------------------------------------
// activation quantisers (bit-exact twins of src/qwen38_cpu_moe.cuh:220-263)
// ---------------------------------------------------------------------------------------------
// Q8_0 of n floats (n multiple of 128) held in shared `xf`; output: quants in task layout
// [g][l][16 B] (word i = values 4l..4l+3 of block 4g+i) and per-block scales as the f16-rounded float.
// by `nthreads` threads (a multiple of 32, whole warps) of which this one is number `thread`
__device__ __forceinline__ void quantize_q8_0_part(const float *xf, int n, uint8_t *q_out, float *d_out, int thread, int nthreads) {
    const int nchunks = n >> 2;    // groups of four values; 8 chunks form a block
#pragma unroll 1
    for (int ch = thread; ch < ((nchunks + 31) & ~31); ch += nthreads) {
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
__device__ __forceinline__ void quantize_q8_0_cta(const float *xf, int n, uint8_t *q_out, float *d_out) {
    quantize_q8_0_part(xf, n, q_out, d_out, threadIdx.x, blockDim.x);
}

// Q8_K of one 256-value superblock by one warp: lane quantises src[8*lane .. 8*lane+7].
__device__ __forceinline__ void quantize_q8_K_warp(const float *src, int lane, uint8_t *q_out_sb, float *d_out) {
    const float4 a = *reinterpret_cast<const float4 *>(src + lane * 8);
    const float4 b = *reinterpret_cast<const float4 *>(src + lane * 8 + 4);
    const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
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
__device__ __forceinline__ float q8_task_row(const uint8_t *task, int nb, const uint8_t *xq, const float *xd, int lane) {
    const int r = lane >> 3, l = lane & 7;
    const uint8_t *wq = task + r * 128 + l * 16;
    const uint8_t *wd = task + nb * 128 + r * nb * 2;
    float acc = 0.0f;
#pragma unroll 4
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

// Two row tasks against the same activation in one pass (the shared expert's gate and up rows): the two fmaf
// chains are independent, so their loads and integer dots overlap. Same operations as two q8_task_row calls.
__device__ __forceinline__ void q8_task_row2(const uint8_t *task_a, const uint8_t *task_b, int nb, const uint8_t *xq,
                                          const float *xd, int lane, float &out_a, float &out_b) {
    const int r = lane >> 3, l = lane & 7;
    const uint8_t *wqa = task_a + r * 128 + l * 16, *wqb = task_b + r * 128 + l * 16;
    const uint8_t *wda = task_a + nb * 128 + r * nb * 2, *wdb = task_b + nb * 128 + r * nb * 2;
    float acc_a = 0.0f, acc_b = 0.0f;
#pragma unroll 8
    for (int g = 0; g < (nb >> 2); ++g) {
        const uint4 wa = *reinterpret_cast<const uint4 *>(wqa + g * 512);
        const uint4 wb = *reinterpret_cast<const uint4 *>(wqb + g * 512);
        const uint4 a = *reinterpret_cast<const uint4 *>(xq + (g * 8 + l) * 16);
        const uint2 da = *reinterpret_cast<const uint2 *>(wda + g * 8);
        const uint2 db = *reinterpret_cast<const uint2 *>(wdb + g * 8);
        const float4 dx = *reinterpret_cast<const float4 *>(xd + g * 4);
        const float sa0 = __fmul_rn(half_bits_to_float(da.x & 0xffffu), dx.x), sb0 = __fmul_rn(half_bits_to_float(db.x & 0xffffu), dx.x);
        const float sa1 = __fmul_rn(half_bits_to_float(da.x >> 16), dx.y), sb1 = __fmul_rn(half_bits_to_float(db.x >> 16), dx.y);
        const float sa2 = __fmul_rn(half_bits_to_float(da.y & 0xffffu), dx.z), sb2 = __fmul_rn(half_bits_to_float(db.y & 0xffffu), dx.z);
        const float sa3 = __fmul_rn(half_bits_to_float(da.y >> 16), dx.w), sb3 = __fmul_rn(half_bits_to_float(db.y >> 16), dx.w);
        acc_a = __fmaf_rn(sa0, static_cast<float>(dp4a_s8(wa.x, a.x, 0)), acc_a);
        acc_b = __fmaf_rn(sb0, static_cast<float>(dp4a_s8(wb.x, a.x, 0)), acc_b);
        acc_a = __fmaf_rn(sa1, static_cast<float>(dp4a_s8(wa.y, a.y, 0)), acc_a);
        acc_b = __fmaf_rn(sb1, static_cast<float>(dp4a_s8(wb.y, a.y, 0)), acc_b);
        acc_a = __fmaf_rn(sa2, static_cast<float>(dp4a_s8(wa.z, a.z, 0)), acc_a);
        acc_b = __fmaf_rn(sb2, static_cast<float>(dp4a_s8(wb.z, a.z, 0)), acc_b);
        acc_a = __fmaf_rn(sa3, static_cast<float>(dp4a_s8(wa.w, a.w, 0)), acc_a);
        acc_b = __fmaf_rn(sb3, static_cast<float>(dp4a_s8(wb.w, a.w, 0)), acc_b);
    }
    out_a = hsum8_lanes(acc_a);
    out_b = hsum8_lanes(acc_b);
}

// ggml_vec_dot_f32 in its AVX2 order by one warp: lane t owns elements = t (mod 32)
// (src/qwen38_cpu_moe.cuh:847-871; n is a multiple of 32 here).
__device__ __noinline__ float dot_f32_warp(const float *a, const float *b, int n, int lane) {
    float s = 0.0f;
#pragma unroll 4
    for (int i = lane; i < n; i += 32) s = __fmaf_rn(a[i], b[i], s);
    s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 16));
    s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 8));
    s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 4));
    s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 1));
    s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 2));
    return s;
}

// ---------------------------------------------------------------------------------------------
// float side of an IQ3_S tile: lanes hold (row, sb) integer partials; the chain over sb of each
// (row, chunk-lane) runs in superblock order with one fmaf per step, then the 8-lane reduction
// (src/qwen38_cpu_moe.cuh:337-375). nsb in {1,2,4,8,16,32}; rows per tile R = 32 / nsb.
// Writes the R row sums to rows_out (shared memory, per warp). Scratch `scr`: R stripes of
// nsb*8+8 floats plus 32 scales.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void iq_tile_rows(const int partial[8], float scale, int nsb, int lane, float *scr,
                                             float *rows_out, float post = 1.0f) {
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
#pragma unroll 1
    for (int it = 0; it < nit; ++it) {
        const int ch = it * 32 + lane;          // chain index = row * 8 + c
        const int rr = ch >> 3, c = ch & 7;
        float acc = 0.0f;
        if (rr < R) {
#pragma unroll 1
            for (int s = 0; s < nsb; ++s) acc = __fmaf_rn(sc[rr * nsb + s], scr[rr * stripe + s * 8 + c], acc);
        }
        acc = hsum8_lanes(acc);
        if (rr < R && c == 0) rows_out[rr] = __fmul_rn(post, acc);       // post is 1 (exact) or IQ2_S's 0.125
    }
    __syncwarp();
}

// One IQ3_S tile (32 blocks, lane = block) against Q8_K activations: integer partials, then the row
// sums into rows_out. `a` / `dx` are this lane's superblock of activations and its scale. The single
// shared copy of the decoder: gate tiles, up tiles and down tiles all come through here.
// partial_dump (optional, global): receives this lane's eight integer partials.
template <int UNROLL = 1>
__device__ __noinline__ void iq3_tile_to_rows(const uint8_t *tile, const uint8_t *a, float dx, int nsb, int lane,
                                              uint32_t lane4x2, const uint8_t *tab, float *scr, float *rows_out,
                                              int *partial_dump) {
    int p[8];
    iq3_block_partials<UNROLL>(tile, lane, a, lane4x2, tab, p);
    if (partial_dump) {
#pragma unroll
        for (int c = 0; c < 8; ++c) partial_dump[c] = p[c];
    }
    const float dw = half_bits_to_float(*reinterpret_cast<const uint16_t *>(tile + kIq3OffD + lane * 2));
    iq_tile_rows(p, __fmul_rn(dw, dx), nsb, lane, scr, rows_out);
}

// The IQ2_S twin.
__device__ __noinline__ void iq2_tile_to_rows(const uint8_t *tile, const uint8_t *a, float dx, int nsb, int lane,
                                              const uint8_t *tab2, float *scr, float *rows_out, int *partial_dump) {
    int p[8];
    iq2_block_partials_range(tile, lane, a, tab2, p, 0, 8);
    if (partial_dump) {
#pragma unroll
        for (int c = 0; c < 8; ++c) partial_dump[c] = p[c];
    }
    const float dw = half_bits_to_float(*reinterpret_cast<const uint16_t *>(tile + kIq2OffD + lane * 2));
    iq_tile_rows(p, __fmul_rn(dw, dx), nsb, lane, scr, rows_out, 0.125f);
}

// Either type (a warp-uniform branch). tab3: lane-private IQ3_S table, tab2: IQ2_S table.
template <int UNROLL = 1>
__device__ __forceinline__ void iq_tile_to_rows_any(int type, const uint8_t *tile, const uint8_t *a, float dx, int nsb,
                                                    int lane, uint32_t lane4x2, const uint8_t *tab3, const uint8_t *tab2,
                                                    float *scr, float *rows_out, int *partial_dump) {
    if (type == kTypeIq2s) iq2_tile_to_rows(tile, a, dx, nsb, lane, tab2, scr, rows_out, partial_dump);
    else iq3_tile_to_rows<UNROLL>(tile, a, dx, nsb, lane, lane4x2, tab3, scr, rows_out, partial_dump);
}

}  // namespace wd
