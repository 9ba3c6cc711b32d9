// Kernels of the plain (dense) Q4_0 decoder step: the per-token path of the reference's Runtime::emit_step
// (src/warodecode.cu:2053-2104) for Llama-style models: embedding row, [residual add + RMSNorm + Q8_0 activation,
// fused QKV product, rotary embedding + cache store, decode attention, output product, residual add + RMSNorm + Q8_0,
// gate/up product, SiLU(g) * u + Q8_0, down product] per layer, output norm, output head with the arg-max.
//
// The reference's kernels carry no float order (src/warodecode.cu:1490-1491) and keep activations in F16. Here every
// step has ONE defined order, activations stay F32, and the results are bit-identical to the CPU restatement in
// oracle/wd_oracle_dense.c. The orders are chosen so that every product keeps the whole GPU busy:
//   row dot     a warp splits a row's blocks over its lanes (lane l: blocks l, l + 32, ... ascending, one
//               fmaf(d_w * d_x, (float)int_dot, acc) per block), then a butterfly ^16 ^8 ^4 ^2 ^1
//   RMSNorm     sum of squares as a binary tree in double (the MoE stack's definition)
//   attention   score dots in the same lane order, p = exp(score - max), sums ascending in the position
// Weights: Q4_0 repacked row by row into [rows][blocks][16 B] quants followed by [rows][blocks] f16 scales, so that a
// warp reads 512 consecutive bytes per step (18 B per 32 weights as in ggml).
#pragma once

#include "wd_dense.cuh"

namespace wd {

constexpr int kDecThreads = 256;

// ggml Q4_0 blocks [rows][nb][18 B] -> [rows][nb][16 B] quants, then [rows][nb] f16 scales.
__global__ void repack_q4_0_rows_kernel(const uint8_t *src, uint8_t *dst, long long nblocks) {
    const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (i >= nblocks) return;
    const uint8_t *s = src + i * 18;
    uint8_t *q = dst + i * 16;
    uint16_t *d = reinterpret_cast<uint16_t *>(dst + nblocks * 16) + i;
    *d = static_cast<uint16_t>(s[0] | (s[1] << 8));
    for (int j = 0; j < 16; ++j) q[j] = s[2 + j];
}

// ggml Q4_0 blocks [rows][nb][18 B] -> per row [nb][16 B] quants followed by [nb] f16 scales (18 * nb bytes per row).
__global__ void repack_q4_0_rowpack_kernel(const uint8_t *src, uint8_t *dst, long long nblocks, int nb) {
    const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (i >= nblocks) return;
    const long long row = i / nb;
    const int b = static_cast<int>(i - row * nb);
    const uint8_t *s = src + i * 18;
    uint8_t *r = dst + row * nb * 18;
    for (int j = 0; j < 16; ++j) r[b * 16 + j] = s[2 + j];
    r[nb * 16 + b * 2] = s[0];
    r[nb * 16 + b * 2 + 1] = s[1];
}

// N(0, sigma) values quantised to ggml Q4_0 blocks by ggml's published rule (quantize_row_q4_0_ref): d = (the value of
// largest magnitude, sign kept) / -8; q = min(15, (int)(v / d + 8.5)); byte j = q[j] | q[j + 16] << 4.
__global__ void synth_q4_0_kernel(uint8_t *dst, long long nblocks, float sigma, uint64_t seed, uint64_t stream_id) {
    const long long b = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (b >= nblocks) return;
    float v[32], amax = 0.0f, vmax = 0.0f;
    for (int i = 0; i < 32; ++i) {
        v[i] = sigma * synth_normal(seed, stream_id, static_cast<uint64_t>(b) * 32 + i);
        if (fabsf(v[i]) > amax) {
            amax = fabsf(v[i]);
            vmax = v[i];
        }
    }
    const float d = vmax / -8.0f;
    const float id = d != 0.0f ? 1.0f / d : 0.0f;
    uint8_t *o = dst + b * 18;
    const uint16_t bits = __half_as_ushort(__float2half_rn(d));
    o[0] = bits & 0xff;
    o[1] = bits >> 8;
    for (int j = 0; j < 16; ++j) {
        const int q0 = min(15, static_cast<int>(v[j] * id + 8.5f));
        const int q1 = min(15, static_cast<int>(v[j + 16] * id + 8.5f));
        o[2 + j] = static_cast<uint8_t>(q0 | (q1 << 4));
    }
}

// Q8_0 of 32 floats held one per lane: quant byte and the f16-rounded scale (ggml's rule, as quantize_q8_0_cta).
__device__ __forceinline__ void q8_0_block_warp(float v, int lane, int8_t *q_out, float *d_out) {
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

// hidden += proj (when given); y = RMSNorm(hidden) * w -> Q8_0 (plain layout: int8 [n], float scale per block).
// One CTA of 256 threads, thread t owns the EPL = n / 256 consecutive elements from t * EPL (EPL in {1, 2, 4, 8, 16}),
// so a Q8_0 block belongs to 32 / EPL neighbouring lanes (residual_rmsnorm_kernel, src/warodecode.cu:1408). The sum of
// squares is the binary tree in double of the MoE stack's RMSNorm. `token` (optional): the step starts here, and
// hidden is first filled with the token's embedding row (embedding_q4_kernel).
template <int EPL>
__device__ __forceinline__ void dense_norm_quant_body(float *hidden, const float *proj, const float *w, int n, float eps, int8_t *xq,
                                                      float *xd, const uint8_t *embd_row, bool embd_q8 = false) {
    __shared__ double red[kDecThreads / 32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float v[EPL];
    if (embd_row != nullptr) {
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            const int e = tid * EPL + i, b = e >> 5, j = e & 31;
            const uint8_t *wb = embd_row + b * (embd_q8 ? 34 : 18);
            const float d = half_bits_to_float(static_cast<uint16_t>(wb[0] | (wb[1] << 8)));
            const int q = embd_q8 ? static_cast<int>(static_cast<int8_t>(wb[2 + j]))
                                  : (j < 16 ? (wb[2 + j] & 0x0f) : (wb[2 + j - 16] >> 4)) - 8;
            v[i] = __fmul_rn(d, static_cast<float>(q));
            hidden[e] = v[i];
        }
    } else {
#pragma unroll
        for (int i = 0; i < EPL; ++i) v[i] = hidden[tid * EPL + i];
        if (proj != nullptr) {
#pragma unroll
            for (int i = 0; i < EPL; ++i) {
                v[i] = __fadd_rn(v[i], proj[tid * EPL + i]);
                hidden[tid * EPL + i] = v[i];
            }
        }
    }
    float nw[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) nw[i] = w != nullptr ? w[tid * EPL + i] : 1.0f;
    double loc[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) loc[i] = __dmul_rn(static_cast<double>(v[i]), static_cast<double>(v[i]));
#pragma unroll
    for (int s = 1; s < EPL; s <<= 1)
#pragma unroll
        for (int i = 0; i + s < EPL; i += 2 * s) loc[i] = __dadd_rn(loc[i], loc[i + s]);
    double ss = loc[0];
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) ss = __dadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, s));
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    double tot[kDecThreads / 32];
#pragma unroll
    for (int i = 0; i < kDecThreads / 32; ++i) tot[i] = red[i];
#pragma unroll
    for (int s = 1; s < kDecThreads / 32; s <<= 1)
#pragma unroll
        for (int i = 0; i + s < kDecThreads / 32; i += 2 * s) tot[i] = __dadd_rn(tot[i], tot[i + s]);
    const float scale = __double2float_rn(
        __ddiv_rn(1.0, __dsqrt_rn(__dadd_rn(__ddiv_rn(tot[0], static_cast<double>(n)), static_cast<double>(eps)))));
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        v[i] = __fmul_rn(v[i], scale);
        if (w != nullptr) v[i] = __fmul_rn(v[i], nw[i]);
        amax = fmaxf(amax, fabsf(v[i]));
    }
#pragma unroll
    for (int s = 1; s < 32 / EPL; s <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, s));
    const float inv = amax != 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
        int q = amax != 0.0f ? __float2int_rn(__fmul_rn(v[i], inv)) : 0;
        q = max(-128, min(127, q));
        xq[tid * EPL + i] = static_cast<int8_t>(q);
    }
    if ((tid * EPL & 31) == 0) xd[(tid * EPL) >> 5] = __half2float(__float2half_rn(__fdiv_rn(amax, 127.0f)));
}

__global__ void __launch_bounds__(kDecThreads) dense_norm_quant_kernel(float *hidden, const float *proj, const float *w, int n,
                                                                     float eps, int8_t *xq, float *xd, const uint8_t *embd,
                                                                     const int *token, int vocab, int embd_q8) {
    grid_dep_launch();
    grid_dep_wait();
    const uint8_t *row = nullptr;     // the embedding table in ggml layout: Q4_0 blocks of 18 bytes, or Q8_0 blocks of 34
    if (embd != nullptr) row = embd + static_cast<size_t>(max(0, min(vocab - 1, *token))) * (n >> 5) * (embd_q8 ? 34 : 18);
    const bool q8 = embd_q8 != 0;
    switch (n / kDecThreads) {
        case 1: dense_norm_quant_body<1>(hidden, proj, w, n, eps, xq, xd, row, q8); break;
        case 2: dense_norm_quant_body<2>(hidden, proj, w, n, eps, xq, xd, row, q8); break;
        case 4: dense_norm_quant_body<4>(hidden, proj, w, n, eps, xq, xd, row, q8); break;
        case 8: dense_norm_quant_body<8>(hidden, proj, w, n, eps, xq, xd, row, q8); break;
        default: dense_norm_quant_body<16>(hidden, proj, w, n, eps, xq, xd, row, q8); break;
    }
}

// y = W x: W Q4_0 in the row layout, x already Q8_0 (plain layout, copied into shared memory once per CTA).
// One warp per row at a time (grid-stride over the rows); see the header for the order. When `key` is given the
// kernel also folds the arg-max of the finite results into it (one atomicMax per warp): key = order_key(value) << 32
// | ~row, so the largest value wins and ties go to the lowest row (dense_argmax_reduce_kernel, :1603-1632).
// Dynamic shared memory: nb * 32 bytes of quants + nb floats.
// R rows per warp at once, U blocks per lane and row in flight: R * U 16-byte loads are issued before the first is
// used. Small matrices take R = 1 and one warp per row, so that every byte of the matrix is requested at once; the
// output head takes R = 4 and walks its rows grid-stride.
template <int R, int U>
__global__ void __launch_bounds__(kDecThreads, 4) dense_gemv_q4_0_kernel(const uint8_t *wp, int rows, int nb, const int8_t *xq,
                                                                       const float *xd, float *y, unsigned long long *key) {
    extern __shared__ __align__(16) uint8_t dsm[];
    grid_dep_launch();
    uint4 *sq = reinterpret_cast<uint4 *>(dsm);
    float *sd = reinterpret_cast<float *>(dsm + static_cast<size_t>(nb) * 32);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const uint4 *q_all = reinterpret_cast<const uint4 *>(wp);
    const uint16_t *d_all = reinterpret_cast<const uint16_t *>(wp + static_cast<size_t>(rows) * nb * 16);
    uint4 w[R][U];
    uint16_t dw[R][U];
    auto load = [&](int row0, int b0) {
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int b = b0 + 32 * u;
                if (b < nb && row0 + r < rows) {
                    w[r][u] = __ldg(q_all + static_cast<size_t>(row0 + r) * nb + b);
                    dw[r][u] = __ldg(d_all + static_cast<size_t>(row0 + r) * nb + b);
                }
            }
    };
    // The weights do not depend on the kernel before this one: the first loads leave before the wait for it, and the
    // activation (its output) is fetched after.
    const int row_first = (blockIdx.x * nwarps + warp) * R;
    if (row_first < rows) load(row_first, lane);
    grid_dep_wait();
    for (int i = threadIdx.x; i < nb * 2; i += blockDim.x) sq[i] = reinterpret_cast<const uint4 *>(xq)[i];
    for (int i = threadIdx.x; i < nb; i += blockDim.x) sd[i] = xd[i];
    __syncthreads();
    unsigned long long best = 0ull;
    for (int row0 = row_first; row0 < rows; row0 += gridDim.x * nwarps * R) {
        float acc[R];
#pragma unroll
        for (int r = 0; r < R; ++r) acc[r] = 0.0f;
#pragma unroll 1
        for (int b0 = lane; b0 < nb; b0 += 32 * U) {
            if (row0 != row_first || b0 != lane) load(row0, b0);
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int b = b0 + 32 * u;
                if (b < nb) {
                    const uint4 lo = sq[2 * b], hi = sq[2 * b + 1];
                    const uint32_t al[4] = {lo.x, lo.y, lo.z, lo.w}, ah[4] = {hi.x, hi.y, hi.z, hi.w};
                    const float dx = sd[b];
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        if (row0 + r < rows) {
                            const uint32_t ww[4] = {w[r][u].x, w[r][u].y, w[r][u].z, w[r][u].w};
                            int s16 = 0;    // 16 * sum of (q - 8) * a: a nibble at the top of its byte with the top bit flipped
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                s16 = dp4a_s8(static_cast<int>(((ww[k] << 4) & 0xf0f0f0f0u) ^ 0x80808080u), static_cast<int>(al[k]), s16);
                                s16 = dp4a_s8(static_cast<int>((ww[k] & 0xf0f0f0f0u) ^ 0x80808080u), static_cast<int>(ah[k]), s16);
                            }
                            acc[r] = __fmaf_rn(__fmul_rn(half_bits_to_float(dw[r][u]), dx), static_cast<float>(s16 >> 4), acc[r]);
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
#pragma unroll
            for (int s = 16; s >= 1; s >>= 1) acc[r] = __fadd_rn(acc[r], __shfl_xor_sync(0xffffffffu, acc[r], s));
        }
        if (lane < R && row0 + lane < rows) {
            float v = acc[0];
#pragma unroll
            for (int r = 1; r < R; ++r) v = lane == r ? acc[r] : v;
            y[row0 + lane] = v;
            if (key != nullptr && v == v && fabsf(v) != INFINITY) {
                const unsigned long long k =
                    (static_cast<unsigned long long>(order_key(v)) << 32) | (0xffffffffu - static_cast<unsigned>(row0 + lane));
                best = k > best ? k : best;
            }
        }
    }
    if (key != nullptr) {
#pragma unroll
        for (int s = 1; s < R; s <<= 1) {
            const unsigned long long o = __shfl_xor_sync(0xffffffffu, best, s);
            best = o > best ? o : best;
        }
        if (lane == 0 && best != 0ull) atomicMax(key, best);
    }
}

// ggml Q8_0 [rows][nb] blocks of 34 bytes -> the row layout of dense_gemv_q8_0_kernel: [rows][nb][32 B] quants, then
// [rows][nb] f16 scales. One thread per block.
__global__ void repack_q8_0_dense_kernel(const uint8_t *src, uint8_t *dst, long long nblocks) {
    const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (i >= nblocks) return;
    const uint8_t *s = src + i * 34;
    uint8_t *q = dst + i * 32;
    uint16_t *d = reinterpret_cast<uint16_t *>(dst + nblocks * 32) + i;
    *d = static_cast<uint16_t>(s[0] | (s[1] << 8));
    for (int j = 0; j < 32; ++j) q[j] = s[2 + j];
}

// y = W x for a Q8_0 matrix (what every 2-D tensor of a model file that is not Q4_0 becomes: planarize_q4,
// src/warodecode.cu:1027-1075), same structure and float order as dense_gemv_q4_0_kernel: lane l takes blocks l, l + 32,
// ..., one fmaf(d_w * d_x, (float)int_dot, acc) per block with the exact integer dot of its 32 values, then the
// butterfly. A block is two 16-byte loads.
template <int R, int U>
__global__ void __launch_bounds__(kDecThreads, 4) dense_gemv_q8_0_kernel(const uint8_t *wp, int rows, int nb, const int8_t *xq,
                                                                       const float *xd, float *y, unsigned long long *key) {
    extern __shared__ __align__(16) uint8_t dsm[];
    grid_dep_launch();
    uint4 *sq = reinterpret_cast<uint4 *>(dsm);
    float *sd = reinterpret_cast<float *>(dsm + static_cast<size_t>(nb) * 32);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const uint4 *q_all = reinterpret_cast<const uint4 *>(wp);
    const uint16_t *d_all = reinterpret_cast<const uint16_t *>(wp + static_cast<size_t>(rows) * nb * 32);
    uint4 wl[R][U], wh[R][U];
    uint16_t dw[R][U];
    auto load = [&](int row0, int b0) {
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int b = b0 + 32 * u;
                if (b < nb && row0 + r < rows) {
                    const size_t blk = static_cast<size_t>(row0 + r) * nb + b;
                    wl[r][u] = __ldg(q_all + 2 * blk);
                    wh[r][u] = __ldg(q_all + 2 * blk + 1);
                    dw[r][u] = __ldg(d_all + blk);
                }
            }
    };
    const int row_first = (blockIdx.x * nwarps + warp) * R;
    if (row_first < rows) load(row_first, lane);     // weights do not depend on the kernel before this one
    grid_dep_wait();
    for (int i = threadIdx.x; i < nb * 2; i += blockDim.x) sq[i] = reinterpret_cast<const uint4 *>(xq)[i];
    for (int i = threadIdx.x; i < nb; i += blockDim.x) sd[i] = xd[i];
    __syncthreads();
    unsigned long long best = 0ull;
    for (int row0 = row_first; row0 < rows; row0 += gridDim.x * nwarps * R) {
        float acc[R];
#pragma unroll
        for (int r = 0; r < R; ++r) acc[r] = 0.0f;
#pragma unroll 1
        for (int b0 = lane; b0 < nb; b0 += 32 * U) {
            if (row0 != row_first || b0 != lane) load(row0, b0);
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int b = b0 + 32 * u;
                if (b < nb) {
                    const uint4 lo = sq[2 * b], hi = sq[2 * b + 1];
                    const float dx = sd[b];
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        if (row0 + r < rows) {
                            int s = dp4a_s8(static_cast<int>(wl[r][u].x), static_cast<int>(lo.x), 0);
                            s = dp4a_s8(static_cast<int>(wl[r][u].y), static_cast<int>(lo.y), s);
                            s = dp4a_s8(static_cast<int>(wl[r][u].z), static_cast<int>(lo.z), s);
                            s = dp4a_s8(static_cast<int>(wl[r][u].w), static_cast<int>(lo.w), s);
                            s = dp4a_s8(static_cast<int>(wh[r][u].x), static_cast<int>(hi.x), s);
                            s = dp4a_s8(static_cast<int>(wh[r][u].y), static_cast<int>(hi.y), s);
                            s = dp4a_s8(static_cast<int>(wh[r][u].z), static_cast<int>(hi.z), s);
                            s = dp4a_s8(static_cast<int>(wh[r][u].w), static_cast<int>(hi.w), s);
                            acc[r] = __fmaf_rn(__fmul_rn(half_bits_to_float(dw[r][u]), dx), static_cast<float>(s), acc[r]);
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
#pragma unroll
            for (int s = 16; s >= 1; s >>= 1) acc[r] = __fadd_rn(acc[r], __shfl_xor_sync(0xffffffffu, acc[r], s));
        }
        if (lane < R && row0 + lane < rows) {
            float v = acc[0];
#pragma unroll
            for (int r = 1; r < R; ++r) v = lane == r ? acc[r] : v;
            y[row0 + lane] = v;
            if (key != nullptr && v == v && fabsf(v) != INFINITY) {
                const unsigned long long k =
                    (static_cast<unsigned long long>(order_key(v)) << 32) | (0xffffffffu - static_cast<unsigned>(row0 + lane));
                best = k > best ? k : best;
            }
        }
    }
    if (key != nullptr) {
#pragma unroll
        for (int s = 1; s < R; s <<= 1) {
            const unsigned long long o = __shfl_xor_sync(0xffffffffu, best, s);
            best = o > best ? o : best;
        }
        if (lane == 0 && best != 0ull) atomicMax(key, best);
    }
}

// The attention of one query head over cache positions 0..pos by one CTA of `nthreads` threads. qs: the rotated q head,
// kn / vn: the new (rotated) k and the new v of position pos (shared memory); kc / vc: the head's KV group in the
// caches, row stride kv_dim; sc: [max_ctx] scores; vbuf: [32][head_dim] staging for the values. Returns the head's
// output element `tid` to threads tid < head_dim. Order (the oracle's): score_t = lane-strided fmaf dot + butterfly,
// times inv_sqrt; m = max; p_t = exp(score_t - m); l and out ascending in t. The loads are arranged so that a warp's
// keys are in flight together and the values come through shared memory in chunks of 32 positions.
__device__ __forceinline__ float dense_attention_core(const float *qs, const float *kn, const float *vn, const float *kc, const float *vc,
                                                      int pos, int kv_dim, int head_dim, float inv_sqrt, float *sc, float *vbuf,
                                                      int nthreads) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = nthreads >> 5;
    const float q0 = qs[lane], q1 = lane + 32 < head_dim ? qs[lane + 32] : 0.0f, q2 = lane + 64 < head_dim ? qs[lane + 64] : 0.0f,
                q3 = lane + 96 < head_dim ? qs[lane + 96] : 0.0f;
#pragma unroll 1
    for (int t0 = warp; t0 <= pos; t0 += 8 * nw) {
        float k0[8], k1[8], k2[8], k3[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {               // every position's loads leave before the first dot
            const int t = t0 + i * nw;
            k0[i] = k1[i] = k2[i] = k3[i] = 0.0f;
            if (t <= pos) {
                const float *k = t == pos ? kn : kc + static_cast<size_t>(t) * kv_dim;
                k0[i] = k[lane];
                if (lane + 32 < head_dim) k1[i] = k[lane + 32];
                if (lane + 64 < head_dim) k2[i] = k[lane + 64];
                if (lane + 96 < head_dim) k3[i] = k[lane + 96];
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int t = t0 + i * nw;
            if (t <= pos) {
                float acc = __fmaf_rn(q0, k0[i], 0.0f);
                if (head_dim > 32) acc = __fmaf_rn(q1, k1[i], acc);
                if (head_dim > 64) acc = __fmaf_rn(q2, k2[i], acc);
                if (head_dim > 96) acc = __fmaf_rn(q3, k3[i], acc);
#pragma unroll
                for (int s = 16; s >= 1; s >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, s));
                if (lane == 0) sc[t] = __fmul_rn(acc, inv_sqrt);
            }
        }
    }
    __syncthreads();
    float m = -INFINITY;
    for (int t = 0; t <= pos; ++t) m = sc[t] > m ? sc[t] : m;
    __syncthreads();
    for (int t = tid; t <= pos; t += nthreads) sc[t] = exp_ggml(__fadd_rn(sc[t], -m));
    float l = 0.0f, acc = 0.0f;
#pragma unroll 1
    for (int c0 = 0; c0 < pos; c0 += 32) {
        const int n = min(32, pos - c0);
        __syncthreads();                            // the scores are final; the previous chunk has been consumed
        for (int i = tid; i < n * head_dim; i += nthreads) {
            const int r = i / head_dim, d = i - r * head_dim;
            vbuf[i] = vc[static_cast<size_t>(c0 + r) * kv_dim + d];
        }
        __syncthreads();
        if (tid < head_dim) {
            for (int r = 0; r < n; ++r) {
                const float p = sc[c0 + r];
                l = __fadd_rn(l, p);
                acc = __fmaf_rn(p, vbuf[r * head_dim + tid], acc);
            }
        }
    }
    __syncthreads();
    if (tid < head_dim) {
        l = __fadd_rn(l, sc[pos]);
        acc = __fmaf_rn(sc[pos], vn[tid], acc);
        return __fdiv_rn(acc, l);
    }
    return 0.0f;
}

// Rotary embedding + cache store + decode attention + Q8_0 of the head's output, one CTA (128 threads) per query head
// (rope_store_kernel :1855 and attention_decode_kernel :1902 of src/warodecode.cu, the latter as two passes; orders in
// the header and in the oracle). The rotary embedding pairs element p with p + head_dim / 2 (GPT-NeoX) and takes
// cos/sin from the table row of *pos. Every CTA rotates its own q head and, for itself, the new k head of its KV
// group; the first CTA of a group also stores the rotated k and the v into the caches [max_ctx][kv_dim]. Cache
// position pos itself is taken from the CTA's own copy, so no CTA waits for another's store.
// head_dim a multiple of 32, at most 128; dynamic shared memory: max_ctx + 32 * head_dim floats.
// EXTRAS: the layer has q/k/v biases (Qwen2-style files: added to the QKV product's rows) and / or RMSNorm weights for
// the q and k heads (Qwen3-style: qk_norm_kernel, src/warodecode.cu:1836), applied in that order before the rotary
// embedding (emit_step :2069-2075). Layers without them run the instantiation that has none of that code.
template <bool EXTRAS>
__global__ void __launch_bounds__(128) dense_attention_kernel(const float *qkv, const float *table, float *kcache, float *vcache,
                                                              const int *pos_ptr, int heads, int kv_heads, int head_dim, int max_ctx,
                                                              float inv_sqrt, int8_t *oq, float *od, const float *bqkv,
                                                              const float *q_norm, const float *k_norm, float eps) {
    extern __shared__ __align__(16) float sc[];        // [max_ctx] scores, then [32][head_dim] value staging
    __shared__ float qs[128], kn[128], vn[128], outv[128];
    float *vbuf = sc + max_ctx;
    grid_dep_launch();
    grid_dep_wait();
    const int h = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int pos = *pos_ptr, kv_dim = kv_heads * head_dim, kvh = (h * kv_heads) / heads, half = head_dim / 2;
    const float *q_raw = qkv + static_cast<size_t>(h) * head_dim;
    const float *k_raw = qkv + static_cast<size_t>(heads + kvh) * head_dim;
    const float *v_raw = qkv + static_cast<size_t>(heads + kv_heads + kvh) * head_dim;
    if constexpr (EXTRAS) {
        __shared__ float qn[128], kn_in[128], vn_in[128];
        __shared__ double nred[2][4];
        float xq_ = 0.0f, xk_ = 0.0f, xv_ = 0.0f;
        if (tid < head_dim) {
            xq_ = q_raw[tid];
            xk_ = k_raw[tid];
            xv_ = v_raw[tid];
            if (bqkv != nullptr) {
                xq_ = __fadd_rn(xq_, bqkv[static_cast<size_t>(h) * head_dim + tid]);
                xk_ = __fadd_rn(xk_, bqkv[static_cast<size_t>(heads + kvh) * head_dim + tid]);
                xv_ = __fadd_rn(xv_, bqkv[static_cast<size_t>(heads + kv_heads + kvh) * head_dim + tid]);
            }
        }
        if (q_norm != nullptr || k_norm != nullptr) {
            // the sum of squares is the binary tree in double over the head's elements, zero-padded to 128 leaves (adding
            // +0.0 changes nothing), thread t owns leaf t
            double sq_ = __dmul_rn(static_cast<double>(xq_), static_cast<double>(xq_));
            double sk_ = __dmul_rn(static_cast<double>(xk_), static_cast<double>(xk_));
#pragma unroll
            for (int s = 1; s < 32; s <<= 1) {
                sq_ = __dadd_rn(sq_, __shfl_xor_sync(0xffffffffu, sq_, s));
                sk_ = __dadd_rn(sk_, __shfl_xor_sync(0xffffffffu, sk_, s));
            }
            if (lane == 0) {
                nred[0][warp] = sq_;
                nred[1][warp] = sk_;
            }
            __syncthreads();
            const double tq = __dadd_rn(__dadd_rn(nred[0][0], nred[0][1]), __dadd_rn(nred[0][2], nred[0][3]));
            const double tk = __dadd_rn(__dadd_rn(nred[1][0], nred[1][1]), __dadd_rn(nred[1][2], nred[1][3]));
            const double hd = static_cast<double>(head_dim), ep = static_cast<double>(eps);
            const float scq = __double2float_rn(__ddiv_rn(1.0, __dsqrt_rn(__dadd_rn(__ddiv_rn(tq, hd), ep))));
            const float sck = __double2float_rn(__ddiv_rn(1.0, __dsqrt_rn(__dadd_rn(__ddiv_rn(tk, hd), ep))));
            if (tid < head_dim) {
                if (q_norm != nullptr) xq_ = __fmul_rn(__fmul_rn(xq_, scq), q_norm[tid]);
                if (k_norm != nullptr) xk_ = __fmul_rn(__fmul_rn(xk_, sck), k_norm[tid]);
            }
        }
        if (tid < head_dim) {
            qn[tid] = xq_;
            kn_in[tid] = xk_;
            vn_in[tid] = xv_;
        }
        __syncthreads();
        q_raw = qn;
        k_raw = kn_in;
        v_raw = vn_in;
    }
    float *kc = kcache + static_cast<size_t>(kvh) * head_dim, *vc = vcache + static_cast<size_t>(kvh) * head_dim;
    const bool writer = h % (heads / kv_heads) == 0;        // the first head of its KV group
    if (tid < half) {
        const float cs = table[(static_cast<size_t>(pos) * half + tid) * 2], sn = table[(static_cast<size_t>(pos) * half + tid) * 2 + 1];
        {
            const float a = q_raw[tid], b = q_raw[tid + half];
            qs[tid] = __fadd_rn(__fmul_rn(a, cs), -__fmul_rn(b, sn));
            qs[tid + half] = __fadd_rn(__fmul_rn(a, sn), __fmul_rn(b, cs));
        }
        const float a = k_raw[tid], b = k_raw[tid + half];
        const float k0 = __fadd_rn(__fmul_rn(a, cs), -__fmul_rn(b, sn)), k1 = __fadd_rn(__fmul_rn(a, sn), __fmul_rn(b, cs));
        kn[tid] = k0;
        kn[tid + half] = k1;
        const float v0 = v_raw[tid], v1 = v_raw[tid + half];
        vn[tid] = v0;
        vn[tid + half] = v1;
        if (writer) {
            const size_t off = static_cast<size_t>(pos) * kv_dim;
            kc[off + tid] = k0;
            kc[off + tid + half] = k1;
            vc[off + tid] = v0;
            vc[off + tid + half] = v1;
        }
    }
    __syncthreads();
    const float o = dense_attention_core(qs, kn, vn, kc, vc, pos, kv_dim, head_dim, inv_sqrt, sc, vbuf, 128);
    if (tid < head_dim) outv[tid] = o;
    __syncthreads();
    if (warp < head_dim / 32) {
        const int b = (h * head_dim) / 32 + warp;
        q8_0_block_warp(outv[warp * 32 + lane], lane, oq + static_cast<size_t>(b) * 32, od + b);
    }
}

// act = SiLU(g) * u for gate_up = [gate rows | up rows], -> Q8_0; one warp per block of 32 (swiglu_kernel, :1956).
__global__ void dense_swiglu_quant_kernel(const float *gate_up, int n, int8_t *xq, float *xd) {
    grid_dep_launch();
    grid_dep_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;     // n is a multiple of 32: whole warps leave together
    const float v = __fmul_rn(silu_ggml(gate_up[i]), gate_up[n + i]);
    q8_0_block_warp(v, threadIdx.x & 31, xq + (i & ~31), xd + (i >> 5));
}

// End of a step: the arg-max key becomes the next token (0 when no logit was finite), is recorded at out[pos + 1],
// the position advances, the key is cleared for the next step (dense_argmax_finish_kernel + increment_pos_kernel).
// `forced` (nullable): forced[pos + 1] >= 0 replaces the generated token (prompt tokens).
__global__ void dense_finish_kernel(unsigned long long *key, int *token, int *pos, int *out, const int *forced) {
    grid_dep_wait();
    const unsigned long long k = *key;
    int t = k == 0ull ? 0 : static_cast<int>(0xffffffffu - static_cast<unsigned>(k & 0xffffffffull));
    const int p = *pos + 1;
    if (forced != nullptr && forced[p] >= 0) t = forced[p];
    out[p] = t;
    *token = t;
    *pos = p;
    *key = 0ull;
}

}  // namespace wd
