// Dense low-bit matvec for the plain decoder path: y = W x with W in Q4_0, x quantised to Q8_0 in the
// kernel's prologue. Replaces q4_0_q8_0_gemv_kernel / q8_0_quantize_half_kernel / planarize_q4
// (src/warodecode.cu:1535-1562, :1504, :1027-1098). The reference's kernel has no fixed float order;
// this one uses ggml's (ggml_vec_dot_q4_0_q8_0, AVX2): per block one fmaf(d_w * d_x, (float)p_c, lane_c)
// for each of the eight chunk-lanes c (four consecutive values each), blocks ascending, then the 8-lane
// tree. Values 0..15 of a block are the low nibbles of its 16 bytes, values 16..31 the high nibbles.
//
// HBM-bound streaming kernel: W is read once with 16-byte loads that a warp issues for 32 consecutive
// rows (lane = row), several blocks in flight per lane; nothing else touches DRAM.
#pragma once

#include "wd_blocks.cuh"

namespace wd {

// Planar layout of a Q4_0 matrix (rows a multiple of 32): tiles of 32 rows; within tile t the quants
// of block b sit at q[(t * nb + b) * 32 + row_in_tile] (16 bytes each), followed after ALL quants by the
// f16 scales in the same order d[(t * nb + b) * 32 + row_in_tile]. 18 bytes per 32 weights as in ggml.
__global__ void repack_q4_0_kernel(const uint8_t *src, uint8_t *dst, int rows, int nb) {
    const long long n = static_cast<long long>(rows) * nb;
    const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (i >= n) return;
    const int row = static_cast<int>(i / nb), b = static_cast<int>(i % nb);
    const uint8_t *blk = src + i * 18;
    const long long o = (static_cast<long long>(row >> 5) * nb + b) * 32 + (row & 31);
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k)
        w[k] = blk[2 + 4 * k] | (blk[3 + 4 * k] << 8) | (blk[4 + 4 * k] << 16) | (static_cast<uint32_t>(blk[5 + 4 * k]) << 24);
    *reinterpret_cast<uint4 *>(dst + o * 16) = make_uint4(w[0], w[1], w[2], w[3]);
    uint16_t *d = reinterpret_cast<uint16_t *>(dst + n * 16);
    d[o] = static_cast<uint16_t>(blk[0] | (blk[1] << 8));
}

// x -> Q8_0 with the plain layout: quants [block][32] int8, scales [block] float (the f16-rounded value).
// Same arithmetic as quantize_q8_0_cta (src/qwen38_cpu_moe.cuh:220-237).
__device__ __forceinline__ void quantize_q8_0_plain_cta(const float *x, int n, uint8_t *q_out, float *d_out) {
    const int nchunks = n >> 2;
    for (int ch = threadIdx.x; ch < ((nchunks + 31) & ~31); ch += blockDim.x) {
        const bool live = ch < nchunks;
        const float4 v = live ? *reinterpret_cast<const float4 *>(x + 4 * ch) : make_float4(0, 0, 0, 0);
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

constexpr int kDenseThreads = 256;
constexpr int kDenseUnroll = 8;      // blocks in flight per lane (128 bytes of quants)

// One warp per tile of 32 rows, lane = row. Dynamic shared memory: cols bytes of quants + cols/32 floats.
// nb must be a multiple of kDenseUnroll.
__global__ void __launch_bounds__(kDenseThreads) q4_0_gemv_kernel(const uint8_t *wp, int rows, int nb, const float *x,
                                                                   float *y) {
    extern __shared__ __align__(16) uint8_t dsm[];
    uint8_t *xq = dsm;
    float *xd = reinterpret_cast<float *>(dsm + nb * 32);
    quantize_q8_0_plain_cta(x, nb * 32, xq, xd);
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int n_tiles = rows >> 5;
    const uint4 *q_all = reinterpret_cast<const uint4 *>(wp);
    const uint16_t *d_all = reinterpret_cast<const uint16_t *>(wp + static_cast<size_t>(rows) * nb * 16);
    const uint4 *a4 = reinterpret_cast<const uint4 *>(xq);
    for (int tile = blockIdx.x * nwarps + warp; tile < n_tiles; tile += gridDim.x * nwarps) {
        const uint4 *q = q_all + static_cast<size_t>(tile) * nb * 32 + lane;
        const uint16_t *d = d_all + static_cast<size_t>(tile) * nb * 32 + lane;
        float acc[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[c] = 0.0f;
#pragma unroll 1
        for (int b0 = 0; b0 < nb; b0 += kDenseUnroll) {
            uint4 w[kDenseUnroll];
            uint16_t dw[kDenseUnroll];
#pragma unroll
            for (int u = 0; u < kDenseUnroll; ++u) {        // the loads first: they stay in flight together
                w[u] = __ldg(q + (b0 + u) * 32);
                dw[u] = __ldg(d + (b0 + u) * 32);
            }
#pragma unroll
            for (int u = 0; u < kDenseUnroll; ++u) {
                const int b = b0 + u;
                const uint4 lo = a4[2 * b], hi = a4[2 * b + 1];
                // a nibble moved to the top of its byte and its top bit flipped is 16 * (q - 8) as int8;
                // the factor 16 goes into the scale (a power of two: exact)
                const float dd = __fmul_rn(__fmul_rn(half_bits_to_float(dw[u]), xd[b]), 0.0625f);
                const uint32_t ww[4] = {w[u].x, w[u].y, w[u].z, w[u].w};
                const uint32_t al[4] = {lo.x, lo.y, lo.z, lo.w}, ah[4] = {hi.x, hi.y, hi.z, hi.w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint32_t l16 = ((ww[k] << 4) & 0xf0f0f0f0u) ^ 0x80808080u;
                    const uint32_t h16 = (ww[k] & 0xf0f0f0f0u) ^ 0x80808080u;
                    acc[k] = __fmaf_rn(dd, static_cast<float>(dp4a_s8(static_cast<int>(l16), static_cast<int>(al[k]), 0)), acc[k]);
                    acc[k + 4] = __fmaf_rn(dd, static_cast<float>(dp4a_s8(static_cast<int>(h16), static_cast<int>(ah[k]), 0)), acc[k + 4]);
                }
            }
        }
        const float r0 = __fadd_rn(acc[0], acc[4]), r1 = __fadd_rn(acc[1], acc[5]);
        const float r2 = __fadd_rn(acc[2], acc[6]), r3 = __fadd_rn(acc[3], acc[7]);
        y[tile * 32 + lane] = __fadd_rn(__fadd_rn(r0, r2), __fadd_rn(r1, r3));
    }
}

// The same product for matrices with few rows, where one warp per tile leaves most of the GPU idle and
// walks a long dependent chain of loads: one CTA per tile of 32 rows. Segments of 64 blocks: the eight
// warps fetch and decode eight blocks each at once (integer sums as int16, the block scale as float, into
// shared memory), then thread (row, chunk-lane) runs its fmaf chain over the segment in block order. The
// float operations and their order are exactly those of q4_0_gemv_kernel.
constexpr int kDenseSeg = 64;
constexpr int kDenseSegSmem = kDenseSeg * 32 * (16 + 4);    // int16[8] + float per (block, row)

__global__ void __launch_bounds__(kDenseThreads) q4_0_gemv_tile_kernel(const uint8_t *wp, int rows, int nb,
                                                                        const float *x, float *y) {
    extern __shared__ __align__(16) uint8_t dsm[];
    uint8_t *xq = dsm;
    float *xd = reinterpret_cast<float *>(dsm + nb * 32);
    uint8_t *seg = dsm + ((nb * 36 + 15) & ~15);
    uint4 *pi = reinterpret_cast<uint4 *>(seg);                              // [block in segment][row] 8 x int16
    float *df = reinterpret_cast<float *>(seg + kDenseSeg * 32 * 16);       // [block in segment][row]
    quantize_q8_0_plain_cta(x, nb * 32, xq, xd);
    __syncthreads();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n_tiles = rows >> 5;
    const uint4 *q_all = reinterpret_cast<const uint4 *>(wp);
    const uint16_t *d_all = reinterpret_cast<const uint16_t *>(wp + static_cast<size_t>(rows) * nb * 16);
    const uint4 *a4 = reinterpret_cast<const uint4 *>(xq);
    const int16_t *ps = reinterpret_cast<const int16_t *>(seg);
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const uint4 *q = q_all + static_cast<size_t>(tile) * nb * 32 + lane;
        const uint16_t *d = d_all + static_cast<size_t>(tile) * nb * 32 + lane;
        float acc = 0.0f;                       // thread (row = tid / 8, chunk-lane = tid % 8)
#pragma unroll 1
        for (int s0 = 0; s0 < nb; s0 += kDenseSeg) {
            const int nseg = min(kDenseSeg, nb - s0);
            // phase A: warp w takes blocks s0 + w * 8 .. + 7 of the segment (lane = row)
            const int bw = warp * kDenseUnroll;
            if (bw < nseg) {
                uint4 w[kDenseUnroll];
                uint16_t dw[kDenseUnroll];
#pragma unroll
                for (int u = 0; u < kDenseUnroll; ++u) {
                    w[u] = __ldg(q + (s0 + bw + u) * 32);
                    dw[u] = __ldg(d + (s0 + bw + u) * 32);
                }
#pragma unroll
                for (int u = 0; u < kDenseUnroll; ++u) {
                    const int b = s0 + bw + u;
                    const uint4 lo = a4[2 * b], hi = a4[2 * b + 1];
                    const uint32_t ww[4] = {w[u].x, w[u].y, w[u].z, w[u].w};
                    const uint32_t al[4] = {lo.x, lo.y, lo.z, lo.w}, ah[4] = {hi.x, hi.y, hi.z, hi.w};
                    int p[8];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint32_t l16 = ((ww[k] << 4) & 0xf0f0f0f0u) ^ 0x80808080u;
                        const uint32_t h16 = (ww[k] & 0xf0f0f0f0u) ^ 0x80808080u;
                        p[k] = dp4a_s8(static_cast<int>(l16), static_cast<int>(al[k]), 0);          // 16 * sum, |.| <= 65,024
                        p[k + 4] = dp4a_s8(static_cast<int>(h16), static_cast<int>(ah[k]), 0);
                    }
                    // the sums are multiples of 16: stored divided by 16 they fit int16
                    uint32_t pk[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        pk[k] = (static_cast<uint32_t>(p[2 * k] >> 4) & 0xffffu) | (static_cast<uint32_t>(p[2 * k + 1] >> 4) << 16);
                    pi[(bw + u) * 32 + lane] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    df[(bw + u) * 32 + lane] = __fmul_rn(half_bits_to_float(dw[u]), xd[b]);
                }
            }
            __syncthreads();
            // phase B: the chains
            const int row = tid >> 3, c = tid & 7;
#pragma unroll 8
            for (int b = 0; b < nseg; ++b)
                acc = __fmaf_rn(df[b * 32 + row], static_cast<float>(ps[(b * 32 + row) * 8 + c]), acc);
            __syncthreads();
        }
        const float r = hsum8_lanes(acc);
        if ((tid & 7) == 0) y[tile * 32 + (tid >> 3)] = r;
    }
}

// ---------------------------------------------------------------------------------------------
// Output head: logits = W x for a Q8_0 matrix [vocab][hidden] fused with the arg-max over the finite
// logits (largest value, ties to the lowest index, non-finite values skipped and reported, token 0 when
// nothing is finite): q38_argmax_kernel (src/qwen38_forward.cuh:450-486) over the Q8_0 GEMV of
// src/qwen38_hc.cuh:1020; the multi-block reduction uses a monotone 64-bit key and atomicMax like
// dense_argmax_reduce_kernel (src/warodecode.cu:1603-1632). Row order of the float operations: ggml's
// Q8_0 x Q8_0 (src/qwen38_cpu_moe.cuh:424-440), the same as q8_task_row.
// Planar layout: tiles of 32 rows; quants of block b of the tile's row r at q[((t * nb + b) * 32 + r) * 2]
// (two 16-byte words), f16 scales after all quants in the same order.
// ---------------------------------------------------------------------------------------------
__global__ void repack_q8_0_planar_kernel(const uint8_t *src, uint8_t *dst, int rows, int nb) {
    const long long n = static_cast<long long>(rows) * nb;
    const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (i >= n) return;
    const int row = static_cast<int>(i / nb), b = static_cast<int>(i % nb);
    const uint8_t *blk = src + i * 34;
    const long long o = (static_cast<long long>(row >> 5) * nb + b) * 32 + (row & 31);
    uint32_t w[8];
#pragma unroll
    for (int k = 0; k < 8; ++k)
        w[k] = blk[2 + 4 * k] | (blk[3 + 4 * k] << 8) | (blk[4 + 4 * k] << 16) | (static_cast<uint32_t>(blk[5 + 4 * k]) << 24);
    uint4 *q = reinterpret_cast<uint4 *>(dst + o * 32);
    q[0] = make_uint4(w[0], w[1], w[2], w[3]);
    q[1] = make_uint4(w[4], w[5], w[6], w[7]);
    uint16_t *d = reinterpret_cast<uint16_t *>(dst + n * 32);
    d[o] = static_cast<uint16_t>(blk[0] | (blk[1] << 8));
}

constexpr int kHeadUnroll = 4;       // blocks in flight per lane (128 bytes of quants)

// key: one u64, zeroed before the launch; flags: [0] set when a non-finite logit was seen
__global__ void __launch_bounds__(kDenseThreads) q8_0_head_kernel(const uint8_t *wp, int rows, int nb, const float *x,
                                                                   float *y, unsigned long long *key, int *flags) {
    extern __shared__ __align__(16) uint8_t dsm[];
    uint8_t *xq = dsm;
    float *xd = reinterpret_cast<float *>(dsm + nb * 32);
    quantize_q8_0_plain_cta(x, nb * 32, xq, xd);
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int n_tiles = rows >> 5;
    const uint4 *q_all = reinterpret_cast<const uint4 *>(wp);
    const uint16_t *d_all = reinterpret_cast<const uint16_t *>(wp + static_cast<size_t>(rows) * nb * 32);
    const uint4 *a4 = reinterpret_cast<const uint4 *>(xq);
    unsigned long long best = 0ull;
    int nonfinite = 0;
    for (int tile = blockIdx.x * nwarps + warp; tile < n_tiles; tile += gridDim.x * nwarps) {
        const uint4 *q = q_all + (static_cast<size_t>(tile) * nb * 32 + lane) * 2;
        const uint16_t *d = d_all + static_cast<size_t>(tile) * nb * 32 + lane;
        float acc[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[c] = 0.0f;
#pragma unroll 1
        for (int b0 = 0; b0 < nb; b0 += kHeadUnroll) {
            uint4 w0[kHeadUnroll], w1[kHeadUnroll];
            uint16_t dw[kHeadUnroll];
#pragma unroll
            for (int u = 0; u < kHeadUnroll; ++u) {
                w0[u] = __ldg(q + (b0 + u) * 64);
                w1[u] = __ldg(q + (b0 + u) * 64 + 1);
                dw[u] = __ldg(d + (b0 + u) * 32);
            }
#pragma unroll
            for (int u = 0; u < kHeadUnroll; ++u) {
                const int b = b0 + u;
                const uint4 lo = a4[2 * b], hi = a4[2 * b + 1];
                const float dd = __fmul_rn(half_bits_to_float(dw[u]), xd[b]);
                const uint32_t ww[8] = {w0[u].x, w0[u].y, w0[u].z, w0[u].w, w1[u].x, w1[u].y, w1[u].z, w1[u].w};
                const uint32_t aa[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
                for (int c = 0; c < 8; ++c)
                    acc[c] = __fmaf_rn(dd, static_cast<float>(dp4a_s8(static_cast<int>(ww[c]), static_cast<int>(aa[c]), 0)), acc[c]);
            }
        }
        const float r0 = __fadd_rn(acc[0], acc[4]), r1 = __fadd_rn(acc[1], acc[5]);
        const float r2 = __fadd_rn(acc[2], acc[6]), r3 = __fadd_rn(acc[3], acc[7]);
        const float v = __fadd_rn(__fadd_rn(r0, r2), __fadd_rn(r1, r3));
        const int row = tile * 32 + lane;
        if (y) y[row] = v;
        if (isfinite(v)) {
            const uint32_t u = __float_as_uint(v + 0.0f);       // -0 and +0 compare equal: one key for both
            const uint32_t mono = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
            const unsigned long long k = (static_cast<unsigned long long>(mono) << 32) | static_cast<uint32_t>(~static_cast<uint32_t>(row));
            best = k > best ? k : best;
        } else {
            nonfinite = 1;
        }
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        const unsigned long long o = __shfl_xor_sync(0xffffffffu, best, s);
        best = o > best ? o : best;
    }
    nonfinite = __any_sync(0xffffffffu, nonfinite);
    if (lane == 0) {
        if (best != 0ull) atomicMax(key, best);
        if (nonfinite) atomicOr(flags, 1);
    }
}

// Embedding row of a Q8_0 table in ggml layout: out[i] = d(block) * q[i] for the row *token
// (token_embd lookup of the decoder, src/qwen38_forward.cuh: embedding gather before layer 0).
__global__ void embed_q8_0_kernel(const uint8_t *table, int rows, int nb, const int *token, float *out) {
    int t = *token;
    t = t < 0 ? 0 : (t >= rows ? rows - 1 : t);
    const uint8_t *row = table + static_cast<size_t>(t) * nb * 34;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < nb * 32; i += gridDim.x * blockDim.x) {
        const uint8_t *blk = row + (i >> 5) * 34;
        const float d = half_bits_to_float(static_cast<uint16_t>(blk[0] | (blk[1] << 8)));
        out[i] = __fmul_rn(d, static_cast<float>(static_cast<int8_t>(blk[2 + (i & 31)])));
    }
}

__global__ void head_finish_kernel(const unsigned long long *key, int *token) {
    const unsigned long long k = *key;
    *token = k == 0ull ? 0 : static_cast<int>(~static_cast<uint32_t>(k & 0xffffffffull));
}

}  // namespace wd
