// Load-time and test-only kernels: ggml -> device-format repacks, the synthetic weight
// generator, and single-purpose wrappers that expose pieces of the fused kernel to unit tests.
#pragma once

#include "wd_moe_fast.cuh"

namespace wd {

// ---------------------------------------------------------------------------------------------
// repack: ggml IQ3_S blocks (110 B: d, qs[64], qh[8], signs[32], scales[4]) -> tiles
// ---------------------------------------------------------------------------------------------
// blockIdx.y walks a batch of matrices `src_stride` / `dst_stride` bytes apart (one launch per layer).
__global__ void repack_iq3s_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, long long nblocks,
                                   long long src_stride, long long dst_stride) {
    const long long b = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (b >= nblocks) return;
    src += blockIdx.y * src_stride;
    dst += blockIdx.y * dst_stride;
    const uint8_t *s = src + b * 110;
    uint8_t *tile = dst + (b >> 5) * kIq3TileBytes;
    const int lane = static_cast<int>(b & 31);
    tile[kIq3OffD + lane * 2] = s[0];
    tile[kIq3OffD + lane * 2 + 1] = s[1];
    for (int i = 0; i < 8; ++i)
        for (int k = 0; k < 8; ++k) tile[i * 256 + lane * 8 + k] = s[2 + i * 8 + k];
    const uint8_t *qh = s + 66, *sg = s + 74;
    for (int i = 0; i < 8; ++i) {
        uint32_t word = 0;
        for (int c = 0; c < 8; ++c) {
            const uint32_t nib = (sg[i * 4 + (c >> 1)] >> (4 * (c & 1))) & 15u;
            for (int j = 0; j < 4; ++j)
                if ((nib >> j) & 1u) word |= 1u << (8 * j + 7 - c);
        }
        *reinterpret_cast<uint32_t *>(tile + kIq3OffSG + i * 128 + lane * 4) = word;
    }
    for (int k = 0; k < 8; ++k) tile[kIq3OffHB + lane * 8 + k] = qh[k];
    for (int k = 0; k < 4; ++k) tile[kIq3OffSC + lane * 4 + k] = s[106 + k];
}

// repack: ggml IQ2_S blocks (82 B) -> tiles of 32 blocks
__global__ void repack_iq2s_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, long long nblocks,
                                   long long src_stride, long long dst_stride) {
    const long long b = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (b >= nblocks) return;
    src += blockIdx.y * src_stride;
    dst += blockIdx.y * dst_stride;
    const uint8_t *s = src + b * 82;
    uint8_t *tile = dst + (b >> 5) * kIq2TileBytes;
    const int lane = static_cast<int>(b & 31);
    tile[kIq2OffD + lane * 2] = s[0];
    tile[kIq2OffD + lane * 2 + 1] = s[1];
    const uint8_t *qs = s + 2, *sg = s + 34, *qh = s + 66, *sc = s + 74;
    for (int i = 0; i < 8; ++i) {
        for (int k = 0; k < 4; ++k) tile[i * 128 + lane * 4 + k] = qs[i * 4 + k];
        uint32_t word = 0;
        for (int c = 0; c < 8; ++c) {
            const uint32_t nib = (sg[i * 4 + (c >> 1)] >> (4 * (c & 1))) & 15u;
            for (int j = 0; j < 4; ++j)
                if ((nib >> j) & 1u) word |= 1u << (8 * j + 7 - c);
        }
        *reinterpret_cast<uint32_t *>(tile + kIq2OffSG + i * 128 + lane * 4) = word;
        tile[kIq2OffQH + lane * 8 + i] = qh[i];
        tile[kIq2OffSC + lane * 8 + i] = sc[i];
    }
}

// repack: ggml Q8_0 [rows][nb] blocks (34 B) -> 4-row tasks
__global__ void repack_q8_0_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, int rows, int nb) {
    const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (i >= static_cast<long long>(rows) * nb) return;
    const int row = static_cast<int>(i / nb), b = static_cast<int>(i % nb);
    const uint8_t *s = src + i * 34;
    uint8_t *task = dst + static_cast<long long>(row >> 2) * nb * 136;
    const int r = row & 3;
    task[nb * 128 + (r * nb + b) * 2] = s[0];
    task[nb * 128 + (r * nb + b) * 2 + 1] = s[1];
    for (int l = 0; l < 8; ++l)
        for (int k = 0; k < 4; ++k) task[(b >> 2) * 512 + r * 128 + l * 16 + (b & 3) * 4 + k] = s[2 + 4 * l + k];
}

// repack: ggml Q8_0 [rows][nb] blocks (34 B) -> one row at a time (the layout q8_row_warp reads): quants
// [g = b / 4][chunk-lane l][16 B] (word b & 3 = values 4l..4l+3 of block b), then the nb f16 scales
__global__ void repack_q8_0_rows_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, int rows, int nb) {
    const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (i >= static_cast<long long>(rows) * nb) return;
    const int row = static_cast<int>(i / nb), b = static_cast<int>(i % nb);
    const uint8_t *s = src + i * 34;
    uint8_t *r = dst + static_cast<long long>(row) * nb * 34;
    r[nb * 32 + b * 2] = s[0];
    r[nb * 32 + b * 2 + 1] = s[1];
    for (int l = 0; l < 8; ++l)
        for (int k = 0; k < 4; ++k) r[(b >> 2) * 128 + l * 16 + (b & 3) * 4 + k] = s[2 + 4 * l + k];
}

// ---------------------------------------------------------------------------------------------
// synthetic weights: counter-based N(0, sigma), quantised to ggml block layouts on the device
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}
// Value `idx` of stream (seed, stream_id): Box-Muller on two 24-bit uniforms.
__device__ __forceinline__ float synth_normal(uint64_t seed, uint64_t stream_id, uint64_t idx) {
    const uint64_t h = mix64(mix64(seed * 0x9e3779b97f4a7c15ull + stream_id) + (idx >> 1));
    const float u1 = (static_cast<float>((h >> 40) & 0xffffffu) + 1.0f) * (1.0f / 16777216.0f);
    const float u2 = static_cast<float>((h >> 8) & 0xffffffu) * (1.0f / 16777216.0f);
    const float rad = sqrtf(-2.0f * logf(u1));
    float sn, cs;
    sincospif(2.0f * u2, &sn, &cs);
    return rad * ((idx & 1) ? sn : cs);
}

__global__ void synth_f32_kernel(float *dst, long long n, float sigma, uint64_t seed, uint64_t stream_id) {
    const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (i < n) dst[i] = sigma * synth_normal(seed, stream_id, static_cast<uint64_t>(i));
}

__global__ void synth_q8_0_kernel(uint8_t *dst, long long nblocks, float sigma, uint64_t seed, uint64_t stream_id) {
    const long long b = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (b >= nblocks) return;
    float v[32], amax = 0.0f;
    for (int i = 0; i < 32; ++i) {
        v[i] = sigma * synth_normal(seed, stream_id, static_cast<uint64_t>(b) * 32 + i);
        amax = fmaxf(amax, fabsf(v[i]));
    }
    const __half dh = __float2half_rn(amax / 127.0f);
    const float d = __half2float(dh);
    const float inv = d > 0.0f ? 1.0f / d : 0.0f;
    uint8_t *o = dst + b * 34;
    const uint16_t bits = __half_as_ushort(dh);
    o[0] = bits & 0xff;
    o[1] = bits >> 8;
    for (int i = 0; i < 32; ++i) o[2 + i] = static_cast<uint8_t>(max(-127, min(127, __float2int_rn(v[i] * inv))));
}

// Nearest codebook entry for each of the 16^4 cells of the magnitude cube (cell centre c + 0.5).
__global__ void synth_iq3s_lut_kernel(const uint16_t *grid_packed, uint16_t *lut) {
    const int cell = blockIdx.x * blockDim.x + threadIdx.x;
    if (cell >= 65536) return;
    float t[4];
    for (int j = 0; j < 4; ++j) t[j] = static_cast<float>((cell >> (12 - 4 * j)) & 15) + 0.5f;
    float best = 1e30f;
    int best_i = 0;
    for (int e = 0; e < 512; ++e) {
        const uint32_t p = grid_packed[e];
        float d2 = 0.0f;
        for (int j = 0; j < 4; ++j) {
            const float g = static_cast<float>(2 * ((p >> (3 * j)) & 7) + 1);
            d2 += (t[j] - g) * (t[j] - g);
        }
        if (d2 < best) {
            best = d2;
            best_i = e;
        }
    }
    lut[cell] = static_cast<uint16_t>(best_i);
}

// One thread per 256-value block: value = d * (1 + 2*s4) * (+-grid); same rule as the host encoder
// (per-32 target unit = max/13, d = max unit / 31, nearest entry by cell lookup).
__global__ void synth_iq3s_kernel(uint8_t *dst, long long first_block, long long nblocks, float sigma, uint64_t seed,
                                  uint64_t stream_id, const uint16_t *lut) {
    const long long b = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (b >= nblocks) return;
    const uint64_t base = static_cast<uint64_t>(first_block + b) * 256;
    float sub_max[8], top = 0.0f;
    for (int i = 0; i < 8; ++i) {
        float m = 0.0f;
        for (int k = 0; k < 32; ++k) m = fmaxf(m, fabsf(sigma * synth_normal(seed, stream_id, base + i * 32 + k)));
        sub_max[i] = m / 13.0f;
        top = fmaxf(top, sub_max[i]);
    }
    const __half dh = __float2half_rn(top / 31.0f);
    const float d = __half2float(dh);
    uint8_t *o = dst + b * 110;
    const uint16_t bits = __half_as_ushort(dh);
    o[0] = bits & 0xff;
    o[1] = bits >> 8;
    uint8_t scales[4] = {0, 0, 0, 0};
    for (int i = 0; i < 8; ++i) {
        int s4 = 0;
        if (d > 0.0f) s4 = max(0, min(15, __float2int_rn((sub_max[i] / d - 1.0f) * 0.5f)));
        scales[i >> 1] |= static_cast<uint8_t>(s4 << (4 * (i & 1)));
        const float unit = (d > 0.0f ? d : 1.0f) * static_cast<float>(1 + 2 * s4);
        uint8_t qh = 0;
        for (int c = 0; c < 8; ++c) {
            uint32_t cell = 0, nib = 0;
            for (int j = 0; j < 4; ++j) {
                const float w = sigma * synth_normal(seed, stream_id, base + i * 32 + c * 4 + j);
                const int q = min(15, static_cast<int>(fminf(fabsf(w) / unit, 15.999f)));
                cell = (cell << 4) | static_cast<uint32_t>(q);
                if (w < 0.0f) nib |= 1u << j;
            }
            const uint32_t idx = lut[cell];
            o[2 + i * 8 + c] = idx & 0xff;
            qh |= static_cast<uint8_t>(((idx >> 8) & 1u) << c);
            if (c & 1) o[74 + i * 4 + (c >> 1)] |= static_cast<uint8_t>(nib << 4);
            else o[74 + i * 4 + (c >> 1)] = static_cast<uint8_t>(nib);
        }
        o[66 + i] = qh;
    }
    for (int k = 0; k < 4; ++k) o[106 + k] = scales[k];
}

// ---------------------------------------------------------------------------------------------
// unit-test wrappers around the fused kernel's device functions
// ---------------------------------------------------------------------------------------------
__global__ void test_router_kernel(const float *logits, int E, int K, float w_scale, int *ids, float *weights,
                                   float *probs) {
    // launched with kThreads threads
    __shared__ float pr[kMaxExperts];
    __shared__ float gsum[kMaxExperts / 8];
    __shared__ float red[kWarps];
    __shared__ float first[2];
    __shared__ uint32_t cand[2 * kWarps * kMaxK];
    __shared__ int sid[kMaxK];
    __shared__ float sw[kMaxK];
    const int t = threadIdx.x;
    RouterScratch rs;
    rs.probs = pr; rs.gsum = gsum; rs.red = red; rs.first = first; rs.cand = cand;
    router_select_cta(t < E ? logits[t] : 0.0f, t + kThreads < E ? logits[t + kThreads] : 0.0f, E, K, w_scale, rs, sid, sw);
    for (int j = threadIdx.x; j < K; j += blockDim.x) {
        ids[j] = sid[j];
        weights[j] = sw[j];
    }
    if (probs)
        for (int i = threadIdx.x; i < E; i += blockDim.x) probs[i] = pr[i];
}

// Quantises n floats both ways with the fused kernel's routines and writes ggml block layouts.
__global__ void test_quantize_kernel(const float *x, int n, uint8_t *q80_blocks, uint8_t *q8k_blocks) {
    extern __shared__ __align__(16) uint8_t tsm[];
    float *xf = reinterpret_cast<float *>(tsm);
    uint8_t *q0 = tsm + n * 4;
    float *d0 = reinterpret_cast<float *>(q0 + n);
    uint8_t *qk = reinterpret_cast<uint8_t *>(d0 + n / 32);
    float *dk = reinterpret_cast<float *>(qk + (n / 256 + 1) * kActSbStride);
    for (int i = threadIdx.x; i < n; i += blockDim.x) xf[i] = x[i];
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (q80_blocks) {
        quantize_q8_0_cta(xf, n, q0, d0);
        __syncthreads();
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            const int b = i >> 5, l = (i & 31) >> 2, k = i & 3;
            q80_blocks[b * 34 + 2 + (i & 31)] = q0[((b >> 2) * 8 + l) * 16 + (b & 3) * 4 + k];
        }
        for (int b = threadIdx.x; b < n / 32; b += blockDim.x) {
            // d0 holds the f16-rounded scale as a float; the conversion back is exact
            *reinterpret_cast<__half *>(q80_blocks + b * 34) = __float2half_rn(d0[b]);
        }
    }
    if (q8k_blocks) {
        for (int sb = warp; sb < n / 256; sb += blockDim.x / 32)
            quantize_q8_K_warp(xf + sb * 256, lane, qk + sb * kActSbStride, &dk[sb]);
        __syncthreads();
        for (int sb = warp; sb < n / 256; sb += blockDim.x / 32) {
            uint8_t *o = q8k_blocks + sb * 292;
            if (lane == 0) *reinterpret_cast<float *>(o) = dk[sb];
            for (int j = 0; j < 8; ++j) o[4 + lane * 8 + j] = qk[sb * kActSbStride + lane * 8 + j];
            if (lane < 16) {
                int s = 0;
                for (int j = 0; j < 16; ++j) s += static_cast<int8_t>(qk[sb * kActSbStride + lane * 16 + j]);
                *reinterpret_cast<int16_t *>(o + 260 + lane * 2) = static_cast<int16_t>(s);
            }
        }
    }
}

// y = W x for a repacked IQ3_S matrix; one warp per tile, tile copied to shared memory with plain
// loads (no bulk copy), same decode and float chain as the fused kernel. x is quantised to Q8_K by
// the same routine. partials (optional): [rows][nsb][8] int32.
__global__ void iq_matvec_tiles_kernel(const uint8_t *tiles, int rows, int nsb, const float *x, float *y,
                                        int *partials, const uint16_t *grid_packed, int type = kTypeIq3s) {
    extern __shared__ __align__(128) uint8_t tsm[];
    uint8_t *tab = tsm;
    uint8_t *xk = tab + kGridTableBytes;
    float *xdk = reinterpret_cast<float *>(xk + nsb * kActSbStride);
    uint8_t *tile_s = reinterpret_cast<uint8_t *>(xdk + 32);
    float *scr_all = reinterpret_cast<float *>(tile_s + (blockDim.x / 32) * kIq3TileBytes);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x / 32;
    if (type == kTypeIq2s) build_iq2_table(tab, grid_packed);     // grid_packed is the codebook of `type`
    else build_grid_table(tab, grid_packed);
    for (int sb = warp; sb < nsb; sb += nw) quantize_q8_K_warp(x + sb * 256, lane, xk + sb * kActSbStride, &xdk[sb]);
    __syncthreads();
    const int R = 32 / nsb, ntiles = rows / R;
    const uint32_t lane4x2 = static_cast<uint32_t>(lane * 4) * 0x0101u;
    uint8_t *ts = tile_s + warp * kIq3TileBytes;
    float *scr = scr_all + warp * 640;          // 544 floats of chain scratch, then 32 row results
    float *rows_out = scr + 576;
    for (int t = blockIdx.x * nw + warp; t < ntiles; t += gridDim.x * nw) {
        const int tb = iq_tile_bytes(type);
        const uint4 *src = reinterpret_cast<const uint4 *>(tiles + static_cast<size_t>(t) * tb);
        for (int i = lane; i < tb / 16; i += 32) reinterpret_cast<uint4 *>(ts)[i] = src[i];
        __syncwarp();
        const int sb = lane % nsb, rl = lane / nsb;
        int *dump = partials ? partials + (static_cast<size_t>(t * R + rl) * nsb + sb) * 8 : nullptr;
        iq_tile_to_rows_any(type, ts, xk + sb * kActSbStride, xdk[sb], nsb, lane, lane4x2, tab, tab, scr, rows_out, dump);
        for (int rr = lane; rr < R; rr += 32) y[t * R + rr] = rows_out[rr];
        __syncwarp();
    }
}

// Measurement: how fast one SM decodes IQ3_S tiles that already sit in shared memory. `warps` warps of every CTA
// run `iters` rounds of one tile each (sixteen pseudo-random tiles, Q8_K activations of `nsb` superblocks);
// cycles[cta] = SM clock cycles of the slowest warp. The decoder is the layer kernels' own (iq3_tile_to_rows).
template <int UNROLL>
__global__ void __launch_bounds__(kThreads, 1) iq3_decoder_rate_kernel(const uint16_t *grid_packed, int nsb, int iters, int warps,
                                                                       unsigned long long *cycles, float *sink) {
    extern __shared__ __align__(128) uint8_t tsm[];
    uint8_t *tab = tsm;
    uint8_t *tiles = tab + kGridTableBytes;                   // 16 tiles
    uint8_t *act = tiles + 16 * kIq3TileBytes;                // 32 superblocks
    float *actd = reinterpret_cast<float *>(act + 32 * kActSbStride);
    float *scr_all = actd + 32;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    build_grid_table(tab, grid_packed);
    for (int i = tid; i < 16 * kIq3TileBytes; i += kThreads) tiles[i] = static_cast<uint8_t>((i * 2654435761u) >> 13);
    for (int i = tid; i < 32 * kActSbStride; i += kThreads) act[i] = static_cast<uint8_t>((i * 40503u) >> 7);
    if (tid < 32) actd[tid] = 0.01f;
    __syncthreads();
    float *scr = scr_all + warp * 640, *rows = scr + 576;
    const uint32_t lane4x2 = static_cast<uint32_t>(lane * 4) * 0x0101u;
    const int sb = lane % nsb;
    float acc = 0.0f;
    const long long t0 = clock64();
    if (warp < warps) {
#pragma unroll 1
        for (int it = 0; it < iters; ++it) {
            iq3_tile_to_rows<UNROLL>(tiles + ((warp + it) & 15) * kIq3TileBytes, act + sb * kActSbStride, actd[sb], nsb, lane, lane4x2,
                                     tab, scr, rows, nullptr);
            acc += rows[lane % (32 / nsb)];
        }
    }
    __syncthreads();
    if (tid == 0) cycles[blockIdx.x] = static_cast<unsigned long long>(clock64() - t0);
    sink[blockIdx.x * kThreads + tid] = acc;
}

// y = W x for a repacked Q8_0 matrix, one warp per 4-row task, x quantised to Q8_0 in shared memory.
__global__ void test_matvec_q8_0_kernel(const uint8_t *tasks, int rows, int nb, const float *x, float *y) {
    extern __shared__ __align__(128) uint8_t tsm[];
    const int n = nb * 32;
    float *xf = reinterpret_cast<float *>(tsm);
    uint8_t *xq = tsm + n * 4;
    float *xd = reinterpret_cast<float *>(xq + n);
    uint8_t *stage = reinterpret_cast<uint8_t *>(xd + nb);
    for (int i = threadIdx.x; i < n; i += blockDim.x) xf[i] = x[i];
    __syncthreads();
    quantize_q8_0_cta(xf, n, xq, xd);
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x / 32;
    const int task_bytes = nb * 136;
    uint8_t *ts = stage + warp * task_bytes;
    for (int t = blockIdx.x * nw + warp; t < rows / 4; t += gridDim.x * nw) {
        const uint4 *src = reinterpret_cast<const uint4 *>(tasks + static_cast<size_t>(t) * task_bytes);
        for (int i = lane; i < task_bytes / 16; i += 32) reinterpret_cast<uint4 *>(ts)[i] = src[i];
        __syncwarp();
        const float v = q8_task_row(ts, nb, xq, xd, lane);
        if ((lane & 7) == 0) y[t * 4 + (lane >> 3)] = v;
        __syncwarp();
    }
}

}  // namespace wd
