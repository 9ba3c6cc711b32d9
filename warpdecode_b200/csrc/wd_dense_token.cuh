// The plain Q4_0 decoder step as ONE persistent cooperative launch per token (the alternative to the graph of
// per-operation kernels in wd_dense_decoder.cuh; same arithmetic, same bits).
//
// Every CTA keeps its own copy of the residual stream in shared memory and owns a fixed share of the rows of every
// matrix. The weights of those rows travel through a ring of shared-memory slots as ONE stream per CTA, in the order
// they are needed (QKV rows, O rows, gate/up row pairs, down rows of layer 0, then layer 1, ..., then the head's
// rows): a warp that has consumed a slot asks at once for the row `ring` entries ahead, so the weight stream never
// waits for an activation and HBM latency is paid once per token, not once per product. Values that cross CTAs
// (QKV outputs, attention outputs, the two branch outputs, the SwiGLU activations, the arg-max candidates) are
// tagged words polled by their consumers, as in the MoE layer kernel: no grid barrier, every wait bounded.
// A phase is: all warps gather what the phase needs and prepare the Q8_0 activation in shared memory (block-wide),
// then the warps walk the CTA's rows of the phase round-robin.
// Exchange words of a phase are overwritten one layer later; two other exchanges lie in between, and a CTA passes an
// exchange only after every CTA has published into it, which each does after its reads of the previous one: no word
// is overwritten before its last reader has it.
#pragma once

#include "wd_dense_decoder.cuh"

namespace wd {

constexpr int kTokThreads = 512;
constexpr int kTokWarps = kTokThreads / 32;
constexpr int kTokMaxRing = 56;

struct DenseLayerDev {
    const uint8_t *wqkv, *wo, *w_gate_up, *w_down;     // row-packed: per row [nb * 16 B quants][nb * 2 B scales]
    const float *attn_norm, *ffn_norm;
    float *kcache, *vcache;                            // [max_ctx][kv_dim] of this layer
};

struct DenseTokenParams {
    int H, heads, kv_heads, head_dim, F, V, n_layers, max_ctx;
    float eps, inv_sqrt;
    const DenseLayerDev *layers;
    const uint8_t *token_embd;        // ggml layout
    const uint8_t *output;            // row-packed
    const float *output_norm;
    const float *rope;                // [max_ctx][head_dim / 2][2]
    int *token, *pos, *out_tokens;
    const int *forced;
    float *logits;                    // [V]
    float *hidden_out;                // [H] the residual stream before the output norm (CTA 0 writes it)
    tagged_t *t_qkv, *t_attn, *t_proj_o, *t_act, *t_proj_d, *t_key;   // [qkv_rows], [qdim], [H], [F], [H], [2 * grid]
    unsigned *sync;                   // [2] error word, [8] tag epoch, [9] count of CTAs that left
    unsigned long long *stamps;       // nullable: [16] SM clock of CTA 0's thread 0 at the steps of layer 1 (profiling)
    unsigned ring, slot_bytes;
    unsigned off_ring, off_bar, off_seq, off_hidden, off_xq, off_xd, off_attn;    // shared memory plan
};

// One row against the Q8_0 activation in shared memory; the row sits in shared memory as [nb * 16 B][nb * 2 B].
// The order is dense_gemv_q4_0_kernel's: lane l takes blocks l, l + 32, ... ascending, then the butterfly.
__device__ __forceinline__ float dense_row_smem(const uint8_t *row, int nb, const uint4 *sq, const float *sd, int lane) {
    const uint4 *q = reinterpret_cast<const uint4 *>(row);
    const uint16_t *d = reinterpret_cast<const uint16_t *>(row + static_cast<size_t>(nb) * 16);
    float acc = 0.0f;
#pragma unroll 2
    for (int b = lane; b < nb; b += 32) {
        const uint4 w = q[b];
        const uint4 lo = sq[2 * b], hi = sq[2 * b + 1];
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
        const uint32_t al[4] = {lo.x, lo.y, lo.z, lo.w}, ah[4] = {hi.x, hi.y, hi.z, hi.w};
        int s16 = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            s16 = dp4a_s8(static_cast<int>(((ww[k] << 4) & 0xf0f0f0f0u) ^ 0x80808080u), static_cast<int>(al[k]), s16);
            s16 = dp4a_s8(static_cast<int>((ww[k] & 0xf0f0f0f0u) ^ 0x80808080u), static_cast<int>(ah[k]), s16);
        }
        acc = __fmaf_rn(__fmul_rn(half_bits_to_float(d[b]), sd[b]), static_cast<float>(s16 >> 4), acc);
    }
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, s));
    return acc;
}

__global__ void __launch_bounds__(kTokThreads, 1) dense_token_kernel(const __grid_constant__ DenseTokenParams P) {
    extern __shared__ __align__(128) uint8_t tsm[];
    uint8_t *ring = tsm + P.off_ring;
    uint64_t *bars = reinterpret_cast<uint64_t *>(tsm + P.off_bar);
    int *ring_seq = reinterpret_cast<int *>(tsm + P.off_seq);
    float *hidden = reinterpret_cast<float *>(tsm + P.off_hidden);
    uint4 *sq = reinterpret_cast<uint4 *>(tsm + P.off_xq);
    int8_t *sq8 = reinterpret_cast<int8_t *>(tsm + P.off_xq);
    float *sd = reinterpret_cast<float *>(tsm + P.off_xd);
    float *att = reinterpret_cast<float *>(tsm + P.off_attn);      // scores [max_ctx], then q, k, v, out [128 each]
    __shared__ double red[kTokWarps];
    __shared__ unsigned long long best_sh[kTokWarps];
    unsigned *err = P.sync + 2;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cta = blockIdx.x, ncta = gridDim.x;
    const int H = P.H, F = P.F, hd = P.head_dim, qdim = P.heads * hd, kv_dim = P.kv_heads * hd, qkv_rows = qdim + 2 * kv_dim;
    const int nbH = H >> 5, nbQ = qdim >> 5, nbF = F >> 5;
    uint32_t epoch;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(epoch) : "l"(P.sync + 8) : "memory");
    const int pos = *P.pos;
    const int ns = static_cast<int>(P.ring);

    // ---- this CTA's stream of rows ------------------------------------------------------------------------------
    auto share = [&](int n) { return n > cta ? (n - cta + ncta - 1) / ncta : 0; };     // rows cta, cta + ncta, ... below n
    const int n_q = share(qkv_rows), n_o = share(H), n_p = share(F), n_d = share(H), n_h = share(P.V);
    const int per_layer = n_q + n_o + 2 * n_p + n_d;
    const int n_stream = P.n_layers * per_layer + n_h;
    // entry j of the stream: where its bytes are and how many
    auto entry = [&](int j, const uint8_t *&src, unsigned &bytes) {
        if (j >= P.n_layers * per_layer) {
            const int r = cta + (j - P.n_layers * per_layer) * ncta;
            bytes = static_cast<unsigned>(nbH) * 18u;
            src = P.output + static_cast<size_t>(r) * bytes;
            return;
        }
        const int l = j / per_layer;
        int o = j - l * per_layer;
        const DenseLayerDev &L = P.layers[l];
        if (o < n_q) {
            bytes = static_cast<unsigned>(nbH) * 18u;
            src = L.wqkv + static_cast<size_t>(cta + o * ncta) * bytes;
        } else if ((o -= n_q) < n_o) {
            bytes = static_cast<unsigned>(nbQ) * 18u;
            src = L.wo + static_cast<size_t>(cta + o * ncta) * bytes;
        } else if ((o -= n_o) < 2 * n_p) {
            bytes = static_cast<unsigned>(nbH) * 18u;
            src = L.w_gate_up + static_cast<size_t>((cta + (o >> 1) * ncta) + (o & 1) * F) * bytes;
        } else {
            o -= 2 * n_p;
            bytes = static_cast<unsigned>(nbF) * 18u;
            src = L.w_down + static_cast<size_t>(cta + o * ncta) * bytes;
        }
    };
    auto issue = [&](int j) {
        const uint8_t *src;
        unsigned bytes;
        entry(j, src, bytes);
        const int slot = j % ns;
        mbar_expect_tx(&bars[slot], bytes);
        bulk_load(ring + static_cast<size_t>(slot) * P.slot_bytes, src, bytes, &bars[slot]);
    };
    // row j of the stream has landed (waits for it); afterwards done(j) lets the slot be used for row j + ring
    auto row_ptr = [&](int j) -> const uint8_t * {
        const int slot = j % ns, round = j / ns;
        if (round > 0) {
            unsigned long long t0 = 0ull;
            for (unsigned it = 0; ld_acquire_shared(&ring_seq[slot]) < round; ++it)
                if (wait_expired(it, t0, err)) break;
        }
        mbar_wait(&bars[slot], static_cast<uint32_t>(round & 1), err);
        return ring + static_cast<size_t>(slot) * P.slot_bytes;
    };
    auto done = [&](int j) {
        __syncwarp();
        if (lane == 0 && j + ns < n_stream) {
            issue(j + ns);
            st_release_shared(&ring_seq[j % ns], (j + ns) / ns);
        }
    };

    if (tid < ns) {
        mbar_init(&bars[tid], 1);
        mbar_fence_init();
        ring_seq[tid] = 0;
    }
    __syncthreads();
    if (tid < min(ns, n_stream)) issue(tid);

    // ---- helpers of the phases ---------------------------------------------------------------------------------
    // hidden (shared, [H]) -> RMSNorm * w -> Q8_0 in sq / sd. H = 512 * EPL, EPL in {1, 2, 4, 8}: thread t owns EPL
    // consecutive elements; the sum of squares is the binary tree in double of the MoE stack's RMSNorm.
    auto norm_quant = [&](const float *w) {
        const int epl = H / kTokThreads;
        float v[8];
        double loc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[i] = i < epl ? hidden[tid * epl + i] : 0.0f;
            loc[i] = __dmul_rn(static_cast<double>(v[i]), static_cast<double>(v[i]));
        }
#pragma unroll
        for (int s = 1; s < 8; s <<= 1)
#pragma unroll
            for (int i = 0; i + s < 8; i += 2 * s)
                if (i + s < epl) loc[i] = __dadd_rn(loc[i], loc[i + s]);
        double ss = loc[0];
#pragma unroll
        for (int s = 1; s < 32; s <<= 1) ss = __dadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, s));
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        double tot[kTokWarps];
#pragma unroll
        for (int i = 0; i < kTokWarps; ++i) tot[i] = red[i];
#pragma unroll
        for (int s = 1; s < kTokWarps; s <<= 1)
#pragma unroll
            for (int i = 0; i + s < kTokWarps; i += 2 * s) tot[i] = __dadd_rn(tot[i], tot[i + s]);
        const float scale = __double2float_rn(
            __ddiv_rn(1.0, __dsqrt_rn(__dadd_rn(__ddiv_rn(tot[0], static_cast<double>(H)), static_cast<double>(P.eps)))));
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (i < epl) {
                v[i] = __fmul_rn(v[i], scale);
                if (w != nullptr) v[i] = __fmul_rn(v[i], w[tid * epl + i]);
                amax = fmaxf(amax, fabsf(v[i]));
            }
        for (int s = 1; s < 32 / epl; s <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, s));
        const float inv = amax != 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (i < epl) {
                int q = amax != 0.0f ? __float2int_rn(__fmul_rn(v[i], inv)) : 0;
                q = max(-128, min(127, q));
                sq8[tid * epl + i] = static_cast<int8_t>(q);
            }
        if (((tid * epl) & 31) == 0) sd[(tid * epl) >> 5] = __half2float(__float2half_rn(__fdiv_rn(amax, 127.0f)));
        __syncthreads();
    };
    // hidden += the n = H values published into `src` with tag `tag`
    auto add_branch = [&](const tagged_t *src, uint32_t tag) {
#pragma unroll 1
        for (int base = 0; base < H; base += 8 * kTokThreads) {         // up to eight words per thread in one round trip
            float v[8];
            const int n = min(8, (H - base - tid + kTokThreads - 1) / kTokThreads);
            wait_tagged<8>(src + base + tid, kTokThreads, n, tag, v, err);
#pragma unroll
            for (int k = 0; k < 8; ++k)
                if (k < n) hidden[base + tid + k * kTokThreads] = __fadd_rn(hidden[base + tid + k * kTokThreads], v[k]);
        }
        __syncthreads();
    };
    // n values published into `src` -> Q8_0 in sq / sd: a warp takes blocks warp, warp + 16, ..., four per round trip
    auto gather_quant = [&](const tagged_t *src, int n, uint32_t tag) {
        const int nblk = n >> 5;
        __syncthreads();        // the rows of the phase before still read the activation this one replaces
#pragma unroll 1
        for (int b0 = warp; b0 < nblk; b0 += 4 * kTokWarps) {
            float v[4];
            const int cnt = min(4, (nblk - b0 + kTokWarps - 1) / kTokWarps);
            wait_tagged<4>(src + b0 * 32 + lane, kTokWarps * 32, cnt, tag, v, err);
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (k < cnt) q8_0_block_warp(v[k], lane, sq8 + (b0 + k * kTokWarps) * 32, sd + b0 + k * kTokWarps);
        }
        __syncthreads();
    };

#define WD_TSTAMP(i)                                                                              \
    if (P.stamps != nullptr && tid == 0 && cta == P.heads && l == 1) {                            \
        unsigned long long c__;                                                                   \
        asm volatile("mov.u64 %0, %%clock64;" : "=l"(c__) : : "memory");                          \
        P.stamps[i] = c__;                                                                        \
    }
    const uint32_t tag0 = epoch + 1u;           // tag of (layer l, phase p) = tag0 + 8 l + p
    int j0 = 0;                                 // first stream entry of the current phase
    // ---- the embedding row starts the residual stream -------------------------------------------------------------
    {
        const int tok = max(0, min(P.V - 1, *P.token));
        const uint8_t *row = P.token_embd + static_cast<size_t>(tok) * nbH * 18;
        for (int e = tid; e < H; e += kTokThreads) {
            const int b = e >> 5, j = e & 31;
            const uint8_t *wb = row + b * 18;
            const float d = half_bits_to_float(static_cast<uint16_t>(wb[0] | (wb[1] << 8)));
            const int q = j < 16 ? (wb[2 + j] & 0x0f) : (wb[2 + j - 16] >> 4);
            hidden[e] = __fmul_rn(d, static_cast<float>(q - 8));
        }
        __syncthreads();
    }
#pragma unroll 1
    for (int l = 0; l < P.n_layers; ++l) {
        const DenseLayerDev L = P.layers[l];
        const uint32_t tg = tag0 + 8u * static_cast<uint32_t>(l);
        // ---- A: (previous layer's down branch) + attention norm; B: QKV rows ---------------------------------------
        WD_TSTAMP(0);
        if (l > 0) add_branch(P.t_proj_d, tg - 8u + 4u);
        WD_TSTAMP(1);
        norm_quant(L.attn_norm);
        WD_TSTAMP(2);
        for (int k = warp; k < n_q; k += kTokWarps) {
            const float v = dense_row_smem(row_ptr(j0 + k), nbH, sq, sd, lane);
            done(j0 + k);
            if (lane == 0) st_tagged(P.t_qkv + cta + k * ncta, v, tg + 0u);
        }
        j0 += n_q;
        WD_TSTAMP(3);
        // ---- C: attention, one CTA per query head -----------------------------------------------------------------
        if (cta < P.heads) {
            const int h = cta, kvh = (h * P.kv_heads) / P.heads, half = hd / 2;
            float *sc = att, *qs = att + P.max_ctx, *kn = qs + 128, *vn = kn + 128, *outv = vn + 128;
            if (tid < 3 * hd) {
                const int which = tid / hd, d = tid - which * hd;
                const int idx = which == 0 ? h * hd + d : which == 1 ? qdim + kvh * hd + d : qdim + kv_dim + kvh * hd + d;
                float v[1];
                wait_tagged<1>(P.t_qkv + idx, 1, 1, tg + 0u, v, err);
                (which == 0 ? qs : which == 1 ? kn : vn)[d] = v[0];
            }
            __syncthreads();
            if (tid < half) {       // rotary embedding of q and of the new k (GPT-NeoX pairing), in place
                const float cs = P.rope[(static_cast<size_t>(pos) * half + tid) * 2], sn = P.rope[(static_cast<size_t>(pos) * half + tid) * 2 + 1];
                const float a = qs[tid], b = qs[tid + half];
                qs[tid] = __fadd_rn(__fmul_rn(a, cs), -__fmul_rn(b, sn));
                qs[tid + half] = __fadd_rn(__fmul_rn(a, sn), __fmul_rn(b, cs));
                const float c = kn[tid], e = kn[tid + half];
                kn[tid] = __fadd_rn(__fmul_rn(c, cs), -__fmul_rn(e, sn));
                kn[tid + half] = __fadd_rn(__fmul_rn(c, sn), __fmul_rn(e, cs));
            }
            __syncthreads();
            float *kc = L.kcache + static_cast<size_t>(kvh) * hd, *vc = L.vcache + static_cast<size_t>(kvh) * hd;
            if (h % (P.heads / P.kv_heads) == 0 && tid < hd) {      // the first head of its KV group stores k and v
                kc[static_cast<size_t>(pos) * kv_dim + tid] = kn[tid];
                vc[static_cast<size_t>(pos) * kv_dim + tid] = vn[tid];
            }
            const float o = dense_attention_core(qs, kn, vn, kc, vc, pos, kv_dim, hd, P.inv_sqrt, sc, outv + 128, kTokThreads);
            if (tid < hd) st_tagged(P.t_attn + h * hd + tid, o, tg + 1u);
            (void)outv;
            __syncthreads();
        }
        // ---- D: attention output -> Q8_0; O rows --------------------------------------------------------------------
        WD_TSTAMP(4);
        gather_quant(P.t_attn, qdim, tg + 1u);
        WD_TSTAMP(5);
        for (int k = warp; k < n_o; k += kTokWarps) {
            const float v = dense_row_smem(row_ptr(j0 + k), nbQ, sq, sd, lane);
            done(j0 + k);
            if (lane == 0) st_tagged(P.t_proj_o + cta + k * ncta, v, tg + 2u);
        }
        j0 += n_o;
        // ---- E: + attention branch, FFN norm; F: gate/up row pairs -> SiLU(g) * u ----------------------------------
        WD_TSTAMP(6);
        add_branch(P.t_proj_o, tg + 2u);
        WD_TSTAMP(7);
        norm_quant(L.ffn_norm);
        WD_TSTAMP(8);
        for (int k = warp; k < n_p; k += kTokWarps) {
            const float g = dense_row_smem(row_ptr(j0 + 2 * k), nbH, sq, sd, lane);
            done(j0 + 2 * k);
            const float u = dense_row_smem(row_ptr(j0 + 2 * k + 1), nbH, sq, sd, lane);
            done(j0 + 2 * k + 1);
            if (lane == 0) st_tagged(P.t_act + cta + k * ncta, __fmul_rn(silu_ggml(g), u), tg + 3u);
        }
        j0 += 2 * n_p;
        // ---- G: activations -> Q8_0; down rows ----------------------------------------------------------------------
        WD_TSTAMP(9);
        gather_quant(P.t_act, F, tg + 3u);
        WD_TSTAMP(10);
        for (int k = warp; k < n_d; k += kTokWarps) {
            const float v = dense_row_smem(row_ptr(j0 + k), nbF, sq, sd, lane);
            done(j0 + k);
            if (lane == 0) st_tagged(P.t_proj_d + cta + k * ncta, v, tg + 4u);
        }
        j0 += n_d;
        WD_TSTAMP(11);
    }
#undef WD_TSTAMP
    // ---- output norm, head rows with the running arg-max -------------------------------------------------------------
    const uint32_t tgl = tag0 + 8u * static_cast<uint32_t>(P.n_layers);
    add_branch(P.t_proj_d, tgl - 8u + 4u);
    if (cta == 0)
        for (int e = tid; e < H; e += kTokThreads) P.hidden_out[e] = hidden[e];
    norm_quant(P.output_norm);
    unsigned long long best = 0ull;
    for (int k = warp; k < n_h; k += kTokWarps) {
        const float v = dense_row_smem(row_ptr(j0 + k), nbH, sq, sd, lane);
        done(j0 + k);
        const int row = cta + k * ncta;
        if (lane == 0) {
            P.logits[row] = v;
            if (v == v && fabsf(v) != INFINITY) {
                const unsigned long long key = (static_cast<unsigned long long>(order_key(v)) << 32) | (0xffffffffu - static_cast<unsigned>(row));
                best = key > best ? key : best;
            }
        }
    }
    if (lane == 0) best_sh[warp] = best;
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < kTokWarps; ++w) best = best_sh[w] > best ? best_sh[w] : best;
        st_tagged(P.t_key + 2 * cta, __uint_as_float(static_cast<uint32_t>(best >> 32)), tgl + 0u);
        st_tagged(P.t_key + 2 * cta + 1, __uint_as_float(static_cast<uint32_t>(best)), tgl + 0u);
    }
    // CTA 0 collects the candidates, fixes the token and advances the position (dense_finish_kernel)
    if (cta == 0) {
        unsigned long long mine = 0ull;
        for (int c = tid; c < ncta; c += kTokThreads) {
            float v[2];
            wait_tagged<2>(P.t_key + 2 * c, 1, 2, tgl + 0u, v, err);
            const unsigned long long key = (static_cast<unsigned long long>(__float_as_uint(v[0])) << 32) | __float_as_uint(v[1]);
            mine = key > mine ? key : mine;
        }
#pragma unroll
        for (int s = 16; s >= 1; s >>= 1) {
            const unsigned long long o = __shfl_xor_sync(0xffffffffu, mine, s);
            mine = o > mine ? o : mine;
        }
        __syncthreads();
        if (lane == 0) best_sh[warp] = mine;
        __syncthreads();
        if (tid == 0) {
            for (int w = 0; w < kTokWarps; ++w) mine = best_sh[w] > mine ? best_sh[w] : mine;
            int t = mine == 0ull ? 0 : static_cast<int>(0xffffffffu - static_cast<unsigned>(mine & 0xffffffffull));
            const int p = pos + 1;
            if (P.forced != nullptr && P.forced[p] >= 0) t = P.forced[p];
            P.out_tokens[p] = t;
            *P.token = t;
            *P.pos = p;
        }
    }
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(P.sync + 9, 1u) == static_cast<unsigned>(ncta) - 1u) {
            P.sync[9] = 0u;
            P.sync[8] = epoch + 8u * static_cast<uint32_t>(P.n_layers) + 8u;
        }
    }
}

}  // namespace wd
