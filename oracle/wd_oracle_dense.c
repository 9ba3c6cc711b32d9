/* CPU oracle of the plain (dense) Q4_0 decoder step. TEST INFRASTRUCTURE: only tests/, the smoke check and the
 * bench's CPU baseline may link or call this file; the product never does.
 *
 * What it restates: the dense decoder step of the reference, Runtime::emit_step (src/warodecode.cu:2053-2104):
 * embedding row (embedding_q4_kernel) -> per layer [residual add + RMSNorm + Q8_0 activation
 * (residual_rmsnorm_kernel :1408), fused QKV product (q4_0_q8_0_gemv_kernel :1535), rotary embedding in the GPT-NeoX
 * pairing and the cache store (rope_store_kernel :1855), decode attention (attention_decode_kernel :1902), output
 * product, residual add + RMSNorm + Q8_0, gate/up product, SiLU(g) * u + Q8_0 (swiglu_kernel :1956), down product]
 * -> residual add + output norm -> output head -> arg-max, largest value, ties to the lowest index
 * (dense_argmax_reduce_kernel :1603-1644).
 *
 * The reference has NO host twin of this path and states that it carries no exactness contract
 * (src/warodecode.cu:1490-1491: dp4a reassociation is fine; activations travel as F16 between its kernels). Parity
 * for the dense path is therefore UNPINNED against the reference: no golden vector or CPU code of the reference
 * exists for it. This file fixes one float order for every step (stated at each function), keeps activations in F32,
 * and the CUDA path must reproduce it bit for bit; the building blocks it shares with the MoE oracle (Q8_0 quantiser,
 * f16 conversions, exp, SiLU, RMSNorm) are pinned against the reference there, and the Q4_0 block decode is pinned
 * against gguf-py (tests/test_oracle_pins.py).
 */
#define _POSIX_C_SOURCE 200809L
#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include "wd_oracle.h"

#define Q4_BYTES 18
#define Q8_BYTES 34

static float mulf(float a, float b) { volatile float r = a * b; return r; }
static float addf(float a, float b) { volatile float r = a + b; return r; }

/* One row of a Q4_0 matrix against a Q8_0 activation, in the order of a warp that splits the row's blocks over
 * its 32 lanes: lane l runs acc = fmaf(d_w * d_x, (float)int_dot(block b), acc) over b = l, l + 32, ... ascending
 * (int_dot = sum of (q - 8) * a over the block's 32 values, exact), then the lanes meet in a butterfly:
 * v += v[lane ^ 16], ^8, ^4, ^2, ^1. Values 0..15 of a block are the low nibbles of its 16 bytes, 16..31 the high. */
float wdo_row_q4_0_q8_0_lanes(const uint8_t *w_row, const uint8_t *y, int cols) {
    const int nb = cols / 32;
    float lane[32];
    for (int l = 0; l < 32; ++l) lane[l] = 0.0f;
    for (int b = 0; b < nb; ++b) {
        const uint8_t *wb = w_row + (size_t)b * Q4_BYTES;
        const uint8_t *yb = y + (size_t)b * Q8_BYTES;
        const int8_t *yq = (const int8_t *)(yb + 2);
        uint16_t dw, dy;
        memcpy(&dw, wb, 2);
        memcpy(&dy, yb, 2);
        int sum = 0;
        for (int j = 0; j < 16; ++j) {
            sum += ((int)(wb[2 + j] & 0x0f) - 8) * yq[j];
            sum += ((int)(wb[2 + j] >> 4) - 8) * yq[j + 16];
        }
        const float d = mulf(wdo_f16_to_f32(dw), wdo_f16_to_f32(dy));
        lane[b & 31] = fmaf(d, (float)sum, lane[b & 31]);
    }
    for (int s = 16; s >= 1; s >>= 1) {
        float next[32];
        for (int l = 0; l < 32; ++l) next[l] = addf(lane[l], lane[l ^ s]);
        memcpy(lane, next, sizeof(lane));
    }
    return lane[0];
}

/* The same for a Q8_0 matrix (the form every 2-D tensor that is not Q4_0 takes in the reference's dense loader,
 * planarize_q4, src/warodecode.cu:1027-1075): int_dot = sum of q_w * a over the block's 32 values. */
float wdo_row_q8_0_q8_0_lanes(const uint8_t *w_row, const uint8_t *y, int cols) {
    const int nb = cols / 32;
    float lane[32];
    for (int l = 0; l < 32; ++l) lane[l] = 0.0f;
    for (int b = 0; b < nb; ++b) {
        const uint8_t *wb = w_row + (size_t)b * Q8_BYTES;
        const uint8_t *yb = y + (size_t)b * Q8_BYTES;
        const int8_t *wq = (const int8_t *)(wb + 2), *yq = (const int8_t *)(yb + 2);
        uint16_t dw, dy;
        memcpy(&dw, wb, 2);
        memcpy(&dy, yb, 2);
        int sum = 0;
        for (int j = 0; j < 32; ++j) sum += (int)wq[j] * (int)yq[j];
        const float d = mulf(wdo_f16_to_f32(dw), wdo_f16_to_f32(dy));
        lane[b & 31] = fmaf(d, (float)sum, lane[b & 31]);
    }
    for (int s = 16; s >= 1; s >>= 1) {
        float next[32];
        for (int l = 0; l < 32; ++l) next[l] = addf(lane[l], lane[l ^ s]);
        memcpy(lane, next, sizeof(lane));
    }
    return lane[0];
}

/* y = W x for W [rows][cols] in ggml Q4_0 or Q8_0 blocks, x already Q8_0. Rows are independent: the thread count does
 * not change a bit. */
typedef struct {
    const uint8_t *w, *xq;
    float *y;
    int cols, r0, r1, type;
} mv_job;

static void *mv_worker(void *arg) {
    const mv_job *j = (const mv_job *)arg;
    const int q8 = j->type == WDO_TYPE_Q8_0;
    const size_t row_bytes = (size_t)(j->cols / 32) * (q8 ? Q8_BYTES : Q4_BYTES);
    for (int r = j->r0; r < j->r1; ++r)
        j->y[r] = q8 ? wdo_row_q8_0_q8_0_lanes(j->w + (size_t)r * row_bytes, j->xq, j->cols)
                     : wdo_row_q4_0_q8_0_lanes(j->w + (size_t)r * row_bytes, j->xq, j->cols);
    return NULL;
}

void wdo_matvec_q4_0(const uint8_t *w, int rows, int cols, const uint8_t *xq, float *y) { wdo_matvec_typed(WDO_TYPE_Q4_0, w, rows, cols, xq, y); }

void wdo_matvec_typed(int type, const uint8_t *w, int rows, int cols, const uint8_t *xq, float *y) {
    long ncpu = sysconf(_SC_NPROCESSORS_ONLN);
    int nt = ncpu > 16 ? 16 : (ncpu < 1 ? 1 : (int)ncpu);
    if (rows < 256) nt = 1;
    mv_job jobs[16];
    pthread_t th[16];
    for (int t = 0; t < nt; ++t) {
        jobs[t].w = w; jobs[t].xq = xq; jobs[t].y = y; jobs[t].cols = cols; jobs[t].type = type;
        jobs[t].r0 = (int)((long long)rows * t / nt);
        jobs[t].r1 = (int)((long long)rows * (t + 1) / nt);
    }
    for (int t = 1; t < nt; ++t)
        if (pthread_create(&th[t], NULL, mv_worker, &jobs[t]) != 0) {       /* no thread: do the share here */
            mv_worker(&jobs[t]);
            th[t] = (pthread_t)0;
            jobs[t].r0 = jobs[t].r1;
        }
    mv_worker(&jobs[0]);
    for (int t = 1; t < nt; ++t)
        if (jobs[t].r0 != jobs[t].r1 || th[t] != (pthread_t)0) {
            if (th[t] != (pthread_t)0) pthread_join(th[t], NULL);
        }
}

/* Embedding row: value i = d(block) * (q - 8), one float multiply (embedding_q4_kernel). */
void wdo_embed_q4_0(const uint8_t *table, int cols, int token, float *out) {
    const uint8_t *row = table + (size_t)token * (size_t)(cols / 32) * Q4_BYTES;
    for (int b = 0; b < cols / 32; ++b) {
        const uint8_t *wb = row + (size_t)b * Q4_BYTES;
        uint16_t dw;
        memcpy(&dw, wb, 2);
        const float d = wdo_f16_to_f32(dw);
        for (int j = 0; j < 16; ++j) {
            out[b * 32 + j] = mulf(d, (float)((int)(wb[2 + j] & 0x0f) - 8));
            out[b * 32 + 16 + j] = mulf(d, (float)((int)(wb[2 + j] >> 4) - 8));
        }
    }
}

/* Embedding row of a Q8_0 table: value i = d(block) * q, one float multiply. */
void wdo_embed_q8_0(const uint8_t *table, int cols, int token, float *out) {
    const uint8_t *row = table + (size_t)token * (size_t)(cols / 32) * Q8_BYTES;
    for (int b = 0; b < cols / 32; ++b) {
        const uint8_t *wb = row + (size_t)b * Q8_BYTES;
        uint16_t dw;
        memcpy(&dw, wb, 2);
        const float d = wdo_f16_to_f32(dw);
        for (int j = 0; j < 32; ++j) out[b * 32 + j] = mulf(d, (float)(int8_t)wb[2 + j]);
    }
}

/* One value of a Q6_K block (210 bytes per 256 values: ql(128) qh(64) scales(16, int8) d(2)); the expression of
 * ggml_q6_k_value, src/ggml_dequant.hpp:102-133: (d * scale) * (v - 32), two float multiplies. */
float wdo_q6_k_value(const uint8_t *blk, int i) {
    const uint8_t *ql = blk, *qh = blk + 128;
    const int8_t *sc = (const int8_t *)(blk + 192);
    uint16_t db;
    memcpy(&db, blk + 208, 2);
    const float d = wdo_f16_to_f32(db);
    const int half = i >> 7, r = i & 127, l = r & 31, q = r >> 5;
    const uint8_t *ql64 = ql + half * 64, *qh32 = qh + half * 32;
    const int8_t *sc8 = sc + half * 8;
    int v;
    if (q == 0) v = (ql64[l] & 0x0f) | (((qh32[l] >> 0) & 3) << 4);
    else if (q == 1) v = (ql64[l + 32] & 0x0f) | (((qh32[l] >> 2) & 3) << 4);
    else if (q == 2) v = (ql64[l] >> 4) | (((qh32[l] >> 4) & 3) << 4);
    else v = (ql64[l + 32] >> 4) | (((qh32[l] >> 6) & 3) << 4);
    return mulf(mulf(d, (float)sc8[(l >> 4) + 2 * q]), (float)(v - 32));
}

/* A row of a tensor that is not Q4_0, turned into Q8_0 blocks the way the reference's dense loader does it on the host
 * (ggml_requantize_row_to_q8_0, src/ggml_dequant.hpp:362-392): per 32 values d = amax / 127 in F32, stored rounded to
 * f16, quant = lround(v / d) with the UNROUNDED d, clamped to [-128, 127]. Source types: Q8_0 (8) and Q6_K (14).
 * Returns 0, or -1 for another type or a column count that does not fit. */
int wdo_requantize_row_to_q8_0(int type, const uint8_t *src, uint8_t *dst, int cols) {
    if (cols % 32 || (type != WDO_TYPE_Q8_0 && type != 14) || (type == 14 && cols % 256)) return -1;
    for (int b = 0; b < cols / 32; ++b) {
        float v[32], amax = 0.0f;
        for (int i = 0; i < 32; ++i) {
            const int idx = b * 32 + i;
            if (type == WDO_TYPE_Q8_0) {
                const uint8_t *bp = src + (size_t)(idx / 32) * Q8_BYTES;
                uint16_t dw;
                memcpy(&dw, bp, 2);
                v[i] = mulf(wdo_f16_to_f32(dw), (float)(int8_t)bp[2 + (idx & 31)]);
            } else {
                v[i] = wdo_q6_k_value(src + (size_t)(idx / 256) * 210, idx & 255);
            }
            if (fabsf(v[i]) > amax) amax = fabsf(v[i]);
        }
        const float d = amax / 127.0f;
        uint8_t *out = dst + (size_t)b * Q8_BYTES;
        const uint16_t dh = wdo_f32_to_f16(d);
        memcpy(out, &dh, 2);
        for (int i = 0; i < 32; ++i) {
            long q = d == 0.0f ? 0 : lroundf(v[i] / d);
            if (q > 127) q = 127;
            if (q < -128) q = -128;
            out[2 + i] = (uint8_t)(int8_t)q;
        }
    }
    return 0;
}

/* cos/sin table of the rotary embedding: angle = pos * theta^(-2p / head_dim) in double, rounded to float once.
 * The product uploads this table, so that both sides rotate with the same factors. [max_ctx][head_dim / 2][2] */
void wdo_rope_table(int max_ctx, int head_dim, double theta, float *table) {
    const int half = head_dim / 2;
    for (int pos = 0; pos < max_ctx; ++pos)
        for (int p = 0; p < half; ++p) {
            const double ang = (double)pos * pow(theta, -2.0 * (double)p / (double)head_dim);
            table[((size_t)pos * half + p) * 2] = (float)cos(ang);
            table[((size_t)pos * half + p) * 2 + 1] = (float)sin(ang);
        }
}

/* GPT-NeoX pairing (rope_store_kernel): pair p rotates elements p and p + head_dim / 2 of a head;
 * x0' = x0 * cos - x1 * sin, x1' = x0 * sin + x1 * cos, each product and sum rounded separately. */
static void rope_head(float *v, int head_dim, const float *cs) {
    const int half = head_dim / 2;
    for (int p = 0; p < half; ++p) {
        const float a = v[p], b = v[p + half], c = cs[2 * p], s = cs[2 * p + 1];
        v[p] = addf(mulf(a, c), -mulf(b, s));
        v[p + half] = addf(mulf(a, s), mulf(b, c));
    }
}

/* Decode attention of one head over cache positions 0..pos (attention_decode_kernel, as two passes):
 * score_t = (q . k_t) * inv_sqrt with the dot product in the warp order (lane l sums d = l, l + 32, ... by fmaf,
 * then the butterfly ^16 .. ^1); m = max score; p_t = exp(score_t - m); l = sum of p_t ascending;
 * out_d = fmaf(p_t, v_t[d], out_d) ascending in t, divided by l at the end. */
static void attention_head(const float *q, const float *kc, const float *vc, size_t kv_stride, int pos, int head_dim,
                           float inv_sqrt, float *out, float *scratch) {
    float m = -INFINITY;
    for (int t = 0; t <= pos; ++t) {
        const float *k = kc + (size_t)t * kv_stride;
        float lane[32];
        for (int l = 0; l < 32; ++l) {
            float acc = 0.0f;
            for (int d = l; d < head_dim; d += 32) acc = fmaf(q[d], k[d], acc);
            lane[l] = acc;
        }
        for (int s = 16; s >= 1; s >>= 1) {
            float next[32];
            for (int l = 0; l < 32; ++l) next[l] = addf(lane[l], lane[l ^ s]);
            memcpy(lane, next, sizeof(lane));
        }
        scratch[t] = mulf(lane[0], inv_sqrt);
        if (scratch[t] > m) m = scratch[t];
    }
    float l = 0.0f;
    for (int t = 0; t <= pos; ++t) {
        scratch[t] = wdo_exp_ggml(addf(scratch[t], -m));
        l = addf(l, scratch[t]);
    }
    for (int d = 0; d < head_dim; ++d) {
        float acc = 0.0f;
        for (int t = 0; t <= pos; ++t) acc = fmaf(scratch[t], vc[(size_t)t * kv_stride + d], acc);
        out[d] = acc / l;
    }
}

/* One decoder step: token at position pos -> next token (greedy). `logits_out` optional [vocab]. The caches
 * [layer][max_ctx][kv_heads * head_dim] are updated in place. Returns the arg-max over the finite logits (largest
 * value, ties to the lowest index; 0 if none is finite). */
int wdo_dense_step(const wdo_dense_model *m, float *kcache, float *vcache, int token, int pos, float *logits_out) {
    const int H = m->hidden, hd = m->head_dim, nh = m->n_heads, nkv = m->n_kv_heads, F = m->ffn, V = m->vocab;
    const int qdim = nh * hd, kvdim = nkv * hd, qkv_rows = qdim + 2 * kvdim;
    const int maxn = H > F ? H : F;
    float *hidden = (float *)malloc(sizeof(float) * H);
    float *norm = (float *)malloc(sizeof(float) * maxn);
    float *qkv = (float *)malloc(sizeof(float) * qkv_rows);
    float *attn = (float *)malloc(sizeof(float) * qdim);
    float *proj = (float *)malloc(sizeof(float) * H);
    float *gu = (float *)malloc(sizeof(float) * 2 * F);
    float *scores = (float *)malloc(sizeof(float) * m->max_ctx);
    uint8_t *xq = (uint8_t *)malloc((size_t)(maxn / 32) * Q8_BYTES);
    float *logits = logits_out ? logits_out : (float *)malloc(sizeof(float) * V);
    const float inv_sqrt = (float)(1.0 / sqrt((double)hd));
    const float *cs = m->rope_table + (size_t)pos * (hd / 2) * 2;
    if (m->token_embd_type == WDO_TYPE_Q8_0) wdo_embed_q8_0(m->token_embd, H, token, hidden);
    else wdo_embed_q4_0(m->token_embd, H, token, hidden);
    for (int li = 0; li < m->n_layers; ++li) {
        const wdo_dense_layer *L = &m->layers[li];
        float *kc = kcache + (size_t)li * m->max_ctx * kvdim, *vc = vcache + (size_t)li * m->max_ctx * kvdim;
        if (li > 0)
            for (int i = 0; i < H; ++i) hidden[i] = addf(hidden[i], proj[i]);
        wdo_rmsnorm(hidden, L->attn_norm, m->rms_eps, H, norm);
        wdo_quantize_q8_0(norm, xq, H / 32);
        wdo_matvec_typed(L->wqkv_type, L->wqkv, qkv_rows, H, xq, qkv);
        /* bias, then the per-head norms, then the rotary embedding: the order of emit_step (src/warodecode.cu:2069-2075:
         * the product adds the bias, qk_norm_kernel :1836 runs before rope_store_kernel) */
        if (L->bqkv)
            for (int i = 0; i < qkv_rows; ++i) qkv[i] = addf(qkv[i], L->bqkv[i]);
        if (L->q_norm)
            for (int h = 0; h < nh; ++h) {
                wdo_rmsnorm(qkv + (size_t)h * hd, L->q_norm, m->rms_eps, hd, norm);
                memcpy(qkv + (size_t)h * hd, norm, sizeof(float) * hd);
            }
        if (L->k_norm)
            for (int h = 0; h < nkv; ++h) {
                wdo_rmsnorm(qkv + qdim + (size_t)h * hd, L->k_norm, m->rms_eps, hd, norm);
                memcpy(qkv + qdim + (size_t)h * hd, norm, sizeof(float) * hd);
            }
        for (int h = 0; h < nh; ++h) rope_head(qkv + (size_t)h * hd, hd, cs);
        for (int h = 0; h < nkv; ++h) rope_head(qkv + qdim + (size_t)h * hd, hd, cs);
        memcpy(kc + (size_t)pos * kvdim, qkv + qdim, sizeof(float) * kvdim);
        memcpy(vc + (size_t)pos * kvdim, qkv + qdim + kvdim, sizeof(float) * kvdim);
        for (int h = 0; h < nh; ++h) {
            const int kvh = (h * nkv) / nh;
            attention_head(qkv + (size_t)h * hd, kc + (size_t)kvh * hd, vc + (size_t)kvh * hd, (size_t)kvdim, pos, hd, inv_sqrt,
                           attn + (size_t)h * hd, scores);
        }
        wdo_quantize_q8_0(attn, xq, qdim / 32);
        wdo_matvec_typed(L->wo_type, L->wo, H, qdim, xq, proj);
        for (int i = 0; i < H; ++i) hidden[i] = addf(hidden[i], proj[i]);
        wdo_rmsnorm(hidden, L->ffn_norm, m->rms_eps, H, norm);
        wdo_quantize_q8_0(norm, xq, H / 32);
        wdo_matvec_typed(L->w_gate_up_type, L->w_gate_up, 2 * F, H, xq, gu);
        for (int i = 0; i < F; ++i) norm[i] = mulf(wdo_silu_ggml(gu[i]), gu[F + i]);
        wdo_quantize_q8_0(norm, xq, F / 32);
        wdo_matvec_typed(L->w_down_type, L->w_down, H, F, xq, proj);
    }
    for (int i = 0; i < H; ++i) hidden[i] = addf(hidden[i], proj[i]);
    wdo_rmsnorm(hidden, m->output_norm, m->rms_eps, H, norm);
    wdo_quantize_q8_0(norm, xq, H / 32);
    wdo_matvec_typed(m->output_type, m->output, V, H, xq, logits);
    int best = 0;
    float bv = -INFINITY;
    for (int i = 0; i < V; ++i)
        if (isfinite(logits[i]) && logits[i] > bv) {
            bv = logits[i];
            best = i;
        }
    if (m->hidden_out) memcpy(m->hidden_out, hidden, sizeof(float) * H);
    free(hidden); free(norm); free(qkv); free(attn); free(proj); free(gu); free(scores); free(xq);
    if (!logits_out) free(logits);
    return best;
}
