/* CPU oracle for the batch-1 MoE decode hot path (TEST INFRASTRUCTURE ONLY).
 *
 * Plain C99, scalar, single-threaded. Each function restates one piece of the
 * reference engine's host arithmetic and cites the lines it follows (paths are
 * relative to the reference project). Build with -ffp-contract=off so that the
 * only fused multiply-adds are the explicit fmaf() calls.
 *
 * Parity status: pinned. tests/test_oracle_pins.py compares every function here
 * bit for bit with the reference's own sources compiled by oracle/build_ref.sh,
 * and with golden vectors that build produced (tests/golden/).
 */
#include "wd_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "../warpdecode_b200/csrc/wd_grids.h"

/* ------------------------------------------------------------------------- */
/* bit casts, half conversion                                                 */
/* ------------------------------------------------------------------------- */
static inline uint32_t f32_bits(float v) { uint32_t b; memcpy(&b, &v, 4); return b; }
static inline float bits_f32(uint32_t b) { float v; memcpy(&v, &b, 4); return v; }

/* IEEE binary16 -> binary32, subnormals included (src/qwen38_cpu_moe.cuh:77-107). */
float wdo_f16_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t e = (h >> 10) & 0x1fu;
    uint32_t m = h & 0x3ffu;
    if (e == 0) {
        if (m == 0) return bits_f32(sign);
        int lead = 0;                       /* normalise the subnormal */
        while (!(m & 0x400u)) { m <<= 1; ++lead; }
        return bits_f32(sign | ((uint32_t)(113 - lead) << 23) | ((m & 0x3ffu) << 13));
    }
    if (e == 31) return bits_f32(sign | 0x7f800000u | (m << 13));
    return bits_f32(sign | ((e + 112u) << 23) | (m << 13));
}

/* binary32 -> binary16, round to nearest even; NaN collapses to infinity exactly
 * as the reference's converter does (src/qwen38_cpu_moe.cuh:109-137). */
uint16_t wdo_f32_to_f16(float value) {
    const uint32_t b = f32_bits(value);
    const uint32_t sign = (b >> 16) & 0x8000u;
    const int e = (int)((b >> 23) & 0xffu) - 127;
    const uint32_t m = b & 0x7fffffu;
    if (e > 15) return (uint16_t)(sign | 0x7c00u);
    if (e < -24) return (uint16_t)sign;
    if (e < -14) {
        const uint32_t shift = (uint32_t)(-e - 1);       /* 13 + (-e - 14) */
        const uint32_t full = m | 0x800000u;
        uint32_t r = full >> shift;
        const uint32_t rest = full & ((1u << shift) - 1u);
        const uint32_t half = 1u << (shift - 1);
        if (rest > half || (rest == half && (r & 1u))) ++r;
        return (uint16_t)(sign | r);
    }
    uint32_t r = m >> 13;
    const uint32_t rest = m & 0x1fffu;
    if (rest > 0x1000u || (rest == 0x1000u && (r & 1u))) {
        ++r;
        if (r == 0x400u) return (uint16_t)(sign | (uint32_t)((e + 16) << 10));
    }
    return (uint16_t)(sign | (uint32_t)((e + 15) << 10) | r);
}

static inline float half_at(const uint8_t *p) {
    uint16_t h;
    memcpy(&h, p, 2);
    return wdo_f16_to_f32(h);
}

/* Single-rounded product / sum that must never become an FMA
 * (src/qwen38_cpu_moe.cuh:144-160, src/qwen38_precision.hpp:14-34). */
static inline float mul_rn(float a, float b) { volatile float r = a * b; return r; }
static inline float add_rn(float a, float b) { volatile float r = a + b; return r; }

uint32_t wdo_iq3s_grid(int index) { return wd_iq3s_unpack(wd_iq3s_grid_packed[index & 511]); }
uint64_t wdo_iq2s_grid(int index) { return wd_iq2s_unpack(wd_iq2s_grid_packed[index & 1023]); }

/* ------------------------------------------------------------------------- */
/* activation quantisers                                                      */
/* ------------------------------------------------------------------------- */

/* ggml quantize_row_q8_0 (src/qwen38_cpu_moe.cuh:220-237): d = f16(amax/127),
 * q = rint(x * (127/amax)) clamped to [-128, 127]; an all-zero block stores 0. */
void wdo_quantize_q8_0(const float *x, uint8_t *blocks, int nblocks) {
    for (int b = 0; b < nblocks; ++b) {
        const float *src = x + (size_t)b * 32;
        uint8_t *blk = blocks + (size_t)b * WDO_Q8_0_BYTES;
        float amax = 0.0f;
        for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(src[i]));
        const uint16_t d = wdo_f32_to_f16(amax / 127.0f);
        memcpy(blk, &d, 2);
        int8_t *q = (int8_t *)(blk + 2);
        if (amax == 0.0f) {
            memset(q, 0, 32);
            continue;
        }
        const float inv = 127.0f / amax;
        for (int i = 0; i < 32; ++i) {
            int v = (int)nearbyintf(src[i] * inv);
            if (v > 127) v = 127;
            if (v < -128) v = -128;
            q[i] = (int8_t)v;
        }
    }
}

/* ggml quantize_row_q8_K (src/qwen38_cpu_moe.cuh:239-263): iscale = -127/amax,
 * q = min(127, rint(x * iscale)), d = 1/iscale, bsums over groups of 16. */
void wdo_quantize_q8_K(const float *x, wdo_q8k *blocks, int nblocks) {
    for (int b = 0; b < nblocks; ++b) {
        const float *src = x + (size_t)b * 256;
        wdo_q8k *blk = &blocks[b];
        float amax = 0.0f;
        for (int i = 0; i < 256; ++i) amax = fmaxf(amax, fabsf(src[i]));
        if (amax == 0.0f) {
            memset(blk, 0, sizeof(*blk));
            continue;
        }
        const float iscale = -127.0f / amax;
        for (int i = 0; i < 256; ++i) {
            int v = (int)nearbyintf(src[i] * iscale);
            if (v > 127) v = 127;
            blk->qs[i] = (int8_t)v;
        }
        for (int j = 0; j < 16; ++j) {
            int s = 0;
            for (int i = 0; i < 16; ++i) s += blk->qs[j * 16 + i];
            blk->bsums[j] = (int16_t)s;
        }
        blk->d = 1.0f / iscale;
    }
}

/* ------------------------------------------------------------------------- */
/* row dot products                                                           */
/* ------------------------------------------------------------------------- */

/* The closing reduction of an 8-lane AVX2 accumulator
 * (src/qwen38_cpu_moe.cuh:290-296). */
static inline float hsum8(const float v[8]) {
    const float r0 = v[0] + v[4];
    const float r1 = v[1] + v[5];
    const float r2 = v[2] + v[6];
    const float r3 = v[3] + v[7];
    return (r0 + r2) + (r1 + r3);
}

/* Q8_0 weights x Q8_0 activation: per 32-value block, chunk-lane l owns values
 * 4l..4l+3 and takes one fmaf(d_w*d_x, int_dot, lane) (src/qwen38_cpu_moe.cuh:424-440). */
float wdo_row_q8_0_q8_0(const uint8_t *w_row, const uint8_t *y, int cols) {
    const int nb = cols / 32;
    float lane[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int b = 0; b < nb; ++b) {
        const uint8_t *wb = w_row + (size_t)b * WDO_Q8_0_BYTES;
        const uint8_t *yb = y + (size_t)b * WDO_Q8_0_BYTES;
        const int8_t *wq = (const int8_t *)(wb + 2);
        const int8_t *yq = (const int8_t *)(yb + 2);
        const float d = half_at(wb) * half_at(yb);
        for (int l = 0; l < 8; ++l) {
            int32_t p = 0;
            for (int j = 0; j < 4; ++j) p += (int32_t)wq[4 * l + j] * (int32_t)yq[4 * l + j];
            lane[l] = fmaf(d, (float)p, lane[l]);
        }
    }
    return hsum8(lane);
}

/* The Q8_0 row dot above for `rows` consecutive rows (an output head of 151,936 rows is too many calls for a Python
 * loop); also returns the index of the largest finite logit, lowest index first, which is the greedy token. */
int wdo_matvec_q8_0_argmax(const uint8_t *w, int rows, int cols, const uint8_t *y, float *out) {
    const size_t rb = (size_t)(cols / 32) * WDO_Q8_0_BYTES;
    int best = 0;
    float best_v = -INFINITY;
    for (int r = 0; r < rows; ++r) {
        const float v = wdo_row_q8_0_q8_0(w + (size_t)r * rb, y, cols);
        if (out) out[r] = v;
        if (v == v && v > best_v && v <= 3.402823466e38f) {
            best_v = v;
            best = r;
        }
    }
    return best;
}

/* IQ3_S weights x Q8_K activation (src/qwen38_cpu_moe.cuh:337-375). Block layout:
 * d(2) qs(64) qh(8) signs(32) scales(4). Chunk-lane c of sub-block ib32 uses grid
 * index qs[8*ib32 + c] | bit (c) of qh[ib32] << 8, sign nibble (c & 1) of
 * signs[4*ib32 + (c >> 1)], and scale 1 + 2*nibble(ib32) of scales[ib32 >> 1]. */
float wdo_row_iq3_s_q8_K(const uint8_t *w_row, const wdo_q8k *y, int cols, int32_t *partials) {
    const int nb = cols / 256;
    float lane[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int sb = 0; sb < nb; ++sb) {
        const uint8_t *blk = w_row + (size_t)sb * WDO_IQ3_S_BYTES;
        const float d = half_at(blk) * y[sb].d;
        const uint8_t *qs = blk + 2, *qh = blk + 66, *signs = blk + 74, *scales = blk + 106;
        const int8_t *a = y[sb].qs;
        for (int c = 0; c < 8; ++c) {
            int32_t partial = 0;
            for (int ib = 0; ib < 8; ++ib) {
                const int nib = (ib & 1) ? (scales[ib >> 1] >> 4) : (scales[ib >> 1] & 15);
                const int ls = 1 + 2 * nib;
                const int idx = qs[ib * 8 + c] | (((qh[ib] >> c) & 1) << 8);
                const uint32_t g = wdo_iq3s_grid(idx);
                const unsigned sg = (unsigned)(signs[ib * 4 + (c >> 1)] >> (4 * (c & 1)));
                int32_t dot = 0;
                for (int j = 0; j < 4; ++j) {
                    const int mag = (int)((g >> (8 * j)) & 0xffu);
                    dot += (int32_t)a[ib * 32 + c * 4 + j] * (((sg >> j) & 1u) ? -mag : mag);
                }
                partial += dot * ls;
            }
            if (partials) partials[sb * 8 + c] = partial;
            lane[c] = fmaf(d, (float)partial, lane[c]);
        }
    }
    return hsum8(lane);
}

/* IQ2_S weights x Q8_K activation (src/qwen38_cpu_moe.cuh:298-335). Block layout:
 * d(2) qs(32) signs(32) qh(8) scales(8). A 10-bit index selects eight magnitudes;
 * chunk-lane c takes the low (even c) or high (odd c) four. Chunks 0..3 use the
 * low scale nibble of scales[ib32], chunks 4..7 the high one; result * 0.125. */
float wdo_row_iq2_s_q8_K(const uint8_t *w_row, const wdo_q8k *y, int cols, int32_t *partials) {
    const int nb = cols / 256;
    float lane[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int sb = 0; sb < nb; ++sb) {
        const uint8_t *blk = w_row + (size_t)sb * WDO_IQ2_S_BYTES;
        const float d = half_at(blk) * y[sb].d;
        const uint8_t *qs = blk + 2, *signs = blk + 34, *qh = blk + 66, *scales = blk + 74;
        const int8_t *a = y[sb].qs;
        for (int c = 0; c < 8; ++c) {
            const int grp = c >> 1, half = c & 1;
            int32_t partial = 0;
            for (int ib = 0; ib < 8; ++ib) {
                const int nib = (c < 4) ? (scales[ib] & 15) : (scales[ib] >> 4);
                const int ls = 1 + 2 * nib;
                const int idx = qs[ib * 4 + grp] | (((qh[ib] >> (2 * grp)) & 3) << 8);
                const uint32_t g = (uint32_t)(wdo_iq2s_grid(idx) >> (32 * half));
                const unsigned sg = (unsigned)(signs[ib * 4 + grp] >> (4 * half));
                int32_t dot = 0;
                for (int j = 0; j < 4; ++j) {
                    const int mag = (int)((g >> (8 * j)) & 0xffu);
                    dot += (int32_t)a[ib * 32 + c * 4 + j] * (((sg >> j) & 1u) ? -mag : mag);
                }
                partial += dot * ls;
            }
            if (partials) partials[sb * 8 + c] = partial;
            lane[c] = fmaf(d, (float)partial, lane[c]);
        }
    }
    return 0.125f * hsum8(lane);
}

static const int8_t k_iq4nl[16] = {-127, -104, -83, -65, -49, -35, -22, -10,
                                   1,    13,   25,  38,  53,  69,  89,  113};

/* IQ4_NL weights x Q8_0 activation (src/qwen38_cpu_moe.cuh:377-422): even and odd
 * blocks accumulate separately, lanes are added, then the 8-lane reduction; a
 * trailing odd block is added as one scalar product. */
float wdo_row_iq4_nl_q8_0(const uint8_t *w_row, const uint8_t *y, int cols) {
    const int nb = cols / 32;
    float even[8] = {0, 0, 0, 0, 0, 0, 0, 0}, odd[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int b = 0;
    for (; b + 1 < nb; b += 2) {
        for (int par = 0; par < 2; ++par) {
            const uint8_t *wb = w_row + (size_t)(b + par) * WDO_IQ4_NL_BYTES;
            const uint8_t *yb = y + (size_t)(b + par) * WDO_Q8_0_BYTES;
            const int8_t *yq = (const int8_t *)(yb + 2);
            const float d = half_at(wb) * half_at(yb);
            float *acc = par ? odd : even;
            for (int l = 0; l < 8; ++l) {
                const int hi = l >> 2;
                int32_t p = 0;
                for (int j = 0; j < 4; ++j) {
                    const int i = 4 * (l & 3) + j;
                    const int nib = hi ? (wb[2 + i] >> 4) : (wb[2 + i] & 15);
                    p += (int32_t)yq[16 * hi + i] * (int32_t)k_iq4nl[nib];
                }
                acc[l] = fmaf(d, (float)p, acc[l]);
            }
        }
    }
    float lane[8];
    for (int l = 0; l < 8; ++l) lane[l] = even[l] + odd[l];
    float sum = hsum8(lane);
    if (b < nb) {
        const uint8_t *wb = w_row + (size_t)b * WDO_IQ4_NL_BYTES;
        const uint8_t *yb = y + (size_t)b * WDO_Q8_0_BYTES;
        const int8_t *yq = (const int8_t *)(yb + 2);
        int s1 = 0, s2 = 0;
        for (int j = 0; j < 16; ++j) {
            s1 += (int)yq[j] * (int)k_iq4nl[wb[2 + j] & 15];
            s2 += (int)yq[j + 16] * (int)k_iq4nl[wb[2 + j] >> 4];
        }
        sum += (half_at(wb) * half_at(yb)) * (float)(s1 + s2);
    }
    return sum;
}

/* Q4_0 weights x Q8_0 activation for the dense matvec (src/warodecode.cu:1535-1562
 * computes (q - 8) * d against Q8_0 activations; that kernel carries no exact
 * float order and the reference has no host twin, so this oracle takes ggml's:
 * ggml_vec_dot_q4_0_q8_0 (AVX2) unpacks the low nibbles of the 16 bytes to values
 * 0..15 and the high nibbles to values 16..31, sums four consecutive products per
 * lane, and does one fmaf(d_w * d_x, (float)p_lane, acc_lane) per block for the
 * eight lanes, blocks ascending, then the same 8-lane tree as the Q8_0 row.
 * No golden vector of the reference covers this function; it is pinned against an independent decoder
 * instead (gguf-py's dequantize plus an exact integer reconstruction, tests/test_oracle_pins.py). */
float wdo_row_q4_0_q8_0(const uint8_t *w_row, const uint8_t *y, int cols) {
    const int nb = cols / 32;
    float lane[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int b = 0; b < nb; ++b) {
        const uint8_t *wb = w_row + (size_t)b * WDO_Q4_0_BYTES;
        const uint8_t *yb = y + (size_t)b * WDO_Q8_0_BYTES;
        const int8_t *yq = (const int8_t *)(yb + 2);
        const float d = half_at(wb) * half_at(yb);
        for (int l = 0; l < 8; ++l) {
            int32_t p = 0;
            for (int j = 0; j < 4; ++j) {
                const int v = 4 * l + j;        /* value index inside the block */
                const int q = v < 16 ? (wb[2 + v] & 15) : (wb[2 + v - 16] >> 4);
                p += (q - 8) * (int)yq[v];
            }
            lane[l] = fmaf(d, (float)p, lane[l]);
        }
    }
    return hsum8(lane);
}

/* ------------------------------------------------------------------------- */
/* transcendentals and the F32 dot                                            */
/* ------------------------------------------------------------------------- */

/* One lane of ggml's AVX2 ggml_v_expf polynomial (src/qwen38_cpu_moe.cuh:816-834,
 * device twin src/qwen38_exact_math.cuh:94-115). */
float wdo_exp_ggml(float x) {
    const float r = 0x1.8p23f;
    const float z = fmaf(x, 0x1.715476p+0f, r);
    const float n = z - r;
    const float b = fmaf(-n, 0x1.7f7d1cp-20f, fmaf(-n, 0x1.62e4p-1f, x));
    const uint32_t e = f32_bits(z) << 23;
    const float k = bits_f32(e + f32_bits(1.0f));
    const float u = b * b;
    const float t0 = fmaf(0x1.0e4020p-7f, b, 0x1.573e2ep-5f);
    const float t1 = fmaf(t0, u, fmaf(0x1.555e66p-3f, b, 0x1.fffdb6p-2f));
    const float j = fmaf(t1, u, 0x1.ffffecp-1f * b);
    if (fabsf(n) <= 126.0f) return fmaf(j, k, k);
    const uint32_t g = n <= 0.0f ? 0x82000000u : 0u;
    const float s1 = bits_f32(g + 0x7f000000u);
    const float s2 = bits_f32(e - g);
    if (fabsf(n) > 192.0f) return s1 * s1;
    return fmaf(s2, j, s2) * s1;
}

/* src/qwen38_cpu_moe.cuh:836-842. */
float wdo_silu_ggml(float x) { return x / (1.0f + wdo_exp_ggml(-x)); }
float wdo_sigmoid_ggml(float x) { return 1.0f / (1.0f + wdo_exp_ggml(-x)); }

/* ggml_vec_dot_f32 in its AVX2 visit order: 32 running sums (element i feeds sum
 * i mod 32), folded 32 -> 16 -> 8 -> 4 -> 1, scalar tail (src/qwen38_cpu_moe.cuh:847-871). */
float wdo_dot_f32(const float *a, const float *b, int n) {
    float s[32];
    for (int i = 0; i < 32; ++i) s[i] = 0.0f;
    const int np = n & ~31;
    for (int i = 0; i < np; i += 32)
        for (int t = 0; t < 32; ++t) s[t] = fmaf(a[i + t], b[i + t], s[t]);
    for (int l = 0; l < 8; ++l) {
        s[l] = s[l] + s[16 + l];
        s[8 + l] = s[8 + l] + s[24 + l];
    }
    for (int l = 0; l < 8; ++l) s[l] = s[l] + s[8 + l];
    float t[4];
    for (int q = 0; q < 4; ++q) t[q] = s[q] + s[q + 4];
    float acc = (t[0] + t[1]) + (t[2] + t[3]);
    for (int c = np; c < n; ++c) acc = acc + a[c] * b[c];
    return acc;
}

/* ------------------------------------------------------------------------- */
/* router                                                                     */
/* ------------------------------------------------------------------------- */

/* ggml_soft_max over the full row (src/qwen38_moe.cuh:711-749): running max,
 * exp_ggml(x - max), groups of eight summed as ((v0+v4)+(v2+v6))+((v1+v5)+(v3+v7))
 * and accumulated ascending into a double, then p * (float)(1/sum). A zero sum
 * leaves the whole row at -inf. */
void wdo_softmax_row(const float *logits, int n, float *probs) {
    float mx = -INFINITY;
    for (int e = 0; e < n; ++e) mx = fmaxf(mx, logits[e]);
    double sum = 0.0;
    int i = 0;
    for (; i + 8 <= n; i += 8) {
        float v[8];
        for (int j = 0; j < 8; ++j) {
            v[j] = wdo_exp_ggml(logits[i + j] - mx);
            probs[i + j] = v[j];
        }
        const float lo = v[0] + v[4], lh = v[2] + v[6], hi = v[1] + v[5], hh = v[3] + v[7];
        sum += (double)((lo + lh) + (hi + hh));
    }
    for (; i < n; ++i) {
        probs[i] = wdo_exp_ggml(logits[i] - mx);
        sum += (double)probs[i];
    }
    if (sum == 0.0) {
        for (int e = 0; e < n; ++e) probs[e] = -INFINITY;
        return;
    }
    const float inv = (float)(1.0 / sum);
    for (int e = 0; e < n; ++e) probs[e] = probs[e] * inv;
}

/* Descending argsort top-k by probability, ties to the lower index; weights are
 * the picked probabilities divided by max((float)double_sum, 2^-14), then scaled
 * unless w_scale is 0 or 1 (src/qwen38_moe.cuh:765-818). A rung that finds nothing
 * above -inf yields id 0 and reads its value back through that id. */
void wdo_router_select(const float *probs, int n, int k, float w_scale, int *ids, float *weights) {
    float top[64];
    if (k > 64) k = 64;
    for (int j = 0; j < k; ++j) {
        float best = -INFINITY;
        int best_id = 0;
        for (int e = 0; e < n; ++e) {
            if (!(probs[e] > best)) continue;
            int taken = 0;
            for (int m = 0; m < j; ++m) taken |= (ids[m] == e);
            if (!taken) {
                best = probs[e];
                best_id = e;
            }
        }
        ids[j] = best_id;
        top[j] = probs[best_id];
    }
    double wsum = 0.0;
    for (int j = 0; j < k; ++j) wsum += (double)top[j];
    const float denom = fmaxf((float)wsum, 6.103515625e-5f);
    for (int j = 0; j < k; ++j) weights[j] = top[j] / denom;
    if (w_scale != 0.0f && w_scale != 1.0f)
        for (int j = 0; j < k; ++j) weights[j] = weights[j] * w_scale;
}

void wdo_router_exact(const float *logits, int n, int k, float w_scale, float *probs, int *ids,
                      float *weights) {
    wdo_softmax_row(logits, n, probs);
    wdo_router_select(probs, n, k, w_scale, ids, weights);
}

/* ------------------------------------------------------------------------- */
/* the MoE block                                                              */
/* ------------------------------------------------------------------------- */
size_t wdo_row_bytes(int type, int cols) {
    switch (type) {
        case WDO_TYPE_F32: return (size_t)cols * 4;
        case WDO_TYPE_Q8_0: return cols % 32 ? 0 : (size_t)(cols / 32) * WDO_Q8_0_BYTES;
        case WDO_TYPE_Q4_0: return cols % 32 ? 0 : (size_t)(cols / 32) * WDO_Q4_0_BYTES;
        case WDO_TYPE_IQ4_NL: return cols % 32 ? 0 : (size_t)(cols / 32) * WDO_IQ4_NL_BYTES;
        case WDO_TYPE_IQ3_S: return cols % 256 ? 0 : (size_t)(cols / 256) * WDO_IQ3_S_BYTES;
        case WDO_TYPE_IQ2_S: return cols % 256 ? 0 : (size_t)(cols / 256) * WDO_IQ2_S_BYTES;
        default: return 0;
    }
}

/* ggml's pairing of weight type and activation quantiser (src/lowbit.cuh:798-803):
 * IQ2_S / IQ3_S consume Q8_K, IQ4_NL / Q8_0 consume Q8_0. */
static int uses_q8k(int type) { return type == WDO_TYPE_IQ3_S || type == WDO_TYPE_IQ2_S; }

static float dot_any(int type, const uint8_t *row, const wdo_q8k *yk, const uint8_t *y0, int cols) {
    switch (type) {
        case WDO_TYPE_IQ3_S: return wdo_row_iq3_s_q8_K(row, yk, cols, NULL);
        case WDO_TYPE_IQ2_S: return wdo_row_iq2_s_q8_K(row, yk, cols, NULL);
        case WDO_TYPE_IQ4_NL: return wdo_row_iq4_nl_q8_0(row, y0, cols);
        default: return wdo_row_q8_0_q8_0(row, y0, cols);
    }
}

/* Composition of one block, in the order the reference engine runs it:
 *   router   : Q8_0-quantised x, Q8_0 GEMV (or, for an F32 router, one
 *              ggml_vec_dot_f32 per expert on the F32 x), (+bias), softmax/top-k
 *              (src/qwen38_moe.cuh:2242-2258, :2323-2361)
 *   experts  : Q8_K-quantised x; per selected expert gate and up rows, silu(g)*u
 *              as a separate rounded product, re-quantise with the quantiser the
 *              down type calls for, down rows (src/qwen38_cpu_moe.cuh:1169-1217)
 *   combine  : out += down * weight with two roundings, in router rank order
 *              (src/qwen38_cpu_moe.cuh:1281-1290)
 *   shared   : sigmoid(dot_f32(gate_vec, x)); Q8_0 gate/up rows, silu*up,
 *              re-quantise Q8_0, Q8_0 down rows (src/qwen38_moe.cuh:3852-3891)
 *   finish   : routed + shared * gate, two roundings (src/qwen38_precision.hpp:32-34) */
int wdo_moe_block(const wdo_moe_weights *w, const float *x, wdo_moe_result *r, int first_expert,
                  int n_local) {
    const int H = w->hidden, F = w->expert_ffn, SF = w->shared_ffn, E = w->n_experts, K = w->top_k;
    if (H <= 0 || H % 256 || F <= 0 || E <= 0 || K <= 0 || K > 64 || K > E) return -1;
    if (F % (uses_q8k(w->down_type) ? 256 : 64)) return -1;
    if (SF % 32 || !r || !r->out) return -1;
    if (!uses_q8k(w->gate_type) || !uses_q8k(w->up_type)) return -2;
    const size_t gate_rb = wdo_row_bytes(w->gate_type, H), up_rb = wdo_row_bytes(w->up_type, H);
    const size_t down_rb = wdo_row_bytes(w->down_type, F), q8_rb_h = wdo_row_bytes(WDO_TYPE_Q8_0, H);
    if (!gate_rb || !up_rb || !down_rb) return -2;

    float *logits = (float *)malloc(sizeof(float) * (size_t)E * 2);
    float *probs = logits + E;
    int *ids = (int *)malloc(sizeof(int) * (size_t)K);
    float *wts = (float *)malloc(sizeof(float) * (size_t)K);
    uint8_t *x_q80 = (uint8_t *)malloc((size_t)(H / 32) * WDO_Q8_0_BYTES);
    wdo_q8k *x_q8k = (wdo_q8k *)malloc(sizeof(wdo_q8k) * (size_t)(H / 256));
    const int FM = F > SF ? F : SF;
    float *gate = (float *)malloc(sizeof(float) * (size_t)FM * 3);
    float *up = gate + FM, *act = up + FM;
    wdo_q8k *a_q8k = (wdo_q8k *)malloc(sizeof(wdo_q8k) * (size_t)(FM / 256 + 1));
    uint8_t *a_q80 = (uint8_t *)malloc((size_t)(FM / 32 + 1) * WDO_Q8_0_BYTES);
    float *eo = (float *)malloc(sizeof(float) * (size_t)H);
    float *routed = (float *)calloc((size_t)H, sizeof(float));

    wdo_quantize_q8_0(x, x_q80, H / 32);
    for (int e = 0; e < E; ++e) {
        logits[e] = w->router_f32 ? wdo_dot_f32(w->router_f32 + (size_t)e * H, x, H)
                                  : wdo_row_q8_0_q8_0(w->router + (size_t)e * q8_rb_h, x_q80, H);
        if (w->router_bias) logits[e] = logits[e] + w->router_bias[e];
    }
    wdo_router_exact(logits, E, K, w->w_scale, probs, ids, wts);

    wdo_quantize_q8_K(x, x_q8k, H / 256);
    for (int j = 0; j < K; ++j) {
        const int e = ids[j];
        if (e < first_expert || e >= first_expert + n_local) {
            if (r->act) memset(r->act + (size_t)j * F, 0, sizeof(float) * (size_t)F);
            if (r->expert_out) memset(r->expert_out + (size_t)j * H, 0, sizeof(float) * (size_t)H);
            continue;
        }
        const uint8_t *g0 = w->gate + (size_t)e * F * gate_rb;
        const uint8_t *u0 = w->up + (size_t)e * F * up_rb;
        const uint8_t *d0 = w->down + (size_t)e * H * down_rb;
        for (int i = 0; i < F; ++i) {
            gate[i] = dot_any(w->gate_type, g0 + (size_t)i * gate_rb, x_q8k, NULL, H);
            up[i] = dot_any(w->up_type, u0 + (size_t)i * up_rb, x_q8k, NULL, H);
        }
        for (int i = 0; i < F; ++i) act[i] = mul_rn(wdo_silu_ggml(gate[i]), up[i]);
        if (uses_q8k(w->down_type)) wdo_quantize_q8_K(act, a_q8k, F / 256);
        else wdo_quantize_q8_0(act, a_q80, F / 32);
        for (int i = 0; i < H; ++i)
            eo[i] = dot_any(w->down_type, d0 + (size_t)i * down_rb, a_q8k, a_q80, F);
        for (int i = 0; i < H; ++i) routed[i] = add_rn(routed[i], mul_rn(eo[i], wts[j]));
        if (r->act) memcpy(r->act + (size_t)j * F, act, sizeof(float) * (size_t)F);
        if (r->expert_out) memcpy(r->expert_out + (size_t)j * H, eo, sizeof(float) * (size_t)H);
    }

    float sgate = 0.0f;
    if (SF > 0) {
        const size_t q8_rb_f = wdo_row_bytes(WDO_TYPE_Q8_0, SF);
        sgate = wdo_sigmoid_ggml(wdo_dot_f32(w->shared_gate_vec, x, H));
        for (int i = 0; i < SF; ++i) {
            gate[i] = wdo_row_q8_0_q8_0(w->shared_gate + (size_t)i * q8_rb_h, x_q80, H);
            up[i] = wdo_row_q8_0_q8_0(w->shared_up + (size_t)i * q8_rb_h, x_q80, H);
        }
        for (int i = 0; i < SF; ++i) act[i] = mul_rn(wdo_silu_ggml(gate[i]), up[i]);
        wdo_quantize_q8_0(act, a_q80, SF / 32);
        for (int i = 0; i < H; ++i) {
            eo[i] = wdo_row_q8_0_q8_0(w->shared_down + (size_t)i * q8_rb_f, a_q80, SF);
            r->out[i] = add_rn(routed[i], mul_rn(eo[i], sgate));
        }
        if (r->shared) memcpy(r->shared, eo, sizeof(float) * (size_t)H);
    } else {
        memcpy(r->out, routed, sizeof(float) * (size_t)H);
        if (r->shared) memset(r->shared, 0, sizeof(float) * (size_t)H);
    }
    if (r->shared_gate) r->shared_gate[0] = sgate;
    if (r->logits) memcpy(r->logits, logits, sizeof(float) * (size_t)E);
    if (r->probs) memcpy(r->probs, probs, sizeof(float) * (size_t)E);
    if (r->ids) memcpy(r->ids, ids, sizeof(int) * (size_t)K);
    if (r->weights) memcpy(r->weights, wts, sizeof(float) * (size_t)K);
    if (r->routed) memcpy(r->routed, routed, sizeof(float) * (size_t)H);

    free(logits); free(ids); free(wts); free(x_q80); free(x_q8k); free(gate);
    free(a_q8k); free(a_q80); free(eo); free(routed);
    return 0;
}

/* Sum of squares as a perfect binary tree over consecutive elements (zero-padded to a power of
 * two), every node one rounded double addition. The tree, not a running sum, is the definition:
 * it is the order a parallel reduction produces, so the CUDA path can match it bit for bit. */
static double sumsq_tree(const float *x, int lo, int width, int n) {
    if (lo >= n) return 0.0;
    if (width == 1) return (double)x[lo] * (double)x[lo];
    const double a = sumsq_tree(x, lo, width / 2, n);
    const double b = sumsq_tree(x, lo + width / 2, width / 2, n);
    return a + b;
}

void wdo_rmsnorm(const float *x, const float *weight, float eps, int n, float *y) {
    int width = 1;
    while (width < n) width *= 2;
    const double ss = sumsq_tree(x, 0, width, n);
    const float scale = (float)(1.0 / sqrt(ss / (double)n + (double)eps));
    for (int i = 0; i < n; ++i) {
        const float v = mul_rn(x[i], scale);
        y[i] = weight ? mul_rn(v, weight[i]) : v;
    }
}
