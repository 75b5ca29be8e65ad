/*
 * krk_oracle.c -- CPU restatement of Kraken's scalar f32 quantized-weight matmul.
 *
 * TEST INFRASTRUCTURE ONLY: the checker for the CUDA path, never part of it.
 * Parity status: PINNED against the compiled reference (oracle/_ref) and the
 * reference suite's known-answer vectors; see krk_oracle.h.
 *
 * Build with -ffp-contract=off: the reference's decoders round every product before
 * the subtract (src/quant.cpp:446-453) and the dot is a chain of separately rounded
 * multiply and add (src/quant.cpp:5579-5589).
 */
#include "krk_oracle.h"

#include <float.h>
#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

/* ---- geometry: src/quant.cpp:1805-1900 ---------------------------------------- */

int krk_oracle_block_size(int wt) {
    switch (wt) {
    case KRK_ORACLE_Q4_0:
    case KRK_ORACLE_Q5_0:
    case KRK_ORACLE_Q5_1:
    case KRK_ORACLE_IQ4_NL:
    case KRK_ORACLE_Q8_0: return 32;
    case KRK_ORACLE_Q2_K:
    case KRK_ORACLE_Q3_K:
    case KRK_ORACLE_Q4_K:
    case KRK_ORACLE_Q5_K:
    case KRK_ORACLE_Q6_K: return 256;
    default: return 0;
    }
}

int krk_oracle_block_bytes(int wt) {
    switch (wt) {
    case KRK_ORACLE_Q4_0: return 18;
    case KRK_ORACLE_Q8_0: return 34;
    case KRK_ORACLE_Q4_K: return 144;
    case KRK_ORACLE_Q6_K: return 210;
    case KRK_ORACLE_Q5_0: return 22;
    case KRK_ORACLE_Q5_1: return 24;
    case KRK_ORACLE_Q5_K: return 176;
    case KRK_ORACLE_Q2_K: return 84;
    case KRK_ORACLE_Q3_K: return 110;
    case KRK_ORACLE_IQ4_NL: return 18;
    default: return 0;
    }
}

size_t krk_oracle_row_bytes(int wt, int64_t n_in) {
    const int bs = krk_oracle_block_size(wt);
    if (bs == 0 || n_in < 0) return 0;
    return (size_t)((n_in + bs - 1) / bs) * (size_t)krk_oracle_block_bytes(wt);
}

/* ---- half -> float: src/common.cpp:161-187 ------------------------------------ */

float krk_oracle_fp16_to_fp32(uint16_t h) {
    const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t expo = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (expo == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else if (expo != 0) {
        bits = sign | ((expo + 112u) << 23) | (man << 13);
    } else if (man == 0) {
        bits = sign;
    } else {
        /* subnormal half: normalise the mantissa into a float exponent */
        int shift = 0;
        while (!(man & 0x400u)) {
            man <<= 1;
            shift++;
        }
        bits = sign | ((uint32_t)(113 - shift) << 23) | ((man & 0x3FFu) << 13);
    }
    float f;
    memcpy(&f, &bits, sizeof f);
    return f;
}

static inline float half_at(const uint8_t *p) {
    return krk_oracle_fp16_to_fp32((uint16_t)(p[0] | (p[1] << 8)));
}

/* ---- per-format block decoders ------------------------------------------------- */

/* src/quant.cpp:381-387 */
static void block_q8_0(const uint8_t *b, float *y) {
    const float d = half_at(b);
    for (int k = 0; k < 32; k++) y[k] = d * (float)(int8_t)b[2 + k];
}

/* src/quant.cpp:331-339: low nibbles are values 0..15, high nibbles 16..31 */
static void block_q4_0(const uint8_t *b, float *y) {
    const float d = half_at(b);
    for (int k = 0; k < 16; k++) {
        y[k] = d * (float)((int)(b[2 + k] & 0xF) - 8);
        y[k + 16] = d * (float)((int)(b[2 + k] >> 4) - 8);
    }
}

/* src/quant.cpp:427-435: the j-th 6-bit scale and 6-bit min out of 12 packed bytes */
static void scale_min_k4(int j, const uint8_t *p, int *sc, int *mn) {
    if (j < 4) {
        *sc = p[j] & 63;
        *mn = p[j + 4] & 63;
    } else {
        *sc = (p[j + 4] & 0xF) | ((p[j - 4] >> 6) << 4);
        *mn = (p[j + 4] >> 4) | ((p[j] >> 6) << 4);
    }
}

/* src/quant.cpp:437-460: value = (d*sc)*q - (dmin*m), both products rounded first */
static void block_q4_k(const uint8_t *b, float *y) {
    const float d = half_at(b);
    const float dmin = half_at(b + 2);
    const uint8_t *packed = b + 4;
    for (int pair = 0; pair < 4; pair++) {
        const uint8_t *q = b + 16 + 32 * pair;
        float *yy = y + 64 * pair;
        int s0, m0, s1, m1;
        scale_min_k4(2 * pair, packed, &s0, &m0);
        scale_min_k4(2 * pair + 1, packed, &s1, &m1);
        const float dl0 = d * (float)s0, mn0 = dmin * (float)m0;
        const float dl1 = d * (float)s1, mn1 = dmin * (float)m1;
        for (int l = 0; l < 32; l++) {
            yy[l] = dl0 * (float)(q[l] & 0xF) - mn0;
            yy[l + 32] = dl1 * (float)(q[l] >> 4) - mn1;
        }
    }
}

/* src/quant.cpp:491-512: value = (d*scale)*(q-32), left to right */
static void block_q6_k(const uint8_t *b, float *y) {
    const float d = half_at(b + 208);
    for (int half = 0; half < 2; half++) {
        const uint8_t *ql = b + 64 * half;
        const uint8_t *qh = b + 128 + 32 * half;
        const int8_t *sc = (const int8_t *)(b + 192) + 8 * half;
        float *yy = y + 128 * half;
        for (int l = 0; l < 32; l++) {
            const int g = l >> 4;
            const int q1 = (ql[l] & 0xF) | ((qh[l] & 3) << 4);
            const int q2 = (ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4);
            const int q3 = (ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4);
            const int q4 = (ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4);
            yy[l] = d * (float)sc[g] * (float)(q1 - 32);
            yy[l + 32] = d * (float)sc[g + 2] * (float)(q2 - 32);
            yy[l + 64] = d * (float)sc[g + 4] * (float)(q3 - 32);
            yy[l + 96] = d * (float)sc[g + 6] * (float)(q4 - 32);
        }
    }
}

/* src/quant.cpp:352-364 */
static void block_q5_0(const uint8_t *b, float *y) {
    const float d = half_at(b);
    uint32_t qh;
    memcpy(&qh, b + 2, 4);
    for (int k = 0; k < 16; k++) {
        const int lo = (b[6 + k] & 0xF) | (int)(((qh >> k) & 1u) << 4);
        const int hi = (b[6 + k] >> 4) | (int)(((qh >> (k + 16)) & 1u) << 4);
        y[k] = d * (float)(lo - 16);
        y[k + 16] = d * (float)(hi - 16);
    }
}

/* src/quant.cpp:366-379 */
static void block_q5_1(const uint8_t *b, float *y) {
    const float d = half_at(b), m = half_at(b + 2);
    uint32_t qh;
    memcpy(&qh, b + 4, 4);
    for (int k = 0; k < 16; k++) {
        const int lo = (b[8 + k] & 0xF) | (int)(((qh >> k) & 1u) << 4);
        const int hi = (b[8 + k] >> 4) | (int)(((qh >> (k + 16)) & 1u) << 4);
        y[k] = d * (float)lo + m;
        y[k + 16] = d * (float)hi + m;
    }
}

/* src/quant.cpp:462-489 */
static void block_q5_k(const uint8_t *b, float *y) {
    const float d = half_at(b), dmin = half_at(b + 2);
    const uint8_t *scales = b + 4, *qh = b + 16, *q = b + 48;
    for (int j = 0; j < 4; j++, q += 32, y += 64) {
        int s0, m0, s1, m1;
        scale_min_k4(2 * j, scales, &s0, &m0);
        scale_min_k4(2 * j + 1, scales, &s1, &m1);
        const float d1 = d * (float)s0, mm1 = dmin * (float)m0, d2 = d * (float)s1, mm2 = dmin * (float)m1;
        const uint8_t u1 = (uint8_t)(1u << (2 * j)), u2 = (uint8_t)(2u << (2 * j));
        for (int l = 0; l < 32; l++) {
            y[l] = d1 * (float)((q[l] & 0xF) + ((qh[l] & u1) ? 16 : 0)) - mm1;
            y[l + 32] = d2 * (float)((q[l] >> 4) + ((qh[l] & u2) ? 16 : 0)) - mm2;
        }
    }
}

/* src/quant.cpp:398-424: 84 bytes = 16 scale bytes (scale in the low nibble, min in the high one), 64 bytes of
 * 2-bit quants, f16 d, f16 dmin. Two 128-value halves; in a half, bit pair j of the 32 quant bytes gives 32
 * values, the first 16 and the last 16 with a scale byte each: y = (d * sc) * q - dmin * m. */
static void block_q2_k(const uint8_t *b, float *y) {
    const float d = half_at(b + 80), dmin = half_at(b + 82);
    int is = 0;
    for (int g = 0; g < 2; g++) {
        const uint8_t *q = b + 16 + 32 * g;
        for (int j = 0; j < 4; j++) {
            for (int h = 0; h < 2; h++) {
                const uint8_t sc = b[is++];
                const float dl = d * (float)(sc & 0xF), ml = dmin * (float)(sc >> 4);
                for (int l = 0; l < 16; l++) y[l + 16 * h] = dl * (float)((q[l + 16 * h] >> (2 * j)) & 3) - ml;
            }
            y += 32;
        }
    }
}

/* src/quant.cpp:514-553: 110 bytes = 32 bytes of high-bit masks, 64 bytes of 2-bit quants, 12 bytes holding
 * sixteen 6-bit scales (low 4 bits in the first 8 bytes' nibbles, high 2 bits in the last 4 bytes), f16 d.
 * q = 2 low bits, minus 4 when the mask bit is clear; y = (d * (scale - 32)) * q. */
static void block_q3_k(const uint8_t *b, float *y) {
    const float d_all = half_at(b + 108);
    const uint8_t *hm = b, *q = b + 32, *sr = b + 96;
    int scales[16];
    for (int j = 0; j < 16; j++) {
        const int lo = j < 8 ? (sr[j] & 0xF) : (sr[j - 8] >> 4);
        const int hi = (sr[8 + (j & 3)] >> (2 * (j >> 2))) & 3;
        scales[j] = (lo | (hi << 4)) - 32;
    }
    int is = 0;
    uint8_t m = 1;
    for (int nn = 0; nn < 2; nn++, q += 32) {
        for (int j = 0; j < 4; j++, m = (uint8_t)(m << 1)) {
            for (int h = 0; h < 2; h++) {
                const float dl = d_all * (float)scales[is++];
                for (int l = 0; l < 16; l++) {
                    const int v = (int)((q[l + 16 * h] >> (2 * j)) & 3) - ((hm[l + 16 * h] & m) ? 0 : 4);
                    *y++ = dl * (float)v;
                }
            }
        }
    }
}

/* src/quant.cpp:88-91, 566-575: f16 d and 16 bytes of nibbles indexing the format's 16-entry non-linear grid;
 * low nibbles are values 0..15, high nibbles 16..31. */
static const int8_t k_iq4nl_grid[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};
static void block_iq4_nl(const uint8_t *b, float *y) {
    const float d = half_at(b);
    for (int k = 0; k < 16; k++) {
        y[k] = d * (float)k_iq4nl_grid[b[2 + k] & 0xF];
        y[k + 16] = d * (float)k_iq4nl_grid[b[2 + k] >> 4];
    }
}

/* src/quant.cpp:1553-1599 */
static void decode_block(int wt, const uint8_t *b, float *y) {
    switch (wt) {
    case KRK_ORACLE_Q8_0: block_q8_0(b, y); break;
    case KRK_ORACLE_Q4_0: block_q4_0(b, y); break;
    case KRK_ORACLE_Q4_K: block_q4_k(b, y); break;
    case KRK_ORACLE_Q6_K: block_q6_k(b, y); break;
    case KRK_ORACLE_Q5_0: block_q5_0(b, y); break;
    case KRK_ORACLE_Q5_1: block_q5_1(b, y); break;
    case KRK_ORACLE_Q5_K: block_q5_k(b, y); break;
    case KRK_ORACLE_Q2_K: block_q2_k(b, y); break;
    case KRK_ORACLE_Q3_K: block_q3_k(b, y); break;
    case KRK_ORACLE_IQ4_NL: block_iq4_nl(b, y); break;
    default: break;
    }
}

int krk_oracle_dequant_rows(float *out, const void *w, int wt, int64_t n_rows, int64_t n_in) {
    const int bs = krk_oracle_block_size(wt);
    const int bb = krk_oracle_block_bytes(wt);
    if (bs == 0 || n_in < 0 || n_rows < 0 || n_in % bs != 0) return -1;
    const int64_t nblk = n_in / bs;
    const uint8_t *p = (const uint8_t *)w;
    for (int64_t r = 0; r < n_rows; r++)
        for (int64_t i = 0; i < nblk; i++, p += bb, out += bs) decode_block(wt, p, out);
    return 0;
}

/* ---- dot and GEMM --------------------------------------------------------------- */

/* src/quant.cpp:5579-5589: decode one block, then sum += w[k]*x[k] in index order */
static float row_dot(int wt, const uint8_t *row, const float *x, int64_t n_in) {
    const int bs = krk_oracle_block_size(wt);
    const int bb = krk_oracle_block_bytes(wt);
    float buf[256];
    float sum = 0.0f;
    for (int64_t i = 0; i < n_in; i += bs, row += bb) {
        decode_block(wt, row, buf);
        for (int k = 0; k < bs; k++) sum += buf[k] * x[i + k];
    }
    return sum;
}

typedef struct {
    float *out;
    const float *x;
    const uint8_t *w;
    int wt;
    int64_t n_out, n_in, rows, o_begin, o_end;
    size_t row_bytes;
} gemm_job;

static void *gemm_worker(void *arg) {
    const gemm_job *j = (const gemm_job *)arg;
    for (int64_t o = j->o_begin; o < j->o_end; o++) {
        const uint8_t *wrow = j->w + (size_t)o * j->row_bytes;
        for (int64_t r = 0; r < j->rows; r++)
            j->out[r * j->n_out + o] = row_dot(j->wt, wrow, j->x + r * j->n_in, j->n_in);
    }
    return NULL;
}

/* src/backend_cpu.cpp:1303-1320: every output is an independent dot, so outputs may
 * be split over threads without changing any bit. */
int krk_oracle_gemm(float *out, const float *x, const void *w, int wt, int64_t n_out,
                    int64_t n_in, int64_t rows, int n_threads) {
    const int bs = krk_oracle_block_size(wt);
    if (bs == 0 || n_in <= 0 || n_in % bs != 0 || n_out < 0 || rows < 0) return -1;
    if (n_out == 0 || rows == 0) return 0;
    if (n_threads < 1) n_threads = 1;
    if (n_threads > 256) n_threads = 256;
    if ((int64_t)n_threads > n_out) n_threads = (int)n_out;
    gemm_job jobs[256];
    pthread_t tids[256];
    for (int t = 0; t < n_threads; t++) {
        gemm_job *j = &jobs[t];
        j->out = out;
        j->x = x;
        j->w = (const uint8_t *)w;
        j->wt = wt;
        j->n_out = n_out;
        j->n_in = n_in;
        j->rows = rows;
        j->row_bytes = krk_oracle_row_bytes(wt, n_in);
        j->o_begin = n_out * t / n_threads;
        j->o_end = n_out * (t + 1) / n_threads;
    }
    if (n_threads == 1) {
        gemm_worker(&jobs[0]);
        return 0;
    }
    for (int t = 0; t < n_threads; t++) pthread_create(&tids[t], NULL, gemm_worker, &jobs[t]);
    for (int t = 0; t < n_threads; t++) pthread_join(tids[t], NULL);
    return 0;
}

/* ---- MoE pieces ------------------------------------------------------------------ */

/* src/engine.cpp:11704-11713 (softmax), :11857-11886 (k picks, strict '>' so a tie
 * keeps the lower id), :11913-11918 (renormalise over the picks, slot order). */
int krk_oracle_route(int32_t *ids, float *wts, const float *logits, int64_t n_tok,
                     int n_expert, int k) {
    if (n_expert <= 0 || k <= 0 || k > n_expert) return -1;
    float *prob = (float *)malloc(sizeof(float) * (size_t)n_expert);
    if (!prob) return -1;
    for (int64_t t = 0; t < n_tok; t++) {
        const float *lg = logits + t * n_expert;
        int32_t *sel = ids + t * k;
        float *wt = wts + t * k;
        float mx = lg[0];
        for (int e = 1; e < n_expert; e++) mx = lg[e] > mx ? lg[e] : mx;
        float sum = 0.0f;
        for (int e = 0; e < n_expert; e++) {
            prob[e] = expf(lg[e] - mx);
            sum += prob[e];
        }
        const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
        for (int e = 0; e < n_expert; e++) prob[e] *= inv;
        for (int s = 0; s < k; s++) {
            int best = -1;
            float bestp = -1.0f;
            for (int e = 0; e < n_expert; e++) {
                int taken = 0;
                for (int p = 0; p < s; p++) taken |= (sel[p] == e);
                if (taken) continue;
                if (prob[e] > bestp) {
                    bestp = prob[e];
                    best = e;
                }
            }
            sel[s] = best;
            wt[s] = best >= 0 ? prob[best] : 0.0f;
        }
        float ksum = 0.0f;
        for (int s = 0; s < k; s++) ksum += wt[s];
        const float kinv = ksum > 0.0f ? 1.0f / ksum : 0.0f;
        for (int s = 0; s < k; s++) wt[s] *= kinv;
    }
    free(prob);
    return 0;
}

/* src/backend_cpu.cpp:2394-2400 */
void krk_oracle_silu_mul(float *out, const float *gate, const float *up, int64_t n) {
    for (int64_t i = 0; i < n; i++) {
        const float g = gate[i];
        out[i] = (g / (1.0f + expf(-g))) * up[i];
    }
}

/* src/backend_cpu.cpp:746-778: rows of the table by token id; an id outside [0, n_vocab) gives a zero row */
int krk_oracle_embed(float *out, const void *table, int wt, int64_t n_vocab, int64_t n_embd,
                     const int32_t *tokens, int64_t n_tok) {
    const size_t rb = krk_oracle_row_bytes(wt, n_embd);
    if (rb == 0 && n_embd != 0) return -1;
    for (int64_t t = 0; t < n_tok; t++) {
        float *dst = out + t * n_embd;
        const int32_t id = tokens[t];
        if (id < 0 || (int64_t)id >= n_vocab) {
            memset(dst, 0, (size_t)n_embd * sizeof(float));
            continue;
        }
        if (krk_oracle_dequant_rows(dst, (const uint8_t *)table + (size_t)id * rb, wt, 1, n_embd) != 0) return -1;
    }
    return 0;
}

/* src/backend_cpu.cpp:862-912: key = logit, clamped to +-softcap, then the repetition penalty where the
 * token's mask bit is set; the k largest keys, descending, ties toward the lower id; -1 / -FLT_MAX past
 * the row's length; mass = sum in index order of exp((key - max) / temp). */
static float topk_key(const float *l, const uint32_t *pm, float rep_pen, float softcap, int32_t i) {
    float v = l[i];
    if (softcap > 0.0f) v = v > softcap ? softcap : (v < -softcap ? -softcap : v);
    if (pm && rep_pen > 0.0f && rep_pen != 1.0f && ((pm[(uint32_t)i >> 5] >> ((uint32_t)i & 31)) & 1u))
        v = v > 0.0f ? v / rep_pen : v * rep_pen;
    return v;
}

int krk_oracle_logits_topk(const float *logits, int64_t n, int k, const uint32_t *pen_mask, float rep_pen,
                           float softcap, float temp, int32_t *ids, float *vals, float *mass_out) {
    if (n < 1 || k < 1) return -1;
    const int64_t keep = n < k ? n : k;
    uint8_t *taken = (uint8_t *)calloc((size_t)n, 1);
    if (!taken) return -1;
    for (int r = 0; r < k; r++) {
        if (r >= keep) {
            ids[r] = -1;
            vals[r] = -FLT_MAX;
            continue;
        }
        int64_t best = -1;
        float bv = 0.0f;
        for (int64_t i = 0; i < n; i++) {   /* first maximum in index order = lower id on ties */
            if (taken[i]) continue;
            const float v = topk_key(logits, pen_mask, rep_pen, softcap, (int32_t)i);
            if (best < 0 || v > bv) {
                best = i;
                bv = v;
            }
        }
        taken[best] = 1;
        ids[r] = (int32_t)best;
        vals[r] = bv;
    }
    free(taken);
    if (mass_out) {
        const float inv = temp > 0.0f ? 1.0f / temp : 1.0f, maxv = vals[0];
        float m = 0.0f;
        for (int64_t i = 0; i < n; i++) m += expf((topk_key(logits, pen_mask, rep_pen, softcap, (int32_t)i) - maxv) * inv);
        *mass_out = m;
    }
    return 0;
}

/* src/backend_cpu.cpp:3193-3220 */
void krk_oracle_scatter_axpy_rows(float *dst, const float *src, const int32_t *rows,
                                  const float *alpha, int64_t n_rows, int64_t n) {
    for (int64_t i = 0; i < n_rows; i++) {
        float *d = dst + (int64_t)rows[i] * n;
        const float *s = src + i * n;
        const float a = alpha[i];
        for (int64_t j = 0; j < n; j++) d[j] += a * s[j];
    }
}

/* Per-expert loop of src/engine.cpp:12353-: experts ascending; for each, the tokens
 * routed to it in token order; gate and up GEMV, silu_mul, down GEMV, weighted
 * scatter-add into the zero-filled output. */
int krk_oracle_moe_ffn(float *y, const float *x, const int32_t *ids, const float *wts,
                       const void *const *gate, const void *const *up,
                       const void *const *down, int wt_gate_up, int wt_down,
                       int n_expert, int k, int64_t n_tok, int64_t n_embd, int64_t n_ff,
                       int n_threads) {
    float *g = (float *)malloc(sizeof(float) * (size_t)n_ff * 3);
    float *dn = (float *)malloc(sizeof(float) * (size_t)n_embd);
    if (!g || !dn) {
        free(g);
        free(dn);
        return -1;
    }
    float *u = g + n_ff, *h = g + 2 * n_ff;
    memset(y, 0, sizeof(float) * (size_t)(n_tok * n_embd));
    int rc = 0;
    for (int e = 0; e < n_expert && rc == 0; e++) {
        if (!gate[e] || !up[e] || !down[e]) continue;
        for (int64_t t = 0; t < n_tok && rc == 0; t++) {
            for (int s = 0; s < k; s++) {
                if (ids[t * k + s] != e) continue;
                const float *xt = x + t * n_embd;
                rc |= krk_oracle_gemm(g, xt, gate[e], wt_gate_up, n_ff, n_embd, 1, n_threads);
                rc |= krk_oracle_gemm(u, xt, up[e], wt_gate_up, n_ff, n_embd, 1, n_threads);
                krk_oracle_silu_mul(h, g, u, n_ff);
                rc |= krk_oracle_gemm(dn, h, down[e], wt_down, n_embd, n_ff, 1, n_threads);
                const int32_t row = (int32_t)t;
                const float a = wts[t * k + s];
                krk_oracle_scatter_axpy_rows(y, dn, &row, &a, 1, n_embd);
            }
        }
    }
    free(g);
    free(dn);
    return rc;
}
