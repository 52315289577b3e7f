/*
 * sg_oracle.c -- CPU restatement of super-gemma's attention hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker that the CUDA kernels are compared
 * against and the timed CPU baseline; nothing in the shipped library links, loads or calls it.
 *
 * The reference (Rust + WGSL) cannot be compiled or run on this project's machines, so every
 * function below restates one piece of it and names the piece (paths are relative to the
 * reference repository).  Pinning: the reference stores no tensors for this path; its tests are
 * seeded generators compared with an f64 oracle.  What can be pinned is pinned in tests/:
 * the closed-form cases of crates/sg-model/src/reference.rs:572-596, the ring-wrap and zero-block
 * cases of crates/sg-gpu/tests/parity_kv.rs, and an independent numpy restatement.
 * Page-table addressing has no reference implementation at all: parity unpinned for that part
 * (it is pinned here only by the property "paged == linear over gathered rows").
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define SGO_NEG_SENTINEL (-3.0e38f) /* attn_decode_*.wgsl: "m = -3.0e38", not -inf */

/* ------------------------------------------------------------------------------------------ */
/* IEEE binary16 <-> binary32, round-to-nearest-even (the `half` crate's from_f32 / to_f32,    */
/* used by crates/sg-gpu/tests/reference/mod.rs:36-52).                                       */
/* ------------------------------------------------------------------------------------------ */
float sgo_f16_to_f32(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: normalise */
            int e = -1;
            do {
                man <<= 1;
                e++;
            } while ((man & 0x400u) == 0);
            bits = sign | (uint32_t)(127 - 15 - e) << 23 | (man & 0x3FFu) << 13;
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | man << 13;
    } else {
        bits = sign | (exp + 127 - 15) << 23 | man << 13;
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

uint16_t sgo_f32_to_f16(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    uint32_t absx = x & 0x7FFFFFFFu;
    if (absx >= 0x7F800000u) /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | (absx > 0x7F800000u ? 0x200u | ((absx >> 13) & 0x3FFu) : 0));
    if (absx >= 0x477FF000u) /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7C00u);
    if (absx < 0x33000001u) /* < 2^-25 (or exactly 2^-25 -> ties to even zero) */
        return sign;
    int e = (int)(absx >> 23) - 127;
    uint32_t man = (absx & 0x7FFFFFu) | 0x800000u;
    int shift = (e < -14) ? (13 + (-14 - e)) : 13; /* bits dropped */
    uint32_t kept = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (kept & 1u)))
        kept++;
    uint32_t out;
    if (e < -14) {
        out = kept; /* subnormal; a carry into bit 10 lands on the smallest normal, correctly */
    } else {
        out = ((uint32_t)(e + 15) << 10) + (kept - 0x400u); /* carry may bump the exponent */
    }
    return (uint16_t)(sign | out);
}

void sgo_f32_to_f16_vec(const float *x, uint16_t *out, size_t n)
{
    for (size_t i = 0; i < n; i++) out[i] = sgo_f32_to_f16(x[i]);
}

void sgo_f16_to_f32_vec(const uint16_t *x, float *out, size_t n)
{
    for (size_t i = 0; i < n; i++) out[i] = sgo_f16_to_f32(x[i]);
}

/* crates/sg-gpu/tests/reference/mod.rs:36-40 `through_f16` */
void sgo_through_f16(const float *x, float *out, size_t n)
{
    for (size_t i = 0; i < n; i++) out[i] = sgo_f16_to_f32(sgo_f32_to_f16(x[i]));
}

/* ------------------------------------------------------------------------------------------ */
/* Test-input generator of the reference's kernel tests: xorshift64* with uniform [-2, 2)     */
/* floats (crates/sg-gpu/tests/reference/mod.rs:8-32).  `state` is the generator word; a zero  */
/* seed is replaced by 1 as `Rng::new` does.                                                   */
/* ------------------------------------------------------------------------------------------ */
void sgo_rng_seed(uint64_t *state, uint64_t seed) { *state = seed ? seed : 1; }

uint64_t sgo_rng_next_u64(uint64_t *state)
{
    uint64_t x = *state;
    x ^= x >> 12;
    x ^= x << 25;
    x ^= x >> 27;
    *state = x;
    return x * 0x2545F4914F6CDD1DULL;
}

void sgo_rng_f32_vec(uint64_t *state, float *out, size_t n)
{
    for (size_t i = 0; i < n; i++) {
        uint64_t top24 = sgo_rng_next_u64(state) >> 40;
        out[i] = (float)top24 / 16777216.0f * 4.0f - 2.0f;
    }
}

/* ------------------------------------------------------------------------------------------ */
/* Q8_0 in the structure-of-arrays page format.                                                */
/* ------------------------------------------------------------------------------------------ */

static float round_ties_even_f32(float v) { return nearbyintf(v); /* default rounding mode */ }

/*
 * Quantise n (multiple of 32) values the way the GPU producer does: d = amax * (1/127) as an f32
 * multiply, scale = RTNE f16(d), id = 1/d (0 for an all-zero block), q = round_half_even(x*id).
 * crates/sg-gpu/shaders/kv_quant_q8.wgsl:36-56 == tests/reference/mod.rs:272-286 `quant_q8_0`.
 */
void sgo_quant_q8_0(const float *x, size_t n, uint16_t *scales, int8_t *quants)
{
    const float inv127 = 1.0f / 127.0f;
    for (size_t b = 0; b < n / 32; b++) {
        const float *blk = x + b * 32;
        float amax = 0.0f;
        for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(blk[i]));
        float d = amax * inv127;
        float id = d > 0.0f ? 1.0f / d : 0.0f;
        scales[b] = sgo_f32_to_f16(d);
        for (int i = 0; i < 32; i++) quants[b * 32 + i] = (int8_t)(int)round_ties_even_f32(blk[i] * id);
    }
}

/*
 * The tolerance-compared helper of the attention tests: d = amax / 127 (a division), clamp to
 * [-128, 127], and the dequantised values d16 * q that the int8 kernels multiply.
 * tests/reference/mod.rs:58-79 `q8_quant`.  `deq` may be NULL.
 */
void sgo_q8_quant_div(const float *x, size_t n, uint16_t *scales, int8_t *quants, float *deq)
{
    for (size_t b = 0; b < n / 32; b++) {
        const float *blk = x + b * 32;
        float amax = 0.0f;
        for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(blk[i]));
        float d = amax / 127.0f;
        float id = d > 0.0f ? 1.0f / d : 0.0f;
        uint16_t d16 = sgo_f32_to_f16(d);
        float dd = sgo_f16_to_f32(d16);
        scales[b] = d16;
        for (int i = 0; i < 32; i++) {
            int q = (int)round_ties_even_f32(blk[i] * id);
            if (q < -128) q = -128;
            if (q > 127) q = 127;
            quants[b * 32 + i] = (int8_t)q;
            if (deq) deq[b * 32 + i] = dd * (float)q;
        }
    }
}

/* x = f16(d * q): kv_dequant_q8.wgsl:26, attn_prefill_global_flash_sp_q8.wgsl:104,
 * tests/reference/mod.rs:289-299 `dequant_q8_0`.  Output as f16 bit patterns. */
void sgo_dequant_q8_0_f16(const uint16_t *scales, const int8_t *quants, size_t n, uint16_t *out)
{
    for (size_t i = 0; i < n; i++) out[i] = sgo_f32_to_f16(sgo_f16_to_f32(scales[i / 32]) * (float)quants[i]);
}

/* kk = f32(scale) * f32(q), not re-rounded: attn_decode_global_q8k.wgsl:82.  The product of an
 * 11-bit significand and an 8-bit integer is exact in f32. */
void sgo_dequant_q8_0_f32(const uint16_t *scales, const int8_t *quants, size_t n, float *out)
{
    for (size_t i = 0; i < n; i++) out[i] = sgo_f16_to_f32(scales[i / 32]) * (float)quants[i];
}

/* ------------------------------------------------------------------------------------------ */
/* KV placement.                                                                               */
/* ------------------------------------------------------------------------------------------ */

/* kv_append.wgsl:15-37: slot = (pos + token) % ring (ring variant) or pos + token (linear). */
void sgo_kv_append(const uint16_t *src, uint16_t *dst, size_t n_tokens, size_t row_len, uint32_t pos,
                   uint32_t ring /* 0 = linear */)
{
    for (size_t t = 0; t < n_tokens; t++) {
        size_t slot = ring ? (pos + t) % ring : pos + t;
        memcpy(dst + slot * row_len, src + t * row_len, row_len * sizeof(uint16_t));
    }
}

/* Logical token -> physical row.  The reference has no page table (its resident global KV is
 * linear); this build defines row = page_table[t / page] * page + t % page, after which the
 * reference's own SoA indexing applies with t := row (attn_decode_global_q8k.wgsl:76-77). */
static inline size_t phys_row(size_t t, const uint32_t *page_table, uint32_t page)
{
    return page_table ? (size_t)page_table[t / page] * page + t % page : t;
}

/* kv_append_global_q8.wgsl:19-60 with the page-table row mapping above (page_table NULL =
 * the reference's linear placement).  src is f16 bits [n_tokens x row_len]. */
void sgo_kv_append_q8(const uint16_t *src, uint16_t *scales, int8_t *quants, size_t n_tokens, size_t row_len,
                      uint32_t pos, const uint32_t *page_table, uint32_t page)
{
    float tmp[32];
    size_t bpr = row_len / 32;
    for (size_t t = 0; t < n_tokens; t++) {
        size_t row = phys_row(pos + t, page_table, page);
        for (size_t b = 0; b < bpr; b++) {
            for (int i = 0; i < 32; i++) tmp[i] = sgo_f16_to_f32(src[t * row_len + b * 32 + i]);
            sgo_quant_q8_0(tmp, 32, scales + row * bpr + b, quants + (row * bpr + b) * 32);
        }
    }
}

/* ------------------------------------------------------------------------------------------ */
/* K/V sources as the kernels see them.                                                        */
/* ------------------------------------------------------------------------------------------ */
typedef struct {
    const uint16_t *f16;        /* f16 rows [row x n_kv x hd], or NULL when quantised */
    const int8_t *quants;       /* Q8_0 quants [row x n_kv x hd] */
    const uint16_t *scales;     /* Q8_0 scales [row x n_kv x hd/32] */
    const uint32_t *page_table; /* NULL = linear */
    uint32_t page;              /* tokens per page */
    uint32_t round_f16;         /* 1: dequantised value re-rounded to f16 (prefill slab), 0: exact f32 */
} sgo_kv_src;

/* Inner-loop conversions through the compiler's _Float16 (exact widening; RTNE narrowing), so
 * the timed baseline is not dominated by bit twiddling.  tests/ check them against the
 * bit-level routines above over all 65536 patterns. */
static inline float h2f(uint16_t h)
{
    _Float16 x;
    memcpy(&x, &h, 2);
    return (float)x;
}
static inline float round_through_f16(float v) { return (float)(_Float16)v; }

float sgo_h2f_fast(uint16_t h) { return h2f(h); }
float sgo_round_through_f16_fast(float v) { return round_through_f16(v); }

static inline void kv_row(const sgo_kv_src *s, size_t t, int kvh, int n_kv, int hd, float *out)
{
    size_t r = phys_row(t, s->page_table, s->page);
    if (s->f16) {
        const uint16_t *p = s->f16 + (r * n_kv + kvh) * hd;
        for (int d = 0; d < hd; d++) out[d] = h2f(p[d]);
    } else {
        const int8_t *qp = s->quants + (r * n_kv + kvh) * hd;
        const uint16_t *sp = s->scales + (r * n_kv + kvh) * (hd / 32);
        for (int b = 0; b < hd / 32; b++) {
            float sc = h2f(sp[b]);
            for (int d = 32 * b; d < 32 * b + 32; d++) {
                float v = sc * (float)qp[d];
                out[d] = s->round_f16 ? round_through_f16(v) : v;
            }
        }
    }
}

/* Materialise a source as linear f32 rows [n_tokens x n_kv x hd] (what the f64 oracle consumes:
 * "dequantised inputs", as parity_attn.rs:756-768 and :1077-1089 do). */
void sgo_kv_materialize(const sgo_kv_src *s, size_t n_tokens, int n_kv, int hd, float *out)
{
#pragma omp parallel for schedule(static)
    for (long t = 0; t < (long)n_tokens; t++)
        for (int h = 0; h < n_kv; h++) kv_row(s, (size_t)t, h, n_kv, hd, out + ((size_t)t * n_kv + h) * hd);
}

/* ------------------------------------------------------------------------------------------ */
/* Ground truth: f64 softmax attention for one (query token, query head) over keys [t0, t1]   */
/* inclusive.  tests/reference/mod.rs:224-263 `attention_head`.  q [m x H x hd], k/v           */
/* [l x KV x hd] as f32 holding f16-representable (or dequantised) values.                     */
/* ------------------------------------------------------------------------------------------ */
void sgo_attention_head(const float *q, const float *k, const float *v, size_t i, int qh, int n_q, int n_kv, int hd,
                        double scale, size_t t0, size_t t1, float *out)
{
    int kvh = qh / (n_q / n_kv);
    const float *qrow = q + (i * n_q + qh) * hd;
    size_t n = t1 - t0 + 1;
    double *sc = (double *)malloc(n * sizeof(double));
    double mx = -INFINITY;
    for (size_t t = t0; t <= t1; t++) {
        const float *krow = k + (t * n_kv + kvh) * hd;
        double dot = 0.0;
        for (int d = 0; d < hd; d++) dot += (double)qrow[d] * (double)krow[d];
        sc[t - t0] = dot * scale;
        if (sc[t - t0] > mx) mx = sc[t - t0];
    }
    double denom = 0.0;
    for (size_t j = 0; j < n; j++) {
        sc[j] = exp(sc[j] - mx);
        denom += sc[j];
    }
    for (int d = 0; d < hd; d++) {
        double acc = 0.0;
        for (size_t j = 0; j < n; j++) acc += sc[j] * (double)v[((t0 + j) * n_kv + kvh) * hd + d];
        out[d] = (float)(acc / denom);
    }
    free(sc);
}

/*
 * Whole-chunk form: m query tokens at absolute positions q0 + i, causal, optional window
 * (0 = none): query i sees keys [max(0, q0+i+1-window), q0+i].  One task per (token, head) as
 * crates/sg-model/src/reference.rs:482-530 `attention` parallelises it.  `tokens`/`heads` select
 * a subset (NULL = all) so long contexts can be sampled; out is [n_tok_sel x n_head_sel x hd].
 */
void sgo_attention_f64(const float *q, const float *k, const float *v, size_t m, size_t q0, int n_q, int n_kv, int hd,
                       size_t window, double scale, const uint32_t *tokens, size_t n_tokens, const uint32_t *heads,
                       size_t n_heads, float *out)
{
    size_t nt = tokens ? n_tokens : m;
    size_t nh = heads ? n_heads : (size_t)n_q;
#pragma omp parallel for schedule(dynamic, 1)
    for (long job = 0; job < (long)(nt * nh); job++) {
        size_t i = tokens ? tokens[job / nh] : (size_t)(job / nh);
        int qh = heads ? (int)heads[job % nh] : (int)(job % nh);
        size_t qpos = q0 + i;
        size_t t0 = (window && qpos + 1 > window) ? qpos + 1 - window : 0;
        sgo_attention_head(q, k, v, i, qh, n_q, n_kv, hd, scale, t0, qpos, out + (size_t)job * hd);
    }
}

/* ------------------------------------------------------------------------------------------ */
/* f32 restatements in the shaders' operation order (secondary check and the timed baseline).  */
/* ------------------------------------------------------------------------------------------ */

/* One streaming-softmax step: attn_decode_global_q8k.wgsl:84-98 (identical in every scalar
 * attention shader). */
static inline void stream_step(const float *qr, const float *kk, const float *vv, int hd, float scale, float *m,
                               float *l, float *acc)
{
    float dot = 0.0f;
    for (int d = 0; d < hd; d++) dot += qr[d] * kk[d];
    float s = dot * scale;
    float m_new = fmaxf(*m, s);
    float corr = expf(*m - m_new);
    float w = expf(s - m_new);
    *l = *l * corr + w;
    for (int d = 0; d < hd; d++) acc[d] = acc[d] * corr + w * vv[d];
    *m = m_new;
}

/*
 * Split-K decode partials.  attn_decode_sliding.wgsl:29-121 / attn_decode_global_q8k.wgsl:18-112:
 * grid (kv head, split); chunk = ceil(kv_len / n_splits); split s covers
 * [min(s*chunk, kv_len), min(s*chunk + chunk, kv_len)); an empty split leaves m = -3e38, l = 0.
 * part[(row * n_splits + split) * (hd + 2)] = acc[hd], m, l with row = i * H + qh.
 * m_q > 1 is this build's multi-query extension (no reference kernel): query i of m_q sees keys
 * t <= kv_len - m_q + i, so m_q = 1 is exactly the reference.
 */
void sgo_decode_partials_f32(const uint16_t *q_f16, const sgo_kv_src *ks, const sgo_kv_src *vs, float *part, int n_q,
                             int n_kv, int hd, uint32_t kv_len, uint32_t n_splits, float scale, uint32_t m_q)
{
    int g = n_q / n_kv;
    uint32_t chunk = (kv_len + n_splits - 1) / n_splits;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int kvh = 0; kvh < n_kv; kvh++) {
        for (long split = 0; split < (long)n_splits; split++) {
            uint32_t t_begin = (uint32_t)split * chunk < kv_len ? (uint32_t)split * chunk : kv_len;
            uint32_t t_end = t_begin + chunk < kv_len ? t_begin + chunk : kv_len;
            int rows = (int)m_q * g;
            float *qr = (float *)malloc(sizeof(float) * (size_t)rows * hd);
            float *acc = (float *)calloc((size_t)rows * hd, sizeof(float));
            float *m = (float *)malloc(sizeof(float) * rows), *l = (float *)calloc(rows, sizeof(float));
            float *kk = (float *)malloc(sizeof(float) * hd), *vv = (float *)malloc(sizeof(float) * hd);
            for (int r = 0; r < rows; r++) {
                int i = r / g, qh = kvh * g + r % g;
                m[r] = SGO_NEG_SENTINEL;
                for (int d = 0; d < hd; d++) qr[r * hd + d] = h2f(q_f16[((size_t)i * n_q + qh) * hd + d]);
            }
            for (uint32_t t = t_begin; t < t_end; t++) {
                kv_row(ks, t, kvh, n_kv, hd, kk);
                kv_row(vs, t, kvh, n_kv, hd, vv);
                for (int r = 0; r < rows; r++) {
                    uint32_t i = (uint32_t)(r / g);
                    if (t + m_q > kv_len + i) continue; /* t > kv_len - m_q + i */
                    stream_step(qr + r * hd, kk, vv, hd, scale, &m[r], &l[r], acc + r * hd);
                }
            }
            for (int r = 0; r < rows; r++) {
                int i = r / g, qh = kvh * g + r % g;
                float *p = part + (((size_t)i * n_q + qh) * n_splits + (size_t)split) * (hd + 2);
                memcpy(p, acc + r * hd, sizeof(float) * hd);
                p[hd] = m[r];
                p[hd + 1] = l[r];
            }
            free(qr); free(acc); free(m); free(l); free(kk); free(vv);
        }
    }
}

/*
 * Split-K combine in fixed ascending split order.  attn_reduce.wgsl:29-56.
 * out_mode 0: out[row*hd + d] = acc/l (f32; the reference stores f16(acc/l), see out_f16).
 * out_mode 1: out[row*(hd+2)] = merged acc[hd], m, l -- this build's unnormalised form for the
 * cross-GPU (m, l, O) exchange; merging those again with out_mode 0 equals merging all splits.
 */
void sgo_reduce_f32(const float *part, float *out, uint16_t *out_f16, size_t rows, int hd, uint32_t n_splits,
                    int out_mode)
{
#pragma omp parallel for schedule(static)
    for (long r = 0; r < (long)rows; r++) {
        float m = SGO_NEG_SENTINEL, l = 0.0f;
        float *acc = (float *)calloc(hd, sizeof(float));
        for (uint32_t s = 0; s < n_splits; s++) {
            const float *p = part + ((size_t)r * n_splits + s) * (hd + 2);
            float ms = p[hd], ls = p[hd + 1];
            float m_new = fmaxf(m, ms);
            float ca = expf(m - m_new), cb = expf(ms - m_new);
            for (int d = 0; d < hd; d++) acc[d] = acc[d] * ca + p[d] * cb;
            l = l * ca + ls * cb;
            m = m_new;
        }
        if (out_mode == 1) {
            float *o = out + (size_t)r * (hd + 2);
            memcpy(o, acc, sizeof(float) * hd);
            o[hd] = m;
            o[hd + 1] = l;
        } else {
            for (int d = 0; d < hd; d++) {
                float y = acc[d] / l;
                if (out) out[(size_t)r * hd + d] = y;
                if (out_f16) out_f16[(size_t)r * hd + d] = sgo_f32_to_f16(y);
            }
        }
        free(acc);
    }
}

/*
 * Scalar streaming prefill over up to two key ranges, in position order:
 *   history positions [t_begin, min(q0, qpos+1)) read from `hist` at row t % ring (ring > 0,
 *   attn_prefill_sliding_ring.wgsl:88-113) or at row t (ring == 0: the linear kernels
 *   attn_prefill_sliding.wgsl:53-57,78 and attn_prefill_global.wgsl:53,74, for which the caller
 *   passes chunk sources = NULL and the whole range comes from `hist`);
 *   chunk positions [max(q0, t_begin), qpos] read from `chunk` at row pos - q0 (:115-140).
 * window 0 = global causal.  out f32 [m x H x hd] (the reference stores f16(acc/l)).
 */
void sgo_prefill_stream_f32(const uint16_t *q_f16, const sgo_kv_src *k_hist, const sgo_kv_src *v_hist,
                            const sgo_kv_src *k_chunk, const sgo_kv_src *v_chunk, float *out, uint16_t *out_f16,
                            size_t m_tokens, uint32_t q0, int n_q, int n_kv, int hd, uint32_t window, uint32_t ring,
                            float scale)
{
    int g = n_q / n_kv;
#pragma omp parallel for collapse(2) schedule(dynamic, 4)
    for (long i = 0; i < (long)m_tokens; i++) {
        for (int kvh = 0; kvh < n_kv; kvh++) {
            uint32_t qpos = q0 + (uint32_t)i;
            uint32_t t_begin = (window && qpos + 1 > window) ? qpos + 1 - window : 0;
            float *qr = (float *)malloc(sizeof(float) * (size_t)g * hd);
            float *acc = (float *)calloc((size_t)g * hd, sizeof(float));
            float m[64], l[64];
            float *kk = (float *)malloc(sizeof(float) * hd), *vv = (float *)malloc(sizeof(float) * hd);
            for (int r = 0; r < g; r++) {
                m[r] = SGO_NEG_SENTINEL;
                l[r] = 0.0f;
                for (int d = 0; d < hd; d++)
                    qr[r * hd + d] = h2f(q_f16[((size_t)i * n_q + kvh * g + r) * hd + d]);
            }
            uint32_t hist_end = k_chunk ? (q0 < qpos + 1 ? q0 : qpos + 1) : qpos + 1;
            for (uint32_t t = t_begin; t < hist_end; t++) {
                size_t row = ring ? t % ring : t;
                kv_row(k_hist, row, kvh, n_kv, hd, kk);
                kv_row(v_hist, row, kvh, n_kv, hd, vv);
                for (int r = 0; r < g; r++) stream_step(qr + r * hd, kk, vv, hd, scale, &m[r], &l[r], acc + r * hd);
            }
            if (k_chunk) {
                uint32_t c_begin = t_begin > q0 ? t_begin - q0 : 0;
                for (uint32_t c = c_begin; c <= (uint32_t)i; c++) {
                    kv_row(k_chunk, c, kvh, n_kv, hd, kk);
                    kv_row(v_chunk, c, kvh, n_kv, hd, vv);
                    for (int r = 0; r < g; r++)
                        stream_step(qr + r * hd, kk, vv, hd, scale, &m[r], &l[r], acc + r * hd);
                }
            }
            for (int r = 0; r < g; r++)
                for (int d = 0; d < hd; d++) {
                    size_t o = ((size_t)i * n_q + kvh * g + r) * hd + d;
                    float y = acc[r * hd + d] / l[r];
                    if (out) out[o] = y;
                    if (out_f16) out_f16[o] = sgo_f32_to_f16(y);
                }
            free(qr); free(acc); free(kk); free(vv);
        }
    }
}

/*
 * Single-pass flash prefill in the tile order of attn_prefill_global_flash_sp.wgsl:118-188 /
 * attn_prefill_global_flash_sp_q8.wgsl (K and V dequantised to f16 first): per tile of `tile_k`
 * keys (64 in the reference) m_new = max(m, s*scale over visible keys), corr = exp(m - m_new),
 * p = exp(s*scale - m_new), l += p in f32 BEFORE P = f16(p), O = O*corr + P*V, out = O / l.
 * Keys come from one linear-or-paged source with round_f16 semantics decided by the source;
 * window 0 = global causal.  `tokens` selects query rows (NULL = all m); out [n_sel x H x hd].
 */
void sgo_prefill_flash_f32(const uint16_t *q_f16, const sgo_kv_src *ks, const sgo_kv_src *vs, float *out,
                           size_t m_tokens, uint32_t q0, int n_q, int n_kv, int hd, uint32_t window, float scale,
                           uint32_t tile_k, const uint32_t *tokens, size_t n_tokens)
{
    size_t nt = tokens ? n_tokens : m_tokens;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (long ti = 0; ti < (long)nt; ti++) {
        for (int qh = 0; qh < n_q; qh++) {
            size_t i = tokens ? tokens[ti] : (size_t)ti;
            int kvh = qh / (n_q / n_kv);
            uint32_t qpos = q0 + (uint32_t)i;
            uint32_t lo = (window && qpos + 1 > window) ? qpos + 1 - window : 0;
            float *qr = (float *)malloc(sizeof(float) * hd), *o = (float *)calloc(hd, sizeof(float));
            float *kk = (float *)malloc(sizeof(float) * hd), *vrow = (float *)malloc(sizeof(float) * hd);
            float *s = (float *)malloc(sizeof(float) * tile_k), *p = (float *)malloc(sizeof(float) * tile_k);
            for (int d = 0; d < hd; d++) qr[d] = h2f(q_f16[(i * n_q + qh) * hd + d]);
            float m = SGO_NEG_SENTINEL, l = 0.0f;
            for (uint32_t k0 = (lo / tile_k) * tile_k; k0 <= qpos; k0 += tile_k) {
                float m_new = m;
                for (uint32_t j = 0; j < tile_k; j++) {
                    uint32_t t = k0 + j;
                    if (t < lo || t > qpos) continue;
                    kv_row(ks, t, kvh, n_kv, hd, kk);
                    float dot = 0.0f;
                    for (int d = 0; d < hd; d++) dot += qr[d] * kk[d];
                    s[j] = dot;
                    m_new = fmaxf(m_new, dot * scale);
                }
                float corr = expf(m - m_new);
                float lsum = l * corr;
                for (uint32_t j = 0; j < tile_k; j++) {
                    uint32_t t = k0 + j;
                    float pj = (t < lo || t > qpos) ? 0.0f : expf(s[j] * scale - m_new);
                    lsum += pj;
                    p[j] = round_through_f16(pj);
                }
                for (int d = 0; d < hd; d++) o[d] *= corr;
                for (uint32_t j = 0; j < tile_k; j++) {
                    if (p[j] == 0.0f) continue;
                    kv_row(vs, k0 + j, kvh, n_kv, hd, vrow);
                    for (int d = 0; d < hd; d++) o[d] += p[j] * vrow[d];
                }
                l = lsum;
                m = m_new;
            }
            for (int d = 0; d < hd; d++) out[((size_t)ti * n_q + qh) * hd + d] = o[d] / l;
            free(qr); free(o); free(kk); free(vrow); free(s); free(p);
        }
    }
}

/* Launchers such as torchrun export OMP_NUM_THREADS=1; the timed baseline asks for what it wants. */
void sgo_set_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int sgo_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
