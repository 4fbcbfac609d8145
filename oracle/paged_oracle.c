/*
 * CPU oracle for the paged-KV hot path, in C (TEST INFRASTRUCTURE, not product
 * code).  Only the tests, the smoke check and the CPU-baseline leg of the
 * benchmark load this library; nothing in the product path does.
 *
 * It restates, loop for loop, the arithmetic of the reference shaders and of
 * the reference's CPU test helper, so that it can serve both as the parity
 * checker at sizes numpy is too slow for and as the timed CPU baseline.
 * Reference sources (paths relative to the reference project root):
 *   metal = Sources/PagedAttentionMetal/kernels.metal
 *   tests = Tests/PagedAttentionMetalTests/PagedAttentionMetalTests.swift
 *   KVCM  = Sources/PagedAttentionMetal/KVCacheManager.swift
 *
 * Pinning: checked in tests/ against golden vectors produced by the
 * reference's own numpy implementation (Reference/paged_attention_sim.py) and
 * against the numpy oracle.  The FP8 codec and the sliding window follow the
 * shader text only (the reference has no vectors for them): parity unpinned
 * for those two.
 *
 * KV pools use the build's layout [block][kv_head][slot][dim]; the reference
 * addresses the same element as [block][slot][kv_head][dim] (metal:1829-1832).
 *
 * Storage type codes: 0 = float32, 1 = float16, 2 = FP8 e4m3 codes with
 * float16 group scales [block][kv_head], 3 = bfloat16.  Queries are float32
 * for type 0, bfloat16 for type 3 and float16 otherwise (metal:1552).  All
 * outputs are float32, before the final rounding to the storage type.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef _Float16 half_t;

static inline float h2f(uint16_t b) { half_t h; memcpy(&h, &b, 2); return (float)h; }
static inline uint16_t f2h(float f) { half_t h = (half_t)f; uint16_t b; memcpy(&b, &h, 2); return b; }
static inline float bf2f(uint16_t b) { uint32_t u = (uint32_t)b << 16; float f; memcpy(&f, &u, 4); return f; }

/* dequant_fp8 (metal:553-562): all-half arithmetic, evaluated left to right,
 * every product rounded to half. */
static inline float dequant_fp8(uint8_t v, uint16_t scale_bits)
{
    int sign = (v >> 7) & 1, e = (v >> 3) & 0xF, m = v & 7;
    if (e == 0 && m == 0) return 0.0f;
    half_t scale; memcpy(&scale, &scale_bits, 2);
    half_t ss = (half_t)((sign ? (half_t)-1.0f : (half_t)1.0f) * scale);
    half_t frac = (half_t)((half_t)m / (half_t)8.0f);
    if (e == 0) {
        half_t t = (half_t)(ss * frac);
        t = (half_t)(t * (half_t)0.015625f);
        return (float)t;
    }
    half_t one_frac = (half_t)((half_t)1.0f + frac);
    half_t t = (half_t)(ss * one_frac);
    half_t p = (half_t)ldexpf(1.0f, e - 7);
    t = (half_t)(t * p);
    return (float)t;
}

/* quantize_fp8 (metal:564-601). */
static inline uint8_t quantize_fp8(uint16_t value_bits, uint16_t scale_bits)
{
    float v = h2f(value_bits) / h2f(scale_bits);
    if (v < -448.0f) v = -448.0f;
    if (v > 448.0f) v = 448.0f;
    unsigned sign = v < 0.0f ? 1u : 0u;
    v = fabsf(v);
    if (v == 0.0f) return 0;
    if (v < 0x1p-6f) {
        int mi = (int)roundf(v * 512.0f);
        if (mi > 7) mi = 7;
        if (mi < 0) mi = 0;
        return (uint8_t)((sign << 7) | (unsigned)mi);
    }
    int ex;
    float mant = frexpf(v, &ex);
    mant = 2.0f * mant;
    ex -= 1;
    if (ex > 8) return (uint8_t)((sign << 7) | 0x7E);
    int eb = ex + 7;
    int mi = (int)roundf((mant - 1.0f) * 8.0f);
    if (mi > 7) { mi = 0; eb++; }
    if (eb > 0xF) return (uint8_t)((sign << 7) | 0x7E);
    if (eb == 0xF && mi > 6) mi = 6;
    return (uint8_t)((sign << 7) | ((unsigned)eb << 3) | (unsigned)mi);
}

void orc_quantize_fp8(const uint16_t *values, const uint16_t *scales, uint8_t *codes, int64_t n)
{
    for (int64_t i = 0; i < n; i++) codes[i] = quantize_fp8(values[i], scales[i]);
}

void orc_dequant_fp8(const uint8_t *codes, const uint16_t *scales, float *out, int64_t n)
{
    for (int64_t i = 0; i < n; i++) out[i] = dequant_fp8(codes[i], scales[i]);
}

/* Load one token row of a pool as float32. */
static inline void load_row(const void *pool, int64_t elem_off, int D, int dtype, uint16_t scale, float *dst)
{
    if (dtype == 0) {
        memcpy(dst, (const float *)pool + elem_off, (size_t)D * 4);
    } else if (dtype == 1) {
        const uint16_t *p = (const uint16_t *)pool + elem_off;
        for (int d = 0; d < D; d++) dst[d] = h2f(p[d]);
    } else if (dtype == 3) {
        const uint16_t *p = (const uint16_t *)pool + elem_off;
        for (int d = 0; d < D; d++) dst[d] = bf2f(p[d]);
    } else {
        const uint8_t *p = (const uint8_t *)pool + elem_off;
        for (int d = 0; d < D; d++) dst[d] = dequant_fp8(p[d], scale);
    }
}

static inline void load_q(const void *q, int64_t elem_off, int D, int dtype, float *dst)
{
    if (dtype == 0) memcpy(dst, (const float *)q + elem_off, (size_t)D * 4);
    else if (dtype == 3) { const uint16_t *p = (const uint16_t *)q + elem_off; for (int d = 0; d < D; d++) dst[d] = bf2f(p[d]); }
    else { const uint16_t *p = (const uint16_t *)q + elem_off; for (int d = 0; d < D; d++) dst[d] = h2f(p[d]); }
}

/* simd_dot_product (metal:620-632): groups of four, then a scalar tail. */
static inline float dot4(const float *a, const float *b, int D)
{
    float sum = 0.0f;
    int d = 0;
    for (; d + 4 <= D; d += 4)
        sum += a[d] * b[d] + a[d + 1] * b[d + 1] + a[d + 2] * b[d + 2] + a[d + 3] * b[d + 3];
    for (; d < D; d++) sum += a[d] * b[d];
    return sum;
}

/*
 * Batched paged decode: paged_decode_single (metal:1417-1482) and its FP8
 * form (metal:1551-1620).  One (sequence, kv head) pair per OpenMP task; the
 * heads of a group walk the same dequantised K/V rows, each with its own
 * online softmax (m, l, acc) in float32 exactly as metal:1472-1477.
 * A sequence of length 0 leaves 0/0 = NaN like the shader.
 */
void orc_decode(const void *q, const void *k_pool, const void *v_pool, const int32_t *tables,
                const uint32_t *lens, float *out, int B, int H, int KVH, int D, int bs, int max_nb,
                int window, int dtype, const uint16_t *k_scale, const uint16_t *v_scale, int nthreads)
{
    const int G = H / KVH;
    const float scale = 1.0f / sqrtf((float)D);                       /* metal:1441 */
#ifdef _OPENMP
    if (nthreads > 0) omp_set_num_threads(nthreads);
#pragma omp parallel for schedule(dynamic, 1)
#endif
    for (int item = 0; item < B * KVH; item++) {
        int b = item / KVH, kvh = item % KVH;
        uint32_t L = lens[b];
        uint32_t ws = (window > 0 && L > (uint32_t)window) ? L - (uint32_t)window : 0; /* metal:1442 */
        uint32_t nb = (L + bs - 1) / bs;
        if (nb > (uint32_t)max_nb) nb = max_nb;                        /* metal:1451-1452 */
        float *qf = (float *)malloc(sizeof(float) * (size_t)G * D);
        float *acc = (float *)calloc((size_t)G * D, sizeof(float));
        float *m = (float *)malloc(sizeof(float) * G), *l = (float *)malloc(sizeof(float) * G);
        float *kr = (float *)malloc(sizeof(float) * D), *vr = (float *)malloc(sizeof(float) * D);
        for (int g = 0; g < G; g++) {
            load_q(q, ((int64_t)b * H + kvh * G + g) * D, D, dtype, qf + (size_t)g * D);
            m[g] = -INFINITY; l[g] = 0.0f;
        }
        const int32_t *bt = tables + (int64_t)b * max_nb;
        for (uint32_t lb = ws / bs; lb < nb; lb++) {                   /* metal:1454-1455 */
            int64_t pb = bt[lb];
            uint16_t ks = 0, vs = 0;
            if (dtype == 2) { ks = k_scale[pb * KVH + kvh]; vs = v_scale[pb * KVH + kvh]; }
            uint32_t start = lb * bs, end = start + bs < L ? start + bs : L;
            for (uint32_t j = start; j < end; j++) {
                if (j < ws) continue;                                  /* metal:1464 */
                int64_t off = ((pb * KVH + kvh) * bs + (j - start)) * (int64_t)D;
                load_row(k_pool, off, D, dtype, ks, kr);
                load_row(v_pool, off, D, dtype, vs, vr);
                for (int g = 0; g < G; g++) {
                    float dot = dot4(qf + (size_t)g * D, kr, D) * scale;
                    float m_old = m[g];
                    m[g] = fmaxf(m[g], dot);
                    float corr = expf(m_old - m[g]);
                    float p = expf(dot - m[g]);
                    l[g] = l[g] * corr + p;
                    float *a = acc + (size_t)g * D;
                    for (int d = 0; d < D; d++) a[d] = a[d] * corr + p * vr[d];
                }
            }
        }
        for (int g = 0; g < G; g++) {
            float *o = out + ((int64_t)b * H + kvh * G + g) * D;
            for (int d = 0; d < D; d++) o[d] = acc[(size_t)g * D + d] / l[g];   /* metal:1481 */
        }
        free(qf); free(acc); free(m); free(l); free(kr); free(vr);
    }
}

/*
 * Single-sequence paged prefill: paged_attention_tiled (metal:693-765), whose
 * CPU counterpart in the reference is cpuAttention (tests:37-63) with the GQA
 * head map of tests:128-148.  Computes rows [q_start, q_start+q_len) of the
 * sequence (the reference's chunk loop, Engine.swift:740-756, ends with exactly
 * these rows) over keys [window_start, seq_len), key j visible iff j <= row
 * when causal (metal:745).  q holds only the q_len rows.  window_start must be
 * a multiple of the block size for the shader's indexing to be meaningful
 * (metal:734-743).  Rows without a visible key come out as 0/0 = NaN.
 */
void orc_prefill(const void *q, const void *k_pool, const void *v_pool, const int32_t *table,
                 float *out, int seq_len, int H, int KVH, int D, int bs, int causal,
                 int window_start, int q_start, int q_len, int dtype, const uint16_t *k_scale,
                 const uint16_t *v_scale, int nthreads)
{
    const int G = H / KVH;
    const float scale = 1.0f / sqrtf((float)D);                       /* metal:719 */
    /* Dequantise the visible keys of each kv head once; rows then share them. */
    int nkeys = seq_len - window_start;
    if (nkeys < 0) nkeys = 0;
    float *kf = (float *)malloc(sizeof(float) * (size_t)(nkeys > 0 ? nkeys : 1) * KVH * D);
    float *vf = (float *)malloc(sizeof(float) * (size_t)(nkeys > 0 ? nkeys : 1) * KVH * D);
#ifdef _OPENMP
    if (nthreads > 0) omp_set_num_threads(nthreads);
#pragma omp parallel for schedule(static)
#endif
    for (int j = window_start; j < seq_len; j++) {
        int64_t pb = table[j / bs];
        for (int kvh = 0; kvh < KVH; kvh++) {
            uint16_t ks = 0, vs = 0;
            if (dtype == 2) { ks = k_scale[pb * KVH + kvh]; vs = v_scale[pb * KVH + kvh]; }
            int64_t off = ((pb * KVH + kvh) * bs + (j % bs)) * (int64_t)D;
            load_row(k_pool, off, D, dtype, ks, kf + ((size_t)kvh * nkeys + (j - window_start)) * D);
            load_row(v_pool, off, D, dtype, vs, vf + ((size_t)kvh * nkeys + (j - window_start)) * D);
        }
    }
#ifdef _OPENMP
#pragma omp parallel for schedule(dynamic, 4)
#endif
    for (int item = 0; item < q_len * H; item++) {
        int r = item / H, h = item % H;
        int row = q_start + r, kvh = h / G;
        float qf[1024];
        float acc[1024];
        load_q(q, ((int64_t)r * H + h) * D, D, dtype, qf);
        for (int d = 0; d < D; d++) acc[d] = 0.0f;
        float m = -INFINITY, l = 0.0f;
        int end = seq_len;
        if (causal && row + 1 < end) end = row + 1;
        for (int j = window_start; j < end; j++) {
            const float *kr = kf + ((size_t)kvh * nkeys + (j - window_start)) * D;
            const float *vr = vf + ((size_t)kvh * nkeys + (j - window_start)) * D;
            float dot = dot4(qf, kr, D) * scale;
            float m_old = m;
            m = fmaxf(m, dot);
            float corr = expf(m_old - m);
            float p = expf(dot - m);
            l = l * corr + p;
            for (int d = 0; d < D; d++) acc[d] = acc[d] * corr + p * vr[d];
        }
        float *o = out + ((int64_t)r * H + h) * D;
        for (int d = 0; d < D; d++) o[d] = acc[d] / l;                 /* metal:763 */
    }
    free(kf); free(vf);
}

/*
 * KV append by slot mapping: kv_cache_append[_f16] (metal:1804-1874).
 * elem_bytes is the size of one stored element; rows are copied verbatim.
 */
void orc_reshape_and_cache(const void *keys, const void *values, void *k_pool, void *v_pool,
                           const int64_t *slots, int T, int KVH, int D, int bs, int elem_bytes)
{
    size_t row = (size_t)D * elem_bytes;
#ifdef _OPENMP
#pragma omp parallel for schedule(static)
#endif
    for (int t = 0; t < T; t++) {
        int64_t blk = slots[t] / bs, off = slots[t] % bs;
        for (int kvh = 0; kvh < KVH; kvh++) {
            size_t dst = (size_t)((blk * KVH + kvh) * bs + off) * row;
            size_t src = ((size_t)t * KVH + kvh) * row;
            memcpy((char *)k_pool + dst, (const char *)keys + src, row);
            memcpy((char *)v_pool + dst, (const char *)values + src, row);
        }
    }
}

/*
 * FP8 append: kv_cache_scale_fp8 (metal:1876-1905) then kv_cache_append_fp8
 * (metal:1907-1961), with the scale group narrowed from the physical block to
 * (block, kv_head).  scratch must hold blocks*KVH*2 floats; it is cleared here
 * as the reference clears it on every call (Engine.swift:1278-1284).
 */
void orc_reshape_and_cache_fp8(const uint16_t *keys, const uint16_t *values, uint8_t *k_codes,
                               uint8_t *v_codes, uint16_t *k_scale, uint16_t *v_scale,
                               const int64_t *slots, int T, int KVH, int D, int bs,
                               int64_t num_blocks, float *scratch)
{
    memset(scratch, 0, sizeof(float) * (size_t)num_blocks * KVH * 2);
    for (int t = 0; t < T; t++) {                                       /* pass 1 */
        int64_t blk = slots[t] / bs;
        for (int kvh = 0; kvh < KVH; kvh++) {
            float ka = 0.0f, va = 0.0f;
            const uint16_t *k = keys + ((size_t)t * KVH + kvh) * D, *v = values + ((size_t)t * KVH + kvh) * D;
            for (int d = 0; d < D; d++) {
                ka = fmaxf(ka, fabsf(h2f(k[d])));
                va = fmaxf(va, fabsf(h2f(v[d])));
            }
            float *s = scratch + (size_t)(blk * KVH + kvh) * 2;
            s[0] = fmaxf(s[0], ka);
            s[1] = fmaxf(s[1], va);
        }
    }
    /* Group scales first (metal:1942-1954), so that every token of a group is
     * quantised with the same, final scale. */
    for (int t = 0; t < T; t++) {
        int64_t blk = slots[t] / bs;
        for (int kvh = 0; kvh < KVH; kvh++) {
            float *s = scratch + (size_t)(blk * KVH + kvh) * 2;
            if (s[0] < 0.0f) continue;                                   /* already done */
            float km = fmaxf(s[0], h2f(k_scale[blk * KVH + kvh]) * 448.0f);
            float vm = fmaxf(s[1], h2f(v_scale[blk * KVH + kvh]) * 448.0f);
            k_scale[blk * KVH + kvh] = km > 0.0f ? f2h(km / 448.0f) : f2h(1.0f);
            v_scale[blk * KVH + kvh] = vm > 0.0f ? f2h(vm / 448.0f) : f2h(1.0f);
            s[0] = -1.0f;
        }
    }
#ifdef _OPENMP
#pragma omp parallel for schedule(static)
#endif
    for (int t = 0; t < T; t++) {                                       /* pass 2 */
        int64_t blk = slots[t] / bs, off = slots[t] % bs;
        for (int kvh = 0; kvh < KVH; kvh++) {
            uint16_t ks = k_scale[blk * KVH + kvh], vs = v_scale[blk * KVH + kvh];
            const uint16_t *k = keys + ((size_t)t * KVH + kvh) * D, *v = values + ((size_t)t * KVH + kvh) * D;
            size_t dst = (size_t)((blk * KVH + kvh) * bs + off) * D;
            for (int d = 0; d < D; d++) {
                k_codes[dst + d] = quantize_fp8(k[d], ks);
                v_codes[dst + d] = quantize_fp8(v[d], vs);
            }
        }
    }
}

/* Copy-on-write block copies: the two memcpy calls of KVCM:183-189, one pair
 * of blocks at a time, in list order. */
void orc_copy_blocks(void *k_pool, void *v_pool, const int32_t *src, const int32_t *dst, int n,
                     int64_t block_bytes)
{
    for (int i = 0; i < n; i++) {
        memcpy((char *)k_pool + dst[i] * block_bytes, (const char *)k_pool + src[i] * block_bytes, (size_t)block_bytes);
        memcpy((char *)v_pool + dst[i] * block_bytes, (const char *)v_pool + src[i] * block_bytes, (size_t)block_bytes);
    }
}

int orc_max_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
