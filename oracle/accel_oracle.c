/*
 * accel_oracle.c -- CPU restatement of golang-design/accel's CPU-backend arithmetic for the
 * quantized decode path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the parity checker and the timed CPU baseline.  It is never linked into, imported
 * by or called from the product library; only the test-suite, the smoke check and the benchmark's
 * CPU-baseline leg may load it.
 *
 * Every function follows the summation ORDER of the reference's generated CPU lowering, with every
 * product and sum rounded to binary32 (build with -ffp-contract=off, no -ffast-math), so that the
 * results are what the reference's CPU backend computes on the same inputs.  The reference
 * executes workgroups in parallel over the host cores; so does this file (OpenMP over workgroups).
 *
 * Pinning: the reference (a Go module) cannot be built in this environment, and its tests hold no
 * committed numeric output vectors; they hold deterministic known-answer fixtures and exactness
 * differentials (nibble order 40-vs-4, constant group, odd-length packing, paged == contiguous and
 * batched == one-at-a-time bit for bit, block-pool page lists).  tests/test_oracle_pins.py replays
 * every one of those against this file.
 *
 * Reference citations are paths inside the accel module.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* How many host threads the parallel loops below use.  A launcher may export OMP_NUM_THREADS=1 to
 * its children (torch.distributed.run does); the timed CPU baseline overrides that here so that it
 * always runs on the cores the host really has. */
ORC_API void orc_set_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

ORC_API int orc_max_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------------------------------ */
/* f32 <-> f16, internal/kernel/narrow.go:67-140                                               */
/* ------------------------------------------------------------------------------------------ */

static inline uint32_t f32_bits(float x) { uint32_t b; memcpy(&b, &x, 4); return b; }
static inline float bits_f32(uint32_t b) { float x; memcpy(&x, &b, 4); return x; }

/* round-to-nearest-even right shift, the helper ToFloat16 uses for both the normal and the
 * subnormal branch (internal/kernel/narrow.go, roundShift). */
static inline uint32_t round_shift(uint32_t v, uint32_t shift)
{
    if (shift == 0) return v;
    if (shift > 31) return 0;
    uint32_t half = 1u << (shift - 1);
    uint32_t mask = (1u << shift) - 1;
    uint32_t q = v >> shift;
    uint32_t rem = v & mask;
    if (rem > half || (rem == half && (q & 1u))) q++;
    return q;
}

ORC_API uint16_t orc_f32_to_f16(float x)
{
    uint32_t b = f32_bits(x);
    uint16_t sign = (uint16_t)((b >> 16) & 0x8000u);
    int32_t exp = (int32_t)((b >> 23) & 0xffu) - 127;
    uint32_t mant = b & 0x7fffffu;

    if ((b & 0x7fffffffu) > 0x7f800000u) return 0x7e00;            /* NaN: canonical quiet */
    if (exp == 128) return (uint16_t)(sign | 0x7c00u);             /* infinity */
    if (exp > 15) return (uint16_t)(sign | 0x7c00u);               /* overflow */
    if (exp < -24) return sign;                                    /* flushed, sign kept */
    if (exp < -14) {                                               /* subnormal */
        mant |= 0x800000u;
        uint32_t shift = (uint32_t)(-exp - 14);
        return (uint16_t)(sign | (uint16_t)round_shift(mant, 13 + shift));
    }
    uint32_t half = ((uint32_t)(exp + 15) << 10) + round_shift(mant, 13);   /* added: carries */
    return (uint16_t)(sign | (uint16_t)half);
}

ORC_API float orc_f16_to_f32(uint16_t h)
{
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = ((uint32_t)h >> 10) & 0x1fu;
    uint32_t mant = (uint32_t)h & 0x3ffu;
    if (exp == 0) {
        if (mant == 0) return bits_f32(sign);
        uint32_t shift = 0;
        while ((mant & 0x400u) == 0) { mant <<= 1; shift++; }
        mant &= 0x3ffu;
        return bits_f32(sign | ((127 - 15 + 1 - shift) << 23) | (mant << 13));
    }
    if (exp == 0x1f) {
        if (mant == 0) return bits_f32(sign | 0x7f800000u);
        return bits_f32(sign | 0x7f800000u | (mant << 13));
    }
    return bits_f32(sign | ((exp + 127 - 15) << 23) | (mant << 13));
}

ORC_API void orc_cast_f32_to_f16(const float *in, uint16_t *out, size_t n)
{   /* internal/kernels/cast.go:30 */
    for (size_t i = 0; i < n; i++) out[i] = orc_f32_to_f16(in[i]);
}

ORC_API void orc_cast_f16_to_f32(const uint16_t *in, float *out, size_t n)
{
    for (size_t i = 0; i < n; i++) out[i] = orc_f16_to_f32(in[i]);
}

/* kmath/kmath.go:40-104: every intrinsic is the double-precision routine rounded once. */
static inline float k_exp(float x) { return (float)exp((double)x); }
static inline float k_log(float x) { return (float)log((double)x); }
static inline float k_sin(float x) { return (float)sin((double)x); }
static inline float k_cos(float x) { return (float)cos((double)x); }
static inline float k_rsqrt(float x) { return (float)(1.0 / sqrt((double)x)); }
static inline float k_max(float x, float y)
{
    if (isnan(x) || isnan(y)) return NAN;
    return x > y ? x : y;
}

/* ------------------------------------------------------------------------------------------ */
/* int4 quantizer, quant/int4.go:71-175                                                        */
/* ------------------------------------------------------------------------------------------ */

/* `group` is quant.Int4Group (128) in the reference; it is a parameter here so that a group-32
 * variant can be restated with the constant changed (that variant has no reference test). */
ORC_API void orc_int4_quantize(const float *w, size_t n, uint32_t *packed, uint16_t *scales,
                               uint16_t *zeros, uint32_t group)
{
    size_t groups = (n + group - 1) / group;
    size_t words = (n + 7) / 8;
    memset(packed, 0, words * sizeof(uint32_t));
#pragma omp parallel for schedule(static)
    for (size_t g = 0; g < groups; g++) {
        size_t lo = g * group;
        size_t hi = lo + group < n ? lo + group : n;
        float lowest = w[lo], highest = w[lo];
        for (size_t i = lo; i < hi; i++) {
            if (w[i] < lowest) lowest = w[i];
            if (w[i] > highest) highest = w[i];
        }
        if (highest == lowest) {                    /* constant group: s = 0, z = value */
            scales[g] = orc_f32_to_f16(0.0f);
            zeros[g] = orc_f32_to_f16(lowest);
            continue;
        }
        float s = (highest - lowest) / 15.0f;
        scales[g] = orc_f32_to_f16(s);
        float s16 = orc_f16_to_f32(scales[g]);
        if (s16 == 0) {                             /* scale underflowed f16 */
            zeros[g] = orc_f32_to_f16(lowest);
            continue;
        }
        float z = -lowest / s16;
        zeros[g] = orc_f32_to_f16(z);
        float z16 = orc_f16_to_f32(zeros[g]);
        for (size_t i = lo; i < hi; i++) {
            double q = nearbyint((double)w[i] / (double)s16 + (double)z16); /* RoundToEven */
            if (q > 15) q = 15;
            if (q < 0) q = 0;
            /* a group is a whole number of words when group % 8 == 0, so no two threads share
             * a word; a trailing partial word belongs to the last group alone. */
            uint32_t shift = 4u * (uint32_t)(i % 8);
            packed[i / 8] = (packed[i / 8] & ~(0xFu << shift)) | ((uint32_t)q << shift);
        }
    }
}

ORC_API uint32_t orc_int4_nibble(const uint32_t *packed, size_t i)
{   /* quant/int4.go:151 */
    return (packed[i / 8] >> (4 * (i % 8))) & 0xFu;
}

ORC_API void orc_int4_dequantize(const uint32_t *packed, const uint16_t *scales,
                                 const uint16_t *zeros, size_t n, float *out, uint32_t group)
{   /* quant/int4.go:160-175 */
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) {
        size_t g = i / group;
        float s = orc_f16_to_f32(scales[g]);
        float z = orc_f16_to_f32(zeros[g]);
        if (s == 0) { out[i] = z; continue; }
        out[i] = ((float)orc_int4_nibble(packed, i) - z) * s;
    }
}

static double ulp16(uint16_t f)
{   /* quant/int4.go:243-253 */
    int e = ((int)f >> 10) & 0x1f;
    if (e == 0x1f) return INFINITY;
    if (e == 0) return ldexp(1.0, -24);
    return ldexp(1.0, e - 25);
}

ORC_API double orc_int4_error_bound(const float *x, const uint16_t *term_scales,
                                    const uint16_t *term_zeros, size_t n)
{   /* quant/int4.go:213-239 */
    const double u = 1.0 / (double)(1 << 24);
    double sum = 0;
    for (size_t i = 0; i < n; i++) {
        double s = (double)orc_f16_to_f32(term_scales[i]);
        double z = (double)orc_f16_to_f32(term_zeros[i]);
        double e;
        if (s == 0) {
            e = ulp16(term_zeros[i]) / 2;
        } else {
            double ds = ulp16(term_scales[i]) / 2 + 2 * u * s;
            double dz = ulp16(term_zeros[i]) / 2 + u * fabs(z);
            e = s / 2 + 15 * ds + dz * s;
        }
        sum += fabs((double)x[i]) * e;
    }
    return sum;
}

static inline float int4_weight(const uint32_t *bq, const uint16_t *bs, const uint16_t *bz,
                                uint64_t w, uint32_t group)
{   /* the decode both int4 kernels spell: internal/kernels/int4.go:74-87 */
    uint32_t code = (bq[w / 8] >> (4 * (w % 8))) & 0xFu;
    uint64_t g = w / group;
    float s = orc_f16_to_f32(bs[g]);
    float z = orc_f16_to_f32(bz[g]);
    float wv = ((float)code - z) * s;
    if (s == 0) wv = z;
    return wv;
}

/* ------------------------------------------------------------------------------------------ */
/* QuantMatVecInt4, internal/kernels/int4.go:60-101 (workgroup 32x16)                          */
/* ------------------------------------------------------------------------------------------ */
ORC_API void orc_quant_matvec_int4(uint32_t N, uint32_t K, const float *a, const uint32_t *bq,
                                   const uint16_t *bs, const uint16_t *bz, float *out,
                                   uint32_t group)
{
    const uint32_t phases = 16;       /* MatVecPhases, internal/kernels/matvec.go:64-67 */
#pragma omp parallel for schedule(static)
    for (uint32_t col = 0; col < N; col++) {
        float part[16];
        for (uint32_t ly = 0; ly < phases; ly++) {
            float acc = 0;
            for (uint32_t k = ly; k < K; k += phases) {
                float wv = int4_weight(bq, bs, bz, (uint64_t)k * N + col, group);
                acc = acc + a[k] * wv;
            }
            part[ly] = acc;
        }
        float sum = 0;
        for (uint32_t p = 0; p < phases; p++) sum = sum + part[p];
        out[col] = sum;
    }
}

/* ------------------------------------------------------------------------------------------ */
/* QuantMatMulInt4, internal/kernels/int4tiled.go:66-137: one accumulator per output element,   */
/* sequential in k; the zero padding of the tiles adds exact zeros and changes no bits.         */
/* ------------------------------------------------------------------------------------------ */
ORC_API void orc_quant_matmul_int4(uint32_t M, uint32_t N, uint32_t K, const float *a,
                                   const uint32_t *bq, const uint16_t *bs, const uint16_t *bz,
                                   float *out, uint32_t group)
{
    /* Dequantize one strip of 16 columns at a time so each weight is decoded once per strip,
     * which is what the tile load does; the arithmetic per output is unchanged. */
    const uint32_t TN = 16;
    uint32_t strips = (N + TN - 1) / TN;
#pragma omp parallel
    {
        float *wcol = (float *)malloc((size_t)K * TN * sizeof(float));
#pragma omp for schedule(dynamic, 4)
        for (uint32_t sidx = 0; sidx < strips; sidx++) {
            uint32_t n0 = sidx * TN;
            uint32_t nn = N - n0 < TN ? N - n0 : TN;
            for (uint32_t k = 0; k < K; k++)
                for (uint32_t j = 0; j < nn; j++)
                    wcol[(size_t)k * TN + j] =
                        int4_weight(bq, bs, bz, (uint64_t)k * N + n0 + j, group);
            for (uint32_t m = 0; m < M; m++) {
                float acc[16];
                for (uint32_t j = 0; j < TN; j++) acc[j] = 0;
                const float *am = a + (size_t)m * K;
                for (uint32_t k = 0; k < K; k++) {
                    float av = am[k];
                    const float *wr = wcol + (size_t)k * TN;
                    for (uint32_t j = 0; j < nn; j++) acc[j] = acc[j] + av * wr[j];
                }
                for (uint32_t j = 0; j < nn; j++) out[(size_t)m * N + n0 + j] = acc[j];
            }
        }
        free(wcol);
    }
}

/* ------------------------------------------------------------------------------------------ */
/* Decode attention: internal/kernels/attention.go:97 (contiguous), paged.go:47,362,            */
/* batched.go:53.  The four share one body that differs only in addressing.                     */
/* ------------------------------------------------------------------------------------------ */
#define ATTN_BLOCK 128u    /* AttnBlock, internal/kernels/attention.go:39 */

typedef struct {
    const float *q;            /* this head's query row */
    const void *k, *v;         /* cache base */
    int f16;                   /* cache dtype */
    const uint32_t *pages;     /* this sequence's page-table row, or NULL for contiguous */
    uint32_t block;            /* positions per page */
    uint32_t kv_heads, head_dim, kv_head;
    uint32_t kv_len;           /* already clamped */
    float scale;
    uint32_t sgw;              /* subgroup width; the CPU profile reports 4
                                  (internal/cpu/profile.go:224-228) */
} attn_unit;

static inline float cache_at(const attn_unit *u, const void *base, uint64_t idx)
{
    return u->f16 ? orc_f16_to_f32(((const uint16_t *)base)[idx]) : ((const float *)base)[idx];
}

static inline uint64_t attn_row(const attn_unit *u, uint32_t pos)
{
    uint64_t phys = u->pages ? (uint64_t)u->pages[pos / u->block] * u->block + pos % u->block
                             : pos;
    return phys * u->kv_heads * u->head_dim + (uint64_t)u->kv_head * u->head_dim;
}

/* One (sequence, head) workgroup of 128 lanes.  out receives head_dim values. */
static void attn_decode_unit(const attn_unit *u, float *out)
{
    const uint32_t D = u->head_dim, sgw = u->sgw, nsg = ATTN_BLOCK / sgw;
    float scores[ATTN_BLOCK], red[ATTN_BLOCK];
    float o[ATTN_BLOCK];
    float m = -3.4e38f, l = 0;
    for (uint32_t i = 0; i < ATTN_BLOCK; i++) o[i] = 0;

    for (uint32_t base = 0; base < u->kv_len; base += ATTN_BLOCK) {
        /* scores: subgroup sg takes positions j = sg, sg + 4*nsg, ... and, per round, the four
         * positions j + r*nsg; lane sgl accumulates four chains over i = sgl, sgl+sgw, ... and
         * the subgroup sum folds lanes in order starting from lane 0's value
         * (internal/kernel/schedule.go:299-313). */
        for (uint32_t sg = 0; sg < nsg; sg++) {
            for (uint32_t j = sg; j < ATTN_BLOCK; j += 4 * nsg) {
                for (uint32_t r = 0; r < 4; r++) {
                    uint32_t jpos = base + j + r * nsg;
                    float dot = 0;
                    for (uint32_t sgl = 0; sgl < sgw; sgl++) {
                        float part = 0;
                        if (jpos < u->kv_len) {
                            uint64_t row = attn_row(u, jpos);
                            float pa = 0, pb = 0, pc = 0, pd = 0;
                            uint32_t i = sgl;
                            while (i + 3 * sgw < D) {
                                pa = pa + u->q[i] * cache_at(u, u->k, row + i);
                                pb = pb + u->q[i + sgw] * cache_at(u, u->k, row + i + sgw);
                                pc = pc + u->q[i + 2 * sgw] * cache_at(u, u->k, row + i + 2 * sgw);
                                pd = pd + u->q[i + 3 * sgw] * cache_at(u, u->k, row + i + 3 * sgw);
                                i = i + 4 * sgw;
                            }
                            while (i < D) {
                                pa = pa + u->q[i] * cache_at(u, u->k, row + i);
                                i = i + sgw;
                            }
                            part = (pa + pb) + (pc + pd);
                        }
                        if (sgl == 0) dot = part; else dot += part;
                    }
                    float sj = -3.4e38f;
                    if (jpos < u->kv_len) sj = dot * u->scale;
                    scores[j + r * nsg] = sj;
                }
            }
        }
        /* block maximum: subgroup fold over consecutive lanes, then a fold of the partials */
        for (uint32_t sg = 0; sg < nsg; sg++) {
            float acc = scores[sg * sgw];
            for (uint32_t t = 1; t < sgw; t++) acc = k_max(acc, scores[sg * sgw + t]);
            red[sg] = acc;
        }
        float block_max = red[0];
        for (uint32_t g = 1; g < nsg; g++) block_max = k_max(block_max, red[g]);

        float next = k_max(m, block_max);
        float alpha = k_exp(m - next);

        float e[ATTN_BLOCK];
        for (uint32_t lane = 0; lane < ATTN_BLOCK; lane++) {
            e[lane] = 0;
            if (base + lane < u->kv_len) e[lane] = k_exp(scores[lane] - next);
        }
        for (uint32_t sg = 0; sg < nsg; sg++) {
            float acc = e[sg * sgw];
            for (uint32_t t = 1; t < sgw; t++) acc += e[sg * sgw + t];
            red[sg] = acc;
        }
        for (uint32_t lane = 0; lane < ATTN_BLOCK; lane++) scores[lane] = e[lane];
        float block_sum = red[0];
        for (uint32_t g = 1; g < nsg; g++) block_sum = block_sum + red[g];
        l = alpha * l + block_sum;
        m = next;

        /* weighted sum of V: lane per output element, four accumulators by j % 4 */
        for (uint32_t lane = 0; lane < D && lane < ATTN_BLOCK; lane++) {
            float ol = alpha * o[lane];
            float o0 = 0, o1 = 0, o2 = 0, o3 = 0;
            for (uint32_t j = 0; j < ATTN_BLOCK; j += 4) {
                uint32_t jj;
                jj = base + j + 0;
                if (jj < u->kv_len) o0 = o0 + scores[j + 0] * cache_at(u, u->v, attn_row(u, jj) + lane);
                jj = base + j + 1;
                if (jj < u->kv_len) o1 = o1 + scores[j + 1] * cache_at(u, u->v, attn_row(u, jj) + lane);
                jj = base + j + 2;
                if (jj < u->kv_len) o2 = o2 + scores[j + 2] * cache_at(u, u->v, attn_row(u, jj) + lane);
                jj = base + j + 3;
                if (jj < u->kv_len) o3 = o3 + scores[j + 3] * cache_at(u, u->v, attn_row(u, jj) + lane);
            }
            o[lane] = ol + ((o0 + o1) + (o2 + o3));
        }
    }
    for (uint32_t lane = 0; lane < D && lane < ATTN_BLOCK; lane++) out[lane] = o[lane] / l;
}

/* AttentionDecode / AttentionDecodeF16 (contiguous cache), internal/kernels/attention.go:97,422.
 * cache_elems is len(k): the capacity is len(k) / (kvHeads*headDim). */
ORC_API void orc_attention_decode(uint32_t q_heads, uint32_t kv_heads, uint32_t head_dim,
                                  float scale, const float *q, const void *k, const void *v,
                                  int cache_f16, uint64_t cache_elems, const uint32_t *lengths,
                                  float *out, uint32_t sgw)
{
    uint32_t capacity = (uint32_t)(cache_elems / ((uint64_t)kv_heads * head_dim));
    uint32_t kv_len = lengths[0];
    if (kv_len > capacity) kv_len = capacity;
#pragma omp parallel for schedule(dynamic, 1)
    for (uint32_t h = 0; h < q_heads; h++) {
        attn_unit u = { q + (size_t)h * head_dim, k, v, cache_f16, NULL, 1, kv_heads, head_dim,
                        h / (q_heads / kv_heads), kv_len, scale, sgw };
        attn_decode_unit(&u, out + (size_t)h * head_dim);
    }
}

/* AttentionDecodePaged / ...F16, internal/kernels/paged.go:47,362.  n_pages is len(pages). */
ORC_API void orc_attention_decode_paged(uint32_t q_heads, uint32_t kv_heads, uint32_t head_dim,
                                        uint32_t block, float scale, const float *q,
                                        const void *k, const void *v, int cache_f16,
                                        const uint32_t *pages, uint32_t n_pages,
                                        const uint32_t *lengths, float *out, uint32_t sgw)
{
    uint32_t capacity = n_pages * block;
    uint32_t kv_len = lengths[0];
    if (kv_len > capacity) kv_len = capacity;
#pragma omp parallel for schedule(dynamic, 1)
    for (uint32_t h = 0; h < q_heads; h++) {
        attn_unit u = { q + (size_t)h * head_dim, k, v, cache_f16, pages, block, kv_heads,
                        head_dim, h / (q_heads / kv_heads), kv_len, scale, sgw };
        attn_decode_unit(&u, out + (size_t)h * head_dim);
    }
}

/* AttentionDecodeBatched, internal/kernels/batched.go:53-350.  The reference registers this
 * kernel for an f32 cache only (tensor/attention.go:383-387); cache_f16 = 1 widens K/V on load
 * the way the paged F16 kernel does and has no reference counterpart. */
ORC_API void orc_attention_decode_batched(uint32_t batch, uint32_t q_heads, uint32_t kv_heads,
                                          uint32_t head_dim, uint32_t block, uint32_t max_pages,
                                          float scale, const float *q, const void *k,
                                          const void *v, int cache_f16, const uint32_t *pages,
                                          const uint32_t *lengths, float *out, uint32_t sgw)
{
    uint32_t capacity = max_pages * block;
    int64_t groups = (int64_t)batch * q_heads;
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t gidx = 0; gidx < groups; gidx++) {
        uint32_t seq = (uint32_t)(gidx / q_heads), h = (uint32_t)(gidx % q_heads);
        uint32_t kv_len = lengths[seq];
        if (kv_len > capacity) kv_len = capacity;
        size_t qbase = ((size_t)seq * q_heads + h) * head_dim;
        attn_unit u = { q + qbase, k, v, cache_f16, pages + (size_t)seq * max_pages, block,
                        kv_heads, head_dim, h / (q_heads / kv_heads), kv_len, scale, sgw };
        attn_decode_unit(&u, out + qbase);
    }
}

/* One query row of a causal attention over a paged (or contiguous) cache: the body shared by
 * AttentionRagged (internal/kernels/ragged.go:61-241) and AttentionPrefill / AttentionPrefillPaged
 * (internal/kernels/prefill.go:409-560).  Positions pos <= limit and pos < kv_len are visible; the
 * loop walks blocks of 128 up to `bound`.  Lane-per-position sequential dot products, binary-tree
 * block maximum and sum over 128 lanes, sequential weighted sum of V per output element. */
static void attn_causal_unit(const attn_unit *up, uint32_t limit, uint32_t bound, float *o_out)
{
    const attn_unit u = *up;
    const float *qr = u.q;
    const void *k = u.k, *v = u.v;
    const uint32_t D = u.head_dim, kv_len = u.kv_len;
    const float scale = u.scale;
    float m = -3.4e38f, l = 0;
    float o[ATTN_BLOCK], scores[ATTN_BLOCK], red[ATTN_BLOCK];
    for (uint32_t t = 0; t < ATTN_BLOCK; t++) o[t] = 0;

    for (uint32_t base = 0; base < bound; base += ATTN_BLOCK) {
        for (uint32_t lane = 0; lane < ATTN_BLOCK; lane++) {
            uint32_t pos = base + lane;
            float score = -3.4e38f;
            if (pos <= limit && pos < kv_len) {
                uint64_t row = attn_row(&u, pos);
                float dot = 0;
                for (uint32_t j = 0; j < D; j++) dot = dot + qr[j] * cache_at(&u, k, row + j);
                score = dot * scale;
            }
            scores[lane] = score;
            red[lane] = score;
        }
        for (uint32_t stride = ATTN_BLOCK / 2; stride > 0; stride /= 2)
            for (uint32_t lane = 0; lane < stride; lane++)
                red[lane] = k_max(red[lane], red[lane + stride]);
        float block_max = red[0];
        float next = k_max(m, block_max);
        float alpha = k_exp(m - next);
        for (uint32_t lane = 0; lane < ATTN_BLOCK; lane++) {
            uint32_t pos = base + lane;
            float e = 0;
            if (pos <= limit && pos < kv_len) e = k_exp(scores[lane] - next);
            scores[lane] = e;
            red[lane] = e;
        }
        for (uint32_t stride = ATTN_BLOCK / 2; stride > 0; stride /= 2)
            for (uint32_t lane = 0; lane < stride; lane++)
                red[lane] = red[lane] + red[lane + stride];
        l = alpha * l + red[0];
        m = next;
        for (uint32_t lane = 0; lane < D && lane < ATTN_BLOCK; lane++) {
            float ol = alpha * o[lane];
            for (uint32_t j = 0; j < ATTN_BLOCK; j++) {
                if (base + j <= limit && base + j < kv_len)
                    ol = ol + scores[j] * cache_at(&u, v, attn_row(&u, base + j) + lane);
            }
            o[lane] = ol;
        }
    }
    for (uint32_t lane = 0; lane < D && lane < ATTN_BLOCK; lane++) o_out[lane] = o[lane] / l;
}

/* AttentionRagged / AttentionRaggedF16, internal/kernels/ragged.go:61-241, raggedf16.go:43. */
ORC_API void orc_attention_ragged(uint32_t tokens, uint32_t batch, uint32_t q_heads,
                                  uint32_t kv_heads, uint32_t head_dim, uint32_t block,
                                  uint32_t max_pages, float scale, const float *q, const void *k,
                                  const void *v, int cache_f16, const uint32_t *pages,
                                  const uint32_t *lengths, const uint32_t *offsets, float *out)
{
    int64_t groups = (int64_t)tokens * q_heads;
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t gidx = 0; gidx < groups; gidx++) {
        uint32_t tok = (uint32_t)(gidx / q_heads), h = (uint32_t)(gidx % q_heads);
        uint32_t kv_head = h / (q_heads / kv_heads);
        size_t qbase = ((size_t)tok * q_heads + h) * head_dim;
        const float *qr = q + qbase;
        float *o_out = out + qbase;
        uint32_t D = head_dim;

        uint32_t seq = 0;
        for (uint32_t r = 0; r < batch; r++)
            if (offsets[r + 1] <= tok) seq = seq + 1;
        if (seq >= batch) {                       /* padding token */
            for (uint32_t lane = 0; lane < D && lane < ATTN_BLOCK; lane++) o_out[lane] = 0;
            continue;
        }
        uint32_t i = tok - offsets[seq];
        uint32_t n = offsets[seq + 1] - offsets[seq];
        uint32_t kv_len = lengths[seq];
        if (kv_len + i < n) {                     /* token with no position */
            for (uint32_t lane = 0; lane < D && lane < ATTN_BLOCK; lane++) o_out[lane] = 0;
            continue;
        }
        uint32_t limit = kv_len + i - n;
        const uint32_t *prow = pages + (size_t)seq * max_pages;
        uint32_t capacity = max_pages * block;
        uint32_t bound = limit + 1;
        if (bound > capacity) bound = capacity;
        if (kv_len > capacity) kv_len = capacity;

        attn_unit u = { qr, k, v, cache_f16, prow, block, kv_heads, head_dim, kv_head, kv_len,
                        scale, 1 };
        attn_causal_unit(&u, limit, bound, o_out);
    }
}

/* AttentionPrefill / AttentionPrefillF16 (contiguous cache), internal/kernels/prefill.go:197-360:
 * q_seq query rows of ONE sequence, row s seeing positions <= base + s.  cache_elems = len(k). */
ORC_API void orc_attention_prefill(uint32_t q_heads, uint32_t kv_heads, uint32_t head_dim, uint32_t q_seq,
                                   uint32_t base, float scale, const float *q, const void *k,
                                   const void *v, int cache_f16, uint64_t cache_elems,
                                   const uint32_t *lengths, float *out)
{
    int64_t groups = (int64_t)q_seq * q_heads;
    uint32_t capacity = (uint32_t)(cache_elems / ((uint64_t)kv_heads * head_dim));
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t gidx = 0; gidx < groups; gidx++) {
        uint32_t s = (uint32_t)(gidx / q_heads), h = (uint32_t)(gidx % q_heads);
        size_t qbase = ((size_t)s * q_heads + h) * head_dim;
        uint32_t kv_len = lengths[0], limit = base + s, bound = limit + 1;
        if (bound > capacity) bound = capacity;
        if (kv_len > capacity) kv_len = capacity;
        attn_unit u = { q + qbase, k, v, cache_f16, NULL, 1, kv_heads, head_dim,
                        h / (q_heads / kv_heads), kv_len, scale, 1 };
        attn_causal_unit(&u, limit, bound, out + qbase);
    }
}

/* AttentionPrefillPaged / AttentionPrefillPagedF16, internal/kernels/prefill.go:409-560,
 * pagedprefillf16.go:31: the same over a page table; n_pages = len(pages). */
ORC_API void orc_attention_prefill_paged(uint32_t q_heads, uint32_t kv_heads, uint32_t head_dim,
                                         uint32_t q_seq, uint32_t base, uint32_t block, float scale,
                                         const float *q, const void *k, const void *v, int cache_f16,
                                         const uint32_t *pages, uint32_t n_pages,
                                         const uint32_t *lengths, float *out)
{
    int64_t groups = (int64_t)q_seq * q_heads;
    uint32_t capacity = n_pages * block;
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t gidx = 0; gidx < groups; gidx++) {
        uint32_t s = (uint32_t)(gidx / q_heads), h = (uint32_t)(gidx % q_heads);
        size_t qbase = ((size_t)s * q_heads + h) * head_dim;
        uint32_t kv_len = lengths[0], limit = base + s, bound = limit + 1;
        if (bound > capacity) bound = capacity;
        if (kv_len > capacity) kv_len = capacity;
        attn_unit u = { q + qbase, k, v, cache_f16, pages, block, kv_heads, head_dim,
                        h / (q_heads / kv_heads), kv_len, scale, 1 };
        attn_causal_unit(&u, limit, bound, out + qbase);
    }
}

/* The definition-level reference the reference's tests compare against: scores, softmax and the
 * weighted sum in binary64 with no blocks, tiles or lanes (internal/kernels/attention_test.go:
 * 29-70), here through a page table.  rows[] lists the physical position of each logical one. */
ORC_API void orc_attention_definition_f64(uint32_t q_heads, uint32_t kv_heads, uint32_t head_dim,
                                          double scale, const float *q, const void *k,
                                          const void *v, int cache_f16, const uint32_t *rows,
                                          uint32_t kv_len, double *out)
{
    uint32_t group = q_heads / kv_heads;
    for (uint32_t h = 0; h < q_heads; h++) {
        uint32_t kvh = h / group;
        double *sc = (double *)malloc(sizeof(double) * (kv_len ? kv_len : 1));
        double mx = -INFINITY;
        for (uint32_t j = 0; j < kv_len; j++) {
            uint64_t row = ((uint64_t)rows[j] * kv_heads + kvh) * head_dim;
            double acc = 0;
            for (uint32_t i = 0; i < head_dim; i++) {
                double kv = cache_f16 ? (double)orc_f16_to_f32(((const uint16_t *)k)[row + i])
                                      : (double)((const float *)k)[row + i];
                acc += (double)q[(size_t)h * head_dim + i] * kv;
            }
            sc[j] = acc * scale;
            if (sc[j] > mx) mx = sc[j];
        }
        double total = 0;
        for (uint32_t j = 0; j < kv_len; j++) { sc[j] = exp(sc[j] - mx); total += sc[j]; }
        for (uint32_t i = 0; i < head_dim; i++) {
            double acc = 0;
            for (uint32_t j = 0; j < kv_len; j++) {
                uint64_t row = ((uint64_t)rows[j] * kv_heads + kvh) * head_dim;
                double vv = cache_f16 ? (double)orc_f16_to_f32(((const uint16_t *)v)[row + i])
                                      : (double)((const float *)v)[row + i];
                acc += sc[j] * vv;
            }
            out[(size_t)h * head_dim + i] = acc / total;
        }
        free(sc);
    }
}

/* ------------------------------------------------------------------------------------------ */
/* Sampling policy on the device: internal/kernels/norm.go:80-137 (Softmax), rowsample.go:42-379 */
/* (the per-row forms), topk.go:59-256, penalty.go:60-141, sample.go:133-171 (the uniform forms). */
/* Workgroups of 128 lanes: lane l walks i = l, l + 128, ...; reductions are binary trees.         */
/* ------------------------------------------------------------------------------------------ */
#define ROW_WIDTH 128u
#define TOP_MAX_ROUNDS 128u   /* internal/kernels/topk.go:30 */

/* Softmax, internal/kernels/norm.go:94-137. */
ORC_API void orc_softmax(uint32_t rows, uint32_t width, const float *x, float *out)
{
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < (int64_t)rows; row++) {
        const float *xr = x + (size_t)row * width;
        float sh[ROW_WIDTH];
        for (uint32_t lid = 0; lid < ROW_WIDTH; lid++) {
            float m = xr[lid % width];
            for (uint32_t i = lid; i < width; i += ROW_WIDTH) m = k_max(m, xr[i]);
            sh[lid] = m;
        }
        for (uint32_t stride = ROW_WIDTH / 2; stride > 0; stride /= 2)
            for (uint32_t lid = 0; lid < stride; lid++) sh[lid] = k_max(sh[lid], sh[lid + stride]);
        float row_max = sh[0];
        for (uint32_t lid = 0; lid < ROW_WIDTH; lid++) {
            float acc = 0;
            for (uint32_t i = lid; i < width; i += ROW_WIDTH) acc = acc + k_exp(xr[i] - row_max);
            sh[lid] = acc;
        }
        for (uint32_t stride = ROW_WIDTH / 2; stride > 0; stride /= 2)
            for (uint32_t lid = 0; lid < stride; lid++) sh[lid] = sh[lid] + sh[lid + stride];
        float total = sh[0];
        for (uint32_t i = 0; i < width; i++) out[(size_t)row * width + i] = k_exp(xr[i] - row_max) / total;
    }
}

/* ScaleRows, rowsample.go:226-236: a factor of zero marks a greedy row and scales by one. */
ORC_API void orc_scale_rows(uint32_t rows, uint32_t vocab, const float *x, const float *factors, float *out)
{
    for (size_t i = 0; i < (size_t)rows * vocab; i++) {
        float f = factors[i / vocab];
        if (f == 0) f = 1;
        out[i] = x[i] * f;
    }
}

/* One extraction round of TopKMask / TopPMask: the largest entry strictly below the frontier in the
 * order (value descending, index ascending), by 128 strided lanes and a binary tree that breaks
 * value ties towards the lower index (topk.go:71-112). */
static void top_round(const float *w, uint32_t vocab, float front_v, uint32_t front_i, float *best_v,
                      uint32_t *best_i)
{
    float best[ROW_WIDTH];
    uint32_t at[ROW_WIDTH];
    for (uint32_t lane = 0; lane < ROW_WIDTH; lane++) {
        float v = -3.4e38f;
        uint32_t idx = vocab;
        for (uint32_t i = lane; i < vocab; i += ROW_WIDTH) {
            float x = w[i];
            int below = x < front_v;
            if (x == front_v && i > front_i) below = 1;
            if (below) {
                int better = x > v;
                if (x == v && i < idx) better = 1;
                if (better) { v = x; idx = i; }
            }
        }
        best[lane] = v;
        at[lane] = idx;
    }
    for (uint32_t stride = 64; stride > 0; stride /= 2)
        for (uint32_t lane = 0; lane < stride; lane++) {
            float a = best[lane], b = best[lane + stride];
            if (b > a) { best[lane] = b; at[lane] = at[lane + stride]; }
            else if (b == a && at[lane + stride] < at[lane]) at[lane] = at[lane + stride];
        }
    *best_v = best[0];
    *best_i = at[0];
}

static void top_keep(const float *w, uint32_t vocab, float front_v, uint32_t front_i, int keep_all, float *out)
{
    for (uint32_t i = 0; i < vocab; i++) {
        float x = w[i];
        int keep = x > front_v;
        if (x == front_v && i <= front_i) keep = 1;
        if (keep_all) keep = 1;
        out[i] = keep ? x : 0.0f;
    }
}

/* TopKMaskRows (rowsample.go:42-120) when ks != NULL: k per row, 0 or >= vocab passes the row
 * through; TopKMask (topk.go:59-130) when ks == NULL: the uniform k, no pass-through. */
ORC_API void orc_topk_mask(uint32_t rows, uint32_t vocab, const float *weights, const uint32_t *ks,
                           uint32_t uniform_k, float *out)
{
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t row = 0; row < (int64_t)rows; row++) {
        const float *w = weights + (size_t)row * vocab;
        uint32_t rounds = ks ? ks[row] : uniform_k;
        if (rounds > TOP_MAX_ROUNDS) rounds = TOP_MAX_ROUNDS;
        if (ks && rounds >= vocab) rounds = 0;
        float front_v = 3.4e38f;
        uint32_t front_i = 0;
        for (uint32_t r = 0; r < rounds; r++) top_round(w, vocab, front_v, front_i, &front_v, &front_i);
        top_keep(w, vocab, front_v, front_i, ks && rounds == 0, out + (size_t)row * vocab);
    }
}

/* TopPMaskRows (rowsample.go:126-220) when ps != NULL: p per row, outside (0, 1) passes the row
 * through; TopPMask (topk.go:153-256) when ps == NULL: the uniform p, always active. */
ORC_API void orc_topp_mask(uint32_t rows, uint32_t vocab, const float *weights, const float *ps,
                           float uniform_p, float *out)
{
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t row = 0; row < (int64_t)rows; row++) {
        const float *w = weights + (size_t)row * vocab;
        float p = ps ? ps[row] : uniform_p;
        int active = ps ? (p > 0 && p < 1) : 1;
        float part[ROW_WIDTH];
        for (uint32_t lane = 0; lane < ROW_WIDTH; lane++) {
            float sum = 0;
            for (uint32_t i = lane; i < vocab; i += ROW_WIDTH) sum = sum + w[i];
            part[lane] = sum;
        }
        for (uint32_t stride = 64; stride > 0; stride /= 2)
            for (uint32_t lane = 0; lane < stride; lane++) part[lane] = part[lane] + part[lane + stride];
        float target = part[0] * p;
        float front_v = 3.4e38f, kept = 0;
        uint32_t front_i = 0;
        for (uint32_t r = 0; r < TOP_MAX_ROUNDS; r++) {
            float bv;
            uint32_t bi;
            if (!(active && kept < target)) break;          /* later rounds change nothing */
            top_round(w, vocab, front_v, front_i, &bv, &bi);
            front_v = bv;
            front_i = bi;
            kept = kept + front_v;
        }
        top_keep(w, vocab, front_v, front_i, !active, out + (size_t)row * vocab);
    }
}

/* SampleRows (rowsample.go:246-300) when factors != NULL: the argmax of a row whose factor is zero,
 * a categorical walk otherwise; SampleCategorical (sample.go:133-171) when factors == NULL. */
ORC_API void orc_sample_rows(uint32_t rows, uint32_t vocab, const float *probs, const float *draws,
                             const float *factors, uint32_t *out)
{
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < (int64_t)rows; r++) {
        const float *p = probs + (size_t)r * vocab;
        if (factors && factors[r] == 0) {
            float v = -3.4e38f;
            uint32_t idx = 0;
            for (uint32_t i = 0; i < vocab; i++) if (p[i] > v) { v = p[i]; idx = i; }
            out[r] = idx;
            continue;
        }
        float draw = draws[r];
        if (draw < 0.0f) draw = 0.0f;
        if (draw > 0.99999994f) draw = 0.99999994f;
        float total = 0;
        for (uint32_t i = 0; i < vocab; i++) total = total + p[i];
        float target = draw * total;
        float acc = 0;
        uint32_t chosen = vocab - 1;
        int found = 0;
        for (uint32_t i = 0; i < vocab; i++) {
            acc = acc + p[i];
            if (!found && acc > target) { chosen = i; found = 1; }
        }
        out[r] = chosen;
    }
}

/* LogitBias, rowsample.go:304-320. */
ORC_API void orc_logit_bias(uint32_t rows, uint32_t vocab, uint32_t slots, const float *logits,
                            const uint32_t *ids, const float *values, float *out)
{
    for (size_t i = 0; i < (size_t)rows * vocab; i++) {
        uint32_t row = (uint32_t)(i / vocab), id = (uint32_t)(i - (size_t)row * vocab);
        float x = logits[i];
        for (uint32_t s = 0; s < slots; s++)
            if (ids[(size_t)row * slots + s] == id) x = x + values[(size_t)row * slots + s];
        out[i] = x;
    }
}

/* PenaltyClearRows, PenaltyCountRows, PenaltyApplyRows (rowsample.go:325-379), which are
 * PenaltyClear / PenaltyCount / PenaltyApply (penalty.go:60-141) with a row axis: the counts are
 * rebuilt from the filled part of each row's history ring, then each counted token is penalised
 * once.  counts [rows][vocab] is written. */
ORC_API void orc_penalty_rows(uint32_t rows, uint32_t vocab, uint32_t history_cap, const float *logits,
                              const uint32_t *history, const uint32_t *filled, const float *repetition,
                              const float *presence, const float *frequency, uint32_t *counts, float *out)
{
    memset(counts, 0, (size_t)rows * vocab * sizeof(uint32_t));
    for (uint32_t row = 0; row < rows; row++)
        for (uint32_t j = 0; j < history_cap && j < filled[row]; j++) {
            uint32_t id = history[(size_t)row * history_cap + j];
            if (id < vocab) counts[(size_t)row * vocab + id] += 1;
        }
    for (size_t i = 0; i < (size_t)rows * vocab; i++) {
        uint32_t row = (uint32_t)(i / vocab);
        float l = logits[i];
        uint32_t c = counts[i];
        if (c == 0) { out[i] = l; continue; }
        float rep = repetition[row];
        if (rep != 0 && rep != 1) {
            if (l > 0) l = l / rep; else l = l * rep;
        }
        out[i] = l - presence[row] - frequency[row] * (float)c;
    }
}

/* ------------------------------------------------------------------------------------------ */
/* int8 weights: quant/quant.go:60-122 (Int8Quantize), :128-134 (Int8Dequantize); one f16 scale */
/* per block of 32 weights along the flat index, quants in [-127, 127].                         */
/* ------------------------------------------------------------------------------------------ */
ORC_API void orc_int8_quantize(const float *w, size_t n, int8_t *quants, uint16_t *scales)
{
    const size_t block = 32;                      /* Int8Block */
    size_t blocks = (n + block - 1) / block;
    for (size_t b = 0; b < blocks; b++) {
        size_t lo = b * block, hi = lo + block < n ? lo + block : n;
        float peak = 0;
        for (size_t i = lo; i < hi; i++) {
            float a = (float)fabs((double)w[i]);
            if (a > peak) peak = a;
        }
        for (size_t i = lo; i < hi; i++) quants[i] = 0;
        if (peak == 0) { scales[b] = orc_f32_to_f16(0.0f); continue; }
        float s = peak / 127.0f;                  /* Int8Max */
        scales[b] = orc_f32_to_f16(s);
        float s16 = orc_f16_to_f32(scales[b]);    /* quantize against the scale the kernel reads */
        if (s16 == 0) continue;                   /* the scale underflowed f16 */
        for (size_t i = lo; i < hi; i++) {
            double q = nearbyint((double)w[i] / (double)s16);      /* round half to even */
            if (q > 127) q = 127;
            if (q < -127) q = -127;
            quants[i] = (int8_t)q;
        }
    }
}

ORC_API void orc_int8_dequantize(const int8_t *quants, const uint16_t *scales, size_t n, float *out)
{
    for (size_t i = 0; i < n; i++) out[i] = (float)quants[i] * orc_f16_to_f32(scales[i / 32]);
}

/* QuantMatVecF32, internal/kernels/matvec.go:204-231 (workgroup 32x16): 16 phases of k per      */
/* column, each acc = acc + a[k] * (q * s), then the phases summed in order.                     */
ORC_API void orc_quant_matvec_f32(uint32_t N, uint32_t K, const float *a, const int8_t *bq,
                                  const uint16_t *bs, float *out)
{
    const uint32_t phases = 16;
#pragma omp parallel for schedule(static)
    for (uint32_t col = 0; col < N; col++) {
        float part[16];
        for (uint32_t ly = 0; ly < phases; ly++) {
            float acc = 0;
            for (uint32_t k = ly; k < K; k += phases) {
                uint64_t w = (uint64_t)k * N + col;
                float q = (float)bq[w];
                float s = orc_f16_to_f32(bs[w / 32]);
                acc = acc + a[k] * (q * s);
            }
            part[ly] = acc;
        }
        float sum = 0;
        for (uint32_t p = 0; p < phases; p++) sum = sum + part[p];
        out[col] = sum;
    }
}

/* QuantMatMulTiledF32, internal/kernels/quant.go:195-243: one accumulator per output element,   */
/* sequential in k, each weight dequantized (q * s, rounded to f32) before the product; the     */
/* zero padding of the tiles adds exact zeros and changes no bits.                              */
ORC_API void orc_quant_matmul_tiled_f32(uint32_t M, uint32_t N, uint32_t K, const float *a,
                                        const int8_t *bq, const uint16_t *bs, float *out)
{
#pragma omp parallel for schedule(static)
    for (uint32_t col = 0; col < N; col++) {
        for (uint32_t m = 0; m < M; m++) {
            const float *am = a + (size_t)m * K;
            float acc = 0;
            for (uint32_t k = 0; k < K; k++) {
                uint64_t w = (uint64_t)k * N + col;
                float wv = (float)bq[w] * orc_f16_to_f32(bs[w / 32]);
                acc = acc + am[k] * wv;
            }
            out[(size_t)m * N + col] = acc;
        }
    }
}

/* ------------------------------------------------------------------------------------------ */
/* Grouped (per-expert) products, internal/kernels/grouped.go:49-97, groupedtiled.go:77-134,    */
/* segment.go:40                                                                                */
/* ------------------------------------------------------------------------------------------ */
ORC_API void orc_segment_offsets(uint32_t rows, const uint32_t *counts, uint32_t *offsets)
{
    uint32_t sum = 0;
    for (uint32_t r = 0; r < rows; r++) { offsets[r] = sum; sum = sum + counts[r]; }
    offsets[rows] = sum;
}

/* One workgroup of 128 lanes per (token, column): strided partials, then a binary tree. */
ORC_API void orc_grouped_matvec(uint32_t tokens, uint32_t experts, uint32_t K, uint32_t N,
                                const float *x, const float *w, const uint32_t *offsets,
                                float *out)
{
    int64_t total = (int64_t)tokens * N;
#pragma omp parallel for schedule(static)
    for (int64_t gidx = 0; gidx < total; gidx++) {
        uint32_t tok = (uint32_t)(gidx / N), col = (uint32_t)(gidx % N);
        uint32_t e = 0;
        for (uint32_t r = 0; r < experts; r++)
            if (offsets[r + 1] <= tok) e = e + 1;
        if (e >= experts) { out[(size_t)tok * N + col] = 0; continue; }
        size_t wbase = (size_t)e * K * N;
        float sh[128];
        for (uint32_t lid = 0; lid < 128; lid++) {
            float acc = 0;
            for (uint32_t k = lid; k < K; k += 128)
                acc = acc + x[(size_t)tok * K + k] * w[wbase + (size_t)k * N + col];
            sh[lid] = acc;
        }
        for (uint32_t stride = 64; stride > 0; stride /= 2)
            for (uint32_t lid = 0; lid < stride; lid++) sh[lid] = sh[lid] + sh[lid + stride];
        out[(size_t)tok * N + col] = sh[0];
    }
}

/* One accumulator per output, sequential in k; rows past offsets[E] (or past `tokens`) are never
 * written. */
ORC_API void orc_grouped_matmul(uint32_t experts, uint32_t tokens, uint32_t K, uint32_t N,
                                const float *x, const float *w, const uint32_t *offsets,
                                float *out)
{
    for (uint32_t e = 0; e < experts; e++) {
        uint32_t first = offsets[e], last = offsets[e + 1];
        if (last > tokens) last = tokens;
        size_t wbase = (size_t)e * K * N;
        int64_t rows = last > first ? (int64_t)(last - first) : 0;
#pragma omp parallel for schedule(static)
        for (int64_t r = 0; r < rows; r++) {
            uint32_t row = first + (uint32_t)r;
            float *acc = (float *)calloc(N, sizeof(float));
            for (uint32_t k = 0; k < K; k++) {
                float xv = x[(size_t)row * K + k];
                const float *wr = w + wbase + (size_t)k * N;
                for (uint32_t n = 0; n < N; n++) acc[n] = acc[n] + xv * wr[n];
            }
            memcpy(out + (size_t)row * N, acc, (size_t)N * sizeof(float));
            free(acc);
        }
    }
}

/* ------------------------------------------------------------------------------------------ */
/* Support operators of a decode step                                                           */
/* ------------------------------------------------------------------------------------------ */
ORC_API void orc_scatter_rows(uint32_t rows, uint32_t width, uint32_t capacity, const void *src,
                              const uint32_t *ids, void *state, uint32_t elem_bytes)
{   /* internal/kernels/elementwise.go:182-233: a row whose id is out of range is dropped */
    for (uint32_t r = 0; r < rows; r++) {
        uint32_t id = ids[r];
        if (id < capacity)
            memcpy((char *)state + (size_t)id * width * elem_bytes,
                   (const char *)src + (size_t)r * width * elem_bytes, (size_t)width * elem_bytes);
    }
}

ORC_API void orc_gather_rows(uint32_t rows, uint32_t width, uint32_t capacity, const float *table,
                             const uint32_t *ids, float *out)
{   /* internal/kernels/elementwise.go:118-131: an id out of range gives a row of zeros */
    for (uint32_t r = 0; r < rows; r++) {
        uint32_t id = ids[r];
        for (uint32_t c = 0; c < width; c++)
            out[(size_t)r * width + c] = id < capacity ? table[(size_t)id * width + c] : 0.0f;
    }
}

ORC_API void orc_rmsnorm(uint32_t rows, uint32_t width, float eps, const float *x, const float *w,
                         float *out)
{   /* internal/kernels/norm.go:46: 128 strided partials, binary tree, RSqrt */
#pragma omp parallel for schedule(static)
    for (uint32_t row = 0; row < rows; row++) {
        size_t base = (size_t)row * width;
        float sh[128];
        for (uint32_t lid = 0; lid < 128; lid++) {
            float acc = 0;
            for (uint32_t i = lid; i < width; i += 128) { float v = x[base + i]; acc = acc + v * v; }
            sh[lid] = acc;
        }
        for (uint32_t stride = 64; stride > 0; stride /= 2)
            for (uint32_t lid = 0; lid < stride; lid++) sh[lid] = sh[lid] + sh[lid + stride];
        float mean = sh[0] / (float)width;
        float scale = k_rsqrt(mean + eps);
        for (uint32_t i = 0; i < width; i++) out[base + i] = x[base + i] * scale * w[i];
    }
}

ORC_API void orc_rope(uint32_t rows, uint32_t width, uint32_t rotary_dim, float base_freq,
                      const uint32_t *positions, float *inout)
{   /* internal/kernels/elementwise.go:267: interleaved pairs (2k, 2k+1), one position per row */
    uint32_t pairs = rotary_dim / 2;
    for (uint32_t r = 0; r < rows; r++) {
        for (uint32_t k = 0; k < pairs; k++) {
            float pos = (float)positions[r];
            float exponent = -2.0f * (float)k / (float)rotary_dim;
            float freq = k_exp(exponent * k_log(base_freq));
            float theta = pos * freq;
            float c = k_cos(theta), s = k_sin(theta);
            size_t lo = (size_t)r * width + 2 * k, hi = lo + 1;
            float x = inout[lo], y = inout[hi];
            inout[lo] = x * c - y * s;
            inout[hi] = x * s + y * c;
        }
    }
}

ORC_API void orc_swiglu(const float *a, const float *b, float *out, size_t n)
{   /* internal/kernels/elementwise.go:85 */
    for (size_t i = 0; i < n; i++) {
        float x = a[i];
        out[i] = x / (1.0f + k_exp(-x)) * b[i];
    }
}

ORC_API void orc_elem_add(const float *a, const float *b, float *out, size_t n)
{   /* internal/kernels/elementwise.go:22 */
    for (size_t i = 0; i < n; i++) out[i] = a[i] + b[i];
}

ORC_API void orc_sample_argmax(uint32_t rows, uint32_t vocab, const float *logits, uint32_t *out)
{   /* internal/kernels/sample.go:50-100: 128 strided lanes, tree, ties to the lowest index */
    for (uint32_t r = 0; r < rows; r++) {
        size_t base = (size_t)r * vocab;
        float best[128];
        uint32_t at[128];
        for (uint32_t lane = 0; lane < 128; lane++) {
            float v = -3.4e38f;
            uint32_t idx = 0;
            for (uint32_t i = lane; i < vocab; i += 128) {
                float x = logits[base + i];
                if (x > v) { v = x; idx = i; }
            }
            best[lane] = v;
            at[lane] = idx;
        }
        for (uint32_t stride = 64; stride > 0; stride /= 2) {
            for (uint32_t lane = 0; lane < stride; lane++) {
                float a = best[lane], b = best[lane + stride];
                if (b > a) { best[lane] = b; at[lane] = at[lane + stride]; }
                else if (b == a && at[lane + stride] < at[lane]) at[lane] = at[lane + stride];
            }
        }
        out[r] = at[0];
    }
}

/* ------------------------------------------------------------------------------------------ */
/* Block pool, tensor/blockpool.go:55-133                                                       */
/* ------------------------------------------------------------------------------------------ */
typedef struct { uint32_t block; uint32_t *free_list; uint32_t n_free; uint32_t cap; } orc_pool;

ORC_API orc_pool *orc_blockpool_new(int blocks, int positions_per_block)
{
    if (blocks <= 0 || positions_per_block <= 0) return NULL;
    orc_pool *p = (orc_pool *)malloc(sizeof(orc_pool));
    p->block = (uint32_t)positions_per_block;
    p->cap = (uint32_t)blocks;
    p->n_free = (uint32_t)blocks;
    p->free_list = (uint32_t *)malloc(sizeof(uint32_t) * (size_t)blocks);
    for (int i = 0; i < blocks; i++) p->free_list[i] = (uint32_t)(blocks - 1 - i);
    return p;
}

ORC_API void orc_blockpool_free_pool(orc_pool *p) { if (p) { free(p->free_list); free(p); } }
ORC_API int orc_blockpool_available(const orc_pool *p) { return (int)p->n_free; }
ORC_API int orc_blockpool_block_size(const orc_pool *p) { return (int)p->block; }

/* Grows `pages` (n_pages entries, capacity >= the returned count) so that it addresses n
 * positions.  Returns the new page count, -1 for a negative n, -2 when the pool would have to
 * evict.  The new pages are the LAST `need` entries of the free list, in list order. */
ORC_API int orc_blockpool_grow(orc_pool *p, uint32_t *pages, int n_pages, int n)
{
    if (n < 0) return -1;
    int want = (int)(((int64_t)n + p->block - 1) / p->block);
    if (want <= n_pages) return n_pages;
    int need = want - n_pages;
    if ((uint32_t)need > p->n_free) return -2;
    for (int i = 0; i < need; i++) pages[n_pages + i] = p->free_list[p->n_free - (uint32_t)need + (uint32_t)i];
    p->n_free -= (uint32_t)need;
    return want;
}

/* Returns how many of the pages were refused because they were already free. */
ORC_API int orc_blockpool_free(orc_pool *p, const uint32_t *pages, int n_pages)
{
    int errs = 0;
    uint8_t *held = (uint8_t *)calloc(p->cap, 1);
    for (uint32_t i = 0; i < p->n_free; i++) held[p->free_list[i]] = 1;
    for (int i = 0; i < n_pages; i++) {
        uint32_t pg = pages[i];
        if (pg >= p->cap || held[pg]) { errs++; continue; }
        held[pg] = 1;
        p->free_list[p->n_free++] = pg;
    }
    free(held);
    return errs;
}

/* ------------------------------------------------------------------------------------------ */
/* Definition-level binary64 product over dequantized weights, as the reference's int4 tests    */
/* build beside themselves (internal/kernels/int4_test.go:121-134): want and the magnitude sum. */
/* ------------------------------------------------------------------------------------------ */
ORC_API void orc_matmul_definition_f64(uint32_t M, uint32_t N, uint32_t K, const float *a,
                                       const float *w_dequant, double *want, double *mag)
{
#pragma omp parallel for schedule(static)
    for (uint32_t n = 0; n < N; n++) {
        for (uint32_t m = 0; m < M; m++) {
            double acc = 0, mg = 0;
            for (uint32_t k = 0; k < K; k++) {
                double t = (double)a[(size_t)m * K + k] * (double)w_dequant[(size_t)k * N + n];
                acc += t;
                mg += fabs(t);
            }
            want[(size_t)m * N + n] = acc;
            if (mag) mag[(size_t)m * N + n] = mg;
        }
    }
}
