// Grouped (per-expert) products over expert-sorted rows: GroupedMatVec (internal/kernels/
// grouped.go:49), GroupedMatMul (groupedtiled.go:77), SegmentOffsets (segment.go:40), and an int4
// form with no reference kernel (each expert's [K,N] matrix quantized on its own).
//
//   out[t][n] = sum_k x[t][k] * w[e(t)][k][n],   rows of expert e are offsets[e] .. offsets[e+1]
//
// The reference's tiled kernel gives one workgroup an (expert, 16-column) strip and walks the
// expert's rows eight at a time, so an expert's matrix is re-read once per eight rows.  Here a CTA
// owns a 128x128 output tile of one expert's segment and steps K by 16 through shared memory with
// an 8x8 register tile per thread, so a matrix is read once per 128 rows.
//
// Edge semantics kept: `last` is clamped to Tokens; an empty expert does nothing; GroupedMatMul
// never writes a row past offsets[E]; GroupedMatVec writes zeros there.
#include <cstdlib>

#include "common.cuh"

namespace ab {

static constexpr int BM = 128, BN = 128, BK = 16, GT = 256;
static constexpr uint32_t kGroup = 128;

struct GroupedParams {
    const float *x;
    const float *w;             // f32 weights, or NULL for int4
    const uint32_t *bq;
    const __half *bs, *bz;
    const uint32_t *offsets;
    float *out;
    uint32_t experts, tokens, K, N;
    uint64_t words_per_expert, groups_per_expert;
    const float *amax;          // int4 tensor-core form: the rows' largest magnitudes (NULL: none)
};

__device__ __forceinline__ bool find_tile(const GroupedParams &p, uint32_t t, uint32_t &e,
                                          uint32_t &row0, uint32_t &last)
{
    if (!p.offsets) {                        // one matrix, no segments: rows 0 .. tokens
        e = 0;
        last = p.tokens;
        row0 = t * BM;
        return row0 < last;
    }
    for (e = 0; e < p.experts; e++) {
        uint32_t first = p.offsets[e];
        last = min(p.offsets[e + 1], p.tokens);
        uint32_t nt = last > first ? (last - first + BM - 1) / BM : 0;
        if (t < nt) { row0 = first + t * BM; return true; }
        t -= nt;
    }
    return false;
}

// grid = (ceil(N/128), row tiles upper bound).  Requires K % 16 == 0 and N % 4 == 0 (f32) or
// N % 128 == 0 (int4).
template <bool INT4>
__global__ void __launch_bounds__(GT) grouped_tile_kernel(const GroupedParams p)
{
    __shared__ __align__(16) float As[BK][BM];
    __shared__ __align__(16) float Bs[BK][BN];
    uint32_t e, row0, last;
    if (!find_tile(p, blockIdx.y, e, row0, last)) return;
    const uint32_t col0 = blockIdx.x * BN;
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[i][j] = 0.f;

    const uint32_t a_row = row0 + (tid >> 1);
    const int a_k = (tid & 1) * 8;
    const int b_k = tid >> 4;
    const uint32_t b_col = col0 + (tid & 15) * 8;
    const float *wbase = INT4 ? nullptr : p.w + (size_t)e * p.K * p.N;

    for (uint32_t k0 = 0; k0 < p.K; k0 += BK) {
        float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
        if (a_row < last) {
            const float *src = p.x + (size_t)a_row * p.K + k0 + a_k;
            a0 = *reinterpret_cast<const float4 *>(src);
            a1 = *reinterpret_cast<const float4 *>(src + 4);
        }
        float bv[8];
#pragma unroll
        for (int j = 0; j < 8; j++) bv[j] = 0.f;
        if (b_col < p.N) {
            if (INT4) {
                size_t wi = (size_t)(k0 + b_k) * p.N + b_col;          // flat weight index
                uint32_t word = p.bq[e * p.words_per_expert + wi / 8];
                size_t g = e * p.groups_per_expert + wi / kGroup;
                float s = __half2float(p.bs[g]), z = __half2float(p.bz[g]);
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    float code = (float)((word >> (4 * j)) & 0xFu);
                    bv[j] = s == 0.f ? z : (code - z) * s;
                }
            } else {
                const float *src = wbase + (size_t)(k0 + b_k) * p.N + b_col;
                float4 b0 = *reinterpret_cast<const float4 *>(src);
                bv[0] = b0.x; bv[1] = b0.y; bv[2] = b0.z; bv[3] = b0.w;
                if (b_col + 4 < p.N) {
                    float4 b1 = *reinterpret_cast<const float4 *>(src + 4);
                    bv[4] = b1.x; bv[5] = b1.y; bv[6] = b1.z; bv[7] = b1.w;
                }
            }
        }
        __syncthreads();
        const int ar = tid >> 1;
        As[a_k + 0][ar] = a0.x; As[a_k + 1][ar] = a0.y; As[a_k + 2][ar] = a0.z; As[a_k + 3][ar] = a0.w;
        As[a_k + 4][ar] = a1.x; As[a_k + 5][ar] = a1.y; As[a_k + 6][ar] = a1.z; As[a_k + 7][ar] = a1.w;
        *reinterpret_cast<float4 *>(&Bs[b_k][(tid & 15) * 8]) = make_float4(bv[0], bv[1], bv[2], bv[3]);
        *reinterpret_cast<float4 *>(&Bs[b_k][(tid & 15) * 8 + 4]) = make_float4(bv[4], bv[5], bv[6], bv[7]);
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; k++) {
            float4 ra0 = *reinterpret_cast<const float4 *>(&As[k][ty * 4]);
            float4 ra1 = *reinterpret_cast<const float4 *>(&As[k][64 + ty * 4]);
            float4 rb0 = *reinterpret_cast<const float4 *>(&Bs[k][tx * 4]);
            float4 rb1 = *reinterpret_cast<const float4 *>(&Bs[k][64 + tx * 4]);
            float ra[8] = {ra0.x, ra0.y, ra0.z, ra0.w, ra1.x, ra1.y, ra1.z, ra1.w};
            float rb[8] = {rb0.x, rb0.y, rb0.z, rb0.w, rb1.x, rb1.y, rb1.z, rb1.w};
#pragma unroll
            for (int i = 0; i < 8; i++)
#pragma unroll
                for (int j = 0; j < 8; j++) acc[i][j] = fmaf(ra[i], rb[j], acc[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < 8; i++) {
        uint32_t row = row0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + i - 4);
        if (row >= last) continue;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            uint32_t col = col0 + h * 64 + tx * 4;
            if (col < p.N)      // N % 4 == 0, so a float4 is inside or outside as a whole
                *reinterpret_cast<float4 *>(p.out + (size_t)row * p.N + col) =
                    make_float4(acc[i][h * 4], acc[i][h * 4 + 1], acc[i][h * 4 + 2], acc[i][h * 4 + 3]);
        }
    }
}

// Any shape: one thread per output element.
template <bool INT4>
__global__ void grouped_generic_kernel(const GroupedParams p, uint32_t rows)
{
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)rows * p.N) return;
    uint32_t tok = (uint32_t)(i / p.N), n = (uint32_t)(i % p.N);
    uint32_t e = 0;
    for (uint32_t r = 0; r < p.experts; r++) e += (p.offsets[r + 1] <= tok) ? 1u : 0u;
    if (e >= p.experts) return;
    if (tok >= min(p.offsets[e + 1], p.tokens)) return;
    float acc = 0.f;
    for (uint32_t k = 0; k < p.K; k++) {
        float wv;
        if (INT4) {
            size_t wi = (size_t)k * p.N + n;
            uint32_t code = (p.bq[e * p.words_per_expert + wi / 8] >> (4 * (wi % 8))) & 0xFu;
            size_t g = e * p.groups_per_expert + wi / kGroup;
            float s = __half2float(p.bs[g]), z = __half2float(p.bz[g]);
            wv = s == 0.f ? z : ((float)code - z) * s;
        } else {
            wv = p.w[((size_t)e * p.K + k) * p.N + n];
        }
        acc = fmaf(p.x[(size_t)tok * p.K + k], wv, acc);
    }
    p.out[i] = acc;
}

// GroupedMatVec's rule for a row that belongs to no expert: zeros (grouped.go:72-77).
__global__ void grouped_zero_tail_kernel(float *out, const uint32_t *offsets, uint32_t experts,
                                         uint32_t rows, uint32_t N)
{
    size_t start = (size_t)min(offsets[experts], rows) * N, end = (size_t)rows * N;
    for (size_t i = start + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < end;
         i += (size_t)gridDim.x * blockDim.x)
        out[i] = 0.f;
}

// ---- int4 experts on the tensor cores ------------------------------------------------------------
// The same arithmetic as the decode-batch int4 kernel (int4_batch.cu), tiled for hundreds of rows
// per expert: a CTA owns 128 rows of one expert x one 128-column quantisation group, so the scale
// and zero of a weight depend on k only and
//   out[m][n] = sum_k (x[m][k] s[k]) code[k][n] - sum_k (x[m][k] s[k]) z[k]
// with x*s rounded to f16 once (the only rounded operand), the 4-bit code masked in place into an
// f16 subnormal (exact; undone per column at the end) and the second sum one more MMA per k step
// with z as its B operand.  A row whose group has scale 0 is the constant z
// (internal/kernels/int4.go:85-87): its x*s is 0 and x*z is added from an f32 side sum.
// Eight warps: warp (r, c) holds rows 32r .. 32r+31 x columns 64c .. 64c+63 (two m16 tiles x eight
// n8 tiles, 64 accumulators per thread).  K advances in chunks of 64: the chunk's x*s goes through
// shared memory (f16, row stride padded against bank conflicts), the codes go from global memory
// straight to registers, one chunk ahead.
static constexpr int kGmThreads = 256, kGmRows = 128, kGmChunk = 64;
static constexpr int kGmStride = kGmChunk * 2 + 32;       // bytes per row of x*s in shared memory (32 mod 128: fragment loads spread over the banks)

__device__ __forceinline__ void gm_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
                 "{%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// grid = (N / 128, row tiles upper bound); K % 64 == 0, N % 128 == 0
__global__ void __launch_bounds__(kGmThreads) grouped_int4_mma_kernel(const GroupedParams p)
{
    __shared__ __align__(16) unsigned char s_a[kGmRows * kGmStride];      // x*s, f16 [128][64]
    __shared__ __align__(8) __half s_s[kGmChunk], s_z[kGmChunk];           // the chunk's scales and zeros
    uint32_t e, row0, last;
    if (!find_tile(p, blockIdx.y, e, row0, last)) return;
    const uint32_t g = blockIdx.x, gpr = p.N / kGroup;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, t = lane & 3;
    const int wr = warp >> 1, wc = warp & 1;
    const __half *bs = p.bs + e * p.groups_per_expert + g, *bz = p.bz + e * p.groups_per_expert + g;
    // this lane's codes: rows 4t .. 4t+3 of every 16-row step, the 8 columns 64 wc + 8 gid .. +7
    const uint32_t *code = p.bq + e * p.words_per_expert + (size_t)(4 * t) * (p.N / 8) + g * 16 + wc * 8 + gid;
    const size_t row_words = p.N / 8;
    // staging of x: pass i covers rows 16 i .. 16 i + 15; thread = (row tid / 16 of the pass, the four
    // k values 4 (tid % 16) ..): a half-warp reads 256 contiguous bytes of a row and its shared
    // stores fall on distinct banks
    const int srow = tid >> 4, skq = tid & 15;
    // every staged row times an exact power of two that puts its largest activation in [2^8, 2^9):
    // x * s stays a normal f16 whatever the activations' magnitude; undone where the sums are stored
    float xscale[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const uint32_t row = row0 + 16 * i + srow;
        xscale[i] = (p.amax && row < last) ? ab_pow2(8 - ab_row_exponent(__float_as_uint(fabsf(__ldg(p.amax + row))))) : 1.f;
    }

    float acc[2][8][4], accz[2][4];
#pragma unroll
    for (int mt = 0; mt < 2; mt++) {
#pragma unroll
        for (int j = 0; j < 8; j++) acc[mt][j][0] = acc[mt][j][1] = acc[mt][j][2] = acc[mt][j][3] = 0.f;
        accz[mt][0] = accz[mt][1] = accz[mt][2] = accz[mt][3] = 0.f;
    }
    float csum[8];
#pragma unroll
    for (int i = 0; i < 8; i++) csum[i] = 0.f;
    bool any_const = false;

    // codes of a chunk: [k16 step][row 4t + i]; two register sets used in turn, so that a chunk's
    // loads are in flight while the other chunk is multiplied
    const uint32_t *cp = code;
    const size_t chunk_words = (size_t)kGmChunk * row_words;
    auto fetch_codes = [&](uint32_t (&dst)[4][4], bool live) {
#pragma unroll
        for (int st = 0; st < 4; st++)
#pragma unroll
            for (int i = 0; i < 4; i++) dst[st][i] = live ? __ldg(cp + (size_t)(16 * st + i) * row_words) : 0u;
        cp += chunk_words;
    };
    auto stage = [&](uint32_t k0) {
        __syncthreads();                                   // the previous chunk's x*s is no longer read
        if (tid < kGmChunk) {
            s_s[tid] = __ldg(bs + (size_t)(k0 + tid) * gpr);
            s_z[tid] = __ldg(bz + (size_t)(k0 + tid) * gpr);
        }
        float4 xv[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t row = row0 + 16 * i + srow;
            xv[i] = row < last ? __ldg(reinterpret_cast<const float4 *>(p.x + (size_t)row * p.K + k0 + 4 * skq))
                               : make_float4(0.f, 0.f, 0.f, 0.f);
            xv[i].x *= xscale[i]; xv[i].y *= xscale[i]; xv[i].z *= xscale[i]; xv[i].w *= xscale[i];
        }
        __syncthreads();
        const uint2 s4 = *reinterpret_cast<const uint2 *>(s_s + 4 * skq);
        const float2 s01 = __half22float2(*reinterpret_cast<const __half2 *>(&s4.x));
        const float2 s23 = __half22float2(*reinterpret_cast<const __half2 *>(&s4.y));
        const bool cst = s01.x == 0.f || s01.y == 0.f || s23.x == 0.f || s23.y == 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const __half2 p01 = __floats2half2_rn(xv[i].x * s01.x, xv[i].y * s01.y);
            const __half2 p23 = __floats2half2_rn(xv[i].z * s23.x, xv[i].w * s23.y);
            uint2 pk;
            pk.x = *reinterpret_cast<const uint32_t *>(&p01);
            pk.y = *reinterpret_cast<const uint32_t *>(&p23);
            *reinterpret_cast<uint2 *>(s_a + (16 * i + srow) * kGmStride + 8 * skq) = pk;
        }
        if (cst) {
            any_const = true;
            const float z0 = __half2float(s_z[4 * skq]), z1 = __half2float(s_z[4 * skq + 1]);
            const float z2 = __half2float(s_z[4 * skq + 2]), z3 = __half2float(s_z[4 * skq + 3]);
#pragma unroll
            for (int i = 0; i < 8; i++) {
                if (s01.x == 0.f) csum[i] = fmaf(xv[i].x, z0, csum[i]);
                if (s01.y == 0.f) csum[i] = fmaf(xv[i].y, z1, csum[i]);
                if (s23.x == 0.f) csum[i] = fmaf(xv[i].z, z2, csum[i]);
                if (s23.y == 0.f) csum[i] = fmaf(xv[i].w, z3, csum[i]);
            }
        }
        __syncthreads();
    };
    const unsigned char *a_base = s_a + (32 * wr + gid) * kGmStride + 8 * t;
    auto multiply = [&](const uint32_t (&cur)[4][4]) {
#pragma unroll
        for (int st = 0; st < 4; st++) {
            // a 16-row step: rows {4t, 4t+1} stand for the MMA's k slots {2t, 2t+1}, {4t+2, 4t+3} for
            // {2t+8, 2t+9} (a free relabelling of k, applied to both operands)
            uint32_t af[2][4];
#pragma unroll
            for (int mt = 0; mt < 2; mt++) {
                const unsigned char *a_lo = a_base + 16 * mt * kGmStride + 32 * st;
                const uint2 lo = *reinterpret_cast<const uint2 *>(a_lo);
                const uint2 hi = *reinterpret_cast<const uint2 *>(a_lo + 8 * kGmStride);
                af[mt][0] = lo.x; af[mt][1] = hi.x; af[mt][2] = lo.y; af[mt][3] = hi.y;
            }
            const uint2 z4 = *reinterpret_cast<const uint2 *>(s_z + 16 * st + 4 * t);
            // a constant row's zero must not reach the MMA (its x*s is 0, but 0 * inf is NaN)
            const uint2 sz4 = *reinterpret_cast<const uint2 *>(s_s + 16 * st + 4 * t);
            uint32_t zb0 = z4.x, zb1 = z4.y;
            if ((sz4.x & 0x7fffu) == 0) zb0 &= 0xffff0000u;
            if ((sz4.x & 0x7fff0000u) == 0) zb0 &= 0x0000ffffu;
            if ((sz4.y & 0x7fffu) == 0) zb1 &= 0xffff0000u;
            if ((sz4.y & 0x7fff0000u) == 0) zb1 &= 0x0000ffffu;
            gm_mma(accz[0], af[0], zb0, zb1);
            gm_mma(accz[1], af[1], zb0, zb1);
            const uint32_t w0 = cur[st][0], w1 = cur[st][1], w2 = cur[st][2], w3 = cur[st][3];
            const uint32_t lo01 = __byte_perm(w0, w1, 0x5410), hi01 = __byte_perm(w0, w1, 0x7632);
            const uint32_t lo23 = __byte_perm(w2, w3, 0x5410), hi23 = __byte_perm(w2, w3, 0x7632);
            const uint32_t src01[4] = {lo01, lo01 >> 8, hi01, hi01 >> 8};
            const uint32_t src23[4] = {lo23, lo23 >> 8, hi23, hi23 >> 8};
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const uint32_t be0 = src01[q] & 0x000F000Fu, be1 = src23[q] & 0x000F000Fu;     // code 2q
                const uint32_t bo0 = src01[q] & 0x00F000F0u, bo1 = src23[q] & 0x00F000F0u;     // code 2q + 1
                gm_mma(acc[0][2 * q], af[0], be0, be1);
                gm_mma(acc[1][2 * q], af[1], be0, be1);
                gm_mma(acc[0][2 * q + 1], af[0], bo0, bo1);
                gm_mma(acc[1][2 * q + 1], af[1], bo0, bo1);
            }
        }
    };

    uint32_t cwa[4][4], cwb[4][4];
    fetch_codes(cwa, true);
    for (uint32_t k0 = 0; k0 < p.K; k0 += 2 * kGmChunk) {
        fetch_codes(cwb, k0 + kGmChunk < p.K);
        stage(k0);
        multiply(cwa);
        fetch_codes(cwa, k0 + 2 * kGmChunk < p.K);
        if (k0 + kGmChunk < p.K) {                         // uniform over the CTA
            stage(k0 + kGmChunk);
            multiply(cwb);
        }
    }
    // side sums over constant rows: sixteen staging threads per row, added in a fixed order
    const int has_const = __syncthreads_or(any_const);
    float *s_const = reinterpret_cast<float *>(s_a);       // [128][16], over x*s (no longer read)
    if (has_const) {
#pragma unroll
        for (int i = 0; i < 8; i++) s_const[(16 * i + srow) * 16 + skq] = csum[i];
        __syncthreads();
    }
    // MMA j's n slot n is column 8 n + j of the warp's 64: the thread holds columns 16 t .. 16 t + 15
    // (n = 2t: j = 0..7, n = 2t+1: j = 0..7) of rows gid and gid + 8 of each m tile
#pragma unroll
    for (int mt = 0; mt < 2; mt++)
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint32_t lr = 32 * wr + 16 * mt + gid + 8 * h, row = row0 + lr;
            if (row >= last) continue;
            float add = -accz[mt][2 * h];
            if (has_const) {
                float cs = 0.f;
#pragma unroll
                for (int q = 0; q < 16; q++) cs += s_const[lr * 16 + q];
                add += cs;
            }
            float *o = p.out + (size_t)row * p.N + (size_t)g * kGroup + 64 * wc + 16 * t;
            const float un = p.amax ? ab_pow2(ab_row_exponent(__float_as_uint(fabsf(__ldg(p.amax + row)))) - 8) : 1.f;
#pragma unroll
            for (int nn = 0; nn < 2; nn++)
#pragma unroll
                for (int j = 0; j < 8; j += 4) {
                    float4 v;
                    v.x = (acc[mt][j][2 * h + nn] * 16777216.f + add) * un;
                    v.y = (acc[mt][j + 1][2 * h + nn] * 1048576.f + add) * un;
                    v.z = (acc[mt][j + 2][2 * h + nn] * 16777216.f + add) * un;
                    v.w = (acc[mt][j + 3][2 * h + nn] * 1048576.f + add) * un;
                    *reinterpret_cast<float4 *>(o + 8 * nn + j) = v;
                }
        }
}

// The same kernel as a plain int4 product for large batches of activation rows (one "expert", no
// segment offsets): QuantMatMulInt4 from about a hundred rows, where 128-row tiles beat passes of
// 16 rows.  K % 64 == 0 and N % 128 == 0.
bool int4_tiles_ok(uint32_t N, uint32_t K) { return N % kGroup == 0 && K % kGmChunk == 0 && N > 0 && K > 0; }

size_t int4_tiles_workspace(uint32_t M) { return align_up((size_t)M * 4, 256); }     // the rows' largest magnitudes

int run_int4_tiles(const Launch &l, float *out, uint32_t M, uint32_t N, uint32_t K)
{
    GroupedParams p{};
    p.x = ptr<const float>(l, 0); p.bq = ptr<const uint32_t>(l, 1);
    p.bs = ptr<const __half>(l, 2); p.bz = ptr<const __half>(l, 3);
    p.offsets = nullptr; p.out = out;
    p.experts = 1; p.tokens = M; p.K = K; p.N = N;
    p.words_per_expert = ((uint64_t)K * N + 7) / 8;
    p.groups_per_expert = ((uint64_t)K * N + kGroup - 1) / kGroup;
    if (!l.ws || l.ws_bytes < int4_tiles_workspace(M))
        return fail(AB_ERR_INVALID, "QuantMatMulInt4 (tiles): needs %zu bytes of workspace, given %zu",
                    int4_tiles_workspace(M), l.ws_bytes);
    float *amax = static_cast<float *>(l.ws);
    int rc = run_row_absmax(l.stream, p.x, amax, M, K, false);
    if (rc) return rc;
    p.amax = amax;
    dim3 grid(N / kGroup, (M + kGmRows - 1) / kGmRows);
    grouped_int4_mma_kernel<<<grid, kGmThreads, 0, l.stream>>>(p); count_launch();
    return check_cuda(cudaGetLastError(), "QuantMatMulInt4 (tiles)");
}

static int run_grouped(Launch &l, GroupedParams &p, bool int4, bool zero_tail, uint32_t out_rows,
                       const char *name)
{
    bool fast = p.K % BK == 0 && (int4 ? p.N % kGroup == 0 : p.N % 4 == 0);
    static const bool simt_only = getenv("AB_GROUPED_SIMT") != nullptr;       // for measurements
    const bool mma = int4 && fast && p.K % kGmChunk == 0 && !simt_only;
    const size_t ws_need = mma ? align_up((size_t)p.tokens * 4, 256) : 0;     // the rows' largest magnitudes
    if (l.query_ws) { l.ws_need = ws_need; return AB_OK; }
    if (p.experts == 0 || p.K == 0 || p.N == 0)
        return fail(AB_ERR_INVALID, "%s: Experts=%u K=%u N=%u", name, p.experts, p.K, p.N);
    if (p.tokens == 0) return AB_OK;
    if (mma) {
        if (!l.ws || l.ws_bytes < ws_need)
            return fail(AB_ERR_INVALID, "%s: needs %zu bytes of workspace, given %zu", name, ws_need, l.ws_bytes);
        float *amax = static_cast<float *>(l.ws);
        int rc = run_row_absmax(l.stream, p.x, amax, p.tokens, p.K, false);
        if (rc) return rc;
        p.amax = amax;
        dim3 grid(p.N / kGroup, (p.tokens + kGmRows - 1) / kGmRows + p.experts);
        grouped_int4_mma_kernel<<<grid, kGmThreads, 0, l.stream>>>(p); count_launch();
    } else if (fast) {
        dim3 grid((p.N + BN - 1) / BN, (p.tokens + BM - 1) / BM + p.experts);
        if (int4) { grouped_tile_kernel<true><<<grid, GT, 0, l.stream>>>(p); count_launch(); }
        else { grouped_tile_kernel<false><<<grid, GT, 0, l.stream>>>(p); count_launch(); }
    } else {
        size_t total = (size_t)p.tokens * p.N;
        unsigned blocks = (unsigned)((total + 127) / 128);
        if (int4) { grouped_generic_kernel<true><<<blocks, 128, 0, l.stream>>>(p, p.tokens); count_launch(); }
        else { grouped_generic_kernel<false><<<blocks, 128, 0, l.stream>>>(p, p.tokens); count_launch(); }
    }
    if (zero_tail)
        grouped_zero_tail_kernel<<<64, 256, 0, l.stream>>>(p.out, p.offsets, p.experts, out_rows, p.N); count_launch();
    note_selection("%s: %s, %u experts over %u rows", name,
                   mma ? "128x128 tensor-core kernel (m16n8k16, f16 operands, f32 accumulate)"
                       : (fast ? "128x128 register-tiled kernel" : "generic kernel"), p.experts, p.tokens);
    return check_cuda(cudaGetLastError(), name);
}

int launch_grouped_matvec(Launch &l)
{   // x, w, offsets, out; GroupedDims{Experts,K,N}; one reference workgroup per (token, column)
    GroupedParams p{};
    p.experts = u32_at(l.u, 0); p.K = u32_at(l.u, 4); p.N = u32_at(l.u, 8);
    uint32_t rows = p.N ? l.len[3] / p.N : 0;          // tokens = len(out) / N
    p.tokens = rows;
    if (l.len[2] < p.experts + 1 || l.len[1] < (uint64_t)p.experts * p.K * p.N ||
        l.len[0] < (uint64_t)rows * p.K)
        return fail(AB_ERR_INVALID, "GroupedMatVec: Experts=%u K=%u N=%u rows=%u; lengths x[%u] "
                    "w[%u] offsets[%u]", p.experts, p.K, p.N, rows, l.len[0], l.len[1], l.len[2]);
    if (!l.query_ws) {
        p.x = ptr<const float>(l, 0); p.w = ptr<const float>(l, 1);
        p.offsets = ptr<const uint32_t>(l, 2); p.out = ptr<float>(l, 3);
    }
    return run_grouped(l, p, false, true, rows, "GroupedMatVec");
}

int launch_grouped_matmul(Launch &l)
{   // GroupedTiledDims{Experts,Tokens,K,N}
    GroupedParams p{};
    p.experts = u32_at(l.u, 0); p.tokens = u32_at(l.u, 4); p.K = u32_at(l.u, 8); p.N = u32_at(l.u, 12);
    if (l.len[2] < p.experts + 1 || l.len[1] < (uint64_t)p.experts * p.K * p.N ||
        l.len[0] < (uint64_t)p.tokens * p.K || l.len[3] < (uint64_t)p.tokens * p.N)
        return fail(AB_ERR_INVALID, "GroupedMatMul: Experts=%u Tokens=%u K=%u N=%u; lengths x[%u] "
                    "w[%u] offsets[%u] out[%u]", p.experts, p.tokens, p.K, p.N, l.len[0], l.len[1],
                    l.len[2], l.len[3]);
    if (!l.query_ws) {
        p.x = ptr<const float>(l, 0); p.w = ptr<const float>(l, 1);
        p.offsets = ptr<const uint32_t>(l, 2); p.out = ptr<float>(l, 3);
    }
    return run_grouped(l, p, false, false, p.tokens, "GroupedMatMul");
}

int launch_grouped_matmul_int4(Launch &l)
{   // x, bq, bs, bz, offsets, out; GroupedTiledDims
    GroupedParams p{};
    p.experts = u32_at(l.u, 0); p.tokens = u32_at(l.u, 4); p.K = u32_at(l.u, 8); p.N = u32_at(l.u, 12);
    uint64_t weights = (uint64_t)p.K * p.N;
    p.words_per_expert = (weights + 7) / 8;
    p.groups_per_expert = (weights + kGroup - 1) / kGroup;
    if (l.len[4] < p.experts + 1 || l.len[1] < p.experts * p.words_per_expert ||
        l.len[2] < p.experts * p.groups_per_expert || l.len[3] < p.experts * p.groups_per_expert ||
        l.len[0] < (uint64_t)p.tokens * p.K || l.len[5] < (uint64_t)p.tokens * p.N)
        return fail(AB_ERR_INVALID, "GroupedMatMulInt4: Experts=%u Tokens=%u K=%u N=%u does not "
                    "match the lengths block", p.experts, p.tokens, p.K, p.N);
    if (!l.query_ws) {
        p.x = ptr<const float>(l, 0); p.bq = ptr<const uint32_t>(l, 1);
        p.bs = ptr<const __half>(l, 2); p.bz = ptr<const __half>(l, 3);
        p.offsets = ptr<const uint32_t>(l, 4); p.out = ptr<float>(l, 5);
    }
    return run_grouped(l, p, true, false, p.tokens, "GroupedMatMulInt4");
}

__global__ void segment_offsets_kernel(const uint32_t *counts, uint32_t *offsets, uint32_t rows)
{   // serial, as the reference's is: a handful of experts
    if (threadIdx.x || blockIdx.x) return;
    uint32_t sum = 0;
    for (uint32_t r = 0; r < rows; r++) { offsets[r] = sum; sum += counts[r]; }
    offsets[rows] = sum;
}

int launch_segment_offsets(Launch &l)
{   // counts, offsets; SegmentDims{Rows}
    if (l.query_ws) { l.ws_need = 0; return AB_OK; }
    uint32_t rows = u32_at(l.u, 0);
    if (l.len[0] < rows || l.len[1] < rows + 1)
        return fail(AB_ERR_INVALID, "SegmentOffsets: Rows=%u, counts[%u], offsets[%u]", rows,
                    l.len[0], l.len[1]);
    segment_offsets_kernel<<<1, 32, 0, l.stream>>>(ptr<const uint32_t>(l, 0), ptr<uint32_t>(l, 1), rows); count_launch();
    return check_cuda(cudaGetLastError(), "SegmentOffsets");
}

}  // namespace ab
