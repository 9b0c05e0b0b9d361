// int4 linear for a decode batch: 1 .. 16 activation rows per pass, weights streamed once from HBM,
// contracted on the tensor cores, K splits summed through the distributed shared memory of a
// thread-block cluster.  One kernel per product, no workspace.
//
// Arithmetic.  With N a multiple of 128 a quantisation group is 128 adjacent columns of one row
// k, so inside a group's columns
//
//   out[m][n] = sum_k (a[m][k] s[k]) code[k][n]  -  sum_k (a[m][k] s[k]) z[k]
//
// a' = a*s is rounded to f16 once; the 4-bit code masked in place into the mantissa of an f16 with
// a zero exponent is the subnormal code * 2^-24 (2^-20 for the odd nibble), exactly, so a pair of
// codes becomes an MMA operand with one AND; the power of two is undone in the epilogue.  The
// second sum is a 17th MMA over the same rounded a' with z as its B operand.  A row of a group
// whose scale is 0 is the constant z (internal/kernels/int4.go:85-87): its a' is 0 and a*z is added
// from a separate f32 sum.
//
// Shape.  A CTA owns G adjacent groups (G x 128 columns) over a K range, four warps per group;
// the cluster is the K splits of those columns.  What decides G: the scale of (row k, group g) is
// a 2-byte value 2*N/128 bytes away from its neighbour in k, so fetching a group's scales costs
// one 32-byte sector per row whatever is done, and the activations are re-read by every column
// tile.  With G = 4 one sector serves four groups and the activation traffic drops fourfold; the
// CTA is then 16 warps, one per SM.
//
// Order of loads.  An SM serves its loads in order, so the small loads the prologue waits for
// (scales, zeros, activations) are issued BEFORE the flood of code loads, never behind it.  The
// prologue stages the whole K range of a' (f16, 16 rows, per group) in shared memory, so the loop
// has no conversion work: per 16-row step a warp does 4 x 8-byte code loads (a private register
// ring, four steps deep), three 8-byte shared loads, 17 MMAs and 48 integer ops for 2048 weights.
// The four warps of a group take alternate steps and add their accumulators in shared memory;
// the CTAs of the cluster then read each other's sums in rank order (deterministic) and write
// the output rows.
#include <cooperative_groups.h>
#include <cuda_fp16.h>

#include <cstdlib>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace ab {

static constexpr uint32_t kGroup = 128;
static constexpr int kBPhases = 4;                    // warps per group: warp p takes steps p, p+4, ...
static constexpr int kBDepth = 4;                     // code steps in flight per warp
static constexpr int kBActBatch = 8;                  // 16-byte activation loads in flight per thread
static constexpr int kBMaxCluster = 16;          // above 8 needs the non-portable cluster size opt-in
static constexpr int kBUsualCluster = 8;

// a' row stride in bytes: kc f16 values, padded so that the eight rows a fragment load touches
// start 32 bytes apart modulo 128 (no bank conflict for 8-byte loads)
__host__ __device__ inline uint32_t batch_a_stride(uint32_t kc) { return (kc * 2 + 127) / 128 * 128 + 32; }
// shared memory: [a' : G x 16 x stride] (re-used for the warps' sums: 4G x 16 x 128 floats)
//                [zeros | scales | zeros as stored : G x kc halfs each] [constant-row sums: G x 16 x 8G floats]
__host__ __device__ inline size_t batch_front(int G, uint32_t kc)
{
    const size_t front = (size_t)G * 16 * batch_a_stride(kc), red = (size_t)kBPhases * G * 16 * 128 * 4;
    return front > red ? front : red;
}
__host__ __device__ inline size_t batch_smem(int G, uint32_t kc)
{
    return batch_front(G, kc) + (size_t)3 * G * kc * 2 + (size_t)G * 16 * 8 * G * 4;
}
// dynamic shared memory a CTA may use when 4 / G of them share an SM
__host__ __device__ constexpr size_t batch_smem_cap(int G) { return (size_t)226 * 1024 / (4 / G) - 1024; }

__device__ __forceinline__ uint2 ldg_stream(const uint2 *p)
{
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
                 "{%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// column c of output row m inside a 16 x 128 sum buffer: rotated inside each 32-column block so
// that the accumulator stores (float4, rows gid, blocks t) spread over all banks
__device__ __forceinline__ int red_at(int m, int c)
{
    const int blk = c >> 5;
    return m * 128 + (c & ~31) + ((c + 4 * blk + 16 * (m & 1)) & 31);
}

// grid = (ceil(N / 128 / G), splits), cluster = (1, splits, 1), 128 G threads.  Warp w works on
// group w / 4 of the tile, steps (w % 4), (w % 4) + 4, ...  In a 16-row step lane (gid = lane/4,
// t = lane%4) reads rows 4t .. 4t+3 of the 16 columns 16*gid .. 16*gid+15 of the group (the MMA's k
// index is a free relabelling: rows {4t,4t+1} stand for its slots {2t,2t+1}, rows {4t+2,4t+3} for
// {2t+8,2t+9}); MMA j takes code j of each of those rows as its B fragment, so it covers columns
// {16*n + j : n = 0..7} and the thread ends up holding out[gid, gid+8][32t .. 32t+31].
template <int G>
__global__ void __launch_bounds__(128 * G, 4 / G)
int4_batch_kernel(const float *__restrict__ a, const uint2 *__restrict__ bq,
                  const __half *__restrict__ bs, const __half *__restrict__ bz,
                  float *__restrict__ out, uint32_t N, uint32_t K, uint32_t kc, uint32_t m0,
                  uint32_t mrows, const float *__restrict__ amax)
{
    constexpr int kThreads = 128 * G, kChunks = 8 * G;      // staging: 16 rows x kChunks 4-wide chunks
    extern __shared__ __align__(16) unsigned char smem[];
    const uint32_t astride = batch_a_stride(kc);
    unsigned char *ap = smem;                                            // a' [G][16][astride]
    float *red = reinterpret_cast<float *>(smem);                        // [4G][16][128], after the loop
    __half *s_z = reinterpret_cast<__half *>(smem + batch_front(G, kc)); // [G][kc]
    __half *s_s = s_z + G * kc;                                          // scales (staging only)
    __half *s_zc = s_s + G * kc;                                         // zeros as stored (constant rows)
    float *cpart = reinterpret_cast<float *>(s_zc + G * kc);             // [G][16][kChunks]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gid = lane >> 2, t = lane & 3;
    const int gi = warp / kBPhases, ph = warp % kBPhases;
    const uint32_t gpr = N / kGroup, g0 = blockIdx.x * G, g = g0 + gi, splits = gridDim.y;
    const bool warp_on = g < gpr;
    const uint32_t kbeg = blockIdx.y * kc, kend = min(K, kbeg + kc);
    const uint32_t nrows = kend > kbeg ? kend - kbeg : 0, nsteps = nrows / 16;      // K % 16 == 0
    const size_t row_u2 = N / 16;
    const uint2 *code_base = bq + (size_t)(kbeg + 4 * t) * row_u2 + (size_t)(warp_on ? g : g0) * 8 + gid;
    // this warp's ring of codes: round r is step ph + 4r
    uint2 cw[kBDepth][4];
    auto fetch = [&](uint2 (&dst)[4], uint32_t round) {
        const uint32_t st = ph + kBPhases * round;
        const bool live = st < nsteps && warp_on;
        const uint2 *src = code_base + (size_t)(live ? st * 16 : 0) * row_u2;
#pragma unroll
        for (int i = 0; i < 4; i++) dst[i] = live ? ldg_stream(src + i * row_u2) : make_uint2(0, 0);
    };

    // 1. scales and zeros of the G groups for every row of the K range and the first batch of
    //    activations, then the first rounds of codes: all issued before any is used.
    //    Scales: when a row's G values start on a 4-byte boundary two groups come with one load
    //    and neighbouring lanes read the same sector.
    constexpr int kPair = G >= 2 ? 2 : 1;                  // groups per metadata load
    constexpr int kPerRow = G / kPair;
    const bool paired = kPair == 2 && gpr % 2 == 0;
    // a CTA never has more than 1408 rows; items = rows x loads per row
    constexpr int kMetaIt = (1408 * kPerRow + kThreads - 1) / kThreads;
    uint32_t sv[kMetaIt], zv[kMetaIt];
#pragma unroll
    for (int i = 0; i < kMetaIt; i++) {
        const uint32_t it = tid + i * kThreads, r = it / kPerRow, gg = (it % kPerRow) * kPair;
        sv[i] = zv[i] = 0;
        if (r < nrows && g0 + gg < gpr) {
            const size_t at = (size_t)(kbeg + r) * gpr + g0 + gg;
            if (paired) {
                sv[i] = __ldg(reinterpret_cast<const uint32_t *>(bs + at));
                zv[i] = __ldg(reinterpret_cast<const uint32_t *>(bz + at));
            } else {
                sv[i] = __ldg(reinterpret_cast<const unsigned short *>(bs + at));
                zv[i] = __ldg(reinterpret_cast<const unsigned short *>(bz + at));
                if (kPair == 2 && g0 + gg + 1 < gpr) {
                    sv[i] |= (uint32_t)__ldg(reinterpret_cast<const unsigned short *>(bs + at + 1)) << 16;
                    zv[i] |= (uint32_t)__ldg(reinterpret_cast<const unsigned short *>(bz + at + 1)) << 16;
                }
            }
        }
    }
    const int m = tid / kChunks, kch = tid % kChunks;      // staging: row m, chunks kch, kch + kChunks, ...
    const bool row_on = (uint32_t)m < mrows;
    const float *arow = a + (size_t)(m0 + (row_on ? m : 0)) * K + kbeg;
    // The row's activations times an exact power of two that puts the largest of the row in
    // [2^8, 2^9) (amax: the rows' largest magnitudes; NULL: as they are): a * s stays a normal f16
    // whatever the activations' magnitude.  Undone where the sums are stored.
    const float pa = (amax && row_on) ? ab_pow2(8 - ab_row_exponent(__float_as_uint(fabsf(__ldg(amax + m0 + m))))) : 1.f;
    float4 av[kBActBatch];
    auto load_acts = [&](uint32_t k0) {
#pragma unroll
        for (int i = 0; i < kBActBatch; i++) {
            const uint32_t k = k0 + 4 * kChunks * i;
            av[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (row_on && k < nrows) {
                const float4 x = __ldg(reinterpret_cast<const float4 *>(arow + k));
                av[i] = make_float4(x.x * pa, x.y * pa, x.z * pa, x.w * pa);
            }
        }
    };
    load_acts(4 * kch);
#pragma unroll
    for (int u = 0; u < kBDepth; u++) fetch(cw[u], u);

    // 2. scales and zeros into shared memory (a group past the last one gets zeros)
    int has_const = 0;
#pragma unroll
    for (int i = 0; i < kMetaIt; i++) {
        const uint32_t it = tid + i * kThreads, r = it / kPerRow, gg = (it % kPerRow) * kPair;
        if (r < nrows) {
#pragma unroll
            for (int h = 0; h < kPair; h++) {
                const unsigned short sb = (unsigned short)(sv[i] >> (16 * h)), zb = (unsigned short)(zv[i] >> (16 * h));
                const bool cst = (sb & 0x7fffu) == 0;
                s_s[(gg + h) * kc + r] = __ushort_as_half(sb);
                s_zc[(gg + h) * kc + r] = __ushort_as_half(zb);
                s_z[(gg + h) * kc + r] = __ushort_as_half(cst ? (unsigned short)0 : zb);
                has_const |= cst && g0 + gg + h < gpr;
            }
        }
    }
    const int any_const = __syncthreads_or(has_const);

    // 3. a' = f16(a * s) per group for 16 activation rows x the K range (rows past the batch are zero)
    {
        float csum[G];
#pragma unroll
        for (int q = 0; q < G; q++) csum[q] = 0.f;
        for (uint32_t k0 = 4 * kch; k0 < nrows; k0 += 4 * kChunks * kBActBatch) {
            if (k0 != 4u * kch) load_acts(k0);
#pragma unroll
            for (int i = 0; i < kBActBatch; i++) {
                const uint32_t k = k0 + 4 * kChunks * i;
                if (k < nrows) {
#pragma unroll
                    for (int q = 0; q < G; q++) {
                        const uint2 s4 = *reinterpret_cast<const uint2 *>(s_s + q * kc + k);
                        const float2 s01 = __half22float2(*reinterpret_cast<const __half2 *>(&s4.x));
                        const float2 s23 = __half22float2(*reinterpret_cast<const __half2 *>(&s4.y));
                        const __half2 p01 = __floats2half2_rn(av[i].x * s01.x, av[i].y * s01.y);
                        const __half2 p23 = __floats2half2_rn(av[i].z * s23.x, av[i].w * s23.y);
                        uint2 pk;
                        pk.x = *reinterpret_cast<const uint32_t *>(&p01);
                        pk.y = *reinterpret_cast<const uint32_t *>(&p23);
                        *reinterpret_cast<uint2 *>(ap + ((size_t)q * 16 + m) * astride + (size_t)k * 2) = pk;
                        if (any_const) {
                            const __half *zc = s_zc + q * kc + k;
                            if (s01.x == 0.f) csum[q] = fmaf(av[i].x, __half2float(zc[0]), csum[q]);
                            if (s01.y == 0.f) csum[q] = fmaf(av[i].y, __half2float(zc[1]), csum[q]);
                            if (s23.x == 0.f) csum[q] = fmaf(av[i].z, __half2float(zc[2]), csum[q]);
                            if (s23.y == 0.f) csum[q] = fmaf(av[i].w, __half2float(zc[3]), csum[q]);
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int q = 0; q < G; q++) cpart[(q * 16 + m) * kChunks + kch] = csum[q];
    }
    __syncthreads();

    // 4. the loop: no barrier, no conversion
    float acc[16][4], accz[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 16; j++) { acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f; }
    const unsigned char *a_lo = ap + ((size_t)gi * 16 + gid) * astride + 8 * t, *a_hi = a_lo + 8 * (size_t)astride;
    const __half *my_z = s_z + gi * kc + 4 * t;

    const uint32_t nrounds = (warp_on && nsteps > (uint32_t)ph) ? (nsteps - ph + kBPhases - 1) / kBPhases : 0;
    for (uint32_t rd0 = 0; rd0 < nrounds; rd0 += kBDepth) {
#pragma unroll
        for (int u = 0; u < kBDepth; u++) {
            const uint32_t rd = rd0 + u, st = ph + kBPhases * rd;
            if (rd < nrounds) {
                const uint2 alo = *reinterpret_cast<const uint2 *>(a_lo + st * 32);
                const uint2 ahi = *reinterpret_cast<const uint2 *>(a_hi + st * 32);
                const uint2 z4 = *reinterpret_cast<const uint2 *>(my_z + st * 16);
                const uint32_t af[4] = {alo.x, ahi.x, alo.y, ahi.y};
                mma_f16(accz, af, z4.x, z4.y);
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    const uint32_t w0 = c ? cw[u][0].y : cw[u][0].x, w1 = c ? cw[u][1].y : cw[u][1].x;
                    const uint32_t w2 = c ? cw[u][2].y : cw[u][2].x, w3 = c ? cw[u][3].y : cw[u][3].x;
                    // 16-bit lanes: low = row 4t (or 4t+2), high = row 4t+1 (or 4t+3)
                    const uint32_t lo01 = __byte_perm(w0, w1, 0x5410), hi01 = __byte_perm(w0, w1, 0x7632);
                    const uint32_t lo23 = __byte_perm(w2, w3, 0x5410), hi23 = __byte_perm(w2, w3, 0x7632);
                    const uint32_t src01[4] = {lo01, lo01 >> 8, hi01, hi01 >> 8};
                    const uint32_t src23[4] = {lo23, lo23 >> 8, hi23, hi23 >> 8};
#pragma unroll
                    for (int p = 0; p < 4; p++) {
                        mma_f16(acc[8 * c + 2 * p], af, src01[p] & 0x000F000Fu, src23[p] & 0x000F000Fu);
                        mma_f16(acc[8 * c + 2 * p + 1], af, src01[p] & 0x00F000F0u, src23[p] & 0x00F000F0u);
                    }
                }
            }
            fetch(cw[u], rd + kBDepth);          // refill the slot just used
        }
    }
    __syncthreads();                             // every warp is done with a' before it becomes red

    // 5. the four warps of a group, through shared memory.  The subnormal placement is undone here
    //    (even codes carried 2^-24, odd codes 2^-20) and the correction, of which every column of
    //    accz holds the same sum, is subtracted.
    {
        float *mine = red + warp * (16 * 128);
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int row = gid + 8 * h;
            const float cz = accz[2 * h];
#pragma unroll
            for (int half = 0; half < 2; half++)
#pragma unroll
                for (int j = 0; j < 16; j += 4) {
                    float4 v;
                    v.x = acc[j][2 * h + half] * 16777216.f - cz;
                    v.y = acc[j + 1][2 * h + half] * 1048576.f - cz;
                    v.z = acc[j + 2][2 * h + half] * 16777216.f - cz;
                    v.w = acc[j + 3][2 * h + half] * 1048576.f - cz;
                    *reinterpret_cast<float4 *>(mine + red_at(row, 32 * t + 16 * half + j)) = v;
                }
        }
    }
    __syncthreads();
    // thread = one column of the tile: group tg, column tc; its sums live in the group's first buffer
    const int tg = tid >> 7, tc = tid & 127;
    const bool col_on = g0 + tg < gpr;
    float *gred = red + (size_t)tg * kBPhases * (16 * 128);
    float *orow = out + (size_t)m0 * N + (size_t)(g0 + tg) * kGroup + tc;
    auto row_unscale = [&](uint32_t mm) {
        return amax ? ab_pow2(ab_row_exponent(__float_as_uint(fabsf(__ldg(amax + m0 + mm)))) - 8) : 1.f;
    };
    {
        float v[16];
#pragma unroll
        for (int mm = 0; mm < 16; mm++) {
            const int at = red_at(mm, tc);
            v[mm] = (uint32_t)mm < mrows
                        ? (gred[at] + gred[16 * 128 + at]) + (gred[2 * 16 * 128 + at] + gred[3 * 16 * 128 + at]) : 0.f;
        }
        if (any_const) {
#pragma unroll
            for (int mm = 0; mm < 16; mm++) {
                float cs = 0.f;
                for (int q = 0; q < kChunks; q++) cs += cpart[(tg * 16 + mm) * kChunks + q];
                v[mm] += cs;
            }
        }
#pragma unroll
        for (int mm = 0; mm < 16; mm++)
            if ((uint32_t)mm < mrows) {
                if (splits > 1) gred[red_at(mm, tc)] = v[mm];
                else if (col_on) orow[(size_t)mm * N] = v[mm] * row_unscale(mm);
            }
    }
    if (splits == 1) return;

    // 6. the K splits: rank r of the cluster adds rows r, r + splits, ... of every CTA's sums
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    const uint32_t rank = cluster.block_rank();
    const float *peer[kBMaxCluster];
#pragma unroll
    for (int q = 0; q < kBMaxCluster; q++) peer[q] = cluster.map_shared_rank(gred, (uint32_t)q < splits ? q : 0);
    for (uint32_t mm = rank; mm < mrows; mm += splits) {
        const int at = red_at(mm, tc);
        float pv[kBMaxCluster];
#pragma unroll
        for (int q = 0; q < kBMaxCluster; q++) pv[q] = (uint32_t)q < splits ? peer[q][at] : 0.f;
        float v = pv[0];
#pragma unroll
        for (int q = 1; q < kBMaxCluster; q++) v += pv[q];
        if (col_on) orow[(size_t)mm * N] = v * row_unscale(mm);
    }
    cluster.sync();                              // nobody leaves while its sums are being read
}

Int4BatchPlan plan_int4_batch(uint32_t M, uint32_t N, uint32_t K)
{
    Int4BatchPlan p{};
    p.ok = N % kGroup == 0 && K % 16 == 0 && N > 0 && K > 0 && M > 0;
    if (!p.ok) return p;
    const uint32_t gpr = N / kGroup, sms = (uint32_t)sm_count();
    // wide matrices: four groups per tile (one scale sector serves four groups, a quarter of the
    // activation traffic); narrow ones: one group per tile, or the SMs run short of CTAs
    uint32_t G = gpr >= 64 ? 4 : 1;
    p.G = (int)G;
    p.tiles = (gpr + G - 1) / G;
    const uint32_t slots = (4u / G) * sms;                         // CTAs resident at once
    uint32_t splits = slots / p.tiles;
    // clusters of more than eight cost more than they save on a full-size product; a small product
    // (a tensor-parallel shard: a few tiles) is a chain of latencies that only more CTAs shorten
    const uint32_t most = p.tiles * kBUsualCluster <= sms ? kBMaxCluster : kBUsualCluster;
    if (splits > most) splits = most;
    if (splits < 1) splits = 1;
    if (splits > (uint32_t)kBMaxCluster) splits = kBMaxCluster;
    uint32_t kc = ((K + splits - 1) / splits + 15) / 16 * 16;
    while (kc > 16 && (batch_smem((int)G, kc) > batch_smem_cap((int)G) || kc > 1408)) kc -= 16;
    p.kc = kc;
    p.splits = (K + kc - 1) / kc;
    // one cluster per tile and one wave of CTAs, or another kernel takes the product
    p.ok = p.splits <= (uint32_t)kBMaxCluster && p.tiles * p.splits <= slots;
    return p;
}

template <int G>
static int launch_batch(const Launch &l, const Int4BatchPlan &p, float *out, uint32_t N, uint32_t K,
                        uint32_t m0, uint32_t mrows, const float *amax)
{
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        int rc = check_cuda(cudaFuncSetAttribute(int4_batch_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)batch_smem_cap(G)), "int4_batch_kernel attributes");
        if (rc) return rc;
        rc = check_cuda(cudaFuncSetAttribute(int4_batch_kernel<G>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1),
                        "int4_batch_kernel attributes");
        if (rc) return rc;
        attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.tiles, p.splits);
    cfg.blockDim = dim3(128 * G);
    cfg.dynamicSmemBytes = batch_smem(G, p.kc);
    cfg.stream = l.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = p.splits;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int rc = check_cuda(cudaLaunchKernelEx(&cfg, int4_batch_kernel<G>, ptr<const float>(l, 0),
                                           ptr<const uint2>(l, 1), ptr<const __half>(l, 2),
                                           ptr<const __half>(l, 3), out, N, K, p.kc, m0, mrows, amax),
                        "int4_batch_kernel");
    count_launch();
    return rc;
}

size_t int4_batch_workspace(uint32_t M) { return align_up((size_t)M * 4, 256); }

// The rows' largest magnitudes first (into the workspace), then passes of 16 rows.
int run_int4_batch(const Launch &l, const Int4BatchPlan &p, float *out, uint32_t M, uint32_t N, uint32_t K)
{
    if (!l.ws || l.ws_bytes < int4_batch_workspace(M))
        return fail(AB_ERR_INVALID, "the int4 batch kernel needs %zu bytes of workspace, given %zu",
                    int4_batch_workspace(M), l.ws_bytes);
    float *amax = static_cast<float *>(l.ws);
    int rc = run_row_absmax(l.stream, ptr<const float>(l, 0), amax, M, K, false);
    if (rc) return rc;
    for (uint32_t m0 = 0; m0 < M; m0 += 16) {
        const uint32_t mrows = M - m0 < 16 ? M - m0 : 16;
        rc = p.G == 4 ? launch_batch<4>(l, p, out, N, K, m0, mrows, amax)
             : p.G == 2 ? launch_batch<2>(l, p, out, N, K, m0, mrows, amax)
                        : launch_batch<1>(l, p, out, N, K, m0, mrows, amax);
        if (rc) return rc;
    }
    return AB_OK;
}

}  // namespace ab
