// int4 linear for a decode batch (1 .. 16 activation rows per pass) on the 5th-generation tensor
// cores: weights streamed once from HBM, expanded to f16 in shared memory, contracted by
// tcgen05.mma into TMEM, K splits summed through the distributed shared memory of a cluster.  One
// kernel per product, no workspace.
//
//   out^T[n][m] = sum_k W^T[n][k] * a'[m][k]        per 128-column quantisation group
//
// The MMA's M dimension is a group's 128 output columns, its N dimension the 16 activation rows,
// its K the rows of the weight matrix.  Inside a group the scale and zero of a weight depend on
// k only, so the scale is folded into the activations (a' = a*s rounded to f16, the only rounded
// operand) and the weight operand is the raw 4-bit code: masked in place into an f16 with a zero
// exponent it IS the subnormal code*2^-24 (or *2^-20 for the odd nibbles), exactly.  One AND per
// pair of weights dequantises; the power of two is undone per column in the epilogue.  The
// zero-point term sum_k a'[m][k] z[k] is summed in f32 on the CUDA cores while a' is staged, from
// the same rounded a' (every product of two f16 is exact in f32).  A row of a group whose scale is
// 0 is the constant z (internal/kernels/int4.go:85-87): its a' is 0 and a*z goes into the same sum.
//
// Why this shape.  The legacy warp-level MMA needs about 7 us of tensor time for a 4096 x 11008
// product at 16 rows, twice the time HBM needs for the codes; tcgen05 does the same contraction in
// a fraction of a microsecond, which leaves the expansion (one AND per two weights, one 16-byte
// shared store per eight) as the only per-weight work.  A CTA owns G adjacent groups over a K
// range, four warps per group, each group an independent pipeline (its own named barrier,
// mbarriers, stage ring and TMEM columns).  G = 4 makes one 32-byte sector of scales serve four
// groups and divides the activation traffic by four.  The loads the prologue waits for (scales,
// zeros, activations) are issued BEFORE the flood of code loads, because an SM serves its loads in
// order.  The prologue stages a' for the CTA's whole K range in the K-major canonical layout, so
// the loop only expands codes: per 32-row stage a thread stores four 16-byte rows of core matrices
// (MN-major canonical layout, 8 x 8 f16 each) and one thread per group issues two K=16 MMAs and
// commits them to the stage's mbarrier; the stage is rewritten only after that barrier flips.
//
// Every wait on an mbarrier is bounded: a wait that runs out sets g_decode_error, the group skips
// its remaining work; the CTA still frees its TMEM and returns.
#include <cooperative_groups.h>
#include <cuda_fp16.h>

#include <cstdlib>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace ab {

static constexpr uint32_t kGroup = 128;
static constexpr int kDRows = 16;                // activation rows per pass = the MMA's N
static constexpr int kDStageRows = 32;           // rows of K per pipeline stage: two K=16 MMAs
static constexpr int kDDepth = 3;                // stages in shared memory per group
static constexpr int kDPre = 8;                  // stages of codes held in registers ahead of use
static constexpr int kDActBatch = 8;             // 16-byte activation loads in flight per thread
static constexpr int kDMaxCluster = 8;
static constexpr uint32_t kDSpinLimit = 1u << 22;

__device__ int g_decode_error;                   // nonzero: a bounded wait ran out

static constexpr uint32_t kDStageBytes = kDStageRows * 128 * 2;    // 8 KB: 32 k x 128 n halfs
static constexpr uint32_t kW_SBO = 128, kW_LBO = 16 * 128;         // n-block stride, k-block stride
static constexpr uint32_t kA_SBO = 128, kA_LBO = (kDRows / 8) * 128;   // m-block stride, k-block stride

__host__ __device__ inline uint32_t round32(uint32_t kc) { return (kc + 31) / 32 * 32; }
// shared memory: [stage rings: G x depth x 8 KB] [a': G x round32(kc) x 32 B]
//                [scales | zeros: G x kc halfs each] [partial zero-point sums: G x 16 x 8G floats]
//                [zero-point sums: G x 16 floats] [mbarriers: G x (depth + 1)] [TMEM base]
__host__ __device__ inline size_t decode_smem(int G, uint32_t kc)
{
    return (size_t)G * kDDepth * kDStageBytes + (size_t)G * round32(kc) * 32 + (size_t)2 * G * kc * 2 +
           (size_t)G * 16 * 8 * G * 4 + (size_t)G * 16 * 4 + (size_t)G * (kDDepth + 1) * 8 + 16;
}
// dynamic shared memory a CTA may use (G = 4: one CTA per SM; G = 2: one or two)
static constexpr size_t kDSmemCap = 225 * 1024;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo)
{
    // start address, leading (K-direction) and stride (MN-direction) byte offsets, all >> 4;
    // descriptor version 1 (bits 46-47); no swizzle (bits 61-63 = 0)
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) |
           ((uint64_t)(sbo >> 4) << 32) | (1ull << 46);
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

// Bounded wait for the phase with the given parity to complete.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity)
{
    const uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i < kDSpinLimit; i++) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\t"
                     "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
    }
    atomicExch(&g_decode_error, 1);
    return false;
}

__device__ __forceinline__ void group_sync(int id)          // the 128 threads of one group
{
    asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory");
}

__device__ __forceinline__ uint4 ldg_codes(const uint4 *p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// Eight codes of one word as eight f16 subnormals, in the order n0,n4 | n1,n5 | n2,n6 | n3,n7.
__device__ __forceinline__ uint4 expand(uint32_t w)
{
    const uint32_t w8 = w >> 8;
    return make_uint4(w & 0x000F000Fu, w & 0x00F000F0u, w8 & 0x000F000Fu, w8 & 0x00F000F0u);
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]),
                   "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
                   "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// grid = (ceil(N / 128 / G), splits), cluster = (1, splits, 1), 128 G threads.  Warp w works on
// group w / 4 of the tile.
template <int G>
__global__ void __launch_bounds__(128 * G)
int4_decode_kernel(const float *__restrict__ a, const uint4 *__restrict__ bq,
                   const __half *__restrict__ bs, const __half *__restrict__ bz,
                   float *__restrict__ out, uint32_t N, uint32_t K, uint32_t kc, uint32_t m0,
                   uint32_t mrows)
{
    constexpr int kThreads = 128 * G, kChunks = 8 * G;      // staging: 16 rows x kChunks 4-wide chunks
    extern __shared__ __align__(128) unsigned char smem[];
    const uint32_t kc32 = round32(kc);
    unsigned char *rings = smem;                                         // [G][depth][8 KB]
    unsigned char *ap = rings + (size_t)G * kDDepth * kDStageBytes;      // a' [G][kc32 / 8][2][8][8] halfs
    __half *s_s = reinterpret_cast<__half *>(ap + (size_t)G * kc32 * 32);    // [G][kc] scales
    __half *s_z = s_s + G * kc;                                              // [G][kc] zeros
    float *cpart = reinterpret_cast<float *>(s_z + G * kc);              // [G][16][kChunks]
    float *corr = cpart + G * 16 * kChunks;                              // [G][16]
    uint64_t *bars = reinterpret_cast<uint64_t *>(corr + G * 16);        // [G][depth] stage free, [G] done
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + G * (kDDepth + 1));
    __shared__ int s_abort;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gi = warp >> 2, wg = warp & 3, tg = tid & 127;            // group, warp and thread in it
    const uint32_t gpr = N / kGroup, g0 = blockIdx.x * G, g = g0 + gi, splits = gridDim.y;
    const bool group_on = g < gpr;
    const uint32_t kbeg = blockIdx.y * kc, kend = min(K, kbeg + kc);
    const uint32_t nrows = kend > kbeg ? kend - kbeg : 0;               // a multiple of 16
    const uint32_t nstages = (nrows + kDStageRows - 1) / kDStageRows;
    const size_t row_u4 = N / 32;                                        // uint4 per row of codes

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < G * (kDDepth + 1); i++) mbar_init(&bars[i], 1);
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // TMEM: 16 f32 columns per group (a power of two >= 32 in all)
    constexpr uint32_t kCols = G * kDRows < 32 ? 32 : G * kDRows;
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(kCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }

    // 1. scales and zeros of the G groups for every row of the K range and the activations, then
    //    the first stages of codes: all issued before any is used.  When a row's G scales start on
    //    a 4-byte boundary two groups come with one load and neighbouring lanes share a sector.
    constexpr int kPair = G >= 2 ? 2 : 1;                  // groups per metadata load
    constexpr int kPerRow = G / kPair;
    const bool paired = kPair == 2 && gpr % 2 == 0;
    constexpr int kMetaIt = (1408 * kPerRow + kThreads - 1) / kThreads;      // a CTA has at most 1408 rows
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
    // staging of a': activation row m, 4-wide chunks kch, kch + kChunks, ...  (m fastest, so that a
    // warp's stores fill whole core matrices)
    const int m = tid & 15, kch = tid >> 4;
    const bool row_on = (uint32_t)m < mrows;
    const float *arow = a + (size_t)(m0 + (row_on ? m : 0)) * K + kbeg;
    float4 av[kDActBatch];
    auto load_acts = [&](uint32_t k0) {
#pragma unroll
        for (int i = 0; i < kDActBatch; i++) {
            const uint32_t k = k0 + 4 * kChunks * i;
            av[i] = (row_on && k < nrows) ? __ldg(reinterpret_cast<const float4 *>(arow + k))
                                          : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    load_acts(4 * kch);
    // this thread's uint4 of every stage: row 8*wg + lane%8, 32-column chunk lane/8.  A quarter-warp
    // stores eight consecutive k-rows of one core matrix: 128 contiguous bytes.
    const int crow = 8 * wg + (lane & 7), cchunk = lane >> 3;
    const uint4 *cbase = bq + (size_t)kbeg * row_u4 + (size_t)(group_on ? g : g0) * 4 + cchunk;
    auto load_codes = [&](uint32_t st) -> uint4 {
        const uint32_t r = st * kDStageRows + crow;
        return (group_on && r < nrows) ? ldg_codes(cbase + (size_t)r * row_u4) : make_uint4(0, 0, 0, 0);
    };
    uint4 pre[kDPre];
#pragma unroll
    for (int p = 0; p < kDPre; p++) pre[p] = load_codes(p);

    // 2. scales and zeros into shared memory (a group past the last one gets zeros)
#pragma unroll
    for (int i = 0; i < kMetaIt; i++) {
        const uint32_t it = tid + i * kThreads, r = it / kPerRow, gg = (it % kPerRow) * kPair;
        if (r < nrows) {
#pragma unroll
            for (int h = 0; h < kPair; h++) {
                s_s[(gg + h) * kc + r] = __ushort_as_half((unsigned short)(sv[i] >> (16 * h)));
                s_z[(gg + h) * kc + r] = __ushort_as_half((unsigned short)(zv[i] >> (16 * h)));
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot + (uint32_t)gi * kDRows;           // this group's columns

    // 3. a' = f16(a * s) per group, K-major core matrices: element (m, k) of a group sits at
    //    (k / 8) * 256 + (m / 8) * 128 + (m % 8) * 16 + (k % 8) * 2.  The zero-point sums ride along.
    {
        float csum[G];
#pragma unroll
        for (int q = 0; q < G; q++) csum[q] = 0.f;
        const uint32_t moff = (uint32_t)(m >> 3) * kA_SBO + (uint32_t)(m & 7) * 16;
        for (uint32_t k0 = 4 * kch; k0 < kc32; k0 += 4 * kChunks * kDActBatch) {
            if (k0 != 4u * kch) load_acts(k0);
#pragma unroll
            for (int i = 0; i < kDActBatch; i++) {
                const uint32_t k = k0 + 4 * kChunks * i;
                if (k < kc32) {
                    const uint32_t koff = (k >> 3) * kA_LBO + (k & 7) * 2 + moff;
#pragma unroll
                    for (int q = 0; q < G; q++) {
                        uint2 pk = make_uint2(0, 0);
                        if (k < nrows) {
                            const uint2 s4 = *reinterpret_cast<const uint2 *>(s_s + q * kc + k);
                            const uint2 z4 = *reinterpret_cast<const uint2 *>(s_z + q * kc + k);
                            const float2 s01 = __half22float2(*reinterpret_cast<const __half2 *>(&s4.x));
                            const float2 s23 = __half22float2(*reinterpret_cast<const __half2 *>(&s4.y));
                            const float2 z01 = __half22float2(*reinterpret_cast<const __half2 *>(&z4.x));
                            const float2 z23 = __half22float2(*reinterpret_cast<const __half2 *>(&z4.y));
                            const __half2 p01 = __floats2half2_rn(av[i].x * s01.x, av[i].y * s01.y);
                            const __half2 p23 = __floats2half2_rn(av[i].z * s23.x, av[i].w * s23.y);
                            const float2 f01 = __half22float2(p01), f23 = __half22float2(p23);
                            // the term subtracted later: a'*z, or -a*z where the scale is zero
                            csum[q] = fmaf(s01.x == 0.f ? -av[i].x : f01.x, z01.x, csum[q]);
                            csum[q] = fmaf(s01.y == 0.f ? -av[i].y : f01.y, z01.y, csum[q]);
                            csum[q] = fmaf(s23.x == 0.f ? -av[i].z : f23.x, z23.x, csum[q]);
                            csum[q] = fmaf(s23.y == 0.f ? -av[i].w : f23.y, z23.y, csum[q]);
                            pk.x = *reinterpret_cast<const uint32_t *>(&p01);
                            pk.y = *reinterpret_cast<const uint32_t *>(&p23);
                        }
                        *reinterpret_cast<uint2 *>(ap + (size_t)q * kc32 * 32 + koff) = pk;
                    }
                }
            }
        }
#pragma unroll
        for (int q = 0; q < G; q++) cpart[(q * 16 + m) * kChunks + kch] = csum[q];
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");       // a' is read by the tensor core
    __syncthreads();
    if (tid < G * 16) {                          // corr[group][row], summed in a fixed order
        float c = 0.f;
        for (int q = 0; q < kChunks; q++) c += cpart[tid * kChunks + q];
        corr[tid] = c;
    }

    // 4. the loop, one pipeline per group: expand a stage of codes, hand it to the tensor core
    constexpr uint32_t idesc = (1u << 4) | (1u << 15) | ((uint32_t)(kDRows >> 3) << 17) | ((128u >> 4) << 24);
    unsigned char *ring = rings + (size_t)gi * kDDepth * kDStageBytes;
    uint64_t *gbars = bars + gi * (kDDepth + 1);
    const uint32_t a_base = smem_u32(ap + (size_t)gi * kc32 * 32);
    bool alive = true;
    if (group_on) {
        for (uint32_t st0 = 0; st0 < nstages; st0 += kDPre) {
#pragma unroll
            for (int pp = 0; pp < kDPre; pp++) {
                const uint32_t st = st0 + pp;
                if (st >= nstages) break;                    // uniform across the group
                const uint32_t buf = st % kDDepth, use = st / kDDepth;
                // the MMAs that last read this buffer (stage st - depth) must have completed
                if (use > 0 && alive) {
                    if (!mbar_wait(&gbars[buf], (use - 1) & 1)) s_abort = 1;
                }
                alive = alive && !s_abort;
                unsigned char *Wt = ring + buf * kDStageBytes;
                if (alive) {
                    const uint4 cw = pre[pp];
                    unsigned char *dstp = Wt + (crow >> 3) * kW_LBO + (crow & 7) * 16 + (cchunk * 4) * kW_SBO;
                    *reinterpret_cast<uint4 *>(dstp) = expand(cw.x);
                    *reinterpret_cast<uint4 *>(dstp + kW_SBO) = expand(cw.y);
                    *reinterpret_cast<uint4 *>(dstp + 2 * kW_SBO) = expand(cw.z);
                    *reinterpret_cast<uint4 *>(dstp + 3 * kW_SBO) = expand(cw.w);
                    pre[pp] = load_codes(st + kDPre);
                    // generic-proxy stores must be visible to the tensor core's (async-proxy) reads
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                }
                group_sync(1 + gi);
                if (tg == 0 && alive) {
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                    for (int k16 = 0; k16 < kDStageRows / 16; k16++) {
                        const uint32_t accum = (st > 0 || k16 > 0) ? 1u : 0u;
                        const uint64_t adesc = make_desc(smem_u32(Wt) + k16 * 2 * kW_LBO, kW_LBO, kW_SBO);
                        const uint64_t bdesc = make_desc(a_base + (st * 2 + k16) * 2 * kA_LBO, kA_LBO, kA_SBO);
                        umma_f16(tmem, adesc, bdesc, idesc, accum);
                    }
                    // arrives on the stage's barrier once these MMAs have finished reading shared memory
                    umma_commit(&gbars[buf]);
                    if (st + 1 == nstages) umma_commit(&gbars[kDDepth]);
                }
            }
        }
        if (nstages > 0 && alive && !mbar_wait(&gbars[kDDepth], 0)) s_abort = 1;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();                             // every group is done with its ring; corr is written
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    alive = !s_abort;

    // 5. accumulators out of TMEM: lane = column of the group (permuted by `expand`), TMEM column =
    //    activation row.  Undo the subnormal placement, subtract the zero-point sum, and park the
    //    16 x 128 tile in the group's ring for the cluster (row-major, one row = 512 bytes).
    float *gred = reinterpret_cast<float *>(ring);
    {
        const int L = 32 * wg + lane;                                    // TMEM lane = MMA row
        const int l8 = L & 7;
        const int col = (L & ~7) + ((l8 >> 1) | ((l8 & 1) << 2));        // 0,4,1,5,2,6,3,7
        const float f = (l8 & 2) ? 1048576.f : 16777216.f;              // rows 2,3,6,7 carried 2^-20
        uint32_t r[16];
#pragma unroll
        for (int i = 0; i < 16; i++) r[i] = 0;
        if (alive && group_on && nstages > 0) tmem_ld16(tmem + ((uint32_t)(32 * wg) << 16), r);
#pragma unroll
        for (int i = 0; i < 16; i++) gred[i * 128 + col] = __uint_as_float(r[i]) * f - corr[gi * 16 + i];
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(*tmem_slot), "r"(kCols) : "memory");

    // thread = one column of the tile: group gi, column tg
    float *orow = out + (size_t)m0 * N + (size_t)g * kGroup + tg;
    if (splits == 1) {
        if (group_on)
            for (uint32_t mm = 0; mm < mrows; mm++) orow[(size_t)mm * N] = gred[mm * 128 + tg];
        return;
    }

    // 6. the K splits: rank r of the cluster adds rows r, r + splits, ... of every CTA's tile
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    const uint32_t rank = cluster.block_rank();
    const float *peer[kDMaxCluster];
#pragma unroll
    for (int q = 0; q < kDMaxCluster; q++) peer[q] = cluster.map_shared_rank(gred, (uint32_t)q < splits ? q : 0);
    for (uint32_t mm = rank; mm < mrows; mm += splits) {
        float pv[kDMaxCluster];
#pragma unroll
        for (int q = 0; q < kDMaxCluster; q++) pv[q] = (uint32_t)q < splits ? peer[q][mm * 128 + tg] : 0.f;
        float v = pv[0];
#pragma unroll
        for (int q = 1; q < kDMaxCluster; q++) v += pv[q];
        if (group_on) orow[(size_t)mm * N] = v;
    }
    cluster.sync();                              // nobody leaves while its tile is being read
}

static uint32_t env_u32(const char *name)
{
    const char *e = getenv(name);
    return e ? (uint32_t)atoi(e) : 0u;
}

Int4DecodePlan plan_int4_decode(uint32_t M, uint32_t N, uint32_t K)
{
    Int4DecodePlan p{};
    p.ok = N % kGroup == 0 && K % 16 == 0 && N > 0 && K > 0 && M > 0;
    if (!p.ok) return p;
    const uint32_t gpr = N / kGroup, sms = (uint32_t)sm_count();
    static const uint32_t forced_g = env_u32("AB_INT4_TILE_GROUPS"), forced_s = env_u32("AB_INT4_SPLITS");
    // the widest tile that still gives most SMs a CTA with a cluster of at most eight K splits
    uint32_t G = 4;
    if ((gpr + 3) / 4 * kDMaxCluster < sms * 3 / 4) G = 2;
    if (forced_g == 2 || forced_g == 4) G = forced_g;
    for (;; G /= 2) {
        p.G = (int)G;
        p.tiles = (gpr + G - 1) / G;
        uint32_t splits = sms / p.tiles;                           // one CTA per SM
        if (forced_s) splits = forced_s;
        if (splits < 1) splits = 1;
        if (splits > (uint32_t)kDMaxCluster) splits = kDMaxCluster;
        uint32_t kc = ((K + splits - 1) / splits + 15) / 16 * 16;
        while (kc > 16 && (decode_smem((int)G, kc) > kDSmemCap || kc > 1408)) kc -= 16;
        p.kc = kc;
        p.splits = (K + kc - 1) / kc;
        if (p.splits <= (uint32_t)kDMaxCluster || G == 2) break;
    }
    p.ok = p.splits <= (uint32_t)kDMaxCluster;                     // deeper K: another kernel takes it
    return p;
}

template <int G>
static int launch_decode(const Launch &l, const Int4DecodePlan &p, float *out, uint32_t N, uint32_t K,
                         uint32_t m0, uint32_t mrows)
{
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        int rc = check_cuda(cudaFuncSetAttribute(int4_decode_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)kDSmemCap), "int4_decode_kernel attributes");
        if (rc) return rc;
        attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.tiles, p.splits);
    cfg.blockDim = dim3(128 * G);
    cfg.dynamicSmemBytes = decode_smem(G, p.kc);
    cfg.stream = l.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = p.splits;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int rc = check_cuda(cudaLaunchKernelEx(&cfg, int4_decode_kernel<G>, ptr<const float>(l, 0),
                                           ptr<const uint4>(l, 1), ptr<const __half>(l, 2),
                                           ptr<const __half>(l, 3), out, N, K, p.kc, m0, mrows),
                        "int4_decode_kernel");
    count_launch();
    return rc;
}

int run_int4_decode(const Launch &l, const Int4DecodePlan &p, float *out, uint32_t M, uint32_t N, uint32_t K)
{
    for (uint32_t m0 = 0; m0 < M; m0 += kDRows) {
        const uint32_t mrows = M - m0 < (uint32_t)kDRows ? M - m0 : kDRows;
        int rc = p.G == 4 ? launch_decode<4>(l, p, out, N, K, m0, mrows)
                          : launch_decode<2>(l, p, out, N, K, m0, mrows);
        if (rc) return rc;
    }
    return AB_OK;
}

int int4_decode_error_flag()
{
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_decode_error, sizeof v) != cudaSuccess) { cudaGetLastError(); return -1; }
    return v;
}

}  // namespace ab
