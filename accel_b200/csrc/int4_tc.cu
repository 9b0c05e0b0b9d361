// int4 linear on the 5th-generation tensor cores (tcgen05 + TMEM), for a batch of activation rows.
//
//   out^T[n][m] = sum_k W^T[n][k] * a'[m][k]            (one 128-column quantisation group per CTA)
//
// The MMA's M dimension is the group's 128 output columns, its N dimension the activation rows
// (16 .. 256 per pass), its K the rows of the weight matrix.  Inside one group the scale and zero of
// a weight depend on k only, so the scale is folded into the activations (a' = a*s, rounded to f16,
// the only rounded operand) and the weight operand is the raw 4-bit code: masked in place into an
// f16 with a zero exponent it IS the subnormal code*2^-24 (or *2^-20 for the odd nibbles), exactly.
// One AND per pair of weights dequantises; the power of two is undone per column in the epilogue.
//
// The zero-point term sum_k a'[m][k] z[k] is a second, thin MMA per step whose weight operand is
// the column of zeros z[k] (an f16 already), accumulated in its own TMEM columns from the same a'
// and subtracted in the epilogue, so the two sums cancel as they do in exact arithmetic.  A group
// with s == 0 is the constant z (internal/kernels/int4.go:85-87): its codes are replaced by zeros
// and its a' by -a, which makes the main product vanish and the subtracted term add a*z.
//
// Data movement.  Codes are read with 128-bit loads eight stages ahead, activations four, in
// registers (the accumulators live in TMEM, so registers are free for that).  The codes are
// expanded to f16 and stored to shared memory in the MN-major canonical layout (8x8 core matrices
// of 128 contiguous bytes: eight k-rows of eight n-values); a' is stored K-major.  One thread
// issues the MMAs of a 64-row stage and commits them to the stage's mbarrier; a stage's shared
// memory (three stages) is rewritten only after that barrier flips.  The accumulator
// (128 lanes x N columns of f32) is read back with tcgen05.ld.
//
// Every wait on an mbarrier is bounded: a wait that runs out sets g_tc_error, the CTA skips its
// remaining work, frees its TMEM and returns.
#include <cuda_fp16.h>

#include "common.cuh"

namespace ab {

static constexpr uint32_t kGroup = 128;
static constexpr int kTcThreads = 128;
static constexpr int kStageRows = 64;            // rows of K per pipeline stage: four K=16 MMAs
static constexpr int kDepth = 3;                 // stages in shared memory
static constexpr int kPre = 8;                   // stages of codes held in registers ahead of use
static constexpr int kPreA = 4;                  // stages of activations held ahead of use
static constexpr uint32_t kSpinLimit = 1u << 22;
static constexpr uint32_t kMaxKc = 2048;

__device__ int g_tc_error;                       // nonzero: a bounded wait ran out

static constexpr uint32_t kABytes = kStageRows * 128 * 2;          // 16 KB: 64 k x 128 n halfs
static constexpr uint32_t kA_SBO = 128, kA_LBO = 16 * 128;        // n-block stride, k-block stride
static constexpr uint32_t kZBytes = kStageRows * 16;               // 1 KB: 64 k-rows of {z, 0 x 7}
static constexpr uint32_t kB_SBO = 128;                           // m-block stride; k-block stride = mblocks*128

__host__ __device__ constexpr uint32_t b_bytes(int nmma) { return (uint32_t)nmma * kStageRows * 2; }
__host__ __device__ constexpr uint32_t stage_bytes(int nmma) { return kABytes + kZBytes + b_bytes(nmma); }
__host__ __device__ constexpr size_t tc_smem(int nmma, uint32_t kc)
{
    return (size_t)kDepth * stage_bytes(nmma) + (size_t)kc * 4 + (size_t)nmma * 4 + 64;
}

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
    for (uint32_t i = 0; i < kSpinLimit; i++) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\t"
                     "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
    }
    atomicExch(&g_tc_error, 1);
    return false;
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

// grid = (N / 128, K splits).  NMMA = activation rows per pass, a multiple of 16 up to 256.
template <int NMMA>
__global__ void __launch_bounds__(kTcThreads)
int4_tc_kernel(const float *__restrict__ a, const uint4 *__restrict__ bq,
               const __half *__restrict__ bs, const __half *__restrict__ bz,
               float *__restrict__ dst, uint32_t M, uint32_t N, uint32_t K, uint32_t kc,
               uint32_t m0, uint32_t mrows)
{
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr uint32_t kStage = stage_bytes(NMMA);
    constexpr uint32_t kB_LBO = (NMMA / 8) * 128;
    constexpr int kRowsPerThread = NMMA / 16;            // 8-element rows of a' per thread per stage
    constexpr bool kPrefetchA = kRowsPerThread <= 2;     // larger batches load a' inside the stage
    __half *ssc = reinterpret_cast<__half *>(smem + kDepth * kStage);   // [kc] scale, -1 where it was 0
    __half *szr = ssc + kc;                                              // [kc] zero
    float *corr = reinterpret_cast<float *>(szr + kc);                   // [NMMA]
    uint64_t *bars = reinterpret_cast<uint64_t *>(corr + NMMA);          // [kDepth] stage free, [1] done
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + kDepth + 1);
    __shared__ int s_abort;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t g = blockIdx.x, gpr = N / kGroup;
    const uint32_t kbeg = blockIdx.y * kc, kend = min(K, kbeg + kc);
    const uint32_t nrows = kend - kbeg, nstages = (nrows + kStageRows - 1) / kStageRows;
    const size_t row_u4 = N / 32;                                        // uint4 per row of codes

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i <= kDepth; i++) mbar_init(&bars[i], 1);
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // TMEM: NMMA columns for the product and NMMA for the zero-point term (a power of two >= 32)
    constexpr uint32_t kCols = 2 * NMMA <= 32 ? 32 : (2 * NMMA <= 64 ? 64 : (2 * NMMA <= 128 ? 128 : (2 * NMMA <= 256 ? 256 : 512)));
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(kCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }

    // This thread's two uint4 of every stage: rows j*32 + 8*warp + lane%8, 32-column chunk lane/8.
    // A quarter-warp stores eight consecutive k-rows of one core matrix: 128 contiguous bytes.
    const int crow = 8 * warp + (lane & 7), cchunk = lane >> 3;
    const uint4 *cbase = bq + (size_t)kbeg * row_u4 + g * 4 + cchunk;
    auto load_codes = [&](uint32_t st, int j) -> uint4 {
        const uint32_t r = st * kStageRows + j * 32 + crow;
        return r < nrows ? ldg_codes(cbase + (size_t)r * row_u4) : make_uint4(0, 0, 0, 0);
    };
    // a' rows of this thread: element e = tid + 128*i -> activation row e % NMMA, k-block e / NMMA
    auto load_act = [&](uint32_t st, int i, float4 &x0, float4 &x1) {
        const int e = tid + kTcThreads * i, m = e % NMMA, kb = e / NMMA;
        const uint32_t kloc = st * kStageRows + kb * 8;
        if ((uint32_t)m < mrows && kloc < nrows) {
            const float *ap = a + (size_t)(m0 + m) * K + kbeg + kloc;
            x0 = __ldg(reinterpret_cast<const float4 *>(ap));
            x1 = __ldg(reinterpret_cast<const float4 *>(ap + 4));
        } else {
            x0 = x1 = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    uint4 pre[kPre][2];
    float4 prea[kPreA][kPrefetchA ? kRowsPerThread : 1][2];
#pragma unroll
    for (int p = 0; p < kPre; p++) {
        pre[p][0] = load_codes(p, 0);
        pre[p][1] = load_codes(p, 1);
    }
    if (kPrefetchA) {
#pragma unroll
        for (int p = 0; p < kPreA; p++)
#pragma unroll
            for (int i = 0; i < kRowsPerThread; i++) load_act(p, i, prea[p][i][0], prea[p][i][1]);
    }
    // the group's scale and zero for every row of the K range; a zero scale becomes -1.  All the
    // loads are issued before the first store, so the prologue pays one memory round trip.
    {
        constexpr int kIters = kMaxKc / kTcThreads;
        __half sv[kIters], zv[kIters];
#pragma unroll
        for (int i = 0; i < kIters; i++) {
            const uint32_t r = tid + i * kTcThreads;
            if (r < nrows) {
                const size_t gi = (size_t)(kbeg + r) * gpr + g;
                sv[i] = __ldg(bs + gi);
                zv[i] = __ldg(bz + gi);
            }
        }
#pragma unroll
        for (int i = 0; i < kIters; i++) {
            const uint32_t r = tid + i * kTcThreads;
            if (r < nrows) {
                ssc[r] = __heq(sv[i], __float2half(0.f)) ? __float2half(-1.f) : sv[i];
                szr[r] = zv[i];
            }
        }
    }
    for (uint32_t r = nrows + tid; r < nstages * kStageRows; r += kTcThreads) {
        ssc[r] = __float2half(0.f);
        szr[r] = __float2half(0.f);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    constexpr uint32_t idesc = (1u << 4) | (1u << 15) | ((uint32_t)(NMMA >> 3) << 17) | ((128u >> 4) << 24);
    bool alive = true;

    for (uint32_t st0 = 0; st0 < nstages; st0 += kPre) {
#pragma unroll
        for (int pp = 0; pp < kPre; pp++) {
            const uint32_t st = st0 + pp;
            if (st >= nstages) break;                    // uniform across the CTA
            const uint32_t buf = st % kDepth, use = st / kDepth;
            // the MMAs that last read this buffer (stage st - kDepth) must have completed
            if (use > 0 && alive) {
                if (!mbar_wait(&bars[buf], (use - 1) & 1)) s_abort = 1;
            }
            alive = alive && !s_abort;
            unsigned char *At = smem + buf * kStage, *Zt = At + kABytes, *Bt = Zt + kZBytes;
            if (alive) {
                // weights: 2 x (four words -> four 16-byte rows of four adjacent core matrices);
                // a row whose scale was zero holds the constant z: its codes are dropped
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    uint4 cw = pre[pp][j];
                    const int r = j * 32 + crow;
                    if (__heq(ssc[st * kStageRows + r], __float2half(-1.f))) cw = make_uint4(0, 0, 0, 0);
                    unsigned char *dstp = At + (r >> 3) * kA_LBO + (r & 7) * 16 + (cchunk * 4) * kA_SBO;
                    *reinterpret_cast<uint4 *>(dstp) = expand(cw.x);
                    *reinterpret_cast<uint4 *>(dstp + kA_SBO) = expand(cw.y);
                    *reinterpret_cast<uint4 *>(dstp + 2 * kA_SBO) = expand(cw.z);
                    *reinterpret_cast<uint4 *>(dstp + 3 * kA_SBO) = expand(cw.w);
                    pre[pp][j] = load_codes(st + kPre, j);
                }
                // the zeros as a one-column weight operand: k-row r holds {z[r], 0 x 7}
                if (tid < kStageRows) {
                    const uint32_t zbits = __half_as_ushort(szr[st * kStageRows + tid]);
                    *reinterpret_cast<uint4 *>(Zt + tid * 16) = make_uint4(zbits, 0, 0, 0);
                }
                // activations: a' = a*s as f16, eight consecutive k per 16-byte row of a K-major
                // core matrix
#pragma unroll
                for (int i = 0; i < kRowsPerThread; i++) {
                    const int e = tid + kTcThreads * i, m = e % NMMA, kb = e / NMMA;
                    float4 x0, x1;
                    if (kPrefetchA) { x0 = prea[pp % kPreA][i][0]; x1 = prea[pp % kPreA][i][1]; }
                    else load_act(st, i, x0, x1);
                    const uint4 s8 = *reinterpret_cast<const uint4 *>(ssc + st * kStageRows + kb * 8);
                    const float2 s01 = __half22float2(*reinterpret_cast<const __half2 *>(&s8.x));
                    const float2 s23 = __half22float2(*reinterpret_cast<const __half2 *>(&s8.y));
                    const float2 s45 = __half22float2(*reinterpret_cast<const __half2 *>(&s8.z));
                    const float2 s67 = __half22float2(*reinterpret_cast<const __half2 *>(&s8.w));
                    const __half2 p0 = __floats2half2_rn(x0.x * s01.x, x0.y * s01.y);
                    const __half2 p1 = __floats2half2_rn(x0.z * s23.x, x0.w * s23.y);
                    const __half2 p2 = __floats2half2_rn(x1.x * s45.x, x1.y * s45.y);
                    const __half2 p3 = __floats2half2_rn(x1.z * s67.x, x1.w * s67.y);
                    *reinterpret_cast<uint4 *>(Bt + kb * kB_LBO + (m >> 3) * kB_SBO + (m & 7) * 16) =
                        make_uint4(*reinterpret_cast<const uint32_t *>(&p0), *reinterpret_cast<const uint32_t *>(&p1),
                                   *reinterpret_cast<const uint32_t *>(&p2), *reinterpret_cast<const uint32_t *>(&p3));
                    if (kPrefetchA) load_act(st + kPreA, i, prea[pp % kPreA][i][0], prea[pp % kPreA][i][1]);
                }
                // generic-proxy stores must be visible to the tensor core's (async-proxy) reads
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            __syncthreads();
            if (tid == 0 && alive) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int k16 = 0; k16 < kStageRows / 16; k16++) {
                    const uint32_t accum = (st > 0 || k16 > 0) ? 1u : 0u;
                    const uint64_t bdesc = make_desc(smem_u32(Bt) + k16 * 2 * kB_LBO, kB_LBO, kB_SBO);
                    umma_f16(tmem, make_desc(smem_u32(At) + k16 * 2 * kA_LBO, kA_LBO, kA_SBO), bdesc, idesc, accum);
                    // the zero-point term: every n-block aliases the one {z,0..} block (stride 0), so
                    // rows 0, 8, 16, ... of this accumulator all hold sum_k z[k] a'[m][k]
                    umma_f16(tmem + NMMA, make_desc(smem_u32(Zt) + k16 * 2 * 128, 128, 0), bdesc, idesc, accum);
                }
                // arrives on the stage's barrier once these MMAs have finished reading shared memory
                umma_commit(&bars[buf]);
                if (st + 1 == nstages) umma_commit(&bars[kDepth]);
            }
        }
    }

    // epilogue: wait for the last MMA, read the accumulators, undo the subnormal placement and the
    // column permutation of `expand`, subtract the zero-point term, write out (or the split's partial)
    if (alive && !mbar_wait(&bars[kDepth], 0)) s_abort = 1;
    __syncthreads();
    alive = alive && !s_abort;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (alive && warp == 0) {
        // lane 0 of the zero-point accumulator holds the term for every activation row
#pragma unroll
        for (int c0 = 0; c0 < NMMA; c0 += 16) {
            uint32_t r[16];
            tmem_ld16(tmem + NMMA + c0, r);
            if (lane == 0) {
#pragma unroll
                for (int i = 0; i < 16; i++) corr[c0 + i] = __uint_as_float(r[i]);
            }
        }
    }
    __syncthreads();
    if (alive) {
        const int L = 32 * warp + lane;                                  // TMEM lane = MMA row
        const int l8 = L & 7;
        const int col = (L & ~7) + ((l8 >> 1) | ((l8 & 1) << 2));        // 0,4,1,5,2,6,3,7
        const float f = (l8 & 2) ? 1048576.f : 16777216.f;              // rows 2,3,6,7 carried 2^-20
        float *o = dst + (size_t)blockIdx.y * M * N + (size_t)g * 128 + col;
#pragma unroll
        for (int c0 = 0; c0 < NMMA; c0 += 16) {
            uint32_t r[16];
            tmem_ld16(tmem + ((uint32_t)(32 * warp) << 16) + c0, r);
#pragma unroll
            for (int i = 0; i < 16; i++) {
                const uint32_t m = c0 + i;
                if (m < mrows) o[(size_t)(m0 + m) * N] = __uint_as_float(r[i]) * f - corr[m];
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kCols) : "memory");
}

Int4TcPlan plan_int4_tc(uint32_t M, uint32_t N, uint32_t K)
{
    Int4TcPlan p{};
    p.ok = N % kGroup == 0 && K % 16 == 0 && N > 0 && K > 0 && M >= 1;
    if (!p.ok) return p;
    p.groups = N / kGroup;
    p.nmma = M > 128 ? 256 : (M > 64 ? 128 : (M > 32 ? 64 : (M > 16 ? 32 : 16)));
    // K range per CTA: enough CTAs for every SM to hold several, but partial tiles (4*M bytes per
    // column per split) kept small against the codes (KC/2 bytes per column)
    const uint32_t mm = M < (uint32_t)p.nmma ? M : (uint32_t)p.nmma;
    uint32_t min_kc = 16 * mm < 256 ? 256 : 16 * mm;
    if (min_kc > kMaxKc) min_kc = kMaxKc;
    uint32_t want = (4u * (uint32_t)sm_count() + p.groups - 1) / p.groups;
    if (want < 1) want = 1;
    uint32_t kc = ((K + want - 1) / want + kStageRows - 1) / kStageRows * kStageRows;
    if (kc < min_kc) kc = min_kc;
    if (kc > kMaxKc) kc = kMaxKc;
    p.kc = kc;
    p.splits = (K + kc - 1) / kc;
    p.ws = p.splits > 1 ? (size_t)p.splits * M * N * sizeof(float) : 0;
    return p;
}

template <int NMMA>
static int launch_tc(const Launch &l, const Int4TcPlan &p, float *dst, uint32_t M, uint32_t N, uint32_t K)
{
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        int rc = check_cuda(cudaFuncSetAttribute(int4_tc_kernel<NMMA>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)tc_smem(NMMA, kMaxKc)), "int4_tc_kernel shared memory");
        if (rc) return rc;
        attr_set[dev] = true;
    }
    dim3 grid(p.groups, p.splits);
    for (uint32_t m0 = 0; m0 < M; m0 += NMMA) {
        int4_tc_kernel<NMMA><<<grid, kTcThreads, tc_smem(NMMA, p.kc), l.stream>>>(
            ptr<const float>(l, 0), ptr<const uint4>(l, 1), ptr<const __half>(l, 2),
            ptr<const __half>(l, 3), dst, M, N, K, p.kc, m0, min((uint32_t)NMMA, M - m0)); count_launch();
    }
    return AB_OK;
}

int run_int4_tc(const Launch &l, const Int4TcPlan &p, float *dst, uint32_t M, uint32_t N, uint32_t K)
{
    switch (p.nmma) {
    case 16: return launch_tc<16>(l, p, dst, M, N, K);
    case 32: return launch_tc<32>(l, p, dst, M, N, K);
    case 64: return launch_tc<64>(l, p, dst, M, N, K);
    case 128: return launch_tc<128>(l, p, dst, M, N, K);
    default: return launch_tc<256>(l, p, dst, M, N, K);
    }
}

int int4_tc_error_flag()
{
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_error, sizeof v) != cudaSuccess) { cudaGetLastError(); return -1; }
    return v;
}

}  // namespace ab
