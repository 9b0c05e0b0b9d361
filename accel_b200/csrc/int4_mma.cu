// int4 linear for a handful of activation rows (the decode batch): weights streamed once from HBM,
// dequantised in registers, contracted on the tensor cores with f32 accumulation.
//
// Why tensor cores at M = 2..64.  At HBM speed a B200 delivers about 12 T int4 weights per second and
// issues about 36 T thread-instructions per second, so a kernel has under three instructions per
// weight.  A CUDA-core FMA per weight AND per activation row cannot fit for more than one or two
// rows; one warp-level MMA covers 128 weights x 16 rows in a single instruction.
//
// What is fed to the MMA.  With N a multiple of 128 a quantisation group is 128 adjacent columns of
// one row k, so inside a 128-column tile the scale s[k] and zero z[k] depend on k only and
//
//   out[m][n] = sum_k (a[m][k] s[k]) code[k][n]  -  sum_k (a[m][k] s[k]) z[k]
//
// The first sum is the MMA: the A operand is a' = a*s rounded to f16, the B operand is the 4-bit
// code itself.  A code masked in place into the mantissa of an f16 with a zero exponent IS the f16
// subnormal code * 2^-24 (or 2^-20 for the next nibble), exactly, so dequantising a pair of codes
// is one AND; the power of two is undone per column in the epilogue.  The second sum is one more
// MMA whose B operand is z (an f16 already), over the SAME rounded a' the others saw, so the two
// sums cancel as they do in exact arithmetic and only one operand (a') is ever rounded: the result
// carries a relative error of 2^-11 per term, against the 1e-3 the path allows.  A group with
// s == 0 is the constant z (internal/kernels/int4.go:85-87): a' = 0 and the second sum takes -a*z.
//
// How the bytes move.  A CTA is four warps, each owning one 128-column group of a 512-column tile,
// all walking the same KC rows of K.  The activations a[0..15][k range] and the four groups' scales
// and zeros are staged once in shared memory and shared by the warps; each thread keeps a private
// ring of cp.async copies of its own codes, eight 16-row steps deep, so the loop has no barrier.
// A warp owns its output columns outright, so nothing is reduced across warps: the accumulators
// go from registers to global memory.  K is split across CTAs only; the partial sums of the
// splits are added by a second, fully parallel kernel.
#include <cuda_fp16.h>

#include <cstdlib>

#include "common.cuh"

namespace ab {

static constexpr uint32_t kGroup = 128;
static constexpr int kMmaWarps = 4;              // one 128-column group each
static constexpr int kMmaThreads = 32 * kMmaWarps;
static constexpr int kDepth = 8;                 // 16-row steps of code copies in flight per thread

// shared memory: [ring: kDepth x 32 B x threads | activations: 16 rows x (KC*4 + 64) B |
//                 scales: 4 x KC halfs | zeros: 4 x KC halfs]
__host__ __device__ constexpr size_t ring_bytes() { return (size_t)kDepth * 32 * kMmaThreads; }
__host__ __device__ constexpr size_t act_stride(int kc) { return (size_t)kc * 4 + 64; }
__host__ __device__ constexpr size_t mma_smem(int kc)
{
    return ring_bytes() + 16 * act_stride(kc) + (size_t)2 * kMmaWarps * kc * 2;
}

template <int BYTES>
__device__ __forceinline__ void cp_async(void *smem, const void *gmem, bool valid)
{
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem);
    const int n = valid ? BYTES : 0;             // 0 source bytes: the destination is zero-filled
    asm volatile("cp.async.ca.shared.global [%0], [%1], %2, %3;" ::"r"(dst), "l"(gmem), "n"(BYTES), "r"(n)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait()
{
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
                 "{%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// grid = (ceil(N / 512), ceil(K / KC)).  In a 16-row step, lane (gid = lane/4, t = lane%4) reads rows
// 4t .. 4t+3 of the 16 columns 16*gid .. 16*gid+15 of its warp's group (the MMA's k index is a free
// relabelling, so rows {4t,4t+1} stand for its slots {2t,2t+1} and rows {4t+2,4t+3} for
// {2t+8,2t+9}); MMA j (j = 0..15) takes code j of each of those rows as its B fragment, so it
// covers columns {16*n + j : n = 0..7} and the thread ends up holding out[gid, gid+8][32t .. 32t+31].
// A 17th MMA per step has the zeros as its B fragment and so accumulates the correction
// sum_k a'[m][k] z[k] from the very a' the others used.
template <int KC>
__global__ void __launch_bounds__(kMmaThreads, 4)
int4_mma_kernel(const float *__restrict__ a, const uint2 *__restrict__ bq,
                const __half *__restrict__ bs, const __half *__restrict__ bz,
                float *__restrict__ dst, uint32_t M, uint32_t N, uint32_t K, uint32_t m0,
                uint32_t mrows)
{
    constexpr size_t kActStride = act_stride(KC);
    extern __shared__ __align__(16) unsigned char smem[];
    unsigned char *acts = smem + ring_bytes();                           // [16][KC*4 + 64 B]
    __half *ssc = reinterpret_cast<__half *>(acts + 16 * kActStride);   // [4][KC] scales
    __half *szr = ssc + kMmaWarps * KC;                                  // [4][KC] zeros
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gid = lane >> 2, t = lane & 3;
    const uint32_t gpr = N / kGroup, g0 = blockIdx.x * kMmaWarps, g = g0 + warp;
    const bool warp_on = g < gpr;
    const uint32_t kbeg = blockIdx.y * KC, kend = min(K, kbeg + KC);
    const uint32_t nrows = kend - kbeg, nsteps = nrows / 16;            // K % 16 == 0
    const size_t row_u2 = N / 16;                                        // uint2 per row of codes
    auto code_slot = [&](uint32_t st, int i) {
        return reinterpret_cast<uint2 *>(smem + (size_t)(st % kDepth) * 32 * kMmaThreads) + i * kMmaThreads + tid;
    };
    const uint2 *code_base = bq + (size_t)(kbeg + 4 * t) * row_u2 + (warp_on ? g : g0) * 8 + gid;
    auto issue = [&](uint32_t st) {
        const bool live = st < nsteps && warp_on;
        const uint2 *src = code_base + (size_t)(live ? st * 16 : 0) * row_u2;
#pragma unroll
        for (int i = 0; i < 4; i++) cp_async<8>(code_slot(st, i), src + i * row_u2, live);
    };

    // 1. the CTA's slice of the activations, a[m0 .. m0+15][kbeg .. kend): 16-byte chunks, rows past
    //    the batch zero-filled, each row padded by 64 B so that the fragment reads spread over banks
    {
        constexpr int chunks_per_row = KC / 4;
        for (int c = tid; c < 16 * chunks_per_row; c += kMmaThreads) {
            const int row = c / chunks_per_row, col = (c % chunks_per_row) * 4;
            const bool ok = (uint32_t)row < mrows && (uint32_t)col < nrows;
            cp_async<16>(acts + row * kActStride + col * 4,
                         a + (size_t)(m0 + (ok ? row : 0)) * K + kbeg + (ok ? col : 0), ok);
        }
        cp_async_commit();
    }
    // 2. the first kDepth steps of this thread's codes, one commit group per step
#pragma unroll
    for (int st = 0; st < kDepth; st++) { issue(st); cp_async_commit(); }
    // 3. the four groups' scale and zero for every row of the K range
    for (uint32_t i = tid; i < nrows * kMmaWarps; i += kMmaThreads) {
        const uint32_t r = i / kMmaWarps, w = i % kMmaWarps;
        if (g0 + w < gpr) {
            const size_t gi = (size_t)(kbeg + r) * gpr + g0 + w;
            ssc[w * KC + r] = __ldg(bs + gi);
            szr[w * KC + r] = __ldg(bz + gi);
        }
    }
    cp_async_wait<kDepth>();                     // the activations have landed
    __syncthreads();
    if (!warp_on) return;

    float acc[16][4], accz[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 16; j++) { acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f; }
    const __half *my_s = ssc + warp * KC + 4 * t, *my_z = szr + warp * KC + 4 * t;
    const unsigned char *a_lo = acts + gid * kActStride + 16 * t, *a_hi = a_lo + 8 * kActStride;

    for (uint32_t st = 0; st < nsteps; st++) {
        cp_async_wait<kDepth - 1>();             // step st's codes have landed
        uint2 cw[4];
#pragma unroll
        for (int i = 0; i < 4; i++) cw[i] = *code_slot(st, i);
        issue(st + kDepth);                      // refill the slot just read
        cp_async_commit();
        const float4 av[2] = {*reinterpret_cast<const float4 *>(a_lo + st * 64),
                              *reinterpret_cast<const float4 *>(a_hi + st * 64)};
        const uint2 s4 = *reinterpret_cast<const uint2 *>(my_s + st * 16);      // s[4t..4t+3]
        const uint2 z4 = *reinterpret_cast<const uint2 *>(my_z + st * 16);      // z[4t..4t+3]
        const float2 s01 = __half22float2(*reinterpret_cast<const __half2 *>(&s4.x));
        const float2 s23 = __half22float2(*reinterpret_cast<const __half2 *>(&s4.y));

        uint32_t af[4];          // a0: (gid, k 4t,4t+1)  a1: (gid+8, same)  a2: (gid, 4t+2,4t+3)  a3
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const __half2 p01 = __floats2half2_rn(av[h].x * s01.x, av[h].y * s01.y);
            const __half2 p23 = __floats2half2_rn(av[h].z * s23.x, av[h].w * s23.y);
            af[h] = *reinterpret_cast<const uint32_t *>(&p01);
            af[h + 2] = *reinterpret_cast<const uint32_t *>(&p23);
        }
        // correction: the zeros as a B fragment.  A row with s == 0 is the constant z: the main
        // MMAs see a' = 0 there, and the correction takes -a so that subtracting it adds a*z.
        const bool any_const = (s01.x == 0.f) | (s01.y == 0.f) | (s23.x == 0.f) | (s23.y == 0.f);
        if (__any_sync(0xffffffffu, any_const)) {
            uint32_t ac[4];
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const __half2 p01 = __floats2half2_rn(av[h].x * (s01.x == 0.f ? -1.f : s01.x),
                                                      av[h].y * (s01.y == 0.f ? -1.f : s01.y));
                const __half2 p23 = __floats2half2_rn(av[h].z * (s23.x == 0.f ? -1.f : s23.x),
                                                      av[h].w * (s23.y == 0.f ? -1.f : s23.y));
                ac[h] = *reinterpret_cast<const uint32_t *>(&p01);
                ac[h + 2] = *reinterpret_cast<const uint32_t *>(&p23);
            }
            mma16816(accz, ac, z4.x, z4.y);
        } else {
            mma16816(accz, af, z4.x, z4.y);
        }
#pragma unroll
        for (int c = 0; c < 2; c++) {
            const uint32_t w0 = c ? cw[0].y : cw[0].x, w1 = c ? cw[1].y : cw[1].x;
            const uint32_t w2 = c ? cw[2].y : cw[2].x, w3 = c ? cw[3].y : cw[3].x;
            // 16-bit lanes: low = row 4t (or 4t+2), high = row 4t+1 (or 4t+3)
            const uint32_t lo01 = __byte_perm(w0, w1, 0x5410), hi01 = __byte_perm(w0, w1, 0x7632);
            const uint32_t lo23 = __byte_perm(w2, w3, 0x5410), hi23 = __byte_perm(w2, w3, 0x7632);
            const uint32_t src01[4] = {lo01, lo01 >> 8, hi01, hi01 >> 8};
            const uint32_t src23[4] = {lo23, lo23 >> 8, hi23, hi23 >> 8};
#pragma unroll
            for (int p = 0; p < 4; p++) {
                // codes 2p and 2p+1 of this word, as f16 subnormals code*2^-24 and code*2^-20
                mma16816(acc[8 * c + 2 * p], af, src01[p] & 0x000F000Fu, src23[p] & 0x000F000Fu);
                mma16816(acc[8 * c + 2 * p + 1], af, src01[p] & 0x00F000F0u, src23[p] & 0x00F000F0u);
            }
        }
    }
    cp_async_wait<0>();

    // registers to global memory: the thread holds rows gid and gid+8, columns 32t .. 32t+31 of its
    // group (MMA j's n-slot 2t is column 32t+j, n-slot 2t+1 is column 32t+16+j).  The subnormal
    // placement is undone here (even codes carried 2^-24, odd codes 2^-20), and the correction,
    // of which every column of accz holds the same sum, is subtracted.
    float *o = dst + (size_t)blockIdx.y * M * N + (size_t)g * 128 + 32 * t;
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const uint32_t row = gid + 8 * h;
        if (row >= mrows) continue;
        const float cz = accz[2 * h];
        float *orow = o + (size_t)(m0 + row) * N;
#pragma unroll
        for (int half = 0; half < 2; half++)
#pragma unroll
            for (int j = 0; j < 16; j += 4) {
                float4 v;
                v.x = acc[j][2 * h + half] * 16777216.f - cz;
                v.y = acc[j + 1][2 * h + half] * 1048576.f - cz;
                v.z = acc[j + 2][2 * h + half] * 16777216.f - cz;
                v.w = acc[j + 3][2 * h + half] * 1048576.f - cz;
                *reinterpret_cast<float4 *>(orow + 16 * half + j) = v;
            }
    }
}

Int4MmaPlan plan_int4_mma(uint32_t M, uint32_t N, uint32_t K)
{
    Int4MmaPlan p{};
    p.ok = N % kGroup == 0 && K % 16 == 0 && N > 0 && K > 0;
    if (!p.ok) return p;
    p.groups = N / kGroup;
    const uint32_t tiles = (p.groups + kMmaWarps - 1) / kMmaWarps;
    // The longest K range per CTA that still gives every SM a few CTAs, but never so short that
    // the partial sums (splits x M x N floats, written and read back) outweigh the codes: a CTA's
    // partial tile is 4*M bytes per column against KC/2 bytes of codes.
    const uint32_t want = 3u * (uint32_t)sm_count();
    const uint32_t floor_kc = M > 8 ? 256 : 128;
    p.kc = 512;
    while (p.kc > floor_kc && tiles * ((K + p.kc - 1) / p.kc) < want) p.kc /= 2;
    p.splits = (K + p.kc - 1) / p.kc;
    p.ws = p.splits > 1 ? (size_t)p.splits * M * N * sizeof(float) : 0;
    return p;
}

template <int KC>
static int launch_mma(const Launch &l, const Int4MmaPlan &p, float *dst, uint32_t M, uint32_t N, uint32_t K)
{
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        int rc = check_cuda(cudaFuncSetAttribute(int4_mma_kernel<KC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)mma_smem(KC)), "int4_mma_kernel shared memory");
        if (rc) return rc;
        attr_set[dev] = true;
    }
    dim3 grid((p.groups + kMmaWarps - 1) / kMmaWarps, p.splits);
    for (uint32_t m0 = 0; m0 < M; m0 += 16) {
        int4_mma_kernel<KC><<<grid, kMmaThreads, mma_smem(KC), l.stream>>>(
            ptr<const float>(l, 0), ptr<const uint2>(l, 1), ptr<const __half>(l, 2),
            ptr<const __half>(l, 3), dst, M, N, K, m0, min(16u, M - m0)); count_launch();
    }
    return AB_OK;
}

// dst is `out` when the plan has one split, else the [splits][M][N] partials the caller sums
int run_int4_mma(const Launch &l, const Int4MmaPlan &p, float *dst, uint32_t M, uint32_t N, uint32_t K)
{
    if (p.kc == 512) return launch_mma<512>(l, p, dst, M, N, K);
    if (p.kc == 256) return launch_mma<256>(l, p, dst, M, N, K);
    return launch_mma<128>(l, p, dst, M, N, K);
}

}  // namespace ab
