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
// How the bytes move.  A CTA owns one 128-column group and 256 or 512 rows of K, small enough that
// EVERYTHING it will read is requested in its first few hundred cycles: every thread issues the
// cp.async copies of its own codes for all of its 16-row steps, the CTA copies its slice of the
// activations and the group's scales and zeros, and only then does anyone wait.  The eight warps
// take the steps in turn and are summed through shared memory; K splits are summed by the last
// CTA of the group to finish.  Many short CTAs that load at once keep far more bytes in flight
// per SM than a few long ones pacing themselves.
#include <cuda_fp16.h>

#include "common.cuh"

namespace ab {

static constexpr uint32_t kGroup = 128;
static constexpr int kMmaThreads = 256;          // 8 warps, all on one 128-column group
static constexpr int kMmaWarps = 8;
static constexpr int kMaxSpw = 4;                // 16-row steps per warp: K range = 128 * SPW rows
static constexpr uint32_t kMaxKc = 128 * kMaxSpw;

// shared memory: [ring: SPW x 32 B x 256 threads | activations: 16 rows x (kc*4 + 64) B | scales,
// zeros: kc halfs each]; the epilogue's [8 warps][16][128] f32 tile reuses it from the start
__host__ __device__ constexpr size_t ring_bytes(int spw) { return (size_t)spw * 32 * kMmaThreads; }
__host__ __device__ constexpr size_t act_stride(int spw) { return (size_t)128 * spw * 4 + 64; }
__host__ __device__ constexpr size_t act_bytes(int spw) { return 16 * act_stride(spw); }
static constexpr size_t kRedBytes = (size_t)kMmaWarps * 16 * 128 * 4 + kMmaWarps * 16 * 4;
static constexpr size_t mma_smem(int spw)
{
    size_t n = ring_bytes(spw) + act_bytes(spw) + (size_t)128 * spw * 4;
    return n > kRedBytes ? n : kRedBytes;
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

// Split-K partials are summed by the last CTA of each column group to finish: every CTA publishes
// its partial tile, bumps the group's counter, and the one that sees the final count adds the
// partials in split order (so the sum is deterministic) and resets the counter.  The counters
// start at zero when the module loads and are left at zero by every launch; launches that overlap
// on the device (two streams) would share them, so this kernel is for one stream at a time.
__device__ unsigned int g_mma_counters[1024];


// grid = (N / 128, K splits of 128*SPW rows).  Warp w takes the 16-row steps w, w+8, ... of the CTA's
// K range.  In a step, lane (gid = lane/4, t = lane%4) reads rows 4t .. 4t+3 of the 16 columns
// 16*gid .. 16*gid+15 of the group (the MMA's k index is a free relabelling, so rows {4t,4t+1}
// stand for its slots {2t,2t+1} and rows {4t+2,4t+3} for {2t+8,2t+9}); MMA j (j = 0..15) takes code
// j of each of those rows as its B fragment, so it covers columns {16*n + j : n = 0..7} and the
// thread ends up holding out[gid, gid+8][32t .. 32t+31].  A 17th MMA per step has the zeros as its
// B fragment and so accumulates the correction sum_k a'[m][k] z[k] from the very a' the others used.
template <int SPW>
__global__ void __launch_bounds__(kMmaThreads, 2)
int4_mma_kernel(const float *__restrict__ a, const uint2 *__restrict__ bq,
                const __half *__restrict__ bs, const __half *__restrict__ bz,
                float *__restrict__ part, float *__restrict__ out, uint32_t M, uint32_t N,
                uint32_t K, uint32_t m0, uint32_t mrows)
{
    constexpr uint32_t kc = 128 * SPW;
    constexpr size_t kRing = ring_bytes(SPW), kActStride = act_stride(SPW);
    extern __shared__ __align__(16) unsigned char smem[];
    unsigned char *acts = smem + kRing;                                  // [16][kc*4 + 64 B]
    __half *ssc = reinterpret_cast<__half *>(acts + act_bytes(SPW));    // [kc] scales
    __half *szr = ssc + kc;                                              // [kc] zeros
    __shared__ int s_last;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gid = lane >> 2, t = lane & 3;
    const uint32_t g = blockIdx.x, gpr = N / kGroup, splits = gridDim.y;
    const uint32_t kbeg = blockIdx.y * kc, kend = min(K, kbeg + kc);
    const uint32_t nrows = kend - kbeg, nsteps = nrows / 16;            // K % 16 == 0
    const size_t row_u2 = N / 16;                                        // uint2 per row of codes
    auto code_slot = [&](int it, int i) {
        return reinterpret_cast<uint2 *>(smem + (size_t)it * 32 * kMmaThreads) + i * kMmaThreads + tid;
    };

    // 1. the CTA's slice of the activations, a[m0 .. m0+15][kbeg .. kend): 16-byte chunks, rows past
    //    the batch zero-filled, each row padded by 64 B so that the fragment reads spread over banks
    {
        constexpr int chunks_per_row = kc / 4;
        for (int c = tid; c < 16 * chunks_per_row; c += kMmaThreads) {
            const int row = c / chunks_per_row, col = (c % chunks_per_row) * 4;
            const bool ok = (uint32_t)row < mrows && (uint32_t)col < nrows;
            cp_async<16>(acts + row * kActStride + col * 4,
                         a + (size_t)(m0 + (ok ? row : 0)) * K + kbeg + (ok ? col : 0), ok);
        }
        cp_async_commit();
    }
    // 2. every code this thread will use, one commit group per step
    {
        const uint2 *code_base = bq + (size_t)(kbeg + 4 * t) * row_u2 + g * 8 + gid;
#pragma unroll
        for (int it = 0; it < SPW; it++) {
            const uint32_t st = warp + it * kMmaWarps;
            const bool live = st < nsteps;
            const uint2 *src = code_base + (size_t)(live ? st * 16 : 0) * row_u2;
#pragma unroll
            for (int i = 0; i < 4; i++) cp_async<8>(code_slot(it, i), src + i * row_u2, live);
            cp_async_commit();
        }
    }
    // 3. the group's scale and zero for every row of the K range
    for (uint32_t r = tid; r < nrows; r += kMmaThreads) {
        const size_t gi = (size_t)(kbeg + r) * gpr + g;
        ssc[r] = __ldg(bs + gi);
        szr[r] = __ldg(bz + gi);
    }
    cp_async_wait<SPW>();                        // the activations have landed
    __syncthreads();

    float acc[16][4], accz[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 16; j++) { acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f; }

#pragma unroll
    for (int it = 0; it < SPW; it++) {
        const uint32_t st = warp + it * kMmaWarps;
        if (st >= nsteps) break;
        if (it == 0) cp_async_wait<SPW - 1>();
        else if (it == 1) cp_async_wait<(SPW > 2 ? SPW - 2 : 0)>();
        else if (it == 2) cp_async_wait<(SPW > 3 ? SPW - 3 : 0)>();
        else cp_async_wait<0>();
        uint2 cw[4];
#pragma unroll
        for (int i = 0; i < 4; i++) cw[i] = *code_slot(it, i);
        const float4 av[2] = {
            *reinterpret_cast<const float4 *>(acts + gid * kActStride + (st * 16 + 4 * t) * 4),
            *reinterpret_cast<const float4 *>(acts + (gid + 8) * kActStride + (st * 16 + 4 * t) * 4)};
        const uint2 s4 = *reinterpret_cast<const uint2 *>(ssc + st * 16 + 4 * t);     // s[4t..4t+3]
        const uint2 z4 = *reinterpret_cast<const uint2 *>(szr + st * 16 + 4 * t);     // z[4t..4t+3]
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
    __syncthreads();                             // every warp is done with the ring and the scales

    float *red = reinterpret_cast<float *>(smem);                        // [8 warps][16 rows][128]
    float *corr = red + kMmaWarps * 16 * 128;                            // [8 warps][16]
    // every column of the correction tile holds the same sum: c0 is row gid, c2 row gid+8
    if (t == 0) { corr[warp * 16 + gid] = accz[0]; corr[warp * 16 + gid + 8] = accz[2]; }
    // Column c of row r lives at r*128 + 32*(c/32) + ((c%32 + 4*(r%8) + c/32) % 32), which puts the
    // 32 lanes of each store on 32 different banks.
    float *mine = red + warp * 16 * 128;
    const int rot = 4 * gid + t;
#pragma unroll
    for (int j = 0; j < 16; j++) {
        const int p0 = 32 * t + ((j + rot) & 31), p1 = 32 * t + ((j + 16 + rot) & 31);
        mine[gid * 128 + p0] = acc[j][0];                      // n-slot 2t   -> column 32t + j
        mine[gid * 128 + p1] = acc[j][1];                      // n-slot 2t+1 -> column 32t + 16 + j
        mine[(gid + 8) * 128 + p0] = acc[j][2];
        mine[(gid + 8) * 128 + p1] = acc[j][3];
    }
    __syncthreads();
    // 2048 outputs, 8 per thread: element e = i*256 + tid -> row e/128, column e%128 (coalesced).
    // The subnormal placement is undone here: even codes carried 2^-24, odd codes 2^-20.
    float *dst = splits > 1 ? part + (size_t)blockIdx.y * M * N : out;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int e = i * kMmaThreads + tid, row = e >> 7, col = e & 127;
        if ((uint32_t)row >= mrows) continue;
        const int phys = row * 128 + (col & ~31) + (((col & 31) + 4 * (row & 7) + (col >> 5)) & 31);
        float v = 0.f, cz = 0.f;
#pragma unroll
        for (int w = 0; w < kMmaWarps; w++) { v += red[w * 16 * 128 + phys]; cz += corr[w * 16 + row]; }
        dst[(size_t)(m0 + row) * N + (size_t)g * 128 + col] = v * ((col & 1) ? 1048576.f : 16777216.f) - cz;
    }
    if (splits == 1) return;

    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned int prev = atomicAdd(&g_mma_counters[g % 1024], 1u);
        s_last = prev == splits - 1;
        if (s_last) g_mma_counters[g % 1024] = 0;               // left at zero for the next launch
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int e = i * kMmaThreads + tid, row = e >> 7, col = e & 127;
        if ((uint32_t)row >= mrows) continue;
        const size_t o = (size_t)(m0 + row) * N + (size_t)g * 128 + col;
        float v = 0.f;
        for (uint32_t sp = 0; sp < splits; sp++) v += __ldcg(part + (size_t)sp * M * N + o);
        out[o] = v;
    }
}

Int4MmaPlan plan_int4_mma(uint32_t M, uint32_t N, uint32_t K)
{
    Int4MmaPlan p{};
    p.ok = N % kGroup == 0 && K % 16 == 0 && N > 0 && K > 0 && N / kGroup <= 1024;
    if (!p.ok) return p;
    p.groups = N / kGroup;
    // 512-row CTAs unless that leaves the machine short of work, then 256
    const uint32_t slots = 2u * (uint32_t)sm_count();
    p.kc = (p.groups * ((K + 511) / 512) >= 2 * slots || K <= 256) ? 512 : 256;
    if (K <= 256) p.kc = 256;
    p.splits = (K + p.kc - 1) / p.kc;
    p.ws = p.splits > 1 ? (size_t)p.splits * M * N * sizeof(float) : 0;
    return p;
}

template <int SPW>
static int launch_mma(const Launch &l, const Int4MmaPlan &p, float *part, float *out, uint32_t M,
                      uint32_t N, uint32_t K)
{
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        int rc = check_cuda(cudaFuncSetAttribute(int4_mma_kernel<SPW>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)mma_smem(SPW)), "int4_mma_kernel shared memory");
        if (rc) return rc;
        attr_set[dev] = true;
    }
    dim3 grid(p.groups, p.splits);
    for (uint32_t m0 = 0; m0 < M; m0 += 16) {
        int4_mma_kernel<SPW><<<grid, kMmaThreads, mma_smem(SPW), l.stream>>>(
            ptr<const float>(l, 0), ptr<const uint2>(l, 1), ptr<const __half>(l, 2),
            ptr<const __half>(l, 3), part, out, M, N, K, m0, min(16u, M - m0)); count_launch();
    }
    return AB_OK;
}

int run_int4_mma(const Launch &l, const Int4MmaPlan &p, float *part, float *out, uint32_t M, uint32_t N,
                 uint32_t K)
{
    return p.kc == 512 ? launch_mma<4>(l, p, part, out, M, N, K) : launch_mma<2>(l, p, part, out, M, N, K);
}

}  // namespace ab
