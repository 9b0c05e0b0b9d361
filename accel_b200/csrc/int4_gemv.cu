// int4 matrix-vector product (QuantMatVecInt4, internal/kernels/int4.go:60) for one activation row:
// the decode shape at batch 1.  HBM-bound: every weight is used once, so the kernel is a streaming
// read of the codes with one FMA per weight.
//
//   out[n] = sum_k (a[k] s[k,g]) code[k,n]  -  sum_k (a[k] s[k,g]) z[k,g]       g = n / 128
//
// Per-weight work is what bounds a CUDA-core kernel here (about 45 M weights against 36 T
// thread-instructions per second), so the inner loop is two instructions per weight:
//   - one logic op turns TWO codes of a word into the f16 pair {16 + c, 16 + c'}: the codes are
//     shifted (one shift per four pairs) onto the top four mantissa bits of an f16 whose exponent
//     field says 16, so no conversion instruction exists;
//   - one mixed-precision FMA per code (f32 += f16 * f16, exact product) accumulates
//     (a s)_f16 * (16 + c) in f32.  The 16 and the zero point leave together:
//     out = acc - sum_k (a s)_f16 (16 + z), summed in f32 from the same rounded (a s).
// a*s is the only rounded operand (f16, relative error 2^-11 per term, against the 1e-3 the path
// allows).  A row of a group whose scale is 0 is the constant z (internal/kernels/int4.go:85-87):
// its (a s) is 0 and the correction takes -a z.
//
// Shape of the kernel.  Many small CTAs (128 threads) that issue all their loads up front: a CTA
// owns W column groups (W = 1 or 2; 64 W contiguous bytes of codes per row) and a K range; 4 W lanes
// cover a row with 128-bit loads, eight loads in flight per thread.  An SM serves its loads in
// order, so the small loads the CTA waits for first (activations, scales, zeros) are issued before
// the code loads.  The K splits of a column tile form a thread-block cluster: every CTA leaves its
// partial row in shared memory and the CTAs add them through distributed shared memory in rank
// order (deterministic), each writing its slice of the columns.  One kernel, no workspace.
#include <cooperative_groups.h>
#include <cuda_fp16.h>

#include <cstdlib>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace ab {

static constexpr uint32_t kGroup = 128;
static constexpr int kRowThreads = 128;
static constexpr int kRowUnroll = 8;
static constexpr uint32_t kRowMaxKc = 768;
static constexpr int kRowMaxCluster = 16;        // 16 needs the non-portable cluster size opt-in

__device__ __forceinline__ uint4 ldg_row(const uint4 *p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ uint32_t opaque(uint32_t v)
{   // keeps a constant in a register, so that (x & imm) | reg is ONE logic instruction
    uint32_t r;
    asm volatile("mov.u32 %0, %1;" : "=r"(r) : "r"(v));
    return r;
}
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c)
{
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// lo += f16(x.lo) * cs, hi += f16(x.hi) * cs, products exact, sums in f32
__device__ __forceinline__ void fma_pair(uint32_t x, unsigned short cs, float &lo, float &hi)
{
    asm("{ .reg .b16 l, h; mov.b32 {l, h}, %2; fma.rn.f32.f16 %0, l, %3, %0; fma.rn.f32.f16 %1, h, %3, %1; }"
        : "+f"(lo), "+f"(hi) : "r"(x), "h"(cs));
}
// eight codes of a word: code i and code i+4 come out of one logic op as the f16 pair
// {16 + code i, 16 + code i+4} (codes on mantissa bits 6..9, exponent field 19)
__device__ __forceinline__ void fma_word(uint32_t w, unsigned short cs, uint32_t magic, float *acc)
{
    fma_pair(and_or(w << 6, 0x03C003C0u, magic), cs, acc[0], acc[4]);
    fma_pair(and_or(w << 2, 0x03C003C0u, magic), cs, acc[1], acc[5]);
    fma_pair(and_or(w >> 2, 0x03C003C0u, magic), cs, acc[2], acc[6]);
    fma_pair(and_or(w >> 6, 0x03C003C0u, magic), cs, acc[3], acc[7]);
}

// grid = (ceil(N / 128 / W), K splits), cluster = (1, splits, 1).
template <int W>
__global__ void __launch_bounds__(kRowThreads)
int4_row_kernel(const float *__restrict__ a, const uint4 *__restrict__ bq, const __half *__restrict__ bs,
                const __half *__restrict__ bz, float *__restrict__ out, uint32_t N, uint32_t K, uint32_t kc)
{
    constexpr int kLanes = 4 * W;                          // lanes per row (16 bytes = 32 columns each)
    constexpr int kRowsPerInstr = kRowThreads / kLanes;    // rows per CTA-wide load
    constexpr int kCols = 128 * W;
    constexpr int kMetaIt = kRowMaxKc / kRowThreads;
    __shared__ unsigned short s_cs[W][kRowMaxKc];          // f16(a s) per group and row of the K range
    __shared__ float s_zw[W][kRowThreads / 32];            // per-warp parts of the correction
    __shared__ float s_zc[W];                              // sum_k (a s)_f16 (16 + z): subtracted at the end
    __shared__ uint32_t s_amax[kRowThreads / 32];          // the warps' largest |a| of the K range (bits)
    __shared__ __align__(16) float s_red[kRowsPerInstr][kCols];
    __shared__ __align__(16) float s_sum[kCols];           // this CTA's partial row, read by the cluster
    const int tid = threadIdx.x, rl = tid / kLanes, c = tid % kLanes;
    const uint32_t gpr = N / kGroup, g0 = blockIdx.x * W, splits = gridDim.y;
    const uint32_t col0 = g0 * kGroup + c * 32;
    const bool col_on = col0 < N;
    const uint32_t kbeg = blockIdx.y * kc, kend = min(K, kbeg + kc), nrows = kend > kbeg ? kend - kbeg : 0;
    const size_t row_u4 = N / 32;
    const uint4 *base = bq + (size_t)kbeg * row_u4 + (col_on ? col0 / 32 : 0);

    // 1. activations, scales and zeros first, then the first batch of codes
    float av[kMetaIt];
    uint32_t sv[kMetaIt], zv[kMetaIt];
    const bool paired = W == 2 && gpr % 2 == 0;            // both groups' values in one 4-byte load
#pragma unroll
    for (int i = 0; i < kMetaIt; i++) {
        const uint32_t r = tid + i * kRowThreads;
        av[i] = 0.f; sv[i] = zv[i] = 0;
        if (r < nrows) {
            av[i] = __ldg(a + kbeg + r);
            const size_t at = (size_t)(kbeg + r) * gpr + g0;
            if (paired) {
                sv[i] = __ldg(reinterpret_cast<const uint32_t *>(bs + at));
                zv[i] = __ldg(reinterpret_cast<const uint32_t *>(bz + at));
            } else {
                sv[i] = __ldg(reinterpret_cast<const unsigned short *>(bs + at));
                zv[i] = __ldg(reinterpret_cast<const unsigned short *>(bz + at));
                if (W == 2 && g0 + 1 < gpr) {
                    sv[i] |= (uint32_t)__ldg(reinterpret_cast<const unsigned short *>(bs + at + 1)) << 16;
                    zv[i] |= (uint32_t)__ldg(reinterpret_cast<const unsigned short *>(bz + at + 1)) << 16;
                }
            }
        }
    }
    uint4 cw[kRowUnroll];
#pragma unroll
    for (int u = 0; u < kRowUnroll; u++) {
        const uint32_t r = rl + u * kRowsPerInstr;
        cw[u] = (col_on && r < nrows) ? ldg_row(base + (size_t)r * row_u4) : make_uint4(0, 0, 0, 0);
    }
    // The activations of this K range times an exact power of two that puts the largest of them in
    // [2^8, 2^9): a * s then stays a normal f16 whatever the activations' magnitude.  Undone when the
    // CTA's sums leave (every CTA of a cluster has its own factor).
    {
        uint32_t mx = 0;
#pragma unroll
        for (int i = 0; i < kMetaIt; i++) mx = max(mx, __float_as_uint(fabsf(av[i])));
        mx = __reduce_max_sync(0xffffffffu, mx);
        if ((tid & 31) == 0) s_amax[tid >> 5] = mx;
    }
    __syncthreads();
    const int ea = ab_row_exponent(max(max(s_amax[0], s_amax[1]), max(s_amax[2], s_amax[3])));
    const float pa = ab_pow2(8 - ea), unscale = ab_pow2(ea - 8);
#pragma unroll
    for (int i = 0; i < kMetaIt; i++) av[i] *= pa;
    // f16(a s) once per (row, group), not once per thread that uses it; the correction
    // sum_k (a s)_f16 (16 + z) (or -a z where the scale is 0) is summed here too, in a fixed order
    {
        float zpart[W];
#pragma unroll
        for (int w = 0; w < W; w++) zpart[w] = 0.f;
#pragma unroll
        for (int i = 0; i < kMetaIt; i++) {
            const uint32_t r = tid + i * kRowThreads;
            if (r < nrows) {
#pragma unroll
                for (int w = 0; w < W; w++) {
                    const float sc = __half2float(__ushort_as_half((unsigned short)(sv[i] >> (16 * w))));
                    const float zr = __half2float(__ushort_as_half((unsigned short)(zv[i] >> (16 * w))));
                    const __half csh = __float2half_rn(av[i] * sc);
                    s_cs[w][r] = __half_as_ushort(csh);
                    zpart[w] = sc == 0.f ? fmaf(-av[i], zr, zpart[w]) : fmaf(__half2float(csh), 16.f + zr, zpart[w]);
                }
            }
        }
#pragma unroll
        for (int w = 0; w < W; w++) {
#pragma unroll
            for (int sh = 16; sh > 0; sh >>= 1) zpart[w] += __shfl_xor_sync(0xffffffffu, zpart[w], sh);
            if ((tid & 31) == 0) s_zw[w][tid >> 5] = zpart[w];
        }
    }
    __syncthreads();
    if (tid < W) s_zc[tid] = (s_zw[tid][0] + s_zw[tid][1]) + (s_zw[tid][2] + s_zw[tid][3]);

    // 2. the loop: two register batches used in turn; a batch's loads go out before the other is used
    float acc[32];
#pragma unroll
    for (int i = 0; i < 32; i++) acc[i] = 0.f;
    const int grp = c >> 2;                                  // which of the tile's groups
    const uint32_t magic = opaque(0x4C004C00u);
    constexpr uint32_t kStep = kRowsPerInstr * kRowUnroll;
    auto fetch = [&](uint4 (&dst)[kRowUnroll], uint32_t r0) {
#pragma unroll
        for (int u = 0; u < kRowUnroll; u++) {
            const uint32_t r = r0 + rl + u * kRowsPerInstr;
            dst[u] = (col_on && r < nrows) ? ldg_row(base + (size_t)r * row_u4) : make_uint4(0, 0, 0, 0);
        }
    };
    auto consume = [&](const uint4 (&src)[kRowUnroll], uint32_t r0) {
#pragma unroll
        for (int u = 0; u < kRowUnroll; u++) {
            const uint32_t r = r0 + rl + u * kRowsPerInstr;
            if (r < nrows) {
                const unsigned short cs = s_cs[grp][r];
                fma_word(src[u].x, cs, magic, acc);
                fma_word(src[u].y, cs, magic, acc + 8);
                fma_word(src[u].z, cs, magic, acc + 16);
                fma_word(src[u].w, cs, magic, acc + 24);
            }
        }
    };
    uint4 cw2[kRowUnroll];
    for (uint32_t r0 = 0; r0 < nrows; r0 += 2 * kStep) {
        fetch(cw2, r0 + kStep);
        consume(cw, r0);
        fetch(cw, r0 + 2 * kStep);
        consume(cw2, r0 + kStep);
    }

    // 3. the row-lanes hold partial sums of the same columns: through shared memory (each 16-byte
    //    store rotated inside its 32-column block, so that the lanes of a row hit different banks)
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
        const float4 v = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
        *reinterpret_cast<float4 *>(&s_red[rl][c * 32 + ((j + 4 * c) & 31)]) = v;
    }
    __syncthreads();
    for (int col = tid; col < kCols; col += kRowThreads) {
        const int at = (col & ~31) | ((col + 4 * (col >> 5)) & 31);
        float v = 0.f;
#pragma unroll
        for (int i = 0; i < kRowsPerInstr; i++) v += s_red[i][at];
        v = (v - s_zc[col >> 7]) * unscale;
        if (splits == 1) {
            if (g0 * kGroup + col < N) out[g0 * kGroup + col] = v;
        } else {
            s_sum[col] = v;
        }
    }
    if (splits == 1) return;

    // 4. the K splits: rank r of the cluster adds a slice of the columns over every CTA's row
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    const uint32_t rank = cluster.block_rank();
    const uint32_t per = (kCols + splits - 1) / splits;
    const uint32_t col = rank * per + tid;
    if ((uint32_t)tid < per && col < (uint32_t)kCols) {
        float pv[kRowMaxCluster];
#pragma unroll
        for (int q = 0; q < kRowMaxCluster; q++)
            pv[q] = (uint32_t)q < splits ? *cluster.map_shared_rank(&s_sum[col], q) : 0.f;
        float v = pv[0];
#pragma unroll
        for (int q = 1; q < kRowMaxCluster; q++) v += pv[q];
        if (g0 * kGroup + col < N) out[g0 * kGroup + col] = v;
    }
    cluster.sync();                              // nobody leaves while its row is being read
}

Int4RowPlan plan_int4_row(uint32_t N, uint32_t K)
{
    Int4RowPlan p{};
    p.ok = N % kGroup == 0 && N > 0 && K > 0;
    if (!p.ok) return p;
    const uint32_t gpr = N / kGroup, sms = (uint32_t)sm_count();
    // measured: about two CTAs per SM and clusters of at most eight do best; two groups per tile
    // for wide matrices (one scale sector serves both), one for narrow ones, unless the K ranges
    // (at most 768 rows) then make more CTAs than fit at once (three per SM at 168 registers)
    auto lay = [&](int W) {
        p.W = W;
        p.tiles = (gpr + W - 1) / W;
        uint32_t splits = 2u * sms / p.tiles;
        if (splits > 8) splits = 8;
        if (splits < 1) splits = 1;
        if (splits > (uint32_t)kRowMaxCluster) splits = kRowMaxCluster;
        uint32_t kc = ((K + splits - 1) / splits + 15) / 16 * 16;
        if (kc > kRowMaxKc) kc = kRowMaxKc;
        p.kc = kc;
        p.splits = (K + kc - 1) / kc;
    };
    lay(gpr >= 64 ? 2 : 1);
    if (p.W == 1 && p.tiles * p.splits > 3 * sms) lay(2);
    p.ok = p.splits <= (uint32_t)kRowMaxCluster;          // deeper K: another kernel takes it
    p.ws = 0;
    return p;
}

template <int W>
static int launch_row(const Launch &l, const Int4RowPlan &p, float *out, uint32_t N, uint32_t K)
{
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        int rc = check_cuda(cudaFuncSetAttribute(int4_row_kernel<W>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1),
                            "int4_row_kernel attributes");
        if (rc) return rc;
        attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.tiles, p.splits);
    cfg.blockDim = dim3(kRowThreads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = l.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = p.splits;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int rc = check_cuda(cudaLaunchKernelEx(&cfg, int4_row_kernel<W>, ptr<const float>(l, 0), ptr<const uint4>(l, 1),
                                           ptr<const __half>(l, 2), ptr<const __half>(l, 3), out, N, K, p.kc),
                        "int4_row_kernel");
    count_launch();
    return rc;
}

int run_int4_row(const Launch &l, const Int4RowPlan &p, float *out, uint32_t N, uint32_t K)
{
    return p.W == 2 ? launch_row<2>(l, p, out, N, K) : launch_row<1>(l, p, out, N, K);
}

}  // namespace ab
