// int4 group-quantized linear: the row kernel (QuantMatVecInt4, internal/kernels/int4.go:60) and the
// batched form (QuantMatMulInt4, internal/kernels/int4tiled.go:66) for small batches.
//
//   out[m][n] = sum_k a[m][k] * w(k,n),   w = s == 0 ? z : (code - z) * s
//
// with code = nibble (k*N+n) of bq (eight per u32, low first) and one f16 scale s and zero z per 128
// consecutive flat weights.  When N is a multiple of 128 a group is 128 adjacent columns of one row
// k, so the kernel streams each row segment once with 128-bit loads and evaluates
//
//   out[m][n] = sum_k (a[m][k]*s) * code  -  sum_k (a[m][k]*s) * z        (s != 0)
//
// in f32: the per-weight work is one integer-to-float conversion and one FMA, and the zero-point
// term costs one FMA per row and group.  A group with s == 0 contributes a[m][k]*z through the
// second sum.  The summation order differs from the reference's, the values do not.
#include <cstdlib>

#include "common.cuh"

namespace ab {

static constexpr uint32_t kGroup = 128;     // quant.Int4Group
static constexpr int kTileCols = 256;       // columns per CTA: 8 lanes x 32 nibbles
static constexpr int kThreads = 256;        // 8 warps, each warp-load covers 4 rows x 256 columns
static constexpr int kRowsPerStep = 32;     // 8 warps x 4 rows
static constexpr int kUnroll = 4;

__device__ __forceinline__ uint4 ldg_stream(const uint4 *p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// The nibble at bit position P of w as a float.  OR-ing the masked nibble into the mantissa of
// 2^(23-P) gives exactly 2^(23-P) + code, and the subtraction is exact, so this is code itself:
// one logic op and one add, no integer-to-float conversion instruction.  P <= 16 keeps the nibble
// inside the mantissa; the three high nibbles come from w >> 12.
template <int P> __device__ __forceinline__ float nib(uint32_t w)
{
    constexpr uint32_t magic = (150u - P) << 23;
    return __uint_as_float((w & (0xFu << P)) | magic) - __uint_as_float(magic);
}

template <int MR>
__device__ __forceinline__ void fma_word(uint32_t w, const float (&c)[MR], float (&acc)[MR][32],
                                         int j)
{
    uint32_t w2 = w >> 12;
    float x[8] = {nib<0>(w), nib<4>(w), nib<8>(w), nib<12>(w),
                  nib<16>(w), nib<8>(w2), nib<12>(w2), nib<16>(w2)};
#pragma unroll
    for (int m = 0; m < MR; m++)
#pragma unroll
        for (int i = 0; i < 8; i++) acc[m][j * 8 + i] = fmaf(c[m], x[i], acc[m][j * 8 + i]);
}

// grid = (column tiles, K splits).  dst is `out` when gridDim.y == 1, else the partials
// [split][M][N] that int4_reduce_kernel sums.
template <int MR>
__global__ void __launch_bounds__(kThreads)
int4_gemv_kernel(const float *__restrict__ a, const uint4 *__restrict__ bq,
                 const __half *__restrict__ bs, const __half *__restrict__ bz,
                 float *__restrict__ dst, uint32_t M, uint32_t N, uint32_t K, uint32_t kc,
                 uint32_t m0, uint32_t mrows)
{
    __shared__ float red[8][kTileCols];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = lane >> 3, c8 = lane & 7;
    const uint32_t col0 = blockIdx.x * kTileCols + c8 * 32;
    const bool active = col0 < N;
    const uint32_t gpr = N / kGroup;                 // groups per row
    const uint32_t g = col0 / kGroup;
    const uint32_t kbeg = blockIdx.y * kc;
    const uint32_t kend = min(K, kbeg + kc);

    float acc[MR][32];
    float zc[MR];
#pragma unroll
    for (int m = 0; m < MR; m++) {
        zc[m] = 0.f;
#pragma unroll
        for (int j = 0; j < 32; j++) acc[m][j] = 0.f;
    }

    if (active) {
        for (uint32_t kk = kbeg + warp * 4 + r; kk < kend; kk += kRowsPerStep * kUnroll) {
            uint4 cw[kUnroll];
            float s[kUnroll], z[kUnroll], av[kUnroll][MR];
#pragma unroll
            for (int u = 0; u < kUnroll; u++) {
                uint32_t k = kk + u * kRowsPerStep;
                bool ok = k < kend;
                uint32_t ks = ok ? k : kbeg;
                cw[u] = ldg_stream(bq + ((size_t)ks * N + col0) / 32);
                s[u] = ok ? __half2float(__ldg(bs + (size_t)ks * gpr + g)) : 0.f;
                z[u] = ok ? __half2float(__ldg(bz + (size_t)ks * gpr + g)) : 0.f;
#pragma unroll
                for (int m = 0; m < MR; m++)
                    av[u][m] = (ok && (uint32_t)m < mrows) ? __ldg(a + (size_t)(m0 + m) * K + ks) : 0.f;
            }
#pragma unroll
            for (int u = 0; u < kUnroll; u++) {
                float c[MR];
#pragma unroll
                for (int m = 0; m < MR; m++) {
                    c[m] = av[u][m] * s[u];
                    // s == 0: the group is the constant z, so the row adds a*z; written as a
                    // subtraction of -a*z because zc is subtracted below
                    zc[m] += (s[u] == 0.f) ? -av[u][m] * z[u] : c[m] * z[u];
                }
                fma_word<MR>(cw[u].x, c, acc, 0);
                fma_word<MR>(cw[u].y, c, acc, 1);
                fma_word<MR>(cw[u].z, c, acc, 2);
                fma_word<MR>(cw[u].w, c, acc, 3);
            }
        }
    }

    // fold the four row-lanes of the warp, then the eight warps through shared memory
#pragma unroll
    for (int m = 0; m < MR; m++) {
#pragma unroll
        for (int j = 0; j < 32; j++) {
            float v = acc[m][j] - zc[m];
            v += __shfl_xor_sync(0xffffffffu, v, 8);
            v += __shfl_xor_sync(0xffffffffu, v, 16);
            acc[m][j] = v;
        }
    }
    const uint32_t col = blockIdx.x * kTileCols + threadIdx.x;
#pragma unroll
    for (int m = 0; m < MR; m++) {
        __syncthreads();
        if (r == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<float4 *>(&red[warp][c8 * 32 + j]) =
                    make_float4(acc[m][j], acc[m][j + 1], acc[m][j + 2], acc[m][j + 3]);
        }
        __syncthreads();
        if ((uint32_t)m < mrows && col < N) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < 8; w++) v += red[w][threadIdx.x];
            dst[((size_t)blockIdx.y * M + m0 + m) * N + col] = v;
        }
    }
}

// Sums the K-split partials [splits][mn] into out: one float4 of outputs per thread, the splits'
// loads independent of one another.
__global__ void int4_reduce_kernel(const float *__restrict__ part, float *__restrict__ out,
                                   uint32_t splits, size_t mn)
{
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= mn) return;
    if (i + 4 <= mn) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
        for (uint32_t s = 0; s < splits; s++) {
            const float4 x = __ldcs(reinterpret_cast<const float4 *>(part + (size_t)s * mn + i));
            v.x += x.x; v.y += x.y; v.z += x.z; v.w += x.w;
        }
        *reinterpret_cast<float4 *>(out + i) = v;
    } else {
        for (size_t j = i; j < mn; j++) {
            float v = 0.f;
            for (uint32_t s = 0; s < splits; s++) v += part[(size_t)s * mn + j];
            out[j] = v;
        }
    }
}

// Any shape: one thread per output, flat weight index, groups that straddle rows and a partial
// last word included (quant/int4.go:67-80).  Slow; it exists so that no shape is refused.
__global__ void int4_generic_kernel(const float *__restrict__ a, const uint32_t *__restrict__ bq,
                                    const __half *__restrict__ bs, const __half *__restrict__ bz,
                                    float *__restrict__ out, uint32_t M, uint32_t N, uint32_t K)
{
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)M * N) return;
    uint32_t m = (uint32_t)(i / N), n = (uint32_t)(i % N);
    float acc = 0.f;
    for (uint32_t k = 0; k < K; k++) {
        size_t w = (size_t)k * N + n;
        uint32_t code = (bq[w / 8] >> (4 * (w % 8))) & 0xFu;
        float s = __half2float(bs[w / kGroup]), z = __half2float(bz[w / kGroup]);
        float wv = s == 0.f ? z : ((float)code - z) * s;
        acc = fmaf(a[(size_t)m * K + k], wv, acc);
    }
    out[i] = acc;
}

struct Int4Plan { bool fast; uint32_t tiles, splits, kc; size_t ws; };

static Int4Plan plan_int4(uint32_t M, uint32_t N, uint32_t K)
{
    Int4Plan p{};
    p.fast = (N % kGroup == 0) && N > 0 && K > 0;
    if (!p.fast) return p;
    p.tiles = (N + kTileCols - 1) / kTileCols;
    uint32_t target = 3u * (uint32_t)sm_count();
    uint32_t splits = (target + p.tiles - 1) / p.tiles;
    uint32_t max_splits = (K + kRowsPerStep - 1) / kRowsPerStep;
    if (splits > max_splits) splits = max_splits;
    if (splits < 1) splits = 1;
    p.kc = ((K + splits - 1) / splits + kRowsPerStep - 1) / kRowsPerStep * kRowsPerStep;
    p.splits = (K + p.kc - 1) / p.kc;
    p.ws = p.splits > 1 ? (size_t)p.splits * M * N * sizeof(float) : 0;
    return p;
}

template <int MR>
static void run_gemv(const Launch &l, const Int4Plan &p, float *dst, uint32_t M, uint32_t N,
                     uint32_t K, uint32_t m0, uint32_t mrows)
{
    dim3 grid(p.tiles, p.splits);
    int4_gemv_kernel<MR><<<grid, kThreads, 0, l.stream>>>(
        ptr<const float>(l, 0), ptr<const uint4>(l, 1), ptr<const __half>(l, 2),
        ptr<const __half>(l, 3), dst, M, N, K, p.kc, m0, mrows); count_launch();
}

static int forced_path()
{
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("AB_INT4_PATH");
        v = !e ? 0 : (!strcmp(e, "tc") ? 1 : (!strcmp(e, "mma") ? 2 : (!strcmp(e, "simt") ? 3 :
            (!strcmp(e, "batch") ? 4 : (!strcmp(e, "row") ? 5 : (!strcmp(e, "tiles") ? 7 : 0))))));
    }
    return v;
}

// From this many activation rows the reference-layout product runs on the tcgen05 tile kernel
// (int4_gemm.cu), which reads the prepacked stream: the three planes are permuted into the
// workspace first, every call (about 20 us for 4096 x 11008, a fifth of the product at 512 rows; a
// host that keeps its weights prepacks them once with ab_int4_prepack and calls the packed entry
// points instead).  Measured on a B200 at 4096 x 11008: 64 rows, 4 passes of the 16-row kernel 73 us
// against 70 us; 512 rows, 351 us on the warp-level tile kernel against 112 us.
static constexpr uint32_t kTcFromRows = 64;
static bool tc_tiles_ok(uint32_t M, uint32_t N, uint32_t K) { return M >= kTcFromRows && int4_stream_ok(M, N, K); }
static size_t tc_tiles_workspace(uint32_t M, uint32_t N, uint32_t K)
{
    return align_up(int4_stream_packed_bytes(N, K), 256) + int4_gemm_workspace(M, K);
}

// The two-kernel tensor-core form (int4_mma.cu) rounds a * s to f16 like the others; it is the
// fallback for products too wide for one wave of clusters, so it gets the rows' power-of-two factors
// from outside: a copy of the activations scaled per row, and the output rows scaled back.
__global__ void __launch_bounds__(256)
int4_scale_rows_kernel(const float *__restrict__ a, const float *__restrict__ amax, float *__restrict__ scaled, uint32_t K)
{
    const float pa = ab_pow2(8 - ab_row_exponent(__float_as_uint(fabsf(amax[blockIdx.x]))));
    const size_t base = (size_t)blockIdx.x * K;
    for (uint32_t k = threadIdx.x; k < K; k += 256) scaled[base + k] = a[base + k] * pa;
}

__global__ void __launch_bounds__(256)
int4_unscale_rows_kernel(float *__restrict__ out, const float *__restrict__ amax, uint32_t N)
{
    const float un = ab_pow2(ab_row_exponent(__float_as_uint(fabsf(amax[blockIdx.x]))) - 8);
    const size_t base = (size_t)blockIdx.x * N;
    for (uint32_t n = threadIdx.x; n < N; n += 256) out[base + n] *= un;
}

static size_t mma_prescale_workspace(uint32_t M, uint32_t K) { return align_up((size_t)M * 4, 256) + align_up((size_t)M * K * 4, 256); }

static int launch_int4(Launch &l, const char *name, uint32_t M, uint32_t N, uint32_t K)
{
    if (N == 0 || K == 0 || M == 0) return fail(AB_ERR_INVALID, "%s: M=%u N=%u K=%u", name, M, N, K);
    Int4Plan p = plan_int4(M, N, K);
    // two or more rows of activations go to the tensor cores; one row stays on the CUDA cores
    Int4MmaPlan mp = plan_int4_mma(M, N, K);
    // AB_INT4_PATH = tiles | tc | batch | mma | simt | row overrides the choice (for
    // measurements and tests)
    const int forced = forced_path();
    // large batches: the tcgen05 tile kernel; AB_INT4_PATH=tiles keeps the warp-level MMA tile
    // kernel (the one the grouped product also uses)
    const bool use_tiles = int4_tiles_ok(N, K) && forced == 7;
    const bool use_tc = !use_tiles && int4_stream_ok(M, N, K) && (forced == 1 || (forced == 0 && tc_tiles_ok(M, N, K)));
    Int4BatchPlan bp = plan_int4_batch(M, N, K);
    const bool use_batch = !use_tc && !use_tiles && bp.ok && (forced == 4 || (forced == 0 && M >= 2));
    const bool use_mma = !use_tc && !use_tiles && !use_batch && mp.ok && (forced == 2 || (forced == 0 && M >= 2));
    // one row: the streaming kernel that sums its own K splits (AB_INT4_PATH=simt keeps the older
    // two-kernel form, which is also the fallback when no counter slot is free)
    Int4RowPlan rp = plan_int4_row(N, K);
    const bool use_row = !use_tc && !use_tiles && !use_mma && !use_batch && rp.ok && M == 1 && forced != 3;
    if (l.query_ws) {
        l.ws_need = use_tiles ? int4_tiles_workspace(M) : use_tc ? tc_tiles_workspace(M, N, K) : (use_batch ? int4_batch_workspace(M) : (use_mma ? align_up(mp.ws, 256) + mma_prescale_workspace(M, K) : (use_row ? 0 : p.ws)));
        return AB_OK;
    }

    uint64_t weights = (uint64_t)K * N;
    if (l.len[0] < (uint64_t)M * K || l.len[1] < (weights + 7) / 8 ||
        l.len[2] < (weights + kGroup - 1) / kGroup || l.len[3] < (weights + kGroup - 1) / kGroup ||
        l.len[4] < (uint64_t)M * N)
        return fail(AB_ERR_INVALID,
                    "%s: M=%u N=%u K=%u needs a[%llu] bq[%llu] bs/bz[%llu] out[%llu]; the lengths "
                    "block says %u %u %u %u %u",
                    name, M, N, K, (unsigned long long)M * K, (unsigned long long)(weights + 7) / 8,
                    (unsigned long long)(weights + kGroup - 1) / kGroup, (unsigned long long)M * N,
                    l.len[0], l.len[1], l.len[2], l.len[3], l.len[4]);
    float *out = ptr<float>(l, 4);
    if (!p.fast) {
        size_t mn = (size_t)M * N;
        int4_generic_kernel<<<(unsigned)((mn + 127) / 128), 128, 0, l.stream>>>(
            ptr<const float>(l, 0), ptr<const uint32_t>(l, 1), ptr<const __half>(l, 2),
            ptr<const __half>(l, 3), out, M, N, K); count_launch();
        note_selection("%s: generic kernel, N=%u is not a multiple of %u", name, N, kGroup);
        return check_cuda(cudaGetLastError(), name);
    }
    if (use_tiles) {
        int rc = run_int4_tiles(l, out, M, N, K);
        if (rc) return rc;
        note_selection("%s: tensor-core tile kernel (128 rows x 128 columns per CTA, m16n8k16, f16 "
                       "operands, f32 accumulate), %u x %u tiles", name, N / kGroup, (M + 127) / 128);
        return AB_OK;
    }
    if (use_tc) {
        const size_t need = tc_tiles_workspace(M, N, K);
        if (need > l.ws_bytes || !l.ws)
            return fail(AB_ERR_INVALID, "%s: needs %zu bytes of workspace, given %zu", name, need, l.ws_bytes);
        unsigned char *packed = static_cast<unsigned char *>(l.ws);
        int rc = run_int4_prepack(l.stream, ptr<const uint32_t>(l, 1), ptr<const uint16_t>(l, 2), ptr<const uint16_t>(l, 3),
                                  packed, N, K);
        if (rc) return rc;
        return run_int4_gemm_mode(l.stream, ptr<const float>(l, 0), packed, 0, out, nullptr, nullptr, 0, 0, M, N, K, N,
                                  packed + align_up(int4_stream_packed_bytes(N, K), 256));
    }
    if (use_batch) {
        int rc = run_int4_batch(l, bp, out, M, N, K);
        if (rc) return rc;
        note_selection("%s: tensor-core kernel (m16n8k16, f16 operands, f32 accumulate), %u tiles of "
                       "%d column groups x a cluster of %u K splits of %u rows, %u pass(es) of 16 "
                       "activation rows", name, bp.tiles, bp.G, bp.splits, bp.kc, (M + 15) / 16);
        return check_cuda(cudaGetLastError(), name);
    }
    if (use_mma) {
        const size_t need = align_up(mp.ws, 256) + mma_prescale_workspace(M, K);
        if (need > l.ws_bytes || !l.ws)
            return fail(AB_ERR_INVALID, "%s: needs %zu bytes of workspace, given %zu", name, need, l.ws_bytes);
        unsigned char *w = static_cast<unsigned char *>(l.ws);
        float *partial = reinterpret_cast<float *>(w);
        float *amax = reinterpret_cast<float *>(w + align_up(mp.ws, 256));
        float *scaled = reinterpret_cast<float *>(w + align_up(mp.ws, 256) + align_up((size_t)M * 4, 256));
        int rc = run_row_absmax(l.stream, ptr<const float>(l, 0), amax, M, K, false);
        if (rc) return rc;
        int4_scale_rows_kernel<<<M, 256, 0, l.stream>>>(ptr<const float>(l, 0), amax, scaled, K); count_launch();
        void *b2[5] = {scaled, l.b[1], l.b[2], l.b[3], l.b[4]};
        Launch l2 = l;
        l2.b = b2;
        float *mdst = mp.splits > 1 ? partial : out;
        rc = run_int4_mma(l2, mp, mdst, M, N, K);
        if (rc) return rc;
        if (mp.splits > 1) {
            size_t mn = (size_t)M * N;
            int4_reduce_kernel<<<(unsigned)((mn / 4 + 128) / 128), 128, 0, l.stream>>>(mdst, out, mp.splits, mn); count_launch();
        }
        int4_unscale_rows_kernel<<<M, 256, 0, l.stream>>>(out, amax, N); count_launch();
        note_selection("%s: tensor-core kernel (m16n8k16, f16 operands, f32 accumulate), %u column "
                       "groups x %u K splits of %u rows, %u pass(es) of 16 activation rows", name,
                       mp.groups, mp.splits, mp.kc, (M + 15) / 16);
        return check_cuda(cudaGetLastError(), name);
    }
    if (use_row) {
        int rc = run_int4_row(l, rp, out, N, K);
        if (rc) return rc;
        note_selection("%s: streaming row kernel (one mixed-precision FMA per weight), %u tiles of %d "
                       "column groups x a cluster of %u K splits of %u rows", name, rp.tiles, rp.W,
                       rp.splits, rp.kc);
        return check_cuda(cudaGetLastError(), name);
    }
    if (p.ws > l.ws_bytes || (p.ws && !l.ws))
        return fail(AB_ERR_INVALID, "%s: needs %zu bytes of workspace, given %zu", name, p.ws,
                    l.ws_bytes);
    float *dst = p.splits > 1 ? reinterpret_cast<float *>(l.ws) : out;
    for (uint32_t m0 = 0; m0 < M;) {
        uint32_t left = M - m0;
        if (left >= 4) { run_gemv<4>(l, p, dst, M, N, K, m0, 4); m0 += 4; }
        else if (left >= 2) { run_gemv<2>(l, p, dst, M, N, K, m0, 2); m0 += 2; }
        else { run_gemv<1>(l, p, dst, M, N, K, m0, 1); m0 += 1; }
    }
    if (p.splits > 1) {
        size_t mn = (size_t)M * N;
        int4_reduce_kernel<<<(unsigned)((mn / 4 + 128) / 128), 128, 0, l.stream>>>(dst, out, p.splits, mn); count_launch();
    }
    note_selection("%s: streaming row kernel, %u column tiles x %u K splits of %u rows, %u row(s) "
                   "of activations per pass", name, p.tiles, p.splits, p.kc, M >= 4 ? 4 : M);
    return check_cuda(cudaGetLastError(), name);
}

int launch_quant_matvec_int4(Launch &l)
{   // GEMMDims{M,N,K}; the reference's matvec leaves M zero (tensor/int4.go:131-133)
    uint32_t N = u32_at(l.u, 4), K = u32_at(l.u, 8);
    return launch_int4(l, "QuantMatVecInt4", 1, N, K);
}

int launch_quant_matmul_int4(Launch &l)
{
    uint32_t M = u32_at(l.u, 0), N = u32_at(l.u, 4), K = u32_at(l.u, 8);
    return launch_int4(l, "QuantMatMulInt4", M, N, K);
}

// ------------------------------------------------------------------------------------------------
// The int4 product for callers that cannot allocate device memory.
//
// Some hosts of this library only ever hand over buffers they were given: a plugin running inside
// another runtime's allocator, a real-time loop that must not call into the driver's allocator once
// it has started, a sandbox that forbids cudaMalloc outright.  They cannot supply the split-K
// workspace the regular entry point asks for.  This entry point carries its own: a fixed array in
// the library's device image, present on every GPU that loads the library for as long as the
// process lives.  The caller passes inputs and the output only.
static constexpr size_t kStaticScratchBytes = 8u << 20;          // 8 MiB: the stated maximum
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

}  // namespace ab

extern "C" AB_API int ab_quant_matmul_int4_noalloc(void *stream, const float *a, const uint32_t *bq,
                                            const uint16_t *bs, const uint16_t *bz, float *out,
                                            uint32_t M, uint32_t N, uint32_t K)
{
    using namespace ab;
    // The array's name is only a handle on the host; the device address has to be asked for, once
    // per device, with that device current.  This first call per device is the set-up.
    static void *scratch_of[64] = {};
    int dev = -1;
    int rc = check_cuda(cudaGetDevice(&dev), "ab_quant_matmul_int4_noalloc");
    if (rc) return rc;
    if (dev < 0 || dev >= 64) return fail(AB_ERR_INVALID, "ab_quant_matmul_int4_noalloc: device %d", dev);
    if (stream) {
        // the array's address is the CURRENT device's: a stream of another device would be handed
        // memory its kernels cannot be assumed to reach
        int sdev = -1;
        rc = check_cuda(cudaStreamGetDevice(static_cast<cudaStream_t>(stream), &sdev),
                        "ab_quant_matmul_int4_noalloc: cudaStreamGetDevice");
        if (rc) return rc;
        if (sdev != dev)
            return fail(AB_ERR_INVALID, "ab_quant_matmul_int4_noalloc: the stream belongs to device %d "
                        "and device %d is current; make the stream's device current first", sdev, dev);
    }
    if (!scratch_of[dev]) {
        void *p = nullptr;
        rc = check_cuda(cudaGetSymbolAddress(&p, g_static_scratch), "cudaGetSymbolAddress(scratch)");
        if (rc) return rc;
        scratch_of[dev] = p;
    }
    if (M == 0) M = 1;                   // the matvec form leaves M zero
    const uint64_t weights = (uint64_t)K * N;
    void *bind[5] = {const_cast<float *>(a), const_cast<uint32_t *>(bq), const_cast<uint16_t *>(bs),
                     const_cast<uint16_t *>(bz), out};
    const uint32_t lens[5] = {(uint32_t)((uint64_t)M * K), (uint32_t)((weights + 7) / 8),
                              (uint32_t)((weights + 127) / 128), (uint32_t)((weights + 127) / 128),
                              (uint32_t)((uint64_t)M * N)};
    Launch q{nullptr, nullptr, lens, 5, nullptr, 0, nullptr, 0, true, 0};
    rc = launch_int4(q, "QuantMatMulInt4 (no-alloc)", M, N, K);
    if (rc) return rc;
    if (q.ws_need > kStaticScratchBytes)
        return fail(AB_ERR_INVALID, "ab_quant_matmul_int4_noalloc: M=%u N=%u K=%u needs %zu bytes of "
                    "scratch and the built-in array holds %zu; use ab_launch with a workspace of your "
                    "own for this shape", M, N, K, q.ws_need, kStaticScratchBytes);
    for (int i = 0; i < 5; i++)
        if (!bind[i] || reinterpret_cast<uintptr_t>(bind[i]) % 16)
            return fail(AB_ERR_INVALID, "ab_quant_matmul_int4_noalloc: argument %d is NULL or not "
                        "16-byte aligned", i);
    Launch l{static_cast<cudaStream_t>(stream), bind, lens, 5, nullptr, 0, scratch_of[dev],
             kStaticScratchBytes, false, 0};
    return launch_int4(l, "QuantMatMulInt4 (no-alloc)", M, N, K);
}
