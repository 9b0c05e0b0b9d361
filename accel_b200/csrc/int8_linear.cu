// int8 linear: out[m][n] = sum_k a[m][k] (q[k][n] s[(k N + n) / 32]), f32 activations, one f16 scale
// per block of 32 weights along the flat [K, N] index (quant/quant.go:60-134).  Replaces
// QuantMatVecF32 (internal/kernels/matvec.go:204-231) and QuantMatMulTiledF32
// (internal/kernels/quant.go:195-243).
//
// The product is HBM-bound on the quants (one byte per weight).  A CTA of 256 threads owns 256
// columns and a range of K: thread (ty, tx) streams rows k = ty, ty + 16, ... of columns 16 tx .. 16 tx + 15,
// one 16-byte load per row (a half warp reads 256 contiguous bytes), with up to 4 activation rows'
// accumulators in registers.  An int8 becomes a float by a byte permute into the mantissa of 2^23
// and one subtraction, exactly.  Partial sums meet in shared memory (the 16 row phases of a CTA) and
// then across the CTAs of a thread-block cluster (the K splits of a column tile) through
// distributed shared memory, in a fixed order: deterministic, no workspace, no atomics.  More than
// 4 activation rows run as passes of 4.  Arithmetic is f32 throughout (q s rounded once, then one
// fused multiply-add per term), so the only difference from the reference kernels is the order of
// the sums.
//
// Shapes whose N is not a multiple of 32 (a block straddles rows) or K not covered by the fast
// path go to a plain kernel, one thread per output.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace ab {

static constexpr int kI8Threads = 256;
static constexpr int kI8Cols = 256;          // columns per CTA
static constexpr int kI8Phases = 16;         // row phases per CTA (threadIdx / 16)
static constexpr int kI8MaxRows = 4;         // activation rows per pass
static constexpr int kI8MaxSplits = 8;       // K splits of a column tile = cluster size

__device__ __forceinline__ float i8_scale(const __half *bs, uint64_t flat)
{
    return __half2float(__ldg(bs + (flat >> 5)));
}

// one output per thread: any N, any K
__global__ void int8_generic_kernel(const float *__restrict__ a, const int8_t *__restrict__ bq,
                                    const __half *__restrict__ bs, float *__restrict__ out, uint32_t M, uint32_t N,
                                    uint32_t K)
{
    const uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (uint64_t)M * N) return;
    const uint32_t m = (uint32_t)(idx / N), n = (uint32_t)(idx % N);
    float acc = 0.f;
    for (uint32_t k = 0; k < K; k++) {
        const uint64_t w = (uint64_t)k * N + n;
        acc = fmaf(a[(size_t)m * K + k], (float)bq[w] * i8_scale(bs, w), acc);
    }
    out[idx] = acc;
}

// four int8 of a word -> four floats, exactly: byte b lands in the mantissa of 2^23 with its sign
// bit flipped (so it reads as b + 128), and 2^23 + 128 is subtracted
__device__ __forceinline__ void i8_unpack4(uint32_t w, float (&f)[4])
{
    const uint32_t u = w ^ 0x80808080u;
    f[0] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7440)) - 8388736.f;
    f[1] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7441)) - 8388736.f;
    f[2] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7442)) - 8388736.f;
    f[3] = __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7443)) - 8388736.f;
}

// grid = (ceil(N / 256), splits), cluster = (1, splits, 1).  MR activation rows (m0 .. m0 + MR - 1).
// Thread (ty, tx): tx = threadIdx % 16 owns columns 16 tx .. 16 tx + 15 (one 16-byte load per row, a
// half warp reads 256 contiguous bytes), ty = threadIdx / 16 the rows k = ty, ty + 16, ...; eight rows
// (four for MR = 4) are in flight per thread, about 10 MB over the device.
template <int MR>
__global__ void __launch_bounds__(kI8Threads)
int8_rows_kernel(const float *__restrict__ a, const int8_t *__restrict__ bq, const __half *__restrict__ bs,
                 float *__restrict__ out, uint32_t N, uint32_t K, uint32_t kc, uint32_t m0)
{
    __shared__ float part[MR][kI8Cols];          // the CTA's sums over its 16 row phases
    cg::cluster_group cluster = cg::this_cluster();
    constexpr int kFlight = MR <= 2 ? 8 : 4;
    const uint32_t tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const uint32_t col = blockIdx.x * kI8Cols + tx * 16;
    const uint32_t kbeg = blockIdx.y * kc, kend = min(K, kbeg + kc);
    const bool on = col < N;                     // N is a multiple of 32: 16 columns are all in or all out
    float acc[MR][16];
#pragma unroll
    for (int m = 0; m < MR; m++)
#pragma unroll
        for (int j = 0; j < 16; j++) acc[m][j] = 0.f;
    if (on) {
        const float *ar = a + (size_t)m0 * K;
        for (uint32_t k = kbeg + ty; k < kend; k += kFlight * kI8Phases) {
            uint4 q[kFlight];
            unsigned short sbits[kFlight];       // raw: converting here would wait for each load in turn
#pragma unroll
            for (int u = 0; u < kFlight; u++) {
                const uint32_t kk = k + u * kI8Phases;
                q[u] = make_uint4(0u, 0u, 0u, 0u);
                sbits[u] = 0;
                if (kk < kend) {
                    const uint64_t flat = (uint64_t)kk * N + col;
                    q[u] = __ldg(reinterpret_cast<const uint4 *>(bq + flat));
                    sbits[u] = __ldg(reinterpret_cast<const unsigned short *>(bs) + (flat >> 5));
                }
            }
            float s[kFlight];
#pragma unroll
            for (int u = 0; u < kFlight; u++) s[u] = __half2float(__ushort_as_half(sbits[u]));
#pragma unroll
            for (int u = 0; u < kFlight; u++) {
                const uint32_t kk = k + u * kI8Phases;
                if (kk < kend) {
                    float w[16];
                    const uint32_t words[4] = {q[u].x, q[u].y, q[u].z, q[u].w};
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        float f[4];
                        i8_unpack4(words[i], f);
#pragma unroll
                        for (int j = 0; j < 4; j++) w[4 * i + j] = f[j] * s[u];
                    }
#pragma unroll
                    for (int m = 0; m < MR; m++) {
                        const float av = __ldg(ar + (size_t)m * K + kk);
#pragma unroll
                        for (int j = 0; j < 16; j++) acc[m][j] = fmaf(av, w[j], acc[m][j]);
                    }
                }
            }
        }
    }
    // the CTA's sums over its 16 phases, added in phase order
    for (int p = 0; p < kI8Phases; p++) {
        if ((int)ty == p) {
#pragma unroll
            for (int m = 0; m < MR; m++)
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    float &dst = part[m][tx * 16 + j];
                    dst = p == 0 ? acc[m][j] : dst + acc[m][j];
                }
        }
        __syncthreads();
    }
    cluster.sync();
    // the K splits, in split order: cluster rank r sums the columns r, r + splits, ... of every row
    const uint32_t splits = gridDim.y, rank = blockIdx.y;
    for (uint32_t i = threadIdx.x * splits + rank; i < MR * kI8Cols; i += kI8Threads * splits) {
        const uint32_t m = i / kI8Cols, c = i % kI8Cols;
        float v = 0.f;
        for (uint32_t sp = 0; sp < splits; sp++) {
            const float *remote = cluster.map_shared_rank(&part[0][0], sp);
            v += remote[m * kI8Cols + c];
        }
        const uint32_t n = blockIdx.x * kI8Cols + c;
        if (n < N) out[(size_t)(m0 + m) * N + n] = v;
    }
    cluster.sync();                              // nobody leaves while its sums are being read
}

template <int MR>
static int launch_rows(cudaStream_t stream, const float *a, const int8_t *bq, const __half *bs, float *out, uint32_t N,
                       uint32_t K, uint32_t splits, uint32_t kc, uint32_t m0)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((N + kI8Cols - 1) / kI8Cols, splits);
    cfg.blockDim = dim3(kI8Threads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = splits;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int rc = check_cuda(cudaLaunchKernelEx(&cfg, int8_rows_kernel<MR>, a, bq, bs, out, N, K, kc, m0), "int8_rows_kernel");
    count_launch();
    return rc;
}

static int launch_int8(Launch &l, const char *name, uint32_t M, uint32_t N, uint32_t K)
{
    if (l.query_ws) { l.ws_need = 0; return AB_OK; }
    if (M == 0 || N == 0 || K == 0) return fail(AB_ERR_INVALID, "%s: M=%u N=%u K=%u", name, M, N, K);
    const uint64_t weights = (uint64_t)K * N;
    if (l.len[0] < (uint64_t)M * K || l.len[1] < weights || l.len[2] < (weights + 31) / 32 || l.len[3] < (uint64_t)M * N)
        return fail(AB_ERR_INVALID, "%s: M=%u N=%u K=%u needs a[%llu] bq[%llu] bs[%llu] out[%llu]; the lengths block "
                    "says %u %u %u %u", name, M, N, K, (unsigned long long)M * K, (unsigned long long)weights,
                    (unsigned long long)(weights + 31) / 32, (unsigned long long)M * N, l.len[0], l.len[1], l.len[2],
                    l.len[3]);
    const float *a = ptr<const float>(l, 0);
    const int8_t *bq = ptr<const int8_t>(l, 1);
    const __half *bs = ptr<const __half>(l, 2);
    float *out = ptr<float>(l, 3);
    if (N % 32 != 0 || reinterpret_cast<uintptr_t>(bq) % 16) {
        const uint64_t mn = (uint64_t)M * N;
        int8_generic_kernel<<<(unsigned)((mn + 127) / 128), 128, 0, l.stream>>>(a, bq, bs, out, M, N, K);
        count_launch();
        note_selection("%s: one thread per output (N=%u is not a multiple of 32, or the quants are not 16-byte "
                       "aligned)", name, N);
        return check_cuda(cudaGetLastError(), name);
    }
    // K splits: enough CTAs for two per SM, at most a cluster of 8, at least 64 rows each
    const uint32_t tiles = (N + kI8Cols - 1) / kI8Cols;
    uint32_t splits = (2u * (uint32_t)sm_count() + tiles - 1) / tiles;
    if (splits > (uint32_t)kI8MaxSplits) splits = kI8MaxSplits;
    while (splits > 1 && K / splits < 64) splits--;
    const uint32_t kc = (K + splits - 1) / splits;
    for (uint32_t m0 = 0; m0 < M;) {
        const uint32_t left = M - m0;
        int rc;
        if (left >= 4) { rc = launch_rows<4>(l.stream, a, bq, bs, out, N, K, splits, kc, m0); m0 += 4; }
        else if (left >= 2) { rc = launch_rows<2>(l.stream, a, bq, bs, out, N, K, splits, kc, m0); m0 += 2; }
        else { rc = launch_rows<1>(l.stream, a, bq, bs, out, N, K, splits, kc, m0); m0 += 1; }
        if (rc) return rc;
    }
    note_selection("%s: int8 streaming kernel (16-byte loads, f32 arithmetic), %u column tiles of 256 x a cluster of "
                   "%u K splits of %u rows, passes of up to 4 activation rows", name, tiles, splits, kc);
    return AB_OK;
}

int launch_quant_matvec_f32(Launch &l)
{   // GEMMDims{M,N,K}; M is 1 (tensor/quantized.go:117-135)
    return launch_int8(l, "QuantMatVecF32", 1, u32_at(l.u, 4), u32_at(l.u, 8));
}

int launch_quant_matmul_tiled_f32(Launch &l)
{
    return launch_int8(l, "QuantMatMulTiledF32", u32_at(l.u, 0), u32_at(l.u, 4), u32_at(l.u, 8));
}

}  // namespace ab
