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
};

__device__ __forceinline__ bool find_tile(const GroupedParams &p, uint32_t t, uint32_t &e,
                                          uint32_t &row0, uint32_t &last)
{
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

static int run_grouped(Launch &l, GroupedParams &p, bool int4, bool zero_tail, uint32_t out_rows,
                       const char *name)
{
    if (l.query_ws) { l.ws_need = 0; return AB_OK; }
    if (p.experts == 0 || p.K == 0 || p.N == 0)
        return fail(AB_ERR_INVALID, "%s: Experts=%u K=%u N=%u", name, p.experts, p.K, p.N);
    if (p.tokens == 0) return AB_OK;
    bool fast = p.K % BK == 0 && (int4 ? p.N % kGroup == 0 : p.N % 4 == 0);
    if (fast) {
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
                   fast ? "128x128 register-tiled kernel" : "generic kernel", p.experts, p.tokens);
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
