// The sampling policy of a decode step on the device: Softmax (internal/kernels/norm.go:94), the
// per-row forms ScaleRows, TopKMaskRows, TopPMaskRows, SampleRows, LogitBias and the three penalty
// kernels (internal/kernels/rowsample.go:42-379), and the uniform forms they generalise (TopKMask,
// TopPMask: topk.go:59-256; SampleCategorical: sample.go:133; PenaltyClear / Count / Apply:
// penalty.go:60-141).  A step that samples on the device reads back one token id per row instead
// of a vocabulary of logits (docs/tutorial/09-a-decode-step.md:86-88).
//
// What is exact.  The masks and the sampled index are index work: they are bit-identical to the
// reference's CPU kernels, which takes the reference's own ORDER of float additions wherever a sum
// decides an index:
//   - Softmax and the top-p total: 128 lanes each sum their strided elements in order, then a binary
//     tree over the lanes, as the reference's workgroup of 128 does;
//   - top-p's kept mass: the frontier values added largest first;
//   - the categorical walk: ONE running sum over the row in index order.  Exactly-zero weights leave a
//     running sum unchanged, so blocks of the row that are all zero (what a mask leaves of most of
//     the vocabulary) are skipped; the rest is summed by one thread from shared memory.
// The extraction rounds of the masks compare, and never add: the largest entry below the frontier in
// (value descending, index ascending) order is the same whoever looks for it.
#include "common.cuh"

namespace ab {

static constexpr int kRowWidth = 128;          // the reference's workgroup for every row kernel
static constexpr uint32_t kTopMaxRounds = 128; // internal/kernels/topk.go:30
static constexpr float kSentinelHi = 3.4e38f, kSentinelLo = -3.4e38f;

static inline unsigned sp_blocks(size_t n, int per) { return (unsigned)((n + per - 1) / per); }

// kmath.Max (kmath/kmath.go:96-104): NaN if either is NaN
__device__ __forceinline__ float k_max(float x, float y)
{
    if (x != x || y != y) return __int_as_float(0x7fc00000);
    return x > y ? x : y;
}
// kmath.Exp (kmath/kmath.go:55): the binary64 exponential rounded once
__device__ __forceinline__ float k_exp(float x) { return (float)exp((double)x); }

// ---------------------------------------------------------------- Softmax
__global__ void __launch_bounds__(kRowWidth) softmax_kernel(const float *__restrict__ x, float *__restrict__ out, uint32_t width)
{
    __shared__ float sh[kRowWidth];
    const uint32_t lid = threadIdx.x;
    const float *xr = x + (size_t)blockIdx.x * width;
    float m = xr[lid % width];
    for (uint32_t i = lid; i < width; i += kRowWidth) m = k_max(m, xr[i]);
    sh[lid] = m;
    __syncthreads();
    for (uint32_t stride = kRowWidth / 2; stride > 0; stride /= 2) {
        if (lid < stride) sh[lid] = k_max(sh[lid], sh[lid + stride]);
        __syncthreads();
    }
    const float row_max = sh[0];
    __syncthreads();
    float acc = 0.f;
    for (uint32_t i = lid; i < width; i += kRowWidth) acc = __fadd_rn(acc, k_exp(__fsub_rn(xr[i], row_max)));
    sh[lid] = acc;
    __syncthreads();
    for (uint32_t stride = kRowWidth / 2; stride > 0; stride /= 2) {
        if (lid < stride) sh[lid] = __fadd_rn(sh[lid], sh[lid + stride]);
        __syncthreads();
    }
    const float total = sh[0];
    for (uint32_t i = lid; i < width; i += kRowWidth)
        out[(size_t)blockIdx.x * width + i] = __fdiv_rn(k_exp(__fsub_rn(xr[i], row_max)), total);
}

int launch_softmax(Launch &l)
{   // x, out; RowDims{Rows,Width,Eps}
    if (l.query_ws) { l.ws_need = 0; return AB_OK; }
    const uint32_t rows = u32_at(l.u, 0), width = u32_at(l.u, 4);
    if (width == 0 || l.len[0] < (uint64_t)rows * width || l.len[1] < (uint64_t)rows * width)
        return fail(AB_ERR_INVALID, "Softmax: Rows=%u Width=%u; x[%u] out[%u]", rows, width, l.len[0], l.len[1]);
    if (rows == 0) return AB_OK;
    softmax_kernel<<<rows, kRowWidth, 0, l.stream>>>(ptr<const float>(l, 0), ptr<float>(l, 1), width);
    count_launch();
    return check_cuda(cudaGetLastError(), "Softmax");
}

// ---------------------------------------------------------------- ScaleRows, LogitBias
__global__ void scale_rows_kernel(const float *__restrict__ x, const float *__restrict__ factors,
                                  float *__restrict__ out, uint32_t vocab, size_t n)
{
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float f = factors[i / vocab];
    if (f == 0.f) f = 1.f;                       // a greedy row keeps its order into the softmax
    out[i] = __fmul_rn(x[i], f);
}

__global__ void logit_bias_kernel(const float *__restrict__ logits, const uint32_t *__restrict__ ids,
                                  const float *__restrict__ values, float *__restrict__ out, uint32_t vocab,
                                  uint32_t slots, size_t n)
{
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint32_t row = (uint32_t)(i / vocab), id = (uint32_t)(i - (size_t)row * vocab);
    float x = logits[i];
    for (uint32_t s = 0; s < slots; s++)
        if (ids[(size_t)row * slots + s] == id) x = __fadd_rn(x, values[(size_t)row * slots + s]);
    out[i] = x;
}

struct RowSampleDims { uint32_t vocab, rows, history, slots; };
static RowSampleDims row_dims_of(const Launch &l)
{
    return RowSampleDims{u32_at(l.u, 0), u32_at(l.u, 4), u32_at(l.u, 8), u32_at(l.u, 12)};
}

int launch_scale_rows(Launch &l)
{   // x, factors, out; RowSampleDims
    if (l.query_ws) { l.ws_need = 0; return AB_OK; }
    const RowSampleDims d = row_dims_of(l);
    const uint64_t n = (uint64_t)d.rows * d.vocab;
    if (d.vocab == 0 || l.len[0] < n || l.len[1] < d.rows || l.len[2] < n)
        return fail(AB_ERR_INVALID, "ScaleRows: Rows=%u Vocab=%u; x[%u] factors[%u] out[%u]", d.rows, d.vocab,
                    l.len[0], l.len[1], l.len[2]);
    if (n == 0) return AB_OK;
    scale_rows_kernel<<<sp_blocks(n, 256), 256, 0, l.stream>>>(ptr<const float>(l, 0), ptr<const float>(l, 1),
                                                              ptr<float>(l, 2), d.vocab, n);
    count_launch();
    return check_cuda(cudaGetLastError(), "ScaleRows");
}

int launch_logit_bias(Launch &l)
{   // logits, ids, values, out; RowSampleDims (Slots = the bias table's width per row)
    if (l.query_ws) { l.ws_need = 0; return AB_OK; }
    const RowSampleDims d = row_dims_of(l);
    const uint64_t n = (uint64_t)d.rows * d.vocab, t = (uint64_t)d.rows * d.slots;
    if (d.vocab == 0 || l.len[0] < n || l.len[1] < t || l.len[2] < t || l.len[3] < n)
        return fail(AB_ERR_INVALID, "LogitBias: Rows=%u Vocab=%u Slots=%u; logits[%u] ids[%u] values[%u] out[%u]",
                    d.rows, d.vocab, d.slots, l.len[0], l.len[1], l.len[2], l.len[3]);
    if (n == 0) return AB_OK;
    logit_bias_kernel<<<sp_blocks(n, 256), 256, 0, l.stream>>>(ptr<const float>(l, 0), ptr<const uint32_t>(l, 1),
                                                              ptr<const float>(l, 2), ptr<float>(l, 3), d.vocab,
                                                              d.slots, n);
    count_launch();
    return check_cuda(cudaGetLastError(), "LogitBias");
}

// ---------------------------------------------------------------- the masks
// One extraction round: the largest entry strictly below the frontier in (value descending, index
// ascending) order.  Every thread ends with the winner.
__device__ void top_round(const float *__restrict__ w, uint32_t vocab, float front_v, uint32_t front_i,
                          float *best, uint32_t *at, float &out_v, uint32_t &out_i)
{
    const uint32_t lane = threadIdx.x;
    float v = kSentinelLo;
    uint32_t idx = vocab;
    for (uint32_t i = lane; i < vocab; i += kRowWidth) {
        const float x = w[i];
        bool below = x < front_v;
        if (x == front_v && i > front_i) below = true;
        if (below) {
            bool better = x > v;
            if (x == v && i < idx) better = true;
            if (better) { v = x; idx = i; }
        }
    }
    best[lane] = v;
    at[lane] = idx;
    __syncthreads();
    for (uint32_t stride = 64; stride > 0; stride /= 2) {
        if (lane < stride) {
            const float a = best[lane], b = best[lane + stride];
            if (b > a) { best[lane] = b; at[lane] = at[lane + stride]; }
            else if (b == a && at[lane + stride] < at[lane]) at[lane] = at[lane + stride];
        }
        __syncthreads();
    }
    out_v = best[0];
    out_i = at[0];
    __syncthreads();
}

__device__ void top_keep(const float *__restrict__ w, float *__restrict__ out, uint32_t vocab, float front_v,
                         uint32_t front_i, bool keep_all)
{
    for (uint32_t i = threadIdx.x; i < vocab; i += kRowWidth) {
        const float x = w[i];
        bool keep = x > front_v;
        if (x == front_v && i <= front_i) keep = true;
        if (keep_all) keep = true;
        out[i] = keep ? x : 0.f;
    }
}

// ks != NULL: TopKMaskRows (k per row; 0, or at least the vocabulary once the bound of 128 rounds has
// been applied, passes the row through).  ks == NULL: TopKMask with the uniform k.
__global__ void __launch_bounds__(kRowWidth)
topk_mask_kernel(const float *__restrict__ weights, const uint32_t *__restrict__ ks, uint32_t uniform_k,
                 float *__restrict__ out, uint32_t vocab)
{
    __shared__ float best[kRowWidth];
    __shared__ uint32_t at[kRowWidth];
    const float *w = weights + (size_t)blockIdx.x * vocab;
    uint32_t rounds = ks ? ks[blockIdx.x] : uniform_k;
    if (rounds > kTopMaxRounds) rounds = kTopMaxRounds;
    if (ks && rounds >= vocab) rounds = 0;
    float front_v = kSentinelHi;
    uint32_t front_i = 0;
    for (uint32_t r = 0; r < rounds; r++) top_round(w, vocab, front_v, front_i, best, at, front_v, front_i);
    top_keep(w, out + (size_t)blockIdx.x * vocab, vocab, front_v, front_i, ks && rounds == 0);
}

// ps != NULL: TopPMaskRows (p per row; outside (0, 1) passes the row through).  ps == NULL: TopPMask.
__global__ void __launch_bounds__(kRowWidth)
topp_mask_kernel(const float *__restrict__ weights, const float *__restrict__ ps, float uniform_p,
                 float *__restrict__ out, uint32_t vocab)
{
    __shared__ float best[kRowWidth];
    __shared__ uint32_t at[kRowWidth];
    const uint32_t lane = threadIdx.x;
    const float *w = weights + (size_t)blockIdx.x * vocab;
    const float p = ps ? ps[blockIdx.x] : uniform_p;
    const bool active = ps ? (p > 0.f && p < 1.f) : true;
    float sum = 0.f;
    for (uint32_t i = lane; i < vocab; i += kRowWidth) sum = __fadd_rn(sum, w[i]);
    best[lane] = sum;
    __syncthreads();
    for (uint32_t stride = 64; stride > 0; stride /= 2) {
        if (lane < stride) best[lane] = __fadd_rn(best[lane], best[lane + stride]);
        __syncthreads();
    }
    const float target = __fmul_rn(best[0], p);
    __syncthreads();
    float front_v = kSentinelHi, kept = 0.f;
    uint32_t front_i = 0;
    // the reference walks all 128 rounds and advances the frontier only while the kept mass is below
    // the target; once it is not, the remaining rounds change nothing
    for (uint32_t r = 0; r < kTopMaxRounds && active && kept < target; r++) {
        float bv;
        uint32_t bi;
        top_round(w, vocab, front_v, front_i, best, at, bv, bi);
        front_v = bv;
        front_i = bi;
        kept = __fadd_rn(kept, front_v);
    }
    top_keep(w, out + (size_t)blockIdx.x * vocab, vocab, front_v, front_i, !active);
}

static int launch_mask(Launch &l, bool topk, bool per_row, const char *name)
{
    if (l.query_ws) { l.ws_need = 0; return AB_OK; }
    uint32_t vocab, rows, uk = 0;
    float up = 0.f;
    const int out_i = per_row ? 2 : 1;
    if (per_row) {                                   // weights, ks | ps, out; RowSampleDims
        const RowSampleDims d = row_dims_of(l);
        vocab = d.vocab; rows = d.rows;
        if (l.len[1] < rows) return fail(AB_ERR_INVALID, "%s: %u rows and %u per-row parameters", name, rows, l.len[1]);
    } else {                                         // weights, out; TopDims{Vocab,K,P}; one workgroup per row
        vocab = u32_at(l.u, 0); uk = u32_at(l.u, 4); up = f32_at(l.u, 8);
        rows = vocab ? l.len[0] / vocab : 0;
    }
    if (vocab == 0 || l.len[0] < (uint64_t)rows * vocab || l.len[out_i] < (uint64_t)rows * vocab)
        return fail(AB_ERR_INVALID, "%s: Rows=%u Vocab=%u; weights[%u] out[%u]", name, rows, vocab, l.len[0], l.len[out_i]);
    if (rows == 0) return AB_OK;
    if (topk)
        topk_mask_kernel<<<rows, kRowWidth, 0, l.stream>>>(ptr<const float>(l, 0), per_row ? ptr<const uint32_t>(l, 1) : nullptr,
                                                          uk, ptr<float>(l, out_i), vocab);
    else
        topp_mask_kernel<<<rows, kRowWidth, 0, l.stream>>>(ptr<const float>(l, 0), per_row ? ptr<const float>(l, 1) : nullptr,
                                                          up, ptr<float>(l, out_i), vocab);
    count_launch();
    return check_cuda(cudaGetLastError(), name);
}
int launch_topk_mask_rows(Launch &l) { return launch_mask(l, true, true, "TopKMaskRows"); }
int launch_topp_mask_rows(Launch &l) { return launch_mask(l, false, true, "TopPMaskRows"); }
int launch_topk_mask(Launch &l) { return launch_mask(l, true, false, "TopKMask"); }
int launch_topp_mask(Launch &l) { return launch_mask(l, false, false, "TopPMask"); }

// ---------------------------------------------------------------- the draw
// One CTA per row.  factors != NULL and factors[row] == 0: the row's argmax (first maximum).  Else
// the categorical walk: total = the row summed in index order; target = draw * total; the first
// index whose running sum exceeds the target, else the last index.
static constexpr int kWalkBlock = 2048;        // weights staged in shared memory per step

__device__ float walk_block(const float *blk, uint32_t n, float acc)
{   // one thread, index order, every addition rounded to f32
    for (uint32_t i = 0; i < n; i++) acc = __fadd_rn(acc, blk[i]);
    return acc;
}

__global__ void __launch_bounds__(kRowWidth)
sample_rows_kernel(const float *__restrict__ probs, const float *__restrict__ draws,
                   const float *__restrict__ factors, uint32_t *__restrict__ out, uint32_t vocab)
{
    __shared__ float blk[kWalkBlock];
    __shared__ float s_v[kRowWidth];
    __shared__ uint32_t s_i[kRowWidth];
    __shared__ float s_acc, s_target;
    __shared__ uint32_t s_found;
    const uint32_t row = blockIdx.x, lane = threadIdx.x;
    const float *p = probs + (size_t)row * vocab;
    if (factors && factors[row] == 0.f) {
        float v = kSentinelLo;
        uint32_t idx = 0;
        for (uint32_t i = lane; i < vocab; i += kRowWidth) {
            const float x = p[i];
            if (x > v) { v = x; idx = i; }               // a lane's indices ascend: its first maximum
        }
        s_v[lane] = v; s_i[lane] = idx;
        __syncthreads();
        for (uint32_t stride = kRowWidth / 2; stride > 0; stride /= 2) {
            if (lane < stride) {
                const float a = s_v[lane], b = s_v[lane + stride];
                if (b > a || (b == a && s_i[lane + stride] < s_i[lane])) { s_v[lane] = b; s_i[lane] = s_i[lane + stride]; }
            }
            __syncthreads();
        }
        // the reference keeps index 0 when nothing exceeds its initial -3.4e38
        if (lane == 0) out[row] = s_v[0] > kSentinelLo ? s_i[0] : 0u;
        return;
    }
    // pass 1: the total; pass 2: the walk.  A block whose weights are all zero changes neither.
    for (int pass = 0; pass < 2; pass++) {
        if (lane == 0) { s_acc = 0.f; s_found = 0xffffffffu; }
        __syncthreads();
        for (uint32_t base = 0; base < vocab; base += kWalkBlock) {
            const uint32_t n = min((uint32_t)kWalkBlock, vocab - base);
            bool any = false;
            for (uint32_t i = lane; i < n; i += kRowWidth) {
                const float x = p[base + i];
                blk[i] = x;
                any |= (x != 0.f) || (x != x);
            }
            if (!__syncthreads_or(any)) continue;        // also orders the stores before thread 0's reads
            if (lane == 0) {
                if (pass == 0) {
                    s_acc = walk_block(blk, n, s_acc);
                } else if (s_found == 0xffffffffu) {
                    float acc = s_acc;
                    const float target = s_target;
                    for (uint32_t i = 0; i < n; i++) {
                        acc = __fadd_rn(acc, blk[i]);
                        if (acc > target) { s_found = base + i; break; }
                    }
                    s_acc = acc;
                }
            }
            __syncthreads();
            if (pass == 1 && s_found != 0xffffffffu) break;
        }
        __syncthreads();
        if (pass == 0 && lane == 0) {
            float draw = draws[row];
            if (draw < 0.f) draw = 0.f;
            if (draw > 0.99999994f) draw = 0.99999994f;
            s_target = __fmul_rn(draw, s_acc);
        }
        __syncthreads();
    }
    if (lane == 0) out[row] = s_found != 0xffffffffu ? s_found : vocab - 1;
}

static int launch_sample(Launch &l, bool per_row, const char *name)
{
    if (l.query_ws) { l.ws_need = 0; return AB_OK; }
    uint32_t vocab, rows;
    const int out_i = per_row ? 3 : 2;
    if (per_row) { const RowSampleDims d = row_dims_of(l); vocab = d.vocab; rows = d.rows; }   // probs, draws, factors, out
    else { vocab = u32_at(l.u, 0); rows = u32_at(l.u, 4); }                                    // probs, draws, out; SampleDims
    if (vocab == 0 || l.len[0] < (uint64_t)rows * vocab || l.len[1] < rows || (per_row && l.len[2] < rows) ||
        l.len[out_i] < rows)
        return fail(AB_ERR_INVALID, "%s: Rows=%u Vocab=%u; probs[%u] draws[%u] out[%u]", name, rows, vocab, l.len[0],
                    l.len[1], l.len[out_i]);
    if (rows == 0) return AB_OK;
    sample_rows_kernel<<<rows, kRowWidth, 0, l.stream>>>(ptr<const float>(l, 0), ptr<const float>(l, 1),
                                                        per_row ? ptr<const float>(l, 2) : nullptr,
                                                        ptr<uint32_t>(l, out_i), vocab);
    count_launch();
    return check_cuda(cudaGetLastError(), name);
}
int launch_sample_rows(Launch &l) { return launch_sample(l, true, "SampleRows"); }
int launch_sample_categorical(Launch &l) { return launch_sample(l, false, "SampleCategorical"); }

// ---------------------------------------------------------------- penalties
__global__ void penalty_count_kernel(const uint32_t *__restrict__ history, const uint32_t *__restrict__ filled,
                                     uint32_t uniform_count, uint32_t *__restrict__ counts, uint32_t vocab,
                                     uint32_t history_cap, size_t n)
{
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint32_t row = (uint32_t)(i / history_cap);
    if ((uint32_t)(i - (size_t)row * history_cap) >= (filled ? filled[row] : uniform_count)) return;
    const uint32_t id = history[i];
    if (id < vocab) atomicAdd(&counts[(size_t)row * vocab + id], 1u);     // integer: exact in any order
}

__global__ void penalty_apply_kernel(const float *__restrict__ logits, const uint32_t *__restrict__ counts,
                                     const float *__restrict__ repetition, const float *__restrict__ presence,
                                     const float *__restrict__ frequency, float u_rep, float u_pres, float u_freq,
                                     float *__restrict__ out, uint32_t vocab, size_t n)
{
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint32_t row = (uint32_t)(i / vocab);
    float lg = logits[i];
    const uint32_t c = counts[i];
    if (c == 0) { out[i] = lg; return; }             // an unseen token comes through bit-identical
    const float rep = repetition ? repetition[row] : u_rep;
    if (rep != 0.f && rep != 1.f) lg = lg > 0.f ? __fdiv_rn(lg, rep) : __fmul_rn(lg, rep);
    out[i] = __fsub_rn(__fsub_rn(lg, presence ? presence[row] : u_pres),
                       __fmul_rn(frequency ? frequency[row] : u_freq, (float)c));
}

int launch_penalty_clear_rows(Launch &l)
{   // counts; RowSampleDims
    if (l.query_ws) { l.ws_need = 0; return AB_OK; }
    const RowSampleDims d = row_dims_of(l);
    const uint64_t n = (uint64_t)d.rows * d.vocab;
    if (l.len[0] < n) return fail(AB_ERR_INVALID, "PenaltyClearRows: Rows=%u Vocab=%u; counts[%u]", d.rows, d.vocab, l.len[0]);
    if (n == 0) return AB_OK;
    return check_cuda(cudaMemsetAsync(l.b[0], 0, n * 4, l.stream), "PenaltyClearRows");
}

int launch_penalty_count_rows(Launch &l)
{   // history, filled, counts; RowSampleDims (History = each row's ring capacity)
    if (l.query_ws) { l.ws_need = 0; return AB_OK; }
    const RowSampleDims d = row_dims_of(l);
    const uint64_t n = (uint64_t)d.rows * d.history;
    if (l.len[0] < n || l.len[1] < d.rows || l.len[2] < (uint64_t)d.rows * d.vocab)
        return fail(AB_ERR_INVALID, "PenaltyCountRows: Rows=%u Vocab=%u History=%u; history[%u] filled[%u] counts[%u]",
                    d.rows, d.vocab, d.history, l.len[0], l.len[1], l.len[2]);
    if (n == 0) return AB_OK;
    penalty_count_kernel<<<sp_blocks(n, 256), 256, 0, l.stream>>>(ptr<const uint32_t>(l, 0), ptr<const uint32_t>(l, 1), 0,
                                                                 ptr<uint32_t>(l, 2), d.vocab, d.history, n);
    count_launch();
    return check_cuda(cudaGetLastError(), "PenaltyCountRows");
}

int launch_penalty_apply_rows(Launch &l)
{   // logits, counts, repetition, presence, frequency, out; RowSampleDims
    if (l.query_ws) { l.ws_need = 0; return AB_OK; }
    const RowSampleDims d = row_dims_of(l);
    const uint64_t n = (uint64_t)d.rows * d.vocab;
    if (d.vocab == 0 || l.len[0] < n || l.len[1] < n || l.len[2] < d.rows || l.len[3] < d.rows || l.len[4] < d.rows ||
        l.len[5] < n)
        return fail(AB_ERR_INVALID, "PenaltyApplyRows: Rows=%u Vocab=%u; logits[%u] counts[%u] out[%u]", d.rows, d.vocab,
                    l.len[0], l.len[1], l.len[5]);
    if (n == 0) return AB_OK;
    penalty_apply_kernel<<<sp_blocks(n, 256), 256, 0, l.stream>>>(ptr<const float>(l, 0), ptr<const uint32_t>(l, 1),
                                                                 ptr<const float>(l, 2), ptr<const float>(l, 3),
                                                                 ptr<const float>(l, 4), 0.f, 0.f, 0.f, ptr<float>(l, 5),
                                                                 d.vocab, n);
    count_launch();
    return check_cuda(cudaGetLastError(), "PenaltyApplyRows");
}

// the uniform forms: PenaltyDims{Vocab,History,Count,Repetition,Presence,Frequency}, one row
int launch_penalty_clear(Launch &l)
{   // counts
    if (l.query_ws) { l.ws_need = 0; return AB_OK; }
    const uint32_t vocab = u32_at(l.u, 0);
    if (l.len[0] < vocab) return fail(AB_ERR_INVALID, "PenaltyClear: Vocab=%u; counts[%u]", vocab, l.len[0]);
    if (vocab == 0) return AB_OK;
    return check_cuda(cudaMemsetAsync(l.b[0], 0, (size_t)vocab * 4, l.stream), "PenaltyClear");
}

int launch_penalty_count(Launch &l)
{   // history, counts
    if (l.query_ws) { l.ws_need = 0; return AB_OK; }
    const uint32_t vocab = u32_at(l.u, 0), cap = u32_at(l.u, 4), count = u32_at(l.u, 8);
    if (l.len[0] < count || l.len[1] < vocab)
        return fail(AB_ERR_INVALID, "PenaltyCount: Vocab=%u History=%u Count=%u; history[%u] counts[%u]", vocab, cap,
                    count, l.len[0], l.len[1]);
    if (count == 0) return AB_OK;
    // one row whose ring is `count` entries long and wholly filled
    penalty_count_kernel<<<sp_blocks(count, 256), 256, 0, l.stream>>>(ptr<const uint32_t>(l, 0), nullptr, count,
                                                                     ptr<uint32_t>(l, 1), vocab, count, count);
    count_launch();
    return check_cuda(cudaGetLastError(), "PenaltyCount");
}

int launch_penalty_apply(Launch &l)
{   // logits, counts, out
    if (l.query_ws) { l.ws_need = 0; return AB_OK; }
    const uint32_t vocab = u32_at(l.u, 0);
    if (l.len[0] < vocab || l.len[1] < vocab || l.len[2] < vocab)
        return fail(AB_ERR_INVALID, "PenaltyApply: Vocab=%u; logits[%u] counts[%u] out[%u]", vocab, l.len[0], l.len[1], l.len[2]);
    if (vocab == 0) return AB_OK;
    penalty_apply_kernel<<<sp_blocks(vocab, 256), 256, 0, l.stream>>>(ptr<const float>(l, 0), ptr<const uint32_t>(l, 1),
                                                                     nullptr, nullptr, nullptr, f32_at(l.u, 12),
                                                                     f32_at(l.u, 16), f32_at(l.u, 20), ptr<float>(l, 2),
                                                                     vocab, vocab);
    count_launch();
    return check_cuda(cudaGetLastError(), "PenaltyApply");
}

}  // namespace ab
