// The operators of a decode step that sit between the int4 products and the attention: RMSNorm
// (internal/kernels/norm.go:46), RoPE (elementwise.go:267), SwiGLU (:85), ElemAdd (:22),
// GatherRows (:118,133), ScatterRows (:182,221), SampleArgmax (sample.go:50), the f16 casts
// (cast.go:30,38), and quant.Int4Quantize (quant/int4.go:71) run on the device.
#include "common.cuh"

namespace ab {

static inline unsigned blocks_for(size_t n, int per) { return (unsigned)((n + per - 1) / per); }

// ---------------------------------------------------------------- RMSNorm
// One CTA per row: x * rsqrt(mean(x^2) + eps) * w.
__global__ void __launch_bounds__(256) rmsnorm_kernel(const float *__restrict__ x,
                                                      const float *__restrict__ w,
                                                      float *__restrict__ out, uint32_t width,
                                                      float eps)
{
    __shared__ float red[8];
    pdl_enter();
    const size_t base = (size_t)blockIdx.x * width;
    float acc = 0.f;
    for (uint32_t i = threadIdx.x; i < width; i += 256) { float v = x[base + i]; acc = fmaf(v, v, acc); }
#pragma unroll
    for (int sh = 16; sh > 0; sh >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, sh);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) total += red[i];
    const float scale = (float)(1.0 / sqrt((double)(total / (float)width + eps)));
    for (uint32_t i = threadIdx.x; i < width; i += 256) out[base + i] = x[base + i] * scale * w[i];
}

int launch_rmsnorm(Launch &l)
{   // x, w, out; RowDims{Rows,Width,Eps}
    if (l.query_ws) { l.ws_need = 0; return AB_OK; }
    uint32_t rows = u32_at(l.u, 0), width = u32_at(l.u, 4);
    float eps = f32_at(l.u, 8);
    if (l.len[0] < (uint64_t)rows * width || l.len[1] < width || l.len[2] < (uint64_t)rows * width)
        return fail(AB_ERR_INVALID, "RMSNorm: Rows=%u Width=%u; x[%u] w[%u] out[%u]", rows, width,
                    l.len[0], l.len[1], l.len[2]);
    if (rows == 0) return AB_OK;
    cudaError_t e = launch_dependent(rmsnorm_kernel, dim3(rows), dim3(256), 0, l.stream, ptr<const float>(l, 0),
                                     ptr<const float>(l, 1), ptr<float>(l, 2), width, eps);
    count_launch();
    return check_cuda(e, "RMSNorm");
}

// ---------------------------------------------------------------- RoPE
// Interleaved pairs (2k, 2k+1), one position per row, in place.  The angle is formed the way the
// reference forms it (f32 exponent, exp/log/cos/sin evaluated in binary64 and rounded once) so
// that large positions do not lose their low bits to an f32 range reduction.
__global__ void rope_kernel(const uint32_t *__restrict__ positions, float *__restrict__ inout,
                            uint32_t rows, uint32_t width, uint32_t rotary, float base)
{
    const uint32_t pairs = rotary / 2;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)rows * pairs) return;
    const uint32_t r = (uint32_t)(i / pairs), k = (uint32_t)(i % pairs);
    const float pos = (float)positions[r];
    const float exponent = __fdiv_rn(__fmul_rn(-2.f, (float)k), (float)rotary);
    const float freq = (float)exp((double)__fmul_rn(exponent, (float)log((double)base)));
    const float theta = __fmul_rn(pos, freq);
    double sd, cd;
    sincos((double)theta, &sd, &cd);
    const float c = (float)cd, s = (float)sd;
    const size_t lo = (size_t)r * width + 2 * k;
    const float x = inout[lo], y = inout[lo + 1];
    inout[lo] = __fsub_rn(__fmul_rn(x, c), __fmul_rn(y, s));
    inout[lo + 1] = __fadd_rn(__fmul_rn(x, s), __fmul_rn(y, c));
}

int launch_rope(Launch &l)
{   // positions, inout; RoPEParams{Rows,Width,RotaryDim,Base}
    if (l.query_ws) { l.ws_need = 0; return AB_OK; }
    uint32_t rows = u32_at(l.u, 0), width = u32_at(l.u, 4), rotary = u32_at(l.u, 8);
    float base = f32_at(l.u, 12);
    if (rotary > width || rotary % 2 || l.len[0] < rows || l.len[1] < (uint64_t)rows * width)
        return fail(AB_ERR_INVALID, "RoPE: Rows=%u Width=%u RotaryDim=%u; positions[%u] inout[%u]",
                    rows, width, rotary, l.len[0], l.len[1]);
    size_t n = (size_t)rows * (rotary / 2);
    if (n == 0) return AB_OK;
    rope_kernel<<<blocks_for(n, 128), 128, 0, l.stream>>>(ptr<const uint32_t>(l, 0),
                                                          ptr<float>(l, 1), rows, width, rotary, base); count_launch();
    return check_cuda(cudaGetLastError(), "RoPE");
}

// ---------------------------------------------------------------- elementwise
__global__ void swiglu_kernel(const float *__restrict__ a, const float *__restrict__ b,
                              float *__restrict__ out, size_t n)
{
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) { float x = a[i]; out[i] = __fdiv_rn(x, 1.f + expf(-x)) * b[i]; }
}

__global__ void add_kernel(const float *__restrict__ a, const float *__restrict__ b,
                           float *__restrict__ out, size_t n)
{
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = a[i] + b[i];
}

static int elementwise3(Launch &l, bool swiglu, const char *name)
{   // a, b, out; the element count is len(out), as the reference's guard reads it
    if (l.query_ws) { l.ws_need = 0; return AB_OK; }
    size_t n = l.len[2];
    if (l.len[0] < n || l.len[1] < n)
        return fail(AB_ERR_INVALID, "%s: out[%u] and inputs [%u] [%u]", name, l.len[2], l.len[0], l.len[1]);
    if (n == 0) return AB_OK;
    if (swiglu) { swiglu_kernel<<<blocks_for(n, 256), 256, 0, l.stream>>>(ptr<const float>(l, 0), ptr<const float>(l, 1), ptr<float>(l, 2), n); count_launch(); }
    else { add_kernel<<<blocks_for(n, 256), 256, 0, l.stream>>>(ptr<const float>(l, 0), ptr<const float>(l, 1), ptr<float>(l, 2), n); count_launch(); }
    return check_cuda(cudaGetLastError(), name);
}
int launch_swiglu(Launch &l) { return elementwise3(l, true, "SwiGLU"); }
int launch_elem_add(Launch &l) { return elementwise3(l, false, "ElemAdd"); }

// ---------------------------------------------------------------- gather / scatter rows
template <typename T>
__global__ void gather_rows_kernel(const T *__restrict__ table, const uint32_t *__restrict__ ids,
                                   float *__restrict__ out, uint32_t rows, uint32_t width,
                                   uint32_t capacity)
{
    pdl_enter();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)rows * width) return;
    uint32_t r = (uint32_t)(i / width), c = (uint32_t)(i % width), id = ids[r];
    float v = 0.f;
    if (id < capacity) {
        if constexpr (sizeof(T) == 2) v = __half2float(table[(size_t)id * width + c]);
        else v = table[(size_t)id * width + c];
    }
    out[i] = v;
}

template <typename T>
__global__ void scatter_rows_kernel(const T *__restrict__ rows_in, const uint32_t *__restrict__ ids,
                                    T *__restrict__ state, uint32_t rows, uint32_t width,
                                    uint32_t capacity)
{
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)rows * width) return;
    uint32_t r = (uint32_t)(i / width), c = (uint32_t)(i % width), id = ids[r];
    if (id < capacity) state[(size_t)id * width + c] = rows_in[i];
}

template <typename T> static int gather(Launch &l, const char *name)
{   // table, ids, out; RowParams{Rows,Width,Capacity}
    if (l.query_ws) { l.ws_need = 0; return AB_OK; }
    uint32_t rows = u32_at(l.u, 0), width = u32_at(l.u, 4), cap = u32_at(l.u, 8);
    if (l.len[0] < (uint64_t)cap * width || l.len[1] < rows || l.len[2] < (uint64_t)rows * width)
        return fail(AB_ERR_INVALID, "%s: Rows=%u Width=%u Capacity=%u; table[%u] ids[%u] out[%u]",
                    name, rows, width, cap, l.len[0], l.len[1], l.len[2]);
    size_t n = (size_t)rows * width;
    if (n == 0) return AB_OK;
    cudaError_t e = launch_dependent(gather_rows_kernel<T>, dim3(blocks_for(n, 256)), dim3(256), 0, l.stream,
                                     ptr<const T>(l, 0), ptr<const uint32_t>(l, 1), ptr<float>(l, 2), rows, width, cap);
    count_launch();
    if (e != cudaSuccess) return check_cuda(e, "GatherRows");
    return check_cuda(cudaGetLastError(), name);
}
template <typename T> static int scatter(Launch &l, const char *name)
{   // rows, ids, state; RowParams
    if (l.query_ws) { l.ws_need = 0; return AB_OK; }
    uint32_t rows = u32_at(l.u, 0), width = u32_at(l.u, 4), cap = u32_at(l.u, 8);
    if (l.len[2] < (uint64_t)cap * width || l.len[1] < rows || l.len[0] < (uint64_t)rows * width)
        return fail(AB_ERR_INVALID, "%s: Rows=%u Width=%u Capacity=%u; rows[%u] ids[%u] state[%u]",
                    name, rows, width, cap, l.len[0], l.len[1], l.len[2]);
    size_t n = (size_t)rows * width;
    if (n == 0) return AB_OK;
    scatter_rows_kernel<T><<<blocks_for(n, 256), 256, 0, l.stream>>>(ptr<const T>(l, 0), ptr<const uint32_t>(l, 1), ptr<T>(l, 2), rows, width, cap); count_launch();
    return check_cuda(cudaGetLastError(), name);
}
int launch_gather_rows(Launch &l) { return gather<float>(l, "GatherRows"); }
int launch_gather_rows_f16(Launch &l) { return gather<__half>(l, "GatherRowsF16"); }
int launch_scatter_rows(Launch &l) { return scatter<float>(l, "ScatterRows"); }
int launch_scatter_rows_f16(Launch &l) { return scatter<__half>(l, "ScatterRowsF16"); }

// ---------------------------------------------------------------- argmax
// One CTA per row; the largest logit, ties to the lowest index (sample.go:50-100).
__global__ void __launch_bounds__(256) argmax_kernel(const float *__restrict__ logits,
                                                     uint32_t *__restrict__ out, uint32_t vocab)
{
    __shared__ float bv[8];
    __shared__ uint32_t bi[8];
    pdl_enter();
    const size_t base = (size_t)blockIdx.x * vocab;
    float v = -3.4e38f;
    uint32_t idx = 0;
    for (uint32_t i = threadIdx.x; i < vocab; i += 256) {
        float x = logits[base + i];
        if (x > v) { v = x; idx = i; }
    }
#pragma unroll
    for (int sh = 16; sh > 0; sh >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, v, sh);
        uint32_t oi = __shfl_xor_sync(0xffffffffu, idx, sh);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
    if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = v; bi[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; w++)
            if (bv[w] > v || (bv[w] == v && bi[w] < idx)) { v = bv[w]; idx = bi[w]; }
        out[blockIdx.x] = idx;
    }
}

// The greedy token of a vocabulary split by columns over `parts` ranks (a tensor-parallel lm_head).
// ArgmaxShard: this rank's logits [rows][width] -> pairs [rows][parts][2] f32 where slot `rank` holds
// (largest logit, its index in the WHOLE vocabulary as a float) and every other slot is zero, so the
// element-wise sum of all ranks' pairs (x + 0 = x exactly) is the gather of their slots: 8 bytes per
// rank and row cross NVLink instead of the padded logits.  ArgmaxMerge picks the largest value,
// the lowest index among equals: the row's SampleArgmax over the unsplit logits
// (internal/kernels/sample.go), since every rank applies the same rule to its columns.
__global__ void __launch_bounds__(256) argmax_shard_kernel(const float *__restrict__ logits, float *__restrict__ pairs,
                                                           uint32_t width, uint32_t parts, uint32_t rank, uint32_t first)
{
    __shared__ float bv[8];
    __shared__ uint32_t bi[8];
    pdl_enter();
    const size_t base = (size_t)blockIdx.x * width;
    float v = -3.4e38f;
    uint32_t idx = 0;
    for (uint32_t i = threadIdx.x; i < width; i += 256) {
        float x = logits[base + i];
        if (x > v) { v = x; idx = i; }
    }
#pragma unroll
    for (int sh = 16; sh > 0; sh >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, v, sh);
        uint32_t oi = __shfl_xor_sync(0xffffffffu, idx, sh);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
    if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = v; bi[threadIdx.x >> 5] = idx; }
    __syncthreads();
    float *row = pairs + (size_t)blockIdx.x * parts * 2;
    for (uint32_t i = threadIdx.x; i < parts * 2; i += 256)
        if (i / 2 != rank) row[i] = 0.f;
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; w++)
            if (bv[w] > v || (bv[w] == v && bi[w] < idx)) { v = bv[w]; idx = bi[w]; }
        row[2 * rank] = v;
        row[2 * rank + 1] = (float)(first + idx);        // exact: the vocabulary is below 2^24
    }
}

__global__ void argmax_merge_kernel(const float *__restrict__ pairs, uint32_t *__restrict__ out, uint32_t rows,
                                    uint32_t parts)
{
    pdl_enter();
    const uint32_t r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    const float *row = pairs + (size_t)r * parts * 2;
    float v = row[0];
    uint32_t idx = (uint32_t)row[1];
    for (uint32_t s = 1; s < parts; s++) {
        const float ov = row[2 * s];
        const uint32_t oi = (uint32_t)row[2 * s + 1];
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
    out[r] = idx;
}

int launch_argmax_shard(Launch &l)
{   // logits, pairs; {Width, Rows, Parts, Rank, First, 0, 0, 0}
    if (l.query_ws) { l.ws_need = 0; return AB_OK; }
    const uint32_t width = u32_at(l.u, 0), rows = u32_at(l.u, 4), parts = u32_at(l.u, 8), rank = u32_at(l.u, 12),
                   first = u32_at(l.u, 16);
    if (parts == 0 || rank >= parts || (uint64_t)first + width > (1u << 24))
        return fail(AB_ERR_INVALID, "ArgmaxShard: Parts=%u Rank=%u First=%u Width=%u; indices are carried as floats "
                    "and stay below 2^24", parts, rank, first, width);
    if (l.len[0] < (uint64_t)rows * width || l.len[1] < (uint64_t)rows * parts * 2)
        return fail(AB_ERR_INVALID, "ArgmaxShard: Rows=%u Width=%u Parts=%u; logits[%u] pairs[%u]", rows, width, parts,
                    l.len[0], l.len[1]);
    if (rows == 0) return AB_OK;
    cudaError_t e = launch_dependent(argmax_shard_kernel, dim3(rows), dim3(256), 0, l.stream, ptr<const float>(l, 0),
                                     ptr<float>(l, 1), width, parts, rank, first);
    count_launch();
    return check_cuda(e, "ArgmaxShard");
}

int launch_argmax_merge(Launch &l)
{   // pairs, out; {Rows, Parts, 0, 0}
    if (l.query_ws) { l.ws_need = 0; return AB_OK; }
    const uint32_t rows = u32_at(l.u, 0), parts = u32_at(l.u, 4);
    if (parts == 0 || l.len[0] < (uint64_t)rows * parts * 2 || l.len[1] < rows)
        return fail(AB_ERR_INVALID, "ArgmaxMerge: Rows=%u Parts=%u; pairs[%u] out[%u]", rows, parts, l.len[0], l.len[1]);
    if (rows == 0) return AB_OK;
    cudaError_t e = launch_dependent(argmax_merge_kernel, dim3((rows + 63) / 64), dim3(64), 0, l.stream,
                                     ptr<const float>(l, 0), ptr<uint32_t>(l, 1), rows, parts);
    count_launch();
    return check_cuda(e, "ArgmaxMerge");
}

int launch_sample_argmax(Launch &l)
{   // logits, out; SampleDims{Vocab,Rows}; rows = len(out), one reference workgroup per row
    if (l.query_ws) { l.ws_need = 0; return AB_OK; }
    uint32_t vocab = u32_at(l.u, 0), rows = l.len[1];
    if (l.len[0] < (uint64_t)rows * vocab)
        return fail(AB_ERR_INVALID, "SampleArgmax: Vocab=%u rows=%u; logits[%u]", vocab, rows, l.len[0]);
    if (rows == 0) return AB_OK;
    cudaError_t e = launch_dependent(argmax_kernel, dim3(rows), dim3(256), 0, l.stream, ptr<const float>(l, 0),
                                     ptr<uint32_t>(l, 1), vocab);
    count_launch();
    return check_cuda(e, "SampleArgmax");
}

// ---------------------------------------------------------------- casts
__global__ void cast_f32_f16_kernel(const float *__restrict__ in, uint16_t *__restrict__ out, size_t n)
{
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = f32_to_f16_ref(in[i]);
}
__global__ void cast_f16_f32_kernel(const __half *__restrict__ in, float *__restrict__ out, size_t n)
{
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __half2float(in[i]);
}
int launch_cast_f32_to_f16(Launch &l)
{
    if (l.query_ws) { l.ws_need = 0; return AB_OK; }
    size_t n = l.len[1];
    if (l.len[0] < n) return fail(AB_ERR_INVALID, "CastF32ToF16: in[%u] out[%u]", l.len[0], l.len[1]);
    if (n) { cast_f32_f16_kernel<<<blocks_for(n, 256), 256, 0, l.stream>>>(ptr<const float>(l, 0), ptr<uint16_t>(l, 1), n); count_launch(); }
    return check_cuda(cudaGetLastError(), "CastF32ToF16");
}
int launch_cast_f16_to_f32(Launch &l)
{
    if (l.query_ws) { l.ws_need = 0; return AB_OK; }
    size_t n = l.len[1];
    if (l.len[0] < n) return fail(AB_ERR_INVALID, "CastF16ToF32: in[%u] out[%u]", l.len[0], l.len[1]);
    if (n) { cast_f16_f32_kernel<<<blocks_for(n, 256), 256, 0, l.stream>>>(ptr<const __half>(l, 0), ptr<float>(l, 1), n); count_launch(); }
    return check_cuda(cudaGetLastError(), "CastF16ToF32");
}


// ---------------------------------------------------------------- per-step inputs of a decode loop
// What a caller's host loop writes before each step (docs/tutorial/11-batching-sequences.md:
// 83-103), computed on the device so that a replayed step can feed the next one without a host
// round trip: the sampled token becomes the input token, its position is the sequence's current
// length, its cache slot is pages[s][pos / Block] * Block + pos % Block, and the length grows by one.
__global__ void decode_step_inputs_kernel(const uint32_t *__restrict__ sampled,
                                          const uint32_t *__restrict__ pages,
                                          uint32_t *__restrict__ tokens, uint32_t *__restrict__ pos_q,
                                          uint32_t *__restrict__ pos_k, uint32_t *__restrict__ slots,
                                          uint32_t *__restrict__ lengths, uint32_t batch, uint32_t hq,
                                          uint32_t hk, uint32_t block, uint32_t max_pages)
{
    pdl_enter();
    const uint32_t s = blockIdx.x;
    if (s >= batch) return;
    const uint32_t pos = lengths[s];
    for (uint32_t i = threadIdx.x; i < hq; i += blockDim.x) pos_q[s * hq + i] = pos;
    for (uint32_t i = threadIdx.x; i < hk; i += blockDim.x) pos_k[s * hk + i] = pos;
    __syncthreads();
    if (threadIdx.x == 0) {
        tokens[s] = sampled[s];
        const uint32_t page = pos / block < max_pages ? pages[(size_t)s * max_pages + pos / block] : 0xffffffffu;
        // past the page table's reach there is no slot: an id ScatterRows drops
        slots[s] = page == 0xffffffffu ? 0xffffffffu : page * block + pos % block;
        lengths[s] = pos + 1;
    }
}

int launch_decode_step_inputs(Launch &l)
{   // sampled, pages, tokens, pos_q, pos_k, slots, lengths; {Batch, QHeads, KVHeads, Block, MaxPages}
    if (l.query_ws) { l.ws_need = 0; return AB_OK; }
    uint32_t batch = u32_at(l.u, 0), hq = u32_at(l.u, 4), hk = u32_at(l.u, 8), block = u32_at(l.u, 12),
             mp = u32_at(l.u, 16);
    if (block == 0 || l.len[0] < batch || l.len[1] < (uint64_t)batch * mp || l.len[2] < batch ||
        l.len[3] < (uint64_t)batch * hq || l.len[4] < (uint64_t)batch * hk || l.len[5] < batch ||
        l.len[6] < batch)
        return fail(AB_ERR_INVALID, "DecodeStepInputs: Batch=%u QHeads=%u KVHeads=%u Block=%u "
                    "MaxPages=%u does not match the lengths block", batch, hq, hk, block, mp);
    if (batch == 0) return AB_OK;
    cudaError_t e = launch_dependent(decode_step_inputs_kernel, dim3(batch), dim3(64), 0, l.stream,
                                     ptr<const uint32_t>(l, 0), ptr<const uint32_t>(l, 1), ptr<uint32_t>(l, 2),
                                     ptr<uint32_t>(l, 3), ptr<uint32_t>(l, 4), ptr<uint32_t>(l, 5), ptr<uint32_t>(l, 6),
                                     batch, hq, hk, block, mp);
    count_launch();
    return check_cuda(e, "DecodeStepInputs");
}

// ---------------------------------------------------------------- quant.Int4Quantize on the device
// One warp per group of 128 weights, four per lane.  Every arithmetic step is the host routine's:
// f32 min/max and (hi-lo)/15, scale and zero round-tripped through f16 with the reference's
// rounding, the code from a binary64 divide and add rounded to nearest even, clamped to [0,15].
__global__ void __launch_bounds__(256) int4_quantize_kernel(const float *__restrict__ w, size_t n,
                                                            uint32_t *__restrict__ packed,
                                                            uint16_t *__restrict__ scales,
                                                            uint16_t *__restrict__ zeros)
{
    const size_t g = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    const size_t lo = g * 128;
    if (lo >= n) return;
    const size_t i0 = lo + (size_t)lane * 4;
    float v[4];
    bool has[4];
#pragma unroll
    for (int j = 0; j < 4; j++) { has[j] = i0 + j < n; v[j] = has[j] ? w[i0 + j] : 0.f; }
    const float first = w[lo];
    float mn = first, mx = first;
#pragma unroll
    for (int j = 0; j < 4; j++) if (has[j]) { mn = fminf(mn, v[j]); mx = fmaxf(mx, v[j]); }
#pragma unroll
    for (int sh = 16; sh > 0; sh >>= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, sh));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, sh));
    }
    uint32_t codes = 0;
    uint16_t s_bits, z_bits;
    if (mx == mn) {
        s_bits = f32_to_f16_ref(0.f);
        z_bits = f32_to_f16_ref(mn);
    } else {
        s_bits = f32_to_f16_ref(__fdiv_rn(__fsub_rn(mx, mn), 15.f));
        const float s16 = f16_bits_to_f32(s_bits);
        if (s16 == 0.f) {
            z_bits = f32_to_f16_ref(mn);
        } else {
            z_bits = f32_to_f16_ref(__fdiv_rn(-mn, s16));
            const double z16 = (double)f16_bits_to_f32(z_bits);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                double q = rint(__dadd_rn(__ddiv_rn((double)v[j], (double)s16), z16));
                q = q > 15.0 ? 15.0 : q;
                q = q < 0.0 ? 0.0 : q;
                if (has[j]) codes |= (uint32_t)q << (4 * j);
            }
        }
    }
    // two lanes make a word: the even lane holds nibbles 0..3, the odd lane 4..7
    const uint32_t other = __shfl_down_sync(0xffffffffu, codes, 1);
    if ((lane & 1) == 0 && i0 < n) packed[i0 / 8] = codes | (other << 16);
    if (lane == 0) { scales[g] = s_bits; zeros[g] = z_bits; }
}

int launch_int4_quantize(Launch &l)
{   // w, packed, scales, zeros; no uniform block; n = len(w)
    if (l.query_ws) { l.ws_need = 0; return AB_OK; }
    size_t n = l.len[0];
    size_t groups = (n + 127) / 128;
    if (l.len[1] < (n + 7) / 8 || l.len[2] < groups || l.len[3] < groups)
        return fail(AB_ERR_INVALID, "Int4Quantize: %zu weights need %zu words and %zu groups; "
                    "packed[%u] scales[%u] zeros[%u]", n, (n + 7) / 8, groups, l.len[1], l.len[2], l.len[3]);
    if (n == 0) return AB_OK;
    int4_quantize_kernel<<<blocks_for(groups, 8), 256, 0, l.stream>>>(
        ptr<const float>(l, 0), n, ptr<uint32_t>(l, 1), ptr<uint16_t>(l, 2), ptr<uint16_t>(l, 3)); count_launch();
    return check_cuda(cudaGetLastError(), "Int4Quantize");
}

}  // namespace ab
