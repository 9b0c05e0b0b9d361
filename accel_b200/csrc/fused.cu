// Fused forms of support operators that follow one another in a decode step.  Extensions: the
// reference records each operator as its own dispatch (ElemAdd, RMSNorm, RoPE, ScatterRows,
// CastF32ToF16); inside a replayed graph every small kernel costs a few microseconds of fixed time,
// and a 7B-shape step has ten of them per layer.  Each fused kernel performs exactly the arithmetic
// of the operators it replaces, in the same order, so its results are bit-identical to the chain.
#include <cuda_fp16.h>

#include "common.cuh"

namespace ab {

static inline unsigned blocks_for(size_t n, int per) { return (unsigned)((n + per - 1) / per); }

// ---------------------------------------------------------------- ElemAdd -> RMSNorm
// sum = x + delta (internal/kernels/elementwise.go:22), norm = sum * rsqrt(mean(sum^2) + eps) * w
// (internal/kernels/norm.go:46).  One CTA per row; the row stays in registers between the two.
template <int PER>
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(const float *__restrict__ x, const float *__restrict__ delta,
                                                          const float *__restrict__ w, float *__restrict__ sum_out,
                                                          float *__restrict__ norm_out, uint32_t width, float eps,
                                                          float *__restrict__ amax_out)
{
    __shared__ float red[8];
    __shared__ uint32_t red_mx[8];
    pdl_enter();
    const size_t base = (size_t)blockIdx.x * width;
    float v[PER];
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < PER; j++) {
        const uint32_t i = threadIdx.x + 256 * j;
        v[j] = 0.f;
        if (i < width) {
            v[j] = __fadd_rn(x[base + i], delta[base + i]);
            sum_out[base + i] = v[j];
            acc = fmaf(v[j], v[j], acc);
        }
    }
#pragma unroll
    for (int sh = 16; sh > 0; sh >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, sh);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) total += red[i];
    const float scale = (float)(1.0 / sqrt((double)(total / (float)width + eps)));
#pragma unroll
    uint32_t mx = 0;
#pragma unroll
    for (int j = 0; j < PER; j++) {
        const uint32_t i = threadIdx.x + 256 * j;
        if (i < width) {
            const float o = v[j] * scale * w[i];
            norm_out[base + i] = o;
            mx = max(mx, __float_as_uint(fabsf(o)));
        }
    }
    if (amax_out) {
        // the row's largest magnitude, for the int4 product that reads the row next (it scales its f16
        // operand by a power of two taken from it): the product then needs no kernel of its own for it
        mx = __reduce_max_sync(0xffffffffu, mx);
        if ((threadIdx.x & 31) == 0) red_mx[threadIdx.x >> 5] = mx;
        __syncthreads();
        if (threadIdx.x == 0) {
#pragma unroll
            for (int i = 1; i < 8; i++) mx = max(mx, red_mx[i]);
            amax_out[blockIdx.x] = __uint_as_float(mx);
        }
    }
}

static int launch_add_rmsnorm_any(Launch &l, bool with_amax);
int launch_add_rmsnorm(Launch &l) { return launch_add_rmsnorm_any(l, false); }
// x, delta, w, sum_out, norm_out, amax_out f32[rows]; RowDims: AddRMSNorm that also leaves every row's largest
// |norm| for the prepacked int4 product that follows (QuantMatMulInt4Packed...A)
int launch_add_rmsnorm_amax(Launch &l) { return launch_add_rmsnorm_any(l, true); }

static int launch_add_rmsnorm_any(Launch &l, bool with_amax)
{   // x, delta, w, sum_out, norm_out[, amax_out]; RowDims{Rows,Width,Eps}
    if (l.query_ws) { l.ws_need = 0; return AB_OK; }
    uint32_t rows = u32_at(l.u, 0), width = u32_at(l.u, 4);
    float eps = f32_at(l.u, 8);
    const uint64_t n = (uint64_t)rows * width;
    if (l.len[0] < n || l.len[1] < n || l.len[2] < width || l.len[3] < n || l.len[4] < n)
        return fail(AB_ERR_INVALID, "AddRMSNorm: Rows=%u Width=%u; x[%u] delta[%u] w[%u] sum[%u] norm[%u]",
                    rows, width, l.len[0], l.len[1], l.len[2], l.len[3], l.len[4]);
    if (width > 256 * 32)
        return fail(AB_ERR_INVALID, "AddRMSNorm: Width=%u (at most %u; use ElemAdd and RMSNorm)", width, 256 * 32);
    if (rows == 0) return AB_OK;
    auto a = ptr<const float>(l, 0), d = ptr<const float>(l, 1), w = ptr<const float>(l, 2);
    auto s = ptr<float>(l, 3), o = ptr<float>(l, 4);
    float *mx = nullptr;
    if (with_amax) {
        if (l.len[5] < rows) return fail(AB_ERR_INVALID, "AddRMSNormAmax: Rows=%u; amax[%u]", rows, l.len[5]);
        mx = ptr<float>(l, 5);
    }
    cudaError_t e;
    if (width <= 256 * 4) e = launch_dependent(add_rmsnorm_kernel<4>, dim3(rows), dim3(256), 0, l.stream, a, d, w, s, o, width, eps, mx);
    else if (width <= 256 * 16) e = launch_dependent(add_rmsnorm_kernel<16>, dim3(rows), dim3(256), 0, l.stream, a, d, w, s, o, width, eps, mx);
    else e = launch_dependent(add_rmsnorm_kernel<32>, dim3(rows), dim3(256), 0, l.stream, a, d, w, s, o, width, eps, mx);
    count_launch();
    return check_cuda(e, "AddRMSNorm");
}

// ---------------------------------------------------------------- RoPE(q), RoPE(k), ScatterRows(k), ScatterRows(v)
// What a decode layer does between its q/k/v products and attention: rotate q and k in place
// (internal/kernels/elementwise.go:267, interleaved pairs, the angle formed as the reference forms
// it), then append this token's k and v rows to the paged cache at the row's slot
// (internal/kernels/elementwise.go:182; a slot >= Capacity is dropped).  For an f16 cache the rows
// are narrowed with the reference's rounding on the way (internal/kernels/cast.go:30).
struct RopeScatterDims { uint32_t batch, q_heads, kv_heads, head_dim, rotary, capacity; float base; uint32_t pad; };

__device__ __forceinline__ void rope_pair(float pos, uint32_t k, uint32_t rotary, float base, float &x, float &y)
{
    const float exponent = __fdiv_rn(__fmul_rn(-2.f, (float)k), (float)rotary);
    const float freq = (float)exp((double)__fmul_rn(exponent, (float)log((double)base)));
    const float theta = __fmul_rn(pos, freq);
    double sd, cd;
    sincos((double)theta, &sd, &cd);
    const float c = (float)cd, s = (float)sd;
    const float x0 = x, y0 = y;
    x = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(y0, s));
    y = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(y0, c));
}

__device__ __forceinline__ void store_cache(float *p, float v) { *p = v; }
__device__ __forceinline__ void store_cache(uint16_t *p, float v) { *p = f32_to_f16_ref(v); }

// work items are pairs of adjacent elements: first the q pairs, then the k pairs, then the v pairs
template <typename T>
__global__ void rope_scatter_kernel(const uint32_t *__restrict__ pos_q, const uint32_t *__restrict__ pos_k,
                                    const uint32_t *__restrict__ slots, float *__restrict__ q,
                                    float *__restrict__ k, const float *__restrict__ v,
                                    T *__restrict__ k_cache, T *__restrict__ v_cache, RopeScatterDims d)
{
    pdl_enter();
    const uint32_t half = d.head_dim / 2, rot_pairs = d.rotary / 2;
    const size_t nq = (size_t)d.batch * d.q_heads * half, nk = (size_t)d.batch * d.kv_heads * half;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < nq) {
        const uint32_t r = (uint32_t)(i / half), p = (uint32_t)(i % half);
        if (p < rot_pairs) {
            float *e = q + (size_t)r * d.head_dim + 2 * p;
            float x = e[0], y = e[1];
            rope_pair((float)pos_q[r], p, d.rotary, d.base, x, y);
            e[0] = x; e[1] = y;
        }
        return;
    }
    i -= nq;
    if (i >= 2 * nk) return;
    const bool is_v = i >= nk;
    if (is_v) i -= nk;
    const uint32_t r = (uint32_t)(i / half), p = (uint32_t)(i % half);      // r = row of [batch * kv_heads]
    const uint32_t b = r / d.kv_heads, h = r % d.kv_heads;
    const size_t at = (size_t)r * d.head_dim + 2 * p;
    float x, y;
    if (is_v) {
        x = v[at]; y = v[at + 1];
    } else {
        x = k[at]; y = k[at + 1];
        if (p < rot_pairs) {
            rope_pair((float)pos_k[r], p, d.rotary, d.base, x, y);
            k[at] = x; k[at + 1] = y;
        }
    }
    const uint32_t slot = slots[b];
    if (slot < d.capacity) {
        T *dst = (is_v ? v_cache : k_cache) + ((size_t)slot * d.kv_heads + h) * d.head_dim + 2 * p;
        store_cache(dst, x);
        store_cache(dst + 1, y);
    }
}

template <typename T> static int rope_scatter(Launch &l, const char *name)
{   // pos_q, pos_k, slots, q, k, v, k_cache, v_cache; RopeScatterDims
    if (l.query_ws) { l.ws_need = 0; return AB_OK; }
    RopeScatterDims d;
    memcpy(&d, l.u, sizeof d);
    const uint64_t nq = (uint64_t)d.batch * d.q_heads * d.head_dim, nk = (uint64_t)d.batch * d.kv_heads * d.head_dim;
    const uint64_t cache = (uint64_t)d.capacity * d.kv_heads * d.head_dim;
    if (d.head_dim % 2 || d.rotary % 2 || d.rotary > d.head_dim || l.len[0] < (uint64_t)d.batch * d.q_heads ||
        l.len[1] < (uint64_t)d.batch * d.kv_heads || l.len[2] < d.batch || l.len[3] < nq || l.len[4] < nk ||
        l.len[5] < nk || l.len[6] < cache || l.len[7] < cache)
        return fail(AB_ERR_INVALID, "%s: Batch=%u QHeads=%u KVHeads=%u HeadDim=%u RotaryDim=%u Capacity=%u; "
                    "pos_q[%u] pos_k[%u] slots[%u] q[%u] k[%u] v[%u] k_cache[%u] v_cache[%u]", name, d.batch,
                    d.q_heads, d.kv_heads, d.head_dim, d.rotary, d.capacity, l.len[0], l.len[1], l.len[2],
                    l.len[3], l.len[4], l.len[5], l.len[6], l.len[7]);
    const size_t items = (size_t)(nq + 2 * nk) / 2;
    if (items == 0) return AB_OK;
    cudaError_t e = launch_dependent(rope_scatter_kernel<T>, dim3(blocks_for(items, 128)), dim3(128), 0, l.stream,
                                     ptr<const uint32_t>(l, 0), ptr<const uint32_t>(l, 1), ptr<const uint32_t>(l, 2),
                                     ptr<float>(l, 3), ptr<float>(l, 4), ptr<const float>(l, 5), ptr<T>(l, 6),
                                     ptr<T>(l, 7), d);
    count_launch();
    return check_cuda(e, name);
}
int launch_rope_scatter_qkv(Launch &l) { return rope_scatter<float>(l, "RopeScatterQKV"); }
int launch_rope_scatter_qkv_f16(Launch &l) { return rope_scatter<uint16_t>(l, "RopeScatterQKVF16"); }

}  // namespace ab
