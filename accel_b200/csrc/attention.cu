// Decode attention over a KV cache: contiguous (internal/kernels/attention.go:97,422), paged
// (paged.go:47,362), batched (batched.go:53) and ragged (ragged.go:61, raggedf16.go:43).
//
// All of them are one computation per (query row, KV head): softmax(q.K^T * scale) V over the
// positions the row may see, with K/V rows reached through a page table,
//
//   physical(j) = pages[j / Block] * Block + j % Block,   row = (physical * KVHeads + kvHead) * HeadDim
//
// The reference walks the cache in blocks of 128 with a running softmax and launches one workgroup
// per QUERY head, so grouped-query heads re-read their shared K/V.  Here a CTA owns one
// (row, KV head, context partition): its warps stream K and V rows once with 128-bit loads, keep
// every query head of the group in registers, and carry their own running (max, sum, output); the
// warps are merged through shared memory and the partitions by a second kernel (split-K).  The
// recurrence is the reference's (alpha = exp(m - m')), applied across warps and partitions instead
// of across blocks, so the result differs from the reference's only by summation order.
//
// Edge semantics kept from the reference: a length beyond the page table's reach is clamped to the
// reach; positions past the length are never read; a zero length gives 0/0 = NaN; ragged padding
// tokens and tokens with no position write zeros.
#include <math_constants.h>

#include <cstdlib>
#include <mutex>

#include "common.cuh"

namespace ab {

static constexpr int kWarps = 4;
static constexpr int kAttnThreads = kWarps * 32;
static constexpr int kPartition = 256;      // positions per context partition when the grid fills the device
static constexpr int kPosUnroll = 4;
static constexpr float kLog2e = 1.4426950408889634f;
static constexpr float kNegBig = -3.0e38f;

enum Mode { kContiguous = 0, kPaged = 1, kBatched = 2, kRagged = 3, kPrefill = 4 };

struct AttnParams {
    const float *q;
    const void *k, *v;
    const uint32_t *pages, *lengths, *offsets;
    float *out;
    float *out_max;     // NULL, or [rows][qH][4]: the largest |out| of the elements each warp of the kernel
                        // that wrote the head wrote (NaN counts as the largest; entries nobody wrote for are 0)
    float *part_o;      // [rows][qH][parts][D]
    float2 *part_ml;    // [rows][qH][parts]
    uint32_t rows;      // sequences (batched), tokens (ragged), 1 otherwise
    uint32_t batch, q_heads, kv_heads, head_dim, block, max_pages, parts;
    uint32_t psize;     // positions per context partition: 256, or 128 / 64 where that many would not fill the SMs
    uint32_t capacity;  // positions the page table (or the contiguous cache) can address
    float scale_log2;   // Scale * log2(e)
    int mode;
    uint32_t base;      // prefill: query row s sees positions <= base + s
};

// One warp wrote a whole head (r4: this lane's four elements, on: the lane holds any): entry 0 of
// the head's four maxima is the largest magnitude, the others 0.  Magnitudes compare by their bit
// patterns, so that a NaN is the largest.  All 32 lanes call.
__device__ __forceinline__ void head_max_store(float *slot, const float4 &r4, bool on, int lane)
{
    uint32_t b = max(max(__float_as_uint(fabsf(r4.x)), __float_as_uint(fabsf(r4.y))),
                     max(__float_as_uint(fabsf(r4.z)), __float_as_uint(fabsf(r4.w))));
    b = __reduce_max_sync(0xffffffffu, on ? b : 0u);
    if (lane < 4) slot[lane] = lane == 0 ? __uint_as_float(b) : 0.f;
}

// What one query row may see.
struct RowView { const uint32_t *pages; uint32_t len; bool zero; };

__device__ __forceinline__ RowView row_view(const AttnParams &p, uint32_t row)
{
    RowView rv{p.pages, 0, false};
    if (p.mode == kRagged) {
        uint32_t seq = 0;
        for (uint32_t r = 0; r < p.batch; r++) seq += (p.offsets[r + 1] <= row) ? 1u : 0u;
        if (seq >= p.batch) { rv.zero = true; return rv; }
        uint32_t i = row - p.offsets[seq], n = p.offsets[seq + 1] - p.offsets[seq];
        uint32_t kv_len = p.lengths[seq];
        if (kv_len + i < n) { rv.zero = true; return rv; }
        uint32_t limit = kv_len + i - n;
        uint32_t vis = min(min(limit + 1, kv_len), p.capacity);
        rv.len = vis;
        rv.pages = p.pages + (size_t)seq * p.max_pages;
    } else if (p.mode == kBatched) {
        rv.len = min(p.lengths[row], p.capacity);
        rv.pages = p.pages + (size_t)row * p.max_pages;
    } else if (p.mode == kPrefill) {
        // one sequence, query row `row` of it: the causal limit and the cache length both bound it
        // (internal/kernels/prefill.go:436-470); base + row + 1 cannot wrap for any cache that exists
        rv.len = min(min(p.base + row + 1, p.lengths[0]), p.capacity);
    } else {
        rv.len = min(p.lengths[0], p.capacity);
    }
    return rv;
}

template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ float4 load(const float *p)
    {
        float4 v;
        asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
                     : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
        return v;
    }
};
template <> struct Vec4<__half> {
    static __device__ __forceinline__ float4 load(const __half *p)
    {
        uint2 raw;
        asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];"
                     : "=r"(raw.x), "=r"(raw.y) : "l"(p));
        float2 a = __half22float2(*reinterpret_cast<__half2 *>(&raw.x));
        float2 b = __half22float2(*reinterpret_cast<__half2 *>(&raw.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
};

// grid = (parts, kv_heads, rows).  G = query heads per KV head.
template <typename T, int G>
__global__ void __launch_bounds__(kAttnThreads)
attn_partition_kernel(const AttnParams p)
{
    // With G > 1 blockIdx.y is a KV head and the CTA serves its G query heads; with G == 1 it is
    // a query head, which also covers group widths that have no instantiation.
    pdl_wait();          // the kernel runs in several waves: its dependent starts as the last one drains
    const uint32_t part = blockIdx.x, row = blockIdx.z;
    const uint32_t hq0 = blockIdx.y * G;
    const uint32_t kvh = G == 1 ? blockIdx.y / (p.q_heads / p.kv_heads) : blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t D = p.head_dim;
    const bool lane_on = (uint32_t)lane * 4 < D;

    const RowView rv = row_view(p, row);
    const uint32_t begin = part * p.psize;
    if (rv.zero) {
        if (part == 0) {
            for (uint32_t i = threadIdx.x; i < G * D; i += kAttnThreads)
                p.out[((size_t)row * p.q_heads + hq0) * D + i] = 0.f;
            if (p.out_max && threadIdx.x < G * 4) p.out_max[((size_t)row * p.q_heads + hq0) * 4 + threadIdx.x] = 0.f;
        }
        return;
    }
    if (begin >= rv.len && !(part == 0)) return;     // partition 0 always reports (len 0 -> NaN)
    const uint32_t end = min(rv.len, begin + p.psize);

    const T *kc = reinterpret_cast<const T *>(p.k);
    const T *vc = reinterpret_cast<const T *>(p.v);
    const size_t row_stride = (size_t)p.kv_heads * D;
    const size_t head_off = (size_t)kvh * D + (size_t)lane * 4;

    float4 qv[G];
#pragma unroll
    for (int g = 0; g < G; g++) {
        qv[g] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (lane_on)
            qv[g] = *reinterpret_cast<const float4 *>(
                p.q + ((size_t)row * p.q_heads + hq0 + g) * D + lane * 4);
        qv[g].x *= p.scale_log2; qv[g].y *= p.scale_log2;
        qv[g].z *= p.scale_log2; qv[g].w *= p.scale_log2;
    }

    float m[G], l[G];
    float4 o[G];
#pragma unroll
    for (int g = 0; g < G; g++) { m[g] = kNegBig; l[g] = 0.f; o[g] = make_float4(0.f, 0.f, 0.f, 0.f); }

    for (uint32_t j0 = begin + warp; j0 < end; j0 += kWarps * kPosUnroll) {
        float4 kv[kPosUnroll], vv[kPosUnroll];
        bool ok[kPosUnroll];
#pragma unroll
        for (int u = 0; u < kPosUnroll; u++) {
            uint32_t j = j0 + u * kWarps;
            ok[u] = j < end;
            kv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            vv[u] = kv[u];
            if (ok[u] && lane_on) {
                size_t phys = rv.pages == nullptr           // a contiguous cache has no page table
                                  ? (size_t)j
                                  : (size_t)__ldg(rv.pages + j / p.block) * p.block + j % p.block;
                const size_t off = phys * row_stride + head_off;
                kv[u] = Vec4<T>::load(kc + off);
                vv[u] = Vec4<T>::load(vc + off);
            }
        }
        float s[kPosUnroll][G];
#pragma unroll
        for (int u = 0; u < kPosUnroll; u++)
#pragma unroll
            for (int g = 0; g < G; g++)
                s[u][g] = qv[g].x * kv[u].x + qv[g].y * kv[u].y + qv[g].z * kv[u].z + qv[g].w * kv[u].w;
#pragma unroll
        for (int sh = 16; sh > 0; sh >>= 1)
#pragma unroll
            for (int u = 0; u < kPosUnroll; u++)
#pragma unroll
                for (int g = 0; g < G; g++) s[u][g] += __shfl_xor_sync(0xffffffffu, s[u][g], sh);
#pragma unroll
        for (int g = 0; g < G; g++) {
            float mx = m[g];
#pragma unroll
            for (int u = 0; u < kPosUnroll; u++) mx = ok[u] ? fmaxf(mx, s[u][g]) : mx;
            const float alpha = exp2f(m[g] - mx);
            m[g] = mx;
            float sum = 0.f;
            float4 acc = make_float4(o[g].x * alpha, o[g].y * alpha, o[g].z * alpha, o[g].w * alpha);
#pragma unroll
            for (int u = 0; u < kPosUnroll; u++) {
                const float e = ok[u] ? exp2f(s[u][g] - mx) : 0.f;
                sum += e;
                acc.x = fmaf(e, vv[u].x, acc.x); acc.y = fmaf(e, vv[u].y, acc.y);
                acc.z = fmaf(e, vv[u].z, acc.z); acc.w = fmaf(e, vv[u].w, acc.w);
            }
            l[g] = l[g] * alpha + sum;
            o[g] = acc;
        }
    }

    // merge the warps
    __shared__ float sm_m[kWarps][G], sm_l[kWarps][G];
    __shared__ float4 sm_o[kWarps][G][32];
#pragma unroll
    for (int g = 0; g < G; g++) {
        if (lane == 0) { sm_m[warp][g] = m[g]; sm_l[warp][g] = l[g]; }
        sm_o[warp][g][lane] = o[g];
    }
    __syncthreads();
    if (warp == 0) {
#pragma unroll
        for (int g = 0; g < G; g++) {
            float mx = sm_m[0][g];
#pragma unroll
            for (int w = 1; w < kWarps; w++) mx = fmaxf(mx, sm_m[w][g]);
            float lt = 0.f;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int w = 0; w < kWarps; w++) {
                const float f = exp2f(sm_m[w][g] - mx);
                lt = fmaf(sm_l[w][g], f, lt);
                const float4 ow = sm_o[w][g][lane];
                acc.x = fmaf(ow.x, f, acc.x); acc.y = fmaf(ow.y, f, acc.y);
                acc.z = fmaf(ow.z, f, acc.z); acc.w = fmaf(ow.w, f, acc.w);
            }
            const size_t qrow = (size_t)row * p.q_heads + hq0 + g;
            if (p.parts == 1) {
                const float4 r4 = make_float4(acc.x / lt, acc.y / lt, acc.z / lt, acc.w / lt);
                if (lane_on) *reinterpret_cast<float4 *>(p.out + qrow * D + lane * 4) = r4;
                if (p.out_max) head_max_store(p.out_max + qrow * 4, r4, lane_on, lane);
            } else {
                if (lane_on)
                    *reinterpret_cast<float4 *>(p.part_o + (qrow * p.parts + part) * D + lane * 4) = acc;
                if (lane == 0) p.part_ml[qrow * p.parts + part] = make_float2(mx, lt);
            }
        }
    }
}

// ---- grouped-query heads: half a warp per position ------------------------------------------------
// With G query heads sharing a KV head, the warp-per-position form spends most of its issue slots on
// shuffles: 5 per (position, head) to sum a dot product over 32 lanes.  Here 16 lanes own a position
// (8 elements each, 32 contiguous bytes of an f32 row), a warp works on two positions at once, and
// the G partial dot products of a lane are summed by a butterfly that halves the number of values a
// lane carries at every step, then handed back to all 16 lanes: G + log2(16) + 1 shuffles for two
// positions x G heads instead of 10 G.  Each half-warp carries its own running (max, sum, output);
// the halves are merged with the warps.
template <typename T> struct Vec8;
template <> struct Vec8<float> {
    static __device__ __forceinline__ void load(const float *p, float (&v)[8])
    {
        asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
                     : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]) : "l"(p));
        asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
                     : "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]) : "l"(p + 4));
    }
};
template <> struct Vec8<__half> {
    static __device__ __forceinline__ void load(const __half *p, float (&v)[8])
    {
        uint4 raw;
        asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(raw.x), "=r"(raw.y), "=r"(raw.z), "=r"(raw.w) : "l"(p));
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
};

static constexpr int kStreams = 2 * kWarps;      // half-warps: independent running softmax states

// grid = (parts, kv_heads, rows); head_dim a multiple of 8, at most 128
// kGqaUnroll = steps per iteration: 2 x kGqaUnroll positions per warp in flight
template <typename T, int G, int kGqaUnroll>
__global__ void __launch_bounds__(kAttnThreads)
attn_partition_gqa_kernel(const AttnParams p)
{
    pdl_wait();
    const uint32_t part = blockIdx.x, row = blockIdx.z, kvh = blockIdx.y;
    const uint32_t hq0 = kvh * G;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, sl = lane & 15, half = lane >> 4;
    const uint32_t D = p.head_dim;
    const bool lane_on = (uint32_t)sl * 8 < D;

    const RowView rv = row_view(p, row);
    const uint32_t begin = part * p.psize;
    if (rv.zero) {
        if (part == 0) {
            for (uint32_t i = threadIdx.x; i < G * D; i += kAttnThreads)
                p.out[((size_t)row * p.q_heads + hq0) * D + i] = 0.f;
            if (p.out_max && threadIdx.x < G * 4) p.out_max[((size_t)row * p.q_heads + hq0) * 4 + threadIdx.x] = 0.f;
        }
        return;
    }
    if (begin >= rv.len && !(part == 0)) return;     // partition 0 always reports (len 0 -> NaN)
    const uint32_t end = min(rv.len, begin + p.psize);

    const T *kc = reinterpret_cast<const T *>(p.k);
    const T *vc = reinterpret_cast<const T *>(p.v);
    const size_t row_stride = (size_t)p.kv_heads * D;
    const size_t head_off = (size_t)kvh * D + (size_t)sl * 8;

    float qv[G][8];
#pragma unroll
    for (int g = 0; g < G; g++)
#pragma unroll
        for (int e = 0; e < 8; e++)
            qv[g][e] = lane_on ? p.q[((size_t)row * p.q_heads + hq0 + g) * D + sl * 8 + e] * p.scale_log2 : 0.f;

    float m[G], l[G], o[G][8];
#pragma unroll
    for (int g = 0; g < G; g++) {
        m[g] = kNegBig; l[g] = 0.f;
#pragma unroll
        for (int e = 0; e < 8; e++) o[g][e] = 0.f;
    }

    // position of (step u, half h) in an iteration: j0 + kWarps * (2u + h)
    for (uint32_t j0 = begin + warp; j0 < end; j0 += kWarps * 2 * kGqaUnroll) {
        float kv[kGqaUnroll][8], vv[kGqaUnroll][8];
        bool ok[kGqaUnroll];
#pragma unroll
        for (int u = 0; u < kGqaUnroll; u++) {
            const uint32_t j = j0 + kWarps * (2 * u + half);
            ok[u] = j < end;
#pragma unroll
            for (int e = 0; e < 8; e++) kv[u][e] = vv[u][e] = 0.f;
            if (ok[u] && lane_on) {
                const size_t phys = rv.pages == nullptr
                                        ? (size_t)j
                                        : (size_t)__ldg(rv.pages + j / p.block) * p.block + j % p.block;
                const size_t off = phys * row_stride + head_off;
                Vec8<T>::load(kc + off, kv[u]);
                Vec8<T>::load(vc + off, vv[u]);
            }
        }
        float sc[kGqaUnroll][G];
#pragma unroll
        for (int u = 0; u < kGqaUnroll; u++) {
            // partial dot products of this lane's 8 elements, one per head
            float s[G];
#pragma unroll
            for (int g = 0; g < G; g++) {
                float a = 0.f;
#pragma unroll
                for (int e = 0; e < 8; e++) a = fmaf(qv[g][e], kv[u][e], a);
                s[g] = a;
            }
            // butterfly over the 16 lanes: every step halves the values a lane carries
            int sh = 8;
#pragma unroll
            for (int n = G; n > 1; n >>= 1, sh >>= 1) {
                const bool upper = (lane & sh) != 0;
#pragma unroll
                for (int i = 0; i < n / 2; i++) {
                    const float send = upper ? s[i] : s[i + n / 2];
                    const float keep = upper ? s[i + n / 2] : s[i];
                    s[i] = keep + __shfl_xor_sync(0xffffffffu, send, sh);
                }
            }
#pragma unroll
            for (; sh >= 1; sh >>= 1) s[0] += __shfl_xor_sync(0xffffffffu, s[0], sh);
            // head g's sum now sits in the lanes whose top bits spell g: hand it to all 16
#pragma unroll
            for (int g = 0; g < G; g++) {
                int src = 0, bit = 8;
#pragma unroll
                for (int n = G; n > 1; n >>= 1, bit >>= 1)
                    if (g & (n >> 1)) src |= bit;
                sc[u][g] = __shfl_sync(0xffffffffu, s[0], (lane & 16) | src);
            }
        }
        // one rescale of the running state per head and iteration, then the positions' terms
#pragma unroll
        for (int g = 0; g < G; g++) {
            float mx = m[g];
#pragma unroll
            for (int u = 0; u < kGqaUnroll; u++) mx = ok[u] ? fmaxf(mx, sc[u][g]) : mx;
            const float alpha = exp2f(m[g] - mx);
            m[g] = mx;
            float sum = 0.f;
#pragma unroll
            for (int q = 0; q < 8; q++) o[g][q] *= alpha;
#pragma unroll
            for (int u = 0; u < kGqaUnroll; u++) {
                const float e = ok[u] ? exp2f(sc[u][g] - mx) : 0.f;
                sum += e;
#pragma unroll
                for (int q = 0; q < 8; q++) o[g][q] = fmaf(e, vv[u][q], o[g][q]);
            }
            l[g] = fmaf(l[g], alpha, sum);
        }
    }

    // merge the half-warps of every warp
    __shared__ float sm_m[kStreams][G], sm_l[kStreams][G];
    __shared__ float4 sm_o[kStreams][G][32];
    const int stream = warp * 2 + half;
#pragma unroll
    for (int g = 0; g < G; g++) {
        if (sl == 0) { sm_m[stream][g] = m[g]; sm_l[stream][g] = l[g]; }
        sm_o[stream][g][2 * sl] = make_float4(o[g][0], o[g][1], o[g][2], o[g][3]);
        sm_o[stream][g][2 * sl + 1] = make_float4(o[g][4], o[g][5], o[g][6], o[g][7]);
    }
    __syncthreads();
    if (warp == 0) {
        const bool out_on = (uint32_t)lane * 4 < D;
#pragma unroll
        for (int g = 0; g < G; g++) {
            float mx = sm_m[0][g];
#pragma unroll
            for (int w = 1; w < kStreams; w++) mx = fmaxf(mx, sm_m[w][g]);
            float lt = 0.f;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int w = 0; w < kStreams; w++) {
                const float f = exp2f(sm_m[w][g] - mx);
                lt = fmaf(sm_l[w][g], f, lt);
                const float4 ow = sm_o[w][g][lane];
                acc.x = fmaf(ow.x, f, acc.x); acc.y = fmaf(ow.y, f, acc.y);
                acc.z = fmaf(ow.z, f, acc.z); acc.w = fmaf(ow.w, f, acc.w);
            }
            const size_t qrow = (size_t)row * p.q_heads + hq0 + g;
            if (p.parts == 1) {
                const float4 r4 = make_float4(acc.x / lt, acc.y / lt, acc.z / lt, acc.w / lt);
                if (out_on) *reinterpret_cast<float4 *>(p.out + qrow * D + lane * 4) = r4;
                if (p.out_max) head_max_store(p.out_max + qrow * 4, r4, out_on, lane);
            } else {
                if (out_on)
                    *reinterpret_cast<float4 *>(p.part_o + (qrow * p.parts + part) * D + lane * 4) = acc;
                if (lane == 0) p.part_ml[qrow * p.parts + part] = make_float2(mx, lt);
            }
        }
    }
}

// ---- grouped-query heads on the tensor cores (head dimension 128) -----------------------------------
// The half-warp kernel above is bound by instruction issue: every (position, head) costs its FMAs
// and shuffles on the CUDA cores.  Here a warp takes 16 positions at a time and both products run as
// mma.sync m16n8k8 (tf32 operands, f32 accumulators) with the HEADS as the 8-wide dimension, so
// nothing is padded but heads G..7:
//   S^T [16 positions x 8 heads] = K tile [16 x 128] . Q^T [128 x 8]            16 MMAs
//   O^T [128 d x 8 heads]       += V tile^T [128 x 16] . P^T [16 x 8]           16 MMAs
// A sum does not care in which order its terms come, so the k index of each product is permuted
// until the fragment a thread needs is 128-bit pieces of a row: of a K row a
// thread (g = lane / 4, t = lane % 4) holds 8 d's of every 32 (rows g and g + 8 of the tile), of a V
// row 16 d's of 128 (positions t, t + 4, t + 8, t + 12), and Q's fragments and the output's rows follow
// the same maps.  K and Q are rounded to tf32 (cvt.rna), P too; V is used as it is (the MMA drops its
// low 13 bits: a bias of at most 2^-11 of the output).  An f16 cache converts exactly.  The running
// softmax is the recurrence of the other kernels per 16 positions; P goes from the accumulator
// layout of S^T to the B layout of the second product by 8 shuffles.
__device__ __forceinline__ uint32_t tf32_rna(float x)
{
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ void mma_tf32(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t half_lo_f32(uint32_t w) { return __float_as_uint(__half2float(__ushort_as_half((unsigned short)(w & 0xffffu)))); }
__device__ __forceinline__ uint32_t half_hi_f32(uint32_t w) { return __float_as_uint(__half2float(__ushort_as_half((unsigned short)(w >> 16)))); }

// Which d a thread's m-th element of a K row's 32-d block c is (m = 0..7), and which d its m-th
// element of a V row is (m = 0..15): the order its 128-bit loads bring them in.
template <typename T> __device__ __forceinline__ uint32_t tc_kd(int c, int m, int t)
{
    return sizeof(T) == 4 ? (uint32_t)(32 * c + 4 * t + (m < 4 ? m : 12 + m)) : (uint32_t)(32 * c + 8 * t + m);
}
template <typename T> __device__ __forceinline__ uint32_t tc_vd(int m, int g)
{
    return sizeof(T) == 4 ? (uint32_t)(32 * (m >> 2) + 4 * g + (m & 3)) : (uint32_t)(64 * (m >> 3) + 8 * g + (m & 7));
}

// grid = (parts, kv_heads, rows); head_dim = 128; G = 2, 4 or 8 query heads per KV head, or G = 1 with
// grid.y = q_heads (an f16 cache without grouping: its 256-byte rows gain from the whole-row copies).
// (Two warps per CTA, so that a warp walks eight tiles of a partition and the start of a CTA weighs
// less, measured no better than four.)
//
// The tiles come through shared memory by cp.async, whole rows at a time (512 bytes of one position
// per instruction at f32, as the one-head kernel reads them: with each thread fetching its own
// fragments, 64 bytes per row and instruction, the kernel stopped at 0.70 of the HBM peak whatever
// the number of warps), and the fragments are read back with 128-bit shared-memory loads; the rows
// are padded (K by 64 bytes, V by 32) so that a quarter-warp's loads fall into different banks.
// A tile belongs to one warp: __syncwarp orders its copies and loads, there is no CTA-wide barrier in
// the loop.  One stage per warp, and three (f32) or four (f16) CTAs per SM: a second stage costs a CTA
// per SM and measured no better, and more warps measured better at every step (f16: 0.49 of the peak at
// 8 warps per SM, 0.58 at 12, 0.70 at 16).
static constexpr int kTcWarps = 4;
static constexpr int kTcThreads = kTcWarps * 32;
template <typename T> __host__ __device__ constexpr int tc_stages() { return 1; }
template <typename T> __host__ __device__ constexpr uint32_t tc_row_bytes() { return 128u * (uint32_t)sizeof(T); }
template <typename T> __host__ __device__ constexpr uint32_t tc_kstride() { return tc_row_bytes<T>() + 64u; }
template <typename T> __host__ __device__ constexpr uint32_t tc_vstride() { return tc_row_bytes<T>() + 32u; }
template <typename T> __host__ __device__ constexpr uint32_t tc_tile_bytes() { return 16u * (tc_kstride<T>() + tc_vstride<T>()); }
template <typename T> __host__ __device__ constexpr size_t tc_smem_bytes() { return (size_t)tc_stages<T>() * kTcWarps * tc_tile_bytes<T>(); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, bool ok)
{   // ok = false fills the 16 bytes with zeros and reads nothing
    const uint32_t n = ok ? 16u : 0u;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ uint4 lds16(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

template <typename T, int G>
__global__ void __launch_bounds__(kTcThreads, sizeof(T) == 4 ? 3 : 4)
attn_partition_gqa_mma_kernel(const AttnParams p)
{
    extern __shared__ __align__(16) unsigned char tc_ring[];
    pdl_wait();
    constexpr uint32_t D = 128;
    constexpr bool F32 = sizeof(T) == 4;
    constexpr int kTcStages = tc_stages<T>();
    constexpr int kVQ = F32 ? 4 : 2;                 // 16-byte pieces of a V row a thread reads
    // G = 1: one query head per CTA, whatever the number of heads that share its KV head
    const uint32_t part = blockIdx.x, row = blockIdx.z;
    const uint32_t kvh = G == 1 ? blockIdx.y / (p.q_heads / p.kv_heads) : blockIdx.y;
    const uint32_t hq0 = G == 1 ? blockIdx.y : kvh * G;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;

    const RowView rv = row_view(p, row);
    const uint32_t begin = part * p.psize;
    if (rv.zero) {
        if (part == 0) {
            for (uint32_t i = threadIdx.x; i < G * D; i += kTcThreads)
                p.out[((size_t)row * p.q_heads + hq0) * D + i] = 0.f;
            if (p.out_max && threadIdx.x < G * 4) p.out_max[((size_t)row * p.q_heads + hq0) * 4 + threadIdx.x] = 0.f;
        }
        return;
    }
    if (begin >= rv.len && !(part == 0)) return;     // partition 0 always reports (len 0 -> NaN)
    const uint32_t end = min(rv.len, begin + p.psize);

    const T *kc = reinterpret_cast<const T *>(p.k);
    const T *vc = reinterpret_cast<const T *>(p.v);
    const size_t row_stride = (size_t)p.kv_heads * D;
    const size_t head_off = (size_t)kvh * D;

    // stage st of this warp: 16 K rows, then 16 V rows
    const uint32_t ring0 = (uint32_t)__cvta_generic_to_shared(tc_ring) + (uint32_t)warp * tc_tile_bytes<T>();
    auto stage = [&](int st) -> uint32_t { return ring0 + (uint32_t)st * kTcWarps * tc_tile_bytes<T>(); };
    constexpr uint32_t KS = tc_kstride<T>(), VS = tc_vstride<T>(), VOFF = 16u * KS;
    // where this thread's fragments lie: K rows g, g + 8 at the d's of block c; V rows t + 4 n at its 16 d's
    const uint32_t koff = (uint32_t)g * KS + (F32 ? 16u * t : 16u * t), voff = VOFF + (uint32_t)t * VS + 16u * g;

    // lane i < 16 finds where position p0 + i of a tile lies; the others get it by shuffle.  The look-up
    // runs one tile ahead of the copies.
    auto lookup = [&](uint32_t p0) -> uint32_t {
        uint32_t phys = 0;
        if (lane < 16 && p0 + lane < end) {
            const uint32_t j = p0 + lane;
            phys = rv.pages == nullptr ? j : __ldg(rv.pages + j / p.block) * p.block + j % p.block;
        }
        return phys;
    };
    // whole rows: an instruction copies one position's 512 bytes (f32) or two positions' 256 (f16) of K,
    // then of V.  Positions past the end are zeros.
    auto issue_tile = [&](uint32_t p0, uint32_t phys, int st) {
        const uint32_t base = stage(st);
        constexpr int kPerInstr = F32 ? 1 : 2;
#pragma unroll
        for (int j = 0; j < 16 / kPerInstr; j++) {
            const int rowi = F32 ? j : 2 * j + (lane >> 4);
            const int chunk = F32 ? lane : (lane & 15);
            const uint32_t ph = __shfl_sync(0xffffffffu, phys, rowi);
            const bool ok = p0 + rowi < end;
            const size_t src = (size_t)ph * row_stride + head_off + (size_t)chunk * (16 / sizeof(T));
            cp_async16(base + (uint32_t)rowi * KS + 16u * chunk, kc + src, ok);
            cp_async16(base + VOFF + (uint32_t)rowi * VS + 16u * chunk, vc + src, ok);
        }
    };

    constexpr uint32_t kStep = 16u * kTcWarps;
    const uint32_t first = begin + 16u * warp;
    uint32_t phys_next;
    {
        uint32_t ph[kTcStages];
#pragma unroll
        for (int k = 0; k < kTcStages; k++) ph[k] = lookup(first + k * kStep);
#pragma unroll
        for (int k = 0; k < kTcStages - 1; k++) {
            if (first + k * kStep < end) issue_tile(first + k * kStep, ph[k], k);
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
        phys_next = ph[kTcStages - 1];
    }

    // Q^T as B fragments: column g is head g (zero past the group), rows in the K fragments' order
    uint32_t qb[16][2];
#pragma unroll
    for (int c = 0; c < 4; c++)
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const float q = g < G ? p.q[((size_t)row * p.q_heads + hq0 + g) * D + tc_kd<T>(c, 2 * i + e, t)] * p.scale_log2 : 0.f;
                qb[4 * c + i][e] = tf32_rna(q);
            }

    float m[2] = {kNegBig, kNegBig}, l[2] = {0.f, 0.f};     // heads 2t, 2t + 1; l: this thread's positions only
    float o[8][4];                                            // O^T: 8 tiles of 16 d's x heads 2t, 2t + 1
#pragma unroll
    for (int mt = 0; mt < 8; mt++)
#pragma unroll
        for (int e = 0; e < 4; e++) o[mt][e] = 0.f;

    int st = 0;                                               // stage of the tile being multiplied
    for (uint32_t p0 = first; p0 < end; p0 += kStep) {
        {   // the tile kTcStages - 1 ahead goes into the stage the previous tile has left
            const uint32_t pi = p0 + (kTcStages - 1) * kStep;
            const int sti = st == 0 ? kTcStages - 1 : st - 1;
            __syncwarp();                             // every lane has read what that stage held
            if (pi < end) issue_tile(pi, phys_next, sti);
            asm volatile("cp.async.commit_group;" ::: "memory");
            phys_next = lookup(pi + kStep);
            asm volatile("cp.async.wait_group %0;" ::"n"(kTcStages - 1) : "memory");
            __syncwarp();                             // ... and sees what the other lanes copied
        }
        const uint32_t tile = stage(st);

        // S^T: sc[0], sc[1] = position g x heads 2t, 2t + 1; sc[2], sc[3] = position g + 8
        float sc[4] = {0.f, 0.f, 0.f, 0.f}, sc2[4] = {0.f, 0.f, 0.f, 0.f};       // two chains of eight MMAs
#pragma unroll
        for (int c = 0; c < 4; c++) {
            uint32_t k0[8], k1[8];                            // rows g and g + 8: the thread's words of block c
            if (F32) {
                const uint4 a = lds16(tile + koff + 128u * c), b = lds16(tile + koff + 128u * c + 64u);
                const uint4 a1 = lds16(tile + koff + 8u * KS + 128u * c), b1 = lds16(tile + koff + 8u * KS + 128u * c + 64u);
                k0[0] = a.x; k0[1] = a.y; k0[2] = a.z; k0[3] = a.w; k0[4] = b.x; k0[5] = b.y; k0[6] = b.z; k0[7] = b.w;
                k1[0] = a1.x; k1[1] = a1.y; k1[2] = a1.z; k1[3] = a1.w; k1[4] = b1.x; k1[5] = b1.y; k1[6] = b1.z; k1[7] = b1.w;
            } else {
                const uint4 a = lds16(tile + koff + 64u * c), a1 = lds16(tile + koff + 8u * KS + 64u * c);
                k0[0] = a.x; k0[1] = a.y; k0[2] = a.z; k0[3] = a.w;
                k1[0] = a1.x; k1[1] = a1.y; k1[2] = a1.z; k1[3] = a1.w;
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {
                uint32_t a0, a1, a2, a3;
                if (F32) {
                    a0 = tf32_rna(__uint_as_float(k0[2 * i])); a2 = tf32_rna(__uint_as_float(k0[2 * i + 1]));
                    a1 = tf32_rna(__uint_as_float(k1[2 * i])); a3 = tf32_rna(__uint_as_float(k1[2 * i + 1]));
                } else {
                    a0 = half_lo_f32(k0[i]); a2 = half_hi_f32(k0[i]);
                    a1 = half_lo_f32(k1[i]); a3 = half_hi_f32(k1[i]);
                }
                mma_tf32((i & 1) ? sc2 : sc, a0, a1, a2, a3, qb[4 * c + i][0], qb[4 * c + i][1]);
            }
        }
#pragma unroll
        for (int e = 0; e < 4; e++) sc[e] += sc2[e];

        // the running softmax of heads 2t, 2t + 1 over these 16 positions
        const bool ok0 = p0 + g < end, ok1 = p0 + g + 8 < end;
        float pc[4], alpha[2];
#pragma unroll
        for (int hh = 0; hh < 2; hh++) {
            float mx = m[hh];
            mx = ok0 ? fmaxf(mx, sc[hh]) : mx;
            mx = ok1 ? fmaxf(mx, sc[2 + hh]) : mx;
#pragma unroll
            for (int sh = 4; sh <= 16; sh <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, sh));
            alpha[hh] = exp2f(m[hh] - mx);
            m[hh] = mx;
            pc[hh] = ok0 ? exp2f(sc[hh] - mx) : 0.f;
            pc[2 + hh] = ok1 ? exp2f(sc[2 + hh] - mx) : 0.f;
            l[hh] = fmaf(l[hh], alpha[hh], pc[hh] + pc[2 + hh]);
        }
        if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
            for (int mt = 0; mt < 8; mt++) { o[mt][0] *= alpha[0]; o[mt][1] *= alpha[1]; o[mt][2] *= alpha[0]; o[mt][3] *= alpha[1]; }
        }
        // P^T as B fragments: thread (g, t) needs P[position t, t + 4 (+ 8)][head g], which the thread of
        // position-row t (or t + 4) that owns heads 2 (g / 2), 2 (g / 2) + 1 holds
        uint32_t pb[2][2];
        {
            const int srcA = t * 4 + (g >> 1), srcB = (t + 4) * 4 + (g >> 1);
            const bool odd = g & 1;
#pragma unroll
            for (int ks = 0; ks < 2; ks++) {
                const float eA = __shfl_sync(0xffffffffu, pc[2 * ks], srcA), oA = __shfl_sync(0xffffffffu, pc[2 * ks + 1], srcA);
                const float eB = __shfl_sync(0xffffffffu, pc[2 * ks], srcB), oB = __shfl_sync(0xffffffffu, pc[2 * ks + 1], srcB);
                pb[ks][0] = tf32_rna(odd ? oA : eA);
                pb[ks][1] = tf32_rna(odd ? oB : eB);
            }
        }
        // O^T += V^T P^T: a 16-byte piece of a V row is four d's (f32: tiles 2q, 2q + 1) or eight (f16:
        // tiles 4q .. 4q + 3) of the thread's sixteen
#pragma unroll
        for (int q = 0; q < kVQ; q++) {
            uint4 v[4];
#pragma unroll
            for (int n = 0; n < 4; n++) v[n] = lds16(tile + voff + 4u * n * VS + 128u * q);
            const uint32_t vw[4][4] = {{v[0].x, v[0].y, v[0].z, v[0].w}, {v[1].x, v[1].y, v[1].z, v[1].w},
                                       {v[2].x, v[2].y, v[2].z, v[2].w}, {v[3].x, v[3].y, v[3].z, v[3].w}};
#pragma unroll
            for (int x = 0; x < (F32 ? 2 : 4); x++) {
                const int mt = F32 ? 2 * q + x : 4 * q + x;
#pragma unroll
                for (int ks = 0; ks < 2; ks++) {
                    uint32_t a0, a1, a2, a3;
                    if (F32) {
                        a0 = vw[2 * ks][2 * x];     a1 = vw[2 * ks][2 * x + 1];
                        a2 = vw[2 * ks + 1][2 * x]; a3 = vw[2 * ks + 1][2 * x + 1];
                    } else {
                        a0 = half_lo_f32(vw[2 * ks][x]);     a1 = half_hi_f32(vw[2 * ks][x]);
                        a2 = half_lo_f32(vw[2 * ks + 1][x]); a3 = half_hi_f32(vw[2 * ks + 1][x]);
                    }
                    mma_tf32(o[mt], a0, a1, a2, a3, pb[ks][0], pb[ks][1]);
                }
            }
        }
        st = st == kTcStages - 1 ? 0 : st + 1;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    // a head's sum is spread over the eight position-rows: add them up
#pragma unroll
    for (int hh = 0; hh < 2; hh++)
#pragma unroll
        for (int sh = 4; sh <= 16; sh <<= 1) l[hh] += __shfl_xor_sync(0xffffffffu, l[hh], sh);

    // merge the warps (their outputs go where the ring was)
    __shared__ float sm_m[kTcWarps][G], sm_l[kTcWarps][G];
    __syncthreads();
    float4 (*sm_o)[G][32] = reinterpret_cast<float4 (*)[G][32]>(tc_ring);
#pragma unroll
    for (int hh = 0; hh < 2; hh++) {
        const int head = 2 * t + hh;
        if (head < G) {
            if (g == 0) { sm_m[warp][head] = m[hh]; sm_l[warp][head] = l[hh]; }
            float *dst = reinterpret_cast<float *>(&sm_o[warp][head][0]);
#pragma unroll
            for (int mt = 0; mt < 8; mt++) {
                dst[tc_vd<T>(2 * mt, g)] = o[mt][hh];
                dst[tc_vd<T>(2 * mt + 1, g)] = o[mt][2 + hh];
            }
        }
    }
    __syncthreads();
    if (warp == 0) {
#pragma unroll
        for (int gg = 0; gg < G; gg++) {
            float mx = sm_m[0][gg];
#pragma unroll
            for (int w = 1; w < kTcWarps; w++) mx = fmaxf(mx, sm_m[w][gg]);
            float lt = 0.f;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int w = 0; w < kTcWarps; w++) {
                const float f = exp2f(sm_m[w][gg] - mx);
                lt = fmaf(sm_l[w][gg], f, lt);
                const float4 ow = sm_o[w][gg][lane];
                acc.x = fmaf(ow.x, f, acc.x); acc.y = fmaf(ow.y, f, acc.y);
                acc.z = fmaf(ow.z, f, acc.z); acc.w = fmaf(ow.w, f, acc.w);
            }
            const size_t qrow = (size_t)row * p.q_heads + hq0 + gg;
            if (p.parts == 1) {
                const float4 r4 = make_float4(acc.x / lt, acc.y / lt, acc.z / lt, acc.w / lt);
                *reinterpret_cast<float4 *>(p.out + qrow * D + lane * 4) = r4;
                if (p.out_max) head_max_store(p.out_max + qrow * 4, r4, true, lane);
            } else {
                *reinterpret_cast<float4 *>(p.part_o + (qrow * p.parts + part) * D + lane * 4) = acc;
                if (lane == 0) p.part_ml[qrow * p.parts + part] = make_float2(mx, lt);
            }
        }
    }
}

// grid = (q_heads, rows), 128 threads; thread d owns output element d.  The partitions' maxima are
// read by all threads side by side (thread t takes partitions t, t + 128, ...) and reduced once; the
// weighted sum then walks the partitions with its loads batched eight at a time: with 64-position
// partitions a 2048-token context has 33 of them, and a loop that waits for each load in turn costs
// more than the partitions themselves.
__global__ void __launch_bounds__(128) attn_combine_kernel(const AttnParams p)
{
    __shared__ float s_mx[4];
    pdl_enter();
    const uint32_t h = blockIdx.x, row = blockIdx.y, d = threadIdx.x;
    const RowView rv = row_view(p, row);
    if (rv.zero) return;
    uint32_t nparts = (rv.len + p.psize - 1) / p.psize;
    if (nparts == 0) nparts = 1;
    const size_t qrow = (size_t)row * p.q_heads + h;
    const float2 *ml = p.part_ml + qrow * p.parts;
    float mx = kNegBig;
    for (uint32_t s = d; s < nparts; s += 128) mx = fmaxf(mx, ml[s].x);
#pragma unroll
    for (int sh = 16; sh > 0; sh >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, sh));
    if ((d & 31) == 0) s_mx[d >> 5] = mx;
    __syncthreads();
    mx = fmaxf(fmaxf(s_mx[0], s_mx[1]), fmaxf(s_mx[2], s_mx[3]));
    const bool on = d < p.head_dim;              // the other threads follow along on element 0 and store nothing
    const float *po = p.part_o + qrow * p.parts * p.head_dim + (on ? d : 0u);
    float lt = 0.f, acc = 0.f;
    uint32_t s = 0;
    for (; s + 8 <= nparts; s += 8) {
        float2 m8[8];
        float o8[8];
#pragma unroll
        for (int i = 0; i < 8; i++) { m8[i] = ml[s + i]; o8[i] = po[(size_t)(s + i) * p.head_dim]; }
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const float f = exp2f(m8[i].x - mx);
            lt = fmaf(m8[i].y, f, lt);
            acc = fmaf(o8[i], f, acc);
        }
    }
    for (; s < nparts; s++) {
        const float2 m1 = ml[s];
        const float f = exp2f(m1.x - mx);
        lt = fmaf(m1.y, f, lt);
        acc = fmaf(po[(size_t)s * p.head_dim], f, acc);
    }
    const float val = acc / lt;
    if (on) p.out[qrow * p.head_dim + d] = val;
    if (p.out_max) {                             // one entry per warp: its 32 elements of the head
        const uint32_t b = __reduce_max_sync(0xffffffffu, on ? __float_as_uint(fabsf(val)) : 0u);
        if ((d & 31) == 0) p.out_max[qrow * 4 + (d >> 5)] = __uint_as_float(b);
    }
}

// the tensor-core kernel's ring is more shared memory than a kernel gets unasked: once per device and kernel
static int tc_prepare(void (*kernel)(const AttnParams), size_t bytes)
{
    static struct { void (*k)(const AttnParams); int dev; } done[64];
    static int ndone = 0;
    static std::mutex mu;                            // launches may come from several host threads
    std::lock_guard<std::mutex> lock(mu);
    int dev = 0;
    cudaGetDevice(&dev);
    for (int i = 0; i < ndone; i++)
        if (done[i].k == kernel && done[i].dev == dev) return AB_OK;
    int rc = check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes),
                        "attn_partition_gqa_mma_kernel shared memory");
    if (rc) return rc;
    if (ndone < 64) { done[ndone].k = kernel; done[ndone].dev = dev; ndone++; }
    return AB_OK;
}

template <typename T>
static int run_attention(Launch &l, AttnParams &p, const char *name)
{
    if (p.kv_heads == 0 || p.q_heads % p.kv_heads != 0)
        return fail(AB_ERR_INVALID, "%s: %u query heads over %u key/value heads", name, p.q_heads,
                    p.kv_heads);
    if (p.head_dim == 0 || p.head_dim % 8 != 0 || p.head_dim > 128)
        return fail(AB_ERR_INVALID, "%s: head dimension %u; it is a multiple of eight and at most "
                    "128", name, p.head_dim);
    if (p.block == 0)
        return fail(AB_ERR_INVALID, "%s: a page table addresses blocks, and Block is 0", name);
    // Positions per partition: 256 where that fills at least three quarters of the SMs' CTA slots; a small grid (a
    // tensor-parallel shard's few KV heads, a short batch) takes 128 or 64 so that the K/V stream is
    // spread over all SMs (the partial results grow by the same factor and stay small).
    {
        const uint32_t group_w = p.q_heads / p.kv_heads;
        const bool grouped = group_w == 2 || group_w == 4 || group_w == 8;
        const uint64_t per_part = (uint64_t)(grouped ? p.kv_heads : p.q_heads) * p.rows;
        const uint64_t slots = 8ull * (uint64_t)sm_count();
        p.psize = 64;
        for (uint32_t ps = kPartition; ps >= 128; ps /= 2)
            if ((uint64_t)((p.capacity + ps - 1) / ps) * per_part * 4 >= slots * 3) { p.psize = ps; break; }
    }
    p.parts = (p.capacity + p.psize - 1) / p.psize;
    if (p.parts == 0) p.parts = 1;
    const size_t o_bytes = align_up((size_t)p.rows * p.q_heads * p.parts * p.head_dim * 4, 256);
    const size_t ml_bytes = (size_t)p.rows * p.q_heads * p.parts * sizeof(float2);
    const size_t need = p.parts > 1 ? o_bytes + ml_bytes : 0;
    if (l.query_ws) { l.ws_need = need; return AB_OK; }
    if (need > l.ws_bytes || (need && !l.ws))
        return fail(AB_ERR_INVALID, "%s: needs %zu bytes of workspace, given %zu", name, need,
                    l.ws_bytes);
    p.part_o = reinterpret_cast<float *>(l.ws);
    p.part_ml = reinterpret_cast<float2 *>(reinterpret_cast<char *>(l.ws) + o_bytes);
    if (p.rows == 0) return AB_OK;

    const uint32_t group = p.q_heads / p.kv_heads;
    // a group width with no instantiation runs one query head per CTA (K/V re-read per head)
    const int G = (group == 2 || group == 4 || group == 8) ? (int)group : 1;
    dim3 grid(p.parts, G == 1 ? p.q_heads : p.kv_heads, p.rows);
    // grouped heads: half a warp per position when the head dimension allows 8 elements per lane
    const bool gqa = G > 1 && p.head_dim % 8 == 0;
    // ... and the tensor cores where the head dimension is 128
    // (an f16 cache without grouping too: whole-row copies serve its 256-byte rows better than the
    // half-warp loads, 0.70 against 0.58-0.63 of the peak)
    const bool gqa_mma = p.head_dim == 128 && (G > 1 || sizeof(T) == 2);
    // an f16 cache without grouping: 16 lanes x 16 bytes cover a row, where a full warp would issue
    // 8-byte loads
    const bool half_rows = sizeof(T) == 2 && group == 1 && p.head_dim % 8 == 0;
#define AB_GQA(GG, UU) lerr = launch_dependent(attn_partition_gqa_kernel<T, GG, UU>, grid, dim3(kAttnThreads), 0, l.stream, p)
#define AB_MHA(GG) lerr = launch_dependent(attn_partition_kernel<T, GG>, grid, dim3(kAttnThreads), 0, l.stream, p)
    cudaError_t lerr = cudaSuccess;
    const bool deep = false;      // four positions in flight per half warp measured no faster than two
#define AB_TC(GG) lerr = tc_prepare(attn_partition_gqa_mma_kernel<T, GG>, tc_smem_bytes<T>()) ? cudaErrorInvalidValue : \
        launch_dependent(attn_partition_gqa_mma_kernel<T, GG>, grid, dim3(kTcThreads), tc_smem_bytes<T>(), l.stream, p)
    if (gqa_mma) {
        if (G == 1) AB_TC(1); else if (G == 2) AB_TC(2); else if (G == 4) AB_TC(4); else AB_TC(8);
    } else
#undef AB_TC
    switch (G) {
    case 1:
        if (half_rows) { if (deep) AB_GQA(1, 4); else AB_GQA(1, 2); }
        else AB_MHA(1);
        break;
    case 2:
        if (gqa) { if (deep) AB_GQA(2, 4); else AB_GQA(2, 2); }
        else AB_MHA(2);
        break;
    case 4:
        if (gqa) { if (deep) AB_GQA(4, 4); else AB_GQA(4, 2); }
        else AB_MHA(4);
        break;
    default:
        if (gqa) AB_GQA(8, 2);
        else AB_MHA(8);
        break;
    }
#undef AB_GQA
#undef AB_MHA
    count_launch();
    if (lerr != cudaSuccess) return check_cuda(lerr, name);
    if (p.parts > 1) {
        dim3 cgrid(p.q_heads, p.rows);
        lerr = launch_dependent(attn_combine_kernel, cgrid, dim3(128), 0, l.stream, p);
        count_launch();
        if (lerr != cudaSuccess) return check_cuda(lerr, name);
    }
    note_selection("%s: split-K decode, %u partition(s) of %d positions, %u query head(s) sharing "
                   "each K/V read, %u row(s), %s per position", name, p.parts, (int)p.psize, group, p.rows,
                   (gqa || (G == 1 && half_rows)) ? "half a warp" : "a warp");
    return check_cuda(cudaGetLastError(), name);
}

// ---- front ends: read the uniform block and the lengths block the way each reference kernel does
static int contiguous(Launch &l, bool f16, const char *name)
{   // q, k, v, lengths, out; AttnDims{QHeads,KVHeads,HeadDim,Scale}
    AttnParams p{};
    p.mode = kContiguous;
    p.q_heads = u32_at(l.u, 0); p.kv_heads = u32_at(l.u, 4); p.head_dim = u32_at(l.u, 8);
    p.scale_log2 = f32_at(l.u, 12) * kLog2e;
    p.rows = 1; p.batch = 1; p.block = 1;
    if (!l.query_ws) {
        p.q = ptr<const float>(l, 0); p.k = l.b[1]; p.v = l.b[2];
        p.lengths = ptr<const uint32_t>(l, 3); p.out = ptr<float>(l, 4);
    }
    uint64_t per = (uint64_t)p.kv_heads * p.head_dim;
    p.capacity = per ? (uint32_t)(l.len[1] / per) : 0;     // len(k) / (kvHeads*headDim)
    return f16 ? run_attention<__half>(l, p, name) : run_attention<float>(l, p, name);
}

static int paged(Launch &l, bool f16, const char *name)
{   // q, k, v, pages, lengths, out; PagedDims{QHeads,KVHeads,HeadDim,Block,Scale}
    AttnParams p{};
    p.mode = kPaged;
    p.q_heads = u32_at(l.u, 0); p.kv_heads = u32_at(l.u, 4); p.head_dim = u32_at(l.u, 8);
    p.block = u32_at(l.u, 12);
    p.scale_log2 = f32_at(l.u, 16) * kLog2e;
    p.rows = 1; p.batch = 1;
    if (!l.query_ws) {
        p.q = ptr<const float>(l, 0); p.k = l.b[1]; p.v = l.b[2];
        p.pages = ptr<const uint32_t>(l, 3); p.lengths = ptr<const uint32_t>(l, 4);
        p.out = ptr<float>(l, 5);
    }
    p.max_pages = l.len[3];
    p.capacity = l.len[3] * p.block;                        // len(pages) * Block
    return f16 ? run_attention<__half>(l, p, name) : run_attention<float>(l, p, name);
}

static int batched(Launch &l, bool f16, bool ragged, const char *name, bool with_max = false)
{   // q, k, v, pages, lengths, [offsets,] out [, outmax]; BatchedDims / RaggedDims
    AttnParams p{};
    p.mode = ragged ? kRagged : kBatched;
    p.batch = u32_at(l.u, 0); p.q_heads = u32_at(l.u, 4); p.kv_heads = u32_at(l.u, 8);
    p.head_dim = u32_at(l.u, 12); p.block = u32_at(l.u, 16); p.max_pages = u32_at(l.u, 20);
    p.scale_log2 = f32_at(l.u, 24) * kLog2e;
    const int out_i = ragged ? 6 : 5;
    uint64_t per = (uint64_t)p.q_heads * p.head_dim;
    p.rows = ragged ? (per ? (uint32_t)(l.len[0] / per) : 0) : p.batch;   // tokens = len(q)/(qH*D)
    p.capacity = p.max_pages * p.block;
    if (l.len[3] < (uint64_t)p.batch * p.max_pages || l.len[4] < p.batch ||
        (ragged && l.len[5] < p.batch + 1) || l.len[out_i] < (uint64_t)p.rows * per ||
        (with_max && l.len[out_i + 1] < (uint64_t)p.rows * p.q_heads * 4))
        return fail(AB_ERR_INVALID, "%s: Batch=%u MaxPages=%u rows=%u and the lengths block says "
                    "pages[%u] lengths[%u] out[%u]%s", name, p.batch, p.max_pages, p.rows, l.len[3],
                    l.len[4], l.len[out_i], with_max ? " (outmax holds rows * QHeads * 4)" : "");
    if (!l.query_ws) {
        p.q = ptr<const float>(l, 0); p.k = l.b[1]; p.v = l.b[2];
        p.pages = ptr<const uint32_t>(l, 3); p.lengths = ptr<const uint32_t>(l, 4);
        p.offsets = ragged ? ptr<const uint32_t>(l, 5) : nullptr;
        p.out = ptr<float>(l, out_i);
        p.out_max = with_max ? ptr<float>(l, out_i + 1) : nullptr;
    }
    return f16 ? run_attention<__half>(l, p, name) : run_attention<float>(l, p, name);
}

// AttentionPrefill(F16) and AttentionPrefillPaged(F16) (internal/kernels/prefill.go:197,409;
// pagedprefillf16.go:31): QSeq query rows of one sequence against its cache, row s seeing the
// positions <= Base + s.  Every row is a decode over its own visible prefix: the split-K decode
// kernels run with one row per query position.
static int prefill(Launch &l, bool f16, bool is_paged, const char *name)
{   // q, k, v, [pages,] lengths, out; PrefillDims{QHeads,KVHeads,HeadDim,QSeq,Base,Scale} or
    // PagedPrefillDims{QHeads,KVHeads,HeadDim,QSeq,Base,Block,Scale}
    AttnParams p{};
    p.mode = kPrefill;
    p.q_heads = u32_at(l.u, 0); p.kv_heads = u32_at(l.u, 4); p.head_dim = u32_at(l.u, 8);
    p.rows = u32_at(l.u, 12); p.base = u32_at(l.u, 16);
    p.block = is_paged ? u32_at(l.u, 20) : 1;
    p.scale_log2 = f32_at(l.u, is_paged ? 24 : 20) * kLog2e;
    p.batch = 1;
    const int len_i = is_paged ? 4 : 3, out_i = is_paged ? 5 : 4;
    const uint64_t per = (uint64_t)p.q_heads * p.head_dim, kvper = (uint64_t)p.kv_heads * p.head_dim;
    if (is_paged) {
        p.max_pages = l.len[3];
        p.capacity = l.len[3] * p.block;                    // len(pages) * Block
    } else {
        p.capacity = kvper ? (uint32_t)(l.len[1] / kvper) : 0;
    }
    if (l.len[0] < (uint64_t)p.rows * per || l.len[out_i] < (uint64_t)p.rows * per || l.len[len_i] < 1)
        return fail(AB_ERR_INVALID, "%s: QSeq=%u QHeads=%u HeadDim=%u and the lengths block says q[%u] lengths[%u] "
                    "out[%u]", name, p.rows, p.q_heads, p.head_dim, l.len[0], l.len[len_i], l.len[out_i]);
    if (!l.query_ws) {
        p.q = ptr<const float>(l, 0); p.k = l.b[1]; p.v = l.b[2];
        p.pages = is_paged ? ptr<const uint32_t>(l, 3) : nullptr;
        p.lengths = ptr<const uint32_t>(l, len_i);
        p.out = ptr<float>(l, out_i);
    }
    return f16 ? run_attention<__half>(l, p, name) : run_attention<float>(l, p, name);
}

int launch_attention_prefill(Launch &l) { return prefill(l, false, false, "AttentionPrefill"); }
int launch_attention_prefill_f16(Launch &l) { return prefill(l, true, false, "AttentionPrefillF16"); }
int launch_attention_prefill_paged(Launch &l) { return prefill(l, false, true, "AttentionPrefillPaged"); }
int launch_attention_prefill_paged_f16(Launch &l) { return prefill(l, true, true, "AttentionPrefillPagedF16"); }

int launch_attention_decode(Launch &l) { return contiguous(l, false, "AttentionDecode"); }
int launch_attention_decode_f16(Launch &l) { return contiguous(l, true, "AttentionDecodeF16"); }
int launch_attention_decode_paged(Launch &l) { return paged(l, false, "AttentionDecodePaged"); }
int launch_attention_decode_paged_f16(Launch &l) { return paged(l, true, "AttentionDecodePagedF16"); }
int launch_attention_decode_batched(Launch &l) { return batched(l, false, false, "AttentionDecodeBatched"); }
int launch_attention_decode_batched_f16(Launch &l) { return batched(l, true, false, "AttentionDecodeBatchedF16"); }
// the same with a seventh binding, outmax f32[Batch][QHeads][4]: a row's largest |out| is the largest of
// its QHeads * 4 entries (for the int4 product that reads out next: its "A" form, AmaxParts = QHeads * 4)
int launch_attention_decode_batched_max(Launch &l) { return batched(l, false, false, "AttentionDecodeBatchedMax", true); }
int launch_attention_decode_batched_f16_max(Launch &l) { return batched(l, true, false, "AttentionDecodeBatchedF16Max", true); }
int launch_attention_ragged(Launch &l) { return batched(l, false, true, "AttentionRagged"); }
int launch_attention_ragged_f16(Launch &l) { return batched(l, true, true, "AttentionRaggedF16"); }

}  // namespace ab
