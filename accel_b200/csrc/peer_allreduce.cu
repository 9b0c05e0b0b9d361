// One-shot all-reduce (sum, f32) over NVLink peer memory, for the row-parallel products of a
// tensor-parallel decode step: 256 KiB per call, 64 calls per step, where a library all-reduce is
// bound by its launch and protocol latency, not by the links.
//
// Every rank owns one buffer that all ranks can address (the caller maps it: CUDA IPC or the
// virtual-memory API; this file only sees pointers):
//
//   [flags: 64 x u32][data A: `capacity` floats][data B: `capacity` floats]
//
// A call with epoch e (1, 2, ...) uses data half e & 1:
//   1. every CTA copies its slice of the input into the rank's OWN buffer;
//   2. the last CTA of the rank to finish that copy stores e into flag[rank] of every peer
//      (release, system scope);
//   3. every CTA waits until all of its own flags are >= e (acquire, system scope; BOUNDED: after
//      kSpinLimit polls the CTA records an error in the rank's state and returns without reading);
//   4. every CTA adds its slice over all ranks' buffers in rank order (plain peer loads that bypass
//      L1; every rank adds in the same order, so all ranks hold bit-identical sums) and writes the
//      output, which may be the input.
// Two halves are enough: a peer can only be two calls ahead of a rank that has not finished reading
// if that rank had signalled the call in between, which it does after its reads (calls of one rank
// are ordered on its stream).  The epoch lives in device memory and is advanced by the kernel, so
// the call can be captured in a CUDA graph and replayed.
//
// No reference counterpart: accel is single-device.  No multicast, no TMA: plain loads and stores.
#include <cstddef>

#include "common.cuh"

namespace ab {

static constexpr int kArThreads = 256;
static constexpr int kArMaxRanks = 8;
static constexpr uint32_t kArFlagWords = 64;
static constexpr uint32_t kArSpinLimit = 1u << 22;       // default: about a second of polling

// spin_limit: polls a CTA spends waiting for its peers before it gives up; 0 means kArSpinLimit
struct ArState { uint32_t epoch, arrived, done, error, spin_limit, reserved[3]; };

__device__ __forceinline__ uint32_t spin_limit_of(const ArState *state)
{
    const uint32_t v = *reinterpret_cast<const volatile uint32_t *>(&state->spin_limit);
    return v ? v : kArSpinLimit;
}
struct ArPeers { float *buf[kArMaxRanks]; };

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float4 ld_peer(const float4 *p)
{
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}

// n4 = elements / 4; capacity4 = floats per data half / 4
__global__ void __launch_bounds__(kArThreads)
peer_allreduce_kernel(ArPeers peers, ArState *state, int rank, int world, const float4 *in,
                      float4 *out, uint32_t n4, uint32_t capacity4)
{
    __shared__ int s_last, s_fail;
    const uint32_t e = *reinterpret_cast<volatile uint32_t *>(&state->epoch) + 1;
    const uint32_t limit = spin_limit_of(state);
    const size_t half = kArFlagWords / 4 + (size_t)(e & 1) * capacity4;      // in float4 units
    float4 *mine = reinterpret_cast<float4 *>(peers.buf[rank]) + half;
    const uint32_t stride = gridDim.x * kArThreads;

    for (uint32_t i = blockIdx.x * kArThreads + threadIdx.x; i < n4; i += stride) mine[i] = in[i];
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        s_fail = 0;
        s_last = atomicAdd(&state->arrived, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (s_last && threadIdx.x < (unsigned)world) {
        __threadfence_system();
        st_release_sys(reinterpret_cast<uint32_t *>(peers.buf[threadIdx.x]) + rank, e);
    }
    if (threadIdx.x < (unsigned)world) {
        const uint32_t *flag = reinterpret_cast<const uint32_t *>(peers.buf[rank]) + threadIdx.x;
        uint32_t polls = 0;
        while ((int32_t)(ld_acquire_sys(flag) - e) < 0) {
            if (++polls >= limit) { s_fail = 1; break; }
        }
    }
    __syncthreads();
    if (s_fail) {
        if (threadIdx.x == 0) atomicExch(&state->error, e);
    } else {
        for (uint32_t i = blockIdx.x * kArThreads + threadIdx.x; i < n4; i += stride) {
            float4 v[kArMaxRanks];
#pragma unroll
            for (int r = 0; r < kArMaxRanks; r++)
                if (r < world) v[r] = ld_peer(reinterpret_cast<const float4 *>(peers.buf[r]) + half + i);
            float4 s = v[0];
#pragma unroll
            for (int r = 1; r < kArMaxRanks; r++)
                if (r < world) { s.x += v[r].x; s.y += v[r].y; s.z += v[r].z; s.w += v[r].w; }
            out[i] = s;
        }
    }
    // the last CTA to leave advances the epoch and re-arms the counters for the next call
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(&state->done, 1u) == gridDim.x - 1) {
            state->arrived = 0;
            state->done = 0;
            __threadfence();
            *reinterpret_cast<volatile uint32_t *>(&state->epoch) = e;
        }
    }
}

// The same all-reduce with the decode layer's next two operators done by its summing stage:
//   sum_out = residual + (sum over ranks of in),   norm_out = RMSNorm(sum_out) * gain
// (ElemAdd, internal/kernels/elementwise.go:22, then RMSNorm, internal/kernels/norm.go:46).  One CTA
// per row: the row's sum of squares never leaves the CTA.  Element tid + 256 j belongs to thread
// tid, the per-thread and cross-warp orders are those of the AddRMSNorm kernel, and ranks are added
// in rank order, so the result is bit-identical to the plain all-reduce followed by AddRMSNorm.
// All of a thread's peer loads (ranks x PER) are issued before the first is used: one NVLink round
// trip, not one per rank.
template <int PER>
__global__ void __launch_bounds__(kArThreads)
peer_allreduce_add_rmsnorm_kernel(ArPeers peers, ArState *state, int rank, int world, const float *in,
                                  const float *residual, const float *gain, float *sum_out, float *norm_out,
                                  uint32_t width, float eps, uint32_t capacity)
{
    __shared__ int s_last, s_fail;
    __shared__ float red[8];
    const uint32_t e = *reinterpret_cast<volatile uint32_t *>(&state->epoch) + 1;
    const uint32_t limit = spin_limit_of(state);
    const size_t half = kArFlagWords + (size_t)(e & 1) * capacity;           // in floats
    const size_t base = (size_t)blockIdx.x * width;
    float *mine = peers.buf[rank] + half + base;
#pragma unroll
    for (int j = 0; j < PER; j++) {
        const uint32_t i = threadIdx.x + kArThreads * j;
        if (i < width) mine[i] = in[base + i];
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        s_fail = 0;
        s_last = atomicAdd(&state->arrived, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (s_last && threadIdx.x < (unsigned)world) {
        __threadfence_system();
        st_release_sys(reinterpret_cast<uint32_t *>(peers.buf[threadIdx.x]) + rank, e);
    }
    if (threadIdx.x < (unsigned)world) {
        const uint32_t *flag = reinterpret_cast<const uint32_t *>(peers.buf[rank]) + threadIdx.x;
        uint32_t polls = 0;
        while ((int32_t)(ld_acquire_sys(flag) - e) < 0) {
            if (++polls >= limit) { s_fail = 1; break; }
        }
    }
    __syncthreads();
    if (s_fail) {
        if (threadIdx.x == 0) atomicExch(&state->error, e);
    } else {
        float v[PER];
        {
            float p[kArMaxRanks][PER];
#pragma unroll
            for (int r = 0; r < kArMaxRanks; r++)
#pragma unroll
                for (int j = 0; j < PER; j++) {
                    const uint32_t i = threadIdx.x + kArThreads * j;
                    p[r][j] = 0.f;
                    if (r < world && i < width)
                        asm volatile("ld.relaxed.sys.global.f32 %0, [%1];"
                                     : "=f"(p[r][j]) : "l"(peers.buf[r] + half + base + i) : "memory");
                }
#pragma unroll
            for (int j = 0; j < PER; j++) {
                float s = p[0][j];
#pragma unroll
                for (int r = 1; r < kArMaxRanks; r++)
                    if (r < world) s += p[r][j];
                v[j] = s;
            }
        }
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < PER; j++) {
            const uint32_t i = threadIdx.x + kArThreads * j;
            if (i < width) {
                v[j] = __fadd_rn(residual[base + i], v[j]);
                sum_out[base + i] = v[j];
                acc = fmaf(v[j], v[j], acc);
            } else {
                v[j] = 0.f;
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
        for (int j = 0; j < PER; j++) {
            const uint32_t i = threadIdx.x + kArThreads * j;
            if (i < width) norm_out[base + i] = v[j] * scale * gain[i];
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(&state->done, 1u) == gridDim.x - 1) {
            state->arrived = 0;
            state->done = 0;
            __threadfence();
            *reinterpret_cast<volatile uint32_t *>(&state->epoch) = e;
        }
    }
}

// ---- in-place forms: the input already lies in the rank's own buffer -----------------------------
// The producer (the row-parallel product) writes its partial result straight into a region of the
// rank's buffer, so the all-reduce has nothing to copy and no grid-wide rendezvous of its own: the
// kernel boundary has already completed the region.  One thread signals every peer, every CTA waits
// for all flags (bounded, as above) and sums its slice of the region over the ranks.
// The caller owns the regions and must not rewrite one until another all-reduce call has passed in
// between (a peer may still be reading it until it has signalled its next call): two regions used
// alternately are enough.
__device__ __forceinline__ bool signal_and_wait(const ArPeers &peers, const ArState *state, int rank, int world,
                                                uint32_t e, int *s_fail)
{
    const uint32_t limit = spin_limit_of(state);
    if (threadIdx.x == 0) *s_fail = 0;
    __syncthreads();
    if (blockIdx.x == 0 && threadIdx.x < (unsigned)world)      // the release is cumulative at system scope
        st_release_sys(reinterpret_cast<uint32_t *>(peers.buf[threadIdx.x]) + rank, e);
    if (threadIdx.x < (unsigned)world) {
        const uint32_t *flag = reinterpret_cast<const uint32_t *>(peers.buf[rank]) + threadIdx.x;
        uint32_t polls = 0;
        while ((int32_t)(ld_acquire_sys(flag) - e) < 0) {
            if (++polls >= limit) { *s_fail = 1; break; }
        }
    }
    __syncthreads();
    return *s_fail == 0;
}

__device__ __forceinline__ void finish_call(ArState *state, uint32_t e)
{
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(&state->done, 1u) == gridDim.x - 1) {
            state->done = 0;
            __threadfence();
            *reinterpret_cast<volatile uint32_t *>(&state->epoch) = e;
        }
    }
}

// offset4: the region's start inside the buffer, in float4 units (flags included)
__global__ void __launch_bounds__(kArThreads)
peer_allreduce_inplace_kernel(ArPeers peers, ArState *state, int rank, int world, size_t offset4, float4 *out,
                              uint32_t n4)
{
    __shared__ int s_fail;
    const uint32_t e = *reinterpret_cast<volatile uint32_t *>(&state->epoch) + 1;
    if (!signal_and_wait(peers, state, rank, world, e, &s_fail)) {
        if (threadIdx.x == 0) atomicExch(&state->error, e);
    } else {
        const uint32_t stride = gridDim.x * kArThreads;
        for (uint32_t i = blockIdx.x * kArThreads + threadIdx.x; i < n4; i += stride) {
            float4 v[kArMaxRanks];
#pragma unroll
            for (int r = 0; r < kArMaxRanks; r++)
                if (r < world) v[r] = ld_peer(reinterpret_cast<const float4 *>(peers.buf[r]) + offset4 + i);
            float4 s = v[0];
#pragma unroll
            for (int r = 1; r < kArMaxRanks; r++)
                if (r < world) { s.x += v[r].x; s.y += v[r].y; s.z += v[r].z; s.w += v[r].w; }
            out[i] = s;
        }
    }
    finish_call(state, e);
}

// One CTA per row; sum_out = residual + sum over ranks, norm_out = RMSNorm(sum_out) * gain, with the
// element-to-thread map and the reduction orders of the AddRMSNorm kernel.
template <int PER>
__global__ void __launch_bounds__(kArThreads)
peer_allreduce_inplace_add_rmsnorm_kernel(ArPeers peers, ArState *state, int rank, int world, size_t offset,
                                          const float *residual, const float *gain, float *sum_out,
                                          float *norm_out, uint32_t width, float eps, float *amax_out)
{
    __shared__ int s_fail;
    __shared__ float red[8];
    __shared__ uint32_t red_mx[8];
    const uint32_t e = *reinterpret_cast<volatile uint32_t *>(&state->epoch) + 1;
    const size_t base = (size_t)blockIdx.x * width;
    if (!signal_and_wait(peers, state, rank, world, e, &s_fail)) {
        if (threadIdx.x == 0) atomicExch(&state->error, e);
    } else {
        // every rank's row in flight at once (up to 8 x PER loads per thread), then added in rank
        // order: one NVLink round trip for the row whatever the number of ranks (with one rank
        // fetched ahead of the adds, 8 ranks cost 8 round trips: 28 us per call against 13 at 2 ranks)
        float v[PER], part[kArMaxRanks][PER];
#pragma unroll
        for (int r = 0; r < kArMaxRanks; r++) {
            if (r < world) {
#pragma unroll
                for (int j = 0; j < PER; j++) {
                    const uint32_t i = threadIdx.x + kArThreads * j;
                    part[r][j] = 0.f;
                    if (i < width)
                        asm volatile("ld.relaxed.sys.global.f32 %0, [%1];"
                                     : "=f"(part[r][j]) : "l"(peers.buf[r] + offset + base + i) : "memory");
                }
            }
        }
#pragma unroll
        for (int j = 0; j < PER; j++) v[j] = part[0][j];
#pragma unroll
        for (int r = 1; r < kArMaxRanks; r++) {
            if (r < world) {
#pragma unroll
                for (int j = 0; j < PER; j++) v[j] = v[j] + part[r][j];
            }
        }
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < PER; j++) {
            const uint32_t i = threadIdx.x + kArThreads * j;
            if (i < width) {
                v[j] = __fadd_rn(residual[base + i], v[j]);
                sum_out[base + i] = v[j];
                acc = fmaf(v[j], v[j], acc);
            } else {
                v[j] = 0.f;
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
        uint32_t mx = 0;
#pragma unroll
        for (int j = 0; j < PER; j++) {
            const uint32_t i = threadIdx.x + kArThreads * j;
            if (i < width) {
                const float o = v[j] * scale * gain[i];
                norm_out[base + i] = o;
                mx = max(mx, __float_as_uint(fabsf(o)));
            }
        }
        if (amax_out) {            // the row's largest |norm|, for the int4 product that reads the row next
            mx = __reduce_max_sync(0xffffffffu, mx);
            if ((threadIdx.x & 31) == 0) red_mx[threadIdx.x >> 5] = mx;
            __syncthreads();
            if (threadIdx.x == 0) {
#pragma unroll
                for (int i = 1; i < kArThreads / 32; i++) mx = max(mx, red_mx[i]);
                amax_out[blockIdx.x] = __uint_as_float(mx);
            }
        }
    }
    finish_call(state, e);
}

}  // namespace ab

extern "C" AB_API size_t ab_peer_allreduce_buffer_bytes(uint32_t capacity_floats)
{
    return (size_t)ab::kArFlagWords * 4 + (size_t)2 * ((capacity_floats + 3) / 4 * 4) * 4;
}

extern "C" AB_API size_t ab_peer_allreduce_state_bytes(void) { return sizeof(ab::ArState); }

extern "C" AB_API int ab_peer_allreduce_f32(void *stream, void *const *peer_buffers, void *state, int rank,
                                            int world, const float *in, float *out, uint32_t n,
                                            uint32_t capacity_floats)
{
    using namespace ab;
    if (world < 1 || world > kArMaxRanks || rank < 0 || rank >= world)
        return fail(AB_ERR_INVALID, "ab_peer_allreduce_f32: rank %d of %d (at most %d ranks)", rank, world,
                    kArMaxRanks);
    if (!peer_buffers || !state || !in || !out)
        return fail(AB_ERR_INVALID, "ab_peer_allreduce_f32: NULL argument");
    const uint32_t cap = (capacity_floats + 3) / 4 * 4;
    if (n == 0 || n % 4 || n > cap)
        return fail(AB_ERR_INVALID, "ab_peer_allreduce_f32: %u elements (a multiple of 4, at most the "
                    "buffer's capacity of %u)", n, cap);
    if (reinterpret_cast<uintptr_t>(in) % 16 || reinterpret_cast<uintptr_t>(out) % 16)
        return fail(AB_ERR_INVALID, "ab_peer_allreduce_f32: input and output must be 16-byte aligned");
    ArPeers peers{};
    for (int r = 0; r < world; r++) {
        if (!peer_buffers[r] || reinterpret_cast<uintptr_t>(peer_buffers[r]) % 16)
            return fail(AB_ERR_INVALID, "ab_peer_allreduce_f32: buffer of rank %d is NULL or unaligned", r);
        peers.buf[r] = static_cast<float *>(peer_buffers[r]);
    }
    const uint32_t n4 = n / 4;
    // every CTA must be resident at once (they wait for peers, not for each other, but a peer's
    // signal needs ALL of that peer's CTAs to have copied): at most one CTA per SM
    uint32_t grid = (n4 + kArThreads - 1) / kArThreads;
    const uint32_t sms = (uint32_t)sm_count();
    if (grid > sms) grid = sms;
    peer_allreduce_kernel<<<grid, kArThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        peers, static_cast<ArState *>(state), rank, world, reinterpret_cast<const float4 *>(in),
        reinterpret_cast<float4 *>(out), n4, cap / 4);
    count_launch();
    return check_cuda(cudaGetLastError(), "ab_peer_allreduce_f32");
}

extern "C" AB_API int ab_peer_allreduce_error(const void *state, uint32_t *failed_call)
{
    using namespace ab;
    ArState h{};
    int rc = check_cuda(cudaMemcpy(&h, state, sizeof h, cudaMemcpyDeviceToHost), "ab_peer_allreduce_error");
    if (rc) return rc;
    if (failed_call) *failed_call = h.error;
    if (h.error) return fail(AB_ERR_TIMEOUT, "ab_peer_allreduce: call %u gave up waiting for its peers", h.error);
    return AB_OK;
}

extern "C" AB_API int ab_peer_allreduce_set_spin_limit(void *state, uint32_t polls)
{
    using namespace ab;
    if (!state) return fail(AB_ERR_INVALID, "ab_peer_allreduce_set_spin_limit: NULL state");
    return check_cuda(cudaMemcpy(static_cast<char *>(state) + offsetof(ArState, spin_limit), &polls, sizeof polls,
                                 cudaMemcpyHostToDevice), "ab_peer_allreduce_set_spin_limit");
}

extern "C" AB_API int ab_peer_allreduce_clear_error(void *state)
{
    using namespace ab;
    if (!state) return fail(AB_ERR_INVALID, "ab_peer_allreduce_clear_error: NULL state");
    const uint32_t zero = 0;
    return check_cuda(cudaMemcpy(static_cast<char *>(state) + offsetof(ArState, error), &zero, sizeof zero,
                                 cudaMemcpyHostToDevice), "ab_peer_allreduce_clear_error");
}

extern "C" AB_API int ab_peer_allreduce_add_rmsnorm_f32(void *stream, void *const *peer_buffers, void *state,
                                                        int rank, int world, const float *in,
                                                        const float *residual, const float *gain,
                                                        float *sum_out, float *norm_out, uint32_t rows,
                                                        uint32_t width, uint32_t eps_bits,
                                                        uint32_t capacity_floats)
{
    using namespace ab;
    if (world < 1 || world > kArMaxRanks || rank < 0 || rank >= world)
        return fail(AB_ERR_INVALID, "ab_peer_allreduce_add_rmsnorm_f32: rank %d of %d (at most %d ranks)", rank,
                    world, kArMaxRanks);
    if (!peer_buffers || !state || !in || !residual || !gain || !sum_out || !norm_out)
        return fail(AB_ERR_INVALID, "ab_peer_allreduce_add_rmsnorm_f32: NULL argument");
    const uint32_t cap = (capacity_floats + 3) / 4 * 4;
    if (rows == 0 || width == 0 || (uint64_t)rows * width > cap)
        return fail(AB_ERR_INVALID, "ab_peer_allreduce_add_rmsnorm_f32: %u rows of %u against a buffer of %u floats",
                    rows, width, cap);
    if (width > (uint32_t)kArThreads * 16 || rows > (uint32_t)sm_count())
        return fail(AB_ERR_INVALID, "ab_peer_allreduce_add_rmsnorm_f32: Width=%u (at most %u), Rows=%u (at most one "
                    "CTA per SM, %d); use ab_peer_allreduce_f32 and AddRMSNorm", width, kArThreads * 16, rows,
                    sm_count());
    ArPeers peers{};
    for (int r = 0; r < world; r++) {
        if (!peer_buffers[r] || reinterpret_cast<uintptr_t>(peer_buffers[r]) % 16)
            return fail(AB_ERR_INVALID, "ab_peer_allreduce_add_rmsnorm_f32: buffer of rank %d is NULL or unaligned", r);
        peers.buf[r] = static_cast<float *>(peer_buffers[r]);
    }
    float eps;
    memcpy(&eps, &eps_bits, 4);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    ArState *sp = static_cast<ArState *>(state);
    if (width <= (uint32_t)kArThreads * 4)
        peer_allreduce_add_rmsnorm_kernel<4><<<rows, kArThreads, 0, st>>>(peers, sp, rank, world, in, residual, gain,
                                                                          sum_out, norm_out, width, eps, cap);
    else
        peer_allreduce_add_rmsnorm_kernel<16><<<rows, kArThreads, 0, st>>>(peers, sp, rank, world, in, residual, gain,
                                                                           sum_out, norm_out, width, eps, cap);
    count_launch();
    return check_cuda(cudaGetLastError(), "ab_peer_allreduce_add_rmsnorm_f32");
}

static int peer_table(const char *what, void *const *peer_buffers, int rank, int world, ab::ArPeers &peers)
{
    using namespace ab;
    if (world < 1 || world > kArMaxRanks || rank < 0 || rank >= world)
        return fail(AB_ERR_INVALID, "%s: rank %d of %d (at most %d ranks)", what, rank, world, kArMaxRanks);
    if (!peer_buffers) return fail(AB_ERR_INVALID, "%s: NULL argument", what);
    for (int r = 0; r < world; r++) {
        if (!peer_buffers[r] || reinterpret_cast<uintptr_t>(peer_buffers[r]) % 16)
            return fail(AB_ERR_INVALID, "%s: buffer of rank %d is NULL or unaligned", what, r);
        peers.buf[r] = static_cast<float *>(peer_buffers[r]);
    }
    return AB_OK;
}

extern "C" AB_API size_t ab_peer_allreduce_region_offset_bytes(uint32_t capacity_floats)
{   // where caller-owned regions may start: behind the flags and the two halves of the copying form
    return ab_peer_allreduce_buffer_bytes(capacity_floats);
}

extern "C" AB_API int ab_peer_allreduce_inplace_f32(void *stream, void *const *peer_buffers, void *state, int rank,
                                                    int world, size_t region_offset_bytes, float *out, uint32_t n,
                                                    size_t buffer_bytes)
{
    using namespace ab;
    const char *what = "ab_peer_allreduce_inplace_f32";
    ArPeers peers{};
    int rc = peer_table(what, peer_buffers, rank, world, peers);
    if (rc) return rc;
    if (!state || !out || reinterpret_cast<uintptr_t>(out) % 16) return fail(AB_ERR_INVALID, "%s: NULL or unaligned argument", what);
    if (n == 0 || n % 4 || region_offset_bytes % 16 || region_offset_bytes < kArFlagWords * 4 ||
        region_offset_bytes + (size_t)n * 4 > buffer_bytes)
        return fail(AB_ERR_INVALID, "%s: %u elements (a multiple of 4) at byte %zu of a buffer of %zu bytes", what,
                    n, region_offset_bytes, buffer_bytes);
    const uint32_t n4 = n / 4;
    uint32_t grid = (n4 + kArThreads - 1) / kArThreads;
    const uint32_t sms = (uint32_t)sm_count();
    if (grid > sms) grid = sms;
    peer_allreduce_inplace_kernel<<<grid, kArThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        peers, static_cast<ArState *>(state), rank, world, region_offset_bytes / 16, reinterpret_cast<float4 *>(out), n4);
    count_launch();
    return check_cuda(cudaGetLastError(), what);
}

extern "C" AB_API int ab_peer_allreduce_inplace_add_rmsnorm_f32(void *stream, void *const *peer_buffers, void *state,
                                                                int rank, int world, size_t region_offset_bytes,
                                                                const float *residual, const float *gain,
                                                                float *sum_out, float *norm_out, uint32_t rows,
                                                                uint32_t width, uint32_t eps_bits,
                                                                size_t buffer_bytes)
{
    return ab_peer_allreduce_inplace_add_rmsnorm_amax_f32(stream, peer_buffers, state, rank, world, region_offset_bytes,
                                                          residual, gain, sum_out, norm_out, rows, width, eps_bits,
                                                          buffer_bytes, nullptr);
}

extern "C" AB_API int ab_peer_allreduce_inplace_add_rmsnorm_amax_f32(void *stream, void *const *peer_buffers, void *state,
                                                                     int rank, int world, size_t region_offset_bytes,
                                                                     const float *residual, const float *gain,
                                                                     float *sum_out, float *norm_out, uint32_t rows,
                                                                     uint32_t width, uint32_t eps_bits,
                                                                     size_t buffer_bytes, float *amax_out)
{
    using namespace ab;
    const char *what = "ab_peer_allreduce_inplace_add_rmsnorm_f32";
    ArPeers peers{};
    int rc = peer_table(what, peer_buffers, rank, world, peers);
    if (rc) return rc;
    if (!state || !residual || !gain || !sum_out || !norm_out) return fail(AB_ERR_INVALID, "%s: NULL argument", what);
    if (rows == 0 || width == 0 || region_offset_bytes % 16 || region_offset_bytes < kArFlagWords * 4 ||
        region_offset_bytes + (size_t)rows * width * 4 > buffer_bytes)
        return fail(AB_ERR_INVALID, "%s: %u rows of %u at byte %zu of a buffer of %zu bytes", what, rows, width,
                    region_offset_bytes, buffer_bytes);
    if (width > (uint32_t)kArThreads * 16 || rows > (uint32_t)sm_count())
        return fail(AB_ERR_INVALID, "%s: Width=%u (at most %u), Rows=%u (at most one CTA per SM, %d)", what, width,
                    kArThreads * 16, rows, sm_count());
    float eps;
    memcpy(&eps, &eps_bits, 4);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    ArState *sp = static_cast<ArState *>(state);
    const size_t off = region_offset_bytes / 4;
    if (width <= (uint32_t)kArThreads * 4)
        peer_allreduce_inplace_add_rmsnorm_kernel<4><<<rows, kArThreads, 0, st>>>(peers, sp, rank, world, off, residual,
                                                                                  gain, sum_out, norm_out, width, eps, amax_out);
    else
        peer_allreduce_inplace_add_rmsnorm_kernel<16><<<rows, kArThreads, 0, st>>>(peers, sp, rank, world, off, residual,
                                                                                   gain, sum_out, norm_out, width, eps, amax_out);
    count_launch();
    return check_cuda(cudaGetLastError(), what);
}
