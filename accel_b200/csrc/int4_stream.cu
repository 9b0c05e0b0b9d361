// int4 linear for decode batches (1 .. 32 activation rows per pass) over PREPACKED weights: the
// weight stream goes from HBM to shared memory by bulk asynchronous copies, from there through
// registers into tensor memory as the A operand of tcgen05.mma, and never exists in shared memory
// as f16.
//
//   out[m][n] = sum_k a[m][k] w(k,n),   w = s == 0 ? z : (code - z) s          (quant/int4.go:160-175,
//                                                                    internal/kernels/int4tiled.go:66)
//
// Inside one 128-column quantisation group the scale and zero of a weight depend on k only, so
//
//   out[m][n] = sum_k B[m][k] code[k][n]  -  sum_k B[m][k] z[k],     B[m][k] = f16(a[m][k] s[k] P_m)
//
// with the code the only thing the tensor core multiplies B by.  B is the one rounded operand (f16,
// 2^-11 per term).  P_m is an exact power of two chosen per activation row from the row's largest
// magnitude and from the group's largest scale, so that B sits in the upper part of the f16 range
// whatever the magnitude of the activations or weights; it is undone in the f32 epilogue.
//
// One MMA per 16 weight rows, D[128 x NB] += A[128 x 16] B[16 x NB] with A in tensor memory:
//   codes  A's 128 rows are the group's 128 columns (one per TMEM lane).  A thread owns a column:
//          the prepacked stream gives it 32 consecutive k of that column as one 16-byte shared
//          memory load; four masks per word turn eight codes into four f16x2 registers whose
//          halves are the f16 SUBNORMALS code * 2^-24 (or * 2^-20: the odd mask keeps the nibble
//          four bits up, and B carries 1/16 there), exactly; tcgen05.st puts 32 k of the column
//          into 16 TMEM columns of its lane.  0.7 instructions per weight, no conversion.
//   zeros  sum_k B[m][k] z[k] on the CUDA cores (fma.rn.f32.f16: exact products of the same rounded
//          B and the stream's f16 zeros, f32 sums), so the two sums cancel as they do in exact
//          arithmetic.  (A second MMA for this term was tried: tcgen05.mma has a floor of about 46
//          cycles per instruction whatever N, so it doubled the loop's time.)
//   B      K-major in shared memory (8 x 8 core matrices, no swizzle), written per 64-row chunk by
//          the expander threads from a (global, f32) and the chunk's scales (in the stream).
// A row whose scale is 0 is the constant z (internal/kernels/int4.go:85-87): its B is 0, the MMA
// skips it, and the threads that build B add a z in f32 (a branch taken only where a scale is 0).
//
// Stream layout (ab_int4_prepack): a header of one float per group, 2^E_s with E_s =
// floor(log2(the group's largest scale)), then per group and per chunk of 64 weight rows 4352
// contiguous bytes: 2 halves x 128 columns x 16 bytes of codes (word i of a column's 16 bytes
// holds k = 8i .. 8i+7 in nibbles 0,4,1,5,2,6,3,7), 64 scales (f16, divided by 2^E_s, and by 16
// where k % 8 is 2, 3, 6 or 7), 64 zeros (f16, times 16 in those rows).  A CTA's K range of one
// group is ONE contiguous run.
//
// Roles in a CTA of 352 threads: warps 0-7 expand codes and build B; warp 8 allocates TMEM; one
// lane each of warps 8 and 10 issues MMAs (two lanes, because one thread gets an MMA out only every
// 46 cycles); the lanes of warp 9 issue the bulk copies six chunks ahead.
// Stages are handed over by mbarriers (copy -> full -> expanders -> ready -> MMA -> commit -> free);
// there is no CTA-wide barrier in the loop.  K splits of a column group form a thread-block
// cluster: every CTA stores its partial rows into the shared memory of the CTA that owns the row
// and arrives on that CTA's mbarrier; the owner adds the splits in split order (deterministic, no
// workspace); one cluster-wide barrier at the end keeps the copies' sources alive.  Every wait is bounded: one that runs out sets g_sm100_error, the CTA skips its
// remaining work, frees its TMEM and returns.
#include <cooperative_groups.h>
#include <cuda_fp16.h>

#include <cstdlib>

#include "common.cuh"
#include "sm100.cuh"

namespace cg = cooperative_groups;

namespace ab {

static constexpr int kSxThreads = 352;
static constexpr int kSxExpanders = 256;
static constexpr int kSxIssuers = 2;               // lanes that issue MMAs (warps 8 and 10)
static constexpr int kSxNC = 6;                   // ring stages in flight from global memory
static constexpr int kSxNA = 3;                   // A (TMEM) and B (shared) stages
__host__ __device__ constexpr uint32_t sx_tmem_cols(int G) { return G == 1 ? 128u : 256u; }   // per group: D (32) + 3 x 32

#ifdef SX_TRACE
// cycle stamps and per-phase cycle sums of CTA (0,0), for tuning builds only
__device__ long long g_sx_trace[64];
#define SX_STAMP(i) do { if (blockIdx.x == 0 && blockIdx.y == 0) g_sx_trace[i] = clock64(); } while (0)
#define SX_ACC(i, t) do { sx_acc[(i) & 7] += clock64() - (t); } while (0)
#define SX_FLUSH(base) do { if (blockIdx.x == 0 && blockIdx.y == 0) for (int q_ = 0; q_ < 8; q_++) g_sx_trace[(base) + q_] += sx_acc[q_]; } while (0)
#define SX_NOW() clock64()
#define SX_DECL() long long sx_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}
__device__ long long g_sx_cta[2048][4];          // per CTA: SM, start, loop end, end (cycles of its SM)
#define SX_CTA(i) do { const unsigned b_ = blockIdx.y * gridDim.x + blockIdx.x; if (b_ < 2048) { \
        if ((i) == 1) { unsigned sm_; asm volatile("mov.u32 %0, %%smid;" : "=r"(sm_)); g_sx_cta[b_][0] = sm_; } \
        g_sx_cta[b_][i] = clock64(); } } while (0)
#else
#define SX_CTA(i) do { } while (0)
#define SX_STAMP(i) do { } while (0)
#define SX_ACC(i, t) do { (void)(t); } while (0)
#define SX_FLUSH(base) do { } while (0)
#define SX_NOW() 0ll
#define SX_DECL() do { } while (0)
#endif

// acc += f16(lo of b) * f16(lo of z) + f16(hi of b) * f16(hi of z): exact products, f32 sums
__device__ __forceinline__ void sx_fma_pairs(float &acc, uint32_t b, uint32_t z)
{
    asm("{\n\t.reg .b16 bl, bh, zl, zh;\n\tmov.b32 {bl, bh}, %1;\n\tmov.b32 {zl, zh}, %2;\n\t"
        "fma.rn.f32.f16 %0, bl, zl, %0;\n\tfma.rn.f32.f16 %0, bh, zh, %0;\n\t}"
        : "+f"(acc) : "r"(b), "r"(z));
}

static constexpr int kSxNB = 16;                                    // activation rows per pass
static constexpr int kSxMaxSplits = 8;                              // K splits of a tile = cluster size
static constexpr int kSxRecvRows = kSxNB + kSxMaxSplits;            // partial rows a CTA receives, rounded up
static constexpr uint32_t kSxLbo = kSxNB * 16u + 16u;              // B: k-block stride (+16: bank spread)
static constexpr uint32_t kSxBStage = 8u * kSxLbo;                 // B: 64 k x 16 rows of one group
__host__ __device__ constexpr size_t sx_smem_bytes(int G)
{
    return (size_t)kSxNC * G * kSxChunkBytes + (size_t)kSxNA * G * kSxBStage + (size_t)G * (kSxRecvRows + kSxNB) * 128 * 4 +
           (size_t)(G + 1) * kSxNB * 4 + (2 * kSxNC + 2 * kSxNA + 2) * 8 + 16 + 128 + 256;
}

// grid = (ceil(N / 128 / G), K splits), cluster = (1, splits, 1); a CTA owns G adjacent column
// groups.  a: [M][K] f32 (M <= 16 rows of this pass), amax: the largest magnitude of each of the M
// rows, or [M][ep.amax_parts] maxima of parts of a row of which the largest counts (NULL: every CTA
// scans its own K range), packed: the stream, ep: where the columns go (and, for the SwiGLU form,
// where the largest |out| of every warp's 32 columns goes).
template <int G>
__global__ void __launch_bounds__(kSxThreads)
int4_stream_kernel(const float *__restrict__ a, const float *__restrict__ amax,
                   const unsigned char *__restrict__ packed, const SxEpilogue ep, uint32_t M, uint32_t N,
                   uint32_t K, uint32_t nchunks_total, uint32_t header_bytes)
{
    extern __shared__ __align__(128) unsigned char sx_raw[];
    constexpr int NB = kSxNB;
    constexpr uint32_t kStage = G * kSxChunkBytes;                   // one ring stage: G groups' chunk
    constexpr uint32_t kA0 = G * 32;                                  // TMEM: D per group (32 columns apart), then A stages
    constexpr uint32_t kSxTmemCols = sx_tmem_cols(G);
    static_assert(kA0 + G * kSxNA * 32 <= kSxTmemCols, "TMEM budget");
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(sx_raw) + 127) & ~(uintptr_t)127);
    unsigned char *ring = smem;
    unsigned char *bring = ring + kSxNC * kStage;
    float *recv = reinterpret_cast<float *>(bring + kSxNA * G * kSxBStage);   // [rows][G][128] partial rows of the K splits
    float *tile = recv + kSxRecvRows * G * 128;                                // [NB][G][128] this CTA's partial rows
    float *unscale = tile + NB * G * 128;                                      // [NB] 2^(E_a - 12)
    float *zsum = unscale + NB;                                                // [G][NB] zero-point term
    uint64_t *w_full = reinterpret_cast<uint64_t *>(zsum + G * NB);
    uint64_t *w_empty = w_full + kSxNC;
    uint64_t *ab_ready = w_empty + kSxNC;
    uint64_t *ab_free = ab_ready + kSxNA;
    uint64_t *done = ab_free + kSxNA;
    uint64_t *red_bar = done + 1;                                              // partial rows have arrived
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(red_bar + 1);
    volatile int *s_abort = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) { SX_STAMP(0); SX_CTA(1); }
    const uint32_t groups = N / 128, g0 = blockIdx.x * G, splits = gridDim.y, split = blockIdx.y;
    const uint32_t gcount = min((uint32_t)G, groups - g0);          // the last tile may hold fewer groups
    const uint32_t c_beg = (uint32_t)((uint64_t)nchunks_total * split / splits);
    const uint32_t c_end = (uint32_t)((uint64_t)nchunks_total * (split + 1) / splits);
    const uint32_t nch = c_end - c_beg;
    const uint32_t kbeg = c_beg * kSxChunkK;
    const unsigned char *stream = packed + header_bytes + ((size_t)g0 * nchunks_total + c_beg) * kSxChunkBytes;
    const size_t group_stride = (size_t)nchunks_total * kSxChunkBytes;

    if (warp == 9) {
        // the copy warp initialises the barriers and starts the first stages at once (the weights
        // depend on nothing that runs before this kernel).  The barriers lie one after another
        // (w_full, w_empty, ab_ready, ab_free, done, red_bar): one lane initialises each, and one
        // lane issues each of the first copies; a single lane doing them in a row spends a few
        // hundred cycles apiece
        constexpr int kBars = 2 * kSxNC + 2 * kSxNA + 2;
        if (lane < kBars) {
            // w_empty, ab_ready: one arrival per expander warp; ab_free, done: one commit per MMA lane
            const uint32_t count = lane < kSxNC ? 1u : lane < 2 * kSxNC + kSxNA ? (uint32_t)(kSxExpanders / 32)
                                   : lane < kBars - 1 ? (uint32_t)kSxIssuers : 1u;
            sx_bar_init(&w_full[lane], count);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncwarp();
        if (lane == 31) {
            *s_abort = 0;
            if (splits > 1) {
                // this CTA owns rows split, split + splits, ... of the tile: their partial sums arrive
                // from every CTA of the cluster as bulk copies that count bytes on red_bar
                const uint32_t owned = M > split ? (M - split + splits - 1) / splits : 0u;
                sx_bar_expect_tx(red_bar, owned * splits * (uint32_t)G * 128u * 4u);
            }
            SX_STAMP(40);
        }
        {   // lane = stage * G + group: the lane of a stage's first group announces the stage's bytes
            const uint32_t st0 = (uint32_t)lane / G, gi = (uint32_t)lane % G;
            if (st0 < (uint32_t)kSxNC && st0 < nch && gi < gcount) {
                if (gi == 0) sx_bar_expect_tx(&w_full[st0], gcount * kSxChunkBytes);
                sx_bulk_load(ring + st0 * kStage + gi * kSxChunkBytes,
                             stream + gi * group_stride + (size_t)st0 * kSxChunkBytes, kSxChunkBytes, &w_full[st0]);
            }
        }
        if (lane == 0) SX_STAMP(41);
    }
    if (warp == 8) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(sx_smem(tmem_slot)), "r"(kSxTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        if (lane == 0) SX_STAMP(42);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    // every CTA of the cluster has initialised its barriers before anyone's partial rows arrive
    // (waited for at the end of the loop, long after)
    if (tid == 0) SX_STAMP(43);
    // (relaxed: the barrier initialisations were published by fence.mbarrier_init above)
    if (splits > 1) asm volatile("barrier.cluster.arrive.relaxed;" ::: "memory");
    if (tid == 0) SX_STAMP(1);
    // a dependent launch may begin now: it only prefetches its own weights until this grid is done
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 9) {
        // ---- the copy lane: the groups' runs of chunks, kSxNC stages ahead of the expanders (the
        //      first stages were issued before the CTA-wide barrier)
        if (lane == 0) {
            SX_DECL();
            for (uint32_t c = kSxNC; c < nch; c++) {     // the first kSxNC stages are already on their way
                const uint32_t st = c % kSxNC;
                long long tt = SX_NOW();
                if (!sx_bar_wait(&w_empty[st], ((c / kSxNC) - 1) & 1)) { *s_abort = 1; break; }
                SX_ACC(0, tt);
                sx_bar_expect_tx(&w_full[st], gcount * kSxChunkBytes);
                for (uint32_t gi = 0; gi < gcount; gi++)
                    sx_bulk_load(ring + st * kStage + gi * kSxChunkBytes,
                                 stream + gi * group_stride + (size_t)c * kSxChunkBytes, kSxChunkBytes, &w_full[st]);
            }
            SX_FLUSH(32);
        }
    } else if (warp == 8 || warp == 10) {
        // ---- the MMA lanes: per group and 16 weight rows, codes (A in tensor memory) times B.  One
        //      thread gets an MMA of this shape out every 46 cycles whatever the tensor pipe has to
        //      do (measured: 8 cycles' worth at N = 16), and several threads overlap, so two lanes
        //      share the work, each with an accumulator of its own (MMAs of different threads are
        //      not ordered among themselves): with two groups a lane takes one group, with one
        //      group a lane takes two of the four k slices and the epilogue adds the two sums
        if (lane == 0) {
            constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(NB >> 3) << 17) | ((128u >> 4) << 24);
            const uint32_t q = warp == 8 ? 0u : 1u;
            const uint32_t gi = G == 2 ? q : 0u, j0 = G == 2 ? 0u : 2u * q, nj = G == 2 ? 4u : 2u;
            const uint32_t dcol = tmem + (G == 2 ? gi * 32u : q * 16u);
            SX_DECL();
            for (uint32_t c = 0; c < nch; c++) {
                const uint32_t ab = c % kSxNA;
                long long tt = SX_NOW();
                if (!sx_bar_wait(&ab_ready[ab], (c / kSxNA) & 1)) { *s_abort = 1; break; }
                SX_ACC(0, tt);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (gi < gcount) {
                    const uint32_t bbase = sx_smem(bring + (ab * G + gi) * kSxBStage);
#pragma unroll 4
                    for (uint32_t jj = 0; jj < nj; jj++) {
                        const uint32_t j = j0 + jj;
                        sx_mma_ts(dcol, tmem + kA0 + (gi * kSxNA + ab) * 32 + 8 * j,
                                  sx_desc(bbase + j * 2 * kSxLbo, kSxLbo, 128), idesc, (c > 0 || jj > 0) ? 1u : 0u);
                    }
                }
                sx_commit(&ab_free[ab]);             // arrives once this lane's MMAs have read A and B
            }
            sx_commit(done);
            if (q == 0) { SX_STAMP(21); SX_FLUSH(24); }
        }
    } else {
        // ---- expanders: warp w puts k-half w/4 of columns 32 (w%4) + lane of every group into TMEM;
        //      thread tid builds B for activation row tid/16 and the weight rows 4 (tid%16) ...
        const int h = warp >> 2;
        const uint32_t tcol = (uint32_t)((warp & 3) * 32 + lane);
        const uint32_t tlane = ((uint32_t)((warp & 3) * 32)) << 16;
        const uint32_t bm = (uint32_t)tid >> 4, bq = (uint32_t)tid & 15u;
        float es[G];                                 // 2^E_s of each group
#pragma unroll
        for (int gi = 0; gi < G; gi++)
            es[gi] = (uint32_t)gi < gcount ? __ldg(reinterpret_cast<const float *>(packed) + g0 + gi) : 1.f;

        // the activations are the previous kernel's output: wait for it (a no-op otherwise)
        asm volatile("griddepcontrol.wait;" ::: "memory");
        uint32_t *amax_s = reinterpret_cast<uint32_t *>(zsum);      // zsum is written after the loop
        if (amax == nullptr) {
            // no row maxima given: all expanders scan the slice [M rows][this CTA's k] together,
            // eight 16-byte loads in flight per thread; a warp's loads lie in one row except
            // where it crosses a row end
            if (tid < NB) amax_s[tid] = 0u;
            asm volatile("bar.sync 1, 256;" ::: "memory");
            const uint32_t kvalid = min(K - kbeg, nch * kSxChunkK), kc4 = kvalid >> 2, total = M * kc4;
            for (uint32_t base0 = (uint32_t)(tid - lane); base0 < total; base0 += kSxExpanders * 8) {   // warp-uniform
                const uint32_t base = base0 + (uint32_t)lane;
                float4 v[8];
                uint32_t row[8];
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const uint32_t idx = base + kSxExpanders * j;
                    row[j] = 0xffffffffu;
                    v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (idx < total) {
                        row[j] = idx / kc4;
                        v[j] = __ldg(reinterpret_cast<const float4 *>(a + (size_t)row[j] * K + kbeg) + (idx - row[j] * kc4));
                    }
                }
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const uint32_t bits = __float_as_uint(fmaxf(fmaxf(fabsf(v[j].x), fabsf(v[j].y)),
                                                                fmaxf(fabsf(v[j].z), fabsf(v[j].w))));
                    const uint32_t r0 = __shfl_sync(0xffffffffu, row[j], 0);
                    if (__all_sync(0xffffffffu, row[j] == r0 || row[j] == 0xffffffffu)) {
                        const uint32_t mx = __reduce_max_sync(0xffffffffu, row[j] == r0 ? bits : 0u);
                        if (lane == 0 && r0 != 0xffffffffu) atomicMax(&amax_s[r0], mx);
                    } else if (row[j] != 0xffffffffu) {
                        atomicMax(&amax_s[row[j]], bits);
                    }
                }
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");
        }
        const bool brow = bm < M;
        uint32_t mb = 0u;
        if (amax == nullptr) {
            mb = brow ? amax_s[bm] : 0u;
        } else if (ep.amax_parts <= 1) {
            mb = brow ? __float_as_uint(fabsf(__ldg(amax + bm))) : 0u;
        } else {
            // the row's maximum is the largest of its entries: the sixteen threads of a row (lanes
            // 16 apart never mix) share the loads
            if (brow)
                for (uint32_t q = bq; q < ep.amax_parts; q += 16)
                    mb = max(mb, __float_as_uint(fabsf(__ldg(amax + (size_t)bm * ep.amax_parts + q))));
#pragma unroll
            for (int sh = 8; sh > 0; sh >>= 1) mb = max(mb, __shfl_xor_sync(0xffffffffu, mb, sh));
        }
        const int ea = sx_row_exponent(mb);
        const float pa = __uint_as_float((uint32_t)(127 + 12 - ea) << 23);            // 2^(12 - E_a)
        const float *ax = a + (size_t)(brow ? bm : 0) * K + kbeg + 4 * bq;            // next activations to load
        const uint32_t k0 = kbeg + 4 * bq;           // K is a multiple of 4: a quad is inside or outside
        uint32_t xleft = (brow && k0 < K) ? min(nch, (K - k0 + kSxChunkK - 1) / kSxChunkK) : 0u;
        float zacc[G], zfx[G];                       // zero-point term; constant rows' term
#pragma unroll
        for (int gi = 0; gi < G; gi++) zacc[gi] = zfx[gi] = 0.f;
        if (amax == nullptr) asm volatile("bar.sync 1, 256;" ::: "memory");    // amax_s (= zsum) is free again
        if (tid == 0) SX_STAMP(2);
        SX_DECL();
        auto load_x = [&]() -> float4 {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (xleft) {
                v = __ldg(reinterpret_cast<const float4 *>(ax));
                ax += kSxChunkK;
                xleft--;
            }
            return v;
        };
        float4 xr[3];                                // this thread's activations, two chunks ahead
        xr[0] = load_x();
        xr[1] = load_x();
        bool alive = true;
        // the loop is unrolled over one period of both rings so that stage addresses are constants
        static_assert(kSxNC % kSxNA == 0, "one unrolled period covers both rings");
        for (uint32_t c0 = 0; c0 < nch && alive; c0 += kSxNC) {
            const uint32_t full_par = (c0 / kSxNC) & 1u;
#pragma unroll
            for (int u = 0; u < kSxNC; u++) {
                const uint32_t c = c0 + u;
                if (c >= nch) break;
                constexpr int kPeriod = kSxNC / kSxNA;
                const int ab = u % kSxNA;
                // stage ab is used for the (c / NA)-th time: kPeriod uses per outer iteration
                const uint32_t free_par = (uint32_t)((c0 / kSxNC) * kPeriod + u / kSxNA - 1) & 1u;
                long long tt = SX_NOW();
                xr[(u + 2) % 3] = load_x();
                SX_ACC(6, tt);
                tt = SX_NOW();
                if (!sx_bar_wait(&w_full[u], full_par)) { *s_abort = 1; alive = false; }
                { SX_ACC(0, tt); if (c == 0) SX_STAMP(3); }
                tt = SX_NOW();
                if (alive && c >= (uint32_t)kSxNA && !sx_bar_wait(&ab_free[ab], free_par)) { *s_abort = 1; alive = false; }
                SX_ACC(1, tt);
                tt = SX_NOW();
                if (!__all_sync(0xffffffffu, alive)) { alive = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned char *stage = ring + u * kStage;
                // A: 32 k of this thread's column of every group
#pragma unroll
                for (int gi = 0; gi < G; gi++) {
                    if ((uint32_t)gi < gcount) {
                        const uint4 cw = *reinterpret_cast<const uint4 *>(stage + gi * kSxChunkBytes + ((uint32_t)h * 128u + tcol) * 16u);
                        uint32_t r[16];
                        const uint32_t w4[4] = {cw.x, cw.y, cw.z, cw.w};
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const uint32_t w = w4[i], w8 = w >> 8;
                            r[4 * i + 0] = w & 0x000F000Fu;
                            r[4 * i + 1] = w & 0x00F000F0u;
                            r[4 * i + 2] = w8 & 0x000F000Fu;
                            r[4 * i + 3] = w8 & 0x00F000F0u;
                        }
                        sx_tmem_st16(tmem + tlane + kA0 + (gi * kSxNA + ab) * 32 + (uint32_t)h * 16u, r);
                    }
                }
                SX_ACC(2, tt);
                tt = SX_NOW();
                // B: row bm, weight rows 4 bq .. 4 bq + 3 of the chunk, one tile per group:
                // f16(a 2^(12 - E_a)) times the group's normalised scale of the row
                if (brow) {
                    const float4 x = xr[u % 3];
                    const float x0 = x.x * pa, x1 = x.y * pa, x2 = x.z * pa, x3 = x.w * pa;
                    const __half2 xh01 = __floats2half2_rn(x0, x1), xh23 = __floats2half2_rn(x2, x3);
#pragma unroll
                    for (int gi = 0; gi < G; gi++) {
                        if ((uint32_t)gi < gcount) {
                            const unsigned char *gs = stage + gi * kSxChunkBytes + kSxCodeBytes;
                            const uint2 sv = *reinterpret_cast<const uint2 *>(gs + 8 * bq);
                            const uint2 zv = *reinterpret_cast<const uint2 *>(gs + 128 + 8 * bq);
                            const __half2 b01 = __hmul2(xh01, *reinterpret_cast<const __half2 *>(&sv.x));
                            const __half2 b23 = __hmul2(xh23, *reinterpret_cast<const __half2 *>(&sv.y));
                            const uint32_t b01u = *reinterpret_cast<const uint32_t *>(&b01);
                            const uint32_t b23u = *reinterpret_cast<const uint32_t *>(&b23);
                            *reinterpret_cast<uint2 *>(bring + (ab * G + gi) * kSxBStage + (bq >> 1) * kSxLbo + (bq & 1) * 8 +
                                                       (bm >> 3) * 128 + (bm & 7) * 16) = make_uint2(b01u, b23u);
                            // the zero-point term, from the same rounded B the tensor core multiplies
                            sx_fma_pairs(zacc[gi], b01u, zv.x);
                            sx_fma_pairs(zacc[gi], b23u, zv.y);
                            // a scale of 0 marks a constant row (rare): its term is a z, in f32
                            if (((sv.x & 0x7fffu) == 0u) | ((sv.x & 0x7fff0000u) == 0u) |
                                ((sv.y & 0x7fffu) == 0u) | ((sv.y & 0x7fff0000u) == 0u)) {
                                const float2 z01 = __half22float2(*reinterpret_cast<const __half2 *>(&zv.x));
                                const float2 z23 = __half22float2(*reinterpret_cast<const __half2 *>(&zv.y));
                                float z = zfx[gi];
                                if ((sv.x & 0x7fffu) == 0u) z = fmaf(-x0, z01.x, z);
                                if ((sv.x & 0x7fff0000u) == 0u) z = fmaf(-x1, z01.y, z);
                                if ((sv.y & 0x7fffu) == 0u) z = fmaf(-x2, z23.x, z);
                                if ((sv.y & 0x7fff0000u) == 0u) z = fmaf(-x3, z23.y, z);
                                zfx[gi] = z;
                            }
                        }
                    }
                }
                SX_ACC(3, tt);
                tt = SX_NOW();
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                SX_ACC(4, tt);
                tt = SX_NOW();
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) {
                    sx_bar_arrive(&ab_ready[ab]);
                    sx_bar_arrive(&w_empty[u]);
                }
                SX_ACC(5, tt);
            }
        }
        if (tid == 0) { SX_STAMP(4); SX_FLUSH(8); SX_CTA(2); }
        if (tid == 224) SX_FLUSH(16);
        // the zero-point term of each activation row (sixteen lanes hold parts of it); the constant
        // rows' part was summed in units that lack the group's power of two
#pragma unroll
        for (int gi = 0; gi < G; gi++) {
            float z = zacc[gi];
            z += zfx[gi] / es[gi];
#pragma unroll
            for (int sh = 8; sh > 0; sh >>= 1) z += __shfl_xor_sync(0xffffffffu, z, sh);
            if (bq == 0) zsum[gi * NB + bm] = z;
        }
        if (bq == 0) unscale[bm] = __uint_as_float((uint32_t)(127 + ea - 12) << 23);
        asm volatile("bar.sync 1, 256;" ::: "memory");          // zsum and unscale are complete
        // read the accumulators: lane = column, TMEM column = activation row
        if (warp < 4) {
            bool ok = !*s_abort && sx_bar_wait(done, 0);
            if (tid == 0) SX_STAMP(5);
            if (!ok) *s_abort = 1;
            ok = __all_sync(0xffffffffu, ok);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (splits > 1) asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
            if (tid == 0) SX_STAMP(9);
            {   // the four warps decide together (they meet at a barrier below)
                uint32_t all;
                asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.and.pred p, 2, 128, q;\n\t"
                             "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(all) : "r"((uint32_t)ok) : "memory");
                ok = all != 0;
            }
            if (ok) {
                const uint32_t rank = split;         // cluster = the K splits of this tile, in order
                // one finished row of the tile: both groups' sums of column tcol
                auto emit = [&](uint32_t m, const float (&v)[G]) {
                    if (G == 2 && ep.swiglu) {
                        const float o = __fdiv_rn(v[0], 1.f + expf(-v[0])) * v[G - 1];
                        ep.out0[(size_t)m * ep.ld0 + (size_t)blockIdx.x * 128 + tcol] = o;
                        if (ep.max_out) {            // this warp's 32 columns of row m (NaN counts as the largest)
                            const uint32_t mx = __reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(o)));
                            if (lane == 0) ep.max_out[(size_t)m * ep.max_ld + blockIdx.x * 4 + warp] = __uint_as_float(mx);
                        }
                    } else {
#pragma unroll
                        for (int gi = 0; gi < G; gi++)
                            if ((uint32_t)gi < gcount) sx_store(ep, m, g0 + gi, tcol, v[gi]);
                    }
                };
                float vals[G][16];
#pragma unroll
                for (int gi = 0; gi < G; gi++) {
                    if ((uint32_t)gi < gcount) {
                        uint32_t r[16];
                        sx_tmem_ld16(tmem + tlane + gi * 32, r);
                        if (G == 1) {                // the second MMA lane's sum, 16 columns on
                            uint32_t r2[16];
                            sx_tmem_ld16(tmem + tlane + 16, r2);
#pragma unroll
                            for (int i = 0; i < 16; i++) r[i] = __float_as_uint(__uint_as_float(r[i]) + __uint_as_float(r2[i]));
                        }
                        if (tid == 0 && gi == 0) SX_STAMP(10);
#pragma unroll
                        for (int i = 0; i < 16; i++)
                            vals[gi][i] = (__uint_as_float(r[i]) * 16777216.f - zsum[gi * NB + i]) * (unscale[i] * es[gi]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; i++) vals[gi][i] = 0.f;
                    }
                }
                if (splits == 1) {
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        if ((uint32_t)i < M) {
                            float v[G];
#pragma unroll
                            for (int gi = 0; gi < G; gi++) v[gi] = vals[gi][i];
                            emit((uint32_t)i, v);
                        }
                    }
                } else {
                    // this CTA's partial rows go through a local tile, from where row i leaves as one
                    // bulk copy into the shared memory of CTA i % splits of the cluster, slot
                    // (i / splits) * splits + rank, counting bytes on that CTA's barrier
#pragma unroll
                    for (int i = 0; i < 16; i++)
#pragma unroll
                        for (int gi = 0; gi < G; gi++) tile[(i * G + gi) * 128 + tcol] = vals[gi][i];
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    asm volatile("bar.sync 2, 128;" ::: "memory");
                    if (lane < NB / 4 && (uint32_t)(lane * 4 + warp) < M) {     // four rows per warp: issuing is slow
                        const uint32_t i = (uint32_t)(lane * 4 + warp), owner = i % splits, slot = (i / splits) * splits + rank;
                        uint32_t raddr, rbar;
                        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
                                     : "=r"(raddr) : "r"(sx_smem(&recv[slot * G * 128])), "r"(owner));
                        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rbar) : "r"(sx_smem(red_bar)), "r"(owner));
                        asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                     ::"r"(raddr), "r"(sx_smem(&tile[i * G * 128])), "r"((uint32_t)(G * 128 * 4)), "r"(rbar) : "memory");
                    }
                    if (tid == 0) SX_STAMP(7);
                    // the rows this CTA owns, from every K split in split order
                    const uint32_t baddr = sx_smem(red_bar);
                    const long long t0 = clock64();
                    bool got = false;
                    for (;;) {
                        uint32_t d;
                        asm volatile("{\n\t.reg .pred p;\n\t"
                                     "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
                                     "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(d) : "r"(baddr), "r"(0u) : "memory");
                        if (d) { got = true; break; }
                        if (clock64() - t0 > kSxWaitCycles) break;
                    }
                    if (!got) { atomicExch(&g_sm100_error, 1); *s_abort = 1; }
                    if (tid == 0) SX_STAMP(8);
                    if (__all_sync(0xffffffffu, got)) {
                        for (uint32_t m = rank, j = 0; m < M; m += splits, j++) {
                            float v[G];
#pragma unroll
                            for (int gi = 0; gi < G; gi++) {
                                v[gi] = 0.f;
                                if ((uint32_t)gi < gcount) {
                                    v[gi] = recv[((j * splits) * G + gi) * 128 + tcol];
                                    for (uint32_t q = 1; q < splits; q++) v[gi] += recv[((j * splits + q) * G + gi) * 128 + tcol];
                                }
                            }
                            emit(m, v);
                        }
                    }
                }
            }
        } else if (splits > 1) {
            asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
        }
    }
    if (warp >= 8 && splits > 1) {
        __syncwarp();                                // the working lane rejoins its warp
        asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
    }
    if (splits > 1) {
        // the bulk copies that carry this CTA's partial rows read its shared memory until they are
        // done, which is when every CTA of the cluster has received its rows: nobody leaves before
        // (relaxed: nothing has to become visible through this barrier; a thread arrives only after
        // it has seen its own CTA's rows complete, in program order, and the release form costs
        // about 2000 cycles more)
        __syncwarp();
        asm volatile("barrier.cluster.arrive.relaxed;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
    }
    if (tid == 0) { SX_STAMP(6); SX_CTA(3); }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 8)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kSxTmemCols) : "memory");
}

// The largest magnitude of each activation row (NaN counts as the largest): one CTA per row.
__global__ void __launch_bounds__(256)
int4_row_absmax_kernel(const float *__restrict__ a, float *__restrict__ amax, uint32_t K)
{
    __shared__ uint32_t part[8];
    // under a programmatic dependent launch: let the product that follows begin its weight prefetch,
    // and wait for the kernel that writes the activations
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const float *row = a + (size_t)blockIdx.x * K;
    uint32_t mx = 0;
    for (uint32_t k = threadIdx.x; k < K; k += 256) mx = max(mx, __float_as_uint(fabsf(row[k])));
    mx = __reduce_max_sync(0xffffffffu, mx);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < 8; i++) mx = max(mx, part[i]);
        amax[blockIdx.x] = __uint_as_float(mx);
    }
}

// ---- prepack ----------------------------------------------------------------------------------------
// Three passes, each reading and writing whole sectors (the permutation also runs per call when a
// large batch arrives in the reference layout, so it is worth keeping near the copy rate).
//
// header word g <- the f16 bits of the group's largest finite scale (scales are non-negative, so
// their bit patterns order like their values).  grid = blocks of 64 weight rows; a thread walks
// groups g, g + 256, ... of its block's rows, so a warp reads 64 contiguous bytes per row.
__global__ void __launch_bounds__(256)
int4_prepack_smax_kernel(const uint16_t *__restrict__ scales, uint32_t *header, uint32_t groups, uint32_t K)
{
    const uint32_t k0 = blockIdx.x * 64, k1 = min(K, k0 + 64);
    for (uint32_t g = threadIdx.x; g < groups; g += 256) {
        uint32_t mx = 0;
        for (uint32_t k = k0; k < k1; k++) {
            const uint32_t sb = scales[(size_t)k * groups + g];
            if (!(sb & 0x8000u) && sb < 0x7c00u) mx = max(mx, sb);
        }
        if (mx) atomicMax(&header[g], mx);
    }
}

// header word g: the largest scale's f16 bits  ->  the float 2^floor(log2(largest scale))
__global__ void int4_prepack_header_kernel(uint32_t *header, uint32_t groups)
{
    const uint32_t g = blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= groups) return;
    const float smax = __half2float(__ushort_as_half((unsigned short)header[g]));
    int es = 0;
    if (smax > 0.f) es = (int)((__float_as_uint(smax) >> 23) & 0xffu) - 127;
    header[g] = (uint32_t)(127 + es) << 23;
}

// Codes.  grid = (groups, ceil(chunks / 8)), 256 threads: 32 threads per chunk of 64 weight rows x 128
// columns.  Thread (h, wc) reads the 32 words that hold rows 32 h .. 32 h + 31 of columns
// 8 wc .. 8 wc + 7 (a half warp reads 64 contiguous bytes per row), transposes the 32 x 8 nibbles in
// registers and writes each column's 16 bytes (32 consecutive k, word i = k 8i .. 8i + 7 in nibbles
// 0,4,1,5,2,6,3,7): 128 contiguous bytes per thread.
__global__ void __launch_bounds__(256)
int4_prepack_codes_kernel(const uint32_t *__restrict__ codes, unsigned char *__restrict__ packed, uint32_t N, uint32_t K,
                          uint32_t nchunks, uint32_t header_bytes)
{
    const uint32_t g = blockIdx.x, c = blockIdx.y * 8 + (threadIdx.x >> 5);
    if (c >= nchunks) return;
    const uint32_t t = threadIdx.x & 31, h = t >> 4, wc = t & 15;
    unsigned char *dst = packed + header_bytes + ((size_t)g * nchunks + c) * kSxChunkBytes;
    const uint32_t kbase = c * kSxChunkK + h * 32;
    const size_t word0 = ((size_t)g * 128 + wc * 8) >> 3;           // N is a multiple of 128: rows start on words
    const size_t row_words = N >> 3;
    uint32_t in[32];
#pragma unroll
    for (int r = 0; r < 32; r++) in[r] = kbase + r < K ? __ldg(codes + (size_t)(kbase + r) * row_words + word0) : 0u;
#pragma unroll
    for (int j = 0; j < 8; j++) {                                   // column 8 wc + j
        uint32_t out[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            uint32_t w = 0;
#pragma unroll
            for (int q = 0; q < 8; q++) {
                const int pos = (q >> 1) + 4 * (q & 1);              // k0 k1 k2 k3 ... -> nibbles 0 4 1 5 2 6 3 7
                w |= ((in[8 * i + q] >> (4 * j)) & 0xFu) << (4 * pos);
            }
            out[i] = w;
        }
        *reinterpret_cast<uint4 *>(dst + (h * 128 + wc * 8 + j) * 16) = make_uint4(out[0], out[1], out[2], out[3]);
    }
}

// Scales and zeros.  grid = (ceil(groups / 32), chunks), 256 threads: the chunk's 64 rows of 32 adjacent
// groups are read row by row (64 contiguous bytes per plane and row), turned in shared memory, and
// written as each group's 64 scales and 64 zeros (128 contiguous bytes each).
//
// Rows whose codes sit four bits up in the A operand (k % 8 in 2, 3, 6, 7) carry 1/16 in their
// scale and 16 in their zero: powers of two, exact unless the value leaves the f16 range.  A
// constant row (scale 0) keeps its value as it is: the kernels add it apart.
__global__ void __launch_bounds__(256)
int4_prepack_meta_kernel(const uint16_t *__restrict__ scales, const uint16_t *__restrict__ zeros,
                         unsigned char *__restrict__ packed, uint32_t N, uint32_t K, uint32_t nchunks, uint32_t header_bytes)
{
    __shared__ uint16_t ss[64][33], zs[64][33];
    const uint32_t groups = N / 128, g0 = blockIdx.x * 32, c = blockIdx.y;
    for (uint32_t i = threadIdx.x; i < 64 * 32; i += 256) {
        const uint32_t kk = i >> 5, gi = i & 31, k = c * kSxChunkK + kk, g = g0 + gi;
        uint16_t sb = 0, zb = 0;
        if (k < K && g < groups) { sb = scales[(size_t)k * groups + g]; zb = zeros[(size_t)k * groups + g]; }
        ss[kk][gi] = sb;
        zs[kk][gi] = zb;
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < 32 * 64; i += 256) {
        const uint32_t gi = i >> 6, kk = i & 63, g = g0 + gi;
        if (g >= groups) continue;
        const uint32_t sb = ss[kk][gi], zb = zs[kk][gi];
        const float es = reinterpret_cast<const float *>(packed)[g];                  // 2^E_s
        float sn = __half2float(__ushort_as_half((unsigned short)sb)) / es;
        float zn = __half2float(__ushort_as_half((unsigned short)zb));
        if ((kk & 2) && (sb & 0x7fffu) != 0u) { sn *= 0.0625f; zn *= 16.f; }
        unsigned char *dst = packed + header_bytes + ((size_t)g * nchunks + c) * kSxChunkBytes + kSxCodeBytes;
        reinterpret_cast<__half *>(dst)[kk] = __float2half_rn(sn);
        reinterpret_cast<__half *>(dst + 128)[kk] = __float2half_rn(zn);
    }
}

bool int4_stream_ok(uint32_t M, uint32_t N, uint32_t K)
{
    return M >= 1 && N > 0 && K > 0 && N % 128 == 0 && K % 4 == 0;
}

size_t int4_stream_packed_bytes(uint32_t N, uint32_t K)
{
    if (N == 0 || N % 128) return 0;
    const size_t nchunks = (K + kSxChunkK - 1) / kSxChunkK;
    return sx_header_bytes(N) + (size_t)(N / 128) * nchunks * kSxChunkBytes;
}

// From how many activation rows a call wants the rows' maxima computed once, ahead of the product:
// every CTA scanning its own slice of a costs more than a small kernel of its own (16 rows of 4096 x
// 11008: 18.6 us against 15.6 us; the whole decode step 8.46 against 7.98 ms).
static constexpr uint32_t kSxAmaxFromRows = 3;

size_t int4_stream_workspace(uint32_t M) { return M >= kSxAmaxFromRows ? align_up((size_t)M * 4, 256) : 0; }

int run_int4_prepack(cudaStream_t stream, const uint32_t *codes, const uint16_t *scales, const uint16_t *zeros,
                     unsigned char *packed, uint32_t N, uint32_t K)
{
    const uint32_t groups = N / 128, nchunks = (K + kSxChunkK - 1) / kSxChunkK;
    const size_t hb = sx_header_bytes(N);
    int rc = check_cuda(cudaMemsetAsync(packed, 0, hb, stream), "int4 prepack header");
    if (rc) return rc;
    int4_prepack_smax_kernel<<<(K + 63) / 64, 256, 0, stream>>>(scales, reinterpret_cast<uint32_t *>(packed), groups, K);
    count_launch();
    int4_prepack_header_kernel<<<(groups + 127) / 128, 128, 0, stream>>>(reinterpret_cast<uint32_t *>(packed), groups);
    count_launch();
    int4_prepack_codes_kernel<<<dim3(groups, (nchunks + 7) / 8), 256, 0, stream>>>(codes, packed, N, K, nchunks, (uint32_t)hb);
    count_launch();
    int4_prepack_meta_kernel<<<dim3((groups + 31) / 32, nchunks), 256, 0, stream>>>(scales, zeros, packed, N, K, nchunks,
                                                                                  (uint32_t)hb);
    count_launch();
    return check_cuda(cudaGetLastError(), "int4 prepack");
}

struct SxPlan { int G; uint32_t tiles, splits, nchunks; };

template <int G> static void sx_config(cudaLaunchConfig_t &cfg, cudaLaunchAttribute *attr, uint32_t tiles, uint32_t splits)
{
    cfg = {};
    cfg.gridDim = dim3(tiles, splits);
    cfg.blockDim = dim3(kSxThreads);
    cfg.dynamicSmemBytes = sx_smem_bytes(G);
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = splits;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
}

template <int G> static int sx_prepare()
{
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        int rc = check_cuda(cudaFuncSetAttribute(int4_stream_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)sx_smem_bytes(G)), "int4_stream_kernel shared memory");
        if (rc) return rc;
        // the kernel touches global memory through bulk copies and a few broadcast loads: all of the
        // SM's memory as shared memory, so that several CTAs fit
        rc = check_cuda(cudaFuncSetAttribute(int4_stream_kernel<G>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                             (int)cudaSharedmemCarveoutMaxShared), "int4_stream_kernel carve-out");
        if (rc) return rc;
        attr_set[dev] = true;
    }
    return AB_OK;
}

// How many clusters of `splits` CTAs the device holds at once.  Clusters do not straddle GPCs, so
// this is less than the CTA slots divided by the cluster size; the runtime's answer is for ONE CTA
// per SM (its occupancy calculation gives a kernel that allocates tensor memory one CTA per SM,
// although several run side by side when their columns fit), so it is scaled by the CTAs per SM
// this kernel's registers, shared memory and tensor-memory columns allow: a lower bound.
template <int G> static uint32_t sx_resident_clusters(uint32_t splits)
{
    static int cached[64][kSxMaxSplits + 1] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (cached[dev][splits] == 0) {
        int n = 0;
        cudaLaunchConfig_t cfg;
        cudaLaunchAttribute attr[1];
        sx_config<G>(cfg, attr, splits, splits);
        cudaFuncAttributes fa{};
        if (sx_prepare<G>() != AB_OK || cudaOccupancyMaxActiveClusters(&n, int4_stream_kernel<G>, &cfg) != cudaSuccess ||
            n <= 0 || cudaFuncGetAttributes(&fa, int4_stream_kernel<G>) != cudaSuccess) {
            cudaGetLastError();
            n = (int)((uint32_t)sm_count() / splits * 3 / 4);           // a cautious guess
            fa.numRegs = 96;
        }
        const uint32_t by_regs = 65536u / ((uint32_t)((fa.numRegs + 7) / 8 * 8) * kSxThreads);
        const uint32_t by_smem = (uint32_t)(233472 / (sx_smem_bytes(G) + 1024));
        const uint32_t by_tmem = 512u / sx_tmem_cols(G);
        uint32_t per_sm = by_regs < by_smem ? by_regs : by_smem;
        if (by_tmem < per_sm) per_sm = by_tmem;
        if (per_sm < 1) per_sm = 1;
        cached[dev][splits] = n * (int)per_sm;
    }
    return (uint32_t)cached[dev][splits];
}

static SxPlan sx_plan(uint32_t N, uint32_t K)
{
    SxPlan p{};
    const uint32_t groups = N / 128;
    p.nchunks = (K + kSxChunkK - 1) / kSxChunkK;
    // A CTA owns two adjacent groups where the matrix is wide enough to fill the SMs that way (the
    // activations are converted once for both).  The K splits of a tile form one cluster: as many
    // as keep every cluster resident at once, at most 8, each with a few chunks to stream.
    p.G = groups >= 64 ? 2 : 1;
#ifdef SX_TRACE
    if (getenv("SX_G")) p.G = atoi(getenv("SX_G"));
#endif
    p.tiles = (groups + p.G - 1) / p.G;
    uint32_t splits = 1;
    for (uint32_t s = kSxMaxSplits; s > 1; s--) {
        if (s * 2 > p.nchunks) continue;
        const uint32_t fit = p.G == 2 ? sx_resident_clusters<2>(s) : sx_resident_clusters<1>(s);
        if (p.tiles <= fit) { splits = s; break; }
    }
#ifdef SX_TRACE
    if (getenv("SX_SPLITS")) splits = (uint32_t)atoi(getenv("SX_SPLITS"));
#endif
    p.splits = splits;
    return p;
}

template <int G>
static int sx_launch(cudaStream_t stream, const float *a, const float *amax, const unsigned char *packed,
                     const SxEpilogue &ep, uint32_t M, uint32_t N, uint32_t K, const SxPlan &p, bool dependent)
{
    int rc = sx_prepare<G>();
    if (rc) return rc;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[2];
    sx_config<G>(cfg, attr, p.tiles, p.splits);
    cfg.stream = stream;
    if (dependent) {
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs = 2;
    }
    const uint32_t hb = (uint32_t)sx_header_bytes(N);
    rc = check_cuda(cudaLaunchKernelEx(&cfg, int4_stream_kernel<G>, a, amax, packed, ep, M, N, K, p.nchunks, hb),
                    "int4_stream_kernel");
    count_launch();
    return rc;
}

int run_row_absmax(cudaStream_t stream, const float *a, float *amax, uint32_t M, uint32_t K, bool dependent)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(M);
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = dependent ? 1 : 0;
    int rc = check_cuda(cudaLaunchKernelEx(&cfg, int4_row_absmax_kernel, a, amax, K), "int4_row_absmax_kernel");
    count_launch();
    return rc;
}

// The product in passes of at most 16 activation rows.  amax: the rows' largest magnitudes if the
// caller has them; else `scratch` (int4_stream_workspace(M) bytes) receives them from a small
// kernel, or, for one or two rows, every CTA finds its own.  mode: kSxPlain (out0 = [M][N]),
// kSxSplit3 (columns [0, n1) -> out0, [n1, n2) -> out1, [n2, N) -> out2, each contiguous) or
// kSxSwiGLU (groups alternate gate, up; out0 = [M][N / 2]).
enum { kSxPlain = 0, kSxSplit3 = 1, kSxSwiGLU = 2 };

static int run_int4_stream_mode(cudaStream_t stream, const float *a, const float *amax, const unsigned char *packed,
                                int mode, float *out0, float *out1, float *out2, uint32_t n1, uint32_t n2, uint32_t M,
                                uint32_t N, uint32_t K, uint32_t ld0, void *scratch, bool dependent,
                                uint32_t amax_parts = 1, float *max_out = nullptr)
{
    SxPlan p = sx_plan(N, K);
    if (mode == kSxSwiGLU && p.G != 2) {             // (gate, up) pairs are tiles of two groups
        p.G = 2;
        p.tiles = (N / 128 + 1) / 2;
        while (p.splits > 1 && p.tiles > sx_resident_clusters<2>(p.splits)) p.splits--;
    }
    if (!amax && M >= kSxAmaxFromRows) {
        if (!scratch) return fail(AB_ERR_INVALID, "the prepacked int4 product of %u rows needs %zu bytes of scratch", M,
                                  int4_stream_workspace(M));
        int rc = run_row_absmax(stream, a, static_cast<float *>(scratch), M, K, dependent);
        if (rc) return rc;
        amax = static_cast<const float *>(scratch);
    }
    for (uint32_t m0 = 0; m0 < M; m0 += kSxNB) {
        const uint32_t rows = M - m0 < (uint32_t)kSxNB ? M - m0 : (uint32_t)kSxNB;
        const float *ap = a + (size_t)m0 * K, *mp = amax ? amax + (size_t)m0 * amax_parts : nullptr;
        SxEpilogue ep{};
        ep.amax_parts = amax_parts;
        if (max_out) {
            ep.max_ld = N / 64;                      // four warps per tile of 256 columns
            ep.max_out = max_out + (size_t)m0 * ep.max_ld;
        }
        ep.g1 = ep.g2 = 0xffffffffu;
        ep.ld0 = ld0;
        ep.out0 = out0 + (size_t)m0 * ld0;
        if (mode == kSxSplit3) {
            ep.g1 = n1 / 128; ep.g2 = n2 / 128;
            ep.ld0 = n1; ep.ld1 = n2 - n1; ep.ld2 = N - n2;
            ep.out0 = out0 + (size_t)m0 * ep.ld0;
            ep.out1 = out1 + (size_t)m0 * ep.ld1;
            ep.out2 = out2 + (size_t)m0 * ep.ld2;
        }
        ep.swiglu = mode == kSxSwiGLU ? 1u : 0u;
        int rc = p.G == 2 ? sx_launch<2>(stream, ap, mp, packed, ep, rows, N, K, p, dependent)
                          : sx_launch<1>(stream, ap, mp, packed, ep, rows, N, K, p, dependent);
        if (rc) return rc;
    }
    note_selection("int4 stream kernel (bulk copies -> shared memory -> tensor memory, tcgen05 M=128 x N=16 x "
                   "K=16, f16 operands, TMEM f32 accumulator), %u tiles of %d column groups x a cluster of %u K "
                   "splits, %u chunks of 64 rows, %u pass(es) of 16 activation rows", p.tiles, p.G, p.splits,
                   p.nchunks, (M + kSxNB - 1) / kSxNB);
    return AB_OK;
}

int run_int4_stream(cudaStream_t stream, const float *a, const float *amax, const unsigned char *packed, float *out,
                    uint32_t M, uint32_t N, uint32_t K, uint32_t ldo, void *scratch, bool dependent, uint32_t amax_parts)
{
    return run_int4_stream_mode(stream, a, amax, packed, kSxPlain, out, nullptr, nullptr, 0, 0, M, N, K, ldo, scratch,
                                dependent, amax_parts ? amax_parts : 1u);
}

int int4_stream_error_flag()
{
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_sm100_error, sizeof v) != cudaSuccess) { cudaGetLastError(); return -1; }
    return v;
}

// ---- dispatch by name: bindings a, packed, out; GEMMDims{M,N,K} ------------------------------------
// Programmatic dependent launch: the product starts while its predecessor in the stream is still
// running, prefetches its weights (which depend on nothing) and waits for the predecessor only
// before it reads the activations.  AB_INT4_PDL=0 launches it the ordinary way (for measurements).
static bool sx_pdl()
{
    static const bool pdl = !(getenv("AB_INT4_PDL") && atoi(getenv("AB_INT4_PDL")) == 0);
    return pdl;
}

// From how many activation rows the tile kernel (int4_gemm.cu: weights dequantised once per CTA,
// 128 rows per tile) takes over from passes of 16 rows of the decode kernel.  Measured at 4096 x
// 11008: a pass of 16 rows 15.6 us, a wave of tiles 52 us whatever the rows: three passes are
// cheaper, four are not.
static constexpr uint32_t kPackedTileFromRows = 49;
static bool packed_tiles(uint32_t M) { return M >= kPackedTileFromRows; }
static size_t packed_workspace(uint32_t M, uint32_t K)
{
    return packed_tiles(M) ? int4_gemm_workspace(M, K) : int4_stream_workspace(M);
}

// The "...A" names take the activation rows' largest magnitudes as a second binding (amax f32[M], what
// AddRMSNormAmax leaves): the decode kernel then needs no kernel of its own for them.  ax = 1 where the
// binding is present; the batch kernel (from kPackedTileFromRows rows) finds its own factors and ignores it.
static int launch_packed(Launch &l, const char *name, uint32_t M, uint32_t N, uint32_t K, int ax = 0)
{
    // the "A" form's fourth uniform word: entries per row of the amax binding (0 or 1: one per row);
    // with P entries a row's maximum is the largest of them (what the attention kernels and the
    // SwiGLU product leave: one per head and warp, one per tile and warp)
    const uint32_t parts = ax && l.ubytes >= 16 && u32_at(l.u, 12) ? u32_at(l.u, 12) : 1u;
    if (!int4_stream_ok(M, N, K))
        return fail(AB_ERR_INVALID, "%s: M=%u N=%u K=%u; the prepacked form needs N a multiple of 128 and K a "
                    "multiple of 4", name, M, N, K);
    const size_t ws = (ax && !packed_tiles(M)) ? 0 : packed_workspace(M, K);
    if (l.query_ws) { l.ws_need = ws; return AB_OK; }
    const size_t need = int4_stream_packed_bytes(N, K);
    if (l.len[0] < (uint64_t)M * K || (uint64_t)l.len[1 + ax] * 4 < need || l.len[2 + ax] < (uint64_t)M * N ||
        (ax && l.len[1] < (uint64_t)M * parts))
        return fail(AB_ERR_INVALID, "%s: M=%u N=%u K=%u needs a[%llu] packed[%zu bytes] out[%llu] (and amax[%llu]); the "
                    "lengths block says %u, %u words, %u", name, M, N, K, (unsigned long long)M * K, need,
                    (unsigned long long)M * N, (unsigned long long)M * parts, l.len[0], l.len[1 + ax], l.len[2 + ax]);
    if (ws > l.ws_bytes || (ws && !l.ws))
        return fail(AB_ERR_INVALID, "%s: needs %zu bytes of workspace, given %zu", name, ws, l.ws_bytes);
    if (packed_tiles(M))
        return run_int4_gemm_mode(l.stream, ptr<const float>(l, 0), ptr<const unsigned char>(l, 1 + ax), kSxPlain,
                                  ptr<float>(l, 2 + ax), nullptr, nullptr, 0, 0, M, N, K, N, l.ws);
    return run_int4_stream(l.stream, ptr<const float>(l, 0), ax ? ptr<const float>(l, 1) : nullptr,
                           ptr<const unsigned char>(l, 1 + ax), ptr<float>(l, 2 + ax), M, N, K, N, l.ws, sx_pdl(), parts);
}

// a, packed, out0, out1, out2; uniform {M, N, K, N1, N2, 0, 0, 0}: columns [0, N1) of the product go to
// out0 [M][N1], [N1, N1 + N2) to out1 [M][N2], the rest to out2 (the fused q | k | v product)
static int launch_split3(Launch &l, const char *name, int ax);
int launch_quant_matmul_int4_packed_split3(Launch &l) { return launch_split3(l, "QuantMatMulInt4PackedSplit3", 0); }
int launch_quant_matmul_int4_packed_split3_a(Launch &l) { return launch_split3(l, "QuantMatMulInt4PackedSplit3A", 1); }

static int launch_split3(Launch &l, const char *name, int ax)
{
    const uint32_t M = u32_at(l.u, 0), N = u32_at(l.u, 4), K = u32_at(l.u, 8), N1 = u32_at(l.u, 12), N2 = u32_at(l.u, 16);
    if (!int4_stream_ok(M, N, K) || N1 % 128 || N2 % 128 || N1 == 0 || N2 == 0 || (uint64_t)N1 + N2 >= N)
        return fail(AB_ERR_INVALID, "%s: M=%u N=%u K=%u N1=%u N2=%u; N, N1 and N2 are multiples of 128 with "
                    "N1 + N2 < N, K a multiple of 4", name, M, N, K, N1, N2);
    const size_t ws = (ax && !packed_tiles(M)) ? 0 : packed_workspace(M, K);
    if (l.query_ws) { l.ws_need = ws; return AB_OK; }
    const uint32_t N3 = N - N1 - N2;
    if (l.len[0] < (uint64_t)M * K || (uint64_t)l.len[1 + ax] * 4 < int4_stream_packed_bytes(N, K) ||
        l.len[2 + ax] < (uint64_t)M * N1 || l.len[3 + ax] < (uint64_t)M * N2 || l.len[4 + ax] < (uint64_t)M * N3 ||
        (ax && l.len[1] < M))
        return fail(AB_ERR_INVALID, "%s: M=%u N=%u K=%u N1=%u N2=%u; a[%u] packed[%u words] out0[%u] out1[%u] out2[%u]",
                    name, M, N, K, N1, N2, l.len[0], l.len[1 + ax], l.len[2 + ax], l.len[3 + ax], l.len[4 + ax]);
    if (ws > l.ws_bytes || (ws && !l.ws))
        return fail(AB_ERR_INVALID, "%s: needs %zu bytes of workspace, given %zu", name, ws, l.ws_bytes);
    if (packed_tiles(M))
        return run_int4_gemm_mode(l.stream, ptr<const float>(l, 0), ptr<const unsigned char>(l, 1 + ax), kSxSplit3,
                                  ptr<float>(l, 2 + ax), ptr<float>(l, 3 + ax), ptr<float>(l, 4 + ax), N1, N1 + N2, M, N, K,
                                  N1, l.ws);
    return run_int4_stream_mode(l.stream, ptr<const float>(l, 0), ax ? ptr<const float>(l, 1) : nullptr,
                                ptr<const unsigned char>(l, 1 + ax), kSxSplit3, ptr<float>(l, 2 + ax), ptr<float>(l, 3 + ax),
                                ptr<float>(l, 4 + ax), N1, N1 + N2, M, N, K, N1, l.ws, sx_pdl());
}

// a, packed, out; GEMMDims{M, N, K}: the 128-column groups of the packed matrix alternate gate, up;
// out [M][N / 2] = SwiGLU(gate, up)
// "...SwiGLUAMax" has a fifth binding, outmax f32[M][N / 64]: entry 4 t + w of a row is the largest
// |out| among the 32 columns warp w of tile t wrote (a tile is 128 output columns), for the product
// that reads out next (its "A" form with AmaxParts = N / 64).  Decode kernel only (fewer than 49 rows).
static int launch_swiglu(Launch &l, const char *name, int ax, int mx = 0);
int launch_quant_matmul_int4_packed_swiglu(Launch &l) { return launch_swiglu(l, "QuantMatMulInt4PackedSwiGLU", 0); }
int launch_quant_matmul_int4_packed_swiglu_a(Launch &l) { return launch_swiglu(l, "QuantMatMulInt4PackedSwiGLUA", 1); }
int launch_quant_matmul_int4_packed_swiglu_a_max(Launch &l) { return launch_swiglu(l, "QuantMatMulInt4PackedSwiGLUAMax", 1, 1); }

static int launch_swiglu(Launch &l, const char *name, int ax, int mx)
{
    const uint32_t M = u32_at(l.u, 0), N = u32_at(l.u, 4), K = u32_at(l.u, 8);
    if (!int4_stream_ok(M, N, K) || N % 256)
        return fail(AB_ERR_INVALID, "%s: M=%u N=%u K=%u; N is a multiple of 256 (gate and up groups in pairs), K a "
                    "multiple of 4", name, M, N, K);
    const size_t ws = (ax && !packed_tiles(M)) ? 0 : packed_workspace(M, K);
    if (l.query_ws) { l.ws_need = ws; return AB_OK; }
    if (l.len[0] < (uint64_t)M * K || (uint64_t)l.len[1 + ax] * 4 < int4_stream_packed_bytes(N, K) ||
        l.len[2 + ax] < (uint64_t)M * (N / 2) || (ax && l.len[1] < M) || (mx && l.len[3 + ax] < (uint64_t)M * (N / 64)))
        return fail(AB_ERR_INVALID, "%s: M=%u N=%u K=%u; a[%u] packed[%u words] out[%u]%s", name, M, N, K, l.len[0],
                    l.len[1 + ax], l.len[2 + ax], mx ? " outmax[M * N / 64]" : "");
    if (ws > l.ws_bytes || (ws && !l.ws))
        return fail(AB_ERR_INVALID, "%s: needs %zu bytes of workspace, given %zu", name, ws, l.ws_bytes);
    if (mx && packed_tiles(M))
        return fail(AB_ERR_INVALID, "%s: M=%u; the form that leaves row maxima runs on the decode kernel, fewer than "
                    "%u rows (use QuantMatMulInt4PackedSwiGLUA)", name, M, kPackedTileFromRows);
    if (packed_tiles(M))
        return run_int4_gemm_mode(l.stream, ptr<const float>(l, 0), ptr<const unsigned char>(l, 1 + ax), kSxSwiGLU,
                                  ptr<float>(l, 2 + ax), nullptr, nullptr, 0, 0, M, N, K, N / 2, l.ws);
    return run_int4_stream_mode(l.stream, ptr<const float>(l, 0), ax ? ptr<const float>(l, 1) : nullptr,
                                ptr<const unsigned char>(l, 1 + ax), kSxSwiGLU, ptr<float>(l, 2 + ax), nullptr, nullptr, 0, 0,
                                M, N, K, N / 2, l.ws, sx_pdl(), 1, mx ? ptr<float>(l, 3 + ax) : nullptr);
}

int launch_quant_matvec_int4_packed(Launch &l)
{
    return launch_packed(l, "QuantMatVecInt4Packed", 1, u32_at(l.u, 4), u32_at(l.u, 8));
}

int launch_quant_matmul_int4_packed(Launch &l)
{
    return launch_packed(l, "QuantMatMulInt4Packed", u32_at(l.u, 0), u32_at(l.u, 4), u32_at(l.u, 8));
}

int launch_quant_matmul_int4_packed_a(Launch &l)
{
    return launch_packed(l, "QuantMatMulInt4PackedA", u32_at(l.u, 0), u32_at(l.u, 4), u32_at(l.u, 8), 1);
}

}  // namespace ab

extern "C" AB_API size_t ab_int4_prepack_bytes(uint32_t K, uint32_t N)
{
    return ab::int4_stream_packed_bytes(N, K);
}

extern "C" AB_API int ab_int4_prepack(void *stream, const uint32_t *codes, const uint16_t *scales,
                                      const uint16_t *zeros, uint32_t K, uint32_t N, void *packed)
{
    using namespace ab;
    if (!codes || !scales || !zeros || !packed) return fail(AB_ERR_INVALID, "ab_int4_prepack: NULL argument");
    if (N == 0 || K == 0 || N % 128)
        return fail(AB_ERR_INVALID, "ab_int4_prepack: K=%u N=%u; N must be a multiple of 128 (whole quantisation "
                    "groups per row)", K, N);
    if (reinterpret_cast<uintptr_t>(packed) % 256)
        return fail(AB_ERR_INVALID, "ab_int4_prepack: the destination must be 256-byte aligned");
    return run_int4_prepack(static_cast<cudaStream_t>(stream), codes, scales, zeros, static_cast<unsigned char *>(packed), N, K);
}

extern "C" AB_API int ab_int4_stream_error(void)
{
    int v = ab::int4_stream_error_flag();
    if (v == 0) v = ab::int4_gemm_error_flag();
    if (v > 0) return ab::fail(AB_ERR_TIMEOUT, "an int4 kernel over the prepacked stream gave up a bounded wait");
    return v < 0 ? AB_ERR_CUDA : AB_OK;
}
