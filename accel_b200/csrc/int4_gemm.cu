// int4 linear for batches of activation rows (from 17 rows up) over the PREPACKED weight stream:
//
//   out[m][n] = sum_k a[m][k] w(k,n),   w = s == 0 ? z : (code - z) s          (quant/int4.go:160-175,
//                                                                    internal/kernels/int4tiled.go:66)
//
// The WEIGHTS are dequantised, not the activations: a tile of 128 columns x 64 weight rows becomes
// f16 once per CTA whatever the number of activation rows, and goes from registers straight into
// tensor memory as the A operand of tcgen05.mma (it never exists in shared memory as f16).  The
// activations are rounded to f16 ONCE per call by a small kernel that also lays them out as the
// MMA's B tiles (K-major 8 x 8 core matrices, 128 rows x 64 k = 16 KB contiguous), so a tile
// arrives in shared memory by one bulk asynchronous copy and needs no tensor map.
//
//   A[n][k]   = f16( (code - z) s / 2^E_s )      E_s = floor(log2(largest scale of the 128-column group))
//   B[m][k]   = f16( a[m][k] 2^(14 - E_a[m]) )   E_a = floor(log2(largest magnitude of row m))
//   out[m][n] = D[n][m] 2^(E_s + E_a - 14),      D = A B^T accumulated in f32 in tensor memory
//
// Both powers of two are exact; they keep the operands inside the f16 range whatever the magnitude
// of weights and activations.  Two rounded operands (2^-11 each per term) instead of the one of the
// decode kernels: bf16 would be 2^-8 per term and misses the 1e-3 bar.
//
// Dequantisation per pair of weights (f16x2): the prepacked word gives the codes as f16 subnormals
// (code 2^-24, or code 2^-20 in the rows whose nibble sits four bits up; the stream's scales and
// zeros carry the matching 1/16 and 16): u = sub 2^15 - z 2^-9 (one fused multiply-add),
// w = u (s 2^9).  A row whose scale is 0 is the constant z (internal/kernels/int4.go:85-87): the
// warp finds such rows with one ballot per chunk and patches them (rare).
//
// A CTA owns G adjacent column groups (G = 1 or 2, sharing one B tile) and 128 activation rows; its
// accumulators are G x 128 TMEM columns.  Roles in a CTA of 320 threads: warps 0-7 dequantise (and
// read the accumulators out at the end); one lane of warp 8 issues the MMAs (M = 128 columns,
// N = 128 activation rows, K = 16 per instruction); warp 9 issues the bulk copies, two lanes per
// stage of a ring of 5 (one group) or 8 (two groups) stages.  Stages are handed over by mbarriers
// (copy -> full -> dequantisers -> a_ready -> MMA -> commit -> a_free and free); there is no
// CTA-wide barrier in the loop.  Every wait is bounded: one that runs
// out sets the error flag, the role leaves its loop, the CTA frees its TMEM and returns.
#include <cuda_fp16.h>

#include <cstdlib>

#include "common.cuh"
#include "sm100.cuh"

namespace ab {

static constexpr int kGmThreads = 320;
static constexpr int kGmExpanderWarps = 8;
static constexpr int kGmBN = 128;                                   // activation rows per tile
static constexpr int kGmNA = 4;                                     // A stages in tensor memory
// stages of the shared-memory ring (weights + B tile): as deep as lets two CTAs of one group, or one
// CTA of two groups, share an SM; what is in flight per SM has to cover the latency of L2
__host__ __device__ constexpr int gm_stages(int G) { return G == 1 ? 5 : 8; }
static constexpr uint32_t kGmLbo = kGmBN * 16;                      // B: stride between 8-k blocks of a tile
static constexpr uint32_t kGmBTile = 8 * kGmLbo;                    // one B tile: 128 rows x 64 k, f16, 16 KB
static constexpr uint32_t kGmPassRows = 4096;                       // activation rows converted per pass
__host__ __device__ constexpr uint32_t gm_stage_bytes(int G) { return (uint32_t)G * kSxChunkBytes + kGmBTile; }
__host__ __device__ constexpr uint32_t gm_tmem_cols(int G) { return G == 1 ? 256u : 512u; }     // D: G x 128, A: G x 4 x 32
__host__ __device__ constexpr size_t gm_smem_bytes(int G)
{
    return (size_t)gm_stages(G) * gm_stage_bytes(G) + kGmBN * 4 + (size_t)kGmExpanderWarps * G * 256 +
           (2 * gm_stages(G) + 2 * kGmNA + 1) * 8 + 16 + 128;
}

#ifdef GM_TRACE
// cycle sums per phase of CTA 0's traced threads, for tuning builds only
__device__ long long g_gm_trace[64];
#define GM_NOW() clock64()
#define GM_ADD(i, t0) do { if (blockIdx.x == 0) atomicAdd(reinterpret_cast<unsigned long long *>(&g_gm_trace[i]), (unsigned long long)(clock64() - (t0))); } while (0)
#define GM_STAMP(i) do { if (blockIdx.x == 0) g_gm_trace[i] = clock64(); } while (0)
#else
#define GM_NOW() 0ll
#define GM_ADD(i, t0) do { (void)(t0); } while (0)
#define GM_STAMP(i) do { } while (0)
#endif

// Which rows a block of 128 tile rows stands for.  Dense product: block rb is rows 128 rb ... of the
// one matrix (table NULL).  Grouped product (rows sorted by expert, internal/kernels/groupedtiled.go:77):
// every expert's segment is cut into blocks of its own, so a tile never mixes experts; entry rb of
// the table holds {expert, first row, rows (1..128)} and *total the number of blocks in use.
struct GmRows {
    const uint4 *table;
    const uint32_t *total;
    unsigned long long expert_stride;      // bytes between the experts' packed matrices
};

// offsets[e] .. offsets[e + 1]: expert e's rows (SegmentOffsets, internal/kernels/segment.go:40).
// One thread: at most a few thousand blocks.
__global__ void gm_group_plan_kernel(const uint32_t *__restrict__ offsets, uint32_t experts, uint32_t tokens,
                                     uint4 *table, uint32_t *total, uint32_t capacity)
{
    if (threadIdx.x || blockIdx.x) return;
    uint32_t n = 0;
    for (uint32_t e = 0; e < experts; e++) {
        const uint32_t lo = min(offsets[e], tokens), hi = min(offsets[e + 1], tokens);
        for (uint32_t r = lo; r < hi && n < capacity; r += kGmBN)
            table[n++] = make_uint4(e, r, min((uint32_t)kGmBN, hi - r), 0u);
    }
    *total = n;
}

// ---- activations: f32 [M][K] -> f16 B tiles + the rows' power-of-two factors ------------------------
// grid = padded rows / 8, one warp per row.  Tile (row block rb, chunk c) is 16 KB at
// (rb * nchunks + c) * 16 KB; inside it element (r, k) sits at (k / 8) * 2048 + (r / 8) * 128 +
// (r % 8) * 16 + (k % 8) * 2.  Rows past M and k past K are zeros.  unscale is
// indexed like the tiles' rows.
__global__ void __launch_bounds__(256)
int4_act_tiles_kernel(const float *__restrict__ a, unsigned char *__restrict__ tiles, float *__restrict__ unscale,
                      uint32_t M, uint32_t K, uint32_t nchunks, const GmRows rows)
{
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t r = blockIdx.x * 8 + warp;            // a row of the tiles
    bool live = r < M;
    uint32_t src = r;                                    // the activation row it holds
    if (rows.table) {
        if ((r >> 7) >= *rows.total) return;             // a block nobody multiplies
        const uint4 e = rows.table[r >> 7];
        live = (r & 127u) < e.z;
        src = e.y + (r & 127u);
    }
    const float *row = a + (size_t)(live ? src : 0) * K;
    uint32_t mx = 0;
    if (live) {
        for (uint32_t k = lane * 4; k < K; k += 128) {
            const float4 v = __ldg(reinterpret_cast<const float4 *>(row + k));
            mx = max(max(mx, __float_as_uint(fabsf(v.x))), __float_as_uint(fabsf(v.y)));
            mx = max(max(mx, __float_as_uint(fabsf(v.z))), __float_as_uint(fabsf(v.w)));
        }
    }
    mx = __reduce_max_sync(0xffffffffu, mx);
    const int ea = sx_row_exponent(mx);
    const float pa = __uint_as_float((uint32_t)(127 + 14 - ea) << 23);                 // 2^(14 - E_a)
    if (lane == 0) unscale[r] = live ? __uint_as_float((uint32_t)(127 + ea - 14) << 23) : 0.f;
    const uint32_t rb = r >> 7, rin = r & 127u;
    unsigned char *base = tiles + (size_t)rb * nchunks * kGmBTile + (rin >> 3) * 128u + (rin & 7u) * 16u;
    for (uint32_t kb = lane; kb < nchunks * 8; kb += 32) {
        const uint32_t k = kb * 8;
        float4 v0 = make_float4(0.f, 0.f, 0.f, 0.f), v1 = v0;
        if (live && k < K) v0 = __ldg(reinterpret_cast<const float4 *>(row + k));
        if (live && k + 4 < K) v1 = __ldg(reinterpret_cast<const float4 *>(row + k + 4));
        const __half2 h0 = __floats2half2_rn(v0.x * pa, v0.y * pa), h1 = __floats2half2_rn(v0.z * pa, v0.w * pa);
        const __half2 h2 = __floats2half2_rn(v1.x * pa, v1.y * pa), h3 = __floats2half2_rn(v1.z * pa, v1.w * pa);
        *reinterpret_cast<uint4 *>(base + (size_t)(kb >> 3) * kGmBTile + (kb & 7u) * kGmLbo) =
            make_uint4(*reinterpret_cast<const uint32_t *>(&h0), *reinterpret_cast<const uint32_t *>(&h1),
                       *reinterpret_cast<const uint32_t *>(&h2), *reinterpret_cast<const uint32_t *>(&h3));
    }
}

// one pair of weights: sub = the two codes as f16 subnormals (code 2^-24, or code 2^-20), up = 2^15
// (or 2^11), nz = -z 2^-9 and s9 = s 2^9 of the two rows:  u = code 2^-9 - z 2^-9 (one fused
// multiply-add, rounded relative to code - z),  w = u s 2^9 = (code - z) s
__device__ __forceinline__ uint32_t gm_dequant(uint32_t sub, uint32_t s9, uint32_t nz, __half2 up)
{
    const __half2 u = __hfma2(*reinterpret_cast<const __half2 *>(&sub), up, *reinterpret_cast<const __half2 *>(&nz));
    const __half2 w = __hmul2(u, *reinterpret_cast<const __half2 *>(&s9));
    return *reinterpret_cast<const uint32_t *>(&w);
}

// grid = column tiles x row blocks (row block fastest, so the CTAs that share a weight tile run
// together and it is read from HBM once).  packed: the stream; tiles, unscale: what
// int4_act_tiles_kernel wrote for these rows; ep: where the columns go; M: rows of this pass.
template <int G>
__global__ void __launch_bounds__(kGmThreads)
int4_gemm_kernel(const unsigned char *__restrict__ packed, const unsigned char *__restrict__ tiles,
                 const float *__restrict__ unscale, const SxEpilogue ep, uint32_t M, uint32_t N, uint32_t nchunks,
                 uint32_t header_bytes, uint32_t nrb, const GmRows rows)
{
    extern __shared__ __align__(128) unsigned char gm_raw[];
    constexpr uint32_t kStage = gm_stage_bytes(G);
    constexpr int kGmNS = gm_stages(G);
    constexpr uint32_t kA0 = G * 128;                                 // TMEM: D per group, then the A stages
    constexpr uint32_t kCols = gm_tmem_cols(G);
    static_assert(kA0 + G * kGmNA * 32 <= kCols, "TMEM budget");
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(gm_raw) + 127) & ~(uintptr_t)127);
    unsigned char *ring = smem;
    float *uns = reinterpret_cast<float *>(ring + kGmNS * kStage);   // [128] the rows' factors
    uint32_t *factors = reinterpret_cast<uint32_t *>(uns + kGmBN);  // [8 warps][G][2][32] a chunk's row factors
    uint64_t *full = reinterpret_cast<uint64_t *>(factors + kGmExpanderWarps * G * 64);
    uint64_t *freeb = full + kGmNS;                                  // the MMAs have read the stage's B tile
    uint64_t *a_ready = freeb + kGmNS;
    uint64_t *a_free = a_ready + kGmNA;                              // the MMAs have read the A stage
    uint64_t *done = a_free + kGmNA;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(done + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) GM_STAMP(0);
    const uint32_t groups = N / 128;
    const uint32_t rb = blockIdx.x % nrb, g0 = (blockIdx.x / nrb) * G;
    // the rows this block stands for: row0 .. row0 + nrows - 1 of the activations and of the output
    uint32_t row0 = rb * kGmBN, nrows = M > row0 ? min((uint32_t)kGmBN, M - row0) : 0u;
    if (rows.table) {
        if (rb >= *rows.total) return;                   // the whole CTA: nothing is set up yet
        const uint4 e = rows.table[rb];
        packed += (size_t)e.x * rows.expert_stride;
        row0 = e.y;
        nrows = e.z;
    }
    const uint32_t gcount = min((uint32_t)G, groups - g0);
    const unsigned char *wsrc = packed + header_bytes + (size_t)g0 * nchunks * kSxChunkBytes;
    const size_t group_stride = (size_t)nchunks * kSxChunkBytes;
    const unsigned char *bsrc = tiles + (size_t)rb * nchunks * kGmBTile;
    const uint32_t stage_tx = gcount * kSxChunkBytes + kGmBTile;

    // Issuing a bulk copy costs its thread a few hundred cycles, more than a chunk's MMAs take: every
    // stage has two lanes of the copy warp of its own, one for the weights (it also announces the
    // stage's bytes) and one for the B tile.
    auto issue = [&](uint32_t c, uint32_t st, int role) {
        unsigned char *dst = ring + st * kStage;
        if (role == 0) {
            sx_bar_expect_tx(&full[st], stage_tx);
            for (uint32_t gi = 0; gi < gcount; gi++)
                sx_bulk_load(dst + gi * kSxChunkBytes, wsrc + gi * group_stride + (size_t)c * kSxChunkBytes,
                             kSxChunkBytes, &full[st]);
        } else {
            sx_bulk_load(dst + G * kSxChunkBytes, bsrc + (size_t)c * kGmBTile, kGmBTile, &full[st]);
        }
    };

    if (warp == 9) {
        if (lane == 0) {
            for (int i = 0; i < kGmNS; i++) { sx_bar_init(&full[i], 1); sx_bar_init(&freeb[i], 1); }
            for (int i = 0; i < kGmNA; i++) { sx_bar_init(&a_ready[i], kGmExpanderWarps / 2); sx_bar_init(&a_free[i], 1); }
            sx_bar_init(done, 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncwarp();
        // the first use of every stage: nothing to wait for
        if (lane < 2 * kGmNS && (uint32_t)(lane >> 1) < nchunks) issue((uint32_t)(lane >> 1), (uint32_t)(lane >> 1), lane & 1);
    }
    if (warp == 8) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(sx_smem(tmem_slot)), "r"(kCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid < kGmBN) {
        uns[tid] = (uint32_t)tid < nrows ? __ldg(unscale + rb * kGmBN + (uint32_t)tid) : 0.f;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    if (tid == 0) GM_STAMP(1);

    if (warp == 9) {
        // ---- the copy lanes: the weights of the CTA's groups and the B tile of every chunk
        if (lane < 2 * kGmNS) {
            const uint32_t st = (uint32_t)(lane >> 1);
            uint32_t use = 1;                        // how many times the stage has been filled
            for (uint32_t c = st + kGmNS; c < nchunks; c += kGmNS, use++) {
                long long tt = GM_NOW();
                if (!sx_bar_wait(&freeb[st], (use - 1) & 1)) break;
                if (lane == 0) GM_ADD(16, tt);
                tt = GM_NOW();
                issue(c, st, lane & 1);
                if (lane == 0) GM_ADD(17, tt);
            }
        }
    } else if (warp == 8) {
        // ---- the MMA lane: D[128 columns x 128 rows] += A (tensor memory) B (shared memory)
        if (lane == 0) {
            constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(kGmBN >> 3) << 17) | ((128u >> 4) << 24);
            bool ok = true;
            for (uint32_t c = 0; c < nchunks && ok; c++) {
                const uint32_t st = c % kGmNS, ab = c % kGmNA;
                // the B tile was written by the copy engine (full), A by the dequantisers (a_ready)
                long long tt = GM_NOW();
                ok = sx_bar_wait(&full[st], (c / kGmNS) & 1);
                GM_ADD(8, tt);
                tt = GM_NOW();
                ok = ok && sx_bar_wait(&a_ready[ab], (c / kGmNA) & 1);
                GM_ADD(9, tt);
                if (!ok) break;
                tt = GM_NOW();
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t bbase = sx_smem(ring + st * kStage + G * kSxChunkBytes);
                for (uint32_t gi = 0; gi < gcount; gi++) {
#pragma unroll
                    for (int j = 0; j < 4; j++)
                        sx_mma_ts(tmem + gi * 128, tmem + kA0 + (gi * kGmNA + ab) * 32 + 8 * j,
                                  sx_desc(bbase + j * 2 * kGmLbo, kGmLbo, 128), idesc, (c > 0 || j > 0) ? 1u : 0u);
                }
                sx_commit(&a_free[ab]);              // both arrive once these MMAs have read A and B
                sx_commit(&freeb[st]);
                GM_ADD(10, tt);
            }
            if (ok) sx_commit(done);
            GM_STAMP(3);
        }
    } else {
        // ---- dequantisers: warps 0-3 take the even chunks, warps 4-7 the odd ones; a thread turns
        //      the 64 weight rows of column 32 (w%4) + lane of every group into f16 and stores them
        //      into the chunk's A stage in tensor memory (two independent halves of 32 rows: their
        //      load and arithmetic latencies overlap)
        const int h = warp >> 2;
        const uint32_t tcol = (uint32_t)((warp & 3) * 32 + lane);
        const uint32_t tlane = ((uint32_t)((warp & 3) * 32)) << 16;
        uint32_t *wscr = factors + warp * (G * 64);
        float es[G];
#pragma unroll
        for (int gi = 0; gi < G; gi++)
            es[gi] = (uint32_t)gi < gcount ? __ldg(reinterpret_cast<const float *>(packed) + g0 + gi) : 1.f;
        const __half2 up0 = __float2half2_rn(32768.f), up1 = __float2half2_rn(2048.f);
        const __half2 zd = __float2half2_rn((lane & 1) ? -0.0001220703125f : -0.001953125f);
        const __half2 su = __float2half2_rn((lane & 1) ? 8192.f : 512.f);
        bool alive = true;
        for (uint32_t c = (uint32_t)h; c < nchunks && alive; c += 2) {
            const uint32_t st = c % kGmNS, ab = c % kGmNA;
            long long tt = GM_NOW();
            if (!sx_bar_wait(&full[st], (c / kGmNS) & 1)) alive = false;
            if (tid == 0) GM_ADD(24, tt);
            tt = GM_NOW();
            if (alive && c >= (uint32_t)kGmNA && !sx_bar_wait(&a_free[ab], ((c / kGmNA) - 1) & 1)) alive = false;
            if (tid == 0) GM_ADD(25, tt);
            tt = GM_NOW();
            if (!__all_sync(0xffffffffu, alive)) { alive = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const unsigned char *stage = ring + st * kStage;
            // The factors of the chunk's 64 weight rows depend on k only: the warp prepares them once,
            // a pair of rows per lane (s 2^9 and -z 2^-9; 2^13 and -2^-13 in the pairs whose nibble
            // sits four bits up), and notes which rows are constants (scale 0).
            uint32_t mlo[G], mhi[G];
#pragma unroll
            for (int gi = 0; gi < G; gi++) {
                const unsigned char *sp = stage + gi * kSxChunkBytes + kSxCodeBytes;
                const uint32_t s2 = reinterpret_cast<const uint32_t *>(sp)[lane];
                const uint32_t z2 = reinterpret_cast<const uint32_t *>(sp + 128)[lane];
                const __half2 sv = __hmul2(*reinterpret_cast<const __half2 *>(&s2), su);
                const __half2 zv = __hmul2(*reinterpret_cast<const __half2 *>(&z2), zd);
                wscr[gi * 64 + lane] = *reinterpret_cast<const uint32_t *>(&sv);
                wscr[gi * 64 + 32 + lane] = *reinterpret_cast<const uint32_t *>(&zv);
                mlo[gi] = __ballot_sync(0xffffffffu, (s2 & 0x7fffu) == 0u);
                mhi[gi] = __ballot_sync(0xffffffffu, (s2 & 0x7fff0000u) == 0u);
            }
            __syncwarp();
#pragma unroll
            for (int gi = 0; gi < G; gi++) {
                if ((uint32_t)gi < gcount) {
                    const unsigned char *gs = stage + gi * kSxChunkBytes;
#pragma unroll
                    for (int hh = 0; hh < 2; hh++) {
                        const uint4 cw = *reinterpret_cast<const uint4 *>(gs + ((uint32_t)hh * 128u + tcol) * 16u);
                        uint32_t r[16];
                        const uint32_t w4[4] = {cw.x, cw.y, cw.z, cw.w};
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const uint4 s4 = *reinterpret_cast<const uint4 *>(wscr + gi * 64 + hh * 16 + 4 * i);
                            const uint4 z4 = *reinterpret_cast<const uint4 *>(wscr + gi * 64 + 32 + hh * 16 + 4 * i);
                            const uint32_t w = w4[i], w8 = w >> 8;
                            r[4 * i + 0] = gm_dequant(w & 0x000F000Fu, s4.x, z4.x, up0);
                            r[4 * i + 1] = gm_dequant(w & 0x00F000F0u, s4.y, z4.y, up1);
                            r[4 * i + 2] = gm_dequant(w8 & 0x000F000Fu, s4.z, z4.z, up0);
                            r[4 * i + 3] = gm_dequant(w8 & 0x00F000F0u, s4.w, z4.w, up1);
                        }
                        const uint32_t lo = (mlo[gi] >> (16 * hh)) & 0xffffu, hi = (mhi[gi] >> (16 * hh)) & 0xffffu;
                        if (lo | hi) {
                            // constant rows: the weight is z whatever the code (the stream keeps z as it is)
                            const float inv = 1.f / es[gi];
                            const __half *zp = reinterpret_cast<const __half *>(gs + kSxCodeBytes + 128) + hh * 32;
#pragma unroll
                            for (int pr = 0; pr < 16; pr++) {
                                if ((lo >> pr) & 1u)
                                    r[pr] = (r[pr] & 0xffff0000u) |
                                            (uint32_t)__half_as_ushort(__float2half_rn(__half2float(zp[2 * pr]) * inv));
                                if ((hi >> pr) & 1u)
                                    r[pr] = (r[pr] & 0x0000ffffu) |
                                            ((uint32_t)__half_as_ushort(__float2half_rn(__half2float(zp[2 * pr + 1]) * inv)) << 16);
                            }
                        }
                        sx_tmem_st16(tmem + tlane + kA0 + (gi * kGmNA + ab) * 32 + (uint32_t)hh * 16u, r);
                    }
                }
            }
            if (tid == 0) GM_ADD(26, tt);
            tt = GM_NOW();
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            if (tid == 0) GM_ADD(27, tt);
            tt = GM_NOW();
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();                            // (also: the warp's factors may be overwritten now)
            if (lane == 0) sx_bar_arrive(&a_ready[ab]);
            if (tid == 0) GM_ADD(28, tt);
        }
        if (tid == 0) GM_STAMP(2);
        // ---- the accumulators: lane = column, TMEM column = activation row of the block
        bool ok = alive && sx_bar_wait(done, 0);
        ok = __all_sync(0xffffffffu, ok);
        if (tid == 0) GM_STAMP(4);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            if (G == 2 && ep.swiglu) {
                // the tile is a (gate, up) pair: out[m][tile * 128 + t] = gate / (1 + exp(-gate)) * up
                // (internal/kernels/elementwise.go:85)
                const uint32_t tile = blockIdx.x / nrb;
#pragma unroll 1
                for (int q = 0; q < 4; q++) {
                    const uint32_t col0 = (uint32_t)h * 64u + (uint32_t)q * 16u;
                    uint32_t rg[16], ru[16];
                    sx_tmem_ld16(tmem + tlane + col0, rg);
                    sx_tmem_ld16(tmem + tlane + 128 + col0, ru);
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const uint32_t m = row0 + col0 + j;
                        if (col0 + j < nrows) {
                            const float f = uns[col0 + j];
                            const float gate = __uint_as_float(rg[j]) * (f * es[0]);
                            const float upv = __uint_as_float(ru[j]) * (f * es[G - 1]);
                            ep.out0[(size_t)m * ep.ld0 + (size_t)tile * 128 + tcol] =
                                __fdiv_rn(gate, 1.f + expf(-gate)) * upv;
                        }
                    }
                }
            } else {
#pragma unroll
                for (int gi = 0; gi < G; gi++) {
                    if ((uint32_t)gi < gcount) {
#pragma unroll 1
                        for (int q = 0; q < 4; q++) {
                            const uint32_t col0 = (uint32_t)h * 64u + (uint32_t)q * 16u;
                            uint32_t r[16];
                            sx_tmem_ld16(tmem + tlane + gi * 128 + col0, r);
#pragma unroll
                            for (int j = 0; j < 16; j++) {
                                const uint32_t m = row0 + col0 + j;
                                if (col0 + j < nrows)
                                    sx_store(ep, m, g0 + gi, tcol, __uint_as_float(r[j]) * (uns[col0 + j] * es[gi]));
                            }
                        }
                    }
                }
            }
        }
    }
    if (tid == 0) GM_STAMP(5);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 8)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kCols) : "memory");
}

// ---- host side --------------------------------------------------------------------------------------
size_t int4_gemm_workspace(uint32_t M, uint32_t K)
{
    const uint32_t rows = M < kGmPassRows ? (M + kGmBN - 1) / kGmBN * kGmBN : kGmPassRows;
    const size_t nchunks = (K + kSxChunkK - 1) / kSxChunkK;
    return align_up((size_t)rows * 4, 256) + (size_t)(rows / kGmBN) * nchunks * kGmBTile;
}

template <int G> static int gm_prepare()
{
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        int rc = check_cuda(cudaFuncSetAttribute(int4_gemm_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)gm_smem_bytes(G)), "int4_gemm_kernel shared memory");
        if (rc) return rc;
        rc = check_cuda(cudaFuncSetAttribute(int4_gemm_kernel<G>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                             (int)cudaSharedmemCarveoutMaxShared), "int4_gemm_kernel carve-out");
        if (rc) return rc;
        attr_set[dev] = true;
    }
    return AB_OK;
}

// One group per CTA, two CTAs per SM, measured faster than two groups per CTA (one CTA per SM,
// half the B-tile traffic, but a single lane issuing every MMA): 4096 x 11008 at 2048 rows 237 us
// against 262 us, at 512 rows 91 us against 105 us.  The SwiGLU epilogue needs the (gate, up) pair
// of groups in one CTA.
static int gm_groups_per_cta(uint32_t M, uint32_t N, bool swiglu)
{
    (void)M; (void)N;
#ifdef GM_TRACE
    if (getenv("GM_G")) return atoi(getenv("GM_G"));
#endif
    return swiglu ? 2 : 1;
}

// The product in passes of at most kGmPassRows activation rows.  mode and the destinations are
// those of the decode kernel's launcher (plain, three column ranges, SwiGLU over (gate, up) pairs).
int run_int4_gemm_mode(cudaStream_t stream, const float *a, const unsigned char *packed, int mode, float *out0,
                       float *out1, float *out2, uint32_t n1, uint32_t n2, uint32_t M, uint32_t N, uint32_t K,
                       uint32_t ld0, void *scratch)
{
    if (!scratch) return fail(AB_ERR_INVALID, "the prepacked int4 product of %u rows needs %zu bytes of scratch", M,
                              int4_gemm_workspace(M, K));
    const uint32_t nchunks = (K + kSxChunkK - 1) / kSxChunkK, groups = N / 128;
    const uint32_t hb = (uint32_t)sx_header_bytes(N);
    const bool swiglu = mode == 2;
    const int G = gm_groups_per_cta(M, N, swiglu);
    int rc = G == 2 ? gm_prepare<2>() : gm_prepare<1>();
    if (rc) return rc;
    const uint32_t pass_rows = M < kGmPassRows ? (M + kGmBN - 1) / kGmBN * kGmBN : kGmPassRows;
    float *unscale = static_cast<float *>(scratch);
    unsigned char *tiles = static_cast<unsigned char *>(scratch) + align_up((size_t)pass_rows * 4, 256);
    for (uint32_t m0 = 0; m0 < M; m0 += kGmPassRows) {
        const uint32_t rows = M - m0 < kGmPassRows ? M - m0 : kGmPassRows;
        const uint32_t nrb = (rows + kGmBN - 1) / kGmBN;
        int4_act_tiles_kernel<<<nrb * (kGmBN / 8), 256, 0, stream>>>(a + (size_t)m0 * K, tiles, unscale, rows, K, nchunks,
                                                                     GmRows{nullptr, nullptr, 0ull});
        count_launch();
        SxEpilogue ep{};
        ep.g1 = ep.g2 = 0xffffffffu;
        ep.ld0 = ld0;
        ep.out0 = out0 + (size_t)m0 * ld0;
        if (mode == 1) {
            ep.g1 = n1 / 128; ep.g2 = n2 / 128;
            ep.ld0 = n1; ep.ld1 = n2 - n1; ep.ld2 = N - n2;
            ep.out0 = out0 + (size_t)m0 * ep.ld0;
            ep.out1 = out1 + (size_t)m0 * ep.ld1;
            ep.out2 = out2 + (size_t)m0 * ep.ld2;
        }
        ep.swiglu = swiglu ? 1u : 0u;
        const uint32_t ctas = ((groups + G - 1) / G) * nrb;
        if (G == 2)
            int4_gemm_kernel<2><<<ctas, kGmThreads, gm_smem_bytes(2), stream>>>(packed, tiles, unscale, ep, rows, N,
                                                                                 nchunks, hb, nrb, GmRows{nullptr, nullptr, 0ull});
        else
            int4_gemm_kernel<1><<<ctas, kGmThreads, gm_smem_bytes(1), stream>>>(packed, tiles, unscale, ep, rows, N,
                                                                                 nchunks, hb, nrb, GmRows{nullptr, nullptr, 0ull});
        count_launch();
        rc = check_cuda(cudaGetLastError(), "int4_gemm_kernel");
        if (rc) return rc;
    }
    note_selection("int4 tile kernel on tcgen05 (weights dequantised to f16 into tensor memory as the A operand, "
                   "activation tiles by bulk copies, M=128 x N=128 x K=16 MMAs, TMEM f32 accumulators), %u column "
                   "tiles of %d groups x %u row blocks of 128, %u chunks of 64 weight rows", (groups + G - 1) / G, G,
                   (M + kGmBN - 1) / kGmBN, nchunks);
    return AB_OK;
}

// ---- grouped product: rows sorted by expert, one prepacked [K, N] matrix per expert --------------------
static uint32_t gm_group_blocks(uint32_t experts, uint32_t tokens) { return (tokens + kGmBN - 1) / kGmBN + experts; }

size_t int4_gemm_grouped_workspace(uint32_t experts, uint32_t tokens, uint32_t K)
{
    const size_t nb = gm_group_blocks(experts, tokens), nchunks = (K + kSxChunkK - 1) / kSxChunkK;
    return align_up(nb * sizeof(uint4), 256) + 256 + align_up(nb * kGmBN * 4, 256) + nb * nchunks * kGmBTile;
}

int run_int4_gemm_grouped(cudaStream_t stream, const float *x, const unsigned char *packed, const uint32_t *offsets,
                          float *out, uint32_t experts, uint32_t tokens, uint32_t N, uint32_t K, void *scratch)
{
    if (tokens == 0 || experts == 0) return AB_OK;
    if (!scratch) return fail(AB_ERR_INVALID, "the grouped prepacked int4 product needs %zu bytes of scratch",
                              int4_gemm_grouped_workspace(experts, tokens, K));
    int rc = gm_prepare<1>();
    if (rc) return rc;
    const uint32_t nb = gm_group_blocks(experts, tokens), nchunks = (K + kSxChunkK - 1) / kSxChunkK, groups = N / 128;
    unsigned char *ws = static_cast<unsigned char *>(scratch);
    uint4 *table = reinterpret_cast<uint4 *>(ws);
    ws += align_up((size_t)nb * sizeof(uint4), 256);
    uint32_t *total = reinterpret_cast<uint32_t *>(ws);
    ws += 256;
    float *unscale = reinterpret_cast<float *>(ws);
    ws += align_up((size_t)nb * kGmBN * 4, 256);
    unsigned char *tiles = ws;
    const GmRows rows{table, total, (unsigned long long)int4_stream_packed_bytes(N, K)};
    gm_group_plan_kernel<<<1, 32, 0, stream>>>(offsets, experts, tokens, table, total, nb);
    count_launch();
    int4_act_tiles_kernel<<<nb * (kGmBN / 8), 256, 0, stream>>>(x, tiles, unscale, tokens, K, nchunks, rows);
    count_launch();
    SxEpilogue ep{};
    ep.g1 = ep.g2 = 0xffffffffu;
    ep.ld0 = N;
    ep.out0 = out;
    int4_gemm_kernel<1><<<groups * nb, kGmThreads, gm_smem_bytes(1), stream>>>(packed, tiles, unscale, ep, tokens, N, nchunks,
                                                                             (uint32_t)sx_header_bytes(N), nb, rows);
    count_launch();
    rc = check_cuda(cudaGetLastError(), "int4_gemm_kernel (grouped)");
    if (rc) return rc;
    note_selection("grouped int4 tile kernel on tcgen05 (every expert's segment in blocks of 128 rows of its own, "
                   "weights dequantised into tensor memory, M=128 x N=128 x K=16 MMAs), %u experts, %u rows, up to "
                   "%u row blocks x %u column groups", experts, tokens, nb, groups);
    return AB_OK;
}

// x f32[T*K], packed (Experts matrices, each ab_int4_prepack_bytes(K, N) bytes, end to end), offsets
// u32[E+1], out f32[T*N]; GroupedTiledDims{Experts,Tokens,K,N}
int launch_grouped_matmul_int4_packed(Launch &l)
{
    const char *name = "GroupedMatMulInt4Packed";
    const uint32_t E = u32_at(l.u, 0), T = u32_at(l.u, 4), K = u32_at(l.u, 8), N = u32_at(l.u, 12);
    if (E == 0 || N == 0 || N % 128 || K == 0 || K % 4)
        return fail(AB_ERR_INVALID, "%s: Experts=%u Tokens=%u K=%u N=%u; N is a multiple of 128 and K of 4", name, E, T, K, N);
    const size_t ws = T ? int4_gemm_grouped_workspace(E, T, K) : 0;
    if (l.query_ws) { l.ws_need = ws; return AB_OK; }
    const size_t per = int4_stream_packed_bytes(N, K);
    if (l.len[0] < (uint64_t)T * K || (uint64_t)l.len[1] * 4 < (uint64_t)E * per || l.len[2] < E + 1 ||
        l.len[3] < (uint64_t)T * N)
        return fail(AB_ERR_INVALID, "%s: Experts=%u Tokens=%u K=%u N=%u needs x[%llu] packed[%llu bytes] offsets[%u] "
                    "out[%llu]; the lengths block says %u, %u words, %u, %u", name, E, T, K, N, (unsigned long long)T * K,
                    (unsigned long long)E * per, E + 1, (unsigned long long)T * N, l.len[0], l.len[1], l.len[2], l.len[3]);
    if (ws > l.ws_bytes || (ws && !l.ws))
        return fail(AB_ERR_INVALID, "%s: needs %zu bytes of workspace, given %zu", name, ws, l.ws_bytes);
    return run_int4_gemm_grouped(l.stream, ptr<const float>(l, 0), ptr<const unsigned char>(l, 1), ptr<const uint32_t>(l, 2),
                                 ptr<float>(l, 3), E, T, N, K, l.ws);
}

int int4_gemm_error_flag()
{
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_sm100_error, sizeof v) != cudaSuccess) { cudaGetLastError(); return -1; }
    return v;
}

}  // namespace ab
