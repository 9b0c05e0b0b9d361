// Device-side pieces shared by the kernels that drive Blackwell's asynchronous units by hand:
// mbarriers with bounded waits, bulk asynchronous copies, tensor memory and tcgen05.mma with the A
// operand in tensor memory; and the layout constants of the prepacked int4 stream those kernels read.
#pragma once
#include <cuda_fp16.h>

#include "common.cuh"

namespace ab {

// ---- the prepacked stream (written by ab_int4_prepack): a header of one float per 128-column group,
// then per group and per chunk of 64 weight rows 4352 contiguous bytes (codes, 64 scales, 64 zeros)
static constexpr uint32_t kSxChunkK = 64;
static constexpr uint32_t kSxCodeBytes = 4096;
static constexpr uint32_t kSxChunkBytes = 4352;
static inline size_t sx_header_bytes(uint32_t N) { return align_up((size_t)(N / 128) * 4, 256); }

static constexpr long long kSxWaitCycles = 1ll << 31;      // about a second

// nonzero: a bounded wait ran out (one copy per translation unit that includes this header)
static __device__ int g_sm100_error;

__device__ __forceinline__ uint32_t sx_smem(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void sx_bar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(sx_smem(bar)), "r"(count));
}
__device__ __forceinline__ void sx_bar_arrive(uint64_t *bar)
{
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(sx_smem(bar)) : "memory");
}
__device__ __forceinline__ void sx_bar_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}"
                 ::"r"(sx_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t sx_bar_try(uint32_t addr, uint32_t parity)
{
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    return done;
}
// Bounded wait for the phase of the given parity; false (and the error flag) when it runs out.
static __device__ __noinline__ bool sx_bar_wait_slow(uint32_t addr, uint32_t parity)
{
    const long long t0 = clock64();
    for (;;) {
        if (sx_bar_try(addr, parity)) return true;
        if (clock64() - t0 > kSxWaitCycles) break;
    }
    atomicExch(&g_sm100_error, 1);
    return false;
}
__device__ __forceinline__ bool sx_bar_wait(uint64_t *bar, uint32_t parity)
{
    const uint32_t addr = sx_smem(bar);
    if (sx_bar_try(addr, parity)) return true;
    if (sx_bar_try(addr, parity)) return true;
    return sx_bar_wait_slow(addr, parity);
}
__device__ __forceinline__ void sx_bulk_load(void *dst, const void *src, uint32_t bytes, uint64_t *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(sx_smem(dst)), "l"(src), "r"(bytes), "r"(sx_smem(bar)) : "memory");
}
__device__ __forceinline__ uint64_t sx_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo)
{   // K-major, no swizzle: start address, K-direction and MN-direction core-matrix strides, all >> 4
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) |
           ((uint64_t)(sbo >> 4) << 32) | (1ull << 46);
}
// D[tmem_d] (+)= A[tmem_a] * B[smem]: the A operand is read from tensor memory
__device__ __forceinline__ void sx_mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void sx_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(sx_smem(bar)) : "memory");
}
__device__ __forceinline__ void sx_tmem_st16(uint32_t taddr, const uint32_t (&r)[16])
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
                   "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
                   "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void sx_tmem_ld16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]),
                   "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
                   "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// The exponent that scales a row: floor(log2(largest magnitude)), clamped; 0 for an all-zero row.
// Bit patterns of non-negative floats order like the floats; Inf and NaN clamp to the top.
__device__ __forceinline__ int sx_row_exponent(uint32_t amax_bits) { return ab_row_exponent(amax_bits); }

// Where the columns go.  Plain: out[m][ld0 .. ].  Split: the columns from group g1 on go to out1 and
// those from group g2 on to out2, each a contiguous matrix of its own (the fused q | k | v product).
// SwiGLU: tiles are (gate, up) pairs of groups and out[m][tile * 128 + t] = gate / (1 + exp(-gate)) * up
// (internal/kernels/elementwise.go:85), the arithmetic of the SwiGLU kernel on the two sums.
struct SxEpilogue {
    float *out0, *out1, *out2;
    uint32_t g1, g2;              // 0xffffffff: no such destination
    uint32_t ld0, ld1, ld2;
    uint32_t swiglu;
    // row maxima in parts: the producer of a matrix leaves, per row, the largest magnitude of each
    // part it wrote (a head, a warp's columns), and the product that reads the matrix takes a row's
    // maximum as the largest of its entries
    uint32_t amax_parts;          // entries per row of the amax binding (1: one maximum per row)
    float *max_out;               // SwiGLU form: [M][max_ld], entry 4 * tile + warp = the largest |out| of the
    uint32_t max_ld;              // 32 columns that warp wrote; NULL: not wanted
};

__device__ __forceinline__ void sx_store(const SxEpilogue &e, uint32_t m, uint32_t g, uint32_t t, float v)
{
    float *base = e.out0;
    uint32_t ld = e.ld0, gb = 0;
    if (g >= e.g2) { base = e.out2; ld = e.ld2; gb = e.g2; }
    else if (g >= e.g1) { base = e.out1; ld = e.ld1; gb = e.g1; }
    base[(size_t)m * ld + (size_t)(g - gb) * 128 + t] = v;
}

}  // namespace ab
