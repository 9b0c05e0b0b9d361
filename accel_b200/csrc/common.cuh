// Shared declarations of the sm_100a kernels and their launchers.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "../../include/accel_b200.h"

namespace ab {

// One dispatch: the reference's argument convention (binding pointers, a lengths block with one
// element count per binding, the std140 uniform block) plus scratch memory.
struct Launch {
    cudaStream_t stream;
    void *const *b;
    const uint32_t *len;
    int nb;
    const uint8_t *u;
    size_t ubytes;
    void *ws;
    size_t ws_bytes;
    bool query_ws;      // true: only compute *ws_need, launch nothing, b may be NULL
    size_t ws_need;
};

typedef int (*launch_fn)(Launch &);

struct KernelEntry {
    const char *name;
    int n_bindings;
    size_t uniform_bytes;   // 0 = the kernel takes no uniform block
    launch_fn fn;
};

int fail(int code, const char *fmt, ...);          // records the thread's last error
void note_selection(const char *fmt, ...);         // records which variant a launch selected
int check_cuda(cudaError_t e, const char *what);   // maps a CUDA error to an ab_status
int sm_count();                                    // SMs of the current device (cached)
void count_launch();                               // one more kernel launch issued by this library

// Programmatic dependent launch.  A kernel launched through launch_dependent may begin while the
// kernel before it in the stream is still running; it must call pdl_enter() (or pdl_wait()) before
// it reads or writes anything that kernel touches.  pdl_trigger() lets the kernel AFTER this one
// begin: at the top of a kernel that fits the device at once, at the end of one that runs in
// several waves (an early dependent would only hold resources the remaining waves need).
// Both instructions do nothing in a kernel launched the ordinary way.  launch_dependent sets the
// attribute only when pdl_enabled() (AB_PDL=1); the int4 products decide for themselves.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_enter() { pdl_trigger(); pdl_wait(); }
#endif
bool pdl_enabled();

template <typename... P, typename... A>
inline cudaError_t launch_dependent(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, A &&...args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<P>(args)...);
}

inline uint32_t u32_at(const uint8_t *u, size_t off) { uint32_t v; memcpy(&v, u + off, 4); return v; }
inline float f32_at(const uint8_t *u, size_t off) { float v; memcpy(&v, u + off, 4); return v; }

template <typename T> inline T *ptr(const Launch &l, int i) { return reinterpret_cast<T *>(l.b[i]); }

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// The f16-operand int4 kernels round a * s to f16.  An exact power of two per activation row, taken
// from the row's largest magnitude and undone in the f32 epilogue, keeps that product a normal f16
// whatever the magnitude of the activations (the reference's f32 arithmetic is scale-invariant).
// floor(log2(largest magnitude)), clamped; 0 for an all-zero row.  Bit patterns of non-negative
// floats order like the floats; Inf and NaN clamp to the top.
__host__ __device__ inline int ab_row_exponent(uint32_t amax_bits)
{
    int ea = amax_bits ? (int)((amax_bits >> 23) & 0xffu) - 127 : 0;
    return ea < -80 ? -80 : (ea > 80 ? 80 : ea);
}
#ifdef __CUDACC__
__device__ __forceinline__ float ab_pow2(int e) { return __uint_as_float((uint32_t)(127 + e) << 23); }
#endif
// the largest magnitude of each of M rows of K floats -> amax[M] (int4_stream.cu)
int run_row_absmax(cudaStream_t stream, const float *a, float *amax, uint32_t M, uint32_t K, bool dependent);

// the tensor-core int4 kernel for small batches (int4_mma.cu), driven by the int4 launcher
struct Int4MmaPlan { bool ok; uint32_t groups, splits, kc; size_t ws; };
Int4MmaPlan plan_int4_mma(uint32_t M, uint32_t N, uint32_t K);
int run_int4_mma(const Launch &l, const Int4MmaPlan &p, float *dst, uint32_t M, uint32_t N, uint32_t K);

// the one-row streaming int4 kernel, K splits summed inside a cluster (int4_gemv.cu)
struct Int4RowPlan { bool ok; int W; uint32_t tiles, splits, kc; size_t ws; };   // W groups per column tile
Int4RowPlan plan_int4_row(uint32_t N, uint32_t K);
int run_int4_row(const Launch &l, const Int4RowPlan &p, float *out, uint32_t N, uint32_t K);

// the decode-batch int4 kernel: 16 rows per pass, K splits summed inside a cluster (int4_batch.cu)
struct Int4BatchPlan { bool ok; int G; uint32_t tiles, splits, kc; };    // G groups per column tile
Int4BatchPlan plan_int4_batch(uint32_t M, uint32_t N, uint32_t K);
size_t int4_batch_workspace(uint32_t M);      // the rows' largest magnitudes
int run_int4_batch(const Launch &l, const Int4BatchPlan &p, float *out, uint32_t M, uint32_t N, uint32_t K);


// the 128 x 128 warp-MMA tile kernel of the grouped product, as a plain int4 product (grouped.cu)
bool int4_tiles_ok(uint32_t N, uint32_t K);
size_t int4_tiles_workspace(uint32_t M);
int run_int4_tiles(const Launch &l, float *out, uint32_t M, uint32_t N, uint32_t K);


// the decode-batch int4 kernel over prepacked weights: bulk copies, tensor memory, tcgen05 (int4_stream.cu)
bool int4_stream_ok(uint32_t M, uint32_t N, uint32_t K);
size_t int4_stream_packed_bytes(uint32_t N, uint32_t K);
int run_int4_prepack(cudaStream_t stream, const uint32_t *codes, const uint16_t *scales, const uint16_t *zeros,
                     unsigned char *packed, uint32_t N, uint32_t K);
size_t int4_stream_workspace(uint32_t M);
int run_int4_stream(cudaStream_t stream, const float *a, const float *amax, const unsigned char *packed, float *out,
                    uint32_t M, uint32_t N, uint32_t K, uint32_t ldo, void *scratch, bool dependent,
                    uint32_t amax_parts = 1);       // amax: [M][amax_parts], a row's maximum is the largest entry
int int4_stream_error_flag();
// the batch int4 kernel over the same prepacked weights: 128-row tiles on tcgen05 (int4_gemm.cu);
// mode 0 plain, 1 three column ranges, 2 SwiGLU over (gate, up) pairs of groups
size_t int4_gemm_workspace(uint32_t M, uint32_t K);
int run_int4_gemm_mode(cudaStream_t stream, const float *a, const unsigned char *packed, int mode, float *out0,
                       float *out1, float *out2, uint32_t n1, uint32_t n2, uint32_t M, uint32_t N, uint32_t K,
                       uint32_t ld0, void *scratch);
int int4_gemm_error_flag();
int launch_grouped_matmul_int4_packed(Launch &);
int launch_quant_matvec_int4_packed(Launch &);
int launch_quant_matmul_int4_packed(Launch &);
int launch_quant_matmul_int4_packed_split3(Launch &);
int launch_quant_matmul_int4_packed_swiglu(Launch &);
int launch_quant_matmul_int4_packed_a(Launch &);
int launch_quant_matmul_int4_packed_split3_a(Launch &);
int launch_quant_matmul_int4_packed_swiglu_a(Launch &);
int launch_quant_matmul_int4_packed_swiglu_a_max(Launch &);
int launch_add_rmsnorm_amax(Launch &);

// launchers, one per reference kernel name (defined beside their kernels)
int launch_quant_matvec_int4(Launch &);
int launch_quant_matvec_f32(Launch &);
int launch_quant_matmul_tiled_f32(Launch &);
int launch_quant_matmul_int4(Launch &);
int launch_attention_decode(Launch &);
int launch_attention_decode_f16(Launch &);
int launch_attention_decode_paged(Launch &);
int launch_attention_decode_paged_f16(Launch &);
int launch_attention_decode_batched(Launch &);
int launch_attention_decode_batched_f16(Launch &);
int launch_attention_decode_batched_max(Launch &);
int launch_attention_decode_batched_f16_max(Launch &);
int launch_attention_ragged(Launch &);
int launch_attention_ragged_f16(Launch &);
int launch_attention_prefill(Launch &);
int launch_attention_prefill_f16(Launch &);
int launch_attention_prefill_paged(Launch &);
int launch_attention_prefill_paged_f16(Launch &);
int launch_grouped_matvec(Launch &);
int launch_grouped_matmul(Launch &);
int launch_grouped_matmul_int4(Launch &);
int launch_segment_offsets(Launch &);
int launch_scatter_rows(Launch &);
int launch_scatter_rows_f16(Launch &);
int launch_gather_rows(Launch &);
int launch_gather_rows_f16(Launch &);
int launch_rmsnorm(Launch &);
int launch_rope(Launch &);
int launch_swiglu(Launch &);
int launch_elem_add(Launch &);
int launch_sample_argmax(Launch &);
int launch_cast_f32_to_f16(Launch &);
int launch_cast_f16_to_f32(Launch &);
int launch_softmax(Launch &);
int launch_scale_rows(Launch &);
int launch_logit_bias(Launch &);
int launch_topk_mask_rows(Launch &);
int launch_topp_mask_rows(Launch &);
int launch_topk_mask(Launch &);
int launch_topp_mask(Launch &);
int launch_sample_rows(Launch &);
int launch_sample_categorical(Launch &);
int launch_penalty_clear_rows(Launch &);
int launch_penalty_count_rows(Launch &);
int launch_penalty_apply_rows(Launch &);
int launch_penalty_clear(Launch &);
int launch_penalty_count(Launch &);
int launch_penalty_apply(Launch &);
int launch_int4_quantize(Launch &);
int launch_decode_step_inputs(Launch &);
int launch_argmax_shard(Launch &);
int launch_argmax_merge(Launch &);
int launch_add_rmsnorm(Launch &);
int launch_rope_scatter_qkv(Launch &);
int launch_rope_scatter_qkv_f16(Launch &);

// f32 -> f16 with the reference's rule: round to nearest even, except that every magnitude below
// 2^-24 becomes a signed zero (internal/kernel/narrow.go:82-83); IEEE rounds (2^-25, 2^-24) up.
__host__ __device__ inline uint16_t f32_to_f16_ref(float x)
{
    uint32_t b;
#ifdef __CUDA_ARCH__
    b = __float_as_uint(x);
#else
    memcpy(&b, &x, 4);
#endif
    uint16_t sign = (uint16_t)((b >> 16) & 0x8000u);
    int32_t exp = (int32_t)((b >> 23) & 0xffu) - 127;
    uint32_t mant = b & 0x7fffffu;
    if ((b & 0x7fffffffu) > 0x7f800000u) return 0x7e00;
    if (exp >= 16) return (uint16_t)(sign | 0x7c00u);
    if (exp < -24) return sign;
    uint32_t shift, base;
    if (exp < -14) { mant |= 0x800000u; shift = 13u + (uint32_t)(-exp - 14); base = 0; }
    else { shift = 13u; base = (uint32_t)(exp + 15) << 10; }
    uint32_t q = mant >> shift, rem = mant & ((1u << shift) - 1u), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) q++;
    return (uint16_t)(sign | (uint16_t)(base + q));
}

__host__ __device__ inline float f16_bits_to_f32(uint16_t h)
{
#ifdef __CUDA_ARCH__
    return __half2float(__ushort_as_half(h));
#else
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16, exp = ((uint32_t)h >> 10) & 0x1fu,
             mant = (uint32_t)h & 0x3ffu, out;
    if (exp == 0) {
        if (mant == 0) out = sign;
        else {
            uint32_t shift = 0;
            while ((mant & 0x400u) == 0) { mant <<= 1; shift++; }
            out = sign | ((127 - 15 + 1 - shift) << 23) | ((mant & 0x3ffu) << 13);
        }
    } else if (exp == 0x1f) out = sign | 0x7f800000u | (mant << 13);
    else out = sign | ((exp + 127 - 15) << 23) | (mant << 13);
    float f;
    memcpy(&f, &out, 4);
    return f;
#endif
}

}  // namespace ab
