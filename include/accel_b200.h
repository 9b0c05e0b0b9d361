/*
 * accel_b200.h -- C ABI of libaccelb200.so, a Blackwell (sm_100a) backend for the quantized decode
 * path of golang-design/accel.
 *
 * The entry points are what accel's cgo-free FFI would bind to put a CUDA backend behind
 * `internal/driver` (the seam between accel's device layer and a backend): integer and pointer
 * arguments only, at most 15 of them, no float passed by value, no callback, no exception or abort
 * across the boundary.  Every function returns 0 or a negative ab_status unless stated otherwise;
 * ab_last_error() gives the thread's last message.
 *
 * Reference citations (file:line) are paths inside the accel module.
 */
#ifndef ACCEL_B200_H
#define ACCEL_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AB_API __attribute__((visibility("default")))

typedef enum ab_status {
    AB_OK = 0,
    AB_ERR_INVALID = -1,      /* an argument the call can check is wrong; nothing was launched   */
    AB_ERR_UNSUPPORTED = -2,  /* no sm_100a kernel under that name: a pipeline-creation error,   */
                              /* never a silent CPU run (pipeline.go:115-119)                    */
    AB_ERR_OOM = -3,          /* allocation failed; the device is NOT lost                       */
    AB_ERR_DEVICE_LOST = -4,  /* sticky: driver.ErrDeviceLost (internal/driver/plan.go:385-391)  */
    AB_ERR_BUSY = -5,         /* a submission of this executable is still in flight              */
    AB_ERR_CUDA = -6,         /* a CUDA call failed for a reason that is not loss                */
    AB_ERR_NO_DEVICE = -7,    /* no CUDA device or driver                                        */
    AB_ERR_TIMEOUT = -8       /* a bounded device-side wait for a peer ran out; nothing is lost   */
} ab_status;

AB_API const char *ab_error_string(int code);
AB_API const char *ab_last_error(void);              /* thread-local, valid until the next call */

/* ------------------------------------------------------------------------------------------ */
/* Adapter and device: driver.Adapter / driver.Device (internal/driver/driver.go:149-190)      */
/* ------------------------------------------------------------------------------------------ */
typedef struct ab_device ab_device;
typedef struct ab_block ab_block;
typedef struct ab_exec ab_exec;
typedef struct ab_fence ab_fence;

typedef struct ab_info {               /* driver.Info */
    char name[128];
    uint8_t token[16];                 /* Adapter.Token(): the device UUID */
    uint64_t total_memory;
    uint32_t sm_count;
    uint32_t cc_major, cc_minor;
    uint32_t max_shared_per_block;
    uint32_t storage_offset_alignment; /* 256, as cuMemAlloc aligns (specs/060-cuda-bringup.md:318) */
    uint32_t subgroup_size;            /* 32 */
} ab_info;

typedef struct ab_open_opts {
    uint32_t struct_size;              /* sizeof(ab_open_opts): the struct may grow */
    int32_t lose_at_submission;        /* >0: report loss at that submission, counted from 1, without
                                          touching the GPU; mirrors CPUOptions.LoseAtSubmission
                                          (accel.go:306-314).  0 = never */
    int32_t use_graphs;                /* 1: replay each executable as a CUDA graph */
} ab_open_opts;

AB_API int ab_init(void);
AB_API int ab_device_count(int *count);
AB_API int ab_device_info(int ordinal, ab_info *out);
AB_API int ab_open(int ordinal, const ab_open_opts *opts, ab_device **out);   /* Adapter.Open  */
AB_API int ab_close(ab_device *dev);   /* refuses (AB_ERR_BUSY) while blocks or executables live */
AB_API int ab_lost(ab_device *dev);    /* Device.Lost(): AB_OK or AB_ERR_DEVICE_LOST              */

/* driver.Block (internal/driver/driver.go:219-238).  kind: */
enum { AB_MEMORY_DEVICE = 0, AB_MEMORY_HOST_VISIBLE = 1 };
AB_API int ab_alloc(ab_device *dev, int kind, size_t bytes, const char *label, ab_block **out);
/* A block over device memory the caller allocated and keeps owning (weights another runtime loaded,
 * a framework's tensor): the block can be named by plans like any other; freeing it releases the
 * handle only.  No accel analogue. */
AB_API int ab_block_import(ab_device *dev, void *device_ptr, size_t bytes, ab_block **out);
AB_API void *ab_block_bytes(ab_block *b);         /* Block.Bytes(): NULL for AB_MEMORY_DEVICE    */
AB_API void *ab_block_device_ptr(ab_block *b);    /* the device address (no accel analogue)      */
AB_API size_t ab_block_size(ab_block *b);
AB_API int ab_block_write(ab_block *b, size_t off, const void *src, size_t n);  /* synchronous   */
AB_API int ab_block_read(ab_block *b, size_t off, void *dst, size_t n);         /* synchronous   */
/* Refused with AB_ERR_BUSY while a live executable names the block, directly or through a bound
 * slot: children are closed before parents (docs/architecture.md:306-310). */
AB_API int ab_block_free(ab_block *b);

/* driver.KernelSupport.SupportsKernel (internal/driver/plan.go:424-428): AB_OK when this library
 * holds an sm_100a kernel for the reference kernel of that name.  digest may be NULL. */
AB_API int ab_supports_kernel(ab_device *dev, const char *name, const char *digest);

/* ------------------------------------------------------------------------------------------ */
/* Plans: driver.Plan / PlanNode / Dispatch / Operand (internal/driver/plan.go:31-201)          */
/* ------------------------------------------------------------------------------------------ */
enum { AB_OP_COPY = 0, AB_OP_HOST_WRITE = 1, AB_OP_DISPATCH = 2 };

typedef struct ab_operand {
    ab_block *block;     /* a fixed block, or NULL when `slot` names a rebindable slot */
    uint32_t slot;       /* 1-based, as accel numbers slots; 0 = none */
    uint32_t _pad;
    uint64_t offset;     /* bytes; a multiple of 256 for a dispatch binding */
    uint64_t size;       /* bytes; a whole number of elements */
} ab_operand;

typedef struct ab_node {
    int32_t op;
    int32_t barrier_before;        /* accepted and ignored: one in-order stream orders every node */
    /* AB_OP_DISPATCH */
    const char *kernel;            /* the reference kernel's name, e.g. "QuantMatVecInt4" */
    const char *digest;            /* optional */
    uint32_t count[3];             /* the reference's workgroup count; ignored (the backend derives
                                      its own launch geometry from uniforms and binding lengths) */
    int32_t n_bindings;
    const ab_operand *bindings;    /* positional, the reference kernel's binding order */
    const void *uniform;           /* std140 bytes of uniform block 0, or NULL */
    uint64_t uniform_bytes;
    /* AB_OP_COPY: bindings[0] = source, bindings[1] = destination (n_bindings = 2).
     * AB_OP_HOST_WRITE: bindings[0] = destination, payload below; the payload is copied into
     * staging the executable owns at compile time and again on ab_exec_set_payload. */
    const void *payload;
    uint64_t payload_bytes;
} ab_node;

typedef struct ab_plan {
    const ab_node *nodes;          /* a valid topological order */
    int32_t n_nodes;
    int32_t n_slots;
    int32_t collect_timings;       /* Plan.CollectTimings: time each submission with an event pair */
    int32_t max_in_flight;         /* CompileOptions.MaxInFlight (tensor/compile.go:19-27): submissions that may be
                                      in flight at once; 0 means 1.  Above one, a submission that finds every
                                      instance busy lowers a spare (own workspace, staging and graph), up to this
                                      many; one more is refused with AB_ERR_BUSY. */
} ab_plan;

typedef struct ab_slot_binding { uint32_t slot; uint32_t _pad; ab_block *block; uint64_t offset; } ab_slot_binding;

/* GraphCompiler.Compile / Executable (internal/driver/plan.go:360-400) */
AB_API int ab_compile(ab_device *dev, const ab_plan *plan, ab_exec **out);
AB_API int ab_exec_rebind(ab_exec *e, const ab_slot_binding *b, int n);            /* all or nothing */
AB_API int ab_exec_set_uniform(ab_exec *e, int node, int index, const void *std140, size_t n);
AB_API int ab_exec_set_payload(ab_exec *e, int node, const void *bytes, size_t n);
AB_API int ab_exec_submit(ab_exec *e, ab_fence **out);     /* begins the work, does not wait */
AB_API int ab_exec_close(ab_exec *e);
/* driver.Fence (internal/driver/plan.go:374-391).  Once the device is lost every outstanding fence
 * reports AB_ERR_DEVICE_LOST.  The executable accepts its next submission as soon as the fence
 * has been waited for, has answered 1 to ab_fence_done, or has been freed (which waits). */
AB_API int ab_fence_wait(ab_fence *f);                     /* AB_ERR_DEVICE_LOST on loss */
AB_API int ab_fence_done(ab_fence *f);                     /* 1 done, 0 running, <0 error */
AB_API uint64_t ab_fence_elapsed_ns(ab_fence *f);          /* driver.Timer.Elapsed; 0 if untimed */
AB_API void ab_fence_free(ab_fence *f);

/* ------------------------------------------------------------------------------------------ */
/* One dispatch on caller-owned device memory and a caller-owned stream.                        */
/* The argument convention is the one accel's GPU targets keep (specs/061-ptx-target.md:152-159,*/
/* internal/mslabi/mslabi.go): binding k is a device pointer with its offset applied, the        */
/* lengths block holds one u32 element count per binding, the uniform block arrives as std140   */
/* bytes.  `stream` is a CUstream / cudaStream_t of the current device (NULL = legacy default). */
/* Kernels that need scratch memory take it from `workspace`; ab_workspace_bytes says how much. */
/* ------------------------------------------------------------------------------------------ */
AB_API int ab_kernel_count(void);
AB_API const char *ab_kernel_name(int index);
AB_API int ab_workspace_bytes(const char *kernel, const uint32_t *lengths, int n_bindings,
                              const void *uniform, size_t uniform_bytes, size_t *bytes);
AB_API int ab_launch(const char *kernel, void *stream, void *const *bindings,
                     const uint32_t *lengths, int n_bindings, const void *uniform,
                     size_t uniform_bytes, void *workspace, size_t workspace_bytes);
/*
 * The int4 product (QuantMatMulInt4; M = 0 or 1 is the matvec) for callers that cannot allocate.
 * No counterpart in the reference: accel's backends allocate through driver.Device.Alloc.  It is
 * here for hosts that may only use memory handed to them (a plugin inside another runtime's
 * allocator, a loop that must not enter the driver's allocator once running, a sandbox without
 * cudaMalloc) and so cannot provide the split-K workspace ab_launch wants.  The scratch is an
 * 8 MiB array built into the library's device image: every GPU that loads the library holds it
 * until the process exits.  A shape that needs more is refused with AB_ERR_INVALID and a message
 * naming the size; nothing is launched.  The call allocates nothing, on the device or through any
 * library.  The first call on each device looks up the array's device address (with that device
 * current); make that first call before starting any stream capture.  All calls share the one
 * array, which keeps the previous call's partial sums (every element read is written first by
 * the same call, so nothing needs clearing); two calls that overlap on the GPU (different
 * streams) race on it, so keep calls to one stream or order them with events.
 * a f32[M*K], bq/bs/bz the packed planes of the [K,N] matrix, out f32[M*N], all device pointers,
 * 16-byte aligned; stream is a cudaStream_t of the current device.
 */
AB_API int ab_quant_matmul_int4_noalloc(void *stream, const float *a, const uint32_t *bq,
                                        const uint16_t *bs, const uint16_t *bz, float *out,
                                        uint32_t M, uint32_t N, uint32_t K);
/* Which variant the last ab_launch of this thread selected, and why: Plan.Selections()
 * (tensor/compile.go:36-41). */
AB_API const char *ab_last_selection(void);
/* How many CUDA kernels this library has launched (or recorded into a stream capture) so far in
 * this process; a caller differences it around a region to count its launches. */
AB_API uint64_t ab_launch_count(void);

/*
 * Kernel names and their bindings (order is ABI) and uniform blocks (std140, little-endian):
 *
 *  QuantMatVecInt4   a f32[K], bq u32, bs f16, bz f16, out f32[N]          GEMMDims{M,N,K}@0,4,8 (16 B)
 *                    internal/kernels/int4.go:60
 *  QuantMatMulInt4   a f32[M*K], bq, bs, bz, out f32[M*N]                  GEMMDims
 *                    internal/kernels/int4tiled.go:66
 *  QuantMatVecF32    a f32[K], bq i8[K*N], bs f16[ceil(K*N/32)], out f32[N]    GEMMDims (M is 1)
 *                    internal/kernels/matvec.go:204
 *  QuantMatMulTiledF32   a f32[M*K], bq i8, bs f16, out f32[M*N]               GEMMDims
 *                    internal/kernels/quant.go:195
 *  AttentionDecode, AttentionDecodeF16     q, k, v, lengths u32[1], out    AttnDims{QHeads,KVHeads,HeadDim,Scale f32}@0,4,8,12 (16 B)
 *                    internal/kernels/attention.go:97,422
 *  AttentionDecodePaged, AttentionDecodePagedF16   q, k, v, pages u32[P], lengths u32[1], out
 *                    PagedDims{QHeads,KVHeads,HeadDim,Block,Scale f32}@0,4,8,12,16 (32 B)   internal/kernels/paged.go:47,362
 *  AttentionDecodeBatched   q f32[B*qH*D], k f32, v f32, pages u32[B*MaxPages], lengths u32[B], out
 *                    BatchedDims{Batch,QHeads,KVHeads,HeadDim,Block,MaxPages,Scale f32}@0..24 (32 B)   internal/kernels/batched.go:53
 *  AttentionDecodeBatchedF16   the same over an f16 cache (no reference kernel of this name; the
 *                    reference reaches an f16 cache for a batch through AttentionRaggedF16)
 *  AttentionRagged, AttentionRaggedF16   q, k, v, pages, lengths u32[B], offsets u32[B+1], out
 *                    RaggedDims = BatchedDims layout                          internal/kernels/ragged.go:61, raggedf16.go:43
 *  GroupedMatVec     x f32[T*K], w f32[E*K*N], offsets u32[E+1], out f32[T*N]   GroupedDims{Experts,K,N}@0,4,8 (16 B)
 *                    internal/kernels/grouped.go:49
 *  GroupedMatMul     same bindings                                          GroupedTiledDims{Experts,Tokens,K,N}@0,4,8,12 (16 B)
 *                    internal/kernels/groupedtiled.go:77
 *  GroupedMatMulInt4 x f32[T*K], bq u32[E*ceil(KN/8)], bs f16[E*ceil(KN/128)], bz f16, offsets u32[E+1], out
 *                    GroupedTiledDims.  No reference kernel: each expert's [K,N] matrix quantized
 *                    on its own with quant.Int4Quantize, result = GroupedMatMul over the dequantized
 *                    weights.
 *  SegmentOffsets    counts u32[R], offsets u32[R+1]                        SegmentDims{Rows}@0 (16 B)   internal/kernels/segment.go:40
 *  ScatterRows, ScatterRowsF16   rows, ids u32, state                        RowParams{Rows,Width,Capacity}@0,4,8 (16 B)
 *                    internal/kernels/elementwise.go:182,221
 *  GatherRows, GatherRowsF16     table, ids u32, out f32                     RowParams   internal/kernels/elementwise.go:118,133
 *  RMSNorm           x, w, out                                              RowDims{Rows,Width,Eps f32}@0,4,8 (16 B)   internal/kernels/norm.go:46
 *  RoPE              positions u32[rows], inout f32                          RoPEParams{Rows,Width,RotaryDim,Base f32}@0,4,8,12 (16 B)
 *                    internal/kernels/elementwise.go:267
 *  SwiGLU, ElemAdd   a, b, out                                               none   internal/kernels/elementwise.go:85,22
 *  SampleArgmax      logits f32[rows*vocab], out u32[rows]                   SampleDims{Vocab,Rows}@0,4 (16 B)   internal/kernels/sample.go:50
 *  CastF32ToF16, CastF16ToF32    in, out                                     none   internal/kernels/cast.go:30,38
 *  AttentionPrefill, AttentionPrefillF16   q f32[QSeq*QHeads*HeadDim], k, v, lengths u32[1], out
 *                    PrefillDims{QHeads,KVHeads,HeadDim,QSeq,Base,Scale f32}@0..20 (32 B)   internal/kernels/prefill.go:66,225
 *  AttentionPrefillPaged, AttentionPrefillPagedF16   q, k, v, pages u32[P], lengths u32[1], out
 *                    PagedPrefillDims{QHeads,KVHeads,HeadDim,QSeq,Base,Block,Scale f32}@0..24 (32 B)
 *                    internal/kernels/prefill.go:409, pagedprefillf16.go:31.  Query row s sees positions <= Base + s.
 *  Softmax           x f32[rows*width], out                                 RowDims   internal/kernels/norm.go:95
 *  ScaleRows         x, factors f32[rows], out                              RowSampleDims{Vocab,Rows,History,Slots}@0..12 (16 B)
 *                    internal/kernels/rowsample.go:226
 *  LogitBias         logits, ids u32[rows*Slots], values f32[rows*Slots], out   RowSampleDims   rowsample.go:304
 *  TopKMaskRows, TopPMaskRows   weights, ks u32[rows] | ps f32[rows], out   RowSampleDims   rowsample.go:42,126
 *  TopKMask, TopPMask           weights, out                                TopDims{Vocab,K,P f32}@0,4,8 (16 B)   topk.go:59,153
 *  SampleRows        probs, draws f32[rows], factors f32[rows], out u32[rows]   RowSampleDims   rowsample.go:246
 *  SampleCategorical probs, draws f32[rows], out u32[rows]                  SampleDims   sample.go:133
 *  PenaltyClearRows / PenaltyCountRows / PenaltyApplyRows   counts u32[rows*Vocab] / history u32[rows*History],
 *                    filled u32[rows], counts / logits, counts, repetition f32[rows], presence, frequency, out
 *                    RowSampleDims   rowsample.go:325,336,356
 *  PenaltyClear / PenaltyCount / PenaltyApply   counts / history, counts / logits, counts, out
 *                    PenaltyDims{Vocab,History,Count,Repetition f32,Presence f32,Frequency f32}@0..20 (32 B)   penalty.go:60,98,136
 *                    Every sampling kernel reproduces the reference's order of sums (128 strided partials and a
 *                    binary tree; the categorical walk in index order), so ids and masks are bit-exact.
 *  QuantMatVecInt4Packed, QuantMatMulInt4Packed   a f32, packed u32 words (ab_int4_prepack), out f32   GEMMDims
 *                    No reference kernel: QuantMatVecInt4 / QuantMatMulInt4 over the load-time prepack of the same
 *                    matrix.  Up to 48 rows: the tcgen05 decode kernel in passes of 16; beyond: the tcgen05 tile kernel.
 *  QuantMatMulInt4PackedSplit3   a, packed, out0 f32[M*N1], out1 f32[M*N2], out2 f32[M*(N-N1-N2)]
 *                    {M,N,K,N1,N2}@0..16 (32 B).  One product whose column ranges land in three matrices (q | k | v).
 *  QuantMatMulInt4PackedSwiGLU   a, packed, out f32[M*N/2]                  GEMMDims.  The 128-column groups of the packed
 *                    matrix alternate gate, up; out = SwiGLU(gate, up) (elementwise.go:85) from the epilogue.
 *  QuantMatMulInt4PackedA, QuantMatMulInt4PackedSplit3A, QuantMatMulInt4PackedSwiGLUA   the three forms above with
 *                    one more binding after a: amax f32[M], every activation row's largest magnitude (what
 *                    AddRMSNormAmax leaves).  The decode kernel scales its f16 operand by a power of two taken from
 *                    it; without the binding a small kernel finds the maxima first.  Bit-identical results.
 *                    QuantMatMulInt4PackedA reads the fourth word of its GEMMDims as AmaxParts: with P > 1 amax is
 *                    f32[M*P] and a row's maximum is the largest of its P entries (what the two kernels below leave).
 *  QuantMatMulInt4PackedSwiGLUAMax   a, amax f32[M], packed, out f32[M*N/2], outmax f32[M*N/64]   GEMMDims.  ...SwiGLUA
 *                    that also leaves the largest |out| of every 32 output columns (NaN counts as the largest), for
 *                    the product that reads out next: its A form with AmaxParts = N/64.  Up to 48 rows.
 *  AttentionDecodeBatchedMax, AttentionDecodeBatchedF16Max   AttentionDecodeBatched(F16) with a seventh binding,
 *                    outmax f32[B*qH*4]: four maxima per head whose largest is the head's largest |out|; the
 *                    product that reads out next takes them as AmaxParts = qH*4.  out is bit-identical.
 *  GroupedMatMulInt4Packed   x f32[T*K], packed (Experts prepacked matrices end to end), offsets u32[E+1], out f32[T*N]
 *                    GroupedTiledDims.  GroupedMatMulInt4 over prepacked experts, on the tcgen05 tile kernel.
 *  ArgmaxShard       logits f32[rows*Width], pairs f32[rows*Parts*2]        {Width,Rows,Parts,Rank,First}@0..16 (32 B)
 *  ArgmaxMerge       pairs f32[rows*Parts*2], out u32[rows]                 {Rows,Parts}@0,4 (16 B).  No reference kernels:
 *                    SampleArgmax over a vocabulary split by columns over Parts ranks; slot Rank of a row's pairs holds
 *                    (largest logit, its index in the whole vocabulary), the other slots zero, so the sum over ranks is
 *                    the gather; the merge takes the largest value, the lowest index among equals.
 *  Int4Quantize      w f32[n], packed u32, scales f16, zeros f16            none.  quant.Int4Quantize
 *                    (quant/int4.go:71) run on the device, bit-identical to the host routine.
 *  DecodeStepInputs  sampled u32[B], pages u32[B*MaxPages], tokens u32[B], pos_q u32[B*QHeads], pos_k u32[B*KVHeads],
 *                    slots u32[B], lengths u32[B]     {Batch,QHeads,KVHeads,Block,MaxPages}@0..16 (32 B).  No reference
 *                    kernel: the per-step host writes of a decode loop (docs/tutorial/11-batching-sequences.md:83-103)
 *                    done on the device, so a replayed step feeds the next without a host round trip.
 *  AddRMSNorm        x, delta, w, sum f32[rows*width], norm f32[rows*width]  RowDims (16 B).  No reference kernel: ElemAdd
 *                    (elementwise.go:22) followed by RMSNorm (norm.go:46) in one launch, sum = x + delta, norm =
 *                    RMSNorm(sum) * w; bit-identical to the two dispatches.  Width <= 8192.
 *  AddRMSNormAmax    x, delta, w, sum, norm, amax f32[rows]                  RowDims.  AddRMSNorm that also writes every
 *                    row's largest |norm| for the ...A product that reads norm next.
 *  RopeScatterQKV, RopeScatterQKVF16   pos_q u32[B*QHeads], pos_k u32[B*KVHeads], slots u32[B], q f32 (in place),
 *                    k f32 (in place), v f32, k_cache, v_cache (f32 / f16 [Capacity, KVHeads, HeadDim])
 *                    {Batch,QHeads,KVHeads,HeadDim,RotaryDim,Capacity,Base f32}@0..24 (32 B).  No reference kernel:
 *                    RoPE on q and on k (elementwise.go:267), then ScatterRows of k and v into the paged cache at
 *                    each row's slot (elementwise.go:182; F16: through CastF32ToF16, cast.go:30), in one launch;
 *                    bit-identical to the four (six) dispatches.
 */

/* ------------------------------------------------------------------------------------------ */
/* Host-side pieces of the path                                                                 */
/* ------------------------------------------------------------------------------------------ */
/* quant.Int4Quantize / Int4Nibble / Int4Dequantize (quant/int4.go:71-175).  packed holds
 * ceil(n/8) words, scales and zeros ceil(n/128) f16 bit patterns each. */
AB_API int ab_int4_quantize(const float *w, size_t n, uint32_t *packed, uint16_t *scales,
                            uint16_t *zeros);
AB_API uint32_t ab_int4_nibble(const uint32_t *packed, size_t i);
AB_API int ab_int4_dequantize(const uint32_t *packed, const uint16_t *scales,
                              const uint16_t *zeros, size_t n, float *out);
/* quant.Int8Quantize / Int8Dequantize (quant/quant.go:60-134): n quants in [-127, 127], ceil(n/32) f16
 * scale bit patterns. */
AB_API int ab_int8_quantize(const float *w, size_t n, int8_t *quants, uint16_t *scales);
AB_API int ab_int8_dequantize(const int8_t *quants, const uint16_t *scales, size_t n, float *out);
/* accel.ToFloat16 / Float16.F32 (internal/kernel/narrow.go:67-140) */
AB_API uint16_t ab_f32_to_f16(const float *x);     /* by pointer: no float crosses by value */
AB_API void ab_f16_to_f32(uint16_t h, float *out);

/* tensor.BlockPool (tensor/blockpool.go:46-133).  Thread-safe. */
typedef struct ab_blockpool ab_blockpool;
AB_API int ab_blockpool_new(int blocks, int positions_per_block, ab_blockpool **out);
AB_API void ab_blockpool_close(ab_blockpool *p);
AB_API int ab_blockpool_block_size(ab_blockpool *p);
AB_API int ab_blockpool_available(ab_blockpool *p);
/* Grow: `pages` holds n_pages entries and has room for ceil(n/block); returns the new count
 * (>= n_pages) or a negative status; the pool never evicts (AB_ERR_OOM). */
AB_API int ab_blockpool_grow(ab_blockpool *p, uint32_t *pages, int n_pages, int n_positions);
/* Free: returns AB_OK, or AB_ERR_INVALID when any page was already free (the others are freed). */
AB_API int ab_blockpool_free(ab_blockpool *p, const uint32_t *pages, int n_pages);
AB_API int ab_blockpool_positions(ab_blockpool *p, int n_pages);

/* Group-aligned column split of an int4 [K,N] matrix for tensor-parallel sharding: shard r of
 * `parts` owns columns [begin, end), both multiples of 128, so each shard's codes, scales and
 * zeros are bit-identical to the same columns of the unsharded matrix. */
AB_API int ab_int4_column_split(uint32_t n_cols, int parts, int rank, uint32_t *begin,
                                uint32_t *end);

/* ---- Load-time prepack of an int4 matrix for the decode-batch kernels ----------------------
 * No reference counterpart: accel's kernels read quant.Int4Quantize's three planes as they are
 * (internal/kernels/int4.go:60-101).  The prepack is a pure permutation of those planes (N a
 * multiple of 128): per 128-column group and per 64 weight rows, the codes of a column contiguous
 * along k with the group's scale / zero pairs behind them, so that one CTA's K range of a group is
 * one contiguous run for a bulk copy; a header keeps one float per group (a power of two from the
 * group's largest scale).  ab_int4_prepack_bytes gives the size of `packed` (device memory,
 * 256-byte aligned); ab_int4_prepack fills it on `stream` from device-resident planes.  The
 * kernels QuantMatVecInt4Packed / QuantMatMulInt4Packed (ab_launch; bindings a, packed, out;
 * GEMMDims) compute what QuantMatVecInt4 / QuantMatMulInt4 compute from the three planes. */
AB_API size_t ab_int4_prepack_bytes(uint32_t K, uint32_t N);
AB_API int ab_int4_prepack(void *stream, const uint32_t *codes, const uint16_t *scales,
                           const uint16_t *zeros, uint32_t K, uint32_t N, void *packed);
/* AB_OK, or AB_ERR_TIMEOUT once a bounded device-side wait of the prepacked kernels has run out
 * (synchronous; sticky for the process). */
AB_API int ab_int4_stream_error(void);

/* ---- One-shot all-reduce over NVLink peer memory (tensor-parallel decode) -----------------
 * No reference counterpart: accel is single-device (the tensor-parallel layer sits above the
 * per-device plan).  Sums `n` f32 values (a multiple of 4) over `world` <= 8 ranks, one process per
 * GPU, and leaves the same bits on every rank (ranks are added in rank order).  `out` may be `in`.
 *
 * Each rank allocates ab_peer_allreduce_buffer_bytes(capacity) bytes that every rank can address
 * (CUDA IPC, the virtual-memory API, or a symmetric-memory allocator), zeroed before the first
 * call on any rank, and passes all ranks' mappings of them, in rank order, as peer_buffers (a HOST
 * array of `world` device pointers, 16-byte aligned).  `state` is
 * ab_peer_allreduce_state_bytes() of this rank's own zeroed device memory; it holds the call
 * counter, so a call can be captured in a CUDA graph and replayed.  Calls of one rank must be
 * ordered on one stream, and every rank must make the same sequence of calls with the same n.
 * The kernels of different ranks wait for one another over NVLink: every rank must run on a GPU
 * of its own.  The wait is bounded (about a second of polling); a rank whose peers never arrive
 * records the failing call in `state`, writes no output and returns normally, and
 * ab_peer_allreduce_error reports AB_ERR_TIMEOUT from then on.  Loads and stores are plain (no
 * multicast, no TMA). */
AB_API size_t ab_peer_allreduce_buffer_bytes(uint32_t capacity_floats);
AB_API size_t ab_peer_allreduce_state_bytes(void);
AB_API int ab_peer_allreduce_f32(void *stream, void *const *peer_buffers, void *state, int rank,
                                 int world, const float *in, float *out, uint32_t n,
                                 uint32_t capacity_floats);
/* The same call with the decode layer's next two operators done by its summing stage (one CTA per
 * row): sum_out = residual + all-reduce(in), norm_out = RMSNorm(sum_out) * gain, bit-identical to
 * ab_peer_allreduce_f32 followed by the AddRMSNorm kernel.  eps_bits is the f32 epsilon's bit
 * pattern (no float crosses the boundary by value).  Width <= 4096, rows <= one per SM; it counts
 * as one call of the same sequence as ab_peer_allreduce_f32 (same buffers, same state). */
AB_API int ab_peer_allreduce_add_rmsnorm_f32(void *stream, void *const *peer_buffers, void *state,
                                             int rank, int world, const float *in,
                                             const float *residual, const float *gain, float *sum_out,
                                             float *norm_out, uint32_t rows, uint32_t width,
                                             uint32_t eps_bits, uint32_t capacity_floats);
/* In-place forms: the rank's partial result already lies in a region of its own buffer (the
 * producing kernel wrote it there), so nothing is copied and the call is a signal, a bounded wait
 * and the sum.  Regions start at or behind ab_peer_allreduce_region_offset_bytes(capacity) and are
 * the caller's to lay out, at the same offset on every rank; a region must not be rewritten until
 * another all-reduce call of this sequence has been made in between (a peer may still be reading
 * it until it has signalled its next call): two regions used alternately are enough.  buffer_bytes
 * is the size every rank allocated.  The calls belong to the same sequence as the copying forms. */
AB_API size_t ab_peer_allreduce_region_offset_bytes(uint32_t capacity_floats);
AB_API int ab_peer_allreduce_inplace_f32(void *stream, void *const *peer_buffers, void *state, int rank,
                                         int world, size_t region_offset_bytes, float *out, uint32_t n,
                                         size_t buffer_bytes);
AB_API int ab_peer_allreduce_inplace_add_rmsnorm_f32(void *stream, void *const *peer_buffers, void *state,
                                                     int rank, int world, size_t region_offset_bytes,
                                                     const float *residual, const float *gain,
                                                     float *sum_out, float *norm_out, uint32_t rows,
                                                     uint32_t width, uint32_t eps_bits, size_t buffer_bytes);
/* The same call that also leaves every row's largest |norm_out| in amax_out[rows] (NULL: none), for
 * the prepacked int4 product that reads norm_out next (QuantMatMulInt4Packed...A). */
AB_API int ab_peer_allreduce_inplace_add_rmsnorm_amax_f32(void *stream, void *const *peer_buffers, void *state,
                                                     int rank, int world, size_t region_offset_bytes,
                                                     const float *residual, const float *gain,
                                                     float *sum_out, float *norm_out, uint32_t rows,
                                                     uint32_t width, uint32_t eps_bits, size_t buffer_bytes, float *amax_out);
/* AB_OK, or AB_ERR_TIMEOUT with *failed_call = the 1-based call that gave up (synchronous). */
AB_API int ab_peer_allreduce_error(const void *state, uint32_t *failed_call);
/* How many polls of a peer's flag a CTA spends before it gives up (0 restores the default, about a
 * second).  A call that gave up still advances the call counter, so the sequence stays aligned
 * with the peers'; ab_peer_allreduce_clear_error forgets the recorded failure.  Both synchronous. */
AB_API int ab_peer_allreduce_set_spin_limit(void *state, uint32_t polls);
AB_API int ab_peer_allreduce_clear_error(void *state);

/* ---- N devices of one process as a group (specs/060-cuda-bringup.md:261-267, 537-548 leave
 * multi-device to a later layer; no accel analogue).  ab_group_open enables peer access between
 * every pair of the named devices (distinct ordinals, at most 8), and gives every rank a zeroed peer
 * buffer of ab_peer_allreduce_buffer_bytes(capacity_floats), a zeroed state block and a non-blocking
 * stream; ab_group_peer_table is the HOST array of the buffers in rank order that the
 * ab_peer_allreduce_* calls take.  A host drives rank r by making ab_group_ordinal(g, r) current and
 * enqueueing on ab_group_stream(g, r); ab_group_all_reduce_f32 enqueues one all-reduce for every rank
 * in turn (in[r], out[r]: device memory of rank r); ab_group_synchronize waits for every rank's stream
 * and reports AB_ERR_TIMEOUT if a bounded wait ran out. */
typedef struct ab_group ab_group;
AB_API int ab_group_open(const int *ordinals, int n, uint32_t capacity_floats, ab_group **out);
AB_API int ab_group_close(ab_group *g);
AB_API int ab_group_size(const ab_group *g);
AB_API int ab_group_ordinal(const ab_group *g, int rank);
AB_API void *ab_group_buffer(const ab_group *g, int rank);
AB_API void *ab_group_state(const ab_group *g, int rank);
AB_API void *ab_group_stream(const ab_group *g, int rank);
AB_API void *const *ab_group_peer_table(const ab_group *g);
AB_API int ab_group_all_reduce_f32(ab_group *g, const float *const *in, float *const *out, uint32_t n);
AB_API int ab_group_synchronize(ab_group *g);

#ifdef __cplusplus
}
#endif
#endif /* ACCEL_B200_H */
