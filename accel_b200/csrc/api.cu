// The C ABI: kernel registry and direct dispatch, the driver seam (device, block, executable,
// fence) shaped like accel's internal/driver, and the host-side pieces of the path (quantizer,
// block pool, shard arithmetic).
#include <algorithm>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <new>
#include <string>
#include <thread>
#include <vector>

#include "common.cuh"

namespace ab {

// ------------------------------------------------------------------------------------------------
// errors
// ------------------------------------------------------------------------------------------------
static thread_local char g_err[1024] = "";
static thread_local char g_sel[512] = "";

int fail(int code, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
    return code;
}

void note_selection(const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_sel, sizeof g_sel, fmt, ap);
    va_end(ap);
}

// Sticky errors mean the context is gone (specs/060-cuda-bringup.md:576-604); out-of-memory and
// argument errors do not.
static bool is_loss(cudaError_t e)
{
    switch (e) {
    case cudaErrorIllegalAddress: case cudaErrorLaunchFailure: case cudaErrorLaunchTimeout:
    case cudaErrorHardwareStackError: case cudaErrorIllegalInstruction:
    case cudaErrorMisalignedAddress: case cudaErrorInvalidAddressSpace: case cudaErrorInvalidPc:
    case cudaErrorECCUncorrectable: case cudaErrorDevicesUnavailable: case cudaErrorAssert:
        return true;
    default: return false;
    }
}

int check_cuda(cudaError_t e, const char *what)
{
    if (e == cudaSuccess) return AB_OK;
    if (e == cudaErrorMemoryAllocation) return fail(AB_ERR_OOM, "%s: out of device memory", what);
    if (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver)
        return fail(AB_ERR_NO_DEVICE, "%s: %s", what, cudaGetErrorString(e));
    if (is_loss(e)) return fail(AB_ERR_DEVICE_LOST, "%s: device lost: %s", what, cudaGetErrorString(e));
    return fail(AB_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

// Whether the support kernels (norms, RoPE, attention, sampling) are launched as programmatic
// dependents too.  Off unless AB_PDL=1: measured on the 7B-shape decode step, dependents that start
// early and wait hold SM resources the running kernel's later waves need (8.97 ms per step against
// 8.01 ms with only the int4 products launched that way).  The kernels still TRIGGER their
// dependents early, which is what lets the product that follows a norm prefetch its weights.
bool pdl_enabled()
{
    static const bool on = getenv("AB_PDL") && atoi(getenv("AB_PDL")) != 0;
    return on;
}

static std::atomic<unsigned long long> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

int sm_count()
{
    static std::mutex mu;
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    std::lock_guard<std::mutex> lk(mu);
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

// ------------------------------------------------------------------------------------------------
// registry: reference kernel name -> launcher
// ------------------------------------------------------------------------------------------------
static const KernelEntry kKernels[] = {
    {"QuantMatVecInt4", 5, 16, launch_quant_matvec_int4},
    {"QuantMatMulInt4", 5, 16, launch_quant_matmul_int4},
    {"QuantMatVecF32", 4, 16, launch_quant_matvec_f32},
    {"QuantMatMulTiledF32", 4, 16, launch_quant_matmul_tiled_f32},
    {"QuantMatVecInt4Packed", 3, 16, launch_quant_matvec_int4_packed},
    {"QuantMatMulInt4Packed", 3, 16, launch_quant_matmul_int4_packed},
    {"QuantMatMulInt4PackedSplit3", 5, 32, launch_quant_matmul_int4_packed_split3},
    {"QuantMatMulInt4PackedSwiGLU", 3, 16, launch_quant_matmul_int4_packed_swiglu},
    {"QuantMatMulInt4PackedA", 4, 16, launch_quant_matmul_int4_packed_a},
    {"QuantMatMulInt4PackedSplit3A", 6, 32, launch_quant_matmul_int4_packed_split3_a},
    {"QuantMatMulInt4PackedSwiGLUA", 4, 16, launch_quant_matmul_int4_packed_swiglu_a},
    {"QuantMatMulInt4PackedSwiGLUAMax", 5, 16, launch_quant_matmul_int4_packed_swiglu_a_max},
    {"AttentionDecode", 5, 16, launch_attention_decode},
    {"AttentionDecodeF16", 5, 16, launch_attention_decode_f16},
    {"AttentionDecodePaged", 6, 32, launch_attention_decode_paged},
    {"AttentionDecodePagedF16", 6, 32, launch_attention_decode_paged_f16},
    {"AttentionDecodeBatched", 6, 32, launch_attention_decode_batched},
    {"AttentionDecodeBatchedF16", 6, 32, launch_attention_decode_batched_f16},
    {"AttentionDecodeBatchedMax", 7, 32, launch_attention_decode_batched_max},
    {"AttentionDecodeBatchedF16Max", 7, 32, launch_attention_decode_batched_f16_max},
    {"AttentionRagged", 7, 32, launch_attention_ragged},
    {"AttentionRaggedF16", 7, 32, launch_attention_ragged_f16},
    {"AttentionPrefill", 5, 32, launch_attention_prefill},
    {"AttentionPrefillF16", 5, 32, launch_attention_prefill_f16},
    {"AttentionPrefillPaged", 6, 32, launch_attention_prefill_paged},
    {"AttentionPrefillPagedF16", 6, 32, launch_attention_prefill_paged_f16},
    {"GroupedMatVec", 4, 16, launch_grouped_matvec},
    {"GroupedMatMul", 4, 16, launch_grouped_matmul},
    {"GroupedMatMulInt4", 6, 16, launch_grouped_matmul_int4},
    {"GroupedMatMulInt4Packed", 4, 16, launch_grouped_matmul_int4_packed},
    {"SegmentOffsets", 2, 16, launch_segment_offsets},
    {"ScatterRows", 3, 16, launch_scatter_rows},
    {"ScatterRowsF16", 3, 16, launch_scatter_rows_f16},
    {"GatherRows", 3, 16, launch_gather_rows},
    {"GatherRowsF16", 3, 16, launch_gather_rows_f16},
    {"RMSNorm", 3, 16, launch_rmsnorm},
    {"RoPE", 2, 16, launch_rope},
    {"SwiGLU", 3, 0, launch_swiglu},
    {"ElemAdd", 3, 0, launch_elem_add},
    {"SampleArgmax", 2, 16, launch_sample_argmax},
    {"ArgmaxShard", 2, 32, launch_argmax_shard},
    {"ArgmaxMerge", 2, 16, launch_argmax_merge},
    {"Softmax", 2, 16, launch_softmax},
    {"ScaleRows", 3, 16, launch_scale_rows},
    {"LogitBias", 4, 16, launch_logit_bias},
    {"TopKMaskRows", 3, 16, launch_topk_mask_rows},
    {"TopPMaskRows", 3, 16, launch_topp_mask_rows},
    {"TopKMask", 2, 16, launch_topk_mask},
    {"TopPMask", 2, 16, launch_topp_mask},
    {"SampleRows", 4, 16, launch_sample_rows},
    {"SampleCategorical", 3, 16, launch_sample_categorical},
    {"PenaltyClearRows", 1, 16, launch_penalty_clear_rows},
    {"PenaltyCountRows", 3, 16, launch_penalty_count_rows},
    {"PenaltyApplyRows", 6, 16, launch_penalty_apply_rows},
    {"PenaltyClear", 1, 32, launch_penalty_clear},
    {"PenaltyCount", 2, 32, launch_penalty_count},
    {"PenaltyApply", 3, 32, launch_penalty_apply},
    {"CastF32ToF16", 2, 0, launch_cast_f32_to_f16},
    {"CastF16ToF32", 2, 0, launch_cast_f16_to_f32},
    {"Int4Quantize", 4, 0, launch_int4_quantize},
    {"DecodeStepInputs", 7, 32, launch_decode_step_inputs},
    {"AddRMSNorm", 5, 16, launch_add_rmsnorm},
    {"AddRMSNormAmax", 6, 16, launch_add_rmsnorm_amax},
    {"RopeScatterQKV", 8, 32, launch_rope_scatter_qkv},
    {"RopeScatterQKVF16", 8, 32, launch_rope_scatter_qkv_f16},
};
static constexpr int kKernelCount = (int)(sizeof(kKernels) / sizeof(kKernels[0]));

static const KernelEntry *find_kernel(const char *name)
{
    if (!name) return nullptr;
    for (int i = 0; i < kKernelCount; i++)
        if (strcmp(kKernels[i].name, name) == 0) return &kKernels[i];
    return nullptr;
}

static int dispatch(const char *name, Launch &l)
{
    const KernelEntry *k = find_kernel(name);
    if (!k)
        return fail(AB_ERR_UNSUPPORTED, "no sm_100a kernel is registered under the name \"%s\"; "
                    "this backend has no CPU fallback", name ? name : "(null)");
    if (l.nb != k->n_bindings)
        return fail(AB_ERR_INVALID, "%s takes %d bindings and %d were given", name, k->n_bindings, l.nb);
    if (k->uniform_bytes && (!l.u || l.ubytes < k->uniform_bytes))
        return fail(AB_ERR_INVALID, "%s takes a %zu-byte uniform block and %zu bytes were given",
                    name, k->uniform_bytes, l.u ? l.ubytes : (size_t)0);
    if (!l.len) return fail(AB_ERR_INVALID, "%s: the lengths block is missing", name);
    if (!l.query_ws) {
        if (!l.b) return fail(AB_ERR_INVALID, "%s: the bindings are missing", name);
        for (int i = 0; i < l.nb; i++) {
            if (!l.b[i] && l.len[i])
                return fail(AB_ERR_INVALID, "%s: binding %d is NULL with %u elements", name, i, l.len[i]);
            if (reinterpret_cast<uintptr_t>(l.b[i]) % 16)
                return fail(AB_ERR_INVALID, "%s: binding %d is not 16-byte aligned; accel hands a "
                            "backend offsets that are multiples of 256", name, i);
        }
    }
    return k->fn(l);
}

// ------------------------------------------------------------------------------------------------
// driver seam objects
// ------------------------------------------------------------------------------------------------
}  // namespace ab

struct ab_device {
    int ordinal;
    cudaStream_t stream;           // explicit, non-blocking; never the NULL stream
    std::atomic<int> live{0};      // blocks + executables
    std::atomic<int> lost{0};
    std::atomic<int> submissions{0};
    int lose_at;
    int use_graphs;
};

struct ab_block {
    ab_device *dev;
    int kind;
    size_t size;
    void *dptr;     // device address (== host address mapping for pinned memory)
    void *hptr;     // host address for AB_MEMORY_HOST_VISIBLE
    std::atomic<int> users{0};     // live executables that name this block (directly or by a slot)
    bool borrowed = false;         // memory the caller owns (ab_block_import): never freed here
};

namespace ab { struct Instance; }

struct ab_fence {
    ab_device *dev;
    ab_exec *exec;
    ab::Instance *inst;    // the executable's instance this submission runs on; NULL once released
    cudaEvent_t start, done;
    bool timed;
    int injected;   // a loss injected on the host
};

namespace ab {
struct Node {
    int op;
    std::string kernel;
    std::vector<ab_operand> bind;
    std::vector<uint8_t> uniform;
    std::vector<void *> ptrs;
    std::vector<uint32_t> lens;
    std::vector<uint8_t> payload;  // a host write's bytes as last set; copied into the instance at submit
    size_t payload_bytes = 0;
    size_t ws = 0;
};
// One lowering of the executable: what a submission owns while it is in flight (CompileOptions.
// MaxInFlight, tensor/compile.go:19-27: "the plan lowers itself again into a spare graph the first
// time a submission finds every instance busy, up to this many, each with its own transient memory").
struct Instance {
    void *workspace = nullptr;
    std::vector<void *> staging;   // per node: the pinned payload of a host write (NULL otherwise)
    cudaGraphExec_t graph = nullptr;
    uint64_t graph_version = 0;    // the executable's version the graph was captured at
    cudaEvent_t ev_start = nullptr, ev_done = nullptr;
    std::atomic<int> busy{0};
};
static size_t elem_bytes_of(const char *kernel, int binding);
}  // namespace ab

struct ab_exec {
    ab_device *dev;
    std::vector<ab::Node> nodes;
    std::vector<ab_slot_binding> slots;    // index = slot - 1
    std::vector<bool> slot_set;
    size_t ws_bytes = 0;
    bool timings = false;
    int max_in_flight = 1;
    std::mutex mu;                         // instances, their busy flags and the version
    std::vector<ab::Instance *> inst;      // at least one; spares are lowered on demand
    uint64_t version = 1;                  // bumped by rebind / set_uniform: graphs captured earlier are stale
    std::vector<ab_block *> held;          // blocks named directly by a node, counted in users
    int busy_count()
    {
        int n = 0;
        for (auto *i : inst) n += i->busy.load();
        return n;
    }
};

namespace ab {

static int set_device(ab_device *d)
{
    if (!d) return fail(AB_ERR_INVALID, "device handle is NULL");
    if (d->lost.load()) return fail(AB_ERR_DEVICE_LOST, "the device was lost; loss is terminal");
    return check_cuda(cudaSetDevice(d->ordinal), "cudaSetDevice");
}

static int note_loss(ab_device *d, int rc)
{
    if (rc == AB_ERR_DEVICE_LOST && d) d->lost.store(1);
    return rc;
}

// Element size of each binding, needed to turn an operand's byte size into the lengths block.
static size_t elem_bytes_of(const char *k, int i)
{
    auto is = [&](const char *n) { return strcmp(k, n) == 0; };
    if (is("QuantMatVecInt4") || is("QuantMatMulInt4")) return (i == 2 || i == 3) ? 2 : 4;
    if (is("GroupedMatMulInt4")) return (i == 2 || i == 3) ? 2 : 4;
    if (is("QuantMatVecF32") || is("QuantMatMulTiledF32")) return i == 1 ? 1 : (i == 2 ? 2 : 4);
    if (is("AttentionPrefillF16") || is("AttentionPrefillPagedF16")) return (i == 1 || i == 2) ? 2 : 4;
    if (is("AttentionDecodeF16") || is("AttentionDecodePagedF16") || is("AttentionDecodeBatchedF16") ||
        is("AttentionDecodeBatchedF16Max") || is("AttentionRaggedF16"))
        return (i == 1 || i == 2) ? 2 : 4;
    if (is("ScatterRowsF16")) return (i == 0 || i == 2) ? 2 : 4;
    if (is("GatherRowsF16")) return i == 0 ? 2 : 4;
    if (is("CastF32ToF16")) return i == 1 ? 2 : 4;
    if (is("CastF16ToF32")) return i == 0 ? 2 : 4;
    if (is("Int4Quantize")) return (i == 2 || i == 3) ? 2 : 4;
    return 4;
}

static int resolve(ab_exec *e, const ab_operand &o, void **out, const char *what, int node, int bi)
{
    ab_block *blk = o.block;
    uint64_t base = 0;
    if (!blk) {
        if (o.slot == 0 || o.slot > e->slots.size())
            return fail(AB_ERR_INVALID, "node %d binding %d (%s) names slot %u of %zu", node, bi,
                        what, o.slot, e->slots.size());
        if (!e->slot_set[o.slot - 1])
            return fail(AB_ERR_INVALID, "node %d binding %d (%s): slot %u is unbound", node, bi, what, o.slot);
        blk = e->slots[o.slot - 1].block;
        base = e->slots[o.slot - 1].offset;
    }
    if (!blk) return fail(AB_ERR_INVALID, "node %d binding %d (%s) has no block", node, bi, what);
    if (base + o.offset + o.size > blk->size)
        return fail(AB_ERR_INVALID, "node %d binding %d (%s): offset %llu + size %llu runs past the "
                    "block's %zu bytes", node, bi, what, (unsigned long long)(base + o.offset),
                    (unsigned long long)o.size, blk->size);
    *out = static_cast<char *>(blk->dptr) + base + o.offset;
    return AB_OK;
}

static int resolve_all(ab_exec *e)
{
    for (size_t n = 0; n < e->nodes.size(); n++) {
        Node &nd = e->nodes[n];
        nd.ptrs.resize(nd.bind.size());
        for (size_t i = 0; i < nd.bind.size(); i++) {
            int rc = resolve(e, nd.bind[i], &nd.ptrs[i], nd.kernel.c_str(), (int)n, (int)i);
            if (rc) return rc;
        }
    }
    return AB_OK;
}

static void free_instance(Instance *in)
{
    if (!in) return;
    if (in->graph) cudaGraphExecDestroy(in->graph);
    if (in->workspace) cudaFree(in->workspace);
    for (void *p : in->staging) if (p) cudaFreeHost(p);
    if (in->ev_start) cudaEventDestroy(in->ev_start);
    if (in->ev_done) cudaEventDestroy(in->ev_done);
    delete in;
}

// A lowering of the executable with transient memory of its own.
static int new_instance(ab_exec *e, Instance **out)
{
    Instance *in = new (std::nothrow) Instance();
    if (!in) return fail(AB_ERR_OOM, "executable instance: host allocation failed");
    int rc = AB_OK;
    if (e->ws_bytes) rc = check_cuda(cudaMalloc(&in->workspace, e->ws_bytes), "executable workspace");
    in->staging.assign(e->nodes.size(), nullptr);
    for (size_t n = 0; n < e->nodes.size() && !rc; n++)
        if (e->nodes[n].op == AB_OP_HOST_WRITE)
            rc = check_cuda(cudaHostAlloc(&in->staging[n], e->nodes[n].payload_bytes, cudaHostAllocDefault),
                            "host-write staging");
    if (!rc) rc = check_cuda(cudaEventCreate(&in->ev_start), "fence events");
    if (!rc) rc = check_cuda(cudaEventCreate(&in->ev_done), "fence events");
    if (rc) { cudaGetLastError(); free_instance(in); return rc; }
    *out = in;
    return AB_OK;
}

static int run_nodes(ab_exec *e, Instance *in, cudaStream_t s)
{
    for (size_t n = 0; n < e->nodes.size(); n++) {
        Node &nd = e->nodes[n];
        if (nd.op == AB_OP_DISPATCH) {
            Launch l{s, nd.ptrs.data(), nd.lens.data(), (int)nd.ptrs.size(),
                     nd.uniform.empty() ? nullptr : nd.uniform.data(), nd.uniform.size(),
                     in->workspace, e->ws_bytes, false, 0};
            int rc = dispatch(nd.kernel.c_str(), l);
            if (rc) return rc;
        } else if (nd.op == AB_OP_COPY) {
            size_t bytes = (size_t)std::min(nd.bind[0].size, nd.bind[1].size);
            // (either side may be a host-visible block: the runtime sorts out the direction)
            int rc = check_cuda(cudaMemcpyAsync(nd.ptrs[1], nd.ptrs[0], bytes, cudaMemcpyDefault, s), "copy node");
            if (rc) return rc;
        } else if (nd.op == AB_OP_HOST_WRITE) {
            size_t bytes = std::min(nd.payload_bytes, (size_t)nd.bind[0].size);
            int rc = check_cuda(cudaMemcpyAsync(nd.ptrs[0], in->staging[n], bytes, cudaMemcpyHostToDevice, s), "host-write node");
            if (rc) return rc;
        }
    }
    return AB_OK;
}

}  // namespace ab

using namespace ab;

// ------------------------------------------------------------------------------------------------
// exported: errors, registry, direct dispatch
// ------------------------------------------------------------------------------------------------
extern "C" {

const char *ab_error_string(int code)
{
    switch (code) {
    case AB_OK: return "ok";
    case AB_ERR_INVALID: return "invalid argument";
    case AB_ERR_UNSUPPORTED: return "no kernel for this name on this backend";
    case AB_ERR_OOM: return "out of memory";
    case AB_ERR_DEVICE_LOST: return "device lost";
    case AB_ERR_BUSY: return "busy";
    case AB_ERR_CUDA: return "CUDA error";
    case AB_ERR_NO_DEVICE: return "no CUDA device";
    case AB_ERR_TIMEOUT: return "a bounded wait for a peer ran out";
    default: return "unknown status";
    }
}

const char *ab_last_error(void) { return g_err; }
const char *ab_last_selection(void) { return g_sel; }
uint64_t ab_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int ab_kernel_count(void) { return kKernelCount; }
const char *ab_kernel_name(int i) { return (i >= 0 && i < kKernelCount) ? kKernels[i].name : nullptr; }

int ab_workspace_bytes(const char *kernel, const uint32_t *lengths, int nb, const void *uniform,
                       size_t ubytes, size_t *bytes)
{
    if (!bytes) return fail(AB_ERR_INVALID, "ab_workspace_bytes: bytes is NULL");
    Launch l{nullptr, nullptr, lengths, nb, static_cast<const uint8_t *>(uniform), ubytes, nullptr, 0, true, 0};
    int rc = dispatch(kernel, l);
    if (rc == AB_OK) *bytes = l.ws_need;
    return rc;
}

int ab_launch(const char *kernel, void *stream, void *const *bindings, const uint32_t *lengths,
              int nb, const void *uniform, size_t ubytes, void *workspace, size_t ws_bytes)
{
    Launch l{static_cast<cudaStream_t>(stream), bindings, lengths, nb,
             static_cast<const uint8_t *>(uniform), ubytes, workspace, ws_bytes, false, 0};
    return dispatch(kernel, l);
}

// ------------------------------------------------------------------------------------------------
// adapter / device / block
// ------------------------------------------------------------------------------------------------
int ab_init(void)
{
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) return check_cuda(e, "ab_init");
    if (n == 0) return fail(AB_ERR_NO_DEVICE, "ab_init: no CUDA device");
    return AB_OK;
}

int ab_device_count(int *count)
{
    if (!count) return fail(AB_ERR_INVALID, "ab_device_count: count is NULL");
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver) { *count = 0; return AB_OK; }
    if (e != cudaSuccess) return check_cuda(e, "ab_device_count");
    *count = n;
    return AB_OK;
}

int ab_device_info(int ord, ab_info *out)
{
    if (!out) return fail(AB_ERR_INVALID, "ab_device_info: out is NULL");
    cudaDeviceProp p;
    int rc = check_cuda(cudaGetDeviceProperties(&p, ord), "ab_device_info");
    if (rc) return rc;
    memset(out, 0, sizeof *out);
    snprintf(out->name, sizeof out->name, "%s", p.name);
    memcpy(out->token, p.uuid.bytes, 16);
    out->total_memory = p.totalGlobalMem;
    out->sm_count = (uint32_t)p.multiProcessorCount;
    out->cc_major = (uint32_t)p.major;
    out->cc_minor = (uint32_t)p.minor;
    out->max_shared_per_block = (uint32_t)p.sharedMemPerBlockOptin;
    out->storage_offset_alignment = 256;
    out->subgroup_size = 32;
    return AB_OK;
}

int ab_open(int ord, const ab_open_opts *opts, ab_device **out)
{
    if (!out) return fail(AB_ERR_INVALID, "ab_open: out is NULL");
    int n = 0;
    int rc = ab_device_count(&n);
    if (rc) return rc;
    if (ord < 0 || ord >= n) return fail(AB_ERR_NO_DEVICE, "ab_open: device %d of %d", ord, n);
    cudaDeviceProp p;
    rc = check_cuda(cudaGetDeviceProperties(&p, ord), "ab_open");
    if (rc) return rc;
    if (p.major != 10)
        return fail(AB_ERR_UNSUPPORTED, "ab_open: %s is compute capability %d.%d and this library "
                    "holds sm_100a code only", p.name, p.major, p.minor);
    rc = check_cuda(cudaSetDevice(ord), "cudaSetDevice");
    if (rc) return rc;
    ab_device *d = new (std::nothrow) ab_device();
    if (!d) return fail(AB_ERR_OOM, "ab_open: host allocation failed");
    d->ordinal = ord;
    d->lose_at = (opts && opts->struct_size >= 8) ? opts->lose_at_submission : 0;
    d->use_graphs = (opts && opts->struct_size >= 12) ? opts->use_graphs : 0;
    rc = check_cuda(cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking), "cudaStreamCreate");
    if (rc) { delete d; return rc; }
    *out = d;
    return AB_OK;
}

int ab_close(ab_device *d)
{
    if (!d) return AB_OK;
    if (d->live.load() > 0)
        return fail(AB_ERR_BUSY, "ab_close: %d block(s) or executable(s) are still live; a device "
                    "with live children refuses to close", d->live.load());
    if (!d->lost.load() && cudaSetDevice(d->ordinal) == cudaSuccess) {
        cudaStreamSynchronize(d->stream);
        cudaStreamDestroy(d->stream);
    }
    delete d;
    return AB_OK;
}

int ab_lost(ab_device *d)
{
    if (!d) return fail(AB_ERR_INVALID, "ab_lost: device is NULL");
    return d->lost.load() ? fail(AB_ERR_DEVICE_LOST, "the device was lost") : AB_OK;
}

int ab_alloc(ab_device *d, int kind, size_t bytes, const char *label, ab_block **out)
{
    if (!out) return fail(AB_ERR_INVALID, "ab_alloc: out is NULL");
    int rc = set_device(d);
    if (rc) return rc;
    if (bytes == 0) return fail(AB_ERR_INVALID, "ab_alloc(%s): zero bytes", label ? label : "");
    ab_block *b = new (std::nothrow) ab_block();
    if (!b) return fail(AB_ERR_OOM, "ab_alloc: host allocation failed");
    b->dev = d; b->kind = kind; b->size = bytes; b->dptr = nullptr; b->hptr = nullptr;
    if (kind == AB_MEMORY_DEVICE) {
        rc = check_cuda(cudaMalloc(&b->dptr, bytes), label ? label : "ab_alloc");
    } else if (kind == AB_MEMORY_HOST_VISIBLE) {
        rc = check_cuda(cudaHostAlloc(&b->hptr, bytes, cudaHostAllocMapped), label ? label : "ab_alloc");
        if (!rc) rc = check_cuda(cudaHostGetDevicePointer(&b->dptr, b->hptr, 0), "cudaHostGetDevicePointer");
    } else {
        rc = fail(AB_ERR_INVALID, "ab_alloc: memory kind %d", kind);
    }
    if (rc) { cudaGetLastError(); delete b; return note_loss(d, rc); }
    d->live.fetch_add(1);
    *out = b;
    return AB_OK;
}

int ab_block_import(ab_device *d, void *device_ptr, size_t bytes, ab_block **out)
{
    if (!out || !device_ptr || bytes == 0) return fail(AB_ERR_INVALID, "ab_block_import: NULL or empty");
    int rc = set_device(d);
    if (rc) return rc;
    cudaPointerAttributes at{};
    rc = check_cuda(cudaPointerGetAttributes(&at, device_ptr), "ab_block_import");
    if (rc) return rc;
    if (at.type != cudaMemoryTypeDevice || at.device != d->ordinal)
        return fail(AB_ERR_INVALID, "ab_block_import: the address is not device memory of device %d", d->ordinal);
    ab_block *b = new (std::nothrow) ab_block();
    if (!b) return fail(AB_ERR_OOM, "ab_block_import: host allocation failed");
    b->dev = d; b->kind = AB_MEMORY_DEVICE; b->size = bytes; b->dptr = device_ptr; b->hptr = nullptr; b->borrowed = true;
    d->live.fetch_add(1);
    *out = b;
    return AB_OK;
}

void *ab_block_bytes(ab_block *b) { return b ? b->hptr : nullptr; }
void *ab_block_device_ptr(ab_block *b) { return b ? b->dptr : nullptr; }
size_t ab_block_size(ab_block *b) { return b ? b->size : 0; }

int ab_block_write(ab_block *b, size_t off, const void *src, size_t n)
{
    if (!b || (!src && n)) return fail(AB_ERR_INVALID, "ab_block_write: NULL argument");
    if (off + n > b->size) return fail(AB_ERR_INVALID, "ab_block_write: %zu + %zu past %zu bytes", off, n, b->size);
    int rc = set_device(b->dev);
    if (rc) return rc;
    if (n == 0) return AB_OK;
    if (b->hptr) { cudaStreamSynchronize(b->dev->stream); memcpy(static_cast<char *>(b->hptr) + off, src, n); return AB_OK; }
    rc = check_cuda(cudaMemcpyAsync(static_cast<char *>(b->dptr) + off, src, n, cudaMemcpyHostToDevice, b->dev->stream), "ab_block_write");
    if (!rc) rc = check_cuda(cudaStreamSynchronize(b->dev->stream), "ab_block_write");
    return note_loss(b->dev, rc);
}

int ab_block_read(ab_block *b, size_t off, void *dst, size_t n)
{
    if (!b || (!dst && n)) return fail(AB_ERR_INVALID, "ab_block_read: NULL argument");
    if (off + n > b->size) return fail(AB_ERR_INVALID, "ab_block_read: %zu + %zu past %zu bytes", off, n, b->size);
    int rc = set_device(b->dev);
    if (rc) return rc;
    if (n == 0) return AB_OK;
    if (b->hptr) { cudaStreamSynchronize(b->dev->stream); memcpy(dst, static_cast<char *>(b->hptr) + off, n); return AB_OK; }
    rc = check_cuda(cudaMemcpyAsync(dst, static_cast<char *>(b->dptr) + off, n, cudaMemcpyDeviceToHost, b->dev->stream), "ab_block_read");
    if (!rc) rc = check_cuda(cudaStreamSynchronize(b->dev->stream), "ab_block_read");
    return note_loss(b->dev, rc);
}

int ab_block_free(ab_block *b)
{
    if (!b) return AB_OK;
    ab_device *d = b->dev;
    // an executable that resolved pointers from this block would read freed memory on its next
    // submission: children are freed before parents (the reference's pools refuse the same way)
    if (b->users.load() > 0)
        return ab::fail(AB_ERR_BUSY, "ab_block_free: %d live executable(s) still name this block; close "
                        "them (or rebind their slots) first", b->users.load());
    if (!d->lost.load() && cudaSetDevice(d->ordinal) == cudaSuccess) {
        cudaStreamSynchronize(d->stream);
        if (b->borrowed) { /* the caller's memory */ }
        else if (b->hptr) cudaFreeHost(b->hptr);
        else cudaFree(b->dptr);
    }
    d->live.fetch_sub(1);
    delete b;
    return AB_OK;
}

int ab_supports_kernel(ab_device *d, const char *name, const char *digest)
{
    (void)d; (void)digest;
    if (!find_kernel(name))
        return fail(AB_ERR_UNSUPPORTED, "no sm_100a kernel is registered under the name \"%s\"",
                    name ? name : "(null)");
    return AB_OK;
}

// ------------------------------------------------------------------------------------------------
// executable / fence
// ------------------------------------------------------------------------------------------------
int ab_compile(ab_device *d, const ab_plan *plan, ab_exec **out)
{
    if (!plan || !out) return fail(AB_ERR_INVALID, "ab_compile: NULL argument");
    int rc = set_device(d);
    if (rc) return rc;
    if (plan->n_nodes < 0 || plan->n_slots < 0 || (plan->n_nodes && !plan->nodes))
        return fail(AB_ERR_INVALID, "ab_compile: %d nodes, %d slots", plan->n_nodes, plan->n_slots);
    ab_exec *e = new (std::nothrow) ab_exec();
    if (!e) return fail(AB_ERR_OOM, "ab_compile: host allocation failed");
    e->dev = d;
    e->timings = plan->collect_timings != 0;
    e->max_in_flight = plan->max_in_flight > 1 ? plan->max_in_flight : 1;
    e->slots.resize((size_t)plan->n_slots);
    e->slot_set.assign((size_t)plan->n_slots, false);
    auto bail = [&](int code) { for (auto *in : e->inst) free_instance(in); delete e; return code; };

    size_t ws_max = 0;
    for (int n = 0; n < plan->n_nodes; n++) {
        const ab_node &src = plan->nodes[n];
        Node nd;
        nd.op = src.op;
        if (src.n_bindings < 0 || (src.n_bindings && !src.bindings))
            return bail(fail(AB_ERR_INVALID, "node %d: %d bindings", n, src.n_bindings));
        nd.bind.assign(src.bindings, src.bindings + src.n_bindings);
        for (int i = 0; i < src.n_bindings; i++)
            if (!nd.bind[i].block && (nd.bind[i].slot == 0 || (int)nd.bind[i].slot > plan->n_slots))
                return bail(fail(AB_ERR_INVALID, "node %d binding %d names slot %u of %d", n, i,
                                 nd.bind[i].slot, plan->n_slots));
        if (src.op == AB_OP_DISPATCH) {
            const KernelEntry *k = find_kernel(src.kernel);
            if (!k)
                return bail(fail(AB_ERR_UNSUPPORTED, "node %d: no sm_100a kernel is registered under "
                                 "the name \"%s\"; this backend has no CPU fallback", n,
                                 src.kernel ? src.kernel : "(null)"));
            nd.kernel = src.kernel;
            if (src.n_bindings != k->n_bindings)
                return bail(fail(AB_ERR_INVALID, "node %d: %s takes %d bindings and %d were given", n,
                                 k->name, k->n_bindings, src.n_bindings));
            if (k->uniform_bytes && (!src.uniform || src.uniform_bytes < k->uniform_bytes))
                return bail(fail(AB_ERR_INVALID, "node %d: %s takes a %zu-byte uniform block", n,
                                 k->name, k->uniform_bytes));
            if (src.uniform && src.uniform_bytes)
                nd.uniform.assign(static_cast<const uint8_t *>(src.uniform),
                                  static_cast<const uint8_t *>(src.uniform) + src.uniform_bytes);
            nd.lens.resize((size_t)src.n_bindings);
            for (int i = 0; i < src.n_bindings; i++) {
                size_t eb = elem_bytes_of(k->name, i);
                if (nd.bind[i].size % eb)
                    return bail(fail(AB_ERR_INVALID, "node %d binding %d of %s is %llu bytes, not a "
                                     "whole number of %zu-byte elements", n, i, k->name,
                                     (unsigned long long)nd.bind[i].size, eb));
                if (nd.bind[i].offset % 256)
                    return bail(fail(AB_ERR_INVALID, "node %d binding %d of %s starts at byte %llu; "
                                     "storage offsets are multiples of 256", n, i, k->name,
                                     (unsigned long long)nd.bind[i].offset));
                nd.lens[i] = (uint32_t)(nd.bind[i].size / eb);
            }
            Launch q{nullptr, nullptr, nd.lens.data(), src.n_bindings,
                     nd.uniform.empty() ? nullptr : nd.uniform.data(), nd.uniform.size(), nullptr, 0, true, 0};
            rc = k->fn(q);
            if (rc) return bail(rc);
            nd.ws = q.ws_need;
            ws_max = std::max(ws_max, nd.ws);
        } else if (src.op == AB_OP_COPY) {
            if (src.n_bindings != 2) return bail(fail(AB_ERR_INVALID, "node %d: a copy has a source and a destination", n));
        } else if (src.op == AB_OP_HOST_WRITE) {
            if (src.n_bindings != 1 || !src.payload || src.payload_bytes == 0)
                return bail(fail(AB_ERR_INVALID, "node %d: a host write has one destination and a payload", n));
            nd.payload_bytes = (size_t)src.payload_bytes;
            nd.payload.assign(static_cast<const uint8_t *>(src.payload),
                              static_cast<const uint8_t *>(src.payload) + nd.payload_bytes);
        } else {
            return bail(fail(AB_ERR_UNSUPPORTED, "node %d: op %d; this is a compute-only backend", n, src.op));
        }
        e->nodes.push_back(std::move(nd));
    }
    e->ws_bytes = ws_max;
    Instance *first = nullptr;
    rc = new_instance(e, &first);
    if (rc) return bail(rc);
    e->inst.push_back(first);
    for (auto &nd : e->nodes)
        for (auto &op : nd.bind)
            if (op.block) { op.block->users.fetch_add(1); e->held.push_back(op.block); }
    d->live.fetch_add(1);
    *out = e;
    return AB_OK;
}

int ab_exec_rebind(ab_exec *e, const ab_slot_binding *b, int n)
{
    if (!e || (n && !b) || n < 0) return fail(AB_ERR_INVALID, "ab_exec_rebind: NULL argument");
    std::lock_guard<std::mutex> lk(e->mu);
    // one submission at a time: the executable is busy until its fence is waited for.  Several in
    // flight: a rebind applies to the submissions that follow (those in flight own their lowering).
    if (e->max_in_flight == 1 && e->busy_count()) return fail(AB_ERR_BUSY, "ab_exec_rebind: a submission is in flight");
    for (int i = 0; i < n; i++) {       // validate everything first: all or nothing
        if (b[i].slot == 0 || b[i].slot > e->slots.size())
            return fail(AB_ERR_INVALID, "ab_exec_rebind: slot %u of %zu", b[i].slot, e->slots.size());
        if (!b[i].block) return fail(AB_ERR_INVALID, "ab_exec_rebind: slot %u has no block", b[i].slot);
        if (b[i].block->dev != e->dev) return fail(AB_ERR_INVALID, "ab_exec_rebind: slot %u's block belongs to another device", b[i].slot);
        if (b[i].offset % 256) return fail(AB_ERR_INVALID, "ab_exec_rebind: slot %u offset %llu is not a multiple of 256", b[i].slot, (unsigned long long)b[i].offset);
    }
    std::vector<ab_slot_binding> saved = e->slots;
    std::vector<bool> saved_set = e->slot_set;
    for (int i = 0; i < n; i++) { e->slots[b[i].slot - 1] = b[i]; e->slot_set[b[i].slot - 1] = true; }
    bool all = std::all_of(e->slot_set.begin(), e->slot_set.end(), [](bool x) { return x; });
    if (all) {
        int rc = resolve_all(e);
        if (rc) { e->slots = saved; e->slot_set = saved_set; return rc; }
    }
    for (int i = 0; i < n; i++) {
        const size_t at = b[i].slot - 1;
        b[i].block->users.fetch_add(1);
        if (saved_set[at] && saved[at].block) saved[at].block->users.fetch_sub(1);
        saved[at] = b[i];                    // a slot named twice in one call: count the last one
        saved_set[at] = true;
    }
    e->version++;
    return AB_OK;
}

int ab_exec_set_uniform(ab_exec *e, int node, int index, const void *bytes, size_t n)
{
    if (!e || !bytes) return fail(AB_ERR_INVALID, "ab_exec_set_uniform: NULL argument");
    std::lock_guard<std::mutex> lk(e->mu);
    if (e->max_in_flight == 1 && e->busy_count()) return fail(AB_ERR_BUSY, "ab_exec_set_uniform: a submission is in flight");
    if (node < 0 || node >= (int)e->nodes.size() || e->nodes[node].op != AB_OP_DISPATCH || index != 0)
        return fail(AB_ERR_INVALID, "ab_exec_set_uniform: node %d block %d", node, index);
    Node &nd = e->nodes[node];
    if (n != nd.uniform.size())
        return fail(AB_ERR_INVALID, "ab_exec_set_uniform: node %d's block is %zu bytes, given %zu", node, nd.uniform.size(), n);
    memcpy(nd.uniform.data(), bytes, n);
    e->version++;
    return AB_OK;
}

int ab_exec_set_payload(ab_exec *e, int node, const void *bytes, size_t n)
{
    if (!e || !bytes) return fail(AB_ERR_INVALID, "ab_exec_set_payload: NULL argument");
    std::lock_guard<std::mutex> lk(e->mu);
    if (e->max_in_flight == 1 && e->busy_count()) return fail(AB_ERR_BUSY, "ab_exec_set_payload: a submission is in flight");
    if (node < 0 || node >= (int)e->nodes.size() || e->nodes[node].op != AB_OP_HOST_WRITE)
        return fail(AB_ERR_INVALID, "ab_exec_set_payload: node %d is not a host write", node);
    Node &nd = e->nodes[node];
    if (n != nd.payload_bytes)
        return fail(AB_ERR_INVALID, "ab_exec_set_payload: node %d's payload is %zu bytes, given %zu", node, nd.payload_bytes, n);
    memcpy(nd.payload.data(), bytes, n);      // copied into the submission's own staging buffer at submit
    return AB_OK;
}

int ab_exec_submit(ab_exec *e, ab_fence **out)
{
    if (!e || !out) return fail(AB_ERR_INVALID, "ab_exec_submit: NULL argument");
    ab_device *d = e->dev;
    int rc = set_device(d);
    if (rc) return rc;
    std::lock_guard<std::mutex> lk(e->mu);
    // an instance nobody is using; else a spare lowered now, up to max_in_flight of them
    Instance *in = nullptr;
    for (auto *cand : e->inst) if (!cand->busy.load()) { in = cand; break; }
    if (!in) {
        if ((int)e->inst.size() >= e->max_in_flight)
            return fail(AB_ERR_BUSY, e->max_in_flight == 1
                        ? "ab_exec_submit: the previous submission has not been waited for; one submission is in "
                          "flight per executable (compile with max_in_flight for more)"
                        : "ab_exec_submit: all %d instances of the executable are in flight", e->max_in_flight);
        rc = new_instance(e, &in);
        if (rc) return rc;
        e->inst.push_back(in);
    }
    in->busy.store(1);
    auto release = [&](int code) { in->busy.store(0); return note_loss(d, code); };
    if (!std::all_of(e->slot_set.begin(), e->slot_set.end(), [](bool x) { return x; }))
        return release(fail(AB_ERR_INVALID, "ab_exec_submit: a slot is unbound"));
    for (auto &nd : e->nodes)
        if (nd.ptrs.size() != nd.bind.size()) { rc = resolve_all(e); if (rc) return release(rc); break; }

    int seq = d->submissions.fetch_add(1) + 1;
    ab_fence *f = new (std::nothrow) ab_fence();
    if (!f) return release(fail(AB_ERR_OOM, "ab_exec_submit: host allocation failed"));
    f->dev = d; f->exec = e; f->inst = in; f->timed = e->timings; f->start = in->ev_start; f->done = in->ev_done;
    f->injected = 0;
    if (d->lose_at > 0 && seq >= d->lose_at) {      // host-side injection: nothing touches the GPU
        d->lost.store(1);
        f->injected = 1;
        *out = f;
        return AB_OK;
    }
    // this submission's payloads: the instance is idle, so its staging buffers are free to write
    for (size_t n = 0; n < e->nodes.size(); n++)
        if (e->nodes[n].op == AB_OP_HOST_WRITE) memcpy(in->staging[n], e->nodes[n].payload.data(), e->nodes[n].payload_bytes);
    if (f->timed) cudaEventRecord(f->start, d->stream);
    if (d->use_graphs) {
        if (in->graph_version != e->version || !in->graph) {
            if (in->graph) { cudaGraphExecDestroy(in->graph); in->graph = nullptr; }
            cudaGraph_t g = nullptr;
            rc = check_cuda(cudaStreamBeginCapture(d->stream, cudaStreamCaptureModeThreadLocal), "graph capture");
            if (!rc) {
                int rn = run_nodes(e, in, d->stream);
                cudaError_t ce = cudaStreamEndCapture(d->stream, &g);
                rc = rn ? rn : check_cuda(ce, "graph capture");
            }
            if (!rc) rc = check_cuda(cudaGraphInstantiate(&in->graph, g, 0), "graph instantiate");
            if (g) cudaGraphDestroy(g);
            if (rc) { delete f; return release(rc); }
            in->graph_version = e->version;
        }
        rc = check_cuda(cudaGraphLaunch(in->graph, d->stream), "graph launch");
    } else {
        rc = run_nodes(e, in, d->stream);
    }
    if (rc) { delete f; return release(rc); }
    rc = check_cuda(cudaEventRecord(f->done, d->stream), "fence");
    if (rc) { delete f; return release(rc); }
    *out = f;
    return AB_OK;
}

// The submission is over for the host: its instance takes the next one.
static void fence_release(ab_fence *f)
{
    if (f->inst) f->inst->busy.store(0);
    f->inst = nullptr;
    f->exec = nullptr;
}

int ab_fence_wait(ab_fence *f)
{
    if (!f) return fail(AB_ERR_INVALID, "ab_fence_wait: fence is NULL");
    if (f->injected) { fence_release(f); return fail(AB_ERR_DEVICE_LOST, "device lost (injected at this submission)"); }
    int rc = check_cuda(cudaEventSynchronize(f->done), "ab_fence_wait");   // needs no current context
    fence_release(f);
    // every outstanding fence reports a loss once the device is lost (internal/driver/plan.go:374-391)
    if (rc == AB_OK && f->dev && f->dev->lost.load())
        return fail(AB_ERR_DEVICE_LOST, "ab_fence_wait: the device was lost");
    return note_loss(f->dev, rc);
}

int ab_fence_done(ab_fence *f)
{
    if (!f) return fail(AB_ERR_INVALID, "ab_fence_done: fence is NULL");
    if (f->dev && f->dev->lost.load() && !f->injected)
        return fail(AB_ERR_DEVICE_LOST, "ab_fence_done: the device was lost");
    // a caller may learn of completion here and never wait: the executable is free again
    auto finished = [&]() { fence_release(f); return 1; };
    if (f->injected) return finished();
    cudaError_t e = cudaEventQuery(f->done);
    if (e == cudaSuccess) return finished();
    if (e == cudaErrorNotReady) return 0;
    return note_loss(f->dev, check_cuda(e, "ab_fence_done"));
}

uint64_t ab_fence_elapsed_ns(ab_fence *f)
{
    if (!f || !f->timed || f->injected) return 0;
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, f->start, f->done) != cudaSuccess) { cudaGetLastError(); return 0; }
    return (uint64_t)((double)ms * 1e6);
}

void ab_fence_free(ab_fence *f)
{
    if (!f) return;
    if (f->inst) {                          // freed unwaited: wait here so the instance is not stuck busy
        if (!f->injected) cudaEventSynchronize(f->done);
        fence_release(f);
    }
    delete f;
}

int ab_exec_close(ab_exec *e)
{
    if (!e) return AB_OK;
    ab_device *d = e->dev;
    if (!d->lost.load() && cudaSetDevice(d->ordinal) == cudaSuccess) {
        cudaStreamSynchronize(d->stream);
        for (auto *in : e->inst) free_instance(in);
    } else {
        for (auto *in : e->inst) delete in;
    }
    e->inst.clear();
    for (ab_block *blk : e->held) blk->users.fetch_sub(1);
    for (size_t i = 0; i < e->slots.size(); i++)
        if (e->slot_set[i] && e->slots[i].block) e->slots[i].block->users.fetch_sub(1);
    d->live.fetch_sub(1);
    delete e;
    return AB_OK;
}

// ------------------------------------------------------------------------------------------------
// host side: quant.Int4Quantize and friends (quant/int4.go:71-175), parallel over groups
// ------------------------------------------------------------------------------------------------
static void quantize_groups(const float *w, size_t n, uint32_t *packed, uint16_t *scales,
                            uint16_t *zeros, size_t g0, size_t g1)
{
    for (size_t g = g0; g < g1; g++) {
        const size_t lo = g * 128, hi = std::min(lo + 128, n);
        float mn = w[lo], mx = w[lo];
        for (size_t i = lo; i < hi; i++) { if (w[i] < mn) mn = w[i]; if (w[i] > mx) mx = w[i]; }
        for (size_t i = lo / 8; i < (hi + 7) / 8; i++) packed[i] = 0;
        if (mx == mn) { scales[g] = f32_to_f16_ref(0.f); zeros[g] = f32_to_f16_ref(mn); continue; }
        scales[g] = f32_to_f16_ref((mx - mn) / 15.0f);
        const float s16 = f16_bits_to_f32(scales[g]);
        if (s16 == 0.f) { zeros[g] = f32_to_f16_ref(mn); continue; }
        zeros[g] = f32_to_f16_ref(-mn / s16);
        const double z16 = (double)f16_bits_to_f32(zeros[g]);
        for (size_t i = lo; i < hi; i++) {
            double q = nearbyint((double)w[i] / (double)s16 + z16);
            q = q > 15.0 ? 15.0 : (q < 0.0 ? 0.0 : q);
            packed[i / 8] |= (uint32_t)q << (4 * (i % 8));
        }
    }
}

int ab_int4_quantize(const float *w, size_t n, uint32_t *packed, uint16_t *scales, uint16_t *zeros)
{
    if (n && (!w || !packed || !scales || !zeros)) return fail(AB_ERR_INVALID, "ab_int4_quantize: NULL argument");
    const size_t groups = (n + 127) / 128;
    unsigned hw = std::thread::hardware_concurrency();
    size_t nt = std::max<size_t>(1, std::min<size_t>(hw ? hw : 1, groups / 256));
    if (nt <= 1) { quantize_groups(w, n, packed, scales, zeros, 0, groups); return AB_OK; }
    std::vector<std::thread> pool;
    const size_t per = (groups + nt - 1) / nt;
    for (size_t t = 0; t < nt; t++) {
        size_t g0 = t * per, g1 = std::min(groups, g0 + per);
        if (g0 >= g1) break;
        pool.emplace_back(quantize_groups, w, n, packed, scales, zeros, g0, g1);
    }
    for (auto &th : pool) th.join();
    return AB_OK;
}

uint32_t ab_int4_nibble(const uint32_t *packed, size_t i) { return (packed[i / 8] >> (4 * (i % 8))) & 0xFu; }

int ab_int4_dequantize(const uint32_t *packed, const uint16_t *scales, const uint16_t *zeros,
                       size_t n, float *out)
{
    if (n && (!packed || !scales || !zeros || !out)) return fail(AB_ERR_INVALID, "ab_int4_dequantize: NULL argument");
    for (size_t i = 0; i < n; i++) {
        const float s = f16_bits_to_f32(scales[i / 128]), z = f16_bits_to_f32(zeros[i / 128]);
        out[i] = s == 0.f ? z : ((float)ab_int4_nibble(packed, i) - z) * s;
    }
    return AB_OK;
}

// quant.Int8Quantize / Int8Dequantize (quant/quant.go:60-134): one f16 scale per 32 weights, quants
// in [-127, 127], quantized against the scale as the kernel reads it back
int ab_int8_quantize(const float *w, size_t n, int8_t *quants, uint16_t *scales)
{
    if (n && (!w || !quants || !scales)) return fail(AB_ERR_INVALID, "ab_int8_quantize: NULL argument");
    const size_t blocks = (n + 31) / 32;
    for (size_t b = 0; b < blocks; b++) {
        const size_t lo = b * 32, hi = std::min(lo + 32, n);
        float peak = 0.f;
        for (size_t i = lo; i < hi; i++) peak = std::max(peak, std::fabs(w[i]));
        for (size_t i = lo; i < hi; i++) quants[i] = 0;
        if (peak == 0.f) { scales[b] = f32_to_f16_ref(0.f); continue; }
        scales[b] = f32_to_f16_ref(peak / 127.0f);
        const float s16 = f16_bits_to_f32(scales[b]);
        if (s16 == 0.f) continue;                       // the scale underflowed f16: zeros reconstruct
        for (size_t i = lo; i < hi; i++) {
            double q = nearbyint((double)w[i] / (double)s16);
            q = q > 127.0 ? 127.0 : (q < -127.0 ? -127.0 : q);
            quants[i] = (int8_t)q;
        }
    }
    return AB_OK;
}

int ab_int8_dequantize(const int8_t *quants, const uint16_t *scales, size_t n, float *out)
{
    if (n && (!quants || !scales || !out)) return fail(AB_ERR_INVALID, "ab_int8_dequantize: NULL argument");
    for (size_t i = 0; i < n; i++) out[i] = (float)quants[i] * f16_bits_to_f32(scales[i / 32]);
    return AB_OK;
}

uint16_t ab_f32_to_f16(const float *x) { return x ? f32_to_f16_ref(*x) : 0; }
void ab_f16_to_f32(uint16_t h, float *out) { if (out) *out = f16_bits_to_f32(h); }

// ------------------------------------------------------------------------------------------------
// tensor.BlockPool (tensor/blockpool.go:46-133)
// ------------------------------------------------------------------------------------------------
}  // extern "C"

struct ab_blockpool {
    int block;
    int total;
    std::mutex mu;
    std::vector<uint32_t> free_list;
};

extern "C" {

int ab_blockpool_new(int blocks, int per, ab_blockpool **out)
{
    if (!out) return fail(AB_ERR_INVALID, "ab_blockpool_new: out is NULL");
    if (blocks <= 0 || per <= 0) return fail(AB_ERR_INVALID, "a pool of %d blocks of %d positions", blocks, per);
    ab_blockpool *p = new (std::nothrow) ab_blockpool();
    if (!p) return fail(AB_ERR_OOM, "ab_blockpool_new: host allocation failed");
    p->block = per; p->total = blocks;
    p->free_list.resize((size_t)blocks);
    for (int i = 0; i < blocks; i++) p->free_list[(size_t)i] = (uint32_t)(blocks - 1 - i);
    *out = p;
    return AB_OK;
}

void ab_blockpool_close(ab_blockpool *p) { delete p; }
int ab_blockpool_block_size(ab_blockpool *p) { return p ? p->block : 0; }
int ab_blockpool_available(ab_blockpool *p)
{
    if (!p) return 0;
    std::lock_guard<std::mutex> lk(p->mu);
    return (int)p->free_list.size();
}

int ab_blockpool_grow(ab_blockpool *p, uint32_t *pages, int n_pages, int n)
{
    if (!p || n_pages < 0) return fail(AB_ERR_INVALID, "ab_blockpool_grow: bad argument");
    if (n < 0) return fail(AB_ERR_INVALID, "%d positions", n);
    const int want = (int)(((int64_t)n + p->block - 1) / p->block);
    if (want <= n_pages) return n_pages;
    if (!pages) return fail(AB_ERR_INVALID, "ab_blockpool_grow: pages is NULL");
    std::lock_guard<std::mutex> lk(p->mu);
    const int need = want - n_pages;
    if ((size_t)need > p->free_list.size())
        return fail(AB_ERR_OOM, "%d positions need %d more block(s) and %zu are free; the pool does "
                    "not evict, because choosing which sequence to truncate is a policy this cannot "
                    "make for you", n, need, p->free_list.size());
    // the new pages are the tail of the free list, in list order; earlier pages never move
    std::copy(p->free_list.end() - need, p->free_list.end(), pages + n_pages);
    p->free_list.resize(p->free_list.size() - (size_t)need);
    return want;
}

int ab_blockpool_free(ab_blockpool *p, const uint32_t *pages, int n_pages)
{
    if (!p || n_pages < 0 || (n_pages && !pages)) return fail(AB_ERR_INVALID, "ab_blockpool_free: bad argument");
    std::lock_guard<std::mutex> lk(p->mu);
    std::vector<bool> held((size_t)p->total, false);
    for (uint32_t f : p->free_list) held[f] = true;
    int bad = 0;
    uint32_t first_bad = 0;
    for (int i = 0; i < n_pages; i++) {
        const uint32_t pg = pages[i];
        if (pg >= (uint32_t)p->total || held[pg]) { if (!bad) first_bad = pg; bad++; continue; }
        held[pg] = true;
        p->free_list.push_back(pg);
    }
    if (bad) return fail(AB_ERR_INVALID, "block %u is already free (%d such block(s))", first_bad, bad);
    return AB_OK;
}

int ab_blockpool_positions(ab_blockpool *p, int n_pages) { return p ? n_pages * p->block : 0; }

int ab_int4_column_split(uint32_t n_cols, int parts, int rank, uint32_t *begin, uint32_t *end)
{
    if (!begin || !end || parts <= 0 || rank < 0 || rank >= parts)
        return fail(AB_ERR_INVALID, "ab_int4_column_split: rank %d of %d", rank, parts);
    if (n_cols % 128)
        return fail(AB_ERR_INVALID, "ab_int4_column_split: %u columns is not a whole number of "
                    "128-column groups, so no split keeps the packing bit-identical", n_cols);
    const uint32_t groups = n_cols / 128, base = groups / (uint32_t)parts, extra = groups % (uint32_t)parts;
    const uint32_t r = (uint32_t)rank;
    const uint32_t g0 = r * base + std::min(r, extra);
    const uint32_t g1 = g0 + base + (r < extra ? 1u : 0u);
    *begin = g0 * 128;
    *end = g1 * 128;
    return AB_OK;
}

}  // extern "C"
