// ab_group: N devices of one process opened together for the tensor-parallel step, so that a host
// without a symmetric-memory allocator of its own (the Go backend: one process, one goroutine per
// device or one thread driving all of them) gets what the one-shot all-reduce needs: peer access
// between every pair, one peer buffer and one state block per device, a stream per device and the
// table of buffer addresses in rank order.  accel is single-device (specs/060-cuda-bringup.md:261-267
// leaves multi-device to a later layer): no reference counterpart.
//
// Memory is plain cudaMalloc with peer access enabled (no multicast objects, no IPC: one process).
// Every rank's kernel runs on a GPU of its own; the calls only enqueue, so one host thread can
// issue a collective for all ranks in turn.
#include <new>

#include "common.cuh"

struct ab_group {
    int n;
    int ord[8];
    void *buf[8];
    void *state[8];
    cudaStream_t stream[8];
    uint32_t capacity;
};

namespace {
struct DeviceGuard {
    int prev = -1;
    DeviceGuard() { if (cudaGetDevice(&prev) != cudaSuccess) { cudaGetLastError(); prev = -1; } }
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};
}  // namespace

extern "C" {

AB_API int ab_group_close(ab_group *g)
{
    if (!g) return AB_OK;
    DeviceGuard guard;
    for (int i = 0; i < g->n; i++) {
        if (cudaSetDevice(g->ord[i]) != cudaSuccess) { cudaGetLastError(); continue; }
        if (g->stream[i]) { cudaStreamSynchronize(g->stream[i]); cudaStreamDestroy(g->stream[i]); }
        if (g->buf[i]) cudaFree(g->buf[i]);
        if (g->state[i]) cudaFree(g->state[i]);
    }
    delete g;
    return AB_OK;
}

AB_API int ab_group_open(const int *ordinals, int n, uint32_t capacity_floats, ab_group **out)
{
    using namespace ab;
    if (!ordinals || !out || n < 1 || n > 8 || capacity_floats == 0)
        return fail(AB_ERR_INVALID, "ab_group_open: %d devices (1 to 8), capacity %u", n, capacity_floats);
    for (int i = 0; i < n; i++)
        for (int j = 0; j < i; j++)
            if (ordinals[i] == ordinals[j])
                return fail(AB_ERR_INVALID, "ab_group_open: device %d is named twice; every rank needs a GPU of its own "
                            "(the ranks' kernels wait for one another)", ordinals[i]);
    DeviceGuard guard;
    ab_group *g = new (std::nothrow) ab_group();
    if (!g) return fail(AB_ERR_OOM, "ab_group_open: host allocation failed");
    g->n = n;
    g->capacity = capacity_floats;
    for (int i = 0; i < n; i++) { g->ord[i] = ordinals[i]; g->buf[i] = g->state[i] = nullptr; g->stream[i] = nullptr; }
    auto bail = [&](int rc) { ab_group_close(g); return rc; };
    for (int i = 0; i < n; i++) {
        int rc = check_cuda(cudaSetDevice(g->ord[i]), "ab_group_open: cudaSetDevice");
        if (rc) return bail(rc);
        for (int j = 0; j < n; j++) {
            if (j == i) continue;
            int can = 0;
            rc = check_cuda(cudaDeviceCanAccessPeer(&can, g->ord[i], g->ord[j]), "cudaDeviceCanAccessPeer");
            if (rc) return bail(rc);
            if (!can)
                return bail(fail(AB_ERR_UNSUPPORTED, "ab_group_open: device %d cannot address device %d's memory", g->ord[i],
                                 g->ord[j]));
            cudaError_t e = cudaDeviceEnablePeerAccess(g->ord[j], 0);
            if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
            else if (e != cudaSuccess) return bail(check_cuda(e, "cudaDeviceEnablePeerAccess"));
        }
        const size_t bb = ab_peer_allreduce_buffer_bytes(capacity_floats), sb = ab_peer_allreduce_state_bytes();
        rc = check_cuda(cudaMalloc(&g->buf[i], bb), "ab_group_open: peer buffer");
        if (!rc) rc = check_cuda(cudaMemset(g->buf[i], 0, bb), "ab_group_open: peer buffer");
        if (!rc) rc = check_cuda(cudaMalloc(&g->state[i], sb), "ab_group_open: state");
        if (!rc) rc = check_cuda(cudaMemset(g->state[i], 0, sb), "ab_group_open: state");
        if (!rc) rc = check_cuda(cudaStreamCreateWithFlags(&g->stream[i], cudaStreamNonBlocking), "ab_group_open: stream");
        if (!rc) rc = check_cuda(cudaDeviceSynchronize(), "ab_group_open");
        if (rc) { cudaGetLastError(); return bail(rc); }
    }
    *out = g;
    return AB_OK;
}

AB_API int ab_group_size(const ab_group *g) { return g ? g->n : 0; }
AB_API int ab_group_ordinal(const ab_group *g, int rank) { return (g && rank >= 0 && rank < g->n) ? g->ord[rank] : -1; }
AB_API void *ab_group_buffer(const ab_group *g, int rank) { return (g && rank >= 0 && rank < g->n) ? g->buf[rank] : nullptr; }
AB_API void *ab_group_state(const ab_group *g, int rank) { return (g && rank >= 0 && rank < g->n) ? g->state[rank] : nullptr; }
AB_API void *ab_group_stream(const ab_group *g, int rank) { return (g && rank >= 0 && rank < g->n) ? g->stream[rank] : nullptr; }
AB_API void *const *ab_group_peer_table(const ab_group *g) { return g ? g->buf : nullptr; }

AB_API int ab_group_all_reduce_f32(ab_group *g, const float *const *in, float *const *out, uint32_t n)
{
    using namespace ab;
    if (!g || !in || !out) return fail(AB_ERR_INVALID, "ab_group_all_reduce_f32: NULL argument");
    DeviceGuard guard;
    for (int r = 0; r < g->n; r++) {
        int rc = check_cuda(cudaSetDevice(g->ord[r]), "ab_group_all_reduce_f32: cudaSetDevice");
        if (rc) return rc;
        rc = ab_peer_allreduce_f32(g->stream[r], g->buf, g->state[r], r, g->n, in[r], out[r], n, g->capacity);
        if (rc) return rc;
    }
    return AB_OK;
}

AB_API int ab_group_synchronize(ab_group *g)
{
    using namespace ab;
    if (!g) return fail(AB_ERR_INVALID, "ab_group_synchronize: NULL group");
    DeviceGuard guard;
    int first = AB_OK;
    for (int r = 0; r < g->n; r++) {
        int rc = check_cuda(cudaSetDevice(g->ord[r]), "ab_group_synchronize: cudaSetDevice");
        if (!rc) rc = check_cuda(cudaStreamSynchronize(g->stream[r]), "ab_group_synchronize");
        if (!rc) rc = ab_peer_allreduce_error(g->state[r], nullptr);
        if (rc && !first) first = rc;
    }
    return first;
}

}  // extern "C"
