// One-shot push all-reduce over peer memory (NVLink / NVSwitch), for the small f32 vectors a
// tensor- or expert-parallel decode step sums across GPUs (a few KB to a few hundred KB), where a
// library collective's fixed cost is several times the matvec it follows.
//
// Every rank owns an arena (one cudaMalloc block, shared with the other ranks of the box through
// CUDA IPC) and carves it into channels at the same offsets on every rank; the channel's layout
// and the per-element protocol (a value travels with its own arrival count in one 8-byte store)
// are in fk_comm.cuh.  The kernel here is the standalone form; the row-split matvec runs the same
// two steps in its epilogue.
//
// Every wait is bounded in time (the caller's limit, two seconds by default) and raises the
// context's error word (60) instead of hanging; the call then returns garbage and the host sees
// the word.
#include "fk_comm.cuh"

#include <string.h>

namespace {

constexpr int AR_THREADS = 256, AR_PER_THREAD = 4;

__global__ void __launch_bounds__(AR_THREADS) allreduce_kernel(FkArChannel ch, const float* __restrict__ src, int n, int accumulate_into,
                                                                float* __restrict__ dst, int* __restrict__ err) {
    asm volatile("griddepcontrol.wait;" ::: "memory");            // src is the previous kernel's output
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int i0 = blockIdx.x * AR_THREADS * AR_PER_THREAD + threadIdx.x;
    float v[AR_PER_THREAD];
    unsigned t[AR_PER_THREAD];
#pragma unroll
    for (int j = 0; j < AR_PER_THREAD; j++) {
        const int i = i0 + j * AR_THREADS;
        if (i < n) {
            v[j] = src[i];
            t[j] = fk_ar_send(ch, i, v[j]);
        }
    }
#pragma unroll
    for (int j = 0; j < AR_PER_THREAD; j++) {
        const int i = i0 + j * AR_THREADS;
        if (i < n) {
            const float s = fk_ar_recv(ch, i, t[j], v[j], err);
            dst[i] = accumulate_into ? dst[i] + s : s;
        }
    }
}

}  // namespace

FK_EXPORT int fk_comm_create(fk_ctx* ctx, size_t arena_bytes, int rank, int world, uint8_t* handle_out, fk_comm** out) {
    if (!ctx || !out || !handle_out) return fk_fail(FK_INVALID, "comm_create: null argument");
    if (world < 1 || world > FK_AR_MAX_WORLD || rank < 0 || rank >= world) return fk_fail(FK_INVALID, "comm_create: rank %d of %d (at most %d)", rank, world, FK_AR_MAX_WORLD);
    FkDeviceGuard g(ctx->device);
    fk_comm* c = new fk_comm();
    c->ctx = ctx;
    c->rank = rank;
    c->world = world;
    c->bytes = (arena_bytes + 255) & ~(size_t)255;
    cudaError_t e = cudaMalloc(&c->arena, c->bytes);
    if (e == cudaSuccess) e = cudaMemset(c->arena, 0, c->bytes);    // flags and counters start at zero
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess && world > 1) e = cudaIpcGetMemHandle(&h, c->arena);
    if (e != cudaSuccess) {
        cudaFree(c->arena);
        delete c;
        return fk_fail(FK_COMM, "comm_create: %s", cudaGetErrorString(e));
    }
    memset(handle_out, 0, 64);
    if (world > 1) memcpy(handle_out, &h, sizeof(h) < 64 ? sizeof(h) : 64);
    for (int q = 0; q < FK_AR_MAX_WORLD; q++) c->peer[q] = nullptr;
    c->peer[rank] = c->arena;
    *out = c;
    return FK_OK;
}

FK_EXPORT int fk_comm_connect(fk_comm* c, const uint8_t* handles) {
    if (!c || !handles) return fk_fail(FK_INVALID, "comm_connect: null argument");
    FkDeviceGuard g(c->ctx->device);
    for (int q = 0; q < c->world; q++) {
        if (q == c->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + 64 * q, sizeof(h) < 64 ? sizeof(h) : 64);
        void* p = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) return fk_fail(FK_COMM, "comm_connect: rank %d cannot map the arena of rank %d: %s", c->rank, q, cudaGetErrorString(e));
        c->peer[q] = (uint8_t*)p;
        c->opened[q] = true;
    }
    c->connected = true;
    return FK_OK;
}

// Test hook: the peers' arenas given as plain device pointers of this GPU (the time-out path is tested on one GPU
// against an arena that nobody writes).
FK_EXPORT int fk_comm_connect_local(fk_comm* c, void* const* peer_arenas_dev) {
    if (!c || !peer_arenas_dev) return fk_fail(FK_INVALID, "comm_connect_local: null argument");
    for (int q = 0; q < c->world; q++)
        if (q != c->rank) c->peer[q] = (uint8_t*)peer_arenas_dev[q];
    c->connected = true;
    return FK_OK;
}

FK_EXPORT int fk_comm_arena(fk_comm* c, void** arena_dev, size_t* bytes) {
    if (!c) return fk_fail(FK_INVALID, "comm_arena: null argument");
    if (arena_dev) *arena_dev = c->arena;
    if (bytes) *bytes = c->bytes;
    return FK_OK;
}

FK_EXPORT int fk_comm_destroy(fk_comm* c) {
    if (!c) return FK_OK;
    FkDeviceGuard g(c->ctx->device);
    cudaDeviceSynchronize();
    for (int q = 0; q < c->world; q++)
        if (c->opened[q]) cudaIpcCloseMemHandle(c->peer[q]);
    cudaFree(c->arena);
    delete c;
    return FK_OK;
}

FK_EXPORT size_t fk_comm_channel_bytes(int world, int n_max) { return fk_ar_channel_bytes(world, n_max); }

int fk_ar_channel(fk_comm* c, size_t channel_off, int n_max, int timeout_us, FkArChannel* ch) {
    if (!c->connected && c->world > 1) return fk_fail(FK_COMM, "all-reduce: the communicator is not connected");
    if (channel_off % 256 || n_max < 1 || channel_off + fk_ar_channel_bytes(c->world, n_max) > c->bytes)
        return fk_fail(FK_INVALID, "all-reduce: a channel of %d floats at offset %zu does not fit the arena of %zu bytes", n_max, channel_off, c->bytes);
    ch->rank = c->rank;
    ch->world = c->world;
    ch->n_max = n_max;
    ch->timeout_ns = (unsigned long long)(timeout_us > 0 ? timeout_us : 2000000) * 1000ull;
    for (int q = 0; q < FK_AR_MAX_WORLD; q++) ch->base[q] = q < c->world ? c->peer[q] + channel_off : nullptr;
    return FK_OK;
}

FK_EXPORT int fk_allreduce(fk_ctx* ctx, void* stream, fk_comm* c, size_t channel_off, int n_max, const float* src_dev, float* dst_dev, int n,
                           int accumulate, int timeout_us) {
    if (!ctx || !c || !src_dev || !dst_dev) return fk_fail(FK_INVALID, "allreduce: null argument");
    if (n < 1 || n > n_max) return fk_fail(FK_INVALID, "allreduce: n=%d outside the channel's 1..%d", n, n_max);
    FkDeviceGuard g(ctx->device);
    FkArChannel ch;
    int rc = fk_ar_channel(c, channel_off, n_max, timeout_us, &ch);
    if (rc) return rc;
    const int parts = (n + AR_THREADS * AR_PER_THREAD - 1) / (AR_THREADS * AR_PER_THREAD);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)parts);
    cfg.blockDim = dim3(AR_THREADS);
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    FK_CUDA(cudaLaunchKernelEx(&cfg, allreduce_kernel, ch, src_dev, n, accumulate, dst_dev, ctx->err_flag), FK_LAUNCH);
    ctx->launches++;
    return FK_OK;
}
