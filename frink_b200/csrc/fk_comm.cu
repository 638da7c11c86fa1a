// One-shot push all-reduce over peer memory (NVLink / NVSwitch), for the small f32 vectors a
// tensor- or expert-parallel decode step sums across GPUs (a few KB to a few hundred KB), where a
// library collective's fixed cost is several times the matvec it follows.
//
// Every rank owns an arena (one cudaMalloc block, shared with the other ranks of the box through
// CUDA IPC) and carves it into channels at the same offsets on every rank.  A channel holds
//   slots [2][world][n_max] f32   -- what every rank contributed, two generations
//   flags [world][FK_AR_FLAGS] u32 -- flags[q][b]: how many times rank q has delivered part b
//   seen  [FK_AR_FLAGS] u32        -- how many all-reduces this rank has finished on part b
// An all-reduce number t (t = seen + 1, counted on the device, so a replayed CUDA graph keeps
// counting) of part b: store the local values into slot (t & 1, my rank) of EVERY rank (plain peer
// stores), make them visible system-wide, store flags[my rank][b] = t on every rank; wait until
// the local flags[q][b] >= t for all q; add the slots in rank order (every rank gets the same
// bits); seen[b] = t.  Two generations are enough: a peer can be at most one all-reduce ahead,
// because its next one needs this rank's next contribution.  No rank reads another rank's
// memory, and nothing here is a multicast.
//
// Every wait is bounded in time (the caller's limit, two seconds by default) and raises the
// context's error word (60) instead of hanging; the call then returns garbage and the host sees
// the word.
#include "fk_comm.cuh"

#include <string.h>

namespace {

__device__ __forceinline__ unsigned long long gtime_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Part b of `n` floats is [b * per, min(n, (b + 1) * per)), per a multiple of 4; one block per part.
__global__ void __launch_bounds__(256) allreduce_kernel(FkArChannel ch, float* __restrict__ buf, int n, int per, int accumulate_into,
                                                         float* __restrict__ dst, int* __restrict__ err) {
    asm volatile("griddepcontrol.wait;" ::: "memory");            // buf is the previous kernel's output
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int b = blockIdx.x, lo = b * per, hi = min(n, lo + per);
    __shared__ unsigned s_target;
    if (threadIdx.x == 0) s_target = fk_ar_seen(ch)[b] + 1u;
    __syncthreads();
    const unsigned target = s_target;
    // 1. my values into my slot on every rank
    for (int q = 0; q < ch.world; q++) {
        float* slot = fk_ar_slot(ch, q, target & 1u, ch.rank);
        for (int i = lo + 4 * (int)threadIdx.x; i < hi; i += 4 * blockDim.x) *(float4*)(slot + i) = *(const float4*)(buf + i);
    }
    __threadfence_system();
    __syncthreads();
    // 2. tell every rank; 3. wait for every rank
    if (threadIdx.x < ch.world) fk_ar_signal(ch, threadIdx.x, b, target);
    if (threadIdx.x < ch.world) fk_ar_wait(ch, threadIdx.x, b, target, err);
    __syncthreads();
    // 4. the sum, in rank order
    for (int i = lo + 4 * (int)threadIdx.x; i < hi; i += 4 * blockDim.x) {
        float4 acc = __ldcg((const float4*)(fk_ar_slot(ch, ch.rank, target & 1u, 0) + i));   // past L1: peers wrote these
        for (int q = 1; q < ch.world; q++) {
            const float4 v = __ldcg((const float4*)(fk_ar_slot(ch, ch.rank, target & 1u, q) + i));
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        if (accumulate_into) {
            const float4 o = *(const float4*)(dst + i);
            acc.x += o.x; acc.y += o.y; acc.z += o.z; acc.w += o.w;
        }
        *(float4*)(dst + i) = acc;
    }
    if (threadIdx.x == 0) fk_ar_seen(ch)[b] = target;
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
    if (channel_off % 256 || channel_off + fk_ar_channel_bytes(c->world, n_max) > c->bytes)
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
    if (n < 1 || n > n_max || (n & 3) || ((uintptr_t)src_dev & 15) || ((uintptr_t)dst_dev & 15))
        return fk_fail(FK_INVALID, "allreduce: n=%d (channel %d) must be a multiple of 4 and the buffers 16-byte aligned", n, n_max);
    FkDeviceGuard g(ctx->device);
    FkArChannel ch;
    int rc = fk_ar_channel(c, channel_off, n_max, timeout_us, &ch);
    if (rc) return rc;
    // parts of at least 4 KB, at most FK_AR_FLAGS of them
    int per = ((n + FK_AR_FLAGS - 1) / FK_AR_FLAGS + 3) & ~3;
    if (per < 1024) per = 1024;
    const int parts = (n + per - 1) / per;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)parts);
    cfg.blockDim = dim3(256);
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    FK_CUDA(cudaLaunchKernelEx(&cfg, allreduce_kernel, ch, (float*)src_dev, n, per, accumulate, dst_dev, ctx->err_flag), FK_LAUNCH);
    ctx->launches++;
    return FK_OK;
}
