// The peer-memory all-reduce's shared pieces: the communicator, the channel a kernel gets, and the
// device-side protocol steps (used by the standalone all-reduce kernel and by the matvec whose
// epilogue is the all-reduce).
#pragma once
#include "fk_common.cuh"

constexpr int FK_AR_MAX_WORLD = 8;
constexpr int FK_AR_FLAGS = 2048;   // parts (flags) per channel

struct fk_comm {
    fk_ctx* ctx = nullptr;
    int rank = 0, world = 1;
    uint8_t* arena = nullptr;       // this rank's block
    size_t bytes = 0;
    uint8_t* peer[FK_AR_MAX_WORLD]; // every rank's block as this process addresses it (peer[rank] == arena)
    bool opened[FK_AR_MAX_WORLD] = {false, false, false, false, false, false, false, false};
    bool connected = false;
};

// What a kernel is given: the channel's base in every rank's arena.
struct FkArChannel {
    uint8_t* base[FK_AR_MAX_WORLD];
    int rank, world, n_max;
    unsigned long long timeout_ns;
};

// slots [2][world][n_max] f32 | flags [world][FK_AR_FLAGS] u32 | seen [FK_AR_FLAGS] u32
__host__ __device__ inline size_t fk_ar_slots_bytes(int world, int n_max) { return ((size_t)2 * world * n_max * 4 + 255) & ~(size_t)255; }
__host__ __device__ inline size_t fk_ar_channel_bytes(int world, int n_max) {
    return fk_ar_slots_bytes(world, n_max) + (size_t)world * FK_AR_FLAGS * 4 + (size_t)FK_AR_FLAGS * 4;
}
int fk_ar_channel(fk_comm* c, size_t channel_off, int n_max, int timeout_us, FkArChannel* ch);

#ifdef __CUDACC__
// slot (generation, from) in the arena of rank `at`
__device__ __forceinline__ float* fk_ar_slot(const FkArChannel& ch, int at, unsigned gen, int from) {
    return (float*)ch.base[at] + ((size_t)gen * ch.world + from) * ch.n_max;
}
__device__ __forceinline__ unsigned* fk_ar_flags(const FkArChannel& ch, int at) {
    return (unsigned*)(ch.base[at] + fk_ar_slots_bytes(ch.world, ch.n_max));
}
__device__ __forceinline__ unsigned* fk_ar_seen(const FkArChannel& ch) { return fk_ar_flags(ch, ch.rank) + (size_t)ch.world * FK_AR_FLAGS; }
// flags[my rank][part] = t on rank q (after the caller's system-wide fence)
__device__ __forceinline__ void fk_ar_signal(const FkArChannel& ch, int q, int part, unsigned t) {
    unsigned* f = fk_ar_flags(ch, q) + (size_t)ch.rank * FK_AR_FLAGS + part;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(t) : "memory");
}
// until rank q has delivered part `part` of all-reduce t here; bounded in time, raises error word 60
__device__ __forceinline__ void fk_ar_wait(const FkArChannel& ch, int q, int part, unsigned t, int* err) {
    const unsigned* f = fk_ar_flags(ch, ch.rank) + (size_t)q * FK_AR_FLAGS + part;
    unsigned long long t0 = 0;
    for (unsigned i = 0;; i++) {
        unsigned v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
        if ((int)(v - t) >= 0) return;
        if ((i & 15) == 15) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (!t0) t0 = now;
            if (now - t0 > ch.timeout_ns || *(volatile int*)err != 0) break;
        }
    }
    atomicCAS(err, 0, 60);   // gave up: the result is garbage from here, the host reads the word
}
#endif
