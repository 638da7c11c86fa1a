// The peer-memory all-reduce's shared pieces: the communicator, the channel a kernel gets, and the
// device-side protocol steps (used by the standalone all-reduce kernel and by the matvec whose
// epilogue is the all-reduce).
//
// A channel holds, at the same offset of every rank's arena,
//   slots [2][world][n_max] of {f32 value, u32 count}   -- what every rank contributed, two generations
//   sent  [n_max] u32                                   -- how many all-reduces this rank has done on element i
// Element i of all-reduce number t (t = sent[i] + 1, counted on the device, so a replayed CUDA graph
// keeps counting): store {value, t} into slot (t & 1, my rank, i) of EVERY other rank -- one 8-byte
// store, which carries its own arrival mark, so no fence and no separate flag follow it -- then read
// the local slots (t & 1, q, i) until their count is t, and add the values in rank order (every rank
// gets the same bits).  Two generations are enough: a peer can be at most one all-reduce ahead on an
// element, because its next one needs this rank's next contribution.  No rank reads another rank's
// memory, and nothing here is a multicast.
#pragma once
#include "fk_common.cuh"

constexpr int FK_AR_MAX_WORLD = 8;

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

__host__ __device__ inline size_t fk_ar_slots_bytes(int world, int n_max) { return (size_t)2 * world * n_max * 8; }
__host__ __device__ inline size_t fk_ar_channel_bytes(int world, int n_max) { return fk_ar_slots_bytes(world, n_max) + (size_t)n_max * 4; }
int fk_ar_channel(fk_comm* c, size_t channel_off, int n_max, int timeout_us, FkArChannel* ch);

#ifdef __CUDACC__
// slot (generation, from, element) in the arena of rank `at`
__device__ __forceinline__ uint2* fk_ar_slot(const FkArChannel& ch, int at, unsigned gen, int from, int i) {
    return (uint2*)ch.base[at] + ((size_t)gen * ch.world + from) * ch.n_max + i;
}
__device__ __forceinline__ unsigned* fk_ar_sent(const FkArChannel& ch) { return (unsigned*)(ch.base[ch.rank] + fk_ar_slots_bytes(ch.world, ch.n_max)); }

// This rank's value of element i to every other rank; returns the all-reduce's number for the element.
__device__ __forceinline__ unsigned fk_ar_send(const FkArChannel& ch, int i, float v) {
    unsigned* s = fk_ar_sent(ch) + i;
    const unsigned t = *s + 1u;
    *s = t;
    for (int q = 0; q < ch.world; q++) {
        if (q == ch.rank) continue;
        uint2* p = fk_ar_slot(ch, q, t & 1u, ch.rank, i);
        asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(t) : "memory");
    }
    return t;
}

// The sum over ranks of element i of all-reduce t, in rank order; v is this rank's own value.  Every wait is
// bounded in time: past the limit the context's error word becomes 60 and the result is garbage.
__device__ __forceinline__ float fk_ar_recv(const FkArChannel& ch, int i, unsigned t, float v, int* err) {
    float acc = 0.0f;
    unsigned long long t0 = 0;
    bool dead = false;
    for (int q = 0; q < ch.world; q++) {
        if (q == ch.rank) {
            acc += v;
            continue;
        }
        const uint2* p = fk_ar_slot(ch, ch.rank, t & 1u, q, i);
        unsigned val = 0, cnt = 0;
        for (unsigned spin = 0; !dead; spin++) {
            asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(val), "=r"(cnt) : "l"(p) : "memory");
            if (cnt == t) break;
            if ((spin & 15) == 15) {
                unsigned long long now;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                if (!t0) t0 = now;
                if (now - t0 > ch.timeout_ns || *(volatile int*)err != 0) dead = true;
            }
        }
        acc += __uint_as_float(val);
    }
    if (dead) fk_raise(err, 60);
    return acc;
}
#endif
