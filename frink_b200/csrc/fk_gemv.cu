// Decode GEMV (batch 1..8) over resident quantized weights, and its indexed
// (one expert per slot) form.
//
// The kernel is HBM-bound, so its shape is set by how many weight bytes it can
// keep in flight.  One persistent block of 16 warps per SM.  Every warp owns a
// private ring of shared-memory stages; a stage holds the packed bytes of two
// weight rows for a range of K, brought in by bulk asynchronous copies
// (cp.async.bulk, completion counted on the stage's own mbarrier).  A warp
// issues the copies for all of its stages before anything else, so a block's
// whole share of a small matrix (96 KB per SM for 8192 x 3072 Q4_K) is
// requested in its first cycles; no register is tied up by bytes in flight and
// no block-wide synchronisation is needed, because the warp that fills a stage
// is the warp that drains it.  While the copies fly the block quantizes the
// activations to q8_1 into shared memory (a float4 per thread, eight lanes per
// run of 32 values, the rule of fk_q8_1_lane; all loads issued before any use).
//
// Draining a stage: a lane owns one 16-byte piece of packed weights per row and
// trip, unpacks it in registers, takes exact int32 dot products against the
// int8 activations with dp4a, scales them into an f32 accumulator per (row,
// batch column); the warp reduces with shuffles.  Weight bytes are read once
// for the whole batch.  Every wait on an mbarrier is bounded and raises the
// context's error word instead of spinning forever.
#include "fk_common.cuh"

#include <cuda.h>
#include <limits.h>
#include <stdlib.h>
#include <algorithm>
#include <string.h>

#include "fk_comm.cuh"

namespace {

constexpr int GEMV_THREADS = 512;   // the tensor-core form (batches of 3..8): one block per SM
constexpr int GEMV_WARPS = GEMV_THREADS / 32;
constexpr int LR = 2;           // weight rows a lane carries at once
constexpr int MAX_STAGES = 4;
constexpr int SMEM_BUDGET = 225 * 1024;
// the general dp4a form: one block of 16 warps per SM
constexpr int DP_THREADS = GEMV_THREADS;
constexpr int DP_WARPS = DP_THREADS / 32;
constexpr int DP_MINB = 1;
constexpr int DP_SMEM_BUDGET = SMEM_BUDGET;
// Half an SM's shared memory: what a block of the Q4_K decode kernel may take, so that the blocks
// of two consecutive launches of a stream are resident on an SM together.
constexpr int HALF_SM_SMEM = 112 * 1024;
constexpr uint32_t WAIT_LIMIT = 1u << 24;
constexpr int MMA_MIN_BATCH = 3;   // from this batch on the tensor-core form is used

struct GemvArgs {
    const uint8_t* w;
    size_t mat_stride;
    size_t plane_off[4];
    size_t plane_stride[4];
    const int* ids;
    const int* n_active;   // indexed form: slots >= *n_active do nothing (null = all run)
    int mat;
    const float* x;
    int x_stride;          // floats between the inputs of consecutive slots
    int x_ld;              // floats between batch rows of x (and of glu_up)
    // fused prologue / epilogue (all optional)
    const float* norm_w;   // RMSNorm weight: the kernel reads rmsnorm(x) * norm_w instead of x
    float norm_eps;
    const float* glu_up;   // gated activation: the kernel reads act(x) * glu_up, x being the gate
    int glu_act;           // 0 SiLU, 1 the clamped gpt-oss form
    int accumulate;        // y += result instead of y = result
    int pair_glu;          // rows are (gate, up) pairs: y[rows/2] = act(gate) * up (1 SiLU, 2 the gpt-oss form)
    int ar_on;             // the epilogue sums the results over the ranks of `ar` (element index: b * rows + row)
    FkArChannel ar;
    const float* bias;     // added to the finished dot products (before the gated activation of pair_glu): [rows], or with ids [n_mats][rows]
    const uint8_t* w2;     // indexed form: slots >= split multiply matrix ids[slot - split] of this second stack (same geometry) with
    int split;             //   the input of slot - split; bias2 is their bias table
    const float* bias2;
    int x_ready;           // indexed form: x was written before the kernel that wrote ids STARTED its work (it is two or more
                           //   launches old), so it may be read -- and the activations prepared -- before the wait on that kernel
    // plan of the Q4_K batch 1..2 kernel (block-owned row ranges)
    int q_lp;              // row pairs a warp tile spans (32, 16 or 8; the rest of the lanes span super-blocks)
    int q_sc_off, q_part_off, q_ring_off, q_bar_off;
#ifdef FK_TRACE
    int trace_slot;
#endif
    float* y;
    int rows, cols, batch;
    int32_t* isums;
    int* err;
    // staging plan (host-computed)
    int trips_per_chunk;   // trips of K a stage covers
    int nchunks;           // stages per row pair
    int nstages;           // ring depth
    int stage_bytes;       // bytes of one stage (its rows, all planes)
    int row_bytes_stage;   // bytes of one row inside a stage
    int act_bytes;         // activation region at the start of shared memory
    // plan of the tensor-core form (batches of 3..8)
    int m_ks;              // warps that share one group of 16 rows, each on its own part of K
    int m_kpart_units;     // units of K per such part
    int m_chunk_units;     // units of K a stage covers
    int m_xs;              // bytes between batch rows of the quantized activations
    int m_sd_off, m_red_off;
    int m_srs[4], m_spo[4];   // stage layout: bytes between rows of plane p, offset of plane p
};

// ------------------------------------------------------------------ PTX glue
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded in polls AND in time (two seconds): a copy that never lands costs the launch
// seconds, not minutes, and the host finds word 50 in the context's error flag.
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, int* err) {
    if (mbar_try_wait(bar, parity)) return;
    const unsigned long long t0 = global_ns();
    for (uint32_t i = 0; i < WAIT_LIMIT; i++) {
        if (mbar_try_wait(bar, parity)) return;
        if ((i & 63) == 63 && (*(volatile int*)err != 0 || global_ns() - t0 > 2000000000ull)) break;
    }
    fk_raise(err, 50);   // gave up: results are garbage from here, the host reads the word
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ uint4 lds16(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ int lds_s8(uint32_t addr) {
    int v;
    asm volatile("ld.shared.s8 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds_u8(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

__device__ __forceinline__ int dp4a4(const uint4& a, const int4& b) {
    int s = __dp4a((int)a.x, b.x, 0);
    s = __dp4a((int)a.y, b.y, s);
    s = __dp4a((int)a.z, b.z, s);
    return __dp4a((int)a.w, b.w, s);
}
// Exact int32 -> f32 for |v| < 2^22 on the integer and FP32 pipes (no conversion unit).
__device__ __forceinline__ float i2f(int v) { return __int_as_float(v + 0x4B400000) - 12582912.0f; }
// roundf(x / d) bit for bit without a division per element.  x * inv (inv within an ulp of 1 / d)
// is within 3e-5 of the rounded quotient for |x / d| <= 127, so its nearest integer is the answer
// unless the product sits within 6e-5 of a half; only then is the quotient itself taken.
__device__ __forceinline__ int q8_quant(float x, float d, float inv) {
    const float t = x * inv;
    const float tm = t + 12582912.0f;   // 1.5 * 2^23: the sum is t rounded to an integer, which its low mantissa bits hold
    const float r = tm - 12582912.0f;
    if (!(fabsf(fabsf(t - r) - 0.5f) >= 6.2e-5f) || !(fabsf(t) < 128.5f)) return (int)roundf(x / d);
    return __float_as_int(tm) - 0x4B400000;
}
// Four E2M1 codes (the four nibbles of the low 16 bits of `w`) to their doubled
// int8 values {0,1,2,3,4,6,8,12} with sign, one per byte, in nibble order.
__device__ __forceinline__ uint32_t e2m1x2_4(uint32_t w) {
    uint32_t pos, neg, out;
    const uint32_t sel = w & 0x7777u;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(pos) : "r"(0x03020100u), "r"(0x0C080604u), "r"(sel));
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(neg) : "r"(0xFDFEFF00u), "r"(0xF4F8FAFCu), "r"(sel));
    const uint32_t pick = 0x3210u | ((w & 0x8888u) >> 1);
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(pos), "r"(neg), "r"(pick));
    return out;
}
// The same codes split by sign: the doubled magnitudes of the four codes in the low 16 bits of `w` whose sign bit is
// CLEAR, zero bytes for the others.  The code nibble itself is the selector: its low three bits pick the magnitude, and
// a set sign bit makes prmt replicate the picked byte's top bit -- clear for every magnitude -- over the byte, i.e. 0.
// e2m1_pos4(w ^ 0x8888) is then the magnitudes of the NEGATIVE codes, and a dot product with the signed values is the
// difference of two dp4a: the same integer as with e2m1x2_4, with fewer instructions per code.
__device__ __forceinline__ uint32_t e2m1_pos4(uint32_t w) {
    uint32_t out;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(0x03020100u), "r"(0x0C080604u), "r"(w));
    return out;
}
__device__ __forceinline__ float e8m0_half(uint32_t e) {
    return __uint_as_float(e < 2 ? (0x00200000u << e) : ((e - 1u) << 23));
}

// ---------------------------------------------------------------------------
// Per-kind geometry.  A "trip" is what one pass of the 32 lanes covers of a row:
//   Q4_K : 4 super-blocks (1024 weights) per HALF warp; a stage holds four rows,
//          lanes 0-15 take rows 0-1, lanes 16-31 rows 2-3.  4 lanes per 144-byte
//          block; lane g owns quant bytes [32g, 32g+32): low nibbles are the 32
//          weights of sub-block 2g, high nibbles those of sub-block 2g+1, so a
//          lane decodes one pair of 6-bit scales per 32 bytes of weights.
//   Q6_K : 4 super-blocks; lane c of a block owns ql bytes [16c, 16c+16) and the
//          matching 16 qh bytes: two runs of 16 weights (groups g_lo, g_lo + 4).
//   Q8_0 : 512 weights; a lane owns 16 int8 (half a block).
//   MXFP4: 1024 weights; a lane owns one block's 16 code bytes.
// ROWS: rows per stage (a lane always carries two of them).  PLANES / TB: bytes
// of each plane one trip of one row occupies in a stage (Q6_K's 4th plane, the
// f16 super-scales, is staged as the whole row).
template <int KIND> struct Geo;
template <> struct Geo<FK_Q4_K> { static constexpr int ROWS = 4, PLANES = 1, TRIP_COLS = 1024, TB0 = 576, TB1 = 0, TB2 = 0; };
template <> struct Geo<FK_Q8_0> { static constexpr int ROWS = 2, PLANES = 2, TRIP_COLS = 512, TB0 = 512, TB1 = 32, TB2 = 0; };
template <> struct Geo<FK_Q6_K> { static constexpr int ROWS = 2, PLANES = 4, TRIP_COLS = 1024, TB0 = 512, TB1 = 256, TB2 = 64; };
template <> struct Geo<FK_MXFP4> { static constexpr int ROWS = 2, PLANES = 2, TRIP_COLS = 1024, TB0 = 512, TB1 = 32, TB2 = 0; };
template <int KIND> __host__ __device__ constexpr int trip_bytes(int p) {
    return p == 0 ? Geo<KIND>::TB0 : (p == 1 ? Geo<KIND>::TB1 : (p == 2 ? Geo<KIND>::TB2 : 0));
}

struct Act {
    const int8_t* q;   // [NB][cols]
    const float* d;    // [NB][cols/32]
    const float* s;    // Q4_K: d * run sum
    const int* b16;    // Q6_K: sums of 16
    int cols, nb32;
};

// Where the pieces of (row r of the stage, plane p) start inside a stage.
template <int KIND>
__device__ __forceinline__ uint32_t plane_at(const GemvArgs& a, uint32_t stage, int r, int p) {
    uint32_t off = stage + r * a.row_bytes_stage;
    if (p > 0) off += Geo<KIND>::TB0 * a.trips_per_chunk;
    if (p > 1) off += Geo<KIND>::TB1 * a.trips_per_chunk;
    if (p > 2) off += Geo<KIND>::TB2 * a.trips_per_chunk;
    return off;
}

__device__ __forceinline__ int dp4a_us(uint32_t a, int b, int c) {   // unsigned bytes of a x signed bytes of b
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// Where 16-byte chunk `c` of a row of quantized activations sits in shared memory.
// The lanes of a quarter warp (one shared-memory access phase) read chunks whose
// natural addresses fall on the same banks (Q4_K: 64 bytes apart per lane, 256 per
// block; Q6_K: groups q and q + 8; MXFP4: 32 bytes apart), so a few low bits of the
// chunk index are XOR-ed with higher ones; every phase then covers all 32 banks.
template <int KIND> __device__ __forceinline__ int act_chunk(int c) {
    if (KIND == FK_Q4_K) return c ^ ((c >> 3) & 3);
    if (KIND == FK_Q6_K) return c ^ (((c >> 3) & 1) << 2);
    if (KIND == FK_MXFP4) return c ^ ((c >> 3) & 1);
    return c;
}

// Q4_K, one trip of the lane's two rows.  The lane's half warp covers 4
// super-blocks; the lane owns sub-blocks 2g, 2g+1 of one of them (64 weights,
// 32 quant bytes) in both rows, against the same 64 activations.
template <int NB, bool DUMP>
__device__ __forceinline__ void eat_q4_k(const GemvArgs& a, const Act& sm, uint32_t stage, int row0, int trip, int tl, int lane,
                                         float (*acc)[NB]) {
    const int nsb = a.cols >> 8;
    const int hw = lane >> 4, sbl = (lane >> 2) & 3, g = lane & 3;
    const int sb = trip * 4 + sbl;
    const bool live_sb = sb < nsb;
    const int sbs = live_sb ? sb : 0;
    const int sh = 16 * (g & 1);
#pragma unroll
    for (int r = 0; r < LR; r++) {
        const int row = row0 + hw * LR + r;
        const bool live = live_sb && row < a.rows;
        const uint32_t blk = stage + (hw * LR + r) * a.row_bytes_stage + (tl * 4 + sbl) * 144;
        uint4 hd = make_uint4(0, 0, 0, 0), q0 = hd, q1 = hd;
        if (live) {
            hd = lds16(blk);
            q0 = lds16(blk + 16 + 32 * g);
            q1 = lds16(blk + 32 + 32 * g);
        }
        // 6-bit scales / mins of sub-blocks 2g, 2g+1: 16-bit word (g & 1) of each of
        // the three scale words; sub-blocks 4..7 borrow their top two bits
        const uint32_t a0 = hd.y >> sh, a1 = hd.z >> sh, a2 = hd.w >> sh;
        const uint32_t sc2 = g < 2 ? (a0 & 0x3F3F) : ((a2 & 0x0F0F) | ((a0 & 0xC0C0) >> 2));
        const uint32_t m2 = g < 2 ? (a1 & 0x3F3F) : (((a2 >> 4) & 0x0F0F) | ((a1 & 0xC0C0) >> 2));
        const float d = fk_h2f((uint16_t)(hd.x & 0xFFFF)), ndmin = -fk_h2f((uint16_t)(hd.x >> 16));
        const float fsc_lo = (float)(uint8_t)sc2, fsc_hi = (float)(uint8_t)(sc2 >> 8);
        const float fm_lo = (float)(uint8_t)m2, fm_hi = (float)(uint8_t)(m2 >> 8);
        const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int b = 0; b < NB; b++) {
            const int8_t* q8 = sm.q + (size_t)b * sm.cols + sbs * 256 + 64 * g;
            const int sw = (2 * sbs + (g >> 1)) & 3;   // act_chunk<FK_Q4_K> for chunks 16 sbs + 4 g + j: j ^ sw
            const int4 u0 = *(const int4*)(q8 + 16 * sw), u1 = *(const int4*)(q8 + 16 * (1 ^ sw)), u2 = *(const int4*)(q8 + 16 * (2 ^ sw)),
                       u3 = *(const int4*)(q8 + 16 * (3 ^ sw));
            const int ulo[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
            const int uhi[8] = {u2.x, u2.y, u2.z, u2.w, u3.x, u3.y, u3.z, u3.w};
            const float2 d8 = *(const float2*)(sm.d + b * sm.nb32 + sbs * 8 + 2 * g);
            const float2 s8 = *(const float2*)(sm.s + b * sm.nb32 + sbs * 8 + 2 * g);
            int il = 0, ih = 0;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                il = __dp4a((int)(w[i] & 0x0F0F0F0Fu), ulo[i], il);
                ih = dp4a_us(w[i] & 0xF0F0F0F0u, uhi[i], ih);   // 16 x the high-nibble dot
            }
            ih >>= 4;
            acc[r][b] += d * (fsc_lo * d8.x * (float)il + fsc_hi * d8.y * (float)ih) + ndmin * (fm_lo * s8.x + fm_hi * s8.y);
            if (DUMP && b == 0 && live) {
                int32_t* o = a.isums + (size_t)row * sm.nb32 + sb * 8 + 2 * g;
                o[0] = il;
                o[1] = ih;
            }
        }
    }
}

// One lane's share of one row for one trip: unpack, dot, scale.  `trip` is the
// trip's index in the row (it places the activations), `tl` its index inside the
// stage (it places the weights).
template <int KIND, int NB, bool DUMP>
__device__ __forceinline__ void eat(const GemvArgs& a, const Act& sm, uint32_t stage, int r, int row, bool row_ok, int trip, int tl,
                                    int lane, float* acc) {
    if (KIND == FK_Q8_0) {
        const int ci = trip * 32 + lane;
        const bool live = ci < (sm.cols >> 4) && row_ok;
        const int cs = ci < (sm.cols >> 4) ? ci : 0;
        uint4 wq = make_uint4(0, 0, 0, 0);
        float dw = 0.0f;
        if (live) {
            wq = lds16(plane_at<KIND>(a, stage, r, 0) + (tl * 32 + lane) * 16);
            dw = fk_h2f((uint16_t)lds_u16(plane_at<KIND>(a, stage, r, 1) + (tl * 16 + (lane >> 1)) * 2));
        }
#pragma unroll
        for (int b = 0; b < NB; b++) {
            const int4 ua = *(const int4*)(sm.q + (size_t)b * sm.cols + cs * 16);
            int is = dp4a4(wq, ua);
            acc[b] += dw * sm.d[b * sm.nb32 + (cs >> 1)] * i2f(is);
            if (DUMP && b == 0) {
                is += __shfl_xor_sync(0xffffffffu, is, 1);
                if (live && !(lane & 1)) a.isums[(size_t)row * sm.nb32 + (ci >> 1)] = is;
            }
        }
    } else if (KIND == FK_Q6_K) {
        const int nsb = sm.cols >> 8, sb = trip * 4 + (lane >> 3);
        const bool live = sb < nsb && row_ok;
        const int sbs = sb < nsb ? sb : 0;
        const int c = lane & 7, hf = c >> 2, q = c & 3;
        const int g_lo = 8 * hf + q, g_hi = g_lo + 4;
        const int shift = 2 * (q >> 1);
        const int bl = tl * 4 + (lane >> 3);   // super-block inside the stage
        uint4 ql = make_uint4(0, 0, 0, 0), qh = ql;
        float f_lo = 0.0f, f_hi = 0.0f;
        if (live) {
            const uint32_t p2 = plane_at<KIND>(a, stage, r, 2);
            ql = lds16(plane_at<KIND>(a, stage, r, 0) + bl * 128 + 16 * c);
            qh = lds16(plane_at<KIND>(a, stage, r, 1) + bl * 64 + 32 * hf + 16 * (q & 1));
            const float d = fk_h2f((uint16_t)lds_u16(plane_at<KIND>(a, stage, r, 3) + sb * 2));   // the whole row's super-scales are staged
            f_lo = d * i2f(lds_s8(p2 + bl * 16 + g_lo));
            f_hi = d * i2f(lds_s8(p2 + bl * 16 + g_hi));
        }
        uint4 vl, vh;
        vl.x = (ql.x & 0x0F0F0F0Fu) | (((qh.x >> shift) & 0x03030303u) << 4);
        vl.y = (ql.y & 0x0F0F0F0Fu) | (((qh.y >> shift) & 0x03030303u) << 4);
        vl.z = (ql.z & 0x0F0F0F0Fu) | (((qh.z >> shift) & 0x03030303u) << 4);
        vl.w = (ql.w & 0x0F0F0F0Fu) | (((qh.w >> shift) & 0x03030303u) << 4);
        vh.x = ((ql.x >> 4) & 0x0F0F0F0Fu) | (((qh.x >> (shift + 4)) & 0x03030303u) << 4);
        vh.y = ((ql.y >> 4) & 0x0F0F0F0Fu) | (((qh.y >> (shift + 4)) & 0x03030303u) << 4);
        vh.z = ((ql.z >> 4) & 0x0F0F0F0Fu) | (((qh.z >> (shift + 4)) & 0x03030303u) << 4);
        vh.w = ((ql.w >> 4) & 0x0F0F0F0Fu) | (((qh.w >> (shift + 4)) & 0x03030303u) << 4);
#pragma unroll
        for (int b = 0; b < NB; b++) {
            const int8_t* q8 = sm.q + (size_t)b * sm.cols + sbs * 256;
            const int4 ua = *(const int4*)(q8 + 16 * act_chunk<FK_Q6_K>(g_lo)), ub = *(const int4*)(q8 + 16 * act_chunk<FK_Q6_K>(g_hi));
            const float d8lo = sm.d[b * sm.nb32 + sbs * 8 + (g_lo >> 1)], d8hi = sm.d[b * sm.nb32 + sbs * 8 + (g_hi >> 1)];
            const int* b16 = sm.b16 + b * (sm.cols >> 4) + sbs * 16;
            // codes are stored +32: sum((c - 32) * u) = sum(c * u) - 32 * sum(u)
            const int il = dp4a4(vl, ua) - 32 * b16[g_lo];
            const int ih = dp4a4(vh, ub) - 32 * b16[g_hi];
            acc[b] += f_lo * d8lo * i2f(il) + f_hi * d8hi * i2f(ih);
            if (DUMP && b == 0 && live) {
                int32_t* o = a.isums + (size_t)row * (sm.cols >> 4) + sb * 16;
                o[g_lo] = il;
                o[g_hi] = ih;
            }
        }
    } else {  // FK_MXFP4
        const int kb = trip * 32 + lane;
        const bool live = kb < sm.nb32 && row_ok;
        const int ks = kb < sm.nb32 ? kb : 0;
        uint4 wq = make_uint4(0, 0, 0, 0);
        float dw = 0.0f;
        if (live) {
            wq = lds16(plane_at<KIND>(a, stage, r, 0) + (tl * 32 + lane) * 16);
            dw = e8m0_half(lds_u8(plane_at<KIND>(a, stage, r, 1) + tl * 32 + lane));
        }
        // magnitudes of the positive and of the negative codes (e2m1_pos4): the block's integer dot is their difference
        const uint4 wn = make_uint4(wq.x ^ 0x88888888u, wq.y ^ 0x88888888u, wq.z ^ 0x88888888u, wq.w ^ 0x88888888u);
        uint4 pa, pb, na, nb;
        pa.x = e2m1_pos4(wq.x); pa.y = e2m1_pos4(wq.x >> 16); pa.z = e2m1_pos4(wq.y); pa.w = e2m1_pos4(wq.y >> 16);
        pb.x = e2m1_pos4(wq.z); pb.y = e2m1_pos4(wq.z >> 16); pb.z = e2m1_pos4(wq.w); pb.w = e2m1_pos4(wq.w >> 16);
        na.x = e2m1_pos4(wn.x); na.y = e2m1_pos4(wn.x >> 16); na.z = e2m1_pos4(wn.y); na.w = e2m1_pos4(wn.y >> 16);
        nb.x = e2m1_pos4(wn.z); nb.y = e2m1_pos4(wn.z >> 16); nb.z = e2m1_pos4(wn.w); nb.w = e2m1_pos4(wn.w >> 16);
#pragma unroll
        for (int b = 0; b < NB; b++) {
            const int8_t* q8 = sm.q + (size_t)b * sm.cols + ks * 32;
            const int sw = 16 * ((ks >> 2) & 1);   // act_chunk<FK_MXFP4> for chunks 2 ks, 2 ks + 1
            const int4 ua = *(const int4*)(q8 + sw), ub = *(const int4*)(q8 + (16 ^ sw));
            const int is = (dp4a4(pa, ua) + dp4a4(pb, ub)) - (dp4a4(na, ua) + dp4a4(nb, ub));
            acc[b] += dw * sm.d[b * sm.nb32 + ks] * i2f(is);
            if (DUMP && b == 0 && live) a.isums[(size_t)row * sm.nb32 + kb] = is;
        }
    }
}

// Bytes of plane p that chunk `kc` of a row occupies, and where they start in
// the row.  Sizes are multiples of 16 (plane strides are), the last chunk of a
// row is clipped to the row.
template <int KIND>
__device__ __forceinline__ void chunk_span(const GemvArgs& a, int p, int kc, uint32_t* off, uint32_t* bytes) {
    if (KIND == FK_Q6_K && p == 3) {   // the f16 super-scales: the whole (padded) row, every chunk
        *off = 0;
        *bytes = (uint32_t)a.plane_stride[3];
        return;
    }
    const uint32_t tb = trip_bytes<KIND>(p);
    const uint32_t o = (uint32_t)kc * a.trips_per_chunk * tb;
    const uint32_t stride = (uint32_t)a.plane_stride[p];
    uint32_t n = a.trips_per_chunk * tb;
    if (o + n > stride) n = stride - o;
    *off = o;
    *bytes = n;
}

#ifdef FK_TRACE
__device__ unsigned long long fk_trace_buf[64][160][12];
__device__ __forceinline__ unsigned long long gtime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define TR(slot_, who_) do { if (who_) fk_trace_buf[a.trace_slot & 63][blockIdx.x][slot_] = gtime(); } while (0)
#define TRMAX(slot_, who_) do { if (who_) atomicMax(&fk_trace_buf[a.trace_slot & 63][blockIdx.x][slot_], gtime()); } while (0)
extern "C" __attribute__((visibility("default"))) int fk_trace_read(void* host, size_t bytes, int clear) {
    if (cudaMemcpyFromSymbol(host, fk_trace_buf, bytes) != cudaSuccess) return 1;
    if (clear) { void* p; cudaGetSymbolAddress(&p, fk_trace_buf); cudaMemset(p, 0, sizeof(fk_trace_buf)); }
    return 0;
}
#else
#define TR(slot_, who_) do { } while (0)
#define TRMAX(slot_, who_) do { } while (0)
#endif

template <int KIND, int NB, bool DUMP>
__global__ void __launch_bounds__(DP_THREADS, DP_MINB) gemv_kernel(const GemvArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    TR(0, threadIdx.x == 0);
    const int cols = a.cols, rows = a.rows;
    const int nb32 = cols >> 5;
    int8_t* sq = (int8_t*)smem;                       // [NB][cols] int8
    float* sd = (float*)(smem + (size_t)NB * cols);   // [NB][nb32] stored scale, widened
    float* ss = sd + NB * nb32;                       // Q4_K: [NB][nb32] scale * run sum
    int* sb16 = (int*)(sd + NB * nb32);               // Q6_K: [NB][cols/16] sums of 16

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int slot = blockIdx.y;
    // The slot table (which expert a slot multiplies, how many slots are live) is written by the
    // previous kernel of the stream, so a launch that has one waits for that kernel before it
    // reads anything; a plain matvec waits later, with its weights already on their way.
    const bool dyn = a.ids != nullptr || a.n_active != nullptr;
    // ... unless x is older than that kernel (x_ready): then only the slot table is waited for, after the activations
    // have been normalized and quantized -- the prologue runs while the kernel that picks the experts still does
    const bool late = dyn && a.x_ready != 0;
    if (dyn && !late) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (!late && a.n_active && slot >= *a.n_active) return;
    const bool second = a.w2 != nullptr && slot >= a.split;          // gate and up in one launch: the up half of the slots
    const int in_slot = second ? slot - a.split : slot;
    int mat = a.ids && !late ? a.ids[in_slot] : a.mat;
    const uint8_t* wb = (second ? a.w2 : a.w) + (size_t)mat * a.mat_stride;
    const float* x = a.x + (size_t)in_slot * a.x_stride;
    const float* bias = second ? a.bias2 : a.bias;
    float* y = a.y + (size_t)slot * a.batch * rows;

    // ---- this warp's ring: stages, then one mbarrier per stage
    const uint32_t sbase = smem_u32(smem);
    const uint32_t ring = sbase + a.act_bytes + warp * (a.nstages * a.stage_bytes);
    const uint32_t bars = sbase + a.act_bytes + DP_WARPS * (a.nstages * a.stage_bytes) + warp * (MAX_STAGES * 8);
    if (lane == 0) {
        for (int s = 0; s < a.nstages; s++) mbar_init(bars + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    TR(8, threadIdx.x == 0);

    // consecutive row groups go to consecutive BLOCKS, so a matrix with fewer groups
    // than warps still spreads over every SM
    const int gwarp = warp * gridDim.x + blockIdx.x;
    const int twarps = gridDim.x * DP_WARPS;
    constexpr int RS = Geo<KIND>::ROWS;               // rows per stage
    const int npairs = (rows + RS - 1) / RS;
    const int my_pairs = gwarp < npairs ? (npairs - gwarp + twarps - 1) / twarps : 0;
    const int njobs = my_pairs * a.nchunks;           // a job = one stage fill = (row pair, K chunk)
    const int ntrips = (cols + Geo<KIND>::TRIP_COLS - 1) / Geo<KIND>::TRIP_COLS;

    // Filling a stage: lane c < ROWS * PLANES copies plane (c % PLANES) of row (c / PLANES);
    // lane 0 announces the byte total first.  Jobs are filled in order, so the stage, the
    // row group and the K chunk of the next fill are carried along instead of divided out,
    // and what a lane copies (plane, offsets, sizes) is worked out once.
    constexpr int P = Geo<KIND>::PLANES;
    const int f_r = lane / P, f_p = lane % P;
    const bool f_on = lane < RS * P;
    const bool f_whole = KIND == FK_Q6_K && f_p == 3;                // the f16 super-scales: the whole row, every chunk
    const size_t f_poff = f_p == 0 ? a.plane_off[0] : f_p == 1 ? a.plane_off[1] : f_p == 2 ? a.plane_off[2] : a.plane_off[3];
    const uint32_t f_pstride = (uint32_t)(f_p == 0 ? a.plane_stride[0] : f_p == 1 ? a.plane_stride[1] : f_p == 2 ? a.plane_stride[2] : a.plane_stride[3]);
    const uint32_t f_chunk = f_whole ? f_pstride : (uint32_t)a.trips_per_chunk * (uint32_t)trip_bytes<KIND>(f_p);
    const uint32_t f_dst = plane_at<KIND>(a, 0u, f_r, f_p);
    const uint8_t* f_src = wb + f_poff + (size_t)f_r * f_pstride;      // (late: set again once the slot table may be read)
    int f_stage = 0, f_kc = 0, f_pair = gwarp;
    auto fill = [&]() {
        const uint32_t stage = ring + f_stage * a.stage_bytes, bar = bars + 8 * f_stage;
        const int row = f_pair * RS + f_r;
        uint32_t off = 0, bytes = 0;
        if (f_on && row < rows) {
            off = f_whole ? 0u : (uint32_t)f_kc * f_chunk;
            bytes = off + f_chunk > f_pstride ? f_pstride - off : f_chunk;
        }
        const uint32_t total = __reduce_add_sync(0xffffffffu, bytes);
        if (lane == 0) mbar_expect_tx(bar, total);
        __syncwarp();
        if (bytes) bulk_g2s(stage + f_dst, f_src + (size_t)f_pair * RS * f_pstride + off, bytes, bar);
        if (++f_stage == a.nstages) f_stage = 0;
        if (++f_kc == a.nchunks) { f_kc = 0; f_pair += twarps; }
    };

    // ---- order of the start-up.  Launched with programmatic stream serialization, this
    // grid may start while the previous kernel of the stream still runs; weights are
    // constants, x (and y) may belong to that kernel.  When the activations fit one pass
    // (the usual decode shapes) the block waits for that kernel FIRST and requests x
    // before its weights: the SM takes its deliveries in order, and x asked for after
    // 96 KB of weights arrives after them, with the quantization and every dot product
    // queued behind it.  In a chain of matvecs the wait is short (a block only starts
    // once its SM's block of the previous launch has left).  Larger activations keep the
    // other order: weights first, then the wait.
    constexpr int QU = 1024 / DP_THREADS;   // float4 a thread holds per pass: 4096 columns per pass
    const int c4 = cols >> 2, items = NB * c4;
    const bool early = items <= DP_THREADS * QU;
    float4 v[QU], vn[QU], vu[QU];
    auto load_acts = [&](int base) {
#pragma unroll
        for (int u = 0; u < QU; u++) {
            const int idx = base + u * DP_THREADS + (int)threadIdx.x;
            v[u] = vn[u] = vu[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (idx < items) {
                const int b = NB == 1 ? 0 : idx / c4, k4 = idx - b * c4;
                if (b < a.batch) {
                    // x and glu_up may be written by the kernel this one overlaps with: read them past L1
                    v[u] = __ldcg((const float4*)(x + (size_t)b * a.x_ld) + k4);
                    if (a.norm_w) vn[u] = __ldg((const float4*)a.norm_w + k4);
                    if (a.glu_up) vu[u] = __ldcg((const float4*)(a.glu_up + (size_t)slot * a.x_stride + (size_t)b * a.x_ld) + k4);
                }
            }
        }
    };
    if (early) {
        if (!dyn) asm volatile("griddepcontrol.wait;" ::: "memory");
        load_acts(0);
    }
    const int pre = njobs < a.nstages ? njobs : a.nstages;
    if (!late)
        for (int q = 0; q < pre; q++) fill();
    TR(1, threadIdx.x == 0);
    if (!early && !dyn) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (!late) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    TR(2, threadIdx.x == 0);

    // ---- activations -> q8_1 in shared memory.  A thread takes one float4, eight
    // lanes make a run of 32; all of a thread's loads go out before any is used,
    // so the block pays one L2 round trip, not one per run.
    __shared__ float s_scale[8];
    __shared__ double s_part[DP_WARPS];
    if (a.norm_w) {
        // fused RMSNorm: squares in f32, summed in f64, the mean rounded to f32, 1/sqrtf(mean + eps)
        for (int b = 0; b < a.batch; b++) {
            double sq = 0.0;
            if (early) {
#pragma unroll
                for (int u = 0; u < QU; u++) {
                    const int idx = u * DP_THREADS + (int)threadIdx.x;
                    if (idx < items && (NB == 1 ? 0 : idx / c4) == b)
                        sq += (double)(v[u].x * v[u].x) + (double)(v[u].y * v[u].y) + (double)(v[u].z * v[u].z) + (double)(v[u].w * v[u].w);
                }
            } else {
                for (int i = threadIdx.x; i < c4; i += DP_THREADS) {
                    const float4 t4 = __ldcg((const float4*)(x + (size_t)b * a.x_ld) + i);
                    sq += (double)(t4.x * t4.x) + (double)(t4.y * t4.y) + (double)(t4.z * t4.z) + (double)(t4.w * t4.w);
                }
            }
            for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
            if (lane == 0) s_part[warp] = sq;
            __syncthreads();
            if (threadIdx.x == 0) {
                double t = 0.0;
                for (int i = 0; i < DP_WARPS; i++) t += s_part[i];
                s_scale[b] = 1.0f / sqrtf((float)(t / (double)cols) + a.norm_eps);
            }
            __syncthreads();
        }
    }
    {
        for (int base = 0; base < items; base += DP_THREADS * QU) {
            if (!early) load_acts(base);
#pragma unroll
            for (int u = 0; u < QU; u++) {
                const int idx = base + u * DP_THREADS + (int)threadIdx.x;
                if (idx < items) {
                    const int b = NB == 1 ? 0 : idx / c4;
                    if (b < a.batch) {
                        if (a.norm_w) {
                            const float sc = s_scale[b];
                            v[u].x = v[u].x * sc * vn[u].x; v[u].y = v[u].y * sc * vn[u].y;
                            v[u].z = v[u].z * sc * vn[u].z; v[u].w = v[u].w * sc * vn[u].w;
                        }
                        if (a.glu_up) {
                            float g[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
                            const float uu[4] = {vu[u].x, vu[u].y, vu[u].z, vu[u].w};
#pragma unroll
                            for (int e = 0; e < 4; e++) {
                                if (a.glu_act == 0) {
                                    g[e] = (g[e] / (1.0f + expf(-g[e]))) * uu[e];
                                } else {
                                    const float xg = fminf(g[e], 7.0f), yu = fminf(fmaxf(uu[e], -7.0f), 7.0f);
                                    g[e] = (xg / (1.0f + expf(1.702f * -xg))) * (yu + 1.0f);
                                }
                            }
                            v[u] = make_float4(g[0], g[1], g[2], g[3]);
                        }
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < QU; u++) {
                if (base + u * DP_THREADS + warp * 32 >= items) continue;   // nothing for this warp here (the same for all its lanes)
                const int idx = base + u * DP_THREADS + (int)threadIdx.x;
                const bool ok = idx < items;
                const int b = !ok || NB == 1 ? 0 : idx / c4, k4 = ok ? idx - b * c4 : 0;
                const int kb = k4 >> 3, quad = k4 & 7;
                // the rule of fk_q8_1_lane over the eight lanes of the run (max and integer sums are order-free)
                unsigned mb = __float_as_uint(fmaxf(fmaxf(fabsf(v[u].x), fabsf(v[u].y)), fmaxf(fabsf(v[u].z), fabsf(v[u].w))));
                mb = max(mb, __shfl_xor_sync(0xffffffffu, mb, 1));
                mb = max(mb, __shfl_xor_sync(0xffffffffu, mb, 2));
                mb = max(mb, __shfl_xor_sync(0xffffffffu, mb, 4));
                const float amax = __uint_as_float(mb);
                TR(9, threadIdx.x == 0 && u == 0 && base == 0);
                const float d = amax / 127.0f;
                int q0 = 0, q1 = 0, q2 = 0, q3 = 0;
                if (amax != 0.0f) {
                    q0 = (int)roundf(v[u].x / d);
                    q1 = (int)roundf(v[u].y / d);
                    q2 = (int)roundf(v[u].z / d);
                    q3 = (int)roundf(v[u].w / d);
                }
                int s16 = q0 + q1 + q2 + q3;
                s16 += __shfl_xor_sync(0xffffffffu, s16, 1);
                s16 += __shfl_xor_sync(0xffffffffu, s16, 2);           // sum of this lane's half run (16 values)
                const int qsum = s16 + __shfl_xor_sync(0xffffffffu, s16, 4);
                if (ok) {
                    int8_t* rowq = sq + (size_t)b * cols;
                    if (KIND == FK_MXFP4) {
                        // each run is kept as (elem j, elem j+16) pairs: the order the nibble decode produces bytes in
                        const int e = 4 * quad;
                        const int qv[4] = {q0, q1, q2, q3};
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const int pos = (((e + i) & 15) << 1) | ((e + i) >> 4);
                            rowq[16 * act_chunk<KIND>(2 * kb + (pos >> 4)) + (pos & 15)] = (int8_t)qv[i];
                        }
                    } else {
                        *(uint32_t*)(rowq + 16 * act_chunk<KIND>(k4 >> 2) + 4 * (k4 & 3)) =
                            (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) | ((uint32_t)(q2 & 0xFF) << 16) | ((uint32_t)(q3 & 0xFF) << 24);
                    }
                    if (KIND == FK_Q6_K && (quad & 3) == 0) sb16[b * (cols >> 4) + 2 * kb + (quad >> 2)] = s16;
                    if (quad == 0) {
                        const float dq = fk_h2f(fk_f2h(d));   // the stored f16 scale, widened
                        sd[b * nb32 + kb] = dq;
                        if (KIND == FK_Q4_K) ss[b * nb32 + kb] = dq * (float)qsum;
                    }
                }
            }
        }
    }
    TR(10, threadIdx.x == 0);
    TR(11, threadIdx.x == DP_THREADS - 1);
    if (late) {
        // the activations are ready in shared memory; now the slot table, then this slot's weights
        asm volatile("griddepcontrol.wait;" ::: "memory");
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
        if (a.n_active && slot >= *a.n_active) return;               // (the whole block: nothing is in flight yet)
        if (a.ids) mat = __ldcg(a.ids + in_slot);
        wb = (second ? a.w2 : a.w) + (size_t)mat * a.mat_stride;
        f_src = wb + f_poff + (size_t)f_r * f_pstride;
        for (int q = 0; q < pre; q++) fill();
    }
    __syncthreads();
    TR(3, threadIdx.x == 0);
    const Act sm{sq, sd, ss, sb16, cols, nb32};

    float acc[LR][NB];
    int pair = gwarp, kc = 0, s = 0;
    uint32_t phase = 0;
    for (int q = 0; q < njobs; q++) {
        const uint32_t stage = ring + s * a.stage_bytes;
        const int row0 = pair * RS;
        if (kc == 0) {
#pragma unroll
            for (int r = 0; r < LR; r++)
#pragma unroll
                for (int b = 0; b < NB; b++) acc[r][b] = 0.0f;
        }
        mbar_wait(bars + 8 * s, phase, a.err);
        TR(4, threadIdx.x == 0 && q == 0);
        const int t0 = kc * a.trips_per_chunk;
        const int t1 = t0 + a.trips_per_chunk < ntrips ? t0 + a.trips_per_chunk : ntrips;
        for (int t = t0; t < t1; t++) {
            if (KIND == FK_Q4_K) {
                eat_q4_k<NB, DUMP>(a, sm, stage, row0, t, t - t0, lane, acc);
            } else {
#pragma unroll
                for (int r = 0; r < LR; r++) eat<KIND, NB, DUMP>(a, sm, stage, r, row0 + r, row0 + r < rows, t, t - t0, lane, acc[r]);
            }
        }
        // every lane has consumed the stage: refill it with the job one ring ahead
        __syncwarp();
        TR(5, threadIdx.x == 0 && q == 0);
        if (q + a.nstages < njobs) fill();
        const bool row_done = kc == a.nchunks - 1;
        if (row_done) {
            // Q4_K: a half warp per row pair; the others: the whole warp on one pair
            const int hw = KIND == FK_Q4_K ? lane >> 4 : 0;
            float done[LR][NB];
#pragma unroll
            for (int r = 0; r < LR; r++)
#pragma unroll
                for (int b = 0; b < NB; b++) {
                    float v = acc[r][b];
                    if (KIND != FK_Q4_K) v += __shfl_xor_sync(0xffffffffu, v, 16);
                    v += __shfl_xor_sync(0xffffffffu, v, 8);
                    v += __shfl_xor_sync(0xffffffffu, v, 4);
                    v += __shfl_xor_sync(0xffffffffu, v, 2);
                    v += __shfl_xor_sync(0xffffffffu, v, 1);
                    done[r][b] = v;
                }
            const bool writer = (lane & 15) == 0 && (KIND == FK_Q4_K || lane == 0);
            if (bias && writer) {
#pragma unroll
                for (int r = 0; r < LR; r++) {
                    const int row = row0 + hw * LR + r;
                    const float bv = row < rows ? bias[(a.ids ? (size_t)mat * rows : 0) + row] : 0.0f;
#pragma unroll
                    for (int b = 0; b < NB; b++) done[r][b] += bv;
                }
            }
            if (a.pair_glu) {
                // rows come as (gate, up) pairs (the merged projection was stacked row-interleaved):
                // the lane holds both, so the gated activation is formed here and written once
                const int prow = (row0 + hw * LR) >> 1;
                if (writer && row0 + hw * LR + 1 < rows) {
#pragma unroll
                    for (int b = 0; b < NB; b++) {
                        if (b >= a.batch) break;
                        const float gt = done[0][b], up = done[1][b];
                        float o;
                        if (a.pair_glu == 1) {
                            o = (gt / (1.0f + expf(-gt))) * up;
                        } else {
                            const float xg = fminf(gt, 7.0f), yu = fminf(fmaxf(up, -7.0f), 7.0f);
                            o = (xg / (1.0f + expf(1.702f * -xg))) * (yu + 1.0f);
                        }
                        y[(size_t)b * (rows >> 1) + prow] = o;
                    }
                }
            } else {
                // row-split across GPUs: every value goes to the peers first, then the peers' values are awaited,
                // so the link's latency is paid once for the lane's LR * NB values
                if (a.ar_on) {
#pragma unroll
                    for (int r = 0; r < LR; r++)
#pragma unroll
                        for (int b = 0; b < NB; b++) {
                            const int row = row0 + hw * LR + r;
                            if (writer && row < rows && b < a.batch) fk_ar_send(a.ar, b * rows + row, done[r][b]);
                        }
                }
#pragma unroll
                for (int r = 0; r < LR; r++)
#pragma unroll
                    for (int b = 0; b < NB; b++) {
                        const int row = row0 + hw * LR + r;
                        if (writer && row < rows && b < a.batch) {
                            float v = done[r][b];
                            if (a.ar_on) v = fk_ar_recv(a.ar, b * rows + row, fk_ar_sent(a.ar)[b * rows + row], v, a.err);
                            float* dst = y + (size_t)b * rows + row;
                            *dst = a.accumulate ? *dst + v : v;
                        }
                    }
            }
        }
        if (++s == a.nstages) { s = 0; phase ^= 1u; }
        if (++kc == a.nchunks) { kc = 0; pair += twarps; }
    }
    TR(6, threadIdx.x == 0);
    TRMAX(7, lane == 0);
}


// ===========================================================================
// Q4_K, batch 1 (the decode matvec proper), for matrices whose share per SM fits a block's
// shared memory.  Once its weights are prefetched across the launch boundary the launch is
// bound by the instructions it issues and the shared-memory wavefronts it makes, so this
// form spends as few of both as the format allows:
//   * a block owns a contiguous range of row pairs and requests ALL of it at its start
//     (one bulk copy per row pair); the block takes half an SM, so the block of the next
//     launch of the stream is resident beside it and has its weights in flight while this
//     one computes (programmatic stream serialization);
//   * a thread takes a unit = one 144-byte super-block of the two rows of a pair: the eight
//     6-bit scales and mins of a block are unpacked four at a time with byte-wide masks, the
//     64 activations of a quarter block are loaded once for both rows, and a block's sums
//     are scaled by d / dmin once;
//   * the lanes of a warp hold DIFFERENT row pairs of the SAME super-block(s): their
//     activation loads are broadcasts (half the wavefronts of distinct addresses), and the
//     row pairs sit 16 bytes more than a multiple of 128 apart, so the weight loads of
//     eight neighbouring lanes fall on different banks;
//   * partial sums of a row meet in shared memory and are added in super-block order, so
//     the result does not depend on how units fell to threads.
#ifndef FK_Q4_THREADS
#define FK_Q4_THREADS 512
#endif
constexpr int Q4_MAX_THREADS = FK_Q4_THREADS;

template <int NB, bool DUMP>
__global__ void __launch_bounds__(Q4_MAX_THREADS, 2) gemv_q4k_kernel(const GemvArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    TR(0, threadIdx.x == 0);
    const int T = blockDim.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = T >> 5;
    const int cols = a.cols, rows = a.rows, nb32 = cols >> 5, nsb = cols >> 8;
    int8_t* sq = (int8_t*)smem;                               // [NB][cols] int8
    float* ssc = (float*)(smem + a.q_sc_off);                  // [NB][nsb][16]: per super-block d[0..7], d * run sum [0..7]
    float* part = (float*)(smem + a.q_part_off);               // [block rows][nsb][NB]
    const uint32_t sbase = smem_u32(smem), ring = sbase + a.q_ring_off, bar = sbase + a.q_bar_off;
    const uint8_t* wb = a.w + (size_t)a.mat * a.mat_stride;
    const float* x = a.x;
    float* y = a.y;
    const uint32_t rb = (uint32_t)a.plane_stride[0];           // bytes of a row
    const uint32_t ps = 2 * rb + 16;                           // bytes between row pairs in shared memory
    // row pairs dealt evenly over the blocks: every SM gets one block of (nearly) the same size
    const int npairs = (rows + 1) >> 1;
    const int pair_lo = (int)(((long long)blockIdx.x * npairs) / gridDim.x);
    const int pair_hi = (int)(((long long)(blockIdx.x + 1) * npairs) / gridDim.x);
    const int np = pair_hi - pair_lo, row_lo = 2 * pair_lo, n = min(rows, 2 * pair_hi) - row_lo;

    if (tid == 0) {
        mbar_init(bar, nwarps);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    TR(8, threadIdx.x == 0);
    if (lane == 0) {
        // this warp's row pairs: warp, warp + nwarps, ...
        uint32_t total = 0;
        for (int p = warp; p < np; p += nwarps) total += (uint32_t)min(2, n - 2 * p) * rb;
        mbar_expect_tx(bar, total);
        for (int p = warp; p < np; p += nwarps)
            bulk_g2s(ring + (uint32_t)p * ps, wb + (size_t)(row_lo + 2 * p) * rb, (uint32_t)min(2, n - 2 * p) * rb, bar);
    }
    TR(1, threadIdx.x == 0);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    TR(2, threadIdx.x == 0);

    // ---- activations -> q8_1 in shared memory (the rule of fk_q8_1_lane; eight lanes make a run)
    const int c4 = cols >> 2, items = NB * c4;
    constexpr int QU = 1024 / Q4_MAX_THREADS;
    for (int base = 0; base < items; base += QU * T) {
        float4 v[QU];
#pragma unroll
        for (int u = 0; u < QU; u++) {
            const int idx = base + u * T + tid;
            v[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (idx < items) {
                const int b = NB == 1 ? 0 : idx / c4, k4 = idx - b * c4;
                // x may be written by the kernel this one overlaps with: read it past L1
                if (b < a.batch) v[u] = __ldcg((const float4*)(x + (size_t)b * a.x_ld) + k4);
            }
        }
#pragma unroll
        for (int u = 0; u < QU; u++) {
            if (base + u * T + warp * 32 >= items) continue;   // nothing for this warp here (the same for all its lanes)
            const int idx = base + u * T + tid;
            const bool ok = idx < items;
            const int b = !ok || NB == 1 ? 0 : idx / c4, k4 = ok ? idx - b * c4 : 0;
            const float4 f = v[u];
            unsigned mb = __float_as_uint(fmaxf(fmaxf(fabsf(f.x), fabsf(f.y)), fmaxf(fabsf(f.z), fabsf(f.w))));
            mb = max(mb, __shfl_xor_sync(0xffffffffu, mb, 1));
            mb = max(mb, __shfl_xor_sync(0xffffffffu, mb, 2));
            mb = max(mb, __shfl_xor_sync(0xffffffffu, mb, 4));
            const float amax = __uint_as_float(mb);
            TR(9, threadIdx.x == 0 && u == 0 && base == 0);
            const float d = amax / 127.0f;
            float inv = 0.0f;
            if (amax != 0.0f) asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(inv) : "f"(d));   // within an ulp of 1 / d (q8_quant wants no more)
            const int q0 = q8_quant(f.x, d, inv), q1 = q8_quant(f.y, d, inv), q2 = q8_quant(f.z, d, inv), q3 = q8_quant(f.w, d, inv);
            int qsum = q0 + q1 + q2 + q3;
            qsum += __shfl_xor_sync(0xffffffffu, qsum, 1);
            qsum += __shfl_xor_sync(0xffffffffu, qsum, 2);
            qsum += __shfl_xor_sync(0xffffffffu, qsum, 4);
            TR(11, threadIdx.x == 0 && u == 0 && base == 0);
            if (ok) {
                *(uint32_t*)(sq + (size_t)b * cols + 4 * k4) =
                    (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) | ((uint32_t)(q2 & 0xFF) << 16) | ((uint32_t)(q3 & 0xFF) << 24);
                if ((k4 & 7) == 0) {
                    const int kb = k4 >> 3;
                    const float dq = fk_h2f(fk_f2h(d));   // the stored f16 scale, widened
                    float* scb = ssc + ((size_t)b * nsb + (kb >> 3)) * 16 + (kb & 7);
                    scb[0] = dq;
                    scb[8] = dq * i2f(qsum);
                }
            }
        }
    }
    TR(10, threadIdx.x == 0);
    __syncthreads();
    TR(3, threadIdx.x == 0);

    // ---- units.  A warp tile is LP row pairs x (32 / LP) super-blocks; tiles go round the warps.
    const int LP = a.q_lp, LS = 32 / LP;
    const int ptiles = (np + LP - 1) / LP, stiles = (nsb + LS - 1) / LS;
    const int lp = lane % LP, ls = lane / LP;
    mbar_wait(bar, 0u, a.err);
    TR(4, threadIdx.x == 0);
    for (int wt = warp; wt < ptiles * stiles; wt += nwarps) {
        const int pt = wt / stiles, stl = wt - pt * stiles;
        const int pr = pt * LP + lp, sb = stl * LS + ls;
        if (pr >= np || sb >= nsb) continue;
        const bool two = 2 * pr + 1 < n;
        const uint32_t blk0 = ring + (uint32_t)pr * ps + (uint32_t)sb * 144u;
        const uint32_t blk[2] = {blk0, two ? blk0 + rb : blk0};
        uint32_t scw[2][2], mnw[2][2];
        float dd[2], dm[2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const uint4 hd = lds16(blk[r]);
            // 6-bit scales and mins of the 8 sub-blocks, one per byte: [0..3] and [4..7]
            scw[r][0] = hd.y & 0x3F3F3F3Fu;
            scw[r][1] = (hd.w & 0x0F0F0F0Fu) | ((hd.y >> 2) & 0x30303030u);
            mnw[r][0] = hd.z & 0x3F3F3F3Fu;
            mnw[r][1] = ((hd.w >> 4) & 0x0F0F0F0Fu) | ((hd.z >> 2) & 0x30303030u);
            dd[r] = fk_h2f((uint16_t)(hd.x & 0xFFFF));
            dm[r] = fk_h2f((uint16_t)(hd.x >> 16));
        }
        float accS[2][NB], accM[2][NB];
#pragma unroll
        for (int r = 0; r < 2; r++)
#pragma unroll
            for (int b = 0; b < NB; b++) accS[r][b] = accM[r][b] = 0.0f;
        // a quarter block (sub-blocks 2q, 2q + 1) per trip; rolled, so the loop body stays in the instruction cache
#pragma unroll 1
        for (int q = 0; q < 4; q++) {
            uint32_t w[2][8];
#pragma unroll
            for (int r = 0; r < 2; r++) {
                const uint4 wa = lds16(blk[r] + 16 + 32 * q), wc = lds16(blk[r] + 32 + 32 * q);
                w[r][0] = wa.x; w[r][1] = wa.y; w[r][2] = wa.z; w[r][3] = wa.w;
                w[r][4] = wc.x; w[r][5] = wc.y; w[r][6] = wc.z; w[r][7] = wc.w;
            }
            // bytes 2 (q & 1), 2 (q & 1) + 1 of the scale / min words of sub-blocks 4 (q >> 1) ..
            const uint32_t sel = (q & 1) ? 0x7652u : 0x7650u;
#pragma unroll
            for (int b = 0; b < NB; b++) {
                const int8_t* q8 = sq + (size_t)b * cols + sb * 256 + 64 * q;
                const int4 u0 = *(const int4*)q8, u1 = *(const int4*)(q8 + 16), u2 = *(const int4*)(q8 + 32), u3 = *(const int4*)(q8 + 48);
                const int ulo[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
                const int uhi[8] = {u2.x, u2.y, u2.z, u2.w, u3.x, u3.y, u3.z, u3.w};
                const float* scb = ssc + ((size_t)b * nsb + sb) * 16 + 2 * q;
                const float2 d8 = *(const float2*)scb, s8 = *(const float2*)(scb + 8);
#pragma unroll
                for (int r = 0; r < 2; r++) {
                    int il = 0, ih = 0;
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        il = __dp4a((int)(w[r][i] & 0x0F0F0F0Fu), ulo[i], il);
                        ih = dp4a_us(w[r][i] & 0xF0F0F0F0u, uhi[i], ih);   // 16 x the high-nibble dot
                    }
                    ih >>= 4;
                    // scale and min bytes as floats: 2^23 + byte, minus 2^23
                    const uint32_t scv = (q & 2) ? scw[r][1] : scw[r][0], mnv = (q & 2) ? mnw[r][1] : mnw[r][0];
                    const float fsl = __uint_as_float(__byte_perm(scv, 0x4B000000u, sel)) - 8388608.0f;
                    const float fsh = __uint_as_float(__byte_perm(scv, 0x4B000000u, sel + 1)) - 8388608.0f;
                    const float fml = __uint_as_float(__byte_perm(mnv, 0x4B000000u, sel)) - 8388608.0f;
                    const float fmh = __uint_as_float(__byte_perm(mnv, 0x4B000000u, sel + 1)) - 8388608.0f;
                    accS[r][b] = fmaf(fsl * d8.x, i2f(il), fmaf(fsh * d8.y, i2f(ih), accS[r][b]));
                    accM[r][b] = fmaf(fml, s8.x, fmaf(fmh, s8.y, accM[r][b]));
                    if (DUMP && b == 0 && (r == 0 || two)) {
                        int32_t* o = a.isums + (size_t)(row_lo + 2 * pr + r) * nb32 + sb * 8 + 2 * q;
                        o[0] = il;
                        o[1] = ih;
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < 2; r++)
#pragma unroll
            for (int b = 0; b < NB; b++)
                if (r == 0 || two) part[((size_t)(2 * pr + r) * nsb + sb) * NB + b] = dd[r] * accS[r][b] - dm[r] * accM[r][b];
    }
    __syncthreads();
    TR(5, threadIdx.x == 0);
    // ---- a row's partial sums, in super-block order
    for (int i = tid; i < n * NB; i += T) {
        const int rr = i / NB, b = i - rr * NB;
        if (b >= a.batch) continue;
        float v = 0.0f;
        for (int k = 0; k < nsb; k++) v += part[((size_t)rr * nsb + k) * NB + b];
        y[(size_t)b * rows + row_lo + rr] = v;
    }
    TR(6, threadIdx.x == 0);
    TRMAX(7, lane == 0);
}

// ===========================================================================
// Batches of 3..8: the per-run integer dots on the int8 tensor-core instruction
// (mma.sync m16n8k32: 16 weight rows x one run of 32 x 8 batch columns), so the
// weights are unpacked once whatever the batch.  A warp owns a group of 16 rows
// for a part of K; KS warps of the same block share a group (rows/16 groups alone
// would leave most warps idle) and their partial sums meet in shared memory in a
// fixed order.  Each lane ends up with rows g, g+8 x batch columns 2t, 2t+1
// (g = lane / 4, t = lane % 4), scales them per run in f32 like the dp4a form,
// and nothing crosses lanes.  The exact int32 dots per run are the same numbers.
constexpr int MM_ROWS = 16;
template <int KIND> struct MGeo;
template <> struct MGeo<FK_Q4_K> { static constexpr int UNIT = 256, PLANES = 1, PB0 = 144, PB1 = 0, PB2 = 0; };
template <> struct MGeo<FK_Q8_0> { static constexpr int UNIT = 256, PLANES = 2, PB0 = 256, PB1 = 16, PB2 = 0; };
template <> struct MGeo<FK_Q6_K> { static constexpr int UNIT = 256, PLANES = 4, PB0 = 128, PB1 = 64, PB2 = 16; };
template <> struct MGeo<FK_MXFP4> { static constexpr int UNIT = 512, PLANES = 2, PB0 = 256, PB1 = 16, PB2 = 0; };
template <int KIND> __host__ __device__ constexpr int unit_bytes(int p) {
    return p == 0 ? MGeo<KIND>::PB0 : (p == 1 ? MGeo<KIND>::PB1 : (p == 2 ? MGeo<KIND>::PB2 : 0));
}

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ float byte_f(uint32_t w, int i) { return (float)((w >> (8 * i)) & 0xFFu); }
// Q6_K codes (0..63, the value + 32) in the four bytes of v -> signed bytes
__device__ __forceinline__ uint32_t q6_signed(uint32_t v) {
    const uint32_t r = v ^ 0x20202020u, neg = r & 0x20202020u;
    return r | (neg << 1) | (neg << 2);
}

// One stage (units cu0..cu1 of K) of the warp's 16 rows against the batch.
template <int KIND>
__device__ __forceinline__ void mma_eat(const GemvArgs& a, uint32_t stage, int cu0, int cu1, uint32_t xrow, const float* sdT, const float* ssT,
                                        int nb32, int lane, float (&acc)[4]) {
    const int g = lane >> 2, t = lane & 3;
    const uint32_t r0 = stage + a.m_spo[0] + g * a.m_srs[0], r8 = r0 + 8 * a.m_srs[0];
    if (KIND == FK_Q4_K) {
        for (int u = cu0; u < cu1; u++) {
            const uint32_t bg = r0 + (u - cu0) * 144, bh = r8 + (u - cu0) * 144;
            const uint4 hg = lds16(bg), hh = lds16(bh);
            // 6-bit scales and mins of the 8 sub-blocks, one per byte: [0..3] and [4..7]
            const uint32_t scg[2] = {hg.y & 0x3F3F3F3Fu, (hg.w & 0x0F0F0F0Fu) | ((hg.y >> 2) & 0x30303030u)};
            const uint32_t mng[2] = {hg.z & 0x3F3F3F3Fu, ((hg.w >> 4) & 0x0F0F0F0Fu) | ((hg.z >> 2) & 0x30303030u)};
            const uint32_t sch[2] = {hh.y & 0x3F3F3F3Fu, (hh.w & 0x0F0F0F0Fu) | ((hh.y >> 2) & 0x30303030u)};
            const uint32_t mnh[2] = {hh.z & 0x3F3F3F3Fu, ((hh.w >> 4) & 0x0F0F0F0Fu) | ((hh.z >> 2) & 0x30303030u)};
            const float dg = fk_h2f((uint16_t)(hg.x & 0xFFFF)), ndming = -fk_h2f((uint16_t)(hg.x >> 16));
            const float dh = fk_h2f((uint16_t)(hh.x & 0xFFFF)), ndminh = -fk_h2f((uint16_t)(hh.x >> 16));
#pragma unroll
            for (int j = 0; j < 4; j++) {      // 32 quant bytes: low nibbles = run 2j, high nibbles = run 2j + 1
                const uint32_t w0 = lds32(bg + 16 + 32 * j + 4 * t), w2 = lds32(bg + 32 + 32 * j + 4 * t);
                const uint32_t w1 = lds32(bh + 16 + 32 * j + 4 * t), w3 = lds32(bh + 32 + 32 * j + 4 * t);
                const int run = u * 8 + 2 * j;
                const uint32_t xl = xrow + run * 32 + 4 * t;
                int dl[4], dh4[4];
                mma_s8(dl, w0 & 0x0F0F0F0Fu, w1 & 0x0F0F0F0Fu, w2 & 0x0F0F0F0Fu, w3 & 0x0F0F0F0Fu, lds32(xl), lds32(xl + 16));
                mma_s8(dh4, (w0 >> 4) & 0x0F0F0F0Fu, (w1 >> 4) & 0x0F0F0F0Fu, (w2 >> 4) & 0x0F0F0F0Fu, (w3 >> 4) & 0x0F0F0F0Fu, lds32(xl + 32),
                       lds32(xl + 48));
                const float2 dxl = *(const float2*)(sdT + run * 8 + 2 * t), dxh = *(const float2*)(sdT + run * 8 + 8 + 2 * t);
                const float2 sxl = *(const float2*)(ssT + run * 8 + 2 * t), sxh = *(const float2*)(ssT + run * 8 + 8 + 2 * t);
                const int jb = 2 * (j & 1);
                const float sgl = dg * byte_f(scg[j >> 1], jb), sgh = dg * byte_f(scg[j >> 1], jb + 1);
                const float shl = dh * byte_f(sch[j >> 1], jb), shh = dh * byte_f(sch[j >> 1], jb + 1);
                const float mgl = ndming * byte_f(mng[j >> 1], jb), mgh = ndming * byte_f(mng[j >> 1], jb + 1);
                const float mhl = ndminh * byte_f(mnh[j >> 1], jb), mhh = ndminh * byte_f(mnh[j >> 1], jb + 1);
                acc[0] += sgl * dxl.x * i2f(dl[0]) + sgh * dxh.x * i2f(dh4[0]) + (mgl * sxl.x + mgh * sxh.x);
                acc[1] += sgl * dxl.y * i2f(dl[1]) + sgh * dxh.y * i2f(dh4[1]) + (mgl * sxl.y + mgh * sxh.y);
                acc[2] += shl * dxl.x * i2f(dl[2]) + shh * dxh.x * i2f(dh4[2]) + (mhl * sxl.x + mhh * sxh.x);
                acc[3] += shl * dxl.y * i2f(dl[3]) + shh * dxh.y * i2f(dh4[3]) + (mhl * sxl.y + mhh * sxh.y);
            }
        }
    } else if (KIND == FK_Q8_0) {
        const uint32_t s0 = stage + a.m_spo[1] + g * a.m_srs[1], s8 = s0 + 8 * a.m_srs[1];
        for (int u = cu0; u < cu1; u++) {
#pragma unroll
            for (int r = 0; r < 8; r++) {
                const int run = u * 8 + r;
                if (run >= nb32) break;
                const uint32_t o = ((u - cu0) * 8 + r) * 32 + 4 * t;
                const uint32_t xl = xrow + run * 32 + 4 * t;
                int d4[4];
                mma_s8(d4, lds32(r0 + o), lds32(r8 + o), lds32(r0 + o + 16), lds32(r8 + o + 16), lds32(xl), lds32(xl + 16));
                const float wg = fk_h2f((uint16_t)lds_u16(s0 + ((u - cu0) * 8 + r) * 2)), wh = fk_h2f((uint16_t)lds_u16(s8 + ((u - cu0) * 8 + r) * 2));
                const float2 dx = *(const float2*)(sdT + run * 8 + 2 * t);
                acc[0] += wg * dx.x * i2f(d4[0]);
                acc[1] += wg * dx.y * i2f(d4[1]);
                acc[2] += wh * dx.x * i2f(d4[2]);
                acc[3] += wh * dx.y * i2f(d4[3]);
            }
        }
    } else if (KIND == FK_MXFP4) {
        const uint32_t s0 = stage + a.m_spo[1] + g * a.m_srs[1], s8 = s0 + 8 * a.m_srs[1];
        for (int u = cu0; u < cu1; u++) {
#pragma unroll 4
            for (int r = 0; r < 16; r++) {
                const int run = u * 16 + r;
                if (run >= nb32) break;
                const uint32_t o = ((u - cu0) * 16 + r) * 16 + 4 * t;
                const uint32_t wg = lds32(r0 + o), wh = lds32(r8 + o);
                // code byte i holds elements i and i + 16; the activations of a run are stored in that (i, i + 16) order
                const uint32_t xl = xrow + run * 32 + 8 * t;
                int d4[4];
                mma_s8(d4, e2m1x2_4(wg), e2m1x2_4(wh), e2m1x2_4(wg >> 16), e2m1x2_4(wh >> 16), lds32(xl), lds32(xl + 4));
                const float fg = e8m0_half(lds_u8(s0 + (u - cu0) * 16 + r)), fh = e8m0_half(lds_u8(s8 + (u - cu0) * 16 + r));
                const float2 dx = *(const float2*)(sdT + run * 8 + 2 * t);
                acc[0] += fg * dx.x * i2f(d4[0]);
                acc[1] += fg * dx.y * i2f(d4[1]);
                acc[2] += fh * dx.x * i2f(d4[2]);
                acc[3] += fh * dx.y * i2f(d4[3]);
            }
        }
    } else {   // FK_Q6_K
        const uint32_t h0 = stage + a.m_spo[1] + g * a.m_srs[1], h8 = h0 + 8 * a.m_srs[1];
        const uint32_t c0 = stage + a.m_spo[2] + g * a.m_srs[2], c8 = c0 + 8 * a.m_srs[2];
        const uint32_t d0 = stage + a.m_spo[3] + g * a.m_srs[3], d8 = d0 + 8 * a.m_srs[3];
        for (int u = cu0; u < cu1; u++) {
            const float dg = fk_h2f((uint16_t)lds_u16(d0 + u * 2)), dh = fk_h2f((uint16_t)lds_u16(d8 + u * 2));   // the whole row's super-scales are staged
            const uint4 scg = lds16(c0 + (u - cu0) * 16), sch = lds16(c8 + (u - cu0) * 16);
            const uint32_t sgw[4] = {scg.x, scg.y, scg.z, scg.w}, shw[4] = {sch.x, sch.y, sch.z, sch.w};
#pragma unroll
            for (int hf = 0; hf < 2; hf++) {
                const uint32_t qh_o = (u - cu0) * 64 + 32 * hf + 4 * t;
                const uint32_t hg0 = lds32(h0 + qh_o), hg1 = lds32(h0 + qh_o + 16), hh0 = lds32(h8 + qh_o), hh1 = lds32(h8 + qh_o + 16);
#pragma unroll
                for (int e = 0; e < 4; e++) {      // elements 128 hf + 32 e ..: ql bytes 64 hf + 32 (e & 1) + l, nibble e >> 1, qh bits 2e
                    const uint32_t ql_o = (u - cu0) * 128 + 64 * hf + 32 * (e & 1) + 4 * t;
                    const int sh = 4 * (e >> 1);
                    const uint32_t lg0 = lds32(r0 + ql_o), lg1 = lds32(r0 + ql_o + 16), lh0 = lds32(r8 + ql_o), lh1 = lds32(r8 + ql_o + 16);
                    const uint32_t ag0 = q6_signed(((lg0 >> sh) & 0x0F0F0F0Fu) | (((hg0 >> (2 * e)) & 0x03030303u) << 4));
                    const uint32_t ag1 = q6_signed(((lg1 >> sh) & 0x0F0F0F0Fu) | (((hg1 >> (2 * e)) & 0x03030303u) << 4));
                    const uint32_t ah0 = q6_signed(((lh0 >> sh) & 0x0F0F0F0Fu) | (((hh0 >> (2 * e)) & 0x03030303u) << 4));
                    const uint32_t ah1 = q6_signed(((lh1 >> sh) & 0x0F0F0F0Fu) | (((hh1 >> (2 * e)) & 0x03030303u) << 4));
                    const int run = u * 8 + hf * 4 + e;
                    const uint32_t xl = xrow + run * 32 + 4 * t;
                    const uint32_t b0 = lds32(xl), b1 = lds32(xl + 16);
                    int dl[4], dh4[4];
                    mma_s8(dl, ag0, ah0, 0u, 0u, b0, b1);     // the first 16 of the run: scale 8 hf + 2 e
                    mma_s8(dh4, 0u, 0u, ag1, ah1, b0, b1);    // the second 16: scale 8 hf + 2 e + 1
                    const int si = 8 * hf + 2 * e;
                    const float fgl = dg * (float)(int8_t)(sgw[si >> 2] >> (8 * (si & 3))), fgh = dg * (float)(int8_t)(sgw[si >> 2] >> (8 * (si & 3) + 8));
                    const float fhl = dh * (float)(int8_t)(shw[si >> 2] >> (8 * (si & 3))), fhh = dh * (float)(int8_t)(shw[si >> 2] >> (8 * (si & 3) + 8));
                    const float2 dx = *(const float2*)(sdT + run * 8 + 2 * t);
                    acc[0] += dx.x * (fgl * i2f(dl[0]) + fgh * i2f(dh4[0]));
                    acc[1] += dx.y * (fgl * i2f(dl[1]) + fgh * i2f(dh4[1]));
                    acc[2] += dx.x * (fhl * i2f(dl[2]) + fhh * i2f(dh4[2]));
                    acc[3] += dx.y * (fhl * i2f(dl[3]) + fhh * i2f(dh4[3]));
                }
            }
        }
    }
}

// The activations of the tensor-core form are quantized ONCE per launch by this kernel
// (a block per batch row), not by every block of the matvec: it writes the exact image
// of the matvec's activation region -- int8 rows `xs` bytes apart (16 more than a row,
// so the eight batch rows of a B fragment fall on different banks), then the stored
// scales as [run][8] and, for Q4_K, scale * run sum as [run][8] -- and each matvec
// block pulls the image in with one bulk copy.  RMSNorm and the gated activation ride
// here when asked for.
constexpr int IMG_THREADS = 1024;
template <int KIND>
__global__ void __launch_bounds__(IMG_THREADS) act_image_kernel(const GemvArgs a, uint8_t* __restrict__ img) {
    const int cols = a.cols, nb32 = cols >> 5, c4 = cols >> 2, b = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int8_t* sq = (int8_t*)img;
    float* sdT = (float*)(img + a.m_sd_off);
    float* ssT = sdT + nb32 * 8;
    const float* x = a.x + (size_t)b * a.x_ld;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __shared__ double s_part[IMG_THREADS / 32];
    __shared__ float s_scale;
    if (a.norm_w) {
        double sqs = 0.0;
        for (int i = threadIdx.x; i < c4; i += IMG_THREADS) {
            const float4 v = __ldcg((const float4*)x + i);   // past L1: the previous kernel of the stream may have written x while this block was resident
            sqs += (double)(v.x * v.x) + (double)(v.y * v.y) + (double)(v.z * v.z) + (double)(v.w * v.w);
        }
        for (int o = 16; o > 0; o >>= 1) sqs += __shfl_xor_sync(0xffffffffu, sqs, o);
        if (lane == 0) s_part[warp] = sqs;
        __syncthreads();
        if (threadIdx.x == 0) {
            double tsum = 0.0;
            for (int i = 0; i < IMG_THREADS / 32; i++) tsum += s_part[i];
            s_scale = 1.0f / sqrtf((float)(tsum / (double)cols) + a.norm_eps);
        }
        __syncthreads();
    }
    // c4 is a multiple of 8, so the eight lanes of a run always hold the same run
    for (int base = 0; base < c4; base += IMG_THREADS) {
        const int k4 = base + (int)threadIdx.x;
        const bool ok = k4 < c4;
        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (ok) {
            v = __ldcg((const float4*)x + k4);
            if (a.norm_w) {
                const float4 nw = __ldg((const float4*)a.norm_w + k4);
                const float sc = s_scale;
                v.x = v.x * sc * nw.x; v.y = v.y * sc * nw.y; v.z = v.z * sc * nw.z; v.w = v.w * sc * nw.w;
            }
            if (a.glu_up) {
                const float4 up = __ldcg((const float4*)(a.glu_up + (size_t)b * a.x_ld) + k4);
                float gt[4] = {v.x, v.y, v.z, v.w};
                const float uu[4] = {up.x, up.y, up.z, up.w};
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    if (a.glu_act == 0) {
                        gt[e] = (gt[e] / (1.0f + expf(-gt[e]))) * uu[e];
                    } else {
                        const float xg = fminf(gt[e], 7.0f), yu = fminf(fmaxf(uu[e], -7.0f), 7.0f);
                        gt[e] = (xg / (1.0f + expf(1.702f * -xg))) * (yu + 1.0f);
                    }
                }
                v = make_float4(gt[0], gt[1], gt[2], gt[3]);
            }
        }
        const int kb = k4 >> 3, quad = k4 & 7;
        unsigned mb = __float_as_uint(fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        mb = max(mb, __shfl_xor_sync(0xffffffffu, mb, 1));
        mb = max(mb, __shfl_xor_sync(0xffffffffu, mb, 2));
        mb = max(mb, __shfl_xor_sync(0xffffffffu, mb, 4));
        const float amax = __uint_as_float(mb);
        const float d = amax / 127.0f;
        int q0 = 0, q1 = 0, q2 = 0, q3 = 0;
        if (amax != 0.0f) {
            q0 = (int)roundf(v.x / d);
            q1 = (int)roundf(v.y / d);
            q2 = (int)roundf(v.z / d);
            q3 = (int)roundf(v.w / d);
        }
        int qsum = q0 + q1 + q2 + q3;
        qsum += __shfl_xor_sync(0xffffffffu, qsum, 1);
        qsum += __shfl_xor_sync(0xffffffffu, qsum, 2);
        qsum += __shfl_xor_sync(0xffffffffu, qsum, 4);
        if (ok) {
            int8_t* rowq = sq + (size_t)b * a.m_xs + kb * 32;
            if (KIND == FK_MXFP4) {
                // a run is kept as (elem j, elem j + 16) pairs: the order the nibble decode produces bytes in
                const int e = 4 * quad;
                const int qv[4] = {q0, q1, q2, q3};
#pragma unroll
                for (int i = 0; i < 4; i++) rowq[(((e + i) & 15) << 1) | ((e + i) >> 4)] = (int8_t)qv[i];
            } else {
                *(uint32_t*)(rowq + 4 * quad) = (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) | ((uint32_t)(q2 & 0xFF) << 16) | ((uint32_t)(q3 & 0xFF) << 24);
            }
            if (quad == 0) {
                const float dq = fk_h2f(fk_f2h(d));
                sdT[kb * 8 + b] = dq;
                if (KIND == FK_Q4_K) ssT[kb * 8 + b] = dq * (float)qsum;
            }
        }
    }
}

template <int KIND>
__global__ void __launch_bounds__(GEMV_THREADS, 1) gemv_mma_kernel(const GemvArgs a, const uint8_t* __restrict__ img,
                                                                   const __grid_constant__ CUtensorMap wmap) {
    extern __shared__ __align__(128) uint8_t smem[];
    TR(0, threadIdx.x == 0);
    const int cols = a.cols, rows = a.rows, nb32 = cols >> 5, batch = a.batch;
    const int xs = a.m_xs;
    int8_t* sq = (int8_t*)smem;                        // [batch][xs] int8
    float* sdT = (float*)(smem + a.m_sd_off);           // [nb32][8] stored scale, widened
    float* ssT = sdT + nb32 * 8;                        // Q4_K: [nb32][8] scale * run sum
    float4* red = (float4*)(smem + a.m_red_off);        // [2][warps][32] partial sums of the K parts
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint8_t* wb = a.w + (size_t)a.mat * a.mat_stride;
    float* y = a.y;

    const uint32_t sbase = smem_u32(smem);
    const uint32_t ring = sbase + a.act_bytes + warp * (a.nstages * a.stage_bytes);
    const uint32_t bars = sbase + a.act_bytes + GEMV_WARPS * (a.nstages * a.stage_bytes) + warp * (MAX_STAGES * 8);
    const uint32_t xbar = sbase + a.act_bytes + GEMV_WARPS * (a.nstages * a.stage_bytes) + GEMV_WARPS * (MAX_STAGES * 8);
    if (lane == 0) {
        for (int s = 0; s < a.nstages; s++) mbar_init(bars + 8 * s, 1);
        if (warp == 0) mbar_init(xbar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    constexpr int UNIT = MGeo<KIND>::UNIT, P = MGeo<KIND>::PLANES;
    const int KS = a.m_ks, gi = warp / KS, kp = warp % KS, GPR = GEMV_WARPS / KS;
    const int ngroups = (rows + MM_ROWS - 1) / MM_ROWS;
    const int units = (cols + UNIT - 1) / UNIT;
    const int u0 = min(units, kp * a.m_kpart_units), u1 = min(units, u0 + a.m_kpart_units);
    const int nch = (u1 - u0 + a.m_chunk_units - 1) / a.m_chunk_units;       // 0 for a part past the end of K
    const int first = gi * gridDim.x + blockIdx.x, gstride = GPR * gridDim.x;
    const int nrounds = first < ngroups ? (ngroups - first + gstride - 1) / gstride : 0;
    const int njobs = nrounds * nch;

    // ---- filling a stage: up to two (row, plane) pieces per lane
    constexpr int NPIECE = (MM_ROWS * P + 31) / 32;
    uint32_t f_dst[NPIECE], f_ub[NPIECE], f_pstride[NPIECE];
    const uint8_t* f_src[NPIECE];
    int f_r[NPIECE];
    bool f_whole[NPIECE];
#pragma unroll
    for (int i = 0; i < NPIECE; i++) {
        const int c = lane + 32 * i, r = c / P, p = c % P;
        f_r[i] = c < MM_ROWS * P ? r : -1;
        f_whole[i] = KIND == FK_Q6_K && p == 3;
        const size_t poff = p == 0 ? a.plane_off[0] : p == 1 ? a.plane_off[1] : p == 2 ? a.plane_off[2] : a.plane_off[3];
        f_pstride[i] = (uint32_t)(p == 0 ? a.plane_stride[0] : p == 1 ? a.plane_stride[1] : p == 2 ? a.plane_stride[2] : a.plane_stride[3]);
        f_ub[i] = (uint32_t)unit_bytes<KIND>(p);
        const int srs = p == 0 ? a.m_srs[0] : p == 1 ? a.m_srs[1] : p == 2 ? a.m_srs[2] : a.m_srs[3];
        const int spo = p == 0 ? a.m_spo[0] : p == 1 ? a.m_spo[1] : p == 2 ? a.m_spo[2] : a.m_spo[3];
        f_dst[i] = (uint32_t)(spo + r * srs);
        f_src[i] = wb + poff + (size_t)r * f_pstride[i];
    }
    int f_stage = 0, f_ch = 0, f_group = first;
    auto fill = [&]() {
        const uint32_t stage = ring + f_stage * a.stage_bytes, bar = bars + 8 * f_stage;
        const int cu0 = u0 + f_ch * a.m_chunk_units, cu1 = min(u1, cu0 + a.m_chunk_units);
        if (KIND == FK_Q4_K) {
            // the 16 rows x chunk of blocks as ONE tiled copy (the matrix is a [rows][row words] tensor);
            // the box always has the full size: rows or blocks past the end arrive as zeros
            if (lane == 0) {
                mbar_expect_tx(bar, (uint32_t)a.stage_bytes);
                asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                             ::"r"(stage), "l"(&wmap), "r"(cu0 * 36), "r"(f_group * MM_ROWS), "r"(bar) : "memory");
            }
            if (++f_stage == a.nstages) f_stage = 0;
            if (++f_ch == nch) { f_ch = 0; f_group += gstride; }
            return;
        }
        uint32_t off[NPIECE], bytes[NPIECE], mine = 0;
#pragma unroll
        for (int i = 0; i < NPIECE; i++) {
            off[i] = 0;
            bytes[i] = 0;
            if (f_r[i] >= 0 && f_group * MM_ROWS + f_r[i] < rows) {
                if (f_whole[i]) {
                    bytes[i] = f_pstride[i];
                } else {
                    off[i] = (uint32_t)cu0 * f_ub[i];
                    bytes[i] = (uint32_t)(cu1 - cu0) * f_ub[i];
                    if (off[i] + bytes[i] > f_pstride[i]) bytes[i] = f_pstride[i] - off[i];   // the ragged end of a row (strides are padded to 16)
                }
                mine += bytes[i];
            }
        }
        const uint32_t total = __reduce_add_sync(0xffffffffu, mine);
        if (lane == 0) mbar_expect_tx(bar, total);
        __syncwarp();
#pragma unroll
        for (int i = 0; i < NPIECE; i++)
            if (bytes[i]) bulk_g2s(stage + f_dst[i], f_src[i] + (size_t)f_group * MM_ROWS * f_pstride[i] + off[i], bytes[i], bar);
        if (++f_stage == a.nstages) f_stage = 0;
        if (++f_ch == nch) { f_ch = 0; f_group += gstride; }
    };
    const int pre = njobs < a.nstages ? njobs : a.nstages;
    for (int q = 0; q < pre; q++) fill();
    TR(1, threadIdx.x == 0);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // ---- the activation image: one bulk copy, every thread waits for it
    if (threadIdx.x == 0) {
        mbar_expect_tx(xbar, (uint32_t)a.m_red_off);
        bulk_g2s(sbase, img, (uint32_t)a.m_red_off, xbar);
    }
    mbar_wait(xbar, 0, a.err);
    TR(3, threadIdx.x == 0);

    const int g = lane >> 2, t = lane & 3;
    const uint32_t xrow = smem_u32(sq) + (uint32_t)min(g, batch - 1) * xs;   // columns past the batch re-read its last row; their sums are dropped
    int s = 0, group = first;
    uint32_t phase = 0;
    for (int round = 0; round < nrounds; round++) {
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int ch = 0; ch < nch; ch++) {
            mbar_wait(bars + 8 * s, phase, a.err);
            TR(4, threadIdx.x == 0 && round == 0 && ch == 0);
            const int cu0 = u0 + ch * a.m_chunk_units, cu1 = min(u1, cu0 + a.m_chunk_units);
            mma_eat<KIND>(a, ring + s * a.stage_bytes, cu0, cu1, xrow, sdT, ssT, nb32, lane, acc);
            __syncwarp();
            TR(5, threadIdx.x == 0 && round == 0 && ch == 0);
            if ((round * nch + ch) + a.nstages < njobs) fill();
            if (++s == a.nstages) { s = 0; phase ^= 1u; }
        }
        if (KS > 1) {
            float4* rb = red + (round & 1) * (GEMV_WARPS * 32);
            rb[warp * 32 + lane] = make_float4(acc[0], acc[1], acc[2], acc[3]);
            asm volatile("bar.sync %0, %1;" ::"r"(1 + gi), "r"(KS * 32) : "memory");
            if (kp == 0) {
                for (int j = 1; j < KS; j++) {
                    const float4 o = rb[(warp + j) * 32 + lane];
                    acc[0] += o.x; acc[1] += o.y; acc[2] += o.z; acc[3] += o.w;
                }
            }
        }
        if (kp == 0) {
            const int rg = group * MM_ROWS + g;
            if (a.pair_glu) {
                // (gate, up) row pairs sit in neighbouring g, i.e. in lanes 4 apart
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float other = __shfl_xor_sync(0xffffffffu, acc[i], 4);
                    const int row = rg + 8 * (i >> 1), b = 2 * t + (i & 1);
                    if (!(g & 1) && row + 1 < rows && b < batch) {
                        const float gt = acc[i], up = other;
                        float o;
                        if (a.pair_glu == 1) {
                            o = (gt / (1.0f + expf(-gt))) * up;
                        } else {
                            const float xg = fminf(gt, 7.0f), yu = fminf(fmaxf(up, -7.0f), 7.0f);
                            o = (xg / (1.0f + expf(1.702f * -xg))) * (yu + 1.0f);
                        }
                        y[(size_t)b * (rows >> 1) + (row >> 1)] = o;
                    }
                }
            } else {
                if (a.ar_on) {
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int row = rg + 8 * (i >> 1), b = 2 * t + (i & 1);
                        if (row < rows && b < batch) fk_ar_send(a.ar, b * rows + row, acc[i]);
                    }
                }
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int row = rg + 8 * (i >> 1), b = 2 * t + (i & 1);
                    if (row < rows && b < batch) {
                        float v = acc[i];
                        if (a.ar_on) v = fk_ar_recv(a.ar, b * rows + row, fk_ar_sent(a.ar)[b * rows + row], v, a.err);
                        float* dst = y + (size_t)b * rows + row;
                        *dst = a.accumulate ? *dst + v : v;
                    }
                }
            }
        }
        group += gstride;
    }
    TR(6, threadIdx.x == 0);
    TRMAX(7, lane == 0);
}

size_t act_smem_bytes(int kind, int nb, int cols) {
    size_t s = (size_t)nb * cols + (size_t)nb * (cols / 32) * 4;
    if (kind == FK_Q4_K) s += (size_t)nb * (cols / 32) * 4;
    if (kind == FK_Q6_K) s += (size_t)nb * (cols / 16) * 4;
    return (s + 127) & ~(size_t)127;
}

// Bytes of one row's share of a stage that covers `t` trips.
template <int KIND>
int row_stage_bytes(const fk_weight_s* w, int t) {
    int b = 0;
    for (int p = 0; p < 3; p++) b += trip_bytes<KIND>(p) * t;
    if (KIND == FK_Q6_K) b += (int)w->plane_stride[3];
    return b;
}

template <int KIND, int NB, bool DUMP>
int launch_one(fk_ctx* ctx, cudaStream_t st, GemvArgs a, const fk_weight_s* w, int slots) {
    const int act = (int)act_smem_bytes(KIND, NB, a.cols);
    const int bars = DP_WARPS * MAX_STAGES * 8;
    const int ntrips = (a.cols + Geo<KIND>::TRIP_COLS - 1) / Geo<KIND>::TRIP_COLS;
    // the largest K chunk that still leaves a ring of two stages (a whole row when it
    // fits): bulk copies pay a fixed cost each, and small ones (a trip of Q6_K's
    // scale planes is 64 and 32 bytes) cost more than the overlap they would buy
    constexpr int RS = Geo<KIND>::ROWS;
    const int ring_budget = (DP_SMEM_BUDGET - act - bars) / DP_WARPS;   // bytes of ring a warp may have
    int t = ntrips;
    while (t > 1 && 2 * RS * row_stage_bytes<KIND>(w, t) > ring_budget) t--;
    if (ring_budget <= 0 || 2 * RS * row_stage_bytes<KIND>(w, t) > ring_budget)
        return fk_fail(FK_UNSUPPORTED, "gemv: %d columns x batch %d does not fit shared memory", a.cols, NB);
    a.trips_per_chunk = t;
    a.nchunks = (ntrips + t - 1) / t;
    a.row_bytes_stage = row_stage_bytes<KIND>(w, t);
    a.stage_bytes = RS * a.row_bytes_stage;
    a.nstages = ring_budget / a.stage_bytes;
    if (a.nstages > MAX_STAGES) a.nstages = MAX_STAGES;
    a.act_bytes = act;
    const size_t smem = (size_t)act + (size_t)DP_WARPS * a.nstages * a.stage_bytes + bars;
    auto kern = gemv_kernel<KIND, NB, DUMP>;
    {
        // raise the kernel's dynamic shared-memory limit only when this launch needs more than any
        // before it on this device (the call costs about as much as the launch itself)
        static std::atomic<int> granted[64];
        const int dev = ctx->device & 63;
        if ((int)smem > granted[dev].load(std::memory_order_relaxed)) {
            FK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), FK_KERNEL);
            granted[dev].store((int)smem, std::memory_order_relaxed);
        }
    }
    const int pairs = (a.rows + RS - 1) / RS;
    const int need = (pairs + 3) / 4;   // at least four row groups a block, else the activation quantization dominates
    // a persistent grid: one block per SM, shared out over the slots
    int per_slot = ctx->sm_count / slots;
    if (per_slot < 1) per_slot = 1;
    dim3 grid((unsigned)(need < per_slot ? need : per_slot), (unsigned)slots);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(DP_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    FK_CUDA(cudaLaunchKernelEx(&cfg, kern, a), FK_LAUNCH);
    ctx->launches++;
    return FK_OK;
}

// Plan and launch of gemv_q4k_kernel; *fits = false (nothing launched) when even two rows a stage
// do not fit beside the activations, and the caller takes the general kernel.
template <int NB, bool DUMP>
int launch_q4k(fk_ctx* ctx, cudaStream_t st, GemvArgs a, const fk_weight_s* w, int slots, bool* fits) {
    *fits = false;
    const int nsb = a.cols / 256;
    const size_t rb = w->plane_stride[0];
    const size_t fixed = (size_t)NB * a.cols + (size_t)NB * nsb * 64 + 64 + 128;   // activations, run scales, barrier, alignment
    const size_t per_pair = 2 * rb + 16 + 2 * (size_t)nsb * NB * 4;                 // a row pair's bytes (padded) and its partial sums
    int per_slot = ctx->sm_count / slots;
    if (per_slot < 1) per_slot = 1;
    // The block's whole share of the matrix must fit its shared memory (half an SM's when possible,
    // so that consecutive launches overlap): nothing is then left to request after the start.
    // Larger matrices amortise their start-up anyway and take the general kernel.
    const int npairs = (a.rows + 1) / 2;
    const int G = std::min(per_slot, (npairs + 3) / 4);
    const int ppb = (npairs + G - 1) / G;      // most row pairs a block gets
    size_t budget = 0;
    for (size_t b : {(size_t)HALF_SM_SMEM, (size_t)SMEM_BUDGET})
        if (!budget && fixed + (size_t)ppb * per_pair <= b) budget = b;
    if (!budget) return FK_OK;
    *fits = true;
    const int T = Q4_MAX_THREADS;
    // lanes of a warp over row pairs (the rest over super-blocks): the split that leaves fewest lanes idle
    int lp = 32, best = INT_MAX;
    for (int c : {32, 16, 8}) {
        const int ls = 32 / c, tiles = ((ppb + c - 1) / c) * ((nsb + ls - 1) / ls);
        const int rounds = (tiles + T / 32 - 1) / (T / 32);
        if (rounds < best) { best = rounds; lp = c; }
    }
    a.q_lp = lp;
    a.q_sc_off = NB * a.cols;
    a.q_part_off = a.q_sc_off + NB * nsb * 64;
    a.q_ring_off = (int)(((size_t)a.q_part_off + 2 * (size_t)ppb * nsb * NB * 4 + 127) & ~(size_t)127);
    a.q_bar_off = a.q_ring_off + (int)((size_t)ppb * (2 * rb + 16));
    const size_t smem = (size_t)a.q_bar_off + 64;
    auto kern = gemv_q4k_kernel<NB, DUMP>;
    {
        static std::atomic<int> granted[64];
        const int dev = ctx->device & 63;
        if ((int)smem > granted[dev].load(std::memory_order_relaxed)) {
            FK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), FK_KERNEL);
            // all of the SM's L1 as shared memory, or two half-SM blocks do not fit together
            FK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared), FK_KERNEL);
            granted[dev].store((int)smem, std::memory_order_relaxed);
        }
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)G);
    cfg.blockDim = dim3((unsigned)T);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    FK_CUDA(cudaLaunchKernelEx(&cfg, kern, a), FK_LAUNCH);
    ctx->launches++;
    return FK_OK;
}

// Plan and launch of the tensor-core form; returns FK_UNSUPPORTED (quietly) when a
// stage of one unit does not fit, and the caller falls back to the dp4a form.
template <int KIND>
int launch_mma(fk_ctx* ctx, cudaStream_t st, GemvArgs a, const fk_weight_s* w, bool* fits) {
    constexpr int UNIT = MGeo<KIND>::UNIT, P = MGeo<KIND>::PLANES;
    *fits = false;
    const int units = (a.cols + UNIT - 1) / UNIT, nb32 = a.cols / 32;
    const int ngroups = (a.rows + MM_ROWS - 1) / MM_ROWS;
    int ks = 1;
    while (ks < GEMV_WARPS && ngroups * ks * 2 <= ctx->sm_count * GEMV_WARPS && ks * 2 <= units) ks *= 2;
    a.m_ks = ks;
    a.m_kpart_units = (units + ks - 1) / ks;
    a.m_xs = a.cols + 16;
    size_t act = (size_t)a.batch * a.m_xs;
    act = (act + 15) & ~(size_t)15;
    a.m_sd_off = (int)act;
    act += (size_t)nb32 * 32 * (KIND == FK_Q4_K ? 2 : 1);
    act = (act + 15) & ~(size_t)15;
    a.m_red_off = (int)act;
    act += 2 * GEMV_WARPS * 32 * 16;
    act = (act + 127) & ~(size_t)127;
    const int bars = GEMV_WARPS * MAX_STAGES * 8 + 16;   // + the barrier of the activation image
    const int ring_budget = ((int)SMEM_BUDGET - (int)act - bars) / GEMV_WARPS;
    auto layout = [&](int cu, int* srs, int* spo) {
        int off = 0;
        for (int p = 0; p < P; p++) {
            int b = (KIND == FK_Q6_K && p == 3) ? (int)w->plane_stride[3] : cu * unit_bytes<KIND>(p);
            b = (b + 15) & ~15;
            // rows 16 mod 32 bytes apart: the eight rows of a fragment load hit different banks
            // (Q4_K arrives as a dense tile: an odd number of 144-byte blocks per chunk does it)
            if ((b & 31) == 0 && KIND != FK_Q4_K) b += 16;
            srs[p] = b;
            spo[p] = off;
            off += MM_ROWS * b;
        }
        return off;
    };
    int srs[4] = {0, 0, 0, 0}, spo[4] = {0, 0, 0, 0};
    int cu = a.m_kpart_units;
    if (KIND == FK_Q4_K) {
        if (cu > 7) cu = 7;                 // a tile is at most 256 words wide
        if ((cu & 1) == 0) cu--;
        while (cu > 1 && 2 * layout(cu, srs, spo) > ring_budget) cu -= 2;
    } else {
        while (cu > 1 && 2 * layout(cu, srs, spo) > ring_budget) cu--;
    }
    const int stage = layout(cu, srs, spo);
    if (ring_budget <= 0 || stage > ring_budget) return FK_UNSUPPORTED;
    *fits = true;
    a.m_chunk_units = cu;
    for (int p = 0; p < 4; p++) { a.m_srs[p] = srs[p]; a.m_spo[p] = spo[p]; }
    a.stage_bytes = stage;
    a.nstages = ring_budget / stage;
    if (a.nstages > MAX_STAGES) a.nstages = MAX_STAGES;
    a.act_bytes = (int)act;
    const size_t smem = act + (size_t)GEMV_WARPS * a.nstages * a.stage_bytes + bars;
    auto kern = gemv_mma_kernel<KIND>;
    {
        // raise the kernel's dynamic shared-memory limit only when this launch needs more than any
        // before it on this device (the call costs about as much as the launch itself)
        static std::atomic<int> granted[64];
        const int dev = ctx->device & 63;
        if ((int)smem > granted[dev].load(std::memory_order_relaxed)) {
            FK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), FK_KERNEL);
            granted[dev].store((int)smem, std::memory_order_relaxed);
        }
    }
    // the activation image lives in the context's scratch block (stream-ordered like its other users)
    const int rcs = fk_ensure_scratch(ctx, st, (size_t)a.m_red_off);
    if (rcs != FK_OK) return rcs;
    const uint8_t* img = ctx->scratch;
    const int gpr = GEMV_WARPS / ks;
    int blocks = (ngroups + gpr - 1) / gpr;
    if (blocks > ctx->sm_count) blocks = ctx->sm_count;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(GEMV_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchConfig_t icfg = cfg;
    icfg.gridDim = dim3((unsigned)a.batch);
    icfg.blockDim = dim3(IMG_THREADS);
    icfg.dynamicSmemBytes = 0;
    alignas(64) CUtensorMap wmap;
    memset(&wmap, 0, sizeof(wmap));
    if (KIND == FK_Q4_K) {
        const int rcm = fk_make_map_u32(&wmap, (void*)(w->dev + (size_t)a.mat * w->mat_stride + w->plane_off[0]), w->plane_stride[0] / 4,
                                        (uint64_t)a.rows, (uint32_t)(36 * cu), MM_ROWS);
        if (rcm != FK_OK) return rcm;
    }
    FK_CUDA(cudaLaunchKernelEx(&icfg, act_image_kernel<KIND>, a, ctx->scratch), FK_LAUNCH);
    FK_CUDA(cudaLaunchKernelEx(&cfg, kern, a, img, wmap), FK_LAUNCH);
    ctx->launches += 2;
    return FK_OK;
}

template <int KIND>
int launch_kind(fk_ctx* ctx, cudaStream_t st, const GemvArgs& a, const fk_weight_s* w, int slots, bool dump) {
    if (!dump && a.batch >= MMA_MIN_BATCH && slots == 1 && !a.ids && !a.bias) {
        bool fits = false;
        const int rc = launch_mma<KIND>(ctx, st, a, w, &fits);
        if (fits) return rc;
    }
    // The block-owned Q4_K kernel takes the plain matvec (and the integer test hook): in a chain of those it is
    // 4.3 us against 5.4 us a launch (8192 x 3072).  It waits for its whole share before the first dot product, which
    // costs it inside a decoder step, where the kernel before a matvec is short and hides nothing (688 against 798
    // tokens per second on the 3B Llama shape): the fused and indexed forms keep the general kernel and its rings.
    const bool plain = !a.ids && !a.n_active && !a.norm_w && !a.glu_up && !a.pair_glu && !a.accumulate && !a.ar_on && !a.bias;
    if (KIND == FK_Q4_K && a.batch <= 1 && (plain || dump)) {
        bool fits = false;
        const int rc = dump ? launch_q4k<1, true>(ctx, st, a, w, slots, &fits) : launch_q4k<1, false>(ctx, st, a, w, slots, &fits);
        if (fits || rc != FK_OK) return rc;
    }
    if (dump) return launch_one<KIND, 1, true>(ctx, st, a, w, slots);
    if (a.batch <= 1) return launch_one<KIND, 1, false>(ctx, st, a, w, slots);
    if (a.batch <= 2) return launch_one<KIND, 2, false>(ctx, st, a, w, slots);
    if (a.batch <= 4) return launch_one<KIND, 4, false>(ctx, st, a, w, slots);
    return launch_one<KIND, 8, false>(ctx, st, a, w, slots);
}

// ---- standalone q8_1 quantizer (36-byte blocks), one warp per run
__global__ void quantize_q8_1_kernel(const float* __restrict__ x, int n_runs, uint8_t* __restrict__ y) {
    const int run = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (run >= n_runs) return;
    const float v = x[(size_t)run * 32 + lane];
    float d_w;
    int qsum;
    const int q = fk_q8_1_lane(v, &d_w, &qsum);
    const float sum = fk_warp_sum(v);  // xor butterfly 16..1, the order the stored sum is defined by
    uint8_t* blk = y + (size_t)run * 36;
    blk[4 + lane] = (uint8_t)(int8_t)q;
    if (lane == 0) {
        *(uint16_t*)blk = fk_f2h(d_w);  // d_w is the f16 scale widened: the conversion back is exact
        *(uint16_t*)(blk + 2) = fk_f2h(sum);
    }
}

}  // namespace

int fk_gemv_launch(fk_ctx* ctx, cudaStream_t st, fk_weight w, const int* ids_dev, int mat, int slots,
                   const float* x_dev, int x_stride, int batch, float* y_dev, int32_t* isums_dev, const int* n_active_dev,
                   const FkGemvFused* fused) {
    GemvArgs a{};
#ifdef FK_TRACE
    static int trace_seq = 0;
    a.trace_slot = trace_seq++;
#endif
    a.n_active = n_active_dev;
    a.x_ld = w->cols;
    if (fused) {
        a.norm_w = fused->norm_w;
        a.norm_eps = fused->norm_eps;
        a.glu_up = fused->glu_up;
        a.glu_act = fused->glu_act;
        a.accumulate = fused->accumulate;
        a.pair_glu = fused->pair_glu;
        if (fused->x_ld) a.x_ld = fused->x_ld;
        a.bias = fused->bias;
        if (fused->w2) {
            a.w2 = fused->w2->dev;
            a.split = slots / 2;
            a.bias2 = fused->bias2;
        }
        a.x_ready = fused->x_ready;
        if (fused->ar) {
            a.ar_on = 1;
            a.ar = *fused->ar;
        }
    }
    a.w = w->dev;
    a.mat_stride = w->mat_stride;
    for (int i = 0; i < 4; i++) {
        a.plane_off[i] = w->plane_off[i];
        a.plane_stride[i] = w->plane_stride[i];
    }
    a.ids = ids_dev;
    a.mat = mat;
    a.x = x_dev;
    a.x_stride = x_stride;
    a.y = y_dev;
    a.rows = w->rows;
    a.cols = w->cols;
    a.batch = batch;
    a.isums = isums_dev;
    a.err = ctx->err_flag;
    const bool dump = isums_dev != nullptr;
    switch (w->kind) {
        case FK_Q4_K: return launch_kind<FK_Q4_K>(ctx, st, a, w, slots, dump);
        case FK_BF16:
            // nothing is quantized (no integer hook); the norm, bias and add-into forms are built, the gated, indexed and
            // row-split ones are not
            if (ids_dev || n_active_dev || isums_dev || (fused && (fused->glu_up || fused->pair_glu || fused->ar)))
                return fk_fail(FK_UNSUPPORTED, "gemv: BF16 has the plain matvec with an optional norm, bias and add-into only");
            return fk_gemv_bf16_launch(ctx, st, w, mat, x_dev, a.x_ld, batch, y_dev, a.norm_w, a.norm_eps, a.bias, a.accumulate);
        case FK_Q5_K:
            // the plain matvec only: the fused, indexed and row-split forms have no Q5_K kernel (the caller composes them
            // from the separate kernels, as it would for any kind this library does not fuse)
            if (ids_dev || n_active_dev || fused) return fk_fail(FK_UNSUPPORTED, "gemv: Q5_K has the plain matvec only");
            return fk_gemv_q5k_launch(ctx, st, w, mat, x_dev, batch, y_dev, isums_dev);
        case FK_Q6_K: return launch_kind<FK_Q6_K>(ctx, st, a, w, slots, dump);
        case FK_Q8_0: return launch_kind<FK_Q8_0>(ctx, st, a, w, slots, dump);
        case FK_MXFP4: return launch_kind<FK_MXFP4>(ctx, st, a, w, slots, dump);
    }
    return fk_fail(FK_UNSUPPORTED, "gemv: kind %d has no kernel", w->kind);
}

FK_EXPORT int fk_quantize_q8_1(fk_ctx* ctx, void* stream, const float* x_dev, int n, uint8_t* y_dev) {
    if (!ctx || !x_dev || !y_dev || n < 0 || n % 32) return fk_fail(FK_INVALID, "quantize_q8_1: n=%d must be a multiple of 32", n);
    if (n == 0) return FK_OK;
    FkDeviceGuard g(ctx->device);
    const int runs = n / 32;
    quantize_q8_1_kernel<<<(runs + 7) / 8, 256, 0, (cudaStream_t)stream>>>(x_dev, runs, y_dev);
    FK_CUDA(cudaGetLastError(), FK_LAUNCH);
    ctx->launches++;
    return FK_OK;
}

// The same with host buffers (what `matvec_reads` of the reference-side crate calls): one upload, one download.
FK_EXPORT int fk_quantize_q8_1_host(fk_ctx* ctx, const float* x_host, int n, uint8_t* y_host) {
    if (!ctx || !x_host || !y_host || n < 0 || n % 32) return fk_fail(FK_INVALID, "quantize_q8_1_host: n=%d must be a multiple of 32", n);
    if (n == 0) return FK_OK;
    FkDeviceGuard g(ctx->device);
    float* xd = nullptr;
    uint8_t* yd = nullptr;
    const size_t yb = (size_t)n / 32 * 36;
    cudaError_t e = cudaMalloc(&xd, (size_t)n * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&yd, yb);
    if (e == cudaSuccess) e = cudaMemcpy(xd, x_host, (size_t)n * sizeof(float), cudaMemcpyHostToDevice);
    int rc = e == cudaSuccess ? fk_quantize_q8_1(ctx, nullptr, xd, n, yd) : fk_fail(FK_LAUNCH, "quantize_q8_1_host: %s", cudaGetErrorString(e));
    if (rc == FK_OK && (e = cudaMemcpy(y_host, yd, yb, cudaMemcpyDeviceToHost)) != cudaSuccess) rc = fk_fail(FK_LAUNCH, "quantize_q8_1_host: %s", cudaGetErrorString(e));
    cudaFree(xd);
    cudaFree(yd);
    return rc;
}

FK_EXPORT int fk_gemv(fk_ctx* ctx, void* stream, fk_weight w, int mat, const float* x_dev, int batch, float* y_dev) {
    if (!ctx || !w || !x_dev || !y_dev) return fk_fail(FK_INVALID, "gemv: null argument");
    if (batch < 1 || batch > 8) return fk_fail(FK_UNSUPPORTED, "gemv: batch %d outside 1..8 (use fk_gemm)", batch);
    if (mat < 0 || mat >= w->n_mats) return fk_fail(FK_INVALID, "gemv: matrix %d of %d", mat, w->n_mats);
    if ((uintptr_t)x_dev & 15) return fk_fail(FK_INVALID, "gemv: x_dev must be 16-byte aligned");
    FkDeviceGuard g(ctx->device);
    return fk_gemv_launch(ctx, (cudaStream_t)stream, w, nullptr, mat, 1, x_dev, 0, batch, y_dev, nullptr, nullptr, nullptr);
}

FK_EXPORT int fk_gemv_fused(fk_ctx* ctx, void* stream, fk_weight w, int mat, const float* x_dev, int x_ld, int batch, float* y_dev,
                            const float* norm_weight_dev, float norm_eps, const float* glu_up_dev, int glu_act, int accumulate, int pair_glu) {
    if (!ctx || !w || !x_dev || !y_dev) return fk_fail(FK_INVALID, "gemv_fused: null argument");
    if (pair_glu < 0 || pair_glu > 2 || (pair_glu && ((w->rows & 1) || accumulate)))
        return fk_fail(FK_INVALID, "gemv_fused: pair_glu %d needs an even number of rows and no accumulate", pair_glu);
    if (batch < 1 || batch > 8) return fk_fail(FK_UNSUPPORTED, "gemv_fused: batch %d outside 1..8", batch);
    if (mat < 0 || mat >= w->n_mats) return fk_fail(FK_INVALID, "gemv_fused: matrix %d of %d", mat, w->n_mats);
    if (x_ld == 0) x_ld = w->cols;
    if (x_ld < w->cols || (x_ld & 3)) return fk_fail(FK_INVALID, "gemv_fused: x_ld %d (columns %d, must be a multiple of 4)", x_ld, w->cols);
    if (((uintptr_t)x_dev & 15) || ((uintptr_t)glu_up_dev & 15) || ((uintptr_t)norm_weight_dev & 15))
        return fk_fail(FK_INVALID, "gemv_fused: inputs must be 16-byte aligned");
    if (glu_act < 0 || glu_act > 1) return fk_fail(FK_UNSUPPORTED, "gemv_fused: activation %d", glu_act);
    FkDeviceGuard g(ctx->device);
    FkGemvFused f{norm_weight_dev, norm_eps, glu_up_dev, glu_act, accumulate, x_ld, pair_glu, nullptr};
    return fk_gemv_launch(ctx, (cudaStream_t)stream, w, nullptr, mat, 1, x_dev, 0, batch, y_dev, nullptr, nullptr, &f);
}

// The row-split matvec of a tensor-parallel decode step with its all-reduce in the epilogue: every rank holds the
// columns [rank * cols, (rank + 1) * cols) of the full matrix as `w`, and
//   y[b][row] (+)= sum over ranks of W_rank x_rank
// -- the lane that finishes a row stores its partial into every peer's channel slot (NVLink) and adds what the peers
// stored here, in rank order, so every rank ends with the same bits.  One launch; the link's latency is paid once at
// the kernel's tail instead of a second kernel's launch, flag and wait.
FK_EXPORT int fk_gemv_fused_allreduce(fk_ctx* ctx, void* stream, fk_weight w, int mat, const float* x_dev, int x_ld, int batch, float* y_dev,
                                      const float* norm_weight_dev, float norm_eps, const float* glu_up_dev, int glu_act, int accumulate,
                                      fk_comm* comm, size_t channel_off, int n_max, int timeout_us) {
    if (!ctx || !w || !x_dev || !y_dev || !comm) return fk_fail(FK_INVALID, "gemv_fused_allreduce: null argument");
    if (batch < 1 || batch > 8) return fk_fail(FK_UNSUPPORTED, "gemv_fused_allreduce: batch %d outside 1..8", batch);
    if (mat < 0 || mat >= w->n_mats) return fk_fail(FK_INVALID, "gemv_fused_allreduce: matrix %d of %d", mat, w->n_mats);
    if (x_ld == 0) x_ld = w->cols;
    if (x_ld < w->cols || (x_ld & 3)) return fk_fail(FK_INVALID, "gemv_fused_allreduce: x_ld %d (columns %d, must be a multiple of 4)", x_ld, w->cols);
    if (((uintptr_t)x_dev & 15) || ((uintptr_t)glu_up_dev & 15) || ((uintptr_t)norm_weight_dev & 15))
        return fk_fail(FK_INVALID, "gemv_fused_allreduce: inputs must be 16-byte aligned");
    if (glu_act < 0 || glu_act > 1) return fk_fail(FK_UNSUPPORTED, "gemv_fused_allreduce: activation %d", glu_act);
    if ((long long)batch * w->rows > n_max) return fk_fail(FK_INVALID, "gemv_fused_allreduce: %d x %d values do not fit a channel of %d", batch, w->rows, n_max);
    FkDeviceGuard g(ctx->device);
    FkArChannel ch;
    const int rc = fk_ar_channel(comm, channel_off, n_max, timeout_us, &ch);
    if (rc) return rc;
    FkGemvFused f{norm_weight_dev, norm_eps, glu_up_dev, glu_act, accumulate, x_ld, 0, comm->world > 1 ? &ch : nullptr};
    return fk_gemv_launch(ctx, (cudaStream_t)stream, w, nullptr, mat, 1, x_dev, 0, batch, y_dev, nullptr, nullptr, &f);
}

FK_EXPORT int fk_gemv_multi(fk_ctx* ctx, void* stream, fk_weight w, const int* ids_dev, int k, const float* x_dev,
                            int x_stride, float* y_dev) {
    if (!ctx || !w || !ids_dev || !x_dev || !y_dev) return fk_fail(FK_INVALID, "gemv_multi: null argument");
    if (k < 1 || k > 65535) return fk_fail(FK_INVALID, "gemv_multi: k=%d", k);
    if (x_stride != 0 && x_stride < w->cols) return fk_fail(FK_INVALID, "gemv_multi: x_stride %d < cols %d", x_stride, w->cols);
    if (((uintptr_t)x_dev & 15) || (x_stride & 3)) return fk_fail(FK_INVALID, "gemv_multi: x_dev must be 16-byte aligned and x_stride a multiple of 4");
    FkDeviceGuard g(ctx->device);
    return fk_gemv_launch(ctx, (cudaStream_t)stream, w, ids_dev, 0, k, x_dev, x_stride, 1, y_dev, nullptr, nullptr, nullptr);
}

FK_EXPORT int fk_gemv_multi_glu(fk_ctx* ctx, void* stream, fk_weight w, const int* ids_dev, int k, const float* gate_dev, const float* up_dev,
                                int x_stride, int glu_act, float* y_dev, const int* n_active_dev) {
    if (!ctx || !w || !ids_dev || !gate_dev || !up_dev || !y_dev) return fk_fail(FK_INVALID, "gemv_multi_glu: null argument");
    if (k < 1 || k > 65535) return fk_fail(FK_INVALID, "gemv_multi_glu: k=%d", k);
    if (glu_act < 0 || glu_act > 1) return fk_fail(FK_UNSUPPORTED, "gemv_multi_glu: activation %d", glu_act);
    if (((uintptr_t)gate_dev & 15) || ((uintptr_t)up_dev & 15) || (x_stride & 3)) return fk_fail(FK_INVALID, "gemv_multi_glu: inputs must be 16-byte aligned");
    FkDeviceGuard g(ctx->device);
    FkGemvFused f{nullptr, 0.0f, up_dev, glu_act, 0, 0, 0, nullptr};
    return fk_gemv_launch(ctx, (cudaStream_t)stream, w, ids_dev, 0, k, gate_dev, x_stride, 1, y_dev, nullptr, n_active_dev, &f);
}

// gpt-oss's projections carry a bias row (crates/frink-models/src/models/gpt_oss.rs:9-12,46); it is added by the lane
// that finishes the row, so a biased projection is still one launch:  y[b] (+)= W rmsnorm?(x[b]) + bias.
FK_EXPORT int fk_gemv_biased(fk_ctx* ctx, void* stream, fk_weight w, int mat, const float* x_dev, int x_ld, int batch, float* y_dev,
                             const float* norm_weight_dev, float norm_eps, const float* bias_dev, int accumulate) {
    if (!ctx || !w || !x_dev || !y_dev) return fk_fail(FK_INVALID, "gemv_biased: null argument");
    if (batch < 1 || batch > 8) return fk_fail(FK_UNSUPPORTED, "gemv_biased: batch %d outside 1..8", batch);
    if (mat < 0 || mat >= w->n_mats) return fk_fail(FK_INVALID, "gemv_biased: matrix %d of %d", mat, w->n_mats);
    if (x_ld == 0) x_ld = w->cols;
    if (x_ld < w->cols || (x_ld & 3)) return fk_fail(FK_INVALID, "gemv_biased: x_ld %d (columns %d, must be a multiple of 4)", x_ld, w->cols);
    if (((uintptr_t)x_dev & 15) || ((uintptr_t)norm_weight_dev & 15)) return fk_fail(FK_INVALID, "gemv_biased: inputs must be 16-byte aligned");
    FkDeviceGuard g(ctx->device);
    FkGemvFused f{norm_weight_dev, norm_eps, nullptr, 0, accumulate, x_ld, 0, nullptr};
    f.bias = bias_dev;
    return fk_gemv_launch(ctx, (cudaStream_t)stream, w, nullptr, mat, 1, x_dev, 0, batch, y_dev, nullptr, nullptr, &f);
}

// The indexed expert matvec with every expert's own bias row (`run_expert_oai`, crates/frink-moe/src/lib.rs:1039-1060):
// slot j:  y[j] = W[ids[j]] in_j + bias[ids[j]],  in_j = x[j] (up_dev null) or act(x[j]) * up[j] (x the BIASED gate).
FK_EXPORT int fk_gemv_multi_biased(fk_ctx* ctx, void* stream, fk_weight w, const int* ids_dev, int k, const float* x_dev, const float* up_dev,
                                   int x_stride, int glu_act, const float* bias_dev, float* y_dev) {
    if (!ctx || !w || !ids_dev || !x_dev || !y_dev || !bias_dev) return fk_fail(FK_INVALID, "gemv_multi_biased: null argument");
    if (w->kind == FK_BF16 || w->kind == FK_Q5_K) return fk_fail(FK_UNSUPPORTED, "gemv_multi_biased: kind %d has no indexed form", w->kind);
    if (k < 1 || k > 65535) return fk_fail(FK_INVALID, "gemv_multi_biased: k=%d", k);
    if (glu_act < 0 || glu_act > 1) return fk_fail(FK_UNSUPPORTED, "gemv_multi_biased: activation %d", glu_act);
    if (x_stride != 0 && x_stride < w->cols) return fk_fail(FK_INVALID, "gemv_multi_biased: x_stride %d < cols %d", x_stride, w->cols);
    if (up_dev && x_stride == 0) return fk_fail(FK_INVALID, "gemv_multi_biased: the gated form reads one row per slot (x_stride 0)");
    if (((uintptr_t)x_dev & 15) || ((uintptr_t)up_dev & 15) || (x_stride & 3)) return fk_fail(FK_INVALID, "gemv_multi_biased: inputs must be 16-byte aligned");
    FkDeviceGuard g(ctx->device);
    FkGemvFused f{nullptr, 0.0f, up_dev, glu_act, 0, 0, 0, nullptr};
    f.bias = bias_dev;
    return fk_gemv_launch(ctx, (cudaStream_t)stream, w, ids_dev, 0, k, x_dev, x_stride, 1, y_dev, nullptr, nullptr, &f);
}

// gate and up of the chosen experts in ONE launch of 2 k slots (they read the same input and have the same shape):
//   y[j]     = gate[ids[j]] in_j (+ gate_bias[ids[j]])        j < k
//   y[k + j] = up[ids[j]]   in_j (+ up_bias[ids[j]])
// in_j = x[j], or rmsnorm(x[j]) * norm_weight when a norm weight is given (the layer's norm folded into the matvec).
int fk_gemv_multi_gate_up_launch(fk_ctx* ctx, void* stream, fk_weight gate, fk_weight up, const int* ids_dev, int k, const float* x_dev,
                                 int x_stride, const float* norm_weight_dev, float norm_eps, const float* gate_bias_dev,
                                 const float* up_bias_dev, float* y_dev, int x_ready) {
    if (!ctx || !gate || !up || !ids_dev || !x_dev || !y_dev) return fk_fail(FK_INVALID, "gemv_multi_gate_up: null argument");
    if (gate->kind != up->kind || gate->rows != up->rows || gate->cols != up->cols || gate->n_mats != up->n_mats || gate->mat_stride != up->mat_stride)
        return fk_fail(FK_INVALID, "gemv_multi_gate_up: gate and up must be stacks of the same kind and shape");
    for (int i = 0; i < 4; i++)
        if (gate->plane_off[i] != up->plane_off[i] || gate->plane_stride[i] != up->plane_stride[i])
            return fk_fail(FK_INVALID, "gemv_multi_gate_up: gate and up are laid out differently");
    if (gate->kind == FK_BF16 || gate->kind == FK_Q5_K) return fk_fail(FK_UNSUPPORTED, "gemv_multi_gate_up: kind %d has no indexed form", gate->kind);
    if ((gate_bias_dev == nullptr) != (up_bias_dev == nullptr)) return fk_fail(FK_INVALID, "gemv_multi_gate_up: the two bias tables come together");
    if (k < 1 || 2 * k > 65535) return fk_fail(FK_INVALID, "gemv_multi_gate_up: k=%d", k);
    if (x_stride != 0 && x_stride < gate->cols) return fk_fail(FK_INVALID, "gemv_multi_gate_up: x_stride %d < cols %d", x_stride, gate->cols);
    if (((uintptr_t)x_dev & 15) || ((uintptr_t)norm_weight_dev & 15) || (x_stride & 3))
        return fk_fail(FK_INVALID, "gemv_multi_gate_up: inputs must be 16-byte aligned and x_stride a multiple of 4");
    FkDeviceGuard g(ctx->device);
    FkGemvFused f{norm_weight_dev, norm_eps, nullptr, 0, 0, 0, 0, nullptr};
    f.bias = gate_bias_dev;
    f.w2 = up;
    f.bias2 = up_bias_dev;
    f.x_ready = x_ready;
    return fk_gemv_launch(ctx, (cudaStream_t)stream, gate, ids_dev, 0, 2 * k, x_dev, x_stride, 1, y_dev, nullptr, nullptr, &f);
}

FK_EXPORT int fk_gemv_multi_gate_up(fk_ctx* ctx, void* stream, fk_weight gate, fk_weight up, const int* ids_dev, int k, const float* x_dev,
                                    int x_stride, const float* norm_weight_dev, float norm_eps, const float* gate_bias_dev,
                                    const float* up_bias_dev, float* y_dev) {
    return fk_gemv_multi_gate_up_launch(ctx, stream, gate, up, ids_dev, k, x_dev, x_stride, norm_weight_dev, norm_eps, gate_bias_dev, up_bias_dev,
                                        y_dev, 0);
}

FK_EXPORT int fk_gemv_multi_active(fk_ctx* ctx, void* stream, fk_weight w, const int* ids_dev, int k, const float* x_dev,
                                   int x_stride, float* y_dev, const int* n_active_dev) {
    if (!ctx || !w || !ids_dev || !x_dev || !y_dev || !n_active_dev) return fk_fail(FK_INVALID, "gemv_multi_active: null argument");
    if (k < 1 || k > 65535) return fk_fail(FK_INVALID, "gemv_multi_active: k=%d", k);
    if (x_stride != 0 && x_stride < w->cols) return fk_fail(FK_INVALID, "gemv_multi_active: x_stride %d < cols %d", x_stride, w->cols);
    if (((uintptr_t)x_dev & 15) || (x_stride & 3)) return fk_fail(FK_INVALID, "gemv_multi_active: x_dev must be 16-byte aligned and x_stride a multiple of 4");
    FkDeviceGuard g(ctx->device);
    return fk_gemv_launch(ctx, (cudaStream_t)stream, w, ids_dev, 0, k, x_dev, x_stride, 1, y_dev, nullptr, n_active_dev, nullptr);
}

FK_EXPORT int fk_gemv_isums(fk_ctx* ctx, void* stream, fk_weight w, int mat, const float* x_dev, int32_t* isums_dev) {
    if (!ctx || !w || !x_dev || !isums_dev) return fk_fail(FK_INVALID, "gemv_isums: null argument");
    if (mat < 0 || mat >= w->n_mats) return fk_fail(FK_INVALID, "gemv_isums: matrix %d of %d", mat, w->n_mats);
    if ((uintptr_t)x_dev & 15) return fk_fail(FK_INVALID, "gemv_isums: x_dev must be 16-byte aligned");
    FkDeviceGuard g(ctx->device);
    // y is not wanted: park it in the context's scratch
    int rc = fk_ensure_scratch(ctx, (cudaStream_t)stream, (size_t)w->rows * sizeof(float));
    if (rc) return rc;
    return fk_gemv_launch(ctx, (cudaStream_t)stream, w, nullptr, mat, 1, x_dev, 0, 1, (float*)ctx->scratch, isums_dev, nullptr, nullptr);
}
