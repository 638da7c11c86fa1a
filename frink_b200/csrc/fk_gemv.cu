// Decode GEMV (batch 1..8) over resident quantized weights, and its indexed
// (one expert per slot) form.
//
// Shape of the kernel: a persistent grid of 512-thread blocks.  Each block
// first quantizes the activations to q8_1 into shared memory (one warp per run
// of 32 values, the rule of fk_q8_1_lane), then its warps walk pairs of weight
// rows.  A lane owns one 16-byte piece of packed weights per row and trip --
// every global load is a 128-bit load of consecutive addresses across the warp
// -- unpacks it in registers, takes exact int32 dot products against the int8
// activations with dp4a, scales them into an f32 accumulator per (row, batch
// column), and the warp reduces with shuffles.  Weight bytes are read once for
// the whole batch.
#include "fk_common.cuh"

namespace {

constexpr int GEMV_THREADS = 512;
constexpr int GEMV_WARPS = GEMV_THREADS / 32;
constexpr int R = 2;  // weight rows a warp carries at once

struct GemvArgs {
    const uint8_t* w;
    size_t mat_stride;
    size_t plane_off[4];
    const int* ids;
    int mat;
    const float* x;
    int x_stride;
    float* y;
    int rows, cols, batch;
    int32_t* isums;
};

__device__ __forceinline__ uint4 ldg16(const uint8_t* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ int dp4a4(const uint4& a, const int4& b) {
    int s = __dp4a((int)a.x, b.x, 0);
    s = __dp4a((int)a.y, b.y, s);
    s = __dp4a((int)a.z, b.z, s);
    return __dp4a((int)a.w, b.w, s);
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
__device__ __forceinline__ float e8m0_half(uint32_t e) {
    return __uint_as_float(e < 2 ? (0x00200000u << e) : ((e - 1u) << 23));
}

// ---------------------------------------------------------------------------
// A "piece" is what one lane holds of one weight row for one trip of the warp
// along K: 16 bytes of packed weights plus the scale words that go with them.
// load() only issues global loads (so a batch of pieces can be in flight
// together); eat() unpacks and accumulates.
//   Q4_K : 8 lanes per 144-byte super-block, a trip covers 4 super-blocks.
//          Lane c owns quant bytes [16c, 16c+16): low nibbles are 16 weights of
//          sub-block 2g, high nibbles 16 weights of sub-block 2g+1 (g = c/2).
//   Q6_K : 8 lanes per super-block; lane c owns ql bytes [16c, 16c+16) and the
//          matching 16 qh bytes: two runs of 16 weights (groups g_lo, g_lo+4).
//   Q8_0 : a lane owns 16 int8 (half a block); a trip covers 512 weights.
//   MXFP4: a lane owns one block's 16 code bytes; a trip covers 1024 weights.
struct Smem {
    const int8_t* q;   // [NB][cols]
    const float* d;    // [NB][cols/32]
    const float* s;    // Q4_K: d * run sum
    const int* b16;    // Q6_K: sums of 16
    int cols, nb32;
};

template <int KIND> struct Piece;

template <> struct Piece<FK_Q4_K> {
    uint4 hd, wq;
    static __device__ __forceinline__ int trips(int cols) { return ((cols >> 8) + 3) >> 2; }
    __device__ __forceinline__ void load(const GemvArgs& a, const uint8_t* wb, int row, int trip, int lane, bool row_ok) {
        const int nsb = a.cols >> 8, sb = trip * 4 + (lane >> 3);
        hd = make_uint4(0, 0, 0, 0);
        wq = make_uint4(0, 0, 0, 0);
        if (row_ok && sb < nsb) {
            const uint8_t* p = wb + ((size_t)row * nsb + sb) * 144;
            hd = ldg16(p);
            wq = ldg16(p + 16 + 16 * (lane & 7));
        }
    }
    template <int NB, bool DUMP>
    __device__ __forceinline__ void eat(const GemvArgs& a, const Smem& sm, int row, int trip, int lane, bool row_ok, float* acc) const {
        const int nsb = a.cols >> 8, sb = trip * 4 + (lane >> 3);
        const bool live = sb < nsb;
        const int sbs = live ? sb : 0;
        const int c = lane & 7, g = c >> 1, h = c & 1;
        // 6-bit scales and mins of sub-blocks 2g, 2g+1, two at a time from the
        // 16-bit words of the 12 packed bytes
        const uint32_t w0 = hd.y, w1 = hd.z, w2 = hd.w;
        uint32_t sc2, m2;
        if (g < 2) {
            const uint32_t s_lo = g ? (w0 >> 16) : (w0 & 0xFFFF), s_hi = g ? (w1 >> 16) : (w1 & 0xFFFF);
            sc2 = s_lo & 0x3F3F;
            m2 = s_hi & 0x3F3F;
        } else {
            const uint32_t A = (g & 1) ? (w2 >> 16) : (w2 & 0xFFFF);
            const uint32_t B = (g & 1) ? (w0 >> 16) : (w0 & 0xFFFF);
            const uint32_t C = (g & 1) ? (w1 >> 16) : (w1 & 0xFFFF);
            sc2 = (A & 0x0F0F) | ((B & 0xC0C0) >> 2);
            m2 = ((A >> 4) & 0x0F0F) | ((C & 0xC0C0) >> 2);
        }
        const float d = fk_h2f((uint16_t)(hd.x & 0xFFFF)), dmin = fk_h2f((uint16_t)(hd.x >> 16));
        const float f_lo = d * (float)(sc2 & 0xFF), f_hi = d * (float)(sc2 >> 8);
        // the two lanes sharing a sub-block (h = 0, 1) each carry half its min term
        const float mm_lo = 0.5f * dmin * (float)(m2 & 0xFF), mm_hi = 0.5f * dmin * (float)(m2 >> 8);
        uint4 lo, hi;
        lo.x = wq.x & 0x0F0F0F0Fu; hi.x = (wq.x >> 4) & 0x0F0F0F0Fu;
        lo.y = wq.y & 0x0F0F0F0Fu; hi.y = (wq.y >> 4) & 0x0F0F0F0Fu;
        lo.z = wq.z & 0x0F0F0F0Fu; hi.z = (wq.z >> 4) & 0x0F0F0F0Fu;
        lo.w = wq.w & 0x0F0F0F0Fu; hi.w = (wq.w >> 4) & 0x0F0F0F0Fu;
#pragma unroll
        for (int b = 0; b < NB; b++) {
            const int8_t* q8 = sm.q + (size_t)b * sm.cols + sbs * 256 + 64 * g + 16 * h;
            const int4 ua = *(const int4*)q8, ub = *(const int4*)(q8 + 32);
            const float2 d8 = *(const float2*)(sm.d + b * sm.nb32 + sbs * 8 + 2 * g);
            const float2 s8 = *(const float2*)(sm.s + b * sm.nb32 + sbs * 8 + 2 * g);
            int il = dp4a4(lo, ua), ih = dp4a4(hi, ub);
            acc[b] += f_lo * d8.x * (float)il + f_hi * d8.y * (float)ih - (mm_lo * s8.x + mm_hi * s8.y);
            if (DUMP && b == 0) {
                il += __shfl_xor_sync(0xffffffffu, il, 1);
                ih += __shfl_xor_sync(0xffffffffu, ih, 1);
                if (live && h == 0 && row_ok) {
                    int32_t* o = a.isums + (size_t)row * sm.nb32 + sb * 8 + 2 * g;
                    o[0] = il;
                    o[1] = ih;
                }
            }
        }
    }
};

template <> struct Piece<FK_Q8_0> {
    uint4 wq;
    uint32_t dbits;
    static __device__ __forceinline__ int trips(int cols) { return ((cols >> 4) + 31) >> 5; }
    __device__ __forceinline__ void load(const GemvArgs& a, const uint8_t* wb, int row, int trip, int lane, bool row_ok) {
        const int ci = trip * 32 + lane;
        wq = make_uint4(0, 0, 0, 0);
        dbits = 0;
        if (row_ok && ci < (a.cols >> 4)) {
            wq = ldg16(wb + a.plane_off[0] + (size_t)row * a.cols + (size_t)ci * 16);
            dbits = __ldg((const uint16_t*)(wb + a.plane_off[1]) + (size_t)row * (a.cols >> 5) + (ci >> 1));
        }
    }
    template <int NB, bool DUMP>
    __device__ __forceinline__ void eat(const GemvArgs& a, const Smem& sm, int row, int trip, int lane, bool row_ok, float* acc) const {
        const int ci = trip * 32 + lane;
        const bool live = ci < (sm.cols >> 4);
        const int cs = live ? ci : 0;
        const float dw = fk_h2f((uint16_t)dbits);
#pragma unroll
        for (int b = 0; b < NB; b++) {
            const int4 ua = *(const int4*)(sm.q + (size_t)b * sm.cols + cs * 16);
            int is = dp4a4(wq, ua);
            acc[b] += dw * sm.d[b * sm.nb32 + (cs >> 1)] * (float)is;
            if (DUMP && b == 0) {
                is += __shfl_xor_sync(0xffffffffu, is, 1);
                if (live && !(lane & 1) && row_ok) a.isums[(size_t)row * sm.nb32 + (ci >> 1)] = is;
            }
        }
    }
};

template <> struct Piece<FK_Q6_K> {
    uint4 ql, qh;
    int sc_lo, sc_hi;
    uint32_t dbits;
    static __device__ __forceinline__ int trips(int cols) { return ((cols >> 8) + 3) >> 2; }
    __device__ __forceinline__ void load(const GemvArgs& a, const uint8_t* wb, int row, int trip, int lane, bool row_ok) {
        const int nsb = a.cols >> 8, sb = trip * 4 + (lane >> 3);
        const int c = lane & 7, hf = c >> 2, q = c & 3;
        ql = make_uint4(0, 0, 0, 0);
        qh = ql;
        sc_lo = sc_hi = 0;
        dbits = 0;
        if (row_ok && sb < nsb) {
            const size_t r = (size_t)row;
            ql = ldg16(wb + a.plane_off[0] + r * (a.cols >> 1) + (size_t)sb * 128 + 16 * c);
            qh = ldg16(wb + a.plane_off[1] + r * (a.cols >> 2) + (size_t)sb * 64 + 32 * hf + 16 * (q & 1));
            const int8_t* sc = (const int8_t*)(wb + a.plane_off[2]) + r * (a.cols >> 4) + sb * 16 + 8 * hf + q;
            sc_lo = __ldg(sc);
            sc_hi = __ldg(sc + 4);
            dbits = __ldg((const uint16_t*)(wb + a.plane_off[3]) + r * nsb + sb);
        }
    }
    template <int NB, bool DUMP>
    __device__ __forceinline__ void eat(const GemvArgs& a, const Smem& sm, int row, int trip, int lane, bool row_ok, float* acc) const {
        const int nsb = sm.cols >> 8, sb = trip * 4 + (lane >> 3);
        const bool live = sb < nsb;
        const int sbs = live ? sb : 0;
        const int c = lane & 7, hf = c >> 2, q = c & 3;
        const int g_lo = 8 * hf + q, g_hi = g_lo + 4;
        const int shift = 2 * (q >> 1);
        const float d = fk_h2f((uint16_t)dbits);
        const float f_lo = d * (float)sc_lo, f_hi = d * (float)sc_hi;
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
            const int4 ua = *(const int4*)(q8 + 16 * g_lo), ub = *(const int4*)(q8 + 16 * g_hi);
            const float d8lo = sm.d[b * sm.nb32 + sbs * 8 + (g_lo >> 1)], d8hi = sm.d[b * sm.nb32 + sbs * 8 + (g_hi >> 1)];
            const int* b16 = sm.b16 + b * (sm.cols >> 4) + sbs * 16;
            // codes are stored +32: sum((c - 32) * u) = sum(c * u) - 32 * sum(u)
            const int il = dp4a4(vl, ua) - 32 * b16[g_lo];
            const int ih = dp4a4(vh, ub) - 32 * b16[g_hi];
            acc[b] += f_lo * d8lo * (float)il + f_hi * d8hi * (float)ih;
            if (DUMP && b == 0 && live && row_ok) {
                int32_t* o = a.isums + (size_t)row * (sm.cols >> 4) + sb * 16;
                o[g_lo] = il;
                o[g_hi] = ih;
            }
        }
    }
};

template <> struct Piece<FK_MXFP4> {
    uint4 wq;
    uint32_t e;
    static __device__ __forceinline__ int trips(int cols) { return ((cols >> 5) + 31) >> 5; }
    __device__ __forceinline__ void load(const GemvArgs& a, const uint8_t* wb, int row, int trip, int lane, bool row_ok) {
        const int kb = trip * 32 + lane;
        wq = make_uint4(0, 0, 0, 0);
        e = 0xFFFFFFFFu;
        if (row_ok && kb < (a.cols >> 5)) {
            wq = ldg16(wb + a.plane_off[0] + (size_t)row * (a.cols >> 1) + (size_t)kb * 16);
            e = __ldg(wb + a.plane_off[1] + (size_t)row * (a.cols >> 5) + kb);
        }
    }
    template <int NB, bool DUMP>
    __device__ __forceinline__ void eat(const GemvArgs& a, const Smem& sm, int row, int trip, int lane, bool row_ok, float* acc) const {
        const int kb = trip * 32 + lane;
        const bool live = kb < sm.nb32;
        const int ks = live ? kb : 0;
        const float dw = e == 0xFFFFFFFFu ? 0.0f : e8m0_half(e);
        uint4 va, vb;
        va.x = e2m1x2_4(wq.x); va.y = e2m1x2_4(wq.x >> 16);
        va.z = e2m1x2_4(wq.y); va.w = e2m1x2_4(wq.y >> 16);
        vb.x = e2m1x2_4(wq.z); vb.y = e2m1x2_4(wq.z >> 16);
        vb.z = e2m1x2_4(wq.w); vb.w = e2m1x2_4(wq.w >> 16);
#pragma unroll
        for (int b = 0; b < NB; b++) {
            const int8_t* q8 = sm.q + (size_t)b * sm.cols + ks * 32;
            const int4 ua = *(const int4*)q8, ub = *(const int4*)(q8 + 16);
            const int is = dp4a4(va, ua) + dp4a4(vb, ub);
            acc[b] += dw * sm.d[b * sm.nb32 + ks] * (float)is;
            if (DUMP && b == 0 && live && row_ok) a.isums[(size_t)row * sm.nb32 + kb] = is;
        }
    }
};

// U = trips whose loads a lane issues back to back before it consumes any.
template <int KIND, int NB, bool DUMP, int U>
__global__ void __launch_bounds__(GEMV_THREADS) gemv_kernel(const GemvArgs a) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int cols = a.cols, rows = a.rows;
    const int nb32 = cols >> 5;
    int8_t* sq = (int8_t*)smem;                       // [NB][cols] int8
    float* sd = (float*)(smem + (size_t)NB * cols);   // [NB][nb32] stored scale, widened
    float* ss = sd + NB * nb32;                       // Q4_K: [NB][nb32] scale * run sum
    int* sb16 = (int*)(sd + NB * nb32);               // Q6_K: [NB][cols/16] sums of 16

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int slot = blockIdx.y;
    const int mat = a.ids ? a.ids[slot] : a.mat;
    const uint8_t* wb = a.w + (size_t)mat * a.mat_stride;
    const float* x = a.x + (size_t)slot * a.x_stride;
    float* y = a.y + (size_t)slot * a.batch * rows;

    const int gwarp = blockIdx.x * GEMV_WARPS + warp;
    const int twarps = gridDim.x * GEMV_WARPS;
    const int ntrips = Piece<KIND>::trips(cols);

    // The first batch of weight loads goes out before the activations are
    // touched, so HBM latency overlaps the quantization.
    Piece<KIND> pc[U][R];
    int rp = gwarp;
#pragma unroll
    for (int u = 0; u < U; u++)
#pragma unroll
        for (int r = 0; r < R; r++)
            pc[u][r].load(a, wb, rp * R + r, u, lane, rp * R + r < rows && u < ntrips);

    // ---- activations -> q8_1 in shared memory
    for (int run = warp; run < NB * nb32; run += GEMV_WARPS) {
        const int b = run / nb32, kb = run - b * nb32;
        const float v = b < a.batch ? x[(size_t)b * cols + kb * 32 + lane] : 0.0f;
        float d;
        int qsum;
        const int q = fk_q8_1_lane(v, &d, &qsum);
        // MXFP4 keeps each run as (elem j, elem j+16) pairs: the order its
        // nibble decode produces bytes in.
        const int pos = KIND == FK_MXFP4 ? (((lane & 15) << 1) | (lane >> 4)) : lane;
        sq[(size_t)b * cols + kb * 32 + pos] = (int8_t)q;
        if (KIND == FK_Q6_K) {
            const int half_sum = __reduce_add_sync(0xffffffffu, lane < 16 ? q : 0);
            if (lane == 0) {
                sb16[b * (cols >> 4) + 2 * kb] = half_sum;
                sb16[b * (cols >> 4) + 2 * kb + 1] = qsum - half_sum;
            }
        }
        if (lane == 0) {
            sd[b * nb32 + kb] = d;
            if (KIND == FK_Q4_K) ss[b * nb32 + kb] = d * (float)qsum;
        }
    }
    __syncthreads();
    Smem sm{sq, sd, ss, sb16, cols, nb32};

    for (; rp * R < rows; rp += twarps) {
        const int row0 = rp * R;
        float acc[R][NB];
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int b = 0; b < NB; b++) acc[r][b] = 0.0f;

        for (int t0 = 0; t0 < ntrips; t0 += U) {
            if (t0 > 0 || rp != gwarp) {
#pragma unroll
                for (int u = 0; u < U; u++)
#pragma unroll
                    for (int r = 0; r < R; r++)
                        pc[u][r].load(a, wb, row0 + r, t0 + u, lane, row0 + r < rows && t0 + u < ntrips);
            }
#pragma unroll
            for (int u = 0; u < U; u++)
#pragma unroll
                for (int r = 0; r < R; r++)
                    pc[u][r].template eat<NB, DUMP>(a, sm, row0 + r, t0 + u, lane, row0 + r < rows && t0 + u < ntrips, acc[r]);
        }
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int b = 0; b < NB; b++) {
                const float s = fk_warp_sum(acc[r][b]);
                if (lane == 0 && row0 + r < rows && b < a.batch) y[(size_t)b * rows + row0 + r] = s;
            }
    }
}

size_t gemv_smem_bytes(int kind, int nb, int cols) {
    size_t s = (size_t)nb * cols + (size_t)nb * (cols / 32) * 4;
    if (kind == FK_Q4_K) s += (size_t)nb * (cols / 32) * 4;
    if (kind == FK_Q6_K) s += (size_t)nb * (cols / 16) * 4;
    return s;
}

template <int KIND, int NB, bool DUMP>
int launch_one(fk_ctx* ctx, cudaStream_t st, const GemvArgs& a, int slots) {
    const size_t smem = gemv_smem_bytes(KIND, NB, a.cols);
    if (smem > 220 * 1024) return fk_fail(FK_UNSUPPORTED, "gemv: %d columns x batch %d needs %zu B of shared memory", a.cols, NB, smem);
    constexpr int U = NB <= 2 ? 3 : (NB <= 4 ? 2 : 1);
    auto kern = gemv_kernel<KIND, NB, DUMP, U>;
    if (smem > 48 * 1024) FK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), FK_KERNEL);
    const int pairs = (a.rows + R - 1) / R;
    const int need = (pairs + GEMV_WARPS - 1) / GEMV_WARPS;
    // a persistent grid: as many blocks as are resident at once, no second wave
    int occ = 0;
    FK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, GEMV_THREADS, smem), FK_KERNEL);
    if (occ < 1) occ = 1;
    int per_slot = (occ * ctx->sm_count + slots - 1) / slots;
    if (per_slot < 1) per_slot = 1;
    dim3 grid((unsigned)(need < per_slot ? need : per_slot), (unsigned)slots);
    kern<<<grid, GEMV_THREADS, smem, st>>>(a);
    FK_CUDA(cudaGetLastError(), FK_LAUNCH);
    ctx->launches++;
    return FK_OK;
}

template <int KIND>
int launch_kind(fk_ctx* ctx, cudaStream_t st, const GemvArgs& a, int slots, bool dump) {
    if (dump) return launch_one<KIND, 1, true>(ctx, st, a, slots);
    if (a.batch <= 1) return launch_one<KIND, 1, false>(ctx, st, a, slots);
    if (a.batch <= 2) return launch_one<KIND, 2, false>(ctx, st, a, slots);
    if (a.batch <= 4) return launch_one<KIND, 4, false>(ctx, st, a, slots);
    return launch_one<KIND, 8, false>(ctx, st, a, slots);
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
                   const float* x_dev, int x_stride, int batch, float* y_dev, int32_t* isums_dev) {
    GemvArgs a;
    a.w = w->dev;
    a.mat_stride = w->mat_stride;
    for (int i = 0; i < 4; i++) a.plane_off[i] = w->plane_off[i];
    a.ids = ids_dev;
    a.mat = mat;
    a.x = x_dev;
    a.x_stride = x_stride;
    a.y = y_dev;
    a.rows = w->rows;
    a.cols = w->cols;
    a.batch = batch;
    a.isums = isums_dev;
    const bool dump = isums_dev != nullptr;
    switch (w->kind) {
        case FK_Q4_K: return launch_kind<FK_Q4_K>(ctx, st, a, slots, dump);
        case FK_Q6_K: return launch_kind<FK_Q6_K>(ctx, st, a, slots, dump);
        case FK_Q8_0: return launch_kind<FK_Q8_0>(ctx, st, a, slots, dump);
        case FK_MXFP4: return launch_kind<FK_MXFP4>(ctx, st, a, slots, dump);
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

FK_EXPORT int fk_gemv(fk_ctx* ctx, void* stream, fk_weight w, int mat, const float* x_dev, int batch, float* y_dev) {
    if (!ctx || !w || !x_dev || !y_dev) return fk_fail(FK_INVALID, "gemv: null argument");
    if (batch < 1 || batch > 8) return fk_fail(FK_UNSUPPORTED, "gemv: batch %d outside 1..8 (use fk_gemm)", batch);
    if (mat < 0 || mat >= w->n_mats) return fk_fail(FK_INVALID, "gemv: matrix %d of %d", mat, w->n_mats);
    FkDeviceGuard g(ctx->device);
    return fk_gemv_launch(ctx, (cudaStream_t)stream, w, nullptr, mat, 1, x_dev, 0, batch, y_dev, nullptr);
}

FK_EXPORT int fk_gemv_multi(fk_ctx* ctx, void* stream, fk_weight w, const int* ids_dev, int k, const float* x_dev,
                            int x_stride, float* y_dev) {
    if (!ctx || !w || !ids_dev || !x_dev || !y_dev) return fk_fail(FK_INVALID, "gemv_multi: null argument");
    if (k < 1 || k > 65535) return fk_fail(FK_INVALID, "gemv_multi: k=%d", k);
    if (x_stride != 0 && x_stride < w->cols) return fk_fail(FK_INVALID, "gemv_multi: x_stride %d < cols %d", x_stride, w->cols);
    FkDeviceGuard g(ctx->device);
    return fk_gemv_launch(ctx, (cudaStream_t)stream, w, ids_dev, 0, k, x_dev, x_stride, 1, y_dev, nullptr);
}

FK_EXPORT int fk_gemv_isums(fk_ctx* ctx, void* stream, fk_weight w, int mat, const float* x_dev, int32_t* isums_dev) {
    if (!ctx || !w || !x_dev || !isums_dev) return fk_fail(FK_INVALID, "gemv_isums: null argument");
    if (mat < 0 || mat >= w->n_mats) return fk_fail(FK_INVALID, "gemv_isums: matrix %d of %d", mat, w->n_mats);
    FkDeviceGuard g(ctx->device);
    // y is not wanted: park it in the context's scratch
    int rc = fk_ensure_scratch(ctx, (size_t)w->rows * sizeof(float));
    if (rc) return rc;
    return fk_gemv_launch(ctx, (cudaStream_t)stream, w, nullptr, mat, 1, x_dev, 0, 1, (float*)ctx->scratch, isums_dev);
}
