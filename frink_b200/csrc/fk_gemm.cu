// Prefill GEMM over resident quantized weights: int8 tensor-core MMA
// (tcgen05.mma kind::i8, accumulators in tensor memory) on q8_1 activations,
// with the exact per-32-run rescale done by the epilogue warps.
//
//   out[t][r] = sum_kb  dw[r][kb] * dx[t][kb] * ( sum_{k in kb} wq[r][k] * xq[t][k] )   (- Q4_K min term)
//
// The inner sum is an exact int32 (one MMA of K = 32 per run kb), so every
// integer this kernel produces equals the GEMV's and the oracle's.  Because the
// weight scale and the activation scale both change every 32 K, an accumulator
// is drained from tensor memory after every K = 32 step and scaled on the CUDA
// cores; that rescale, not the tensor pipe, bounds this kernel.
//
// One CTA = 128 weight rows x BN tokens, E + 4 warps with fixed roles:
//   warps 0..E-1  epilogue (E = 4 per 32 token columns: 16 for BN = 128): TMEM ->
//               registers (tcgen05.ld), f32 rescale, store
//   next 2      unpack: packed weights (global) -> int8 tile in shared memory
//               (128-byte swizzle, the layout the MMA descriptor names)
//   next 1      TMA producer: activation int8 tile + its scale tiles (and the
//               weight tile itself for Q8_0, whose int8 plane needs no unpacking)
//   last        MMA issuer (one elected lane) + TMEM allocation
// Stages (K = 128 each) and TMEM accumulators are rings guarded by mbarriers;
// every wait is bounded and raises the context's error word instead of
// spinning forever.
#include "fk_common.cuh"

#ifndef FK_I2F_MASK
#define FK_I2F_MASK 15
#endif
#ifndef FK_EPI_F32X2
#define FK_EPI_F32X2 1
#endif

#include "fk_tc.cuh"

namespace {
using namespace fk_tc;

#ifdef FK_TRACE
__device__ unsigned long long fk_gemm_trace[4][512];
__device__ __forceinline__ unsigned long long gtime_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define GTR(k_, i_, who_) do { if ((who_) && blockIdx.x == 0 && blockIdx.y == 0 && (i_) < 512) fk_gemm_trace[k_][i_] = gtime_ns(); } while (0)
#else
#define GTR(k_, i_, who_) do { } while (0)
#endif

constexpr int BM = 128;           // weight rows per CTA (MMA M)
constexpr int KSTAGE = 128;       // K per pipeline stage (4 MMAs of K = 32)
constexpr int NSTAGE = 4;
constexpr int UNPACK_WARPS = 2;
// epilogue warps: four (one per TMEM lane quadrant) for every 32 token columns of the tile
__host__ __device__ constexpr int epi_warps(int bn) { return bn / 32 * 4; }
__host__ __device__ constexpr int gemm_threads(int bn) { return (epi_warps(bn) + UNPACK_WARPS + 2) * 32; }

struct GemmArgs {
    const uint8_t* w;         // matrix 0 of the weight handle
    size_t mat_stride;
    size_t plane_off[4];
    size_t plane_stride[4];
    int kind, rows, cols;
    int mat;                  // dense: the matrix; grouped: ignored
    const int* tile_expert;   // grouped: expert of each token tile (nullptr = dense)
    const int* n_tiles_dev;   // grouped: number of live token tiles (nullptr = all of gridDim.y)
    const int* out_row;       // padded token row -> output row, -1 = padding
    float* out;
    int32_t* isums;           // test hook: the raw accumulators, [token][rows][cols / run] (nullptr = off)
    int* err;
};

// Shared memory map (offsets from a 1024-byte aligned base).
template <int BN> struct Smem {
    static constexpr int A_BYTES = BM * KSTAGE;          // 16 KB
    static constexpr int B_BYTES = BN * KSTAGE;
    static constexpr int DX_BYTES = 4 * BN * 4;          // [4 runs][BN] f32
    static constexpr int STAGE = A_BYTES + B_BYTES + 2 * DX_BYTES;
    static constexpr int BARS = NSTAGE * STAGE;          // barrier block
    static constexpr int TOTAL = BARS + 256 + 1024;      // + alignment slack
    static constexpr int NACC = 512 / BN;                // TMEM accumulator ring
};

// Weight scale of row `row`, run `kb`; Q4_K also the min scale.  Q6_K rows are
// (weight row, half-run) pairs, see the unpack warps.
struct WScale { float dw, mw; };

template <int KIND>
__device__ __forceinline__ void load_wscales(const GemmArgs& a, const uint8_t* wb, int row, bool row_ok, int kb0, int nkb, WScale* ws) {
    // scales of runs kb0 .. kb0+3 of this thread's row
#pragma unroll
    for (int j = 0; j < 4; j++) ws[j] = {0.0f, 0.0f};
    if (!row_ok) return;
    if (KIND == FK_Q4_K) {
        const int sb = kb0 >> 3;
        const uint4 hd = ldg16(wb + ((size_t)row * (a.cols >> 8) + sb) * 144);
        const float d = fk_h2f((uint16_t)(hd.x & 0xFFFF)), dmin = fk_h2f((uint16_t)(hd.x >> 16));
        const uint32_t s[3] = {hd.y, hd.z, hd.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int q = (kb0 & 7) + j;  // sub-block 0..7
            uint32_t sc, m;
            if (q < 4) {
                sc = (s[0] >> (8 * q)) & 63;
                m = (s[1] >> (8 * q)) & 63;
            } else {
                const uint32_t b = (s[2] >> (8 * (q - 4))) & 0xFF;
                sc = (b & 0x0F) | ((((s[0] >> (8 * (q - 4))) & 0xFF) >> 6) << 4);
                m = (b >> 4) | ((((s[1] >> (8 * (q - 4))) & 0xFF) >> 6) << 4);
            }
            if (kb0 + j < nkb) ws[j] = {d * (float)sc, dmin * (float)m};
        }
    } else if (KIND == FK_Q8_0) {
        const uint16_t* dp = (const uint16_t*)(wb + a.plane_off[1] + (size_t)row * a.plane_stride[1]);
#pragma unroll
        for (int j = 0; j < 4; j++)
            if (kb0 + j < nkb) ws[j].dw = fk_h2f(__ldg(dp + kb0 + j));
    } else if (KIND == FK_MXFP4) {
        const uint8_t* ep = wb + a.plane_off[1] + (size_t)row * a.plane_stride[1];
#pragma unroll
        for (int j = 0; j < 4; j++)
            if (kb0 + j < nkb) ws[j].dw = e8m0_half(__ldg(ep + kb0 + j));
    } else {  // FK_Q6_K: `row` = 2 * weight row + half; its scale of run kb is sc[2 * kb + half]
        const int wrow = row >> 1, half = row & 1;
        const int sb = kb0 >> 3;
        const float d = fk_h2f(__ldg((const uint16_t*)(wb + a.plane_off[3] + (size_t)wrow * a.plane_stride[3]) + sb));
        const int8_t* sc = (const int8_t*)(wb + a.plane_off[2] + (size_t)wrow * a.plane_stride[2]) + 2 * kb0 + half;
#pragma unroll
        for (int j = 0; j < 4; j++)
            if (kb0 + j < nkb) ws[j].dw = d * (float)__ldg(sc + 2 * j);
    }
}

// Packed bytes of one weight row for stage `st` (K range [128 st, 128 st + 128)),
// as loaded (nothing decoded yet, so the loads of the next stage can be in
// flight while this stage is written).
template <int KIND> struct RawRow { uint4 q[KIND == FK_Q6_K ? 6 : 4]; };

template <int KIND>
__device__ __forceinline__ void load_raw(const GemmArgs& a, const uint8_t* wb, int wrow, bool ok, int st, RawRow<KIND>& raw) {
    constexpr int N = KIND == FK_Q6_K ? 6 : 4;
#pragma unroll
    for (int i = 0; i < N; i++) raw.q[i] = make_uint4(0, 0, 0, 0);
    const int k0 = st * KSTAGE;
    if (!ok || k0 >= a.cols || KIND == FK_Q8_0) return;
    if (KIND == FK_Q4_K) {
        // 128 weights = 64 quant bytes: two groups of 32 bytes
        const uint8_t* p = wb + ((size_t)wrow * (a.cols >> 8) + (k0 >> 8)) * 144 + 16 + ((k0 >> 7) & 1) * 64;
#pragma unroll
        for (int i = 0; i < 4; i++) raw.q[i] = ldg16(p + 16 * i);
    } else if (KIND == FK_MXFP4) {
        const uint8_t* p = wb + a.plane_off[0] + (size_t)wrow * (a.cols >> 1) + (k0 >> 1);
#pragma unroll
        for (int b = 0; b < 4; b++)
            if (k0 + 32 * b < a.cols) raw.q[b] = ldg16(p + 16 * b);
    } else {  // FK_Q6_K: 64 ql bytes + 32 qh bytes of this half super-block
        const int sb = k0 >> 8, hf = (k0 >> 7) & 1;
        const uint8_t* ql = wb + a.plane_off[0] + (size_t)wrow * (a.cols >> 1) + (size_t)sb * 128 + 64 * hf;
        const uint8_t* qh = wb + a.plane_off[1] + (size_t)wrow * (a.cols >> 2) + (size_t)sb * 64 + 32 * hf;
#pragma unroll
        for (int i = 0; i < 4; i++) raw.q[i] = ldg16(ql + 16 * i);
        raw.q[4] = ldg16(qh);
        raw.q[5] = ldg16(qh + 16);
    }
}

__device__ __forceinline__ void store_tile_row(uint8_t* a_tile, int r, const uint4* o) {
    uint8_t* dst = a_tile + r * 128;
#pragma unroll
    for (int c = 0; c < 8; c++) *(uint4*)(dst + ((c ^ (r & 7)) << 4)) = o[c];
}

// Decode one weight row's 128 weights of a stage to int8 and write them as tile
// row(s), eight 16-byte chunks each at their swizzled places.  Q4_K, MXFP4:
// tile row `r`.  Q6_K: tile rows 2 r' and 2 r' + 1 (r = 2 r'), the codes minus
// 32 with the 16 weights of the OTHER half of every run of 32 zeroed, so that
// one K = 32 MMA yields the exact dot of a 16-weight scale group.
template <int KIND>
__device__ __forceinline__ void store_raw(const RawRow<KIND>& raw, int r, uint8_t* a_tile) {
    uint4 o[8];
    if (KIND == FK_Q4_K) {
        // low nibbles are the first 32 weights of a 32-byte group, high nibbles the next 32
#pragma unroll
        for (int g = 0; g < 2; g++) {
            const uint4 q0 = raw.q[2 * g], q1 = raw.q[2 * g + 1];
            o[4 * g + 0] = make_uint4(q0.x & 0x0F0F0F0Fu, q0.y & 0x0F0F0F0Fu, q0.z & 0x0F0F0F0Fu, q0.w & 0x0F0F0F0Fu);
            o[4 * g + 1] = make_uint4(q1.x & 0x0F0F0F0Fu, q1.y & 0x0F0F0F0Fu, q1.z & 0x0F0F0F0Fu, q1.w & 0x0F0F0F0Fu);
            o[4 * g + 2] = make_uint4((q0.x >> 4) & 0x0F0F0F0Fu, (q0.y >> 4) & 0x0F0F0F0Fu, (q0.z >> 4) & 0x0F0F0F0Fu, (q0.w >> 4) & 0x0F0F0F0Fu);
            o[4 * g + 3] = make_uint4((q1.x >> 4) & 0x0F0F0F0Fu, (q1.y >> 4) & 0x0F0F0F0Fu, (q1.z >> 4) & 0x0F0F0F0Fu, (q1.w >> 4) & 0x0F0F0F0Fu);
        }
        store_tile_row(a_tile, r, o);
    } else if (KIND == FK_MXFP4) {
        // bytes come out as (elem j, elem j+16) pairs, the order the activation
        // plane of this kind is stored in; an absent block (past the last column) is zeros
#pragma unroll
        for (int b = 0; b < 4; b++) {
            const uint4 q = raw.q[b];
            o[2 * b] = make_uint4(e2m1x2_4(q.x), e2m1x2_4(q.x >> 16), e2m1x2_4(q.y), e2m1x2_4(q.y >> 16));
            o[2 * b + 1] = make_uint4(e2m1x2_4(q.z), e2m1x2_4(q.z >> 16), e2m1x2_4(q.w), e2m1x2_4(q.w >> 16));
        }
        store_tile_row(a_tile, r, o);
    } else if (KIND == FK_Q6_K) {
        const uint32_t hh[8] = {raw.q[4].x, raw.q[4].y, raw.q[4].z, raw.q[4].w, raw.q[5].x, raw.q[5].y, raw.q[5].z, raw.q[5].w};
        uint4 o1[8];
        // element e = 32 * qd + l (qd = 0..3, l = 0..31): ql byte (l + 32 * (qd & 1)),
        // nibble (qd >> 1), qh byte l bits [2 qd, 2 qd + 2)
#pragma unroll
        for (int qd = 0; qd < 4; qd++) {
            const uint4 l0 = raw.q[2 * (qd & 1)], l1 = raw.q[2 * (qd & 1) + 1];
            const uint32_t ll[8] = {l0.x, l0.y, l0.z, l0.w, l1.x, l1.y, l1.z, l1.w};
            uint32_t v[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const uint32_t nib = (qd >> 1) ? ((ll[i] >> 4) & 0x0F0F0F0Fu) : (ll[i] & 0x0F0F0F0Fu);
                const uint32_t c6 = nib | (((hh[i] >> (2 * qd)) & 0x03030303u) << 4);
                v[i] = __vsub4(c6, 0x20202020u);
            }
            o[2 * qd] = make_uint4(v[0], v[1], v[2], v[3]);       // half 0 keeps the first 16 of the run
            o[2 * qd + 1] = make_uint4(0, 0, 0, 0);
            o1[2 * qd] = make_uint4(0, 0, 0, 0);
            o1[2 * qd + 1] = make_uint4(v[4], v[5], v[6], v[7]);  // half 1 the last 16
        }
        store_tile_row(a_tile, r, o);
        store_tile_row(a_tile, r + 1, o1);
    }
}

template <int KIND, int BN, bool DUMP>
__global__ void __launch_bounds__(gemm_threads(BN), 1)
gemm_kernel(const GemmArgs a, const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_dx,
            const __grid_constant__ CUtensorMap map_sx, const __grid_constant__ CUtensorMap map_w) {
    using S = Smem<BN>;
    constexpr int EPI_WARPS = epi_warps(BN);
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const int ttile = blockIdx.y;
    if (a.n_tiles_dev && ttile >= *a.n_tiles_dev) return;
    const int mat = a.tile_expert ? a.tile_expert[ttile] : a.mat;
    const uint8_t* wb = a.w + (size_t)mat * a.mat_stride;
    // Q6_K tile rows are (weight row, half) pairs: 64 weight rows per CTA
    constexpr int WROWS = KIND == FK_Q6_K ? BM / 2 : BM;
    const int wrow0 = blockIdx.x * WROWS;
    const int tok0 = ttile * BN;
    const int nkb = a.cols >> 5;
    const int nst = (nkb + 3) >> 2;

    // barriers: full_b[NSTAGE], full_a[NSTAGE], empty[NSTAGE], acc_full[NACC], acc_empty[NACC], then the TMEM base word
    const uint32_t bar0 = sbase + S::BARS;
    auto full_b = [&](int s) { return bar0 + 8u * s; };
    auto full_a = [&](int s) { return bar0 + 8u * (NSTAGE + s); };
    auto empty = [&](int s) { return bar0 + 8u * (2 * NSTAGE + s); };
    auto acc_full = [&](int b) { return bar0 + 8u * (3 * NSTAGE + b); };
    auto acc_empty = [&](int b) { return bar0 + 8u * (3 * NSTAGE + S::NACC + b); };
    uint32_t* tmem_word = (uint32_t*)(smem + S::BARS + 8 * (3 * NSTAGE + 2 * S::NACC));

    if (threadIdx.x == 0) {
        for (int s = 0; s < NSTAGE; s++) {
            mbar_init(full_b(s), 1);
            mbar_init(full_a(s), UNPACK_WARPS);
            mbar_init(empty(s), 1 + EPI_WARPS);
        }
        for (int b = 0; b < S::NACC; b++) {
            mbar_init(acc_full(b), 1);
            mbar_init(acc_empty(b), EPI_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == EPI_WARPS + UNPACK_WARPS + 1) {  // the MMA warp owns tensor memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_word)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_word;

    if (warp < EPI_WARPS) {
        // ------------------------------------------------------------ epilogue
        const int quad = warp & 3, chalf = warp >> 2;
        const int r = quad * 32 + lane;                // tile row = TMEM lane
        const int row = KIND == FK_Q6_K ? 2 * wrow0 + r : wrow0 + r;   // scale row id (pair id for Q6_K)
        const bool row_ok = (KIND == FK_Q6_K ? (wrow0 + (r >> 1)) : (wrow0 + r)) < a.rows;
        constexpr int CW = 32;                         // token columns this warp owns
        float acc[CW];
#pragma unroll
        for (int i = 0; i < CW; i++) acc[i] = 0.0f;
        const uint32_t taddr0 = tmem_base + ((uint32_t)(quad * 32) << 16) + chalf * CW;
        WScale ws[4], ws_next[4];
        load_wscales<KIND>(a, wb, row, row_ok, 0, nkb, ws_next);
        // TMEM reads are double-buffered in halves of 16 columns: while one half is
        // scaled the next one (or the next run's first) is already in flight, so a warp's
        // chain per run is its arithmetic, not the accumulator hand-off latency.
        uint32_t v[2][16];
        auto issue = [&](int kb, int c, uint32_t* dst) {
            const int buf = kb % S::NACC;
            if (c == 0) {
                mbar_wait(acc_full(buf), (kb / S::NACC) & 1, a.err, 11);
                tc_fence_after();
                GTR(1, kb, warp == 0 && lane == 0);
            }
            tc_ld16(taddr0 + buf * BN + c * 16, dst);
        };
        issue(0, 0, v[0]);
        tc_wait_ld();
        tc_ld_fence<16>(v[0]);
        for (int st = 0; st < nst; st++) {
            const int s = st % NSTAGE;
#pragma unroll
            for (int j = 0; j < 4; j++) ws[j] = ws_next[j];
            if (st + 1 < nst) load_wscales<KIND>(a, wb, row, row_ok, 4 * (st + 1), nkb, ws_next);
            mbar_wait(full_b(s), (st / NSTAGE) & 1, a.err, 10);   // the scale tiles of this stage have landed
            // the stage's scale tiles: dx [4][BN] then (Q4_K) sx [4][BN], as shared-space addresses
            const uint32_t sdx_s = sbase + s * S::STAGE + S::A_BYTES + S::B_BYTES;
            // Rolled on purpose: the unrolled body falls out of the instruction cache.
#pragma unroll 1
            for (int j = 0; j < 4; j++) {
                const int kb = 4 * st + j;
                if (kb >= nkb) break;
                const float dw = j == 0 ? ws[0].dw : (j == 1 ? ws[1].dw : (j == 2 ? ws[2].dw : ws[3].dw));
                const float mw = j == 0 ? ws[0].mw : (j == 1 ? ws[1].mw : (j == 2 ? ws[2].mw : ws[3].mw));
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    uint32_t* cur = v[c];
                    uint32_t* nxt = v[c ^ 1];
                    const int kb_n = c == 0 ? kb : kb + 1, c_n = c ^ 1;
                    if (kb_n < nkb) issue(kb_n, c_n, nxt);
                    const uint32_t dxs = sdx_s + (uint32_t)(j * BN + chalf * CW + c * 16) * 4u;
                    if (DUMP && row_ok) {
                        // the exact integers of this run, before any scale touches them
                        const int orow_d = KIND == FK_Q6_K ? wrow0 + (r >> 1) : wrow0 + r;
                        const int nruns = KIND == FK_Q6_K ? a.cols >> 4 : nkb, run = KIND == FK_Q6_K ? 2 * kb + (r & 1) : kb;
                        for (int i = 0; i < 16; i++) {
                            const int dst = a.out_row[tok0 + chalf * CW + c * 16 + i];
                            if (dst >= 0) a.isums[((size_t)dst * a.rows + orow_d) * nruns + run] = (int32_t)cur[i];
                        }
                    }
#pragma unroll
                    for (int i = 0; i < 16; i += 4) {
                        const float4 dx = lds128(dxs + 4u * i);
                        const float dxa[4] = {dx.x, dx.y, dx.z, dx.w};
                        float sxa[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                        if (KIND == FK_Q4_K) {
                            const float4 sx = lds128(dxs + 16u * BN + 4u * i);
                            sxa[0] = sx.x; sxa[1] = sx.y; sxa[2] = sx.z; sxa[3] = sx.w;
                        }
#if FK_EPI_F32X2
                        // two columns per instruction on the packed f32x2 path; int32 -> f32 (exact, |C| < 2^22)
                        // either on the conversion unit (bit of FK_I2F_MASK set: one issue slot, a quarter of
                        // the rate) or by the magic-number add on the integer and FP32 pipes (two slots)
#pragma unroll
                        for (int e = 0; e < 4; e += 2) {
                            constexpr int M2 = FK_I2F_MASK;
                            float2 f2;
                            if (((M2 >> e) & 3) == 3) {
                                f2 = make_float2((float)(int)cur[i + e], (float)(int)cur[i + e + 1]);
                            } else if (((M2 >> e) & 3) == 0) {
                                f2 = __fadd2_rn(make_float2(__int_as_float((int)cur[i + e] + 0x4B400000), __int_as_float((int)cur[i + e + 1] + 0x4B400000)),
                                                make_float2(-12582912.0f, -12582912.0f));
                            } else {
                                f2.x = ((M2 >> e) & 1) ? (float)(int)cur[i + e] : __int_as_float((int)cur[i + e] + 0x4B400000) - 12582912.0f;
                                f2.y = ((M2 >> e) & 2) ? (float)(int)cur[i + e + 1] : __int_as_float((int)cur[i + e + 1] + 0x4B400000) - 12582912.0f;
                            }
                            const float2 s2 = __fmul2_rn(make_float2(dw, dw), make_float2(dxa[e], dxa[e + 1]));
                            float2 t2 = __ffma2_rn(s2, f2, make_float2(acc[c * 16 + i + e], acc[c * 16 + i + e + 1]));
                            if (KIND == FK_Q4_K) t2 = __ffma2_rn(make_float2(-mw, -mw), make_float2(sxa[e], sxa[e + 1]), t2);
                            acc[c * 16 + i + e] = t2.x;
                            acc[c * 16 + i + e + 1] = t2.y;
                        }
#else
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            // exact int32 -> f32 for |C| < 2^22: by the magic-number add on the integer and
                            // FP32 pipes, or (elements whose bit of FK_I2F_MASK is set) by the conversion unit,
                            // which costs one issue slot instead of two but runs at a quarter of the rate
                            const float f = ((FK_I2F_MASK >> e) & 1) ? (float)(int)cur[i + e]
                                                                     : __int_as_float((int)cur[i + e] + 0x4B400000) - 12582912.0f;
                            float t = fmaf(dw * dxa[e], f, acc[c * 16 + i + e]);
                            if (KIND == FK_Q4_K) t = fmaf(-mw, sxa[e], t);
                            acc[c * 16 + i + e] = t;
                        }
#endif
                    }
                    tc_wait_ld();
                    tc_ld_fence<16>(nxt);
                    GTR(2, kb, warp == 0 && lane == 0 && c == 1);
                    if (kb_n < nkb && c_n == 1) {   // both halves of that accumulator are in registers: hand it back
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(acc_empty(kb_n % S::NACC));
                    }
                }
            }
            // this warp is done with the stage's scale tiles
            __syncwarp();
            if (lane == 0) mbar_arrive(empty(s));
        }
        // ---- store: out[out_row[token]][weight row]
        const int orow = KIND == FK_Q6_K ? wrow0 + (r >> 1) : wrow0 + r;
        const bool writer = row_ok && (KIND != FK_Q6_K || !(r & 1));
#pragma unroll 4
        for (int i = 0; i < CW; i++) {
            float v0 = acc[i];
            if (KIND == FK_Q6_K) v0 += __shfl_xor_sync(0xffffffffu, v0, 1);   // the two halves of a weight row sit in neighbouring lanes
            const int dst = a.out_row[tok0 + chalf * CW + i];
            if (writer && dst >= 0) a.out[(size_t)dst * a.rows + orow] = v0;
        }
    } else if (warp < EPI_WARPS + UNPACK_WARPS) {
        // ------------------------------------------------- weight unpack warps
        if (KIND != FK_Q8_0) {
            // 64 threads: Q6_K one weight row (two tile rows) each, the others two rows each
            constexpr int NR = KIND == FK_Q6_K ? 1 : 2;
            const int t = (warp - EPI_WARPS) * 32 + lane;
            RawRow<KIND> cur[NR], nxt[NR];
#pragma unroll
            for (int i = 0; i < NR; i++) load_raw<KIND>(a, wb, wrow0 + t + 64 * i, wrow0 + t + 64 * i < a.rows, 0, cur[i]);
            for (int st = 0; st < nst; st++) {
                const int s = st % NSTAGE;
                if (st + 1 < nst) {
#pragma unroll
                    for (int i = 0; i < NR; i++) load_raw<KIND>(a, wb, wrow0 + t + 64 * i, wrow0 + t + 64 * i < a.rows, st + 1, nxt[i]);
                }
                if (st >= NSTAGE) mbar_wait(empty(s), ((st / NSTAGE) - 1) & 1, a.err, 20);
#pragma unroll
                for (int i = 0; i < NR; i++) store_raw<KIND>(cur[i], KIND == FK_Q6_K ? 2 * t : t + 64 * i, smem + s * S::STAGE);
                fence_proxy_async();   // generic-proxy writes -> visible to the tensor core's reads
                __syncwarp();
                if (lane == 0) mbar_arrive(full_a(s));
                GTR(3, st, warp == EPI_WARPS && lane == 0);
#pragma unroll
                for (int i = 0; i < NR; i++) cur[i] = nxt[i];
            }
        }
    } else if (warp == EPI_WARPS + UNPACK_WARPS) {
        // --------------------------------------------------------- TMA producer
        if (lane == 0) {
            constexpr uint32_t TX = S::B_BYTES + S::DX_BYTES + (KIND == FK_Q4_K ? S::DX_BYTES : 0) + (KIND == FK_Q8_0 ? S::A_BYTES : 0);
            for (int st = 0; st < nst; st++) {
                const int s = st % NSTAGE;
                if (st >= NSTAGE) mbar_wait(empty(s), ((st / NSTAGE) - 1) & 1, a.err, 30);
                const uint32_t sa = sbase + s * S::STAGE;
                mbar_expect_tx(full_b(s), TX);
                tma_load_2d(sa + S::A_BYTES, &map_q, st * KSTAGE, tok0, full_b(s));
                tma_load_2d(sa + S::A_BYTES + S::B_BYTES, &map_dx, tok0, 4 * st, full_b(s));
                if (KIND == FK_Q4_K) tma_load_2d(sa + S::A_BYTES + S::B_BYTES + S::DX_BYTES, &map_sx, tok0, 4 * st, full_b(s));
                if (KIND == FK_Q8_0) tma_load_3d(sa, &map_w, st * KSTAGE, wrow0, mat, full_b(s));   // [matrix][row][k]: rows past a matrix's end read as zeros
            }
        }
    } else {
        // ----------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t IDESC = umma_idesc_i8(BM, BN);
            for (int st = 0; st < nst; st++) {
                const int s = st % NSTAGE;
                mbar_wait(full_b(s), (st / NSTAGE) & 1, a.err, 40);
                if (KIND != FK_Q8_0) mbar_wait(full_a(s), (st / NSTAGE) & 1, a.err, 41);
                tc_fence_after();
                const uint32_t sa = sbase + s * S::STAGE;
                const uint64_t da = umma_desc(sa), db = umma_desc(sa + S::A_BYTES);
                for (int j = 0; j < 4; j++) {
                    const int kb = 4 * st + j;
                    if (kb >= nkb) break;
                    const int buf = kb % S::NACC;
                    if (kb >= S::NACC) mbar_wait(acc_empty(buf), ((kb / S::NACC) - 1) & 1, a.err, 42);
                    tc_fence_after();
                    // K advances 32 bytes inside the 128-byte swizzle atom: +2 in the 16-byte address field
                    GTR(0, kb, true);
                    tc_mma_i8(tmem_base + buf * BN, da + 2 * j, db + 2 * j, IDESC);
                    tc_commit(acc_full(buf));
                }
                tc_commit(empty(s));   // arrives once the MMAs that read this stage are done
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == EPI_WARPS + UNPACK_WARPS + 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

// ---------------------------------------------------------------------------
// Activation plan: q8_1 of every (padded) token row into an int8 plane
// [n_pad][kpad] (row-major, K inner; MXFP4 keeps each run as (j, j+16) pairs)
// plus run-major scale planes dx[nkb][n_pad] and, for Q4_K, sx = dx * run sum.
__global__ void quantize_acts_kernel(const float* __restrict__ x, const int* __restrict__ src_row, int n_pad, int cols, int kind,
                                     int8_t* __restrict__ q, float* __restrict__ dx, float* __restrict__ sx) {
    const int nkb = cols >> 5;
    const long long run = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (run >= (long long)n_pad * nkb) return;
    const int t = (int)(run / nkb), kb = (int)(run - (long long)t * nkb);
    const int src = src_row[t];
    const float v = src >= 0 ? x[(size_t)src * cols + kb * 32 + lane] : 0.0f;
    float d;
    int qsum;
    const int qv = fk_q8_1_lane(v, &d, &qsum);
    const int pos = kind == FK_MXFP4 ? (((lane & 15) << 1) | (lane >> 4)) : lane;
    q[(size_t)t * cols + kb * 32 + pos] = (int8_t)qv;
    if (lane == 0) {
        dx[(size_t)kb * n_pad + t] = d;
        if (sx) sx[(size_t)kb * n_pad + t] = d * (float)qsum;
    }
}

// The same for the kinds whose int8 plane keeps the elements in order (all but MXFP4): a thread takes four values, eight
// lanes make a run, rows past the live tiles (`*n_tiles_dev * bn`, grouped form) are left alone -- no tile reads them.
__global__ void quantize_acts4_kernel(const float* __restrict__ x, const int* __restrict__ src_row, int n_pad, int cols, int8_t* __restrict__ q,
                                      float* __restrict__ dx, float* __restrict__ sx, const int* __restrict__ n_tiles_dev, int bn) {
    const int nkb = cols >> 5;
    const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long run = gid >> 3;
    const int part = (int)(gid & 7);
    const int n_live = n_tiles_dev ? min(n_pad, *n_tiles_dev * bn) : n_pad;
    const bool ok = run < (long long)n_live * nkb;          // whole groups of eight lanes are in or out
    const int t = ok ? (int)(run / nkb) : 0, kb = ok ? (int)(run - (long long)t * nkb) : 0;
    const int src = ok ? src_row[t] : -1;
    float4 f = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (src >= 0) f = __ldg((const float4*)(x + (size_t)src * cols + kb * 32) + part);
    unsigned mb = __float_as_uint(fmaxf(fmaxf(fabsf(f.x), fabsf(f.y)), fmaxf(fabsf(f.z), fabsf(f.w))));
    mb = max(mb, __shfl_xor_sync(0xffffffffu, mb, 1));
    mb = max(mb, __shfl_xor_sync(0xffffffffu, mb, 2));
    mb = max(mb, __shfl_xor_sync(0xffffffffu, mb, 4));
    const float amax = __uint_as_float(mb);
    const float d = amax / 127.0f;
    int q0 = 0, q1 = 0, q2 = 0, q3 = 0;
    if (amax != 0.0f) {
        q0 = (int)roundf(f.x / d); q1 = (int)roundf(f.y / d); q2 = (int)roundf(f.z / d); q3 = (int)roundf(f.w / d);
    }
    int qsum = q0 + q1 + q2 + q3;
    qsum += __shfl_xor_sync(0xffffffffu, qsum, 1);
    qsum += __shfl_xor_sync(0xffffffffu, qsum, 2);
    qsum += __shfl_xor_sync(0xffffffffu, qsum, 4);
    if (!ok) return;
    *(uint32_t*)(q + (size_t)t * cols + kb * 32 + part * 4) =
        (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) | ((uint32_t)(q2 & 0xFF) << 16) | ((uint32_t)(q3 & 0xFF) << 24);
    if (part == 0) {
        const float dq = fk_h2f(fk_f2h(d));
        dx[(size_t)kb * n_pad + t] = dq;
        if (sx) sx[(size_t)kb * n_pad + t] = dq * (float)qsum;
    }
}

// Dense plan: padded row t reads token t (t < m) and writes output row t.
__global__ void dense_plan_kernel(int m, int n_pad, int* src_row, int* out_row) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < n_pad) {
        src_row[t] = t < m ? t : -1;
        out_row[t] = t < m ? t : -1;
    }
}

// Grouped plan (one block): every expert's rows padded up to whole tiles of BN.
// Permuted row p of expert e lands at pad_off[e] + (p - group_off[e]).  The offsets are a serial scan by one thread
// (a few hundred additions); everything else is spread over the block: a thread finds its row's expert by bisecting
// the group offsets in shared memory.
__global__ void grouped_plan_kernel(const int* __restrict__ group_off, const int* __restrict__ gather, int n_experts, int bn,
                                    int n_pad, int* src_row, int* out_row, int* tile_expert, int* n_tiles) {
    extern __shared__ int sm_plan[];  // pad_off [n_experts + 1] | group_off [n_experts + 1]
    int* pad_off = sm_plan;
    int* goff = sm_plan + n_experts + 1;
    for (int e = threadIdx.x; e <= n_experts; e += blockDim.x) goff[e] = group_off[e];
    __syncthreads();
    if (threadIdx.x == 0) {
        int acc = 0;
        for (int e = 0; e < n_experts; e++) {
            pad_off[e] = acc;
            acc += (goff[e + 1] - goff[e] + bn - 1) / bn * bn;
        }
        pad_off[n_experts] = acc;
        *n_tiles = acc / bn;
    }
    for (int t = threadIdx.x; t < n_pad; t += blockDim.x) {
        src_row[t] = -1;
        out_row[t] = -1;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x)
        for (int tl = pad_off[e] / bn; tl < pad_off[e + 1] / bn; tl++) tile_expert[tl] = e;
    const int pairs = goff[n_experts];
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        int lo = 0, hi = n_experts;          // the expert e with goff[e] <= p < goff[e + 1] (empty experts are skipped by the bisection)
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (goff[mid] <= p) lo = mid; else hi = mid;
        }
        const int dst = pad_off[lo] + (p - goff[lo]);
        src_row[dst] = gather ? gather[p] : p;
        out_row[dst] = p;
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::mutex mu;
    std::lock_guard<std::mutex> lk(mu);
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// 2-D row-major tensor [outer][inner] of `esize`-byte elements, box [box_outer][box_inner].
int make_map(CUtensorMap* map, CUtensorMapDataType dt, int esize, void* base, uint64_t inner, uint64_t outer, uint32_t box_inner,
             uint32_t box_outer, CUtensorMapSwizzle sw) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fk_fail(FK_DRIVER_INIT, "gemm: the driver does not export cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {inner * (uint64_t)esize};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, dt, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fk_fail(FK_LAUNCH, "gemm: cuTensorMapEncodeTiled failed (%d) for a [%llu][%llu] tensor", (int)r,
                                          (unsigned long long)outer, (unsigned long long)inner);
    return FK_OK;
}

// The int8 plane of a stack of Q8_0 matrices as a [n_mats][rows][cols] tensor, box [1][BM][KSTAGE].
int make_map_q8_0(CUtensorMap* map, const fk_weight_s* w) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fk_fail(FK_DRIVER_INIT, "gemm: the driver does not export cuTensorMapEncodeTiled");
    cuuint64_t dims[3] = {(cuuint64_t)w->cols, (cuuint64_t)w->rows, (cuuint64_t)w->n_mats};
    cuuint64_t strides[2] = {(cuuint64_t)w->plane_stride[0], (cuuint64_t)w->mat_stride};
    cuuint32_t box[3] = {(cuuint32_t)KSTAGE, (cuuint32_t)BM, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, w->dev + w->plane_off[0], dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fk_fail(FK_LAUNCH, "gemm: cuTensorMapEncodeTiled failed (%d) for %d Q8_0 matrices of %d x %d", (int)r, w->n_mats, w->rows, w->cols);
    return FK_OK;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

template <int KIND, int BN, bool DUMP = false>
int launch_gemm(fk_ctx* ctx, cudaStream_t st, const GemmArgs& a, const CUtensorMap& mq, const CUtensorMap& mdx, const CUtensorMap& msx,
                const CUtensorMap& mw, int n_token_tiles) {
    auto kern = gemm_kernel<KIND, BN, DUMP>;
    constexpr int SMEM = Smem<BN>::TOTAL;
    FK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM), FK_KERNEL);
    constexpr int WROWS = KIND == FK_Q6_K ? BM / 2 : BM;
    dim3 grid((a.rows + WROWS - 1) / WROWS, n_token_tiles);
    kern<<<grid, gemm_threads(BN), SMEM, st>>>(a, mq, mdx, msx, mw);
    FK_CUDA(cudaGetLastError(), FK_LAUNCH);
    ctx->launches++;
    return FK_OK;
}

template <int BN>
int launch_by_kind(fk_ctx* ctx, cudaStream_t st, const GemmArgs& a, const CUtensorMap& mq, const CUtensorMap& mdx, const CUtensorMap& msx,
                   const CUtensorMap& mw, int n_token_tiles) {
    if (a.isums && BN == 128) {
        switch (a.kind) {
            case FK_Q4_K: return launch_gemm<FK_Q4_K, 128, true>(ctx, st, a, mq, mdx, msx, mw, n_token_tiles);
            case FK_Q6_K: return launch_gemm<FK_Q6_K, 128, true>(ctx, st, a, mq, mdx, msx, mw, n_token_tiles);
            case FK_Q8_0: return launch_gemm<FK_Q8_0, 128, true>(ctx, st, a, mq, mdx, msx, mw, n_token_tiles);
            case FK_MXFP4: return launch_gemm<FK_MXFP4, 128, true>(ctx, st, a, mq, mdx, msx, mw, n_token_tiles);
        }
    }
    switch (a.kind) {
        case FK_Q4_K: return launch_gemm<FK_Q4_K, BN>(ctx, st, a, mq, mdx, msx, mw, n_token_tiles);
        case FK_Q6_K: return launch_gemm<FK_Q6_K, BN>(ctx, st, a, mq, mdx, msx, mw, n_token_tiles);
        case FK_Q8_0: return launch_gemm<FK_Q8_0, BN>(ctx, st, a, mq, mdx, msx, mw, n_token_tiles);
        case FK_MXFP4: return launch_gemm<FK_MXFP4, BN>(ctx, st, a, mq, mdx, msx, mw, n_token_tiles);
    }
    return fk_fail(FK_UNSUPPORTED, "gemm: kind %d has no kernel", a.kind);
}

// Shared body of fk_gemm (group_off == nullptr) and fk_gemm_grouped.
int gemm_common(fk_ctx* ctx, cudaStream_t st, fk_weight w, int mat, const int* group_off, const int* gather, const float* x,
                int n_tokens, float* out, int32_t* isums = nullptr) {
    const bool grouped = group_off != nullptr;
    if (w->kind == FK_Q5_K || w->kind == FK_BF16)   // before anything is enqueued: the caller takes batches of 8 through the matvec
        return fk_fail(FK_UNSUPPORTED, "gemm: kind %d has the plain matvec only", w->kind);
    const int bn = grouped ? 64 : 128;
    const int n_tiles_max = grouped ? (n_tokens + bn - 1) / bn + w->n_mats : (n_tokens + bn - 1) / bn;
    const int n_pad = n_tiles_max * bn;
    const int nkb = w->cols / 32;
    // scratch: q plane | dx | sx | src_row | out_row | tile_expert | n_tiles
    size_t off_q = 0, off_dx = align_up(off_q + (size_t)n_pad * w->cols, 1024);
    size_t off_sx = align_up(off_dx + (size_t)nkb * n_pad * 4, 1024);
    size_t off_src = align_up(off_sx + (size_t)nkb * n_pad * 4, 1024);
    size_t off_out = off_src + (size_t)n_pad * 4, off_te = off_out + (size_t)n_pad * 4;
    size_t off_nt = off_te + (size_t)n_tiles_max * 4, total = off_nt + 16;
    int rc = fk_ensure_scratch(ctx, st, total);
    if (rc) return rc;
    uint8_t* sc = ctx->scratch;
    int8_t* q = (int8_t*)(sc + off_q);
    float* dx = (float*)(sc + off_dx);
    float* sx = (float*)(sc + off_sx);
    int* src_row = (int*)(sc + off_src);
    int* out_row = (int*)(sc + off_out);
    int* tile_expert = (int*)(sc + off_te);
    int* n_tiles = (int*)(sc + off_nt);

    if (grouped) {
        grouped_plan_kernel<<<1, 1024, 2 * (w->n_mats + 1) * sizeof(int), st>>>(group_off, gather, w->n_mats, bn, n_pad, src_row, out_row,
                                                                             tile_expert, n_tiles);
    } else {
        dense_plan_kernel<<<(n_pad + 255) / 256, 256, 0, st>>>(n_tokens, n_pad, src_row, out_row);
    }
    FK_CUDA(cudaGetLastError(), FK_LAUNCH);
    const long long runs = (long long)n_pad * nkb;
    if (w->kind == FK_MXFP4)
        quantize_acts_kernel<<<(unsigned)((runs + 7) / 8), 256, 0, st>>>(x, src_row, n_pad, w->cols, w->kind, q, dx, nullptr);
    else
        quantize_acts4_kernel<<<(unsigned)((runs + 31) / 32), 256, 0, st>>>(x, src_row, n_pad, w->cols, q, dx, w->kind == FK_Q4_K ? sx : nullptr,
                                                                            grouped ? n_tiles : nullptr, bn);
    FK_CUDA(cudaGetLastError(), FK_LAUNCH);
    ctx->launches += 2;

    CUtensorMap mq, mdx, msx, mw;
    if ((rc = make_map(&mq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, q, w->cols, n_pad, KSTAGE, bn, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
    if ((rc = make_map(&mdx, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, dx, n_pad, nkb, bn, 4, CU_TENSOR_MAP_SWIZZLE_NONE))) return rc;
    if ((rc = make_map(&msx, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, sx, n_pad, nkb, bn, 4, CU_TENSOR_MAP_SWIZZLE_NONE))) return rc;
    mw = mq;
    if (w->kind == FK_Q8_0 && (rc = make_map_q8_0(&mw, w))) return rc;
    GemmArgs a;
    a.w = w->dev;
    a.mat_stride = w->mat_stride;
    for (int i = 0; i < 4; i++) { a.plane_off[i] = w->plane_off[i]; a.plane_stride[i] = w->plane_stride[i]; }
    a.kind = w->kind;
    a.rows = w->rows;
    a.cols = w->cols;
    a.mat = mat;
    a.tile_expert = grouped ? tile_expert : nullptr;
    a.n_tiles_dev = grouped ? n_tiles : nullptr;
    a.out_row = out_row;
    a.out = out;
    a.isums = isums;
    a.err = ctx->err_flag;
    return grouped ? launch_by_kind<64>(ctx, st, a, mq, mdx, msx, mw, n_tiles_max) : launch_by_kind<128>(ctx, st, a, mq, mdx, msx, mw, n_tiles_max);
}

}  // namespace

#ifdef FK_TRACE
extern "C" __attribute__((visibility("default"))) int fk_gemm_trace_read(void* host, size_t bytes) {
    return cudaMemcpyFromSymbol(host, fk_gemm_trace, bytes) == cudaSuccess ? 0 : 1;
}
#endif

// General 2-D map for the other kernel files: dtype 0 = uint8, 1 = uint16, 2 = uint32, 3 = float32;
// swizzle 0 = none, 1 = 32 B, 2 = 64 B, 3 = 128 B.
int fk_make_map_2d(void* map, int dtype, void* base, uint64_t inner, uint64_t outer, uint32_t box_inner, uint32_t box_outer, int swizzle) {
    static const CUtensorMapDataType dt[4] = {CU_TENSOR_MAP_DATA_TYPE_UINT8, CU_TENSOR_MAP_DATA_TYPE_UINT16, CU_TENSOR_MAP_DATA_TYPE_UINT32,
                                              CU_TENSOR_MAP_DATA_TYPE_FLOAT32};
    static const int es[4] = {1, 2, 4, 4};
    static const CUtensorMapSwizzle sw[4] = {CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_SWIZZLE_128B};
    return make_map((CUtensorMap*)map, dt[dtype], es[dtype], base, inner, outer, box_inner, box_outer, sw[swizzle]);
}

// A [outer][inner] tensor of 32-bit words, unswizzled, for the other kernel files.
int fk_make_map_u32(void* map, void* base, uint64_t inner_words, uint64_t outer, uint32_t box_inner, uint32_t box_outer) {
    return make_map((CUtensorMap*)map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, base, inner_words, outer, box_inner, box_outer, CU_TENSOR_MAP_SWIZZLE_NONE);
}

FK_EXPORT int fk_gemm(fk_ctx* ctx, void* stream, fk_weight w, int mat, const float* x_dev, int m, float* out_dev) {
    if (!ctx || !w || !x_dev || !out_dev) return fk_fail(FK_INVALID, "gemm: null argument");
    if (m < 1) return fk_fail(FK_INVALID, "gemm: m=%d", m);
    if (mat < 0 || mat >= w->n_mats) return fk_fail(FK_INVALID, "gemm: matrix %d of %d", mat, w->n_mats);
    FkDeviceGuard g(ctx->device);
    return gemm_common(ctx, (cudaStream_t)stream, w, mat, nullptr, nullptr, x_dev, m, out_dev);
}

FK_EXPORT int fk_gemm_isums(fk_ctx* ctx, void* stream, fk_weight w, int mat, const float* x_dev, int m, float* out_dev, int32_t* isums_dev) {
    if (!ctx || !w || !x_dev || !out_dev || !isums_dev) return fk_fail(FK_INVALID, "gemm_isums: null argument");
    if (m < 1) return fk_fail(FK_INVALID, "gemm_isums: m=%d", m);
    if (mat < 0 || mat >= w->n_mats) return fk_fail(FK_INVALID, "gemm_isums: matrix %d of %d", mat, w->n_mats);
    FkDeviceGuard g(ctx->device);
    return gemm_common(ctx, (cudaStream_t)stream, w, mat, nullptr, nullptr, x_dev, m, out_dev, isums_dev);
}

FK_EXPORT int fk_gemm_grouped(fk_ctx* ctx, void* stream, fk_weight w, const int* group_off_dev, const int* gather_dev,
                              const float* x_dev, int pairs, float* out_dev) {
    if (!ctx || !w || !group_off_dev || !x_dev || !out_dev) return fk_fail(FK_INVALID, "gemm_grouped: null argument");
    if (pairs < 1) return fk_fail(FK_INVALID, "gemm_grouped: pairs=%d", pairs);
    FkDeviceGuard g(ctx->device);
    return gemm_common(ctx, (cudaStream_t)stream, w, 0, group_off_dev, gather_dev, x_dev, pairs, out_dev);
}

// ---------------------------------------------------------------------------
// fk_gemm without any allocation.
//
// Some callers cannot allocate device memory at the moment they need a GEMM: a
// host thread that is inside a CUDA stream capture (cudaMalloc is not allowed
// there), a serving loop that must not hit the implicit device-wide
// synchronisation of cudaMalloc/cudaFree, or a process whose memory budget was
// handed out up front.  fk_gemm grows the context's scratch block on demand,
// so it is not for them.  This variant keeps its scratch (the int8 activation
// plane, the two scale planes and the row tables) in the fixed array below,
// which every GPU that loads this library holds from load to exit.
constexpr size_t FK_GEMM_STATIC_BYTES = 6u << 20;   // 6 MiB: e.g. 512 tokens x 8192 columns
static __device__ __align__(256) uint8_t fk_gemm_static_scratch[FK_GEMM_STATIC_BYTES];

namespace {
// In host code the array's name is only a handle; the device address comes from
// cudaGetSymbolAddress, asked once per device with that device current.
std::mutex g_static_mu;
uint8_t* g_static_ptr[64] = {nullptr};

int static_scratch(fk_ctx* ctx, uint8_t** out) {
    std::lock_guard<std::mutex> lk(g_static_mu);
    if (ctx->device < 0 || ctx->device >= 64) return fk_fail(FK_INVALID, "gemm_static: device %d", ctx->device);
    if (!g_static_ptr[ctx->device]) {
        void* p = nullptr;
        FK_CUDA(cudaGetSymbolAddress(&p, fk_gemm_static_scratch), FK_DRIVER_INIT);
        g_static_ptr[ctx->device] = (uint8_t*)p;
    }
    *out = g_static_ptr[ctx->device];
    return FK_OK;
}
}  // namespace

FK_EXPORT int fk_gemm_static(fk_ctx* ctx, void* stream, fk_weight w, int mat, const float* x_dev, int m, float* out_dev) {
    if (!ctx || !w || !x_dev || !out_dev) return fk_fail(FK_INVALID, "gemm_static: null argument");
    if (m < 1) return fk_fail(FK_INVALID, "gemm_static: m=%d", m);
    if (mat < 0 || mat >= w->n_mats) return fk_fail(FK_INVALID, "gemm_static: matrix %d of %d", mat, w->n_mats);
    FkDeviceGuard g(ctx->device);
    cudaStream_t st = (cudaStream_t)stream;
    const int bn = 128;
    const int n_tiles = (m + bn - 1) / bn, n_pad = n_tiles * bn, nkb = w->cols / 32;
    // the same carve-up as fk_gemm's: q plane | dx | sx | src_row | out_row
    const size_t off_dx = align_up((size_t)n_pad * w->cols, 1024);
    const size_t off_sx = align_up(off_dx + (size_t)nkb * n_pad * 4, 1024);
    const size_t off_src = align_up(off_sx + (size_t)nkb * n_pad * 4, 1024);
    const size_t off_out = off_src + (size_t)n_pad * 4, total = off_out + (size_t)n_pad * 4;
    if (total > FK_GEMM_STATIC_BYTES)
        return fk_fail(FK_INVALID, "gemm_static: %d tokens x %d columns needs %zu bytes of scratch, the fixed block holds %zu (use fk_gemm)",
                       m, w->cols, total, (size_t)FK_GEMM_STATIC_BYTES);
    uint8_t* sc = nullptr;
    int rc = static_scratch(ctx, &sc);
    if (rc) return rc;
    int8_t* q = (int8_t*)sc;
    float* dx = (float*)(sc + off_dx);
    float* sx = (float*)(sc + off_sx);
    int* src_row = (int*)(sc + off_src);
    int* out_row = (int*)(sc + off_out);
    // Nothing in the block has to start at zero: the two kernels below write every
    // word the GEMM reads (padding rows included) before it reads them.
    dense_plan_kernel<<<(n_pad + 255) / 256, 256, 0, st>>>(m, n_pad, src_row, out_row);
    FK_CUDA(cudaGetLastError(), FK_LAUNCH);
    const long long runs = (long long)n_pad * nkb;
    quantize_acts_kernel<<<(unsigned)((runs + 7) / 8), 256, 0, st>>>(x_dev, src_row, n_pad, w->cols, w->kind, q, dx, w->kind == FK_Q4_K ? sx : nullptr);
    FK_CUDA(cudaGetLastError(), FK_LAUNCH);
    ctx->launches += 2;
    CUtensorMap mq, mdx, msx, mw;
    if ((rc = make_map(&mq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, q, w->cols, n_pad, KSTAGE, bn, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
    if ((rc = make_map(&mdx, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, dx, n_pad, nkb, bn, 4, CU_TENSOR_MAP_SWIZZLE_NONE))) return rc;
    if ((rc = make_map(&msx, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, sx, n_pad, nkb, bn, 4, CU_TENSOR_MAP_SWIZZLE_NONE))) return rc;
    mw = mq;
    if (w->kind == FK_Q8_0 && (rc = make_map_q8_0(&mw, w))) return rc;
    GemmArgs a;
    a.w = w->dev;
    a.mat_stride = w->mat_stride;
    for (int i = 0; i < 4; i++) { a.plane_off[i] = w->plane_off[i]; a.plane_stride[i] = w->plane_stride[i]; }
    a.kind = w->kind;
    a.rows = w->rows;
    a.cols = w->cols;
    a.mat = mat;
    a.tile_expert = nullptr;
    a.n_tiles_dev = nullptr;
    a.out_row = out_row;
    a.out = out_dev;
    a.isums = nullptr;
    a.err = ctx->err_flag;
    return launch_by_kind<128>(ctx, st, a, mq, mdx, msx, mw, n_tiles);
}

// The error word kernels raise when a bounded wait gives up: 0 = none.
FK_EXPORT int fk_device_error(fk_ctx* ctx, int* code, int reset) {
    if (!ctx || !code) return fk_fail(FK_INVALID, "device_error: null argument");
    FkDeviceGuard g(ctx->device);
    FK_CUDA(cudaMemcpy(code, ctx->err_flag, sizeof(int), cudaMemcpyDeviceToHost), FK_LAUNCH);
    if (reset && *code) {
        FK_CUDA(cudaMemset(ctx->err_flag, 0, sizeof(int)), FK_LAUNCH);
        *ctx->err_pin = 0;
    }
    return FK_OK;
}
