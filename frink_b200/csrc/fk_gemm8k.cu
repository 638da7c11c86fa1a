// Prefill GEMM for the K-quants on Q8_K activations (frink's CPU activation rule: one f32 scale
// and sixteen 16-value sums per 256 values, crates/frink-quant/src/act_quant.rs:69-104), whose
// integers are frink's CPU vec_dot itself (crates/frink-quant/src/lib.rs:822-869):
//
//   out[t][r] = sum over super-blocks sb of  da[t][sb] * ( d[r][sb] * S - dmin[r][sb] * M )
//   S = sum_j sc[r][sb][j] * ( sum_{k in sub-block j} nib[r][k] * q[t][k] )      exact int32
//   M = sum_j m[r][sb][j] * ( sum of q[t] over sub-block j )                       exact
//
// With one activation scale per super-block the 6-bit sub-block scales are integers that fold
// into the int8 operand: sc = 8 s1 + s0 (both below 8), nib * s1 and nib * s0 fit a byte, and
// S = 8 * HI + LO with HI, LO two int8 tensor-core contractions over the whole super-block.  M is
// a third, small contraction (K = 16 on the f16 path: the mins against the sixteen 16-value sums,
// all exact).  The accumulators are drained once per 256 K instead of once per 32.
//
// One CTA = 128 weight rows x 128 tokens: three accumulators (HI, LO, M) of 128 tensor-memory
// columns each.  The unpacked weights never touch shared memory: the A operand lives in tensor
// memory (the remaining 128 columns hold one super-block: 4 stages of K = 64, hi and lo), so an
// MMA reads shared memory only for the activations.  A super-block is an MMA phase (16 int8 MMAs
// of N = 128 at the tensor core's full rate and one small f16 one) and an epilogue phase; the
// unpack of the next super-block and all copies run under both.  22 warps with fixed roles:
//   warps 0..15  epilogue (TMEM lane quadrant = warp & 3, 32 of the 128 token columns each):
//                four per scheduler, so one warp's tensor-memory loads fly under another's arithmetic
//   warps 16..19 unpack: packed Q4_K block (shared memory, staged by TMA) -> nib * s1, nib * s0
//                -> tensor memory (tcgen05.st), and the mins / d / dmin of the block
//   warp 20      TMA producer: weight blocks, activation tiles, their scales and 16-value sums
//   warp 21      MMA issuer + tensor-memory allocation
// Every wait is bounded and raises the context's error word instead of spinning forever.
#include "fk_tc.cuh"

#include <type_traits>

namespace {
using namespace fk_tc;

#ifdef FK_TRACE
__device__ unsigned long long fk_gemm8k_trace[16][64];
__device__ __forceinline__ unsigned long long gtime_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define GTR(k_, i_, who_) do { if ((who_) && blockIdx.x == 0 && blockIdx.y == 0 && (i_) < 64) fk_gemm8k_trace[k_][i_] = gtime_ns(); } while (0)
#define GTW(k_, i_, who_, stmt_) do { const unsigned long long t__ = gtime_ns(); stmt_; if ((who_) && blockIdx.x == 0 && blockIdx.y == 0 && (i_) < 64) fk_gemm8k_trace[k_][i_] += gtime_ns() - t__; } while (0)
#else
#define GTR(k_, i_, who_) do { } while (0)
#define GTW(k_, i_, who_, stmt_) do { stmt_; } while (0)
#endif

constexpr int BM = 128, BN = 128;
constexpr int EPI_WARPS = 16, UNPACK_WARPS = 4;
constexpr int EC = 32;   // token columns an epilogue warp owns
constexpr int THREADS = (EPI_WARPS + UNPACK_WARPS + 2) * 32;
constexpr int WS = 3;   // weight blocks in flight (one super-block of 128 rows each)
constexpr int BS = 4;   // activation tiles in flight (128 tokens x K = 128)
constexpr int XS = 2;   // per-super-block extras in flight (activation scales, 16-value sums)
constexpr int W_BYTES = BM * 144, B_BYTES = BN * 128, BP_BYTES = BN * 32, DA_BYTES = BN * 4, X_BYTES = BP_BYTES + 1024;
constexpr int AP_BYTES = BM * 32, DD_BYTES = BM * 8;
constexpr int OFF_W = 0, OFF_B = OFF_W + WS * W_BYTES, OFF_X = OFF_B + BS * B_BYTES, OFF_AP = OFF_X + XS * X_BYTES;
constexpr int OFF_DD = OFF_AP + 2 * AP_BYTES, OFF_BAR = OFF_DD + 2 * DD_BYTES, SMEM_TOTAL = OFF_BAR + 512 + 1024;
// tensor-memory columns
constexpr int COL_HI = 0, COL_LO = 128, COL_MN = 256;
constexpr int COL_A = 384;        // stage s (K = 64): hi at 32 s, lo at 32 s + 16

struct Args8k {
    const int* out_row;   // padded token row -> output row, -1 = padding
    float* out;
    int32_t* isums;       // test hook: [token][rows][super-blocks][2] = S, M (nullptr = off)
    int rows, cols;
    int* err;
};

template <bool DUMP>
__global__ void __launch_bounds__(THREADS, 1)
gemm8k_q4k_kernel(const Args8k a, const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_q,
                  const __grid_constant__ CUtensorMap map_bs, const __grid_constant__ CUtensorMap map_da) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wrow0 = blockIdx.x * BM, tok0 = blockIdx.y * BN;
    const int nsb = a.cols >> 8;

    const uint32_t bar0 = sbase + OFF_BAR;
    int nb = 0;
    auto bars = [&](int n) { const uint32_t b = bar0 + 8u * nb; nb += n; return b; };
    const uint32_t w_full = bars(WS), w_empty = bars(WS), b_full = bars(BS), b_empty = bars(BS), x_full = bars(XS), x_empty = bars(XS);
    const uint32_t a_full = bars(4), a_empty = bars(4), ap_full = bars(2), ap_empty = bars(2), acc_full = bars(1), acc_empty = bars(1);
    uint32_t* tmem_word = (uint32_t*)(smem + OFF_BAR + 8 * nb);

    if (threadIdx.x == 0) {
        for (int i = 0; i < WS; i++) { mbar_init(w_full + 8 * i, 1); mbar_init(w_empty + 8 * i, UNPACK_WARPS); }
        for (int i = 0; i < BS; i++) { mbar_init(b_full + 8 * i, 1); mbar_init(b_empty + 8 * i, 1); }
        for (int i = 0; i < XS; i++) { mbar_init(x_full + 8 * i, 1); mbar_init(x_empty + 8 * i, 1 + EPI_WARPS); }
        for (int i = 0; i < 4; i++) { mbar_init(a_full + 8 * i, UNPACK_WARPS); mbar_init(a_empty + 8 * i, 1); }
        for (int i = 0; i < 2; i++) { mbar_init(ap_full + 8 * i, UNPACK_WARPS); mbar_init(ap_empty + 8 * i, 1 + EPI_WARPS); }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, EPI_WARPS);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == EPI_WARPS + UNPACK_WARPS + 1) {   // the MMA warp owns tensor memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_word)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_word;

    if (warp < EPI_WARPS) {
        // ------------------------------------------------------------------ epilogue
        const int quad = warp & 3, cg = warp >> 2;
        const int r = quad * 32 + lane, row = wrow0 + r;
        const int col0 = cg * EC;                             // first token column of this warp inside the tile
        const uint32_t tl = tmem_base + ((uint32_t)(quad * 32) << 16) + cg * EC;
        float acc[EC];
#pragma unroll
        for (int i = 0; i < EC; i++) acc[i] = 0.0f;
        for (int sb = 0; sb < nsb; sb++) {
            const int xs = sb % XS, ap = sb & 1;
            mbar_wait_parked(ap_full + 8 * ap, (sb >> 1) & 1, a.err, 60);
            const float2 dd = *(const float2*)(smem + OFF_DD + ap * DD_BYTES + r * 8);
            mbar_wait_parked(x_full + 8 * xs, (sb / XS) & 1, a.err, 61);
            const uint32_t das = sbase + OFF_X + xs * X_BYTES + BP_BYTES + (uint32_t)col0 * 4u;
            mbar_wait_parked(acc_full, sb & 1, a.err, 62);
            tc_fence_after();
            GTR(10, sb, threadIdx.x == 0);
#pragma unroll
            for (int c = 0; c < EC / 8; c++) {
                uint32_t hi[8], lo[8], mn[8];
                tc_ld8(tl + COL_HI + c * 8, hi);
                tc_ld8(tl + COL_LO + c * 8, lo);
                tc_ld8(tl + COL_MN + c * 8, mn);
                tc_wait_ld();
                tc_ld_fence<8>(hi);
                tc_ld_fence<8>(lo);
                tc_ld_fence<8>(mn);
#pragma unroll
                for (int i = 0; i < 8; i += 4) {
                    const float4 da4 = lds128(das + (uint32_t)(c * 8 + i) * 4u);
                    // S = 8 HI + LO.  Columns 0, 1 of the four: both halves made floats by the 2^23 trick (exact: each is
                    // below 2^22) and joined by one fused multiply-add, which rounds the exact sum once; columns 2, 3: the
                    // integer sum through the conversion unit, which rounds the same way.  Two pipes share the work.
                    const float2 fh = __fadd2_rn(make_float2(__int_as_float((int)hi[i] + 0x4B400000), __int_as_float((int)hi[i + 1] + 0x4B400000)),
                                                 make_float2(-12582912.0f, -12582912.0f));
                    const float2 fl = __fadd2_rn(make_float2(__int_as_float((int)lo[i] + 0x4B400000), __int_as_float((int)lo[i + 1] + 0x4B400000)),
                                                 make_float2(-12582912.0f, -12582912.0f));
                    const float2 s01 = __ffma2_rn(fh, make_float2(8.0f, 8.0f), fl);
                    const float2 s23 = make_float2((float)(8 * (int)hi[i + 2] + (int)lo[i + 2]), (float)(8 * (int)hi[i + 3] + (int)lo[i + 3]));
                    const float2 m01 = make_float2(__uint_as_float(mn[i]), __uint_as_float(mn[i + 1]));
                    const float2 m23 = make_float2(__uint_as_float(mn[i + 2]), __uint_as_float(mn[i + 3]));
                    const float2 nd = make_float2(-dd.y, -dd.y), dv = make_float2(dd.x, dd.x);
                    const float2 t01 = __ffma2_rn(nd, m01, __fmul2_rn(dv, s01));
                    const float2 t23 = __ffma2_rn(nd, m23, __fmul2_rn(dv, s23));
                    const float2 a01 = __ffma2_rn(make_float2(da4.x, da4.y), t01, make_float2(acc[c * 8 + i], acc[c * 8 + i + 1]));
                    const float2 a23 = __ffma2_rn(make_float2(da4.z, da4.w), t23, make_float2(acc[c * 8 + i + 2], acc[c * 8 + i + 3]));
                    acc[c * 8 + i] = a01.x; acc[c * 8 + i + 1] = a01.y; acc[c * 8 + i + 2] = a23.x; acc[c * 8 + i + 3] = a23.y;
                    if (DUMP && row < a.rows) {
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            const int dst = a.out_row[tok0 + col0 + c * 8 + i + e];
                            if (dst >= 0) {
                                int32_t* o = a.isums + (((size_t)dst * a.rows + row) * nsb + sb) * 2;
                                o[0] = 8 * (int)hi[i + e] + (int)lo[i + e];
                                o[1] = (int)__uint_as_float(mn[i + e]);
                            }
                        }
                    }
                }
            }
            // the accumulators, this block's scales and this super-block's activation scales are free again
            tc_fence_before();
            __syncwarp();
            GTR(13, sb, threadIdx.x == 0);
            if (lane == 0) {
                mbar_arrive(acc_empty);
                mbar_arrive(x_empty + 8 * xs);
                mbar_arrive(ap_empty + 8 * ap);
            }
        }
        if (row < a.rows) {
#pragma unroll
            for (int i = 0; i < EC; i++) {
                const int dst = a.out_row[tok0 + col0 + i];
                if (dst >= 0) a.out[(size_t)dst * a.rows + row] = acc[i];
            }
        }
    } else if (warp < EPI_WARPS + UNPACK_WARPS) {
        // -------------------------------------------------------------------- unpack
        const int quad = warp & 3, r = quad * 32 + lane;
        const uint32_t ta = tmem_base + ((uint32_t)(quad * 32) << 16) + COL_A;
        for (int sb = 0; sb < nsb; sb++) {
            const int ws = sb % WS, ap = sb & 1;
            mbar_wait_parked(w_full + 8 * ws, (sb / WS) & 1, a.err, 70);
            const uint32_t blk = sbase + OFF_W + ws * W_BYTES + (uint32_t)r * 144u;
            const uint4 hd = lds16(blk);
            // 6-bit scales and mins of the 8 sub-blocks, one per byte: [0..3] and [4..7]
            const uint32_t scw[2] = {hd.y & 0x3F3F3F3Fu, (hd.w & 0x0F0F0F0Fu) | ((hd.y >> 2) & 0x30303030u)};
            const uint32_t mnw[2] = {hd.z & 0x3F3F3F3Fu, ((hd.w >> 4) & 0x0F0F0F0Fu) | ((hd.z >> 2) & 0x30303030u)};
            if (sb >= 2) mbar_wait_parked(ap_empty + 8 * ap, ((sb >> 1) - 1) & 1, a.err, 71);
            *(float2*)(smem + OFF_DD + ap * DD_BYTES + r * 8) = make_float2(fk_h2f((uint16_t)(hd.x & 0xFFFF)), fk_h2f((uint16_t)(hd.x >> 16)));
            {
                // the mins as f16, each twice (one per 16-value sum of its sub-block): a 128 x 16 K-major operand in
                // 8-row x 16-byte core matrices, the two along K 128 bytes apart, 8-row groups 256 bytes apart
                uint32_t mh[8];
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const uint32_t m = (mnw[j >> 2] >> (8 * (j & 3))) & 0xFFu;
                    const uint32_t hb = (uint32_t)__half_as_ushort(__uint2half_rn(m));
                    mh[j] = hb | (hb << 16);
                }
                uint8_t* dst = smem + OFF_AP + ap * AP_BYTES + (r >> 3) * 256 + (r & 7) * 16;
                *(uint4*)dst = make_uint4(mh[0], mh[1], mh[2], mh[3]);
                *(uint4*)(dst + 128) = make_uint4(mh[4], mh[5], mh[6], mh[7]);
            }
            fence_proxy_async();   // generic-proxy writes -> visible to the tensor core's reads
            __syncwarp();
            if (lane == 0) mbar_arrive(ap_full + 8 * ap);
            const uint32_t s1w[2] = {(scw[0] >> 3) & 0x07070707u, (scw[1] >> 3) & 0x07070707u};
            const uint32_t s0w[2] = {scw[0] & 0x07070707u, scw[1] & 0x07070707u};
#pragma unroll
            for (int s = 0; s < 4; s++) {
                const uint4 q0 = lds16(blk + 16 + 32 * s), q1 = lds16(blk + 32 + 32 * s);
                const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
                const int sh = 16 * (s & 1);
                const uint32_t a1 = (s1w[s >> 1] >> sh) & 0xFFu, b1 = (s1w[s >> 1] >> (sh + 8)) & 0xFFu;
                const uint32_t a0 = (s0w[s >> 1] >> sh) & 0xFFu, b0 = (s0w[s >> 1] >> (sh + 8)) & 0xFFu;
                uint32_t hi[16], lo[16];
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const uint32_t ln = w[i] & 0x0F0F0F0Fu, hn = (w[i] >> 4) & 0x0F0F0F0Fu;   // sub-block 2s, sub-block 2s + 1
                    hi[i] = ln * a1;       // four byte-wide products at once: each is below 128
                    hi[8 + i] = hn * b1;
                    lo[i] = ln * a0;
                    lo[8 + i] = hn * b0;
                }
                if (sb >= 1) {
                    mbar_wait_parked(a_empty + 8 * s, (sb - 1) & 1, a.err, 72);
                    tc_fence_after();
                }
                tc_st16(ta + 32 * s, hi);
                tc_st16(ta + 32 * s + 16, lo);
                tc_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(a_full + 8 * s);
#ifdef FK_TRACE
                if (lane == 0 && blockIdx.x == 0 && blockIdx.y == 0 && sb < 64 && s == 3) atomicMax(&fk_gemm8k_trace[11][sb], gtime_ns());
#endif
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(w_empty + 8 * ws);
        }
    } else if (warp == EPI_WARPS + UNPACK_WARPS) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            for (int sb = 0; sb < nsb; sb++) {
                const int ws = sb % WS, xs = sb % XS;
                if (sb >= WS) mbar_wait_parked_thread(w_empty + 8 * ws, ((sb / WS) - 1) & 1, a.err, 80);
                mbar_expect_tx(w_full + 8 * ws, W_BYTES);
                tma_load_2d(sbase + OFF_W + ws * W_BYTES, &map_w, sb * 36, wrow0, w_full + 8 * ws);
                if (sb >= XS) mbar_wait_parked_thread(x_empty + 8 * xs, ((sb / XS) - 1) & 1, a.err, 81);
                mbar_expect_tx(x_full + 8 * xs, BP_BYTES + DA_BYTES);
                tma_load_2d(sbase + OFF_X + xs * X_BYTES, &map_bs, sb * 16, tok0, x_full + 8 * xs);
                tma_load_2d(sbase + OFF_X + xs * X_BYTES + BP_BYTES, &map_da, tok0, sb, x_full + 8 * xs);
                for (int t = 0; t < 2; t++) {
                    const int kt = 2 * sb + t, bt = kt % BS;
                    if (kt >= BS) mbar_wait_parked_thread(b_empty + 8 * bt, ((kt / BS) - 1) & 1, a.err, 82);
                    mbar_expect_tx(b_full + 8 * bt, B_BYTES);
                    tma_load_2d(sbase + OFF_B + bt * B_BYTES, &map_q, kt * 128, tok0, b_full + 8 * bt);
                }
            }
        }
    } else {
        // -------------------------------------------------------------------- MMA issuer
        // One lane issues every MMA, and what it executes between two of them is time the tensor core
        // idles.  So the whole warp walks the loop in uniform control flow (only the instructions
        // themselves are predicated on the lane) and super-blocks are taken two at a time: ring slots
        // then depend on the parity only, every descriptor is a constant offset from the shared-memory
        // base, and the accumulate flags are constants.
        {
            constexpr uint32_t IDESC_I8 = umma_idesc_i8(BM, BN), IDESC_F16 = umma_idesc_f16(BM, BN);
            const uint32_t on = lane == 0 ? 1u : 0u;
            const uint32_t ta = tmem_base + COL_A, d_hi = tmem_base + COL_HI, d_lo = tmem_base + COL_LO, d_mn = tmem_base + COL_MN;
            auto super_block = [&](auto parity, int sb) {
                constexpr int P = decltype(parity)::value;      // sb & 1: activation tiles 2 P, 2 P + 1 of the ring of 4, extras slot P, A' slot P
                static_assert(BS == 4 && XS == 2, "ring slots are tied to the parity of the super-block");
                // the K = 128 activation tiles (128-byte swizzle, 8-row groups 1024 bytes apart); the mins (f16, K = 16, plain core
                // matrices 128 bytes apart along K, 8-row groups 256 apart); the 16-value sums (f16, 32-byte swizzle, groups 256 apart)
                const uint64_t db0 = umma_desc(sbase + OFF_B + (2 * P) * B_BYTES), db1 = umma_desc(sbase + OFF_B + (2 * P + 1) * B_BYTES);
                const uint64_t dap = umma_desc_of(sbase + OFF_AP + P * AP_BYTES, 128, 256, 0);
                const uint64_t dbp = umma_desc_of(sbase + OFF_X + P * X_BYTES, 16, 256, 6);
                GTR(12, sb, lane == 0);
                if (sb >= 1) mbar_wait_spin(acc_empty, (sb - 1) & 1, a.err, 90);
                GTR(0, sb, lane == 0);
#pragma unroll
                for (int s = 0; s < 4; s++) {
                    GTW((s == 0 ? 4 : s == 1 ? 6 : s == 2 ? 8 : 9), sb, lane == 0, mbar_wait_spin(a_full + 8 * s, sb & 1, a.err, 91));
                    if (s == 0) mbar_wait_spin(b_full + 8 * (2 * P), (sb >> 1) & 1, a.err, 92);
                    if (s == 2) mbar_wait_spin(b_full + 8 * (2 * P + 1), (sb >> 1) & 1, a.err, 92);
                    tc_fence_after();
                    const uint64_t db = s < 2 ? db0 : db1;
#pragma unroll
                    for (int j = 0; j < 2; j++) {
                        const uint64_t dbk = db + 2 * ((s & 1) * 2 + j);   // K advances 32 bytes inside the 128-byte swizzle atom
                        tc_mma_i8_ts_if(on, d_hi, ta + 32 * s + 8 * j, dbk, IDESC_I8, (s | j) ? 1u : 0u);
                        tc_mma_i8_ts_if(on, d_lo, ta + 32 * s + 16 + 8 * j, dbk, IDESC_I8, (s | j) ? 1u : 0u);
                    }
                    GTR(1 + 2 * s, sb, lane == 0);
                    tc_commit_if(on, a_empty + 8 * s);                         // this stage of A may be overwritten
                    if (s == 1) tc_commit_if(on, b_empty + 8 * (2 * P));       // and these activation tiles
                    if (s == 3) tc_commit_if(on, b_empty + 8 * (2 * P + 1));
                }
                mbar_wait_spin(x_full + 8 * P, (sb >> 1) & 1, a.err, 93); mbar_wait_spin(ap_full + 8 * P, (sb >> 1) & 1, a.err, 94);
                tc_fence_after();
                tc_mma_f16_ss_if(on, d_mn, dap, dbp, IDESC_F16, 0u); tc_commit_if(on, acc_full);
                GTR(2, sb, lane == 0);
                tc_commit_if(on, x_empty + 8 * P);
                tc_commit_if(on, ap_empty + 8 * P);
            };
            for (int sb = 0; sb < nsb; sb += 2) {
                super_block(std::integral_constant<int, 0>{}, sb);
                if (sb + 1 < nsb) super_block(std::integral_constant<int, 1>{}, sb + 1);
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

// Activations -> Q8_K (act_quant.rs:69-104): per 256 values amax, iscale = 127 / amax, q = the product rounded to
// nearest-even and clamped to +-127, d = 1 / iscale, and the sums of every 16 quants.  One warp per (padded token,
// super-block); planes: q [n_pad][cols] int8, d [nsb][n_pad] f32, sums [n_pad][nsb * 16] f16 (each below 2048: exact).
__global__ void quantize_q8k_kernel(const float* __restrict__ x, const int* __restrict__ src_row, int n_pad, int cols, int8_t* __restrict__ q,
                                    float* __restrict__ da, uint16_t* __restrict__ bs) {
    const int nsb = cols >> 8;
    const long long unit = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (unit >= (long long)n_pad * nsb) return;
    const int t = (int)(unit / nsb), sb = (int)(unit - (long long)t * nsb);
    const int src = src_row[t];
    float v[8];
    if (src >= 0) {
        const float4* p = (const float4*)(x + (size_t)src * cols + sb * 256 + lane * 8);
        const float4 a0 = __ldg(p), a1 = __ldg(p + 1);
        v[0] = a0.x; v[1] = a0.y; v[2] = a0.z; v[3] = a0.w; v[4] = a1.x; v[5] = a1.y; v[6] = a1.z; v[7] = a1.w;
    } else {
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = 0.0f;
    }
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) m = fmaxf(m, fabsf(v[i]));
    const float amax = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(m)));
    int qi[8], s = 0;
    float d = 0.0f;
    if (amax != 0.0f) {
        const float iscale = __fdiv_rn(127.0f, amax);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const float r = fminf(fmaxf(rintf(__fmul_rn(iscale, v[i])), -127.0f), 127.0f);
            qi[i] = (int)r;
            s += qi[i];
        }
        d = __fdiv_rn(1.0f, iscale);
    } else {
#pragma unroll
        for (int i = 0; i < 8; i++) qi[i] = 0;
    }
    uint2 pk;
    pk.x = (uint32_t)(qi[0] & 0xFF) | ((uint32_t)(qi[1] & 0xFF) << 8) | ((uint32_t)(qi[2] & 0xFF) << 16) | ((uint32_t)(qi[3] & 0xFF) << 24);
    pk.y = (uint32_t)(qi[4] & 0xFF) | ((uint32_t)(qi[5] & 0xFF) << 8) | ((uint32_t)(qi[6] & 0xFF) << 16) | ((uint32_t)(qi[7] & 0xFF) << 24);
    *(uint2*)(q + (size_t)t * cols + sb * 256 + lane * 8) = pk;
    const int s16 = s + __shfl_xor_sync(0xffffffffu, s, 1);
    if (!(lane & 1)) bs[((size_t)t * nsb + sb) * 16 + (lane >> 1)] = __half_as_ushort(__int2half_rn(s16));
    if (lane == 0) da[(size_t)sb * n_pad + t] = d;
}

__global__ void dense_plan8k_kernel(int m, int n_pad, int* src_row, int* out_row) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < n_pad) {
        src_row[t] = t < m ? t : -1;
        out_row[t] = t < m ? t : -1;
    }
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int gemm8k(fk_ctx* ctx, cudaStream_t st, fk_weight w, int mat, const float* x, int m, float* out, int32_t* isums) {
    if (w->kind != FK_Q4_K) return fk_fail(FK_UNSUPPORTED, "gemm_q8k: kind %d (Q4_K only)", w->kind);
    const int n_tiles = (m + BN - 1) / BN, n_pad = n_tiles * BN, nsb = w->cols / 256;
    // scratch: q plane | d | 16-value sums | src_row | out_row
    const size_t off_da = align_up((size_t)n_pad * w->cols, 1024);
    const size_t off_bs = align_up(off_da + (size_t)nsb * n_pad * 4, 1024);
    const size_t off_src = align_up(off_bs + (size_t)n_pad * nsb * 32, 1024);
    const size_t off_out = off_src + (size_t)n_pad * 4, total = off_out + (size_t)n_pad * 4;
    int rc = fk_ensure_scratch(ctx, st, total);
    if (rc) return rc;
    uint8_t* sc = ctx->scratch;
    int8_t* q = (int8_t*)sc;
    float* da = (float*)(sc + off_da);
    uint16_t* bs = (uint16_t*)(sc + off_bs);
    int* src_row = (int*)(sc + off_src);
    int* out_row = (int*)(sc + off_out);
    dense_plan8k_kernel<<<(n_pad + 255) / 256, 256, 0, st>>>(m, n_pad, src_row, out_row);
    FK_CUDA(cudaGetLastError(), FK_LAUNCH);
    const long long units = (long long)n_pad * nsb;
    quantize_q8k_kernel<<<(unsigned)((units + 7) / 8), 256, 0, st>>>(x, src_row, n_pad, w->cols, q, da, bs);
    FK_CUDA(cudaGetLastError(), FK_LAUNCH);
    alignas(64) CUtensorMap mw, mq, mbs, mda;
    uint8_t* wbase = w->dev + (size_t)mat * w->mat_stride + w->plane_off[0];
    if ((rc = fk_make_map_2d(&mw, 2, wbase, w->plane_stride[0] / 4, (uint64_t)w->rows, 36, BM, 0))) return rc;
    if ((rc = fk_make_map_2d(&mq, 0, q, (uint64_t)w->cols, (uint64_t)n_pad, 128, BN, 3))) return rc;
    if ((rc = fk_make_map_2d(&mbs, 1, bs, (uint64_t)nsb * 16, (uint64_t)n_pad, 16, BN, 1))) return rc;
    if ((rc = fk_make_map_2d(&mda, 3, da, (uint64_t)n_pad, (uint64_t)nsb, BN, 1, 0))) return rc;
    Args8k a;
    a.out_row = out_row;
    a.out = out;
    a.isums = isums;
    a.rows = w->rows;
    a.cols = w->cols;
    a.err = ctx->err_flag;
    dim3 grid((w->rows + BM - 1) / BM, n_tiles);
    if (isums) {
        FK_CUDA(cudaFuncSetAttribute(gemm8k_q4k_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL), FK_KERNEL);
        gemm8k_q4k_kernel<true><<<grid, THREADS, SMEM_TOTAL, st>>>(a, mw, mq, mbs, mda);
    } else {
        FK_CUDA(cudaFuncSetAttribute(gemm8k_q4k_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL), FK_KERNEL);
        gemm8k_q4k_kernel<false><<<grid, THREADS, SMEM_TOTAL, st>>>(a, mw, mq, mbs, mda);
    }
    FK_CUDA(cudaGetLastError(), FK_LAUNCH);
    ctx->launches += 3;
    return FK_OK;
}

}  // namespace

#ifdef FK_TRACE
FK_EXPORT int fk_gemm8k_trace_read(void* host, size_t bytes) {
    return cudaMemcpyFromSymbol(host, fk_gemm8k_trace, bytes) == cudaSuccess ? 0 : 1;
}
#endif

FK_EXPORT int fk_gemm_q8k(fk_ctx* ctx, void* stream, fk_weight w, int mat, const float* x_dev, int m, float* out_dev) {
    if (!ctx || !w || !x_dev || !out_dev) return fk_fail(FK_INVALID, "gemm_q8k: null argument");
    if (m < 1) return fk_fail(FK_INVALID, "gemm_q8k: m=%d", m);
    if (mat < 0 || mat >= w->n_mats) return fk_fail(FK_INVALID, "gemm_q8k: matrix %d of %d", mat, w->n_mats);
    FkDeviceGuard g(ctx->device);
    return gemm8k(ctx, (cudaStream_t)stream, w, mat, x_dev, m, out_dev, nullptr);
}

FK_EXPORT int fk_gemm_q8k_isums(fk_ctx* ctx, void* stream, fk_weight w, int mat, const float* x_dev, int m, float* out_dev, int32_t* isums_dev) {
    if (!ctx || !w || !x_dev || !out_dev || !isums_dev) return fk_fail(FK_INVALID, "gemm_q8k_isums: null argument");
    if (m < 1) return fk_fail(FK_INVALID, "gemm_q8k_isums: m=%d", m);
    if (mat < 0 || mat >= w->n_mats) return fk_fail(FK_INVALID, "gemm_q8k_isums: matrix %d of %d", mat, w->n_mats);
    FkDeviceGuard g(ctx->device);
    return gemm8k(ctx, (cudaStream_t)stream, w, mat, x_dev, m, out_dev, isums_dev);
}
