// Q5_K decode matvec (crates/frink-quant/src/lib.rs:424-515, 873-939; block: f16 d, f16 dmin, 12 bytes of
// 6-bit scales and mins as Q4_K's, 32 bytes qh, 128 bytes of nibbles = 176 bytes per 256 weights).
// Real Q4_K_M files carry this format in some tensors; it gets the plain matvec (batch 1..8) with the same
// q8_1 activation rule and the same exact per-run integers as the other kinds, not the tuned rings of the
// Q4_K path: a warp walks the super-blocks of one row four at a time (a lane on 16 nibble bytes = 32 weights),
// weights read straight from global memory (16-byte loads, every byte once), the quantized activations from
// shared memory.  HBM-bound on large matrices, latency-bound on small ones.
#include "fk_common.cuh"

namespace {

constexpr int Q5_THREADS = 256, Q5_WARPS = Q5_THREADS / 32;

struct Q5Args {
    const uint8_t* w;      // 176-byte blocks, row-major
    size_t row_bytes;
    const float* x;        // [batch][cols]
    float* y;              // [batch][rows]
    int32_t* isums;        // test hook: [rows][cols / 32] (batch row 0), nullptr = off
    int rows, cols, batch;
};

__device__ __forceinline__ int dp4a_ss(int a, int b, int c) { return __dp4a(a, b, c); }

template <int NB, bool DUMP>
__global__ void __launch_bounds__(Q5_THREADS) gemv_q5k_kernel(const Q5Args a) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int cols = a.cols, nb32 = cols >> 5, nsb = cols >> 8;
    int8_t* sq = (int8_t*)smem;                                   // [NB][cols]
    float* sd = (float*)(smem + (size_t)NB * cols);               // [NB][nb32] f16-rounded scale of the run
    float* ss = sd + (size_t)NB * nb32;                           // [NB][nb32] scale * sum of the run's quants
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // ---- activations -> q8_1 (the rule of fk_q8_1_lane: d = amax / 127, q = roundf(x / d), the scale stored as f16);
    // a thread takes float4s, eight lanes make a run of 32, four loads are in flight per thread
    {
        const int c4 = cols >> 2, items = NB * c4;
        constexpr int QU = 4;
        for (int base = 0; base < items; base += QU * Q5_THREADS) {
            float4 v[QU];
#pragma unroll
            for (int u = 0; u < QU; u++) {
                const int idx = base + u * Q5_THREADS + (int)threadIdx.x;
                v[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (idx < items) {
                    const int b = idx / c4, k4 = idx - b * c4;
                    if (b < a.batch) v[u] = __ldg((const float4*)(a.x + (size_t)b * cols) + k4);
                }
            }
#pragma unroll
            for (int u = 0; u < QU; u++) {
                const int idx = base + u * Q5_THREADS + (int)threadIdx.x;
                const bool ok = idx < items;                       // whole groups of eight lanes are in or out: items is a multiple of 8
                const int b = ok ? idx / c4 : 0, k4 = ok ? idx - b * c4 : 0;
                const float4 f = v[u];
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
                if (ok) {
                    *(uint32_t*)(sq + (size_t)b * cols + 4 * k4) =
                        (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) | ((uint32_t)(q2 & 0xFF) << 16) | ((uint32_t)(q3 & 0xFF) << 24);
                    if ((k4 & 7) == 0) {
                        const float dq = fk_h2f(fk_f2h(d));
                        sd[b * nb32 + (k4 >> 3)] = dq;
                        ss[b * nb32 + (k4 >> 3)] = dq * (float)qsum;
                    }
                }
            }
        }
    }
    __syncthreads();
    // ---- rows round the warps of the grid.  A warp takes four super-blocks of its row at a time: lane = (super-block
    // sbo of the four, 64-element group g, half h of the group's 32 bytes), 16 nibble bytes = 32 weights a lane, so the
    // scale decode is paid once per 32 weights.  The words of up to three such trips are requested before the first is used.
    const int sbo = lane >> 3, g = (lane >> 1) & 3, h = lane & 1;
    const int wid = blockIdx.x * Q5_WARPS + warp, nw = gridDim.x * Q5_WARPS;
    constexpr int SU = 3;
    for (int row = wid; row < a.rows; row += nw) {
        const uint8_t* rp = a.w + (size_t)row * a.row_bytes;
        float acc[NB];
#pragma unroll
        for (int b = 0; b < NB; b++) acc[b] = 0.0f;
        for (int sb0 = 0; sb0 < nsb; sb0 += 4 * SU) {
            uint4 hdv[SU], qhv[SU], qlv[SU];
#pragma unroll
            for (int u = 0; u < SU; u++) {
                const int sbc = min(sb0 + 4 * u + sbo, nsb - 1);                // past the end: re-read the last block (not used)
                const uint8_t* blk = rp + (size_t)sbc * 176;
                hdv[u] = __ldg((const uint4*)blk);                              // d, dmin, scales
                qhv[u] = __ldg((const uint4*)(blk + 16) + h);                   // qh[16 h .. 16 h + 15]
                qlv[u] = __ldg((const uint4*)(blk + 48) + 2 * g + h);           // nibbles of elements 64 g + 16 h .. (low), + 32 (high)
            }
#pragma unroll
            for (int u = 0; u < SU; u++) {
                const int sb = sb0 + 4 * u + sbo;
                const bool live = sb < nsb;
                const uint4 hd = hdv[u];
                const uint32_t qh[4] = {qhv[u].x, qhv[u].y, qhv[u].z, qhv[u].w}, ql[4] = {qlv[u].x, qlv[u].y, qlv[u].z, qlv[u].w};
                // 6-bit scales and mins of sub-blocks 2 g and 2 g + 1, one per byte: [0..3] and [4..7]
                const uint32_t scw = g < 2 ? (hd.y & 0x3F3F3F3Fu) : ((hd.w & 0x0F0F0F0Fu) | ((hd.y >> 2) & 0x30303030u));
                const uint32_t mnw = g < 2 ? (hd.z & 0x3F3F3F3Fu) : (((hd.w >> 4) & 0x0F0F0F0Fu) | ((hd.z >> 2) & 0x30303030u));
                const int sh = 16 * (g & 1);
                const float d = live ? fk_h2f((uint16_t)(hd.x & 0xFFFF)) : 0.0f, dmin = live ? fk_h2f((uint16_t)(hd.x >> 16)) : 0.0f;
                const float dsc0 = d * (float)((scw >> sh) & 0xFFu), dsc1 = d * (float)((scw >> (sh + 8)) & 0xFFu);
                const float dm0 = h == 0 ? dmin * (float)((mnw >> sh) & 0xFFu) : 0.0f;        // the mins count once per sub-block
                const float dm1 = h == 0 ? dmin * (float)((mnw >> (sh + 8)) & 0xFFu) : 0.0f;
                uint32_t lo[4], hi[4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    lo[i] = (ql[i] & 0x0F0F0F0Fu) | (((qh[i] >> (2 * g)) & 0x01010101u) << 4);
                    hi[i] = ((ql[i] >> 4) & 0x0F0F0F0Fu) | (((qh[i] >> (2 * g + 1)) & 0x01010101u) << 4);
                }
                const int sbs = live ? sb : 0, kb0 = sbs * 8 + 2 * g;
#pragma unroll
                for (int b = 0; b < NB; b++) {
                    const int8_t* q8 = sq + (size_t)b * cols + sbs * 256 + 64 * g + 16 * h;
                    const int4 xl = *(const int4*)q8, xh = *(const int4*)(q8 + 32);
                    int il = dp4a_ss((int)lo[0], xl.x, 0), ih = dp4a_ss((int)hi[0], xh.x, 0);
                    il = dp4a_ss((int)lo[1], xl.y, il); ih = dp4a_ss((int)hi[1], xh.y, ih);
                    il = dp4a_ss((int)lo[2], xl.z, il); ih = dp4a_ss((int)hi[2], xh.z, ih);
                    il = dp4a_ss((int)lo[3], xl.w, il); ih = dp4a_ss((int)hi[3], xh.w, ih);
                    const float2 dx = *(const float2*)(sd + b * nb32 + kb0), sx = *(const float2*)(ss + b * nb32 + kb0);
                    acc[b] += dsc0 * dx.x * (float)il + dsc1 * dx.y * (float)ih - (dm0 * sx.x + dm1 * sx.y);
                    if (DUMP && b == 0) {
                        const int sl = il + __shfl_xor_sync(0xffffffffu, il, 1), sh_ = ih + __shfl_xor_sync(0xffffffffu, ih, 1);
                        if (h == 0 && live) {
                            a.isums[(size_t)row * nb32 + kb0] = sl;
                            a.isums[(size_t)row * nb32 + kb0 + 1] = sh_;
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int b = 0; b < NB; b++) {
            const float v = fk_warp_sum(acc[b]);      // xor butterfly: the same order on every run
            if (lane == 0 && b < a.batch) a.y[(size_t)b * a.rows + row] = v;
        }
    }
}

template <int NB, bool DUMP>
int launch(fk_ctx* ctx, cudaStream_t st, const Q5Args& a) {
    const size_t smem = (size_t)NB * a.cols + 2 * (size_t)NB * (a.cols / 32) * sizeof(float);
    if (smem > 200 * 1024) return fk_fail(FK_UNSUPPORTED, "gemv (Q5_K): %d columns x batch %d need %zu bytes of shared memory", a.cols, a.batch, smem);
    auto kern = gemv_q5k_kernel<NB, DUMP>;
    FK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), FK_KERNEL);
    int per_sm = (int)((220 * 1024) / (smem + 1024));
    per_sm = per_sm < 1 ? 1 : per_sm > 6 ? 6 : per_sm;
    int blocks = ctx->sm_count * per_sm;
    const int need = (a.rows + Q5_WARPS - 1) / Q5_WARPS;
    if (blocks > need) blocks = need;
    kern<<<(unsigned)blocks, Q5_THREADS, smem, st>>>(a);
    FK_CUDA(cudaGetLastError(), FK_LAUNCH);
    ctx->launches++;
    return FK_OK;
}

}  // namespace

int fk_gemv_q5k_launch(fk_ctx* ctx, cudaStream_t st, fk_weight w, int mat, const float* x_dev, int batch, float* y_dev, int32_t* isums_dev) {
    Q5Args a{};
    a.w = w->dev + (size_t)mat * w->mat_stride + w->plane_off[0];
    a.row_bytes = w->plane_stride[0];
    a.x = x_dev;
    a.y = y_dev;
    a.isums = isums_dev;
    a.rows = w->rows;
    a.cols = w->cols;
    a.batch = batch;
    if (isums_dev) return launch<1, true>(ctx, st, a);
    if (batch <= 1) return launch<1, false>(ctx, st, a);
    if (batch <= 2) return launch<2, false>(ctx, st, a);
    if (batch <= 4) return launch<4, false>(ctx, st, a);
    return launch<8, false>(ctx, st, a);
}
