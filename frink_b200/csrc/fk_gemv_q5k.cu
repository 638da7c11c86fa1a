// Q5_K decode matvec (crates/frink-quant/src/lib.rs:424-515, 873-939; block: f16 d, f16 dmin, 12 bytes of
// 6-bit scales and mins as Q4_K's, 32 bytes qh, 128 bytes of nibbles = 176 bytes per 256 weights).
// Real Q4_K_M files carry this format in some tensors; it gets the plain matvec (batch 1..8) with the same
// q8_1 activation rule and the same exact per-run integers as the other kinds, not the tuned rings of the
// Q4_K path: a warp walks the super-blocks of one row at a time, its 32 lanes on the 32 four-byte words of a
// super-block's nibbles, weights read straight from global memory (coalesced 128-byte lines, every byte once),
// the quantized activations from shared memory.  HBM-bound on large matrices, latency-bound on small ones.
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
    // ---- activations -> q8_1 (one warp per run of 32, the rule of fk_q8_1_lane)
    for (int run = warp; run < NB * nb32; run += Q5_WARPS) {
        const int b = run / nb32, kb = run - b * nb32;
        float v = 0.0f;
        if (b < a.batch) v = a.x[(size_t)b * cols + kb * 32 + lane];
        float d_w;
        int qsum;
        const int q = fk_q8_1_lane(v, &d_w, &qsum);
        sq[(size_t)b * cols + kb * 32 + lane] = (int8_t)q;
        if (lane == 0) {
            sd[b * nb32 + kb] = d_w;
            ss[b * nb32 + kb] = d_w * (float)qsum;
        }
    }
    __syncthreads();
    // ---- rows round the warps of the grid; lane = (64-element group g, word li of its 8)
    const int g = lane >> 3, li = lane & 7;
    const int wid = blockIdx.x * Q5_WARPS + warp, nw = gridDim.x * Q5_WARPS;
    for (int row = wid; row < a.rows; row += nw) {
        const uint8_t* rp = a.w + (size_t)row * a.row_bytes;
        float acc[NB];
#pragma unroll
        for (int b = 0; b < NB; b++) acc[b] = 0.0f;
#pragma unroll 2
        for (int sb = 0; sb < nsb; sb++) {
            const uint8_t* blk = rp + (size_t)sb * 176;
            const uint4 hd = __ldg((const uint4*)blk);                       // d, dmin, scales: the same for all lanes
            const uint32_t qh = __ldg((const uint32_t*)(blk + 16) + li);
            const uint32_t ql = __ldg((const uint32_t*)(blk + 48) + 8 * g + li);
            // codes of elements 64 g + 4 li .. + 3 (low nibbles, bit 2 g of qh) and 64 g + 32 + 4 li .. (high, bit 2 g + 1)
            const uint32_t lo = (ql & 0x0F0F0F0Fu) | (((qh >> (2 * g)) & 0x01010101u) << 4);
            const uint32_t hi = ((ql >> 4) & 0x0F0F0F0Fu) | (((qh >> (2 * g + 1)) & 0x01010101u) << 4);
            // 6-bit scales and mins of sub-blocks 2 g and 2 g + 1, one per byte: [0..3] and [4..7]
            const uint32_t scw = g < 2 ? (hd.y & 0x3F3F3F3Fu) : ((hd.w & 0x0F0F0F0Fu) | ((hd.y >> 2) & 0x30303030u));
            const uint32_t mnw = g < 2 ? (hd.z & 0x3F3F3F3Fu) : (((hd.w >> 4) & 0x0F0F0F0Fu) | ((hd.z >> 2) & 0x30303030u));
            const int sh = 16 * (g & 1);
            const float sc0 = (float)((scw >> sh) & 0xFFu), sc1 = (float)((scw >> (sh + 8)) & 0xFFu);
            const float m0 = (float)((mnw >> sh) & 0xFFu), m1 = (float)((mnw >> (sh + 8)) & 0xFFu);
            const float d = fk_h2f((uint16_t)(hd.x & 0xFFFF)), dmin = fk_h2f((uint16_t)(hd.x >> 16));
            const int kb0 = sb * 8 + 2 * g;
#pragma unroll
            for (int b = 0; b < NB; b++) {
                const int8_t* q8 = sq + (size_t)b * cols + sb * 256 + 64 * g + 4 * li;
                const int il = dp4a_ss((int)lo, *(const int*)q8, 0), ih = dp4a_ss((int)hi, *(const int*)(q8 + 32), 0);
                float t = d * (sc0 * sd[b * nb32 + kb0] * (float)il + sc1 * sd[b * nb32 + kb0 + 1] * (float)ih);
                if (li == 0) t -= dmin * (m0 * ss[b * nb32 + kb0] + m1 * ss[b * nb32 + kb0 + 1]);   // the mins, once per sub-block
                acc[b] += t;
                if (DUMP && b == 0) {
                    int sl = il, sh_ = ih;
                    sl += __shfl_xor_sync(0xffffffffu, sl, 1); sh_ += __shfl_xor_sync(0xffffffffu, sh_, 1);
                    sl += __shfl_xor_sync(0xffffffffu, sl, 2); sh_ += __shfl_xor_sync(0xffffffffu, sh_, 2);
                    sl += __shfl_xor_sync(0xffffffffu, sl, 4); sh_ += __shfl_xor_sync(0xffffffffu, sh_, 4);
                    if (li == 0) {
                        a.isums[(size_t)row * nb32 + kb0] = sl;
                        a.isums[(size_t)row * nb32 + kb0 + 1] = sh_;
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
