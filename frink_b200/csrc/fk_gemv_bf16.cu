// BF16 weights (ggml type 30; crates/frink-quant/src/lib.rs:232-250: the upper half of an f32, widened exactly):
// gpt-oss keeps its attention projections in this format.  Nothing is quantized here -- the activations stay f32 and the
// products are accumulated in f32 -- so this matvec shares only the calling convention with the block formats.
// A warp per row, a lane on 8 weights (one 16-byte load) per trip, four trips in flight; the activations come through
// the read-only cache (every warp of an SM reads the same vector).  Plain matvec for batches of 1..8, and the
// elementwise pieces a gpt-oss layer adds around its projections (bias rows).
#include "fk_common.cuh"

namespace {

constexpr int BF_THREADS = 256, BF_WARPS = BF_THREADS / 32;

template <int NB>
__global__ void __launch_bounds__(BF_THREADS) gemv_bf16_kernel(const uint16_t* __restrict__ w, size_t row_elems, const float* __restrict__ x,
                                                               float* __restrict__ y, int rows, int cols, int batch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int wid = blockIdx.x * BF_WARPS + warp, nw = gridDim.x * BF_WARPS;
    const int c8 = cols >> 3;                               // 16-byte chunks of a row
    for (int row = wid; row < rows; row += nw) {
        const uint4* rp = (const uint4*)(w + (size_t)row * row_elems);
        float acc[NB];
#pragma unroll
        for (int b = 0; b < NB; b++) acc[b] = 0.0f;
        for (int c0 = 0; c0 < c8; c0 += 4 * 32) {
            uint4 wv[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int c = c0 + u * 32 + lane;
                wv[u] = c < c8 ? __ldg(rp + c) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int c = c0 + u * 32 + lane;
                if (c >= c8) continue;
                const uint32_t ww[4] = {wv[u].x, wv[u].y, wv[u].z, wv[u].w};
                float f[8];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    f[2 * i] = __uint_as_float(ww[i] << 16);              // element 2 i: the low half of the word
                    f[2 * i + 1] = __uint_as_float(ww[i] & 0xFFFF0000u);
                }
#pragma unroll
                for (int b = 0; b < NB; b++) {
                    if (b >= batch) break;
                    const float4 x0 = __ldg((const float4*)(x + (size_t)b * cols) + 2 * c), x1 = __ldg((const float4*)(x + (size_t)b * cols) + 2 * c + 1);
                    acc[b] = fmaf(f[0], x0.x, fmaf(f[1], x0.y, fmaf(f[2], x0.z, fmaf(f[3], x0.w, acc[b]))));
                    acc[b] = fmaf(f[4], x1.x, fmaf(f[5], x1.y, fmaf(f[6], x1.z, fmaf(f[7], x1.w, acc[b]))));
                }
            }
        }
#pragma unroll
        for (int b = 0; b < NB; b++) {
            const float v = fk_warp_sum(acc[b]);             // xor butterfly: the same order on every run
            if (lane == 0 && b < batch) y[(size_t)b * rows + row] = v;
        }
    }
}

// y[r][c] += bias[c] (ids == nullptr) or bias[ids[r]][c]: a projection's bias row, or every expert slot's own
__global__ void add_bias_kernel(float* __restrict__ y, const float* __restrict__ bias, const int* __restrict__ ids, int n_rows, int cols) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)n_rows * cols) return;
    const int r = (int)(i / cols), c = (int)(i - (size_t)r * cols);
    y[i] += bias[(ids ? (size_t)ids[r] * cols : 0) + c];
}

}  // namespace

int fk_gemv_bf16_launch(fk_ctx* ctx, cudaStream_t st, fk_weight w, int mat, const float* x_dev, int batch, float* y_dev) {
    if (w->cols & 7) return fk_fail(FK_UNSUPPORTED, "gemv (BF16): %d columns is not a multiple of 8", w->cols);
    const uint16_t* wp = (const uint16_t*)(w->dev + (size_t)mat * w->mat_stride + w->plane_off[0]);
    const size_t row_elems = w->plane_stride[0] / 2;
    int blocks = ctx->sm_count * 8;
    const int need = (w->rows + BF_WARPS - 1) / BF_WARPS;
    if (blocks > need) blocks = need;
    if (batch <= 1) gemv_bf16_kernel<1><<<blocks, BF_THREADS, 0, st>>>(wp, row_elems, x_dev, y_dev, w->rows, w->cols, batch);
    else if (batch <= 2) gemv_bf16_kernel<2><<<blocks, BF_THREADS, 0, st>>>(wp, row_elems, x_dev, y_dev, w->rows, w->cols, batch);
    else if (batch <= 4) gemv_bf16_kernel<4><<<blocks, BF_THREADS, 0, st>>>(wp, row_elems, x_dev, y_dev, w->rows, w->cols, batch);
    else gemv_bf16_kernel<8><<<blocks, BF_THREADS, 0, st>>>(wp, row_elems, x_dev, y_dev, w->rows, w->cols, batch);
    FK_CUDA(cudaGetLastError(), FK_LAUNCH);
    ctx->launches++;
    return FK_OK;
}

// gpt-oss adds a bias to q, k, v and the attention output, to the router logits and to every expert projection
// (crates/frink-models/src/models/gpt_oss.rs:9-12,46; crates/frink-moe/src/lib.rs:1039-1060 `run_expert_oai`).
// y [n_rows][cols] += bias [cols], or with ids_dev [n_rows] (expert of every slot) += bias [n_bias][cols] row ids[r].
FK_EXPORT int fk_add_bias(fk_ctx* ctx, void* stream, float* y_dev, const float* bias_dev, const int* ids_dev, int n_rows, int cols) {
    if (!ctx || !y_dev || !bias_dev || n_rows < 1 || cols < 1) return fk_fail(FK_INVALID, "add_bias: bad argument");
    FkDeviceGuard g(ctx->device);
    const size_t n = (size_t)n_rows * cols;
    add_bias_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(y_dev, bias_dev, ids_dev, n_rows, cols);
    FK_CUDA(cudaGetLastError(), FK_LAUNCH);
    ctx->launches++;
    return FK_OK;
}
