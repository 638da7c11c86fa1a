// BF16 weights (ggml type 30; crates/frink-quant/src/lib.rs:232-250: the upper half of an f32, widened exactly):
// gpt-oss keeps its attention projections in this format.  Nothing is quantized here -- the activations stay f32 and the
// products are accumulated in f32 -- so this matvec shares only the calling convention with the block formats.
// A warp per row, a lane on 8 weights (one 16-byte load) per trip, four trips in flight; the activations come through
// the read-only cache (every warp of an SM reads the same vector).  Batches of 1..8; optionally the RMSNorm of the
// input in the prologue, a bias row and add-into-y in the epilogue (a gpt-oss projection is one launch), and the
// standalone bias add for outputs of the GEMM path.
#include "fk_common.cuh"

namespace {

constexpr int BF_THREADS = 256, BF_WARPS = BF_THREADS / 32;

// NORM: the block first stages rmsnorm(x[b]) * norm_w for its batch rows in shared memory (every block repeats the few
// thousand multiply-adds).  The sum of squares is not added in the order of the separate norm launch: the fused form
// agrees with it to rounding, not to the bit, as in the block-format matvecs.
template <int NB, bool NORM>
__global__ void __launch_bounds__(BF_THREADS) gemv_bf16_kernel(const uint16_t* __restrict__ w, size_t row_elems, const float* __restrict__ x, int x_ld,
                                                               float* __restrict__ y, int rows, int cols, int batch,
                                                               const float* __restrict__ norm_w, float eps, const float* __restrict__ bias,
                                                               int accumulate) {
    extern __shared__ __align__(16) float xs[];              // NORM: [NB][cols]
    __shared__ float red[BF_WARPS];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (NORM) {
        for (int b = 0; b < NB && b < batch; b++) {
            float ss = 0.0f;
            for (int c = threadIdx.x; c < cols; c += BF_THREADS) {
                const float v = x[(size_t)b * x_ld + c];
                ss = fmaf(v, v, ss);
            }
            ss = fk_warp_sum(ss);
            if (lane == 0) red[warp] = ss;
            __syncthreads();
            float tot = 0.0f;
#pragma unroll
            for (int i = 0; i < BF_WARPS; i++) tot += red[i];
            const float scale = rsqrtf(tot / (float)cols + eps);
            for (int c = threadIdx.x; c < cols; c += BF_THREADS) xs[(size_t)b * cols + c] = x[(size_t)b * x_ld + c] * scale * norm_w[c];
            __syncthreads();
        }
    }
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
                    float4 x0, x1;
                    if (NORM) {
                        x0 = ((const float4*)(xs + (size_t)b * cols))[2 * c];
                        x1 = ((const float4*)(xs + (size_t)b * cols))[2 * c + 1];
                    } else {
                        x0 = __ldg((const float4*)(x + (size_t)b * x_ld) + 2 * c);
                        x1 = __ldg((const float4*)(x + (size_t)b * x_ld) + 2 * c + 1);
                    }
                    acc[b] = fmaf(f[0], x0.x, fmaf(f[1], x0.y, fmaf(f[2], x0.z, fmaf(f[3], x0.w, acc[b]))));
                    acc[b] = fmaf(f[4], x1.x, fmaf(f[5], x1.y, fmaf(f[6], x1.z, fmaf(f[7], x1.w, acc[b]))));
                }
            }
        }
#pragma unroll
        for (int b = 0; b < NB; b++) {
            float v = fk_warp_sum(acc[b]);                   // xor butterfly: the same order on every run
            if (lane == 0 && b < batch) {
                if (bias) v += bias[row];
                float* dst = y + (size_t)b * rows + row;
                *dst = accumulate ? *dst + v : v;
            }
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

template <int NB>
static int launch_bf16(fk_ctx* ctx, cudaStream_t st, int blocks, const uint16_t* wp, size_t row_elems, const float* x, int x_ld, float* y, int rows,
                       int cols, int batch, const float* norm_w, float eps, const float* bias, int accumulate) {
    if (norm_w) {
        const size_t smem = (size_t)NB * cols * sizeof(float);
        if (smem > 200 * 1024) return fk_fail(FK_UNSUPPORTED, "gemv (BF16): a fused norm over %d rows of %d columns does not fit shared memory", NB, cols);
        if (smem > 48 * 1024) FK_CUDA(cudaFuncSetAttribute(gemv_bf16_kernel<NB, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), FK_LAUNCH);
        gemv_bf16_kernel<NB, true><<<blocks, BF_THREADS, smem, st>>>(wp, row_elems, x, x_ld, y, rows, cols, batch, norm_w, eps, bias, accumulate);
    } else {
        gemv_bf16_kernel<NB, false><<<blocks, BF_THREADS, 0, st>>>(wp, row_elems, x, x_ld, y, rows, cols, batch, nullptr, 0.0f, bias, accumulate);
    }
    FK_CUDA(cudaGetLastError(), FK_LAUNCH);
    ctx->launches++;
    return FK_OK;
}

int fk_gemv_bf16_launch(fk_ctx* ctx, cudaStream_t st, fk_weight w, int mat, const float* x_dev, int x_ld, int batch, float* y_dev,
                        const float* norm_w, float norm_eps, const float* bias, int accumulate) {
    if (w->cols & 7) return fk_fail(FK_UNSUPPORTED, "gemv (BF16): %d columns is not a multiple of 8", w->cols);
    const uint16_t* wp = (const uint16_t*)(w->dev + (size_t)mat * w->mat_stride + w->plane_off[0]);
    const size_t row_elems = w->plane_stride[0] / 2;
    int blocks = ctx->sm_count * 8;
    const int need = (w->rows + BF_WARPS - 1) / BF_WARPS;
    if (blocks > need) blocks = need;
    if (x_ld == 0) x_ld = w->cols;
    if (batch <= 1) return launch_bf16<1>(ctx, st, blocks, wp, row_elems, x_dev, x_ld, y_dev, w->rows, w->cols, batch, norm_w, norm_eps, bias, accumulate);
    if (batch <= 2) return launch_bf16<2>(ctx, st, blocks, wp, row_elems, x_dev, x_ld, y_dev, w->rows, w->cols, batch, norm_w, norm_eps, bias, accumulate);
    if (batch <= 4) return launch_bf16<4>(ctx, st, blocks, wp, row_elems, x_dev, x_ld, y_dev, w->rows, w->cols, batch, norm_w, norm_eps, bias, accumulate);
    return launch_bf16<8>(ctx, st, blocks, wp, row_elems, x_dev, x_ld, y_dev, w->rows, w->cols, batch, norm_w, norm_eps, bias, accumulate);
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
