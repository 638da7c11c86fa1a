// BF16 weights (ggml type 30; crates/frink-quant/src/lib.rs:232-250: the upper half of an f32, widened exactly):
// gpt-oss keeps its attention projections in this format.  Nothing is quantized here -- the activations stay f32 and the
// products are accumulated in f32 -- so this matvec shares only the calling convention with the block formats.
// One or two warps per row, a lane on 8 weights (one 16-byte load) at a time with up to eight such loads in flight; the
// activations come through the read-only cache (every warp of an SM reads the same vector).  Batches of 1..8; optionally the RMSNorm of the
// input in the prologue, a bias row and add-into-y in the epilogue (a gpt-oss projection is one launch), and the
// standalone bias add for outputs of the GEMM path.
#include "fk_common.cuh"

namespace {

constexpr int BF_THREADS = 256, BF_WARPS = BF_THREADS / 32;

// NORM: the block first stages rmsnorm(x[b]) * norm_w for its batch rows in shared memory (every block repeats the few
// thousand multiply-adds).  The sum of squares is not added in the order of the separate norm launch: the fused form
// agrees with it to rounding, not to the bit, as in the block-format matvecs.
// S warps share a row (each on its own run of K, the partial sums added in warp order by the first of them), so that a
// matrix of a few thousand rows still has every SM's load queues full; U 16-byte loads a lane has in flight.
// The grid may start while the previous kernel of the stream still runs (programmatic stream serialization): weights
// are constants, so a warp requests its first trip of them BEFORE it waits for that kernel, and touches x, the bias and
// y only after.
template <int NB, bool NORM, int S, int U>
__global__ void __launch_bounds__(BF_THREADS) gemv_bf16_kernel(const uint16_t* __restrict__ w, size_t row_elems, const float* __restrict__ x, int x_ld,
                                                               float* __restrict__ y, int rows, int cols, int batch,
                                                               const float* __restrict__ norm_w, float eps, const float* __restrict__ bias,
                                                               int accumulate) {
    extern __shared__ __align__(16) float xs[];              // NORM: [NB][cols]
    __shared__ float red[BF_WARPS];
    __shared__ float part[BF_WARPS][NB];
    constexpr int RPB = BF_WARPS / S;                        // rows a block works on at a time
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rin = warp / S, prt = warp % S;
    const int c8 = cols >> 3;                                // 16-byte chunks of a row
    const int cpp = S == 1 ? c8 : ((((c8 + S - 1) / S) + 31) & ~31);   // chunks of a row one of its S warps takes
    const int cb = prt * cpp, ce = cb + cpp < c8 ? cb + cpp : c8;
    uint4 wv[U];
    auto request = [&](int row, int c0) {
        // every load unconditional, on a clamped address (what lies past the row's end is not used): they go out together
        const uint4* rp = (const uint4*)(w + (size_t)(row < rows ? row : rows - 1) * row_elems);
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int c = c0 + u * 32 + lane;
            wv[u] = __ldg(rp + (c < ce ? c : 0));
        }
    };
    int rbase = blockIdx.x * RPB;
    request(rbase + rin, cb);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (NORM) {
        constexpr int XP = 16;                               // values of a row a thread holds (rows of up to 4096 columns)
        const bool held = cols <= BF_THREADS * XP;
#pragma unroll 1
        for (int b = 0; b < NB && b < batch; b++) {          // (not unrolled: one row's values in registers at a time)
            float ss = 0.0f;
            float xv[XP], nv[XP];
            if (held) {
                // the row and the norm weight are read once, every load on a clamped index so that they all go out together
#pragma unroll
                for (int u = 0; u < XP; u++) {
                    const int c = threadIdx.x + u * BF_THREADS, cc = c < cols ? c : 0;
                    xv[u] = x[(size_t)b * x_ld + cc];
                    nv[u] = __ldg(norm_w + cc);
                }
#pragma unroll
                for (int u = 0; u < XP; u++)
                    if ((int)threadIdx.x + u * BF_THREADS < cols) ss = fmaf(xv[u], xv[u], ss);
            } else {
                for (int c = threadIdx.x; c < cols; c += BF_THREADS) {
                    const float v = x[(size_t)b * x_ld + c];
                    ss = fmaf(v, v, ss);
                }
            }
            ss = fk_warp_sum(ss);
            if (lane == 0) red[warp] = ss;
            __syncthreads();
            float tot = 0.0f;
#pragma unroll
            for (int i = 0; i < BF_WARPS; i++) tot += red[i];
            const float scale = rsqrtf(tot / (float)cols + eps);
            if (held) {
#pragma unroll
                for (int u = 0; u < XP; u++) {
                    const int c = threadIdx.x + u * BF_THREADS;
                    if (c < cols) xs[(size_t)b * cols + c] = xv[u] * scale * nv[u];
                }
            } else {
                for (int c = threadIdx.x; c < cols; c += BF_THREADS) xs[(size_t)b * cols + c] = x[(size_t)b * x_ld + c] * scale * norm_w[c];
            }
            __syncthreads();
        }
    }
    bool requested = true;                                   // the first trip of the first row is already on its way
    for (; rbase < rows; rbase += gridDim.x * RPB) {         // (the same trip count for every warp of the block: it meets at a barrier)
        const int row = rbase + rin;
        float acc[NB];
#pragma unroll
        for (int b = 0; b < NB; b++) acc[b] = 0.0f;
        for (int c0 = cb; c0 < ce; c0 += U * 32) {
            if (!requested) request(row, c0);
            requested = false;
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int c = c0 + u * 32 + lane;
                if (c >= ce) continue;
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
        requested = false;
#pragma unroll
        for (int b = 0; b < NB; b++) acc[b] = fk_warp_sum(acc[b]);   // xor butterfly: the same order on every run
        if (S > 1) {
            if (lane == 0)
#pragma unroll
                for (int b = 0; b < NB; b++) part[warp][b] = acc[b];
            __syncthreads();
            if (prt == 0)
#pragma unroll
                for (int b = 0; b < NB; b++) {
                    float v = part[warp][b];
#pragma unroll
                    for (int s2 = 1; s2 < S; s2++) v += part[warp + s2][b];
                    acc[b] = v;
                }
            __syncthreads();
        }
        if (prt == 0 && lane == 0 && row < rows) {
#pragma unroll
            for (int b = 0; b < NB; b++) {
                if (b >= batch) break;
                float v = acc[b];
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

template <int NB, int S, int U>
static int launch_bf16(fk_ctx* ctx, cudaStream_t st, const uint16_t* wp, size_t row_elems, const float* x, int x_ld, float* y, int rows,
                       int cols, int batch, const float* norm_w, float eps, const float* bias, int accumulate) {
    constexpr int RPB = BF_WARPS / S;
    const size_t norm_smem = norm_w ? (size_t)NB * cols * sizeof(float) : 0;
    if (norm_smem > 200 * 1024) return fk_fail(FK_UNSUPPORTED, "gemv (BF16): a fused norm over %d rows of %d columns does not fit shared memory", NB, cols);
    // one wave: as many blocks as are resident at once (the rows are dealt out in a grid-stride loop)
    int per_sm = 0;
    if (norm_w) {
        if (norm_smem > 48 * 1024) FK_CUDA(cudaFuncSetAttribute(gemv_bf16_kernel<NB, true, S, U>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)norm_smem), FK_LAUNCH);
        FK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemv_bf16_kernel<NB, true, S, U>, BF_THREADS, norm_smem), FK_LAUNCH);
    } else {
        FK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemv_bf16_kernel<NB, false, S, U>, BF_THREADS, 0), FK_LAUNCH);
    }
    if (per_sm < 1) per_sm = 1;
    int blocks = ctx->sm_count * per_sm;
    const int need = (rows + RPB - 1) / RPB;
    if (blocks > need) blocks = need;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(BF_THREADS);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (norm_w) {
        auto kern = gemv_bf16_kernel<NB, true, S, U>;
        cfg.dynamicSmemBytes = norm_smem;
        FK_CUDA(cudaLaunchKernelEx(&cfg, kern, wp, row_elems, x, x_ld, y, rows, cols, batch, norm_w, eps, bias, accumulate), FK_LAUNCH);
    } else {
        auto kern = gemv_bf16_kernel<NB, false, S, U>;
        FK_CUDA(cudaLaunchKernelEx(&cfg, kern, wp, row_elems, x, x_ld, y, rows, cols, batch, (const float*)nullptr, 0.0f, bias, accumulate), FK_LAUNCH);
    }
    ctx->launches++;
    return FK_OK;
}

int fk_gemv_bf16_launch(fk_ctx* ctx, cudaStream_t st, fk_weight w, int mat, const float* x_dev, int x_ld, int batch, float* y_dev,
                        const float* norm_w, float norm_eps, const float* bias, int accumulate) {
    if (w->cols & 7) return fk_fail(FK_UNSUPPORTED, "gemv (BF16): %d columns is not a multiple of 8", w->cols);
    const uint16_t* wp = (const uint16_t*)(w->dev + (size_t)mat * w->mat_stride + w->plane_off[0]);
    const size_t row_elems = w->plane_stride[0] / 2;
    if (x_ld == 0) x_ld = w->cols;
    // a matrix with fewer rows than the device holds warps: two warps a row, so that every SM has loads in flight
    const bool split = w->rows < ctx->sm_count * 48 && w->cols >= 1024;
#define FK_BF16_GO(NB_, S_, U_) \
    return launch_bf16<NB_, S_, U_>(ctx, st, wp, row_elems, x_dev, x_ld, y_dev, w->rows, w->cols, batch, norm_w, norm_eps, bias, accumulate)
    if (batch <= 1) { if (split) FK_BF16_GO(1, 2, 8); FK_BF16_GO(1, 1, 8); }
    if (batch <= 2) { if (split) FK_BF16_GO(2, 2, 8); FK_BF16_GO(2, 1, 8); }
    if (batch <= 4) { if (split) FK_BF16_GO(4, 2, 4); FK_BF16_GO(4, 1, 4); }
    if (split) FK_BF16_GO(8, 2, 4);
    FK_BF16_GO(8, 1, 4);
#undef FK_BF16_GO
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
