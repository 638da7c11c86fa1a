// MoE plumbing around the expert matmuls: router logits, top-k routing, the
// token permutation that makes each expert's rows contiguous, the gated
// activation between the two expert matmuls, and the weighted combine.
#include "fk_common.cuh"

namespace {

constexpr int TOPK_PER_LANE = 8;  // n_experts <= 256
constexpr int TOPK_MAX_K = 16;

// One warp per token.  Selection is by (biased) logit, ties to the lower
// expert id; weights by `mode` (0 softmax over all, 1 renormalised over the
// chosen, 2 softmax over the chosen only), written in selection order.
// The whole warp calls this for token t; the logits are read with L2-coherent loads because
// the fused kernel below reads what other blocks of the same launch have just written.
__device__ __forceinline__ void route_token(const float* logits, const float* bias, int n_experts, int k, int mode, int t, int lane,
                                            int* ids_out, float* w_out) {
    const float NEG_INF = __int_as_float(0xff800000);
    const float* lg = logits + (size_t)t * n_experts;
    float v[TOPK_PER_LANE];
#pragma unroll
    for (int j = 0; j < TOPK_PER_LANE; j++) {
        const int e = lane + 32 * j;
        v[j] = e < n_experts ? __ldcg(lg + e) + (bias ? bias[e] : 0.0f) : NEG_INF;
    }
    float mx = NEG_INF;
#pragma unroll
    for (int j = 0; j < TOPK_PER_LANE; j++) mx = fmaxf(mx, v[j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < TOPK_PER_LANE; j++)
        if (lane + 32 * j < n_experts) sum += expf(v[j] - mx);
    sum = fk_warp_sum(sum);

    float cv[TOPK_MAX_K];
    int ci[TOPK_MAX_K];
#pragma unroll 1
    for (int s = 0; s < k; s++) {
        float bv = NEG_INF;
        int bi = 0x7fffffff;
#pragma unroll
        for (int j = 0; j < TOPK_PER_LANE; j++) {
            const int e = lane + 32 * j;
            if (e < n_experts && (v[j] > bv || (v[j] == bv && e < bi))) { bv = v[j]; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        cv[s] = bv;
        ci[s] = bi;
#pragma unroll
        for (int j = 0; j < TOPK_PER_LANE; j++)
            if (lane + 32 * j == bi) v[j] = NEG_INF;
    }
    if (lane != 0) return;
    int* ids = ids_out + (size_t)t * k;
    float* w = w_out + (size_t)t * k;
    if (mode == 2) {
        float es = 0.0f;
        for (int s = 0; s < k; s++) es += expf(cv[s] - cv[0]);
        for (int s = 0; s < k; s++) {
            const float e = expf(cv[s] - cv[0]);
            w[s] = es > 0.0f ? e / es : e;
            ids[s] = ci[s];
        }
        return;
    }
    float ts = 0.0f;
    for (int s = 0; s < k; s++) {
        const float p = expf(cv[s] - mx) / sum;
        w[s] = p;
        ts += p;
        ids[s] = ci[s];
    }
    if (mode == 1)
        for (int s = 0; s < k; s++) w[s] = w[s] / ts;
}

__global__ void route_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int n_experts, int k,
                             int mode, int batch, int* __restrict__ ids_out, float* __restrict__ w_out) {
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= batch) return;
    route_token(logits, bias, n_experts, k, mode, t, threadIdx.x & 31, ids_out, w_out);
}

// logits[t][e] = router[e] . x[t], one warp per (e, t); f32 throughout.
__global__ void router_logits_kernel(const float* __restrict__ w, const float* __restrict__ x, float* __restrict__ out,
                                     int rows, int cols) {
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float* wr = w + (size_t)row * cols;
    const float* xt = x + (size_t)blockIdx.y * cols;
    float acc = 0.0f;
    for (int i = lane; i < cols; i += 32) acc += wr[i] * xt[i];
    acc = fk_warp_sum(acc);
    if (lane == 0) out[(size_t)blockIdx.y * rows + row] = acc;
}

// router_logits_kernel and route_kernel in one launch: the block that arrives last (a counter
// of the context, rewound by that block) routes every token, a warp per token.
__global__ void router_route_kernel(const float* __restrict__ w, const float* __restrict__ x, float* __restrict__ logits, int rows, int cols,
                                    const float* __restrict__ bias, int k, int mode, int batch, int* __restrict__ ids_out,
                                    float* __restrict__ w_out, unsigned* __restrict__ cnt, const float* __restrict__ norm_w, float norm_eps) {
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    // The sum of a lane runs over i = lane, lane + 32, ... in that order (the order the separate logits kernel uses), so
    // a warp walks its row alone; what can be parallel is the memory: the router's weights are constants, and a lane
    // requests its whole share of the row (up to RU steps, 3072 columns) BEFORE the wait for the kernel that writes x --
    // this grid may start while that kernel still runs -- on clamped indices, so that every load is unconditional and
    // they all go out together.  x (normalized, if asked) is staged once a block in shared memory.
    constexpr int RU = 96;
    extern __shared__ __align__(16) float xs[];                  // [cols]
    const float* wr = w + (size_t)(row < rows ? row : 0) * cols;
    const float* xt = x + (size_t)blockIdx.y * cols;
    float wa[RU];
#pragma unroll
    for (int u = 0; u < RU; u++) {
        const int i = lane + 32 * u;
        wa[u] = __ldg(wr + (i < cols ? i : 0));
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // norm_w: x is the residual stream and the router reads rmsnorm(x) * norm_w -- the values the separate norm launch
    // writes (squares in f32, summed in f64, the mean rounded to f32; element = x * scale * weight), formed on the fly
    float scale = 1.0f;
    if (norm_w) {
        __shared__ double sq_part[32];
        double sq = 0.0;
        for (int i0 = threadIdx.x; i0 < cols; i0 += 8 * blockDim.x) {     // eight loads in flight a thread
            float xv[8];
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const int i = i0 + u * blockDim.x;
                xv[u] = xt[i < cols ? i : 0];
            }
#pragma unroll
            for (int u = 0; u < 8; u++)
                if (i0 + u * (int)blockDim.x < cols) sq += (double)(xv[u] * xv[u]);
        }
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        if (lane == 0) sq_part[threadIdx.x >> 5] = sq;
        __syncthreads();
        double t = 0.0;
        for (int i = 0; i < (int)(blockDim.x >> 5); i++) t += sq_part[i];
        scale = 1.0f / sqrtf((float)(t / (double)cols) + norm_eps);
    }
    for (int i0 = threadIdx.x; i0 < cols; i0 += 8 * blockDim.x) {
        float xv[8], nv[8];
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const int i = i0 + u * blockDim.x, ic = i < cols ? i : 0;
            xv[u] = xt[ic];
            nv[u] = norm_w ? __ldg(norm_w + ic) : 1.0f;
        }
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const int i = i0 + u * blockDim.x;
            if (i < cols) xs[i] = norm_w ? xv[u] * scale * nv[u] : xv[u];
        }
    }
    __syncthreads();
    if (row < rows) {
        float acc = 0.0f;
        for (int i0 = lane; i0 < cols; i0 += 32 * RU) {
            if (i0 != lane) {
#pragma unroll
                for (int u = 0; u < RU; u++) {
                    const int i = i0 + 32 * u;
                    wa[u] = __ldg(wr + (i < cols ? i : 0));
                }
            }
#pragma unroll
            for (int u = 0; u < RU; u++) {
                const int i = i0 + 32 * u;
                if (i < cols) acc += wa[u] * xs[i];
            }
        }
        acc = fk_warp_sum(acc);
        if (lane == 0) logits[(size_t)blockIdx.y * rows + row] = acc;
    }
    __shared__ bool last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) last = atomicAdd(cnt, 1u) == gridDim.x * gridDim.y - 1;
    __syncthreads();
    if (!last) return;
    __threadfence();
    for (int t = threadIdx.x >> 5; t < batch; t += blockDim.x >> 5) route_token(logits, bias, rows, k, mode, t, lane, ids_out, w_out);
    if (threadIdx.x == 0) *cnt = 0;
}

// Stable counting sort of the (token, slot) pairs by expert, in one block: counts by shared-memory
// atomics, offsets by one thread, then the pairs are placed in pair order (chunk by chunk, warp by warp,
// lane by lane), so pairs keep ascending order inside a group and the result is the same on every run.
__global__ void permute_kernel(const int* __restrict__ ids, int pairs, int k, int n_experts, int* __restrict__ group_off,
                               int* __restrict__ gather, int* __restrict__ pair_of) {
    extern __shared__ int counts[];  // [n_experts + 1]: counts, then each expert's next free place
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int e = threadIdx.x; e <= n_experts; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = ids[p];
        if (e >= 0 && e < n_experts) atomicAdd(&counts[e], 1);      // integer counts: the order of the additions does not matter
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int acc = 0;
        for (int e = 0; e < n_experts; e++) {
            const int c = counts[e];
            counts[e] = acc;
            group_off[e] = acc;
            acc += c;
        }
        counts[n_experts] = acc;
        group_off[n_experts] = acc;
    }
    __syncthreads();
    // Places, in pair order: a chunk of blockDim pairs at a time; inside a chunk the warps take turns (warp w holds pairs
    // before warp w + 1's), and inside a warp the lanes with the same expert are ranked by lane.
    for (int p0 = 0; p0 < pairs; p0 += blockDim.x) {
        const int p = p0 + threadIdx.x;
        int e = p < pairs ? ids[p] : -1;
        if (e >= n_experts) e = -1;
        const unsigned same = __match_any_sync(0xffffffffu, e);
        const int rank = __popc(same & ((1u << lane) - 1u)), leader = __ffs(same) - 1;
        int base = 0;
        for (int w = 0; w < nwarps; w++) {
            if (warp == w && e >= 0 && lane == leader) {
                base = counts[e];
                counts[e] = base + __popc(same);
            }
            __syncthreads();
        }
        base = __shfl_sync(0xffffffffu, base, leader);
        if (e >= 0) {
            gather[base + rank] = p / k;
            pair_of[p] = base + rank;
        }
    }
}

__global__ void glu_kernel(const float* __restrict__ gate, const float* __restrict__ up, size_t n, int act, float* __restrict__ out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float g = gate[i], u = up[i];
    if (act == 0) {
        out[i] = (g / (1.0f + expf(-g))) * u;
    } else {
        const float x = fminf(g, 7.0f);
        const float y = fminf(fmaxf(u, -7.0f), 7.0f);
        out[i] = (x / (1.0f + expf(1.702f * -x))) * (y + 1.0f);
    }
}

__global__ void combine_kernel(const float* __restrict__ y, const int* __restrict__ pair_of, const float* __restrict__ w,
                               int k, int n, float* __restrict__ out, int add) {
    // launched with programmatic stream serialization: wait for the kernel that wrote y, and let the next one (a
    // matvec that requests its weights before it waits in turn) be scheduled now
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const int t = blockIdx.y;
    if (i >= n) return;
    float acc = 0.0f;
    for (int j = 0; j < k; j++) {
        const int p = pair_of ? pair_of[t * k + j] : t * k + j;
        acc += y[(size_t)p * n + i] * w[t * k + j];
    }
    out[(size_t)t * n + i] = add ? out[(size_t)t * n + i] + acc : acc;   // the sum is formed from zero either way
}

// One warp: the chosen experts of one token that fall in [e0, e0 + n_local), packed
// to the front in routing order with their weights; the rest padded with expert 0 /
// weight 0.  *out_n = how many.
__global__ void local_slots_kernel(const int* __restrict__ ids, const float* __restrict__ w, int k, int e0, int n_local,
                                   int* __restrict__ out_ids, float* __restrict__ out_w, int* __restrict__ out_n) {
    const int lane = threadIdx.x;
    const int id = lane < k ? ids[lane] : -1;
    const bool mine = id >= e0 && id < e0 + n_local;
    const unsigned m = __ballot_sync(0xffffffffu, mine);
    const int n = __popc(m);
    if (lane < k) {
        out_ids[lane] = 0;
        out_w[lane] = 0.0f;
    }
    __syncwarp();
    if (mine) {
        const int p = __popc(m & ((1u << lane) - 1u));
        out_ids[p] = id - e0;
        out_w[p] = w[lane];
    }
    if (lane == 0) *out_n = n;
}

// Expert-parallel prefill with replicated activations: pair i keeps its expert as a local id when a rank owns it,
// else it joins the dummy group n_local with weight 0 (the grouped GEMM never reads that group).
__global__ void localize_kernel(const int* __restrict__ ids, const float* __restrict__ w, int n, int e0, int n_local,
                                int* __restrict__ ids_out, float* __restrict__ w_out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int id = ids[i];
    const bool mine = id >= e0 && id < e0 + n_local;
    ids_out[i] = mine ? id - e0 : n_local;
    w_out[i] = mine ? w[i] : 0.0f;
}

// A decode batch under expert parallelism: of the `pairs` (row, chosen expert) pairs of b rows (pair i belongs to row
// i / k), those whose expert lies in [e0, e0 + n_local) are packed to the front as slots, in pair order:
//   out_ids[p] local expert, out_src[p] row of the slot's activation (both 0 past the last slot),
//   out_pair_of[i] slot of pair i (0 for another rank's pair), out_w[i] its weight (0 for another rank's pair),
//   *out_n the number of slots.  One block; pairs <= 256.
__global__ void __launch_bounds__(256) local_pairs_kernel(const int* __restrict__ ids, const float* __restrict__ w, int pairs, int k, int e0,
                                                          int n_local, int* __restrict__ out_ids, int* __restrict__ out_src,
                                                          int* __restrict__ out_pair_of, float* __restrict__ out_w, int* __restrict__ out_n) {
    __shared__ int s_cnt[8];
    const int i = threadIdx.x, lane = i & 31, warp = i >> 5;
    const int id = i < pairs ? ids[i] : -1;
    const bool mine = id >= e0 && id < e0 + n_local;
    const unsigned m = __ballot_sync(0xffffffffu, mine);
    if (lane == 0) s_cnt[warp] = __popc(m);
    if (i < pairs) {
        out_ids[i] = 0;
        out_src[i] = 0;
    }
    __syncthreads();
    int before = 0, total = 0;
    for (int v = 0; v < 8; v++) {
        if (v < warp) before += s_cnt[v];
        total += s_cnt[v];
    }
    const int p = before + __popc(m & ((1u << lane) - 1u));
    if (mine) {
        out_ids[p] = id - e0;
        out_src[p] = i / k;
    }
    if (i < pairs) {
        out_pair_of[i] = mine ? p : 0;
        out_w[i] = mine ? w[i] : 0.0f;
    }
    if (i == 0) *out_n = total;
}

// y[r][c] += bias[expert of permuted row r][c]: the rows of a grouped GEMM's output are sorted by expert, group_off [E + 1]
// says where each expert's rows start, so a thread finds its row's expert by bisection
__global__ void add_bias_grouped_kernel(float* __restrict__ y, const float* __restrict__ bias, const int* __restrict__ group_off, int n_experts,
                                        int n_rows, int cols) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)n_rows * cols) return;
    const int r = (int)(i / cols), c = (int)(i - (size_t)r * cols);
    int lo = 0, hi = n_experts;                      // the expert e with group_off[e] <= r < group_off[e + 1]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (group_off[mid] <= r) lo = mid; else hi = mid;
    }
    y[i] += bias[(size_t)lo * cols + c];
}

// out[j] = x[j / k] for j < rows * k: every slot of a decode batch gets its row's activation.
__global__ void repeat_rows_kernel(const float* __restrict__ x, int cols4, int k, size_t n4, float* __restrict__ out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n4) return;
    const size_t slot = i / cols4, c = i - slot * cols4;
    ((float4*)out)[i] = ((const float4*)x)[(slot / k) * cols4 + c];
}

// Every kernel of a decode step asks for the same shared-memory carve-out as the GEMV
// (the maximum): an SM that alternates between kernels with different carve-outs
// re-partitions its L1 between them, which costs more than these kernels run.
template <typename K> void fk_carveout(K kern) {
    static thread_local const void* done[64];
    static thread_local int n = 0;
    for (int i = 0; i < n; i++) if (done[i] == (const void*)kern) return;
    cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (n < 64) done[n++] = (const void*)kern;
}
#define FK_CARVEOUT(k) fk_carveout(k)

}  // namespace

FK_EXPORT int fk_moe_local_slots(fk_ctx* ctx, void* stream, const int* ids_dev, const float* w_dev, int k, int e0, int n_local,
                                 int* out_ids_dev, float* out_w_dev, int* out_n_dev) {
    if (!ctx || !ids_dev || !w_dev || !out_ids_dev || !out_w_dev || !out_n_dev) return fk_fail(FK_INVALID, "moe_local_slots: null argument");
    if (k < 1 || k > 32) return fk_fail(FK_UNSUPPORTED, "moe_local_slots: k=%d (limit 32)", k);
    FkDeviceGuard g(ctx->device);
    FK_CARVEOUT(local_slots_kernel);
    local_slots_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(ids_dev, w_dev, k, e0, n_local, out_ids_dev, out_w_dev, out_n_dev);
    FK_CUDA(cudaGetLastError(), FK_LAUNCH);
    ctx->launches++;
    return FK_OK;
}

FK_EXPORT int fk_moe_local_pairs(fk_ctx* ctx, void* stream, const int* ids_dev, const float* w_dev, int pairs, int k, int e0, int n_local,
                                 int* out_ids_dev, int* out_src_dev, int* out_pair_of_dev, float* out_w_dev, int* out_n_dev) {
    if (!ctx || !ids_dev || !w_dev || !out_ids_dev || !out_src_dev || !out_pair_of_dev || !out_w_dev || !out_n_dev)
        return fk_fail(FK_INVALID, "moe_local_pairs: null argument");
    if (k < 1 || pairs < 1 || pairs > 256 || pairs % k) return fk_fail(FK_UNSUPPORTED, "moe_local_pairs: %d pairs of k=%d (limit 256)", pairs, k);
    FkDeviceGuard g(ctx->device);
    FK_CARVEOUT(local_pairs_kernel);
    local_pairs_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(ids_dev, w_dev, pairs, k, e0, n_local, out_ids_dev, out_src_dev, out_pair_of_dev, out_w_dev,
                                                            out_n_dev);
    FK_CUDA(cudaGetLastError(), FK_LAUNCH);
    ctx->launches++;
    return FK_OK;
}

FK_EXPORT int fk_moe_localize(fk_ctx* ctx, void* stream, const int* ids_dev, const float* w_dev, int pairs, int e0, int n_local,
                              int* out_ids_dev, float* out_w_dev) {
    if (!ctx || !ids_dev || !w_dev || !out_ids_dev || !out_w_dev) return fk_fail(FK_INVALID, "moe_localize: null argument");
    if (pairs < 1 || n_local < 1) return fk_fail(FK_INVALID, "moe_localize: pairs %d, local experts %d", pairs, n_local);
    FkDeviceGuard g(ctx->device);
    localize_kernel<<<(pairs + 255) / 256, 256, 0, (cudaStream_t)stream>>>(ids_dev, w_dev, pairs, e0, n_local, out_ids_dev, out_w_dev);
    FK_CUDA(cudaGetLastError(), FK_LAUNCH);
    ctx->launches++;
    return FK_OK;
}

FK_EXPORT int fk_moe_route(fk_ctx* ctx, void* stream, const float* logits_dev, const float* bias_dev, int n_experts,
                           int k, int mode, int batch, int* ids_dev, float* w_dev) {
    if (!ctx || !logits_dev || !ids_dev || !w_dev) return fk_fail(FK_INVALID, "moe_route: null argument");
    if (n_experts < 1 || n_experts > 32 * TOPK_PER_LANE) return fk_fail(FK_UNSUPPORTED, "moe_route: %d experts (limit %d)", n_experts, 32 * TOPK_PER_LANE);
    if (k < 1 || k > TOPK_MAX_K || k > n_experts) return fk_fail(FK_UNSUPPORTED, "moe_route: k=%d (limit %d, experts %d)", k, TOPK_MAX_K, n_experts);
    if (mode < 0 || mode > 2) return fk_fail(FK_INVALID, "moe_route: mode %d", mode);
    if (batch < 1) return fk_fail(FK_INVALID, "moe_route: batch %d", batch);
    FkDeviceGuard g(ctx->device);
    FK_CARVEOUT(route_kernel);
    route_kernel<<<(batch + 3) / 4, 128, 0, (cudaStream_t)stream>>>(logits_dev, bias_dev, n_experts, k, mode, batch, ids_dev, w_dev);
    FK_CUDA(cudaGetLastError(), FK_LAUNCH);
    ctx->launches++;
    return FK_OK;
}

FK_EXPORT int fk_router_logits(fk_ctx* ctx, void* stream, const float* router_dev, const float* x_dev, int n_experts,
                               int cols, int batch, float* logits_dev) {
    if (!ctx || !router_dev || !x_dev || !logits_dev) return fk_fail(FK_INVALID, "router_logits: null argument");
    if (n_experts < 1 || cols < 1 || batch < 1 || batch > 65535) return fk_fail(FK_INVALID, "router_logits: %d x %d, batch %d", n_experts, cols, batch);
    FkDeviceGuard g(ctx->device);
    dim3 grid((n_experts + 7) / 8, batch);
    FK_CARVEOUT(router_logits_kernel);
    router_logits_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(router_dev, x_dev, logits_dev, n_experts, cols);
    FK_CUDA(cudaGetLastError(), FK_LAUNCH);
    ctx->launches++;
    return FK_OK;
}

static int router_route_launch(fk_ctx* ctx, void* stream, const float* router_dev, const float* x_dev, int n_experts, int cols, int batch,
                               const float* bias_dev, int k, int mode, float* logits_dev, int* ids_dev, float* w_dev, const float* norm_w,
                               float norm_eps) {
    if (!ctx || !router_dev || !x_dev || !logits_dev || !ids_dev || !w_dev) return fk_fail(FK_INVALID, "router_route: null argument");
    if (n_experts < 1 || n_experts > 32 * TOPK_PER_LANE) return fk_fail(FK_UNSUPPORTED, "router_route: %d experts (limit %d)", n_experts, 32 * TOPK_PER_LANE);
    if (k < 1 || k > TOPK_MAX_K || k > n_experts) return fk_fail(FK_UNSUPPORTED, "router_route: k=%d (limit %d, experts %d)", k, TOPK_MAX_K, n_experts);
    if (mode < 0 || mode > 2 || batch < 1 || batch > 65535 || cols < 1) return fk_fail(FK_INVALID, "router_route: mode %d, batch %d, cols %d", mode, batch, cols);
    FkDeviceGuard g(ctx->device);
    dim3 grid((n_experts + 7) / 8, batch);
    FK_CARVEOUT(router_route_kernel);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(256);
    cfg.stream = (cudaStream_t)stream;
    cfg.dynamicSmemBytes = (size_t)cols * sizeof(float);             // x (normalized), staged once a block
    if (cfg.dynamicSmemBytes > 200 * 1024) return fk_fail(FK_UNSUPPORTED, "router_route: %d columns do not fit shared memory", cols);
    if (cfg.dynamicSmemBytes > 48 * 1024)
        FK_CUDA(cudaFuncSetAttribute(router_route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)cfg.dynamicSmemBytes), FK_LAUNCH);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    FK_CUDA(cudaLaunchKernelEx(&cfg, router_route_kernel, router_dev, x_dev, logits_dev, n_experts, cols, bias_dev, k, mode, batch, ids_dev, w_dev,
                               (unsigned*)(ctx->argmax_cnt + 64), norm_w, norm_eps), FK_LAUNCH);
    ctx->launches++;
    return FK_OK;
}

FK_EXPORT int fk_router_route(fk_ctx* ctx, void* stream, const float* router_dev, const float* x_dev, int n_experts, int cols, int batch,
                              const float* bias_dev, int k, int mode, float* logits_dev, int* ids_dev, float* w_dev) {
    return router_route_launch(ctx, stream, router_dev, x_dev, n_experts, cols, batch, bias_dev, k, mode, logits_dev, ids_dev, w_dev, nullptr, 0.0f);
}

FK_EXPORT int fk_moe_permute(fk_ctx* ctx, void* stream, const int* ids_dev, int pairs, int k, int n_experts,
                             int* group_off_dev, int* gather_dev, int* pair_of_dev) {
    if (!ctx || !ids_dev || !group_off_dev || !gather_dev || !pair_of_dev) return fk_fail(FK_INVALID, "moe_permute: null argument");
    if (pairs < 1 || k < 1 || n_experts < 1 || n_experts > 4096) return fk_fail(FK_INVALID, "moe_permute: pairs %d, k %d, experts %d", pairs, k, n_experts);
    FkDeviceGuard g(ctx->device);
    FK_CARVEOUT(permute_kernel);
    permute_kernel<<<1, 1024, (n_experts + 1) * sizeof(int), (cudaStream_t)stream>>>(ids_dev, pairs, k, n_experts, group_off_dev, gather_dev, pair_of_dev);
    FK_CUDA(cudaGetLastError(), FK_LAUNCH);
    ctx->launches++;
    return FK_OK;
}

FK_EXPORT int fk_glu(fk_ctx* ctx, void* stream, const float* gate_dev, const float* up_dev, size_t n, int act, float* out_dev) {
    if (!ctx || !gate_dev || !up_dev || !out_dev) return fk_fail(FK_INVALID, "glu: null argument");
    if (act < 0 || act > 1) return fk_fail(FK_UNSUPPORTED, "glu: activation %d", act);
    if (n == 0) return FK_OK;
    FkDeviceGuard g(ctx->device);
    FK_CARVEOUT(glu_kernel);
    glu_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(gate_dev, up_dev, n, act, out_dev);
    FK_CUDA(cudaGetLastError(), FK_LAUNCH);
    ctx->launches++;
    return FK_OK;
}

static cudaError_t launch_combine(dim3 grid, cudaStream_t st, const float* y, const int* pair_of, const float* w, int k, int n, float* out, int add) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, combine_kernel, y, pair_of, w, k, n, out, add);
}

FK_EXPORT int fk_moe_combine(fk_ctx* ctx, void* stream, const float* y_dev, const int* pair_of_dev, const float* w_dev,
                             int batch, int k, int n, float* out_dev) {
    if (!ctx || !y_dev || !w_dev || !out_dev) return fk_fail(FK_INVALID, "moe_combine: null argument");
    if (batch < 1 || batch > 65535 || k < 1 || n < 1) return fk_fail(FK_INVALID, "moe_combine: batch %d, k %d, n %d", batch, k, n);
    FkDeviceGuard g(ctx->device);
    dim3 grid((n + 255) / 256, batch);
    FK_CARVEOUT(combine_kernel);
    FK_CUDA(launch_combine(grid, (cudaStream_t)stream, y_dev, pair_of_dev, w_dev, k, n, out_dev, 0), FK_LAUNCH);
    ctx->launches++;
    return FK_OK;
}

FK_EXPORT int fk_moe_combine_add(fk_ctx* ctx, void* stream, const float* y_dev, const int* pair_of_dev, const float* w_dev,
                             int batch, int k, int n, float* out_dev) {
    if (!ctx || !y_dev || !w_dev || !out_dev) return fk_fail(FK_INVALID, "moe_combine_add: null argument");
    if (batch < 1 || batch > 65535 || k < 1 || n < 1) return fk_fail(FK_INVALID, "moe_combine_add: batch %d, k %d, n %d", batch, k, n);
    FkDeviceGuard g(ctx->device);
    dim3 grid((n + 255) / 256, batch);
    FK_CARVEOUT(combine_kernel);
    FK_CUDA(launch_combine(grid, (cudaStream_t)stream, y_dev, pair_of_dev, w_dev, k, n, out_dev, 1), FK_LAUNCH);
    ctx->launches++;
    return FK_OK;
}

// ---- the routed layer in one call --------------------------------------------------------------
namespace {
struct MoeWs {
    size_t logits, ids, w, group_off, gather, pair_of, xr, g, u, y, total;
};
MoeWs moe_ws(int n_experts, int k, int hidden, int ffn, int batch) {
    MoeWs m{};
    size_t off = 0;
    auto take = [&](size_t bytes) { const size_t at = off; off += (bytes + 255) & ~(size_t)255; return at; };
    const size_t pairs = (size_t)batch * k;
    m.logits = take((size_t)batch * n_experts * 4);
    m.ids = take(pairs * 4);
    m.w = take(pairs * 4);
    m.group_off = take(((size_t)n_experts + 1) * 4);
    m.gather = take(pairs * 4);
    m.pair_of = take(pairs * 4);
    m.xr = take(batch <= 8 && batch > 1 ? pairs * hidden * 4 : 0);
    m.g = take(2 * pairs * ffn * 4);                 // gate rows, then the up rows directly behind them (one launch may write both)
    m.u = m.g + pairs * ffn * 4;
    m.y = take(pairs * hidden * 4);
    m.total = off;
    return m;
}
}  // namespace

FK_EXPORT size_t fk_moe_layer_workspace(int n_experts, int k, int hidden, int ffn, int batch) {
    if (n_experts < 1 || k < 1 || hidden < 1 || ffn < 1 || batch < 1) return 0;
    return moe_ws(n_experts, k, hidden, ffn, batch).total;
}

// The resident routed layer (crates/frink-cuda/src/prefill/moe_device.rs:241-438) as one call: router, top-k, and
//   batch <= 8 : every (row, expert) pair a slot of one indexed matvec per projection, GLU in the down projection;
//   batch  > 8 : pairs grouped by expert, one grouped GEMM per projection;
// then the weighted combine in routing order, written to out_dev or added into it.
static int moe_layer_impl(fk_ctx* ctx, void* stream, const float* router_dev, const float* router_bias_dev, fk_weight gate, fk_weight up,
                          fk_weight down, const float* gate_b, const float* up_b, const float* down_b, int k, int mode, int act, const float* x_dev,
                          int batch, float* out_dev, int accumulate, void* workspace_dev, size_t workspace_bytes,
                          const float* norm_w = nullptr, float norm_eps = 0.0f) {
    if (!ctx || !router_dev || !gate || !up || !down || !x_dev || !out_dev || !workspace_dev) return fk_fail(FK_INVALID, "moe_layer: null argument");
    const int E = gate->n_mats, hidden = gate->cols, ffn = gate->rows;
    if (up->n_mats != E || down->n_mats != E || up->rows != ffn || up->cols != hidden || down->rows != hidden || down->cols != ffn)
        return fk_fail(FK_INVALID, "moe_layer: gate %d x [%d x %d], up %d x [%d x %d], down %d x [%d x %d] do not form an expert FFN", E, ffn, hidden,
                       up->n_mats, up->rows, up->cols, down->n_mats, down->rows, down->cols);
    if (batch < 1 || k < 1 || k > E) return fk_fail(FK_INVALID, "moe_layer: batch %d, k %d of %d experts", batch, k, E);
    if (((uintptr_t)workspace_dev & 255) || ((uintptr_t)x_dev & 15)) return fk_fail(FK_INVALID, "moe_layer: workspace must be 256-byte aligned, x 16-byte aligned");
    const MoeWs m = moe_ws(E, k, hidden, ffn, batch);
    if (workspace_bytes < m.total) return fk_fail(FK_INVALID, "moe_layer: workspace of %zu bytes, %zu needed (fk_moe_layer_workspace)", workspace_bytes, m.total);
    uint8_t* ws = (uint8_t*)workspace_dev;
    float* logits = (float*)(ws + m.logits);
    int* ids = (int*)(ws + m.ids);
    float* w = (float*)(ws + m.w);
    float *g = (float*)(ws + m.g), *u = (float*)(ws + m.u), *y = (float*)(ws + m.y);
    const int pairs = batch * k;
    int rc;
    auto combine = accumulate ? fk_moe_combine_add : fk_moe_combine;
    if (norm_w && batch > 8) return fk_fail(FK_UNSUPPORTED, "moe_layer_normed: the norm is folded into the decode form only (batch <= 8), got %d rows", batch);
    if (batch <= 8) {
        if ((rc = router_route_launch(ctx, stream, router_dev, x_dev, E, hidden, batch, router_bias_dev, k, mode, logits, ids, w, norm_w, norm_eps))) return rc;
        const float* xin = x_dev;
        int x_stride = 0;
        if (batch > 1) {
            float* xr = (float*)(ws + m.xr);
            FkDeviceGuard gd(ctx->device);
            const size_t n4 = (size_t)pairs * (hidden / 4);
            if (hidden & 3) return fk_fail(FK_INVALID, "moe_layer: hidden %d must be a multiple of 4", hidden);
            FK_CARVEOUT(repeat_rows_kernel);
            repeat_rows_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x_dev, hidden / 4, k, n4, xr);
            FK_CUDA(cudaGetLastError(), FK_LAUNCH);
            ctx->launches++;
            xin = xr;
            x_stride = hidden;
        }
        if (norm_w) {
            // x is the residual stream: the norm rides in the router's and the matvec's prologue, and gate and up (same
            // input, same shape) are the two halves of ONE launch of 2 * pairs slots -- four launches for the layer
            if (gate->kind == FK_BF16 || gate->kind == FK_Q5_K) return fk_fail(FK_UNSUPPORTED, "moe_layer_normed: kind %d has no indexed form", gate->kind);
            // one row: x is the caller's residual stream, complete before the router started, so the matvec may normalize
            // and quantize it while the router still picks the experts (several rows: x was repeated by the launch before)
            if ((rc = fk_gemv_multi_gate_up_launch(ctx, stream, gate, up, ids, pairs, xin, x_stride, norm_w, norm_eps, gate_b, up_b, g,
                                                   batch == 1 ? 1 : 0)))
                return rc;
            if (down_b) rc = fk_gemv_multi_biased(ctx, stream, down, ids, pairs, g, u, ffn, act, down_b, y);
            else rc = fk_gemv_multi_glu(ctx, stream, down, ids, pairs, g, u, ffn, act, y, nullptr);
            if (rc) return rc;
            return combine(ctx, stream, y, nullptr, w, batch, k, hidden, out_dev);
        }
        if (gate_b) {
            // every slot's bias row is added by the lane that finishes the row: still three launches
            if ((rc = fk_gemv_multi_biased(ctx, stream, gate, ids, pairs, xin, nullptr, x_stride, 0, gate_b, g))) return rc;
            if ((rc = fk_gemv_multi_biased(ctx, stream, up, ids, pairs, xin, nullptr, x_stride, 0, up_b, u))) return rc;
            if ((rc = fk_gemv_multi_biased(ctx, stream, down, ids, pairs, g, u, ffn, act, down_b, y))) return rc;
            return combine(ctx, stream, y, nullptr, w, batch, k, hidden, out_dev);
        }
        if ((rc = fk_gemv_multi(ctx, stream, gate, ids, pairs, xin, x_stride, g))) return rc;
        if ((rc = fk_gemv_multi(ctx, stream, up, ids, pairs, xin, x_stride, u))) return rc;
        if ((rc = fk_gemv_multi_glu(ctx, stream, down, ids, pairs, g, u, ffn, act, y, nullptr))) return rc;
        return combine(ctx, stream, y, nullptr, w, batch, k, hidden, out_dev);
    }
    int* group_off = (int*)(ws + m.group_off);
    int* gather = (int*)(ws + m.gather);
    int* pair_of = (int*)(ws + m.pair_of);
    if ((rc = fk_router_logits(ctx, stream, router_dev, x_dev, E, hidden, batch, logits))) return rc;
    if ((rc = fk_moe_route(ctx, stream, logits, router_bias_dev, E, k, mode, batch, ids, w))) return rc;
    if ((rc = fk_moe_permute(ctx, stream, ids, pairs, k, E, group_off, gather, pair_of))) return rc;
    auto add_bias = [&](float* t, const float* bias, int cols) -> int {
        if (!bias) return FK_OK;
        FkDeviceGuard gd(ctx->device);
        const size_t n = (size_t)pairs * cols;
        add_bias_grouped_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(t, bias, group_off, E, pairs, cols);
        FK_CUDA(cudaGetLastError(), FK_LAUNCH);
        ctx->launches++;
        return FK_OK;
    };
    if ((rc = fk_gemm_grouped(ctx, stream, gate, group_off, gather, x_dev, pairs, g))) return rc;
    if ((rc = add_bias(g, gate_b, ffn))) return rc;
    if ((rc = fk_gemm_grouped(ctx, stream, up, group_off, gather, x_dev, pairs, u))) return rc;
    if ((rc = add_bias(u, up_b, ffn))) return rc;
    if ((rc = fk_glu(ctx, stream, g, u, (size_t)pairs * ffn, act, g))) return rc;
    if ((rc = fk_gemm_grouped(ctx, stream, down, group_off, nullptr, g, pairs, y))) return rc;
    if ((rc = add_bias(y, down_b, hidden))) return rc;
    return combine(ctx, stream, y, pair_of, w, batch, k, hidden, out_dev);
}

FK_EXPORT int fk_moe_layer(fk_ctx* ctx, void* stream, const float* router_dev, const float* router_bias_dev, fk_weight gate, fk_weight up,
                           fk_weight down, int k, int mode, int act, const float* x_dev, int batch, float* out_dev, int accumulate,
                           void* workspace_dev, size_t workspace_bytes) {
    return moe_layer_impl(ctx, stream, router_dev, router_bias_dev, gate, up, down, nullptr, nullptr, nullptr, k, mode, act, x_dev, batch, out_dev,
                          accumulate, workspace_dev, workspace_bytes);
}

// The decode form of the routed layer on the RESIDUAL stream: x_dev is un-normalized, the layer's RMSNorm (weight
// norm_weight_dev) is folded into the router and into the gate / up launch, which is one launch for both projections.
// Bias tables are optional (all three or none).  batch <= 8 only.
FK_EXPORT int fk_moe_layer_normed(fk_ctx* ctx, void* stream, const float* router_dev, const float* router_bias_dev, fk_weight gate, fk_weight up,
                                  fk_weight down, const float* gate_bias_dev, const float* up_bias_dev, const float* down_bias_dev, int k, int mode,
                                  int act, const float* norm_weight_dev, float norm_eps, const float* x_dev, int batch, float* out_dev,
                                  int accumulate, void* workspace_dev, size_t workspace_bytes) {
    if (!norm_weight_dev) return fk_fail(FK_INVALID, "moe_layer_normed: null norm weight");
    const int nb = (gate_bias_dev != nullptr) + (up_bias_dev != nullptr) + (down_bias_dev != nullptr);
    if (nb != 0 && nb != 3) return fk_fail(FK_INVALID, "moe_layer_normed: the three bias tables come together");
    return moe_layer_impl(ctx, stream, router_dev, router_bias_dev, gate, up, down, gate_bias_dev, up_bias_dev, down_bias_dev, k, mode, act, x_dev,
                          batch, out_dev, accumulate, workspace_dev, workspace_bytes, norm_weight_dev, norm_eps);
}

// gpt-oss's routed layer (`run_expert_oai`, crates/frink-moe/src/lib.rs:1039-1060): fk_moe_layer whose expert projections
// each carry a bias table [n_experts][rows]; the activation (act = 1, the clamped form) is applied to the BIASED gate and up.
FK_EXPORT int fk_moe_layer_biased(fk_ctx* ctx, void* stream, const float* router_dev, const float* router_bias_dev, fk_weight gate, fk_weight up,
                                  fk_weight down, const float* gate_bias_dev, const float* up_bias_dev, const float* down_bias_dev, int k, int mode,
                                  int act, const float* x_dev, int batch, float* out_dev, int accumulate, void* workspace_dev,
                                  size_t workspace_bytes) {
    if (!gate_bias_dev || !up_bias_dev || !down_bias_dev) return fk_fail(FK_INVALID, "moe_layer_biased: the three bias tables come together");
    return moe_layer_impl(ctx, stream, router_dev, router_bias_dev, gate, up, down, gate_bias_dev, up_bias_dev, down_bias_dev, k, mode, act, x_dev,
                          batch, out_dev, accumulate, workspace_dev, workspace_bytes);
}
