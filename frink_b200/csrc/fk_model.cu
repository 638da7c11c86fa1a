// The decoder glue around the quantized matmuls, enough to run a dense
// Llama-shaped or a routed Qwen3-MoE-shaped decoder on the device and report
// prefill / decode tokens per second: embedding row gather, RMSNorm (with the
// residual add folded in), RoPE, causal grouped-query attention over an f32 KV
// buffer, greedy argmax.  All f32; none of these is on the graded matmul path,
// so they are written for clarity first.
#include "fk_common.cuh"

namespace {

// ---- embedding gather: out[i] = dequantized row ids[i]  (the kind's own dequant)
__device__ __forceinline__ float e8m0_scale(uint32_t e) { return __uint_as_float(e == 0 ? 0x00400000u : (e << 23)); }

__global__ void get_rows_kernel(const uint8_t* __restrict__ wb, size_t o0, size_t o1, size_t o2, size_t o3, size_t s0, size_t s1, size_t s2,
                                size_t s3, int kind, int rows, int cols, const int* __restrict__ ids, float* __restrict__ out) {
    const int i = blockIdx.y;
    int row = ids[i];
    if (row < 0 || row >= rows) row = 0;
    float* o = out + (size_t)i * cols;
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < cols; e += gridDim.x * blockDim.x) {
        float v;
        if (kind == FK_Q8_0) {
            const float d = fk_h2f(*(const uint16_t*)(wb + o1 + (size_t)row * s1 + (e >> 5) * 2));
            v = (float)*(const int8_t*)(wb + o0 + (size_t)row * s0 + e) * d;
        } else if (kind == FK_Q4_K) {
            const uint8_t* blk = wb + o0 + (size_t)row * s0 + (size_t)(e >> 8) * 144;
            const int j = (e & 255) >> 5, l = e & 31;
            const uint8_t* sc = blk + 4;
            int scv, mv;
            if (j < 4) {
                scv = sc[j] & 63;
                mv = sc[j + 4] & 63;
            } else {
                scv = (sc[j + 4] & 0x0F) | ((sc[j - 4] >> 6) << 4);
                mv = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4);
            }
            const float d = fk_h2f(*(const uint16_t*)blk), dmin = fk_h2f(*(const uint16_t*)(blk + 2));
            const uint8_t q = blk[16 + (j >> 1) * 32 + l];
            const int nib = (j & 1) ? (q >> 4) : (q & 0x0F);
            v = (d * (float)scv) * (float)nib - dmin * (float)mv;
        } else if (kind == FK_Q6_K) {
            const int sb = e >> 8, w = e & 255, hf = w >> 7, t = w & 127, qd = t >> 5, l = t & 31;
            const uint8_t ql = wb[o0 + (size_t)row * s0 + (size_t)sb * 128 + 64 * hf + l + 32 * (qd & 1)];
            const uint8_t qh = wb[o1 + (size_t)row * s1 + (size_t)sb * 64 + 32 * hf + l];
            const int nib = (qd >> 1) ? (ql >> 4) : (ql & 0x0F);
            const int c6 = (nib | (((qh >> (2 * qd)) & 3) << 4)) - 32;
            const int sc = *(const int8_t*)(wb + o2 + (size_t)row * s2 + sb * 16 + (w >> 4));
            const float d = fk_h2f(*(const uint16_t*)(wb + o3 + (size_t)row * s3 + sb * 2));
            v = d * (float)sc * (float)c6;
        } else {  // FK_MXFP4
            const int b = e >> 5, l = e & 31;
            const uint8_t code = wb[o0 + (size_t)row * s0 + (size_t)b * 16 + (l & 15)];
            const int c = (l >> 4) ? (code >> 4) : (code & 0x0F);
            const float kv[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
            const float m = kv[c & 7];
            v = e8m0_scale(wb[o1 + (size_t)row * s1 + b]) * ((c & 8) ? -m : m);
        }
        o[e] = v;
    }
}

// ---- RMSNorm: if `res` is given, x += res first (and the sum is written back to x).
// Squares in f32, summed in f64, the mean rounded to f32, 1/sqrtf(mean + eps): the
// reference's order up to the association of the f64 sum.
__global__ void rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ res, const float* __restrict__ w, int cols, float eps,
                               float* __restrict__ out) {
    const int r = blockIdx.x;
    float* xr = x + (size_t)r * cols;
    const float* rr = res ? res + (size_t)r * cols : nullptr;
    double s = 0.0;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
        float v = xr[i];
        if (rr) {
            v += rr[i];
            xr[i] = v;
        }
        s += (double)(v * v);
    }
    __shared__ double part[32];
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x < 32) {
        double t = threadIdx.x < (blockDim.x >> 5) ? part[threadIdx.x] : 0.0;
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (threadIdx.x == 0) part[0] = t;
    }
    __syncthreads();
    const float mean = (float)(part[0] / (double)cols);
    const float scale = 1.0f / sqrtf(mean + eps);
    float* orow = out + (size_t)r * cols;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) orow[i] = xr[i] * scale * w[i];
}

// ---- RoPE in place over [n_rows][n_heads][head_dim]; row r sits at *pos + r.
__global__ void rope_kernel(float* __restrict__ x, int n_rows, int n_heads, int head_dim, const int* __restrict__ pos, float theta, int neox) {
    const int half = head_dim / 2;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t per_row = (size_t)n_heads * half;
    if (idx >= (size_t)n_rows * per_row) return;
    const int row = (int)(idx / per_row), rem = (int)(idx % per_row), h = rem / half, i = rem % half;
    float* v = x + ((size_t)row * n_heads + h) * head_dim;
    const float freq = 1.0f / powf(theta, (float)(2 * i) / (float)head_dim);
    const float angle = (float)(*pos + row) * freq;
    float s, c;
    sincosf(angle, &s, &c);
    const int ia = neox ? i : 2 * i, ib = neox ? i + half : 2 * i + 1;
    const float a = v[ia], b = v[ib];
    v[ia] = a * c - b * s;
    v[ib] = a * s + b * c;
}

// rope(q), rope(k), and the cache append of k and v, one launch.
__global__ void rope_kv_kernel(float* __restrict__ q, float* __restrict__ k, const float* __restrict__ v, int q_ld, int kv_ld, int n_rows,
                               int n_heads, int n_kv, int head_dim, const int* __restrict__ pos, float theta, int neox,
                               float* __restrict__ kc, float* __restrict__ vc) {
    const int half = head_dim / 2;
    const int p0 = *pos;
    const int per_row = (n_heads + n_kv) * half;            // rotation pairs per row, q heads first
    const int kvw = n_kv * head_dim;
    const int total = n_rows * per_row;
    for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
        const int row = idx / per_row, rem = idx % per_row, hh = rem / half, i = rem % half;
        const float freq = 1.0f / powf(theta, (float)(2 * i) / (float)head_dim);
        float s, c;
        sincosf((float)(p0 + row) * freq, &s, &c);
        const int ia = neox ? i : 2 * i, ib = neox ? i + half : 2 * i + 1;
        if (hh < n_heads) {
            float* vv = q + (size_t)row * q_ld + hh * head_dim;
            const float a = vv[ia], b = vv[ib];
            vv[ia] = a * c - b * s;
            vv[ib] = a * s + b * c;
        } else {
            const int kh = hh - n_heads;
            float* vv = k + (size_t)row * kv_ld + kh * head_dim;
            const float a = vv[ia], b = vv[ib];
            const float ra = a * c - b * s, rb = a * s + b * c;
            vv[ia] = ra;
            vv[ib] = rb;
            float* dk = kc + (size_t)(p0 + row) * kvw + kh * head_dim;
            dk[ia] = ra;
            dk[ib] = rb;
            const float* sv = v + (size_t)row * kv_ld + kh * head_dim;
            float* dv = vc + (size_t)(p0 + row) * kvw + kh * head_dim;
            dv[ia] = sv[ia];
            dv[ib] = sv[ib];
        }
    }
}

__global__ void add_kernel(float* __restrict__ a, const float* __restrict__ b, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) a[i] += b[i];
}

// ---- KV append: rows [*pos, *pos + n_rows) of the cache <- src
__global__ void kv_append_kernel(float* __restrict__ cache, const float* __restrict__ src, size_t row_elems, int n_rows, const int* __restrict__ pos) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < row_elems * n_rows) cache[(size_t)(*pos) * row_elems + i] = src[i];
}

// ---- causal grouped-query attention.  One block per (query row, head), 4 warps;
// warp w takes key tiles w, w + 4, ...; inside a tile lane j scores key j against
// the query (held in shared memory), the tile's probabilities stay in the lanes
// and reach the V accumulation by shuffle (lane l owns channels 4l..4l+3).
// Query row r sits at *pos + r and sees keys 0 ..= *pos + r of the K/V buffers
// [T][n_kv][head_dim].  head_dim <= 128, a multiple of 4.
constexpr int ATT_WARPS = 4;
__global__ void __launch_bounds__(ATT_WARPS * 32)
attn_kernel(const float* __restrict__ q, const float* __restrict__ kbuf, const float* __restrict__ vbuf, int n_heads, int n_kv, int head_dim,
            const int* __restrict__ pos, float scale, float* __restrict__ out) {
    __shared__ __align__(16) float sq[128];
    __shared__ float sm_m[ATT_WARPS], sm_s[ATT_WARPS];
    __shared__ __align__(16) float sm_acc[ATT_WARPS][128];
    const int r = blockIdx.x, h = blockIdx.y, kvh = h / (n_heads / n_kv);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_keys = *pos + r + 1;
    const float* qr = q + ((size_t)r * n_heads + h) * head_dim;
    for (int i = threadIdx.x; i < head_dim; i += blockDim.x) sq[i] = qr[i];
    __syncthreads();
    const size_t kv_stride = (size_t)n_kv * head_dim;
    float m = -INFINITY, s = 0.0f;
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    const bool owns = 4 * lane < head_dim;
    for (int t0 = warp * 32; t0 < n_keys; t0 += ATT_WARPS * 32) {
        const int key = t0 + lane;
        float sc = -INFINITY;
        if (key < n_keys) {
            const float4* kr = (const float4*)(kbuf + (size_t)key * kv_stride + (size_t)kvh * head_dim);
            float d = 0.0f;
            for (int i = 0; i < head_dim / 4; i++) {
                const float4 kv = kr[i], qv = *(const float4*)(sq + 4 * i);
                d += kv.x * qv.x + kv.y * qv.y + kv.z * qv.z + kv.w * qv.w;
            }
            sc = d * scale;
        }
        float tm = sc;
        for (int o = 16; o > 0; o >>= 1) tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, o));
        const float m_new = fmaxf(m, tm);
        const float p = key < n_keys ? expf(sc - m_new) : 0.0f;
        float ts = p;
        for (int o = 16; o > 0; o >>= 1) ts += __shfl_xor_sync(0xffffffffu, ts, o);
        const float corr = expf(m - m_new);   // exp(-inf) = 0 on the first tile
        s = s * corr + ts;
        acc.x *= corr; acc.y *= corr; acc.z *= corr; acc.w *= corr;
        const int cnt = min(32, n_keys - t0);
        for (int j = 0; j < cnt; j++) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            if (owns) {
                const float4 vv = *(const float4*)(vbuf + (size_t)(t0 + j) * kv_stride + (size_t)kvh * head_dim + 4 * lane);
                acc.x += pj * vv.x; acc.y += pj * vv.y; acc.z += pj * vv.z; acc.w += pj * vv.w;
            }
        }
        m = m_new;
    }
    if (lane == 0) { sm_m[warp] = m; sm_s[warp] = s; }
    if (owns) *(float4*)(&sm_acc[warp][4 * lane]) = acc;
    __syncthreads();
    if (warp == 0 && owns) {
        float gm = -INFINITY;
        for (int w = 0; w < ATT_WARPS; w++) gm = fmaxf(gm, sm_m[w]);
        float gs = 0.0f;
        float4 o = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int w = 0; w < ATT_WARPS; w++) {
            const float c = sm_m[w] == -INFINITY ? 0.0f : expf(sm_m[w] - gm);
            gs += sm_s[w] * c;
            const float4 a = *(const float4*)(&sm_acc[w][4 * lane]);
            o.x += a.x * c; o.y += a.y * c; o.z += a.z * c; o.w += a.w * c;
        }
        const float inv = 1.0f / gs;
        float* orow = out + ((size_t)r * n_heads + h) * head_dim + 4 * lane;
        orow[0] = o.x * inv; orow[1] = o.y * inv; orow[2] = o.z * inv; orow[3] = o.w * inv;
    }
}

// ---- the same attention for a prefill batch: a block takes 32 consecutive query rows
// of one head, 8 warps x 4 rows; K and V tiles of 32 keys are staged once in shared
// memory (K rows padded by 4 floats so lanes scoring different keys hit different
// banks) and shared by the block's 32 rows.
constexpr int PF_ROWS = 32, PF_WARPS = 8, PF_RPW = PF_ROWS / PF_WARPS;
__global__ void __launch_bounds__(PF_WARPS * 32)
attn_prefill_kernel(const float* __restrict__ q, const float* __restrict__ kbuf, const float* __restrict__ vbuf, int n_q, int n_heads, int n_kv,
                    int head_dim, const int* __restrict__ pos, float scale, float* __restrict__ out) {
    extern __shared__ __align__(16) float sm[];
    const int kpad = head_dim + 4;
    float* sq = sm;                          // [32][head_dim]
    float* sk = sq + PF_ROWS * head_dim;     // [32][head_dim + 4]
    float* sv = sk + 32 * kpad;              // [32][head_dim]
    const int r0 = blockIdx.x * PF_ROWS, h = blockIdx.y, kvh = h / (n_heads / n_kv);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int p0 = *pos;
    const size_t kv_stride = (size_t)n_kv * head_dim;
    const int hd4 = head_dim >> 2;
    for (int i = threadIdx.x; i < PF_ROWS * hd4; i += blockDim.x) {
        const int rr = i / hd4, c = i % hd4;
        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (r0 + rr < n_q) v = *(const float4*)(q + ((size_t)(r0 + rr) * n_heads + h) * head_dim + 4 * c);
        *(float4*)(sq + rr * head_dim + 4 * c) = v;
    }
    float m[PF_RPW], s[PF_RPW];
    float4 acc[PF_RPW];
#pragma unroll
    for (int i = 0; i < PF_RPW; i++) { m[i] = -INFINITY; s[i] = 0.0f; acc[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f); }
    const bool owns = 4 * lane < head_dim;
    const int last_row = min(n_q, r0 + PF_ROWS) - 1;
    const int n_keys_max = p0 + last_row + 1;
    for (int t0 = 0; t0 < n_keys_max; t0 += 32) {
        __syncthreads();
        for (int i = threadIdx.x; i < 32 * hd4; i += blockDim.x) {
            const int kk = i / hd4, c = i % hd4;
            float4 kv4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f), vv4 = kv4;
            if (t0 + kk < n_keys_max) {
                kv4 = *(const float4*)(kbuf + (size_t)(t0 + kk) * kv_stride + (size_t)kvh * head_dim + 4 * c);
                vv4 = *(const float4*)(vbuf + (size_t)(t0 + kk) * kv_stride + (size_t)kvh * head_dim + 4 * c);
            }
            *(float4*)(sk + kk * kpad + 4 * c) = kv4;
            *(float4*)(sv + kk * head_dim + 4 * c) = vv4;
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < PF_RPW; i++) {
            const int rr = warp * PF_RPW + i, r = r0 + rr;
            if (r >= n_q) continue;
            const int n_keys = p0 + r + 1;
            if (t0 >= n_keys) continue;
            const int key = t0 + lane;
            float sc = -INFINITY;
            if (key < n_keys) {
                float d = 0.0f;
                const float* kr = sk + lane * kpad;
                const float* qr = sq + rr * head_dim;
                for (int c = 0; c < hd4; c++) {
                    const float4 kv4 = *(const float4*)(kr + 4 * c), qv = *(const float4*)(qr + 4 * c);
                    d += kv4.x * qv.x + kv4.y * qv.y + kv4.z * qv.z + kv4.w * qv.w;
                }
                sc = d * scale;
            }
            float tm = sc;
            for (int o = 16; o > 0; o >>= 1) tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, o));
            const float m_new = fmaxf(m[i], tm);
            const float p = key < n_keys ? expf(sc - m_new) : 0.0f;
            float ts = p;
            for (int o = 16; o > 0; o >>= 1) ts += __shfl_xor_sync(0xffffffffu, ts, o);
            const float corr = expf(m[i] - m_new);
            s[i] = s[i] * corr + ts;
            acc[i].x *= corr; acc[i].y *= corr; acc[i].z *= corr; acc[i].w *= corr;
            const int cnt = min(32, n_keys - t0);
            for (int j = 0; j < cnt; j++) {
                const float pj = __shfl_sync(0xffffffffu, p, j);
                if (owns) {
                    const float4 vv = *(const float4*)(sv + j * head_dim + 4 * lane);
                    acc[i].x += pj * vv.x; acc[i].y += pj * vv.y; acc[i].z += pj * vv.z; acc[i].w += pj * vv.w;
                }
            }
            m[i] = m_new;
        }
    }
#pragma unroll
    for (int i = 0; i < PF_RPW; i++) {
        const int r = r0 + warp * PF_RPW + i;
        if (r < n_q && owns) {
            const float inv = 1.0f / s[i];
            float* orow = out + ((size_t)r * n_heads + h) * head_dim + 4 * lane;
            orow[0] = acc[i].x * inv; orow[1] = acc[i].y * inv; orow[2] = acc[i].z * inv; orow[3] = acc[i].w * inv;
        }
    }
}

// ---- greedy argmax of each row (ties -> lower index); also advances *pos_inc if given
__global__ void argmax_kernel(const float* __restrict__ x, int n, int* __restrict__ out) {
    const float* xr = x + (size_t)blockIdx.x * n;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = xr[i];
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
    __shared__ float sv[32];
    __shared__ int si[32];
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x < 32) {
        bv = threadIdx.x < (blockDim.x >> 5) ? sv[threadIdx.x] : -INFINITY;
        bi = threadIdx.x < (blockDim.x >> 5) ? si[threadIdx.x] : 0x7fffffff;
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (threadIdx.x == 0) out[blockIdx.x] = bi;
    }
}

__global__ void add_int_kernel(int* p, int v) { *p += v; }

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

#define FK_LAUNCH_CHECK() do { FK_CUDA(cudaGetLastError(), FK_LAUNCH); ctx->launches++; } while (0)

FK_EXPORT int fk_get_rows(fk_ctx* ctx, void* stream, fk_weight w, int mat, const int* ids_dev, int n, float* out_dev) {
    if (!ctx || !w || !ids_dev || !out_dev || n < 1 || n > 65535) return fk_fail(FK_INVALID, "get_rows: bad argument");
    if (mat < 0 || mat >= w->n_mats) return fk_fail(FK_INVALID, "get_rows: matrix %d of %d", mat, w->n_mats);
    FkDeviceGuard g(ctx->device);
    dim3 grid((w->cols + 255) / 256 > 8 ? 8 : (w->cols + 255) / 256, n);
    FK_CARVEOUT(get_rows_kernel);
    get_rows_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(w->dev + (size_t)mat * w->mat_stride, w->plane_off[0], w->plane_off[1], w->plane_off[2],
                                                           w->plane_off[3], w->plane_stride[0], w->plane_stride[1], w->plane_stride[2],
                                                           w->plane_stride[3], w->kind, w->rows, w->cols, ids_dev, out_dev);
    FK_LAUNCH_CHECK();
    return FK_OK;
}

FK_EXPORT int fk_rmsnorm(fk_ctx* ctx, void* stream, float* x_dev, const float* residual_dev, const float* weight_dev, int n_rows, int cols,
                         float eps, float* out_dev) {
    if (!ctx || !x_dev || !weight_dev || !out_dev || n_rows < 1 || cols < 1) return fk_fail(FK_INVALID, "rmsnorm: bad argument");
    FkDeviceGuard g(ctx->device);
    FK_CARVEOUT(rmsnorm_kernel);
    rmsnorm_kernel<<<n_rows, 256, 0, (cudaStream_t)stream>>>(x_dev, residual_dev, weight_dev, cols, eps, out_dev);
    FK_LAUNCH_CHECK();
    return FK_OK;
}

FK_EXPORT int fk_rope(fk_ctx* ctx, void* stream, float* x_dev, int n_rows, int n_heads, int head_dim, const int* pos_dev, float theta, int neox) {
    if (!ctx || !x_dev || !pos_dev || n_rows < 1 || n_heads < 1 || head_dim < 2 || (head_dim & 1)) return fk_fail(FK_INVALID, "rope: bad argument");
    FkDeviceGuard g(ctx->device);
    const size_t n = (size_t)n_rows * n_heads * (head_dim / 2);
    FK_CARVEOUT(rope_kernel);
    rope_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x_dev, n_rows, n_heads, head_dim, pos_dev, theta, neox);
    FK_LAUNCH_CHECK();
    return FK_OK;
}

FK_EXPORT int fk_rope_kv(fk_ctx* ctx, void* stream, float* q_dev, float* k_dev, const float* v_dev, int q_ld, int kv_ld, int n_rows,
                         int n_heads, int n_kv, int head_dim, const int* pos_dev, float theta, int neox, float* k_cache_dev, float* v_cache_dev) {
    if (!ctx || !q_dev || !k_dev || !v_dev || !pos_dev || !k_cache_dev || !v_cache_dev) return fk_fail(FK_INVALID, "rope_kv: null argument");
    if (n_rows < 1 || n_heads < 1 || n_kv < 1 || head_dim < 2 || (head_dim & 1)) return fk_fail(FK_INVALID, "rope_kv: bad shape");
    FkDeviceGuard g(ctx->device);
    const int total = n_rows * (n_heads + n_kv) * (head_dim / 2);
    int blocks = (total + 255) / 256;
    if (blocks > 4096) blocks = 4096;
    FK_CARVEOUT(rope_kv_kernel);
    rope_kv_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(q_dev, k_dev, v_dev, q_ld, kv_ld, n_rows, n_heads, n_kv, head_dim, pos_dev, theta,
                                                           neox, k_cache_dev, v_cache_dev);
    FK_LAUNCH_CHECK();
    return FK_OK;
}

FK_EXPORT int fk_add(fk_ctx* ctx, void* stream, float* a_dev, const float* b_dev, size_t n) {
    if (!ctx || !a_dev || !b_dev) return fk_fail(FK_INVALID, "add: null argument");
    if (n == 0) return FK_OK;
    FkDeviceGuard g(ctx->device);
    FK_CARVEOUT(add_kernel);
    add_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(a_dev, b_dev, n);
    FK_LAUNCH_CHECK();
    return FK_OK;
}

FK_EXPORT int fk_kv_append(fk_ctx* ctx, void* stream, float* cache_dev, const float* src_dev, size_t row_elems, int n_rows, const int* pos_dev) {
    if (!ctx || !cache_dev || !src_dev || !pos_dev || n_rows < 1) return fk_fail(FK_INVALID, "kv_append: bad argument");
    FkDeviceGuard g(ctx->device);
    const size_t n = row_elems * n_rows;
    FK_CARVEOUT(kv_append_kernel);
    kv_append_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(cache_dev, src_dev, row_elems, n_rows, pos_dev);
    FK_LAUNCH_CHECK();
    return FK_OK;
}

FK_EXPORT int fk_attention(fk_ctx* ctx, void* stream, const float* q_dev, const float* k_dev, const float* v_dev, int n_q, int n_heads, int n_kv,
                           int head_dim, const int* pos_dev, float scale, float* out_dev) {
    if (!ctx || !q_dev || !k_dev || !v_dev || !pos_dev || !out_dev) return fk_fail(FK_INVALID, "attention: null argument");
    if (n_q < 1 || n_heads < 1 || n_kv < 1 || n_heads % n_kv || head_dim > 128 || (head_dim & 3) || n_heads > 65535)
        return fk_fail(FK_UNSUPPORTED, "attention: %d queries, %d/%d heads of %d", n_q, n_heads, n_kv, head_dim);
    FkDeviceGuard g(ctx->device);
    if (n_q >= 16) {
        const size_t smem = (size_t)(PF_ROWS * head_dim + 32 * (head_dim + 4) + 32 * head_dim) * sizeof(float);
        FK_CUDA(cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), FK_KERNEL);
        FK_CARVEOUT(attn_prefill_kernel);
        attn_prefill_kernel<<<dim3((n_q + PF_ROWS - 1) / PF_ROWS, n_heads), PF_WARPS * 32, smem, (cudaStream_t)stream>>>(
            q_dev, k_dev, v_dev, n_q, n_heads, n_kv, head_dim, pos_dev, scale, out_dev);
    } else {
        FK_CARVEOUT(attn_kernel);
        attn_kernel<<<dim3(n_q, n_heads), ATT_WARPS * 32, 0, (cudaStream_t)stream>>>(q_dev, k_dev, v_dev, n_heads, n_kv, head_dim, pos_dev, scale, out_dev);
    }
    FK_LAUNCH_CHECK();
    return FK_OK;
}

FK_EXPORT int fk_argmax(fk_ctx* ctx, void* stream, const float* x_dev, int n_rows, int n, int* out_dev) {
    if (!ctx || !x_dev || !out_dev || n_rows < 1 || n < 1) return fk_fail(FK_INVALID, "argmax: bad argument");
    FkDeviceGuard g(ctx->device);
    FK_CARVEOUT(argmax_kernel);
    argmax_kernel<<<n_rows, 1024, 0, (cudaStream_t)stream>>>(x_dev, n, out_dev);
    FK_LAUNCH_CHECK();
    return FK_OK;
}

FK_EXPORT int fk_add_int(fk_ctx* ctx, void* stream, int* p_dev, int v) {
    if (!ctx || !p_dev) return fk_fail(FK_INVALID, "add_int: null argument");
    FkDeviceGuard g(ctx->device);
    FK_CARVEOUT(add_int_kernel);
    add_int_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(p_dev, v);
    FK_LAUNCH_CHECK();
    return FK_OK;
}
