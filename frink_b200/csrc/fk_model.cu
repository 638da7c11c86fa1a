// The decoder glue around the quantized matmuls, enough to run a dense
// Llama-shaped or a routed Qwen3-MoE-shaped decoder on the device and report
// prefill / decode tokens per second: embedding row gather, RMSNorm (with the
// residual add folded in), RoPE, causal grouped-query attention over an f32 KV
// buffer, greedy argmax.  All f32; none of these is on the graded matmul path,
// so they are written for clarity first.
#include "fk_common.cuh"

namespace {

__device__ __forceinline__ void fk_pdl_sync() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}


// ---- embedding gather: out[i] = dequantized row ids[i]  (the kind's own dequant)
__device__ __forceinline__ float e8m0_scale(uint32_t e) { return __uint_as_float(e == 0 ? 0x00400000u : (e << 23)); }

__global__ void get_rows_kernel(const uint8_t* __restrict__ wb, size_t o0, size_t o1, size_t o2, size_t o3, size_t s0, size_t s1, size_t s2,
                                size_t s3, int kind, int rows, int cols, const int* __restrict__ ids, float* __restrict__ out) {
    fk_pdl_sync();
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
        } else if (kind == FK_BF16) {
            v = __uint_as_float((uint32_t)*(const uint16_t*)(wb + o0 + (size_t)row * s0 + (size_t)e * 2) << 16);
        } else if (kind == FK_Q5_K) {
            const uint8_t* blk = wb + o0 + (size_t)row * s0 + (size_t)(e >> 8) * 176;
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
            const uint8_t q = blk[48 + (j >> 1) * 32 + l];
            const int code = ((j & 1) ? (q >> 4) : (q & 0x0F)) + (((blk[16 + l] >> j) & 1) << 4);
            v = (d * (float)scv) * (float)code - dmin * (float)mv;
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
    fk_pdl_sync();
    const int r = blockIdx.x;
    float* xr = x + (size_t)r * cols;
    const float* rr = res ? res + (size_t)r * cols : nullptr;
    const bool vec = (cols & 3) == 0;       // rows then start on 16-byte boundaries (bases come from 256-byte aligned allocations)
    double s = 0.0;
    if (vec) {
        for (int i = threadIdx.x; i < (cols >> 2); i += blockDim.x) {
            float4 v = ((const float4*)xr)[i];
            if (rr) {
                const float4 q = ((const float4*)rr)[i];
                v.x += q.x; v.y += q.y; v.z += q.z; v.w += q.w;
                ((float4*)xr)[i] = v;
            }
            s += (double)(v.x * v.x) + (double)(v.y * v.y) + (double)(v.z * v.z) + (double)(v.w * v.w);
        }
    } else {
        for (int i = threadIdx.x; i < cols; i += blockDim.x) {
            float v = xr[i];
            if (rr) {
                v += rr[i];
                xr[i] = v;
            }
            s += (double)(v * v);
        }
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
    if (vec) {
        for (int i = threadIdx.x; i < (cols >> 2); i += blockDim.x) {
            const float4 v = ((const float4*)xr)[i], g = ((const float4*)w)[i];
            ((float4*)orow)[i] = make_float4(v.x * scale * g.x, v.y * scale * g.y, v.z * scale * g.z, v.w * scale * g.w);
        }
    } else {
        for (int i = threadIdx.x; i < cols; i += blockDim.x) orow[i] = xr[i] * scale * w[i];
    }
}

// Rows [p0, p0 + n_rows) must lie inside a cache of `cache_rows` rows: otherwise the kernel does nothing (every block
// returns before its first access) and the context's error word becomes 95.
__device__ __forceinline__ bool fk_cache_overrun(int p0, int n_rows, int cache_rows, int* err) {
    if (p0 >= 0 && p0 + n_rows <= cache_rows) return false;
    if (threadIdx.x == 0) fk_raise(err, 95);
    return true;
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
                               float* __restrict__ kc, float* __restrict__ vc, const float* __restrict__ q_norm, const float* __restrict__ k_norm,
                               float eps, int cache_rows, int* __restrict__ err) {
    fk_pdl_sync();
    // a warp per (row, head), q heads first; a lane takes rotation pairs lane, lane + 32, ...
    const int half = head_dim / 2;
    const int p0 = *pos;
    if (fk_cache_overrun(p0, n_rows, cache_rows, err)) return;
    const int kvw = n_kv * head_dim;
    const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
    const int total = n_rows * (n_heads + n_kv);
    for (int item = blockIdx.x * wpb + (threadIdx.x >> 5); item < total; item += gridDim.x * wpb) {
        const int row = item / (n_heads + n_kv), hh = item % (n_heads + n_kv);
        const bool is_q = hh < n_heads;
        const int kh = hh - n_heads;
        float* vv = is_q ? q + (size_t)row * q_ld + hh * head_dim : k + (size_t)row * kv_ld + kh * head_dim;
        const float* nw = is_q ? q_norm : k_norm;
        float scale = 1.0f;
        if (nw) {
            // the per-head RMSNorm of Qwen3 (squares in f32, sum in f64) ahead of the rotation
            double sq = 0.0;
            for (int i = lane; i < head_dim; i += 32) sq += (double)(vv[i] * vv[i]);
            for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
            scale = 1.0f / sqrtf((float)(sq / (double)head_dim) + eps);
        }
        for (int i = lane; i < half; i += 32) {
            const float freq = 1.0f / powf(theta, (float)(2 * i) / (float)head_dim);
            float sn, cs;
            sincosf((float)(p0 + row) * freq, &sn, &cs);
            const int ia = neox ? i : 2 * i, ib = neox ? i + half : 2 * i + 1;
            float xa = vv[ia], xb = vv[ib];
            if (nw) {
                xa = xa * scale * nw[ia];
                xb = xb * scale * nw[ib];
            }
            const float ra = xa * cs - xb * sn, rb = xa * sn + xb * cs;
            vv[ia] = ra;
            vv[ib] = rb;
            if (!is_q) {
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
}

__global__ void add_kernel(float* __restrict__ a, const float* __restrict__ b, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) a[i] += b[i];
}

// ---- KV append: rows [*pos, *pos + n_rows) of the cache <- src
__global__ void kv_append_kernel(float* __restrict__ cache, const float* __restrict__ src, size_t row_elems, int n_rows, const int* __restrict__ pos,
                                 int cache_rows, int* __restrict__ err) {
    if (fk_cache_overrun(*pos, n_rows, cache_rows, err)) return;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < row_elems * n_rows) cache[(size_t)(*pos) * row_elems + i] = src[i];
}

// ---- causal grouped-query attention for a few query rows (decode).  Query row r sits at
// *pos + r and sees keys 0 ..= *pos + r of the K/V buffers [T][n_kv][head_dim];
// head_dim <= 128, a multiple of 4.  The keys of one (row, head) are cut over
// gridDim.x blocks (the grid is fixed so that a captured launch stays valid while
// *pos grows; the cut is made on the device).  A block walks its keys in tiles of 64:
// eight lanes share one key's dot product (coalesced 128-byte pieces of the K row),
// the tile's probabilities sit in two registers per lane, and warp w folds V rows
// w, w + 4, ... with lane l owning channels 4l..4l+3.  Each block parks (max, sum,
// unnormalised output) in the workspace; the block that arrives last for the
// (row, head) merges them and rewinds the arrival counter.
constexpr int AD_WARPS = 4, AD_TK = 64, AD_REC = 132, AD_MAX_SPLITS = 64, AD_MAX_CNT = 4096;
// One decode row with the step's RoPE and cache append folded in (on != 0, one query row):
// q arrives unrotated and is (normed and) rotated in shared memory; the newest key and value
// are taken from the projection's output (k_new / v_new), rotated in shared memory by every
// block whose share of the keys holds that position, and written to the caches by the blocks
// of the first query head of each KV group.  No block reads that position from the caches.
struct AttnFuse {
    const float* k_new;
    const float* v_new;
    float* kc;
    float* vc;
    const float* q_norm;
    const float* k_norm;
    float theta, eps;
    int neox, on;
    // independent sequences (seq_stride != 0): query row r is sequence r's newest token, at position pos[r], with its own
    // caches r * seq_stride floats further on; k_new / v_new rows are k_ld / v_ld floats apart
    size_t seq_stride;
    int k_ld, v_ld;
    // gpt-oss attention (crates/frink-core/src/attention.rs:312-322, 960-1000): a query sees only the `window` most recent
    // keys including its own (0 = all), and one learned logit per query head (`sinks`, null = none) joins the softmax's
    // denominator without contributing to the output
    int window;
    const float* sinks;
};
__global__ void __launch_bounds__(AD_WARPS * 32)
attn_kernel(const float* __restrict__ q, int q_ld, const float* __restrict__ kbuf, const float* __restrict__ vbuf, int n_heads, int n_kv, int head_dim,
            const int* __restrict__ pos, float scale, float* __restrict__ out, float* __restrict__ ws, unsigned* __restrict__ cnt, const AttnFuse f,
            int cache_rows, int* __restrict__ err) {
    fk_pdl_sync();
    const bool per_seq = f.seq_stride != 0;
    const int p_row = per_seq ? pos[blockIdx.z] : *pos + (int)blockIdx.z;     // this query row's position
    if (per_seq ? fk_cache_overrun(p_row, 1, cache_rows, err) : fk_cache_overrun(*pos, (int)gridDim.z, cache_rows, err)) return;
    if (per_seq) {
        kbuf += (size_t)blockIdx.z * f.seq_stride;
        vbuf += (size_t)blockIdx.z * f.seq_stride;
    }
    __shared__ __align__(16) float sk_new[128];
    __shared__ __align__(16) float sv_new[128];
    __shared__ double s_red[AD_WARPS];
    __shared__ __align__(16) float sq[128];
    __shared__ float s_p[AD_TK];
    __shared__ __align__(16) float s_acc[AD_WARPS][128];
    __shared__ bool last;
    const int split = blockIdx.x, S = gridDim.x, h = blockIdx.y, r = blockIdx.z, kvh = h / (n_heads / n_kv);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, sub = lane & 7;
    const int n_keys = p_row + 1;
    const int k_lo = f.window > 0 ? max(0, n_keys - f.window) : 0;     // first visible key
    const int chunk = ((n_keys - k_lo + S - 1) / S + 15) & ~15;
    const int c0 = k_lo + split * chunk, c1 = min(n_keys, c0 + chunk);
    const float* qr = q + (size_t)r * q_ld + (size_t)h * head_dim;
    for (int i = threadIdx.x; i < head_dim; i += blockDim.x) sq[i] = qr[i];
    __syncthreads();
    const size_t kv_stride = (size_t)n_kv * head_dim;
    const int p_new = n_keys - 1;
    const bool has_new = f.on && c0 <= p_new && p_new < c1;
    if (f.on) {
        // (head norm and) rotation of one head held in shared memory, at position p_new; same
        // arithmetic as rope_kv_kernel
        auto rope_head = [&](float* buf, const float* nw) {
            float nscale = 1.0f;
            if (nw) {
                double sqs = 0.0;
                for (int i = threadIdx.x; i < head_dim; i += blockDim.x) sqs += (double)(buf[i] * buf[i]);
                for (int o = 16; o > 0; o >>= 1) sqs += __shfl_xor_sync(0xffffffffu, sqs, o);
                if (lane == 0) s_red[warp] = sqs;
                __syncthreads();
                double tsum = 0.0;
                for (int i = 0; i < AD_WARPS; i++) tsum += s_red[i];
                nscale = 1.0f / sqrtf((float)(tsum / (double)head_dim) + f.eps);
                __syncthreads();
            }
            const int half = head_dim >> 1;
            for (int i = threadIdx.x; i < half; i += blockDim.x) {
                const float freq = 1.0f / powf(f.theta, (float)(2 * i) / (float)head_dim);
                float sn, cs;
                sincosf((float)p_new * freq, &sn, &cs);
                const int ia = f.neox ? i : 2 * i, ib = f.neox ? i + half : 2 * i + 1;
                float xa = buf[ia], xb = buf[ib];
                if (nw) {
                    xa = xa * nscale * nw[ia];
                    xb = xb * nscale * nw[ib];
                }
                buf[ia] = xa * cs - xb * sn;
                buf[ib] = xa * sn + xb * cs;
            }
            __syncthreads();
        };
        rope_head(sq, f.q_norm);
        if (has_new) {
            for (int i = threadIdx.x; i < head_dim; i += blockDim.x) {
                sk_new[i] = f.k_new[(size_t)r * f.k_ld + (size_t)kvh * head_dim + i];
                sv_new[i] = f.v_new[(size_t)r * f.v_ld + (size_t)kvh * head_dim + i];
            }
            __syncthreads();
            rope_head(sk_new, f.k_norm);
            if (h % (n_heads / n_kv) == 0) {
                for (int i = threadIdx.x; i < head_dim; i += blockDim.x) {
                    const size_t at = (size_t)r * f.seq_stride + (size_t)p_new * kv_stride + (size_t)kvh * head_dim + i;
                    f.kc[at] = sk_new[i];
                    f.vc[at] = sv_new[i];
                }
            }
        }
    }
    const int hd4 = head_dim >> 2;
    float m = -INFINITY, s = 0.0f;
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    const bool owns = lane < hd4;
    for (int t0 = c0; t0 < c1; t0 += AD_TK) {
        const int nk = min(AD_TK, c1 - t0);
        // this warp's V rows are requested now, beside the K rows, and used after the softmax
        float4 vv[AD_TK / AD_WARPS];
#pragma unroll
        for (int jj = 0; jj < AD_TK / AD_WARPS; jj++) {
            const int j = warp + AD_WARPS * jj;
            vv[jj] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (j < nk && owns)
                vv[jj] = (has_new && t0 + j == p_new) ? *(const float4*)(sv_new + 4 * lane)
                                                      : *(const float4*)(vbuf + (size_t)(t0 + j) * kv_stride + (size_t)kvh * head_dim + 4 * lane);
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int j = warp * 16 + i * 4 + (lane >> 3);
            float d = 0.0f;
            if (j < nk) {
                const float4* kr = (has_new && t0 + j == p_new) ? (const float4*)sk_new
                                                                : (const float4*)(kbuf + (size_t)(t0 + j) * kv_stride + (size_t)kvh * head_dim);
#pragma unroll 4
                for (int f = sub; f < hd4; f += 8) {
                    const float4 kv = kr[f], qv = *(const float4*)(sq + 4 * f);
                    d += kv.x * qv.x + kv.y * qv.y + kv.z * qv.z + kv.w * qv.w;
                }
            }
            d += __shfl_xor_sync(0xffffffffu, d, 4);
            d += __shfl_xor_sync(0xffffffffu, d, 2);
            d += __shfl_xor_sync(0xffffffffu, d, 1);
            if (sub == 0 && j < nk) s_p[j] = d * scale;
        }
        __syncthreads();
        // every warp works out the tile's max and sum for itself (same values in all four)
        const float sc0 = lane < nk ? s_p[lane] : -INFINITY, sc1 = lane + 32 < nk ? s_p[lane + 32] : -INFINITY;
        float tm = fmaxf(sc0, sc1);
        for (int o = 16; o > 0; o >>= 1) tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, o));
        const float m_new = fmaxf(m, tm);
        const float p0 = lane < nk ? expf(sc0 - m_new) : 0.0f, p1 = lane + 32 < nk ? expf(sc1 - m_new) : 0.0f;
        float ts = p0 + p1;
        for (int o = 16; o > 0; o >>= 1) ts += __shfl_xor_sync(0xffffffffu, ts, o);
        const float corr = expf(m - m_new);   // exp(-inf) = 0 on the first tile
        s = s * corr + ts;
        acc.x *= corr; acc.y *= corr; acc.z *= corr; acc.w *= corr;
#pragma unroll
        for (int jj = 0; jj < AD_TK / AD_WARPS; jj++) {
            const int j = warp + AD_WARPS * jj;
            const float pj = __shfl_sync(0xffffffffu, jj < 8 ? p0 : p1, j & 31);
            acc.x += pj * vv[jj].x; acc.y += pj * vv[jj].y; acc.z += pj * vv[jj].z; acc.w += pj * vv[jj].w;
        }
        m = m_new;
        __syncthreads();
    }
    *(float4*)(&s_acc[warp][4 * lane]) = acc;
    __syncthreads();
    float* rec = ws + ((size_t)(r * n_heads + h) * S + split) * AD_REC;
    if (threadIdx.x < head_dim) {
        const int t = threadIdx.x;
        rec[t] = s_acc[0][t] + s_acc[1][t] + s_acc[2][t] + s_acc[3][t];
    }
    if (threadIdx.x == 0) { rec[128] = m; rec[129] = s; }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) last = atomicAdd(&cnt[r * n_heads + h], 1u) == (unsigned)(S - 1);
    __syncthreads();
    if (!last) return;
    __threadfence();
    // merge: warp 0 turns the parked maxima into one weight per block, then each thread
    // folds its channel over the blocks (loads that do not wait on one another)
    __shared__ float s_c[AD_MAX_SPLITS];
    __shared__ float s_gs;
    const float* all = ws + (size_t)(r * n_heads + h) * S * AD_REC;
    if (warp == 0) {
        const bool h0 = lane < S, h1 = lane + 32 < S;
        const float m0 = h0 ? __ldcg(all + lane * AD_REC + 128) : -INFINITY, m1 = h1 ? __ldcg(all + (lane + 32) * AD_REC + 128) : -INFINITY;
        const float s0 = h0 ? __ldcg(all + lane * AD_REC + 129) : 0.0f, s1 = h1 ? __ldcg(all + (lane + 32) * AD_REC + 129) : 0.0f;
        float gm = fmaxf(m0, m1);
        for (int o = 16; o > 0; o >>= 1) gm = fmaxf(gm, __shfl_xor_sync(0xffffffffu, gm, o));
        const float w0 = m0 == -INFINITY ? 0.0f : expf(m0 - gm), w1 = m1 == -INFINITY ? 0.0f : expf(m1 - gm);   // -inf: an empty share
        float gs = s0 * w0 + s1 * w1;
        for (int o = 16; o > 0; o >>= 1) gs += __shfl_xor_sync(0xffffffffu, gs, o);
        if (h0) s_c[lane] = w0;
        if (h1) s_c[lane + 32] = w1;
        if (lane == 0) s_gs = f.sinks ? gs + expf(f.sinks[h] - gm) : gs;      // the sink's share of the softmax, none of the output
    }
    __syncthreads();
    if (threadIdx.x < head_dim) {
        float o = 0.0f;
#pragma unroll 8
        for (int i = 0; i < S; i++) o += __ldcg(all + i * AD_REC + threadIdx.x) * s_c[i];
        out[((size_t)r * n_heads + h) * head_dim + threadIdx.x] = o / s_gs;
    }
    if (threadIdx.x == 0) cnt[r * n_heads + h] = 0;
}

// ---- the same attention for a prefill batch: a block takes 32 consecutive query rows
// of one head, 8 warps x 4 rows; K and V tiles of 32 keys are staged once in shared
// memory (K rows padded by 4 floats so lanes scoring different keys hit different
// banks) and shared by the block's 32 rows.
constexpr int PF_ROWS = 32, PF_WARPS = 8, PF_RPW = PF_ROWS / PF_WARPS;
__global__ void __launch_bounds__(PF_WARPS * 32)
attn_prefill_kernel(const float* __restrict__ q, int q_ld, const float* __restrict__ kbuf, const float* __restrict__ vbuf, int n_q, int n_heads, int n_kv,
                    int head_dim, const int* __restrict__ pos, float scale, float* __restrict__ out, int cache_rows, int* __restrict__ err,
                    int window, const float* __restrict__ sinks) {
    if (fk_cache_overrun(*pos, n_q, cache_rows, err)) return;
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
        if (r0 + rr < n_q) v = *(const float4*)(q + (size_t)(r0 + rr) * q_ld + (size_t)h * head_dim + 4 * c);
        *(float4*)(sq + rr * head_dim + 4 * c) = v;
    }
    float m[PF_RPW], s[PF_RPW];
    float4 acc[PF_RPW];
#pragma unroll
    for (int i = 0; i < PF_RPW; i++) { m[i] = -INFINITY; s[i] = 0.0f; acc[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f); }
    const bool owns = 4 * lane < head_dim;
    const int last_row = min(n_q, r0 + PF_ROWS) - 1;
    const int n_keys_max = p0 + last_row + 1;
    // with a window, the block's first row sees the oldest key: tiles before it are skipped (32-aligned, so the tiles are
    // the same as without a window)
    const int t_first = window > 0 ? (max(0, p0 + r0 + 1 - window) & ~31) : 0;
    for (int t0 = t_first; t0 < n_keys_max; t0 += 32) {
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
        // the warp's rows together: a key's row of K (and of V below) is read once from shared memory for all of them.
        // Every row's own sums run in the same order as if it were alone.
        const int key = t0 + lane;
        int nk[PF_RPW], lo[PF_RPW];
        bool act[PF_RPW];
        float d[PF_RPW], p[PF_RPW];
#pragma unroll
        for (int i = 0; i < PF_RPW; i++) {
            const int r = r0 + warp * PF_RPW + i;
            nk[i] = p0 + r + 1;
            lo[i] = window > 0 ? max(0, nk[i] - window) : 0;
            act[i] = r < n_q && t0 < nk[i] && t0 + 32 > lo[i];
            d[i] = 0.0f;
            p[i] = 0.0f;
        }
        bool any = false;
#pragma unroll
        for (int i = 0; i < PF_RPW; i++) any = any || act[i];
        if (!any) continue;                                  // none of the warp's rows sees this tile
        {
            const float* kr = sk + lane * kpad;
            const float* qr = sq + warp * PF_RPW * head_dim;
            for (int c = 0; c < hd4; c++) {
                const float4 kv4 = *(const float4*)(kr + 4 * c);
#pragma unroll
                for (int i = 0; i < PF_RPW; i++) {
                    const float4 qv = *(const float4*)(qr + i * head_dim + 4 * c);
                    d[i] += kv4.x * qv.x + kv4.y * qv.y + kv4.z * qv.z + kv4.w * qv.w;
                }
            }
        }
        int cnt = 0;
#pragma unroll
        for (int i = 0; i < PF_RPW; i++) {
            if (!act[i]) continue;
            const bool vis = key < nk[i] && key >= lo[i];
            const float sc = vis ? d[i] * scale : -INFINITY;
            float tm = sc;
            for (int o = 16; o > 0; o >>= 1) tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, o));
            const float m_new = fmaxf(m[i], tm);
            p[i] = vis ? expf(sc - m_new) : 0.0f;
            float ts = p[i];
            for (int o = 16; o > 0; o >>= 1) ts += __shfl_xor_sync(0xffffffffu, ts, o);
            const float corr = expf(m[i] - m_new);
            s[i] = s[i] * corr + ts;
            acc[i].x *= corr; acc[i].y *= corr; acc[i].z *= corr; acc[i].w *= corr;
            m[i] = m_new;
            cnt = max(cnt, min(32, nk[i] - t0));
        }
        for (int j = 0; j < cnt; j++) {
            float4 vv = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (owns) vv = *(const float4*)(sv + j * head_dim + 4 * lane);
#pragma unroll
            for (int i = 0; i < PF_RPW; i++) {
                const float pj = __shfl_sync(0xffffffffu, p[i], j);
                acc[i].x += pj * vv.x; acc[i].y += pj * vv.y; acc[i].z += pj * vv.z; acc[i].w += pj * vv.w;
            }
        }
    }
#pragma unroll
    for (int i = 0; i < PF_RPW; i++) {
        const int r = r0 + warp * PF_RPW + i;
        if (r < n_q && owns) {
            const float inv = 1.0f / (sinks ? s[i] + expf(sinks[h] - m[i]) : s[i]);
            float* orow = out + ((size_t)r * n_heads + h) * head_dim + 4 * lane;
            orow[0] = acc[i].x * inv; orow[1] = acc[i].y * inv; orow[2] = acc[i].z * inv; orow[3] = acc[i].w * inv;
        }
    }
}

// ---- greedy argmax of each row (ties -> lower index, NaN never wins).  A row is cut
// over gridDim.x blocks; each folds its slice into one 64-bit key (order-preserving
// float bits above, ~index below, so an unsigned max picks the largest value and
// then the lowest index), parks it in the context's workspace, and the block that
// arrives last for the row reduces the parked keys and rewinds the row's counter.
constexpr int ARGMAX_MAX_BLOCKS = 64, ARGMAX_MAX_ROWS = 64;
__device__ __forceinline__ unsigned long long argmax_key(float v, int i) {
    unsigned u = __float_as_uint(v != v ? -INFINITY : v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ((unsigned long long)u << 32) | (unsigned)(~i);
}
__global__ void __launch_bounds__(256)
argmax_kernel(const float* __restrict__ x, int n, int* __restrict__ out, unsigned long long* __restrict__ ws, unsigned* __restrict__ cnt) {
    fk_pdl_sync();
    const int row = blockIdx.y;
    const float* xr = x + (size_t)row * n;
    unsigned long long best = 0ull;
    if ((n & 3) == 0 && !((uintptr_t)x & 15)) {
        for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < (n >> 2); i += gridDim.x * blockDim.x) {
            const float4 v = ((const float4*)xr)[i];
            best = max(best, max(max(argmax_key(v.x, 4 * i), argmax_key(v.y, 4 * i + 1)), max(argmax_key(v.z, 4 * i + 2), argmax_key(v.w, 4 * i + 3))));
        }
    } else {
        for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) best = max(best, argmax_key(xr[i], i));
    }
    __shared__ unsigned long long sk[8];
    __shared__ bool last;
    for (int o = 16; o > 0; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
    if ((threadIdx.x & 31) == 0) sk[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < 8; i++) best = max(best, sk[i]);
        ws[row * ARGMAX_MAX_BLOCKS + blockIdx.x] = best;
        __threadfence();
        last = atomicAdd(&cnt[row], 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (last && threadIdx.x < 32) {
        __threadfence();
        unsigned long long b = 0ull;
        for (int i = threadIdx.x; i < (int)gridDim.x; i += 32) b = max(b, ((volatile unsigned long long*)ws)[row * ARGMAX_MAX_BLOCKS + i]);
        for (int o = 16; o > 0; o >>= 1) b = max(b, __shfl_xor_sync(0xffffffffu, b, o));
        if (threadIdx.x == 0) {
            out[row] = (int)(~(unsigned)(b & 0xffffffffull));
            cnt[row] = 0;
        }
    }
}

__global__ void add_int_kernel(int* p, int v) {
    fk_pdl_sync();
    *p += v;
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

// Launch with programmatic stream serialization: the grid may be scheduled while the previous
// kernel of the stream still runs; the kernels below call fk_pdl_sync() before they touch
// global memory, which waits for that kernel to complete (and lets the next grid be scheduled).
template <typename... KArgs, typename... Args>
cudaError_t fk_launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

#define FK_LAUNCH_CHECK() do { FK_CUDA(cudaGetLastError(), FK_LAUNCH); ctx->launches++; } while (0)

FK_EXPORT int fk_get_rows(fk_ctx* ctx, void* stream, fk_weight w, int mat, const int* ids_dev, int n, float* out_dev) {
    if (!ctx || !w || !ids_dev || !out_dev || n < 1 || n > 65535) return fk_fail(FK_INVALID, "get_rows: bad argument");
    if (mat < 0 || mat >= w->n_mats) return fk_fail(FK_INVALID, "get_rows: matrix %d of %d", mat, w->n_mats);
    FkDeviceGuard g(ctx->device);
    dim3 grid((w->cols + 255) / 256 > 8 ? 8 : (w->cols + 255) / 256, n);
    FK_CARVEOUT(get_rows_kernel);
    FK_CUDA(fk_launch_pdl(get_rows_kernel, grid, dim3(256), 0, (cudaStream_t)stream, w->dev + (size_t)mat * w->mat_stride, w->plane_off[0], w->plane_off[1], w->plane_off[2],
                                                           w->plane_off[3], w->plane_stride[0], w->plane_stride[1], w->plane_stride[2],
                                                           w->plane_stride[3], w->kind, w->rows, w->cols, ids_dev, out_dev), FK_LAUNCH);
    FK_LAUNCH_CHECK();
    return FK_OK;
}

FK_EXPORT int fk_rmsnorm(fk_ctx* ctx, void* stream, float* x_dev, const float* residual_dev, const float* weight_dev, int n_rows, int cols,
                         float eps, float* out_dev) {
    if (!ctx || !x_dev || !weight_dev || !out_dev || n_rows < 1 || cols < 1) return fk_fail(FK_INVALID, "rmsnorm: bad argument");
    FkDeviceGuard g(ctx->device);
    const bool aligned = !(((uintptr_t)x_dev | (uintptr_t)residual_dev | (uintptr_t)weight_dev | (uintptr_t)out_dev) & 15);
    if ((cols & 3) == 0 && !aligned) return fk_fail(FK_INVALID, "rmsnorm: buffers must be 16-byte aligned");
    int threads = n_rows <= 8 ? ((cols / 4 + 31) / 32) * 32 : 256;
    threads = threads < 64 ? 64 : threads > 1024 ? 1024 : threads;
    FK_CARVEOUT(rmsnorm_kernel);
    FK_CUDA(fk_launch_pdl(rmsnorm_kernel, dim3(n_rows), dim3(threads), 0, (cudaStream_t)stream, x_dev, residual_dev, weight_dev, cols, eps, out_dev), FK_LAUNCH);
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
                         int n_heads, int n_kv, int head_dim, const int* pos_dev, float theta, int neox, float* k_cache_dev, float* v_cache_dev,
                         const float* q_norm_dev, const float* k_norm_dev, float norm_eps, int cache_rows) {
    if (!ctx || !q_dev || !k_dev || !v_dev || !pos_dev || !k_cache_dev || !v_cache_dev) return fk_fail(FK_INVALID, "rope_kv: null argument");
    if (cache_rows < n_rows) return fk_fail(FK_INVALID, "rope_kv: %d rows into caches of %d rows", n_rows, cache_rows);
    if (n_rows < 1 || n_heads < 1 || n_kv < 1 || head_dim < 2 || (head_dim & 1)) return fk_fail(FK_INVALID, "rope_kv: bad shape");
    FkDeviceGuard g(ctx->device);
    if ((q_norm_dev == nullptr) != (k_norm_dev == nullptr)) return fk_fail(FK_INVALID, "rope_kv: q and k norm weights come together");
    const int total = n_rows * (n_heads + n_kv);          // a warp each, four warps per block
    int blocks = (total + 3) / 4;
    if (blocks > 4096) blocks = 4096;
    FK_CARVEOUT(rope_kv_kernel);
    FK_CUDA(fk_launch_pdl(rope_kv_kernel, dim3(blocks), dim3(128), 0, (cudaStream_t)stream, q_dev, k_dev, v_dev, q_ld, kv_ld, n_rows, n_heads, n_kv,
                          head_dim, pos_dev, theta, neox, k_cache_dev, v_cache_dev, q_norm_dev, k_norm_dev, norm_eps, cache_rows, ctx->err_flag), FK_LAUNCH);
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

FK_EXPORT int fk_kv_append(fk_ctx* ctx, void* stream, float* cache_dev, const float* src_dev, size_t row_elems, int n_rows, const int* pos_dev,
                           int cache_rows) {
    if (!ctx || !cache_dev || !src_dev || !pos_dev || n_rows < 1) return fk_fail(FK_INVALID, "kv_append: bad argument");
    if (cache_rows < n_rows) return fk_fail(FK_INVALID, "kv_append: %d rows into a cache of %d rows", n_rows, cache_rows);
    FkDeviceGuard g(ctx->device);
    const size_t n = row_elems * n_rows;
    FK_CARVEOUT(kv_append_kernel);
    kv_append_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(cache_dev, src_dev, row_elems, n_rows, pos_dev, cache_rows, ctx->err_flag);
    FK_LAUNCH_CHECK();
    return FK_OK;
}

FK_EXPORT int fk_attention(fk_ctx* ctx, void* stream, const float* q_dev, int q_ld, const float* k_dev, const float* v_dev, int n_q, int n_heads,
                           int n_kv, int head_dim, const int* pos_dev, float scale, float* out_dev, int cache_rows, int window,
                           const float* sinks_dev) {
    if (!ctx || !q_dev || !k_dev || !v_dev || !pos_dev || !out_dev) return fk_fail(FK_INVALID, "attention: null argument");
    if (cache_rows < n_q || window < 0) return fk_fail(FK_INVALID, "attention: %d queries over caches of %d rows, window %d", n_q, cache_rows, window);
    if (n_q < 1 || n_heads < 1 || n_kv < 1 || n_heads % n_kv || head_dim > 128 || (head_dim & 3) || n_heads > 65535)
        return fk_fail(FK_UNSUPPORTED, "attention: %d queries, %d/%d heads of %d", n_q, n_heads, n_kv, head_dim);
    if (q_ld == 0) q_ld = n_heads * head_dim;
    if (q_ld < n_heads * head_dim || (q_ld & 3) || ((uintptr_t)q_dev & 15)) return fk_fail(FK_INVALID, "attention: query row stride %d", q_ld);
    FkDeviceGuard g(ctx->device);
    if (n_q >= 16) {
        const size_t smem = (size_t)(PF_ROWS * head_dim + 32 * (head_dim + 4) + 32 * head_dim) * sizeof(float);
        FK_CUDA(cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), FK_KERNEL);
        FK_CARVEOUT(attn_prefill_kernel);
        attn_prefill_kernel<<<dim3((n_q + PF_ROWS - 1) / PF_ROWS, n_heads), PF_WARPS * 32, smem, (cudaStream_t)stream>>>(
            q_dev, q_ld, k_dev, v_dev, n_q, n_heads, n_kv, head_dim, pos_dev, scale, out_dev, cache_rows, ctx->err_flag, window, sinks_dev);
    } else {
        if (n_q * n_heads > AD_MAX_CNT) return fk_fail(FK_UNSUPPORTED, "attention: %d rows x %d heads", n_q, n_heads);
        int splits = 4 * ctx->sm_count / (n_heads * n_q);
        splits = splits < 1 ? 1 : splits > AD_MAX_SPLITS ? AD_MAX_SPLITS : splits;
        const int rc = fk_ensure_scratch(ctx, (cudaStream_t)stream, (size_t)n_q * n_heads * splits * AD_REC * sizeof(float));
        if (rc != FK_OK) return rc;
        FK_CARVEOUT(attn_kernel);
        AttnFuse nofuse{};
        nofuse.window = window;
        nofuse.sinks = sinks_dev;
        FK_CUDA(fk_launch_pdl(attn_kernel, dim3(splits, n_heads, n_q), dim3(AD_WARPS * 32), 0, (cudaStream_t)stream, q_dev, q_ld, k_dev, v_dev,
                              n_heads, n_kv, head_dim, pos_dev, scale, out_dev, (float*)ctx->scratch, ctx->attn_cnt, nofuse, cache_rows, ctx->err_flag), FK_LAUNCH);
    }
    FK_LAUNCH_CHECK();
    return FK_OK;
}

FK_EXPORT int fk_attention_rope_kv(fk_ctx* ctx, void* stream, const float* q_dev, const float* k_new_dev, const float* v_new_dev, float* k_cache_dev,
                                   float* v_cache_dev, int n_heads, int n_kv, int head_dim, const int* pos_dev, float scale, float theta, int neox,
                                   const float* q_norm_dev, const float* k_norm_dev, float norm_eps, float* out_dev, int cache_rows, int window,
                                   const float* sinks_dev) {
    if (!ctx || !q_dev || !k_new_dev || !v_new_dev || !k_cache_dev || !v_cache_dev || !pos_dev || !out_dev)
        return fk_fail(FK_INVALID, "attention_rope_kv: null argument");
    if (window < 0) return fk_fail(FK_INVALID, "attention_rope_kv: window %d", window);
    if (cache_rows < 1) return fk_fail(FK_INVALID, "attention_rope_kv: caches of %d rows", cache_rows);
    if (n_heads < 1 || n_kv < 1 || n_heads % n_kv || head_dim > 128 || (head_dim & 3) || n_heads > AD_MAX_CNT)
        return fk_fail(FK_UNSUPPORTED, "attention_rope_kv: %d/%d heads of %d", n_heads, n_kv, head_dim);
    if ((q_norm_dev == nullptr) != (k_norm_dev == nullptr)) return fk_fail(FK_INVALID, "attention_rope_kv: q and k norm weights come together");
    if (((uintptr_t)q_dev | (uintptr_t)k_new_dev | (uintptr_t)v_new_dev) & 15) return fk_fail(FK_INVALID, "attention_rope_kv: inputs must be 16-byte aligned");
    FkDeviceGuard g(ctx->device);
    int splits = 4 * ctx->sm_count / n_heads;
    splits = splits < 1 ? 1 : splits > AD_MAX_SPLITS ? AD_MAX_SPLITS : splits;
    const int rc = fk_ensure_scratch(ctx, (cudaStream_t)stream, (size_t)n_heads * splits * AD_REC * sizeof(float));
    if (rc != FK_OK) return rc;
    AttnFuse f{k_new_dev, v_new_dev, k_cache_dev, v_cache_dev, q_norm_dev, k_norm_dev, theta, norm_eps, neox, 1, 0, 0, 0, window, sinks_dev};
    FK_CARVEOUT(attn_kernel);
    FK_CUDA(fk_launch_pdl(attn_kernel, dim3(splits, n_heads, 1), dim3(AD_WARPS * 32), 0, (cudaStream_t)stream, q_dev, n_heads * head_dim, (const float*)k_cache_dev,
                          (const float*)v_cache_dev, n_heads, n_kv, head_dim, pos_dev, scale, out_dev, (float*)ctx->scratch, ctx->attn_cnt, f, cache_rows,
                          ctx->err_flag), FK_LAUNCH);
    FK_LAUNCH_CHECK();
    return FK_OK;
}

// One decode step of n_seqs independent sequences: row r of q / k_new / v_new is sequence r's newest token at position
// pos[r]; sequence r's caches start r * seq_stride floats into k_cache_dev / v_cache_dev.
FK_EXPORT int fk_attention_rope_kv_seqs(fk_ctx* ctx, void* stream, const float* q_dev, int q_ld, const float* k_new_dev, const float* v_new_dev, int k_ld,
                                        int v_ld, float* k_cache_dev, float* v_cache_dev, size_t seq_stride, int n_seqs, int n_heads, int n_kv, int head_dim,
                                        const int* pos_dev, float scale, float theta, int neox, const float* q_norm_dev, const float* k_norm_dev,
                                        float norm_eps, float* out_dev, int cache_rows, int window, const float* sinks_dev) {
    if (!ctx || !q_dev || !k_new_dev || !v_new_dev || !k_cache_dev || !v_cache_dev || !pos_dev || !out_dev)
        return fk_fail(FK_INVALID, "attention_rope_kv_seqs: null argument");
    if (n_seqs < 1 || n_heads < 1 || n_kv < 1 || n_heads % n_kv || head_dim > 128 || (head_dim & 3) || n_seqs * n_heads > AD_MAX_CNT)
        return fk_fail(FK_UNSUPPORTED, "attention_rope_kv_seqs: %d sequences, %d/%d heads of %d", n_seqs, n_heads, n_kv, head_dim);
    if ((q_norm_dev == nullptr) != (k_norm_dev == nullptr)) return fk_fail(FK_INVALID, "attention_rope_kv_seqs: q and k norm weights come together");
    if ((((uintptr_t)q_dev | (uintptr_t)k_new_dev | (uintptr_t)v_new_dev) & 15) || (q_ld & 3) || (k_ld & 3) || (v_ld & 3) || q_ld < n_heads * head_dim ||
        k_ld < n_kv * head_dim || v_ld < n_kv * head_dim)
        return fk_fail(FK_INVALID, "attention_rope_kv_seqs: inputs must be 16-byte aligned, row strides multiples of 4 and at least a row");
    if (cache_rows < 1 || seq_stride < (size_t)cache_rows * n_kv * head_dim)
        return fk_fail(FK_INVALID, "attention_rope_kv_seqs: caches of %d rows, %zu floats apart", cache_rows, seq_stride);
    FkDeviceGuard g(ctx->device);
    int splits = 4 * ctx->sm_count / (n_heads * n_seqs);
    splits = splits < 1 ? 1 : splits > AD_MAX_SPLITS ? AD_MAX_SPLITS : splits;
    const int rc = fk_ensure_scratch(ctx, (cudaStream_t)stream, (size_t)n_seqs * n_heads * splits * AD_REC * sizeof(float));
    if (rc != FK_OK) return rc;
    AttnFuse f{k_new_dev, v_new_dev, k_cache_dev, v_cache_dev, q_norm_dev, k_norm_dev, theta, norm_eps, neox, 1, seq_stride, k_ld, v_ld, window, sinks_dev};
    FK_CARVEOUT(attn_kernel);
    FK_CUDA(fk_launch_pdl(attn_kernel, dim3(splits, n_heads, n_seqs), dim3(AD_WARPS * 32), 0, (cudaStream_t)stream, q_dev, q_ld, (const float*)k_cache_dev,
                          (const float*)v_cache_dev, n_heads, n_kv, head_dim, pos_dev, scale, out_dev, (float*)ctx->scratch, ctx->attn_cnt, f, cache_rows,
                          ctx->err_flag), FK_LAUNCH);
    FK_LAUNCH_CHECK();
    return FK_OK;
}

FK_EXPORT int fk_argmax(fk_ctx* ctx, void* stream, const float* x_dev, int n_rows, int n, int* out_dev) {
    if (!ctx || !x_dev || !out_dev || n_rows < 1 || n < 1) return fk_fail(FK_INVALID, "argmax: bad argument");
    if (n_rows > ARGMAX_MAX_ROWS) return fk_fail(FK_UNSUPPORTED, "argmax: %d rows (at most %d per call)", n_rows, ARGMAX_MAX_ROWS);
    FkDeviceGuard g(ctx->device);
    int blocks = (n + 2047) / 2048;
    blocks = blocks < 1 ? 1 : blocks > ARGMAX_MAX_BLOCKS ? ARGMAX_MAX_BLOCKS : blocks;
    FK_CARVEOUT(argmax_kernel);
    FK_CUDA(fk_launch_pdl(argmax_kernel, dim3(blocks, n_rows), dim3(256), 0, (cudaStream_t)stream, x_dev, n, out_dev, ctx->argmax_ws, ctx->argmax_cnt), FK_LAUNCH);
    FK_LAUNCH_CHECK();
    return FK_OK;
}

FK_EXPORT int fk_add_int(fk_ctx* ctx, void* stream, int* p_dev, int v) {
    if (!ctx || !p_dev) return fk_fail(FK_INVALID, "add_int: null argument");
    FkDeviceGuard g(ctx->device);
    FK_CARVEOUT(add_int_kernel);
    FK_CUDA(fk_launch_pdl(add_int_kernel, dim3(1), dim3(1), 0, (cudaStream_t)stream, p_dev, v), FK_LAUNCH);
    FK_LAUNCH_CHECK();
    return FK_OK;
}
