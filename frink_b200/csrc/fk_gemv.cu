// Decode GEMV (batch 1..8) over resident quantized weights, and its indexed
// (one expert per slot) form.
//
// Shape of the kernel: a persistent grid of 512-thread blocks.  Each block
// first quantizes the activations to q8_1 into shared memory (one warp per run
// of 32 values, the rule of fk_q8_1_lane), then its warps walk pairs of weight
// rows.  A lane owns one 16-byte piece of packed weights per row and trip --
// every global load is a 128-bit load of consecutive addresses across the warp
// -- unpacks it in registers, takes exact int32 dot products against the int8
// activations with dp4a, scales them into an f32 accumulator per (row, batch
// column), and the warp reduces with shuffles.  Weight bytes are read once for
// the whole batch.
#include "fk_common.cuh"

namespace {

constexpr int GEMV_THREADS = 512;
constexpr int GEMV_WARPS = GEMV_THREADS / 32;
constexpr int R = 2;  // weight rows a warp carries at once

struct GemvArgs {
    const uint8_t* w;
    size_t mat_stride;
    size_t plane_off[4];
    const int* ids;
    int mat;
    const float* x;
    int x_stride;
    float* y;
    int rows, cols, batch;
    int32_t* isums;
};

__device__ __forceinline__ uint4 ldg16(const uint8_t* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ int dp4a4(const uint4& a, const int4& b) {
    int s = __dp4a((int)a.x, b.x, 0);
    s = __dp4a((int)a.y, b.y, s);
    s = __dp4a((int)a.z, b.z, s);
    return __dp4a((int)a.w, b.w, s);
}
__device__ __forceinline__ uint32_t byte_of(uint32_t s0, uint32_t s1, uint32_t s2, int k) {
    const uint32_t w = k < 4 ? s0 : (k < 8 ? s1 : s2);
    return (w >> (8 * (k & 3))) & 0xFFu;
}
// 6-bit scale and min of Q4_K sub-block j from the 12 packed bytes.
__device__ __forceinline__ void q4k_scale_min(uint32_t s0, uint32_t s1, uint32_t s2, int j, int* sc, int* m) {
    if (j < 4) {
        *sc = byte_of(s0, s1, s2, j) & 63;
        *m = byte_of(s0, s1, s2, j + 4) & 63;
    } else {
        const uint32_t b = byte_of(s0, s1, s2, j + 4);
        *sc = (b & 0x0F) | ((byte_of(s0, s1, s2, j - 4) >> 6) << 4);
        *m = (b >> 4) | ((byte_of(s0, s1, s2, j) >> 6) << 4);
    }
}
// Four E2M1 codes (the four nibbles of the low 16 bits of `w`) to their doubled
// int8 values {0,1,2,3,4,6,8,12} with sign, one per byte, in nibble order.
__device__ __forceinline__ uint32_t e2m1x2_4(uint32_t w) {
    uint32_t pos, neg, out;
    const uint32_t sel = w & 0x7777u;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(pos) : "r"(0x03020100u), "r"(0x0C080604u), "r"(sel));
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(neg) : "r"(0xFDFEFF00u), "r"(0xF4F8FAFCu), "r"(sel));
    const uint32_t pick = 0x3210u | ((w & 0x8888u) >> 1);
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(pos), "r"(neg), "r"(pick));
    return out;
}
__device__ __forceinline__ float e8m0_half(uint32_t e) {
    return __uint_as_float(e < 2 ? (0x00200000u << e) : ((e - 1u) << 23));
}

template <int KIND, int NB, bool DUMP>
__global__ void __launch_bounds__(GEMV_THREADS) gemv_kernel(const GemvArgs a) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int cols = a.cols, rows = a.rows;
    const int nb32 = cols >> 5;
    int8_t* sq = (int8_t*)smem;                       // [NB][cols] int8
    float* sd = (float*)(smem + (size_t)NB * cols);   // [NB][nb32] stored scale, widened
    float* ss = sd + NB * nb32;                       // Q4_K: [NB][nb32] scale * run sum
    int* sb16 = (int*)(sd + NB * nb32);               // Q6_K: [NB][cols/16] sums of 16

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int slot = blockIdx.y;
    const int mat = a.ids ? a.ids[slot] : a.mat;
    const uint8_t* wb = a.w + (size_t)mat * a.mat_stride;
    const float* x = a.x + (size_t)slot * a.x_stride;
    float* y = a.y + (size_t)slot * a.batch * rows;

    // ---- activations -> q8_1 in shared memory
    for (int run = warp; run < NB * nb32; run += GEMV_WARPS) {
        const int b = run / nb32, kb = run - b * nb32;
        const float v = b < a.batch ? x[(size_t)b * cols + kb * 32 + lane] : 0.0f;
        float d;
        int qsum;
        const int q = fk_q8_1_lane(v, &d, &qsum);
        // MXFP4 keeps each run as (elem j, elem j+16) pairs: the order its
        // nibble decode produces bytes in.
        const int pos = KIND == FK_MXFP4 ? (((lane & 15) << 1) | (lane >> 4)) : lane;
        sq[(size_t)b * cols + kb * 32 + pos] = (int8_t)q;
        if (KIND == FK_Q6_K) {
            const int half_sum = __reduce_add_sync(0xffffffffu, lane < 16 ? q : 0);
            if (lane == 0) {
                sb16[b * (cols >> 4) + 2 * kb] = half_sum;
                sb16[b * (cols >> 4) + 2 * kb + 1] = qsum - half_sum;
            }
        }
        if (lane == 0) {
            sd[b * nb32 + kb] = d;
            if (KIND == FK_Q4_K) ss[b * nb32 + kb] = d * (float)qsum;
        }
    }
    __syncthreads();

    const int gwarp = blockIdx.x * GEMV_WARPS + warp;
    const int twarps = gridDim.x * GEMV_WARPS;

    for (int rp = gwarp; rp * R < rows; rp += twarps) {
        const int row0 = rp * R;
        float acc[R][NB];
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int b = 0; b < NB; b++) acc[r][b] = 0.0f;

        if (KIND == FK_Q4_K) {
            const int nsb = cols >> 8;
            const size_t row_bytes = (size_t)nsb * 144;
            const int c = lane & 7, g = c >> 1, h = c & 1;
            for (int sb0 = 0; sb0 < nsb; sb0 += 4) {
                const int sb = sb0 + (lane >> 3);
                const bool live = sb < nsb;
                const int sbs = live ? sb : 0;
                uint4 wq[R];
                float f_lo[R], f_hi[R], mm_lo[R], mm_hi[R];
#pragma unroll
                for (int r = 0; r < R; r++) {
                    uint4 hd = make_uint4(0, 0, 0, 0);
                    wq[r] = make_uint4(0, 0, 0, 0);
                    if (live && row0 + r < rows) {
                        const uint8_t* p = wb + (size_t)(row0 + r) * row_bytes + (size_t)sb * 144;
                        hd = ldg16(p);
                        wq[r] = ldg16(p + 16 + 16 * c);
                    }
                    const float d = fk_h2f((uint16_t)(hd.x & 0xFFFF)), dmin = fk_h2f((uint16_t)(hd.x >> 16));
                    int sc0, m0, sc1, m1;
                    q4k_scale_min(hd.y, hd.z, hd.w, 2 * g, &sc0, &m0);
                    q4k_scale_min(hd.y, hd.z, hd.w, 2 * g + 1, &sc1, &m1);
                    f_lo[r] = d * (float)sc0;
                    f_hi[r] = d * (float)sc1;
                    // the two lanes sharing a sub-block (h = 0, 1) each carry half its min term
                    mm_lo[r] = 0.5f * dmin * (float)m0;
                    mm_hi[r] = 0.5f * dmin * (float)m1;
                }
#pragma unroll
                for (int b = 0; b < NB; b++) {
                    const int8_t* q8 = sq + (size_t)b * cols + sbs * 256 + 64 * g + 16 * h;
                    const int4 ua = *(const int4*)q8, ub = *(const int4*)(q8 + 32);
                    const float2 d8 = *(const float2*)(sd + b * nb32 + sbs * 8 + 2 * g);
                    const float2 s8 = *(const float2*)(ss + b * nb32 + sbs * 8 + 2 * g);
#pragma unroll
                    for (int r = 0; r < R; r++) {
                        uint4 lo, hi;
                        lo.x = wq[r].x & 0x0F0F0F0Fu; hi.x = (wq[r].x >> 4) & 0x0F0F0F0Fu;
                        lo.y = wq[r].y & 0x0F0F0F0Fu; hi.y = (wq[r].y >> 4) & 0x0F0F0F0Fu;
                        lo.z = wq[r].z & 0x0F0F0F0Fu; hi.z = (wq[r].z >> 4) & 0x0F0F0F0Fu;
                        lo.w = wq[r].w & 0x0F0F0F0Fu; hi.w = (wq[r].w >> 4) & 0x0F0F0F0Fu;
                        int il = dp4a4(lo, ua), ih = dp4a4(hi, ub);
                        acc[r][b] += f_lo[r] * d8.x * (float)il + f_hi[r] * d8.y * (float)ih -
                                     (mm_lo[r] * s8.x + mm_hi[r] * s8.y);
                        if (DUMP && b == 0) {
                            il += __shfl_xor_sync(0xffffffffu, il, 1);
                            ih += __shfl_xor_sync(0xffffffffu, ih, 1);
                            if (live && h == 0 && row0 + r < rows) {
                                int32_t* o = a.isums + (size_t)(row0 + r) * nb32 + sb * 8 + 2 * g;
                                o[0] = il;
                                o[1] = ih;
                            }
                        }
                    }
                }
            }
        } else if (KIND == FK_Q8_0) {
            const uint8_t* qsp = wb + a.plane_off[0];
            const uint16_t* dp = (const uint16_t*)(wb + a.plane_off[1]);
            const int nchunk = cols >> 4;
            for (int c0 = 0; c0 < nchunk; c0 += 32) {
                const int ci = c0 + lane;
                const bool live = ci < nchunk;
                const int cs = live ? ci : 0;
                uint4 wq[R];
                float dw[R];
#pragma unroll
                for (int r = 0; r < R; r++) {
                    wq[r] = make_uint4(0, 0, 0, 0);
                    dw[r] = 0.0f;
                    if (live && row0 + r < rows) {
                        wq[r] = ldg16(qsp + (size_t)(row0 + r) * cols + (size_t)ci * 16);
                        dw[r] = fk_h2f(__ldg(dp + (size_t)(row0 + r) * nb32 + (ci >> 1)));
                    }
                }
#pragma unroll
                for (int b = 0; b < NB; b++) {
                    const int4 ua = *(const int4*)(sq + (size_t)b * cols + cs * 16);
                    const float d8 = sd[b * nb32 + (cs >> 1)];
#pragma unroll
                    for (int r = 0; r < R; r++) {
                        int is = dp4a4(wq[r], ua);
                        acc[r][b] += dw[r] * d8 * (float)is;
                        if (DUMP && b == 0) {
                            is += __shfl_xor_sync(0xffffffffu, is, 1);
                            if (live && !(lane & 1) && row0 + r < rows)
                                a.isums[(size_t)(row0 + r) * nb32 + (ci >> 1)] = is;
                        }
                    }
                }
            }
        } else if (KIND == FK_Q6_K) {
            const uint8_t* qlp = wb + a.plane_off[0];
            const uint8_t* qhp = wb + a.plane_off[1];
            const int8_t* scp = (const int8_t*)(wb + a.plane_off[2]);
            const uint16_t* dp = (const uint16_t*)(wb + a.plane_off[3]);
            const int nsb = cols >> 8;
            const int c = lane & 7, hf = c >> 2, q = c & 3;
            const int g_lo = 8 * hf + q, g_hi = g_lo + 4;
            const int shift = 2 * (q >> 1);
            for (int sb0 = 0; sb0 < nsb; sb0 += 4) {
                const int sb = sb0 + (lane >> 3);
                const bool live = sb < nsb;
                const int sbs = live ? sb : 0;
                uint4 vl[R], vh[R];
                float f_lo[R], f_hi[R];
#pragma unroll
                for (int r = 0; r < R; r++) {
                    uint4 ql = make_uint4(0, 0, 0, 0), qh = ql;
                    f_lo[r] = 0.0f;
                    f_hi[r] = 0.0f;
                    if (live && row0 + r < rows) {
                        const size_t row = (size_t)(row0 + r);
                        ql = ldg16(qlp + row * (cols >> 1) + (size_t)sb * 128 + 16 * c);
                        qh = ldg16(qhp + row * (cols >> 2) + (size_t)sb * 64 + 32 * hf + 16 * (q & 1));
                        const int8_t* sc = scp + row * (cols >> 4) + sb * 16;
                        const float d = fk_h2f(__ldg(dp + row * nsb + sb));
                        f_lo[r] = d * (float)__ldg(sc + g_lo);
                        f_hi[r] = d * (float)__ldg(sc + g_hi);
                    }
                    vl[r].x = (ql.x & 0x0F0F0F0Fu) | (((qh.x >> shift) & 0x03030303u) << 4);
                    vl[r].y = (ql.y & 0x0F0F0F0Fu) | (((qh.y >> shift) & 0x03030303u) << 4);
                    vl[r].z = (ql.z & 0x0F0F0F0Fu) | (((qh.z >> shift) & 0x03030303u) << 4);
                    vl[r].w = (ql.w & 0x0F0F0F0Fu) | (((qh.w >> shift) & 0x03030303u) << 4);
                    vh[r].x = ((ql.x >> 4) & 0x0F0F0F0Fu) | (((qh.x >> (shift + 4)) & 0x03030303u) << 4);
                    vh[r].y = ((ql.y >> 4) & 0x0F0F0F0Fu) | (((qh.y >> (shift + 4)) & 0x03030303u) << 4);
                    vh[r].z = ((ql.z >> 4) & 0x0F0F0F0Fu) | (((qh.z >> (shift + 4)) & 0x03030303u) << 4);
                    vh[r].w = ((ql.w >> 4) & 0x0F0F0F0Fu) | (((qh.w >> (shift + 4)) & 0x03030303u) << 4);
                }
#pragma unroll
                for (int b = 0; b < NB; b++) {
                    const int8_t* q8 = sq + (size_t)b * cols + sbs * 256;
                    const int4 ua = *(const int4*)(q8 + 16 * g_lo), ub = *(const int4*)(q8 + 16 * g_hi);
                    const float d8lo = sd[b * nb32 + sbs * 8 + (g_lo >> 1)], d8hi = sd[b * nb32 + sbs * 8 + (g_hi >> 1)];
                    const int s_lo = sb16[b * (cols >> 4) + sbs * 16 + g_lo], s_hi = sb16[b * (cols >> 4) + sbs * 16 + g_hi];
#pragma unroll
                    for (int r = 0; r < R; r++) {
                        // codes are stored +32: sum((c - 32) * u) = sum(c * u) - 32 * sum(u)
                        const int il = dp4a4(vl[r], ua) - 32 * s_lo;
                        const int ih = dp4a4(vh[r], ub) - 32 * s_hi;
                        acc[r][b] += f_lo[r] * d8lo * (float)il + f_hi[r] * d8hi * (float)ih;
                        if (DUMP && b == 0 && live && row0 + r < rows) {
                            int32_t* o = a.isums + (size_t)(row0 + r) * (cols >> 4) + sb * 16;
                            o[g_lo] = il;
                            o[g_hi] = ih;
                        }
                    }
                }
            }
        } else {  // FK_MXFP4
            const uint8_t* cp = wb + a.plane_off[0];
            const uint8_t* ep = wb + a.plane_off[1];
            for (int k0 = 0; k0 < nb32; k0 += 32) {
                const int kb = k0 + lane;
                const bool live = kb < nb32;
                const int ks = live ? kb : 0;
                uint4 va[R], vb[R];
                float dw[R];
#pragma unroll
                for (int r = 0; r < R; r++) {
                    uint4 wq = make_uint4(0, 0, 0, 0);
                    dw[r] = 0.0f;
                    if (live && row0 + r < rows) {
                        wq = ldg16(cp + (size_t)(row0 + r) * (cols >> 1) + (size_t)kb * 16);
                        dw[r] = e8m0_half(__ldg(ep + (size_t)(row0 + r) * nb32 + kb));
                    }
                    va[r].x = e2m1x2_4(wq.x); va[r].y = e2m1x2_4(wq.x >> 16);
                    va[r].z = e2m1x2_4(wq.y); va[r].w = e2m1x2_4(wq.y >> 16);
                    vb[r].x = e2m1x2_4(wq.z); vb[r].y = e2m1x2_4(wq.z >> 16);
                    vb[r].z = e2m1x2_4(wq.w); vb[r].w = e2m1x2_4(wq.w >> 16);
                }
#pragma unroll
                for (int b = 0; b < NB; b++) {
                    const int8_t* q8 = sq + (size_t)b * cols + ks * 32;
                    const int4 ua = *(const int4*)q8, ub = *(const int4*)(q8 + 16);
                    const float d8 = sd[b * nb32 + ks];
#pragma unroll
                    for (int r = 0; r < R; r++) {
                        const int is = dp4a4(va[r], ua) + dp4a4(vb[r], ub);
                        acc[r][b] += dw[r] * d8 * (float)is;
                        if (DUMP && b == 0 && live && row0 + r < rows)
                            a.isums[(size_t)(row0 + r) * nb32 + kb] = is;
                    }
                }
            }
        }

#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int b = 0; b < NB; b++) {
                const float s = fk_warp_sum(acc[r][b]);
                if (lane == 0 && row0 + r < rows && b < a.batch) y[(size_t)b * rows + row0 + r] = s;
            }
    }
}

size_t gemv_smem_bytes(int kind, int nb, int cols) {
    size_t s = (size_t)nb * cols + (size_t)nb * (cols / 32) * 4;
    if (kind == FK_Q4_K) s += (size_t)nb * (cols / 32) * 4;
    if (kind == FK_Q6_K) s += (size_t)nb * (cols / 16) * 4;
    return s;
}

template <int KIND, int NB, bool DUMP>
int launch_one(fk_ctx* ctx, cudaStream_t st, const GemvArgs& a, int slots) {
    const size_t smem = gemv_smem_bytes(KIND, NB, a.cols);
    if (smem > 220 * 1024) return fk_fail(FK_UNSUPPORTED, "gemv: %d columns x batch %d needs %zu B of shared memory", a.cols, NB, smem);
    auto kern = gemv_kernel<KIND, NB, DUMP>;
    if (smem > 48 * 1024) FK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), FK_KERNEL);
    const int pairs = (a.rows + R - 1) / R;
    const int need = (pairs + GEMV_WARPS - 1) / GEMV_WARPS;
    int per_slot = (2 * ctx->sm_count + slots - 1) / slots;
    if (per_slot < 1) per_slot = 1;
    dim3 grid((unsigned)(need < per_slot ? need : per_slot), (unsigned)slots);
    kern<<<grid, GEMV_THREADS, smem, st>>>(a);
    FK_CUDA(cudaGetLastError(), FK_LAUNCH);
    ctx->launches++;
    return FK_OK;
}

template <int KIND>
int launch_kind(fk_ctx* ctx, cudaStream_t st, const GemvArgs& a, int slots, bool dump) {
    if (dump) return launch_one<KIND, 1, true>(ctx, st, a, slots);
    if (a.batch <= 1) return launch_one<KIND, 1, false>(ctx, st, a, slots);
    if (a.batch <= 2) return launch_one<KIND, 2, false>(ctx, st, a, slots);
    if (a.batch <= 4) return launch_one<KIND, 4, false>(ctx, st, a, slots);
    return launch_one<KIND, 8, false>(ctx, st, a, slots);
}

// ---- standalone q8_1 quantizer (36-byte blocks), one warp per run
__global__ void quantize_q8_1_kernel(const float* __restrict__ x, int n_runs, uint8_t* __restrict__ y) {
    const int run = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (run >= n_runs) return;
    const float v = x[(size_t)run * 32 + lane];
    float d_w;
    int qsum;
    const int q = fk_q8_1_lane(v, &d_w, &qsum);
    const float sum = fk_warp_sum(v);  // xor butterfly 16..1, the order the stored sum is defined by
    uint8_t* blk = y + (size_t)run * 36;
    blk[4 + lane] = (uint8_t)(int8_t)q;
    if (lane == 0) {
        *(uint16_t*)blk = fk_f2h(d_w);  // d_w is the f16 scale widened: the conversion back is exact
        *(uint16_t*)(blk + 2) = fk_f2h(sum);
    }
}

}  // namespace

int fk_gemv_launch(fk_ctx* ctx, cudaStream_t st, fk_weight w, const int* ids_dev, int mat, int slots,
                   const float* x_dev, int x_stride, int batch, float* y_dev, int32_t* isums_dev) {
    GemvArgs a;
    a.w = w->dev;
    a.mat_stride = w->mat_stride;
    for (int i = 0; i < 4; i++) a.plane_off[i] = w->plane_off[i];
    a.ids = ids_dev;
    a.mat = mat;
    a.x = x_dev;
    a.x_stride = x_stride;
    a.y = y_dev;
    a.rows = w->rows;
    a.cols = w->cols;
    a.batch = batch;
    a.isums = isums_dev;
    const bool dump = isums_dev != nullptr;
    switch (w->kind) {
        case FK_Q4_K: return launch_kind<FK_Q4_K>(ctx, st, a, slots, dump);
        case FK_Q6_K: return launch_kind<FK_Q6_K>(ctx, st, a, slots, dump);
        case FK_Q8_0: return launch_kind<FK_Q8_0>(ctx, st, a, slots, dump);
        case FK_MXFP4: return launch_kind<FK_MXFP4>(ctx, st, a, slots, dump);
    }
    return fk_fail(FK_UNSUPPORTED, "gemv: kind %d has no kernel", w->kind);
}

FK_EXPORT int fk_quantize_q8_1(fk_ctx* ctx, void* stream, const float* x_dev, int n, uint8_t* y_dev) {
    if (!ctx || !x_dev || !y_dev || n < 0 || n % 32) return fk_fail(FK_INVALID, "quantize_q8_1: n=%d must be a multiple of 32", n);
    if (n == 0) return FK_OK;
    FkDeviceGuard g(ctx->device);
    const int runs = n / 32;
    quantize_q8_1_kernel<<<(runs + 7) / 8, 256, 0, (cudaStream_t)stream>>>(x_dev, runs, y_dev);
    FK_CUDA(cudaGetLastError(), FK_LAUNCH);
    ctx->launches++;
    return FK_OK;
}

FK_EXPORT int fk_gemv(fk_ctx* ctx, void* stream, fk_weight w, int mat, const float* x_dev, int batch, float* y_dev) {
    if (!ctx || !w || !x_dev || !y_dev) return fk_fail(FK_INVALID, "gemv: null argument");
    if (batch < 1 || batch > 8) return fk_fail(FK_UNSUPPORTED, "gemv: batch %d outside 1..8 (use fk_gemm)", batch);
    if (mat < 0 || mat >= w->n_mats) return fk_fail(FK_INVALID, "gemv: matrix %d of %d", mat, w->n_mats);
    FkDeviceGuard g(ctx->device);
    return fk_gemv_launch(ctx, (cudaStream_t)stream, w, nullptr, mat, 1, x_dev, 0, batch, y_dev, nullptr);
}

FK_EXPORT int fk_gemv_multi(fk_ctx* ctx, void* stream, fk_weight w, const int* ids_dev, int k, const float* x_dev,
                            int x_stride, float* y_dev) {
    if (!ctx || !w || !ids_dev || !x_dev || !y_dev) return fk_fail(FK_INVALID, "gemv_multi: null argument");
    if (k < 1 || k > 65535) return fk_fail(FK_INVALID, "gemv_multi: k=%d", k);
    if (x_stride != 0 && x_stride < w->cols) return fk_fail(FK_INVALID, "gemv_multi: x_stride %d < cols %d", x_stride, w->cols);
    FkDeviceGuard g(ctx->device);
    return fk_gemv_launch(ctx, (cudaStream_t)stream, w, ids_dev, 0, k, x_dev, x_stride, 1, y_dev, nullptr);
}

FK_EXPORT int fk_gemv_isums(fk_ctx* ctx, void* stream, fk_weight w, int mat, const float* x_dev, int32_t* isums_dev) {
    if (!ctx || !w || !x_dev || !isums_dev) return fk_fail(FK_INVALID, "gemv_isums: null argument");
    if (mat < 0 || mat >= w->n_mats) return fk_fail(FK_INVALID, "gemv_isums: matrix %d of %d", mat, w->n_mats);
    FkDeviceGuard g(ctx->device);
    // y is not wanted: park it in the context's scratch
    int rc = fk_ensure_scratch(ctx, (size_t)w->rows * sizeof(float));
    if (rc) return rc;
    return fk_gemv_launch(ctx, (cudaStream_t)stream, w, nullptr, mat, 1, x_dev, 0, 1, (float*)ctx->scratch, isums_dev);
}
