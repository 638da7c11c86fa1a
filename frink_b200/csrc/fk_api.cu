// Context, resident weights (upload + de-interleave), and the host-buffer
// launch surface of the C ABI.
#include "fk_common.cuh"

#include <string.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>

// ------------------------------------------------------------------ errors
static thread_local char g_err[512] = "";

void fk_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}
int fk_fail(int status, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return status;
}
FK_EXPORT const char* fk_last_error(void) { return g_err; }
FK_EXPORT int fk_block_bytes(int kind) { return fk_kind_block_bytes(kind); }
FK_EXPORT int fk_block_elems(int kind) { return fk_kind_block_elems(kind); }

// ----------------------------------------------------------------- context
FK_EXPORT int fk_init(int device, fk_ctx** out) {
    if (!out) return fk_fail(FK_INVALID, "init: null out");
    *out = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) return fk_fail(FK_DRIVER_INIT, "no usable CUDA driver: %s", cudaGetErrorString(e));
    if (device < 0 || device >= n) return fk_fail(FK_DRIVER_INIT, "device %d of %d", device, n);
    cudaDeviceProp prop;
    FK_CUDA(cudaGetDeviceProperties(&prop, device), FK_DRIVER_INIT);
    if (prop.major != 10)
        return fk_fail(FK_UNSUPPORTED, "device %d is sm_%d%d; this library holds sm_100a code only", device, prop.major, prop.minor);
    fk_ctx* ctx = new (std::nothrow) fk_ctx();
    if (!ctx) return fk_fail(FK_DRIVER_INIT, "out of host memory");
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->mem_bytes = prop.totalGlobalMem;
    snprintf(ctx->name, sizeof(ctx->name), "%s", prop.name);
    FkDeviceGuard g(device);
    e = cudaMalloc(&ctx->err_flag, 16);
    if (e == cudaSuccess) e = cudaMemset(ctx->err_flag, 0, 16);
    if (e == cudaSuccess) e = cudaHostAlloc((void**)&ctx->err_pin, sizeof(int), cudaHostAllocMapped);
    if (e == cudaSuccess) {
        *ctx->err_pin = 0;
        int* mirror_dev = nullptr;
        e = cudaHostGetDevicePointer((void**)&mirror_dev, ctx->err_pin, 0);
        if (e == cudaSuccess) e = cudaMemcpy((char*)ctx->err_flag + 8, &mirror_dev, sizeof(mirror_dev), cudaMemcpyHostToDevice);
    }
    if (e == cudaSuccess) e = cudaMalloc(&ctx->argmax_ws, 64 * 64 * sizeof(unsigned long long));
    // 64 counters of the argmax rows, then (index 64) the arrival counter of the fused router
    if (e == cudaSuccess) e = cudaMalloc(&ctx->argmax_cnt, 128 * sizeof(unsigned));
    if (e == cudaSuccess) e = cudaMemset(ctx->argmax_cnt, 0, 128 * sizeof(unsigned));
    if (e == cudaSuccess) e = cudaMalloc(&ctx->attn_cnt, 4096 * sizeof(unsigned));
    if (e == cudaSuccess) e = cudaMemset(ctx->attn_cnt, 0, 4096 * sizeof(unsigned));
    if (e != cudaSuccess) {
        delete ctx;
        return fk_fail(FK_DRIVER_INIT, "context allocation: %s", cudaGetErrorString(e));
    }
    *out = ctx;
    return FK_OK;
}

FK_EXPORT void fk_destroy(fk_ctx* ctx) {
    if (!ctx) return;
    FkDeviceGuard g(ctx->device);
    fk_forget_resident(ctx);
    cudaFree(ctx->x_dev);
    cudaFree(ctx->y_dev);
    if (ctx->x_pin) cudaFreeHost(ctx->x_pin);
    if (ctx->y_pin) cudaFreeHost(ctx->y_pin);
    cudaFree(ctx->scratch);
    for (uint8_t* p : ctx->scratch_retired) cudaFree(p);
    cudaFree(ctx->err_flag);
    if (ctx->err_pin) cudaFreeHost(ctx->err_pin);
    cudaFree(ctx->argmax_ws);
    cudaFree(ctx->argmax_cnt);
    cudaFree(ctx->attn_cnt);
    delete ctx;
}

FK_EXPORT int fk_device_info(fk_ctx* ctx, char* name, size_t cap, int* sm_count, size_t* mem_bytes) {
    if (!ctx) return fk_fail(FK_INVALID, "device_info: null context");
    if (name && cap) snprintf(name, cap, "%s", ctx->name);
    if (sm_count) *sm_count = ctx->sm_count;
    if (mem_bytes) *mem_bytes = ctx->mem_bytes;
    return FK_OK;
}

FK_EXPORT int fk_counters(fk_ctx* ctx, uint64_t* h2d, uint64_t* d2h, uint64_t* launches, int reset) {
    if (!ctx) return fk_fail(FK_INVALID, "counters: null context");
    if (h2d) *h2d = ctx->h2d.load();
    if (d2h) *d2h = ctx->d2h.load();
    if (launches) *launches = ctx->launches.load();
    if (reset) { ctx->h2d = 0; ctx->d2h = 0; ctx->launches = 0; }
    return FK_OK;
}

// The workspace only grows, and a block that was ever handed out is kept until fk_destroy: its address is inside
// launches that may still be queued, and inside CUDA graphs that may be replayed at any later time.  Growth allocates,
// which a stream capture does not allow: a call that needs more than is reserved while `st` is being captured fails
// with FK_INVALID (reserve with fk_reserve_scratch before capturing).
int fk_ensure_scratch(fk_ctx* ctx, cudaStream_t st, size_t bytes) {
    std::lock_guard<std::recursive_mutex> lk(ctx->mu);
    if (bytes <= ctx->scratch_cap) return FK_OK;
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cs) == cudaSuccess && cs != cudaStreamCaptureStatusNone)
        return fk_fail(FK_INVALID, "the workspace has %zu bytes and this call needs %zu: it cannot grow inside a stream capture (fk_reserve_scratch first)",
                       ctx->scratch_cap, bytes);
    size_t cap = bytes + (bytes >> 1) + 4096;
    if (cap < FK_SCRATCH_MIN) cap = FK_SCRATCH_MIN;
    uint8_t* p = nullptr;
    FK_CUDA(cudaMalloc(&p, cap), FK_LAUNCH);
    if (ctx->scratch) ctx->scratch_retired.push_back(ctx->scratch);
    ctx->scratch = p;
    ctx->scratch_cap = cap;
    return FK_OK;
}

FK_EXPORT int fk_reserve_scratch(fk_ctx* ctx, size_t bytes) {
    if (!ctx) return fk_fail(FK_INVALID, "reserve_scratch: null context");
    FkDeviceGuard g(ctx->device);
    return fk_ensure_scratch(ctx, nullptr, bytes);
}

// ------------------------------------------------------- weight registration
namespace {
size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

// GGUF blocks -> planes (layouts in fk_common.cuh).  One thread per block; run
// once per tensor.
__global__ void split_q8_0(const uint8_t* __restrict__ src, size_t n_blocks, int bpr, int8_t* __restrict__ qs, size_t qs_stride,
                           uint8_t* __restrict__ d, size_t d_stride) {
    const size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    const size_t row = b / bpr, i0 = b % bpr;
    const uint8_t* s = src + b * 34;
    *(uint16_t*)(d + row * d_stride + i0 * 2) = (uint16_t)(s[0] | (s[1] << 8));
    int8_t* q = qs + row * qs_stride + i0 * 32;
    for (int i = 0; i < 32; i++) q[i] = (int8_t)s[2 + i];
}
__global__ void split_q6_k(const uint8_t* __restrict__ src, size_t n_blocks, int bpr, uint8_t* __restrict__ ql, size_t ql_stride,
                           uint8_t* __restrict__ qh, size_t qh_stride, uint8_t* __restrict__ sc, size_t sc_stride,
                           uint8_t* __restrict__ d, size_t d_stride) {
    const size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    const size_t row = b / bpr, i0 = b % bpr;
    const uint8_t* s = src + b * 210;
    for (int i = 0; i < 128; i++) ql[row * ql_stride + i0 * 128 + i] = s[i];
    for (int i = 0; i < 64; i++) qh[row * qh_stride + i0 * 64 + i] = s[128 + i];
    for (int i = 0; i < 16; i++) sc[row * sc_stride + i0 * 16 + i] = s[192 + i];
    *(uint16_t*)(d + row * d_stride + i0 * 2) = (uint16_t)(s[208] | (s[209] << 8));
}
__global__ void split_mxfp4(const uint8_t* __restrict__ src, size_t n_blocks, int bpr, uint8_t* __restrict__ codes, size_t c_stride,
                            uint8_t* __restrict__ e, size_t e_stride) {
    const size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    const size_t row = b / bpr, i0 = b % bpr;
    const uint8_t* s = src + b * 17;
    e[row * e_stride + i0] = s[0];
    for (int i = 0; i < 16; i++) codes[row * c_stride + i0 * 16 + i] = s[1 + i];
}

int make_weight(fk_ctx* ctx, const uint8_t* raw_dev, size_t len, int kind, int n_mats, int rows, int cols,
                cudaStream_t st, fk_weight* out) {
    const int bb = fk_kind_block_bytes(kind), be = fk_kind_block_elems(kind);
    fk_weight w = new (std::nothrow) fk_weight_s();
    if (!w) return fk_fail(FK_LAUNCH, "out of host memory");
    w->kind = kind;
    w->n_mats = n_mats;
    w->rows = rows;
    w->cols = cols;
    w->gguf_row_bytes = (size_t)(cols / be) * bb;
    w->gguf_bytes = len;
    w->device = ctx->device;
    const size_t n = (size_t)rows * cols;
    auto pad16 = [](size_t v) { return (v + 15) & ~(size_t)15; };
    size_t stride[4] = {0, 0, 0, 0};
    const size_t c = (size_t)cols;
    switch (kind) {
        case FK_Q4_K: case FK_Q5_K: case FK_BF16: stride[0] = w->gguf_row_bytes; break;
        case FK_Q8_0: stride[0] = c; stride[1] = pad16(c / 16); break;
        case FK_Q6_K: stride[0] = c / 2; stride[1] = c / 4; stride[2] = c / 16; stride[3] = pad16(c / 256 * 2); break;
        case FK_MXFP4: stride[0] = c / 2; stride[1] = pad16(c / 32); break;
    }
    size_t off = 0;
    for (int i = 0; i < 4; i++) {
        w->plane_off[i] = off;
        w->plane_stride[i] = stride[i];
        off += align256((size_t)rows * stride[i]) + (stride[i] ? 256 : 0);   // slack: rounded-up copies may read past the last row
    }
    w->mat_stride = off;
    cudaError_t e = cudaMalloc(&w->dev, (size_t)n_mats * w->mat_stride);
    if (e != cudaSuccess) {
        delete w;
        return fk_fail(FK_LAUNCH, "weights: cudaMalloc of %zu bytes: %s", (size_t)n_mats * off, cudaGetErrorString(e));
    }
    const size_t mat_raw = (size_t)rows * w->gguf_row_bytes;
    const size_t blocks = n / be;
    const int bpr = cols / be;
    const unsigned grid = (unsigned)((blocks + 255) / 256);
    e = cudaMemsetAsync(w->dev, 0, (size_t)n_mats * w->mat_stride, st);   // row padding of the scale planes reads as zeros
    for (int m = 0; m < n_mats && e == cudaSuccess; m++) {
        const uint8_t* src = raw_dev + (size_t)m * mat_raw;
        uint8_t* dst = w->dev + (size_t)m * w->mat_stride;
        switch (kind) {
            case FK_Q4_K: case FK_Q5_K: case FK_BF16:
                e = cudaMemcpyAsync(dst, src, mat_raw, cudaMemcpyDeviceToDevice, st);
                break;
            case FK_Q8_0:
                split_q8_0<<<grid, 256, 0, st>>>(src, blocks, bpr, (int8_t*)(dst + w->plane_off[0]), w->plane_stride[0],
                                                 dst + w->plane_off[1], w->plane_stride[1]);
                break;
            case FK_Q6_K:
                split_q6_k<<<grid, 256, 0, st>>>(src, blocks, bpr, dst + w->plane_off[0], w->plane_stride[0], dst + w->plane_off[1],
                                                 w->plane_stride[1], dst + w->plane_off[2], w->plane_stride[2], dst + w->plane_off[3],
                                                 w->plane_stride[3]);
                break;
            case FK_MXFP4:
                split_mxfp4<<<grid, 256, 0, st>>>(src, blocks, bpr, dst + w->plane_off[0], w->plane_stride[0], dst + w->plane_off[1],
                                                  w->plane_stride[1]);
                break;
        }
        if (e == cudaSuccess) e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) {
        cudaFree(w->dev);
        delete w;
        return fk_fail(FK_LAUNCH, "weights: de-interleave failed: %s", cudaGetErrorString(e));
    }
    *out = w;
    return FK_OK;
}

int check_shape(const char* who, size_t len, int kind, int n_mats, int rows, int cols) {
    const int bb = fk_kind_block_bytes(kind), be = fk_kind_block_elems(kind);
    if (bb < 0) return fk_fail(FK_UNSUPPORTED, "%s: kind %d is not one of Q8_0, Q4_K, Q5_K, Q6_K, MXFP4, BF16", who, kind);
    if (n_mats < 1 || rows < 1 || cols < 1) return fk_fail(FK_INVALID, "%s: %d matrices of %d x %d", who, n_mats, rows, cols);
    if (cols % be) return fk_fail(FK_INVALID, "%s: %d columns is not a whole number of %d-element blocks", who, cols, be);
    if (cols % 32) return fk_fail(FK_INVALID, "%s: %d columns is not a whole number of q8_1 runs", who, cols);
    const size_t want = (size_t)n_mats * rows * (size_t)(cols / be) * bb;
    if (len != want) return fk_fail(FK_INVALID, "%s: %zu bytes given, shape needs %zu", who, len, want);
    return FK_OK;
}
}  // namespace

FK_EXPORT int fk_register_weights_dev(fk_ctx* ctx, const uint8_t* gguf_bytes_dev, size_t len, int kind, int n_mats,
                                      int rows, int cols, void* stream, fk_weight* out) {
    if (!ctx || !gguf_bytes_dev || !out) return fk_fail(FK_INVALID, "register_weights_dev: null argument");
    int rc = check_shape("register_weights_dev", len, kind, n_mats, rows, cols);
    if (rc) return rc;
    FkDeviceGuard g(ctx->device);
    return make_weight(ctx, gguf_bytes_dev, len, kind, n_mats, rows, cols, (cudaStream_t)stream, out);
}

FK_EXPORT int fk_register_weights(fk_ctx* ctx, const uint8_t* gguf_bytes_host, size_t len, int kind, int n_mats,
                                  int rows, int cols, fk_weight* out) {
    if (!ctx || !gguf_bytes_host || !out) return fk_fail(FK_INVALID, "register_weights: null argument");
    int rc = check_shape("register_weights", len, kind, n_mats, rows, cols);
    if (rc) return rc;
    FkDeviceGuard g(ctx->device);
    uint8_t* raw = nullptr;
    FK_CUDA(cudaMalloc(&raw, len), FK_LAUNCH);
    cudaError_t e = cudaMemcpy(raw, gguf_bytes_host, len, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        cudaFree(raw);
        return fk_fail(FK_LAUNCH, "register_weights: upload: %s", cudaGetErrorString(e));
    }
    ctx->h2d += len;
    rc = make_weight(ctx, raw, len, kind, n_mats, rows, cols, nullptr, out);
    cudaFree(raw);
    return rc;
}

FK_EXPORT int fk_release_weights(fk_ctx* ctx, fk_weight w) {
    if (!ctx || !w) return fk_fail(FK_INVALID, "release_weights: null argument");
    FkDeviceGuard g(ctx->device);
    cudaFree(w->dev);
    delete w;
    return FK_OK;
}

FK_EXPORT int fk_weight_shape(fk_weight w, int* kind, int* n_mats, int* rows, int* cols, size_t* gguf_bytes) {
    if (!w) return fk_fail(FK_INVALID, "weight_shape: null weight");
    if (kind) *kind = w->kind;
    if (n_mats) *n_mats = w->n_mats;
    if (rows) *rows = w->rows;
    if (cols) *cols = w->cols;
    if (gguf_bytes) *gguf_bytes = w->gguf_bytes;
    return FK_OK;
}

// ------------------------------------------------ host-buffer launch surface
namespace {
// 64 eight-byte samples spread over the buffer, folded with its length: cheap
// enough for every call, and a remapped file at the same address fails it.
uint64_t fingerprint(const uint8_t* p, size_t len) {
    uint64_t h = 0xcbf29ce484222325ull ^ len;
    const size_t n = 64;
    for (size_t i = 0; i < n; i++) {
        size_t off = len > 8 ? (size_t)((long double)(len - 8) * i / (n - 1)) : 0;
        uint64_t v = 0;
        memcpy(&v, p + off, len >= 8 ? 8 : len);
        h = (h ^ v) * 0x100000001b3ull;
    }
    return h;
}

int resident(fk_ctx* ctx, int kind, const uint8_t* host, size_t len, int rows, int cols, fk_weight* out) {
    const uint64_t fp = fingerprint(host, len);
    {
        std::lock_guard<std::recursive_mutex> lk(ctx->mu);
        auto it = ctx->resident.find({host, len});
        if (it != ctx->resident.end()) {
            fk_weight w = it->second.second;
            if (it->second.first == fp && w->kind == kind && w->rows == rows && w->cols == cols) {
                *out = w;
                return FK_OK;
            }
            fk_release_weights(ctx, w);
            ctx->resident.erase(it);
        }
    }
    fk_weight w = nullptr;
    int rc = fk_register_weights(ctx, host, len, kind, 1, rows, cols, &w);
    if (rc) return rc;
    std::lock_guard<std::recursive_mutex> lk(ctx->mu);
    ctx->resident[{host, len}] = {fp, w};
    *out = w;
    return FK_OK;
}

int grow(float** p, size_t* cap, size_t floats) {
    if (floats <= *cap) return FK_OK;
    if (*p) cudaFree(*p);
    *p = nullptr;
    *cap = 0;
    FK_CUDA(cudaMalloc(p, floats * sizeof(float)), FK_LAUNCH);
    *cap = floats;
    return FK_OK;
}
int grow_pinned(float** p, float** dev_alias, size_t* cap, size_t floats, bool mapped) {
    if (floats <= *cap) return FK_OK;
    if (*p) cudaFreeHost(*p);
    *p = nullptr;
    *cap = 0;
    FK_CUDA(cudaHostAlloc((void**)p, floats * sizeof(float), mapped ? cudaHostAllocMapped : cudaHostAllocDefault), FK_LAUNCH);
    if (dev_alias) FK_CUDA(cudaHostGetDevicePointer((void**)dev_alias, *p, 0), FK_LAUNCH);
    *cap = floats;
    return FK_OK;
}

// The end of a host-buffer call: one synchronize, then the error word's host mirror.  A kernel that gave up a bounded wait (or refused a cache overrun) left a code there: the
// results are garbage and the call says so (frink-core's contract: `Err` -> fall back, weight_matrix.rs:3454-3493).
int finish_host_call(fk_ctx* ctx, const char* what) {
    FK_CUDA(cudaStreamSynchronize(nullptr), FK_LAUNCH);
    const int code = *(volatile int*)ctx->err_pin;      // written by the kernel that raised (fk_raise), visible after the synchronize
    if (code) {
        cudaMemset(ctx->err_flag, 0, sizeof(int));
        *ctx->err_pin = 0;
        return fk_fail(FK_LAUNCH, "%s: a kernel gave up a bounded wait (device error word %d); the result is not valid", what, code);
    }
    return FK_OK;
}
}  // namespace

FK_EXPORT int fk_forget_resident(fk_ctx* ctx) {
    if (!ctx) return fk_fail(FK_INVALID, "forget_resident: null context");
    std::lock_guard<std::recursive_mutex> lk(ctx->mu);
    FkDeviceGuard g(ctx->device);
    for (auto& kv : ctx->resident) {
        cudaFree(kv.second.second->dev);
        delete kv.second.second;
    }
    ctx->resident.clear();
    return FK_OK;
}

FK_EXPORT int fk_launch_mul_mm(fk_ctx* ctx, int kind, const uint8_t* weights_host, size_t len, const float* x_batch_host,
                               int n_rows, int n_cols, int batch, int row_bytes, float* out_host) {
    if (!ctx || !weights_host || !x_batch_host || !out_host) return fk_fail(FK_INVALID, "launch: null argument");
    const int bb = fk_kind_block_bytes(kind), be = fk_kind_block_elems(kind);
    if (bb < 0) return fk_fail(FK_UNSUPPORTED, "launch: kind %d has no kernel here", kind);
    if (batch < 1) return fk_fail(FK_INVALID, "launch: batch %d", batch);
    if (n_cols % be || (size_t)row_bytes != (size_t)(n_cols / be) * bb)
        return fk_fail(FK_INVALID, "launch: row_bytes %d does not match %d columns of kind %d", row_bytes, n_cols, kind);
    FkDeviceGuard g(ctx->device);
    fk_weight w = nullptr;
    int rc = resident(ctx, kind, weights_host, len, n_rows, n_cols, &w);
    if (rc) return rc;
    // one stream (the default one) and one pair of staging buffers: calls from
    // several host threads take turns, as the reference's do on its one stream
    std::lock_guard<std::recursive_mutex> lk(ctx->mu);
    const size_t xn = (size_t)batch * n_cols, yn = (size_t)batch * n_rows;
    if ((rc = grow(&ctx->x_dev, &ctx->x_cap, xn))) return rc;
    if (batch <= 8) {
        // the decode shape: a few KB each way, so the call is all latency.  x goes through a
        // pinned buffer (a truly asynchronous copy), and the kernel writes y straight into
        // mapped host memory, which saves the copy back and its launch.
        if ((rc = grow_pinned(&ctx->x_pin, nullptr, &ctx->x_pin_cap, xn, false))) return rc;
        if ((rc = grow_pinned(&ctx->y_pin, &ctx->y_pin_dev, &ctx->y_pin_cap, yn, true))) return rc;
        memcpy(ctx->x_pin, x_batch_host, xn * sizeof(float));
        FK_CUDA(cudaMemcpyAsync(ctx->x_dev, ctx->x_pin, xn * sizeof(float), cudaMemcpyHostToDevice, nullptr), FK_LAUNCH);
        ctx->h2d += xn * sizeof(float);
        rc = fk_gemv_launch(ctx, nullptr, w, nullptr, 0, 1, ctx->x_dev, 0, batch, ctx->y_pin_dev, nullptr, nullptr, nullptr);
        if (rc) return rc;
        if ((rc = finish_host_call(ctx, "launch"))) return rc;
        memcpy(out_host, ctx->y_pin, yn * sizeof(float));
        ctx->d2h += yn * sizeof(float);
        return FK_OK;
    }
    if ((rc = grow(&ctx->y_dev, &ctx->y_cap, yn))) return rc;
    FK_CUDA(cudaMemcpyAsync(ctx->x_dev, x_batch_host, xn * sizeof(float), cudaMemcpyHostToDevice, nullptr), FK_LAUNCH);
    ctx->h2d += xn * sizeof(float);
    {
        rc = fk_gemm(ctx, nullptr, w, 0, ctx->x_dev, batch, ctx->y_dev);
    }
    if (rc) return rc;
    FK_CUDA(cudaMemcpyAsync(out_host, ctx->y_dev, yn * sizeof(float), cudaMemcpyDeviceToHost, nullptr), FK_LAUNCH);
    if ((rc = finish_host_call(ctx, "launch_mul_mm"))) return rc;
    ctx->d2h += yn * sizeof(float);
    return FK_OK;
}

FK_EXPORT int fk_launch_matvec(fk_ctx* ctx, int kind, const uint8_t* weights_host, size_t len, const float* x_host,
                               int rows, int row_bytes, int n_blocks_per_row, float* y_host) {
    const int be = fk_kind_block_elems(kind);
    if (be < 0) return fk_fail(FK_UNSUPPORTED, "launch_matvec: kind %d has no kernel here", kind);
    return fk_launch_mul_mm(ctx, kind, weights_host, len, x_host, rows, n_blocks_per_row * be, 1, row_bytes, y_host);
}

namespace {
// One launch description of a multi-matvec call, checked and made resident.
int prepare_launch(fk_ctx* ctx, const fk_matvec_launch* l, int n_cols, const char* what, fk_weight* w) {
    if (!l || !l->weights_host) return fk_fail(FK_INVALID, "%s: null launch", what);
    const int bb = fk_kind_block_bytes(l->kind), be = fk_kind_block_elems(l->kind);
    if (bb < 0) return fk_fail(FK_UNSUPPORTED, "%s: kind %d has no kernel here", what, l->kind);
    if (l->rows < 1 || l->n_blocks_per_row < 1 || l->n_blocks_per_row * be != n_cols || (size_t)l->row_bytes != (size_t)l->n_blocks_per_row * bb)
        return fk_fail(FK_INVALID, "%s: %d rows, %d blocks of kind %d per row (%d bytes) against %d columns", what, l->rows, l->n_blocks_per_row, l->kind,
                       l->row_bytes, n_cols);
    return resident(ctx, l->kind, l->weights_host, l->len, l->rows, n_cols, w);
}
}  // namespace

// `gpu::launch_matvec_multi` (crates/frink-cuda/src/matvec_launch.rs:495-536): x goes up once, the n matvecs are
// enqueued back to back on resident weights, every result comes down, one synchronize at the edge.
FK_EXPORT int fk_launch_matvec_multi(fk_ctx* ctx, const float* x_host, int n_cols, const fk_matvec_launch* launches, int n, float* const* y_hosts) {
    if (!ctx || !x_host || (n > 0 && (!launches || !y_hosts))) return fk_fail(FK_INVALID, "launch_matvec_multi: null argument");
    if (n <= 0) return FK_OK;
    if (n > 64 || n_cols < 1) return fk_fail(FK_INVALID, "launch_matvec_multi: %d launches of %d columns", n, n_cols);
    FkDeviceGuard g(ctx->device);
    fk_weight ws[64];
    size_t total = 0;
    for (int i = 0; i < n; i++) {
        const int rc = prepare_launch(ctx, &launches[i], n_cols, "launch_matvec_multi", &ws[i]);
        if (rc) return rc;
        if (!y_hosts[i]) return fk_fail(FK_INVALID, "launch_matvec_multi: null output %d", i);
        total += ((size_t)launches[i].rows + 3) & ~(size_t)3;
    }
    std::lock_guard<std::recursive_mutex> lk(ctx->mu);
    int rc;
    if ((rc = grow(&ctx->x_dev, &ctx->x_cap, (size_t)n_cols))) return rc;
    if ((rc = grow_pinned(&ctx->x_pin, nullptr, &ctx->x_pin_cap, (size_t)n_cols, false))) return rc;
    if ((rc = grow_pinned(&ctx->y_pin, &ctx->y_pin_dev, &ctx->y_pin_cap, total, true))) return rc;
    memcpy(ctx->x_pin, x_host, (size_t)n_cols * sizeof(float));
    FK_CUDA(cudaMemcpyAsync(ctx->x_dev, ctx->x_pin, (size_t)n_cols * sizeof(float), cudaMemcpyHostToDevice, nullptr), FK_LAUNCH);
    ctx->h2d += (size_t)n_cols * sizeof(float);
    size_t off = 0;
    for (int i = 0; i < n; i++) {
        rc = fk_gemv_launch(ctx, nullptr, ws[i], nullptr, 0, 1, ctx->x_dev, 0, 1, ctx->y_pin_dev + off, nullptr, nullptr, nullptr);
        if (rc) return rc;
        off += ((size_t)launches[i].rows + 3) & ~(size_t)3;
    }
    if ((rc = finish_host_call(ctx, "launch_matvec_multi"))) return rc;
    off = 0;
    for (int i = 0; i < n; i++) {
        memcpy(y_hosts[i], ctx->y_pin + off, (size_t)launches[i].rows * sizeof(float));
        ctx->d2h += (size_t)launches[i].rows * sizeof(float);
        off += ((size_t)launches[i].rows + 3) & ~(size_t)3;
    }
    return FK_OK;
}

// `gpu::launch_dense_ffn_swiglu` (matvec_launch.rs:554-574): gate and up matvecs, SiLU(gate) * up, the down matvec,
// all on the device; one upload of x and one download of the result.  The gated activation rides in the down
// projection's prologue (no launch of its own).
FK_EXPORT int fk_launch_dense_ffn_swiglu(fk_ctx* ctx, const fk_matvec_launch* gate, const fk_matvec_launch* up, const fk_matvec_launch* down,
                                         const float* x_host, int n_cols, float* y_host) {
    if (!ctx || !gate || !up || !down || !x_host || !y_host) return fk_fail(FK_INVALID, "launch_dense_ffn_swiglu: null argument");
    if (gate->rows != up->rows) return fk_fail(FK_INVALID, "launch_dense_ffn_swiglu: gate has %d rows, up %d", gate->rows, up->rows);
    FkDeviceGuard g(ctx->device);
    fk_weight wg, wu, wd;
    int rc;
    if ((rc = prepare_launch(ctx, gate, n_cols, "launch_dense_ffn_swiglu (gate)", &wg))) return rc;
    if ((rc = prepare_launch(ctx, up, n_cols, "launch_dense_ffn_swiglu (up)", &wu))) return rc;
    if ((rc = prepare_launch(ctx, down, gate->rows, "launch_dense_ffn_swiglu (down)", &wd))) return rc;
    std::lock_guard<std::recursive_mutex> lk(ctx->mu);
    const size_t ffn = (size_t)gate->rows;
    if ((rc = grow(&ctx->x_dev, &ctx->x_cap, (size_t)n_cols))) return rc;
    if ((rc = grow(&ctx->y_dev, &ctx->y_cap, 2 * ffn))) return rc;
    if ((rc = grow_pinned(&ctx->x_pin, nullptr, &ctx->x_pin_cap, (size_t)n_cols, false))) return rc;
    if ((rc = grow_pinned(&ctx->y_pin, &ctx->y_pin_dev, &ctx->y_pin_cap, (size_t)down->rows, true))) return rc;
    memcpy(ctx->x_pin, x_host, (size_t)n_cols * sizeof(float));
    FK_CUDA(cudaMemcpyAsync(ctx->x_dev, ctx->x_pin, (size_t)n_cols * sizeof(float), cudaMemcpyHostToDevice, nullptr), FK_LAUNCH);
    ctx->h2d += (size_t)n_cols * sizeof(float);
    float* g_dev = ctx->y_dev;
    float* u_dev = ctx->y_dev + ffn;
    if ((rc = fk_gemv_launch(ctx, nullptr, wg, nullptr, 0, 1, ctx->x_dev, 0, 1, g_dev, nullptr, nullptr, nullptr))) return rc;
    if ((rc = fk_gemv_launch(ctx, nullptr, wu, nullptr, 0, 1, ctx->x_dev, 0, 1, u_dev, nullptr, nullptr, nullptr))) return rc;
    FkGemvFused f{nullptr, 0.0f, u_dev, 0, 0, (int)ffn, 0, nullptr};
    if ((rc = fk_gemv_launch(ctx, nullptr, wd, nullptr, 0, 1, g_dev, 0, 1, ctx->y_pin_dev, nullptr, nullptr, &f))) return rc;
    if ((rc = finish_host_call(ctx, "launch_dense_ffn_swiglu"))) return rc;
    memcpy(y_host, ctx->y_pin, (size_t)down->rows * sizeof(float));
    ctx->d2h += (size_t)down->rows * sizeof(float);
    return FK_OK;
}
