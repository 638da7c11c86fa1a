// Shared declarations of the sm_100a backend: context, resident weights and
// their device layouts, error plumbing, small device helpers.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stddef.h>
#include <atomic>
#include <map>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

#include "../../include/frink_b200.h"

#define FK_EXPORT extern "C" __attribute__((visibility("default")))

// ---------------------------------------------------------------------------
// Device layouts of resident weights.
//
// The ABI takes GGUF bytes.  Q4_K blocks (144 B, 16-byte aligned) stay as they
// are.  The other three formats have block sizes (210, 34, 17 B) that defeat
// 16-byte loads and TMA, so registration de-interleaves each matrix into
// planes with the SAME total bytes (plus alignment padding of a few bytes per
// matrix):
//   Q8_0 : qs   [rows][cols]      int8      | d  [rows][cols/32]  f16
//   Q6_K : ql   [rows][cols/2]    u8        | qh [rows][cols/4]   u8
//          sc   [rows][cols/16]   int8      | d  [rows][cols/256] f16
//   MXFP4: code [rows][cols/2]    u8        | e  [rows][cols/32]  u8 (E8M0)
// Every plane starts on a 256-byte boundary and every plane's row stride is a
// multiple of 16 bytes (the small scale planes are padded per row), so any row
// range of any plane can be moved with 16-byte loads or bulk copies.  Bytes
// inside a plane keep the GGUF block's own order, so the nibble/bit pairing
// rules of the formats are unchanged.
struct fk_weight_s {
    int kind;
    int n_mats;
    int rows;
    int cols;
    size_t gguf_bytes;      // n_mats * rows * row_bytes (what the caller gave)
    size_t gguf_row_bytes;  // bytes of one row in GGUF form
    size_t mat_stride;      // device bytes between consecutive matrices
    size_t plane_off[4];    // byte offset of each plane inside one matrix
    size_t plane_stride[4]; // bytes between consecutive rows of each plane (multiples of 16)
    uint8_t* dev;           // device allocation (n_mats * mat_stride)
    int device;
};

struct fk_ctx {
    int device;
    int sm_count;
    size_t mem_bytes;
    char name[128];
    std::recursive_mutex mu;   // recursive: the host-buffer surface holds it across launches that may grow the scratch block
    // host-buffer surface: (host ptr, len) -> (fingerprint, weights)
    std::map<std::pair<const void*, size_t>, std::pair<uint64_t, fk_weight>> resident;
    // scratch for the host-buffer surface, grown on demand
    float* x_dev = nullptr;
    size_t x_cap = 0;
    float* y_dev = nullptr;
    size_t y_cap = 0;
    // pinned host staging of the host-buffer surface (batch <= 8): x is copied from here,
    // y is written by the kernel straight into mapped host memory
    float* x_pin = nullptr;
    size_t x_pin_cap = 0;
    float* y_pin = nullptr;
    float* y_pin_dev = nullptr;
    size_t y_pin_cap = 0;
    // GEMM / MoE scratch (activation q8_1 planes), grown on demand
    uint8_t* scratch = nullptr;
    size_t scratch_cap = 0;
    std::vector<uint8_t*> scratch_retired;   // outgrown blocks: queued launches and captured graphs may still name them
    // device word kernels raise when a bounded wait gives up
    int* err_flag = nullptr;       // 16 bytes on the device: the error word, and at byte 8 the device address of its host mirror
    int* err_pin = nullptr;        // the mirror: mapped pinned host memory, written by the kernel that raises (fk_raise)
    // argmax: per-(row, block) keys and per-row arrival counters (64 x 64 keys, 64 counters);
    // one argmax in flight per context
    unsigned long long* argmax_ws = nullptr;
    unsigned* argmax_cnt = nullptr;
    // decode attention: arrival counters per (query row, head), 4096 of them
    unsigned* attn_cnt = nullptr;
    std::atomic<uint64_t> h2d{0}, d2h{0}, launches{0};
};

// error plumbing ------------------------------------------------------------
void fk_set_error(const char* fmt, ...);
int fk_fail(int status, const char* fmt, ...);
#define FK_CUDA(call, status)                                                            \
    do {                                                                                 \
        cudaError_t e__ = (call);                                                        \
        if (e__ != cudaSuccess)                                                          \
            return fk_fail((status), "%s: %s (%s:%d)", #call, cudaGetErrorString(e__), __FILE__, __LINE__); \
    } while (0)

struct FkDeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit FkDeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
        if (prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
    }
    ~FkDeviceGuard() {
        int cur = -1;
        if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
    }
};

static inline int fk_kind_block_bytes(int kind) {
    switch (kind) { case FK_Q8_0: return 34; case FK_Q4_K: return 144; case FK_Q5_K: return 176; case FK_Q6_K: return 210; case FK_MXFP4: return 17; case FK_BF16: return 2; }
    return -1;
}
static inline int fk_kind_block_elems(int kind) {
    switch (kind) { case FK_Q8_0: return 32; case FK_Q4_K: return 256; case FK_Q5_K: return 256; case FK_Q6_K: return 256; case FK_MXFP4: return 32; case FK_BF16: return 1; }
    return -1;
}
// activations per exact integer run (the weight-scale granularity)
static inline int fk_kind_run(int kind) { return kind == FK_Q6_K ? 16 : 32; }

// internal entry points of the kernel files ----------------------------------
struct FkGemvFused {
    const float* norm_w;
    float norm_eps;
    const float* glu_up;
    int glu_act;
    int accumulate;
    int x_ld;
    int pair_glu;                   // rows are (gate, up) pairs: write act(gate) * up, rows / 2 outputs
    const struct FkArChannel* ar;   // sum the results over the ranks of this channel in the epilogue (null: no)
    const float* bias = nullptr;    // [rows] added to the result; with ids: [n_mats][rows], slot j gets the row of matrix ids[j]
    // a second stack of matrices of the same geometry (indexed form only): the launch has 2 k slots, slot k + j multiplies
    // matrix ids[j] of w2 with slot j's input (bias2 its bias table) -- gate and up of the chosen experts in one launch
    fk_weight w2 = nullptr;
    const float* bias2 = nullptr;
    // indexed form: x is at least two launches old (older than the kernel that writes ids), so the activations may be
    // prepared before the wait on that kernel
    int x_ready = 0;
};
int fk_gemv_multi_gate_up_launch(fk_ctx* ctx, void* stream, fk_weight gate, fk_weight up, const int* ids_dev, int k, const float* x_dev,
                                 int x_stride, const float* norm_weight_dev, float norm_eps, const float* gate_bias_dev,
                                 const float* up_bias_dev, float* y_dev, int x_ready);
int fk_gemv_launch(fk_ctx* ctx, cudaStream_t st, fk_weight w, const int* ids_dev, int mat, int slots,
                   const float* x_dev, int x_stride, int batch, float* y_dev, int32_t* isums_dev, const int* n_active_dev,
                   const FkGemvFused* fused);
constexpr size_t FK_SCRATCH_MIN = (size_t)64 << 20;
int fk_ensure_scratch(fk_ctx* ctx, cudaStream_t st, size_t bytes);
int fk_gemv_bf16_launch(fk_ctx* ctx, cudaStream_t st, fk_weight w, int mat, const float* x_dev, int x_ld, int batch, float* y_dev,
                        const float* norm_w, float norm_eps, const float* bias, int accumulate);
int fk_gemv_q5k_launch(fk_ctx* ctx, cudaStream_t st, fk_weight w, int mat, const float* x_dev, int batch, float* y_dev, int32_t* isums_dev);
// `map` points at a CUtensorMap (128 bytes, 64-byte aligned): [outer][inner] 32-bit words, no swizzle
int fk_make_map_2d(void* map, int dtype, void* base, uint64_t inner, uint64_t outer, uint32_t box_inner, uint32_t box_outer, int swizzle);
int fk_make_map_u32(void* map, void* base, uint64_t inner_words, uint64_t outer, uint32_t box_inner, uint32_t box_outer);

// device helpers --------------------------------------------------------------
#ifdef __CUDACC__
// A kernel gives up (a bounded wait ran out, a cache would overrun): the first code wins the context's error word, and
// the winner also stores it into the word's host mirror (mapped pinned memory whose device address sits 8 bytes after
// the word), so that a host-buffer call sees it after its one synchronize without a copy of its own.
__device__ __forceinline__ void fk_raise(int* err, int code) {
    if (atomicCAS(err, 0, code) == 0) {
        int* mirror = *(int**)(err + 2);
        if (mirror) {
            *(volatile int*)mirror = code;
            __threadfence_system();
        }
    }
}
__device__ __forceinline__ float fk_h2f(uint16_t h) { return __half2float(__ushort_as_half(h)); }
__device__ __forceinline__ uint16_t fk_f2h(float f) { return __half_as_ushort(__float2half_rn(f)); }

__device__ __forceinline__ float fk_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// One 32-value run of the q8_1 activation rule, one value per lane of a full
// warp: amax over the run, d = amax / 127 (f32), q = roundf(x / d) with that
// unrounded d, stored scale f16(d).  Returns q; *d_f16 = the stored scale
// widened back to f32 (what every dot multiplies by), *qsum = the run's
// integer sum of q.
__device__ __forceinline__ int fk_q8_1_lane(float x, float* d_f16, int* qsum) {
    const unsigned amax_bits = __reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(x)));
    const float amax = __uint_as_float(amax_bits);
    const float d = amax / 127.0f;
    const int q = (amax == 0.0f) ? 0 : (int)roundf(x / d);
    *d_f16 = fk_h2f(fk_f2h(d));
    *qsum = __reduce_add_sync(0xffffffffu, q);
    return q;
}
#endif
