/* frink_b200 -- C ABI of the B200 (sm_100a) backend for frink's
 * dequantize-inside-the-matmul path.
 *
 * This library takes the place of frink-cuda's kernel set behind frink-core's
 * `WeightMatrix` backend seam.  Every entry point below names the frink
 * interface it replaces (file:line inside the frink project, v0.63.0).  All
 * functions return an `fk_status`; a failing call leaves a message that
 * `fk_last_error` returns (per calling thread).  No host allocation crosses
 * the ABI (callers pass every output buffer).
 *
 * Threads: calls on different contexts are independent; calls on one context
 * are serialised where they touch its tables (registration, residency).  The
 * GEMM, the batch 3..8 matvec, the split attention and fk_gemv_isums use ONE
 * workspace of the context, in stream order: two streams (or threads) must not
 * have such calls of one context in flight together.  The workspace only grows
 * and an outgrown block is kept until fk_destroy, so a launch that is queued,
 * or captured in a CUDA graph, never points at freed memory; growing it
 * allocates, which a stream capture forbids, so a call that needs more than is
 * reserved while its stream is being captured fails with FK_INVALID -- run the
 * call once before capturing, or fk_reserve_scratch.  64 MiB are taken on
 * first use.
 *
 * Pointers named `*_dev` are CUDA device pointers on the context's device,
 * pointers named `*_host` are ordinary host memory.  `stream` is a
 * `cudaStream_t` passed as `void*` (NULL = the legacy default stream).
 *
 * Weight bytes are ALWAYS the unmodified GGUF block bytes of the tensor
 * (row-major, `row_bytes = cols / block_elems * block_bytes`); the library
 * uploads them once and may rearrange them on the device.
 */
#ifndef FRINK_B200_H
#define FRINK_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Mirrors `CudaError::{DriverInit, KernelCompile, Launch, Unsupported}`
 * (crates/frink-cuda/src/gpu.rs:91-104).  UNSUPPORTED keeps its contract: the
 * caller must use a path that can compute the result, never something else. */
typedef enum fk_status {
    FK_OK = 0,
    FK_DRIVER_INIT = 1,
    FK_KERNEL = 2,
    FK_LAUNCH = 3,
    FK_UNSUPPORTED = 4,
    FK_COMM = 5,
    FK_INVALID = 6
} fk_status;

/* Block formats, by ggml type tag (crates/frink-core/src/weight_matrix.rs:43,
 * `QuantKind`; layouts crates/frink-quant/src/lib.rs:73-75,176-197,5560-5571). */
typedef enum fk_kind {
    FK_Q8_0 = 8,   /* 34 B / 32 weights  */
    FK_Q4_K = 12,  /* 144 B / 256 weights */
    FK_Q5_K = 13,  /* 176 B / 256 weights: the plain matvec (fk_gemv, fk_gemv_isums, fk_launch_matvec) and fk_get_rows only */
    FK_Q6_K = 14,  /* 210 B / 256 weights */
    FK_BF16 = 30,  /* 2 B / weight, not quantized (gpt-oss attention projections): the plain matvec on f32 activations and fk_get_rows only */
    FK_MXFP4 = 39  /* 17 B / 32 weights  */
} fk_kind;

typedef struct fk_ctx fk_ctx;
typedef struct fk_weight_s* fk_weight;
typedef struct fk_comm fk_comm;

/* ---- context ------------------------------------------------------------
 * Replaces `gpu::shared_device` / `gpu::probe` (crates/frink-cuda/src/
 * gpu.rs:121-222): one context per device, created once, used from any thread. */
int fk_init(int device, fk_ctx** out);
void fk_destroy(fk_ctx* ctx);
const char* fk_last_error(void);
/* name[<=cap], SM count, global memory bytes: `CudaInfo` (gpu.rs:106-119). */
int fk_device_info(fk_ctx* ctx, char* name, size_t cap, int* sm_count, size_t* mem_bytes);
/* Counters since the last reset: H2D bytes, D2H bytes, kernel launches made
 * by this library (crates/frink-cuda/src/counters.rs, xfer.rs). */
int fk_counters(fk_ctx* ctx, uint64_t* h2d_bytes, uint64_t* d2h_bytes, uint64_t* launches, int reset);
/* The word a kernel raises when one of its bounded waits gives up (0 = none);
 * no counterpart in the reference, whose kernels have no waits. */
int fk_device_error(fk_ctx* ctx, int* code, int reset);
int fk_block_bytes(int kind);
int fk_block_elems(int kind);

/* ---- resident weights ---------------------------------------------------
 * Replaces `resident_cuda_weights` (crates/frink-cuda/src/resident.rs): the
 * GGUF bytes of `n_mats` equally shaped matrices (1 for a dense projection,
 * `n_expert` for a stacked expert tensor), uploaded once.  `len` must equal
 * n_mats * rows * row_bytes. */
int fk_register_weights(fk_ctx* ctx, const uint8_t* gguf_bytes_host, size_t len, int kind, int n_mats,
                        int rows, int cols, fk_weight* out);
/* The same from bytes already on the device (copied; the source may be freed). */
int fk_register_weights_dev(fk_ctx* ctx, const uint8_t* gguf_bytes_dev, size_t len, int kind, int n_mats,
                            int rows, int cols, void* stream, fk_weight* out);
int fk_release_weights(fk_ctx* ctx, fk_weight w);
int fk_weight_shape(fk_weight w, int* kind, int* n_mats, int* rows, int* cols, size_t* gguf_bytes);

/* ---- activation quantizer ----------------------------------------------
 * Replaces `quantize_q8_1` (crates/frink-cuda/src/matvec_kinds/dp4a/
 * kernels.rs:113-143): n f32 (n % 32 == 0) -> n/32 `block_q8_1` of 36 bytes
 * (f16 d = amax/127, f16 sum, 32 x int8 = roundf(x/d)).  The GEMV and GEMM
 * below quantize their activations with exactly this rule, fused. */
int fk_quantize_q8_1(fk_ctx* ctx, void* stream, const float* x_dev, int n, uint8_t* y_dev);
/* The same with host buffers: n floats in, n / 32 blocks of 36 bytes out (`matvec_reads`,
 * crates/frink-cuda/src/matvec_kinds/dp4a.rs:291-303, is this followed by d * q). */
int fk_quantize_q8_1_host(fk_ctx* ctx, const float* x_host, int n, uint8_t* y_host);

/* ---- decode GEMV, batch 1..8 ---------------------------------------------
 * Replaces `q4_k_matvec_dp4a`, `q6_k_matvec_dp4a`, `q8_0_matvec_dp4a`,
 * `mxfp4_matvec_dp4a` and their launch (kernels.rs:243-465,
 * crates/frink-cuda/src/dp4a_launch.rs:185-246).
 * y_dev[b * rows + r] = W[mat][r] . q8_1(x_dev[b * cols ..]),  0 <= b < batch. */
int fk_gemv(fk_ctx* ctx, void* stream, fk_weight w, int mat, const float* x_dev, int batch, float* y_dev);

/* fk_gemv with the elementwise neighbours of a decode step folded in (the reference
 * runs them as separate kernels: `fused_add_rmsnorm_f32` crates/frink-cuda/src/gpu.rs:459,
 * `silu_mul_f32` src/glu.rs:68, `add_rows_f32` src/prefill/kernels.rs:70).  All optional:
 * norm_weight_dev: the matvec reads rmsnorm(x) * norm_weight (squares summed in f64);
 * glu_up_dev: the matvec reads act(x) * glu_up, x being the gate (act 0 SiLU, 1 gpt-oss);
 * accumulate != 0: y += W x (the residual add).  x_ld = floats between batch rows of x
 * and glu_up (0 = cols).
 * pair_glu (0 none, 1 SiLU, 2 gpt-oss): the matrix holds gate and up stacked row-interleaved
 * (gate row i, up row i, ...); the launch writes act(gate_i) * up_i, rows / 2 values per
 * batch row, so the down projection reads the activated vector directly. */
int fk_gemv_fused(fk_ctx* ctx, void* stream, fk_weight w, int mat, const float* x_dev, int x_ld, int batch, float* y_dev,
                  const float* norm_weight_dev, float norm_eps, const float* glu_up_dev, int glu_act, int accumulate, int pair_glu);

/* Indexed expert GEMV: the `FX_MULTI` form (kernels.rs:166-179,
 * dp4a_launch.rs:256-314).  Slot j (0 <= j < k) multiplies matrix
 * `ids_dev[j]` of `w` with x_dev[j * x_stride ..] (x_stride 0 = one shared
 * input) into y_dev[j * rows ..]. */
int fk_gemv_multi(fk_ctx* ctx, void* stream, fk_weight w, const int* ids_dev, int k, const float* x_dev,
                  int x_stride, float* y_dev);

/* fk_gemv_multi reading act(gate[j]) * up[j] instead of x[j] (the down projection of the
 * chosen experts with `silu_mul_f32` / the gpt-oss activation of src/glu.rs:68 folded
 * in); n_active_dev may be null (all k slots run). */
int fk_gemv_multi_glu(fk_ctx* ctx, void* stream, fk_weight w, const int* ids_dev, int k, const float* gate_dev, const float* up_dev,
                      int x_stride, int glu_act, float* y_dev, const int* n_active_dev);
/* fk_gemv_multi whose slots >= *n_active_dev do nothing (their outputs are left as
 * they are).  Expert-parallel decode runs only the chosen experts a rank owns
 * without a host round trip for the count; no counterpart in the single-device
 * reference. */
int fk_gemv_multi_active(fk_ctx* ctx, void* stream, fk_weight w, const int* ids_dev, int k, const float* x_dev,
                         int x_stride, float* y_dev, const int* n_active_dev);

/* Biased projections of a gpt-oss layer (crates/frink-models/src/models/gpt_oss.rs:9-12,46) as one launch:
 *   y[b] (+)= W rmsnorm?(x[b]) + bias        (norm_weight_dev, bias_dev may be null; bias_dev is [rows]).
 * Every kind with a matvec except Q5_K; BF16 included (its only fused forms are these). */
int fk_gemv_biased(fk_ctx* ctx, void* stream, fk_weight w, int mat, const float* x_dev, int x_ld, int batch, float* y_dev,
                   const float* norm_weight_dev, float norm_eps, const float* bias_dev, int accumulate);
/* fk_gemv_multi / fk_gemv_multi_glu with every expert's own bias row (`run_expert_oai`, crates/frink-moe/src/
 * lib.rs:1039-1060): slot j: y[j] = W[ids[j]] in_j + bias_dev[ids[j]], in_j = x[j], or act(x[j]) * up[j] when
 * up_dev is given (x then being the biased gate); bias_dev is [n_mats][rows]. */
int fk_gemv_multi_biased(fk_ctx* ctx, void* stream, fk_weight w, const int* ids_dev, int k, const float* x_dev, const float* up_dev,
                         int x_stride, int glu_act, const float* bias_dev, float* y_dev);

/* gate and up of the chosen experts in one launch of 2 k slots (same input, same shape; the reference shares one
 * quantized input between them, crates/frink-cuda/src/dp4a_launch.rs:56-62): y_dev [2 k][rows], rows j < k from
 * `gate`, rows k + j from `up`, both of expert ids_dev[j] on input j.  norm_weight_dev (optional): the input is
 * rmsnorm(x[j]) * norm_weight; the bias tables ([n_mats][rows]) are optional and come together. */
int fk_gemv_multi_gate_up(fk_ctx* ctx, void* stream, fk_weight gate, fk_weight up, const int* ids_dev, int k, const float* x_dev,
                          int x_stride, const float* norm_weight_dev, float norm_eps, const float* gate_bias_dev,
                          const float* up_bias_dev, float* y_dev);

/* Test hook (the reference's twins expose the same integers,
 * crates/frink-cuda/src/dp4a_twin.rs:142-231): the exact int32 dot of every
 * run of 32 activations (16 for Q6_K) of every row against q8_1(x), computed
 * by the GEMV kernel's own inner loop.  isums_dev is [rows][cols / run]. */
int fk_gemv_isums(fk_ctx* ctx, void* stream, fk_weight w, int mat, const float* x_dev, int32_t* isums_dev);

/* ---- prefill GEMM ---------------------------------------------------------
 * Replaces `mul_mm_launch::launch_mul_mm` / `enqueue_mmq` (crates/frink-cuda/
 * src/mul_mm_launch.rs:40-68, src/mmq/mod.rs:30-133):
 * out_dev[t * rows + r] = W[mat][r] . q8_1(x_dev[t * cols ..]),  0 <= t < m. */
int fk_gemm(fk_ctx* ctx, void* stream, fk_weight w, int mat, const float* x_dev, int m, float* out_dev);

/* Test hook, the GEMM's counterpart of fk_gemv_isums (the reference's GEMM twins expose the
 * same integers, crates/frink-cuda/src/mmq/mod.rs:230-432): fk_gemm that also writes the
 * exact int32 dot of every run of 32 activations (16 for Q6_K) as the tensor cores
 * delivered it, before any scale: isums_dev is [m][rows][cols / run]. */
int fk_gemm_isums(fk_ctx* ctx, void* stream, fk_weight w, int mat, const float* x_dev, int m, float* out_dev, int32_t* isums_dev);

/* The prefill GEMM on frink's CPU activation rule: Q8_K activations (one f32 scale and sixteen
 * 16-value sums per 256 values, `quantize_activations_q8_k`, crates/frink-quant/src/act_quant.rs:
 * 69-104) against Q4_K weights, the integers of `dot_q4_k_q8` (crates/frink-quant/src/lib.rs:
 * 822-869) taken on the tensor cores over whole super-blocks.  Its results match frink's CPU
 * batched path (`WeightMatrix::apply_batch_with_acts`, crates/frink-core/src/weight_matrix.rs:1716)
 * to f32 summation order; they differ from fk_gemm's by the activation quantizer (q8_1 there).
 * Other kinds return FK_UNSUPPORTED (use fk_gemm). */
int fk_gemm_q8k(fk_ctx* ctx, void* stream, fk_weight w, int mat, const float* x_dev, int m, float* out_dev);
/* Test hook: fk_gemm_q8k that also writes, per (token, row, super-block), the two exact integers
 * of the CPU vec_dot (sum of scale * sub-block dot, sum of min * sub-block sum) as the tensor
 * cores delivered them: isums_dev is [m][rows][cols / 256][2]. */
int fk_gemm_q8k_isums(fk_ctx* ctx, void* stream, fk_weight w, int mat, const float* x_dev, int m, float* out_dev, int32_t* isums_dev);

/* fk_gemm for callers that cannot allocate device memory when they need it (a
 * thread inside a stream capture, a serving loop that must avoid cudaMalloc's
 * device-wide synchronisation, a process on a fixed memory budget).  It has no
 * counterpart in the reference.  Same arguments and results as fk_gemm; its
 * scratch lives in a fixed 6 MiB block inside the library (held by every GPU
 * that loads it, from load to exit) and the call makes no cudaMalloc/cudaFree.
 * Shapes whose scratch does not fit (about m_padded * (cols + cols / 4) bytes,
 * m padded to 128) are refused with FK_INVALID.  The first call on a device
 * looks the block's address up (cudaGetSymbolAddress); make that call before
 * any stream capture.  Every call shares the block: two calls that overlap on
 * the GPU (different streams, no ordering) race; calls on one stream do not. */
int fk_gemm_static(fk_ctx* ctx, void* stream, fk_weight w, int mat, const float* x_dev, int m, float* out_dev);

/* Grouped (per-expert) GEMM, the `FX_GROUPED` form (src/mmq/mod.rs:144-226):
 * rows [group_off[e], group_off[e+1]) of the permuted activation list belong to
 * expert e; permuted row p reads x_dev[gather_dev[p] * cols ..] (gather NULL =
 * identity) and writes out_dev[p * rows ..]. */
int fk_gemm_grouped(fk_ctx* ctx, void* stream, fk_weight w, const int* group_off_dev, const int* gather_dev,
                    const float* x_dev, int pairs, float* out_dev);

/* ---- MoE routing, permute, activation, combine ----------------------------
 * `moe_topk_f32` (crates/frink-cuda/src/prefill/kernels.rs:178-267): mode 0
 * softmax over all experts, 1 the same renormalised over the chosen, 2 top-k by
 * (biased) logit then softmax over the chosen (gpt-oss).  Ties -> lower id. */
int fk_moe_route(fk_ctx* ctx, void* stream, const float* logits_dev, const float* bias_dev, int n_experts,
                 int k, int mode, int batch, int* ids_dev, float* w_dev);
/* fk_router_logits and fk_moe_route in one launch (the decode step of a routed layer): the
 * logits are still written (logits_dev [batch][n_experts]); one call in flight per context. */
int fk_router_route(fk_ctx* ctx, void* stream, const float* router_dev, const float* x_dev, int n_experts, int cols, int batch,
                    const float* bias_dev, int k, int mode, float* logits_dev, int* ids_dev, float* w_dev);
/* `router_f32_matvec` (kernels.rs:356-378): logits[t][e] = router[e] . x[t]. */
int fk_router_logits(fk_ctx* ctx, void* stream, const float* router_dev, const float* x_dev, int n_experts,
                     int cols, int batch, float* logits_dev);
/* `moe_count_i32` + `moe_offsets_i32` + `moe_scatter_i32` (kernels.rs:271-308):
 * pairs = batch * k (token p / k, slot p % k) grouped by expert, tokens in
 * ascending order inside a group.  group_off_dev[n_experts + 1],
 * gather_dev[pairs] (token of each permuted row), pair_of_dev[pairs]. */
int fk_moe_permute(fk_ctx* ctx, void* stream, const int* ids_dev, int pairs, int k, int n_experts,
                   int* group_off_dev, int* gather_dev, int* pair_of_dev);
/* Expert-parallel decode (no reference counterpart): of one token's k routed
 * experts, those in [e0, e0 + n_local) packed to the front in routing order as
 * local ids with their weights (the rest: expert 0, weight 0); *out_n = count. */
int fk_moe_local_slots(fk_ctx* ctx, void* stream, const int* ids_dev, const float* w_dev, int k, int e0, int n_local,
                       int* out_ids_dev, float* out_w_dev, int* out_n_dev);
/* The same for a decode batch of b rows (pairs = b * k <= 256, pair i belongs to row i / k): the pairs
 * whose expert lies in [e0, e0 + n_local) become slots 0 .. *out_n - 1 in pair order -- out_ids[p] the
 * local expert and out_src[p] the row whose activation slot p reads (0 past the last slot);
 * out_pair_of[i] is the slot of pair i and out_w[i] its weight (slot 0, weight 0 for a pair another
 * rank owns), the arguments fk_moe_combine takes. */
int fk_moe_local_pairs(fk_ctx* ctx, void* stream, const int* ids_dev, const float* w_dev, int pairs, int k, int e0, int n_local,
                       int* out_ids_dev, int* out_src_dev, int* out_pair_of_dev, float* out_w_dev, int* out_n_dev);
/* Expert-parallel prefill over replicated activations (no reference counterpart): every rank routes
 * all tokens; pair i keeps its expert as the local id ids[i] - e0 when e0 <= ids[i] < e0 + n_local,
 * else it gets the id n_local (a group no expert serves) and weight 0. */
int fk_moe_localize(fk_ctx* ctx, void* stream, const int* ids_dev, const float* w_dev, int pairs, int e0, int n_local,
                    int* out_ids_dev, float* out_w_dev);
/* `silu_mul_f32` / `swiglu_oai_f32` (crates/frink-cuda/src/glu.rs:42,68):
 * act 0 = silu(gate) * up, 1 = gpt-oss clamped SwiGLU (alpha 1.702, limit 7). */
int fk_glu(fk_ctx* ctx, void* stream, const float* gate_dev, const float* up_dev, size_t n, int act,
           float* out_dev);
/* `moe_combine_rows_f32` (kernels.rs:332-352): out[t] = sum_j w[t][j] *
 * y[pair_of[t*k+j]] from zero in routing order (pair_of NULL = identity). */
int fk_moe_combine(fk_ctx* ctx, void* stream, const float* y_dev, const int* pair_of_dev, const float* w_dev,
                   int batch, int k, int n, float* out_dev);
/* fk_moe_combine that adds the combined rows into out (the residual stream) instead of
 * overwriting it; the weighted sum itself is still formed from zero in routing order. */
int fk_moe_combine_add(fk_ctx* ctx, void* stream, const float* y_dev, const int* pair_of_dev, const float* w_dev,
                   int batch, int k, int n, float* out_dev);

/* The resident routed layer as ONE call (`prefill::moe_device`, crates/frink-cuda/src/prefill/
 * moe_device.rs:241-438): router logits and top-k, the three expert projections with the
 * gated activation, the weighted combine in routing order.  gate / up / down are stacked expert
 * handles (n_mats experts of [ffn x hidden], [ffn x hidden], [hidden x ffn]); x_dev
 * [batch][hidden]; out_dev [batch][hidden] is written, or added into when accumulate != 0.
 * batch <= 8 takes the indexed matvecs (every (row, expert) pair a slot), larger batches the
 * grouped GEMMs.  workspace_dev: fk_moe_layer_workspace(...) bytes of device memory, 256-byte
 * aligned, owned by the caller (nothing is allocated here).  mode / act as in fk_moe_route /
 * fk_glu. */
size_t fk_moe_layer_workspace(int n_experts, int k, int hidden, int ffn, int batch);
int fk_moe_layer(fk_ctx* ctx, void* stream, const float* router_dev, const float* router_bias_dev, fk_weight gate, fk_weight up,
                 fk_weight down, int k, int mode, int act, const float* x_dev, int batch, float* out_dev, int accumulate,
                 void* workspace_dev, size_t workspace_bytes);
/* gpt-oss's routed layer (`run_expert_oai`, crates/frink-moe/src/lib.rs:1039-1060): fk_moe_layer whose three
 * expert projections carry a bias table each ([n_experts][ffn], [n_experts][ffn], [n_experts][hidden]); the
 * activation is applied to the biased gate and up.  Decode batches add the bias in the matvec's epilogue;
 * the grouped GEMM path adds it with a launch per projection. */
int fk_moe_layer_biased(fk_ctx* ctx, void* stream, const float* router_dev, const float* router_bias_dev, fk_weight gate, fk_weight up,
                        fk_weight down, const float* gate_bias_dev, const float* up_bias_dev, const float* down_bias_dev, int k, int mode,
                        int act, const float* x_dev, int batch, float* out_dev, int accumulate, void* workspace_dev,
                        size_t workspace_bytes);

/* The decode form (batch <= 8) of the routed layer on the RESIDUAL stream: x_dev is un-normalized and the layer's
 * RMSNorm (`rmsnorm_rows_f32`, crates/frink-cuda/src/prefill/kernels.rs:26) is folded into the router and into the
 * gate / up launch, which is ONE indexed launch for both projections (fk_gemv_multi_gate_up): four launches a layer.
 * Bias tables: all three or none (null).  out_dev may be x_dev with accumulate != 0 (the layer added into the stream). */
int fk_moe_layer_normed(fk_ctx* ctx, void* stream, const float* router_dev, const float* router_bias_dev, fk_weight gate, fk_weight up,
                        fk_weight down, const float* gate_bias_dev, const float* up_bias_dev, const float* down_bias_dev, int k, int mode,
                        int act, const float* norm_weight_dev, float norm_eps, const float* x_dev, int batch, float* out_dev,
                        int accumulate, void* workspace_dev, size_t workspace_bytes);

/* ---- decoder glue (next-row components: enough to run a decoder and report
 * prefill / decode tokens per second; f32 throughout) -------------------------
 * `get_rows` (crates/frink-cuda/src/get_rows.rs:52): out[i] = dequantized row ids[i]. */
int fk_get_rows(fk_ctx* ctx, void* stream, fk_weight w, int mat, const int* ids_dev, int n, float* out_dev);
/* `rmsnorm_rows_f32` / `fused_add_rmsnorm_f32` (crates/frink-cuda/src/prefill/kernels.rs:26,
 * src/gpu.rs:459): if residual_dev is given, x += residual first (kept in x); then
 * out = x * (1/sqrt(mean(x^2) + eps)) * weight, squares summed in f64
 * (crates/frink-core/src/matmul.rs:87-95). */
int fk_rmsnorm(fk_ctx* ctx, void* stream, float* x_dev, const float* residual_dev, const float* weight_dev, int n_rows, int cols,
               float eps, float* out_dev);
/* `rope_rows_f32` (kernels.rs:402): in place over [n_rows][n_heads][head_dim]; row r is
 * at position *pos_dev + r; neox 0 rotates pairs (2i, 2i+1), else (i, i + head_dim/2). */
int fk_rope(fk_ctx* ctx, void* stream, float* x_dev, int n_rows, int n_heads, int head_dim, const int* pos_dev, float theta, int neox);
/* rope of q and k and the KV append of one step in one launch: q [n][n_heads*hd] and
 * k [n][n_kv*hd] are rotated in place (rows at *pos + r), then k and v rows are
 * written to the caches at *pos.  q_ld / kv_ld = floats between rows.  q_norm_dev /
 * k_norm_dev (both or neither, [head_dim]): the per-head RMSNorm of Qwen3 applied to
 * q and k ahead of the rotation.
 *
 * cache_rows (here and in the three calls below) is the number of rows T the K/V buffers hold.
 * The position lives on the device, so the host cannot refuse an overrun: a kernel that finds
 * *pos + rows > cache_rows does nothing at all and raises the device error word 95. */
int fk_rope_kv(fk_ctx* ctx, void* stream, float* q_dev, float* k_dev, const float* v_dev, int q_ld, int kv_ld, int n_rows, int n_heads,
               int n_kv, int head_dim, const int* pos_dev, float theta, int neox, float* k_cache_dev, float* v_cache_dev,
               const float* q_norm_dev, const float* k_norm_dev, float norm_eps, int cache_rows);
/* Grow the context's workspace to at least `bytes` (it never shrinks). */
int fk_reserve_scratch(fk_ctx* ctx, size_t bytes);
/* gpt-oss's projection biases (crates/frink-models/src/models/gpt_oss.rs:9-12,46; `run_expert_oai`,
 * crates/frink-moe/src/lib.rs:1039-1060): y [n_rows][cols] += bias [cols]; with ids_dev [n_rows] (the expert of every
 * slot of an indexed matvec) += row ids[r] of bias [n_experts][cols]. */
int fk_add_bias(fk_ctx* ctx, void* stream, float* y_dev, const float* bias_dev, const int* ids_dev, int n_rows, int cols);
/* `add_rows_f32` (kernels.rs:70): a += b. */
int fk_add(fk_ctx* ctx, void* stream, float* a_dev, const float* b_dev, size_t n);
/* `kv_append_f32` (kernels.rs:664): cache rows [*pos, *pos + n_rows) <- src. */
int fk_kv_append(fk_ctx* ctx, void* stream, float* cache_dev, const float* src_dev, size_t row_elems, int n_rows, const int* pos_dev,
                 int cache_rows);
/* window, sinks_dev (this call and the two below; gpt-oss, crates/frink-core/src/attention.rs:312-322,960-1000):
 * window > 0: a query sees only the `window` most recent keys including its own (0 = all); sinks_dev
 * [n_heads] (NULL = none): one logit per query head that joins the softmax's denominator, unscaled, and
 * contributes nothing to the output.
 * `causal_gqa_prefill_f32` / `decode_attn_*` (kernels.rs:488, src/decode_attn.rs:125):
 * query row r at position *pos + r attends keys 0..=*pos + r of K/V [T][n_kv][head_dim].
 * q_ld = floats between query rows (0 = n_heads * head_dim).  With fewer than 16 query rows
 * the keys are split over many blocks that meet in a workspace of the context: one such
 * call in flight per context. */
int fk_attention(fk_ctx* ctx, void* stream, const float* q_dev, int q_ld, const float* k_dev, const float* v_dev, int n_q, int n_heads,
                 int n_kv, int head_dim, const int* pos_dev, float scale, float* out_dev, int cache_rows, int window,
                 const float* sinks_dev);
/* One decode row: fk_rope_kv and fk_attention in one launch.  q [n_heads*head_dim], k_new and
 * v_new [n_kv*head_dim] are the projection's outputs for the token at *pos (unrotated); the
 * caches hold positions 0 .. *pos - 1 and receive the rotated k and v at *pos.  q_norm_dev /
 * k_norm_dev as in fk_rope_kv.  One call in flight per context. */
int fk_attention_rope_kv(fk_ctx* ctx, void* stream, const float* q_dev, const float* k_new_dev, const float* v_new_dev, float* k_cache_dev,
                         float* v_cache_dev, int n_heads, int n_kv, int head_dim, const int* pos_dev, float scale, float theta, int neox,
                         const float* q_norm_dev, const float* k_norm_dev, float norm_eps, float* out_dev, int cache_rows, int window, const float* sinks_dev);
/* The same step for n_seqs independent sequences in one launch (batched decode): row r of q
 * (rows q_ld floats apart), k_new and v_new (k_ld / v_ld apart) is sequence r's token at position
 * pos_dev[r]; sequence r's caches begin r * seq_stride floats into k_cache_dev / v_cache_dev and
 * hold cache_rows rows each.  out_dev [n_seqs][n_heads*head_dim].  A sequence whose position
 * has reached cache_rows is skipped and raises the error word 95. */
int fk_attention_rope_kv_seqs(fk_ctx* ctx, void* stream, const float* q_dev, int q_ld, const float* k_new_dev, const float* v_new_dev, int k_ld,
                              int v_ld, float* k_cache_dev, float* v_cache_dev, size_t seq_stride, int n_seqs, int n_heads, int n_kv, int head_dim,
                              const int* pos_dev, float scale, float theta, int neox, const float* q_norm_dev, const float* k_norm_dev,
                              float norm_eps, float* out_dev, int cache_rows, int window, const float* sinks_dev);
/* Greedy sampling: index of the largest of each row, ties to the lower index; at most
 * 64 rows per call, and one call in flight per context (it uses a workspace of the context). */
int fk_argmax(fk_ctx* ctx, void* stream, const float* x_dev, int n_rows, int n, int* out_dev);
/* *p += v on the device (the position word of a captured decode step). */
int fk_add_int(fk_ctx* ctx, void* stream, int* p_dev, int v);

/* ---- multi-GPU: peer-memory all-reduce ---------------------------------------
 * The reference is single-device (crates/frink-cuda/src/gpu.rs:219); these have no counterpart
 * there.  One process per GPU of one box.  Every rank creates an arena and publishes its 64-byte
 * handle (CUDA IPC) to the others by whatever transport the host has (torch.distributed here);
 * fk_comm_connect maps the peers' arenas.  An arena is carved into channels at the same offsets
 * on every rank, fk_comm_channel_bytes(world, n_max) bytes each (256-byte aligned offsets); a
 * channel serves all-reduces of up to n_max floats, one at a time.
 *
 * fk_allreduce: dst = (accumulate ? dst : 0) + sum over ranks of src, the same bits on every
 * rank (values are added in rank order).  One kernel: every value is stored into every peer's
 * slot together with the all-reduce's number for that element (one 8-byte store, so no fence
 * and no separate flag), the local slots are read until their number matches -- a wait bounded
 * by timeout_us (0 = two seconds) that raises the device error word 60 instead of hanging --
 * and summed.  The per-element numbers live on the device, so a captured launch may be
 * replayed.  Every rank must issue the same all-reduces on a channel in the same order.
 *
 * fk_gemv_fused_allreduce: fk_gemv_fused (without pair_glu) on this rank's column range of a
 * row-split matrix, the sum over ranks done by the matvec's own epilogue (element b * rows + row
 * of the channel): the tensor-parallel form of the wo / down projections of a decode step. */
int fk_comm_create(fk_ctx* ctx, size_t arena_bytes, int rank, int world, uint8_t* handle_out_64, fk_comm** out);
int fk_comm_connect(fk_comm* comm, const uint8_t* handles_world_x_64);
/* Test hook: peers given as device pointers of this GPU (the time-out path is tested on one GPU). */
int fk_comm_connect_local(fk_comm* comm, void* const* peer_arenas_dev);
int fk_comm_arena(fk_comm* comm, void** arena_dev, size_t* bytes);
int fk_comm_destroy(fk_comm* comm);
size_t fk_comm_channel_bytes(int world, int n_max);
int fk_allreduce(fk_ctx* ctx, void* stream, fk_comm* comm, size_t channel_off, int n_max, const float* src_dev, float* dst_dev, int n,
                 int accumulate, int timeout_us);
int fk_gemv_fused_allreduce(fk_ctx* ctx, void* stream, fk_weight w, int mat, const float* x_dev, int x_ld, int batch, float* y_dev,
                            const float* norm_weight_dev, float norm_eps, const float* glu_up_dev, int glu_act, int accumulate,
                            fk_comm* comm, size_t channel_off, int n_max, int timeout_us);

/* ---- host-buffer launch surface -------------------------------------------
 * What frink-core binds (crates/frink-core/src/weight_matrix/gpu_backend.rs:
 * 247-273,563-565): host slices in, host slice out, one call per projection.
 * Weights are kept resident, keyed by (pointer, length) plus a byte-sample
 * fingerprint, as crates/frink-cuda/src/resident.rs does.
 *
 * `gpu::launch_<kind>_matvec(weights, x, rows, row_bytes, n_blocks_per_row)`
 * (crates/frink-cuda/src/gpu.rs:319-446). */
int fk_launch_matvec(fk_ctx* ctx, int kind, const uint8_t* weights_host, size_t len, const float* x_host,
                     int rows, int row_bytes, int n_blocks_per_row, float* y_host);

/* `MatvecLaunch` (crates/frink-cuda/src/matvec_launch.rs:485-493) without the kernel names: the
 * GGML type tag selects the kernel.  `weights_host` must be a stable slice (the mmap'd tensor):
 * residency is keyed by (pointer, length). */
typedef struct fk_matvec_launch {
    int kind;
    const uint8_t* weights_host;
    size_t len;
    int rows;
    int row_bytes;
    int n_blocks_per_row;
} fk_matvec_launch;
/* `gpu::launch_matvec_multi` (matvec_launch.rs:495-536): x (n_cols floats) goes up once, the n
 * matvecs are enqueued back to back, y_hosts[i] receives launches[i].rows floats; one
 * synchronize.  n <= 64. */
int fk_launch_matvec_multi(fk_ctx* ctx, const float* x_host, int n_cols, const fk_matvec_launch* launches, int n, float* const* y_hosts);
/* `gpu::launch_dense_ffn_swiglu` (matvec_launch.rs:554-574): y = down (SiLU(gate x) * (up x)),
 * one upload of x, one download of y (down->rows floats); the gated activation is formed in
 * the down projection's prologue. */
int fk_launch_dense_ffn_swiglu(fk_ctx* ctx, const fk_matvec_launch* gate, const fk_matvec_launch* up, const fk_matvec_launch* down,
                               const float* x_host, int n_cols, float* y_host);
/* All fk_launch_* calls read the device error word before they return: if a kernel of the call
 * gave up a bounded wait the call answers FK_LAUNCH (the message names the code) and clears
 * the word. */
/* `mul_mm_launch::launch_mul_mm(kind, weights, x_batch, n_rows, n_cols, batch,
 * row_bytes)` (crates/frink-cuda/src/mul_mm_launch.rs:40-68);
 * out_host[token * n_rows + row].  batch 1..8 takes the GEMV. */
int fk_launch_mul_mm(fk_ctx* ctx, int kind, const uint8_t* weights_host, size_t len, const float* x_batch_host,
                     int n_rows, int n_cols, int batch, int row_bytes, float* out_host);
/* Drops every weight the host-buffer surface made resident. */
int fk_forget_resident(fk_ctx* ctx);

#ifdef __cplusplus
}
#endif
#endif /* FRINK_B200_H */
