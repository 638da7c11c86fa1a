//! Raw declarations of `libfrink_b200.so`'s C ABI, one per entry point of `include/frink_b200.h`, in the
//! header's order and with the header's argument names (written by `bindings/rust/gen_sys.py`).  Semantics,
//! units and the frink interface each call replaces are documented in the header; nothing here adds behaviour.
#![allow(non_camel_case_types)]
use std::os::raw::{c_char, c_int, c_void};

/// Opaque context (`fk_ctx`): one per device, created by `fk_init`.
#[repr(C)]
pub struct FkCtx {
    _private: [u8; 0],
}
/// Opaque resident weights (`struct fk_weight_s`).
#[repr(C)]
pub struct FkWeightS {
    _private: [u8; 0],
}
pub type FkWeight = *mut FkWeightS;
/// Opaque peer-memory communicator (`fk_comm`).
#[repr(C)]
pub struct FkComm {
    _private: [u8; 0],
}
/// `fk_matvec_launch`: one matvec of a multi-matvec call.
#[repr(C)]
#[derive(Clone, Copy)]
pub struct FkMatvecLaunch {
    pub kind: c_int,
    pub weights_host: *const u8,
    pub len: usize,
    pub rows: c_int,
    pub row_bytes: c_int,
    pub n_blocks_per_row: c_int,
}

/// `fk_status`.
pub const FK_OK: c_int = 0;
pub const FK_DRIVER_INIT: c_int = 1;
pub const FK_KERNEL: c_int = 2;
pub const FK_LAUNCH: c_int = 3;
pub const FK_UNSUPPORTED: c_int = 4;
pub const FK_COMM: c_int = 5;
pub const FK_INVALID: c_int = 6;

/// GGML type tags the library has kernels for.
pub const FK_Q8_0: c_int = 8;
pub const FK_Q4_K: c_int = 12;
pub const FK_Q5_K: c_int = 13;
pub const FK_Q6_K: c_int = 14;
pub const FK_MXFP4: c_int = 39;

extern "C" {
    pub fn fk_init(device: c_int, out: *mut *mut FkCtx) -> c_int;
    pub fn fk_destroy(ctx: *mut FkCtx);
    pub fn fk_last_error() -> *const c_char;
    pub fn fk_device_info(
        ctx: *mut FkCtx,
        name: *mut c_char,
        cap: usize,
        sm_count: *mut c_int,
        mem_bytes: *mut usize,
    ) -> c_int;
    pub fn fk_counters(
        ctx: *mut FkCtx,
        h2d_bytes: *mut u64,
        d2h_bytes: *mut u64,
        launches: *mut u64,
        reset: c_int,
    ) -> c_int;
    pub fn fk_device_error(ctx: *mut FkCtx, code: *mut c_int, reset: c_int) -> c_int;
    pub fn fk_block_bytes(kind: c_int) -> c_int;
    pub fn fk_block_elems(kind: c_int) -> c_int;
    pub fn fk_register_weights(
        ctx: *mut FkCtx,
        gguf_bytes_host: *const u8,
        len: usize,
        kind: c_int,
        n_mats: c_int,
        rows: c_int,
        cols: c_int,
        out: *mut FkWeight,
    ) -> c_int;
    pub fn fk_register_weights_dev(
        ctx: *mut FkCtx,
        gguf_bytes_dev: *const u8,
        len: usize,
        kind: c_int,
        n_mats: c_int,
        rows: c_int,
        cols: c_int,
        stream: *mut c_void,
        out: *mut FkWeight,
    ) -> c_int;
    pub fn fk_release_weights(ctx: *mut FkCtx, w: FkWeight) -> c_int;
    pub fn fk_weight_shape(
        w: FkWeight,
        kind: *mut c_int,
        n_mats: *mut c_int,
        rows: *mut c_int,
        cols: *mut c_int,
        gguf_bytes: *mut usize,
    ) -> c_int;
    pub fn fk_quantize_q8_1(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        x_dev: *const f32,
        n: c_int,
        y_dev: *mut u8,
    ) -> c_int;
    pub fn fk_quantize_q8_1_host(ctx: *mut FkCtx, x_host: *const f32, n: c_int, y_host: *mut u8) -> c_int;
    pub fn fk_gemv(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        w: FkWeight,
        mat: c_int,
        x_dev: *const f32,
        batch: c_int,
        y_dev: *mut f32,
    ) -> c_int;
    pub fn fk_gemv_fused(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        w: FkWeight,
        mat: c_int,
        x_dev: *const f32,
        x_ld: c_int,
        batch: c_int,
        y_dev: *mut f32,
        norm_weight_dev: *const f32,
        norm_eps: f32,
        glu_up_dev: *const f32,
        glu_act: c_int,
        accumulate: c_int,
        pair_glu: c_int,
    ) -> c_int;
    pub fn fk_gemv_multi(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        w: FkWeight,
        ids_dev: *const c_int,
        k: c_int,
        x_dev: *const f32,
        x_stride: c_int,
        y_dev: *mut f32,
    ) -> c_int;
    pub fn fk_gemv_multi_glu(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        w: FkWeight,
        ids_dev: *const c_int,
        k: c_int,
        gate_dev: *const f32,
        up_dev: *const f32,
        x_stride: c_int,
        glu_act: c_int,
        y_dev: *mut f32,
        n_active_dev: *const c_int,
    ) -> c_int;
    pub fn fk_gemv_multi_active(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        w: FkWeight,
        ids_dev: *const c_int,
        k: c_int,
        x_dev: *const f32,
        x_stride: c_int,
        y_dev: *mut f32,
        n_active_dev: *const c_int,
    ) -> c_int;
    pub fn fk_gemv_biased(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        w: FkWeight,
        mat: c_int,
        x_dev: *const f32,
        x_ld: c_int,
        batch: c_int,
        y_dev: *mut f32,
        norm_weight_dev: *const f32,
        norm_eps: f32,
        bias_dev: *const f32,
        accumulate: c_int,
    ) -> c_int;
    pub fn fk_gemv_multi_biased(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        w: FkWeight,
        ids_dev: *const c_int,
        k: c_int,
        x_dev: *const f32,
        up_dev: *const f32,
        x_stride: c_int,
        glu_act: c_int,
        bias_dev: *const f32,
        y_dev: *mut f32,
    ) -> c_int;
    pub fn fk_gemv_multi_gate_up(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        gate: FkWeight,
        up: FkWeight,
        ids_dev: *const c_int,
        k: c_int,
        x_dev: *const f32,
        x_stride: c_int,
        norm_weight_dev: *const f32,
        norm_eps: f32,
        gate_bias_dev: *const f32,
        up_bias_dev: *const f32,
        y_dev: *mut f32,
    ) -> c_int;
    pub fn fk_gemv_isums(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        w: FkWeight,
        mat: c_int,
        x_dev: *const f32,
        isums_dev: *mut i32,
    ) -> c_int;
    pub fn fk_gemm(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        w: FkWeight,
        mat: c_int,
        x_dev: *const f32,
        m: c_int,
        out_dev: *mut f32,
    ) -> c_int;
    pub fn fk_gemm_isums(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        w: FkWeight,
        mat: c_int,
        x_dev: *const f32,
        m: c_int,
        out_dev: *mut f32,
        isums_dev: *mut i32,
    ) -> c_int;
    pub fn fk_gemm_q8k(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        w: FkWeight,
        mat: c_int,
        x_dev: *const f32,
        m: c_int,
        out_dev: *mut f32,
    ) -> c_int;
    pub fn fk_gemm_q8k_isums(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        w: FkWeight,
        mat: c_int,
        x_dev: *const f32,
        m: c_int,
        out_dev: *mut f32,
        isums_dev: *mut i32,
    ) -> c_int;
    pub fn fk_gemm_static(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        w: FkWeight,
        mat: c_int,
        x_dev: *const f32,
        m: c_int,
        out_dev: *mut f32,
    ) -> c_int;
    pub fn fk_gemm_grouped(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        w: FkWeight,
        group_off_dev: *const c_int,
        gather_dev: *const c_int,
        x_dev: *const f32,
        pairs: c_int,
        out_dev: *mut f32,
    ) -> c_int;
    pub fn fk_moe_route(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        logits_dev: *const f32,
        bias_dev: *const f32,
        n_experts: c_int,
        k: c_int,
        mode: c_int,
        batch: c_int,
        ids_dev: *mut c_int,
        w_dev: *mut f32,
    ) -> c_int;
    pub fn fk_router_route(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        router_dev: *const f32,
        x_dev: *const f32,
        n_experts: c_int,
        cols: c_int,
        batch: c_int,
        bias_dev: *const f32,
        k: c_int,
        mode: c_int,
        logits_dev: *mut f32,
        ids_dev: *mut c_int,
        w_dev: *mut f32,
    ) -> c_int;
    pub fn fk_router_logits(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        router_dev: *const f32,
        x_dev: *const f32,
        n_experts: c_int,
        cols: c_int,
        batch: c_int,
        logits_dev: *mut f32,
    ) -> c_int;
    pub fn fk_moe_permute(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        ids_dev: *const c_int,
        pairs: c_int,
        k: c_int,
        n_experts: c_int,
        group_off_dev: *mut c_int,
        gather_dev: *mut c_int,
        pair_of_dev: *mut c_int,
    ) -> c_int;
    pub fn fk_moe_local_slots(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        ids_dev: *const c_int,
        w_dev: *const f32,
        k: c_int,
        e0: c_int,
        n_local: c_int,
        out_ids_dev: *mut c_int,
        out_w_dev: *mut f32,
        out_n_dev: *mut c_int,
    ) -> c_int;
    pub fn fk_moe_local_pairs(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        ids_dev: *const c_int,
        w_dev: *const f32,
        pairs: c_int,
        k: c_int,
        e0: c_int,
        n_local: c_int,
        out_ids_dev: *mut c_int,
        out_src_dev: *mut c_int,
        out_pair_of_dev: *mut c_int,
        out_w_dev: *mut f32,
        out_n_dev: *mut c_int,
    ) -> c_int;
    pub fn fk_moe_localize(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        ids_dev: *const c_int,
        w_dev: *const f32,
        pairs: c_int,
        e0: c_int,
        n_local: c_int,
        out_ids_dev: *mut c_int,
        out_w_dev: *mut f32,
    ) -> c_int;
    pub fn fk_glu(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        gate_dev: *const f32,
        up_dev: *const f32,
        n: usize,
        act: c_int,
        out_dev: *mut f32,
    ) -> c_int;
    pub fn fk_moe_combine(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        y_dev: *const f32,
        pair_of_dev: *const c_int,
        w_dev: *const f32,
        batch: c_int,
        k: c_int,
        n: c_int,
        out_dev: *mut f32,
    ) -> c_int;
    pub fn fk_moe_combine_add(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        y_dev: *const f32,
        pair_of_dev: *const c_int,
        w_dev: *const f32,
        batch: c_int,
        k: c_int,
        n: c_int,
        out_dev: *mut f32,
    ) -> c_int;
    pub fn fk_moe_layer_workspace(n_experts: c_int, k: c_int, hidden: c_int, ffn: c_int, batch: c_int) -> usize;
    pub fn fk_moe_layer(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        router_dev: *const f32,
        router_bias_dev: *const f32,
        gate: FkWeight,
        up: FkWeight,
        down: FkWeight,
        k: c_int,
        mode: c_int,
        act: c_int,
        x_dev: *const f32,
        batch: c_int,
        out_dev: *mut f32,
        accumulate: c_int,
        workspace_dev: *mut c_void,
        workspace_bytes: usize,
    ) -> c_int;
    pub fn fk_moe_layer_biased(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        router_dev: *const f32,
        router_bias_dev: *const f32,
        gate: FkWeight,
        up: FkWeight,
        down: FkWeight,
        gate_bias_dev: *const f32,
        up_bias_dev: *const f32,
        down_bias_dev: *const f32,
        k: c_int,
        mode: c_int,
        act: c_int,
        x_dev: *const f32,
        batch: c_int,
        out_dev: *mut f32,
        accumulate: c_int,
        workspace_dev: *mut c_void,
        workspace_bytes: usize,
    ) -> c_int;
    pub fn fk_moe_layer_normed(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        router_dev: *const f32,
        router_bias_dev: *const f32,
        gate: FkWeight,
        up: FkWeight,
        down: FkWeight,
        gate_bias_dev: *const f32,
        up_bias_dev: *const f32,
        down_bias_dev: *const f32,
        k: c_int,
        mode: c_int,
        act: c_int,
        norm_weight_dev: *const f32,
        norm_eps: f32,
        x_dev: *const f32,
        batch: c_int,
        out_dev: *mut f32,
        accumulate: c_int,
        workspace_dev: *mut c_void,
        workspace_bytes: usize,
    ) -> c_int;
    pub fn fk_get_rows(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        w: FkWeight,
        mat: c_int,
        ids_dev: *const c_int,
        n: c_int,
        out_dev: *mut f32,
    ) -> c_int;
    pub fn fk_rmsnorm(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        x_dev: *mut f32,
        residual_dev: *const f32,
        weight_dev: *const f32,
        n_rows: c_int,
        cols: c_int,
        eps: f32,
        out_dev: *mut f32,
    ) -> c_int;
    pub fn fk_rope(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        x_dev: *mut f32,
        n_rows: c_int,
        n_heads: c_int,
        head_dim: c_int,
        pos_dev: *const c_int,
        theta: f32,
        neox: c_int,
    ) -> c_int;
    pub fn fk_rope_kv(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        q_dev: *mut f32,
        k_dev: *mut f32,
        v_dev: *const f32,
        q_ld: c_int,
        kv_ld: c_int,
        n_rows: c_int,
        n_heads: c_int,
        n_kv: c_int,
        head_dim: c_int,
        pos_dev: *const c_int,
        theta: f32,
        neox: c_int,
        k_cache_dev: *mut f32,
        v_cache_dev: *mut f32,
        q_norm_dev: *const f32,
        k_norm_dev: *const f32,
        norm_eps: f32,
        cache_rows: c_int,
    ) -> c_int;
    pub fn fk_reserve_scratch(ctx: *mut FkCtx, bytes: usize) -> c_int;
    pub fn fk_add_bias(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        y_dev: *mut f32,
        bias_dev: *const f32,
        ids_dev: *const c_int,
        n_rows: c_int,
        cols: c_int,
    ) -> c_int;
    pub fn fk_add(ctx: *mut FkCtx, stream: *mut c_void, a_dev: *mut f32, b_dev: *const f32, n: usize) -> c_int;
    pub fn fk_kv_append(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        cache_dev: *mut f32,
        src_dev: *const f32,
        row_elems: usize,
        n_rows: c_int,
        pos_dev: *const c_int,
        cache_rows: c_int,
    ) -> c_int;
    pub fn fk_attention(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        q_dev: *const f32,
        q_ld: c_int,
        k_dev: *const f32,
        v_dev: *const f32,
        n_q: c_int,
        n_heads: c_int,
        n_kv: c_int,
        head_dim: c_int,
        pos_dev: *const c_int,
        scale: f32,
        out_dev: *mut f32,
        cache_rows: c_int,
        window: c_int,
        sinks_dev: *const f32,
    ) -> c_int;
    pub fn fk_attention_rope_kv(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        q_dev: *const f32,
        k_new_dev: *const f32,
        v_new_dev: *const f32,
        k_cache_dev: *mut f32,
        v_cache_dev: *mut f32,
        n_heads: c_int,
        n_kv: c_int,
        head_dim: c_int,
        pos_dev: *const c_int,
        scale: f32,
        theta: f32,
        neox: c_int,
        q_norm_dev: *const f32,
        k_norm_dev: *const f32,
        norm_eps: f32,
        out_dev: *mut f32,
        cache_rows: c_int,
        window: c_int,
        sinks_dev: *const f32,
    ) -> c_int;
    pub fn fk_attention_rope_kv_seqs(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        q_dev: *const f32,
        q_ld: c_int,
        k_new_dev: *const f32,
        v_new_dev: *const f32,
        k_ld: c_int,
        v_ld: c_int,
        k_cache_dev: *mut f32,
        v_cache_dev: *mut f32,
        seq_stride: usize,
        n_seqs: c_int,
        n_heads: c_int,
        n_kv: c_int,
        head_dim: c_int,
        pos_dev: *const c_int,
        scale: f32,
        theta: f32,
        neox: c_int,
        q_norm_dev: *const f32,
        k_norm_dev: *const f32,
        norm_eps: f32,
        out_dev: *mut f32,
        cache_rows: c_int,
        window: c_int,
        sinks_dev: *const f32,
    ) -> c_int;
    pub fn fk_argmax(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        x_dev: *const f32,
        n_rows: c_int,
        n: c_int,
        out_dev: *mut c_int,
    ) -> c_int;
    pub fn fk_add_int(ctx: *mut FkCtx, stream: *mut c_void, p_dev: *mut c_int, v: c_int) -> c_int;
    pub fn fk_comm_create(
        ctx: *mut FkCtx,
        arena_bytes: usize,
        rank: c_int,
        world: c_int,
        handle_out_64: *mut u8,
        out: *mut *mut FkComm,
    ) -> c_int;
    pub fn fk_comm_connect(comm: *mut FkComm, handles_world_x_64: *const u8) -> c_int;
    pub fn fk_comm_connect_local(comm: *mut FkComm, peer_arenas_dev: *const *mut c_void) -> c_int;
    pub fn fk_comm_arena(comm: *mut FkComm, arena_dev: *mut *mut c_void, bytes: *mut usize) -> c_int;
    pub fn fk_comm_destroy(comm: *mut FkComm) -> c_int;
    pub fn fk_comm_channel_bytes(world: c_int, n_max: c_int) -> usize;
    pub fn fk_allreduce(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        comm: *mut FkComm,
        channel_off: usize,
        n_max: c_int,
        src_dev: *const f32,
        dst_dev: *mut f32,
        n: c_int,
        accumulate: c_int,
        timeout_us: c_int,
    ) -> c_int;
    pub fn fk_gemv_fused_allreduce(
        ctx: *mut FkCtx,
        stream: *mut c_void,
        w: FkWeight,
        mat: c_int,
        x_dev: *const f32,
        x_ld: c_int,
        batch: c_int,
        y_dev: *mut f32,
        norm_weight_dev: *const f32,
        norm_eps: f32,
        glu_up_dev: *const f32,
        glu_act: c_int,
        accumulate: c_int,
        comm: *mut FkComm,
        channel_off: usize,
        n_max: c_int,
        timeout_us: c_int,
    ) -> c_int;
    pub fn fk_launch_matvec(
        ctx: *mut FkCtx,
        kind: c_int,
        weights_host: *const u8,
        len: usize,
        x_host: *const f32,
        rows: c_int,
        row_bytes: c_int,
        n_blocks_per_row: c_int,
        y_host: *mut f32,
    ) -> c_int;
    pub fn fk_launch_matvec_multi(
        ctx: *mut FkCtx,
        x_host: *const f32,
        n_cols: c_int,
        launches: *const FkMatvecLaunch,
        n: c_int,
        y_hosts: *const *mut f32,
    ) -> c_int;
    pub fn fk_launch_dense_ffn_swiglu(
        ctx: *mut FkCtx,
        gate: *const FkMatvecLaunch,
        up: *const FkMatvecLaunch,
        down: *const FkMatvecLaunch,
        x_host: *const f32,
        n_cols: c_int,
        y_host: *mut f32,
    ) -> c_int;
    pub fn fk_launch_mul_mm(
        ctx: *mut FkCtx,
        kind: c_int,
        weights_host: *const u8,
        len: usize,
        x_batch_host: *const f32,
        n_rows: c_int,
        n_cols: c_int,
        batch: c_int,
        row_bytes: c_int,
        out_host: *mut f32,
    ) -> c_int;
    pub fn fk_forget_resident(ctx: *mut FkCtx) -> c_int;
}
