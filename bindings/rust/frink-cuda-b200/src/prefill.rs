//! `frink_cuda::prefill` (the resident stack: crates/frink-cuda/src/prefill/moe_device.rs:241-438, layer.rs:44):
//! weights registered once and kept on the device, activations as device pointers on a caller's stream.
//! The routed layer is one call here; the pieces it is made of are in `frink-b200-sys` for callers that shard
//! the experts over devices.
//!
//! Device pointers are raw (`*const f32` / `*mut f32`): this crate owns no device memory besides the weights,
//! the caller's allocator does (as `frink-cuda`'s `DeviceBuffer`s do in the reference).
use std::ffi::c_void;

use frink_b200_sys as sys;

use crate::gpu::{ctx, status, CudaError};

/// A stack of `n_mats` matrices of one block format, resident on the device (`fk_register_weights`): what the
/// reference keeps per tensor in `resident.rs`.  Released on drop.
pub struct ResidentWeights {
    handle: sys::FkWeight,
}

// SAFETY: the handle is an opaque pointer into the library, which serialises what must be serialised.
unsafe impl Send for ResidentWeights {}
unsafe impl Sync for ResidentWeights {}

impl ResidentWeights {
    /// `gguf` are the tensor's GGUF bytes: `n_mats` matrices of `rows` x `cols`, `tag` the GGML type tag.
    pub fn new(gguf: &[u8], tag: i32, n_mats: usize, rows: usize, cols: usize) -> Result<Self, CudaError> {
        let mut handle: sys::FkWeight = std::ptr::null_mut();
        // SAFETY: the slice outlives the call (the bytes are copied to the device before it returns).
        status(unsafe {
            sys::fk_register_weights(ctx()?, gguf.as_ptr(), gguf.len(), tag, n_mats as i32, rows as i32, cols as i32, &mut handle)
        })?;
        Ok(Self { handle })
    }

    pub(crate) fn raw(&self) -> sys::FkWeight {
        self.handle
    }
}

impl Drop for ResidentWeights {
    fn drop(&mut self) {
        if let Ok(c) = ctx() {
            // SAFETY: a handle this context made, released once.
            unsafe { sys::fk_release_weights(c, self.handle) };
        }
    }
}

/// The bias tables of gpt-oss's experts (`run_expert_oai`, crates/frink-moe/src/lib.rs:1039-1060), device pointers:
/// `[n_experts][ffn]`, `[n_experts][ffn]`, `[n_experts][hidden]`.
#[derive(Clone, Copy)]
pub struct ExpertBiases {
    pub gate: *const f32,
    pub up: *const f32,
    pub down: *const f32,
}

/// One routed layer, resident: the router matrix (f32 `[n_experts][hidden]`, device pointer, with its optional
/// bias), the three expert stacks, the routing rule and the activation (`0` SiLU, `1` the clamped gpt-oss form).
pub struct MoeLayer {
    pub router: *const f32,
    pub router_bias: *const f32, // null: none
    pub gate: ResidentWeights,
    pub up: ResidentWeights,
    pub down: ResidentWeights,
    pub biases: Option<ExpertBiases>,
    pub n_experts: usize,
    pub hidden: usize,
    pub ffn: usize,
    pub k: usize,
    pub mode: i32,
    pub act: i32,
}

impl MoeLayer {
    /// Bytes of 256-byte-aligned device workspace a call with `batch` rows needs (`fk_moe_layer_workspace`).
    pub fn workspace_bytes(&self, batch: usize) -> usize {
        // SAFETY: a pure function of its arguments.
        unsafe { sys::fk_moe_layer_workspace(self.n_experts as i32, self.k as i32, self.hidden as i32, self.ffn as i32, batch as i32) }
    }

    /// `out[batch][hidden]` = (or `+=` with `accumulate`) the layer applied to `x[batch][hidden]`, both on the device.
    /// Up to 8 rows take the indexed matvecs, more the grouped GEMMs.
    ///
    /// # Safety
    /// `x`, `out`, `workspace` and the layer's pointers must be device memory of this process's context, of the sizes
    /// named above, and must stay valid until `stream` has run the call.
    pub unsafe fn run(&self, stream: *mut c_void, x: *const f32, batch: usize, out: *mut f32, accumulate: bool, workspace: *mut c_void,
                      workspace_bytes: usize) -> Result<(), CudaError> {
        let c = ctx()?;
        let rc = match self.biases {
            None => sys::fk_moe_layer(c, stream, self.router, self.router_bias, self.gate.raw(), self.up.raw(), self.down.raw(), self.k as i32,
                                      self.mode, self.act, x, batch as i32, out, accumulate as i32, workspace, workspace_bytes),
            Some(b) => sys::fk_moe_layer_biased(c, stream, self.router, self.router_bias, self.gate.raw(), self.up.raw(), self.down.raw(), b.gate,
                                                b.up, b.down, self.k as i32, self.mode, self.act, x, batch as i32, out, accumulate as i32,
                                                workspace, workspace_bytes),
        };
        status(rc)
    }

    /// The decode form on the RESIDUAL stream (at most 8 rows): `x` is un-normalized, the layer's RMSNorm (`norm_weight`,
    /// `eps`) is folded into the router and the gate / up launch, and the result is added into `x` itself -- four launches.
    ///
    /// # Safety
    /// As `run`; `x` is read and written.
    pub unsafe fn run_on_residual(&self, stream: *mut c_void, x: *mut f32, batch: usize, norm_weight: *const f32, eps: f32, workspace: *mut c_void,
                                  workspace_bytes: usize) -> Result<(), CudaError> {
        let (gb, ub, db) = match self.biases {
            Some(b) => (b.gate, b.up, b.down),
            None => (std::ptr::null(), std::ptr::null(), std::ptr::null()),
        };
        status(sys::fk_moe_layer_normed(ctx()?, stream, self.router, self.router_bias, self.gate.raw(), self.up.raw(), self.down.raw(), gb, ub, db,
                                        self.k as i32, self.mode, self.act, norm_weight, eps, x as *const f32, batch as i32, x, 1, workspace,
                                        workspace_bytes))
    }
}

/// The device's error word (bounded waits that gave up, a KV cache that would overflow): 0 = none.  `reset` clears it.
pub fn device_error(reset: bool) -> Result<i32, CudaError> {
    let mut code = 0i32;
    // SAFETY: `code` is a valid out-pointer.
    status(unsafe { sys::fk_device_error(ctx()?, &mut code, reset as i32) })?;
    Ok(code)
}
