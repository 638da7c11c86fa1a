//! `frink_cuda::gpu`: the error type, the process-wide device and the per-kind host-buffer matvecs
//! (reference: crates/frink-cuda/src/gpu.rs:91-104, 172-222, 319-446).
use std::ffi::CStr;
use std::sync::OnceLock;

use frink_b200_sys as sys;

pub use crate::matvec_launch::{launch_dense_ffn_swiglu, launch_matvec_multi, MatvecLaunch};

/// Same variants and meaning as the reference's `CudaError`.  `Unsupported` keeps its contract: the caller must use
/// a path that can compute the result, never something else.
#[derive(Debug, thiserror::Error)]
pub enum CudaError {
    #[error("CUDA driver init: {0}")]
    DriverInit(String),
    #[error("kernel: {0}")]
    KernelCompile(String),
    #[error("launch: {0}")]
    Launch(String),
    #[error("unsupported on the CUDA path: {0}")]
    Unsupported(String),
}

/// An `fk_status` as a `Result`; the message is the library's (`fk_last_error`, per thread).
pub(crate) fn status(rc: i32) -> Result<(), CudaError> {
    if rc == sys::FK_OK {
        return Ok(());
    }
    // SAFETY: fk_last_error returns a NUL-terminated string owned by the library, valid until this thread's next call.
    let msg = unsafe { CStr::from_ptr(sys::fk_last_error()) }.to_string_lossy().into_owned();
    Err(match rc {
        sys::FK_DRIVER_INIT => CudaError::DriverInit(msg),
        sys::FK_KERNEL => CudaError::KernelCompile(msg),
        sys::FK_UNSUPPORTED => CudaError::Unsupported(msg),
        _ => CudaError::Launch(msg), // FK_LAUNCH, FK_COMM, FK_INVALID
    })
}

struct Ctx(*mut sys::FkCtx);
// SAFETY: the library serialises what must be serialised on a context (see the header's threading note).
unsafe impl Send for Ctx {}
unsafe impl Sync for Ctx {}

/// The process-wide context of device 0 (`gpu::shared_device`): created on first use, kept for the process.
pub(crate) fn ctx() -> Result<*mut sys::FkCtx, CudaError> {
    static CTX: OnceLock<Result<Ctx, String>> = OnceLock::new();
    let got = CTX.get_or_init(|| {
        let mut p: *mut sys::FkCtx = std::ptr::null_mut();
        // SAFETY: `p` is a valid out-pointer.
        match status(unsafe { sys::fk_init(0, &mut p) }) {
            Ok(()) => Ok(Ctx(p)),
            Err(e) => Err(e.to_string()),
        }
    });
    match got {
        Ok(c) => Ok(c.0),
        Err(m) => Err(CudaError::DriverInit(m.clone())),
    }
}

fn launch_matvec(tag: i32, weights: &[u8], x: &[f32], rows: usize, row_bytes: usize, n_blocks_per_row: usize) -> Result<Vec<f32>, CudaError> {
    let mut y = vec![0f32; rows];
    // SAFETY: the slices outlive the call (it synchronizes before returning); `y` holds `rows` floats.
    status(unsafe {
        sys::fk_launch_matvec(ctx()?, tag, weights.as_ptr(), weights.len(), x.as_ptr(), rows as i32, row_bytes as i32, n_blocks_per_row as i32, y.as_mut_ptr())
    })?;
    Ok(y)
}

macro_rules! matvec {
    ($name:ident, $tag:expr) => {
        /// Same contract as the reference's function of this name (gpu.rs:319-446): `weights` are the tensor's GGUF
        /// bytes (kept resident by pointer and length), `x` one activation row, the result `rows` floats.
        pub fn $name(weights: &[u8], x: &[f32], rows: usize, row_bytes: usize, n_blocks_per_row: usize) -> Result<Vec<f32>, CudaError> {
            launch_matvec($tag, weights, x, rows, row_bytes, n_blocks_per_row)
        }
    };
}
matvec!(launch_q8_0_matvec, sys::FK_Q8_0);
matvec!(launch_q4_k_matvec, sys::FK_Q4_K);
matvec!(launch_q5_k_matvec, sys::FK_Q5_K);
matvec!(launch_q6_k_matvec, sys::FK_Q6_K);
matvec!(launch_mxfp4_matvec, sys::FK_MXFP4);

/// Drops every resident weight buffer (the reference's cache clear on model unload).
pub fn forget_resident() -> Result<(), CudaError> {
    // SAFETY: a valid context.
    status(unsafe { sys::fk_forget_resident(ctx()?) })
}
