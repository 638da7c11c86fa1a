//! `frink_cuda::mul_mm_launch::launch_mul_mm` (reference: crates/frink-cuda/src/mul_mm_launch.rs:40-68).
use frink_b200_sys as sys;

use crate::gpu::{ctx, status, CudaError};
use crate::mul_mm::{validate_shape, MulMmKind};

/// `out[b][r] = sum_c W[r][c] x_batch[b][c]` for a batch of activation rows; weights resident by pointer and length.
/// Batches of up to 8 rows take the matvec path inside the library, larger ones the tensor-core GEMM.
pub fn launch_mul_mm(kind: &MulMmKind, weights: &[u8], x_batch: &[f32], n_rows: usize, n_cols: usize, batch: usize, row_bytes: usize) -> Result<Vec<f32>, CudaError> {
    validate_shape(kind, n_rows, n_cols, batch, row_bytes).map_err(CudaError::Launch)?;
    if x_batch.len() != batch * n_cols || weights.len() != n_rows * row_bytes {
        return Err(CudaError::Launch(format!("{}: {} activations for {batch} x {n_cols}, {} weight bytes for {n_rows} x {row_bytes}", kind.name, x_batch.len(), weights.len())));
    }
    let mut out = vec![0f32; batch * n_rows];
    // SAFETY: sizes checked above; the call synchronizes before it returns.
    status(unsafe {
        sys::fk_launch_mul_mm(ctx()?, kind.tag, weights.as_ptr(), weights.len(), x_batch.as_ptr(), n_rows as i32, n_cols as i32, batch as i32, row_bytes as i32, out.as_mut_ptr())
    })?;
    Ok(out)
}
