//! `frink_cuda::matvec_launch`: several matvecs over one upload of the activation, and the dense SwiGLU FFN
//! on the device (reference: crates/frink-cuda/src/matvec_launch.rs:485-574).
use frink_b200_sys as sys;

use crate::gpu::{ctx, status, CudaError};
use crate::matvec_kinds;

/// One matvec of a multi-matvec call.  `kernel_src` and `module_name` belong to the reference's run-time compiler
/// and are kept so that call sites compile unchanged; the kind is looked up by `fn_name`.
/// `weights` must be a stable slice (the mmap'd tensor), never a per-call copy: residency is keyed by pointer and length.
#[derive(Clone, Copy)]
pub struct MatvecLaunch<'a> {
    pub kernel_src: &'static str,
    pub module_name: &'static str,
    pub fn_name: &'static str,
    pub weights: &'a [u8],
    pub rows: usize,
    pub row_bytes: usize,
    pub n_blocks_per_row: usize,
}

fn c_launch(l: &MatvecLaunch<'_>) -> Result<sys::FkMatvecLaunch, CudaError> {
    let kind = matvec_kinds::kind_by_name(l.fn_name).ok_or_else(|| CudaError::Unsupported(format!("no kernel for {}", l.fn_name)))?;
    Ok(sys::FkMatvecLaunch {
        kind: kind.tag,
        weights_host: l.weights.as_ptr(),
        len: l.weights.len(),
        rows: l.rows as i32,
        row_bytes: l.row_bytes as i32,
        n_blocks_per_row: l.n_blocks_per_row as i32,
    })
}

/// `x` goes up once, the matvecs are enqueued back to back on resident weights, every result comes down.
pub fn launch_matvec_multi(x: &[f32], launches: &[MatvecLaunch<'_>]) -> Result<Vec<Vec<f32>>, CudaError> {
    if launches.is_empty() {
        return Ok(Vec::new());
    }
    let cl = launches.iter().map(c_launch).collect::<Result<Vec<_>, _>>()?;
    let mut outs: Vec<Vec<f32>> = launches.iter().map(|l| vec![0f32; l.rows]).collect();
    let ptrs: Vec<*mut f32> = outs.iter_mut().map(|o| o.as_mut_ptr()).collect();
    // SAFETY: every pointer is valid for the sizes the descriptions state; the call synchronizes before it returns.
    status(unsafe { sys::fk_launch_matvec_multi(ctx()?, x.as_ptr(), x.len() as i32, cl.as_ptr(), cl.len() as i32, ptrs.as_ptr()) })?;
    Ok(outs)
}

/// `down (SiLU(gate x) * (up x))` with one upload of `x` and one download of the result.
pub fn launch_dense_ffn_swiglu(gate: &MatvecLaunch<'_>, up: &MatvecLaunch<'_>, down: &MatvecLaunch<'_>, x: &[f32]) -> Result<Vec<f32>, CudaError> {
    let (g, u, d) = (c_launch(gate)?, c_launch(up)?, c_launch(down)?);
    let mut y = vec![0f32; down.rows];
    // SAFETY: as above.
    status(unsafe { sys::fk_launch_dense_ffn_swiglu(ctx()?, &g, &u, &d, x.as_ptr(), x.len() as i32, y.as_mut_ptr()) })?;
    Ok(y)
}
