//! `frink_cuda::matvec_kinds`: the table `frink-core` derives its decode capability set from
//! (reference: crates/frink-cuda/src/matvec_kinds/mod.rs:50-60, 102, 240).
use frink_b200_sys as sys;

#[derive(Debug, Clone, Copy)]
pub struct MatvecKind {
    /// GGUF quant name, `QuantKind::name()`.
    pub name: &'static str,
    /// Kept for call sites; nothing is compiled at run time here.
    pub module_name: &'static str,
    /// The reference kernel this library's kernel stands in for.
    pub fn_name: &'static str,
    /// GGML type tag = the library's `fk_kind`.
    pub tag: i32,
    pub block_bytes: usize,
    pub block_elems: usize,
}

pub const KINDS: &[MatvecKind] = &[
    MatvecKind { name: "Q4_K", module_name: "frink_b200", fn_name: "q4_k_matvec", tag: sys::FK_Q4_K, block_bytes: 144, block_elems: 256 },
    MatvecKind { name: "Q5_K", module_name: "frink_b200", fn_name: "q5_k_matvec", tag: sys::FK_Q5_K, block_bytes: 176, block_elems: 256 },
    MatvecKind { name: "Q6_K", module_name: "frink_b200", fn_name: "q6_k_matvec", tag: sys::FK_Q6_K, block_bytes: 210, block_elems: 256 },
    MatvecKind { name: "Q8_0", module_name: "frink_b200", fn_name: "q8_0_matvec", tag: sys::FK_Q8_0, block_bytes: 34, block_elems: 32 },
    MatvecKind { name: "MXFP4", module_name: "frink_b200", fn_name: "mxfp4_matvec", tag: sys::FK_MXFP4, block_bytes: 17, block_elems: 32 },
];

/// By quant name or by kernel name (with or without the reference's `_dp4a` suffix); `None` = no kernel here.
pub fn kind_by_name(name: &str) -> Option<&'static MatvecKind> {
    let key = name.to_ascii_lowercase();
    let key = key.strip_suffix("_dp4a").unwrap_or(&key);
    KINDS.iter().find(|k| k.name.eq_ignore_ascii_case(key) || k.fn_name == key)
}

pub mod dp4a {
    //! What a decode matvec reads of its input (reference: matvec_kinds/dp4a.rs:291-303).
    use frink_b200_sys as sys;

    use crate::gpu::{ctx, status, CudaError};

    /// The q8_1 rounding of `x`, run by run of 32, as the kernels read it -- obtained from the library's own
    /// quantizer (`fk_quantize_q8_1` through device buffers), so a test that compares against "what the kernel
    /// read" uses the kernel's bytes.  Inputs that are not whole runs come back unchanged.
    pub fn matvec_reads(fn_name: &str, _n_blocks: usize, x: &[f32]) -> Result<Vec<f32>, CudaError> {
        if super::kind_by_name(fn_name).is_none() || x.len() % 32 != 0 {
            return Ok(x.to_vec());
        }
        let mut blocks = vec![0u8; x.len() / 32 * 36];
        // SAFETY: `blocks` holds 36 bytes per run of 32 values.
        status(unsafe { sys::fk_quantize_q8_1_host(ctx()?, x.as_ptr(), x.len() as i32, blocks.as_mut_ptr()) })?;
        let mut out = Vec::with_capacity(x.len());
        for b in blocks.chunks_exact(36) {
            let d = crate::mul_mm::f16_to_f32(u16::from_le_bytes([b[0], b[1]]));
            out.extend(b[4..].iter().map(|&q| d * (q as i8) as f32));
        }
        Ok(out)
    }
}
