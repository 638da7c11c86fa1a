//! `frink_cuda::mul_mm`: the prefill GEMM's kind table and the batch threshold
//! (reference: crates/frink-cuda/src/mul_mm.rs:154-190, 258, 282-296, 634).
use frink_b200_sys as sys;

#[derive(Debug, Clone, Copy)]
pub struct MulMmKind {
    pub name: &'static str,
    pub module_name: &'static str,
    pub fn_name: &'static str,
    pub block_bytes: usize,
    pub block_elems: usize,
    /// GGML type tag = the library's `fk_kind`.
    pub tag: i32,
}

pub const KINDS: &[MulMmKind] = &[
    MulMmKind { name: "Q4_K", module_name: "frink_b200", fn_name: "mul_mm_q4_k", block_bytes: 144, block_elems: 256, tag: sys::FK_Q4_K },
    MulMmKind { name: "Q6_K", module_name: "frink_b200", fn_name: "mul_mm_q6_k", block_bytes: 210, block_elems: 256, tag: sys::FK_Q6_K },
    MulMmKind { name: "Q8_0", module_name: "frink_b200", fn_name: "mul_mm_q8_0", block_bytes: 34, block_elems: 32, tag: sys::FK_Q8_0 },
    MulMmKind { name: "MXFP4", module_name: "frink_b200", fn_name: "mul_mm_mxfp4", block_bytes: 17, block_elems: 32, tag: sys::FK_MXFP4 },
];

pub fn kind_by_name(name: &str) -> Option<&'static MulMmKind> {
    KINDS.iter().find(|k| k.name.eq_ignore_ascii_case(name))
}

/// From this batch on a GEMM beats repeated matvecs.  The matvec here reads the weights once for up to 8 rows, so the
/// threshold is 9 (the reference's own value is lower: its matvec reads the weights once per row).
pub fn worth_a_gemm(batch: usize) -> bool {
    batch > 8
}

/// Shapes the GEMM takes: whole blocks per row, a row size that matches them.
pub fn validate_shape(kind: &MulMmKind, n_rows: usize, n_cols: usize, batch: usize, row_bytes: usize) -> Result<(), String> {
    if n_rows == 0 || batch == 0 || n_cols == 0 || n_cols % kind.block_elems != 0 {
        return Err(format!("{}: {n_rows} x {n_cols}, batch {batch}: columns must be whole blocks of {}", kind.name, kind.block_elems));
    }
    if row_bytes != n_cols / kind.block_elems * kind.block_bytes {
        return Err(format!("{}: row_bytes {row_bytes} does not match {n_cols} columns", kind.name));
    }
    Ok(())
}

/// IEEE half to f32.
pub fn f16_to_f32(bits: u16) -> f32 {
    let sign = ((bits & 0x8000) as u32) << 16;
    let exp = ((bits >> 10) & 0x1f) as u32;
    let man = (bits & 0x3ff) as u32;
    let word = match (exp, man) {
        (0, 0) => sign,
        (0, m) => {
            let shift = m.leading_zeros() - 21; // bring the leading one to bit 10
            sign | ((127 - 15 + 1 - shift) << 23) | (((m << shift) & 0x3ff) << 13)
        }
        (31, m) => sign | 0x7f80_0000 | (m << 13),
        (e, m) => sign | ((e + 127 - 15) << 23) | (m << 13),
    };
    f32::from_bits(word)
}
