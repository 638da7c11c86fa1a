//! Drop-in for `frink-cuda` on the dequantize-inside-the-matmul path: the module paths, names, signatures and
//! error enum that `frink-core` calls (`crates/frink-core/src/weight_matrix/gpu_backend.rs:247-273,438-712`),
//! with bodies that call `libfrink_b200.so` through `frink-b200-sys`.
//!
//! Only the four kinds with kernels in the library are listed in the tables (`Q4_K`, `Q6_K`, `Q8_0`, `MXFP4`);
//! `frink-core` derives its capability set from the tables and sends every other kind to its next backend.
//!
//! This crate has not been compiled where it was written (no Rust toolchain there); the same calls are tested
//! through the library's C ABI from C++ and Python.
pub mod gpu;
pub mod matvec_kinds;
pub mod matvec_launch;
pub mod mul_mm;
pub mod mul_mm_launch;
pub mod prefill;

pub use gpu::CudaError;
