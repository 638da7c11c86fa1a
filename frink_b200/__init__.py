"""frink_b200: a B200 (sm_100a) backend for frink's dequantize-inside-the-matmul path.

The compute lives in `libfrink_b200.so` (hand-written CUDA behind the C ABI of
`include/frink_b200.h`).  The modules here mirror the launch surface frink-core
binds of frink-cuda (`gpu`, `matvec_kinds`, `mul_mm`, `mul_mm_launch`, `prefill`)
plus a device-tensor layer (`device`) and the multi-GPU sharding (`parallel`).
"""
from ._lib import CudaError, DriverInit, Invalid, KernelCompile, Launch, Unsupported  # noqa: F401

Q8_0, Q4_K, Q6_K, MXFP4 = 8, 12, 14, 39
__all__ = ["Q8_0", "Q4_K", "Q6_K", "MXFP4", "CudaError", "DriverInit", "KernelCompile", "Launch", "Unsupported", "Invalid"]
