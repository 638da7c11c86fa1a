"""`frink_cuda::mul_mm_launch::launch_mul_mm` (crates/frink-cuda/src/mul_mm_launch.rs:40-68)."""
import ctypes as C

import numpy as np

from . import _lib, mul_mm
from ._lib import check, lib


def launch_mul_mm(kind, weights, x_batch, n_rows, n_cols, batch, row_bytes):
    """Host slices in, `out[token * n_rows + row]` out.  `kind` is a `MulMmKind`
    or its name."""
    k = kind if hasattr(kind, "tag") else mul_mm.kind_by_name(kind)
    if k is None:
        raise _lib.Unsupported(f"no GEMM for {kind}")
    from . import device
    w = np.ascontiguousarray(weights, np.uint8)
    x = np.ascontiguousarray(x_batch, np.float32)
    if x.size != batch * n_cols:
        raise _lib.Invalid(f"x_batch has {x.size} values, {batch} x {n_cols} wanted")
    out = np.empty(batch * n_rows, np.float32)
    check(lib().fk_launch_mul_mm(device.context(), k.tag, w.ctypes.data_as(C.c_void_p), w.size, x.ctypes.data_as(C.c_void_p),
                                 n_rows, n_cols, batch, row_bytes, out.ctypes.data_as(C.c_void_p)))
    return out
