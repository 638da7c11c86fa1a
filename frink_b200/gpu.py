"""Host-buffer launch surface: mirror of `frink_cuda::gpu`
(crates/frink-cuda/src/gpu.rs:91-157,319-446 and src/matvec_launch.rs:485-570).

Borrowed host bytes and host f32 in, a freshly owned host array out, weights
kept resident by (pointer, length) + fingerprint.  Same names, argument meaning
and error behaviour as the functions frink-core binds."""
import ctypes as C
from dataclasses import dataclass
from typing import Optional

import numpy as np

from . import _lib, matvec_kinds
from ._lib import CudaError, DriverInit, KernelCompile, Launch, Unsupported, check, lib  # noqa: F401


@dataclass
class CudaInfo:
    device_count: int
    first_device_name: Optional[str]
    total_vram_bytes: int
    free_vram_bytes: int


def probe():
    """`gpu::probe`: None on any failure to find a usable device, never raises."""
    try:
        import torch
        if not torch.cuda.is_available():
            return None
        from . import device
        ctx = device.context()
        name = C.create_string_buffer(128)
        sms, mem = C.c_int(), C.c_size_t()
        check(lib().fk_device_info(ctx, name, 128, C.byref(sms), C.byref(mem)))
        free, total = torch.cuda.mem_get_info(torch.cuda.current_device())
        return CudaInfo(torch.cuda.device_count(), name.value.decode(), int(total), int(free))
    except Exception:
        return None


def _ctx():
    """The context the host-buffer calls run on: the process's current CUDA device at first use.  The reference's
    `shared_device` is device 0 (one GPU); with one process per GPU every rank must stay on its own device --
    bound to device 0, eight ranks took turns on one GPU and a 31 us call became a millisecond."""
    from . import device
    return device.context()


def _host(a, dt):
    """A C-contiguous array of dtype `dt` (the input itself when it already is one) and its address."""
    if not (isinstance(a, np.ndarray) and a.dtype == dt and a.flags.c_contiguous):
        a = np.ascontiguousarray(a, dt)
    return a, a.ctypes.data


_KIND = {}
_CTX = []


def _launch_matvec(kind_name, weights, x, rows, row_bytes, n_blocks_per_row):
    # the call is ~20 us of GPU work, so the wrapper keeps its own share small: kinds and the
    # context are looked up once, addresses go over as plain integers
    kind = _KIND.get(kind_name)
    if kind is None:
        kind = _KIND[kind_name] = matvec_kinds.kind_by_name(kind_name)
    if not _CTX:
        _CTX.append(_ctx())
    w, wp = _host(weights, np.uint8)
    xv, xp = _host(x, np.float32)
    if xv.size != n_blocks_per_row * kind.block_elems:
        raise _lib.Invalid(f"{kind.fn_name}: x has {xv.size} values, the row has {n_blocks_per_row * kind.block_elems}")
    y = np.empty(rows, np.float32)
    check(lib().fk_launch_matvec(_CTX[0], kind.tag, wp, w.size, xp, rows, row_bytes, n_blocks_per_row, y.ctypes.data))
    return y


def launch_q4_k_matvec(weights, x, rows, row_bytes, n_blocks_per_row):
    return _launch_matvec("Q4_K", weights, x, rows, row_bytes, n_blocks_per_row)


def launch_q5_k_matvec(weights, x, rows, row_bytes, n_blocks_per_row):
    return _launch_matvec("Q5_K", weights, x, rows, row_bytes, n_blocks_per_row)


def launch_q6_k_matvec(weights, x, rows, row_bytes, n_blocks_per_row):
    return _launch_matvec("Q6_K", weights, x, rows, row_bytes, n_blocks_per_row)


def launch_q8_0_matvec(weights, x, rows, row_bytes, n_blocks_per_row):
    return _launch_matvec("Q8_0", weights, x, rows, row_bytes, n_blocks_per_row)


def launch_mxfp4_matvec(weights, x, rows, row_bytes, n_blocks_per_row):
    return _launch_matvec("MXFP4", weights, x, rows, row_bytes, n_blocks_per_row)


@dataclass
class MatvecLaunch:
    """`gpu::MatvecLaunch` (matvec_launch.rs:485-493).  `kernel_src` and
    `module_name` belong to the reference's run-time compiler and are kept only
    so call sites read the same; this library's kernels are compiled ahead of time."""
    fn_name: str
    weights: np.ndarray
    rows: int
    row_bytes: int
    n_blocks_per_row: int
    kernel_src: str = ""
    module_name: str = ""


def matvec_launch_meta(kind_name):
    k = matvec_kinds.kind_by_name(kind_name)
    if k is None:
        return None
    return ("", "frink_b200", k.fn_name)


def _kind_of(launch):
    k = matvec_kinds.kind_by_name(launch.fn_name)
    if k is None:
        raise Unsupported(f"no kernel for {launch.fn_name}")
    return k


class _CLaunch(C.Structure):
    """`fk_matvec_launch` of the C ABI."""
    _fields_ = [("kind", C.c_int), ("weights_host", C.c_void_p), ("len", C.c_size_t), ("rows", C.c_int), ("row_bytes", C.c_int),
                ("n_blocks_per_row", C.c_int)]


def _c_launch(l):
    k = _kind_of(l)
    w, wp = _host(l.weights, np.uint8)
    return _CLaunch(k.tag, wp, w.size, l.rows, l.row_bytes, l.n_blocks_per_row), k, w


def launch_matvec_multi(x, launches):
    """`gpu::launch_matvec_multi` (matvec_launch.rs:495-535): one upload of `x`,
    one matvec per launch, outputs downloaded after all were enqueued
    (`fk_launch_matvec_multi`)."""
    if not launches:
        return []
    if not _CTX:
        _CTX.append(_ctx())
    xv, xp = _host(x, np.float32)
    cl = [_c_launch(l) for l in launches]
    arr = (_CLaunch * len(cl))(*[c[0] for c in cl])
    outs = [np.empty(l.rows, np.float32) for l in launches]
    ptrs = (C.c_void_p * len(outs))(*[o.ctypes.data for o in outs])
    check(lib().fk_launch_matvec_multi(_CTX[0], xp, xv.size, arr, len(cl), ptrs))
    return outs


def launch_dense_ffn_swiglu(gate, up, down, x):
    """`gpu::launch_dense_ffn_swiglu` (matvec_launch.rs:537-570): x up once,
    gate and up matvecs, silu(gate)*up, down matvec, one download
    (`fk_launch_dense_ffn_swiglu`)."""
    if not _CTX:
        _CTX.append(_ctx())
    xv, xp = _host(x, np.float32)
    g, u, d = _c_launch(gate), _c_launch(up), _c_launch(down)
    y = np.empty(down.rows, np.float32)
    check(lib().fk_launch_dense_ffn_swiglu(_CTX[0], C.byref(g[0]), C.byref(u[0]), C.byref(d[0]), xp, xv.size, y.ctypes.data))
    return y
