"""Device-tensor layer over the C ABI: torch CUDA tensors in, torch CUDA tensors
out, on torch's current stream.  torch is used for device memory and streams
only; every computation is a call into `libfrink_b200.so`."""
import ctypes as C
import threading

import numpy as np
import torch

from . import _lib
from ._lib import check, lib

_contexts = {}
_lock = threading.Lock()


def context(device=None):
    """The process-wide context of `device` (`gpu::shared_device`,
    crates/frink-cuda/src/gpu.rs:172-222): created once, used from any thread."""
    if not torch.cuda.is_available():
        raise _lib.DriverInit("no CUDA device is visible; this backend has no CPU path")
    idx = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    with _lock:
        if idx not in _contexts:
            p = C.c_void_p()
            check(lib().fk_init(idx, C.byref(p)))
            _contexts[idx] = p
        return _contexts[idx]


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _f32(t):
    assert t.is_cuda and t.dtype == torch.float32, "expects a float32 CUDA tensor"
    return t.contiguous()


def _i32(t):
    assert t.is_cuda and t.dtype == torch.int32, "expects an int32 CUDA tensor"
    return t.contiguous()


def counters(reset=False, device=None):
    h, d, n = C.c_uint64(), C.c_uint64(), C.c_uint64()
    check(lib().fk_counters(context(device), C.byref(h), C.byref(d), C.byref(n), int(reset)))
    return {"h2d_bytes": h.value, "d2h_bytes": d.value, "launches": n.value}


def device_error(reset=True, device=None):
    """The word a kernel raises when a bounded wait gave up (0 = none)."""
    code = C.c_int()
    check(lib().fk_device_error(context(device), C.byref(code), int(reset)))
    return code.value


class Weights:
    """Resident quantized weights: `n_mats` equally shaped matrices given as
    their GGUF block bytes (numpy / CPU tensor: uploaded; CUDA tensor: copied
    on the device)."""

    def __init__(self, gguf_bytes, kind, rows, cols, n_mats=1, device=None):
        self.kind, self.rows, self.cols, self.n_mats = int(kind), int(rows), int(cols), int(n_mats)
        self._ctx = context(device)
        self._h = C.c_void_p()
        if isinstance(gguf_bytes, torch.Tensor) and gguf_bytes.is_cuda:
            raw = gguf_bytes.contiguous().view(torch.uint8)
            check(lib().fk_register_weights_dev(self._ctx, _ptr(raw), raw.numel(), self.kind, self.n_mats,
                                                self.rows, self.cols, _stream(), C.byref(self._h)))
            self.gguf_bytes = raw.numel()
        else:
            raw = np.ascontiguousarray(gguf_bytes.numpy() if isinstance(gguf_bytes, torch.Tensor) else gguf_bytes, np.uint8).ravel()
            check(lib().fk_register_weights(self._ctx, raw.ctypes.data_as(C.c_void_p), raw.size, self.kind, self.n_mats,
                                            self.rows, self.cols, C.byref(self._h)))
            self.gguf_bytes = raw.size

    @property
    def handle(self):
        if not self._h:
            raise _lib.Invalid("weights were released")
        return self._h

    def release(self):
        if self._h:
            check(lib().fk_release_weights(self._ctx, self._h))
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


def quantize_q8_1(x):
    """f32 CUDA tensor (numel % 32 == 0) -> uint8 CUDA tensor of 36-byte q8_1 blocks."""
    x = _f32(x)
    y = torch.empty(x.numel() // 32 * 36, dtype=torch.uint8, device=x.device)
    check(lib().fk_quantize_q8_1(context(x.device), _stream(), _ptr(x), x.numel(), _ptr(y)))
    return y


def quantize_q8_1_host(x):
    xd = torch.from_numpy(np.ascontiguousarray(x, np.float32).ravel()).cuda()
    return quantize_q8_1(xd).cpu().numpy()


def gemv(w, x, mat=0, out=None):
    """y[b, r] = W[mat][r] . q8_1(x[b]); x is [cols] or [batch <= 8, cols]."""
    x = _f32(x)
    batch = 1 if x.dim() == 1 else x.shape[0]
    assert x.shape[-1] == w.cols, f"x has {x.shape[-1]} columns, weights have {w.cols}"
    y = out if out is not None else torch.empty((batch, w.rows), dtype=torch.float32, device=x.device)
    check(lib().fk_gemv(w._ctx, _stream(), w.handle, mat, _ptr(x), batch, _ptr(y)))
    return y if x.dim() > 1 or out is not None else y[0]


def gemv_multi(w, ids, x, out=None):
    """Slot j: matrix ids[j] of `w` times x[j] (or the one shared x) -> out[j]."""
    ids, x = _i32(ids), _f32(x)
    k = ids.numel()
    stride = 0 if x.dim() == 1 else x.stride(0)
    y = out if out is not None else torch.empty((k, w.rows), dtype=torch.float32, device=x.device)
    check(lib().fk_gemv_multi(w._ctx, _stream(), w.handle, _ptr(ids), k, _ptr(x), stride, _ptr(y)))
    return y


def gemv_isums(w, x, mat=0):
    x = _f32(x)
    run = 16 if w.kind == 14 else 32
    out = torch.empty((w.rows, w.cols // run), dtype=torch.int32, device=x.device)
    check(lib().fk_gemv_isums(w._ctx, _stream(), w.handle, mat, _ptr(x), _ptr(out)))
    return out


def gemm(w, x, mat=0, out=None):
    """out[t, r] = W[mat][r] . q8_1(x[t]); x is [m, cols]."""
    x = _f32(x)
    assert x.dim() == 2 and x.shape[1] == w.cols
    y = out if out is not None else torch.empty((x.shape[0], w.rows), dtype=torch.float32, device=x.device)
    check(lib().fk_gemm(w._ctx, _stream(), w.handle, mat, _ptr(x), x.shape[0], _ptr(y)))
    return y


def gemm_static(w, x, mat=0, out=None):
    """`gemm` through the entry point that allocates nothing on the device: its
    scratch is a fixed block inside the library, so it can be used where device
    allocation is off limits (`out` must then be given: torch allocating the
    result would defeat the point).  Shapes too large for the block raise Invalid."""
    x = _f32(x)
    assert x.dim() == 2 and x.shape[1] == w.cols
    y = out if out is not None else torch.empty((x.shape[0], w.rows), dtype=torch.float32, device=x.device)
    check(lib().fk_gemm_static(w._ctx, _stream(), w.handle, mat, _ptr(x), x.shape[0], _ptr(y)))
    return y


def gemm_grouped(w, group_off, gather, x, pairs, out=None):
    """Permuted row p (expert e where group_off[e] <= p < group_off[e+1]) reads
    x[gather[p]] and writes out[p]."""
    x, group_off = _f32(x), _i32(group_off)
    gather = _i32(gather) if gather is not None else None
    y = out if out is not None else torch.empty((pairs, w.rows), dtype=torch.float32, device=x.device)
    check(lib().fk_gemm_grouped(w._ctx, _stream(), w.handle, _ptr(group_off), _ptr(gather), _ptr(x), pairs, _ptr(y)))
    return y


def router_logits(router, x):
    router, x = _f32(router), _f32(x)
    x2 = x if x.dim() == 2 else x[None]
    out = torch.empty((x2.shape[0], router.shape[0]), dtype=torch.float32, device=x.device)
    check(lib().fk_router_logits(context(x.device), _stream(), _ptr(router), _ptr(x2), router.shape[0], router.shape[1],
                                 x2.shape[0], _ptr(out)))
    return out


def moe_route(logits, k, mode, bias=None):
    logits = _f32(logits)
    l2 = logits if logits.dim() == 2 else logits[None]
    ids = torch.empty((l2.shape[0], k), dtype=torch.int32, device=logits.device)
    w = torch.empty((l2.shape[0], k), dtype=torch.float32, device=logits.device)
    b = _f32(bias) if bias is not None else None
    check(lib().fk_moe_route(context(logits.device), _stream(), _ptr(l2), _ptr(b), l2.shape[1], k, mode, l2.shape[0],
                             _ptr(ids), _ptr(w)))
    return ids, w


def moe_permute(ids, n_experts):
    ids = _i32(ids)
    pairs, k = ids.numel(), ids.shape[-1]
    dev = ids.device
    group_off = torch.empty(n_experts + 1, dtype=torch.int32, device=dev)
    gather = torch.empty(pairs, dtype=torch.int32, device=dev)
    pair_of = torch.empty(pairs, dtype=torch.int32, device=dev)
    check(lib().fk_moe_permute(context(dev), _stream(), _ptr(ids), pairs, k, n_experts, _ptr(group_off), _ptr(gather), _ptr(pair_of)))
    return group_off, gather, pair_of


def glu(gate, up, act=0, out=None):
    gate, up = _f32(gate), _f32(up)
    y = out if out is not None else torch.empty_like(gate)
    check(lib().fk_glu(context(gate.device), _stream(), _ptr(gate), _ptr(up), gate.numel(), act, _ptr(y)))
    return y


def moe_combine(y, pair_of, w, batch, k, out=None):
    y, w = _f32(y), _f32(w)
    n = y.shape[-1]
    o = out if out is not None else torch.empty((batch, n), dtype=torch.float32, device=y.device)
    check(lib().fk_moe_combine(context(y.device), _stream(), _ptr(y), _ptr(_i32(pair_of)) if pair_of is not None else None,
                               _ptr(w), batch, k, n, _ptr(o)))
    return o
