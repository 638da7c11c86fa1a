"""ctypes/numpy face of the CPU oracle (`libfrink_oracle.so`).

TEST INFRASTRUCTURE ONLY.  Importable from `tests/`, from `__graft_entry__.smoke()`
and from `bench.py`'s CPU-baseline legs; the shipped package never imports it.
Each wrapper names the oracle function it calls; the citations of the reference
functions those restate are in `frink_oracle.cpp`.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libfrink_oracle.so")

# ggml type tags, shared with include/frink_b200.h
Q8_0, Q4_K, Q5_K, Q6_K, MXFP4, BF16 = 8, 12, 13, 14, 39, 30
KINDS = {"q8_0": Q8_0, "q4_k": Q4_K, "q5_k": Q5_K, "q6_k": Q6_K, "mxfp4": MXFP4, "bf16": BF16}


def build(force=False):
    """Compile the oracle with the Makefile beside it (g++, no GPU needed)."""
    src = os.path.join(_HERE, "frink_oracle.cpp")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libfrink_oracle.so"], stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_SO)
        u8p, f32p, i8p, i16p, i32p, f64p = (C.c_void_p,) * 6
        L.fko_f16_to_f32.restype = C.c_float
        L.fko_f16_to_f32.argtypes = [C.c_uint16]
        L.fko_f32_to_f16.restype = C.c_uint16
        L.fko_f32_to_f16.argtypes = [C.c_float]
        L.fko_dequant.restype = C.c_long
        L.fko_dequant.argtypes = [C.c_int, u8p, C.c_long, f32p]
        L.fko_dot_f32_scalar.restype = C.c_float
        L.fko_dot_f32_scalar.argtypes = [C.c_int, u8p, C.c_int, f32p]
        L.fko_dot_dequant_f64.restype = C.c_double
        L.fko_dot_dequant_f64.argtypes = [C.c_int, u8p, C.c_int, f32p]
        L.fko_quantize_q8_k.argtypes = [f32p, C.c_int, i8p, f32p, i16p]
        L.fko_quantize_q8_0_act.argtypes = [f32p, C.c_int, C.c_int, i8p, f32p]
        L.fko_quantize_q8_1.argtypes = [f32p, C.c_int, u8p]
        L.fko_q8_1_dequant.argtypes = [u8p, C.c_int, f32p]
        L.fko_dot_q8.restype = C.c_float
        L.fko_dot_q8.argtypes = [C.c_int, u8p, C.c_int, i8p, f32p, i16p]
        L.fko_dp4a_row.restype = C.c_float
        L.fko_dp4a_row.argtypes = [C.c_int, u8p, u8p, C.c_int, C.c_int]
        L.fko_row_isums.argtypes = [C.c_int, u8p, C.c_int, u8p, i32p]
        L.fko_encode.restype = C.c_long
        L.fko_encode.argtypes = [C.c_int, f32p, C.c_long, u8p]
        L.fko_encode_mt.restype = C.c_long
        L.fko_encode_mt.argtypes = [C.c_int, f32p, C.c_long, u8p, C.c_int]
        L.fko_nearest_int.argtypes = [C.c_float]
        L.fko_row_isums_q4k_q8k.argtypes = [u8p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
        L.fko_matvec_f32.argtypes = [C.c_int, u8p, C.c_int, C.c_int, f32p, C.c_int, f32p, C.c_int, C.c_int]
        L.fko_matmul_q8.argtypes = [C.c_int, u8p, C.c_int, C.c_int, f32p, C.c_int, f32p, C.c_int]
        L.fko_matmul_f64.argtypes = [C.c_int, u8p, C.c_int, C.c_int, f32p, C.c_int, f64p, C.c_int]
        L.fko_route_top_k.argtypes = [f32p, f32p, C.c_int, C.c_int, C.c_int, C.c_int, i32p, f32p]
        L.fko_silu_mul.argtypes = [f32p, f32p, C.c_int, f32p]
        L.fko_swiglu_oai.argtypes = [f32p, f32p, C.c_int, C.c_float, C.c_float, f32p]
        L.fko_combine.argtypes = [f32p, f32p, C.c_int, C.c_int, f32p]
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def block_bytes(kind):
    return lib().fko_block_bytes(kind)


def block_elems(kind):
    return lib().fko_block_elems(kind)


def row_bytes(kind, cols):
    return cols // block_elems(kind) * block_bytes(kind)


def runs_per_block(kind):
    return lib().fko_runs_per_block(kind)


def host_threads():
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


def dequant(kind, raw):
    raw = _c(raw, np.uint8).ravel()
    out = np.empty(raw.size // block_bytes(kind) * block_elems(kind), np.float32)
    n = lib().fko_dequant(kind, _p(raw), raw.size, _p(out))
    assert n == out.size, "byte length is not a whole number of blocks"
    return out


def encode(kind, x, threads=None):
    """f32 -> GGUF blocks of `kind` with the reference's encoders."""
    x = _c(x, np.float32).ravel()
    assert x.size % block_elems(kind) == 0
    out = np.empty(x.size // block_elems(kind) * block_bytes(kind), np.uint8)
    n = lib().fko_encode_mt(kind, _p(x), x.size, _p(out), threads or host_threads())
    assert n == out.size
    return out


def dot_f32_scalar(kind, row, x):
    row, x = _c(row, np.uint8).ravel(), _c(x, np.float32)
    return float(lib().fko_dot_f32_scalar(kind, _p(row), row.size // block_bytes(kind), _p(x)))


def dot_dequant_f64(kind, row, x):
    row, x = _c(row, np.uint8).ravel(), _c(x, np.float32)
    return float(lib().fko_dot_dequant_f64(kind, _p(row), row.size // block_bytes(kind), _p(x)))


def quantize_q8_k(x):
    x = _c(x, np.float32).ravel()
    q = np.empty(x.size, np.int8)
    d = np.empty(x.size // 256, np.float32)
    bs = np.empty(x.size // 16, np.int16)
    lib().fko_quantize_q8_k(_p(x), x.size, _p(q), _p(d), _p(bs))
    return q, d, bs


def quantize_q8_0_act(x, form=1):
    x = _c(x, np.float32).ravel()
    q = np.empty(x.size, np.int8)
    d = np.empty(x.size // 32, np.float32)
    lib().fko_quantize_q8_0_act(_p(x), x.size, form, _p(q), _p(d))
    return q, d


def quantize_q8_1(x):
    """f32 (multiple of 32 long) -> `block_q8_1` bytes, 36 per 32 values."""
    x = _c(x, np.float32).ravel()
    out = np.empty(x.size // 32 * 36, np.uint8)
    lib().fko_quantize_q8_1(_p(x), x.size, _p(out))
    return out


def q8_1_dequant(y):
    y = _c(y, np.uint8).ravel()
    out = np.empty(y.size // 36 * 32, np.float32)
    lib().fko_q8_1_dequant(_p(y), y.size // 36, _p(out))
    return out


def q8_1_round(x):
    """`x` as a q8_1 kernel reads it: through the quantizer and back."""
    shape = np.shape(x)
    return q8_1_dequant(quantize_q8_1(x)).reshape(shape)


def dot_q8(kind, row, x):
    """The reference's CPU integer vec_dot of one row (Q8_K / Q8_0 activations)."""
    row = _c(row, np.uint8).ravel()
    nblk = row.size // block_bytes(kind)
    if kind in (Q4_K, Q5_K, Q6_K):
        q, d, bs = quantize_q8_k(x)
        return float(lib().fko_dot_q8(kind, _p(row), nblk, _p(q), _p(d), _p(bs)))
    q, d = quantize_q8_0_act(x, 1)
    return float(lib().fko_dot_q8(kind, _p(row), nblk, _p(q), _p(d), None))


def matrix_isums_q4k_q8k(w, rows, cols, x):
    """The exact integers of the reference's CPU Q4_K vec_dot on Q8_K activations, per super-block:
    [rows, cols / 256, 2] = (sum of scale * sub-block dot, sum of min * sub-block sum)."""
    w = _c(w, np.uint8).ravel()
    q, d, bs = quantize_q8_k(x)
    nblk = cols // 256
    rb = nblk * 144
    out = np.empty((rows, nblk, 2), np.int32)
    for r in range(rows):
        lib().fko_row_isums_q4k_q8k(_p(w[r * rb:(r + 1) * rb]), nblk, _p(q), _p(bs), _p(out[r]))
    return out


def dp4a_row(kind, row, y, nwarps=4):
    row, y = _c(row, np.uint8).ravel(), _c(y, np.uint8).ravel()
    return float(lib().fko_dp4a_row(kind, _p(row), _p(y), row.size // block_bytes(kind), nwarps))


def matrix_isums(kind, w, rows, cols, y):
    """Exact per-run integer dots of every row of `w` against q8_1 bytes `y`."""
    w, y = _c(w, np.uint8).ravel(), _c(y, np.uint8).ravel()
    nblk = cols // block_elems(kind)
    rb = nblk * block_bytes(kind)
    rpb = runs_per_block(kind)
    out = np.empty((rows, nblk * rpb), np.int32)
    for r in range(rows):
        lib().fko_row_isums(kind, _p(w[r * rb:(r + 1) * rb]), nblk, _p(y), _p(out[r]))
    return out


def matvec_f32(kind, w, rows, cols, x, threads=1, simd=False):
    """The reference's x86 decode path: fused f32 dot per row, rows over threads."""
    w = _c(w, np.uint8).ravel()
    x = _c(x, np.float32).reshape(-1, cols)
    y = np.empty((x.shape[0], rows), np.float32)
    rc = lib().fko_matvec_f32(kind, _p(w), rows, cols, _p(x), x.shape[0], _p(y), threads, int(simd))
    assert rc == 0
    return y


def matmul_q8(kind, w, rows, cols, x, threads=1):
    """The reference's CPU batched path: Q8_K / Q8_0 activations, integer row dots."""
    w = _c(w, np.uint8).ravel()
    x = _c(x, np.float32).reshape(-1, cols)
    out = np.empty((x.shape[0], rows), np.float32)
    rc = lib().fko_matmul_q8(kind, _p(w), rows, cols, _p(x), x.shape[0], _p(out), threads)
    assert rc == 0
    return out


def matmul_f64(kind, w, rows, cols, x, threads=None):
    """f64 dequantize-then-dot of every row: what the fp32 tolerance is taken against."""
    w = _c(w, np.uint8).ravel()
    x = _c(x, np.float32).reshape(-1, cols)
    out = np.empty((x.shape[0], rows), np.float64)
    rc = lib().fko_matmul_f64(kind, _p(w), rows, cols, _p(x), x.shape[0], _p(out), threads or host_threads())
    assert rc == 0
    return out


def route_top_k(logits, k, mode, bias=None):
    logits = _c(logits, np.float32)
    batch, n = logits.reshape(-1, logits.shape[-1]).shape
    ids = np.empty((batch, k), np.int32)
    w = np.empty((batch, k), np.float32)
    b = _c(bias, np.float32) if bias is not None else None
    lib().fko_route_top_k(_p(logits), _p(b) if b is not None else None, n, k, mode, batch, _p(ids), _p(w))
    return ids, w


def silu_mul(gate, up):
    gate, up = _c(gate, np.float32), _c(up, np.float32)
    out = np.empty_like(gate)
    lib().fko_silu_mul(_p(gate), _p(up), gate.size, _p(out))
    return out


def swiglu_oai(gate, up, alpha=1.702, limit=7.0):
    gate, up = _c(gate, np.float32), _c(up, np.float32)
    out = np.empty_like(gate)
    lib().fko_swiglu_oai(_p(gate), _p(up), gate.size, alpha, limit, _p(out))
    return out


def combine(ys, w):
    ys, w = _c(ys, np.float32), _c(w, np.float32)
    k, n = ys.shape
    out = np.empty(n, np.float32)
    lib().fko_combine(_p(ys), _p(w), k, n, _p(out))
    return out
