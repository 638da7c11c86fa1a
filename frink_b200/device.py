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


def gemv_fused(w, x, out=None, mat=0, norm_weight=None, eps=0.0, glu_up=None, glu_act=0, accumulate=False, pair_glu=0, allreduce=None, bias=None):
    """gemv with its elementwise neighbours folded in: reads rmsnorm(x) * norm_weight, or
    act(x) * glu_up (x the gate), and/or adds into `out` instead of overwriting it.
    x (and glu_up) are [batch <= 8, cols] with any row stride that is a multiple of 4.
    pair_glu (1 SiLU, 2 gpt-oss): `w` holds gate and up row-interleaved; the result is
    act(gate) * up, [batch, rows / 2].
    allreduce = (`frink_b200.comm.Comm`, channel): `w` is this rank's column range of a row-split
    matrix and the result is summed over the ranks by the matvec's epilogue.
    bias [rows]: added to the result by the same launch (`fk_gemv_biased`; with a norm and/or accumulate only)."""
    assert x.is_cuda and x.dtype == torch.float32 and x.dim() == 2 and x.stride(1) == 1
    batch, ld = x.shape[0], x.stride(0) if x.shape[0] > 1 else max(x.stride(0), w.cols)
    if glu_up is not None:
        assert glu_up.shape == x.shape and glu_up.stride(1) == 1 and (batch == 1 or glu_up.stride(0) == x.stride(0))
    y = out if out is not None else torch.empty((batch, w.rows // 2 if pair_glu else w.rows), dtype=torch.float32, device=x.device)
    if bias is not None:
        assert glu_up is None and not pair_glu and allreduce is None and bias.numel() == w.rows
        check(lib().fk_gemv_biased(w._ctx, _stream(), w.handle, mat, _ptr(x), ld, batch, _ptr(y),
                                   _ptr(_f32(norm_weight)) if norm_weight is not None else None, float(eps), _ptr(_f32(bias)), int(bool(accumulate))))
        return y
    if allreduce is not None:
        comm, (off, n_max) = allreduce
        assert not pair_glu
        check(lib().fk_gemv_fused_allreduce(w._ctx, _stream(), w.handle, mat, _ptr(x), ld, batch, _ptr(y),
                                            _ptr(_f32(norm_weight)) if norm_weight is not None else None, float(eps),
                                            _ptr(glu_up) if glu_up is not None else None, int(glu_act), int(bool(accumulate)),
                                            comm._h, off, n_max, comm.timeout_us))
        return y
    check(lib().fk_gemv_fused(w._ctx, _stream(), w.handle, mat, _ptr(x), ld, batch, _ptr(y),
                              _ptr(_f32(norm_weight)) if norm_weight is not None else None, float(eps),
                              _ptr(glu_up) if glu_up is not None else None, int(glu_act), int(bool(accumulate)),
                              int(pair_glu)))
    return y


def rope_kv(q, k, v, n_heads, n_kv, head_dim, pos, theta, neox, k_cache, v_cache, q_norm=None, k_norm=None, eps=0.0):
    """One launch: (Qwen3: per-head RMSNorm of q and k,) rotate q and k in place (rows at
    pos[0] + r) and append k, v to the caches.  q, k, v may be column slices of one buffer."""
    n = q.shape[0]
    assert k.stride(0) == v.stride(0) or n == 1
    check(lib().fk_rope_kv(context(q.device), _stream(), _ptr(q), _ptr(k), _ptr(v), q.stride(0), k.stride(0), n, n_heads, n_kv, head_dim,
                           _ptr(_i32(pos)), float(theta), int(neox), _ptr(k_cache), _ptr(v_cache),
                           _ptr(_f32(q_norm)) if q_norm is not None else None, _ptr(_f32(k_norm)) if k_norm is not None else None, float(eps),
                           min(k_cache.shape[0], v_cache.shape[0])))


def gemv_multi(w, ids, x, out=None, bias=None):
    """Slot j: matrix ids[j] of `w` times x[j] (or the one shared x) -> out[j]; with bias [n_mats, rows], + bias[ids[j]]."""
    ids, x = _i32(ids), _f32(x)
    k = ids.numel()
    stride = 0 if x.dim() == 1 else x.stride(0)
    y = out if out is not None else torch.empty((k, w.rows), dtype=torch.float32, device=x.device)
    if bias is not None:
        check(lib().fk_gemv_multi_biased(w._ctx, _stream(), w.handle, _ptr(ids), k, _ptr(x), None, stride, 0, _ptr(_f32(bias)), _ptr(y)))
        return y
    check(lib().fk_gemv_multi(w._ctx, _stream(), w.handle, _ptr(ids), k, _ptr(x), stride, _ptr(y)))
    return y


def gemv_multi_glu(w, ids, gate, up, act=0, out=None, n_active=None, bias=None):
    """Slot j: matrix ids[j] of `w` times act(gate[j]) * up[j] -> out[j] (gate, up: [k, cols]); with bias, + bias[ids[j]]."""
    ids, gate, up = _i32(ids), _f32(gate), _f32(up)
    k = ids.numel()
    assert gate.shape == up.shape and gate.dim() == 2 and gate.shape[0] == k
    y = out if out is not None else torch.empty((k, w.rows), dtype=torch.float32, device=gate.device)
    if bias is not None:
        assert n_active is None
        check(lib().fk_gemv_multi_biased(w._ctx, _stream(), w.handle, _ptr(ids), k, _ptr(gate), _ptr(up), gate.stride(0), int(act), _ptr(_f32(bias)), _ptr(y)))
        return y
    check(lib().fk_gemv_multi_glu(w._ctx, _stream(), w.handle, _ptr(ids), k, _ptr(gate), _ptr(up), gate.stride(0), int(act), _ptr(y),
                                  _ptr(_i32(n_active)) if n_active is not None else None))
    return y


def gemv_multi_active(w, ids, x, n_active, out):
    """gemv_multi whose slots >= n_active[0] (a device word) are skipped; `out` keeps its contents there."""
    ids, x = _i32(ids), _f32(x)
    stride = 0 if x.dim() == 1 else x.stride(0)
    check(lib().fk_gemv_multi_active(w._ctx, _stream(), w.handle, _ptr(ids), ids.numel(), _ptr(x), stride, _ptr(out), _ptr(_i32(n_active))))
    return out


def moe_local_slots(ids, w, e0, n_local):
    ids, w = _i32(ids).reshape(-1), _f32(w).reshape(-1)
    k = ids.numel()
    oi = torch.empty(k, dtype=torch.int32, device=ids.device)
    ow = torch.empty(k, dtype=torch.float32, device=ids.device)
    on = torch.empty(1, dtype=torch.int32, device=ids.device)
    check(lib().fk_moe_local_slots(context(ids.device), _stream(), _ptr(ids), _ptr(w), k, e0, n_local, _ptr(oi), _ptr(ow), _ptr(on)))
    return oi, ow, on


def add_bias_(y, bias, ids=None):
    """y [n, cols] += bias [cols], or += bias[ids[r]] row by row (the expert of every slot): gpt-oss's projection biases."""
    y2 = y if y.dim() == 2 else y[None]
    assert y2.is_contiguous() and y2.dtype == torch.float32
    check(lib().fk_add_bias(context(y.device), _stream(), _ptr(y2), _ptr(_f32(bias)), _ptr(_i32(ids)) if ids is not None else None, y2.shape[0], y2.shape[1]))
    return y


def gemv_multi_gate_up(gate, up, ids, x, norm_weight=None, eps=0.0, gate_bias=None, up_bias=None, out=None):
    """gate and up of the chosen experts in one launch: out [2 k, rows], rows j < k = gate[ids[j]] in_j, rows k + j =
    up[ids[j]] in_j (in_j = x[j] or the one shared x; with norm_weight, its RMSNorm), plus the experts' bias rows."""
    ids, x = _i32(ids), _f32(x)
    k = ids.numel()
    stride = 0 if x.dim() == 1 else x.stride(0)
    y = out if out is not None else torch.empty((2 * k, gate.rows), dtype=torch.float32, device=x.device)
    check(lib().fk_gemv_multi_gate_up(gate._ctx, _stream(), gate.handle, up.handle, _ptr(ids), k, _ptr(x), stride,
                                      _ptr(_f32(norm_weight)) if norm_weight is not None else None, float(eps),
                                      _ptr(_f32(gate_bias)) if gate_bias is not None else None,
                                      _ptr(_f32(up_bias)) if up_bias is not None else None, _ptr(y)))
    return y


def moe_layer(layer, x, out=None, accumulate=False, biases=None, norm=None):
    """The routed layer in one call (`fk_moe_layer`): `layer` carries router, router_bias, gate / up / down (stacked
    `Weights`), k, mode, act; x [batch, hidden] or [hidden].  The workspace is kept on the layer object, per batch size.
    biases = (gate_b, up_b, down_b), each [n_experts, rows]: gpt-oss's form (`fk_moe_layer_biased`).
    norm = (weight, eps): x is the un-normalized residual stream (at most 8 rows) and the layer's RMSNorm is folded into
    the router and the gate / up launch (`fk_moe_layer_normed`: four launches)."""
    x2 = _f32(x) if x.dim() == 2 else _f32(x)[None]
    batch = x2.shape[0]
    g = layer.gate
    ws = layer.__dict__.setdefault("_ws", {})
    if batch not in ws:
        need = lib().fk_moe_layer_workspace(g.n_mats, layer.k, g.cols, g.rows, batch)
        ws[batch] = torch.empty(need + 256, dtype=torch.uint8, device=x2.device)
    buf = ws[batch]
    base = (buf.data_ptr() + 255) & ~255
    assert not accumulate or out is not None
    o = out if out is not None else torch.empty((batch, g.cols), dtype=torch.float32, device=x2.device)
    o2 = o if o.dim() == 2 else o[None]
    rb = _ptr(_f32(layer.router_bias)) if layer.router_bias is not None else None
    if norm is not None:
        gb, ub, db = (_f32(t) for t in biases) if biases is not None else (None, None, None)
        check(lib().fk_moe_layer_normed(g._ctx, _stream(), _ptr(_f32(layer.router)), rb, g.handle, layer.up.handle, layer.down.handle,
                                        _ptr(gb) if gb is not None else None, _ptr(ub) if ub is not None else None,
                                        _ptr(db) if db is not None else None, layer.k, int(layer.mode), int(layer.act),
                                        _ptr(_f32(norm[0])), float(norm[1]), _ptr(x2), batch, _ptr(o2),
                                        int(bool(accumulate)), C.c_void_p(base), buf.numel() - (base - buf.data_ptr())))
        return o if x.dim() == 2 or out is not None else o[0]
    if biases is not None:
        gb, ub, db = (_f32(t) for t in biases)
        assert gb.shape == (g.n_mats, g.rows) and ub.shape == gb.shape and db.shape == (g.n_mats, g.cols)
        check(lib().fk_moe_layer_biased(g._ctx, _stream(), _ptr(_f32(layer.router)), rb, g.handle, layer.up.handle, layer.down.handle,
                                        _ptr(gb), _ptr(ub), _ptr(db), layer.k, int(layer.mode), int(layer.act), _ptr(x2), batch, _ptr(o2),
                                        int(bool(accumulate)), C.c_void_p(base), buf.numel() - (base - buf.data_ptr())))
        return o if x.dim() == 2 or out is not None else o[0]
    check(lib().fk_moe_layer(g._ctx, _stream(), _ptr(_f32(layer.router)), rb,
                             g.handle, layer.up.handle, layer.down.handle, layer.k, int(layer.mode), int(layer.act), _ptr(x2), batch, _ptr(o2),
                             int(bool(accumulate)), C.c_void_p(base), buf.numel() - (base - buf.data_ptr())))
    return o if x.dim() == 2 or out is not None else o[0]


def moe_local_pairs(ids, w, e0, n_local):
    """ids, w [b, k] -> (local expert per slot, source row per slot, slot of each pair, weight of each pair, slot count):
    the pairs this rank's experts serve, packed to the front as slots."""
    ids, w = _i32(ids), _f32(w)
    k, pairs = ids.shape[-1], ids.numel()
    oi = torch.empty(pairs, dtype=torch.int32, device=ids.device)
    src, po = torch.empty_like(oi), torch.empty_like(oi)
    ow = torch.empty(pairs, dtype=torch.float32, device=ids.device)
    on = torch.empty(1, dtype=torch.int32, device=ids.device)
    check(lib().fk_moe_local_pairs(context(ids.device), _stream(), _ptr(ids), _ptr(w), pairs, k, e0, n_local, _ptr(oi), _ptr(src), _ptr(po), _ptr(ow),
                                   _ptr(on)))
    return oi, src, po, ow, on


def moe_localize(ids, w, e0, n_local):
    """ids, w [batch, k] -> local ids (n_local where another rank owns the expert) and weights (0 there)."""
    ids, w = _i32(ids), _f32(w)
    oi, ow = torch.empty_like(ids), torch.empty_like(w)
    check(lib().fk_moe_localize(context(ids.device), _stream(), _ptr(ids), _ptr(w), ids.numel(), e0, n_local, _ptr(oi), _ptr(ow)))
    return oi, ow


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
    if w.kind in (13, 30):
        # Q5_K and BF16 have no GEMM kernel (fk_gemm answers UNSUPPORTED): batches of 8 through the matvec, the same integers
        for i in range(0, x.shape[0], 8):
            gemv(w, x[i:i + 8], mat=mat, out=y[i:i + 8])
        return y
    check(lib().fk_gemm(w._ctx, _stream(), w.handle, mat, _ptr(x), x.shape[0], _ptr(y)))
    return y


def gemm_isums(w, x, mat=0):
    """(out, isums): `gemm` plus the exact int32 dot of every run, [m, rows, cols / run]."""
    x = _f32(x)
    run = 16 if w.kind == 14 else 32
    y = torch.empty((x.shape[0], w.rows), dtype=torch.float32, device=x.device)
    isums = torch.empty((x.shape[0], w.rows, w.cols // run), dtype=torch.int32, device=x.device)
    check(lib().fk_gemm_isums(w._ctx, _stream(), w.handle, mat, _ptr(x), x.shape[0], _ptr(y), _ptr(isums)))
    return y, isums


def gemm_q8k(w, x, mat=0, out=None):
    """out[t, r] = W[mat][r] . q8_k(x[t]): the GEMM on frink's CPU activation rule (Q4_K weights)."""
    x = _f32(x)
    assert x.dim() == 2 and x.shape[1] == w.cols
    y = out if out is not None else torch.empty((x.shape[0], w.rows), dtype=torch.float32, device=x.device)
    check(lib().fk_gemm_q8k(w._ctx, _stream(), w.handle, mat, _ptr(x), x.shape[0], _ptr(y)))
    return y


def gemm_q8k_isums(w, x, mat=0):
    """(out, isums): `gemm_q8k` plus the exact integers per super-block, [m, rows, cols / 256, 2]."""
    x = _f32(x)
    y = torch.empty((x.shape[0], w.rows), dtype=torch.float32, device=x.device)
    isums = torch.empty((x.shape[0], w.rows, w.cols // 256, 2), dtype=torch.int32, device=x.device)
    check(lib().fk_gemm_q8k_isums(w._ctx, _stream(), w.handle, mat, _ptr(x), x.shape[0], _ptr(y), _ptr(isums)))
    return y, isums


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


def router_route(router, x, k, mode, bias=None):
    """router_logits followed by moe_route, one launch: (ids [batch, k], weights [batch, k])."""
    router, x = _f32(router), _f32(x)
    x2 = x if x.dim() == 2 else x[None]
    n, e = x2.shape[0], router.shape[0]
    logits = torch.empty((n, e), dtype=torch.float32, device=x.device)
    ids = torch.empty((n, k), dtype=torch.int32, device=x.device)
    w = torch.empty((n, k), dtype=torch.float32, device=x.device)
    b = _f32(bias) if bias is not None else None
    check(lib().fk_router_route(context(x.device), _stream(), _ptr(router), _ptr(x2), e, router.shape[1], n, _ptr(b), k, mode, _ptr(logits),
                                _ptr(ids), _ptr(w)))
    return ids, w


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


def moe_combine(y, pair_of, w, batch, k, out=None, accumulate=False):
    """accumulate: add the combined rows into `out` (the residual stream) instead of overwriting it."""
    y, w = _f32(y), _f32(w)
    n = y.shape[-1]
    assert not accumulate or out is not None
    o = out if out is not None else torch.empty((batch, n), dtype=torch.float32, device=y.device)
    fn = lib().fk_moe_combine_add if accumulate else lib().fk_moe_combine
    check(fn(context(y.device), _stream(), _ptr(y), _ptr(_i32(pair_of)) if pair_of is not None else None, _ptr(w), batch, k, n, _ptr(o)))
    return o


# ---- decoder glue -----------------------------------------------------------
def get_rows(w, ids, mat=0, out=None):
    ids = _i32(ids)
    o = out if out is not None else torch.empty((ids.numel(), w.cols), dtype=torch.float32, device=ids.device)
    check(lib().fk_get_rows(w._ctx, _stream(), w.handle, mat, _ptr(ids), ids.numel(), _ptr(o)))
    return o


def rmsnorm(x, weight, eps, residual=None, out=None):
    """out = rmsnorm(x (+ residual)) * weight; with `residual`, x is updated in place to the sum."""
    assert x.is_cuda and x.dtype == torch.float32 and x.is_contiguous()
    x2 = x if x.dim() == 2 else x[None]
    o = out if out is not None else torch.empty_like(x2)
    r = _f32(residual) if residual is not None else None
    check(lib().fk_rmsnorm(context(x.device), _stream(), _ptr(x2), _ptr(r), _ptr(_f32(weight)), x2.shape[0], x2.shape[1], float(eps), _ptr(o)))
    return o if x.dim() == 2 else o[0]


def rope(x, n_heads, head_dim, pos, theta, neox=False):
    """In place; x is [n_rows, n_heads * head_dim], `pos` an int32 device word."""
    assert x.is_cuda and x.dtype == torch.float32 and x.is_contiguous()
    n_rows = 1 if x.dim() == 1 else x.shape[0]
    check(lib().fk_rope(context(x.device), _stream(), _ptr(x), n_rows, n_heads, head_dim, _ptr(_i32(pos)), float(theta), int(neox)))
    return x


def add_(a, b):
    assert a.is_contiguous() and b.is_contiguous()
    check(lib().fk_add(context(a.device), _stream(), _ptr(a), _ptr(_f32(b)), a.numel()))
    return a


def kv_append(cache, src, pos):
    """cache [T, row] rows [*pos, *pos + n) <- src [n, row]."""
    src = _f32(src)
    n = 1 if src.dim() == 1 else src.shape[0]
    check(lib().fk_kv_append(context(cache.device), _stream(), _ptr(cache), _ptr(src), cache.shape[1], n, _ptr(_i32(pos)), cache.shape[0]))


def _sinks(sinks):
    return _ptr(_f32(sinks)) if sinks is not None else None


def attention(q, k_cache, v_cache, n_heads, n_kv, head_dim, pos, scale=None, out=None, window=0, sinks=None):
    """q: [n, n_heads * head_dim] with any row stride that is a multiple of 4 floats (a column
    slice of a merged q/k/v output works), or one row.  window > 0: only the `window` most recent
    keys; sinks [n_heads]: gpt-oss's per-head logit in the softmax's denominator."""
    assert q.is_cuda and q.dtype == torch.float32 and q.stride(-1) == 1
    q2 = q if q.dim() == 2 else q[None]
    o = out if out is not None else torch.empty((q2.shape[0], n_heads * head_dim), dtype=torch.float32, device=q.device)
    sc = float(scale) if scale is not None else head_dim ** -0.5
    ld = q2.stride(0) if q2.shape[0] > 1 else 0
    check(lib().fk_attention(context(q.device), _stream(), _ptr(q2), ld, _ptr(k_cache), _ptr(v_cache), q2.shape[0], n_heads, n_kv, head_dim,
                             _ptr(_i32(pos)), sc, _ptr(o), min(k_cache.shape[0], v_cache.shape[0]), int(window), _sinks(sinks)))
    return o if q.dim() == 2 else o[0]


def attention_rope_kv(q, k_new, v_new, k_cache, v_cache, n_heads, n_kv, head_dim, pos, theta, neox=False, q_norm=None, k_norm=None, eps=0.0,
                      scale=None, out=None, window=0, sinks=None):
    """One decode row: rotate q and the new k at pos[0] (after Qwen3's head norms when given),
    append k and v to the caches and attend over positions 0 ..= pos[0], in one launch.
    q [1, n_heads*head_dim], k_new / v_new [1, n_kv*head_dim] (column slices are fine)."""
    assert q.shape[0] == 1 and q.stride(-1) == 1 and k_new.stride(-1) == 1 and v_new.stride(-1) == 1
    o = out if out is not None else torch.empty((1, n_heads * head_dim), dtype=torch.float32, device=q.device)
    sc = float(scale) if scale is not None else head_dim ** -0.5
    check(lib().fk_attention_rope_kv(context(q.device), _stream(), _ptr(q), _ptr(k_new), _ptr(v_new), _ptr(k_cache), _ptr(v_cache), n_heads, n_kv,
                                     head_dim, _ptr(_i32(pos)), sc, float(theta), int(neox),
                                     _ptr(_f32(q_norm)) if q_norm is not None else None, _ptr(_f32(k_norm)) if k_norm is not None else None,
                                     float(eps), _ptr(o), min(k_cache.shape[0], v_cache.shape[0]), int(window), _sinks(sinks)))
    return o


def attention_rope_kv_seqs(q, k_new, v_new, k_caches, v_caches, n_heads, n_kv, head_dim, pos, theta, neox=False, q_norm=None, k_norm=None,
                           eps=0.0, scale=None, out=None, window=0, sinks=None):
    """One decode step of independent sequences: row r of q / k_new / v_new (column slices are fine) is sequence r's
    token at position pos[r]; k_caches / v_caches are [n_seqs, T, n_kv*head_dim]."""
    n = q.shape[0]
    assert k_caches.dim() == 3 and k_caches.is_contiguous() and v_caches.is_contiguous() and k_caches.shape == v_caches.shape and k_caches.shape[0] >= n
    assert q.stride(-1) == 1 and k_new.stride(-1) == 1 and v_new.stride(-1) == 1
    assert pos.dtype == torch.int32 and pos.numel() >= n
    o = out if out is not None else torch.empty((n, n_heads * head_dim), dtype=torch.float32, device=q.device)
    sc = float(scale) if scale is not None else head_dim ** -0.5
    check(lib().fk_attention_rope_kv_seqs(context(q.device), _stream(), _ptr(q), q.stride(0), _ptr(k_new), _ptr(v_new), k_new.stride(0), v_new.stride(0),
                                          _ptr(k_caches), _ptr(v_caches), k_caches.stride(0), n, n_heads, n_kv, head_dim, _ptr(pos), sc,
                                          float(theta), int(neox), _ptr(_f32(q_norm)) if q_norm is not None else None,
                                          _ptr(_f32(k_norm)) if k_norm is not None else None, float(eps), _ptr(o), k_caches.shape[1],
                                          int(window), _sinks(sinks)))
    return o


def argmax(x, out=None):
    x = _f32(x)
    x2 = x if x.dim() == 2 else x[None]
    o = out if out is not None else torch.empty(x2.shape[0], dtype=torch.int32, device=x.device)
    check(lib().fk_argmax(context(x.device), _stream(), _ptr(x2), x2.shape[0], x2.shape[1], _ptr(o)))
    return o


def add_int_(p, v):
    check(lib().fk_add_int(context(p.device), _stream(), _ptr(_i32(p)), int(v)))
