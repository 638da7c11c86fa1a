"""A CPU stand-in for `frink_b200.device` built on the oracle, for the tests of
the host-side sharding logic (`frink_b200.parallel`) under gloo.  TEST ONLY."""
import numpy as np
import torch

from oracle import frink_oracle as fo


class Weights:
    def __init__(self, raw, kind, rows, cols, n_mats=1, device=None):
        self.raw = np.ascontiguousarray(raw, np.uint8).ravel().copy()
        self.kind, self.rows, self.cols, self.n_mats = kind, rows, cols, n_mats
        self.per = rows * fo.row_bytes(kind, cols)

    def mat(self, m):
        return self.raw[m * self.per:(m + 1) * self.per]


def _mm(w, m, x):
    x = np.ascontiguousarray(x, np.float32).reshape(-1, w.cols)
    xq = x if w.kind == fo.BF16 else fo.q8_1_round(x)          # BF16 weights meet f32 activations; the block formats q8_1's
    return fo.matmul_f64(w.kind, w.mat(m), w.rows, w.cols, xq, threads=1).astype(np.float32)


def gemv(w, x, mat=0, out=None):
    y = torch.from_numpy(_mm(w, mat, x.numpy()))
    return y if x.dim() > 1 else y[0]


def gemm(w, x, mat=0, out=None):
    return torch.from_numpy(_mm(w, mat, x.numpy()))


def gemv_multi(w, ids, x, out=None):
    xs = x.numpy()
    return torch.from_numpy(np.stack([_mm(w, int(e), xs if xs.ndim == 1 else xs[j])[0] for j, e in enumerate(ids.tolist())]))


def gemm_grouped(w, group_off, gather, x, pairs, out=None):
    off = group_off.tolist()
    xs = x.numpy()
    y = np.zeros((pairs, w.rows), np.float32)
    for e in range(w.n_mats):
        lo, hi = off[e], off[e + 1]
        if hi > lo:
            idx = gather.numpy()[lo:hi] if gather is not None else np.arange(lo, hi)
            y[lo:hi] = _mm(w, e, xs[idx])
    return torch.from_numpy(y)


def glu(g, u, act=0, out=None):
    f = fo.silu_mul if act == 0 else fo.swiglu_oai
    return torch.from_numpy(f(g.numpy().ravel(), u.numpy().ravel()).reshape(g.shape))


def router_logits(router, x):
    x2 = x if x.dim() == 2 else x[None]
    return (x2.double() @ router.double().T).float()


def moe_route(logits, k, mode, bias=None):
    l2 = logits if logits.dim() == 2 else logits[None]
    ids, w = fo.route_top_k(l2.numpy(), k, mode, None if bias is None else bias.numpy())
    return torch.from_numpy(ids), torch.from_numpy(w)


def moe_permute(ids, n_experts):
    flat = ids.numpy().ravel()
    k = ids.shape[-1]
    order = np.argsort(flat, kind="stable")
    off = np.concatenate([[0], np.cumsum(np.bincount(flat, minlength=n_experts))]).astype(np.int32)
    pair_of = np.empty(flat.size, np.int32)
    pair_of[order] = np.arange(flat.size, dtype=np.int32)
    return torch.from_numpy(off), torch.from_numpy((order // k).astype(np.int32)), torch.from_numpy(pair_of)


def moe_localize(ids, w, e0, n_local):
    mine = (ids >= e0) & (ids < e0 + n_local)
    return torch.where(mine, ids - e0, torch.full_like(ids, n_local)).to(torch.int32), torch.where(mine, w, torch.zeros_like(w))


def moe_local_pairs(ids, w, e0, n_local):
    flat, wf = ids.reshape(-1), w.reshape(-1)
    k = ids.shape[-1]
    mine = (flat >= e0) & (flat < e0 + n_local)
    n = int(mine.sum())
    slot = torch.cumsum(mine.to(torch.int32), 0) - 1
    lid = torch.zeros_like(flat)
    src = torch.zeros_like(flat)
    lid[:n] = flat[mine] - e0
    src[:n] = (torch.arange(flat.numel())[mine] // k).to(torch.int32)
    pair_of = torch.where(mine, slot, torch.zeros_like(slot)).to(torch.int32)
    return lid.to(torch.int32), src.to(torch.int32), pair_of, torch.where(mine, wf, torch.zeros_like(wf)), torch.tensor([n], dtype=torch.int32)


def gemv_multi_active(w, ids, x, n_active, out):
    n = int(n_active[0])
    if n:
        out[:n] = gemv_multi(w, ids[:n], x[:n] if x.dim() == 2 else x)
    return out


def moe_combine(y, pair_of, w, batch, k, out=None, accumulate=False):
    ys, ws = y.numpy(), w.numpy().reshape(batch, k)
    po = pair_of.numpy() if pair_of is not None else np.arange(batch * k)
    r = torch.from_numpy(np.stack([fo.combine(ys[po[t * k:(t + 1) * k]], ws[t]) for t in range(batch)]))
    if accumulate:
        out.add_(r)
        return out
    return r


def gemv_multi_glu(w, ids, gate, up, act=0, out=None, n_active=None):
    if n_active is not None:
        n = int(n_active[0])
        if n:
            out[:n] = gemv_multi(w, ids[:n], glu(gate[:n].contiguous(), up[:n].contiguous(), act))
        return out
    return gemv_multi(w, ids, glu(gate, up, act))


# ---- the decoder glue, so that `frink_b200.decoder.Decoder` runs on CPU ranks
def get_rows(w, ids):
    rb = fo.row_bytes(w.kind, w.cols)
    return torch.from_numpy(np.stack([fo.dequant(w.kind, w.raw[int(t) * rb:(int(t) + 1) * rb]) for t in ids.tolist()]).astype(np.float32))


def rmsnorm(x, w, eps, residual=None, out=None):
    from tests import oracle_decoder as od
    if residual is not None:
        x.add_(residual)          # the device kernel leaves x + residual in x
    return torch.from_numpy(od.rmsnorm(x.numpy(), w.numpy(), eps))


def rope(x, n_heads, head_dim, pos, theta, neox=False):
    from tests import oracle_decoder as od
    x.copy_(torch.from_numpy(od.rope(x.numpy().copy(), n_heads, head_dim, int(pos[0]), theta, neox)))
    return x


def kv_append(cache, src, pos):
    p = int(pos[0])
    cache[p:p + src.shape[0]] = src


def attention(q, k_cache, v_cache, n_heads, n_kv, head_dim, pos, scale=None, out=None, window=0, sinks=None):
    p0, n, grp = int(pos[0]), q.shape[0], n_heads // n_kv
    qn, K, V = q.numpy().astype(np.float64), k_cache.numpy().astype(np.float64), v_cache.numpy().astype(np.float64)
    o = np.zeros((n, n_heads * head_dim), np.float32)
    for r in range(n):
        T = p0 + r + 1
        for h in range(n_heads):
            kv = h // grp
            lo = max(0, T - window) if window else 0
            s = K[lo:T, kv * head_dim:(kv + 1) * head_dim] @ qn[r, h * head_dim:(h + 1) * head_dim] * head_dim ** -0.5
            mx = max(s.max(), float(sinks[h])) if sinks is not None else s.max()
            p = np.exp(s - mx)
            den = p.sum() + (np.exp(float(sinks[h]) - mx) if sinks is not None else 0.0)
            o[r, h * head_dim:(h + 1) * head_dim] = p @ V[lo:T, kv * head_dim:(kv + 1) * head_dim] / den
    return torch.from_numpy(o)


def argmax(x, out=None):
    x2 = x if x.dim() == 2 else x[None]
    return torch.argmax(x2, dim=1).to(torch.int32)


def add_bias_(y, bias, ids=None):
    y2 = y if y.dim() == 2 else y[None]
    y2.add_(bias if ids is None else bias[ids.long()])
    return y


def add_(a, b):
    a.add_(b)


def add_int_(p, v):
    p.add_(v)


def gemv_fused(w, x, out=None, mat=0, norm_weight=None, eps=0.0, glu_up=None, glu_act=0, accumulate=False, pair_glu=0, bias=None):
    """The fused matvec of the device layer, composed from the separate CPU steps."""
    h = x.clone()
    if norm_weight is not None:
        h = rmsnorm(h, norm_weight, eps)
    if glu_up is not None:
        h = glu(h.contiguous(), glu_up.contiguous(), glu_act)
    y = gemv(w, h, mat=mat)
    if bias is not None:
        y = y + bias
    if pair_glu:
        y = glu(y[:, 0::2].contiguous(), y[:, 1::2].contiguous(), pair_glu - 1)
    if out is None:
        return y
    if accumulate:
        out.add_(y)
    else:
        out.copy_(y)
    return out


def rope_kv(q, k, v, n_heads, n_kv, head_dim, pos, theta, neox, k_cache, v_cache, q_norm=None, k_norm=None, eps=0.0):
    qc, kc = q.contiguous(), k.contiguous()
    if q_norm is not None:
        qc = rmsnorm(qc.view(-1, head_dim), q_norm, eps).view(qc.shape[0], -1).contiguous()
        kc = rmsnorm(kc.view(-1, head_dim), k_norm, eps).view(kc.shape[0], -1).contiguous()
    rope(qc, n_heads, head_dim, pos, theta, neox)
    rope(kc, n_kv, head_dim, pos, theta, neox)
    q.copy_(qc)
    k.copy_(kc)
    kv_append(k_cache, kc, pos)
    kv_append(v_cache, v.contiguous(), pos)
