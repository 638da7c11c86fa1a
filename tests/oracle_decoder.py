"""CPU oracle of the decoder pipeline, composed from the oracle's pieces: every
matmul is the f64 dequantize-then-dot of the q8_1-rounded activation (what the
device kernels read), RMSNorm sums f32 squares in f64
(crates/frink-core/src/matmul.rs:87-95), RoPE as
crates/frink-cuda/src/prefill/kernels.rs:402, causal GQA softmax in f64; routed
layers as crates/frink-moe/src/lib.rs:567 (route), :1068 (run_expert), :1246 (combine
from zero in routing order); Qwen3's per-head q/k RMSNorm ahead of the rotation
(crates/frink-core/src/matmul.rs:63).  Written against the reference's graph, not
against frink_b200.decoder: it shares no code with the device decoder.  TEST ONLY."""
import numpy as np

from oracle import frink_oracle as fo


def rmsnorm(x, w, eps):
    x = np.asarray(x, np.float32)
    sq = (x * x).astype(np.float32).astype(np.float64).sum(axis=-1, keepdims=True)
    mean = (sq / x.shape[-1]).astype(np.float32)
    scale = (np.float32(1.0) / np.sqrt(mean + np.float32(eps))).astype(np.float32)
    return (x * scale * w).astype(np.float32)


def rope(x, n_heads, hd, pos0, theta, neox):
    x = x.reshape(x.shape[0], n_heads, hd).copy()
    half = hd // 2
    i = np.arange(half, dtype=np.float32)
    freq = (np.float32(1.0) / np.power(np.float32(theta), (2 * i / np.float32(hd)).astype(np.float32))).astype(np.float32)
    for r in range(x.shape[0]):
        ang = (np.float32(pos0 + r) * freq).astype(np.float32)
        s, c = np.sin(ang).astype(np.float32), np.cos(ang).astype(np.float32)
        ia, ib = (np.arange(half), np.arange(half) + half) if neox else (2 * np.arange(half), 2 * np.arange(half) + 1)
        a, b = x[r][:, ia].copy(), x[r][:, ib].copy()
        x[r][:, ia] = a * c - b * s
        x[r][:, ib] = a * s + b * c
    return x.reshape(x.shape[0], n_heads * hd)


def lin(kind, raw, rows, cols, x):
    return fo.matmul_f64(kind, raw, rows, cols, fo.q8_1_round(np.ascontiguousarray(x, np.float32))).astype(np.float32)


class OracleDecoder:
    def __init__(self, cfg, layers, tok_embd, tok_kind, out_norm, output=None, output_kind=None):
        self.cfg, self.layers, self.tok, self.tok_kind, self.out_norm = cfg, layers, tok_embd, tok_kind, np.asarray(out_norm, np.float32)
        self.head, self.head_kind = (tok_embd, tok_kind) if output is None else (output, output_kind)
        self.k = [np.zeros((0, cfg.n_kv * cfg.head_dim), np.float32) for _ in layers]
        self.v = [np.zeros((0, cfg.n_kv * cfg.head_dim), np.float32) for _ in layers]
        self.pos = 0
        rb = fo.row_bytes(tok_kind, cfg.hidden)
        self.embd_row = lambda t: fo.dequant(tok_kind, self.tok[t * rb:(t + 1) * rb])

    def forward(self, ids):
        c = self.cfg
        hd, H = c.head_dim, c.hidden
        x = np.stack([self.embd_row(int(t)) for t in ids]).astype(np.float32)
        n = x.shape[0]
        for li, L in enumerate(self.layers):
            k = L.kinds
            h = rmsnorm(x, np.asarray(L.attn_norm, np.float32), c.eps)
            q = lin(k["wq"], L.wq, c.n_heads * hd, H, h)
            kk = lin(k["wk"], L.wk, c.n_kv * hd, H, h)
            v = lin(k["wv"], L.wv, c.n_kv * hd, H, h)
            if c.qk_norm:
                q = rmsnorm(q.reshape(-1, hd), np.asarray(L.q_norm, np.float32), c.eps).reshape(n, -1)
                kk = rmsnorm(kk.reshape(-1, hd), np.asarray(L.k_norm, np.float32), c.eps).reshape(n, -1)
            q = rope(q, c.n_heads, hd, self.pos, c.rope_theta, c.neox)
            kk = rope(kk, c.n_kv, hd, self.pos, c.rope_theta, c.neox)
            self.k[li] = np.concatenate([self.k[li], kk])
            self.v[li] = np.concatenate([self.v[li], v])
            a = np.zeros((n, c.n_heads * hd), np.float32)
            grp = c.n_heads // c.n_kv
            for r in range(n):
                T = self.pos + r + 1
                for hh in range(c.n_heads):
                    kv = hh // grp
                    K = self.k[li][:T, kv * hd:(kv + 1) * hd].astype(np.float64)
                    V = self.v[li][:T, kv * hd:(kv + 1) * hd].astype(np.float64)
                    s = K @ q[r, hh * hd:(hh + 1) * hd].astype(np.float64) * (hd ** -0.5)
                    p = np.exp(s - s.max())
                    a[r, hh * hd:(hh + 1) * hd] = (p @ V / p.sum()).astype(np.float32)
            x = (x + lin(k["wo"], L.wo, H, c.n_heads * hd, a)).astype(np.float32)
            h2 = rmsnorm(x, np.asarray(L.ffn_norm, np.float32), c.eps)
            if c.n_experts:
                x = (x + self.routed(L, h2)).astype(np.float32)
                continue
            g = lin(k["gate"], L.gate, c.ffn, H, h2)
            u = lin(k["up"], L.up, c.ffn, H, h2)
            act = fo.silu_mul(g.ravel(), u.ravel()).reshape(g.shape)
            x = (x + lin(k["down"], L.down, H, c.ffn, act)).astype(np.float32)
        hn = rmsnorm(x[-1:], self.out_norm, c.eps)
        logits = lin(self.head_kind, self.head, c.vocab, H, hn)[0]
        self.pos += n
        return logits

    def routed(self, L, h):
        """Router logits in f32, top-k with ties to the lower id, every chosen expert's SwiGLU FFN,
        weighted sum from zero in routing order."""
        c = self.cfg
        H, F, kind = c.hidden, c.ffn, L.kinds["experts"]
        logits = (h.astype(np.float32) @ np.asarray(L.router, np.float32).T).astype(np.float32)
        ids, w = fo.route_top_k(logits, c.top_k, c.route_mode)
        pg, pd = F * fo.row_bytes(kind, H), H * fo.row_bytes(kind, F)
        gate, up, down = (np.ascontiguousarray(t, np.uint8).ravel() for t in (L.gate, L.up, L.down))
        out = np.zeros((h.shape[0], H), np.float32)
        for t in range(h.shape[0]):
            ys = []
            for e in ids[t]:
                g = lin(kind, gate[e * pg:(e + 1) * pg], F, H, h[t:t + 1])[0]
                u = lin(kind, up[e * pg:(e + 1) * pg], F, H, h[t:t + 1])[0]
                ys.append(lin(kind, down[e * pd:(e + 1) * pd], H, F, fo.silu_mul(g, u)[None])[0])
            out[t] = fo.combine(np.stack(ys), w[t])
        return out

    def generate(self, prompt, n_new, margins=None):
        out = []
        logits = self.forward(prompt)
        for _ in range(n_new):
            t = int(np.argmax(logits))
            out.append(t)
            if margins is not None:      # gap between the chosen logit and the runner-up, relative to the logits' spread
                top2 = np.partition(logits, -2)[-2:]
                margins.append(float((top2[1] - top2[0]) / max(float(np.std(logits)), 1e-30)))
            if len(out) < n_new:
                logits = self.forward([t])
        return out
