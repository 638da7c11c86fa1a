"""Shared fixtures for the tests: seeded synthetic tensors and the reference's
own fixture generator for the K-quant encoder goldens."""
import json
import os

import numpy as np

from oracle import frink_oracle as fo

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "frink_goldens.json")


def goldens():
    with open(GOLDEN) as f:
        t = json.load(f)["tables"]
    return {k: v["values"] for k, v in t.items()}


def xorshift_unit(n, seed):
    """The reference fixtures' generator: 32-bit xorshift, top 24 bits to [-1, 1)
    (crates/frink-quant/src/encode.rs:138-150, encode/testdata.rs:92-100)."""
    out = np.empty(n, np.float32)
    s = seed & 0xFFFFFFFF
    for i in range(n):
        s ^= (s << 13) & 0xFFFFFFFF
        s ^= s >> 17
        s ^= (s << 5) & 0xFFFFFFFF
        out[i] = np.float32(np.float32(s >> 8) / np.float32(8388608.0)) - np.float32(1.0)
    return out


def k_quant_fixture(real_weight_bits):
    """crates/frink-quant/src/encode/testdata.rs:90-135: four shaped synthetic
    super-blocks rounded through f16, then eight real-weight super-blocks given
    as f16 bit patterns."""
    gains = [0.02, 0.05, 0.1, 0.25]
    v = xorshift_unit(4 * 8 * 32, 0xB54CDA26)
    out = np.empty(4 * 256, np.float32)
    for sub in range(32):
        for i in range(32):
            x = np.float32(v[sub * 32 + i])
            if sub == 8:
                s = np.float32(0.0)
            elif sub == 9:
                s = np.float32(0.125)
            elif sub == 10:
                s = np.float32(abs(x) * np.float32(0.05) + np.float32(0.01))
            elif sub == 11:
                s = np.float32(-(np.float32(abs(x) * np.float32(0.05)) + np.float32(0.01)))
            elif sub == 17:
                s = np.float32(x * np.float32(1e-4))
            else:
                s = np.float32(x * np.float32(gains[sub % 4]))
            out[sub * 32 + i] = np.float32(np.float16(s))
    real = np.array(real_weight_bits, np.uint16).view(np.float16).astype(np.float32)
    return np.concatenate([out, real])


def synth_weights(rows, cols, seed):
    """Synthetic weight matrix of the benchmark's distribution, N(0, 0.02^2)."""
    rng = np.random.default_rng(seed)
    return (rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(0.02)).astype(np.float32)


def synth_acts(batch, cols, seed):
    rng = np.random.default_rng(seed)
    return rng.standard_normal((batch, cols), dtype=np.float32)


def rel_l2(got, want):
    got = np.asarray(got, np.float64).ravel()
    want = np.asarray(want, np.float64).ravel()
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))


def max_abs_over_inf(got, want):
    got = np.asarray(got, np.float64).ravel()
    want = np.asarray(want, np.float64).ravel()
    return float(np.max(np.abs(got - want)) / max(np.max(np.abs(want)), 1e-30))


def tiny_gpt_oss(seed=5):
    """A two-layer model of gpt-oss's layer form: BF16 attention projections with biases, sinks, layer 0 windowed,
    four MXFP4 experts (top 2) with a bias per expert projection, the clamped SwiGLU and a router bias."""
    from frink_b200.decoder import DecoderConfig, LayerWeights
    cfg = DecoderConfig(n_layers=2, hidden=256, n_heads=8, n_kv=2, head_dim=64, ffn=256, vocab=512, rope_theta=150000.0, eps=1e-5, neox=True,
                        n_experts=4, top_k=2, route_mode=1, oai=True, sliding_window=8, swa_period=2)
    rng = np.random.default_rng(seed)
    H, hd, E = cfg.hidden, cfg.head_dim, cfg.n_experts
    bf = lambda r, c, s: fo.encode(fo.BF16, (rng.standard_normal((r, c)) * s).astype(np.float32))
    mx = lambda r, c: np.concatenate([fo.encode(fo.MXFP4, (rng.standard_normal((r, c)) * 0.05).astype(np.float32)) for _ in range(E)])
    vec = lambda n, s=0.1: (rng.standard_normal(n) * s).astype(np.float32)
    layers = []
    for _ in range(cfg.n_layers):
        layers.append(LayerWeights(
            attn_norm=1 + vec(H), wq=bf(cfg.n_heads * hd, H, 0.05), wk=bf(cfg.n_kv * hd, H, 0.05), wv=bf(cfg.n_kv * hd, H, 0.05),
            wo=bf(H, cfg.n_heads * hd, 0.05), ffn_norm=1 + vec(H), gate=mx(cfg.ffn, H), up=mx(cfg.ffn, H), down=mx(H, cfg.ffn),
            router=(rng.standard_normal((E, H)) * 0.5).astype(np.float32), sinks=vec(cfg.n_heads, 1.0),
            bq=vec(cfg.n_heads * hd), bk=vec(cfg.n_kv * hd), bv=vec(cfg.n_kv * hd), bo=vec(H), router_bias=vec(E, 0.5),
            gate_b=vec(E * cfg.ffn).reshape(E, cfg.ffn), up_b=vec(E * cfg.ffn).reshape(E, cfg.ffn), down_b=vec(E * H).reshape(E, H),
            kinds={"wq": fo.BF16, "wk": fo.BF16, "wv": fo.BF16, "wo": fo.BF16, "experts": fo.MXFP4}))
    tok = fo.encode(fo.BF16, rng.standard_normal((cfg.vocab, H)).astype(np.float32))
    head = fo.encode(fo.BF16, (rng.standard_normal((cfg.vocab, H)) * 0.5).astype(np.float32))
    return cfg, layers, tok, (1 + vec(H)).astype(np.float32), head
