"""The decoder's host logic on CPU: `frink_b200.decoder.Decoder` driven through the
oracle-backed stand-in for the device ops, against the oracle pipeline.  Covers the
batched path (more than 8 rows), the fused decode path (merged q/k/v and gate/up,
norm and GLU folded into the matvecs, residual adds in place) and the position word."""
import numpy as np
import torch

from oracle import frink_oracle as fo
from tests import cpu_ops
from tests import oracle_decoder as od
from tests.helpers import rel_l2


def _model(uniform):
    from frink_b200.decoder import DecoderConfig, LayerWeights
    cfg = DecoderConfig(n_layers=2, hidden=256, n_heads=4, n_kv=2, head_dim=64, ffn=512, vocab=300)
    rng = np.random.default_rng(17)
    H, hd = cfg.hidden, cfg.head_dim
    layers = []
    for _ in range(cfg.n_layers):
        kd = {"wq": fo.Q4_K, "wk": fo.Q4_K, "wv": fo.Q4_K if uniform else fo.Q6_K, "wo": fo.Q4_K, "gate": fo.Q4_K, "up": fo.Q4_K, "down": fo.Q6_K}
        enc = lambda name, r, c: fo.encode(kd[name], (rng.standard_normal((r, c)) * 0.05).astype(np.float32))
        norm = lambda n: (1 + 0.1 * rng.standard_normal(n)).astype(np.float32)
        layers.append(LayerWeights(attn_norm=norm(H), wq=enc("wq", cfg.n_heads * hd, H), wk=enc("wk", cfg.n_kv * hd, H), wv=enc("wv", cfg.n_kv * hd, H),
                                   wo=enc("wo", H, cfg.n_heads * hd), ffn_norm=norm(H), gate=enc("gate", cfg.ffn, H), up=enc("up", cfg.ffn, H),
                                   down=enc("down", H, cfg.ffn), kinds=kd))
    tok = fo.encode(fo.Q8_0, rng.standard_normal((cfg.vocab, H)).astype(np.float32))
    head = fo.encode(fo.Q8_0, (rng.standard_normal((cfg.vocab, H)) * 0.5).astype(np.float32))
    return cfg, layers, tok, (1 + 0.1 * rng.standard_normal(H)).astype(np.float32), head


def test_decoder_host_logic_matches_the_oracle_pipeline():
    from frink_b200.decoder import Decoder
    for uniform in (False, True):
        cfg, layers, tok, out_norm, head = _model(uniform)
        dec = Decoder(cfg, layers, tok, fo.Q8_0, out_norm, output=head, output_kind=fo.Q8_0, max_seq=32, ops=cpu_ops, device="cpu")
        ora = od.OracleDecoder(cfg, layers, tok, fo.Q8_0, out_norm, head, fo.Q8_0)
        prompt = np.random.default_rng(5).integers(0, cfg.vocab, 10).astype(np.int32)
        lg = dec.forward(torch.from_numpy(prompt)).numpy()[0]          # 10 rows: the batched path
        assert rel_l2(lg, ora.forward(prompt)) <= 1e-5
        assert int(dec.pos[0]) == 10
        nxt = np.array([int(np.argmax(lg))], np.int32)
        lg1 = dec.forward(torch.from_numpy(nxt)).numpy()[0]            # one row: the fused decode path
        assert rel_l2(lg1, ora.forward(nxt)) <= 1e-5
        three = np.array([3, 1, 4], np.int32)
        lg3 = dec.forward(torch.from_numpy(three)).numpy()[0]          # three rows through the fused path
        assert rel_l2(lg3, ora.forward(three)) <= 1e-5
        assert int(dec.pos[0]) == 14


def test_gpt_oss_routed_layer_host_logic_against_the_oracle_composition():
    """`prefill.run_device_routed_oai` (router bias, per-expert bias rows, the clamped SwiGLU on the biased gate and up)
    on the CPU ops, for a few rows (slots of the indexed matvecs) and for more than eight (pairs grouped by expert, the
    expert of every permuted row found from the group offsets), against the reference's composition written out:
    route_top_k -> per expert gate/up + bias -> swiglu_oai -> down + bias -> combine
    (crates/frink-moe/src/lib.rs:567, 1039-1060, 1246)."""
    from frink_b200 import prefill
    E, k, H, F = 6, 2, 128, 96
    rng = np.random.default_rng(31)
    raws = {n: [fo.encode(fo.MXFP4, (rng.standard_normal((r, c)) * 0.05).astype(np.float32)) for _ in range(E)]
            for n, r, c in (("gate", F, H), ("up", F, H), ("down", H, F))}
    mk = lambda n, r, c: cpu_ops.Weights(np.concatenate(raws[n]), fo.MXFP4, r, c, n_mats=E)
    router = (rng.standard_normal((E, H)) * 0.5).astype(np.float32)
    rb = (rng.standard_normal(E) * 0.5).astype(np.float32)
    gb, ub, db = (rng.standard_normal((E, n)).astype(np.float32) * 0.2 for n in (F, F, H))
    layer = prefill.RoutedLayer(torch.from_numpy(router), mk("gate", F, H), mk("up", F, H), mk("down", H, F), k=k, mode=1, act=1,
                                router_bias=torch.from_numpy(rb))
    biases = tuple(torch.from_numpy(b) for b in (gb, ub, db))
    x = rng.standard_normal((12, H)).astype(np.float32)

    def want_rows(xs):
        ids, w = fo.route_top_k((xs @ router.T).astype(np.float32), k, 1, rb)
        out = np.zeros((xs.shape[0], H), np.float32)
        for t in range(xs.shape[0]):
            ys = []
            for e in ids[t]:
                xq = fo.q8_1_round(xs[t])
                g = fo.matmul_f64(fo.MXFP4, raws["gate"][e], F, H, xq)[0].astype(np.float32) + gb[e]
                u = fo.matmul_f64(fo.MXFP4, raws["up"][e], F, H, xq)[0].astype(np.float32) + ub[e]
                ys.append(fo.matmul_f64(fo.MXFP4, raws["down"][e], H, F, fo.q8_1_round(fo.swiglu_oai(g, u)))[0].astype(np.float32) + db[e])
            out[t] = fo.combine(np.stack(ys), w[t])
        return out

    for rows in (1, 3, 12):
        got = prefill.run_device_routed_oai(layer, biases, torch.from_numpy(x[:rows]), cpu_ops).numpy()
        assert rel_l2(got, want_rows(x[:rows])) <= 1e-5, rows
    # added into a residual stream instead of returned
    res = torch.from_numpy(rng.standard_normal((3, H)).astype(np.float32))
    base = res.numpy().copy()
    prefill.run_device_routed_oai(layer, biases, torch.from_numpy(x[:3]), cpu_ops, residual=res)
    assert rel_l2(res.numpy(), base + want_rows(x[:3])) <= 1e-5
