"""The decoder glue and a whole small model against the CPU oracle pipeline:
each glue kernel on its own, then greedy decoding of a random-init Llama-shaped
model (the parity-sized stand-in for BASELINE config 3) token for token."""
import numpy as np
import pytest
import torch

from oracle import frink_oracle as fo
from tests import oracle_decoder as od
from tests.helpers import rel_l2, synth_weights

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kind", [fo.Q6_K, fo.Q4_K, fo.Q8_0, fo.MXFP4])
def test_get_rows_is_the_host_dequant(kind):
    from frink_b200 import device
    rows, cols = 50, 768 if kind != fo.MXFP4 else 960
    raw = fo.encode(kind, synth_weights(rows, cols, 3))
    w = device.Weights(raw, kind, rows, cols)
    ids = np.array([7, 0, 49, 7], np.int32)
    got = device.get_rows(w, torch.from_numpy(ids).cuda()).cpu().numpy()
    want = fo.dequant(kind, raw).reshape(rows, cols)[ids]
    assert np.array_equal(got, want)   # bit for bit, as the reference's get_rows is


def test_rmsnorm_rope_attention_argmax():
    from frink_b200 import device
    rng = np.random.default_rng(0)
    x = rng.standard_normal((5, 3072)).astype(np.float32)
    r = rng.standard_normal((5, 3072)).astype(np.float32)
    w = rng.standard_normal(3072).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    got = device.rmsnorm(xd, torch.from_numpy(w).cuda(), 1e-5, residual=torch.from_numpy(r).cuda()).cpu().numpy()
    assert np.array_equal(xd.cpu().numpy(), x + r)
    assert np.allclose(got, od.rmsnorm(x + r, w, 1e-5), rtol=2e-6, atol=1e-7)
    for neox in (False, True):
        q = rng.standard_normal((6, 4 * 128)).astype(np.float32)
        pos = torch.tensor([37], dtype=torch.int32).cuda()
        got = device.rope(torch.from_numpy(q).cuda(), 4, 128, pos, 500000.0, neox).cpu().numpy()
        assert np.allclose(got, od.rope(q, 4, 128, 37, 500000.0, neox), rtol=1e-4, atol=2e-5)
    # attention: 3 query rows at positions 20..22 over 23 keys, 8 heads / 2 kv heads
    nh, nkv, hd, T0, nq = 8, 2, 64, 20, 3
    K = rng.standard_normal((T0 + nq, nkv * hd)).astype(np.float32)
    V = rng.standard_normal((T0 + nq, nkv * hd)).astype(np.float32)
    Q = rng.standard_normal((nq, nh * hd)).astype(np.float32)
    pos = torch.tensor([T0], dtype=torch.int32).cuda()
    got = device.attention(torch.from_numpy(Q).cuda(), torch.from_numpy(K).cuda(), torch.from_numpy(V).cuda(), nh, nkv, hd, pos).cpu().numpy()
    want = np.zeros_like(Q)
    for rr in range(nq):
        for h in range(nh):
            kv = h // (nh // nkv)
            s = K[:T0 + rr + 1, kv * hd:(kv + 1) * hd].astype(np.float64) @ Q[rr, h * hd:(h + 1) * hd].astype(np.float64) * hd ** -0.5
            p = np.exp(s - s.max())
            want[rr, h * hd:(h + 1) * hd] = p @ V[:T0 + rr + 1, kv * hd:(kv + 1) * hd].astype(np.float64) / p.sum()
    assert np.allclose(got, want, rtol=1e-4, atol=1e-5)
    lg = rng.standard_normal((3, 5000)).astype(np.float32)
    lg[1, 77] = lg[1, 4000] = 9.0
    assert list(device.argmax(torch.from_numpy(lg).cuda()).cpu().numpy()) == [int(np.argmax(lg[0])), 77, int(np.argmax(lg[2]))]


def small_llama(seed=1):
    from frink_b200.decoder import DecoderConfig, LayerWeights
    cfg = DecoderConfig(n_layers=2, hidden=512, n_heads=4, n_kv=2, head_dim=128, ffn=1024, vocab=2048)
    rng = np.random.default_rng(seed)
    H, hd = cfg.hidden, cfg.head_dim
    layers = []
    for li in range(cfg.n_layers):
        kd = {"wq": fo.Q4_K, "wk": fo.Q4_K, "wv": fo.Q6_K, "wo": fo.Q4_K, "gate": fo.Q4_K, "up": fo.Q4_K, "down": fo.Q6_K}
        enc = lambda name, r, c, s: fo.encode(kd[name], (rng.standard_normal((r, c)) * s).astype(np.float32))
        layers.append(LayerWeights(
            attn_norm=1 + 0.1 * rng.standard_normal(H), wq=enc("wq", cfg.n_heads * hd, H, 0.05), wk=enc("wk", cfg.n_kv * hd, H, 0.05),
            wv=enc("wv", cfg.n_kv * hd, H, 0.05), wo=enc("wo", H, cfg.n_heads * hd, 0.05), ffn_norm=1 + 0.1 * rng.standard_normal(H),
            gate=enc("gate", cfg.ffn, H, 0.05), up=enc("up", cfg.ffn, H, 0.05), down=enc("down", H, cfg.ffn, 0.05), kinds=kd))
    # an untied head with clear margins: token identity should test the pipeline, not f32 coin flips on flat logits
    tok = fo.encode(fo.Q6_K, rng.standard_normal((cfg.vocab, H)).astype(np.float32))
    head = fo.encode(fo.Q6_K, (rng.standard_normal((cfg.vocab, H)) * 0.5).astype(np.float32))
    return cfg, layers, tok, (1 + 0.1 * rng.standard_normal(H)).astype(np.float32), head


def test_small_llama_greedy_tokens_match_the_oracle():
    from frink_b200.decoder import Decoder
    cfg, layers, tok, out_norm, head = small_llama()
    dec = Decoder(cfg, layers, tok, fo.Q6_K, out_norm, output=head, output_kind=fo.Q6_K, max_seq=128)
    ora = od.OracleDecoder(cfg, layers, tok, fo.Q6_K, out_norm, head, fo.Q6_K)
    prompt = np.random.default_rng(0x70C).integers(0, cfg.vocab, 20).astype(np.int32)
    # logits after the prompt (prefill takes the GEMM path: 20 rows)
    lg = dec.forward(torch.from_numpy(prompt).cuda()).cpu().numpy()[0]
    lo = ora.forward(prompt)
    assert rel_l2(lg, lo) <= 1e-3
    dec.reset()
    ora = od.OracleDecoder(cfg, layers, tok, fo.Q6_K, out_norm, head, fo.Q6_K)
    n_new = 24
    got = dec.generate(torch.from_numpy(prompt).cuda(), n_new)
    want = ora.generate(list(prompt), n_new)
    first = next((i for i in range(n_new) if got[i] != want[i]), None)
    assert first is None, f"first divergence at generated token {first}: {got[first]} vs {want[first]}"
    # the captured-graph decode loop reproduces the eager one
    dec.reset()
    assert dec.generate(torch.from_numpy(prompt).cuda(), n_new, use_graph=True) == got
