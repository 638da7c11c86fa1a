"""The decoder glue and a whole small model against the CPU oracle pipeline:
each glue kernel on its own, then greedy decoding of a random-init Llama-shaped
model (the parity-sized stand-in for the 3B Llama shape) token for token."""
import numpy as np
import pytest
import torch

from oracle import frink_oracle as fo
from tests import oracle_decoder as od
from tests.helpers import rel_l2, synth_weights, tiny_gpt_oss

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


@pytest.mark.parametrize("kind", [fo.Q4_K, fo.Q6_K, fo.Q8_0, fo.MXFP4])
@pytest.mark.parametrize("batch", [1, 3])
def test_fused_gemv_equals_the_separate_kernels(kind, batch):
    """The matvec with RMSNorm / SiLU*up in its prologue and the residual add in its
    epilogue against the same steps as separate launches (which the other tests tie
    to the oracle)."""
    from frink_b200 import device
    rng = np.random.default_rng(5 + batch)
    rows, cols = 520, 1024
    # One kernel serves the plain and the fused launch of a shape, so the two agree bit for bit -- except Q4_K at batch 1,
    # where the plain matvec has a kernel of its own (another f32 summation order; both are tied to the oracle elsewhere).
    if kind == fo.Q4_K and batch == 1:
        same = lambda a, b: torch.allclose(a, b, rtol=2e-5, atol=2e-6 * float(b.abs().max()))
    else:
        same = torch.equal
    w = device.Weights(fo.encode(kind, synth_weights(rows, cols, 11)), kind, rows, cols)
    x = torch.from_numpy(rng.standard_normal((batch, cols)).astype(np.float32)).cuda()
    nw = torch.from_numpy((1 + 0.1 * rng.standard_normal(cols)).astype(np.float32)).cuda()
    want = device.gemv(w, device.rmsnorm(x.clone(), nw, 1e-5))
    got = device.gemv_fused(w, x, norm_weight=nw, eps=1e-5)
    assert torch.allclose(got, want, rtol=1e-5, atol=1e-6)
    # gate | up as the two halves of one wider buffer, as the merged projection leaves them
    gu = torch.from_numpy(rng.standard_normal((batch, 2 * cols)).astype(np.float32)).cuda()
    for act in (0, 1):
        want = device.gemv(w, device.glu(gu[:, :cols].contiguous(), gu[:, cols:].contiguous(), act))
        got = device.gemv_fused(w, gu[:, :cols], glu_up=gu[:, cols:], glu_act=act)
        assert same(got, want)
    # rows read as (gate, up) pairs: the gated activation formed in the epilogue
    full = device.gemv(w, x)
    for act in (0, 1):
        want = device.glu(full[:, 0::2].contiguous(), full[:, 1::2].contiguous(), act)
        got = device.gemv_fused(w, x, pair_glu=act + 1)
        assert got.shape == (batch, rows // 2) and same(got, want)
    res = torch.from_numpy(rng.standard_normal((batch, rows)).astype(np.float32)).cuda()
    out = res.clone()
    device.gemv_fused(w, x, out=out, accumulate=True)
    assert same(out, res + device.gemv(w, x))
    assert device.device_error() == 0


def test_rope_kv_strided_attention_and_wide_argmax():
    from frink_b200 import device
    rng = np.random.default_rng(9)
    nh, nkv, hd, n, p0 = 8, 2, 128, 3, 11
    hq, kvw = nh * hd, nkv * hd
    qkv = torch.from_numpy(rng.standard_normal((n, hq + 2 * kvw)).astype(np.float32)).cuda()
    pos = torch.tensor([p0], dtype=torch.int32).cuda()
    for neox in (False, True):
        q0, k0, v0 = (t.contiguous() for t in (qkv[:, :hq], qkv[:, hq:hq + kvw], qkv[:, hq + kvw:]))
        kc0 = torch.from_numpy(rng.standard_normal((32, kvw)).astype(np.float32)).cuda()
        vc0 = torch.from_numpy(rng.standard_normal((32, kvw)).astype(np.float32)).cuda()
        kc1, vc1 = kc0.clone(), vc0.clone()
        device.rope(q0, nh, hd, pos, 1e4, neox)
        device.rope(k0, nkv, hd, pos, 1e4, neox)
        device.kv_append(kc0, k0, pos)
        device.kv_append(vc0, v0, pos)
        buf = qkv.clone()
        q1, k1, v1 = buf[:, :hq], buf[:, hq:hq + kvw], buf[:, hq + kvw:]
        device.rope_kv(q1, k1, v1, nh, nkv, hd, pos, 1e4, neox, kc1, vc1)
        assert torch.equal(q1, q0) and torch.equal(k1, k0) and torch.equal(kc1, kc0) and torch.equal(vc1, vc0)
        # Qwen3's per-head q/k RMSNorm folded into the same launch
        qn = torch.from_numpy((1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)).cuda()
        kn = torch.from_numpy((1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)).cuda()
        q2, k2, v2 = (t.contiguous() for t in (qkv[:, :hq], qkv[:, hq:hq + kvw], qkv[:, hq + kvw:]))
        q2 = device.rmsnorm(q2.view(-1, hd), qn, 1e-6).view(n, -1)
        k2 = device.rmsnorm(k2.view(-1, hd), kn, 1e-6).view(n, -1)
        kc2, vc2 = kc0.clone(), vc0.clone()
        device.rope_kv(q2, k2, v2, nh, nkv, hd, pos, 1e4, neox, kc2, vc2)
        buf3 = qkv.clone()
        kc3, vc3 = kc0.clone(), vc0.clone()
        device.rope_kv(buf3[:, :hq], buf3[:, hq:hq + kvw], buf3[:, hq + kvw:], nh, nkv, hd, pos, 1e4, neox, kc3, vc3, q_norm=qn, k_norm=kn, eps=1e-6)
        assert torch.allclose(buf3[:, :hq], q2, rtol=1e-6, atol=1e-7) and torch.allclose(kc3, kc2, rtol=1e-6, atol=1e-7) and torch.equal(vc3, vc2)
        # a query that is a column slice of a wider buffer
        a0 = device.attention(q0, kc0, vc0, nh, nkv, hd, pos)
        a1 = device.attention(q1, kc1, vc1, nh, nkv, hd, pos)
        assert torch.equal(a0, a1)
    # argmax over a vocabulary-sized row: many blocks per row, ties inside and across blocks
    lg = rng.standard_normal((3, 128256)).astype(np.float32)
    lg[1, 120000] = lg[1, 513] = lg[1, 70001] = 9.5
    lg[2, 128255] = 11.0
    lg[0, 5] = np.nan
    want = [int(np.nanargmax(lg[0])), 513, 128255]
    for _ in range(2):   # the second call finds the arrival counters rewound
        assert list(device.argmax(torch.from_numpy(lg).cuda()).cpu().numpy()) == want


def small_llama(seed=1, uniform=False):
    from frink_b200.decoder import DecoderConfig, LayerWeights
    cfg = DecoderConfig(n_layers=2, hidden=512, n_heads=4, n_kv=2, head_dim=128, ffn=1024, vocab=2048)
    rng = np.random.default_rng(seed)
    H, hd = cfg.hidden, cfg.head_dim
    layers = []
    for li in range(cfg.n_layers):
        kd = {"wq": fo.Q4_K, "wk": fo.Q4_K, "wv": fo.Q4_K if uniform else fo.Q6_K, "wo": fo.Q4_K, "gate": fo.Q4_K, "up": fo.Q4_K, "down": fo.Q6_K}
        enc = lambda name, r, c, s: fo.encode(kd[name], (rng.standard_normal((r, c)) * s).astype(np.float32))
        layers.append(LayerWeights(
            attn_norm=1 + 0.1 * rng.standard_normal(H), wq=enc("wq", cfg.n_heads * hd, H, 0.05), wk=enc("wk", cfg.n_kv * hd, H, 0.05),
            wv=enc("wv", cfg.n_kv * hd, H, 0.05), wo=enc("wo", H, cfg.n_heads * hd, 0.05), ffn_norm=1 + 0.1 * rng.standard_normal(H),
            gate=enc("gate", cfg.ffn, H, 0.05), up=enc("up", cfg.ffn, H, 0.05), down=enc("down", H, cfg.ffn, 0.05), kinds=kd))
    # an untied head with clear margins: token identity should test the pipeline, not f32 coin flips on flat logits
    tok = fo.encode(fo.Q6_K, rng.standard_normal((cfg.vocab, H)).astype(np.float32))
    head = fo.encode(fo.Q6_K, (rng.standard_normal((cfg.vocab, H)) * 0.5).astype(np.float32))
    return cfg, layers, tok, (1 + 0.1 * rng.standard_normal(H)).astype(np.float32), head


@pytest.mark.parametrize("uniform", [False, True])
def test_small_llama_greedy_tokens_match_the_oracle(uniform):
    """uniform: q, k and v share a block format and run as one merged, norm-fused matvec;
    otherwise v is Q6_K (the usual K-quant mix) and the norm stays a kernel of its own."""
    from frink_b200.decoder import Decoder
    cfg, layers, tok, out_norm, head = small_llama(uniform=uniform)
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


def recipe_llama(seed=7):
    """A Llama-shaped model small enough for the f64 oracle, quantized with the Q4_K_M recipe
    (crates/frink-cli/src/quantize/recipe.rs `use_more_bits`: Q6_K for attn_v and ffn_down on the
    layers the rule names, Q4_K elsewhere, a Q6_K embedding)."""
    from frink_b200.decoder import DecoderConfig, LayerWeights
    cfg = DecoderConfig(n_layers=4, hidden=1024, n_heads=8, n_kv=2, head_dim=128, ffn=2816, vocab=4096)
    rng = np.random.default_rng(seed)
    H, hd, n = cfg.hidden, cfg.head_dim, cfg.n_layers
    more = lambda i: i < n // 8 or i >= 7 * n // 8 or (i - n // 8) % 3 == 2
    layers = []
    for li in range(n):
        hi = fo.Q6_K if more(li) else fo.Q4_K
        kd = {"wq": fo.Q4_K, "wk": fo.Q4_K, "wv": hi, "wo": fo.Q4_K, "gate": fo.Q4_K, "up": fo.Q4_K, "down": hi}
        enc = lambda name, r, c, s: fo.encode(kd[name], (rng.standard_normal((r, c)) * s).astype(np.float32))
        layers.append(LayerWeights(
            attn_norm=1 + 0.1 * rng.standard_normal(H), wq=enc("wq", cfg.n_heads * hd, H, 0.02), wk=enc("wk", cfg.n_kv * hd, H, 0.02),
            wv=enc("wv", cfg.n_kv * hd, H, 0.02), wo=enc("wo", H, cfg.n_heads * hd, 0.02), ffn_norm=1 + 0.1 * rng.standard_normal(H),
            gate=enc("gate", cfg.ffn, H, 0.02), up=enc("up", cfg.ffn, H, 0.02), down=enc("down", H, cfg.ffn, 0.02), kinds=kd))
    assert [L.kinds["down"] for L in layers] == [fo.Q4_K, fo.Q4_K, fo.Q6_K, fo.Q6_K]
    tok = fo.encode(fo.Q6_K, rng.standard_normal((cfg.vocab, H)).astype(np.float32))
    head = fo.encode(fo.Q6_K, (rng.standard_normal((cfg.vocab, H)) * 0.5).astype(np.float32))
    return cfg, layers, tok, (1 + 0.1 * rng.standard_normal(H)).astype(np.float32), head


def decisive_head(cfg, tok, beta=0.08, seed=99):
    """An output head whose logits have a usable top-1 margin.  Random-init logits are nearly flat
    (the gap between the two largest of 4096 Gaussian logits is below 1e-3 of their spread somewhere
    in any 128 steps), far below what the order of f32 sums does to a stack of q8_1 quantizers.  So
    every token t gets a successor s(t) whose head row leans towards t's embedding (strength beta);
    at beta = 0.08 the planted successor wins about four steps in five and the model's own logits
    decide the rest, so the sequence still depends on every layer."""
    rng = np.random.default_rng(seed)
    succ = rng.permutation(cfg.vocab)
    hf = (rng.standard_normal((cfg.vocab, cfg.hidden)) * 0.5).astype(np.float32)
    hf[succ] += np.float32(beta) * fo.dequant(fo.Q6_K, tok).reshape(cfg.vocab, cfg.hidden)
    return fo.encode(fo.Q6_K, hf), succ


def test_greedy_decode_of_128_tokens_is_token_identical():
    """128 greedy tokens after a 32-token prompt, eager and from the captured graph, against the
    oracle pipeline (the harness frink's `verify` uses: crates/frink-cli/src/verify_engine.rs:70-93
    compares token ids and reports the first divergence).

    Token identity can only be asked where the logit margins exceed what the order of f32 sums
    does: an activation that lands on the other side of a q8_1 rounding boundary moves a matmul's
    output by 1e-4, the next quantizers amplify that, and after four layers the logits of the two
    pipelines differ by several 1e-3 of their spread (printed below, and bounded).  The head is
    therefore `decisive_head`; the oracle's smallest top-2 margin over the 128 steps is 0.04 of the
    spread, printed with the result."""
    from frink_b200.decoder import Decoder
    cfg, layers, tok, out_norm, _ = recipe_llama()
    head, succ = decisive_head(cfg, tok)
    dec = Decoder(cfg, layers, tok, fo.Q6_K, out_norm, output=head, output_kind=fo.Q6_K, max_seq=256)
    ora = od.OracleDecoder(cfg, layers, tok, fo.Q6_K, out_norm, head, fo.Q6_K)
    prompt = np.random.default_rng(0x70C).integers(0, cfg.vocab, 32).astype(np.int32)
    n_new = 128
    margins = []
    want = ora.generate(list(prompt), n_new, margins=margins)
    planted = sum(1 for a, b in zip([int(prompt[-1])] + want[:-1], want) if succ[a] == b)
    assert min(margins) > 3e-2 and len(set(want)) == n_new and planted < 110
    lg = dec.forward(torch.from_numpy(prompt).cuda()).cpu().numpy()[0]
    lo = od.OracleDecoder(cfg, layers, tok, fo.Q6_K, out_norm, head, fo.Q6_K).forward(prompt)
    dist = float(np.abs(lg - lo).max() / np.std(lo))
    print(f"prefill logits: rel-L2 to the oracle {rel_l2(lg, lo):.2e}, largest difference {dist:.2e} of the logits' spread; "
          f"{planted} of {n_new} steps take the planted successor")
    assert rel_l2(lg, lo) <= 2e-2 and dist <= 5e-2     # measured: 7.5e-3 and 2.9e-2
    dec.reset()
    got = dec.generate(torch.from_numpy(prompt).cuda(), n_new)
    first = next((i for i in range(n_new) if got[i] != want[i]), None)
    print(f"128-token greedy decode: first divergence {first}; smallest top-2 logit margin {min(margins):.3e} (in units of the logits' spread) "
          f"at token {int(np.argmin(margins))}; {len(set(want))} distinct tokens")
    assert first is None, f"first divergence at generated token {first}: {got[first]} vs {want[first]} (margin there {margins[first]:.3e})"
    dec.reset()
    assert dec.generate(torch.from_numpy(prompt).cuda(), n_new, use_graph=True) == want
    from frink_b200 import device
    assert device.device_error() == 0


def test_small_qwen3_moe_decoder_matches_an_independent_oracle():
    """The routed graph (per-head q/k norms, split-half RoPE, router -> top-k -> experts ->
    combine) against `tests/oracle_decoder.py`, which composes the oracle's functions in the
    reference's order and shares no code with `frink_b200.decoder`: logits of a prefill and of
    decode rows, then greedy tokens."""
    from frink_b200.decoder import Decoder
    from tests.test_parallel_cpu import _tiny_model
    cfg, layers, tok, out_norm, head = _tiny_model(True)
    dev = Decoder(cfg, layers, tok, fo.Q8_0, out_norm, output=head, output_kind=fo.Q8_0, max_seq=64)
    ora = od.OracleDecoder(cfg, layers, tok, fo.Q8_0, out_norm, head, fo.Q8_0)
    prompt = np.random.default_rng(3).integers(0, cfg.vocab, 12).astype(np.int32)
    for ids in (prompt, np.array([7], np.int32), np.array([5, 9, 2], np.int32)):
        got = dev.forward(torch.from_numpy(ids).cuda()).cpu().numpy()[0]
        want = ora.forward(ids)
        assert rel_l2(got, want) <= 1e-3, len(ids)
    dev.reset()
    ora = od.OracleDecoder(cfg, layers, tok, fo.Q8_0, out_norm, head, fo.Q8_0)
    want = ora.generate(list(prompt), 24)
    assert dev.generate(torch.from_numpy(prompt).cuda(), 24) == want
    from frink_b200 import device
    assert device.device_error() == 0


def test_small_qwen3_moe_decoder_matches_the_cpu_decoder():
    """A routed model with per-head q/k norms and split-half RoPE: the device decoder (grouped
    GEMM prefill, indexed-expert fused decode) against the same decoder run on the oracle-backed
    CPU ops."""
    from frink_b200.decoder import Decoder
    from tests import cpu_ops
    from tests.test_parallel_cpu import _tiny_model
    cfg, layers, tok, out_norm, head = _tiny_model(True)
    dev = Decoder(cfg, layers, tok, fo.Q8_0, out_norm, output=head, output_kind=fo.Q8_0, max_seq=32)
    cpu = Decoder(cfg, layers, tok, fo.Q8_0, out_norm, output=head, output_kind=fo.Q8_0, max_seq=32, ops=cpu_ops, device="cpu")
    prompt = np.random.default_rng(3).integers(0, cfg.vocab, 12).astype(np.int32)
    for ids in (prompt, np.array([7], np.int32), np.array([5, 9, 2], np.int32)):
        got = dev.forward(torch.from_numpy(ids).cuda()).cpu().numpy()
        want = cpu.forward(torch.from_numpy(ids)).numpy()
        assert rel_l2(got, want) <= 1e-3, len(ids)
    from frink_b200 import device
    assert device.device_error() == 0


@pytest.mark.parametrize("neox,norms", [(False, False), (True, True)])
def test_one_row_attention_with_rope_and_cache_append_folded_in(neox, norms):
    """`fk_attention_rope_kv` against `fk_rope_kv` followed by `fk_attention`: same caches,
    same output (the key split over blocks is the same, so is the arithmetic per key)."""
    from frink_b200 import device
    rng = np.random.default_rng(21)
    nh, nkv, hd, p0 = 8, 2, 128, 150
    hq, kvw = nh * hd, nkv * hd
    qkv = torch.from_numpy(rng.standard_normal((1, hq + 2 * kvw)).astype(np.float32)).cuda()
    kc = torch.from_numpy(rng.standard_normal((256, kvw)).astype(np.float32)).cuda()
    vc = torch.from_numpy(rng.standard_normal((256, kvw)).astype(np.float32)).cuda()
    qn = torch.from_numpy((1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)).cuda() if norms else None
    kn = torch.from_numpy((1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)).cuda() if norms else None
    for pos_v in (p0, 0, 63, 64):
        pos = torch.tensor([pos_v], dtype=torch.int32).cuda()
        b0, k0, v0 = qkv.clone(), kc.clone(), vc.clone()
        device.rope_kv(b0[:, :hq], b0[:, hq:hq + kvw], b0[:, hq + kvw:], nh, nkv, hd, pos, 1e4, neox, k0, v0, q_norm=qn, k_norm=kn, eps=1e-6)
        want = device.attention(b0[:, :hq], k0, v0, nh, nkv, hd, pos)
        b1, k1, v1 = qkv.clone(), kc.clone(), vc.clone()
        got = device.attention_rope_kv(b1[:, :hq], b1[:, hq:hq + kvw], b1[:, hq + kvw:], k1, v1, nh, nkv, hd, pos, 1e4, neox, q_norm=qn, k_norm=kn, eps=1e-6)
        assert torch.equal(b1, qkv)                                  # the projection's output is left as it was
        assert torch.allclose(k1, k0, rtol=1e-6, atol=1e-7) and torch.equal(v1, v0)
        assert torch.allclose(got, want, rtol=1e-5, atol=1e-6), pos_v
    assert device.device_error() == 0


def test_rows_past_the_kv_caches_are_refused_on_the_host_and_on_the_device():
    """The decoder counts positions on the host and raises before launching; the kernels themselves, whose
    position word lives on the device, do nothing and raise error word 95 when *pos + rows passes the caches."""
    from frink_b200 import device
    from frink_b200.decoder import Decoder
    cfg, layers, tok, out_norm, head = small_llama(uniform=True)
    dec = Decoder(cfg, layers, tok, fo.Q6_K, out_norm, output=head, output_kind=fo.Q6_K, max_seq=24)
    prompt = torch.from_numpy(np.random.default_rng(1).integers(0, cfg.vocab, 20).astype(np.int32)).cuda()
    t = dec.prefill(prompt)
    for _ in range(4):
        t = dec.decode_step(t)
    with pytest.raises(ValueError):
        dec.decode_step(t)                      # position 24 of 24
    dec.reset()
    dec.prefill(prompt)
    for _ in range(3):
        dec.decode_step(t)
    with pytest.raises(ValueError):
        dec.capture_decode(t)                   # the two warm-up steps would need rows 23 and 24
    with pytest.raises(ValueError):
        dec.forward(prompt)                     # 20 more rows at 23
    assert device.device_error() == 0
    # the device-side guard: a cache of 8 rows, position 7, two rows
    kc, vc = torch.zeros((8, 256), device="cuda"), torch.zeros((8, 256), device="cuda")
    pos = torch.tensor([7], dtype=torch.int32, device="cuda")
    q, k, v = torch.randn(2, 512, device="cuda"), torch.randn(2, 256, device="cuda"), torch.randn(2, 256, device="cuda")
    device.rope_kv(q, k, v, 4, 2, 128, pos, 10000.0, False, kc, vc)
    torch.cuda.synchronize()
    assert device.device_error() == 95 and not kc.any() and not vc.any()
    device.kv_append(kc, k, pos)
    torch.cuda.synchronize()
    assert device.device_error() == 95 and not kc.any()
    out = torch.full((2, 512), 3.0, device="cuda")
    device.attention(q, kc, vc, 4, 2, 128, pos, out=out)
    torch.cuda.synchronize()
    assert device.device_error() == 95 and bool((out == 3.0).all())
    pos.fill_(8)
    out1 = torch.full((1, 512), 3.0, device="cuda")
    device.attention_rope_kv(q[:1], k[:1], v[:1], kc, vc, 4, 2, 128, pos, 10000.0, out=out1)
    torch.cuda.synchronize()
    assert device.device_error() == 95 and bool((out1 == 3.0).all()) and not kc.any()
    pos.fill_(6)                                # rows 6 and 7 fit
    device.rope_kv(q, k, v, 4, 2, 128, pos, 10000.0, False, kc, vc)
    torch.cuda.synchronize()
    assert device.device_error() == 0 and kc[6:].any() and not kc[:6].any()


def test_the_workspace_never_moves_under_a_captured_graph(monkeypatch):
    """A call that needs more workspace than is reserved fails inside a stream capture instead of allocating there;
    outside a capture the workspace grows, and the block a graph captured earlier points at stays alive and untouched
    by the move."""
    import ctypes as C
    from frink_b200 import _lib, device
    from frink_b200._lib import check, lib
    idx = torch.cuda.current_device()
    device.context()
    fresh = C.c_void_p()
    check(lib().fk_init(idx, C.byref(fresh)))
    monkeypatch.setitem(device._contexts, idx, fresh)          # a context whose workspace is still empty
    try:
        raw = fo.encode(fo.Q8_0, synth_weights(256, 1024, 1))
        w = device.Weights(raw, fo.Q8_0, 256, 1024)
        small = torch.randn(64, 1024, device="cuda")
        big = torch.randn(70000, 1024, device="cuda")          # ~80 MB of q8_1 image: more than the 64 MiB taken on first use
        y, ybig = torch.empty(64, 256, device="cuda"), torch.empty(70000, 256, device="cuda")
        device.gemm(w, small, out=y)                           # first use reserves the minimum
        torch.cuda.synchronize()
        want = y.clone()
        g = torch.cuda.CUDAGraph()
        with pytest.raises(_lib.Invalid):
            with torch.cuda.graph(g):
                device.gemm(w, big, out=ybig)
        torch.cuda.synchronize()
        g2 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g2):
            device.gemm(w, small, out=y)
        device.gemm(w, big, out=ybig)                          # grows the workspace: the old block stays
        torch.cuda.synchronize()
        assert torch.isfinite(ybig).all()
        y.zero_()
        g2.replay()
        torch.cuda.synchronize()
        assert torch.equal(y, want) and device.device_error() == 0
        w.release()
    finally:
        lib().fk_destroy(fresh)


@pytest.mark.parametrize("moe", [False, True, "oai"])
def test_a_decode_batch_of_independent_sequences_matches_each_sequence_alone(moe):
    """Eight sequences with prompts of different lengths, decoded together (one token each per step, their own KV
    caches and positions, one launch per op for the whole batch), against each sequence decoded alone."""
    from frink_b200 import device
    from frink_b200.decoder import Decoder
    if moe == "oai":
        # gpt-oss's layer form: biased BF16 projections (one launch each), sinks, a windowed layer, biased MXFP4 experts
        cfg, layers, tok, out_norm, head = tiny_gpt_oss()
        mk = lambda: Decoder(cfg, layers, tok, fo.BF16, out_norm, output=head, output_kind=fo.BF16, max_seq=64)
    elif moe:
        from tests.test_parallel_cpu import _tiny_model
        cfg, layers, tok, out_norm, head = _tiny_model(True)
        mk = lambda: Decoder(cfg, layers, tok, fo.Q8_0, out_norm, output=head, output_kind=fo.Q8_0, max_seq=64)
    else:
        cfg, layers, tok, out_norm, head = small_llama(uniform=True)
        mk = lambda: Decoder(cfg, layers, tok, fo.Q6_K, out_norm, output=head, output_kind=fo.Q6_K, max_seq=64)
    n_seqs, steps = 8, 6
    rng = np.random.default_rng(17)
    prompts = [torch.from_numpy(rng.integers(0, cfg.vocab, 5 + 3 * s).astype(np.int32)).cuda() for s in range(n_seqs)]
    solo = mk()
    want_tok, want_logits = [], []
    for p in prompts:
        solo.reset()
        t = solo.prefill(p)
        toks, lgs = [int(t.item())], []
        for _ in range(steps):
            lg = solo.forward(t)
            lgs.append(lg.cpu().numpy()[0])
            t = device.argmax(lg)
            toks.append(int(t.item()))
        want_tok.append(toks)
        want_logits.append(lgs)
    dec = mk()
    dec.alloc_seqs(n_seqs)
    cur = torch.cat([dec.prefill_seq(s, prompts[s]) for s in range(n_seqs)])
    got_tok = [[int(c)] for c in cur.tolist()]
    worst = 0.0
    for i in range(steps):
        lg = dec.forward_seqs(cur)
        for s in range(n_seqs):
            worst = max(worst, rel_l2(lg[s].cpu().numpy(), want_logits[s][i]))
        cur = device.argmax(lg)
        for s, c in enumerate(cur.tolist()):
            got_tok[s].append(int(c))
    assert device.device_error() == 0
    # the batched step takes the tensor-core matvec (8 rows) where the single row takes the dp4a one: same integers,
    # another f32 summation order, and q8_1 re-rounding of the activations downstream of it
    assert worst <= 5e-3, worst
    assert got_tok == want_tok
    # the captured step continues where the eager ones stopped
    g, out = dec.capture_decode_seqs(cur)
    dec.replay_seqs()
    torch.cuda.synchronize()
    lg = None
    assert out.shape[0] == n_seqs and device.device_error() == 0
    assert dec._seq_pos_host == [int(p) for p in dec.seq_pos.tolist()]


def test_prefill_on_q8k_activations_stays_close_to_the_q8_1_pipeline():
    """`Decoder(prefill_acts="q8_k")`: a prompt's Q4_K projections take the GEMM on Q8_K activations (its integers are
    frink's CPU vec_dot's, tests/test_gemm_q8k_gpu.py); the logits after a 64-token prompt stay within the distance two
    8-bit activation quantizers put between two pipelines, and where the oracle's margin is decisive the greedy
    continuation is the same."""
    from frink_b200.decoder import Decoder
    cfg, layers, tok, out_norm, _ = recipe_llama()
    head, _ = decisive_head(cfg, tok)
    prompt = torch.from_numpy(np.random.default_rng(0x70C).integers(0, cfg.vocab, 64).astype(np.int32)).cuda()
    a = Decoder(cfg, layers, tok, fo.Q6_K, out_norm, output=head, output_kind=fo.Q6_K, max_seq=128)
    b = Decoder(cfg, layers, tok, fo.Q6_K, out_norm, output=head, output_kind=fo.Q6_K, max_seq=128, prefill_acts="q8_k")
    la, lb = a.forward(prompt).cpu().numpy()[0], b.forward(prompt).cpu().numpy()[0]
    r = rel_l2(lb, la)
    print(f"q8_k prefill against q8_1 prefill: rel-L2 {r:.2e}")
    assert r <= 5e-2
    top2 = np.sort(la)[-2:]
    if (top2[1] - top2[0]) / np.std(la) > 0.2:
        assert int(np.argmax(la)) == int(np.argmax(lb))
    a.reset()
    b.reset()
    ga, gb = a.generate(prompt, 16), b.generate(prompt, 16)
    same = sum(x == y for x, y in zip(ga, gb))
    print(f"greedy continuation: {same} of 16 tokens equal")
    from frink_b200 import device
    assert device.device_error() == 0


@pytest.mark.parametrize("n_q", [1, 5, 40])
@pytest.mark.parametrize("window,with_sinks", [(0, True), (48, False), (48, True), (7, True)])
def test_sliding_window_and_sinks(n_q, window, with_sinks):
    """gpt-oss attention (crates/frink-core/src/attention.rs:312-322, 960-1000): only the `window` most recent keys
    are seen, and a per-head sink logit joins the softmax's denominator -- the split-key decode kernel (1 and 5 rows)
    and the prefill kernel (40 rows) against a float64 restatement."""
    from frink_b200 import device
    from tests import cpu_ops
    n_heads, n_kv, hd, p0 = 8, 2, 64, 100
    rng = np.random.default_rng(31 + n_q + window)
    kc = torch.from_numpy(rng.standard_normal((256, n_kv * hd)).astype(np.float32))
    vc = torch.from_numpy(rng.standard_normal((256, n_kv * hd)).astype(np.float32))
    q = torch.from_numpy(rng.standard_normal((n_q, n_heads * hd)).astype(np.float32))
    sinks = torch.from_numpy((rng.standard_normal(n_heads) * 2).astype(np.float32)) if with_sinks else None
    pos = torch.tensor([p0], dtype=torch.int32)
    want = cpu_ops.attention(q, kc, vc, n_heads, n_kv, hd, pos, window=window, sinks=sinks).numpy()
    got = device.attention(q.cuda(), kc.cuda(), vc.cuda(), n_heads, n_kv, hd, pos.cuda(), window=window,
                           sinks=None if sinks is None else sinks.cuda()).cpu().numpy()
    assert rel_l2(got, want) <= 2e-6
    if with_sinks and window == 0:
        plain = device.attention(q.cuda(), kc.cuda(), vc.cuda(), n_heads, n_kv, hd, pos.cuda()).cpu().numpy()
        assert rel_l2(got, plain) > 1e-3           # the sink takes weight away from the real keys
    assert device.device_error() == 0


def test_fused_decode_attention_with_window_and_sinks_for_one_and_many_sequences():
    from frink_b200 import device
    n_heads, n_kv, hd, window = 8, 2, 64, 20
    rng = np.random.default_rng(77)
    sinks = torch.from_numpy(rng.standard_normal(n_heads).astype(np.float32)).cuda()
    kcs = torch.from_numpy(rng.standard_normal((3, 128, n_kv * hd)).astype(np.float32)).cuda()
    vcs = torch.from_numpy(rng.standard_normal((3, 128, n_kv * hd)).astype(np.float32)).cuda()
    pos = torch.tensor([90, 5, 33], dtype=torch.int32, device="cuda")
    q = torch.from_numpy(rng.standard_normal((3, n_heads * hd)).astype(np.float32)).cuda()
    k = torch.from_numpy(rng.standard_normal((3, n_kv * hd)).astype(np.float32)).cuda()
    v = torch.from_numpy(rng.standard_normal((3, n_kv * hd)).astype(np.float32)).cuda()
    # reference: per sequence, the separate kernels (rotation + append, then attention with the same window and sinks)
    want = []
    for s_ in range(3):
        kc, vc = kcs[s_].clone(), vcs[s_].clone()
        q1, k1 = q[s_:s_ + 1].clone(), k[s_:s_ + 1].clone()
        device.rope_kv(q1, k1, v[s_:s_ + 1], n_heads, n_kv, hd, pos[s_:s_ + 1], 10000.0, False, kc, vc)
        want.append(device.attention(q1, kc, vc, n_heads, n_kv, hd, pos[s_:s_ + 1], window=window, sinks=sinks))
    want = torch.cat(want)
    one = device.attention_rope_kv(q[:1].clone(), k[:1].clone(), v[:1], kcs[0].clone(), vcs[0].clone(), n_heads, n_kv, hd, pos[:1], 10000.0,
                                   window=window, sinks=sinks)
    assert rel_l2(one.cpu().numpy(), want[:1].cpu().numpy()) <= 2e-6
    many = device.attention_rope_kv_seqs(q.clone(), k.clone(), v, kcs.clone(), vcs.clone(), n_heads, n_kv, hd, pos, 10000.0, window=window, sinks=sinks)
    assert rel_l2(many.cpu().numpy(), want.cpu().numpy()) <= 2e-6
    assert device.device_error() == 0


def test_decoder_with_alternating_windowed_layers_and_sinks_matches_the_cpu_decoder():
    """gpt-oss's attention pattern on a small dense model: layer 0 windowed (8 keys), layer 1 full, a sink logit per
    head in both -- prompt through the prefill kernel, then single rows and a few rows through the split-key kernel
    (fused with rotation and cache append for one row), against the same decoder on the oracle-backed CPU ops."""
    import dataclasses
    from frink_b200.decoder import Decoder
    from tests import cpu_ops
    cfg, layers, tok, out_norm, head = small_llama(uniform=True)
    cfg = dataclasses.replace(cfg, sliding_window=8, swa_period=2)
    rng = np.random.default_rng(41)
    layers = [dataclasses.replace(L, sinks=rng.standard_normal(cfg.n_heads).astype(np.float32)) for L in layers]
    assert [cfg.window_of(i) for i in range(2)] == [8, 0]
    dev = Decoder(cfg, layers, tok, fo.Q6_K, out_norm, output=head, output_kind=fo.Q6_K, max_seq=64)
    cpu = Decoder(cfg, layers, tok, fo.Q6_K, out_norm, output=head, output_kind=fo.Q6_K, max_seq=64, ops=cpu_ops, device="cpu")
    prompt = rng.integers(0, cfg.vocab, 20).astype(np.int32)
    for ids in (prompt, np.array([7], np.int32), np.array([11], np.int32), np.array([5, 9, 2], np.int32), np.array([3], np.int32)):
        got = dev.forward(torch.from_numpy(ids).cuda()).cpu().numpy()
        want = cpu.forward(torch.from_numpy(ids)).numpy()
        # two f32 pipelines: mostly equal to 1e-5, but one activation on the other side of a q8_1 rounding boundary moves
        # the logits by up to 1e-2 (with or without window and sinks); the kernels themselves are held to 2e-6 above
        assert rel_l2(got, want) <= 2e-2, len(ids)
    # and the window matters: the same model without it answers differently
    plain = Decoder(dataclasses.replace(cfg, sliding_window=0), layers, tok, fo.Q6_K, out_norm, output=head, output_kind=fo.Q6_K, max_seq=64)
    a = plain.forward(torch.from_numpy(prompt).cuda()).cpu().numpy()
    dev.reset()
    b = dev.forward(torch.from_numpy(prompt).cuda()).cpu().numpy()
    assert rel_l2(b, a) > 5e-2
    from frink_b200 import device
    assert device.device_error() == 0


def test_gpt_oss_layer_form_matches_the_cpu_decoder():
    """The gpt-oss pieces assembled: prompt (grouped MXFP4 GEMMs with expert biases, prefill attention with window and
    sinks, BF16 projections in batches of 8), single rows and a few rows (indexed matvecs), eager and from a captured
    graph, against the same decoder on the oracle-backed CPU ops."""
    from frink_b200.decoder import Decoder
    from tests import cpu_ops
    cfg, layers, tok, out_norm, head = tiny_gpt_oss()
    dev = Decoder(cfg, layers, tok, fo.BF16, out_norm, output=head, output_kind=fo.BF16, max_seq=64)
    cpu = Decoder(cfg, layers, tok, fo.BF16, out_norm, output=head, output_kind=fo.BF16, max_seq=64, ops=cpu_ops, device="cpu")
    prompt = np.random.default_rng(3).integers(0, cfg.vocab, 12).astype(np.int32)
    worst = 0.0
    for ids in (prompt, np.array([7], np.int32), np.array([5, 9, 2], np.int32), np.array([100], np.int32)):
        got = dev.forward(torch.from_numpy(ids).cuda()).cpu().numpy()
        want = cpu.forward(torch.from_numpy(ids)).numpy()
        worst = max(worst, rel_l2(got, want))
    print(f"gpt-oss layer form, device against CPU ops: worst rel-L2 {worst:.2e}")
    assert worst <= 2e-2
    dev.reset()
    eager = dev.generate(torch.from_numpy(prompt).cuda(), 6)
    dev.reset()
    assert dev.generate(torch.from_numpy(prompt).cuda(), 6, use_graph=True) == eager
    from frink_b200 import device
    assert device.device_error() == 0
