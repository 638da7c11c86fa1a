"""Pins the CPU oracle against the reference's own golden vectors and
known-answer tests (extracted by tests/golden/make_goldens.py)."""
import numpy as np
import pytest

from oracle import frink_oracle as fo
from tests.helpers import goldens, k_quant_fixture, xorshift_unit

G = goldens()


def u8(name):
    return np.array(G[name], np.uint8)


def test_f16_conversions_match_ieee():
    bits = np.arange(0, 65536, dtype=np.uint16)
    want = bits.view(np.float16).astype(np.float32)
    got = np.array([fo.lib().fko_f16_to_f32(int(b)) for b in bits[::7]], np.float32)
    w = want[::7]
    ok = (got == w) | (np.isnan(got) & np.isnan(w))
    assert ok.all()
    rng = np.random.default_rng(1)
    xs = np.concatenate([
        rng.standard_normal(4000).astype(np.float32) * np.float32(10) ** rng.integers(-8, 6, 4000).astype(np.float32),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e-8, 5.96e-8, 2.98e-8, 6.1e-5, 0.5 + 2 ** -12], np.float32),
    ])
    for x in xs:
        h = np.float32(x).astype(np.float16).view(np.uint16)
        assert fo.lib().fko_f32_to_f16(float(x)) == int(h), x


# crates/frink-quant/src/lib.rs:6532, :6556, :7056, :7124 (dequant goldens, 1e-3)
@pytest.mark.parametrize("kind,block,gold", [
    (fo.Q4_K, "Q4_K_TEST_BLOCK", "Q4_K_GOLDEN"),
    (fo.Q5_K, "Q5_K_TEST_BLOCK", "Q5_K_GOLDEN"),
    (fo.Q6_K, "Q6_K_TEST_BLOCK", "Q6_K_GOLDEN"),
    (fo.Q6_K, "Q6_K_SIGNED_SCALES_TEST_BLOCK", "Q6_K_SIGNED_SCALES_GOLDEN"),
    (fo.Q6_K, "Q6_K_SIGNED_TEST_BLOCK", "Q6_K_SIGNED_GOLDEN"),
    (fo.MXFP4, "MXFP4_GGUF_TEST_BLOCKS", "MXFP4_GGUF_GOLDEN"),
])
def test_dequant_matches_reference_golden(kind, block, gold):
    got = fo.dequant(kind, u8(block))
    want = np.array(G[gold], np.float32)
    assert got.shape == want.shape
    assert np.max(np.abs(got - want)) < 1e-3
    # the goldens are printed to six digits; hold the oracle to that too
    assert np.allclose(got, want, rtol=2e-5, atol=1e-6)


def test_dequant_agrees_with_gguf_py():
    quants = pytest.importorskip("gguf.quants")
    import gguf
    rng = np.random.default_rng(7)
    for kind, qt in [(fo.Q4_K, gguf.GGMLQuantizationType.Q4_K), (fo.Q5_K, gguf.GGMLQuantizationType.Q5_K),
                     (fo.Q6_K, gguf.GGMLQuantizationType.Q6_K),
                     (fo.Q8_0, gguf.GGMLQuantizationType.Q8_0), (fo.MXFP4, gguf.GGMLQuantizationType.MXFP4)]:
        w = (rng.standard_normal(8 * 256) * 0.02).astype(np.float32)
        raw = fo.encode(kind, w, threads=1)
        want = quants.dequantize(raw.reshape(1, -1), qt).ravel()
        got = fo.dequant(kind, raw)
        assert np.allclose(got, want, rtol=1e-6, atol=1e-9), kind


# crates/frink-quant/src/encode.rs:165-216 (byte-identical to llama.cpp's encoder)
def test_q8_0_encoder_matches_llama_cpp_bytes():
    x = xorshift_unit(64, 0x12345678)
    assert np.array_equal(fo.encode(fo.Q8_0, x, threads=1), u8("LLAMA_CPP_Q8_0_GOLDEN"))
    tie = np.array(G["TIE_BLOCK_F16_BITS"], np.uint16).view(np.float16).astype(np.float32)
    assert np.array_equal(fo.encode(fo.Q8_0, tie, threads=1), u8("LLAMA_CPP_TIE_BLOCK_GOLDEN"))


# crates/frink-quant/src/encode/q4_k.rs:279, encode/q6_k.rs (goldens over k_quant_fixture)
@pytest.mark.parametrize("kind,gold", [(fo.Q4_K, "LLAMA_CPP_Q4_K_GOLDEN"), (fo.Q5_K, "LLAMA_CPP_Q5_K_GOLDEN"), (fo.Q6_K, "LLAMA_CPP_Q6_K_GOLDEN")])
def test_k_quant_encoders_match_llama_cpp_bytes(kind, gold):
    x = k_quant_fixture(G["REAL_WEIGHT_BLOCKS"])
    assert x.size == 12 * 256
    got = fo.encode(kind, x, threads=1)
    want = u8(gold)
    bb = fo.block_bytes(kind)
    bad = [b for b in range(12) if not np.array_equal(got[b * bb:(b + 1) * bb], want[b * bb:(b + 1) * bb])]
    assert not bad, f"super-blocks {bad} differ from llama.cpp's bytes"
    assert np.array_equal(fo.encode(kind, x, threads=4), want)


# crates/frink-quant/src/encode/fit.rs:601-612
def test_nearest_int_rounds_ties_to_even():
    n = fo.lib().fko_nearest_int
    assert [n(0.5), n(1.5), n(2.5), n(-0.5), n(-1.5), n(3.7), n(-3.7), n(3.2)] == [0, 2, 2, 0, -2, 4, -4, 3]


# crates/frink-quant/src/act_quant.rs:215-300 (libggml-produced known answers)
def _blk(head, n):
    x = np.zeros(n, np.float32)
    x[:len(head)] = head
    return x


def test_q8_k_known_answers():
    q, d, bs = fo.quantize_q8_k(_blk([127.0, 2.5, -3.5, 0.5, -0.5, 126.5], 256))
    assert d[0] == 1.0 and list(q[:6]) == [127, 2, -4, 0, 0, 126] and bs[0] == 127 + 2 - 4 + 126
    amax = np.array([0x3FE46A64], np.uint32).view(np.float32)[0]
    x = np.array([0x3DD7D365], np.uint32).view(np.float32)[0]
    q, d, _ = fo.quantize_q8_k(_blk([-amax, x], 256))
    assert d.view(np.uint32)[0] == 0x3C6636D1 and list(q[:2]) == [-127, 8]
    qn, dn, _ = fo.quantize_q8_k(_blk([-127.0, 2.5], 256))
    qp, dp, _ = fo.quantize_q8_k(_blk([127.0, -2.5], 256))
    assert (dn[0], dp[0]) == (1.0, 1.0) and (qn[1], qp[1]) == (2, -2) and np.array_equal(qn, -qp)
    q, d, bs = fo.quantize_q8_k(np.zeros(256, np.float32))
    assert d[0] == 0.0 and not q.any() and not bs.any()


def test_q8_0_activation_known_answers():
    x = _blk([127.0, 2.5, -3.5, 0.5, 1.5], 32)
    for form, want in [(0, [127, 2, -4, 0, 2]), (1, [127, 2, -4, 0, 2]), (2, [127, 3, -4, 1, 2])]:
        q, d = fo.quantize_q8_0_act(x, form)
        assert d[0] == 1.0 and list(q[:5]) == want
    q, d = fo.quantize_q8_0_act(_blk([1.0, 0.5], 32), 0)
    assert d[0] == np.array([0x2008], np.uint16).view(np.float16).astype(np.float32)[0]
    assert d[0] != np.float32(1.0) / np.float32(127.0) and list(q[:2]) == [127, 64]
    x = _blk(np.array([0x4013E709, 0x3CDF99C0], np.uint32).view(np.float32), 32)
    q, d = fo.quantize_q8_0_act(x, 0)
    assert d[0] == np.array([0x24A9], np.uint16).view(np.float16).astype(np.float32)[0] and list(q[:2]) == [127, 2]
    assert fo.quantize_q8_0_act(x, 1)[0][1] == 1
    for form in (0, 1, 2):
        q, d = fo.quantize_q8_0_act(np.zeros(32, np.float32), form)
        assert d[0] == 0.0 and not q.any()


def _weights(kind, n_blocks, seed):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal(n_blocks * fo.block_elems(kind)) * 0.02).astype(np.float32)
    return fo.encode(kind, w, threads=1)


ALL = [fo.Q4_K, fo.Q6_K, fo.Q8_0, fo.MXFP4]
WITH_Q5 = ALL + [fo.Q5_K]      # Q5_K has no dp4a twin in the reference (its GPU matvec is generated from the dequant)


# crates/frink-quant/src/lib.rs:6544, :6568, :7068 (fused dot == dequantize-then-dot)
@pytest.mark.parametrize("kind", WITH_Q5)
def test_fused_f32_dot_matches_dequant_then_dot(kind):
    nb = 3 * (256 // fo.block_elems(kind))
    row = _weights(kind, nb, 11)
    x = np.sin(np.arange(nb * fo.block_elems(kind), dtype=np.float32) * np.float32(0.017))
    want = float(np.dot(fo.dequant(kind, row).astype(np.float64), x.astype(np.float64)))
    got = fo.dot_f32_scalar(kind, row, x)
    assert abs(got - want) < 1e-4 * max(1.0, abs(want))
    assert abs(fo.dot_dequant_f64(kind, row, x) - want) < 1e-12 * max(1.0, abs(want))
    if kind == fo.Q4_K and fo.lib().fko_has_avx2():
        y = fo.matvec_f32(kind, row, 1, x.size, x, threads=1, simd=True)
        assert abs(float(y[0, 0]) - want) < 1e-4 * max(1.0, abs(want))


# crates/frink-quant/src/lib.rs:5624-5810, legacy_q8.rs:453-524 (the integer dot
# tracks the float dot within the activation quantization error)
@pytest.mark.parametrize("kind", WITH_Q5)
def test_cpu_integer_dot_tracks_float_dot(kind):
    nb = 4 * (256 // fo.block_elems(kind))
    row = _weights(kind, nb, 5)
    rng = np.random.default_rng(6)
    x = rng.standard_normal(nb * fo.block_elems(kind)).astype(np.float32)
    w = fo.dequant(kind, row)
    scale = float(np.sum(np.abs(w.astype(np.float64) * x)))
    assert abs(fo.dot_q8(kind, row, x) - fo.dot_dequant_f64(kind, row, x)) < 2e-2 * scale


# crates/frink-cuda/src/dp4a_twin.rs:402-440: each dp4a twin equals the f64
# dequantize-then-dot of ITS q8_1 input to 1e-5 of the term scale
@pytest.mark.parametrize("kind", ALL)
@pytest.mark.parametrize("nwarps", [1, 2, 4])
def test_dp4a_twin_matches_dequant_dot_of_its_q8_1_input(kind, nwarps):
    for n_blocks, seed in [(1, 3), (3, 7), (6, 11), (16, 13), (37, 17)]:
        row = _weights(kind, n_blocks, seed)
        rng = np.random.default_rng(seed)
        x = rng.standard_normal(n_blocks * fo.block_elems(kind)).astype(np.float32)
        y = fo.quantize_q8_1(x)
        got = fo.dp4a_row(kind, row, y, nwarps)
        w = fo.dequant(kind, row).astype(np.float64)
        xq = fo.q8_1_dequant(y).astype(np.float64)
        want = float(np.dot(w, xq))
        scale = max(float(np.sum(np.abs(w * xq))), 1e-6)
        assert abs(got - want) / scale < 1e-5, (kind, nwarps, n_blocks)


# crates/frink-cuda/src/dp4a_twin.rs:520-560 (quantizer known answers)
def test_q8_1_quantizer_layout_and_values():
    rng = np.random.default_rng(3)
    x = rng.standard_normal(96).astype(np.float32)
    x[:32] = 0.0
    y = fo.quantize_q8_1(x)
    assert y.size == 3 * 36 and not y[:36].any()
    b1 = y[36:72]
    s = np.frombuffer(b1[2:4].tobytes(), np.float16)[0]
    assert abs(float(s) - float(x[32:64].sum())) <= abs(float(x[32:64].sum())) * 1e-3 + 1e-3
    b2 = y[72:108]
    amax = np.abs(x[64:96]).max()
    d = np.frombuffer(b2[0:2].tobytes(), np.float16)[0]
    assert d == np.float16(np.float32(amax) / np.float32(127.0))
    assert (np.abs(b2[4:].view(np.int8).astype(np.int32)) == 127).any()
    # the integers are what the dp4a word dots add up
    assert np.array_equal(fo.q8_1_dequant(y)[64:96], b2[4:].view(np.int8).astype(np.float32) * np.float32(d))


@pytest.mark.parametrize("kind", WITH_Q5)
def test_per_run_isums_reassemble_the_dp4a_twin(kind):
    """The exact per-run integers, scaled the way the block format says, give the
    dequantize-then-dot of the q8_1 input: ties the integer oracle to the formats."""
    n_blocks = 2 * (256 // fo.block_elems(kind))
    cols = n_blocks * fo.block_elems(kind)
    row = _weights(kind, n_blocks, 23)
    rng = np.random.default_rng(24)
    x = rng.standard_normal(cols).astype(np.float32)
    y = fo.quantize_q8_1(x)
    isums = fo.matrix_isums(kind, row, 1, cols, y)[0]
    w = fo.dequant(kind, row).astype(np.float64)
    yq = y.reshape(-1, 36)
    d8 = yq[:, :2].copy().view(np.float16).astype(np.float64).ravel()
    q8 = yq[:, 4:].view(np.int8).astype(np.int64)
    if kind == fo.Q8_0:
        dw = row.reshape(-1, 34)[:, :2].copy().view(np.float16).astype(np.float64).ravel()
        got = float(np.sum(dw * d8 * isums))
    elif kind == fo.MXFP4:
        e = row.reshape(-1, 17)[:, 0].astype(np.int64)
        got = float(np.sum(np.ldexp(1.0, e - 127) * 0.5 * d8 * isums))
    else:
        # per-run weight scale read back from the dequantized row: w = a*code - b
        got = None
    want = float(np.dot(w, fo.q8_1_dequant(y).astype(np.float64)))
    if got is not None:
        assert abs(got - want) < 1e-9 * max(1.0, float(np.sum(np.abs(w))))
    assert isums.dtype == np.int32 and isums.size == n_blocks * fo.runs_per_block(kind)
    assert np.all(np.abs(isums) <= 127 * 127 * 32)
    assert q8.shape == (cols // 32, 32)


# crates/frink-moe/src/lib.rs:1345-1400 (routing), :2219 (ties take the lower id)
def test_routing_known_answers():
    ids, w = fo.route_top_k(np.array([[0.1, 5.0, 0.2, 3.0, -1.0]], np.float32), 2, 1)
    assert list(ids[0]) == [1, 3] and abs(w.sum() - 1) < 1e-5 and w[0, 0] > w[0, 1]
    logits = np.arange(1, 9, dtype=np.float32)[None]
    for k in range(1, 9):
        assert abs(fo.route_top_k(logits, k, 1)[1].sum() - 1) < 1e-5
    ids, w = fo.route_top_k(logits, 3, 0)
    assert list(ids[0]) == [7, 6, 5]
    assert np.allclose(w[0], [0.6323223, 0.2326232, 0.0855683], atol=1e-4) and abs(w.sum() - 0.9505138) < 1e-4
    ids1, w1 = fo.route_top_k(logits, 3, 1)
    assert np.array_equal(ids1, ids) and np.allclose(w[0] / w.sum(), w1[0], atol=1e-4)
    ids, w = fo.route_top_k(np.array([[1.0, 3.0, 3.0, 0.0]], np.float32), 2, 1)
    assert list(ids[0]) == [1, 2]
    # gpt-oss: top-k by biased logit, softmax over the chosen
    lg = np.array([[0.5, 2.0, 1.0, -1.0]], np.float32)
    ids, w = fo.route_top_k(lg, 2, 2, bias=np.array([0, 0, 2.0, 0], np.float32))
    assert list(ids[0]) == [2, 1]
    e = np.exp(np.array([3.0, 2.0]) - 3.0)
    assert np.allclose(w[0], e / e.sum(), atol=1e-6)


# crates/frink-moe/src/lib.rs:988-999, :1246-1263
def test_glu_and_combine():
    g = np.array([-8.0, -1.0, 0.0, 1.0, 9.0], np.float32)
    u = np.array([0.5, -9.0, 2.0, 0.0, 8.0], np.float32)
    x = np.minimum(g, 7.0)
    y = np.clip(u, -7.0, 7.0)
    want = x / (1 + np.exp(1.702 * -x)) * (y + 1)
    assert np.allclose(fo.swiglu_oai(g, u), want, rtol=1e-6)
    assert np.allclose(fo.silu_mul(g, u), g / (1 + np.exp(-g)) * u, rtol=1e-6)
    ys = np.array([[1.0, 2.0], [10.0, 20.0]], np.float32)
    assert np.array_equal(fo.combine(ys, np.array([0.25, 0.5], np.float32)), np.array([5.25, 10.5], np.float32))
