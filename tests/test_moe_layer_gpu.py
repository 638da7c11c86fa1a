"""The routed MoE layer (decode and prefill forms) against the oracle's
composition of the reference's host functions: route_top_k -> per expert
gate/up -> SwiGLU -> down -> combine in routing order."""
import numpy as np
import pytest
import torch

from oracle import frink_oracle as fo
from tests.helpers import max_abs_over_inf, rel_l2, synth_weights

pytestmark = pytest.mark.gpu


def oracle_layer(raws, kind, router, x, k, mode, hidden, ffn, act):
    """crates/frink-moe/src/lib.rs:567 (route), :1068 (run_expert), :1246 (combine), with
    every matvec taken on the q8_1-rounded activation the device reads."""
    logits = (x.astype(np.float32) @ router.T.astype(np.float32)).astype(np.float32)
    ids, w = fo.route_top_k(logits, k, mode)
    out = np.zeros((x.shape[0], hidden), np.float32)
    for t in range(x.shape[0]):
        ys = []
        for e in ids[t]:
            g = fo.matmul_f64(kind, raws["gate"][e], ffn, hidden, fo.q8_1_round(x[t]))[0].astype(np.float32)
            u = fo.matmul_f64(kind, raws["up"][e], ffn, hidden, fo.q8_1_round(x[t]))[0].astype(np.float32)
            a = fo.silu_mul(g, u) if act == 0 else fo.swiglu_oai(g, u)
            ys.append(fo.matmul_f64(kind, raws["down"][e], hidden, ffn, fo.q8_1_round(a))[0].astype(np.float32))
        out[t] = fo.combine(np.stack(ys), w[t])
    return ids, out


def build_layer(kind, n_exp, hidden, ffn, k, mode, act, seed):
    from frink_b200 import device, prefill
    rng = np.random.default_rng(seed)
    raws = {n: [fo.encode(kind, synth_weights(r, c, seed + 10 * i + j)) for j in range(n_exp)]
            for i, (n, r, c) in enumerate((("gate", ffn, hidden), ("up", ffn, hidden), ("down", hidden, ffn)))}
    router = (rng.standard_normal((n_exp, hidden)) * 0.5).astype(np.float32)
    mk = lambda n, r, c: device.Weights(np.concatenate(raws[n]), kind, r, c, n_mats=n_exp)
    layer = prefill.RoutedLayer(torch.from_numpy(router).cuda(), mk("gate", ffn, hidden), mk("up", ffn, hidden), mk("down", hidden, ffn),
                                k=k, mode=mode, act=act)
    return raws, router, layer


@pytest.mark.parametrize("kind,hidden,ffn,act,mode", [(fo.Q4_K, 512, 768, 0, 1), (fo.MXFP4, 576, 576, 1, 2), (fo.Q6_K, 256, 512, 0, 0)])
def test_routed_layer_decode_and_prefill(kind, hidden, ffn, act, mode):
    from frink_b200 import device, prefill
    n_exp, k = 16, 4
    raws, router, layer = build_layer(kind, n_exp, hidden, ffn, k, mode, act, 900)
    rng = np.random.default_rng(4)
    x = rng.standard_normal((40, hidden)).astype(np.float32)
    ids_want, want = oracle_layer(raws, kind, router, x, k, mode, hidden, ffn, act)
    xd = torch.from_numpy(x).cuda()
    ids, _ = prefill.route(layer, xd)
    assert np.array_equal(ids.cpu().numpy(), ids_want)
    got_b = prefill.run_device_routed_batch(layer, xd).cpu().numpy()
    torch.cuda.synchronize()
    assert device.device_error() == 0
    assert rel_l2(got_b, want) <= 1e-3 and max_abs_over_inf(got_b, want) <= 2e-3
    got_d = prefill.run_device_routed(layer, xd[:3]).cpu().numpy()
    assert rel_l2(got_d, want[:3]) <= 1e-3 and max_abs_over_inf(got_d, want[:3]) <= 2e-3
    # decode and prefill read the same integers: they agree to f32 summation noise
    assert rel_l2(got_d, got_b[:3]) <= 5e-6


def oracle_layer_grouped(raws, kind, router, x, k, mode, hidden, ffn, act):
    """`oracle_layer` with the tokens of an expert taken together (the same numbers: each output
    row depends on its own token only), so that a 512-token, 128-expert case finishes in seconds."""
    logits = (x.astype(np.float32) @ router.T.astype(np.float32)).astype(np.float32)
    ids, w = fo.route_top_k(logits, k, mode)
    n = x.shape[0]
    ys = np.zeros((n, k, hidden), np.float32)
    xq = fo.q8_1_round(x)
    for e in np.unique(ids):
        t, j = np.nonzero(ids == e)
        g = fo.matmul_f64(kind, raws["gate"][e], ffn, hidden, xq[t]).astype(np.float32)
        u = fo.matmul_f64(kind, raws["up"][e], ffn, hidden, xq[t]).astype(np.float32)
        a = (fo.silu_mul(g.ravel(), u.ravel()) if act == 0 else fo.swiglu_oai(g.ravel(), u.ravel())).reshape(g.shape)
        ys[t, j] = fo.matmul_f64(kind, raws["down"][e], hidden, ffn, fo.q8_1_round(a)).astype(np.float32)
    out = np.stack([fo.combine(ys[t], w[t]) for t in range(n)])
    return ids, out


def test_config4_shaped_routed_layer():
    """The routed layer at the Qwen3-30B-A3B shape: 128 experts, top-8 (softmax, renormalised),
    hidden 2048, expert FFN 768, Q4_K experts -- decode rows and a 512-token prefill."""
    from frink_b200 import device, prefill
    n_exp, k, hidden, ffn, kind = 128, 8, 2048, 768, fo.Q4_K
    raws, router, layer = build_layer(kind, n_exp, hidden, ffn, k, 1, 0, 4000)
    x = np.random.default_rng(44).standard_normal((512, hidden)).astype(np.float32)
    ids_want, want = oracle_layer_grouped(raws, kind, router, x, k, 1, hidden, ffn, 0)
    xd = torch.from_numpy(x).cuda()
    ids, _ = prefill.route(layer, xd)
    assert np.array_equal(ids.cpu().numpy(), ids_want)
    assert len(np.unique(ids_want)) > 100          # the router spreads the tokens: most experts are exercised
    got = prefill.run_device_routed_batch(layer, xd).cpu().numpy()
    torch.cuda.synchronize()
    assert device.device_error() == 0
    assert rel_l2(got, want) <= 1e-3 and max_abs_over_inf(got, want) <= 2e-3, (rel_l2(got, want), max_abs_over_inf(got, want))
    got_d = prefill.run_device_routed(layer, xd[:8]).cpu().numpy()
    assert rel_l2(got_d, want[:8]) <= 1e-3 and max_abs_over_inf(got_d, want[:8]) <= 2e-3
    # decode and prefill take their gate / up sums in different f32 orders; where that moves a gated
    # activation across a q8_1 rounding boundary the down projection's input differs by one step
    assert rel_l2(got_d, got[:8]) <= 1e-3


def test_biased_routed_layer_one_call_against_the_composition_and_the_oracle():
    """gpt-oss's routed layer (`run_expert_oai`, crates/frink-moe/src/lib.rs:1039-1060) as one C call: the biases ride
    in the indexed matvecs' epilogues (decode) or follow the grouped GEMMs (prefill).  Bit-identical to the same layer
    composed from the separate entry points, and equal to the oracle's composition with the bias rows added."""
    import types
    from frink_b200 import device, prefill
    kind, n_exp, k, hidden, ffn, mode, act = fo.MXFP4, 8, 2, 576, 320, 1, 1
    raws, router, layer = build_layer(kind, n_exp, hidden, ffn, k, mode, act, 1200)
    rng = np.random.default_rng(9)
    gb, ub, db = (rng.standard_normal((n_exp, n)).astype(np.float32) * 0.2 for n in (ffn, ffn, hidden))
    biases = tuple(torch.from_numpy(b).cuda() for b in (gb, ub, db))
    x = rng.standard_normal((40, hidden)).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    separate = types.SimpleNamespace(**{n: getattr(device, n) for n in dir(device) if not n.startswith("_") and n != "moe_layer"})
    for rows in (1, 4, 8, 40):
        one = prefill.run_device_routed_oai(layer, biases, xd[:rows])
        assert torch.equal(one, prefill.run_device_routed_oai(layer, biases, xd[:rows], separate)), rows
        res = torch.randn(rows, hidden, device="cuda")
        want = res + one
        prefill.run_device_routed_oai(layer, biases, xd[:rows], residual=res)
        assert torch.equal(res, want), rows
    # the oracle's composition on three rows
    logits = (x[:3] @ router.T).astype(np.float32)
    ids, w = fo.route_top_k(logits, k, mode)
    want = np.zeros((3, hidden), np.float32)
    for t in range(3):
        ys = []
        for e in ids[t]:
            xq = fo.q8_1_round(x[t])
            g = fo.matmul_f64(kind, raws["gate"][e], ffn, hidden, xq)[0].astype(np.float32) + gb[e]
            u = fo.matmul_f64(kind, raws["up"][e], ffn, hidden, xq)[0].astype(np.float32) + ub[e]
            ys.append(fo.matmul_f64(kind, raws["down"][e], hidden, ffn, fo.q8_1_round(fo.swiglu_oai(g, u)))[0].astype(np.float32) + db[e])
        want[t] = fo.combine(np.stack(ys), w[t])
    got = prefill.run_device_routed_oai(layer, biases, xd[:3]).cpu().numpy()
    assert rel_l2(got, want) <= 1e-3 and max_abs_over_inf(got, want) <= 2e-3
    assert device.device_error() == 0


@pytest.mark.parametrize("kind,biased", [(fo.MXFP4, True), (fo.Q4_K, False), (fo.Q8_0, False)])
def test_routed_layer_on_the_residual_stream_is_the_separate_launches_to_the_bit(kind, biased):
    """fk_moe_layer_normed: the RMSNorm folded into the router and the matvec, gate and up as the two halves of one
    launch.  The same routes and the same output bits as norm launch + fk_moe_layer(_biased), for 1, 3 and 8 rows; and
    fk_gemv_multi_gate_up alone against the two indexed launches."""
    from frink_b200 import device, prefill
    n_exp, k, hidden, ffn, mode, act = 8, 2, 512, 256, 1, 1 if biased else 0
    raws, router, layer = build_layer(kind, n_exp, hidden, ffn, k, mode, act, 1500)
    rng = np.random.default_rng(21)
    biases = None
    if biased:
        biases = tuple(torch.from_numpy(rng.standard_normal((n_exp, n)).astype(np.float32) * 0.2).cuda() for n in (ffn, ffn, hidden))
    nw = torch.from_numpy((1.0 + 0.1 * rng.standard_normal(hidden)).astype(np.float32)).cuda()
    eps = 1e-5
    x = torch.from_numpy(rng.standard_normal((8, hidden)).astype(np.float32) * 1.7).cuda()
    for rows in (1, 3, 8):
        res = x[:rows].clone()
        h = device.rmsnorm(res.clone(), nw, eps)
        want = res + (device.moe_layer(layer, h, biases=biases) if biased else device.moe_layer(layer, h))
        got = res.clone()
        device.moe_layer(layer, got, out=got, accumulate=True, biases=biases, norm=(nw, eps))
        assert torch.equal(got, want), rows
    # the two-projection launch alone
    ids = torch.tensor([5, 1, 5], dtype=torch.int32, device="cuda")
    xs = x[:3].contiguous()
    both = device.gemv_multi_gate_up(layer.gate, layer.up, ids, xs)
    assert torch.equal(both[:3], device.gemv_multi(layer.gate, ids, xs)) and torch.equal(both[3:], device.gemv_multi(layer.up, ids, xs))
    h3 = device.rmsnorm(xs.clone(), nw, eps)
    both = device.gemv_multi_gate_up(layer.gate, layer.up, ids, xs, norm_weight=nw, eps=eps)
    assert torch.equal(both[:3], device.gemv_multi(layer.gate, ids, h3)) and torch.equal(both[3:], device.gemv_multi(layer.up, ids, h3))
    with pytest.raises(Exception):
        device.moe_layer(layer, x.repeat(2, 1), norm=(nw, eps))        # 16 rows: the folded form is the decode form
    assert device.device_error() == 0
