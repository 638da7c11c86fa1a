"""MoE plumbing kernels against the oracle: routing (ids exact, weights to f32
rounding), the expert permutation, the gated activations and the combine."""
import numpy as np
import pytest
import torch

from oracle import frink_oracle as fo
from tests.helpers import synth_weights

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n_experts,k,mode", [(128, 8, 1), (128, 4, 2), (64, 6, 0), (8, 2, 1), (256, 16, 1), (5, 5, 0)])
def test_route_matches_oracle(n_experts, k, mode):
    from frink_b200 import device
    rng = np.random.default_rng(n_experts + k)
    logits = rng.standard_normal((33, n_experts)).astype(np.float32)
    logits[3, :] = 0.25          # all tied: lower ids first
    logits[4, 1] = logits[4, 0]  # a tie at the top
    bias = rng.standard_normal(n_experts).astype(np.float32) if mode == 2 else None
    ids, w = device.moe_route(torch.from_numpy(logits).cuda(), k, mode, None if bias is None else torch.from_numpy(bias).cuda())
    wi, ww = fo.route_top_k(logits, k, mode, bias)
    assert np.array_equal(ids.cpu().numpy(), wi)
    assert np.allclose(w.cpu().numpy(), ww, rtol=2e-6, atol=1e-8)


def test_permute_groups_pairs_by_expert_in_token_order():
    from frink_b200 import device
    rng = np.random.default_rng(2)
    n_experts, k, batch = 128, 8, 512
    ids = np.stack([rng.choice(n_experts, k, replace=False) for _ in range(batch)]).astype(np.int32)
    off, gather, pair_of = [t.cpu().numpy() for t in device.moe_permute(torch.from_numpy(ids).cuda(), n_experts)]
    flat = ids.ravel()
    assert off[0] == 0 and off[-1] == batch * k and np.array_equal(np.diff(off), np.bincount(flat, minlength=n_experts))
    order = np.argsort(flat, kind="stable")
    assert np.array_equal(gather, order // k)
    assert np.array_equal(pair_of[order], np.arange(batch * k))
    # one pair, and an expert nobody chose
    off, gather, pair_of = [t.cpu().numpy() for t in device.moe_permute(torch.tensor([[2]], dtype=torch.int32).cuda(), 4)]
    assert list(off) == [0, 0, 0, 1, 1] and list(gather) == [0] and list(pair_of) == [0]


def test_glu_combine_and_router_logits():
    from frink_b200 import device
    rng = np.random.default_rng(3)
    g = (rng.standard_normal(5000) * 4).astype(np.float32)
    u = (rng.standard_normal(5000) * 4).astype(np.float32)
    gd, ud = torch.from_numpy(g).cuda(), torch.from_numpy(u).cuda()
    assert np.allclose(device.glu(gd, ud, 0).cpu().numpy(), fo.silu_mul(g, u), rtol=2e-6, atol=1e-7)
    assert np.allclose(device.glu(gd, ud, 1).cpu().numpy(), fo.swiglu_oai(g, u), rtol=2e-6, atol=1e-7)
    batch, k, n = 7, 4, 333
    ys = rng.standard_normal((batch * k, n)).astype(np.float32)
    w = rng.random((batch, k)).astype(np.float32)
    perm = rng.permutation(batch * k).astype(np.int32)
    out = device.moe_combine(torch.from_numpy(ys).cuda(), torch.from_numpy(perm).cuda(), torch.from_numpy(w).cuda(), batch, k).cpu().numpy()
    for t in range(batch):
        want = fo.combine(ys[perm[t * k:(t + 1) * k]], w[t])
        assert np.allclose(out[t], want, rtol=1e-6, atol=1e-6)
    router = (rng.standard_normal((128, 2048)) * 0.02).astype(np.float32)
    x = rng.standard_normal((5, 2048)).astype(np.float32)
    lg = device.router_logits(torch.from_numpy(router).cuda(), torch.from_numpy(x).cuda()).cpu().numpy()
    assert np.allclose(lg, x.astype(np.float64) @ router.astype(np.float64).T, rtol=1e-4, atol=1e-5)


def test_local_slots_and_active_count_for_expert_parallel_decode():
    """The device-side half of expert-parallel decode: routed ids -> this rank's local
    slots, weights and count (`fk_moe_local_slots`), and the indexed matvec that runs
    only that many slots (`fk_gemv_multi_active`), leaving the other outputs alone."""
    from frink_b200 import device
    n_exp, rows, cols, k = 8, 96, 768, 6
    raws = np.concatenate([fo.encode(fo.Q4_K, synth_weights(rows, cols, 700 + e)) for e in range(n_exp)])
    w = device.Weights(raws, fo.Q4_K, rows, cols, n_mats=n_exp)
    ids = np.array([5, 1, 7, 2, 4, 0], np.int32)
    wt = np.array([0.3, 0.1, 0.2, 0.15, 0.05, 0.2], np.float32)
    x = torch.from_numpy(np.random.default_rng(3).standard_normal(cols).astype(np.float32)).cuda()
    for e0, n_local in ((4, 4), (0, 4), (6, 2), (0, 8)):
        li, lw, ln = device.moe_local_slots(torch.from_numpy(ids).cuda(), torch.from_numpy(wt).cuda(), e0, n_local)
        mine = [(int(i) - e0, float(v)) for i, v in zip(ids, wt) if e0 <= i < e0 + n_local]
        n = int(ln.item())
        assert n == len(mine)
        assert [(int(a), float(b)) for a, b in zip(li[:n].cpu(), lw[:n].cpu())] == [(a, np.float32(b)) for a, b in mine]
        assert not lw[n:].cpu().numpy().any()
        # the weights of this rank's experts alone, as the rank holds them
        per = rows * fo.row_bytes(fo.Q4_K, cols)
        wl = device.Weights(raws[e0 * per:(e0 + n_local) * per], fo.Q4_K, rows, cols, n_mats=n_local)
        out = torch.full((k, rows), 7.0, device="cuda")
        device.gemv_multi_active(wl, li, x, ln, out)
        want = device.gemv_multi(wl, li[:n].contiguous(), x) if n else None
        got = out.cpu().numpy()
        if n:
            assert np.array_equal(got[:n], want.cpu().numpy())
        assert np.all(got[n:] == 7.0)
    assert device.device_error() == 0


def test_indexed_down_projection_with_glu_and_combine_into_the_residual():
    """`fk_gemv_multi_glu` = GLU kernel + `fk_gemv_multi`, bit for bit; `fk_moe_combine_add` =
    residual + `fk_moe_combine`."""
    from frink_b200 import device
    n_exp, rows, cols, k = 6, 128, 512, 4
    raws = np.concatenate([fo.encode(fo.Q4_K, synth_weights(rows, cols, 800 + e)) for e in range(n_exp)])
    w = device.Weights(raws, fo.Q4_K, rows, cols, n_mats=n_exp)
    rng = np.random.default_rng(11)
    ids = torch.tensor([4, 0, 5, 2], dtype=torch.int32).cuda()
    g = torch.from_numpy(rng.standard_normal((k, cols)).astype(np.float32)).cuda()
    u = torch.from_numpy(rng.standard_normal((k, cols)).astype(np.float32)).cuda()
    for act in (0, 1):
        want = device.gemv_multi(w, ids, device.glu(g, u, act))
        got = device.gemv_multi_glu(w, ids, g, u, act)
        assert torch.equal(got, want)
    wt = torch.from_numpy(rng.random(k).astype(np.float32)).cuda()
    res = torch.from_numpy(rng.standard_normal((1, rows)).astype(np.float32)).cuda()
    out = res.clone()
    device.moe_combine(got, None, wt, 1, k, out=out, accumulate=True)
    assert torch.equal(out, res + device.moe_combine(got, None, wt, 1, k))
    assert device.device_error() == 0


@pytest.mark.parametrize("n_experts,k,mode,batch", [(128, 8, 1, 1), (64, 6, 0, 3), (128, 4, 2, 8)])
def test_fused_router_equals_logits_then_route(n_experts, k, mode, batch):
    from frink_b200 import device
    rng = np.random.default_rng(n_experts + k)
    hidden = 2048
    router = torch.from_numpy((rng.standard_normal((n_experts, hidden)) * 0.05).astype(np.float32)).cuda()
    x = torch.from_numpy(rng.standard_normal((batch, hidden)).astype(np.float32)).cuda()
    want_ids, want_w = device.moe_route(device.router_logits(router, x), k, mode)
    for _ in range(2):      # the second call finds the arrival counter rewound
        ids, w = device.router_route(router, x, k, mode)
        assert torch.equal(ids, want_ids) and torch.equal(w, want_w)
