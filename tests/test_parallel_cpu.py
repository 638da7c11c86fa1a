"""Host-side sharding logic of `frink_b200.parallel` on CPU: world_size-2 gloo
ranks with the oracle standing in for the device kernels.  Checks that the
sharded result equals the unsharded one (bit-exact where the design promises it)."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import frink_oracle as fo
from tests.helpers import rel_l2, synth_weights


def _run(rank, world, port, fn, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ret[rank] = fn(rank, world)
    finally:
        dist.destroy_process_group()


def spawn(fn, world=2):
    port = 29500 + os.getpid() % 2000
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_run, args=(world, port, fn, ret), nprocs=world, join=True)
    return [ret[r] for r in range(world)]


def test_shard_helpers():
    from frink_b200 import parallel
    raw = fo.encode(fo.Q4_K, synth_weights(8, 1024, 1))
    a, r = parallel.shard_rows(raw, fo.Q4_K, 8, 1024, 1, 2)
    assert r == 4 and np.array_equal(a, raw[4 * 576:])
    b, c = parallel.shard_cols(raw, fo.Q4_K, 8, 1024, 1, 2)
    assert c == 512 and np.array_equal(b.reshape(8, 288), raw.reshape(8, 576)[:, 288:])
    # a K shard dequantizes to the K range of the full matrix
    assert np.array_equal(fo.dequant(fo.Q4_K, b).reshape(8, 512), fo.dequant(fo.Q4_K, raw).reshape(8, 1024)[:, 512:])
    with pytest.raises(ValueError):
        parallel.shard_cols(fo.encode(fo.Q4_K, synth_weights(2, 768, 1)), fo.Q4_K, 2, 768, 0, 2)   # 3 blocks over 2 ranks
    with pytest.raises(ValueError):
        parallel.shard_rows(raw, fo.Q4_K, 8, 1024, 0, 3)


def _tp_case(rank, world):
    from frink_b200 import parallel
    from tests import cpu_ops
    hidden, ffn = 512, 1024
    g = fo.encode(fo.Q4_K, synth_weights(ffn, hidden, 11))
    u = fo.encode(fo.Q4_K, synth_weights(ffn, hidden, 12))
    d = fo.encode(fo.Q6_K, synth_weights(hidden, ffn, 13))
    x = torch.from_numpy(np.random.default_rng(5).standard_normal((3, hidden)).astype(np.float32))
    col = parallel.ColumnParallelLinear(cpu_ops, g, fo.Q4_K, ffn, hidden, gather=True)
    y_col = col(x).numpy()
    ffn_tp = parallel.TensorParallelFFN(cpu_ops, g, u, d, fo.Q4_K, fo.Q6_K, hidden, ffn)
    y_ffn = ffn_tp(x).numpy()
    return y_col, y_ffn


def test_tensor_parallel_matches_single_rank():
    from tests import cpu_ops
    hidden, ffn = 512, 1024
    g = fo.encode(fo.Q4_K, synth_weights(ffn, hidden, 11))
    u = fo.encode(fo.Q4_K, synth_weights(ffn, hidden, 12))
    d = fo.encode(fo.Q6_K, synth_weights(hidden, ffn, 13))
    x = torch.from_numpy(np.random.default_rng(5).standard_normal((3, hidden)).astype(np.float32))
    wg, wu, wd = cpu_ops.Weights(g, fo.Q4_K, ffn, hidden), cpu_ops.Weights(u, fo.Q4_K, ffn, hidden), cpu_ops.Weights(d, fo.Q6_K, hidden, ffn)
    want_col = cpu_ops.gemv(wg, x).numpy()
    want_ffn = cpu_ops.gemv(wd, cpu_ops.glu(cpu_ops.gemv(wg, x), cpu_ops.gemv(wu, x))).numpy()
    for y_col, y_ffn in spawn(_tp_case):
        assert np.array_equal(y_col, want_col)                 # whole rows: nothing changes
        assert rel_l2(y_ffn, want_ffn) <= 1e-5                # K split: only the f32 summation order
    

def _ep_case(rank, world):
    from frink_b200 import parallel
    from tests import cpu_ops
    n_exp, hidden, ffn, k = 8, 256, 512, 2
    raws = {n: np.concatenate([fo.encode(fo.Q4_K, synth_weights(r, c, 100 * i + e)) for e in range(n_exp)])
            for i, (n, r, c) in enumerate((("gate", ffn, hidden), ("up", ffn, hidden), ("down", hidden, ffn)))}
    router = torch.from_numpy((np.random.default_rng(1).standard_normal((n_exp, hidden)) * 0.5).astype(np.float32))
    ep = parallel.ExpertParallelLayer(cpu_ops, router, raws["gate"], raws["up"], raws["down"], fo.Q4_K, n_exp, hidden, ffn, k)
    x = torch.from_numpy(np.random.default_rng(2).standard_normal((6, hidden)).astype(np.float32))
    dec = ep.decode(x[0]).numpy()
    per = 6 // world
    pre = ep.prefill(x[rank * per:(rank + 1) * per]).numpy()
    rows = ep.decode_rows(x).numpy()          # a decode batch: all six rows replicated on every rank
    return dec, pre, rows


def test_expert_parallel_matches_single_rank():
    from frink_b200 import prefill
    from tests import cpu_ops
    n_exp, hidden, ffn, k = 8, 256, 512, 2
    raws = {n: np.concatenate([fo.encode(fo.Q4_K, synth_weights(r, c, 100 * i + e)) for e in range(n_exp)])
            for i, (n, r, c) in enumerate((("gate", ffn, hidden), ("up", ffn, hidden), ("down", hidden, ffn)))}
    router = torch.from_numpy((np.random.default_rng(1).standard_normal((n_exp, hidden)) * 0.5).astype(np.float32))
    mk = lambda n, r, c: cpu_ops.Weights(raws[n], fo.Q4_K, r, c, n_mats=n_exp)
    layer = prefill.RoutedLayer(router, mk("gate", ffn, hidden), mk("up", ffn, hidden), mk("down", hidden, ffn), k=k, mode=1)
    x = torch.from_numpy(np.random.default_rng(2).standard_normal((6, hidden)).astype(np.float32))
    want = prefill.run_device_routed_batch(layer, x, cpu_ops).numpy()
    want_dec = prefill.run_device_routed(layer, x[0], cpu_ops).numpy()
    assert rel_l2(want_dec, want[0]) <= 1e-6
    res = spawn(_ep_case)
    for rank, (dec, pre, rows) in enumerate(res):
        assert rel_l2(rows, want) <= 1e-6                      # the slot form of a decode batch
        assert rel_l2(dec, want_dec) <= 1e-6                   # partial sums all-reduced: order of two adds
        assert np.array_equal(pre, want[rank * 3:(rank + 1) * 3])   # dispatch/combine keeps the single-rank order: same bits


def _ep_ragged_case(rank, world):
    """9 rows over 4 ranks: shares of 3, 3, 3 and NONE -- the last rank still has to make every collective call."""
    from frink_b200 import parallel
    from tests import cpu_ops
    n_exp, hidden, ffn, k = 8, 256, 512, 2
    raws = {n: np.concatenate([fo.encode(fo.Q4_K, synth_weights(r, c, 100 * i + e)) for e in range(n_exp)])
            for i, (n, r, c) in enumerate((("gate", ffn, hidden), ("up", ffn, hidden), ("down", hidden, ffn)))}
    router = torch.from_numpy((np.random.default_rng(1).standard_normal((n_exp, hidden)) * 0.5).astype(np.float32))
    ep = parallel.ExpertParallelLayer(cpu_ops, router, raws["gate"], raws["up"], raws["down"], fo.Q4_K, n_exp, hidden, ffn, k)
    x = torch.from_numpy(np.random.default_rng(2).standard_normal((9, hidden)).astype(np.float32))
    per = -(-9 // world)
    lo, hi = min(9, rank * per), min(9, (rank + 1) * per)
    sharded = ep.prefill(x[lo:hi].contiguous()).numpy()     # tokens sharded: two all-to-alls, also from the rank with no rows
    replicated = ep.prefill_replicated(x).numpy()           # activations replicated: one all-reduce
    return lo, hi, sharded, replicated


def test_expert_parallel_prefill_with_a_rank_that_has_no_rows():
    from frink_b200 import prefill
    from tests import cpu_ops
    n_exp, hidden, ffn, k = 8, 256, 512, 2
    raws = {n: np.concatenate([fo.encode(fo.Q4_K, synth_weights(r, c, 100 * i + e)) for e in range(n_exp)])
            for i, (n, r, c) in enumerate((("gate", ffn, hidden), ("up", ffn, hidden), ("down", hidden, ffn)))}
    router = torch.from_numpy((np.random.default_rng(1).standard_normal((n_exp, hidden)) * 0.5).astype(np.float32))
    mk = lambda n, r, c: cpu_ops.Weights(raws[n], fo.Q4_K, r, c, n_mats=n_exp)
    layer = prefill.RoutedLayer(router, mk("gate", ffn, hidden), mk("up", ffn, hidden), mk("down", hidden, ffn), k=k, mode=1)
    x = torch.from_numpy(np.random.default_rng(2).standard_normal((9, hidden)).astype(np.float32))
    want = prefill.run_device_routed_batch(layer, x, cpu_ops).numpy()
    res = spawn(_ep_ragged_case, world=4)
    assert [hi - lo for lo, hi, _, _ in res] == [3, 3, 3, 0]
    for lo, hi, sharded, replicated in res:
        assert np.array_equal(sharded, want[lo:hi])               # dispatch / combine keeps the single-rank order: same bits
        assert rel_l2(replicated, want) <= 1e-6                   # partial sums all-reduced: the order of a few adds
    for r in res[1:]:
        assert np.array_equal(r[3], res[0][3])                    # and every rank ends with the same rows


def _tiny_model(moe):
    from frink_b200.decoder import DecoderConfig, LayerWeights
    rng = np.random.default_rng(21)
    if moe:
        cfg = DecoderConfig(n_layers=2, hidden=512, n_heads=8, n_kv=2, head_dim=64, ffn=256, vocab=512, n_experts=4, top_k=2, route_mode=1,
                            neox=True, qk_norm=True)
    else:
        cfg = DecoderConfig(n_layers=2, hidden=512, n_heads=8, n_kv=2, head_dim=64, ffn=512, vocab=512)
    H, hd = cfg.hidden, cfg.head_dim
    enc = lambda kind, r, c: fo.encode(kind, (rng.standard_normal((r, c)) * 0.05).astype(np.float32))
    layers = []
    for _ in range(cfg.n_layers):
        norm = lambda n: (1 + 0.1 * rng.standard_normal(n)).astype(np.float32)
        common = dict(attn_norm=norm(H), wq=enc(fo.Q4_K, cfg.n_heads * hd, H), wk=enc(fo.Q4_K, cfg.n_kv * hd, H), wv=enc(fo.Q4_K, cfg.n_kv * hd, H),
                      wo=enc(fo.Q4_K, H, cfg.n_heads * hd), ffn_norm=norm(H))
        if moe:
            st = lambda r, c: np.concatenate([enc(fo.Q4_K, r, c) for _ in range(cfg.n_experts)])
            layers.append(LayerWeights(**common, gate=st(cfg.ffn, H), up=st(cfg.ffn, H), down=st(H, cfg.ffn),
                                       router=(rng.standard_normal((cfg.n_experts, H)) * 0.5).astype(np.float32), q_norm=norm(hd), k_norm=norm(hd),
                                       kinds={"wq": fo.Q4_K, "wk": fo.Q4_K, "wv": fo.Q4_K, "wo": fo.Q4_K, "experts": fo.Q4_K}))
        else:
            layers.append(LayerWeights(**common, gate=enc(fo.Q4_K, cfg.ffn, H), up=enc(fo.Q4_K, cfg.ffn, H), down=enc(fo.Q4_K, H, cfg.ffn),
                                       kinds={k: fo.Q4_K for k in ("wq", "wk", "wv", "wo", "gate", "up", "down")}))
    tok = fo.encode(fo.Q8_0, rng.standard_normal((cfg.vocab, H)).astype(np.float32))
    head = fo.encode(fo.Q8_0, (rng.standard_normal((cfg.vocab, H)) * 0.5).astype(np.float32))
    return cfg, layers, tok, norm(H), head


def _decoder_logits(moe, group_world, dense_parallel=True):
    from frink_b200.decoder import Decoder
    from tests import cpu_ops
    cfg, layers, tok, out_norm, head = _tiny_model(moe)
    dec = Decoder(cfg, layers, tok, fo.Q8_0, out_norm, output=head, output_kind=fo.Q8_0, max_seq=32, ops=cpu_ops, device="cpu",
                  dense_parallel=dense_parallel)
    assert dec.world == group_world
    prompt = torch.from_numpy(np.random.default_rng(3).integers(0, cfg.vocab, 12).astype(np.int32))
    lg_prefill = dec.forward(prompt).numpy().copy()            # 12 rows: the batched path
    lg_decode = dec.forward(torch.tensor([7], dtype=torch.int32)).numpy().copy()   # one row at position 12
    return lg_prefill, lg_decode


def _decoder_dense_case(rank, world):
    return _decoder_logits(False, world)


def _decoder_moe_case(rank, world):
    return _decoder_logits(True, world)


def _decoder_moe_replicated_case(rank, world):
    return _decoder_logits(True, world, dense_parallel=False)


def _decoder_oai_logits(rank, world):
    from frink_b200.decoder import Decoder
    from tests import cpu_ops
    from tests.helpers import tiny_gpt_oss
    cfg, layers, tok, out_norm, head = tiny_gpt_oss()
    dec = Decoder(cfg, layers, tok, fo.BF16, out_norm, output=head, output_kind=fo.BF16, max_seq=32, ops=cpu_ops, device="cpu",
                  dense_parallel=False)
    assert dec.world == world
    prompt = torch.from_numpy(np.random.default_rng(3).integers(0, cfg.vocab, 12).astype(np.int32))
    outs = [dec.forward(prompt).numpy().copy()]                                        # 12 rows: grouped GEMMs with the bias rows
    outs.append(dec.forward(torch.tensor([7], dtype=torch.int32)).numpy().copy())      # one row
    outs.append(dec.forward(torch.tensor([5, 9, 2], dtype=torch.int32)).numpy().copy())   # a few rows: slots
    return outs


def test_gpt_oss_form_with_sharded_experts_matches_one_rank():
    """gpt-oss's layer form on two ranks: attention (and its biases) replicated, the experts AND their bias rows spread
    over the ranks, the router bias replicated.  Prompt rows, one row and a few rows against the same decoder on one rank."""
    want = spawn(_decoder_oai_logits, world=1)[0]
    got = spawn(_decoder_oai_logits, world=2)
    for r in range(2):
        for a, b in zip(got[r], want):
            assert rel_l2(a, b) <= 1e-4
    for a, b in zip(got[0], got[1]):
        assert np.array_equal(a, b)
    # the tensor-parallel plan has no gpt-oss variant: refused when the decoder is built
    msgs = spawn(_oai_tp_refused, world=2)
    assert all(m and "tensor-parallel" in m for m in msgs)


def _oai_tp_refused(rank, world):
    from frink_b200.decoder import Decoder
    from tests import cpu_ops
    from tests.helpers import tiny_gpt_oss
    cfg, layers, tok, out_norm, head = tiny_gpt_oss()
    try:
        Decoder(cfg, layers, tok, fo.BF16, out_norm, output=head, output_kind=fo.BF16, max_seq=32, ops=cpu_ops, device="cpu")
    except ValueError as e:
        return str(e)
    return None


def test_decoder_with_replicated_attention_and_sharded_experts_matches_one_rank():
    """The plan for routed models on more ranks than KV heads: attention on every rank, experts
    spread over the ranks.  Prefill (dispatch/combine) and the fused decode path."""
    want = spawn(_decoder_moe_case, world=1)[0]
    got = spawn(_decoder_moe_replicated_case, world=2)
    for r in range(2):
        for a, b in zip(got[r], want):
            assert rel_l2(a, b) <= 1e-4
    for a, b in zip(got[0], got[1]):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("moe", [False, True])
def test_decoder_sharded_over_two_ranks_matches_one(moe):
    """The whole decoder under TP (dense) and TP+EP (routed) on two gloo ranks against the
    same decoder on one rank: same collectives on every rank (no deadlock), same logits up
    to the f32 summation order of the K-split projections."""
    want = spawn(_decoder_moe_case if moe else _decoder_dense_case, world=1)[0]
    got = spawn(_decoder_moe_case if moe else _decoder_dense_case, world=2)
    for r in range(2):
        for a, b in zip(got[r], want):
            assert rel_l2(a, b) <= 1e-4
    for a, b in zip(got[0], got[1]):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("kind", [fo.Q4_K, fo.Q6_K])
def test_a_k_range_cut_inside_blocks_is_the_product_restricted_to_the_window(kind):
    """3072 columns over 8 ranks: 384 columns a rank, one and a half 256-wide blocks.  Each rank holds whole
    blocks with the columns outside its window masked (scales zeroed, quants untouched); the partial
    products over the padded inputs add up to the unsharded product, and what a rank's shard decodes to
    is the matrix inside its window and zero outside."""
    from frink_b200 import parallel
    rows, cols, world = 24, 3072, 8
    raw = fo.encode(kind, synth_weights(rows, cols, 21))
    x = np.random.default_rng(3).standard_normal((2, cols)).astype(np.float32)
    xq = fo.q8_1_round(x)
    want = fo.matmul_f64(kind, raw, rows, cols, xq)
    full = fo.dequant(kind, raw).reshape(rows, cols)
    total = np.zeros_like(want)
    for rank in range(world):
        loc, cl, off, width = parallel.shard_cols_window(raw, kind, rows, cols, rank, world)
        assert width == 384 and cl == 512 and off in (0, 128)
        lo = rank * width
        dq = fo.dequant(kind, loc).reshape(rows, cl)
        assert np.array_equal(dq[:, off:off + width], full[:, lo:lo + width])
        assert not dq[:, :off].any() and not dq[:, off + width:].any()
        xp = np.full((2, cl), 7.0, np.float32)           # anything finite outside the window
        xp[:, off:off + width] = x[:, lo:lo + width]
        total += fo.matmul_f64(kind, loc, rows, cl, fo.q8_1_round(xp))
    assert rel_l2(total, want) <= 1e-6


def _row_window_case(rank, world):
    from frink_b200 import parallel
    from tests import cpu_ops
    raw = fo.encode(fo.Q4_K, synth_weights(16, 1536, 31))
    x = torch.from_numpy(np.random.default_rng(6).standard_normal((2, 1536)).astype(np.float32))
    lin = parallel.RowParallelLinear(cpu_ops, raw, fo.Q4_K, 16, 1536, input_is_sharded=True)
    assert lin.window is not None and lin.cols_local == 512
    return lin(x[:, rank * 384:(rank + 1) * 384].contiguous()).numpy()


def test_row_split_over_four_ranks_of_six_blocks():
    """1536 columns (six Q4_K blocks) over four ranks: every rank's 384 columns are cut inside a block."""
    from tests import cpu_ops
    raw = fo.encode(fo.Q4_K, synth_weights(16, 1536, 31))
    x = torch.from_numpy(np.random.default_rng(6).standard_normal((2, 1536)).astype(np.float32))
    want = cpu_ops.gemv(cpu_ops.Weights(raw, fo.Q4_K, 16, 1536), x).numpy()
    for y in spawn(_row_window_case, world=4):
        assert rel_l2(y, want) <= 1e-5
