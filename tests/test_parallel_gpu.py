"""TP / EP over NCCL on two GPUs (skipped where fewer are visible): each rank's
local work is the single-GPU path, so the sharded results are held to the
single-GPU results computed in the same process."""
import os

import numpy as np
import pytest
import torch

from oracle import frink_oracle as fo
from tests.helpers import rel_l2, synth_weights

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, ret):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from frink_b200 import device, parallel, prefill
        hidden, ffn, n_exp, k = 1024, 2048, 8, 2
        g = fo.encode(fo.Q4_K, synth_weights(ffn, hidden, 11))
        u = fo.encode(fo.Q4_K, synth_weights(ffn, hidden, 12))
        d = fo.encode(fo.Q6_K, synth_weights(hidden, ffn, 13))
        rng = np.random.default_rng(5)
        x = torch.from_numpy(rng.standard_normal((64, hidden)).astype(np.float32)).cuda()
        out = {}
        # dense TP: decode (batch 2, GEMV) and prefill (64 tokens, GEMM)
        tp = parallel.TensorParallelFFN(device, g, u, d, fo.Q4_K, fo.Q6_K, hidden, ffn)
        wg, wu, wd = device.Weights(g, fo.Q4_K, ffn, hidden), device.Weights(u, fo.Q4_K, ffn, hidden), device.Weights(d, fo.Q6_K, hidden, ffn)
        ref_dec = device.gemv(wd, device.glu(device.gemv(wg, x[:2]), device.gemv(wu, x[:2])))
        ref_pre = device.gemm(wd, device.glu(device.gemm(wg, x), device.gemm(wu, x)))
        out["tp_dec"] = rel_l2(tp(x[:2]).cpu().numpy(), ref_dec.cpu().numpy())
        out["tp_pre"] = rel_l2(tp(x).cpu().numpy(), ref_pre.cpu().numpy())
        # experts EP
        raws = {n: np.concatenate([fo.encode(fo.Q4_K, synth_weights(r, c, 100 * i + e)) for e in range(n_exp)])
                for i, (n, r, c) in enumerate((("gate", 512, hidden), ("up", 512, hidden), ("down", hidden, 512)))}
        router = torch.from_numpy((rng.standard_normal((n_exp, hidden)) * 0.5).astype(np.float32)).cuda()
        mk = lambda n, r, c: device.Weights(raws[n], fo.Q4_K, r, c, n_mats=n_exp)
        layer = prefill.RoutedLayer(router, mk("gate", 512, hidden), mk("up", 512, hidden), mk("down", hidden, 512), k=k, mode=1)
        ep = parallel.ExpertParallelLayer(device, router, raws["gate"], raws["up"], raws["down"], fo.Q4_K, n_exp, hidden, 512, k)
        ref = prefill.run_device_routed_batch(layer, x).cpu().numpy()
        per = 64 // world
        got = ep.prefill(x[rank * per:(rank + 1) * per].contiguous()).cpu().numpy()
        out["ep_pre_equal"] = bool(np.array_equal(got, ref[rank * per:(rank + 1) * per]))
        out["ep_dec"] = rel_l2(ep.decode(x[0]).cpu().numpy(), prefill.run_device_routed(layer, x[0]).cpu().numpy())
        torch.cuda.synchronize()
        out["err"] = device.device_error()
        ret[rank] = out
    finally:
        dist.destroy_process_group()


def test_tp_and_ep_over_nccl_match_single_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, 29400 + os.getpid() % 500, ret), nprocs=2, join=True)
    for r in range(2):
        o = ret[r]
        assert o["err"] == 0
        assert o["tp_dec"] <= 1e-5 and o["tp_pre"] <= 1e-5, o
        assert o["ep_pre_equal"] and o["ep_dec"] <= 1e-6, o
