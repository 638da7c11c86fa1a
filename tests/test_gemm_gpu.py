"""Parity of the tcgen05 prefill GEMM and its grouped (per-expert) form against
the CPU oracle, through the C ABI.  Same bar as the GEMV: relative L2 <= 1e-3,
max-abs <= 2e-3 * |y|_inf against the f64 dequantize-then-dot of the q8_1-rounded
activations; and because GEMV and GEMM share one activation rule and exact
per-run integers, the two kernels must agree to f32 summation-order noise."""
import numpy as np
import pytest
import torch

from oracle import frink_oracle as fo
from tests.helpers import max_abs_over_inf, rel_l2, synth_acts, synth_weights

pytestmark = pytest.mark.gpu
REL_L2, MAX_ABS = 1e-3, 2e-3
KINDS = [fo.Q8_0, fo.Q4_K, fo.Q6_K, fo.MXFP4]


def _no_device_error():
    from frink_b200 import device
    torch.cuda.synchronize()
    assert device.device_error() == 0, "a bounded wait inside the GEMM gave up"


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("rows,cols,m", [(128, 256, 128), (256, 1024, 64), (200, 768, 100), (384, 3072, 512), (64, 2048, 9)])
def test_gemm_matches_oracle(kind, rows, cols, m):
    from frink_b200 import device
    raw = fo.encode(kind, synth_weights(rows, cols, 11 + rows))
    x = synth_acts(m, cols, 12 + m)
    w = device.Weights(raw, kind, rows, cols)
    out = torch.full((m, rows), float("nan"), device="cuda")
    device.gemm(w, torch.from_numpy(x).cuda(), out=out)
    _no_device_error()
    got = out.cpu().numpy()
    want = fo.matmul_f64(kind, raw, rows, cols, fo.q8_1_round(x))
    assert np.isfinite(got).all()
    assert rel_l2(got, want) <= REL_L2 and max_abs_over_inf(got, want) <= MAX_ABS, (rel_l2(got, want), max_abs_over_inf(got, want))
    # the GEMV of the same rows (batch <= 8) reads the same integers
    y = device.gemv(w, torch.from_numpy(x[:8]).cuda()).cpu().numpy()
    assert rel_l2(got[:8], y) <= 2e-6
    # deterministic
    again = device.gemm(w, torch.from_numpy(x).cuda()).cpu().numpy()
    assert np.array_equal(got, again)


def test_gemm_mxfp4_2880_columns():
    from frink_b200 import device
    rows, cols, m = 256, 2880, 130
    raw = fo.encode(fo.MXFP4, synth_weights(rows, cols, 5))
    x = synth_acts(m, cols, 6)
    w = device.Weights(raw, fo.MXFP4, rows, cols)
    got = device.gemm(w, torch.from_numpy(x).cuda()).cpu().numpy()
    _no_device_error()
    want = fo.matmul_f64(fo.MXFP4, raw, rows, cols, fo.q8_1_round(x))
    assert rel_l2(got, want) <= REL_L2 and max_abs_over_inf(got, want) <= MAX_ABS


@pytest.mark.parametrize("kind", [fo.Q4_K, fo.Q6_K, fo.MXFP4])
def test_grouped_gemm_matches_oracle(kind):
    from frink_b200 import device
    n_exp, rows, cols, batch, k = 8, 192, 1024 if kind != fo.MXFP4 else 960, 70, 2
    rng = np.random.default_rng(21)
    raws = [fo.encode(kind, synth_weights(rows, cols, 500 + e)) for e in range(n_exp)]
    w = device.Weights(np.concatenate(raws), kind, rows, cols, n_mats=n_exp)
    x = synth_acts(batch, cols, 22)
    ids = np.stack([rng.choice(n_exp - 1, k, replace=False) for _ in range(batch)]).astype(np.int32)  # expert 7 stays empty
    off, gather, pair_of = device.moe_permute(torch.from_numpy(ids).cuda(), n_exp)
    out = device.gemm_grouped(w, off, gather, torch.from_numpy(x).cuda(), batch * k)
    _no_device_error()
    got = out.cpu().numpy()
    off_h, gather_h = off.cpu().numpy(), gather.cpu().numpy()
    xq = fo.q8_1_round(x)
    for e in range(n_exp):
        lo, hi = off_h[e], off_h[e + 1]
        if hi == lo:
            continue
        want = fo.matmul_f64(kind, raws[e], rows, cols, xq[gather_h[lo:hi]])
        assert rel_l2(got[lo:hi], want) <= REL_L2 and max_abs_over_inf(got[lo:hi], want) <= MAX_ABS, e


def test_config2_shape_full_size():
    """A cell of the prefill sweep at full size: M = 512, 8192 x 3072, Q4_K."""
    from frink_b200 import device
    rows, cols, m = 8192, 3072, 512
    raw = fo.encode(fo.Q4_K, synth_weights(rows, cols, 0x5EED))
    x = synth_acts(m, cols, 0xAC7)
    w = device.Weights(raw, fo.Q4_K, rows, cols)
    got = device.gemm(w, torch.from_numpy(x).cuda()).cpu().numpy()
    _no_device_error()
    # the oracle on all 4.2 M outputs takes seconds with host threads
    want = fo.matmul_f64(fo.Q4_K, raw, rows, cols, fo.q8_1_round(x))
    assert rel_l2(got, want) <= REL_L2 and max_abs_over_inf(got, want) <= MAX_ABS
