"""BF16 weights (gpt-oss attention projections; crates/frink-quant/src/lib.rs:232-250) and the gpt-oss bias add:
nothing is quantized, so the matvec is held to the f64 dot of the widened weights with the raw activations."""
import numpy as np
import pytest
import torch

from oracle import frink_oracle as fo
from tests.helpers import rel_l2, synth_acts, synth_weights

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,cols", [(512, 2880), (4096, 2880), (100, 64)])
@pytest.mark.parametrize("batch", [1, 3, 8])
def test_bf16_matvec(rows, cols, batch):
    from frink_b200 import device
    raw = fo.encode(fo.BF16, synth_weights(rows, cols, 3))
    w = device.Weights(raw, fo.BF16, rows, cols)
    x = synth_acts(batch, cols, 4)
    y = torch.full((batch, rows), float("nan"), device="cuda")
    device.gemv(w, torch.from_numpy(x).cuda(), out=y)
    want = fo.matmul_f64(fo.BF16, raw, rows, cols, x)
    assert rel_l2(y.cpu().numpy(), want) <= 1e-5
    assert torch.equal(y, device.gemv(w, torch.from_numpy(x).cuda()))
    w.release()


def test_bf16_get_rows_gemm_fallback_and_bias():
    from frink_b200 import _lib, device
    rows, cols = 256, 512
    raw = fo.encode(fo.BF16, synth_weights(rows, cols, 5))
    w = device.Weights(raw, fo.BF16, rows, cols)
    ids = torch.tensor([3, 0, 255], dtype=torch.int32, device="cuda")
    assert np.array_equal(device.get_rows(w, ids).cpu().numpy(), fo.dequant(fo.BF16, raw).reshape(rows, cols)[[3, 0, 255]])
    x = torch.from_numpy(synth_acts(20, cols, 6)).cuda()
    big = device.gemm(w, x)                  # no GEMM kernel: batches of 8 through the matvec
    assert torch.equal(big[8:16], device.gemv(w, x[8:16]))
    with pytest.raises(_lib.Unsupported):
        device.gemv_isums(w, x[0])
    # biases: one row for a projection, a row per expert slot for an indexed matvec
    y = torch.randn(6, rows, device="cuda")
    b1 = torch.randn(rows, device="cuda")
    want = y + b1
    assert torch.equal(device.add_bias_(y.clone(), b1), want)
    be = torch.randn(4, rows, device="cuda")
    slot_ids = torch.tensor([2, 0, 3, 3, 1, 0], dtype=torch.int32, device="cuda")
    assert torch.equal(device.add_bias_(y.clone(), be, slot_ids), y + be[slot_ids.long()])
    assert device.device_error() == 0
    w.release()


@pytest.mark.parametrize("batch", [1, 3, 8])
def test_bf16_matvec_with_norm_bias_and_accumulate(batch):
    """A gpt-oss projection as one launch: y (+)= W rmsnorm(x) + bias, against an f64 restatement; without the norm the
    biased launch is bit-identical to the plain matvec followed by the bias add."""
    from frink_b200 import _lib, device
    rows, cols, eps = 640, 2880, 1e-5
    raw = fo.encode(fo.BF16, synth_weights(rows, cols, 11))
    w = device.Weights(raw, fo.BF16, rows, cols)
    x = synth_acts(batch, cols, 12)
    rng = np.random.default_rng(13)
    nw = (1.0 + 0.1 * rng.standard_normal(cols)).astype(np.float32)
    bias = rng.standard_normal(rows).astype(np.float32)
    y0 = rng.standard_normal((batch, rows)).astype(np.float32)
    xd, nwd, bd = (torch.from_numpy(a).cuda() for a in (x, nw, bias))
    x64 = x.astype(np.float64)
    h = x64 / np.sqrt((x64 * x64).mean(axis=1, keepdims=True) + eps) * nw
    W = fo.dequant(fo.BF16, raw).reshape(rows, cols).astype(np.float64)
    want = h @ W.T + bias
    got = device.gemv_fused(w, xd, norm_weight=nwd, eps=eps, bias=bd)
    assert rel_l2(got.cpu().numpy(), want) <= 2e-6
    # add-into, reading x with a row stride (a column slice of a wider buffer)
    wide = torch.zeros((batch, cols + 64), device="cuda")
    wide[:, :cols] = xd
    acc = torch.from_numpy(y0).cuda()
    device.gemv_fused(w, wide[:, :cols], out=acc, norm_weight=nwd, eps=eps, bias=bd, accumulate=True)
    assert rel_l2(acc.cpu().numpy(), y0 + want) <= 2e-6
    # the norm alone (the output head of the decode step)
    assert rel_l2(device.gemv_fused(w, xd, norm_weight=nwd, eps=eps).cpu().numpy(), h @ W.T) <= 2e-6
    # no norm: the same bits as the separate launches
    assert torch.equal(device.gemv_fused(w, xd, bias=bd), device.add_bias_(device.gemv(w, xd), bd))
    with pytest.raises(_lib.Unsupported):
        device.gemv_fused(w, xd, glu_up=xd)
    assert device.device_error() == 0
    w.release()


@pytest.mark.parametrize("kind", ["mxfp4", "q4_k", "q8_0"])
def test_indexed_matvec_with_expert_bias_rows(kind):
    """fk_gemv_multi_biased: the bias row of every slot's expert added by the matvec itself -- the same bits as the
    indexed matvec followed by the bias launch, plain and with the gated activation in front."""
    from frink_b200 import device
    k_ = getattr(fo, kind.upper())
    E, rows, cols = 6, 320, 512
    raw = np.concatenate([fo.encode(k_, synth_weights(rows, cols, 20 + e)) for e in range(E)])
    w = device.Weights(raw, k_, rows, cols, n_mats=E)
    ids = torch.tensor([4, 0, 5, 4], dtype=torch.int32, device="cuda")
    bias = torch.randn(E, rows, device="cuda")
    x1 = torch.from_numpy(synth_acts(1, cols, 30)[0]).cuda()
    xs = torch.from_numpy(synth_acts(4, cols, 31)).cuda()
    up = torch.from_numpy(synth_acts(4, cols, 32)).cuda()
    assert torch.equal(device.gemv_multi(w, ids, x1, bias=bias), device.add_bias_(device.gemv_multi(w, ids, x1), bias, ids))
    assert torch.equal(device.gemv_multi(w, ids, xs, bias=bias), device.add_bias_(device.gemv_multi(w, ids, xs), bias, ids))
    for act in (0, 1):
        assert torch.equal(device.gemv_multi_glu(w, ids, xs, up, act, bias=bias),
                           device.add_bias_(device.gemv_multi_glu(w, ids, xs, up, act), bias, ids))
    # the single-matrix form on a block format (two rows: the plain and the biased launch then take the same kernel,
    # so the sums are added in the same order)
    b1 = torch.randn(rows, device="cuda")
    w1 = device.Weights(raw[:len(raw) // E], k_, rows, cols)
    assert torch.equal(device.gemv_fused(w1, xs[:2], bias=b1), device.add_bias_(device.gemv(w1, xs[:2]), b1))
    assert torch.allclose(device.gemv_fused(w1, xs, bias=b1), device.add_bias_(device.gemv(w1, xs), b1), rtol=1e-4, atol=1e-4)
    assert device.device_error() == 0
    w.release()
    w1.release()
