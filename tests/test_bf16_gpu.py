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
