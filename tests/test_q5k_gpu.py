"""Q5_K (row f-2 of the scope: real Q4_K_M files carry it): the plain decode matvec and get_rows against the oracle,
which is pinned for this format by the reference's dequant golden and llama.cpp's encoder bytes
(tests/test_oracle_goldens.py)."""
import numpy as np
import pytest
import torch

from oracle import frink_oracle as fo
from tests.helpers import max_abs_over_inf, rel_l2, synth_acts, synth_weights

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,cols", [(64, 256), (96, 1024), (300, 3072)])
def test_per_run_integers_and_quantizer_are_exact(rows, cols):
    from frink_b200 import device
    raw = fo.encode(fo.Q5_K, synth_weights(rows, cols, 5))
    w = device.Weights(raw, fo.Q5_K, rows, cols)
    x = synth_acts(1, cols, 6)
    got = device.gemv_isums(w, torch.from_numpy(x[0]).cuda()).cpu().numpy()
    want = fo.matrix_isums(fo.Q5_K, raw, rows, cols, fo.quantize_q8_1(x[0]))
    assert np.array_equal(got, want)
    w.release()


@pytest.mark.parametrize("batch", [1, 2, 3, 4, 8])
def test_matvec_matches_the_dequant_dot_of_its_activations(batch):
    from frink_b200 import device
    rows, cols = 1000, 3072
    raw = fo.encode(fo.Q5_K, synth_weights(rows, cols, 7))
    w = device.Weights(raw, fo.Q5_K, rows, cols)
    x = synth_acts(batch, cols, 8)
    y = torch.full((batch, rows), float("nan"), device="cuda")
    device.gemv(w, torch.from_numpy(x).cuda(), out=y)
    got = y.cpu().numpy()
    want = fo.matmul_f64(fo.Q5_K, raw, rows, cols, fo.q8_1_round(x))
    assert rel_l2(got, want) <= 1e-3 and max_abs_over_inf(got, want) <= 2e-3
    # distance to frink's CPU integer path (Q8_K activations): two 8-bit activation quantizers apart
    cpu = fo.matmul_q8(fo.Q5_K, raw, rows, cols, x)
    assert rel_l2(got, cpu) <= 1.2e-2
    # run to run
    y2 = device.gemv(w, torch.from_numpy(x).cuda())
    assert torch.equal(y, y2) and device.device_error() == 0
    w.release()


def test_get_rows_host_surface_and_what_is_refused():
    from frink_b200 import _lib, device, gpu
    rows, cols = 128, 512
    raw = fo.encode(fo.Q5_K, synth_weights(rows, cols, 9))
    w = device.Weights(raw, fo.Q5_K, rows, cols)
    ids = torch.tensor([0, 5, 127, 64], dtype=torch.int32, device="cuda")
    got = device.get_rows(w, ids).cpu().numpy()
    want = fo.dequant(fo.Q5_K, raw).reshape(rows, cols)[[0, 5, 127, 64]]
    assert np.array_equal(got, want)
    x = synth_acts(20, cols, 10)
    xd = torch.from_numpy(x).cuda()
    # host-buffer matvec = the device matvec
    y_host = gpu.launch_q5_k_matvec(raw, x[0], rows, fo.row_bytes(fo.Q5_K, cols), cols // 256)
    assert np.array_equal(y_host, device.gemv(w, xd[:1]).cpu().numpy()[0])
    # more than 8 rows: no GEMM kernel -- the C call says UNSUPPORTED before it enqueues anything, the Python layer
    # takes batches of 8 through the matvec
    with pytest.raises(_lib.Unsupported):
        _lib.check(_lib.lib().fk_gemm(w._ctx, None, w.handle, 0, xd.data_ptr(), 20, torch.empty((20, rows), device="cuda").data_ptr()))
    big = device.gemm(w, xd).cpu().numpy()
    assert np.array_equal(big[:8], device.gemv(w, xd[:8]).cpu().numpy()) and np.array_equal(big[16:], device.gemv(w, xd[16:]).cpu().numpy())
    with pytest.raises(_lib.Unsupported):
        device.gemv_fused(w, xd[:1], accumulate=True, out=torch.zeros((1, rows), device="cuda"))
    assert device.device_error() == 0
    w.release()
