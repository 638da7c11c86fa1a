"""The Q8_K-activation prefill GEMM (Q4_K weights) against frink's CPU integer path restated in
the oracle (`quantize_activations_q8_k` + `dot_q4_k_q8`, crates/frink-quant/src/act_quant.rs:69-104,
src/lib.rs:822-869): the per-super-block integers are exact, the f32 results agree with the CPU
path to summation order (relative L2 <= 1e-3, max-abs <= 2e-3 * |y|_inf), through the C ABI."""
import numpy as np
import pytest
import torch

from oracle import frink_oracle as fo
from tests.helpers import max_abs_over_inf, rel_l2, synth_acts, synth_weights

pytestmark = pytest.mark.gpu
REL_L2, MAX_ABS = 1e-3, 2e-3


def _no_device_error():
    from frink_b200 import device
    torch.cuda.synchronize()
    assert device.device_error() == 0, "a bounded wait inside the GEMM gave up"


@pytest.mark.parametrize("rows,cols,m", [(128, 256, 128), (200, 1024, 37), (384, 3072, 300)])
def test_integers_are_the_cpu_vec_dot_integers(rows, cols, m):
    from frink_b200 import device
    raw = fo.encode(fo.Q4_K, synth_weights(rows, cols, 31 + rows))
    x = synth_acts(m, cols, 32 + m)
    w = device.Weights(raw, fo.Q4_K, rows, cols)
    out, isums = device.gemm_q8k_isums(w, torch.from_numpy(x).cuda())
    _no_device_error()
    got = isums.cpu().numpy()
    for t in range(0, m, max(1, m // 16)):
        want = fo.matrix_isums_q4k_q8k(raw, rows, cols, x[t])
        assert np.array_equal(got[t], want), f"token {t}"
    cpu = fo.matmul_q8(fo.Q4_K, raw, rows, cols, x, threads=fo.host_threads())
    assert rel_l2(out.cpu().numpy(), cpu) <= REL_L2 and max_abs_over_inf(out.cpu().numpy(), cpu) <= MAX_ABS


@pytest.mark.parametrize("rows,cols,m", [(256, 512, 1), (130, 768, 129), (3072, 3072, 512), (8192, 3072, 512), (3072, 8192, 512)])
def test_matches_the_cpu_batched_path(rows, cols, m):
    from frink_b200 import device
    raw = fo.encode(fo.Q4_K, synth_weights(rows, cols, 41 + rows))
    x = synth_acts(m, cols, 42 + m)
    w = device.Weights(raw, fo.Q4_K, rows, cols)
    out = torch.full((m, rows), float("nan"), device="cuda")      # every element must be written
    device.gemm_q8k(w, torch.from_numpy(x).cuda(), out=out)
    _no_device_error()
    got = out.cpu().numpy()
    assert np.isfinite(got).all()
    cpu = fo.matmul_q8(fo.Q4_K, raw, rows, cols, x, threads=fo.host_threads())
    assert rel_l2(got, cpu) <= REL_L2 and max_abs_over_inf(got, cpu) <= MAX_ABS, (rel_l2(got, cpu), max_abs_over_inf(got, cpu))
    assert np.array_equal(got, device.gemm_q8k(w, torch.from_numpy(x).cuda()).cpu().numpy())   # deterministic


def test_other_kinds_are_refused():
    from frink_b200 import _lib, device
    raw = fo.encode(fo.Q8_0, synth_weights(64, 256, 1))
    w = device.Weights(raw, fo.Q8_0, 64, 256)
    with pytest.raises(_lib.Unsupported):
        device.gemm_q8k(w, torch.zeros((4, 256), device="cuda"))
