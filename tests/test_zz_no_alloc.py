"""The GEMM entry point that allocates nothing on the device (`fk_gemm_static`).

It exists for callers that cannot allocate device memory at the moment they
need a GEMM (inside a stream capture, in a serving loop that must not trigger
cudaMalloc's synchronisation, or on a fixed memory budget): its scratch is a
fixed block inside the library.  Here it is called through the C ABI twice in a
row and held to the ordinary entry point's output, and a shape too large for
the block must be refused with a clear error.  Collected last on purpose."""
import numpy as np
import pytest
import torch

from oracle import frink_oracle as fo
from tests.helpers import rel_l2, synth_acts, synth_weights

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kind", [fo.Q4_K, fo.Q8_0])
def test_gemm_static_matches_gemm_on_two_calls_in_a_row(kind):
    from frink_b200 import device
    rows, cols = 384, 2048
    raw = fo.encode(kind, synth_weights(rows, cols, 71))
    w = device.Weights(raw, kind, rows, cols)
    out = torch.empty((200, rows), dtype=torch.float32, device="cuda")
    for call, m in enumerate((200, 77)):   # the second call reuses the block with a different shape
        x = torch.from_numpy(synth_acts(m, cols, 72 + call)).cuda()
        want = device.gemm(w, x).cpu().numpy()
        out.fill_(float("nan"))
        got = device.gemm_static(w, x, out=out[:m]).cpu().numpy()
        torch.cuda.synchronize()
        assert device.device_error() == 0
        assert np.isfinite(got).all()
        assert rel_l2(got, want) <= 1e-3          # the tolerance of the GEMM tests ...
        assert np.array_equal(got, want)          # ... and in fact the same bits: same kernels, same inputs


def test_gemm_static_refuses_what_does_not_fit():
    from frink_b200 import _lib, device
    rows, cols = 128, 8192
    w = device.Weights(fo.encode(fo.Q8_0, synth_weights(rows, cols, 73)), fo.Q8_0, rows, cols)
    x = torch.zeros((1024, cols), device="cuda")
    out = torch.empty((1024, rows), device="cuda")
    with pytest.raises(_lib.Invalid, match="fixed block"):
        device.gemm_static(w, x, out=out)
