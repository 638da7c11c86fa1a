"""The peer-memory all-reduce on ONE GPU: the single-rank case, and the bounded wait -- an
all-reduce of a two-rank communicator whose peer never shows up gives up after its time limit,
raises the device error word and leaves the context usable (no rank exits, nothing hangs)."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_single_rank_allreduce_is_a_copy():
    from frink_b200 import device
    from frink_b200._lib import check, lib
    ctx = device.context()
    h, handle = C.c_void_p(), (C.c_uint8 * 64)()
    check(lib().fk_comm_create(ctx, 1 << 20, 0, 1, handle, C.byref(h)))
    x = torch.randn(3072, device="cuda")
    y = torch.full_like(x, 2.0)
    s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    check(lib().fk_allreduce(ctx, s, h, 0, 3072, C.c_void_p(x.data_ptr()), C.c_void_p(y.data_ptr()), 3072, 1, 0))
    torch.cuda.synchronize()
    assert torch.equal(y, x + 2.0) and device.device_error() == 0
    check(lib().fk_comm_destroy(h))


def test_a_peer_that_never_arrives_times_out_with_an_error_word():
    from frink_b200 import device
    from frink_b200._lib import check, lib
    ctx = device.context()
    assert device.device_error() == 0
    a, b, handle = C.c_void_p(), C.c_void_p(), (C.c_uint8 * 64)()
    check(lib().fk_comm_create(ctx, 1 << 20, 0, 2, handle, C.byref(a)))     # "rank 0" of two
    check(lib().fk_comm_create(ctx, 1 << 20, 1, 2, handle, C.byref(b)))     # the arena that stands for rank 1: nobody runs it
    arena_b = C.c_void_p()
    check(lib().fk_comm_arena(b, C.byref(arena_b), None))
    peers = (C.c_void_p * 2)(None, arena_b)
    check(lib().fk_comm_connect_local(a, peers))
    x = torch.randn(1024, device="cuda")
    y = torch.empty_like(x)
    s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    check(lib().fk_allreduce(ctx, s, a, 0, 1024, C.c_void_p(x.data_ptr()), C.c_void_p(y.data_ptr()), 1024, 0, 3000))   # 3 ms limit
    e1.record()
    torch.cuda.synchronize()
    assert 2.0 <= e0.elapsed_time(e1) <= 200.0            # it waited its limit, not forever
    # the host-buffer surface reads the word before it returns: the next such call fails with it instead of handing back
    # numbers that a broken launch may have produced, and clears it
    from frink_b200 import gpu
    from oracle import frink_oracle as fo
    from tests.helpers import synth_weights
    raw4 = fo.encode(fo.Q4_K, synth_weights(64, 256, 2))
    xh = np.random.default_rng(1).standard_normal(256).astype(np.float32)
    with pytest.raises(gpu.Launch, match="60"):
        gpu.launch_q4_k_matvec(raw4, xh, 64, 144, 1)
    assert device.device_error() == 0
    assert np.isfinite(gpu.launch_q4_k_matvec(raw4, xh, 64, 144, 1)).all()
    # the device-pointer calls leave the word to the caller
    check(lib().fk_allreduce(ctx, s, a, 0, 1024, C.c_void_p(x.data_ptr()), C.c_void_p(y.data_ptr()), 1024, 0, 3000))
    torch.cuda.synchronize()
    assert device.device_error() == 60                    # read and reset
    assert device.device_error() == 0
    # the context is as usable as before
    from oracle import frink_oracle as fo
    from tests.helpers import synth_weights
    raw = fo.encode(fo.Q8_0, synth_weights(64, 256, 1))
    w = device.Weights(raw, fo.Q8_0, 64, 256)
    xv = np.random.default_rng(0).standard_normal(256).astype(np.float32)
    got = device.gemv(w, torch.from_numpy(xv).cuda()).cpu().numpy()
    want = fo.matmul_f64(fo.Q8_0, raw, 64, 256, fo.q8_1_round(xv))[0]
    assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 1e-3
    check(lib().fk_comm_destroy(a))
    check(lib().fk_comm_destroy(b))


class _Raw:
    """Device memory at `ptr` as something torch can wrap."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


@pytest.mark.parametrize("batch", [1, 4])
def test_matvec_with_the_allreduce_in_its_epilogue_adds_what_the_peer_delivered(batch):
    """One GPU stands for rank 0 of two.  The peer's records ({value, all-reduce number} per element, the
    layout of the channel) are written into rank 0's slots by the test before the launch, as a peer's
    stores would have; the matvec then must return its own rows plus those values -- twice, so both
    generations of slots are used -- and a third launch, whose records nobody delivers, must give up
    with the error word."""
    from frink_b200 import device
    from frink_b200._lib import check, lib
    from oracle import frink_oracle as fo
    from tests.helpers import synth_weights
    ctx = device.context()
    assert device.device_error() == 0
    rows, cols, n_max, arena = 512, 1024, 8 * 512, 1 << 20
    a, b, handle = C.c_void_p(), C.c_void_p(), (C.c_uint8 * 64)()
    check(lib().fk_comm_create(ctx, arena, 0, 2, handle, C.byref(a)))
    check(lib().fk_comm_create(ctx, arena, 1, 2, handle, C.byref(b)))
    pa, pb = C.c_void_p(), C.c_void_p()
    check(lib().fk_comm_arena(a, C.byref(pa), None))
    check(lib().fk_comm_arena(b, C.byref(pb), None))
    check(lib().fk_comm_connect_local(a, (C.c_void_p * 2)(None, pb)))
    mem = torch.as_tensor(_Raw(pa.value, arena), device="cuda").view(torch.int32)
    slots = mem[:2 * 2 * n_max * 2].view(2, 2, n_max, 2)          # [generation][from][element][value bits, number]
    raw = fo.encode(fo.Q4_K, synth_weights(rows, cols, 3))
    w = device.Weights(raw, fo.Q4_K, rows, cols)
    rng = np.random.default_rng(5)
    s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for t in (1, 2, 3):
        x = torch.from_numpy(rng.standard_normal((batch, cols)).astype(np.float32)).cuda()
        peer = torch.from_numpy(rng.standard_normal((batch, rows)).astype(np.float32)).cuda()
        base = torch.from_numpy(rng.standard_normal((batch, rows)).astype(np.float32)).cuda()
        if t < 3:
            slots[t & 1, 1, :batch * rows, 0] = peer.view(torch.int32).ravel()
            slots[t & 1, 1, :batch * rows, 1] = t
        y = base.clone()
        check(lib().fk_gemv_fused_allreduce(ctx, s, w.handle, 0, C.c_void_p(x.data_ptr()), cols, batch, C.c_void_p(y.data_ptr()), None, 0.0, None, 0, 1,
                                            a, 0, n_max, 3000))
        torch.cuda.synchronize()
        if t < 3:
            assert device.device_error() == 0
            want = (device.gemv(w, x) + peer) + base
            assert torch.allclose(y, want, rtol=1e-5, atol=1e-5)       # `want` may come from another kernel's summation order
        else:
            assert device.device_error() == 60
    # what rank 0 sent: its own rows, numbered, in the peer's arena
    memb = torch.as_tensor(_Raw(pb.value, arena), device="cuda").view(torch.int32)
    sent = memb[:2 * 2 * n_max * 2].view(2, 2, n_max, 2)[1, 0, :batch * rows]
    assert bool((sent[:, 1] == 3).all())
    assert torch.allclose(sent[:, 0].view(torch.float32).view(batch, rows), device.gemv(w, x), rtol=1e-5, atol=1e-5)
    w.release()
    check(lib().fk_comm_destroy(a))
    check(lib().fk_comm_destroy(b))
