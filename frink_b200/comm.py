"""The peer-memory all-reduce of the C ABI (`fk_comm_*`, `fk_allreduce`) for one process per GPU
of one box: `Comm` creates this rank's arena, swaps the CUDA IPC handles through
`torch.distributed`, maps the peers, and hands out channels (the same offsets on every rank, so
every rank must ask for the same channels in the same order).

The reference is single-device; nothing here mirrors reference code."""
import ctypes as C

import torch
import torch.distributed as dist

from ._lib import check, lib
from .device import _ptr, _stream, context


class Comm:
    def __init__(self, group=None, arena_bytes=256 << 20, timeout_us=0):
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.timeout_us = int(timeout_us)
        self._ctx = context()
        self._h = C.c_void_p()
        handle = (C.c_uint8 * 64)()
        check(lib().fk_comm_create(self._ctx, arena_bytes, self.rank, self.world, handle, C.byref(self._h)))
        mine = torch.tensor(list(handle), dtype=torch.uint8, device="cuda")
        allh = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(allh, mine, group=group)
        flat = bytes(torch.stack(allh).cpu().numpy().tobytes())
        self._handles = (C.c_uint8 * (64 * self.world)).from_buffer_copy(flat)
        check(lib().fk_comm_connect(self._h, self._handles))
        dist.barrier(group=group)       # every arena is mapped everywhere before anyone stores into a peer
        self.arena_bytes, self._next = arena_bytes, 0

    def channel(self, n_max):
        """A channel for all-reduces of up to n_max floats: (offset, n_max)."""
        n_max = int(n_max)
        size = (lib().fk_comm_channel_bytes(self.world, n_max) + 255) & ~255
        off = self._next
        if off + size > self.arena_bytes:
            raise MemoryError(f"the all-reduce arena of {self.arena_bytes} bytes is full")
        self._next += size
        return off, n_max

    def all_reduce(self, channel, src, dst=None, accumulate=False):
        """dst (default: src, in place) = (dst if accumulate else 0) + sum over ranks of src."""
        off, n_max = channel
        assert src.is_cuda and src.dtype == torch.float32 and src.is_contiguous()
        dst = src if dst is None else dst
        check(lib().fk_allreduce(self._ctx, _stream(), self._h, off, n_max, _ptr(src), _ptr(dst), src.numel(), int(bool(accumulate)), self.timeout_us))
        return dst

    def close(self):
        if self._h:
            check(lib().fk_comm_destroy(self._h))
            self._h = C.c_void_p()
