"""A host model of the peer-memory all-reduce's record protocol (frink_b200/csrc/fk_comm.cuh),
run as threads that interleave freely: every "rank" owns slots[2][world][n] of packed
{value bits, count} 64-bit records and a local sent[n]; an element's value goes to every other
rank's slot (generation = count & 1, one atomic 64-bit store) and the local slots are polled until
their count matches.  The model checks what the device code relies on: two generations are enough
whatever the interleaving, the sum is the same on every rank, ranks may run ahead of one another by
at most one all-reduce, all-reduces of different lengths may share a channel, and a rank whose
peer never shows up gives up after its limit with an error instead of spinning for ever."""
import random
import threading
import time

import numpy as np
import pytest


class Channel:
    def __init__(self, world, n):
        self.world, self.n = world, n
        # slots[rank][generation, from, element] as one uint64 per record (a numpy element store is one atomic write)
        self.slots = [np.zeros((2, world, n), np.uint64) for _ in range(world)]
        self.sent = [np.zeros(n, np.uint32) for _ in range(world)]


def pack(v, t):
    return np.uint64((int(np.float32(v).view(np.uint32)) << 32) | int(t))


def send(ch, rank, i, v):
    t = int(ch.sent[rank][i]) + 1
    ch.sent[rank][i] = t
    for q in range(ch.world):
        if q != rank:
            ch.slots[q][t & 1, rank, i] = pack(v, t)
    return t


def recv(ch, rank, i, t, v, limit):
    acc = np.float32(0.0)
    for q in range(ch.world):
        if q == rank:
            acc = np.float32(acc + np.float32(v))
            continue
        spins = 0
        while True:
            rec = int(ch.slots[rank][t & 1, q, i])
            if rec & 0xFFFFFFFF == t:
                break
            spins += 1
            if spins > limit:
                return None                       # the device raises error word 60 here
            if spins % 64 == 0:
                time.sleep(0)
        acc = np.float32(acc + np.uint32(rec >> 32).view(np.float32))
    return acc


def all_reduce(ch, rank, x, n, limit=2_000_000, jitter=None):
    """The standalone kernel: all sends first, then all receives."""
    ts = [send(ch, rank, i, x[i]) for i in range(n)]
    if jitter:
        time.sleep(jitter())
    out = np.empty(n, np.float32)
    for i in range(n):
        r = recv(ch, rank, i, ts[i], x[i], limit)
        if r is None:
            return None
        out[i] = r
    return out


@pytest.mark.parametrize("world", [2, 4])
def test_many_all_reduces_on_one_channel_under_free_interleaving(world):
    n_max, rounds = 24, 60
    ch = Channel(world, n_max)
    rng = np.random.default_rng(3)
    lens = rng.integers(1, n_max + 1, rounds)                 # different lengths share the channel
    data = rng.standard_normal((rounds, world, n_max)).astype(np.float32)
    results = [[None] * rounds for _ in range(world)]
    ahead = []

    def worker(rank):
        rnd = random.Random(rank)
        for r in range(rounds):
            n = int(lens[r])
            results[rank][r] = all_reduce(ch, rank, data[r, rank], n, jitter=lambda: rnd.random() * 2e-4)
            ahead.append(max(int(ch.sent[rank][0]) - int(ch.sent[q][0]) for q in range(world)))

    th = [threading.Thread(target=worker, args=(r,)) for r in range(world)]
    for t in th:
        t.start()
    for t in th:
        t.join(120)
    assert not any(t.is_alive() for t in th)
    for r in range(rounds):
        n = int(lens[r])
        want = np.zeros(n, np.float32)
        for q in range(world):                                 # rank order, f32
            want = (want + data[r, q, :n]).astype(np.float32)
        for rank in range(world):
            assert results[rank][r] is not None
            assert np.array_equal(results[rank][r], want), (r, rank)     # the same bits on every rank
    assert max(ahead) <= 1                                      # nobody finishes two all-reduces ahead of a peer


def test_a_peer_that_never_arrives_ends_the_wait_with_an_error():
    ch = Channel(2, 8)
    x = np.ones(8, np.float32)
    t0 = time.time()
    assert all_reduce(ch, 0, x, 8, limit=2000) is None
    assert time.time() - t0 < 5.0
    # what it sent is in the peer's slots, numbered 1, in generation 1
    assert all(int(ch.slots[1][1, 0, i]) & 0xFFFFFFFF == 1 for i in range(8))
    # the late peer then finds rank 0's values and completes its own all-reduce
    got = all_reduce(ch, 1, 2 * x, 8, limit=2000)
    assert got is not None and np.array_equal(got, 3 * x)
