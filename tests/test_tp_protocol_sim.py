"""Host-side simulation of the one-shot peer-memory exchange (csrc/model.cu, tp_exchange.h): ranks are
threads, peer memory is shared numpy arrays.  It checks the protocol's invariants without a GPU:
two parity sets of slots are enough because a rank can run at most one exchange ahead, the fixed
rank-order sum is bit-identical on every rank, and a rank that stops arriving makes the others give up
after a bounded number of polls with a status instead of hanging (the failure is injected on the host)."""
import threading
import time

import numpy as np

MAX_RANKS = 8
SLOT = 64  # floats per slot in the simulation (the library uses 8192)


class Area:
    """One rank's exchange area: [parity][source rank][SLOT] floats, then flags [parity][source rank]."""

    def __init__(self):
        self.slots = np.zeros((2, MAX_RANKS, SLOT), np.float32)
        self.flags = np.zeros((2, MAX_RANKS), np.uint32)


def reached(flag, epoch) -> bool:
    """(int)(flag - epoch) >= 0 in 32-bit arithmetic, as the kernel compares epochs"""
    return ((int(flag) - int(epoch)) & 0xFFFFFFFF) < 0x80000000


def exchange(rank, n, areas, epoch, partial, poll_limit, delay=0.0):
    """One exchange as the kernel does it; returns (sum or None, status)."""
    par = epoch & 1
    for r in range(n):                       # 1. push this rank's vector into every rank's area
        areas[r].slots[par, rank, :] = partial
    if delay:
        time.sleep(delay)
    for r in range(n):                       # flag after the data (the kernel fences in between)
        areas[r].flags[par, rank] = epoch
    for src in range(n):                     # 2. bounded poll of all flags in this rank's own area
        for _ in range(poll_limit):
            if reached(areas[rank].flags[par, src], epoch):
                break
            time.sleep(0)
        else:
            return None, "timeout"
    acc = np.zeros(SLOT, np.float32)         # 3. sum in rank order
    for src in range(n):
        acc = acc + areas[rank].slots[par, src, :]
    return acc, "ok"


def _run(n, epochs, slow_rank=None, dead_after=None, poll_limit=200000):
    areas = [Area() for _ in range(n)]
    rng = np.random.default_rng(7)
    data = rng.standard_normal((epochs + 1, n, SLOT)).astype(np.float32)
    results = [[None] * (epochs + 1) for _ in range(n)]
    status = ["ok"] * n

    def worker(rank):
        for e in range(1, epochs + 1):
            if dead_after is not None and rank == dead_after[0] and e > dead_after[1]:
                return                        # the rank leaves between exchanges and never arrives again
            delay = 0.002 if rank == slow_rank and e % 3 == 0 else 0.0
            out, st = exchange(rank, n, areas, e, data[e, rank], poll_limit, delay)
            if st != "ok":
                status[rank] = st
                return
            results[rank][e] = out

    threads = [threading.Thread(target=worker, args=(r,)) for r in range(n)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=60)
    assert not any(t.is_alive() for t in threads), "a simulated rank hung"
    return data, results, status


def test_sums_are_identical_on_every_rank_and_two_parities_suffice():
    for n in (2, 4, 8):
        data, results, status = _run(n, epochs=40, slow_rank=n - 1)
        assert status == ["ok"] * n
        for e in range(1, 41):
            exp = np.zeros(SLOT, np.float32)
            for src in range(n):
                exp = exp + data[e, src]
            for r in range(n):
                assert np.array_equal(results[r][e].view(np.uint32), exp.view(np.uint32)), (n, e, r)


def test_a_rank_that_leaves_makes_the_others_give_up_with_a_status():
    data, results, status = _run(4, epochs=10, dead_after=(2, 4), poll_limit=2000)
    assert status[2] == "ok"                       # it simply stopped
    assert all(status[r] == "timeout" for r in (0, 1, 3))
    for r in (0, 1, 3):                            # everything before the failure completed, bit-identical
        for e in range(1, 5):
            assert results[r][e] is not None and np.array_equal(results[r][e], results[0][e])
        assert results[r][5] is None


def test_epoch_comparison_survives_wraparound():
    a = Area()
    a.flags[1, 0] = np.uint32(0xFFFFFFFE)          # a flag from just before the counter wrapped
    assert not reached(a.flags[1, 0], 3)           # is older than epoch 3
    a.flags[1, 0] = np.uint32(5)
    assert reached(a.flags[1, 0], 3)
