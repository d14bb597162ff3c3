"""Host-side model of the in-kernel tensor-parallel exchange protocol (csrc/include/tp_comm.cuh), run with CPU threads.

Every "rank" is a thread with, per site, a slot buffer [size] (slot r written by rank r), signal words [size]
(word r = pushes rank r completed) and a private epoch counter.  A layer alternates two sites (o_proj, down_proj) exactly as
the model does; threads sleep for random times between the phases so that ranks drift apart as far as the protocol allows.

Checked: (a) every rank reads, at every step, exactly the values all ranks produced for that step: a slot is never
overwritten while a peer still reads it, although no rank ever waits for its peers before producing; (b) every rank
computes the same sum; (c) a rank that never signals makes the others' bounded waits run out and report a status, not hang.
The failure is made on the host (a thread that withholds its flag); nothing here touches a GPU.
"""
import random
import threading
import time

STATUS_FLAG_TIMEOUT = 4


class Site:
    def __init__(self, size):
        self.slots = [[None] * size for _ in range(size)]       # [owner rank][source rank]
        self.signal = [[0] * size for _ in range(size)]         # [owner rank][source rank]
        self.epoch = [0] * size                                 # private, per rank


def produce(site, rank, size, value, rng, withhold=False):
    for p in range(size):                                       # push into every rank's copy (peer stores)
        site.slots[p][rank] = value
        if rng.random() < 0.3:
            time.sleep(rng.random() * 2e-4)
    site.epoch[rank] += 1
    if not withhold:
        for p in range(size):                                   # release: the data above is visible before the flag
            site.signal[p][rank] = site.epoch[rank]


def consume(site, rank, size, timeout_s, status):
    want = site.epoch[rank]
    t0 = time.perf_counter()
    for r in range(size):
        while site.signal[rank][r] - want < 0:                  # acquire
            if time.perf_counter() - t0 > timeout_s:
                status[rank] |= STATUS_FLAG_TIMEOUT
                return None
            time.sleep(1e-5)
    return list(site.slots[rank])                               # rank order: same result on every rank


def run_ranks(size, steps, timeout_s, silent_rank=None, silent_from=None, seed=0):
    sites = [Site(size), Site(size)]
    status = [0] * size
    seen = [[] for _ in range(size)]

    def rank_main(rank):
        rng = random.Random(seed * 100 + rank)
        for k in range(steps):
            site = sites[k & 1]
            withhold = rank == silent_rank and silent_from is not None and k >= silent_from
            time.sleep(rng.random() * 3e-4)
            produce(site, rank, size, (k, rank), rng, withhold)
            time.sleep(rng.random() * 3e-4)
            got = consume(site, rank, size, timeout_s, status)
            if got is None:
                return
            seen[rank].append(got)

    threads = [threading.Thread(target=rank_main, args=(r,)) for r in range(size)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=30)
    assert not any(t.is_alive() for t in threads), "a rank hung"
    return seen, status


def test_alternating_sites_never_lose_or_mix_data():
    for size in (2, 4, 8):
        seen, status = run_ranks(size, steps=60, timeout_s=5.0, seed=size)
        assert status == [0] * size
        for rank in range(size):
            assert len(seen[rank]) == 60
            for k, got in enumerate(seen[rank]):
                assert got == [(k, r) for r in range(size)], (size, rank, k, got)


def test_a_silent_rank_times_out_the_others_instead_of_hanging():
    seen, status = run_ranks(4, steps=20, timeout_s=0.75, silent_rank=2, silent_from=7, seed=3)
    for rank in range(4):
        assert status[rank] & STATUS_FLAG_TIMEOUT            # every wait ran out (rank 2 waits for itself too)
        assert len(seen[rank]) == 7                           # the steps before the silence completed everywhere
