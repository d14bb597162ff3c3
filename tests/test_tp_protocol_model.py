"""Host-side model of the in-kernel tensor-parallel exchange protocol (csrc/include/tp_comm.cuh), run with CPU threads.

Every "rank" is a thread.  Per site a rank owns a partial buffer (its own GEMM output, written locally, READ BY PEERS),
signal words [size] (word r = productions rank r completed) and a private epoch counter; all ranks share the layout of
one broadcast buffer `y` per rank (row r written by rank r into every rank's copy) with its own "gather" site.
A layer alternates two sites (o_proj, down_proj) exactly as the model does, and each exchange is either

  one-shot   produce locally, signal all; every rank waits for all signals and reads every rank's partial, or
  two-shot   produce locally, signal all; rank r waits for all signals, reduces only "row" r, writes it into every
             rank's `y`, signals at the gather site and waits until every rank has done so (wanted epoch = the
             value read before arriving + 1, as in the kernel), then reads its whole `y`.

Threads sleep for random times between the phases so that ranks drift apart as far as the protocol allows.

Checked: (a) every rank reads, at every step, exactly the values all ranks produced for that step: a partial buffer is
never overwritten while a peer still reads it, and `y` is never overwritten while its owner still reads it, although
no rank ever waits for its peers before producing; (b) every rank computes the same result; (c) a rank that is late
but within the limit delays the others and nothing else; (d) a rank that never signals makes the others' bounded
waits run out and report a status, not hang.  Failures are made on the host (a thread that sleeps or withholds its
flag); nothing here touches a GPU.
"""
import random
import threading
import time

STATUS_FLAG_TIMEOUT = 2


class Site:
    def __init__(self, size):
        self.part = [None] * size                               # [owner rank]: that rank's partial (peers read it)
        self.signal = [[0] * size for _ in range(size)]         # [owner rank][source rank]
        self.epoch = [0] * size                                 # private, per rank


class Gather(Site):
    def __init__(self, size):
        super().__init__(size)
        self.y = [[None] * size for _ in range(size)]           # [owner rank][row]: row r is written by rank r


def produce(site, rank, size, value, withhold=False):
    site.part[rank] = value                                     # a local store
    site.epoch[rank] += 1
    if not withhold:
        for p in range(size):                                   # release: the data above is visible before the flag
            site.signal[p][rank] = site.epoch[rank]


def wait_all(site, rank, size, want, timeout_s, status):
    t0 = time.perf_counter()
    for r in range(size):
        while site.signal[rank][r] - want < 0:                  # acquire
            if time.perf_counter() - t0 > timeout_s:
                status[rank] |= STATUS_FLAG_TIMEOUT
                return False
            time.sleep(1e-5)
    return True


def consume_one_shot(site, rank, size, timeout_s, status, rng):
    if not wait_all(site, rank, size, site.epoch[rank], timeout_s, status):
        return None
    got = []
    for r in range(size):                                       # pull every rank's partial (rank order)
        got.append(site.part[r])
        if rng.random() < 0.3:
            time.sleep(rng.random() * 2e-4)
    return got


def consume_two_shot(site, gather, rank, size, timeout_s, status, rng):
    want_rows = gather.epoch[rank] + 1                          # read before arriving
    if not wait_all(site, rank, size, site.epoch[rank], timeout_s, status):
        return None
    row = tuple(site.part[r] for r in range(size))              # "reduce" row `rank`: needs every rank's partial
    for p in range(size):                                       # broadcast it into every rank's y
        gather.y[p][rank] = row
        if rng.random() < 0.3:
            time.sleep(rng.random() * 2e-4)
    gather.epoch[rank] += 1
    for p in range(size):
        gather.signal[p][rank] = gather.epoch[rank]
    if not wait_all(gather, rank, size, want_rows, timeout_s, status):
        return None
    rows = list(gather.y[rank])
    assert all(r == rows[0] for r in rows), ("rows of one exchange differ", rank, rows)
    return list(rows[0])


def run_ranks(size, steps, timeout_s, silent_rank=None, silent_from=None, late_rank=None, late_at=None, late_s=0.0, seed=0):
    sites = [Site(size), Site(size)]
    gather = Gather(size)
    status = [0] * size
    seen = [[] for _ in range(size)]
    kinds = [random.Random(seed).random() < 0.5 for _ in range(steps)]      # the same choice on every rank

    def rank_main(rank):
        rng = random.Random(seed * 100 + rank)
        for k in range(steps):
            site = sites[k & 1]
            withhold = rank == silent_rank and silent_from is not None and k >= silent_from
            time.sleep(rng.random() * 3e-4)
            if rank == late_rank and k == late_at:
                time.sleep(late_s)
            produce(site, rank, size, (k, rank), withhold)
            time.sleep(rng.random() * 3e-4)
            if kinds[k]:
                got = consume_two_shot(site, gather, rank, size, timeout_s, status, rng)
            else:
                got = consume_one_shot(site, rank, size, timeout_s, status, rng)
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


def test_a_late_rank_within_the_limit_only_delays_the_others():
    seen, status = run_ranks(4, steps=20, timeout_s=5.0, late_rank=1, late_at=9, late_s=0.4, seed=5)
    assert status == [0] * 4
    for rank in range(4):
        assert [got for got in seen[rank]] == [[(k, r) for r in range(4)] for k in range(20)]


def test_a_silent_rank_times_out_the_others_instead_of_hanging():
    seen, status = run_ranks(4, steps=20, timeout_s=0.75, silent_rank=2, silent_from=7, seed=3)
    for rank in range(4):
        assert status[rank] & STATUS_FLAG_TIMEOUT            # every wait ran out (rank 2 waits for itself too)
        assert len(seen[rank]) == 7                           # the steps before the silence completed everywhere
