"""The shared-memory control channel: ordering, acknowledgements, error reporting, bounded waits.
Failures are made on the host: a follower that reports an error, one that never acknowledges, one that exits."""
import multiprocessing as mp
import time

import numpy as np
import pytest

from tinyllmforge_b200.engine import rpc


def _follower(name, rank, world, n_msgs, fail_at, out_q):
    ch = rpc.ShmChannel(name, world, rank, create=False, timeout_s=20)
    ch.hello()
    got = []
    try:
        for i in range(n_msgs):
            kind, data = ch.receive(timeout_s=20)
            if kind == rpc.KIND_EXIT:
                break
            if i == fail_at:
                ch.report_failure("boom at message %d" % i)
                return
            got.append(int(data.view(np.int32).sum()))
    finally:
        out_q.put((rank, got))
        ch.close()


def test_broadcast_in_order_to_two_followers():
    ctx = mp.get_context("spawn")
    name = rpc.unique_name("t")
    ch = rpc.ShmChannel(name, 3, 0, create=True, timeout_s=20)
    q = ctx.Queue()
    ps = [ctx.Process(target=_follower, args=(name, r, 3, 50, -1, q)) for r in (1, 2)]
    [p.start() for p in ps]
    try:
        ch.wait_hello()
        sums = []
        for i in range(50):
            payload = np.arange(i + 1, dtype=np.int32)
            sums.append(int(payload.sum()))
            ch.publish(rpc.KIND_STEP, payload)
        ch.drain()
        res = dict(q.get(timeout=20) for _ in ps)
        assert res[1] == sums and res[2] == sums
    finally:
        [p.join(10) for p in ps]
        ch.close()


def test_follower_failure_surfaces_on_rank0():
    ctx = mp.get_context("spawn")
    name = rpc.unique_name("t")
    ch = rpc.ShmChannel(name, 2, 0, create=True, timeout_s=20)
    q = ctx.Queue()
    p = ctx.Process(target=_follower, args=(name, 1, 2, 10, 2, q))
    p.start()
    try:
        ch.wait_hello()
        with pytest.raises(rpc.PeerFailed, match="boom at message 2"):
            for i in range(10):
                ch.publish(rpc.KIND_STEP, np.ones(4, dtype=np.int32))
            ch.drain()
    finally:
        p.join(10)
        ch.close()


def test_publish_times_out_when_nobody_acknowledges():
    name = rpc.unique_name("t")
    ch = rpc.ShmChannel(name, 2, 0, create=True, timeout_s=0.3)
    try:
        ch.publish(rpc.KIND_STEP, np.ones(4, dtype=np.int32))      # first message needs no earlier ack
        t0 = time.monotonic()
        with pytest.raises(rpc.ChannelTimeout):
            ch.publish(rpc.KIND_STEP, np.ones(4, dtype=np.int32))
        assert time.monotonic() - t0 < 5
    finally:
        ch.close()


def test_liveness_probe_beats_the_deadline():
    name = rpc.unique_name("t")
    ch = rpc.ShmChannel(name, 2, 0, create=True, timeout_s=60)

    def dead():
        raise rpc.PeerFailed("rank 1 exited with code 1")
    ch.liveness = dead
    try:
        ch.publish(rpc.KIND_STEP, None)
        t0 = time.monotonic()
        with pytest.raises(rpc.PeerFailed):
            ch.publish(rpc.KIND_STEP, None)
        assert time.monotonic() - t0 < 5
    finally:
        ch.close()


def test_oversized_message_rejected():
    name = rpc.unique_name("t")
    ch = rpc.ShmChannel(name, 1, 0, create=True, capacity=1024)
    try:
        with pytest.raises(ValueError):
            ch.publish(rpc.KIND_STEP, np.zeros(1000, dtype=np.int32))
    finally:
        ch.close()
