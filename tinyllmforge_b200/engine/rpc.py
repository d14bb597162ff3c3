"""Control plane between rank 0 and the other tensor-parallel ranks: a sequence-numbered
shared-memory broadcast channel with bounded waits.

Parity: tinyvllm/engine/model_runner.py:48-60,80-106 (a 1 MiB ``SharedMemory`` segment named
"tinyvllm", a pickled ``[method, *args]`` with a length prefix, one ``multiprocessing.Event`` per
worker, no reply and no error channel, waits that never time out).

Here:
  * the segment name is unique per engine, and the creator unlinks it on close, so two engines on
    one host do not collide and a crashed run does not poison the next one;
  * messages are raw bytes (the packed step buffer), not pickled object graphs;
  * rank 0 publishes message ``n`` only after every follower acknowledged ``n - 1``; followers
    acknowledge after copying the payload out, and report failure through a status word plus a text
    area, so rank 0 can raise a clean error instead of hanging in the next collective;
  * every wait has a deadline and calls a liveness probe while it waits.

Segment layout (little-endian int64 words, then bytes):
    [0] seq   [1] kind   [2] nbytes   [3] pid of the creator (rank 0)
    [4 + r]   ack word of follower r (r = 1..world-1)  = last seq it consumed
    [16 + r]  status word of follower r (0 ok, 1 failed)
    [24 + r]  pid of follower r once it attached
    [32...]   64 words of error text (UTF-8), then the payload.
"""
from __future__ import annotations

import os
import time
import uuid
from multiprocessing import shared_memory

import numpy as np

KIND_STEP, KIND_EXIT, KIND_PING, KIND_CALL = 1, 2, 3, 4
_WORDS_HDR = 32
_ERR_BYTES = 512
_PAYLOAD_OFF = _WORDS_HDR * 8 + _ERR_BYTES


class ChannelTimeout(RuntimeError):
    pass


class PeerFailed(RuntimeError):
    pass


def unique_name(prefix: str = "tlf") -> str:
    return f"{prefix}_{os.getpid()}_{uuid.uuid4().hex[:10]}"


class ShmChannel:
    def __init__(self, name: str, world_size: int, rank: int, create: bool, capacity: int = 8 << 20,
                 timeout_s: float = 120.0):
        assert world_size <= 8       # status words [16 + r] and pid words [24 + r] must not overlap
        self.name, self.world_size, self.rank, self.timeout_s = name, world_size, rank, timeout_s
        self.owner = create
        if create:
            self.shm = shared_memory.SharedMemory(name=name, create=True, size=_PAYLOAD_OFF + capacity)
            self.shm.buf[:_PAYLOAD_OFF] = bytes(_PAYLOAD_OFF)
            np.ndarray((_WORDS_HDR,), dtype=np.int64, buffer=self.shm.buf)[3] = os.getpid()
        else:
            self.shm = shared_memory.SharedMemory(name=name)
            # Only the creator may unlink.  A process started by the creator through multiprocessing shares
            # its resource tracker (nothing to do); an independently launched rank has its own tracker,
            # which would unlink the segment when that rank exits, so take the segment off its list.
            import multiprocessing
            if multiprocessing.parent_process() is None:
                try:
                    from multiprocessing import resource_tracker
                    resource_tracker.unregister(self.shm._name, "shared_memory")
                except Exception:
                    pass
        self.capacity = self.shm.size - _PAYLOAD_OFF
        self.words = np.ndarray((_WORDS_HDR,), dtype=np.int64, buffer=self.shm.buf, offset=0)
        self.payload = np.ndarray((self.capacity,), dtype=np.uint8, buffer=self.shm.buf, offset=_PAYLOAD_OFF)
        self.seq = 0
        # callable raising if a peer died. Rank 0 installs a probe of its child processes; a follower
        # probes the creator's pid, so it may wait for work without a deadline yet never outlive rank 0.
        self.liveness = None if create else self._owner_alive

    def _owner_alive(self):
        pid = int(self.words[3])
        try:
            os.kill(pid, 0)
        except ProcessLookupError:
            raise PeerFailed(f"rank 0 (pid {pid}) is gone") from None
        except PermissionError:
            pass

    # ------------------------------------------------------------------ waiting
    def _wait(self, cond, what: str, timeout_s: float | None = None):
        deadline = time.monotonic() + (self.timeout_s if timeout_s is None else timeout_s)
        spins = 0
        while not cond():
            spins += 1
            if spins < 2000:
                continue
            if spins % 64 == 0:
                if self.liveness is not None:
                    self.liveness()
                if time.monotonic() > deadline:
                    raise ChannelTimeout(f"rank {self.rank}: timed out waiting for {what}")
            time.sleep(0 if spins < 20000 else 0.0002)

    # ------------------------------------------------------------------ rank 0
    def _check_followers(self):
        for r in range(1, self.world_size):
            if self.words[16 + r] != 0:
                raise PeerFailed(f"rank {r} reported: {self.read_error()}")

    def publish(self, kind: int, data: np.ndarray | bytes | None = None) -> None:
        """Send one message to every follower (rank 0 only)."""
        assert self.rank == 0
        w = self.words

        def all_acked():
            self._check_followers()
            return all(w[4 + r] >= self.seq for r in range(1, self.world_size))

        self._wait(all_acked, f"acknowledgement of message {self.seq}")
        n = 0
        if data is not None:
            raw = np.frombuffer(data, dtype=np.uint8) if isinstance(data, (bytes, bytearray)) else data.view(np.uint8).reshape(-1)
            n = raw.shape[0]
            if n > self.capacity:
                raise ValueError(f"message of {n} bytes exceeds the channel capacity {self.capacity}")
            self.payload[:n] = raw
        w[1], w[2] = kind, n
        self.seq += 1
        w[0] = self.seq            # publishing store: after the payload (x86 keeps store order)

    def drain(self, timeout_s: float | None = None) -> None:
        """Wait until every follower consumed the last message."""
        w = self.words

        def all_acked():
            self._check_followers()
            return all(w[4 + r] >= self.seq for r in range(1, self.world_size))
        self._wait(all_acked, "followers to drain", timeout_s)

    def wait_hello(self, timeout_s: float | None = None) -> None:
        """Rank 0: wait until every follower process attached to the channel (words 24 + r)."""
        w = self.words

        def all_here():
            self._check_followers()
            return all(w[24 + r] != 0 for r in range(1, self.world_size))
        self._wait(all_here, "follower processes to start", timeout_s)

    # ------------------------------------------------------------------ followers
    def hello(self) -> None:
        self.words[24 + self.rank] = os.getpid()

    def receive(self, timeout_s: float | None = float("inf")) -> tuple[int, np.ndarray]:
        """Wait for the next message; returns (kind, payload copy as uint8).  The default has no
        deadline (an idle engine is not an error) but ends with ``PeerFailed`` when rank 0 is gone."""
        w = self.words
        nxt = self.seq + 1
        self._wait(lambda: w[0] >= nxt, f"message {nxt}", timeout_s)
        kind, n = int(w[1]), int(w[2])
        data = self.payload[:n].copy()
        self.seq = nxt
        w[4 + self.rank] = nxt
        return kind, data

    def report_failure(self, text: str) -> None:
        raw = text.encode("utf-8", "replace")[:_ERR_BYTES - 1]
        off = _WORDS_HDR * 8
        self.shm.buf[off:off + len(raw)] = raw
        self.shm.buf[off + len(raw)] = 0
        self.words[16 + self.rank] = 1

    def read_error(self) -> str:
        off = _WORDS_HDR * 8
        raw = bytes(self.shm.buf[off:off + _ERR_BYTES])
        return raw.split(b"\0", 1)[0].decode("utf-8", "replace")

    # ------------------------------------------------------------------ teardown
    def close(self) -> None:
        if self.shm is None:
            return
        self.words = self.payload = None
        try:
            self.shm.close()
            if self.owner:
                self.shm.unlink()
        except (FileNotFoundError, BufferError):
            pass
        self.shm = None
