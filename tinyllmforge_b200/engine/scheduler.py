"""Prefill-first batch scheduler with recompute preemption.

Parity: tinyvllm/engine/scheduler.py:7-72.  Policy is the reference's:

* if any waiting request fits (sequence slots, token budget counted on the
  tokens that still need computing, KV blocks), the step is a prefill of as many
  waiting requests as fit, in arrival order;
* otherwise the step decodes every running request; when the pool cannot hold a
  request's next KV entry the newest running request is preempted (all its
  blocks freed, pushed to the front of the waiting queue, recomputed later);
* a request finishes on EOS (unless ``ignore_eos``) or after ``max_tokens``.

The admission test charges the same quantity it compares (uncached tokens),
where the reference compares the full length but charges the uncached part
(tinyvllm/engine/scheduler.py:29,33).
"""
from __future__ import annotations

from collections import deque

from ..config import Config
from .kv_blocks import KVBlockPool
from .request import Request, RequestStatus


PLACEHOLDER = -2          # token id not read back yet (never equals an EOS id, never a valid id)


class Scheduler:
    def __init__(self, config: Config):
        self.max_num_seqs = config.max_num_seqs
        self.max_num_batched_tokens = config.max_num_batched_tokens
        self.eos = config.eos
        self.pool = KVBlockPool(config.num_kvcache_blocks, config.kvcache_block_size)
        self.waiting: deque[Request] = deque()
        self.running: deque[Request] = deque()
        self.num_preemptions = 0

    def is_finished(self) -> bool:
        return not self.waiting and not self.running

    def add(self, req: Request) -> None:
        if len(req) > self.max_num_batched_tokens:
            raise ValueError(f"prompt of {len(req)} tokens exceeds max_num_batched_tokens={self.max_num_batched_tokens}")
        if self.pool.blocks_needed(len(req) + 1) > self.pool.num_blocks:
            raise ValueError("prompt does not fit in the KV cache")
        self.waiting.append(req)

    def schedule(self, defer_seal: bool = False) -> tuple[list[Request], bool]:
        """Pick the next batch. Returns (requests, is_prefill).  ``defer_seal``: see ``KVBlockPool.grow``."""
        batch: list[Request] = []
        budget = self.max_num_batched_tokens
        while self.waiting and len(self.running) < self.max_num_seqs:
            req = self.waiting[0]
            # An upper bound on the work is the whole length; the exact charge is known after admit().
            if len(req) > budget or not self.pool.can_admit(req):
                break
            self.pool.admit(req)
            budget -= len(req) - req.num_cached_tokens
            req.status = RequestStatus.RUNNING
            self.waiting.popleft()
            self.running.append(req)
            batch.append(req)
        if batch:
            return batch, True

        # decode: walk the running queue oldest first
        pending = self.running
        self.running = deque()
        while pending:
            req = pending.popleft()
            while not self.pool.can_grow(req):
                if pending:
                    self._preempt(pending.pop())
                else:
                    self._preempt(req)
                    req = None
                    break
            if req is None:
                break
            self.pool.grow(req, defer_seal)
            batch.append(req)
        self.running.extend(batch)
        if not batch:
            raise RuntimeError("the KV cache cannot hold a single running request; raise gpu_memory_utilization "
                               "or lower max_model_len")
        return batch, False

    def _preempt(self, req: Request) -> None:
        req.status = RequestStatus.WAITING
        req.num_preemptions += 1
        self.num_preemptions += 1
        self.pool.release(req)
        self.waiting.appendleft(req)

    def has_waiting(self) -> bool:
        return bool(self.waiting)

    def postprocess(self, batch: list[Request], token_ids: list[int]) -> list[Request]:
        """Append the sampled tokens; retire finished requests. Returns the finished ones.
        The pipelined engine loop passes ``PLACEHOLDER`` ids and patches the real ones in later."""
        finished = []
        for req, tok in zip(batch, token_ids):
            req.token_ids.append(tok)
            if (not req.ignore_eos and tok == self.eos) or req.num_completion_tokens >= req.max_tokens:
                req.status = RequestStatus.FINISHED
                self.pool.release(req)
                finished.append(req)
        if finished:
            if len(finished) == len(self.running):
                self.running.clear()
            else:
                self.running = deque(r for r in self.running if r.status is RequestStatus.RUNNING)
        return finished
