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

Not in the reference (it rejects such prompts): with ``chunked_prefill`` a prompt longer
than the token budget is admitted alone and prefilled over consecutive steps, one budget
worth of tokens at a time; it joins the running queue when its last chunk is scheduled,
and its blocks become visible to the prefix cache only as their chunks are scheduled.
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
        self.chunked = bool(config.chunked_prefill)
        self.max_model_len = config.max_model_len
        self.partial: Request | None = None       # admitted, holds its blocks, prompt not completely prefilled yet
        self.last_admit_cached = 0                # prefix-cache tokens of the requests admitted by the last schedule()

    def is_finished(self) -> bool:
        return not self.waiting and not self.running and self.partial is None

    def add(self, req: Request) -> None:
        if len(req) > self.max_num_batched_tokens and not self.chunked:
            raise ValueError(f"prompt of {len(req)} tokens exceeds max_num_batched_tokens={self.max_num_batched_tokens} "
                             "(chunked_prefill=True admits it)")
        if len(req) >= self.max_model_len and self.chunked:
            raise ValueError(f"prompt of {len(req)} tokens does not fit max_model_len={self.max_model_len}")
        if self.pool.blocks_needed(len(req) + 1) > self.pool.num_blocks:
            raise ValueError("prompt does not fit in the KV cache")
        self.waiting.append(req)

    def schedule(self, defer_seal: bool = False) -> tuple[list[Request], bool]:
        """Pick the next batch. Returns (requests, is_prefill).  ``defer_seal``: see ``KVBlockPool.grow``."""
        batch: list[Request] = []
        budget = self.max_num_batched_tokens
        self.last_admit_cached = 0
        if self.partial is not None:                       # the next chunk of a long prompt, alone
            req = self.partial
            req.prefill_end = min(len(req), req.num_computed_tokens + budget)
            self.pool.seal_computed(req, req.prefill_end)
            if req.prefill_end == len(req):                # last chunk: the request decodes from the next step on
                self.partial = None
                req.status = RequestStatus.RUNNING
                self.running.append(req)
            return [req], True
        while self.waiting and len(self.running) < self.max_num_seqs:
            req = self.waiting[0]
            if self.chunked and len(req) > self.max_num_batched_tokens:
                # can never be prefilled whole: first chunk, in a step of its own
                if batch or not self.pool.can_admit(req):
                    break
                first = self.max_num_batched_tokens
                self.pool.admit(req, seal_upto=first)
                self.last_admit_cached += req.num_cached_tokens
                req.num_computed_tokens = req.num_cached_tokens
                req.prefill_end = min(len(req), req.num_computed_tokens + first)
                self.pool.seal_computed(req, req.prefill_end)
                self.waiting.popleft()
                self.partial = req                         # a prefix hit cannot complete it: the prompt exceeds the budget by itself...
                if req.prefill_end == len(req):            # ...unless most of it was cached
                    self.partial = None
                    req.status = RequestStatus.RUNNING
                    self.running.append(req)
                return [req], True
            # An upper bound on the work is the whole length; the exact charge is known after admit().
            if len(req) > budget or not self.pool.can_admit(req):
                break
            self.pool.admit(req)
            self.last_admit_cached += req.num_cached_tokens
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

    def finish_early(self, req: Request) -> None:
        """Retire a request whose newest KNOWN token ended it (EOS) although a later step that still contains it has
        been scheduled already (the pipelined engine loop schedules one step ahead of the tokens it has read back).
        Its blocks go back to the pool at once: the step in flight may still write the surplus token's KV entry into
        the request's last block, but every later step runs after it on the same stream, and a partly filled or
        unsealed block is never found through the prefix cache."""
        if req.status is RequestStatus.FINISHED:
            return
        was_running = req.status is RequestStatus.RUNNING
        req.status = RequestStatus.FINISHED
        if req.block_table:
            self.pool.release(req)
        if was_running:
            self.running = deque(r for r in self.running if r is not req)
        else:                                              # preempted in the meantime: it waits for a prefill it no longer needs
            self.waiting = deque(r for r in self.waiting if r is not req)

    def has_waiting(self) -> bool:
        """True if the next step may be a prefill."""
        return bool(self.waiting) or self.partial is not None

    def postprocess(self, batch: list[Request], token_ids: list[int]) -> list[Request]:
        """Append the sampled tokens; retire finished requests. Returns the finished ones.
        The pipelined engine loop passes ``PLACEHOLDER`` ids and patches the real ones in later."""
        finished = []
        for req, tok in zip(batch, token_ids):
            if req.status is RequestStatus.FINISHED:       # retired by finish_early() while this step was in flight
                continue
            if req is self.partial:                        # a chunk in the middle of a long prompt: no token yet
                req.num_computed_tokens = req.prefill_end
                continue
            if req.prefill_end >= 0:                       # last (or only) chunk of a chunked prompt: back to the normal state
                req.num_computed_tokens = req.prefill_end = -1
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
