"""Paged KV-cache bookkeeping with hash-based prefix reuse (host side, no tensors).

Parity: tinyvllm/engine/block_manager.py:8-139.  Same observable policy:

* a block's identity is a *chained* 64-bit hash: hash(parent_hash, the block's
  token ids), so equal hashes imply an equal whole prefix (block_manager.py:36-42);
* only full blocks are hashed; a hit needs the dictionary entry **and** equal
  token ids; after the first miss every later block of the request is a miss
  (block_manager.py:66-98);
* releasing a request keeps hash and token ids on its freed blocks, so they stay
  reusable until the allocator recycles them, oldest-freed first
  (block_manager.py:100-107);
* growth during decode: a new block when the newest token opens one, and the
  last block is sealed (hashed, registered) when it becomes full
  (block_manager.py:110-139).

Differences: state lives in flat per-block arrays and the free list is an
insertion-ordered dict, so reviving a specific freed block is O(1) (the
reference's ``deque.remove`` is O(free blocks)); the number of cached tokens
is capped at ``len(request) - 1`` so a fully cached prompt still computes its
last token (the reference produces an empty query in that case).
"""
from __future__ import annotations

import struct
from collections import OrderedDict

from .request import Request

try:  # a hashing library; the hash value is not part of any interface
    import xxhash

    def _hash64(parent: int, payload: bytes) -> int:
        h = xxhash.xxh64()
        if parent != -1:
            h.update(struct.pack("<q", parent))
        h.update(payload)
        return h.intdigest() & 0x7FFFFFFFFFFFFFFF
except ImportError:  # pragma: no cover
    import hashlib

    def _hash64(parent: int, payload: bytes) -> int:
        h = hashlib.blake2b(digest_size=8)
        if parent != -1:
            h.update(struct.pack("<q", parent))
        h.update(payload)
        return int.from_bytes(h.digest(), "little") & 0x7FFFFFFFFFFFFFFF


def chain_hash(token_ids, parent: int = -1) -> int:
    """Hash of one full block given the hash of the block before it (-1: none)."""
    return _hash64(parent, struct.pack(f"<{len(token_ids)}q", *token_ids))


class KVBlockPool:
    def __init__(self, num_blocks: int, block_size: int):
        if num_blocks <= 0:
            raise ValueError("the KV pool needs at least one block")
        self.num_blocks = num_blocks
        self.block_size = block_size
        self.ref_count = [0] * num_blocks
        self.block_hash = [-1] * num_blocks
        self.block_tokens: list[tuple | None] = [None] * num_blocks
        self.free: "OrderedDict[int, None]" = OrderedDict((i, None) for i in range(num_blocks))
        self.hash_to_block: dict[int, int] = {}
        # counters for the stats object
        self.prefix_hit_tokens = 0
        self.prefix_query_tokens = 0

    # ------------------------------------------------------------------ helpers
    @property
    def num_free(self) -> int:
        return len(self.free)

    def blocks_needed(self, num_tokens: int) -> int:
        return (num_tokens + self.block_size - 1) // self.block_size

    def _take(self, block_id: int) -> None:
        """Move a free block to the used state, forgetting its old identity."""
        del self.free[block_id]
        old = self.block_hash[block_id]
        if old != -1 and self.hash_to_block.get(old) == block_id:
            del self.hash_to_block[old]
        self.block_hash[block_id] = -1
        self.block_tokens[block_id] = None
        self.ref_count[block_id] = 1

    def _take_oldest(self) -> int:
        block_id = next(iter(self.free))
        self._take(block_id)
        return block_id

    def _seal(self, block_id: int, h: int, tokens: tuple) -> None:
        self.block_hash[block_id] = h
        self.block_tokens[block_id] = tokens
        self.hash_to_block[h] = block_id

    # ------------------------------------------------------------------ prefill
    def can_admit(self, req: Request) -> bool:
        return len(self.free) >= self.blocks_needed(len(req))

    def admit(self, req: Request, seal_upto: int | None = None) -> None:
        """Give ``req`` a block table covering all its tokens, reusing cached prefix blocks.

        ``seal_upto``: only blocks that end at or before this token count are registered for reuse now (chunked prefill:
        a block must not be found by other requests before the step that computes it has been scheduled);
        ``seal_computed`` registers the rest later."""
        assert not req.block_table, "request already holds blocks"
        bs = self.block_size
        n = len(req)
        if seal_upto is None:
            seal_upto = n
        toks = req.token_ids
        parent = -1
        missed = False
        cached = 0
        for i in range(self.blocks_needed(n)):
            chunk = tuple(toks[i * bs:(i + 1) * bs])
            full = len(chunk) == bs
            h = chain_hash(chunk, parent) if full else -1
            block_id = -1
            if not missed and full:
                cand = self.hash_to_block.get(h, -1)
                if cand != -1 and self.block_tokens[cand] == chunk:
                    block_id = cand
            if block_id == -1:
                missed = True
                block_id = self._take_oldest()
            else:
                cached += bs
                if self.ref_count[block_id] > 0:
                    self.ref_count[block_id] += 1
                else:                      # freed but not yet recycled: revive it as is
                    del self.free[block_id]
                    self.ref_count[block_id] = 1
            if full:
                if self.block_hash[block_id] != h and (i + 1) * bs <= seal_upto:
                    self._seal(block_id, h, chunk)
                parent = h
            req.block_table.append(block_id)
        req.num_cached_tokens = min(cached, n - 1)
        self.prefix_hit_tokens += req.num_cached_tokens
        self.prefix_query_tokens += n

    def seal_computed(self, req: Request, upto: int) -> None:
        """Register the prompt blocks of ``req`` that end at or before token ``upto`` and are not registered yet (in order:
        a block's hash chains on its predecessor's)."""
        bs = self.block_size
        for index in range(min(upto // bs, len(req.block_table))):
            self._seal_block(req, index, (index + 1) * bs)

    def release(self, req: Request) -> None:
        for block_id in reversed(req.block_table):
            self.ref_count[block_id] -= 1
            assert self.ref_count[block_id] >= 0
            if self.ref_count[block_id] == 0:
                self.free[block_id] = None
        req.block_table.clear()
        req.num_cached_tokens = 0
        req.num_computed_tokens = req.prefill_end = -1

    # ------------------------------------------------------------------ decode
    def can_grow(self, req: Request) -> bool:
        """True if the pool can hold the KV entry of ``req``'s newest token."""
        return len(self.free) >= (1 if len(req) % self.block_size == 1 else 0)

    def grow(self, req: Request, defer_seal: bool = False) -> None:
        """Make room for the newest token's KV entry; seal the last block when it fills up.

        ``defer_seal``: the pipelined engine loop schedules a step before the previous step's tokens have been read
        back, so the newest token id is still a placeholder.  The block it completes is then sealed one step later
        (when the next block is opened), by which time every token of it is known."""
        bs = self.block_size
        n = len(req)
        rem = n % bs
        if rem == 1:
            if defer_seal and len(req.block_table) >= 1:
                self._seal_block(req, len(req.block_table) - 1, n - 1)
            req.block_table.append(self._take_oldest())
        elif rem == 0 and not defer_seal:
            self._seal_block(req, len(req.block_table) - 1, n)

    def _seal_block(self, req: Request, index: int, end: int) -> None:
        """Hash and register block ``index`` of ``req``, whose last token is token ``end - 1``."""
        block_id = req.block_table[index]
        if self.block_hash[block_id] != -1 or self.ref_count[block_id] != 1:
            return
        parent = self.block_hash[req.block_table[index - 1]] if index > 0 else -1
        if index > 0 and parent == -1:
            return                                  # the chain is broken (an earlier block was never sealed)
        chunk = tuple(req.token_ids[end - self.block_size:end])
        self._seal(block_id, chain_hash(chunk, parent), chunk)

    # ------------------------------------------------------------------ checks (tests)
    def check_invariants(self) -> None:
        used = {i for i, r in enumerate(self.ref_count) if r > 0}
        free = set(self.free)
        assert used.isdisjoint(free)
        assert used | free == set(range(self.num_blocks))
        for h, b in self.hash_to_block.items():
            assert self.block_hash[b] == h
