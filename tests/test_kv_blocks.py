"""KV block pool: chained-hash prefix cache, reference counting, reuse of freed blocks, growth and sealing.
Behaviour model: tinyvllm/engine/block_manager.py:36-139."""
import random

from hypothesis import given, settings, strategies as st

from tinyllmforge_b200 import SamplingParams
from tinyllmforge_b200.engine.kv_blocks import KVBlockPool, chain_hash
from tinyllmforge_b200.engine.request import Request


def req(tokens, **kw):
    return Request(list(tokens), SamplingParams(**kw))


def test_chain_hash_depends_on_prefix():
    a = chain_hash([1, 2, 3, 4])
    assert a == chain_hash([1, 2, 3, 4])
    assert chain_hash([1, 2, 3, 4], parent=a) != a
    assert chain_hash([1, 2, 3, 5]) != a


def test_admit_without_sharing_takes_blocks_in_order():
    pool = KVBlockPool(8, 4)
    r = req(range(10))
    assert pool.can_admit(r)
    pool.admit(r)
    assert r.block_table == [0, 1, 2] and r.num_cached_tokens == 0
    assert pool.num_free == 5
    pool.check_invariants()


def test_prefix_hit_shares_full_blocks_only():
    pool = KVBlockPool(16, 4)
    a = req([1, 2, 3, 4, 5, 6, 7, 8, 9])
    pool.admit(a)
    b = req([1, 2, 3, 4, 5, 6, 7, 8, 10, 11])
    pool.admit(b)
    assert b.block_table[:2] == a.block_table[:2] and b.block_table[2] != a.block_table[2]
    assert b.num_cached_tokens == 8
    assert pool.ref_count[a.block_table[0]] == 2
    pool.check_invariants()


def test_miss_latches_after_first_difference():
    pool = KVBlockPool(16, 4)
    a = req([1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12])
    pool.admit(a)
    b = req([1, 2, 3, 4, 0, 0, 0, 0, 9, 10, 11, 12, 13])
    pool.admit(b)
    assert b.num_cached_tokens == 4          # block 3 has equal tokens but a different prefix -> different hash
    assert b.block_table[0] == a.block_table[0] and b.block_table[2] != a.block_table[2]


def test_freed_blocks_stay_reusable_until_recycled():
    pool = KVBlockPool(4, 4)
    a = req([1, 2, 3, 4, 5, 6, 7, 8, 9])
    pool.admit(a)
    table = list(a.block_table)
    pool.release(a)
    assert pool.num_free == 4
    b = req([1, 2, 3, 4, 5, 6, 7, 8, 9])
    pool.admit(b)
    assert b.block_table[:2] == table[:2] and b.num_cached_tokens == 8
    pool.check_invariants()


def test_fully_cached_prompt_still_computes_last_token():
    pool = KVBlockPool(8, 4)
    a = req([1, 2, 3, 4, 5, 6, 7, 8])
    pool.admit(a)
    b = req([1, 2, 3, 4, 5, 6, 7, 8])
    pool.admit(b)
    assert b.block_table == a.block_table
    assert b.num_cached_tokens == 7           # the reference would report 8 and build an empty query


def test_grow_allocates_and_seals():
    pool = KVBlockPool(8, 4)
    r = req([1, 2, 3])
    pool.admit(r)
    r.append_token(4)
    assert pool.can_grow(r)
    pool.grow(r)                               # len 4: last block becomes full -> sealed
    assert len(r.block_table) == 1 and pool.block_hash[r.block_table[0]] == chain_hash([1, 2, 3, 4])
    r.append_token(5)
    pool.grow(r)                               # len 5: needs a second block
    assert len(r.block_table) == 2
    other = req([1, 2, 3, 4, 9])
    pool.admit(other)
    assert other.block_table[0] == r.block_table[0] and other.num_cached_tokens == 4


def test_can_grow_false_when_pool_empty():
    pool = KVBlockPool(1, 4)
    r = req([1, 2, 3, 4])
    pool.admit(r)
    r.append_token(5)
    assert not pool.can_grow(r)


@settings(max_examples=60, deadline=None)
@given(st.integers(0, 10_000), st.sampled_from([4, 8, 16]))
def test_random_workload_keeps_invariants(seed, bs):
    rng = random.Random(seed)
    pool = KVBlockPool(48, bs)
    prefixes = [[rng.randrange(50) for _ in range(rng.randrange(1, 4 * bs))] for _ in range(3)]
    live = []
    for _ in range(200):
        op = rng.random()
        if op < 0.4:
            toks = list(rng.choice(prefixes)) + [rng.randrange(50) for _ in range(rng.randrange(0, 2 * bs))]
            r = req(toks)
            if pool.can_admit(r):
                pool.admit(r)
                assert len(r.block_table) == pool.blocks_needed(len(r))
                assert 0 <= r.num_cached_tokens < len(r)
                # cached prefix => the shared blocks really hold the same tokens
                for i in range(r.num_cached_tokens // bs):
                    assert pool.block_tokens[r.block_table[i]] == tuple(toks[i * bs:(i + 1) * bs])
                live.append(r)
        elif op < 0.8 and live:
            r = rng.choice(live)
            r.append_token(rng.randrange(50))
            if pool.can_grow(r):
                pool.grow(r)
                assert len(r.block_table) == pool.blocks_needed(len(r))
            else:
                r.token_ids.pop()
        elif live:
            r = live.pop(rng.randrange(len(live)))
            pool.release(r)
        pool.check_invariants()
        # a block is writable by at most one request: every block after the shared prefix has ref_count 1
        for r in live:
            assert all(pool.ref_count[b] >= 1 for b in r.block_table)
            assert pool.ref_count[r.block_table[-1]] == 1 or len(r) % bs == 0
