"""The packed step descriptor: layout, padding conventions, round trip through raw bytes."""
import numpy as np

from tinyllmforge_b200 import SamplingParams
from tinyllmforge_b200.engine.request import Request
from tinyllmforge_b200.engine.step_batch import StepBatch, build_decode, build_prefill


def _req(n, table, cached=0, temp=0.5):
    r = Request(list(range(100, 100 + n)), SamplingParams(temperature=temp))
    r.block_table = list(table)
    r.num_cached_tokens = cached
    return r


def test_prefill_layout_with_cached_prefix():
    a = _req(10, [3, 5, 9], cached=0)
    b = _req(7, [2, 4], cached=4, temp=0.0)
    sb = build_prefill([a, b], block_size=4, step_index=12, seed=(5 << 32) | 7)
    assert sb.is_prefill and sb.num_seqs == 2 and sb.num_tokens == 13
    assert sb.max_seqlen_q == 10 and sb.max_seqlen_k == 10 and sb.step_index == 12 and sb.seed == (5 << 32) | 7
    assert sb.cu_seqlens_q.tolist() == [0, 10, 13]
    assert sb.context_lens.tolist() == [10, 7]
    assert sb.last_index.tolist() == [9, 12]
    assert sb.input_ids.tolist() == list(range(100, 110)) + [104, 105, 106]
    assert sb.positions.tolist() == list(range(10)) + [4, 5, 6]
    # slot = block_table[pos // bs] * bs + pos % bs
    assert sb.slot_mapping.tolist()[:5] == [12, 13, 14, 15, 20]
    assert sb.slot_mapping.tolist()[10:] == [16, 17, 18]
    assert sb.block_tables.tolist() == [[3, 5, 9], [2, 4, -1]]
    assert np.allclose(sb.temperatures, [0.5, 0.0])


def test_decode_padding_uses_skip_values_and_true_positions():
    a = _req(9, [1, 2, 6])
    b = _req(4, [7])
    sb = build_decode([a, b], block_size=4, pad_to=4, table_width=5)
    assert not sb.is_prefill and sb.num_seqs == 2 and sb.padded_seqs == 4 and sb.table_width == 5
    assert sb.input_ids.tolist() == [108, 103, 0, 0]
    assert sb.positions.tolist() == [8, 3, 0, 0]                 # index of the token being written: len - 1
    assert sb.slot_mapping.tolist() == [6 * 4 + 0, 7 * 4 + 3, -1, -1]
    assert sb.context_lens.tolist() == [9, 4, 0, 0]
    assert sb.block_tables.tolist()[0] == [1, 2, 6, -1, -1] and sb.block_tables.tolist()[2] == [-1] * 5
    assert sb.cu_seqlens_q.tolist() == [0, 1, 2, 2, 2]


def test_offsets_depend_only_on_bucket_and_width():
    a = build_decode([_req(3, [0])], 4, pad_to=8, table_width=6)
    b = build_decode([_req(9, [1, 2, 3]), _req(5, [4, 5])], 4, pad_to=8, table_width=6)
    assert a.offsets == b.offsets and a.num_words == b.num_words
    assert all(off % 4 == 0 for off, _ in a.offsets.values())


def test_round_trip_through_bytes():
    sb = build_decode([_req(9, [1, 2, 6])], 4, step_index=3, seed=11)
    raw = sb.buf.tobytes()
    sb2 = StepBatch(np.frombuffer(raw, dtype=np.int32))
    assert sb2.input_ids.tolist() == sb.input_ids.tolist() and sb2.seed == 11 and sb2.step_index == 3


def test_incremental_decode_builder_equals_full_rebuild():
    """Drive a scheduler through a workload; every decode step built incrementally must equal the full build."""
    import random
    from tinyllmforge_b200.config import Config, preset
    from tinyllmforge_b200.engine.scheduler import Scheduler
    from tinyllmforge_b200.engine.step_batch import DecodeBuilder
    rng = random.Random(0)
    cfg = Config("x", hf_config=preset("tiny"), num_kvcache_blocks=400, kvcache_block_size=8, device="cpu",
                 max_num_seqs=16, max_num_batched_tokens=512, max_model_len=512)
    s = Scheduler(cfg)
    for _ in range(12):
        s.add(Request([rng.randrange(100) for _ in range(rng.randint(3, 40))],
                      SamplingParams(max_tokens=rng.randint(2, 40), ignore_eos=True)))
    builder = DecodeBuilder(8)
    fast = steps = 0
    while not s.is_finished():
        reqs, is_prefill = s.schedule()
        if not is_prefill:
            for pad, width in ((None, None), (16, 64)):
                b = DecodeBuilder(8) if pad is None else builder
                was_cached = b.reqs is not None and b.reqs == reqs
                got = b.build(reqs, steps, 7, pad, width)
                want = build_decode(reqs, 8, steps, 7, pad_to=pad, table_width=width)
                assert got.num_words == want.num_words
                assert np.array_equal(got.buf[:got.num_words], want.buf[:want.num_words]), steps
                fast += bool(was_cached)
        steps += 1
        s.postprocess(reqs, [rng.randrange(100) for _ in reqs])
    assert fast > 10
