"""Scheduler policy: prefill first, budgets, decode growth, recompute preemption of the newest request,
finish conditions.  Behaviour model: tinyvllm/engine/scheduler.py:22-72."""
import pytest

from tinyllmforge_b200 import SamplingParams
from tinyllmforge_b200.config import Config, preset
from tinyllmforge_b200.engine.request import Request, RequestStatus
from tinyllmforge_b200.engine.scheduler import Scheduler


def make(num_blocks=64, block_size=4, max_seqs=8, budget=64, eos=-1):
    cfg = Config("x", hf_config=preset("tiny"), num_kvcache_blocks=num_blocks, kvcache_block_size=16, device="cpu",
                 max_num_seqs=max_seqs, max_num_batched_tokens=budget, max_model_len=budget, eos=eos)
    s = Scheduler(cfg)
    s.pool.__init__(num_blocks, block_size)
    return s


_base = [0]


def R(n, **kw):
    """A request of n tokens that shares no prefix with any other request."""
    _base[0] += 1000
    return Request(list(range(_base[0], _base[0] + n)), SamplingParams(**kw))


def test_prefill_first_in_arrival_order_within_budget():
    s = make(budget=20)
    a, b, c = R(8), R(8), R(8)
    for r in (a, b, c):
        s.add(r)
    batch, is_prefill = s.schedule()
    assert is_prefill and batch == [a, b]                 # 8 + 8 <= 20 < 24
    assert all(r.status is RequestStatus.RUNNING for r in batch)
    batch, is_prefill = s.schedule()
    assert is_prefill and batch == [c]
    batch, is_prefill = s.schedule()
    assert not is_prefill and batch == [a, b, c]


def test_max_num_seqs_limits_admission():
    s = make(max_seqs=2)
    for _ in range(3):
        s.add(R(4))
    batch, _ = s.schedule()
    assert len(batch) == 2


def test_budget_counts_uncached_tokens_only():
    s = make(budget=20, block_size=4)
    a = R(16)
    s.add(a)
    s.schedule()
    s.postprocess([a], [99])
    b = Request(a.prompt_token_ids + [5, 6], SamplingParams())       # shares 16 cached tokens
    c = R(6)
    s.add(b)
    s.add(c)
    batch, is_prefill = s.schedule()
    assert b.num_cached_tokens == 16                      # b is charged 2 tokens, not 18 ...
    assert is_prefill and batch == [b, c]                 # ... so c (6 tokens) still fits: 18 + 6 > 20 >= 2 + 6


def test_decode_preempts_newest_and_requeues_at_front():
    s = make(num_blocks=4, block_size=4, budget=64)
    a, b = R(8), R(8)
    s.add(a)
    s.add(b)
    batch, _ = s.schedule()
    assert batch == [a, b] and s.pool.num_free == 0
    s.postprocess(batch, [7, 7])                          # both now 9 tokens: each needs a new block, none free
    batch, is_prefill = s.schedule()
    assert not is_prefill and batch == [a]
    assert b.status is RequestStatus.WAITING and s.waiting[0] is b and b.block_table == []
    assert b.num_preemptions == 1 and s.num_preemptions == 1
    assert len(b) == 9                                    # the generated token is kept and recomputed later


def test_finish_on_max_tokens_and_eos():
    s = make(eos=42)
    a = R(4, max_tokens=2)
    b = R(4, max_tokens=10)
    c = R(4, max_tokens=10, ignore_eos=True)
    for r in (a, b, c):
        s.add(r)
    batch, _ = s.schedule()
    done = s.postprocess(batch, [1, 42, 42])
    assert done == [b] and b.is_finished and b.block_table == []
    batch, _ = s.schedule()
    assert batch == [a, c]
    done = s.postprocess(batch, [1, 1])
    assert done == [a] and a.completion_token_ids == [1, 1]
    assert list(s.running) == [c]


def test_oversized_prompt_rejected():
    s = make(budget=16)
    with pytest.raises(ValueError):
        s.add(R(17))


def test_bench_workload_shape():
    """The reference's bench.py workload: 9 prefill steps (142,827 tokens) then 1,023 decode steps
    (133,710 tokens), batch 256 -> 1, no preemption with >= 800 blocks of 256."""
    import sys, os
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from bench import make_workload
    prompts, max_tokens = make_workload()
    assert sum(map(len, prompts)) == 142827 and sum(max_tokens) == 133966
    cfg = Config("x", hf_config=preset("qwen3-0.6b"), num_kvcache_blocks=800, device="cpu")
    s = Scheduler(cfg)
    for p, m in zip(prompts, max_tokens):
        s.add(Request(p, SamplingParams(temperature=0.6, max_tokens=m, ignore_eos=True)))
    pre = dec = pre_tok = dec_tok = 0
    while not s.is_finished():
        batch, is_prefill = s.schedule()
        if is_prefill:
            pre += 1
            pre_tok += sum(len(r) - r.num_cached_tokens for r in batch)
        else:
            dec += 1
            dec_tok += len(batch)
        s.postprocess(batch, [0] * len(batch))
    assert (pre, dec, pre_tok, dec_tok, s.num_preemptions) == (9, 1023, 142827, 133710, 0)


def test_chunked_prefill_schedules_a_long_prompt_over_several_steps():
    from tinyllmforge_b200 import preset
    from tinyllmforge_b200.config import Config
    cfg = Config.from_kwargs("x", hf_config=preset("tiny"), device="cpu", load_format="dummy", skip_tokenizer_init=True,
                             kvcache_block_size=8, num_kvcache_blocks=64, max_num_seqs=4, max_model_len=256,
                             max_num_batched_tokens=32, chunked_prefill=True)
    sch = Scheduler(cfg)
    short, long = Request(list(range(10))), Request(list(range(100, 180)))         # 80 tokens > budget 32
    sch.add(short)
    sch.add(long)
    batch, is_prefill = sch.schedule()
    assert is_prefill and batch == [short]
    sch.postprocess(batch, [1])
    spans = []
    while sch.has_waiting():
        batch, is_prefill = sch.schedule()
        assert is_prefill and batch == [long]
        spans.append((long.num_computed_tokens, long.prefill_end))
        before = len(long)
        sch.postprocess(batch, [7])
        assert len(long) == before + (0 if sch.partial is long else 1)
    assert spans == [(0, 32), (32, 64), (64, 80)]
    assert len(long) == 81 and long.num_computed_tokens == -1 and long in sch.running
    # blocks were registered chunk by chunk: all ten full prompt blocks are reusable now
    other = Request(list(range(100, 180)) + [5])
    sch.add(other)
    batch, is_prefill = sch.schedule()
    assert is_prefill and batch == [other] and other.num_cached_tokens == 80
    batch2, is_prefill2 = sch.schedule()
    assert not is_prefill2 and set(batch2) == {short, long, other}
