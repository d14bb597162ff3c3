"""Property test of the engine loops with a fake worker (no model): whatever the prompts, lengths, pool size and
sequence limit, the loop that runs one step ahead of the tokens it has read back must retire every request with exactly
the tokens of the plain loop, keep the KV pool consistent and give every block back.  In half of the cases the pipelined
engine also has a token budget so small that long prompts are prefilled in chunks.  A second property does the same with
requests that stop on an EOS id the fake worker emits often: the pipelined loop then schedules one step too many for
such a request and must drop the surplus token, free the blocks and never seal a block with a token that was not read back.

The fake worker "samples" a deterministic function of (the sequence's input token, its position), taken from the packed
step buffer exactly as a real worker would see it, including the device-side hand-over of the previous step's tokens
(``src_rows``)."""
import numpy as np
import pytest
from hypothesis import HealthCheck, given, settings, strategies as st

from tinyllmforge_b200 import SamplingParams, preset
from tinyllmforge_b200.config import Config
from tinyllmforge_b200.engine.engine import LLMEngine
from tinyllmforge_b200.engine.scheduler import Scheduler
from tinyllmforge_b200.engine.stats import EngineStats
from tinyllmforge_b200.engine.step_batch import DecodeBuilder


class FakeWorker:
    def __init__(self, modulus=997):
        self.prev = np.zeros(0, dtype=np.int64)
        self.steps = 0
        self.modulus = modulus          # tokens are drawn from [0, modulus): a small one makes any given id frequent
        self.fail_at = None             # step whose collect() reports a kernel error, as the real worker does from the status word

    def decode_padding(self, n):
        return None, None

    def launch(self, sb):
        n = sb.num_seqs
        if sb.is_prefill:
            last = sb.last_index[:n]
            ids, pos = sb.input_ids[last].astype(np.int64), sb.positions[last].astype(np.int64)
        else:
            ids, pos = sb.input_ids[:n].astype(np.int64).copy(), sb.positions[:n].astype(np.int64)
            src = sb.src_rows[:n]
            take = src >= 0
            ids[take] = self.prev[src[take]]
        assert (ids >= 0).all(), "a placeholder token reached the worker"
        toks = (ids * 31 + pos * 7 + 3) % self.modulus
        self.prev = toks
        self.steps += 1
        return toks.tolist()

    def collect(self, ticket):
        if self.fail_at is not None and self.steps >= self.fail_at:
            raise RuntimeError("a CUDA kernel reported: peer flag wait ran out")
        return ticket

    def run(self, sb):
        return self.collect(self.launch(sb))


def make_engine(num_blocks, max_seqs, pipelined, budget=128, eos=-1, modulus=997):
    cfg = Config.from_kwargs("fake", hf_config=preset("tiny"), device="cpu", load_format="dummy", skip_tokenizer_init=True,
                             kvcache_block_size=8, num_kvcache_blocks=num_blocks, max_num_seqs=max_seqs, max_model_len=128,
                             max_num_batched_tokens=budget, chunked_prefill=budget < 128, extra={"pipeline": pipelined}, eos=eos)
    eng = LLMEngine.__new__(LLMEngine)            # the loops only: no model, no processes
    eng.config, eng.worker, eng.scheduler, eng.stats = cfg, FakeWorker(modulus), Scheduler(cfg), EngineStats()
    eng.chan, eng.procs, eng.launcher_mode, eng._closed, eng._trace = None, [], False, False, None
    eng._nvtx, eng._nvtx_open, eng.step_index, eng.tokenizer, eng.rank = False, False, 0, None, 0
    eng.decode_builder = DecodeBuilder(cfg.kvcache_block_size)
    return eng


workload = st.lists(st.tuples(st.lists(st.integers(0, 50), min_size=1, max_size=30), st.integers(1, 24)), min_size=1, max_size=10)


@settings(max_examples=100, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(reqs=workload, num_blocks=st.integers(10, 30), max_seqs=st.integers(1, 6), shared=st.booleans(),
       budget=st.sampled_from([128, 128, 16, 24]))
def test_pipelined_loop_matches_plain_loop(reqs, num_blocks, max_seqs, shared, budget):
    if shared:                                    # a common prefix, so that blocks are shared and revived
        reqs = [([7, 7, 7, 7, 9, 9, 9, 9, 1, 2, 3, 4, 5, 6, 7, 8] + p, m) for p, m in reqs]
    results = []
    for pipelined in (True, False):
        # the pipelined engine may also prefill long prompts in chunks (a small token budget); the plain one never does
        eng = make_engine(num_blocks, max_seqs, pipelined, budget if pipelined else 128)
        prompts = [p for p, _ in reqs]
        sps = [SamplingParams(temperature=0.0, max_tokens=m, ignore_eos=True) for _, m in reqs]
        outs = eng.generate(prompts, sps, use_tqdm=False)
        pool = eng.scheduler.pool
        pool.check_invariants()
        assert pool.num_free == pool.num_blocks and eng.scheduler.is_finished()
        assert [len(o["token_ids"]) for o in outs] == [m for _, m in reqs]
        # a second call that extends the first request's text must find consistent cached blocks (hashes of known tokens only)
        again = eng.generate([prompts[0] + outs[0]["token_ids"]], SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True), use_tqdm=False)
        results.append(([o["token_ids"] for o in outs], again[0]["token_ids"], eng.stats.preemptions))
    assert results[0][0] == results[1][0]
    assert results[0][1] == results[1][1]


@settings(max_examples=100, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(reqs=workload, num_blocks=st.integers(10, 30), max_seqs=st.integers(1, 6), shared=st.booleans(),
       budget=st.sampled_from([128, 128, 16, 24]), eos=st.integers(0, 6), some_ignore=st.booleans())
def test_pipelined_loop_matches_plain_loop_when_requests_stop_on_eos(reqs, num_blocks, max_seqs, shared, budget, eos, some_ignore):
    """Tokens come from [0, 7), so the EOS id is hit about every seventh token: most requests stop on it, at random
    steps, often several in one step, sometimes in the step in which they would have reached max_tokens anyway."""
    if shared:
        reqs = [([7, 7, 7, 7, 9, 9, 9, 9, 1, 2, 3, 4, 5, 6, 7, 8] + p, m) for p, m in reqs]
    results = []
    for pipelined in (True, False):
        eng = make_engine(num_blocks, max_seqs, pipelined, budget if pipelined else 128, eos=eos, modulus=7)
        prompts = [p for p, _ in reqs]
        sps = [SamplingParams(temperature=0.0, max_tokens=m, ignore_eos=some_ignore and i % 3 == 0) for i, (_, m) in enumerate(reqs)]
        outs = eng.generate(prompts, sps, use_tqdm=False)
        pool = eng.scheduler.pool
        pool.check_invariants()
        assert pool.num_free == pool.num_blocks and eng.scheduler.is_finished()
        for o, sp in zip(outs, sps):
            toks = o["token_ids"]
            assert 1 <= len(toks) <= sp.max_tokens and all(0 <= t < 7 for t in toks)
            if not sp.ignore_eos:
                assert eos not in toks[:-1]                              # nothing after the first EOS
                assert toks[-1] == eos or len(toks) == sp.max_tokens
        # blocks sealed for the prefix cache hold only tokens that were read back: extending a finished text hits consistently
        again = eng.generate([prompts[0] + outs[0]["token_ids"]], SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True), use_tqdm=False)
        results.append(([o["token_ids"] for o in outs], again[0]["token_ids"]))
    assert results[0] == results[1]


def test_a_kernel_error_in_the_last_step_of_a_call_raises_from_that_call():
    """The worker checks the kernels' status word with every step it collects, the final drain included: an error in the
    very last decode step of generate() must surface from that call, not from the next one."""
    from tinyllmforge_b200.engine.engine import EngineDeadError
    for pipelined in (True, False):
        eng = make_engine(30, 4, pipelined)
        eng.worker.fail_at = 1 + 5                  # one prefill step + five decode steps: the last step of the call below
        with pytest.raises((EngineDeadError, RuntimeError), match="CUDA kernel reported"):
            eng.generate([[1, 2, 3]], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True), use_tqdm=False)
