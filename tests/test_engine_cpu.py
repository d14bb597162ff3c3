"""End to end on CPU: the tiny Qwen3 architecture (2 layers, hidden 256, 4/2 heads of 64, vocab 4096, fp32),
KV block size 16, 4 random prompts of 16..64 tokens, 32 greedy tokens each.

* TP=1 reproduces a plain Hugging Face greedy loop token for token.
* TP=2 over gloo (two processes, shared-memory control channel) reproduces TP=1.
* prefix caching, preemption and sampling behave as specified.
* a follower that dies is reported as EngineDeadError (failure made on the host: the process exits).
"""
import os
import random
import signal
import time

import pytest
import torch

from tinyllmforge_b200 import LLM, SamplingParams, preset
from tinyllmforge_b200.engine.engine import EngineDeadError
from tinyllmforge_b200.utils.synth import write_checkpoint


@pytest.fixture(scope="module")
def ckpt(tmp_path_factory):
    path = str(tmp_path_factory.mktemp("tiny_e2e"))
    write_checkpoint(path, preset("tiny"), seed=0, std=0.2, norm_std=0.1)
    return path


@pytest.fixture(scope="module")
def prompts():
    rng = random.Random(0)
    return [[rng.randrange(4096) for _ in range(rng.randint(16, 64))] for _ in range(4)]


def _llm(ckpt, **kw):
    base = dict(kvcache_block_size=16, device="cpu", max_model_len=512, max_num_batched_tokens=512, num_kvcache_blocks=96)
    base.update(kw)
    return LLM(ckpt, **base)


GREEDY = SamplingParams(temperature=0.0, max_tokens=32, ignore_eos=True)


@pytest.fixture(scope="module")
def tp1_tokens(ckpt, prompts):
    llm = _llm(ckpt)
    outs = llm.generate(prompts, GREEDY, use_tqdm=False)
    stats = llm.stats.to_dict()
    llm.exit()
    return [o["token_ids"] for o in outs], stats


def test_tp1_matches_transformers_greedy(ckpt, prompts, tp1_tokens):
    from transformers import AutoModelForCausalLM
    hf = AutoModelForCausalLM.from_pretrained(ckpt, dtype=torch.float32).eval()
    toks, stats = tp1_tokens
    for p, got in zip(prompts, toks):
        ids = list(p)
        with torch.no_grad():
            for _ in range(32):
                ids.append(int(hf(torch.tensor([ids])).logits[0, -1].argmax()))
        assert got == ids[len(p):]
    assert len({tuple(t) for t in toks}) > 1 and all(len(set(t)) > 4 for t in toks)      # not degenerate
    assert stats["prefill_steps"] == 1 and stats["decode_steps"] == 31 and stats["decode_tokens"] == 4 * 31


def test_tp2_gloo_matches_tp1(ckpt, prompts, tp1_tokens):
    llm = _llm(ckpt, tensor_parallel_size=2)
    try:
        outs = llm.generate(prompts, GREEDY, use_tqdm=False)
        assert [o["token_ids"] for o in outs] == tp1_tokens[0]
        # a second call on the same engine (followers stay alive between calls)
        outs2 = llm.generate(prompts[:2], GREEDY, use_tqdm=False)
        assert [o["token_ids"] for o in outs2] == tp1_tokens[0][:2]
    finally:
        llm.exit()
    assert all(not p.is_alive() for p in llm.procs)


def test_prefix_cache_skips_shared_prompt_and_keeps_tokens(ckpt):
    rng = random.Random(1)
    shared = [rng.randrange(4096) for _ in range(48)]
    ps = [shared + [rng.randrange(4096) for _ in range(8)] for _ in range(3)]
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    llm = _llm(ckpt)
    first = llm.generate([ps[0]], sp, use_tqdm=False)              # populates the cache
    rest = llm.generate(ps, sp, use_tqdm=False)
    assert llm.stats.prefix_cached_tokens == 3 * 48
    assert rest[0]["token_ids"] == first[0]["token_ids"]
    llm.exit()
    cold = _llm(ckpt)
    want = cold.generate(ps, sp, use_tqdm=False)
    cold.exit()
    assert [o["token_ids"] for o in rest] == [o["token_ids"] for o in want]


def test_preemption_recomputes_and_keeps_tokens(ckpt, prompts, tp1_tokens):
    need = max(-(-(len(p) + 32) // 16) for p in prompts)
    llm = _llm(ckpt, num_kvcache_blocks=need + 4)                   # far too small for four sequences at once
    outs = llm.generate(prompts, GREEDY, use_tqdm=False)
    assert llm.stats.preemptions > 0 or llm.stats.prefill_steps > 1
    assert [o["token_ids"] for o in outs] == tp1_tokens[0]
    llm.exit()


def test_sampling_is_seeded_and_temperature_matters(ckpt, prompts):
    sp = SamplingParams(temperature=1.0, max_tokens=16, ignore_eos=True)
    a = _llm(ckpt, seed=7)
    ta = [o["token_ids"] for o in a.generate(prompts, sp, use_tqdm=False)]
    a.exit()
    b = _llm(ckpt, seed=7)
    tb = [o["token_ids"] for o in b.generate(prompts, sp, use_tqdm=False)]
    b.exit()
    c = _llm(ckpt, seed=8)
    tc = [o["token_ids"] for o in c.generate(prompts, sp, use_tqdm=False)]
    c.exit()
    assert ta == tb and ta != tc


def test_eos_and_max_tokens_stop(ckpt, prompts, tp1_tokens):
    eos = tp1_tokens[0][0][5]                                       # sixth greedy token of request 0
    llm = _llm(ckpt, eos=eos, skip_tokenizer_init=True)
    out = llm.generate([prompts[0]], SamplingParams(temperature=0.0, max_tokens=32), use_tqdm=False)[0]["token_ids"]
    first = tp1_tokens[0][0].index(eos)
    assert out == tp1_tokens[0][0][:first + 1]
    out = llm.generate([prompts[0]], SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True), use_tqdm=False)
    assert out[0]["token_ids"] == tp1_tokens[0][0][:3]
    llm.exit()


def test_string_prompts_use_the_checkpoint_tokenizer(ckpt):
    llm = _llm(ckpt)
    out = llm.generate(["w1 w2 w3 w4"], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True), use_tqdm=False)
    assert len(out[0]["token_ids"]) == 4 and isinstance(out[0]["text"], str)
    llm.exit()


def test_dead_follower_is_reported_not_hung(ckpt, prompts):
    llm = _llm(ckpt, tensor_parallel_size=2, rpc_timeout_s=20)
    try:
        llm.generate(prompts[:1], SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True), use_tqdm=False)
        os.kill(llm.procs[0].pid, signal.SIGKILL)                   # between steps: nothing in flight
        llm.procs[0].join(10)
        t0 = time.monotonic()
        with pytest.raises(EngineDeadError):
            llm.generate(prompts, GREEDY, use_tqdm=False)
        assert time.monotonic() - t0 < 60
    finally:
        llm.exit()


def test_pipelined_loop_equals_step_by_step_loop(ckpt):
    """The loop that schedules step t+1 before it reads step t's tokens (used when no request can stop on a token
    value) must produce the same tokens as the plain loop: sampling, different lengths, a KV pool small enough to
    force preemption, and a prompt that shares a prefix produced by an earlier decode."""
    rng = random.Random(5)
    prompts = [[rng.randrange(4096) for _ in range(rng.randint(5, 70))] for _ in range(6)]
    sps = [SamplingParams(temperature=0.8 if i % 2 else 0.0, max_tokens=20 + 7 * i, ignore_eos=True) for i in range(6)]
    results = {}
    for pipelined in (True, False):
        llm = _llm(ckpt, num_kvcache_blocks=14, max_num_seqs=4, seed=3, extra={"pipeline": pipelined})
        outs = llm.generate(prompts, sps, use_tqdm=False)
        first = [o["token_ids"] for o in outs]
        # second call: prompt + completion of the first call -> its sealed decode blocks must be reusable and right
        again = llm.generate([prompts[0] + first[0]], SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True), use_tqdm=False)
        llm.scheduler.pool.check_invariants()
        results[pipelined] = (first, again[0]["token_ids"], llm.stats.to_dict())
        llm.exit()
    assert results[True][0] == results[False][0]
    assert results[True][1] == results[False][1]
    assert results[True][2]["preemptions"] > 0
    assert all(len(t) == sp.max_tokens for t, sp in zip(results[True][0], sps))
    assert all(tok >= 0 for t in results[True][0] for tok in t)


def test_step_trace_has_one_line_per_step(ckpt, prompts, tmp_path):
    """``trace_path``: one JSON line per engine step with the phase times, in the pipelined loop and in the plain one."""
    import json
    for pipelined in (True, False):
        path = str(tmp_path / f"trace_{pipelined}.jsonl")
        llm = _llm(ckpt, trace_path=path, extra={"pipeline": pipelined})
        llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True), use_tqdm=False)
        steps = llm.stats.prefill_steps + llm.stats.decode_steps
        llm.exit()
        lines = [json.loads(l) for l in open(path)]
        assert len(lines) == steps and [l["step"] for l in lines] == list(range(steps))
        assert lines[0]["prefill"] and not lines[-1]["prefill"] and all(l["run_ms"] >= 0 for l in lines)


def test_pipelined_loop_short_requests(ckpt, prompts):
    """Requests that finish on their first or second token (the step that produced the token is still in flight when the
    request is retired) and an empty follow-up call."""
    results = {}
    for pipelined in (True, False):
        llm = _llm(ckpt, seed=1, extra={"pipeline": pipelined})
        sps = [SamplingParams(temperature=0.0, max_tokens=1 + (i % 3), ignore_eos=True) for i in range(len(prompts))]
        outs = llm.generate(prompts, sps, use_tqdm=False)
        assert llm.generate([], [], use_tqdm=False) == []
        results[pipelined] = [o["token_ids"] for o in outs]
        assert llm.scheduler.pool.num_free == llm.scheduler.pool.num_blocks
        llm.exit()
    assert results[True] == results[False]
    assert [len(t) for t in results[True]] == [1 + (i % 3) for i in range(len(prompts))]


def test_chunked_prefill_matches_whole_prompt_prefill(ckpt):
    """A prompt longer than the token budget is prefilled in several steps (not in the reference, which rejects it): same
    tokens as with a budget that takes the prompt whole; a later prompt reuses the long prompt's blocks through the prefix
    cache; pipelined and plain loops agree."""
    rng = random.Random(9)
    long_prompt = [rng.randrange(4096) for _ in range(150)]
    prompts = [[rng.randrange(4096) for _ in range(20)], long_prompt, [rng.randrange(4096) for _ in range(33)],
               long_prompt[:100] + [rng.randrange(4096) for _ in range(70)]]
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    whole = _llm(ckpt, max_model_len=400)
    want = [o["token_ids"] for o in whole.generate(prompts, sp, use_tqdm=False)]
    whole.exit()
    with pytest.raises(ValueError):
        _llm(ckpt, max_model_len=400, max_num_batched_tokens=64)
    for pipelined in (True, False):
        llm = _llm(ckpt, max_model_len=400, max_num_batched_tokens=64, chunked_prefill=True, extra={"pipeline": pipelined})
        got = [o["token_ids"] for o in llm.generate(prompts, sp, use_tqdm=False)]
        st = llm.stats.to_dict()
        llm.scheduler.pool.check_invariants()
        assert llm.scheduler.pool.num_free == llm.scheduler.pool.num_blocks
        llm.exit()
        assert got == want
        assert st["prefill_steps"] >= 3 + 3 + 1               # 150 tokens and 170 tokens at 64 per step, plus the short ones
        assert st["prefix_cached_tokens"] >= 96                # the fourth prompt found the long prompt's first six blocks
