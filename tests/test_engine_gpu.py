"""The engine on one GPU: a 3-layer model with the Qwen3-0.6B layer shapes and random weights, through ``LLM.generate``.

* the loop that runs one step ahead of the GPU gives exactly the tokens of the plain loop (same kernels, same order);
* CUDA-graph replay agrees with eager execution;
* a prompt prefilled in chunks (longer than the token budget) and a prompt served from the prefix cache agree with the same
  prompt prefilled whole (different kernels' tile shapes: agreement of greedy tokens, not bit equality).
"""
import random

import pytest
import torch

pytestmark = pytest.mark.gpu


def _agree(a, b):
    return sum(x == y for s, t in zip(a, b) for x, y in zip(s, t)) / sum(len(s) for s in a)


@pytest.fixture(scope="module")
def setup():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from tinyllmforge_b200 import preset
    cfg = preset("qwen3-0.6b", num_hidden_layers=3, vocab_size=8192)
    rng = random.Random(0)
    prompts = [[rng.randrange(8192) for _ in range(rng.randint(20, 300))] for _ in range(10)]
    prompts.append([rng.randrange(8192) for _ in range(1300)])
    prompts.append(prompts[-1][:1024] + [rng.randrange(8192) for _ in range(100)])
    return cfg, prompts


def _run(cfg, prompts, **kw):
    from tinyllmforge_b200 import LLM, SamplingParams
    base = dict(hf_config=cfg, load_format="dummy", skip_tokenizer_init=True, max_model_len=2048, max_num_batched_tokens=4096,
                max_num_seqs=16, num_kvcache_blocks=96, gpu_memory_utilization=0.5)
    base.update(kw)
    llm = LLM("gpu-engine-test", **base)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=16, ignore_eos=True), use_tqdm=False)
    llm.worker.ops.check_status()
    stats = llm.stats.to_dict()
    llm.exit()
    return [o["token_ids"] for o in outs], stats


def test_engine_loops_graphs_chunks_and_prefix_cache_agree(setup):
    cfg, prompts = setup
    base, st = _run(cfg, prompts)
    assert all(len(t) == 16 for t in base)
    assert st["prefix_cached_tokens"] >= 1024                       # the last prompt reused the one before it
    plain, _ = _run(cfg, prompts, extra={"pipeline": False})
    assert plain == base
    eager, _ = _run(cfg, prompts, enforce_eager=True)
    assert _agree(eager, base) > 0.9
    chunked, st_c = _run(cfg, prompts, max_num_batched_tokens=512, chunked_prefill=True)
    assert st_c["prefill_steps"] > st["prefill_steps"]
    assert _agree(chunked, base) > 0.9
