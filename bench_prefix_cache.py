"""Prefix-cache workload: R requests share one P-token random prefix, each followed by a distinct S-token suffix,
O output tokens each (defaults 128 x (4096 + 256) -> 256 on the Qwen3-8B architecture).  Reports the prefill tokens
skipped through hash-based block reuse and end-to-end output tokens/s, with the cache warm (the shared prefix was
prefilled by an earlier request, as in a serving system) and cold.

    python bench_prefix_cache.py [--model qwen3-8b] [--gpus N] [--requests 128] [--prefix 4096] [--suffix 256] [--out 256]

With --gpus N > 1 launch under torchrun (one rank per GPU), like bench.py.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from random import Random

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--requests", type=int, default=128)
    ap.add_argument("--prefix", type=int, default=4096)
    ap.add_argument("--suffix", type=int, default=256)
    ap.add_argument("--out", type=int, default=256)
    args = ap.parse_args()
    import torch
    from tinyllmforge_b200 import LLM, SamplingParams, preset

    rank = int(os.environ.get("RANK", "0")) if args.gpus > 1 else 0
    rng = Random(0)
    prefix = [rng.randrange(10000) for _ in range(args.prefix)]
    prompts = [prefix + [rng.randrange(10000) for _ in range(args.suffix)] for _ in range(args.requests)]
    sp = SamplingParams(temperature=0.6, max_tokens=args.out, ignore_eos=True)
    max_len = args.prefix + args.suffix + args.out + 256
    llm = LLM(args.model, hf_config=preset(args.model), load_format="dummy", skip_tokenizer_init=True,
              tensor_parallel_size=args.gpus, max_model_len=max_len, max_num_batched_tokens=max(16384, max_len),
              max_num_seqs=max(args.requests, 16))
    results = {}
    llm.generate(prompts[:2], SamplingParams(temperature=0.6, max_tokens=4, ignore_eos=True), use_tqdm=False)   # warm-up + fills the cache
    for name in ("warm", "cold"):
        if name == "cold" and rank == 0:       # forget every cached block
            pool = llm.scheduler.pool
            pool.hash_to_block.clear()
            pool.block_hash = [-1] * pool.num_blocks
        before = llm.stats.prefix_cached_tokens if rank == 0 else 0
        computed_before = llm.stats.prefill_tokens if rank == 0 else 0
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        llm.generate(prompts, sp, use_tqdm=False)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        if rank == 0:
            results[name] = {"seconds": round(dt, 3), "output_tok_per_s": round(args.requests * args.out / dt, 1),
                             "prefill_tokens_skipped": llm.stats.prefix_cached_tokens - before,
                             "prefill_tokens_computed": llm.stats.prefill_tokens - computed_before}
    if rank == 0:
        print(json.dumps({"workload": vars(args), "total_prompt_tokens": args.requests * (args.prefix + args.suffix), **results}))
    llm.exit()


if __name__ == "__main__":
    main()
