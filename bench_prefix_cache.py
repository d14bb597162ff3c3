"""Prefix-cache workload: R requests share one P-token random prefix, each followed by a distinct S-token suffix,
O output tokens each (defaults 128 x (4096 + 256) -> 256 on the Qwen3-8B architecture).  Reports the prefill tokens
skipped through hash-based block reuse and output tokens/s (device-timed engine steps, max over ranks, and end to end),
with the cache warm (the shared prefix was prefilled by an earlier request, as in a serving system) and cold.

    python bench_prefix_cache.py [--model qwen3-8b] [--gpus N] [--requests 128] [--prefix 4096] [--suffix 256] [--out 256]
                                 [--impl ours|reference]

With --gpus N > 1 launch under torchrun (one rank per GPU), like bench.py.  ``--impl reference`` runs the reference
engine from ``baseline/_ref`` (its prefix cache is always on: tinyvllm/engine/block_manager.py:66-98) on the same
requests, with a safetensors checkpoint of the architecture written under /tmp.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from random import Random

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def make_prompts(args):
    rng = Random(0)
    prefix = [rng.randrange(10000) for _ in range(args.prefix)]
    return [prefix + [rng.randrange(10000) for _ in range(args.suffix)] for _ in range(args.requests)]


def run_ours(args, prompts, max_len):
    import torch
    from bench import max_over_ranks
    from tinyllmforge_b200 import LLM, SamplingParams, preset
    n = args.gpus
    rank = int(os.environ.get("RANK", "0")) if n > 1 else 0
    sp = SamplingParams(temperature=0.6, max_tokens=args.out, ignore_eos=True)
    llm = LLM(args.model, hf_config=preset(args.model), load_format="dummy", skip_tokenizer_init=True,
              tensor_parallel_size=n, max_model_len=max_len, max_num_batched_tokens=max(16384, max_len),
              max_num_seqs=max(args.requests, 16), comm=args.comm, extra={"device_timing": True})
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
        if n > 1:
            torch.distributed.barrier()
        llm.worker.reset_counters()
        t0 = time.perf_counter()
        llm.generate(prompts, sp, use_tqdm=False)
        torch.cuda.synchronize()
        dt = max_over_ranks(time.perf_counter() - t0, n)
        dev = max_over_ranks(llm.worker.device_ms, n) / 1e3
        if rank == 0:
            results[name] = {"seconds": round(dt, 3), "output_tok_per_s": round(args.requests * args.out / dt, 1),
                             "device_seconds": round(dev, 3), "output_tok_per_s_device": round(args.requests * args.out / dev, 1),
                             "prefill_tokens_skipped": llm.stats.prefix_cached_tokens - before,
                             "prefill_tokens_computed": llm.stats.prefill_tokens - computed_before}
    llm.exit()
    return results if rank == 0 else None


def run_reference(args, prompts, max_len):
    from bench import ReferenceHarness, ensure_checkpoint
    n = args.gpus
    if n > 1 and int(os.environ.get("RANK", "0")) != 0:
        return None
    import torch
    h = ReferenceHarness(n, 600.0, 900.0)
    try:
        LLM, SamplingParams = h.load()
        path = ensure_checkpoint(args.model, 0)
    except Exception as e:
        return {"unavailable": f"{type(e).__name__}: {e}"}
    sp = SamplingParams(temperature=0.6, max_tokens=args.out, ignore_eos=True)
    results = {"shims": h.shims}
    h.arm("start", h.start_timeout)
    try:
        llm = LLM(path, enforce_eager=False, max_model_len=max_len, max_num_batched_tokens=max(16384, max_len),
                  max_num_seqs=max(args.requests, 16), tensor_parallel_size=n)
        h.arm("finish its passes", h.run_timeout)
        llm.generate(prompts[:2], SamplingParams(temperature=0.6, max_tokens=4, ignore_eos=True), use_tqdm=False)
        for name in ("warm", "cold"):
            if name == "cold":                 # forget every cached block (tinyvllm/engine/block_manager.py:26-32)
                bm = llm.scheduler.block_manager
                bm.hash_to_block_id.clear()
                for b in bm.blocks:
                    b.hash = -1
            torch.cuda.synchronize()
            h.reset()
            t0 = time.perf_counter()
            llm.generate(prompts, sp, use_tqdm=False)
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            dev = h.acc["ms"] / 1e3
            computed = sum(t for p, _, t, _ in h.step_times if p)
            results[name] = {"seconds": round(dt, 3), "output_tok_per_s": round(args.requests * args.out / dt, 1),
                             "device_seconds": round(dev, 3), "output_tok_per_s_device": round(args.requests * args.out / dev, 1),
                             "prefill_tokens_skipped": h.acc["cached"], "prefill_tokens_computed": computed}
        h.disarm()
    except Exception as e:
        h.disarm()
        h.kill_children()
        return {"unavailable": f"the reference engine failed: {type(e).__name__}: {str(e)[:300]}", "shims": h.shims}
    return results


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--requests", type=int, default=128)
    ap.add_argument("--prefix", type=int, default=4096)
    ap.add_argument("--suffix", type=int, default=256)
    ap.add_argument("--out", type=int, default=256)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"])
    args = ap.parse_args()
    prompts = make_prompts(args)
    max_len = args.prefix + args.suffix + args.out + 256
    res = run_reference(args, prompts, max_len) if args.impl == "reference" else run_ours(args, prompts, max_len)
    if res is not None:
        print(json.dumps({"impl": args.impl, "workload": vars(args), "total_prompt_tokens": args.requests * (args.prefix + args.suffix), **res}), flush=True)


if __name__ == "__main__":
    main()
