"""Decode-heavy workload on a large architecture: R requests of P random prompt tokens and O output tokens each (defaults
64 x (2048 in, 512 out) on the Qwen3-32B architecture, random-init weights), bf16 or block-scaled fp8 weights.  Reports
output tokens/s (device time of the engine steps, max over ranks; and end to end), and the mean decode step time.

    python bench_decode.py [--model qwen3-32b] [--gpus N] [--requests 64] [--prompt 2048] [--out 512]
                           [--quantization fp8_block] [--impl ours|reference]

With --gpus N > 1 launch under torchrun (one rank per GPU), like bench.py.  ``--impl reference`` runs the reference
engine from ``baseline/_ref`` on the same requests (bf16 only; its weights are initialised on the device instead of
being read from a 64 GB checkpoint, which the result line lists under "shims").
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from random import Random

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def make_prompts(args, p):          # fresh token ids per pass: no prefix-cache hits across passes
    rng = Random(p)
    return [[rng.randrange(10000) for _ in range(args.prompt)] for _ in range(args.requests)]


def summary(args, total, dev_ms, wall, step_times, extra):
    from bench import step_breakdown
    return {"impl": args.impl, "workload": vars(args), "output_tok_per_s_device": round(total / (dev_ms / 1e3), 1),
            "output_tok_per_s_end_to_end": round(total / wall, 1), "device_s_per_pass": round(dev_ms / 1e3 / args.passes, 3),
            **step_breakdown(step_times), **extra}


def run_ours(args, max_len):
    import torch
    from bench import max_over_ranks
    from tinyllmforge_b200 import LLM, SamplingParams, preset
    n = args.gpus
    rank = int(os.environ.get("RANK", "0")) if n > 1 else 0
    kw = dict(tensor_parallel_size=n, max_model_len=max_len, max_num_batched_tokens=max(16384, max_len),
              max_num_seqs=max(args.requests, 16), comm=args.comm, extra={"device_timing": True})
    if args.quantization != "none":
        kw["quantization"] = args.quantization
    llm = LLM(args.model, hf_config=preset(args.model), load_format="dummy", skip_tokenizer_init=True, **kw)
    sp = SamplingParams(temperature=0.6, max_tokens=args.out, ignore_eos=True)
    for p in range(args.warmup):
        llm.generate(make_prompts(args, p)[:max(2, args.requests // 8)], SamplingParams(temperature=0.6, max_tokens=8, ignore_eos=True), use_tqdm=False)
    torch.cuda.synchronize()
    if n > 1:
        torch.distributed.barrier()
    llm.worker.reset_counters()
    t0 = time.perf_counter()
    for p in range(args.passes):
        llm.generate(make_prompts(args, 100 + p), sp, use_tqdm=False)
    torch.cuda.synchronize()
    if n > 1:
        torch.distributed.barrier()
    wall = max_over_ranks(time.perf_counter() - t0, n)
    dev_ms = max_over_ranks(llm.worker.device_ms, n)
    res = None
    if rank == 0:
        res = summary(args, args.passes * args.requests * args.out, dev_ms, wall, llm.worker.step_times,
                      {"gpu_launches": llm.worker.kernel_launches})
    llm.exit()
    return res


def run_reference(args, max_len):
    from bench import ReferenceHarness
    n = args.gpus
    if n > 1 and int(os.environ.get("RANK", "0")) != 0:
        return None
    if args.quantization != "none":
        return {"impl": "reference", "unavailable": "the reference has no fp8 path"}
    import torch
    from tinyllmforge_b200 import preset
    from tinyllmforge_b200.utils.synth import write_checkpoint
    h = ReferenceHarness(n, 600.0, 900.0)
    try:
        LLM, SamplingParams = h.load()
        from baseline import ref_repairs
        os.environ["FORGE_REF_DUMMY_LOAD"] = "1"             # read by the spawned workers of a TP > 1 run
        h.shims.append(ref_repairs.apply_dummy_load())
        path = write_checkpoint(f"/tmp/forge_cfg_{args.model}", preset(args.model), weights=False)
    except Exception as e:
        return {"impl": "reference", "unavailable": f"{type(e).__name__}: {e}"}
    sp = SamplingParams(temperature=0.6, max_tokens=args.out, ignore_eos=True)
    h.arm("start", h.start_timeout)
    try:
        llm = LLM(path, enforce_eager=False, max_model_len=max_len, max_num_batched_tokens=max(16384, max_len),
                  max_num_seqs=max(args.requests, 16), tensor_parallel_size=n)
        h.arm("finish its passes", h.run_timeout)
        for p in range(args.warmup):
            llm.generate(make_prompts(args, p)[:max(2, args.requests // 8)], SamplingParams(temperature=0.6, max_tokens=8, ignore_eos=True), use_tqdm=False)
        torch.cuda.synchronize()
        h.reset()
        t0 = time.perf_counter()
        for p in range(args.passes):
            llm.generate(make_prompts(args, 100 + p), sp, use_tqdm=False)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        h.disarm()
    except Exception as e:
        h.disarm()
        h.kill_children()
        return {"impl": "reference", "unavailable": f"the reference engine failed: {type(e).__name__}: {str(e)[:300]}", "shims": h.shims}
    return summary(args, args.passes * args.requests * args.out, h.acc["ms"], wall, h.step_times, {"shims": h.shims})


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-32b")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--out", type=int, default=512)
    ap.add_argument("--passes", type=int, default=1)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--quantization", default="none", choices=["none", "fp8_block"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()
    max_len = args.prompt + args.out + 64
    res = run_reference(args, max_len) if args.impl == "reference" else run_ours(args, max_len)
    if res is not None:
        print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
