"""Decode-heavy workload on a large architecture: R requests of P random prompt tokens and O output tokens each (defaults
64 x (2048 in, 512 out) on the Qwen3-32B architecture, random-init weights), bf16 or block-scaled fp8 weights.  Reports
output tokens/s (device time of the engine steps, max over ranks; and end to end), and the mean decode step time.

    python bench_decode.py [--model qwen3-32b] [--gpus N] [--requests 64] [--prompt 2048] [--out 512] [--quantization fp8_block]

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
    ap.add_argument("--model", default="qwen3-32b")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--out", type=int, default=512)
    ap.add_argument("--passes", type=int, default=1)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--quantization", default="none", choices=["none", "fp8_block"])
    args = ap.parse_args()
    import torch
    from bench import max_over_ranks
    from tinyllmforge_b200 import LLM, SamplingParams, preset

    n = args.gpus
    rank = int(os.environ.get("RANK", "0")) if n > 1 else 0
    max_len = args.prompt + args.out + 64
    kw = dict(tensor_parallel_size=n, max_model_len=max_len, max_num_batched_tokens=max(16384, max_len),
              max_num_seqs=max(args.requests, 16), comm=args.comm, extra={"device_timing": True})
    if args.quantization != "none":
        kw["quantization"] = args.quantization
    llm = LLM(args.model, hf_config=preset(args.model), load_format="dummy", skip_tokenizer_init=True, **kw)
    sp = SamplingParams(temperature=0.6, max_tokens=args.out, ignore_eos=True)

    def prompts(p):          # fresh token ids per pass: no prefix-cache hits across passes
        rng = Random(p)
        return [[rng.randrange(10000) for _ in range(args.prompt)] for _ in range(args.requests)]

    for p in range(args.warmup):
        llm.generate(prompts(p)[:max(2, args.requests // 8)], SamplingParams(temperature=0.6, max_tokens=8, ignore_eos=True), use_tqdm=False)
    torch.cuda.synchronize()
    if n > 1:
        torch.distributed.barrier()
    llm.worker.reset_counters()
    st0 = (llm.stats.prefill_steps, llm.stats.decode_steps)
    t0 = time.perf_counter()
    for p in range(args.passes):
        llm.generate(prompts(100 + p), sp, use_tqdm=False)
    torch.cuda.synchronize()
    if n > 1:
        torch.distributed.barrier()
    wall = max_over_ranks(time.perf_counter() - t0, n)
    dev_ms = max_over_ranks(llm.worker.device_ms, n)
    if rank == 0:
        total = args.passes * args.requests * args.out
        decode_steps = llm.stats.decode_steps - st0[1]
        print(json.dumps({"workload": vars(args), "output_tok_per_s_device": round(total / (dev_ms / 1e3), 1),
                          "output_tok_per_s_end_to_end": round(total / wall, 1), "device_s_per_pass": round(dev_ms / 1e3 / args.passes, 3),
                          "prefill_steps": llm.stats.prefill_steps - st0[0], "decode_steps": decode_steps,
                          "gpu_launches": llm.worker.kernel_launches}))
    llm.exit()


if __name__ == "__main__":
    main()
