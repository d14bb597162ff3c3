"""Headline benchmark: the reference's ``bench.py`` workload (256 random-token requests, prompt and output
lengths uniform in [100, 1024], temperature 0.6, ignore_eos) on a random-init Qwen3 architecture.

    python bench.py --gpus N --steps K --warmup W [--model qwen3-0.6b] [--impl ours|reference]

One "step" is one complete ``LLM.generate`` pass over the 256 requests (the reference's timed region,
bench.py:54-56).  Metric: output tokens per second = K * sum(max_tokens) / time.

* ``value``: device-timed.  Every engine step (host-to-device copy of the packed step inputs, forward,
  sampling, device-to-host copy of the tokens) is bracketed by CUDA events on the launching stream; the
  per-step times are summed per rank and the maximum over ranks is taken.
* ``e2e``: wall clock of the same ``generate`` calls through the public API, i.e. additionally the
  scheduler, step building, control-plane publishing and output assembly.

With N > 1 (launched by torchrun, one rank per GPU) the model runs tensor-parallel over the N GPUs.
``--impl reference`` runs the unmodified reference engine from ``baseline/_ref`` on the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from random import randint, seed

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

NUM_SEQS, MAX_IN, MAX_OUT = 256, 1024, 1024


def make_workload():
    """Same draw order as the reference's bench.py:40-49."""
    seed(0)
    prompts = [[randint(0, 10000) for _ in range(randint(100, MAX_IN))] for _ in range(NUM_SEQS)]
    max_tokens = [randint(100, MAX_OUT) for _ in range(NUM_SEQS)]
    return prompts, max_tokens


def prompts_for_pass(prompts, p: int):
    """Pass p of the benchmark: the same lengths (the same work), different token ids, so that the prefix cache
    cannot serve one pass from the blocks of an earlier one.  Pass 0 is the reference's workload verbatim."""
    if p == 0:
        return prompts
    return [[(t + 7919 * p) % 10001 for t in q] for q in prompts]


# ---------------------------------------------------------------------------------------------- clocks
class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        self.gpu = gpu_index
        self.path = f"/tmp/clocks_{os.getpid()}.csv"

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(self.gpu)], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                p = [x.strip() for x in line.split(",")]
                if len(p) < 9:
                    continue
                try:
                    sm.append(float(p[1]))
                    mx.append(float(p[2]))
                except ValueError:
                    continue
                for name, val in zip(names, p[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        os.unlink(self.path)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------- checkpoint
def ensure_checkpoint(model: str, rank: int) -> str:
    """Seeded random-init checkpoint (config.json + safetensors + offline tokenizer) under /tmp, written once."""
    from tinyllmforge_b200 import preset
    from tinyllmforge_b200.utils.synth import write_checkpoint
    path = os.environ.get("FORGE_BENCH_CKPT", f"/tmp/forge_ckpt_{model}")
    done = os.path.join(path, "DONE")
    if rank == 0 and not os.path.exists(done):
        write_checkpoint(path, preset(model), seed=0)
        open(done, "w").close()
    t0 = time.time()
    while not os.path.exists(done):
        if time.time() - t0 > 1800:
            raise RuntimeError("timed out waiting for rank 0 to write the checkpoint")
        time.sleep(0.5)
    return path


def max_over_ranks(x: float, n: int) -> float:
    if n == 1:
        return x
    import torch
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


# ---------------------------------------------------------------------------------------------- our engine
def run_ours(args) -> dict:
    import torch
    from tinyllmforge_b200 import LLM, SamplingParams, preset

    n = args.gpus
    rank = int(os.environ.get("RANK", "0")) if n > 1 else 0
    prompts, max_tokens = make_workload()
    sps = [SamplingParams(temperature=0.6, ignore_eos=True, max_tokens=m) for m in max_tokens]
    kw = dict(enforce_eager=False, max_model_len=4096, tensor_parallel_size=n, comm=args.comm, extra={"device_timing": True})
    if args.quantization != "none":
        kw["quantization"] = args.quantization
    if args.load == "dummy":
        llm = LLM(args.model, hf_config=preset(args.model), load_format="dummy", skip_tokenizer_init=True, **kw)
    else:
        llm = LLM(ensure_checkpoint(args.model, rank), **kw)
    worker = llm.worker

    passes = iter(range(1 << 30))

    def one_pass():
        return llm.generate(prompts_for_pass(prompts, next(passes)), sps, use_tqdm=False)

    for _ in range(args.warmup):
        one_pass()
    torch.cuda.synchronize()
    if n > 1:
        torch.distributed.barrier()
    sampler = ClockSampler(torch.cuda.current_device())
    if rank == 0:
        sampler.start()
    worker.reset_counters()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        outs = one_pass()
    torch.cuda.synchronize()
    if n > 1:
        torch.distributed.barrier()
    wall = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else None
    dev_ms = max_over_ranks(worker.device_ms, n)
    wall = max_over_ranks(wall, n)
    result = None
    if rank == 0:
        assert all(len(o["token_ids"]) == m for o, m in zip(outs, max_tokens))
        total = args.steps * sum(max_tokens)
        st = llm.stats
        result = {
            "metric": "output_tokens_per_second", "value": total / (dev_ms / 1e3), "unit": "tok/s", "n_gpus": n,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16" if args.quantization == "none" else "bf16 activations, fp8 e4m3 block-scaled weights",
            "data": "synthetic", "impl": "ours",
            "config": {"model": args.model, "global_batch": NUM_SEQS, "seq_len": "prompt U[100,1024] + output U[100,1024]",
                       "parallelism": f"tp{n}", "comm": args.comm if n > 1 else "none", "weights": "random-init N(0,0.02), seed 0", "step": "one generate() pass over 256 requests; every pass uses fresh token ids of the same lengths (no cross-pass prefix-cache hits)",
                       "l2": "inputs larger than L2: every engine step streams the weights and the KV cache (> 126 MB)",
                       "timing": "value: sum of per-engine-step CUDA-event times, max over ranks; e2e: wall clock of generate()"},
            "e2e": {"value": total / wall, "unit": "tok/s", "h2d_bytes_per_step": worker.h2d_bytes // args.steps,
                    "d2h_bytes_per_step": worker.d2h_bytes // args.steps, "wall_s_per_step": wall / args.steps},
            "gpu_launches": worker.kernel_launches,
            "engine_steps_per_pass": (st.prefill_steps + st.decode_steps) // (args.steps + args.warmup),
            "clocks": clocks,
        }
    llm.exit()
    return result


# ---------------------------------------------------------------------------------------------- reference engine
def run_reference(args) -> dict:
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "tinyvllm")):
        return {"impl": "reference", "unavailable": "baseline/_ref/tinyvllm is not installed"}
    n = args.gpus
    rank = int(os.environ.get("RANK", "0")) if n > 1 else 0
    if n > 1 and rank != 0:
        return None            # the reference spawns its own worker processes from rank 0; the launcher's other ranks stand by
    import torch
    sys.path.insert(0, ref_dir)
    shims = []
    try:
        # The reference was written against transformers 4.x, where a Qwen3 config has `rope_theta` and
        # `rope_scaling is None`.  transformers 5.x folds both into a `rope_parameters` dict, which the
        # reference then passes to an lru_cache'd function (unhashable) and asserts to be None.  Give the
        # loaded config object its 4.x attribute names back; the reference's own files stay untouched.
        import transformers
        if int(transformers.__version__.split(".")[0]) >= 5:
            orig_from_pretrained = transformers.AutoConfig.from_pretrained

            def from_pretrained_compat(*a, **k):
                cfg = orig_from_pretrained(*a, **k)
                rp = getattr(cfg, "rope_parameters", None) or {}
                theta = rp.get("rope_theta", 1000000.0)
                cfg.rope_scaling = None
                cfg.rope_theta = theta
                return cfg
            transformers.AutoConfig.from_pretrained = from_pretrained_compat
            shims.append("transformers>=5 config: restored legacy rope_theta / rope_scaling=None attributes")
        from tinyvllm import LLM, SamplingParams
        from tinyvllm.engine.model_runner import ModelRunner
        if n > 1:
            # as written the reference cannot start with more than one GPU: repair the four spots in memory
            from baseline import ref_repairs
            shims += ["TP>1 run-time repairs: " + r for r in ref_repairs.apply()]
    except Exception as e:  # missing dependency of the reference
        return {"impl": "reference", "unavailable": f"import failed: {type(e).__name__}: {e}"}
    path = ensure_checkpoint(args.model, 0)
    prompts, max_tokens = make_workload()
    sps = [SamplingParams(temperature=0.6, ignore_eos=True, max_tokens=m) for m in max_tokens]

    # timing instrumentation only: CUDA events around the reference's own per-step device work
    acc = {"ms": 0.0, "steps": 0, "h2d": 0, "d2h": 0}
    orig_run = ModelRunner.run

    def timed_run(self, seqs, is_prefill):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = orig_run(self, seqs, is_prefill)
        e1.record()
        e1.synchronize()
        acc["ms"] += e0.elapsed_time(e1)
        acc["steps"] += 1
        ntok = sum(len(s) - s.num_cached_tokens for s in seqs) if is_prefill else len(seqs)
        acc["h2d"] += ntok * 20 + len(seqs) * 8        # ids + positions (int64), slots (int32), lens, temperatures
        acc["d2h"] += len(seqs) * 8
        return out

    ModelRunner.run = timed_run
    # Under torchrun the reference's own rendezvous ("tcp://localhost:2333", rank 0 hosts the store) would be turned
    # into a client of the launcher's agent store by these variables; the reference is its own launcher.
    for k in [k for k in os.environ if k.startswith("TORCHELASTIC")]:
        os.environ.pop(k)

    def kill_children():
        try:
            import psutil
            for c in psutil.Process(os.getpid()).children(recursive=True):
                c.kill()
        except Exception:
            pass

    def give_up(what, limit):    # watchdogs: never sit in a rendezvous or a lost collective until the caller's limit
        print(json.dumps({"impl": "reference", "unavailable": f"the reference engine did not {what} within {limit:.0f} s"}), flush=True)
        kill_children()
        os._exit(0)
    import threading
    watchdog = threading.Timer(args.ref_start_timeout, give_up, ("start", args.ref_start_timeout))
    watchdog.daemon = True
    watchdog.start()
    try:
        llm = LLM(path, enforce_eager=False, max_model_len=4096, tensor_parallel_size=n)
        watchdog.cancel()
        watchdog = threading.Timer(args.ref_run_timeout, give_up, ("finish its passes", args.ref_run_timeout))
        watchdog.daemon = True
        watchdog.start()
        for p in range(args.warmup):
            llm.generate(prompts_for_pass(prompts, p), sps, use_tqdm=False)
        torch.cuda.synchronize()
        sampler = ClockSampler(torch.cuda.current_device())
        sampler.start()
        acc.update(ms=0.0, steps=0, h2d=0, d2h=0)
        t0 = time.perf_counter()
        for p in range(args.steps):
            outs = llm.generate(prompts_for_pass(prompts, args.warmup + p), sps, use_tqdm=False)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        clocks = sampler.stop()
        watchdog.cancel()
    except Exception as e:       # the reference's own code failed (it has no error handling of its own): report, do not crash
        watchdog.cancel()
        kill_children()
        return {"impl": "reference", "unavailable": f"the reference engine failed: {type(e).__name__}: {str(e)[:300]}", "shims": shims}
    total = args.steps * sum(max_tokens)
    return {
        "metric": "output_tokens_per_second", "value": total / (acc["ms"] / 1e3), "unit": "tok/s", "n_gpus": n,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": acc["ms"] / args.steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "reference",
        "config": {"model": args.model, "global_batch": NUM_SEQS, "seq_len": "prompt U[100,1024] + output U[100,1024]",
                   "parallelism": f"tp{n}", "weights": "random-init N(0,0.02), seed 0", "step": "one generate() pass over 256 requests; every pass uses fresh token ids of the same lengths (no cross-pass prefix-cache hits)",
                   "l2": "inputs larger than L2", "timing": "value: CUDA events around ModelRunner.run on rank 0 (every step ends in a "
                   "collective and a host sync, so rank 0 spans the slowest rank), summed; e2e: wall clock of generate()"},
        "e2e": {"value": total / wall, "unit": "tok/s", "h2d_bytes_per_step": acc["h2d"] // args.steps,
                "d2h_bytes_per_step": acc["d2h"] // args.steps, "wall_s_per_step": wall / args.steps},
        "engine_steps_per_pass": acc["steps"] // args.steps, "clocks": clocks, "shims": shims,
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default=os.environ.get("FORGE_BENCH_MODEL", "qwen3-0.6b"))
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"],
                    help="tensor-parallel exchange: in-kernel NVLink pushes (fused) or torch.distributed/NCCL calls")
    ap.add_argument("--ref-start-timeout", type=float, default=300.0, help="seconds the reference engine gets to start")
    ap.add_argument("--ref-run-timeout", type=float, default=1500.0, help="seconds the reference engine gets for all its passes")
    ap.add_argument("--quantization", default="none", choices=["none", "fp8_block"],
                    help="fp8_block: e4m3 weights with 128 x 128 block scales for the four projections of every layer (not the headline)")
    ap.add_argument("--load", default="auto", choices=["auto", "dummy"],
                    help="auto: write and load a safetensors checkpoint; dummy: random-init on the device (large models)")
    args = ap.parse_args()
    out = run_reference(args) if args.impl == "reference" else run_ours(args)
    if out is not None:
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
