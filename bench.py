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
* ``decode_step_ms`` / ``prefill_ms``: means of the per-step device times, overall and at decode batches of 256, ~64
  and 1 sequences; ``exposed_comm_pct`` (N > 1, this engine): share of the decode step time that disappears when the
  exchange kernels run on their own rank's data only (no waits, no peer traffic), measured on one extra pass.
* ``extras``: the same workload on the Qwen3-8B architecture at the same N (2 passes after 1 warm-up, in a child
  process before the headline run) and, at N = 8, the prefix-cache and the decode-heavy 32B workloads.

With N > 1 (launched by torchrun, one rank per GPU) the model runs tensor-parallel over the N GPUs.
``--impl reference`` runs the unmodified reference engine from ``baseline/_ref`` on the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import signal
import statistics
import subprocess
import sys
import threading
import time
from random import randint, seed

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

NUM_SEQS, MAX_IN, MAX_OUT = 256, 1024, 1024
HEADLINE_MODEL = "qwen3-0.6b"
T_START = time.monotonic()          # the run's time budget counts from here
MIN_CHILD_S = 45.0                   # an extra workload with less time left than this is skipped


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


def workload_config(model: str, n: int) -> dict:
    """The ``config`` entry of the result line: the same keys and values for both engines."""
    return {"model": model, "global_batch": NUM_SEQS, "seq_len": "prompt U[100,1024] + output U[100,1024]", "parallelism": f"tp{n}",
            "weights": "random-init N(0,0.02), seed 0",
            "step": "one generate() pass over 256 requests; every pass uses fresh token ids of the same lengths (no cross-pass prefix-cache hits)",
            "l2": "inputs larger than L2: every engine step streams the weights and the KV cache (> 126 MB)"}


def step_breakdown(step_times) -> dict:
    """Means over (is_prefill, sequences, tokens, device ms) records: decode steps overall and at batches of 256, 57..64
    and 1 sequences, prefill steps overall."""
    def mean(xs):
        xs = list(xs)
        return round(sum(xs) / len(xs), 4) if xs else None
    dec = [(s, ms) for p, s, _, ms in step_times if not p]
    pre = [(t, ms) for p, _, t, ms in step_times if p]
    return {"decode_step_ms": {"mean": mean(ms for _, ms in dec), "batch_256": mean(ms for s, ms in dec if s == 256),
                               "batch_57_64": mean(ms for s, ms in dec if 57 <= s <= 64), "batch_1": mean(ms for s, ms in dec if s == 1),
                               "steps": len(dec)},
            "prefill_ms": {"mean_per_step": mean(ms for _, ms in pre), "mean_tokens_per_step": mean(t for t, _ in pre), "steps": len(pre)}}


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
    from tinyllmforge_b200.utils.synth import checkpoint_bytes, write_checkpoint
    path = os.environ.get("FORGE_BENCH_CKPT", f"/tmp/forge_ckpt_{model}")
    done = os.path.join(path, "DONE")
    if rank == 0 and not os.path.exists(done):
        import torch
        need = checkpoint_bytes(preset(model))
        os.makedirs(path, exist_ok=True)
        free = shutil.disk_usage(path).free
        if free < need * 1.1 + (1 << 30):
            raise RuntimeError(f"a {need / 1e9:.0f} GB checkpoint does not fit the {free / 1e9:.0f} GB free under {path}")
        write_checkpoint(path, preset(model), seed=0, device="cuda" if torch.cuda.is_available() and need > (4 << 30) else "cpu")
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

    def sync_all():
        torch.cuda.synchronize()
        if n > 1:
            torch.distributed.barrier()

    for _ in range(args.warmup):
        one_pass()
    sync_all()
    sampler = ClockSampler(torch.cuda.current_device())
    if rank == 0:
        sampler.start()
    worker.reset_counters()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        outs = one_pass()
    sync_all()
    wall = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else None
    dev_ms = max_over_ranks(worker.device_ms, n)
    wall = max_over_ranks(wall, n)
    launches, h2d, d2h = worker.kernel_launches, worker.h2d_bytes, worker.d2h_bytes
    breakdown = step_breakdown(worker.step_times)
    decode_ms = max_over_ranks(sum(ms for p, _, _, ms in worker.step_times if not p) / args.steps, n)

    # exposed communication: one more pass with the exchange kernels working on this rank's data only (no waits, no peer
    # traffic; the sampled tokens are meaningless, the schedule is the same because every request ignores EOS)
    exposed = None
    fused = getattr(worker.ops, "fused", None)
    if n > 1 and fused is not None:
        fused.set_local_only(True)
        sync_all()
        worker.reset_counters()
        one_pass()
        sync_all()
        fused.set_local_only(False)
        local_decode_ms = max_over_ranks(sum(ms for p, _, _, ms in worker.step_times if not p), n)
        local_ms = max_over_ranks(worker.device_ms, n)
        sync_all()
        exposed = {"exposed_comm_pct": round(100.0 * (decode_ms - local_decode_ms) / decode_ms, 2),
                   "decode_ms_per_pass": round(decode_ms, 2), "decode_ms_per_pass_without_exchange": round(local_decode_ms, 2),
                   "pass_ms_without_exchange": round(local_ms, 2)}
    result = None
    if rank == 0:
        assert all(len(o["token_ids"]) == m for o, m in zip(outs, max_tokens))
        total = args.steps * sum(max_tokens)
        st = llm.stats
        result = {
            "metric": "output_tokens_per_second", "value": total / (dev_ms / 1e3), "unit": "tok/s", "n_gpus": n,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16" if args.quantization == "none" else "bf16 activations, fp8 e4m3 block-scaled weights",
            "data": "synthetic", "impl": "ours", "config": workload_config(args.model, n),
            "e2e": {"value": total / wall, "unit": "tok/s", "h2d_bytes_per_step": h2d // args.steps,
                    "d2h_bytes_per_step": d2h // args.steps, "wall_s_per_step": wall / args.steps},
            "gpu_launches": launches,
            "engine_steps_per_pass": (st.prefill_steps + st.decode_steps) // (args.steps + args.warmup + (1 if exposed else 0)),
            **breakdown,
            "clocks": clocks,
            "notes": {"comm": args.comm if n > 1 else "none",
                      "timing": "value: sum of per-engine-step CUDA-event times, max over ranks; e2e: wall clock of generate()"},
        }
        if exposed:
            result.update(exposed)
    llm.exit()
    return result


# ---------------------------------------------------------------------------------------------- reference engine
class ReferenceHarness:
    """Imports the reference from ``baseline/_ref`` with the documented shims, wraps ``ModelRunner.run`` in CUDA events
    (timing only) and guards construction and the passes with watchdogs (the reference has no error handling: a lost
    rendezvous or collective would sit until the caller's limit)."""

    def __init__(self, n: int, start_timeout: float, run_timeout: float):
        self.n, self.start_timeout, self.run_timeout = n, start_timeout, run_timeout
        self.shims: list[str] = []
        self.acc = {"ms": 0.0, "steps": 0, "h2d": 0, "d2h": 0, "cached": 0}
        self.step_times: list = []
        self.watchdog = None

    def load(self):
        """Returns (LLM, SamplingParams) or raises."""
        import torch
        ref_dir = os.path.join(ROOT, "baseline", "_ref")
        sys.path.insert(0, ref_dir)
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
                cfg.rope_scaling = None
                cfg.rope_theta = rp.get("rope_theta", 1000000.0)
                return cfg
            transformers.AutoConfig.from_pretrained = from_pretrained_compat
            self.shims.append("transformers>=5 config: restored legacy rope_theta / rope_scaling=None attributes")
        from tinyvllm import LLM, SamplingParams
        from tinyvllm.engine.model_runner import ModelRunner
        if self.n > 1:
            # as written the reference cannot start with more than one GPU: repair the defective spots in memory
            from baseline import ref_repairs
            self.shims += ["TP>1 run-time repairs: " + r for r in ref_repairs.apply()]
        acc, step_times = self.acc, self.step_times
        orig_run = ModelRunner.run

        def timed_run(runner, seqs, is_prefill):    # timing instrumentation only: CUDA events around the reference's own per-step device work
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = orig_run(runner, seqs, is_prefill)
            e1.record()
            e1.synchronize()
            ms = e0.elapsed_time(e1)
            ntok = sum(len(s) - s.num_cached_tokens for s in seqs) if is_prefill else len(seqs)
            acc["ms"] += ms
            acc["steps"] += 1
            acc["h2d"] += ntok * 20 + len(seqs) * 8        # ids + positions (int64), slots (int32), lens, temperatures
            acc["d2h"] += len(seqs) * 8
            if is_prefill:
                acc["cached"] += sum(s.num_cached_tokens for s in seqs)
            step_times.append((is_prefill, len(seqs), ntok, ms))
            return out

        ModelRunner.run = timed_run
        # Under torchrun the reference's own rendezvous ("tcp://localhost:2333", rank 0 hosts the store) would be turned
        # into a client of the launcher's agent store by these variables; the reference is its own launcher.
        for k in [k for k in os.environ if k.startswith("TORCHELASTIC")]:
            os.environ.pop(k)
        return LLM, SamplingParams

    def reset(self):
        self.acc.update(ms=0.0, steps=0, h2d=0, d2h=0, cached=0)
        self.step_times.clear()

    @staticmethod
    def kill_children():
        try:
            import psutil
            for c in psutil.Process(os.getpid()).children(recursive=True):
                c.kill()
        except Exception:
            pass

    def arm(self, what: str, limit: float):
        self.disarm()

        def give_up():
            print(json.dumps({"impl": "reference", "unavailable": f"the reference engine did not {what} within {limit:.0f} s"}), flush=True)
            self.kill_children()
            os._exit(0)
        self.watchdog = threading.Timer(limit, give_up)
        self.watchdog.daemon = True
        self.watchdog.start()

    def disarm(self):
        if self.watchdog is not None:
            self.watchdog.cancel()
            self.watchdog = None


def run_reference(args) -> dict:
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "tinyvllm")):
        return {"impl": "reference", "unavailable": "baseline/_ref/tinyvllm is not installed"}
    n = args.gpus
    rank = int(os.environ.get("RANK", "0")) if n > 1 else 0
    if n > 1 and rank != 0:
        return None            # the reference spawns its own worker processes from rank 0; the launcher's other ranks stand by
    import torch
    h = ReferenceHarness(n, args.ref_start_timeout, args.ref_run_timeout)
    try:
        LLM, SamplingParams = h.load()
    except Exception as e:  # missing dependency of the reference
        return {"impl": "reference", "unavailable": f"import failed: {type(e).__name__}: {e}"}
    try:
        path = ensure_checkpoint(args.model, 0)
    except Exception as e:
        return {"impl": "reference", "unavailable": f"no checkpoint: {type(e).__name__}: {e}"}
    prompts, max_tokens = make_workload()
    sps = [SamplingParams(temperature=0.6, ignore_eos=True, max_tokens=m) for m in max_tokens]
    h.arm("start", args.ref_start_timeout)
    try:
        llm = LLM(path, enforce_eager=False, max_model_len=4096, tensor_parallel_size=n)
        h.arm("finish its passes", args.ref_run_timeout)
        for p in range(args.warmup):
            llm.generate(prompts_for_pass(prompts, p), sps, use_tqdm=False)
        torch.cuda.synchronize()
        sampler = ClockSampler(torch.cuda.current_device())
        sampler.start()
        h.reset()
        t0 = time.perf_counter()
        for p in range(args.steps):
            llm.generate(prompts_for_pass(prompts, args.warmup + p), sps, use_tqdm=False)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        clocks = sampler.stop()
        h.disarm()
    except Exception as e:       # the reference's own code failed (it has no error handling of its own): report, do not crash
        h.disarm()
        h.kill_children()
        return {"impl": "reference", "unavailable": f"the reference engine failed: {type(e).__name__}: {str(e)[:300]}", "shims": h.shims}
    acc = h.acc
    total = args.steps * sum(max_tokens)
    return {
        "metric": "output_tokens_per_second", "value": total / (acc["ms"] / 1e3), "unit": "tok/s", "n_gpus": n,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": acc["ms"] / args.steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "reference",
        "config": workload_config(args.model, n),
        "e2e": {"value": total / wall, "unit": "tok/s", "h2d_bytes_per_step": acc["h2d"] // args.steps,
                "d2h_bytes_per_step": acc["d2h"] // args.steps, "wall_s_per_step": wall / args.steps},
        "engine_steps_per_pass": acc["steps"] // args.steps, **step_breakdown(h.step_times), "clocks": clocks, "shims": h.shims,
        "notes": {"timing": "value: CUDA events around ModelRunner.run on rank 0 (every step ends in a collective and a host sync, "
                            "so rank 0 spans the slowest rank), summed; e2e: wall clock of generate()"},
    }


# ---------------------------------------------------------------------------------------------- extras (child processes)
def child_env(n: int, port_offset: int, for_reference: bool) -> dict:
    """Environment of a child benchmark.  This engine under torchrun: the same rank variables, a rendezvous port of its
    own, and no launcher-agent store (rank 0 of the child hosts the store).  The reference: a plain single process."""
    env = {k: v for k, v in os.environ.items() if not k.startswith("TORCHELASTIC")}
    if for_reference:
        for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "GROUP_RANK", "LOCAL_WORLD_SIZE", "ROLE_RANK", "ROLE_WORLD_SIZE"):
            env.pop(k, None)
    elif n > 1:
        env["MASTER_ADDR"] = "127.0.0.1"
        env["MASTER_PORT"] = str(int(os.environ.get("MASTER_PORT", "29500")) + port_offset)
    return env


def run_child(cmd: list[str], env: dict, timeout_s: float) -> dict | None:
    """Runs a benchmark script in a process group of its own, returns the last JSON line it printed (None if it printed
    none: a non-zero rank).  At the time limit the whole group is ended (the reference starts worker processes)."""
    if timeout_s < MIN_CHILD_S:
        return {"unavailable": f"skipped: {timeout_s:.0f} s left of the run's time budget"}
    p = subprocess.Popen([sys.executable] + cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, cwd=ROOT,
                         start_new_session=True)
    try:
        stdout, stderr = p.communicate(timeout=timeout_s)
    except subprocess.TimeoutExpired:
        try:
            os.killpg(p.pid, signal.SIGKILL)          # the group this call created, nothing else
        except ProcessLookupError:
            pass
        p.communicate()
        return {"unavailable": f"did not finish within {timeout_s:.0f} s"}
    for line in reversed(stdout.strip().splitlines()):
        if line.startswith("{"):
            try:
                return json.loads(line)
            except ValueError:
                continue
    if p.returncode != 0:
        return {"unavailable": f"exit code {p.returncode}: {stderr.strip()[-300:]}"}
    return None


def run_extras(args) -> dict:
    """BASELINE configs beyond the headline, measured with the same engine arm at the same N.  Each runs in a child
    process BEFORE the headline engine is built (a fresh process frees every byte and the fixed rendezvous port of the
    reference); a failure or a timeout becomes an ``unavailable`` entry and never touches the headline number.
    All of them together get what ``--time-budget`` leaves after the headline's own estimated time: a workload that
    would not fit is skipped, not cut short in the middle of the headline."""
    n, ref = args.gpus, args.impl == "reference"
    rank = int(os.environ.get("RANK", "0")) if n > 1 else 0
    if ref and rank != 0:
        return {}
    per_pass = (6.2 if ref else 4.5)                       # seconds, the slowest N measured (N=1)
    headline_s = (100.0 if ref else 75.0) + (args.steps + args.warmup + 1) * per_pass * (1.10 if ref else 1.15)
    deadline = T_START + args.time_budget - headline_s

    def left() -> float:
        return min(args.extras_timeout, deadline - time.monotonic())
    common = ["--gpus", str(n), "--impl", args.impl, "--comm", args.comm]
    keep = ("metric", "value", "unit", "ms_per_step", "steps", "warmup", "e2e", "decode_step_ms", "prefill_ms", "exposed_comm_pct",
            "gpu_launches", "unavailable", "shims")
    out = {}
    r = run_child(["bench.py", "--model", "qwen3-8b", "--steps", "2", "--warmup", "1", "--no-extras"] + common +
                  ([] if ref else ["--load", "dummy"]), child_env(n, 101, ref), left())
    if r is not None:
        out[f"config3_qwen3_8b_tp{n}"] = {k: r[k] for k in keep if k in r}
    if n == 8:
        r = run_child(["bench_prefix_cache.py"] + common, child_env(n, 102, ref), left())
        if r is not None:
            out["config5_prefix_cache_qwen3_8b_tp8"] = r
        for q in ("none", "fp8_block"):
            if ref and q != "none":
                continue                  # the reference has no fp8 path
            r = run_child(["bench_decode.py", "--quantization", q] + common, child_env(n, 103 + (q != "none"), ref), left())
            if r is not None:
                out["config4_qwen3_32b_tp8_" + ("bf16" if q == "none" else "fp8_block")] = r
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default=os.environ.get("FORGE_BENCH_MODEL", HEADLINE_MODEL))
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"],
                    help="tensor-parallel exchange: in-kernel NVLink exchange (fused) or torch.distributed/NCCL calls")
    ap.add_argument("--ref-start-timeout", type=float, default=600.0, help="seconds the reference engine gets to start")
    ap.add_argument("--ref-run-timeout", type=float, default=1500.0, help="seconds the reference engine gets for all its passes")
    ap.add_argument("--quantization", default="none", choices=["none", "fp8_block"],
                    help="fp8_block: e4m3 weights with 128 x 128 block scales for the four projections of every layer (not the headline)")
    ap.add_argument("--load", default="auto", choices=["auto", "dummy"],
                    help="auto: write and load a safetensors checkpoint; dummy: random-init on the device (large models)")
    ap.add_argument("--no-extras", action="store_true", help="only the named model's workload (what the child runs use)")
    ap.add_argument("--extras-timeout", type=float, default=600.0, help="most seconds one extra workload's child process gets")
    ap.add_argument("--time-budget", type=float, default=800.0,
                    help="seconds the whole run should fit in: the extra workloads get what the headline's estimated time leaves")
    args = ap.parse_args()
    extras = None
    if not args.no_extras and args.model == HEADLINE_MODEL and args.quantization == "none" and os.environ.get("FORGE_BENCH_EXTRAS", "1") != "0":
        extras = run_extras(args)
    out = run_reference(args) if args.impl == "reference" else run_ours(args)
    if out is not None:
        if extras:
            out["extras"] = extras
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
