"""The engine: request intake, the schedule -> run -> postprocess loop, rank management.

Parity: tinyvllm/engine/llm_engine.py:15-101 (``LLMEngine``): ``add_request``, ``step``,
``is_finished``, ``generate`` (outputs sorted by request id as ``{"text", "token_ids"}`` dicts), ``exit``.

Two ways to get tensor-parallel ranks:
  * spawn mode (the reference's): ``LLM(..., tensor_parallel_size=N)`` in one process starts N-1
    follower processes;
  * launcher mode: when the process was started by ``torchrun`` (``WORLD_SIZE == tensor_parallel_size``)
    every rank constructs ``LLM`` itself; rank 0 schedules, the others execute the published steps inside
    their own ``generate`` call and return an empty list.

A follower that dies or reports an error surfaces on rank 0 as ``EngineDeadError`` at the next step
(the reference hangs in its next collective).
"""
from __future__ import annotations

import atexit
import json
import os
import time

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ..config import Config
from ..parallel.comm import TPGroup, find_free_port
from ..sampling_params import SamplingParams
from . import rpc
from .request import Request
from .scheduler import PLACEHOLDER, Scheduler
from .stats import EngineStats
from .step_batch import DecodeBuilder, build_prefill
from .worker import Worker, follower_loop, follower_main


class EngineDeadError(RuntimeError):
    pass


def _load_tokenizer(config: Config):
    if config.skip_tokenizer_init:
        return None
    if not any(os.path.exists(os.path.join(config.model, f)) for f in ("tokenizer.json", "tokenizer.model", "vocab.json")):
        return None
    from transformers import AutoTokenizer
    return AutoTokenizer.from_pretrained(config.model, use_fast=True)


class LLMEngine:
    def __init__(self, model: str, **kwargs):
        self.config = config = Config.from_kwargs(model, **kwargs)
        tp_size = config.tensor_parallel_size
        self.procs: list = []
        self.chan: rpc.ShmChannel | None = None
        self.worker: Worker | None = None
        self._closed = False
        self.step_index = 0
        self.stats = EngineStats()
        self._trace = open(config.trace_path, "a") if config.trace_path else None
        self._nvtx = bool(config.extra.get("nvtx", False)) and config.device == "cuda"
        self._nvtx_open = False

        env_world = int(os.environ.get("WORLD_SIZE", "1"))
        self.launcher_mode = tp_size > 1 and env_world == tp_size and "RANK" in os.environ
        self.rank = int(os.environ["RANK"]) if self.launcher_mode else 0
        try:
            if config.device == "cuda":
                local = int(os.environ.get("LOCAL_RANK", self.rank)) if self.launcher_mode else 0
                torch.cuda.set_device(local)
            if tp_size == 1:
                tp = TPGroup()
            elif self.launcher_mode:
                tp = TPGroup.init(self.rank, tp_size, config.device, "env://", config.rpc_timeout_s)
                name = [rpc.unique_name()] if self.rank == 0 else [None]
                if self.rank == 0:
                    self.chan = rpc.ShmChannel(name[0], tp_size, 0, create=True, timeout_s=config.rpc_timeout_s)
                dist.broadcast_object_list(name, src=0)
                if self.rank != 0:
                    self.chan = rpc.ShmChannel(name[0], tp_size, self.rank, create=False, timeout_s=config.rpc_timeout_s)
            else:
                name = rpc.unique_name()
                self.chan = rpc.ShmChannel(name, tp_size, 0, create=True, timeout_s=config.rpc_timeout_s)
                init_method = f"tcp://127.0.0.1:{find_free_port()}"
                ctx = mp.get_context("spawn")
                for r in range(1, tp_size):
                    p = ctx.Process(target=follower_main, args=(config, r, name, init_method), daemon=True)
                    p.start()
                    self.procs.append(p)
                self.chan.liveness = self._check_followers_alive
                self.chan.wait_hello()
                tp = TPGroup.init(0, tp_size, config.device, init_method, config.rpc_timeout_s)
            self.tp = tp
            self.worker = Worker(config, self.rank, tp)
            tp.barrier()
        except BaseException:
            self.exit()
            raise
        self.tokenizer = _load_tokenizer(config) if self.rank == 0 else None
        if self.tokenizer is not None and self.tokenizer.eos_token_id is not None:
            config.eos = self.tokenizer.eos_token_id
        self.scheduler = Scheduler(config) if self.rank == 0 else None
        self.decode_builder = DecodeBuilder(config.kvcache_block_size)
        atexit.register(self.exit)

    # ------------------------------------------------------------------ liveness
    def _check_followers_alive(self) -> None:
        for r, p in enumerate(self.procs, start=1):
            if not p.is_alive():
                msg = self.chan.read_error() if self.chan is not None else ""
                raise EngineDeadError(f"tensor-parallel rank {r} exited with code {p.exitcode}. {msg}")

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt: str | list[int], sampling_params: SamplingParams = SamplingParams()) -> int:
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("string prompts need tokenizer files in the model directory; pass token ids instead")
            prompt = self.tokenizer.encode(prompt)
        room = self.config.max_model_len - len(prompt)
        if room < 1:
            raise ValueError(f"prompt of {len(prompt)} tokens leaves no room under max_model_len={self.config.max_model_len}")
        req = Request(prompt, sampling_params)
        req.max_tokens = min(req.max_tokens, room)
        self.scheduler.add(req)
        return req.req_id

    def is_finished(self) -> bool:
        return self.scheduler.is_finished()

    # ------------------------------------------------------------------ one step
    # ------------------------------------------------------------------ tracing
    def _mark(self, name: str | None) -> None:
        """NVTX range per phase of a step (schedule / build / run / postprocess) when ``extra={"nvtx": True}``: closes
        the open range and opens ``name`` (None: just close).  Shows the host phases on a profiler's timeline."""
        if not self._nvtx:
            return
        if self._nvtx_open:
            torch.cuda.nvtx.range_pop()
        self._nvtx_open = name is not None
        if name is not None:
            torch.cuda.nvtx.range_push(name)

    def _trace_step(self, index, is_prefill, seqs, tokens, t0, t1, t2, t3, t4) -> None:
        if self._trace is not None:
            self._trace.write(json.dumps({"step": index, "prefill": is_prefill, "seqs": seqs, "tokens": tokens,
                                          "schedule_ms": (t1 - t0) * 1e3, "build_ms": (t2 - t1) * 1e3, "run_ms": (t3 - t2) * 1e3,
                                          "post_ms": (t4 - t3) * 1e3}) + "\n")

    def step(self):
        """schedule -> build -> (publish) -> run -> postprocess.  Returns (finished, signed token count):
        finished = [(req_id, completion_token_ids)], count > 0: prefill tokens, < 0: decode sequences."""
        st = self.stats
        t0 = time.perf_counter()
        self._mark("schedule")
        reqs, is_prefill = self.scheduler.schedule()
        t1 = time.perf_counter()
        self._mark("build")
        bs = self.config.kvcache_block_size
        if is_prefill:
            sb = build_prefill(reqs, bs, self.step_index, self.config.seed)
            self.decode_builder.reset()
        else:
            pad, width = self.worker.decode_padding(len(reqs))
            sb = self.decode_builder.build(reqs, self.step_index, self.config.seed, pad, width)
        t2 = time.perf_counter()
        self._mark("run")
        try:
            if self.chan is not None:
                if self.procs:
                    self._check_followers_alive()       # learn of a dead rank on the host, before the next collective
                self.chan.publish(rpc.KIND_STEP, sb.buf[:sb.num_words])
            token_ids = self.worker.run(sb)
        except (rpc.PeerFailed, rpc.ChannelTimeout) as e:
            raise EngineDeadError(str(e)) from e
        except RuntimeError as e:
            # a collective that lost its peer fails with a backend error: say which rank went away
            if self.chan is not None:
                try:
                    self._check_followers_alive()
                    self.chan._check_followers()
                except (EngineDeadError, rpc.PeerFailed) as dead:
                    raise EngineDeadError(f"{dead} (while running a step: {e})") from e
            raise
        t3 = time.perf_counter()
        self._mark("postprocess")
        self.step_index += 1
        st.add_device_time(is_prefill, getattr(self.worker, "last_step_ms", None))
        finished = self.scheduler.postprocess(reqs, token_ids)
        t4 = time.perf_counter()
        self._mark(None)

        st.schedule_s += t1 - t0
        st.build_s += t2 - t1
        st.run_s += t3 - t2
        st.postprocess_s += t4 - t3
        if is_prefill:
            st.prefill_steps += 1
            st.prefill_tokens += sb.num_tokens
            st.prefix_cached_tokens += self.scheduler.last_admit_cached
            count = sb.num_tokens
        else:
            st.decode_steps += 1
            st.decode_tokens += len(reqs)
            st.decode_batch_hist[len(reqs)] += 1
            count = -len(reqs)
        st.preemptions = self.scheduler.num_preemptions
        st.finished_requests += len(finished)
        self._trace_step(self.step_index - 1, is_prefill, len(reqs), sb.num_tokens, t0, t1, t2, t3, t4)
        return [(r.req_id, r.completion_token_ids) for r in finished], count

    # ------------------------------------------------------------------ generate
    def generate(self, prompts: list[str] | list[list[int]], sampling_params: SamplingParams | list[SamplingParams],
                 use_tqdm: bool = True) -> list[dict]:
        if self.rank != 0:          # launcher mode: execute rank 0's steps until it marks the end of this call
            kind = follower_loop(self.worker, self.chan)
            if kind == rpc.KIND_EXIT:
                self.exit()
            return []
        if not isinstance(sampling_params, list):
            sampling_params = [sampling_params] * len(prompts)
        if len(sampling_params) != len(prompts):
            raise ValueError("need one SamplingParams per prompt")
        pbar = None
        if use_tqdm:
            from tqdm.auto import tqdm
            pbar = tqdm(total=len(prompts), desc="Generating", dynamic_ncols=True)
        ids = [self.add_request(p, sp) for p, sp in zip(prompts, sampling_params)]
        outputs: dict[int, list[int]] = {}
        prefill_tps = decode_tps = 0.0
        pipelined = self._can_pipeline()
        try:
            if pipelined:
                self._run_pipelined(outputs, pbar)
            while not self.is_finished():
                t = time.perf_counter()
                finished, count = self.step()
                if pbar is not None:
                    dt = time.perf_counter() - t
                    if count > 0:
                        prefill_tps = count / dt
                    else:
                        decode_tps = -count / dt
                    pbar.set_postfix({"Prefill": f"{int(prefill_tps)}tok/s", "Decode": f"{int(decode_tps)}tok/s"})
                    pbar.update(len(finished))
                for req_id, toks in finished:
                    outputs[req_id] = toks
        finally:
            if pbar is not None:
                pbar.close()
            if self.launcher_mode and self.chan is not None and not self._closed:
                self.chan.publish(rpc.KIND_PING)
        result = []
        for req_id in ids:
            toks = outputs[req_id]
            text = self.tokenizer.decode(toks) if self.tokenizer is not None else ""
            result.append({"text": text, "token_ids": toks})
        return result

    # ------------------------------------------------------------------ pipelined loop
    def _can_pipeline(self) -> bool:
        """The host runs one step ahead of the tokens it reads back.  Lengths, finish-by-max_tokens, block growth and
        slots do not depend on token values, and the values themselves travel device-to-device.  A request that may
        stop on EOS is scheduled one step ahead on the assumption that it does not stop; when its token turns out to
        be EOS the surplus token of the step already in flight is dropped (see ``_run_pipelined``)."""
        return bool(self.config.extra.get("pipeline", True))

    def _run_pipelined(self, outputs: dict, pbar) -> None:
        """schedule/build/launch step t+1, THEN read step t's tokens: scheduling, building, publishing and output
        handling overlap with the GPU.  Prefill steps are launched only when nothing is in flight (a preempted
        request must have all its real tokens before it is prefilled again).

        EOS: step t+1 is launched before step t's tokens are known, so a request whose step-t token is EOS also sits
        in step t+1.  When the EOS is read, the request is retired with the tokens up to the EOS, its blocks are
        freed (later steps run after the one in flight, and blocks are sealed for the prefix cache only with tokens
        that were read back), and the token step t+1 computes for it is ignored."""
        sch, st, bs = self.scheduler, self.stats, self.config.kvcache_block_size
        eos = self.config.eos
        inflight = None             # (reqs, ticket, finished requests) of the step not yet read back

        def drain():
            nonlocal inflight
            if inflight is None:
                return
            reqs, ticket, finished, was_prefill = inflight
            inflight = None
            try:
                toks = self.worker.collect(ticket)
            except RuntimeError as e:
                raise EngineDeadError(str(e)) from e
            st.add_device_time(was_prefill, getattr(self.worker, "last_step_ms", None))
            early = 0
            for (r, idx), tok in zip(reqs, toks):
                if idx < 0 or idx >= len(r.token_ids):   # no token expected (chunk of a long prompt), or retired before this step was read
                    continue
                r.token_ids[idx] = tok
                if tok == eos and not r.ignore_eos and idx + 1 - r.num_prompt_tokens < r.max_tokens:
                    # stops here, one step (or, preempted in between, no step) after the host moved on
                    del r.token_ids[idx + 1:]
                    sch.finish_early(r)
                    outputs[r.req_id] = r.completion_token_ids
                    early += 1
            for r in finished:
                outputs[r.req_id] = r.completion_token_ids
            st.finished_requests += early
            if pbar is not None:
                pbar.update(len(finished) + early)

        while not sch.is_finished():
            if sch.has_waiting() and inflight is not None:
                drain()                                  # the next step may be a prefill: needs real token ids
                if sch.is_finished():                    # the tokens just read ended the last requests (EOS)
                    break
            t0 = time.perf_counter()
            self._mark("schedule")
            reqs, is_prefill = sch.schedule(defer_seal=True)
            t1 = time.perf_counter()
            self._mark("build")
            if is_prefill:
                sb = build_prefill(reqs, bs, self.step_index, self.config.seed)
                self.decode_builder.reset()
            else:
                pad, width = self.worker.decode_padding(len(reqs))
                sb = self.decode_builder.build(reqs, self.step_index, self.config.seed, pad, width)
                src = sb.src_rows
                src[:] = -1
                if inflight is not None:
                    prev_row = {id(r): i for i, (r, _) in enumerate(inflight[0])}
                    src[:len(reqs)] = [prev_row.get(id(r), -1) for r in reqs]
            t2 = time.perf_counter()
            self._mark("launch")
            try:
                if self.chan is not None:
                    if self.procs:
                        self._check_followers_alive()
                    self.chan.publish(rpc.KIND_STEP, sb.buf[:sb.num_words])
                ticket = self.worker.launch(sb)
            except (rpc.PeerFailed, rpc.ChannelTimeout) as e:
                raise EngineDeadError(str(e)) from e
            t3 = time.perf_counter()
            self._mark("collect previous + postprocess")
            self.step_index += 1
            drain()                                      # read the PREVIOUS step while this one runs
            partial = sch.partial                        # a long prompt in the middle of its prefill receives no token
            # a request the drain above retired (EOS in the previous step) is still part of this step: its token is dropped
            retired = {id(r) for r in reqs if r.is_finished}
            finished = sch.postprocess(reqs, [PLACEHOLDER] * len(reqs))
            inflight = ([(r, -1 if (r is partial or id(r) in retired) else len(r.token_ids) - 1) for r in reqs], ticket, finished, is_prefill)
            t4 = time.perf_counter()
            self._mark(None)
            st.schedule_s += t1 - t0
            st.build_s += t2 - t1
            st.run_s += t3 - t2
            st.postprocess_s += t4 - t3
            if is_prefill:
                st.prefill_steps += 1
                st.prefill_tokens += sb.num_tokens
                st.prefix_cached_tokens += self.scheduler.last_admit_cached
            else:
                st.decode_steps += 1
                st.decode_tokens += len(reqs)
                st.decode_batch_hist[len(reqs)] += 1
            st.preemptions = sch.num_preemptions
            st.finished_requests += len(finished)
            self._trace_step(self.step_index - 1, is_prefill, len(reqs), sb.num_tokens, t0, t1, t2, t3, t4)
        drain()

    # ------------------------------------------------------------------ teardown
    def exit(self) -> None:
        if self._closed:
            return
        self._closed = True
        try:
            if self.chan is not None and self.rank == 0 and self.procs:      # launcher-mode ranks leave on their own
                try:
                    self.chan.publish(rpc.KIND_EXIT)
                    self.chan.drain(timeout_s=10.0)
                except Exception:
                    pass
            if self.worker is not None:
                self.worker.close()
                self.worker = None
            for p in self.procs:
                p.join(timeout=15.0)
                if p.is_alive():
                    p.terminate()
            if getattr(self, "tp", None) is not None:
                self.tp.close()
        finally:
            if self.chan is not None:
                self.chan.close()
                self.chan = None
            if self._trace is not None:
                self._trace.close()
                self._trace = None
