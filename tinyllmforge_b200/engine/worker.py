"""Per-rank executor: owns the model shard, the KV cache, the step staging buffers and the CUDA graphs.

Parity: tinyvllm/engine/model_runner.py:15-308 (``ModelRunner``): distributed init, model build and
load, warm-up, KV-cache sizing, batch -> tensors, eager/graph execution, sampling, and the follower
loop of ranks 1..tp-1.

Differences that matter:
  * a step arrives as ONE packed int32 buffer (``StepBatch``) that is copied to the device with a single
    transfer into a static buffer; kernels read typed views of it, so a replayed graph needs no
    per-tensor copies (the reference fills five graph tensors per replay, model_runner.py:252-257);
  * logits, the cross-rank token choice and sampling run INSIDE the captured graph (the reference
    computes logits and gathers them after the replay, model_runner.py:261);
  * every rank computes the sampled token, so followers need no result channel, and a follower that
    fails reports it through the channel's status word.
"""
from __future__ import annotations

import traceback

import numpy as np
import torch

from ..config import Config
from ..models.qwen3 import Qwen3ForCausalLM
from ..ops.ref import RefOps
from ..parallel.comm import TPGroup
from ..utils.weights import init_dummy_weights, load_weights
from . import rpc
from .step_batch import (HEADER_WORDS, SECTIONS, StepBatch, build_decode, build_prefill, section_offsets)


class DeviceBatch:
    """Typed device views over a packed step buffer, plus the host copies of the scalars."""

    def __init__(self, sb: StepBatch, words: torch.Tensor):
        self.is_prefill = sb.is_prefill
        self.num_seqs, self.num_tokens = sb.num_seqs, sb.num_tokens
        self.padded_seqs, self.padded_tokens = sb.padded_seqs, sb.padded_tokens
        self.table_width = sb.table_width
        self.max_seqlen_q, self.max_seqlen_k = sb.max_seqlen_q, sb.max_seqlen_k
        self.step_index, self.seed = sb.step_index, sb.seed
        self.words = words
        self.header = words[:HEADER_WORDS]
        for name in SECTIONS:
            off, n = sb.offsets[name]
            v = words[off:off + n]
            if name == "temperatures":
                v = v.view(torch.float32)
            elif name == "block_tables":
                v = v.view(sb.padded_seqs, sb.table_width)
            setattr(self, name, v)


def graph_buckets(max_num_seqs: int) -> list[int]:
    """Decode batch sizes with a captured graph: 1, 2, 4, 8, then every 16 up to min(max_num_seqs, 512)
    (tinyvllm/engine/model_runner.py:287)."""
    top = min(max_num_seqs, 512)
    return [b for b in (1, 2, 4, 8) if b <= top] + list(range(16, top + 1, 16))


class Worker:
    def __init__(self, config: Config, rank: int, tp: TPGroup):
        self.config, self.rank, self.tp = config, rank, tp
        hf = config.hf_config
        self.block_size = config.kvcache_block_size
        self.is_cuda = config.device == "cuda"
        self.device = torch.device("cuda", torch.cuda.current_device()) if self.is_cuda else torch.device("cpu")
        self.table_width = (config.max_model_len + self.block_size - 1) // self.block_size
        self.buckets = [] if (config.enforce_eager or not self.is_cuda) else graph_buckets(config.max_num_seqs)
        self.graphs: dict[int, object] = {}
        self.graph_launches: dict[int, int] = {}
        self.time_steps = bool(config.extra.get("device_timing", False))
        self.prev_tokens_host = np.zeros(0, dtype=np.int64)
        self.num_steps = 0
        self.last_step_ms: float | None = None      # device time of the step collected last (with extra={"device_timing": True})
        self.reset_counters()

        if self.is_cuda:
            from ..ops.cuda import CudaOps
            ops = CudaOps(config, tp, self.device)
        else:
            ops = RefOps
        self.ops = ops
        with torch.inference_mode():
            self.model = Qwen3ForCausalLM(hf, tp, config.dtype, self.device, ops, max_positions=config.max_model_len)
            if config.load_format == "dummy":
                init_dummy_weights(self.model, config.seed)
            else:
                load_weights(self.model, config.model)
            if (self.is_cuda and tp.size == 1 and config.quantization is None and config.dtype == torch.bfloat16
                    and config.extra.get("fold_norms", True) and not hf.attention_bias):
                self.model.fold_norm_weights()      # add + RMSNorm become GEMM epilogues (models/qwen3.py)
            if config.quantization == "fp8_block":
                from ..ops.quant import Fp8BlockWeight
                for l in self.model.layers:          # the four projections of every block; embeddings and LM head stay bf16
                    for lin in (l.qkv_proj, l.o_proj, l.gate_up_proj, l.down_proj):
                        lin.weight = Fp8BlockWeight.quantize(lin.weight)
            if self.is_cuda and tp.size > 1 and config.comm == "fused":
                ops.enable_fused_comm(hf.hidden_size, config.max_num_batched_tokens, config.comm_timeout_s)
            # staging: the largest step is a full prefill (3 token-sized sections) or the widest decode bucket
            max_seqs = config.max_num_seqs
            _, words_prefill = section_offsets(config.max_num_batched_tokens, max_seqs, self.table_width)
            self.max_words = words_prefill
            if self.is_cuda:
                # two staging buffers: the host fills one while the copy out of the other may still be in flight
                self.host_words = [torch.empty(self.max_words, dtype=torch.int32, pin_memory=True) for _ in range(2)]
                self.dev_words = torch.zeros(self.max_words, dtype=torch.int32, device=self.device)
                # sampled tokens of a step, followed by one word that receives the kernels' status word of that step
                self.status_slot = max(max_seqs, 512)
                self.host_tokens = [torch.zeros(self.status_slot + 1, dtype=torch.int32, pin_memory=True) for _ in range(2)]
                self.prev_tokens_dev = torch.zeros(1, dtype=torch.int32, device=self.device)
            self._allocate_kv_cache()
            if self.buckets:
                self._capture_graphs()

    def reset_counters(self) -> None:
        """Zero the per-run measurements: device time of the steps (CUDA events), bytes staged in each
        direction, and the number of this library's kernels launched (graph replays count their nodes)."""
        self.device_ms = 0.0
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.kernel_launches = 0
        self.step_times: list[tuple[bool, int, int, float]] = []      # (is_prefill, sequences, tokens, device ms) per timed step
        if getattr(self, "ops", None) is not None and hasattr(self.ops, "launches"):
            self.ops.launches = 0

    # ------------------------------------------------------------------ KV cache
    def _kv_block_bytes(self) -> int:
        hf = self.config.hf_config
        kvh = hf.num_key_value_heads // self.tp.size
        return 2 * hf.num_hidden_layers * self.block_size * kvh * hf.head_dim * torch.finfo(self.config.dtype).bits // 8

    def _warmup(self) -> None:
        """One full-budget prefill so the allocator's peak reflects the largest step
        (tinyvllm/engine/model_runner.py:108-116)."""
        cfg = self.config
        seq_len = min(cfg.max_model_len, cfg.max_num_batched_tokens)      # chunked prefill: a step never exceeds the budget
        n = max(1, min(cfg.max_num_batched_tokens // seq_len, cfg.max_num_seqs))
        from .request import Request
        reqs = []
        nblk = (seq_len + self.block_size - 1) // self.block_size
        for i in range(n):
            r = Request([0] * seq_len)
            r.block_table = list(range(i * nblk, (i + 1) * nblk))
            reqs.append(r)
        self.run(build_prefill(reqs, self.block_size))

    def _allocate_kv_cache(self) -> None:
        cfg, hf = self.config, self.config.hf_config
        kvh = hf.num_key_value_heads // self.tp.size
        block_bytes = self._kv_block_bytes()
        if cfg.num_kvcache_blocks <= 0:
            if self.is_cuda:
                # temporary cache just large enough for the warm-up prefill
                n_tmp = max(1, min(cfg.max_num_batched_tokens // min(cfg.max_model_len, cfg.max_num_batched_tokens), cfg.max_num_seqs)) * self.table_width
                self.model.bind_kv_cache(torch.zeros(hf.num_hidden_layers, 2, n_tmp, kvh, self.block_size, hf.head_dim,
                                                     dtype=cfg.dtype, device=self.device))
                torch.cuda.reset_peak_memory_stats()
                self._warmup()
                torch.cuda.synchronize()
                self.model.kv_cache = None
                torch.cuda.empty_cache()
                free, total = torch.cuda.mem_get_info()
                stats = torch.cuda.memory_stats()
                peak, cur = stats["allocated_bytes.all.peak"], stats["allocated_bytes.all.current"]
                budget = int(total * cfg.gpu_memory_utilization) - (total - free) - (peak - cur)
                n = budget // block_bytes
            else:
                n = max(64, min(cfg.max_num_seqs, 16) * self.table_width)
            # every rank must agree on the pool size: take the minimum
            if self.tp.size > 1:
                t = torch.tensor([n], dtype=torch.int64, device=self.device)
                torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MIN, group=self.tp.group)
                n = int(t.item())
            if n <= 0:
                raise RuntimeError("no memory left for the KV cache; raise gpu_memory_utilization")
            cfg.num_kvcache_blocks = int(n)
        self.model.bind_kv_cache(torch.zeros(hf.num_hidden_layers, 2, cfg.num_kvcache_blocks, kvh, self.block_size,
                                             hf.head_dim, dtype=cfg.dtype, device=self.device))

    # ------------------------------------------------------------------ execution
    def decode_padding(self, num_seqs: int) -> tuple[int | None, int | None]:
        """(bucket, table width) rank 0 must pad a decode step to, or (None, None) for eager."""
        for b in self.buckets:
            if b >= num_seqs:
                return b, self.table_width
        return None, None

    def _stage(self, sb: StepBatch) -> DeviceBatch:
        n = sb.num_words
        if not self.is_cuda:
            return DeviceBatch(sb, torch.from_numpy(sb.buf[:n]))
        host = self.host_words[self.num_steps & 1]
        host[:n].numpy()[:] = sb.buf[:n]
        self.dev_words[:n].copy_(host[:n], non_blocking=True)
        return DeviceBatch(sb, self.dev_words[:n])

    @torch.inference_mode()
    def launch(self, sb: StepBatch):
        """Start one step and return a ticket for :meth:`collect`.  Nothing here waits for the GPU, so the caller
        may schedule and build the next step while this one runs.  When ``sb.src_rows`` names rows of the previous
        step, the input tokens are taken from that step's sampled tokens on the device."""
        if not self.is_cuda:
            src = sb.src_rows[:sb.num_seqs]
            if not sb.is_prefill and (src >= 0).any():
                ids = sb.input_ids
                take = src >= 0
                ids[:sb.num_seqs][take] = self.prev_tokens_host[src[take]]
            tokens = self.model.step(self._stage(sb))[:sb.num_seqs]
            self.prev_tokens_host = np.asarray(tokens.tolist(), dtype=np.int64)
            self.num_steps += 1
            return ("cpu", self.prev_tokens_host.tolist())
        timed = self.time_steps
        e0 = None
        if timed:
            e0 = torch.cuda.Event(enable_timing=True)
            e0.record()
        batch = self._stage(sb)
        if not sb.is_prefill and self.feed_rows(sb):
            self.ops.C.feed_tokens(batch.input_ids[:sb.num_seqs], batch.src_rows, self.prev_tokens_dev)
            self.kernel_launches += 1
        graph = None if sb.is_prefill else self.graphs.get(sb.padded_seqs)
        if graph is not None and sb.table_width == self.table_width:
            graph.replay()
            tokens = self.graph_tokens[sb.padded_seqs]
            self.kernel_launches += self.graph_launches[sb.padded_seqs]
        else:
            before = self.ops.launches
            tokens = self.model.step(batch)
            self.kernel_launches += self.ops.launches - before
        n = sb.num_seqs
        self.prev_tokens_dev = tokens                  # stays on the device: the next step may take its inputs from here
        host = self.host_tokens[self.num_steps & 1]
        host[:n].copy_(tokens[:n], non_blocking=True)
        # the status word of the kernels travels with the tokens: every step is checked, and the check costs no sync
        host[self.status_slot:].copy_(self.ops.status[:1], non_blocking=True)
        done = torch.cuda.Event(enable_timing=timed)
        done.record()
        self.h2d_bytes += sb.nbytes
        self.d2h_bytes += n * 4 + 4
        self.num_steps += 1
        return ("cuda", host, n, e0, done, (sb.is_prefill, sb.num_seqs, sb.num_tokens))

    @staticmethod
    def feed_rows(sb: StepBatch) -> bool:
        return bool((sb.src_rows[:sb.num_seqs] >= 0).any())

    def collect(self, ticket) -> list[int]:
        """Wait for a launched step; returns the sampled token of each of its sequences."""
        if ticket[0] == "cpu":
            return ticket[1]
        _, host, n, e0, done, shape = ticket
        done.synchronize()
        self.last_step_ms = None
        if e0 is not None:
            ms = e0.elapsed_time(done)
            self.device_ms += ms
            self.last_step_ms = ms
            self.step_times.append((shape[0], shape[1], shape[2], ms))
        word = int(host[self.status_slot])
        if word:
            self.ops.raise_status(word)
        return host[:n].tolist() if self.rank == 0 else []

    def run(self, sb: StepBatch) -> list[int]:
        """Execute one step and wait for it."""
        return self.collect(self.launch(sb))

    @torch.inference_mode()
    def _capture_graphs(self) -> None:
        """One graph per decode bucket, largest first so they share one memory pool
        (tinyvllm/engine/model_runner.py:289-297).  Inputs are views of the static step buffer."""
        from .request import Request
        self.graph_tokens: dict[int, torch.Tensor] = {}
        pool = None
        for b in reversed(self.buckets):
            reqs = []
            for i in range(b):
                r = Request([0, 0])
                r.block_table = [i % self.config.num_kvcache_blocks]
                reqs.append(r)
            sb = build_decode(reqs, self.block_size, pad_to=b, table_width=self.table_width)
            batch = self._stage(sb)
            self.model.step(batch)                       # warm-up outside capture
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            before = self.ops.launches
            with torch.cuda.graph(g, pool=pool):
                self.graph_tokens[b] = self.model.step(batch)
            self.graph_launches[b] = self.ops.launches - before
            pool = pool or g.pool()
            self.graphs[b] = g
        torch.cuda.synchronize()

    def close(self) -> None:
        self.graphs.clear()
        if hasattr(self.ops, "close"):
            self.ops.close()
        if self.is_cuda:
            torch.cuda.synchronize()


# ---------------------------------------------------------------------- follower process
def follower_loop(worker: Worker, chan: rpc.ShmChannel) -> int:
    """Ranks 1..tp-1: execute every published step until told to exit (KIND_EXIT) or until rank 0 marks
    the end of a ``generate`` call (KIND_PING); returns which (tinyvllm/engine/model_runner.py:73-89)."""
    pending = None
    while True:
        kind, data = chan.receive()
        if kind in (rpc.KIND_EXIT, rpc.KIND_PING):
            if pending is not None:
                worker.collect(pending)
            return kind
        if kind == rpc.KIND_STEP:
            # Launch first, then wait for the step before: the GPU always has the next step queued, and this
            # rank is never more than one step ahead of what it has checked.
            ticket = worker.launch(StepBatch(data.view(np.int32)))
            if pending is not None:
                worker.collect(pending)
            pending = ticket


def follower_main(config: Config, rank: int, chan_name: str, init_method: str) -> None:
    """Entry point of a spawned follower process.  The channel exists before this process starts, so a
    failure at any point, start-up included, reaches rank 0 through the status word."""
    chan = rpc.ShmChannel(chan_name, config.tensor_parallel_size, rank, create=False, timeout_s=config.rpc_timeout_s)
    tp = None
    try:
        chan.hello()
        if config.device == "cuda":
            torch.cuda.set_device(rank)
        tp = TPGroup.init(rank, config.tensor_parallel_size, config.device, init_method, config.rpc_timeout_s)
        worker = Worker(config, rank, tp)
        tp.barrier()
        follower_loop(worker, chan)
        worker.close()
    except BaseException as e:                        # report, then die: rank 0 turns this into an error
        chan.report_failure(f"{type(e).__name__}: {e} | {traceback.format_exc()[-300:]}")
        raise
    finally:
        chan.close()
        if tp is not None:
            tp.close()
