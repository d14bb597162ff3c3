"""Run-time repairs that let the reference engine start at tensor_parallel_size > 1.

As written the reference cannot run on more than one GPU (four independent defects, all on the multi-process
path).  To measure "the reference at TP = 2/4/8" its installed copy under ``baseline/_ref`` is left byte-identical
and the four spots are replaced in memory, in the parent and (through ``worker_entry``) in every spawned worker:

  B1  tinyvllm/engine/llm_engine.py:26   worker ``args`` is a set literal holding an unhashable dataclass
  B2  tinyvllm/engine/sequence.py:75-85  ``__setstate__`` unpacks ``state[-1]`` and assigns a read-only property
  B3  tinyvllm/engine/model_runner.py:104  ``write_shm(method_name, args)`` forgets to splat ``args``
  B4  tinyvllm/layers/embed_head.py:69   ``self.tp.rank`` typo; logits concatenated along the batch, not the vocabulary
  B14 tinyvllm/layers/linear.py:128-130  QKVParallelLinear hands the PER-RANK output size to a base class that divides
      by the TP size again, so the parameter is tp times too small and the k/v shards do not fit (found when the
      repaired engine first reached weight loading at TP = 2)

Each replacement restates the surrounding reference lines with only the defect removed.  Single-GPU runs do not
use this module.
"""
from __future__ import annotations

import atexit


def apply() -> list[str]:
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F
    from tinyvllm.engine import llm_engine, model_runner, sequence
    from tinyvllm.layers import embed_head
    from tinyvllm.utils.context import get_context

    Sequence, ModelRunner = sequence.Sequence, model_runner.ModelRunner

    # B2 -------------------------------------------------------------------------------------------------
    def getstate(self):
        return (self.num_tokens, self.num_prompt_tokens, self.num_cached_tokens, self.block_table,
                self.token_ids if self.num_completion_tokens == 0 else self.last_token)

    def setstate(self, state):
        self.num_tokens, self.num_prompt_tokens, self.num_cached_tokens, self.block_table = state[:-1]
        if self.num_completion_tokens == 0:
            self.token_ids = state[-1]
        else:
            self.last_token = state[-1]
    Sequence.__getstate__, Sequence.__setstate__ = getstate, setstate

    # B3 -------------------------------------------------------------------------------------------------
    def call(self, method_name, *args):
        if self.world_size > 1 and self.rank == 0:
            self.write_shm(method_name, *args)
        return getattr(self, method_name, None)(*args)
    ModelRunner.call = call

    # B4 -------------------------------------------------------------------------------------------------
    def lm_head_forward(self, x):
        context = get_context()
        if context.is_prefill:
            x = x[context.cu_seqlens_q[1:] - 1].contiguous()
        logits = F.linear(x, self.weight, self.bias)
        if self.tp_size > 1:
            all_logits = [torch.empty_like(logits) for _ in range(self.tp_size)] if self.tp_rank == 0 else None
            dist.gather(logits, all_logits, 0)
            logits = torch.cat(all_logits, -1) if self.tp_rank == 0 else None
        return logits
    embed_head.ParallelLMHead.forward = lm_head_forward

    # B14 ------------------------------------------------------------------------------------------------
    from tinyvllm.layers import linear

    def qkv_init(self, hidden_size, head_size, total_num_heads, total_num_kv_heads=None, bias=False):
        self.head_size = head_size
        self.total_num_heads = total_num_heads
        self.total_num_kv_heads = total_num_kv_heads or total_num_heads
        tp_size = dist.get_world_size()
        self.num_heads = linear.divide(self.total_num_heads, tp_size)
        self.num_kv_heads = linear.divide(self.total_num_kv_heads, tp_size)
        output_size = (self.total_num_heads + 2 * self.total_num_kv_heads) * head_size     # full size: the base class shards it
        linear.ColumnParallelLinear.__init__(self, hidden_size, output_size, bias)
    linear.QKVParallelLinear.__init__ = qkv_init

    # B1 -------------------------------------------------------------------------------------------------
    def engine_init(self, model, **kwargs):
        from dataclasses import fields
        import torch.multiprocessing as mp
        from transformers import AutoTokenizer
        Config = llm_engine.Config
        config_fields = {f.name for f in fields(Config)}
        config = Config(model, **{k: v for k, v in kwargs.items() if k in config_fields})
        self.ps, self.events = [], []
        ctx = mp.get_context("spawn")
        for i in range(1, config.tensor_parallel_size):
            event = ctx.Event()
            process = ctx.Process(target=worker_entry, args=(config, i, event))
            process.start()
            self.ps.append(process)
            self.events.append(event)
        self.model_runner = ModelRunner(config, 0, self.events)
        self.tokenizer = AutoTokenizer.from_pretrained(config.model, use_fast=True)
        config.eos = self.tokenizer.eos_token_id
        self.scheduler = llm_engine.Scheduler(config)
        atexit.register(self.exit)
    llm_engine.LLMEngine.__init__ = engine_init
    return ["B1 worker args tuple", "B2 Sequence pickling", "B3 RPC args splat", "B4 LM-head gather along vocabulary",
            "B14 QKV parameter size"]


def apply_dummy_load() -> str:
    """Replace the reference's checkpoint loader (tinyvllm/utils/loader.py:11-30) by a random initialisation on the
    device, for architectures whose safetensors files would be tens of GB (Qwen3-32B: 64 GB, read in full by every
    rank).  Weight values do not change what the timed region does; loading is outside it."""
    import torch
    from tinyvllm.engine import model_runner

    def dummy_load(model, path):
        g = torch.Generator(device="cuda").manual_seed(0)
        for _, p in model.named_parameters():
            if p.dim() >= 2:
                p.data.normal_(0.0, 0.02, generator=g)
            else:
                p.data.fill_(1.0)
    model_runner.load_model = dummy_load
    return "checkpoint loader replaced by on-device random init N(0, 0.02)"


def worker_entry(config, rank, event):
    """Spawn target of ranks 1..tp-1: repair this interpreter, then run the reference's worker as it would."""
    import os
    apply()
    if os.environ.get("FORGE_REF_DUMMY_LOAD") == "1":
        apply_dummy_load()
    from tinyvllm.engine.model_runner import ModelRunner
    ModelRunner(config, rank, event)
