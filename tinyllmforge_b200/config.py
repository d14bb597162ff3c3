"""Engine and model configuration.

Parity: tinyvllm/config.py:5-26 (same field names and defaults for the fields
the reference has) and tinyvllm/engine/llm_engine.py:18-20 (built from the
keyword arguments of ``LLM``).  Differences, all deliberate:

* unknown keyword arguments raise instead of being dropped silently;
* the KV block size may be any power of two >= 16 on the GPU and >= 8 on the CPU
  path (the reference's flash-attn call needs a multiple of 256);
* ``config.json`` is parsed directly into :class:`ModelConfig`, so building an
  engine does not import ``transformers``;
* extra optional fields: ``seed``, ``dtype``, ``device``, ``comm``,
  ``quantization``, ``load_format``, ``skip_tokenizer_init``, ``chunked_prefill``.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, fields
from typing import Any, Optional

import torch

_DTYPES = {
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float16": torch.float16, "fp16": torch.float16, "half": torch.float16,
    "float32": torch.float32, "fp32": torch.float32, "float": torch.float32,
}


def parse_dtype(value) -> torch.dtype:
    if isinstance(value, torch.dtype):
        return value
    key = str(value).replace("torch.", "")
    if key not in _DTYPES:
        raise ValueError(f"unsupported dtype {value!r}")
    return _DTYPES[key]


@dataclass
class ModelConfig:
    """The subset of a Hugging Face Qwen3 ``config.json`` the engine uses.

    Parity: the attributes read from ``hf_config`` at tinyvllm/models/qwen3.py:140-150
    and tinyvllm/engine/model_runner.py:118-127.
    """
    hidden_size: int = 1024
    num_hidden_layers: int = 28
    num_attention_heads: int = 16
    num_key_value_heads: int = 8
    head_dim: int = 128
    intermediate_size: int = 3072
    vocab_size: int = 151936
    rope_theta: float = 1_000_000.0
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = True
    max_position_embeddings: int = 40960
    torch_dtype: str = "bfloat16"
    attention_bias: bool = False
    hidden_act: str = "silu"
    eos_token_id: int = -1
    model_type: str = "qwen3"

    @classmethod
    def from_dict(cls, d: dict) -> "ModelConfig":
        known = {f.name for f in fields(cls)}
        kw = {k: v for k, v in d.items() if k in known and v is not None}
        if "torch_dtype" not in kw and "dtype" in d and d["dtype"] is not None:
            kw["torch_dtype"] = d["dtype"]
        if "torch_dtype" in kw:
            kw["torch_dtype"] = str(kw["torch_dtype"]).replace("torch.", "")
        if "head_dim" not in kw and "hidden_size" in kw and "num_attention_heads" in kw:
            kw["head_dim"] = kw["hidden_size"] // kw["num_attention_heads"]
        rope = d.get("rope_parameters") or {}
        if "rope_theta" not in kw and "rope_theta" in rope:
            kw["rope_theta"] = rope["rope_theta"]
        eos = kw.get("eos_token_id", -1)
        if isinstance(eos, (list, tuple)):
            kw["eos_token_id"] = int(eos[0]) if eos else -1
        scaling = d.get("rope_scaling")
        if scaling not in (None, {}) and (scaling.get("rope_type", scaling.get("type")) not in (None, "default")):
            raise ValueError("rope_scaling is not supported (the reference asserts it is None, "
                             "tinyvllm/layers/rotary_embedding.py:68)")
        cfg = cls(**kw)
        cfg.validate()
        return cfg

    @classmethod
    def from_dir(cls, path: str) -> "ModelConfig":
        with open(os.path.join(path, "config.json")) as f:
            return cls.from_dict(json.load(f))

    def to_hf_dict(self) -> dict:
        d = {f.name: getattr(self, f.name) for f in fields(self)}
        d["architectures"] = ["Qwen3ForCausalLM"]
        d["rope_scaling"] = None
        d["use_cache"] = True
        d["max_window_layers"] = self.num_hidden_layers
        d["use_sliding_window"] = False
        d["sliding_window"] = None
        d["attention_dropout"] = 0.0
        d["initializer_range"] = 0.02
        if d["eos_token_id"] < 0:
            d["eos_token_id"] = None
        return d

    def validate(self):
        if self.model_type not in ("qwen3",):
            raise ValueError(f"unsupported model_type {self.model_type!r}; supported: qwen3")
        if self.hidden_act != "silu":
            raise ValueError("only the SiLU-gated MLP is supported")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ValueError("num_attention_heads must be a multiple of num_key_value_heads")
        if self.head_dim % 2:
            raise ValueError("head_dim must be even for rotary embedding")

    @property
    def dtype(self) -> torch.dtype:
        return parse_dtype(self.torch_dtype)


# Architectures named by the benchmark definition; weights are random-init.
PRESETS = {
    "tiny": dict(hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                 head_dim=64, intermediate_size=512, vocab_size=4096, tie_word_embeddings=True,
                 max_position_embeddings=4096, torch_dtype="float32"),
    "qwen3-0.6b": dict(hidden_size=1024, num_hidden_layers=28, num_attention_heads=16, num_key_value_heads=8,
                       head_dim=128, intermediate_size=3072, vocab_size=151936, tie_word_embeddings=True),
    "qwen3-1.7b": dict(hidden_size=2048, num_hidden_layers=28, num_attention_heads=16, num_key_value_heads=8,
                       head_dim=128, intermediate_size=6144, vocab_size=151936, tie_word_embeddings=True),
    "qwen3-4b": dict(hidden_size=2560, num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8,
                     head_dim=128, intermediate_size=9728, vocab_size=151936, tie_word_embeddings=True),
    "qwen3-8b": dict(hidden_size=4096, num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8,
                     head_dim=128, intermediate_size=12288, vocab_size=151936, tie_word_embeddings=False),
    "qwen3-14b": dict(hidden_size=5120, num_hidden_layers=40, num_attention_heads=40, num_key_value_heads=8,
                      head_dim=128, intermediate_size=17408, vocab_size=151936, tie_word_embeddings=False),
    "qwen3-32b": dict(hidden_size=5120, num_hidden_layers=64, num_attention_heads=64, num_key_value_heads=8,
                      head_dim=128, intermediate_size=25600, vocab_size=151936, tie_word_embeddings=False),
}


def preset(name: str, **overrides) -> ModelConfig:
    if name not in PRESETS:
        raise KeyError(f"unknown preset {name!r}; known: {sorted(PRESETS)}")
    return ModelConfig.from_dict({**PRESETS[name], **overrides})


@dataclass
class Config:
    model: str
    max_num_batched_tokens: int = 16384
    max_num_seqs: int = 512
    max_model_len: int = 4096
    gpu_memory_utilization: float = 0.9
    tensor_parallel_size: int = 1
    enforce_eager: bool = False
    hf_config: Optional[ModelConfig] = None
    eos: int = -1
    kvcache_block_size: int = 256
    num_kvcache_blocks: int = -1
    # --- fields the reference does not have ---
    seed: int = 0
    dtype: Optional[Any] = None              # None: the checkpoint's torch_dtype
    device: str = "auto"                     # "auto" | "cuda" | "cpu"
    comm: str = "fused"                      # "fused": in-kernel NVLink collectives; "nccl": torch.distributed calls
    quantization: Optional[str] = None       # None | "fp8_block"
    load_format: str = "auto"                # "auto": read *.safetensors; "dummy": seeded N(0, 0.02) weights
    skip_tokenizer_init: bool = False
    rpc_timeout_s: float = 120.0             # bound on every control-plane wait between ranks
    comm_timeout_s: float = 10.0             # bound on every device-side wait for a peer's flag (comm="fused")
    trace_path: Optional[str] = None         # per-step JSONL trace
    chunked_prefill: bool = False            # prompts longer than max_num_batched_tokens are prefilled over several steps
    extra: dict = field(default_factory=dict)

    def __post_init__(self):
        if self.hf_config is None:
            if not os.path.isdir(self.model):
                raise FileNotFoundError(f"model directory not found: {self.model}")
            self.hf_config = ModelConfig.from_dir(self.model)
        elif isinstance(self.hf_config, dict):
            self.hf_config = ModelConfig.from_dict(self.hf_config)
        bs = self.kvcache_block_size
        if bs < 8 or bs & (bs - 1):
            raise ValueError(f"kvcache_block_size must be a power of two >= 8, got {bs}")
        if not 1 <= self.tensor_parallel_size <= 8:
            raise ValueError("tensor_parallel_size must be in [1, 8] (single host)")
        hf = self.hf_config
        if hf.num_key_value_heads % self.tensor_parallel_size or hf.num_attention_heads % self.tensor_parallel_size:
            raise ValueError("attention heads and KV heads must divide evenly by tensor_parallel_size")
        if hf.vocab_size % self.tensor_parallel_size:
            raise ValueError("vocab_size must divide evenly by tensor_parallel_size")
        self.max_model_len = min(self.max_model_len, hf.max_position_embeddings)
        if self.max_num_batched_tokens < self.max_model_len and not self.chunked_prefill:
            raise ValueError("max_num_batched_tokens must be >= max_model_len (prompts are prefilled whole; "
                             "chunked_prefill=True lifts this)")
        if self.max_num_batched_tokens < self.kvcache_block_size:
            raise ValueError("max_num_batched_tokens must be at least one KV block")
        if self.device == "auto":
            self.device = "cuda" if torch.cuda.is_available() else "cpu"
        if self.device not in ("cuda", "cpu"):
            raise ValueError(f"device must be 'cuda' or 'cpu', got {self.device!r}")
        if self.device == "cuda" and bs < 16:
            raise ValueError(f"kvcache_block_size must be >= 16 on the GPU (the attention kernels' smallest tile), got {bs}")
        if not self.comm_timeout_s > 0:
            raise ValueError("comm_timeout_s must be positive")
        if self.comm not in ("fused", "nccl"):
            raise ValueError("comm must be 'fused' or 'nccl'")
        if self.quantization not in (None, "fp8_block"):
            raise ValueError("quantization must be None or 'fp8_block'")
        if self.load_format not in ("auto", "dummy"):
            raise ValueError("load_format must be 'auto' or 'dummy'")
        self.dtype = parse_dtype(self.dtype) if self.dtype is not None else hf.dtype
        if self.eos < 0 and hf.eos_token_id is not None:
            self.eos = hf.eos_token_id

    @classmethod
    def from_kwargs(cls, model: str, **kwargs) -> "Config":
        known = {f.name for f in fields(cls)}
        unknown = sorted(set(kwargs) - known)
        if unknown:
            raise TypeError(f"unknown engine option(s): {unknown}; valid: {sorted(known - {'model'})}")
        return cls(model, **kwargs)
