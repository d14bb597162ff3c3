"""Synthetic Hugging Face checkpoint directories (config.json + safetensors + an offline tokenizer).

No model files or network exist where the benchmarks run, and the benchmark definition asks for
random-init N(0, 0.02) weights of a named architecture.  The directory written here is loadable by
this engine, by ``transformers`` and by the reference engine (which needs ``config.json``, HF tensor
names and ``AutoTokenizer`` files: tinyvllm/config.py:24, tinyvllm/utils/loader.py:11-30,
tinyvllm/engine/llm_engine.py:32).
"""
from __future__ import annotations

import json
import os

import torch

from ..config import ModelConfig


def hf_tensor_shapes(cfg: ModelConfig) -> dict[str, tuple]:
    H, d, I, V = cfg.hidden_size, cfg.head_dim, cfg.intermediate_size, cfg.vocab_size
    nh, nkv = cfg.num_attention_heads, cfg.num_key_value_heads
    shapes = {"model.embed_tokens.weight": (V, H), "model.norm.weight": (H,)}
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        shapes.update({
            p + "self_attn.q_proj.weight": (nh * d, H), p + "self_attn.k_proj.weight": (nkv * d, H),
            p + "self_attn.v_proj.weight": (nkv * d, H), p + "self_attn.o_proj.weight": (H, nh * d),
            p + "self_attn.q_norm.weight": (d,), p + "self_attn.k_norm.weight": (d,),
            p + "mlp.gate_proj.weight": (I, H), p + "mlp.up_proj.weight": (I, H), p + "mlp.down_proj.weight": (H, I),
            p + "input_layernorm.weight": (H,), p + "post_attention_layernorm.weight": (H,),
        })
    if not cfg.tie_word_embeddings:
        shapes["lm_head.weight"] = (V, H)
    return shapes


def write_tokenizer(path: str, vocab_size: int) -> None:
    """A tiny word-level tokenizer (tokenizer.json) so ``AutoTokenizer.from_pretrained`` works offline."""
    from tokenizers import Tokenizer, models, pre_tokenizers

    n_words = min(vocab_size - 3, 2000)
    vocab = {"<unk>": 0, "<eos>": 1, "<pad>": 2}
    for i in range(n_words):
        vocab[f"w{i}"] = 3 + i
    tok = Tokenizer(models.WordLevel(vocab=vocab, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    tok.save(os.path.join(path, "tokenizer.json"))
    with open(os.path.join(path, "tokenizer_config.json"), "w") as f:
        json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "unk_token": "<unk>", "eos_token": "<eos>",
                   "pad_token": "<pad>", "model_max_length": 1 << 20}, f)
    with open(os.path.join(path, "special_tokens_map.json"), "w") as f:
        json.dump({"unk_token": "<unk>", "eos_token": "<eos>", "pad_token": "<pad>"}, f)


def checkpoint_bytes(cfg: ModelConfig) -> int:
    """Size of the safetensors data ``write_checkpoint`` produces for ``cfg``."""
    itemsize = torch.finfo(cfg.dtype).bits // 8
    return sum(itemsize * int(torch.Size(shape).numel()) for shape in hf_tensor_shapes(cfg).values())


def write_checkpoint(path: str, cfg: ModelConfig, seed: int = 0, std: float = 0.02, tokenizer: bool = True,
                     shard_bytes: int = 4 << 30, norm_std: float = 0.0, device: str = "cpu", weights: bool = True) -> str:
    """Write ``config.json`` and seeded random weights under HF names; returns ``path``.
    Matrices are N(0, std); norm weights are 1 (+ N(0, norm_std) when asked, which makes tests sharper).
    ``device="cuda"`` draws the numbers on the GPU (a multi-GB checkpoint then takes seconds instead of minutes; the
    values differ from the CPU generator's for the same seed).  ``weights=False`` writes only ``config.json`` and the
    tokenizer (for engines that initialise their weights on the device)."""
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    d = cfg.to_hf_dict()
    if tokenizer:
        d["eos_token_id"] = 1
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(d, f, indent=1)
    if not weights:
        if tokenizer:
            write_tokenizer(path, cfg.vocab_size)
        return path
    gen = torch.Generator(device=device).manual_seed(seed)
    dtype = cfg.dtype
    itemsize = torch.finfo(dtype).bits // 8
    # plan the shards first so the files can carry the "-i-of-n" names transformers expects
    plan, cur, size = [], [], 0
    for name, shape in hf_tensor_shapes(cfg).items():
        cur.append((name, shape))
        size += itemsize * int(torch.Size(shape).numel())
        if size >= shard_bytes:
            plan.append(cur)
            cur, size = [], 0
    if cur:
        plan.append(cur)
    weight_map = {}
    for i, group in enumerate(plan):
        fname = "model.safetensors" if len(plan) == 1 else f"model-{i + 1:05d}-of-{len(plan):05d}.safetensors"
        shard = {}
        for name, shape in group:
            if len(shape) == 1:
                t = torch.ones(shape, dtype=dtype)
                if norm_std > 0:
                    t = (t.float() + torch.empty(shape, device=device).normal_(0.0, norm_std, generator=gen).cpu()).to(dtype)
            else:
                t = torch.empty(shape, dtype=torch.float32, device=device).normal_(0.0, std, generator=gen).to(dtype).cpu()
            shard[name] = t
            weight_map[name] = fname
        save_file(shard, os.path.join(path, fname), metadata={"format": "pt"})
    if len(plan) > 1:
        with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
            json.dump({"metadata": {}, "weight_map": weight_map}, f)
    if tokenizer:
        write_tokenizer(path, cfg.vocab_size)
    return path
