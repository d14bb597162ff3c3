"""Hugging Face safetensors -> sharded local weights.

Parity: tinyvllm/utils/loader.py:7-30 and the per-layer ``weight_loader`` methods
(tinyvllm/layers/linear.py:75-80,96-105,134-150,172-177; tinyvllm/layers/embed_head.py:24-30).
Same name protocol (q/k/v -> qkv_proj, gate/up -> gate_up_proj), but each rank reads from disk only the
slice it owns (``safe_open(...).get_slice``) instead of every rank reading every full tensor, and
missing or unexpected tensors are reported instead of ignored.

``init_dummy_weights`` fills a model with seeded N(0, 0.02) values (norm weights 1) without touching the
disk: the benchmark definition asks for random-init weights of a named architecture.
"""
from __future__ import annotations

import glob
import os

import torch


def load_weights(model, path: str, strict: bool = True) -> None:
    from safetensors import safe_open

    files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"no *.safetensors files in {path}")
    wanted = {name: (param, owner, sid) for name, param, owner, sid in model.named_parameters()}
    seen = set()
    for file in files:
        with safe_open(file, "pt", "cpu") as f:
            for name in f.keys():
                if name not in wanted:
                    if name == "lm_head.weight" and model.cfg.tie_word_embeddings:
                        continue
                    if strict and "rotary_emb.inv_freq" not in name:
                        raise KeyError(f"unexpected tensor {name!r} in {file}")
                    continue
                param, owner, sid = wanted[name]
                sl = f.get_slice(name)
                shape = tuple(sl.get_shape())
                if owner is None:
                    param.copy_(f.get_tensor(name))
                else:
                    def read_slice(dim, start, length, _sl=sl, _nd=len(shape)):
                        if _nd == 1 or dim == 0:
                            return _sl[start:start + length]
                        return _sl[:, start:start + length]
                    owner.load(param, read_slice, shape, sid)
                seen.add(name)
    missing = sorted(set(wanted) - seen)
    if strict and missing:
        raise KeyError(f"checkpoint is missing {len(missing)} tensors, e.g. {missing[:4]}")


@torch.no_grad()
def init_dummy_weights(model, seed: int = 0, std: float = 0.02) -> None:
    """Seeded N(0, std) for matrices, ones for norm weights. Each rank draws its own shard
    (seed mixed with the rank), so no rank materialises a full tensor."""
    dev = model.device
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed * 1000003 + model.tp.rank)
    for name, param, owner, _ in model.named_parameters():
        if owner is None:
            param.fill_(1.0)
        elif name.endswith(".bias"):
            param.zero_()
        else:
            param.normal_(0.0, std, generator=gen)
