"""Megatron-style tensor-parallel layers: who owns which slice of which weight.

Parity:
  ReplicatedLinear            tinyvllm/layers/linear.py:27-49
  ColumnParallelLinear        tinyvllm/layers/linear.py:52-83   (output rows split)
  MergedColumnParallelLinear  tinyvllm/layers/linear.py:86-105  (gate and up each split, concatenated per rank)
  QKVParallelLinear           tinyvllm/layers/linear.py:113-150 (q, k, v head groups split, concatenated per rank)
  RowParallelLinear           tinyvllm/layers/linear.py:153-184 (input columns split, SUM over ranks)
  VocabParallelEmbedding      tinyvllm/layers/embed_head.py:9-42
  ParallelLMHead              tinyvllm/layers/embed_head.py:45-70

These are plain objects (no ``nn.Module``): each owns its shard, knows which slice of a full
Hugging Face tensor belongs to it (``shard_slices``; the loader reads only that slice from disk) and
runs the matching op of the model's op set.  The reference attaches a ``weight_loader`` method to
every parameter and reads whole tensors on every rank (tinyvllm/utils/loader.py:11-30).
"""
from __future__ import annotations

import torch

from .comm import TPGroup


def _div(a: int, b: int) -> int:
    assert a % b == 0, f"{a} is not divisible by {b}"
    return a // b


class LinearBase:
    def __init__(self, in_features: int, out_features: int, tp: TPGroup, dtype, device, bias: bool = False):
        self.tp = tp
        self.in_features, self.out_features = in_features, out_features
        self.weight = torch.empty(out_features, in_features, dtype=dtype, device=device)
        self.bias = torch.zeros(out_features, dtype=dtype, device=device) if bias else None

    def parameters(self):
        yield "weight", self.weight
        if self.bias is not None:
            yield "bias", self.bias

    # Slices of the full tensor -> slices of the local tensor. Each entry:
    # (dim, full_start, length, local_start). ``shard_id`` selects the packed sub-matrix.
    def shard_slices(self, full_shape, shard_id=None):
        return [(0, 0, full_shape[0], 0)]

    def load(self, param: torch.Tensor, read_slice, full_shape, shard_id=None) -> None:
        """``read_slice(dim, start, length)`` returns that slice of the full tensor (CPU)."""
        for dim, start, length, local in self.shard_slices(full_shape, shard_id):
            src = read_slice(dim, start, length)
            param.narrow(dim if param.dim() > 1 else 0, local, length).copy_(src)


class ReplicatedLinear(LinearBase):
    def forward(self, ops, x):
        y = ops.linear(x, self.weight)
        return y if self.bias is None else y + self.bias


class ColumnParallelLinear(LinearBase):
    def __init__(self, in_features, out_features, tp: TPGroup, dtype, device, bias=False):
        self.full_out = out_features
        super().__init__(in_features, _div(out_features, tp.size), tp, dtype, device, bias)

    def shard_slices(self, full_shape, shard_id=None):
        n = self.out_features
        return [(0, self.tp.rank * n, n, 0)]

    def forward(self, ops, x):
        y = ops.linear(x, self.weight)
        return y if self.bias is None else y + self.bias


class MergedColumnParallelLinear(ColumnParallelLinear):
    """Several column-parallel matrices stacked along the output dim (gate_proj, up_proj)."""

    def __init__(self, in_features, output_sizes: list[int], tp: TPGroup, dtype, device, bias=False):
        self.output_sizes = list(output_sizes)
        super().__init__(in_features, sum(output_sizes), tp, dtype, device, bias)

    def shard_slices(self, full_shape, shard_id=None):
        assert shard_id is not None
        n = _div(self.output_sizes[shard_id], self.tp.size)
        local = sum(self.output_sizes[:shard_id]) // self.tp.size
        return [(0, self.tp.rank * n, n, local)]

    def forward_silu_mul(self, ops, x):
        assert len(self.output_sizes) == 2 and self.bias is None
        return ops.linear_silu_mul(x, self.weight)


class QKVParallelLinear(ColumnParallelLinear):
    def __init__(self, hidden_size, head_dim, num_heads, num_kv_heads, tp: TPGroup, dtype, device, bias=False):
        self.head_dim = head_dim
        self.num_heads = _div(num_heads, tp.size)
        self.num_kv_heads = _div(num_kv_heads, tp.size)
        super().__init__(hidden_size, (num_heads + 2 * num_kv_heads) * head_dim, tp, dtype, device, bias)

    def shard_slices(self, full_shape, shard_id=None):
        assert shard_id in ("q", "k", "v")
        qn, kn = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        n, local = {"q": (qn, 0), "k": (kn, qn), "v": (kn, qn + kn)}[shard_id]
        return [(0, self.tp.rank * n, n, local)]


class RowParallelLinear(LinearBase):
    def __init__(self, in_features, out_features, tp: TPGroup, dtype, device, bias=False):
        self.full_in = in_features
        super().__init__(_div(in_features, tp.size), out_features, tp, dtype, device, bias)

    def shard_slices(self, full_shape, shard_id=None):
        if len(full_shape) == 1:      # bias: replicated, added on rank 0 only
            return [(0, 0, full_shape[0], 0)]
        n = self.in_features
        return [(1, self.tp.rank * n, n, 0)]

    def forward(self, ops, x):
        y = ops.linear(x, self.weight)
        if self.bias is not None and self.tp.rank == 0:
            y = y + self.bias
        return ops.tp_all_reduce(y, self.tp)


class VocabParallelEmbedding:
    def __init__(self, vocab_size, hidden_size, tp: TPGroup, dtype, device):
        self.tp = tp
        self.vocab_size = vocab_size
        self.shard = _div(vocab_size, tp.size)
        self.vocab_start = tp.rank * self.shard
        self.weight = torch.empty(self.shard, hidden_size, dtype=dtype, device=device)

    def parameters(self):
        yield "weight", self.weight

    def shard_slices(self, full_shape, shard_id=None):
        return [(0, self.vocab_start, self.shard, 0)]

    load = LinearBase.load

    def forward(self, ops, ids):
        y = ops.embedding(ids, self.weight, self.vocab_start)
        return ops.tp_all_reduce(y, self.tp)


class ParallelLMHead(VocabParallelEmbedding):
    """Vocab-sharded output projection.  ``forward`` returns this rank's logits shard
    ``[rows, vocab / tp]``; ``ops.sample`` then reduces each shard to one (score, id) pair per row and
    only those pairs cross ranks.  ``full_logits`` is the materialising variant (the reference gathers
    whole shards to rank 0: tinyvllm/layers/embed_head.py:63-70)."""

    def forward(self, ops, hidden):
        return ops.linear(hidden, self.weight)

    def full_logits(self, ops, hidden):
        return self.tp.all_gather_cat(ops.linear(hidden, self.weight), dim=-1)
