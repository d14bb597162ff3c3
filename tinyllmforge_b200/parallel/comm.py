"""Tensor-parallel group: rank bookkeeping and the library-collective path.

Parity: the reference uses the default ``torch.distributed`` process group as its
tensor-parallel group (tinyvllm/layers/linear.py:20-21, tinyvllm/engine/model_runner.py:26-31)
with ``all_reduce`` (linear.py:183, embed_head.py:41), ``gather`` (embed_head.py:66-67) and
``barrier``.  This class is that path (NCCL on GPUs, gloo on CPU).  The in-kernel NVLink
collectives live in ``parallel/symm.py`` and ``ops/cuda.py``; they are selected by
``Config.comm == "fused"`` and fall back to nothing: a missing extension raises.

Rendezvous uses a caller-supplied free port on 127.0.0.1 (the reference hard-wires
port 2333, so two engines on one host collide).
"""
from __future__ import annotations

import datetime
import socket

import torch
import torch.distributed as dist


def find_free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class TPGroup:
    """World == tensor-parallel group, as in the reference. ``size == 1`` needs no process group."""

    def __init__(self, rank: int = 0, size: int = 1, group=None):
        self.rank = rank
        self.size = size
        self.group = group
        self._owns_pg = False

    @classmethod
    def init(cls, rank: int, size: int, device: str, init_method: str | None, timeout_s: float = 120.0) -> "TPGroup":
        if size == 1:
            return cls(0, 1)
        if dist.is_initialized():
            # launched under torchrun or by a test harness: reuse the default group
            assert dist.get_world_size() == size and dist.get_rank() == rank
            return cls(rank, size, dist.group.WORLD)
        backend = "nccl" if device == "cuda" else "gloo"
        kw = {}
        if device == "cuda":
            kw["device_id"] = torch.device("cuda", torch.cuda.current_device())
        dist.init_process_group(backend, init_method=init_method, world_size=size, rank=rank,
                                timeout=datetime.timedelta(seconds=timeout_s), **kw)
        g = cls(rank, size, dist.group.WORLD)
        g._owns_pg = True
        return g

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.size > 1:
            dist.all_reduce(x, group=self.group)
        return x

    def all_gather_cat(self, x: torch.Tensor, dim: int = -1) -> torch.Tensor:
        if self.size == 1:
            return x
        parts = [torch.empty_like(x) for _ in range(self.size)]
        dist.all_gather(parts, x.contiguous(), group=self.group)
        return torch.cat(parts, dim=dim)

    def all_gather_stack(self, x: torch.Tensor) -> torch.Tensor:
        """[size, *x.shape]"""
        if self.size == 1:
            return x[None]
        out = torch.empty(self.size * x.numel(), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous().view(-1), group=self.group)
        return out.view((self.size,) + tuple(x.shape))

    def barrier(self) -> None:
        if self.size > 1:
            dist.barrier(group=self.group)

    def close(self) -> None:
        if self._owns_pg and dist.is_initialized():
            dist.destroy_process_group()
            self._owns_pg = False
