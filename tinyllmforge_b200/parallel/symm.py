"""Symmetric memory for the in-kernel tensor-parallel exchange.

Every rank allocates the same region through ``torch.distributed._symmetric_memory`` (which exchanges the
handles between the processes and maps every peer's copy into this process); the kernels of this package then
read and write peers' memory directly over NVLink.  Only allocation and handle exchange are delegated; no
collective of that module is used.

Region layout (identical on every rank, byte offsets):
    signals   NUM_SITES x 8 words        word [site][r] = pushes rank r has completed at that site
    pairs     tp x 512 x {float, int}    sampler candidates, slot r written by rank r
    embed     max_tokens x H bf16        embedding rows, each written by the rank that owns the token id
    slots_o   tp x 256 x H bf16          o_proj partial sums, slot r written by rank r
    slots_d   tp x 256 x H bf16          down_proj partial sums
    slots_ar  tp x 256 x H bf16          operands of the standalone all-reduce / barrier

Replaces the NCCL calls at tinyvllm/layers/linear.py:183 and tinyvllm/layers/embed_head.py:41,66-67.
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch

SITE_EMBED, SITE_O, SITE_DOWN, SITE_SAMPLE, SITE_ALLREDUCE = 0, 1, 2, 3, 4
NUM_SITES = 8
MAX_PUSH_ROWS = 256          # rows the decode GEMM can push (its token limit)
MAX_PAIR_ROWS = 512


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


@dataclass
class Site:
    """Addresses one rank needs to take part in the exchange at one site."""
    index: int
    slot_ptrs: list[int]       # peer p -> where this rank writes its data in p's memory
    signal_ptrs: list[int]     # peer p -> this rank's signal word in p's memory
    local_slots: int           # where this rank reads
    slot_stride: int           # distance between slots, in bf16 elements
    num_slots: int             # slots to combine when reading
    local_signal: int
    arrive: int
    epoch: int
    mc_slot: int = 0           # NVLS multicast address of this rank's slot (0: no multicast support)


class FusedTPComm:
    def __init__(self, tp, hidden_size: int, max_tokens: int, device: torch.device, timeout_s: float = 2.0):
        import torch.distributed._symmetric_memory as symm_mem

        self.tp, self.rank, self.size = tp, tp.rank, tp.size
        self.hidden = hidden_size
        self.timeout_ns = int(timeout_s * 1e9)
        H = hidden_size
        off = {}
        cur = 0
        for name, nbytes in (("signals", NUM_SITES * 8 * 4), ("pairs", self.size * MAX_PAIR_ROWS * 8),
                             ("embed", max_tokens * H * 2), ("slots_o", self.size * MAX_PUSH_ROWS * H * 2),
                             ("slots_d", self.size * MAX_PUSH_ROWS * H * 2), ("slots_ar", self.size * MAX_PUSH_ROWS * H * 2)):
            off[name] = cur
            cur = _align(cur + nbytes)
        self.offsets, self.nbytes = off, cur
        self.region = symm_mem.empty(cur, dtype=torch.uint8, device=device)
        self.region.zero_()
        self.handle = symm_mem.rendezvous(self.region, group=tp.group)
        self.bases = [int(p) for p in self.handle.buffer_ptrs]
        self.multicast_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        if os.environ.get("FORGE_NVLS", "1") == "0":
            self.multicast_ptr = 0
        self.counters = torch.zeros(2 * NUM_SITES, dtype=torch.int32, device=device)     # private: arrive, epoch per site
        torch.cuda.synchronize()
        tp.barrier()                       # nobody pushes before every region is zeroed

        me = self.bases[self.rank]
        cbase = self.counters.data_ptr()

        def site(index, name, slot_bytes, shared_slot=False):
            return Site(
                index=index,
                slot_ptrs=[b + off[name] + (0 if shared_slot else self.rank * slot_bytes) for b in self.bases],
                signal_ptrs=[b + off["signals"] + (index * 8 + self.rank) * 4 for b in self.bases],
                local_slots=me + off[name], slot_stride=slot_bytes // 2, num_slots=1 if shared_slot else self.size,
                local_signal=me + off["signals"] + index * 8 * 4,
                arrive=cbase + (2 * index) * 4, epoch=cbase + (2 * index + 1) * 4,
                mc_slot=(self.multicast_ptr + off[name] + (0 if shared_slot else self.rank * slot_bytes)) if self.multicast_ptr else 0)

        self.sites = {
            SITE_EMBED: site(SITE_EMBED, "embed", max_tokens * H * 2, shared_slot=True),
            SITE_O: site(SITE_O, "slots_o", MAX_PUSH_ROWS * H * 2),
            SITE_DOWN: site(SITE_DOWN, "slots_d", MAX_PUSH_ROWS * H * 2),
            SITE_SAMPLE: site(SITE_SAMPLE, "pairs", MAX_PAIR_ROWS * 8),
            SITE_ALLREDUCE: site(SITE_ALLREDUCE, "slots_ar", MAX_PUSH_ROWS * H * 2),
        }
        self.max_tokens = max_tokens

    def close(self):
        self.handle = None
        self.region = None
