"""Symmetric memory for the in-kernel tensor-parallel exchange.

Every rank allocates the same region through ``torch.distributed._symmetric_memory`` (which exchanges the
handles between the processes, maps every peer's copy into this process and, where the driver supports it,
binds all copies to one NVSwitch multicast address); the kernels of this package then read and write peers'
memory directly over NVLink, or all copies at once through the multicast address (``multimem.ld_reduce`` /
``multimem.st``).  Only allocation and handle exchange are delegated; no collective of that module is used.

Region layout (identical on every rank, byte offsets):
    signals   NUM_SITES x 8 words        word [site][r] = productions rank r has completed at that site
    pairs     tp x 512 x {float, int}    sampler candidates, slot r written by rank r
    embed     max_tokens x H bf16        embedding rows, each written by the rank that owns the token id
    part_o    max_tokens x H bf16        THIS rank's o_proj partial sums (peers pull the sum of all ranks' copies)
    part_d    max_tokens x H bf16        the same for down_proj
    part_ar   256 x H bf16               operand of the standalone all-reduce / barrier
    y         max_tokens x H bf16        normalised rows, each broadcast by the rank that reduced it (two-shot exchange)
    ll_o      tp x ceil(256/tp) x H words   decode-sized o_proj exchange: tagged partial rows this rank owns, one area per
    ll_d                                    source rank (every bf16 pair travels as {payload, tag}); the same for down_proj
    ll_y      256 x H words              tagged normalised rows sent by their owners

Replaces the NCCL calls at tinyvllm/layers/linear.py:183 and tinyvllm/layers/embed_head.py:41,66-67.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field

import torch

SITE_EMBED, SITE_O, SITE_DOWN, SITE_SAMPLE, SITE_ALLREDUCE, SITE_GATHER = 0, 1, 2, 3, 4, 5
NUM_SITES = 8
MAX_ALLREDUCE_ROWS = 256     # rows of `hidden` elements the standalone all-reduce accepts
MAX_PAIR_ROWS = 512
MAX_TAGGED_ROWS = 256        # rows of a decode-sized exchange (the weight-tile GEMM's limit)


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


@dataclass
class Site:
    """Addresses one rank needs to take part in the exchange at one site."""
    index: int
    signal_ptrs: list[int]     # peer p -> this rank's signal word in p's memory
    local_signal: int          # this rank's signal words (one per rank)
    arrive: int                # private counters
    epoch: int
    buf_ptrs: list[int] = field(default_factory=list)    # every rank's copy of the site's buffer, rank order
    local_buf: int = 0         # this rank's copy
    mc_buf: int = 0            # NVSwitch multicast address of the buffer (0: no multicast support)
    slot_ptrs: list[int] = field(default_factory=list)   # per-rank slots (pairs): peer p -> slot [rank] in p's buffer
    slot_stride: int = 0       # distance between slots, in bf16 elements
    ll_ptrs: list[int] = field(default_factory=list)     # every rank's tagged-word buffer of the site, rank order
    ll_local: int = 0


class FusedTPComm:
    def __init__(self, tp, hidden_size: int, max_tokens: int, device: torch.device, timeout_s: float = 10.0):
        import torch.distributed._symmetric_memory as symm_mem

        self.tp, self.rank, self.size = tp, tp.rank, tp.size
        self.hidden = hidden_size
        self.max_tokens = max_tokens
        self.timeout_ns = int(timeout_s * 1e9)
        # one-shot (every rank pulls every row) moves tp x the tensor per direction, two-shot ~1x plus a second flag
        # round: switch over when the extra bytes cost more than that round
        self.two_shot_bytes = int(os.environ.get("FORGE_TP_TWO_SHOT_BYTES", str(2 << 20)))
        H = hidden_size
        self.tagged = os.environ.get("FORGE_TP_TAGGED", "1") != "0"      # decode-sized exchanges as tagged words (else: pulls)
        self.tagged_rows_per_rank = (MAX_TAGGED_ROWS + self.size - 1) // self.size
        ll_bytes = self.size * self.tagged_rows_per_rank * H * 4
        rows_bytes = max_tokens * H * 2
        off = {}
        cur = 0
        for name, nbytes in (("signals", NUM_SITES * 8 * 4), ("pairs", self.size * MAX_PAIR_ROWS * 8), ("embed", rows_bytes),
                             ("part_o", rows_bytes), ("part_d", rows_bytes), ("part_ar", MAX_ALLREDUCE_ROWS * H * 2),
                             ("y", rows_bytes), ("ll_o", ll_bytes), ("ll_d", ll_bytes), ("ll_y", MAX_TAGGED_ROWS * H * 4)):
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
        # private words: arrive, epoch per site, then the measurement-mode switch
        self.counters = torch.zeros(2 * NUM_SITES + 2, dtype=torch.int32, device=device)
        torch.cuda.synchronize()
        tp.barrier()                       # nobody produces before every region is zeroed

        me = self.bases[self.rank]
        cbase = self.counters.data_ptr()
        self.local_only = cbase + 2 * NUM_SITES * 4
        mc = self.multicast_ptr

        def site(index, name=None, slot_bytes=0):
            s = Site(index=index,
                     signal_ptrs=[b + off["signals"] + (index * 8 + self.rank) * 4 for b in self.bases],
                     local_signal=me + off["signals"] + index * 8 * 4,
                     arrive=cbase + (2 * index) * 4, epoch=cbase + (2 * index + 1) * 4)
            if name is not None:
                s.buf_ptrs = [b + off[name] for b in self.bases]
                s.local_buf = me + off[name]
                s.mc_buf = mc + off[name] if mc else 0
                if slot_bytes:
                    s.slot_ptrs = [b + off[name] + self.rank * slot_bytes for b in self.bases]
                    s.slot_stride = slot_bytes // 2
            if index in (SITE_O, SITE_DOWN, SITE_GATHER):
                ll = {SITE_O: "ll_o", SITE_DOWN: "ll_d", SITE_GATHER: "ll_y"}[index]
                s.ll_ptrs = [b + off[ll] for b in self.bases]
                s.ll_local = me + off[ll]
            return s

        self.sites = {
            SITE_EMBED: site(SITE_EMBED, "embed"),
            SITE_O: site(SITE_O, "part_o"),
            SITE_DOWN: site(SITE_DOWN, "part_d"),
            SITE_SAMPLE: site(SITE_SAMPLE, "pairs", MAX_PAIR_ROWS * 8),
            SITE_ALLREDUCE: site(SITE_ALLREDUCE, "part_ar"),
            SITE_GATHER: site(SITE_GATHER, "y"),
        }

    def use_tagged(self, rows: int, width: int) -> bool:
        """Decode-sized exchange of the model's hidden width: tagged words pushed from the GEMM epilogue."""
        return self.tagged and rows <= MAX_TAGGED_ROWS and width == self.hidden and width % 8 == 0

    def two_shot(self, rows: int, width: int) -> bool:
        """Reduce-scatter + all-gather instead of every rank pulling every row?  Depends only on the shape, so all
        ranks decide alike."""
        return (self.size - 1) * rows * width * 2 > self.two_shot_bytes

    def y_view(self, rows: int, width: int) -> torch.Tensor:
        """The first ``rows x width`` bf16 elements of this rank's broadcast buffer as a tensor."""
        o = self.offsets["y"]
        return self.region[o:o + rows * width * 2].view(torch.bfloat16).view(rows, width)

    def set_local_only(self, on: bool) -> None:
        """Measurement mode (stream-ordered): the exchange kernels skip their waits and peer traffic and work on this
        rank's own data only.  Results are wrong on purpose; the time difference to a normal run is the exposed
        communication.  Callers synchronise all ranks (device and host) before switching either way."""
        with torch.inference_mode():           # the counters may have been created under inference mode (the worker's constructor)
            self.counters[2 * NUM_SITES] = 1 if on else 0

    def close(self):
        self.handle = None
        self.region = None
