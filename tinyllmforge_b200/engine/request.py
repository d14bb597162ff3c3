"""Per-request generation state.

Parity: tinyvllm/engine/sequence.py:6-85.  The reference's ``Sequence`` also
knows how to pickle itself for its worker RPC; here workers receive a flat
integer step descriptor instead (see ``step_batch.py``), so a request never
leaves rank 0 and carries no block-size constant of its own: the block size
is a property of the KV pool.
"""
from __future__ import annotations

from enum import Enum, auto
from itertools import count

from ..sampling_params import SamplingParams


class RequestStatus(Enum):
    WAITING = auto()
    RUNNING = auto()
    FINISHED = auto()


class Request:
    __slots__ = ("req_id", "status", "token_ids", "num_prompt_tokens", "num_cached_tokens", "num_computed_tokens", "prefill_end",
                 "block_table", "temperature", "max_tokens", "ignore_eos", "num_preemptions")

    _ids = count()

    def __init__(self, prompt_token_ids: list[int], sampling_params: SamplingParams = SamplingParams()):
        if len(prompt_token_ids) == 0:
            raise ValueError("a request needs at least one prompt token")
        self.req_id = next(Request._ids)
        self.status = RequestStatus.WAITING
        self.token_ids = list(prompt_token_ids)
        self.num_prompt_tokens = len(self.token_ids)
        self.num_cached_tokens = 0
        # chunked prefill (a prompt longer than the token budget is prefilled over several steps): tokens whose KV entries
        # exist already, and the end of the range the current prefill step covers.  -1: not in use (the step starts at
        # num_cached_tokens and covers the whole request).
        self.num_computed_tokens = -1
        self.prefill_end = -1
        self.block_table: list[int] = []
        self.temperature = float(sampling_params.temperature)
        self.max_tokens = int(sampling_params.max_tokens)
        self.ignore_eos = bool(sampling_params.ignore_eos)
        self.num_preemptions = 0

    def __len__(self) -> int:
        return len(self.token_ids)

    @property
    def num_tokens(self) -> int:
        return len(self.token_ids)

    @property
    def last_token(self) -> int:
        return self.token_ids[-1]

    @property
    def is_finished(self) -> bool:
        return self.status is RequestStatus.FINISHED

    @property
    def num_completion_tokens(self) -> int:
        return len(self.token_ids) - self.num_prompt_tokens

    @property
    def prompt_token_ids(self) -> list[int]:
        return self.token_ids[:self.num_prompt_tokens]

    @property
    def completion_token_ids(self) -> list[int]:
        return self.token_ids[self.num_prompt_tokens:]

    def append_token(self, token_id: int) -> None:
        self.token_ids.append(token_id)

    def __repr__(self) -> str:
        return (f"Request(id={self.req_id}, {self.status.name}, tokens={len(self.token_ids)}, "
                f"prompt={self.num_prompt_tokens}, cached={self.num_cached_tokens}, blocks={len(self.block_table)})")
