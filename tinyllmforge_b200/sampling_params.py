"""Per-request sampling options.

Parity: tinyvllm/sampling_params.py:3-11 (temperature, max_tokens, ignore_eos).
`temperature == 0` selects greedy decoding, as the reference's sampler does
(tinyvllm/layers/sampler.py:21).
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 1.0
    max_tokens: int = 64
    ignore_eos: bool = False

    def __post_init__(self):
        if self.temperature < 0.0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if self.max_tokens < 1:
            raise ValueError(f"max_tokens must be >= 1, got {self.max_tokens}")
