"""Engine counters (the reference records nothing beyond a tqdm postfix, tinyvllm/engine/llm_engine.py:82-96)."""
from __future__ import annotations

import json
from collections import Counter
from dataclasses import dataclass, field


@dataclass
class EngineStats:
    prefill_steps: int = 0
    decode_steps: int = 0
    prefill_tokens: int = 0            # tokens actually computed in prefill steps
    prefix_cached_tokens: int = 0      # prompt tokens skipped thanks to the prefix cache
    decode_tokens: int = 0
    preemptions: int = 0
    finished_requests: int = 0
    schedule_s: float = 0.0
    build_s: float = 0.0
    run_s: float = 0.0
    postprocess_s: float = 0.0
    # device time of the steps (CUDA events around each step on this rank; filled when extra={"device_timing": True})
    prefill_device_ms: float = 0.0
    decode_device_ms: float = 0.0
    decode_batch_hist: Counter = field(default_factory=Counter)

    def add_device_time(self, is_prefill: bool, ms: float | None) -> None:
        if ms is not None:
            if is_prefill:
                self.prefill_device_ms += ms
            else:
                self.decode_device_ms += ms

    def to_dict(self) -> dict:
        d = {k: v for k, v in self.__dict__.items() if k != "decode_batch_hist"}
        d["decode_step_device_ms"] = self.decode_device_ms / self.decode_steps if self.decode_steps and self.decode_device_ms else None
        d["prefill_step_device_ms"] = self.prefill_device_ms / self.prefill_steps if self.prefill_steps and self.prefill_device_ms else None
        d["decode_batch_hist"] = {int(k): int(v) for k, v in sorted(self.decode_batch_hist.items())}
        return d

    def to_json(self) -> str:
        return json.dumps(self.to_dict())
