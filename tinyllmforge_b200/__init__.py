"""B200-native offline LLM inference engine.

    from tinyllmforge_b200 import LLM, SamplingParams
    llm = LLM(model_dir, tensor_parallel_size=1)
    outs = llm.generate(prompts_or_token_ids, SamplingParams(temperature=0.6, max_tokens=256))

Public surface parity: tinyvllm/__init__.py:1-2.
"""
from .llm import LLM
from .sampling_params import SamplingParams
from .config import Config, ModelConfig, preset

__all__ = ["LLM", "SamplingParams", "Config", "ModelConfig", "preset"]
__version__ = "0.1.0"
