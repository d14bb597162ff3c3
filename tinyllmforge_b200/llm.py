"""``LLM``: the user-facing name of the engine (tinyvllm/llm.py:4-5)."""
from .engine.engine import LLMEngine


class LLM(LLMEngine):
    pass
