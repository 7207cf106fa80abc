"""User-facing ``LLM`` class (reference ``prism_infer/llm.py:6-9``)."""

from .engine.llm_engine import LLMEngine


class LLM(LLMEngine):
    """Stable public entry point of the inference engine."""
