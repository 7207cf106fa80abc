"""B200-native Qwen3-VL inference engine: ``from prism_infer_b200 import LLM, SamplingParams``.

``LLM`` is loaded lazily so importing the package (for its config, ops or analysis
modules) does not pull in the engine.
"""

from .sampling_params import SamplingParams

__version__ = "0.1.0"
__all__ = ["LLM", "SamplingParams", "__version__"]


def __getattr__(name):
    if name == "LLM":
        from .llm import LLM

        return LLM
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
