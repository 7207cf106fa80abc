"""Request-level generation parameters (reference ``prism_infer/sampling_params.py:6-18``)."""

from dataclasses import dataclass


@dataclass
class SamplingParams:
    """``temperature == 0`` selects greedy decoding; ``ignore_eos`` decodes to ``max_tokens``."""

    temperature: float = 1.0
    max_tokens: int = 64
    ignore_eos: bool = False

    def __post_init__(self) -> None:
        if self.temperature < 0:
            raise ValueError("temperature must be non-negative")
        if self.max_tokens <= 0:
            raise ValueError("max_tokens must be positive")
