"""KV compression modes and what each implies for the runtime.

Seven modes as in the reference (``prism_infer/engine/compression.py:25-50``): ``off``,
``visual_prune`` (logical holes in the block table, eager only), ``visual_compact``
(physical compaction, bf16), ``fp8_kv`` / ``visual_compact_fp8`` (unit-scale E4M3),
``scaled_fp8_kv`` / ``visual_compact_scaled_fp8`` (E4M3 with one fp32 scale per token and
KV head).  E4M3FN max is 448, the scale floor 1e-6, K and V are scaled separately
(``prism_infer/engine/kv_quantization.py:9-13``).
"""

from __future__ import annotations

from dataclasses import dataclass

FP8_E4M3_MAX = 448.0
FP8_SCALE_FLOOR = 1.0e-6


@dataclass(frozen=True)
class CompressionTraits:
    mode: str
    kv_mode: int            # 0 bf16, 1 fp8, 2 scaled fp8
    compacts: bool          # physically removes dropped visual rows
    logical_prune: bool     # leaves holes instead
    graph_safe: bool


_TABLE = {
    "off": CompressionTraits("off", 0, False, False, True),
    "visual_prune": CompressionTraits("visual_prune", 0, False, True, False),
    "visual_compact": CompressionTraits("visual_compact", 0, True, False, True),
    "fp8_kv": CompressionTraits("fp8_kv", 1, False, False, True),
    "visual_compact_fp8": CompressionTraits("visual_compact_fp8", 1, True, False, True),
    "scaled_fp8_kv": CompressionTraits("scaled_fp8_kv", 2, False, False, True),
    "visual_compact_scaled_fp8": CompressionTraits("visual_compact_scaled_fp8", 2, True, False, True),
}


def traits(mode: str) -> CompressionTraits:
    try:
        return _TABLE[mode]
    except KeyError:
        raise ValueError(f"unsupported compression_mode {mode!r}") from None


def kv_bytes_per_token(num_layers: int, kv_heads: int, head_dim: int, kv_mode: int) -> int:
    """K and V, all layers, one token (payload + scales)."""
    rows = 2 * num_layers * kv_heads
    return rows * head_dim * (2 if kv_mode == 0 else 1) + (rows * 4 if kv_mode == 2 else 0)


@dataclass(frozen=True)
class CompressionMetadata:
    """Per-step record attached to batch metrics."""

    mode: str
    compacted_sequences: int = 0
    rows_moved: int = 0
    pages_released: int = 0
    visual_tokens_dropped: int = 0
