"""Validated Qwen3-VL architecture description.

The engine never reads a Hugging Face config object directly: it converts the
``config.json`` dictionary (or an ``AutoConfig`` instance) into the frozen
dataclasses below once and every later layer (weight sharding, kernels, KV sizing)
reads these.  Mirrors the contract of the reference's
``prism_infer/models/qwen3_vl_architecture.py:117-428`` (canonical 8B constants at
``:18-44``): interleaved M-RoPE only, no attention bias, SiLU text MLP, GELU-tanh
vision MLP.
"""

from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field
from typing import Any, Mapping

SUPPORTED_MODEL_TYPES = frozenset({"qwen3_vl"})


def _get(cfg: Any, *names: str, default: Any = ...) -> Any:
    for name in names:
        if isinstance(cfg, Mapping):
            if name in cfg:
                return cfg[name]
        elif hasattr(cfg, name):
            return getattr(cfg, name)
    if default is not ...:
        return default
    raise ValueError(f"Qwen3-VL config is missing required field {' or '.join(names)}")


@dataclass(frozen=True)
class TextArch:
    vocab_size: int = 151_936
    hidden_size: int = 4_096
    num_layers: int = 36
    num_heads: int = 32
    num_kv_heads: int = 8
    head_dim: int = 128
    intermediate_size: int = 12_288
    rope_theta: float = 5_000_000.0
    rms_norm_eps: float = 1.0e-6
    mrope_section: tuple[int, int, int] = (24, 20, 20)
    max_position_embeddings: int = 262_144
    tie_word_embeddings: bool = False

    def __post_init__(self) -> None:
        if self.num_heads % self.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if self.head_dim % 2:
            raise ValueError("head_dim must be even")
        if sum(self.mrope_section) != self.head_dim // 2:
            raise ValueError(
                f"mrope_section {self.mrope_section} must sum to head_dim/2 = {self.head_dim // 2}"
            )
        if len(self.mrope_section) != 3:
            raise ValueError("mrope_section needs three entries (T, H, W)")

    @property
    def q_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim


@dataclass(frozen=True)
class VisionArch:
    hidden_size: int = 1_152
    depth: int = 27
    num_heads: int = 16
    intermediate_size: int = 4_304
    in_channels: int = 3
    patch_size: int = 16
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    num_position_embeddings: int = 2_304
    out_hidden_size: int = 4_096
    deepstack_visual_indexes: tuple[int, ...] = (8, 16, 24)
    rope_theta: float = 10_000.0
    layer_norm_eps: float = 1.0e-6

    def __post_init__(self) -> None:
        if self.hidden_size % self.num_heads:
            raise ValueError("vision hidden_size must be a multiple of num_heads")
        side = int(round(self.num_position_embeddings**0.5))
        if side * side != self.num_position_embeddings:
            raise ValueError("num_position_embeddings must be a perfect square")
        if (self.head_dim // 2) % 2:
            raise ValueError("vision head_dim/2 must be even for 2-D rotary embedding")
        for idx in self.deepstack_visual_indexes:
            if not 0 <= idx < self.depth:
                raise ValueError(f"deepstack index {idx} outside vision depth {self.depth}")

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads

    @property
    def patch_input_dim(self) -> int:
        return self.in_channels * self.temporal_patch_size * self.patch_size * self.patch_size

    @property
    def merge_unit(self) -> int:
        return self.spatial_merge_size * self.spatial_merge_size

    @property
    def merged_dim(self) -> int:
        return self.hidden_size * self.merge_unit

    @property
    def grid_per_side(self) -> int:
        return int(round(self.num_position_embeddings**0.5))


@dataclass(frozen=True)
class Qwen3VLArch:
    text: TextArch = field(default_factory=TextArch)
    vision: VisionArch = field(default_factory=VisionArch)
    image_token_id: int = 151_655
    video_token_id: int = 151_656
    vision_start_token_id: int = 151_652
    vision_end_token_id: int = 151_653
    eos_token_id: int = 151_645
    model_type: str = "qwen3_vl"

    def __post_init__(self) -> None:
        if self.model_type not in SUPPORTED_MODEL_TYPES:
            raise ValueError(f"unsupported model_type {self.model_type!r}")
        if self.vision.out_hidden_size != self.text.hidden_size:
            raise ValueError("vision out_hidden_size must equal text hidden_size")
        ids = (self.image_token_id, self.video_token_id, self.vision_start_token_id)
        if len(set(ids)) != 3:
            raise ValueError(f"visual special token ids must be distinct: {ids}")

    # ---- factories -----------------------------------------------------------
    @classmethod
    def qwen3_vl_8b(cls) -> "Qwen3VLArch":
        return cls()

    def rank_shard(self, n: int) -> "Qwen3VLArch":
        """Architecture whose language model equals one rank's share of an ``n``-way
        tensor-parallel split (for single-GPU profiling of the per-rank kernel chain)."""
        import dataclasses

        validate_tensor_parallel(self, n)
        t = self.text
        text = dataclasses.replace(t, num_heads=t.num_heads // n, num_kv_heads=t.num_kv_heads // n,
                                   intermediate_size=t.intermediate_size // n, vocab_size=t.vocab_size // n)
        return dataclasses.replace(self, text=text)

    @classmethod
    def qwen3_vl_8b_2layer(cls) -> "Qwen3VLArch":
        """Qwen3-VL-8B widths (hidden 4096, 32 / 8 heads of 128, MLP 12288, vocabulary 151936, vision
        hidden 1152) with two decoder and two vision layers: every kernel runs at its production
        shape, and an end-to-end comparison against the oracle stays cheap."""
        import dataclasses

        full = cls()
        return dataclasses.replace(
            full, text=dataclasses.replace(full.text, num_layers=2),
            vision=dataclasses.replace(full.vision, depth=2, deepstack_visual_indexes=(0, 1)))

    @classmethod
    def tiny(cls) -> "Qwen3VLArch":
        """The small CPU test model: 2+2 layers, hidden 256/128, head_dim 64."""
        return cls(
            text=TextArch(
                vocab_size=1024,
                hidden_size=256,
                num_layers=2,
                num_heads=4,
                num_kv_heads=2,
                head_dim=64,
                intermediate_size=512,
                mrope_section=(8, 12, 12),
                max_position_embeddings=4096,
            ),
            vision=VisionArch(
                hidden_size=128,
                depth=2,
                num_heads=4,
                intermediate_size=256,
                num_position_embeddings=256,
                out_hidden_size=256,
                deepstack_visual_indexes=(1,),
            ),
            image_token_id=1001,
            video_token_id=1002,
            vision_start_token_id=1003,
            vision_end_token_id=1004,
            eos_token_id=1005,
        )

    @classmethod
    def from_hf_config(cls, cfg: Any) -> "Qwen3VLArch":
        model_type = _get(cfg, "model_type")
        if model_type not in SUPPORTED_MODEL_TYPES:
            raise ValueError(f"unsupported model_type {model_type!r}")
        tcfg = _get(cfg, "text_config")
        vcfg = _get(cfg, "vision_config")
        rope = _get(tcfg, "rope_scaling", "rope_parameters", default=None) or {}
        section = tuple(_get(rope, "mrope_section", default=(24, 20, 20)))
        if _get(rope, "mrope_interleaved", default=True) is False:
            raise ValueError("only interleaved M-RoPE is supported")
        if _get(tcfg, "attention_bias", default=False):
            raise ValueError("attention bias is not supported")
        if _get(tcfg, "hidden_act", default="silu") != "silu":
            raise ValueError("text MLP activation must be silu")
        vact = _get(vcfg, "hidden_act", default="gelu_pytorch_tanh")
        if vact not in ("gelu_pytorch_tanh", "gelu_tanh"):
            raise ValueError("vision MLP activation must be gelu (tanh)")
        theta = _get(tcfg, "rope_theta", default=None)
        if theta is None:
            theta = _get(rope, "rope_theta", default=5_000_000.0)
        hidden = int(_get(tcfg, "hidden_size"))
        heads = int(_get(tcfg, "num_attention_heads"))
        text = TextArch(
            vocab_size=int(_get(tcfg, "vocab_size")),
            hidden_size=hidden,
            num_layers=int(_get(tcfg, "num_hidden_layers")),
            num_heads=heads,
            num_kv_heads=int(_get(tcfg, "num_key_value_heads")),
            head_dim=int(_get(tcfg, "head_dim", default=hidden // heads)),
            intermediate_size=int(_get(tcfg, "intermediate_size")),
            rope_theta=float(theta),
            rms_norm_eps=float(_get(tcfg, "rms_norm_eps", default=1e-6)),
            mrope_section=section,  # type: ignore[arg-type]
            max_position_embeddings=int(_get(tcfg, "max_position_embeddings", default=262_144)),
            tie_word_embeddings=bool(
                _get(cfg, "tie_word_embeddings", default=_get(tcfg, "tie_word_embeddings", default=False))
            ),
        )
        vision = VisionArch(
            hidden_size=int(_get(vcfg, "hidden_size")),
            depth=int(_get(vcfg, "depth")),
            num_heads=int(_get(vcfg, "num_heads")),
            intermediate_size=int(_get(vcfg, "intermediate_size")),
            in_channels=int(_get(vcfg, "in_channels", default=3)),
            patch_size=int(_get(vcfg, "patch_size")),
            temporal_patch_size=int(_get(vcfg, "temporal_patch_size", default=2)),
            spatial_merge_size=int(_get(vcfg, "spatial_merge_size", default=2)),
            num_position_embeddings=int(_get(vcfg, "num_position_embeddings")),
            out_hidden_size=int(_get(vcfg, "out_hidden_size")),
            deepstack_visual_indexes=tuple(_get(vcfg, "deepstack_visual_indexes", default=(8, 16, 24))),
        )
        eos = _get(cfg, "eos_token_id", default=_get(tcfg, "eos_token_id", default=151_645))
        if isinstance(eos, (list, tuple)):
            eos = eos[0]
        return cls(
            text=text,
            vision=vision,
            image_token_id=int(_get(cfg, "image_token_id")),
            video_token_id=int(_get(cfg, "video_token_id")),
            vision_start_token_id=int(_get(cfg, "vision_start_token_id")),
            vision_end_token_id=int(_get(cfg, "vision_end_token_id", default=151_653)),
            eos_token_id=int(eos if eos is not None else 151_645),
            model_type=model_type,
        )

    @classmethod
    def from_pretrained(cls, path: str) -> "Qwen3VLArch":
        with open(os.path.join(path, "config.json"), "r", encoding="utf-8") as fh:
            return cls.from_hf_config(json.load(fh))

    def to_hf_config(self) -> dict[str, Any]:
        """A ``config.json`` dictionary Hugging Face ``AutoConfig`` accepts."""
        t, v = self.text, self.vision
        return {
            "architectures": ["Qwen3VLForConditionalGeneration"],
            "model_type": self.model_type,
            "image_token_id": self.image_token_id,
            "video_token_id": self.video_token_id,
            "vision_start_token_id": self.vision_start_token_id,
            "vision_end_token_id": self.vision_end_token_id,
            "tie_word_embeddings": t.tie_word_embeddings,
            "eos_token_id": self.eos_token_id,
            "text_config": {
                "model_type": "qwen3_vl_text",
                "vocab_size": t.vocab_size,
                "hidden_size": t.hidden_size,
                "num_hidden_layers": t.num_layers,
                "num_attention_heads": t.num_heads,
                "num_key_value_heads": t.num_kv_heads,
                "head_dim": t.head_dim,
                "intermediate_size": t.intermediate_size,
                "rope_theta": t.rope_theta,
                "rms_norm_eps": t.rms_norm_eps,
                "hidden_act": "silu",
                "attention_bias": False,
                "max_position_embeddings": t.max_position_embeddings,
                "rope_scaling": {
                    "mrope_interleaved": True,
                    "mrope_section": list(t.mrope_section),
                    "rope_type": "default",
                },
                "dtype": "bfloat16",
            },
            "vision_config": {
                "model_type": "qwen3_vl",
                "hidden_size": v.hidden_size,
                "depth": v.depth,
                "num_heads": v.num_heads,
                "intermediate_size": v.intermediate_size,
                "in_channels": v.in_channels,
                "patch_size": v.patch_size,
                "temporal_patch_size": v.temporal_patch_size,
                "spatial_merge_size": v.spatial_merge_size,
                "num_position_embeddings": v.num_position_embeddings,
                "out_hidden_size": v.out_hidden_size,
                "deepstack_visual_indexes": list(v.deepstack_visual_indexes),
                "hidden_act": "gelu_pytorch_tanh",
            },
        }

    def describe(self) -> dict[str, Any]:
        return asdict(self)


def validate_tensor_parallel(arch: Qwen3VLArch, tp: int) -> None:
    """Every sharded dimension must divide evenly (reference ``engine/llm_engine.py:117-143``)."""
    if tp < 1:
        raise ValueError("tensor_parallel_size must be >= 1")
    t = arch.text
    for name, value in (
        ("num_heads", t.num_heads),
        ("num_kv_heads", t.num_kv_heads),
        ("hidden_size", t.hidden_size),
        ("intermediate_size", t.intermediate_size),
        ("vocab_size", t.vocab_size),
    ):
        if value % tp:
            raise ValueError(f"tensor_parallel_size {tp} does not divide text {name}={value}")
