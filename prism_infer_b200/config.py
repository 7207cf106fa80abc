"""Engine configuration.

Seven frozen domain dataclasses plus a strict flat-keyword adapter so that
``LLM(model, **kwargs)`` accepts the same option names as the reference
(``prism_infer/config.py:569-701``): an unknown key raises ``TypeError``, invalid values
raise at construction, and cross-domain rules are checked once (``:511-567``).  Knobs
that configure ``torch.compile`` in the reference are accepted and validated but are
no-ops here: every decode op is a hand-written kernel and the CUDA-graph backend is the
default.  ``Config`` resolves the model directory (``config.json``) or a ``random:<name>``
spec into the architecture description and the derived KV geometry.
"""

from __future__ import annotations

import os
from dataclasses import dataclass, field, fields, replace
from math import isfinite
from typing import Any, Mapping

from .models.architecture import Qwen3VLArch, validate_tensor_parallel

COMPRESSION_MODES = (
    "off", "visual_prune", "visual_compact", "fp8_kv", "visual_compact_fp8", "scaled_fp8_kv",
    "visual_compact_scaled_fp8",
)
PAGE_SIZES = (16, 32, 64, 128, 256)
BACKENDS = ("eager", "compile", "cuda_graph", "compile_graph")
POLICIES = ("fcfs", "vision_aware", "slo_aware")
DEFAULT_TP_TIMEOUT = 120


def _int(v: Any, name: str, lo: int | None = None) -> int:
    if isinstance(v, bool) or not isinstance(v, int):
        raise TypeError(f"{name} must be an integer, got {v!r}")
    if lo is not None and v < lo:
        raise ValueError(f"{name} must be >= {lo}, got {v}")
    return v


def _bool(v: Any, name: str) -> bool:
    if not isinstance(v, bool):
        raise TypeError(f"{name} must be a bool, got {v!r}")
    return v


def _num(v: Any, name: str) -> float:
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not isfinite(float(v)):
        raise TypeError(f"{name} must be a finite number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class ModelConfig:
    model: str
    max_model_len: int = 4096
    tensor_parallel_size: int = 1
    tensor_parallel_timeout_seconds: int = DEFAULT_TP_TIMEOUT
    logits_precision: str = "model"
    mlp_projection_mode: str = "packed"
    seed: int = 0

    def __post_init__(self) -> None:
        if not isinstance(self.model, str) or not self.model:
            raise ValueError("model must be a checkpoint directory or 'random:<arch>'")
        if not self.model.startswith("random:") and not os.path.isdir(self.model):
            raise ValueError(f"model must be an existing local directory: {self.model!r}")
        _int(self.max_model_len, "max_model_len", 1)
        _int(self.tensor_parallel_size, "tensor_parallel_size", 1)
        _int(self.tensor_parallel_timeout_seconds, "tensor_parallel_timeout_seconds", 1)
        if self.logits_precision not in ("fp32", "model", "selective_fp32"):
            raise ValueError(f"unsupported logits_precision {self.logits_precision!r}")
        if self.mlp_projection_mode not in ("legacy", "packed"):
            raise ValueError(f"unsupported mlp_projection_mode {self.mlp_projection_mode!r}")


@dataclass(frozen=True)
class CacheConfig:
    gpu_memory_utilization: float = 0.9
    page_size: int = 256
    num_gpu_blocks: int = -1
    cpu_kv_cache_ratio: float = 0.5
    enable_prefix_caching: bool = True
    compression_mode: str = "off"
    enable_visual_pruning_shadow: bool = False
    visual_pruning_keep_ratio: float = 0.6
    visual_pruning_min_keep_tokens: int = 32
    visual_pruning_video_min_keep_tokens: int | None = None
    visual_pruning_strategy: str = "uniform"
    visual_pruning_attention_last_n_layers: int = 1

    def __post_init__(self) -> None:
        u = _num(self.gpu_memory_utilization, "gpu_memory_utilization")
        if not 0.0 < u <= 1.0:
            raise ValueError("gpu_memory_utilization must be in (0, 1]")
        if self.page_size not in PAGE_SIZES:
            raise ValueError(f"kvcache_block_size must be one of {PAGE_SIZES}, got {self.page_size!r}")
        if self.num_gpu_blocks != -1:
            _int(self.num_gpu_blocks, "num_kvcache_blocks", 1)
        if _num(self.cpu_kv_cache_ratio, "cpu_kv_cache_ratio") < 0:
            raise ValueError("cpu_kv_cache_ratio must be non-negative")
        _bool(self.enable_prefix_caching, "enable_prefix_caching")
        if not isinstance(self.compression_mode, str):
            raise TypeError(f"compression_mode must be a string, got {self.compression_mode!r}")
        if self.compression_mode not in COMPRESSION_MODES:
            raise ValueError(f"unsupported compression_mode {self.compression_mode!r}")
        r = _num(self.visual_pruning_keep_ratio, "visual_pruning_keep_ratio")
        if not 0.0 < r <= 1.0:
            raise ValueError("visual_pruning_keep_ratio must be in (0, 1]")
        _int(self.visual_pruning_min_keep_tokens, "visual_pruning_min_keep_tokens", 1)
        if self.visual_pruning_video_min_keep_tokens is not None:
            _int(self.visual_pruning_video_min_keep_tokens, "visual_pruning_video_min_keep_tokens", 1)
        if self.visual_pruning_strategy not in ("uniform", "attention", "score"):
            raise ValueError(f"unsupported visual_pruning_strategy {self.visual_pruning_strategy!r}")
        _int(self.visual_pruning_attention_last_n_layers, "visual_pruning_attention_last_n_layers", 1)


@dataclass(frozen=True)
class SchedulerConfig:
    max_num_batched_tokens: int = 16384
    max_num_seqs: int = 512
    enable_chunked_prefill: bool = True
    max_chunk_size: int = 512
    scheduler_policy: str = "fcfs"
    max_queue_size: int | None = None
    max_consecutive_prefill_batches: int = 1
    heavy_prefill_vision_patch_threshold: int = 4096
    min_decode_batches_between_heavy_prefills: int = 32
    max_light_prefill_bypasses_per_heavy: int = 2

    def __post_init__(self) -> None:
        _int(self.max_num_batched_tokens, "max_num_batched_tokens", 1)
        _int(self.max_num_seqs, "max_num_seqs", 1)
        _bool(self.enable_chunked_prefill, "enable_chunked_prefill")
        _int(self.max_chunk_size, "max_chunk_size", 1)
        if self.scheduler_policy not in POLICIES:
            raise ValueError(f"unsupported scheduler_policy {self.scheduler_policy!r}")
        if self.max_queue_size is not None:
            _int(self.max_queue_size, "max_queue_size", 0)
        _int(self.max_consecutive_prefill_batches, "max_consecutive_prefill_batches", 1)
        _int(self.heavy_prefill_vision_patch_threshold, "heavy_prefill_vision_patch_threshold", 1)
        _int(self.min_decode_batches_between_heavy_prefills, "min_decode_batches_between_heavy_prefills", 0)
        _int(self.max_light_prefill_bypasses_per_heavy, "max_light_prefill_bypasses_per_heavy", 0)


@dataclass(frozen=True)
class MultimodalConfig:
    image_min_pixels: int | None = None
    image_max_pixels: int | None = None
    video_max_pixels: int | None = None
    max_vision_patches_per_batch: int = 8192
    vision_encoder_microbatch_patches: int = 4096
    vision_attention_backend: str = "sdpa"
    enable_vision_tensor_cudagraph: bool = False
    enable_visual_embedding_cache: bool = False
    visual_embedding_cache_bytes: int = 256 << 20
    # string prompts of multimodal requests are wrapped in the checkpoint's chat turns: "auto" = when the
    # tokenizer ships a chat template (instruction-tuned checkpoints), "always", or "never"
    chat_template: str = "auto"
    # "always": preprocess media with the checkpoint's own Hugging Face processor (needs its processor
    # files and transformers) instead of the built-in one, which has the same output contract
    hf_processor: str = "never"

    def __post_init__(self) -> None:
        if self.chat_template not in ("auto", "always", "never"):
            raise ValueError(f"chat_template must be 'auto', 'always' or 'never', got {self.chat_template!r}")
        if self.hf_processor not in ("always", "never"):
            raise ValueError(f"hf_processor must be 'always' or 'never', got {self.hf_processor!r}")
        for n in ("image_min_pixels", "image_max_pixels", "video_max_pixels"):
            v = getattr(self, n)
            if v is not None:
                _int(v, n, 1)
        _int(self.max_vision_patches_per_batch, "max_vision_patches_per_batch", 1)
        _int(self.vision_encoder_microbatch_patches, "vision_encoder_microbatch_patches", 1)
        if self.max_vision_patches_per_batch < self.vision_encoder_microbatch_patches:
            raise ValueError("max_vision_patches_per_batch must be >= vision_encoder_microbatch_patches")
        if self.vision_attention_backend not in ("sdpa", "flash_attn"):
            raise ValueError(f"unsupported vision_attention_backend {self.vision_attention_backend!r}")
        _bool(self.enable_vision_tensor_cudagraph, "enable_vision_tensor_cudagraph")
        _bool(self.enable_visual_embedding_cache, "enable_visual_embedding_cache")


@dataclass(frozen=True)
class ExecutionConfig:
    backend: str = "cuda_graph"
    compile_region: str = "none"
    compile_mode: str = "default"
    compile_emulate_precision_casts: bool = True
    compile_force_same_precision: bool = False
    allow_unsafe_compile: bool = False
    paged_decode_block_n: int = 32
    fused_qk_rmsnorm: bool = True
    fused_qk_mrope: bool = True
    fused_add_rmsnorm: bool = True
    packed_kv_projection: bool = True
    cooperative_prefill: bool = False
    cooperative_prefill_layer_quantum: int = 4
    cooperative_prefill_vision_block_quantum: int = 4
    # adaptive cooperative prefill (0 = off): with sequences decoding, fewer than `coalesce_min_seqs` waiting requests are
    # held back for up to this many milliseconds (less when a deadline reserve ends earlier) so that one prefill serves
    # several; a prefill of at least that many requests runs in one piece; a smaller one runs in layer quanta only when it
    # carries a heavy visual input or the decode batch has reached a quarter of max_num_seqs
    cooperative_prefill_coalesce_ms: float = 0.0
    cooperative_prefill_coalesce_min_seqs: int = 3
    programmatic_dependent_launch: bool = True
    decode_run_ahead: bool = True             # launch the next greedy decode graph before the host has read this one's tokens
    device_status_check_interval: int = 256   # engine steps between reads of the kernels' status words (0 = never)

    def __post_init__(self) -> None:
        if self.backend not in BACKENDS:
            raise ValueError(f"unsupported execution_backend: {self.backend!r}")
        if self.compile_region not in ("none", "attention", "qkv", "layer", "model"):
            raise ValueError(f"unsupported decode_compile_region {self.compile_region!r}")
        if self.paged_decode_block_n not in (16, 32, 64, 128, 256):
            raise ValueError("paged_decode_block_n must be a power of two in [16, 256]")
        for n in ("fused_qk_rmsnorm", "fused_qk_mrope", "fused_add_rmsnorm", "packed_kv_projection",
                  "cooperative_prefill", "programmatic_dependent_launch", "decode_run_ahead"):
            _bool(getattr(self, n), n)
        _int(self.cooperative_prefill_layer_quantum, "cooperative_prefill_layer_quantum", 1)
        _int(self.cooperative_prefill_vision_block_quantum, "cooperative_prefill_vision_block_quantum", 1)
        _int(self.cooperative_prefill_coalesce_min_seqs, "cooperative_prefill_coalesce_min_seqs", 2)
        if isinstance(self.cooperative_prefill_coalesce_ms, bool) or not isinstance(self.cooperative_prefill_coalesce_ms, (int, float)) \
                or not 0 <= self.cooperative_prefill_coalesce_ms <= 10_000:
            raise ValueError("cooperative_prefill_coalesce_ms must be a number of milliseconds in [0, 10000]")
        _int(self.device_status_check_interval, "device_status_check_interval", 0)

    @property
    def uses_graphs(self) -> bool:
        return self.backend in ("cuda_graph", "compile_graph")


@dataclass(frozen=True)
class QuantizationConfig:
    """Derived from the compression mode; weight / activation quantisation is rejected."""

    kv_dtype: str = "bf16"        # bf16 | fp8_e4m3
    kv_scaled: bool = False
    weight_quantization: str | None = None
    activation_quantization: str | None = None

    def __post_init__(self) -> None:
        if self.weight_quantization is not None or self.activation_quantization is not None:
            raise ValueError("weight and activation quantisation are not supported")

    @classmethod
    def from_mode(cls, mode: str) -> "QuantizationConfig":
        if mode in ("fp8_kv", "visual_compact_fp8"):
            return cls("fp8_e4m3", False)
        if mode in ("scaled_fp8_kv", "visual_compact_scaled_fp8"):
            return cls("fp8_e4m3", True)
        return cls()


@dataclass(frozen=True)
class ServingConfig:
    ingress_capacity: int = 64


_FLAT = {
    "model": {
        "max_model_len": "max_model_len", "tensor_parallel_size": "tensor_parallel_size",
        "tensor_parallel_timeout_seconds": "tensor_parallel_timeout_seconds",
        "logits_precision": "logits_precision", "mlp_projection_mode": "mlp_projection_mode", "seed": "seed",
    },
    "multimodal": {
        "image_min_pixels": "image_min_pixels", "image_max_pixels": "image_max_pixels",
        "video_max_pixels": "video_max_pixels",
        "max_vision_patches_per_batch": "max_vision_patches_per_batch",
        "vision_encoder_microbatch_patches": "vision_encoder_microbatch_patches",
        "vision_attention_backend": "vision_attention_backend",
        "enable_vision_tensor_cudagraph": "enable_vision_tensor_cudagraph",
        "enable_visual_embedding_cache": "enable_visual_embedding_cache",
        "visual_embedding_cache_bytes": "visual_embedding_cache_bytes",
        "chat_template": "chat_template", "hf_processor": "hf_processor",
    },
    "cache": {
        "gpu_memory_utilization": "gpu_memory_utilization", "kvcache_block_size": "page_size",
        "num_kvcache_blocks": "num_gpu_blocks", "cpu_kv_cache_ratio": "cpu_kv_cache_ratio",
        "enable_prefix_caching": "enable_prefix_caching", "compression_mode": "compression_mode",
        "enable_visual_pruning_shadow": "enable_visual_pruning_shadow",
        "visual_pruning_keep_ratio": "visual_pruning_keep_ratio",
        "visual_pruning_min_keep_tokens": "visual_pruning_min_keep_tokens",
        "visual_pruning_video_min_keep_tokens": "visual_pruning_video_min_keep_tokens",
        "visual_pruning_strategy": "visual_pruning_strategy",
        "visual_pruning_attention_last_n_layers": "visual_pruning_attention_last_n_layers",
    },
    "scheduler": {
        "max_num_batched_tokens": "max_num_batched_tokens", "max_num_seqs": "max_num_seqs",
        "enable_chunked_prefill": "enable_chunked_prefill", "max_chunk_size": "max_chunk_size",
        "scheduler_policy": "scheduler_policy", "max_queue_size": "max_queue_size",
        "max_consecutive_prefill_batches": "max_consecutive_prefill_batches",
        "heavy_prefill_vision_patch_threshold": "heavy_prefill_vision_patch_threshold",
        "min_decode_batches_between_heavy_prefills": "min_decode_batches_between_heavy_prefills",
        "max_light_prefill_bypasses_per_heavy": "max_light_prefill_bypasses_per_heavy",
    },
    "execution": {
        "decode_compile_region": "compile_region", "decode_compile_mode": "compile_mode",
        "decode_compile_emulate_precision_casts": "compile_emulate_precision_casts",
        "decode_compile_force_same_precision": "compile_force_same_precision",
        "allow_unsafe_decode_compile": "allow_unsafe_compile",
        "paged_decode_block_n": "paged_decode_block_n",
        "enable_fused_qk_rmsnorm": "fused_qk_rmsnorm", "enable_fused_qk_mrope": "fused_qk_mrope",
        "enable_fused_add_rmsnorm": "fused_add_rmsnorm", "enable_packed_kv_projection": "packed_kv_projection",
        "enable_cooperative_prefill": "cooperative_prefill",
        "cooperative_prefill_layer_quantum": "cooperative_prefill_layer_quantum",
        "cooperative_prefill_vision_block_quantum": "cooperative_prefill_vision_block_quantum",
        "cooperative_prefill_coalesce_ms": "cooperative_prefill_coalesce_ms",
        "cooperative_prefill_coalesce_min_seqs": "cooperative_prefill_coalesce_min_seqs",
        "enable_programmatic_dependent_launch": "programmatic_dependent_launch",
        "enable_decode_run_ahead": "decode_run_ahead",
        "device_status_check_interval": "device_status_check_interval",
    },
}
_CONTROL = {"enforce_eager", "execution_backend"}
FLAT_OPTION_NAMES = frozenset(k for group in _FLAT.values() for k in group) | _CONTROL


@dataclass(frozen=True)
class PrismConfig:
    model: ModelConfig
    cache: CacheConfig = field(default_factory=CacheConfig)
    scheduler: SchedulerConfig = field(default_factory=SchedulerConfig)
    multimodal: MultimodalConfig = field(default_factory=MultimodalConfig)
    execution: ExecutionConfig = field(default_factory=ExecutionConfig)
    quantization: QuantizationConfig = field(default_factory=QuantizationConfig)
    serving: ServingConfig = field(default_factory=ServingConfig)

    def __post_init__(self) -> None:
        mode = self.cache.compression_mode
        object.__setattr__(self, "quantization", QuantizationConfig.from_mode(mode))
        if mode == "visual_prune" and self.execution.uses_graphs:
            raise ValueError("compression_mode 'visual_prune' is a logical (eager-only) mode")
        if self.cache.visual_pruning_strategy == "attention" and self.execution.uses_graphs and mode == "visual_prune":
            raise ValueError("attention pruning needs the eager backend")
        tp = self.model.tensor_parallel_size
        if tp > 1 and self.model.logits_precision != "model":
            raise ValueError("tensor parallel execution requires logits_precision='model'")
        if self.execution.cooperative_prefill and tp != 1:
            raise ValueError("enable_cooperative_prefill currently supports TP1 only")
        if self.scheduler.max_chunk_size > self.scheduler.max_num_batched_tokens:
            raise ValueError("max_chunk_size must not exceed max_num_batched_tokens")

    @classmethod
    def from_flat_options(cls, model: str, options: Mapping[str, object]) -> "PrismConfig":
        unknown = sorted(set(options) - FLAT_OPTION_NAMES)
        if unknown:
            raise TypeError("unknown Prism config option(s): " + ", ".join(repr(n) for n in unknown))

        def pick(group: str) -> dict[str, object]:
            return {dst: options[src] for src, dst in _FLAT[group].items() if src in options}

        region = options.get("decode_compile_region", "none")
        if not isinstance(region, str):
            raise TypeError(f"decode_compile_region must be a string, got {region!r}")
        eager = _bool(options.get("enforce_eager", False), "enforce_eager")
        explicit = options.get("execution_backend")
        if explicit is None:
            if region != "none" and not eager:
                raise ValueError("decode torch.compile region and CUDA Graph are mutually exclusive")
            backend = "compile" if region != "none" else ("eager" if eager else "cuda_graph")
        else:
            if explicit not in BACKENDS:
                raise ValueError(f"unsupported execution_backend: {explicit!r}")
            backend = str(explicit)
            if "enforce_eager" in options and eager != (backend not in ("cuda_graph", "compile_graph")):
                raise ValueError(
                    f"enforce_eager conflicts with execution_backend: enforce_eager={eager}, backend={backend!r}"
                )
        exe = pick("execution")
        exe["backend"] = backend
        return cls(
            model=ModelConfig(model=model, **pick("model")),
            cache=CacheConfig(**pick("cache")),
            scheduler=SchedulerConfig(**pick("scheduler")),
            multimodal=MultimodalConfig(**pick("multimodal")),
            execution=ExecutionConfig(**exe),
        )


_RANDOM_ARCHS = {
    "tiny": Qwen3VLArch.tiny,
    "qwen3-vl-8b": Qwen3VLArch.qwen3_vl_8b,
    "qwen3_vl_8b": Qwen3VLArch.qwen3_vl_8b,
    "qwen3-vl-8b-2layer": Qwen3VLArch.qwen3_vl_8b_2layer,
    # profiling aids: the language-model compute of ONE rank of an n-way tensor-parallel group
    # (heads, KV heads, MLP width and vocabulary divided by n), run without any exchange
    "qwen3-vl-8b-tp2-shard": lambda: Qwen3VLArch.qwen3_vl_8b().rank_shard(2),
    "qwen3-vl-8b-tp4-shard": lambda: Qwen3VLArch.qwen3_vl_8b().rank_shard(4),
    "qwen3-vl-8b-tp8-shard": lambda: Qwen3VLArch.qwen3_vl_8b().rank_shard(8),
}


def resolve_arch(model: str) -> Qwen3VLArch:
    if model.startswith("random:"):
        name = model.split(":", 1)[1]
        if name not in _RANDOM_ARCHS:
            raise ValueError(f"unknown random architecture {name!r}; known: {sorted(_RANDOM_ARCHS)}")
        return _RANDOM_ARCHS[name]()
    return Qwen3VLArch.from_pretrained(model)


class Config:
    """Resolved runtime configuration: domains + architecture + derived capacities."""

    def __init__(self, model: "str | PrismConfig", arch: Qwen3VLArch | None = None, **flat_options: object) -> None:
        if isinstance(model, PrismConfig):
            if flat_options:
                raise TypeError("flat options cannot be combined with a PrismConfig")
            self.prism = model
            self._flat_options = {}
        else:
            self.prism = PrismConfig.from_flat_options(model, flat_options)
            self._flat_options = dict(flat_options)  # replayed verbatim by spawned worker ranks
        self.arch = arch if arch is not None else resolve_arch(self.prism.model.model)
        validate_tensor_parallel(self.arch, self.prism.model.tensor_parallel_size)
        self.max_model_len = min(self.prism.model.max_model_len, self.arch.text.max_position_embeddings)
        if self.prism.scheduler.max_num_batched_tokens < self.max_model_len and not self.prism.scheduler.enable_chunked_prefill:
            raise ValueError("max_num_batched_tokens must be >= max_model_len when chunked prefill is off")
        self.eos = self.arch.eos_token_id
        self.num_kvcache_blocks = self.prism.cache.num_gpu_blocks
        self.num_cpu_blocks = 0

    # flat read access used across the engine ------------------------------------
    _flat_domain: dict[str, str] = {}  # field name -> domain, resolved once (the step loop reads flat names)

    def __getattr__(self, name: str) -> Any:
        prism = self.__dict__.get("prism")
        if prism is not None:
            dom = Config._flat_domain.get(name)
            if dom is None:
                for cand in ("model", "cache", "scheduler", "multimodal", "execution", "quantization", "serving"):
                    if name in {f.name for f in fields(getattr(prism, cand))}:
                        dom = Config._flat_domain[name] = cand
                        break
            if dom is not None:
                return getattr(getattr(prism, dom), name)
        raise AttributeError(name)

    @property
    def tp(self) -> int:
        return self.prism.model.tensor_parallel_size

    @property
    def kvcache_block_size(self) -> int:
        return self.prism.cache.page_size

    @property
    def kv_mode(self) -> int:
        q = self.prism.quantization
        return 0 if q.kv_dtype == "bf16" else (2 if q.kv_scaled else 1)

    @property
    def compacts_visual_tokens(self) -> bool:
        return self.prism.cache.compression_mode in ("visual_compact", "visual_compact_fp8", "visual_compact_scaled_fp8")

    def kv_bytes_per_page(self) -> int:
        """Bytes of one page across all layers, K and V, on one rank (payload + scales)."""
        t = self.arch.text
        rows = 2 * t.num_layers * (t.num_kv_heads // self.tp) * self.kvcache_block_size
        elem = 2 if self.kv_mode == 0 else 1
        return rows * t.head_dim * elem + (rows * 4 if self.kv_mode == 2 else 0)

    def with_cache_capacity(self, gpu_blocks: int, cpu_blocks: int) -> "Config":
        self.num_kvcache_blocks = int(gpu_blocks)
        self.num_cpu_blocks = int(cpu_blocks)
        return self

    def replace_domain(self, **domains: Any) -> "Config":
        return Config(replace(self.prism, **domains), arch=self.arch)
