"""Checkpoint tensors under their Hugging Face names: shapes, random init, safetensors IO.

The engine keeps HF names as the single naming scheme (reference
``prism_infer/utils/loader.py:17-36`` and ``prism_infer/models/qwen3_vl.py:1205-1222``):
``model.language_model.layers.N.self_attn.q_proj.weight``,
``model.visual.blocks.N.attn.qkv.weight``, ``model.visual.merger.linear_fc1.weight``,
``model.visual.deepstack_merger_list.K.*``, ``lm_head.weight``.
"""

from __future__ import annotations

import glob
import json
import os
from typing import Callable, Iterator

import torch

from .architecture import Qwen3VLArch

LM = "model.language_model"
VIS = "model.visual"


def weight_shapes(arch: Qwen3VLArch) -> dict[str, tuple[int, ...]]:
    """Name -> shape of every checkpoint tensor, in load order."""
    t, v = arch.text, arch.vision
    s: dict[str, tuple[int, ...]] = {}
    s[f"{VIS}.patch_embed.proj.weight"] = (
        v.hidden_size, v.in_channels, v.temporal_patch_size, v.patch_size, v.patch_size)
    s[f"{VIS}.patch_embed.proj.bias"] = (v.hidden_size,)
    s[f"{VIS}.pos_embed.weight"] = (v.num_position_embeddings, v.hidden_size)
    for i in range(v.depth):
        b = f"{VIS}.blocks.{i}"
        for n in ("norm1", "norm2"):
            s[f"{b}.{n}.weight"] = (v.hidden_size,)
            s[f"{b}.{n}.bias"] = (v.hidden_size,)
        s[f"{b}.attn.qkv.weight"] = (3 * v.hidden_size, v.hidden_size)
        s[f"{b}.attn.qkv.bias"] = (3 * v.hidden_size,)
        s[f"{b}.attn.proj.weight"] = (v.hidden_size, v.hidden_size)
        s[f"{b}.attn.proj.bias"] = (v.hidden_size,)
        s[f"{b}.mlp.linear_fc1.weight"] = (v.intermediate_size, v.hidden_size)
        s[f"{b}.mlp.linear_fc1.bias"] = (v.intermediate_size,)
        s[f"{b}.mlp.linear_fc2.weight"] = (v.hidden_size, v.intermediate_size)
        s[f"{b}.mlp.linear_fc2.bias"] = (v.hidden_size,)

    def merger(prefix: str, norm_dim: int) -> None:
        s[f"{prefix}.norm.weight"] = (norm_dim,)
        s[f"{prefix}.norm.bias"] = (norm_dim,)
        s[f"{prefix}.linear_fc1.weight"] = (v.merged_dim, v.merged_dim)
        s[f"{prefix}.linear_fc1.bias"] = (v.merged_dim,)
        s[f"{prefix}.linear_fc2.weight"] = (v.out_hidden_size, v.merged_dim)
        s[f"{prefix}.linear_fc2.bias"] = (v.out_hidden_size,)

    merger(f"{VIS}.merger", v.hidden_size)
    for k in range(len(v.deepstack_visual_indexes)):
        merger(f"{VIS}.deepstack_merger_list.{k}", v.merged_dim)

    s[f"{LM}.embed_tokens.weight"] = (t.vocab_size, t.hidden_size)
    for i in range(t.num_layers):
        p = f"{LM}.layers.{i}"
        s[f"{p}.input_layernorm.weight"] = (t.hidden_size,)
        s[f"{p}.self_attn.q_proj.weight"] = (t.q_size, t.hidden_size)
        s[f"{p}.self_attn.k_proj.weight"] = (t.kv_size, t.hidden_size)
        s[f"{p}.self_attn.v_proj.weight"] = (t.kv_size, t.hidden_size)
        s[f"{p}.self_attn.o_proj.weight"] = (t.hidden_size, t.q_size)
        s[f"{p}.self_attn.q_norm.weight"] = (t.head_dim,)
        s[f"{p}.self_attn.k_norm.weight"] = (t.head_dim,)
        s[f"{p}.post_attention_layernorm.weight"] = (t.hidden_size,)
        s[f"{p}.mlp.gate_proj.weight"] = (t.intermediate_size, t.hidden_size)
        s[f"{p}.mlp.up_proj.weight"] = (t.intermediate_size, t.hidden_size)
        s[f"{p}.mlp.down_proj.weight"] = (t.hidden_size, t.intermediate_size)
    s[f"{LM}.norm.weight"] = (t.hidden_size,)
    if not t.tie_word_embeddings:
        s["lm_head.weight"] = (t.vocab_size, t.hidden_size)
    return s


def _is_norm_weight(name: str) -> bool:
    return name.endswith("norm.weight") or "layernorm.weight" in name or ".norm1.weight" in name \
        or ".norm2.weight" in name


def iter_random_weights(
    arch: Qwen3VLArch,
    *,
    dtype: torch.dtype = torch.bfloat16,
    device: str | torch.device = "cpu",
    seed: int = 0,
) -> Iterator[tuple[str, torch.Tensor]]:
    """Deterministic random checkpoint, one tensor at a time (never the whole model).

    Each tensor has its own generator seeded from ``(seed, index)`` so any subset can be
    regenerated, on CPU or GPU; values are produced in fp32 on CPU-sized chunks only for
    small tensors, large ones are drawn on ``device`` directly.
    """
    device = torch.device(device)
    for index, (name, shape) in enumerate(weight_shapes(arch).items()):
        gen = torch.Generator(device=device)
        gen.manual_seed(seed * 1_000_003 + index)
        if _is_norm_weight(name):
            w = 1.0 + 0.05 * torch.randn(shape, generator=gen, device=device, dtype=torch.float32)
        elif name.endswith(".bias"):
            w = 0.02 * torch.randn(shape, generator=gen, device=device, dtype=torch.float32)
        elif name.endswith("embed_tokens.weight") or name.endswith("pos_embed.weight"):
            w = 0.05 * torch.randn(shape, generator=gen, device=device, dtype=torch.float32)
        else:
            fan_in = 1
            for d in shape[1:]:
                fan_in *= d
            w = torch.randn(shape, generator=gen, device=device, dtype=dtype if device.type == "cuda" else torch.float32)
            w = w * (fan_in ** -0.5)
        yield name, w.to(dtype)


def random_weights(arch: Qwen3VLArch, *, dtype=torch.float32, device="cpu", seed: int = 0) -> dict[str, torch.Tensor]:
    return dict(iter_random_weights(arch, dtype=dtype, device=device, seed=seed))


def iter_safetensors(path: str) -> Iterator[tuple[str, torch.Tensor]]:
    """Yield ``(hf_name, cpu_tensor)`` for every tensor in ``path/*.safetensors``."""
    from safetensors import safe_open

    files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"no *.safetensors files under {path}")
    for file in files:
        with safe_open(file, "pt", "cpu") as fh:
            for name in fh.keys():
                yield name, fh.get_tensor(name)


def save_checkpoint(
    path: str,
    arch: Qwen3VLArch,
    tensors: Iterator[tuple[str, torch.Tensor]] | dict[str, torch.Tensor],
    *,
    shard_bytes: int = 4 << 30,
) -> None:
    """Write an HF-style directory: ``config.json`` plus sharded ``*.safetensors``."""
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(arch.to_hf_config(), fh, indent=1)
    items = tensors.items() if isinstance(tensors, dict) else tensors
    shard: dict[str, torch.Tensor] = {}
    size = 0
    index = 0
    weight_map: dict[str, str] = {}

    def flush() -> None:
        nonlocal shard, size, index
        if not shard:
            return
        fname = f"model-{index:05d}.safetensors"
        save_file(shard, os.path.join(path, fname))
        for k in shard:
            weight_map[k] = fname
        shard, size, index = {}, 0, index + 1

    for name, tensor in items:
        t = tensor.detach().to("cpu").contiguous()
        shard[name] = t
        size += t.numel() * t.element_size()
        if size >= shard_bytes:
            flush()
    flush()
    with open(os.path.join(path, "model.safetensors.index.json"), "w", encoding="utf-8") as fh:
        json.dump({"metadata": {}, "weight_map": weight_map}, fh)


def open_weight_source(
    model: str, arch: Qwen3VLArch, *, dtype: torch.dtype, device, seed: int = 0
) -> Callable[[], Iterator[tuple[str, torch.Tensor]]]:
    """``model`` is a checkpoint directory, or ``random:<anything>`` for random init."""
    if model.startswith("random:") or not glob.glob(os.path.join(model, "*.safetensors")):
        return lambda: iter_random_weights(arch, dtype=dtype, device=device, seed=seed)
    return lambda: iter_safetensors(model)
