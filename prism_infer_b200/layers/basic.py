"""Stand-alone normalisation, activation and rotary modules (reference
``prism_infer/layers/layernorm.py:8-54``, ``layers/activation.py:8-17``,
``layers/rotary_embedding.py:9-86``).

The Qwen3-VL path does not go through these classes: its decoder layer calls the fused kernels
directly (add + RMSNorm with the residual carried in bf16, QK-norm + M-RoPE + KV store, the
dual-GEMM SwiGLU).  They exist for code that composes a model out of modules, and they run the
same kernels: on a CUDA tensor ``RMSNorm`` launches ``prism_add_rmsnorm`` and ``SiluAndMul``
launches ``prism_swiglu``; on a CPU tensor both evaluate the plain PyTorch form of the same
arithmetic.  Inputs may have any number of leading dimensions.
"""

from __future__ import annotations

import torch
from torch import nn

from .. import ops


def _positive_int(name: str, value) -> int:
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ValueError(f"{name} must be a positive integer, got {value!r}")
    return value


class RMSNorm(nn.Module):
    """``y = x / rms(x) * weight``; with ``residual`` the sum ``x + residual`` is normalised and
    also returned (rounded to the input dtype) as the next residual."""

    def __init__(self, hidden_size: int, eps: float = 1e-6) -> None:
        super().__init__()
        self.hidden_size = _positive_int("hidden_size", hidden_size)
        self.eps = float(eps)
        self.weight = nn.Parameter(torch.ones(hidden_size))

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        w = self.weight if self.weight.dtype == x.dtype else self.weight.to(x.dtype)
        if residual is None:
            return ops.rmsnorm(x2.contiguous(), w, self.eps).view(shape)
        # the kernel updates the residual in place: work on a copy so the caller's tensor survives
        carried = residual.reshape(-1, shape[-1]).clone()
        normed, carried = ops.add_rmsnorm(w, self.eps, x=x2.contiguous(), residual=carried)
        return normed.view(shape), carried.view(shape)


class SiluAndMul(nn.Module):
    """SwiGLU over a concatenated ``[gate | up]`` last dimension."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.shape[-1] % 2:
            raise ValueError(f"the last dimension holds gate and up halves, got {x.shape[-1]}")
        lead = x.shape[:-1]
        y = ops.swiglu(x.reshape(-1, x.shape[-1]).contiguous())
        return y.view(*lead, x.shape[-1] // 2)


def apply_rotary_emb(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Half-split rotary: ``(x1, x2) -> (x1 cos - x2 sin, x2 cos + x1 sin)`` in fp32."""
    half = x.shape[-1] // 2
    xf = x.float()
    lo, hi = xf[..., :half], xf[..., half:]
    return torch.cat((lo * cos - hi * sin, hi * cos + lo * sin), dim=-1).to(x.dtype)


class RotaryEmbedding(nn.Module):
    """One-axis rotary table ``[max_positions, 1, head_size]`` = ``[cos | sin]`` and its
    application to query and key ``[T, heads, head_size]``.  Only full-width rotation
    (``rotary_dim == head_size``) is supported, as in the reference."""

    def __init__(self, head_size: int, rotary_dim: int, max_position_embeddings: int, base: float) -> None:
        super().__init__()
        _positive_int("head_size", head_size)
        _positive_int("rotary_dim", rotary_dim)
        if rotary_dim != head_size:
            raise ValueError(f"partial rotary dimensions are unsupported: rotary_dim={rotary_dim}, head_size={head_size}")
        if rotary_dim % 2:
            raise ValueError(f"rotary_dim must be even, got {rotary_dim}")
        if max_position_embeddings <= 0:
            raise ValueError(f"max_position_embeddings must be positive, got {max_position_embeddings}")
        if base <= 0:
            raise ValueError(f"RoPE base must be positive, got {base}")
        self.head_size = head_size
        exponent = torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim
        angle = torch.arange(max_position_embeddings, dtype=torch.float32)[:, None] * (1.0 / base ** exponent)[None, :]
        self.register_buffer("cos_sin_cache", torch.cat((angle.cos(), angle.sin()), dim=-1)[:, None, :], persistent=False)

    def forward(self, positions: torch.Tensor, query: torch.Tensor, key: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        table = self.cos_sin_cache[positions]
        half = table.shape[-1] // 2
        cos, sin = table[..., :half], table[..., half:]
        return apply_rotary_emb(query, cos, sin), apply_rotary_emb(key, cos, sin)


_ROPE_CACHE: dict[tuple, RotaryEmbedding] = {}


def get_rope(head_size: int, rotary_dim: int, max_position: int, base: float, rope_scaling: dict | None = None) -> RotaryEmbedding:
    """Shared table per configuration (reference ``layers/rotary_embedding.py:73-86``); scaled
    variants are rejected rather than silently ignored."""
    if rope_scaling is not None:
        raise NotImplementedError("rope_scaling is not supported by the one-axis rotary table")
    key = (head_size, rotary_dim, max_position, float(base))
    if key not in _ROPE_CACHE:
        _ROPE_CACHE[key] = RotaryEmbedding(head_size, rotary_dim, max_position, base)
    return _ROPE_CACHE[key]
