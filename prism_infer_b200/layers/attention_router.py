"""Attention module: store the step's K/V in the paged cache, then route to the kernel that
fits the step (reference ``prism_infer/layers/attention.py:69-111`` routes, ``:85-502`` whole).

Routes, chosen from the step's ``AttnMeta`` (the reference reads the same facts from a context
variable; here the metadata is an explicit argument):

=========================================  ====================================================
step                                       kernel
=========================================  ====================================================
prefill, no history (first chunk, no hit)  ``ops.varlen_attention`` over the fresh bf16 K/V rows
                                           (tcgen05 flash attention for head size 128)
prefill with history (later chunk, hit)    ``ops.paged_prefill_attention`` over the cache pages
decode                                     ``ops.paged_decode_attention`` (split-KV + merge)
=========================================  ====================================================

The cache's mode (bf16, unit-scale FP8, per-token-scaled FP8) is a property of the ``KVCache``
and is handled inside the store and the paged kernels.  The flagship model does not use this
class on its hot path: there the store is fused with QK-RMSNorm and M-RoPE in one kernel
(``ops.qk_norm_rope_store``); the module serves models whose rotary step is separate.
"""

from __future__ import annotations

import torch
from torch import nn

from .. import ops
from ..models.qwen3_vl import AttnMeta


class Attention(nn.Module):
    def __init__(self, num_heads: int, head_dim: int, scale: float | None = None, num_kv_heads: int | None = None,
                 layer: int = 0) -> None:
        super().__init__()
        num_kv_heads = num_kv_heads or num_heads
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads {num_heads} is not a multiple of num_kv_heads {num_kv_heads}")
        if scale is not None and abs(scale - head_dim ** -0.5) > 1e-6 * head_dim ** -0.5:
            raise ValueError("the kernels use the softmax scale head_dim ** -0.5")
        self.num_heads, self.num_kv_heads, self.head_dim, self.layer = num_heads, num_kv_heads, head_dim, layer
        self.cache: ops.KVCache | None = None

    def bind_cache(self, cache: ops.KVCache, layer: int | None = None) -> None:
        """The runner binds every layer to the one KV allocation after sizing it."""
        self.cache = cache
        if layer is not None:
            self.layer = layer

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, meta: AttnMeta) -> torch.Tensor:
        """``q [T, Hq*D]``, ``k, v [T, Hkv*D]`` (or already split into heads) -> ``[T, Hq*D]``."""
        T = q.shape[0]
        q = q.view(T, self.num_heads, self.head_dim)
        k = k.view(T, self.num_kv_heads, self.head_dim)
        v = v.view(T, self.num_kv_heads, self.head_dim)
        cache = self.cache
        if cache is not None:
            ops.store_kv(k, v, meta.slots, cache, self.layer)
        if meta.is_prefill:
            if meta.no_history or cache is None:
                out = ops.varlen_attention(q, k, v, meta.cu_seqlens_q, meta.max_q_len, causal=True)
            else:
                out = ops.paged_prefill_attention(q, cache, self.layer, meta.cu_seqlens_q, meta.kv_lens, meta.block_tables,
                                                  meta.max_q_len, cu_seqlens_kv=meta.cu_seqlens_kv, total_kv=meta.total_kv,
                                                  max_kv_len=meta.max_kv_len)
        else:
            if cache is None:
                raise RuntimeError("decode needs a bound KV cache")
            out = ops.paged_decode_attention(q, cache, self.layer, meta.block_tables, meta.context_lens, nsplit=meta.nsplit,
                                             workspace=meta.workspace)
        return out.reshape(T, self.num_heads * self.head_dim)
