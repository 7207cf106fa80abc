"""Functional op layer.

CUDA tensors run the hand-written sm_100a kernels from ``libprism_b200.so`` and raise if
the library is missing; CPU tensors run the plain-PyTorch statement of the same op, which
is what the CPU test-suite and the tiny CPU model use.  Shapes and the KV-cache layout
(payload ``[blocks, Hkv, page, D]``, scales ``[blocks, Hkv, page]``) are identical on both
paths.  The op set mirrors the reference's ``prism_infer/ops`` package
(``paged_decode_attention``, ``store_kvcache``, ``compact_kv_slots``, ``fused_qk_rmsnorm``,
``fused_add_rmsnorm``, ``fused_silu_mul``, dual-GEMM SwiGLU) plus the library calls it
leaves to cuBLAS / FlashAttention / cuDNN.
"""

from __future__ import annotations

import math
from typing import Optional, Sequence

import torch
import torch.nn.functional as F

from . import native

KV_BF16, KV_FP8, KV_FP8_SCALED = 0, 1, 2
FP8_MAX = 448.0
FP8_SCALE_FLOOR = 1.0e-6
SM_COUNT = 148

_PDL = False


def set_pdl(enabled: bool) -> None:
    """Launch kernels with programmatic stream serialization (overlapped prologues)."""
    global _PDL
    _PDL = bool(enabled)


def pdl_enabled() -> bool:
    return _PDL


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _s() -> int:
    return torch.cuda.current_stream().cuda_stream


def _pdl() -> int:
    return 1 if _PDL else 0


# ------------------------------------------------------------------------------- GEMM
SPLIT_K_MAX_TOKENS = 511  # from 512 tokens the persistent GEMM (several tiles per CTA) takes over


def choose_splits(m: int, k: int, tokens: int) -> int:
    """Split-K factor that fills the 148 SMs: for a weight-streaming GEMM (at most 128 tokens, one token
    tile) and for the short prefills above it (up to 511 tokens, one or two token tiles), where a
    row-parallel projection with 32 weight tiles would otherwise keep a fifth of the SMs busy."""
    if tokens > SPLIT_K_MAX_TOKENS:
        return 1
    tiles = (m + 127) // 128
    if tokens > 128:
        tiles *= (tokens + 255) // 256  # upper bound of the kernel's own tile choice (128 or 256 tokens)
    kb = (k + 63) // 64
    # one CTA per SM is resident (the operand ring fills shared memory), so more CTAs than
    # SMs means a second, mostly empty wave: stay at or below the SM count
    want = max(1, SM_COUNT // tiles)
    return max(1, min(want, kb // 4 if kb >= 8 else 1, 16))


def linear(
    x: torch.Tensor,
    w: torch.Tensor,
    *,
    bias: Optional[torch.Tensor] = None,
    act: Optional[str] = None,
    residual: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    bn: int = 0,
    stages: int = 0,
) -> torch.Tensor:
    """``act(x @ w.T + bias) (+ residual)``; x ``[T, K]``, w ``[M, K]`` -> ``[T, M]``."""
    T, K = x.shape
    M = w.shape[0]
    if not x.is_cuda:
        y = F.linear(x, w, bias)
        if act == "gelu_tanh":
            y = F.gelu(y, approximate="tanh")
        elif act == "gelu":
            y = F.gelu(y)
        if residual is not None:
            y = y + residual
        if out is not None:
            out.copy_(y)
            return out
        return y
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    assert x.stride(1) == 1 and w.stride(1) == 1
    if out is None:
        out = torch.empty((T, M), dtype=torch.bfloat16, device=x.device)
    code = {None: 0, "gelu_tanh": 1, "gelu": 2}[act]
    native.call(
        "prism_gemm_wx", _p(w), _p(x), _p(out), M, T, K, w.stride(0), x.stride(0), out.stride(0), M,
        _p(bias), _p(residual), residual.stride(0) if residual is not None else 0, code, 0, 0, 1, 0, 0,
        bn, stages, _s(), _pdl(),
    )
    return out


def linear_partial(
    x: torch.Tensor, w: torch.Tensor, splits: int, out: Optional[torch.Tensor] = None, *, bn: int = 0, stages: int = 0
) -> torch.Tensor:
    """Split-K GEMM: fp32 partial slabs ``[S, T, M]`` whose sum over S is ``x @ w.T``."""
    T, K = x.shape
    M = w.shape[0]
    if not x.is_cuda:
        y = F.linear(x.float(), w.float())
        if out is None:
            return y.unsqueeze(0)
        out.zero_()
        out[0].copy_(y)
        return out
    eff = effective_splits(K, splits)
    if out is None:
        out = torch.empty((eff, T, M), dtype=torch.float32, device=x.device)
    assert out.shape[0] >= eff and out.is_contiguous()
    native.call(
        "prism_gemm_wx", _p(w), _p(x), _p(out), M, T, K, w.stride(0), x.stride(0), out.stride(1), M,
        None, None, 0, 0, 0, 0, eff, 1, out.stride(0), bn, stages, _s(), _pdl(),
    )
    return out[:eff]


def effective_splits(k: int, splits: int) -> int:
    kb = (k + 63) // 64
    splits = max(1, min(splits, kb))
    per = (kb + splits - 1) // splits
    return (kb + per - 1) // per


def gate_up_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, out: Optional[torch.Tensor] = None, *, bn: int = 0) -> torch.Tensor:
    """``silu(x @ Wg.T) * (x @ Wu.T)`` with ``w_gate_up = [Wg ; Wu]`` of shape ``[2I, K]``."""
    T, K = x.shape
    I = w_gate_up.shape[0] // 2
    if not x.is_cuda:
        gu = F.linear(x, w_gate_up)
        y = F.silu(gu[:, :I]) * gu[:, I:]
        if out is not None:
            out.copy_(y)
            return out
        return y
    if out is None:
        out = torch.empty((T, I), dtype=torch.bfloat16, device=x.device)
    native.call(
        "prism_gemm_wx", _p(w_gate_up), _p(x), _p(out), I, T, K, w_gate_up.stride(0), x.stride(0), out.stride(0),
        2 * I, None, None, 0, 0, 1, I, 1, 0, 0, bn, 0, _s(), _pdl(),
    )
    return out


import os as _os

# Launch tuning, fixed where a measurement settled it (the numbers are in the profiles next to the repo's
# benchmarks); tests set the attributes directly.
# smallest decode batch that uses the tensor-core (mma) decode-attention kernel: on the headline decode step
# (batch 1, context ~1650) it measured 0.17 ms faster than the SIMT kernel
DECODE_MMA_MIN_BATCH = 1
# operand-ring depth of the decode-sized o_proj GEMM (0 = as deep as fits)
O_PROJ_STAGES = 0
# tcgen05 attention for contiguous bf16 K / V (prefill without history, the vision tower)
ATTN_TC_ENABLED = True
# prefill over the paged cache (chunked prefill, prefix hits) at head dimension 128: gather the visible keys from
# their pages once per layer, then the same tcgen05 kernel (False: the mma.sync kernel that reads the pages itself)
PAGED_PREFILL_TC_ENABLED = True
# the gathered rows cost 4 x KV heads x head dimension bytes per visible key (K and V in bf16): above this total the
# page-reading kernel runs instead (a prefill step over very many long histories), so the scratch stays inside the
# memory the KV sizing leaves free
PAGED_PREFILL_TC_MAX_SCRATCH_BYTES = 2 << 30
# prefill GEMMs of at least this many tokens run the persistent form, tokens on the TMEM lanes
PERSISTENT_ROWMAJOR = True
PERSISTENT_MIN_TOKENS = 512
# shared-memory cap of decode-sized GEMM launches (0 = none)
SMALL_TILE_SMEM_CAP = 0
# tensor-parallel prefill: GEMM -> reduce-scatter / reduce + norm -> all-gather kernels; PRISM_TP_PREFILL_FUSED=0
# selects the NCCL all-reduce arm the benchmarks compare against
TP_PREFILL_FUSED = _os.environ.get("PRISM_TP_PREFILL_FUSED", "1") != "0"


def apply_tuning() -> None:
    """Push the process-wide launch tuning into the native library (CUDA only)."""
    native.call("prism_gemm_set_small_tile_smem_cap", SMALL_TILE_SMEM_CAP)
    native.call("prism_gemm_set_persistent_min_tokens", PERSISTENT_MIN_TOKENS)
    native.call("prism_gemm_set_persistent_rowmajor", 1 if PERSISTENT_ROWMAJOR else 0)


# ------------------------------------------------------------------------- norm family
def add_rmsnorm(
    weight: torch.Tensor,
    eps: float,
    *,
    x: Optional[torch.Tensor] = None,
    partials: Optional[torch.Tensor] = None,
    residual: Optional[torch.Tensor] = None,
    extra: Optional[torch.Tensor] = None,
    extra_index: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    write_out: bool = True,
) -> tuple[Optional[torch.Tensor], torch.Tensor]:
    """Returns ``(normed, new_residual)``.

    ``delta`` is ``x`` or the sum of the fp32 ``partials [P, T, H]``;
    ``new_residual = residual + delta (+ extra[extra_index])``; ``residual`` is updated in
    place when given, otherwise ``new_residual`` is a fresh tensor (or ``x`` itself).
    """
    src = x if x is not None else partials[0]
    T, H = src.shape
    if not src.is_cuda:
        delta = x if x is not None else partials.sum(0).to(weight.dtype)
        added = delta if residual is None else residual + delta
        if extra is not None:
            mask = extra_index >= 0
            added = added.clone()
            added[mask] = added[mask] + extra[extra_index[mask].long()]
        if residual is not None:
            residual.copy_(added)
            added = residual
        normed = None
        if write_out:
            af = added.float()
            normed = (af * torch.rsqrt(af.pow(2).mean(-1, keepdim=True) + eps)).to(added.dtype) * weight
            if out is not None:
                out.copy_(normed)
                normed = out
        return normed, added
    if residual is None:
        new_res = torch.empty((T, H), dtype=torch.bfloat16, device=src.device)
    else:
        new_res = residual
    if write_out and out is None:
        out = torch.empty((T, H), dtype=torch.bfloat16, device=src.device)
    P = 0 if partials is None else partials.shape[0]
    native.call(
        "prism_add_rmsnorm", _p(partials), partials.stride(0) if partials is not None else 0, P, _p(x),
        _p(residual), _p(new_res), _p(extra), _p(extra_index), _p(weight), _p(out) if write_out else None,
        T, H, float(eps), _s(), _pdl(),
    )
    return (out if write_out else None), new_res


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    if not x.is_cuda:
        xf = x.float()
        y = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * weight
        if out is not None:
            out.copy_(y)
            return out
        return y
    T, H = x.shape
    if out is None:
        out = torch.empty_like(x)
    native.call("prism_add_rmsnorm", None, 0, 0, _p(x), None, None, None, None, _p(weight), _p(out), T, H,
                float(eps), _s(), _pdl())
    return out


def layernorm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    if not x.is_cuda:
        return F.layer_norm(x, (x.shape[-1],), w, b, eps)
    x2 = x.reshape(-1, x.shape[-1])
    assert x2.is_contiguous()
    out = torch.empty_like(x2)
    native.call("prism_layernorm", _p(x2), _p(w), _p(b), _p(out), x2.shape[0], x2.shape[1], float(eps), _s(), _pdl())
    return out.view(x.shape)


# ------------------------------------------------------------------- KV cache container
class KVCache:
    """One allocation for every layer: payload ``[2, L, blocks, Hkv, page, D]`` (+ scales)."""

    def __init__(self, num_layers: int, num_blocks: int, num_kv_heads: int, page: int, head_dim: int,
                 mode: int, device, dtype: torch.dtype = torch.bfloat16, pin_memory: bool = False):
        self.num_layers, self.num_blocks, self.num_kv_heads = num_layers, num_blocks, num_kv_heads
        self.page, self.head_dim, self.mode = page, head_dim, mode
        shape = (2, num_layers, num_blocks, num_kv_heads, page, head_dim)
        pdtype = dtype if mode == KV_BF16 else torch.float8_e4m3fn
        kw = dict(device=device)
        if pin_memory:
            kw = dict(device="cpu", pin_memory=True)
        self.payload = torch.zeros(shape, dtype=pdtype, **kw)
        self.scales = torch.zeros(shape[:-1], dtype=torch.float32, **kw) if mode == KV_FP8_SCALED else None

    def k(self, layer: int) -> torch.Tensor:
        return self.payload[0, layer]

    def v(self, layer: int) -> torch.Tensor:
        return self.payload[1, layer]

    def k_scale(self, layer: int) -> Optional[torch.Tensor]:
        return None if self.scales is None else self.scales[0, layer]

    def v_scale(self, layer: int) -> Optional[torch.Tensor]:
        return None if self.scales is None else self.scales[1, layer]

    @property
    def n_slabs(self) -> int:
        return 2 * self.num_layers

    def bytes_per_page(self) -> int:
        n = 2 * self.num_layers * self.num_kv_heads * self.page
        return n * self.head_dim * self.payload.element_size() + (n * 4 if self.scales is not None else 0)

    def dequant(self, kv: int, layer: int) -> torch.Tensor:
        """``[blocks, Hkv, page, D]`` fp32 view of what attention sees."""
        x = self.payload[kv, layer].float()
        if self.scales is not None:
            x = x * self.scales[kv, layer].unsqueeze(-1)
        return x


def quantize_fp8_rows(x: torch.Tensor, scaled: bool) -> tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Reference quantiser: per last-dim row ``scale = max(absmax/448, 1e-6)``."""
    xf = x.float()
    if scaled:
        scale = (xf.abs().amax(-1) / FP8_MAX).clamp_min(FP8_SCALE_FLOOR)
        q = (xf / scale.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
        return q, scale
    return xf.clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn), None


def _rope_tables(head_dim: int, theta: float, section: Sequence[int], device) -> tuple[torch.Tensor, torch.Tensor]:
    from ..models.position import mrope_axis_table, mrope_inv_freq

    key = (head_dim, float(theta), tuple(section), str(device))
    hit = _ROPE_CACHE.get(key)
    if hit is None:
        hit = (mrope_inv_freq(head_dim, theta).to(device), mrope_axis_table(section, head_dim // 2).to(device))
        _ROPE_CACHE[key] = hit
    return hit


_ROPE_CACHE: dict = {}


def qk_norm_rope_store(
    *,
    qkv: Optional[torch.Tensor],
    partials: Optional[torch.Tensor],
    positions: torch.Tensor,
    q_weight: torch.Tensor,
    k_weight: torch.Tensor,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    theta: float,
    section: Sequence[int],
    eps: float,
    slots: torch.Tensor,
    cache: KVCache,
    layer: int,
    q_out: Optional[torch.Tensor] = None,
    apply_norm: bool = True,
    apply_rope: bool = True,
    k_writeback: bool = False,
) -> torch.Tensor:
    """Per-head RMSNorm of q/k, interleaved M-RoPE, then K/V written to the paged cache.
    With ``k_writeback`` (CUDA, bf16 ``qkv`` source) the normalised, rotated K also replaces
    its slice of ``qkv`` so a prefill without history can attend over ``qkv`` directly.

    ``qkv [T, (Hq + 2 Hkv) * D]`` (or fp32 split-K ``partials [P, T, ...]``), ``positions
    [3, T]`` int32, ``slots [T]`` int64 flat slot (``block * page + offset``, negative =
    do not store).  Returns ``q [T, Hq, D]``.
    """
    src = qkv if qkv is not None else partials[0]
    T = src.shape[0]
    Hq, Hkv, D = num_heads, num_kv_heads, head_dim
    if not src.is_cuda:
        from ..models.position import mrope_cos_sin, rotate_half

        full = qkv if qkv is not None else partials.sum(0).to(q_weight.dtype)
        q, k, v = full.split([Hq * D, Hkv * D, Hkv * D], dim=-1)
        q, k, v = q.reshape(T, Hq, D), k.reshape(T, Hkv, D), v.reshape(T, Hkv, D)
        if apply_norm:
            def _n(z, w):
                zf = z.float()
                return (zf * torch.rsqrt(zf.pow(2).mean(-1, keepdim=True) + eps)).to(z.dtype) * w
            q, k = _n(q, q_weight), _n(k, k_weight)
        if apply_rope:
            cos, sin = mrope_cos_sin(positions.long(), D, theta, section)
            def _r(z):
                zf = z.float()
                return (zf * cos[:, None, :] + rotate_half(zf) * sin[:, None, :]).to(z.dtype)
            q, k = _r(q), _r(k)
        store_kv(k, v, slots, cache, layer)
        if k_writeback and qkv is not None:
            qkv[:, Hq * D:(Hq + Hkv) * D] = k.reshape(T, Hkv * D)
        if q_out is not None:
            q_out.copy_(q)
            return q_out
        return q.contiguous()
    inv_freq, axis = _rope_tables(D, theta, section, src.device)
    if q_out is None:
        q_out = torch.empty((T, Hq, D), dtype=torch.bfloat16, device=src.device)
    assert positions.dtype == torch.int32 and positions.is_contiguous() and slots.dtype == torch.int64
    native.call(
        "prism_qk_norm_rope_store", _p(qkv), _p(partials), partials.stride(0) if partials is not None else 0,
        0 if partials is None else partials.shape[0], src.stride(0), _p(positions), _p(q_weight), _p(k_weight),
        _p(inv_freq), _p(axis), _p(q_out), q_out.stride(0), _p(slots), _p(cache.k(layer)), _p(cache.v(layer)),
        _p(cache.k_scale(layer)), _p(cache.v_scale(layer)), T, Hq, Hkv, D, cache.page, cache.mode,
        1 if apply_norm else 0, 1 if apply_rope else 0, float(eps), 1 if (k_writeback and qkv is not None) else 0, _s(), _pdl(),
    )
    return q_out


def store_kv(k: torch.Tensor, v: torch.Tensor, slots: torch.Tensor, cache: KVCache, layer: int) -> None:
    """Scatter ``k, v [T, Hkv, D]`` to flat ``slots`` (negative = skip), quantising per the cache mode."""
    T, Hkv, D = k.shape
    if k.is_cuda:
        packed = torch.cat((torch.empty((T, 0), dtype=k.dtype, device=k.device), k.reshape(T, -1), v.reshape(T, -1)), dim=1)
        one = torch.ones(D, dtype=k.dtype, device=k.device)
        pos = torch.zeros((3, T), dtype=torch.int32, device=k.device)
        inv_freq, axis = _rope_tables(D, 10000.0, (D // 2, 0, 0), k.device)
        native.call(
            "prism_qk_norm_rope_store", _p(packed), None, 0, 0, packed.stride(0), _p(pos), _p(one), _p(one),
            _p(inv_freq), _p(axis), None, 0, _p(slots), _p(cache.k(layer)), _p(cache.v(layer)),
            _p(cache.k_scale(layer)), _p(cache.v_scale(layer)), T, 0, Hkv, D, cache.page, cache.mode, 0, 0,
            1e-6, 0, _s(), _pdl(),
        )
        return
    keep = slots >= 0
    if not bool(keep.any()):
        return
    sl = slots[keep].long()
    blk, off = sl // cache.page, sl % cache.page
    for kv, x in ((0, k[keep]), (1, v[keep])):
        if cache.mode == KV_BF16:
            cache.payload[kv, layer][blk, :, off] = x.to(cache.payload.dtype)
        else:
            qx, scale = quantize_fp8_rows(x, cache.mode == KV_FP8_SCALED)
            cache.payload[kv, layer][blk, :, off] = qx
            if scale is not None:
                cache.scales[kv, layer][blk, :, off] = scale


def swiglu(gu: Optional[torch.Tensor] = None, partials: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None):
    src = gu if gu is not None else partials[0]
    T, I2 = src.shape
    I = I2 // 2
    if not src.is_cuda:
        full = gu if gu is not None else partials.sum(0)
        y = F.silu(full[:, :I]) * full[:, I:]
        if out is not None:
            out.copy_(y)
            return out
        return y.to(src.dtype) if gu is not None else y
    if out is None:
        out = torch.empty((T, I), dtype=torch.bfloat16, device=src.device)
    native.call("prism_swiglu", _p(gu), _p(partials), partials.stride(0) if partials is not None else 0,
                0 if partials is None else partials.shape[0], _p(out), T, I, _s(), _pdl())
    return out


def embed(ids: torch.Tensor, table: torch.Tensor, *, visual: Optional[torch.Tensor] = None,
          vis_index: Optional[torch.Tensor] = None, vocab_start: int = 0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rows of ``table`` (a vocabulary shard starting at ``vocab_start``; ids outside give
    zeros) with ``visual[vis_index[t]]`` substituted where ``vis_index[t] >= 0``."""
    T, H = ids.shape[0], table.shape[1]
    if not table.is_cuda:
        local = ids - vocab_start
        ok = (local >= 0) & (local < table.shape[0])
        y = table[local.clamp(0, table.shape[0] - 1)] * ok[:, None].to(table.dtype)
        if visual is not None and vis_index is not None:
            m = vis_index >= 0
            y = y.clone()
            y[m] = visual[vis_index[m].long()].to(y.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    if out is None:
        out = torch.empty((T, H), dtype=torch.bfloat16, device=table.device)
    assert ids.dtype == torch.int64
    # first kernel of a step: it may follow a memcpy node, so it takes a full dependency
    native.call("prism_embed", _p(ids), _p(table), _p(visual), _p(vis_index), _p(out), T, H, vocab_start,
                vocab_start + table.shape[0], _s(), 0)
    return out


# --------------------------------------------------------------------------- attention
def decode_splits(batch: int, num_kv_heads: int) -> int:
    want = max(1, (2 * SM_COUNT) // max(1, batch * num_kv_heads))
    return int(min(32, want))


_DECODE_COUNTERS: dict = {}


def _decode_counters(device, n: int) -> torch.Tensor:
    """Zero-initialised, self-resetting arrival counters shared by all decode launches."""
    t = _DECODE_COUNTERS.get(str(device))
    if t is None or t.numel() < n:
        t = torch.zeros(max(n, 8192), dtype=torch.int32, device=device)
        _DECODE_COUNTERS[str(device)] = t
    return t


def paged_decode_attention(
    q: torch.Tensor, cache: KVCache, layer: int, block_tables: torch.Tensor, context_lens: torch.Tensor,
    *, nsplit: int = 0, out: Optional[torch.Tensor] = None, workspace: Optional[tuple[torch.Tensor, torch.Tensor]] = None,
    use_mma: Optional[bool] = None,
) -> torch.Tensor:
    """``q [B, Hq, D]`` against the paged cache; ``block_tables [B, maxblk]`` int32 (-1 = hole)."""
    B, Hq, D = q.shape
    scale = 1.0 / math.sqrt(D)
    if not q.is_cuda:
        outs = []
        kd, vd = cache.dequant(0, layer), cache.dequant(1, layer)
        G = Hq // cache.num_kv_heads
        for b in range(B):
            n = int(context_lens[b])
            if n == 0:
                outs.append(torch.zeros((Hq, D), dtype=q.dtype))
                continue
            pos = torch.arange(n)
            blk = block_tables[b, (pos // cache.page).long()].long()
            ok = blk >= 0
            k = kd[blk.clamp_min(0), :, pos % cache.page]  # [n, Hkv, D]
            v = vd[blk.clamp_min(0), :, pos % cache.page]
            k = k.repeat_interleave(G, dim=1)
            v = v.repeat_interleave(G, dim=1)
            s = torch.einsum("hd,nhd->hn", q[b].float(), k) * scale
            s = s.masked_fill(~ok[None, :], float("-inf"))
            p = torch.softmax(s, dim=-1)
            outs.append(torch.einsum("hn,nhd->hd", p, v).to(q.dtype))
        y = torch.stack(outs)
        if out is not None:
            out.copy_(y)
            return out
        return y
    if nsplit <= 0:
        nsplit = decode_splits(B, cache.num_kv_heads)
    if out is None:
        out = torch.empty_like(q)
    part_o = part_ml = None
    if nsplit > 1:
        if workspace is None:
            part_o = torch.empty((B, Hq, nsplit, D), dtype=torch.float32, device=q.device)
            part_ml = torch.empty((B, Hq, nsplit, 2), dtype=torch.float32, device=q.device)
        else:
            part_o, part_ml = workspace
    assert block_tables.dtype == torch.int32 and context_lens.dtype == torch.int32
    native.call(
        "prism_paged_decode", _p(q), _p(cache.k(layer)), _p(cache.v(layer)), _p(cache.k_scale(layer)),
        _p(cache.v_scale(layer)), _p(block_tables), _p(context_lens), _p(part_o), _p(part_ml), _p(out),
        _p(_decode_counters(q.device, B * cache.num_kv_heads)) if nsplit > 1 else None,
        B, Hq, cache.num_kv_heads, D, cache.page, block_tables.shape[1], cache.num_blocks, nsplit, cache.mode, scale,
        1 if (use_mma if use_mma is not None else B >= DECODE_MMA_MIN_BATCH) else 0, _s(), _pdl(),
    )
    return out


def varlen_attention(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor, max_len: int, *,
    causal: bool, out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Ragged self-attention over contiguous segments; ``q [T, Hq, D]``, ``k, v [T, Hkv, D]``
    (views into a packed projection are fine: only the last dim must be dense)."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    scale = 1.0 / math.sqrt(D)
    if not q.is_cuda:
        y = torch.empty((T, Hq, D), dtype=q.dtype)
        cu = cu_seqlens.tolist()
        G = Hq // Hkv
        for a, b in zip(cu[:-1], cu[1:]):
            o = F.scaled_dot_product_attention(
                q[a:b].transpose(0, 1).unsqueeze(0).float(),
                k[a:b].repeat_interleave(G, dim=1).transpose(0, 1).unsqueeze(0).float(),
                v[a:b].repeat_interleave(G, dim=1).transpose(0, 1).unsqueeze(0).float(),
                is_causal=causal,
            )
            y[a:b] = o.squeeze(0).transpose(0, 1).to(q.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    if out is None:
        out = torch.empty((T, Hq, D), dtype=torch.bfloat16, device=q.device)
    assert q.stride(2) == 1 and q.stride(1) == D and k.stride(1) == D and v.stride(1) == D
    assert k.stride(0) == v.stride(0) and cu_seqlens.dtype == torch.int32
    if (ATTN_TC_ENABLED and D in (128, 72) and q.stride(0) % 8 == 0 and k.stride(0) % 8 == 0
            and (q.data_ptr() | k.data_ptr() | v.data_ptr() | out.data_ptr()) % 16 == 0):
        # the tcgen05 / TMEM kernel (head dimension 128, or 72 padded to 80)
        native.call(
            "prism_flash_attention_tc", _p(q), q.stride(0), _p(k), _p(v), k.stride(0), _p(out), out.stride(0),
            _p(cu_seqlens), T, cu_seqlens.shape[0] - 1, int(max_len), Hq, Hkv, D, 1 if causal else 0, scale, _s(), _pdl(),
        )
        return out
    native.call(
        "prism_flash_attention", _p(q), q.stride(0), _p(out), out.stride(0), _p(cu_seqlens), _p(k), _p(v),
        k.stride(0), None, None, None, None, None, None, 0, 0, 1, cu_seqlens.shape[0] - 1, int(max_len), Hq, Hkv, D,
        0, 1 if causal else 0, scale, _s(), _pdl(),
    )
    return out


_GATHERED_KV: dict = {}  # device -> (rows, width, K rows, V rows): the gathered keys of the layer under way


def _gathered_kv_rows(device: torch.device, rows: int, width: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Scratch for the keys and values that ``paged_prefill_attention`` gathers from their pages; one pair per
    device, reused by every layer (launches of one stream run in order), grown in steps of 4096 rows."""
    have = _GATHERED_KV.get(device)
    if have is None or have[0] < rows or have[1] != width:
        cap = -(-rows // 4096) * 4096
        have = (cap, width, torch.empty((cap, width), dtype=torch.bfloat16, device=device),
                torch.empty((cap, width), dtype=torch.bfloat16, device=device))
        _GATHERED_KV[device] = have
    return have[2], have[3]


def paged_prefill_attention(
    q: torch.Tensor, cache: KVCache, layer: int, cu_seqlens_q: torch.Tensor, kv_lens: torch.Tensor,
    block_tables: torch.Tensor, max_q_len: int, *, out: Optional[torch.Tensor] = None,
    cu_seqlens_kv: Optional[torch.Tensor] = None, total_kv: int = 0, max_kv_len: int = 0,
) -> torch.Tensor:
    """Causal attention of the new tokens ``q [T, Hq, D]`` over the paged cache.

    Sequence ``s`` owns rows ``cu_seqlens_q[s]:cu_seqlens_q[s+1]``; it sees ``kv_lens[s]``
    cached keys (history, shared prefix pages and this chunk, already stored), the last
    ``q_len`` of which are the chunk itself.

    With ``cu_seqlens_kv`` (``[S+1]`` int32, the running sum of ``kv_lens``), ``total_kv`` and ``max_kv_len``
    (host integers) and head dimension 128, the keys are gathered from their pages once and the tcgen05 kernel
    runs over them; without them the mma.sync kernel reads the pages itself.
    """
    T, Hq, D = q.shape
    scale = 1.0 / math.sqrt(D)
    if not q.is_cuda:
        y = torch.empty((T, Hq, D), dtype=q.dtype)
        kd, vd = cache.dequant(0, layer), cache.dequant(1, layer)
        G = Hq // cache.num_kv_heads
        cu = cu_seqlens_q.tolist()
        for s, (a, b) in enumerate(zip(cu[:-1], cu[1:])):
            n = int(kv_lens[s])
            pos = torch.arange(n)
            blk = block_tables[s, (pos // cache.page).long()].long()
            ok = blk >= 0
            k = kd[blk.clamp_min(0), :, pos % cache.page].repeat_interleave(G, dim=1)
            v = vd[blk.clamp_min(0), :, pos % cache.page].repeat_interleave(G, dim=1)
            sc = torch.einsum("qhd,nhd->hqn", q[a:b].float(), k) * scale
            qpos = torch.arange(b - a) + (n - (b - a))
            mask = (pos[None, :] <= qpos[:, None]) & ok[None, :]
            sc = sc.masked_fill(~mask[None], float("-inf"))
            y[a:b] = torch.einsum("hqn,nhd->qhd", torch.softmax(sc, dim=-1), v).to(q.dtype)
        if out is not None:
            out.copy_(y)
            return out
        return y
    if out is None:
        out = torch.empty((T, Hq, D), dtype=torch.bfloat16, device=q.device)
    assert q.stride(2) == 1 and q.stride(1) == D
    assert cu_seqlens_q.dtype == torch.int32 and kv_lens.dtype == torch.int32 and block_tables.dtype == torch.int32
    if (ATTN_TC_ENABLED and PAGED_PREFILL_TC_ENABLED and D == 128 and cu_seqlens_kv is not None and total_kv > 0
            and 4 * int(total_kv) * cache.num_kv_heads * D <= PAGED_PREFILL_TC_MAX_SCRATCH_BYTES
            and q.stride(0) % 8 == 0 and (q.data_ptr() | out.data_ptr()) % 16 == 0):
        assert cu_seqlens_kv.dtype == torch.int32 and cu_seqlens_kv.shape == cu_seqlens_q.shape and max_kv_len <= total_kv
        k_rows, v_rows = _gathered_kv_rows(q.device, total_kv, cache.num_kv_heads * D)
        native.call(
            "prism_paged_prefill_tc", _p(q), q.stride(0), _p(out), out.stride(0), _p(cu_seqlens_q), _p(cu_seqlens_kv),
            _p(cache.k(layer)), _p(cache.v(layer)), _p(cache.k_scale(layer)), _p(cache.v_scale(layer)), _p(block_tables),
            block_tables.shape[1], cache.num_blocks, cache.page, _p(k_rows), _p(v_rows), T, int(total_kv),
            cu_seqlens_q.shape[0] - 1, int(max_q_len), int(max_kv_len), Hq, cache.num_kv_heads, D, cache.mode, scale,
            _s(), _pdl(),
        )
        return out
    native.call(
        "prism_flash_attention", _p(q), q.stride(0), _p(out), out.stride(0), _p(cu_seqlens_q), None, None, 0,
        _p(cache.k(layer)), _p(cache.v(layer)), _p(cache.k_scale(layer)), _p(cache.v_scale(layer)),
        _p(block_tables), _p(kv_lens), block_tables.shape[1], cache.num_blocks, cache.page, cu_seqlens_q.shape[0] - 1,
        int(max_q_len),
        Hq, cache.num_kv_heads, D, 1 if cache.mode == KV_BF16 else 2, 1, scale, _s(), _pdl(),
    )
    return out


# ------------------------------------------------------------------------ KV maintenance
def kv_page_copy(src: KVCache, dst: KVCache, src_blocks: Sequence[int], dst_blocks: Sequence[int],
                 rows: Optional[Sequence[int]] = None) -> None:
    """Copy (the first ``rows[i]`` tokens of) page ``src_blocks[i]`` to ``dst_blocks[i]``
    in every layer, K and V, payload and scales.  ``src`` and ``dst`` may be the same
    cache (copy-on-write, prefix copies) or a device cache and a pinned host pool (swap)."""
    n = len(src_blocks)
    if n == 0:
        return
    on_gpu = src.payload.is_cuda or dst.payload.is_cuda
    if not on_gpu:
        for i in range(n):
            r = src.page if rows is None else int(rows[i])
            dst.payload[:, :, dst_blocks[i], :, :r] = src.payload[:, :, src_blocks[i], :, :r]
            if src.scales is not None:
                dst.scales[:, :, dst_blocks[i], :, :r] = src.scales[:, :, src_blocks[i], :, :r]
        return
    dev = src.payload.device if src.payload.is_cuda else dst.payload.device
    sb = torch.tensor(list(src_blocks), dtype=torch.int32, device=dev)
    db = torch.tensor(list(dst_blocks), dtype=torch.int32, device=dev)
    nr = None if rows is None else torch.tensor(list(rows), dtype=torch.int32, device=dev)
    es = src.payload.element_size()
    native.call(
        "prism_kv_page_copy", _p(src.payload), _p(dst.payload), src.payload.stride(1) * es, dst.payload.stride(1) * es,
        src.head_dim * es, _p(src.scales), _p(dst.scales),
        src.scales.stride(1) * 4 if src.scales is not None else 0,
        dst.scales.stride(1) * 4 if dst.scales is not None else 0,
        _p(sb), _p(db), _p(nr), n, src.num_kv_heads, src.page, src.n_slabs, _s(),
    )


def kv_compact(cache: KVCache, src_slots: torch.Tensor, dst_slots: torch.Tensor) -> None:
    """Move the rows at flat ``src_slots`` to ``dst_slots`` in every layer (payload and
    scales), safe for overlapping ranges: gather into scratch, then scatter."""
    R = int(src_slots.shape[0])
    if R == 0:
        return
    if not cache.payload.is_cuda:
        sb, so = src_slots.long() // cache.page, src_slots.long() % cache.page
        db, do = dst_slots.long() // cache.page, dst_slots.long() % cache.page
        tmp = cache.payload[:, :, sb, :, so].clone()
        cache.payload[:, :, db, :, do] = tmp
        if cache.scales is not None:
            tmp_s = cache.scales[:, :, sb, :, so].clone()
            cache.scales[:, :, db, :, do] = tmp_s
        return
    es = cache.payload.element_size()
    rb = cache.head_dim * es
    rows = cache.n_slabs * cache.num_kv_heads * R
    temp = torch.empty(rows * rb, dtype=torch.uint8, device=cache.payload.device)
    stemp = torch.empty(rows, dtype=torch.float32, device=cache.payload.device) if cache.scales is not None else None
    native.call(
        "prism_kv_compact", _p(cache.payload), cache.payload.stride(1) * es, rb, _p(cache.scales),
        cache.scales.stride(1) * 4 if cache.scales is not None else 0, _p(temp), _p(stemp),
        _p(src_slots), _p(dst_slots), R, cache.num_kv_heads, cache.page, cache.n_slabs, _s(),
    )


# ------------------------------------------------------------------------------ sampler
def sample(
    logits: torch.Tensor, temperature: Optional[torch.Tensor] = None, *, seed: int = 0,
    step: Optional[torch.Tensor] = None, vocab_offset: int = 0, out: Optional[torch.Tensor] = None,
    out_val: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Token per row of fp32 ``logits [B, V]`` (or split slabs ``[P, B, V]``): arg-max where
    ``temperature`` is 0 / absent (lowest id wins ties), exponential-race sample elsewhere."""
    slabs = logits if logits.dim() == 3 else logits.unsqueeze(0)
    P, B, V = slabs.shape
    if not logits.is_cuda:
        full = slabs.sum(0).float()
        if temperature is not None and bool((temperature > 0).any()):
            gen = torch.Generator().manual_seed(int(seed) + (int(step.item()) if step is not None else 0))
            t = temperature.clamp_min(1e-10)[:, None]
            e = torch.empty_like(full).exponential_(1.0, generator=gen)
            noisy = torch.softmax(full / t, dim=-1) / e
            tok = torch.where(temperature > 0, noisy.argmax(-1), full.argmax(-1))
        else:
            tok = full.argmax(-1)
        tok = tok + vocab_offset
        if out_val is not None:
            out_val.copy_(full.max(-1).values)
        if out is not None:
            out.copy_(tok)
            return out
        return tok
    assert slabs.dtype == torch.float32 and slabs.stride(2) == 1
    if out is None:
        out = torch.empty((B,), dtype=torch.int64, device=logits.device)
    chunks = max(1, min(64, (V + 2047) // 2048, (4 * SM_COUNT) // B)) if V > 8192 else 1
    cand_val = cand_id = None
    if chunks > 1:
        cand_val = torch.empty((chunks, B), dtype=torch.float32, device=logits.device)
        cand_id = torch.empty((chunks, B), dtype=torch.int64, device=logits.device)
    native.call("prism_sample", _p(slabs), slabs.stride(1), slabs.stride(0), P, _p(temperature), _p(out), _p(out_val),
                B, V, vocab_offset, int(seed) & 0xFFFFFFFFFFFFFFFF, _p(step), _p(cand_val), _p(cand_id), chunks,
                _s(), _pdl())
    return out


# ------------------------------------------------------------------ FP8 candidate LM head
LM_HEAD_FP8_MAX_BATCH = 4  # the kernel's limit; measured, the candidate head beats the bf16 head at one row only
LM_HEAD_FP8_BATCH = 1      # rows up to which Qwen3VLModel.sample uses it


def quantize_lm_head_fp8(weight: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Row-scaled E4M3 copy of the LM head ``[V, H]`` for candidate generation: ``(codes uint8 [V, H], scale
    fp32 [V])`` with ``weight ~ codes * scale[:, None]`` (reference
    ``prism_infer/models/qwen3_vl.py:1723-1743``).  Done once at load time."""
    w = weight.float()
    scale = (w.abs().amax(dim=1) / 448.0).clamp_min(1e-12)
    codes = (w / scale[:, None]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    return codes.view(torch.uint8).contiguous(), scale.contiguous()


def lm_head_fp8_greedy(hidden: torch.Tensor, codes: torch.Tensor, scale: torch.Tensor, weight: torch.Tensor, *,
                       vocab_offset: int = 0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Greedy token per row of ``hidden [B, H]`` (B at most 4): candidates from the E4M3 head, exact fp32 rerank
    with the bf16 rows of ``weight``, lowest id on ties.  The CPU statement is the exact arg-max."""
    B, H = hidden.shape
    V = weight.shape[0]
    if not hidden.is_cuda:
        tok = F.linear(hidden.float(), weight.float()).argmax(-1) + vocab_offset
        if out is not None:
            out.copy_(tok)
            return out
        return tok
    assert B <= LM_HEAD_FP8_MAX_BATCH and hidden.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
    assert codes.dtype == torch.uint8 and codes.shape == (V, H) and codes.is_contiguous() and scale.dtype == torch.float32
    import ctypes as _ct

    plan = (_ct.c_int * 3)()
    native.call("prism_lm_head_fp8_plan", _ct.cast(plan, _ct.c_void_p))
    n_cand, n_list = int(plan[0]), int(plan[1])
    dev = hidden.device
    cand_val = torch.empty((B, n_cand), dtype=torch.float32, device=dev)
    cand_id = torch.empty((B, n_cand), dtype=torch.int32, device=dev)
    list_val = torch.empty((n_list, B), dtype=torch.float32, device=dev)
    list_id = torch.empty((n_list, B), dtype=torch.int64, device=dev)
    if out is None:
        out = torch.empty((B,), dtype=torch.int64, device=dev)
    native.call("prism_lm_head_fp8_candidates", _p(codes), _p(scale), _p(weight), weight.stride(0), _p(hidden), hidden.stride(0),
                B, V, H, vocab_offset, _p(cand_val), _p(cand_id), _p(list_val), _p(list_id), _s(), _pdl())
    native.call("prism_merge_candidates", _p(list_val), _p(list_id), _p(out), n_list, B, _s(), _pdl())
    return out


# ------------------------------------------------------------------------------- vision
def pos_embed_add(x: torch.Tensor, table: torch.Tensor, idx: torch.Tensor, wt: torch.Tensor) -> torch.Tensor:
    """In place ``x[n] += sum_k wt[k, n] * table[idx[k, n]]`` (bilinear 4-corner plan)."""
    if not x.is_cuda:
        x += (table[idx].float() * wt[:, :, None]).sum(0).to(x.dtype)
        return x
    native.call("prism_pos_embed_add", _p(x), _p(table), _p(idx), _p(wt), x.shape[0], x.shape[1], _s(), _pdl())
    return x


def vit_rope(qkv: torch.Tensor, coords: torch.Tensor, inv_freq: torch.Tensor, heads: int, hd: int) -> torch.Tensor:
    """In-place 2-D rotary on q and k of a packed ``[N, 3 * heads * hd]`` projection."""
    N = qkv.shape[0]
    if not qkv.is_cuda:
        from ..models.position import rotate_half

        ang = torch.cat((coords[:, 0:1].float() * inv_freq[None], coords[:, 1:2].float() * inv_freq[None]), dim=-1)
        ang = torch.cat((ang, ang), dim=-1)
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        view = qkv.view(N, 3, heads, hd)
        for i in (0, 1):
            z = view[:, i].float()
            view[:, i] = (z * cos + rotate_half(z) * sin).to(qkv.dtype)
        return qkv
    assert qkv.is_contiguous() and coords.dtype == torch.int32
    native.call("prism_vit_rope", _p(qkv), _p(coords), _p(inv_freq), N, heads, hd, _s(), _pdl())
    return qkv
