"""Host side of the persistent decode kernel (``csrc/decode_layers.cu``): all decoder layers of
a decode step of at most 16 tokens in one cooperative launch.

``DecodeLayersPlan`` is built once per (model weights, KV cache): it writes one descriptor per
layer (four weight tensor maps, the norm weights, the layer's K / V page arrays) into device
memory and asks the library for the grid size and the number of partial slabs each GEMM needs
with its stream-K split.  ``run`` launches one step; its work buffers are allocated once per
token count, so a CUDA graph can capture the launch.  The loop it replaces is
``Qwen3VLModel.forward`` for decode (reference ``prism_infer/models/qwen3_vl.py:925-1022``).
"""

from __future__ import annotations

import ctypes
import os
import struct

import torch

from . import native

MAX_TOKENS = 16
# 0 switches the persistent kernel off (the per-layer kernel chain runs instead)
ENABLED = os.environ.get("PRISM_DECODE_LAYERS", "1") != "0"

_ARG_NAMES = (
    "layers", "n_layers", "T", "H", "Hq", "Hkv", "D", "I", "m_qkv", "page", "max_blocks", "num_blocks", "kv_mode",
    "nsplit", "eps_bits", "scale_bits", "x0", "positions", "slots", "block_tables", "context_lens", "inv_freq", "axis",
    "residual", "xw", "attn", "act", "ssq", "part_o", "part_ml", "attn_counters", "gbar", "abort", "part_qkv",
    "part_oproj", "part_gu", "part_down", "grid", "timeline", "pf_depth", "tp", "rank", "epoch", "tile_counters",
) + tuple(f"xch{s}_{r}" for s in (0, 1) for r in range(8))
TIMELINE_STAMPS = 20  # 13 phase boundaries of a layer + 7 stamps inside the CTA's first attention item
TIMELINE_PHASES = 13
# weight tiles (16 KB each) the producer requests into L2 ahead of its shared-memory ring, so that HBM keeps
# streaming while the ring waits for a barrier or a pointwise phase; 0 switches the requests off
PREFETCH_UNITS = int(os.environ.get("PRISM_DECODE_PREFETCH_UNITS", "24"))


def _f32_bits(x: float) -> int:
    return struct.unpack("<I", struct.pack("<f", float(x)))[0]


def supported(*, hidden: int, heads: int, kv_heads: int, head_dim: int, intermediate: int) -> bool:
    """Shapes the kernel handles: head dimension 64 or 128, 1 / 2 / 4 / 8 query heads per KV head
    with 128 to 512 query values per KV head, hidden and MLP widths multiples of 128."""
    if head_dim not in (64, 128) or kv_heads <= 0 or heads % kv_heads:
        return False
    gq = heads // kv_heads
    if gq not in (1, 2, 4, 8) or not 128 <= gq * head_dim <= 512:
        return False
    return hidden % 128 == 0 and intermediate % 128 == 0 and (heads * head_dim) % 64 == 0 and hidden <= 8192


class DecodeLayersPlan:
    def __init__(self, layers, cache, *, hidden: int, heads: int, kv_heads: int, head_dim: int, intermediate: int,
                 eps: float, inv_freq: torch.Tensor, axis: torch.Tensor, tp: int = 1, rank: int = 0, epoch_ptr: int = 0,
                 exchange_ptrs: tuple[list[int], list[int]] | None = None) -> None:
        """``layers``: the model's ``LayerWeights`` (packed qkv / o / gate_up / down and norm weights);
        ``cache``: the ``ops.KVCache`` the layers write and read.  Sizes are per rank.  Tensor-parallel
        ranks pass the device address of the step-epoch word and, for each of the two exchange
        buffers, every rank's address of it (``tp * 16 * hidden`` 8-byte words each, in peer-mapped
        memory); the kernel then all-reduces the row-parallel projections and the embedding itself."""
        self.tp, self.rank, self.epoch_ptr = int(tp), int(rank), int(epoch_ptr)
        self.exchange_ptrs = exchange_ptrs
        if self.tp > 1 and (exchange_ptrs is None or not epoch_ptr or len(exchange_ptrs[0]) < tp or len(exchange_ptrs[1]) < tp):
            raise ValueError("tensor-parallel decode needs the epoch word and both exchange buffers of every rank")
        lib = native.lib()
        self.device = cache.payload.device
        self.cache = cache
        self.H, self.Hq, self.Hkv, self.D, self.I = hidden, heads, kv_heads, head_dim, intermediate
        self.m_qkv = (heads + 2 * kv_heads) * head_dim
        self.eps = float(eps)
        self.n_layers = len(layers)
        self.inv_freq = inv_freq.to(self.device, torch.float32).contiguous()
        self.axis = axis.to(self.device, torch.int32).contiguous()
        plan = (ctypes.c_int * 6)()
        native.call("prism_decode_layers_plan", hidden, self.m_qkv, heads * head_dim, intermediate,
                    ctypes.cast(plan, ctypes.c_void_p))
        self.grid, self.slabs, self.stages = int(plan[0]), [int(plan[i]) for i in range(1, 5)], int(plan[5])
        nbytes = int(lib.prism_decode_layer_desc_bytes())
        host = torch.zeros(self.n_layers * nbytes, dtype=torch.uint8)
        for i, l in enumerate(layers):
            native.call(
                "prism_decode_layer_desc", host.data_ptr() + i * nbytes, l.qkv.data_ptr(), self.m_qkv, l.o.data_ptr(),
                l.gate_up.data_ptr(), l.down.data_ptr(), hidden, heads * head_dim, intermediate, l.input_norm.data_ptr(),
                l.post_norm.data_ptr(), l.q_norm.data_ptr(), l.k_norm.data_ptr(), cache.k(i).data_ptr(),
                cache.v(i).data_ptr(), native.ptr(cache.k_scale(i)), native.ptr(cache.v_scale(i)))
        self._keep = [t for l in layers for t in (l.qkv, l.o, l.gate_up, l.down, l.input_norm, l.post_norm, l.q_norm, l.k_norm)]
        self.descs = host.to(self.device)
        self.gbar = torch.zeros(1, dtype=torch.int64, device=self.device)
        self.abort = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.counters = torch.zeros(MAX_TOKENS * max(1, kv_heads), dtype=torch.int32, device=self.device)
        self.ssq = torch.zeros(2 * MAX_TOKENS * 64, dtype=torch.float32, device=self.device)
        self.tile_counters = torch.zeros(3 * 512, dtype=torch.int32, device=self.device)
        self._work: dict[tuple[int, int], dict[str, torch.Tensor]] = {}
        self.timeline: torch.Tensor | None = None  # set by record_timeline(): SM clock stamps per CTA, layer, phase boundary

    def splits(self, tokens: int) -> int:
        """Context splits per (sequence, KV head): about one attention work item per CTA."""
        return max(1, min(32, self.grid // max(1, tokens * self.Hkv)))

    def _buffers(self, T: int, nsplit: int) -> dict[str, torch.Tensor]:
        key = (T, nsplit)
        w = self._work.get(key)
        if w is None:
            dev, bf, f32 = self.device, torch.bfloat16, torch.float32
            Ms = (self.m_qkv, self.H, 2 * self.I, self.H)
            w = {
                "residual": torch.zeros((T, self.H), dtype=bf, device=dev),
                "xw": torch.zeros((T, self.H), dtype=bf, device=dev),
                "attn": torch.zeros((T, self.Hq * self.D), dtype=bf, device=dev),
                "act": torch.zeros((T, self.I), dtype=bf, device=dev),
                "part_o": torch.zeros((T, self.Hq, nsplit, self.D), dtype=f32, device=dev),
                "part_ml": torch.zeros((T, self.Hq, nsplit, 2), dtype=f32, device=dev),
            }
            for name, P, M in zip(("part_qkv", "part_oproj", "part_gu", "part_down"), self.slabs, Ms):
                w[name] = torch.zeros((P, T, M), dtype=f32, device=dev)
            self._work[key] = w
        return w

    def run(self, x0: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, block_tables: torch.Tensor,
            context_lens: torch.Tensor, *, nsplit: int = 0) -> torch.Tensor:
        """One decode step.  ``x0 [T, H]`` bf16 embedding rows, ``positions [3, T]`` int32, ``slots [T]``
        int64, ``block_tables [T, max_blocks]`` int32, ``context_lens [T]`` int32 (new token included).
        Returns the hidden state before the final norm, ``[T, H]`` bf16 (a buffer owned by the plan)."""
        T = int(x0.shape[0])
        assert 1 <= T <= MAX_TOKENS and x0.dtype == torch.bfloat16 and x0.is_contiguous()
        assert positions.dtype == torch.int32 and slots.dtype == torch.int64
        assert block_tables.dtype == torch.int32 and context_lens.dtype == torch.int32 and block_tables.is_contiguous()
        nsplit = nsplit or self.splits(T)
        w = self._buffers(T, nsplit)
        vals = dict(
            layers=self.descs.data_ptr(), n_layers=self.n_layers, T=T, H=self.H, Hq=self.Hq, Hkv=self.Hkv, D=self.D, I=self.I,
            m_qkv=self.m_qkv, page=self.cache.page, max_blocks=block_tables.shape[1], num_blocks=self.cache.num_blocks,
            kv_mode=self.cache.mode, nsplit=nsplit, eps_bits=_f32_bits(self.eps), scale_bits=_f32_bits(self.D ** -0.5),
            x0=x0.data_ptr(), positions=positions.data_ptr(), slots=slots.data_ptr(), block_tables=block_tables.data_ptr(),
            context_lens=context_lens.data_ptr(), inv_freq=self.inv_freq.data_ptr(), axis=self.axis.data_ptr(),
            residual=w["residual"].data_ptr(), xw=w["xw"].data_ptr(), attn=w["attn"].data_ptr(), act=w["act"].data_ptr(),
            ssq=self.ssq.data_ptr(), part_o=w["part_o"].data_ptr(), part_ml=w["part_ml"].data_ptr(),
            attn_counters=self.counters.data_ptr(), gbar=self.gbar.data_ptr(), abort=self.abort.data_ptr(),
            part_qkv=w["part_qkv"].data_ptr(), part_oproj=w["part_oproj"].data_ptr(), part_gu=w["part_gu"].data_ptr(),
            part_down=w["part_down"].data_ptr(), grid=self.grid,
            timeline=0 if self.timeline is None else self.timeline.data_ptr(), pf_depth=PREFETCH_UNITS,
            tp=self.tp, rank=self.rank, epoch=self.epoch_ptr, tile_counters=self.tile_counters.data_ptr(),
        )
        for slot in (0, 1):
            for r in range(8):
                vals[f"xch{slot}_{r}"] = self.exchange_ptrs[slot][r] if (self.tp > 1 and r < self.tp) else 0
        args = (ctypes.c_longlong * len(_ARG_NAMES))(*[int(vals[n]) for n in _ARG_NAMES])
        native.call("prism_decode_layers", ctypes.cast(args, ctypes.c_void_p), len(_ARG_NAMES),
                    torch.cuda.current_stream().cuda_stream)
        return w["residual"]

    def record_timeline(self, on: bool = True) -> None:
        """Profiling aid: have worker thread 0 of every CTA store its SM clock at each phase boundary
        (``[grid, layers, 20]`` int64 in ``self.timeline``: 13 phase boundaries, then 7 stamps inside the CTA's
        first attention item of the layer; differences within one CTA are cycles)."""
        self.timeline = torch.zeros((self.grid, self.n_layers, TIMELINE_STAMPS), dtype=torch.int64, device=self.device) if on else None

    def reset(self) -> None:
        """Clear the abort word after a reported failure (a set word makes every later launch return at once)."""
        self.abort.zero_()
        self.counters.zero_()
        self.tile_counters.zero_()
