"""Host side of the persistent decode kernel (``csrc/decode_layers.cu``): all decoder layers of
a decode step of at most 4 tokens in one cooperative launch, the SMs handing values to one
another as ``{value, sequence number}`` words.

``DecodeLayersPlan`` is built once per (model weights, KV cache): it writes one descriptor per
layer (four weight tensor maps, the norm weights, the layer's K / V page arrays) into device
memory and asks the library for the grid size and the number of partial slabs each GEMM needs
with its stream-K split.  ``run`` launches one step; every buffer it touches is allocated when the
plan is built, so a CUDA graph can capture the launch.  The loop it replaces is
``Qwen3VLModel.forward`` for decode (reference ``prism_infer/models/qwen3_vl.py:925-1022``).
"""

from __future__ import annotations

import ctypes
import os
import struct

import torch

from . import native

MAX_TOKENS = 4
# Off unless PRISM_DECODE_LAYERS=1: measured on a B200 (Qwen3-VL-8B, one sequence of 1600 tokens) the step
# takes 5.0 ms through this kernel against 3.85 ms through the per-layer kernel chain.  Its weight stream runs at
# the chain's rate, but each of the nine all-to-all hand-offs of a layer costs two dependent memory round
# trips of about 3 us each, more than the kernel boundary it replaces; benchmarks/profile_decode_layers.py
# prints the timeline.
ENABLED = os.environ.get("PRISM_DECODE_LAYERS", "0") == "1"

# order of enum DLArg in csrc/decode_layers.cu
_ARG_NAMES = (
    "layers", "n_layers", "T", "H", "Hq", "Hkv", "D", "I", "m_qkv", "page", "max_blocks", "num_blocks", "kv_mode",
    "nsplit", "eps_bits", "scale_bits", "state", "plan_generation", "arena", "arena_bytes", "x0", "positions", "slots",
    "block_tables", "context_lens", "inv_freq", "axis", "out", "xw_in", "xw_post", "ssq_in", "ssq_post", "attn_part", "attn",
    "act", "abort", "part_qkv", "part_oproj", "part_gu", "part_down", "grid", "timeline", "pf_depth",
)
TIMELINE_STAMPS = 16  # worker thread 0's time stamps at the step boundaries of a layer (see benchmarks/profile_decode_layers.py)
# weight tiles (16 KB each) the producer requests into L2 ahead of its shared-memory ring, so that HBM keeps
# streaming while the ring waits for the activations of the next GEMM; 0 switches the requests off
PREFETCH_UNITS = int(os.environ.get("PRISM_DECODE_PREFETCH_UNITS", "24"))
MAX_SPLITS = 32

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
                 eps: float, inv_freq: torch.Tensor, axis: torch.Tensor) -> None:
        """``layers``: the model's ``LayerWeights`` (packed qkv / o / gate_up / down and norm weights);
        ``cache``: the ``ops.KVCache`` the layers write and read.  One GPU only (tensor-parallel ranks
        run the per-layer chain)."""
        lib = native.lib()
        self.device = cache.payload.device
        self.cache = cache
        self.H, self.Hq, self.Hkv, self.D, self.I = hidden, heads, kv_heads, head_dim, intermediate
        self.m_qkv = (heads + 2 * kv_heads) * head_dim
        self.eps = float(eps)
        self.n_layers = len(layers)
        self.inv_freq = inv_freq.to(self.device, torch.float32).contiguous()
        self.axis = axis.to(self.device, torch.int32).contiguous()
        plan = (ctypes.c_int * 8)()
        native.call("prism_decode_layers_plan", hidden, self.m_qkv, heads * head_dim, intermediate,
                    ctypes.cast(plan, ctypes.c_void_p))
        self.grid, self.slabs = int(plan[0]), [int(plan[i]) for i in range(1, 5)]
        self.xslots, self.stages = int(plan[5]), (int(plan[6]), int(plan[7]))  # ring depth at 1 and at 4 tokens
        self.max_tokens = min(MAX_TOKENS, self.grid // max(1, kv_heads))  # one attention work item per CTA
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
        self.state = torch.zeros(2, dtype=torch.int64, device=self.device)  # {sequence base, wrap generation}
        self.generation = torch.zeros(1, dtype=torch.int64, device=self.device)
        self.abort = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.out = torch.zeros((MAX_TOKENS, hidden), dtype=torch.bfloat16, device=self.device)
        # every buffer of {value, sequence} words lives in one arena (the kernel zeroes it when the numbers wrap)
        T = MAX_TOKENS
        sizes = {"xw_in": T * hidden, "xw_post": T * hidden, "ssq_in": T * 64, "ssq_post": T * 64,
                 "attn_part": T * heads * MAX_SPLITS * (head_dim + 2), "attn": T * heads * head_dim, "act": T * intermediate}
        for name, P, M in zip(("part_qkv", "part_oproj", "part_gu", "part_down"), self.slabs,
                              (self.m_qkv, hidden, 2 * intermediate, hidden)):
            sizes[name] = P * T * M
        self._offsets, total = {}, 0
        for name, words in sizes.items():
            self._offsets[name] = total
            total += (words + 1) // 2 * 2  # 16-byte alignment
        self.arena = torch.zeros(total, dtype=torch.int64, device=self.device)
        self.timeline: torch.Tensor | None = None  # set by record_timeline(): SM clock stamps per CTA, layer, step boundary

    def splits(self, tokens: int) -> int:
        """Context splits per (sequence, KV head): one attention work item per CTA at most."""
        return max(1, min(MAX_SPLITS, self.grid // max(1, tokens * self.Hkv)))

    def run(self, x0: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, block_tables: torch.Tensor,
            context_lens: torch.Tensor, *, nsplit: int = 0) -> torch.Tensor:
        """One decode step.  ``x0 [T, H]`` bf16 embedding rows, ``positions [3, T]`` int32, ``slots [T]``
        int64, ``block_tables [T, max_blocks]`` int32, ``context_lens [T]`` int32 (new token included).
        Returns the hidden state before the final norm, ``[T, H]`` bf16 (a buffer owned by the plan)."""
        T = int(x0.shape[0])
        assert 1 <= T <= self.max_tokens and x0.dtype == torch.bfloat16 and x0.is_contiguous()
        assert positions.dtype == torch.int32 and slots.dtype == torch.int64
        assert block_tables.dtype == torch.int32 and context_lens.dtype == torch.int32 and block_tables.is_contiguous()
        nsplit = nsplit or self.splits(T)
        base = self.arena.data_ptr()
        vals = dict(
            layers=self.descs.data_ptr(), n_layers=self.n_layers, T=T, H=self.H, Hq=self.Hq, Hkv=self.Hkv, D=self.D, I=self.I,
            m_qkv=self.m_qkv, page=self.cache.page, max_blocks=block_tables.shape[1], num_blocks=self.cache.num_blocks,
            kv_mode=self.cache.mode, nsplit=nsplit, eps_bits=_f32_bits(self.eps), scale_bits=_f32_bits(self.D ** -0.5),
            state=self.state.data_ptr(), plan_generation=self.generation.data_ptr(), arena=base,
            arena_bytes=self.arena.numel() * 8, x0=x0.data_ptr(), positions=positions.data_ptr(), slots=slots.data_ptr(),
            block_tables=block_tables.data_ptr(), context_lens=context_lens.data_ptr(), inv_freq=self.inv_freq.data_ptr(),
            axis=self.axis.data_ptr(), out=self.out.data_ptr(), abort=self.abort.data_ptr(), grid=self.grid,
            timeline=0 if self.timeline is None else self.timeline.data_ptr(), pf_depth=PREFETCH_UNITS,
        )
        for name, off in self._offsets.items():
            vals[name] = base + 8 * off
        args = (ctypes.c_longlong * len(_ARG_NAMES))(*[int(vals[n]) for n in _ARG_NAMES])
        native.call("prism_decode_layers", ctypes.cast(args, ctypes.c_void_p), len(_ARG_NAMES),
                    torch.cuda.current_stream().cuda_stream)
        return self.out[:T]

    def record_timeline(self, on: bool = True) -> None:
        """Profiling aid: have worker thread 0 of every CTA store the GPU-wide timer at each step boundary of a
        layer (``[grid, layers, 16]`` int64 nanoseconds in ``self.timeline``)."""
        self.timeline = torch.zeros((self.grid, self.n_layers, TIMELINE_STAMPS), dtype=torch.int64, device=self.device) if on else None

    def reset(self) -> None:
        """Clear the abort word after a reported failure (a set word makes every later launch return at once)."""
        self.abort.zero_()
