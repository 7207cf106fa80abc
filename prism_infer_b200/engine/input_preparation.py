"""Host-side construction of one step's model inputs (reference
``prism_infer/engine/input_preparation.py:51-668``).

``StepInputs`` is a flat bundle of CPU tensors and small integers: it is what rank 0 hands
to its own runner and ships to the tensor-parallel workers, so workers never need
``Sequence`` objects.  Slot mappings and context lengths use *physical* KV positions
(after compaction), M-RoPE positions use logical ones.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import numpy as np
import torch

from .contracts import BatchPlan, Phase
from .sequence import Sequence


def _pack_tensor(t: Optional[torch.Tensor]):
    """Tensor -> picklable (numpy array, torch dtype name).  The default tensor pickle goes through
    torch's storage serialisation (about 50 us per tensor each way); a numpy array is a memcpy,
    which matters because these objects cross the tensor-parallel control plane every step."""
    if t is None:
        return None
    t = t.detach().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy(), "bfloat16"
    return t.numpy(), None


def _unpack_tensor(packed) -> Optional[torch.Tensor]:
    if packed is None:
        return None
    arr, special = packed
    t = torch.from_numpy(arr)
    return t.view(torch.bfloat16) if special == "bfloat16" else t


class _TensorStatePickle:
    """Mixin: dataclass fields holding CPU tensors travel as numpy arrays."""

    def __getstate__(self):
        return {k: (("__tensor__", _pack_tensor(v)) if isinstance(v, torch.Tensor) else v) for k, v in self.__dict__.items()}

    def __setstate__(self, state):
        for k, v in state.items():
            if isinstance(v, tuple) and len(v) == 2 and isinstance(v[0], str) and v[0] == "__tensor__":
                v = _unpack_tensor(v[1])
            self.__dict__[k] = v


@dataclass
class VisionJob(_TensorStatePickle):
    """Patches one sequence still has to push through the vision tower."""

    seq_id: int
    pixel_values: torch.Tensor            # [N, patch_dim]
    grid_thw: list[tuple[int, int, int]]
    cache_key: Optional[str] = None


@dataclass
class StepInputs(_TensorStatePickle):
    kind: str                              # "prefill" | "decode"
    input_ids: torch.Tensor                # [T] int64
    positions: torch.Tensor                # [3, T] int32
    slots: torch.Tensor                    # [T] int64
    block_tables: torch.Tensor             # [S, max_blocks] int32
    temperatures: torch.Tensor             # [S] fp32 (0 = greedy)
    # prefill only
    cu_seqlens_q: Optional[torch.Tensor] = None   # [S+1] int32
    kv_lens: Optional[torch.Tensor] = None        # [S] int32
    max_q_len: int = 0
    sample_rows: Optional[torch.Tensor] = None    # [n] int64 flattened row of each finishing sequence
    sample_seq: list[int] = field(default_factory=list)   # index into the plan of those sequences
    vis_index: Optional[torch.Tensor] = None      # [T] int32
    vision_jobs: list[VisionJob] = field(default_factory=list)
    vision_rows: list[tuple[int, int, int]] = field(default_factory=list)  # (seq_id, first row, rows) in vis order
    release_visual: list[int] = field(default_factory=list)
    # attention pruning strategy: (seq_id, first row, rows, visual token indices) of the sequences to score
    score_rows: list[tuple[int, int, int, tuple[int, ...]]] = field(default_factory=list)
    score_layers: list[int] = field(default_factory=list)
    # decode only
    context_lens: Optional[torch.Tensor] = None   # [B] int32

    # ---- fixed binary form of a decode step for the tensor-parallel command channel ----------
    # int64 words [batch, table width, 0, 0 | ids[B] | slots[B]] followed by int32 words
    # [positions[3B] | context_lens[B] | temperature bits[B] | block_tables[B * W]].  A decode step
    # is sent every few milliseconds; pickling its six small tensors costs about 80 us per step
    # (write + read), this form a tenth of that, and the workers start their step that much sooner.
    def pack_decode(self, area: memoryview) -> int:
        """Write the step into ``area``; returns the bytes used, or 0 when this step does not fit
        the fixed form (not a decode step, unexpected dtypes, area too small)."""
        if self.kind != "decode" or self.context_lens is None or self.block_tables.dim() != 2:
            return 0
        B, W = (int(v) for v in self.block_tables.shape)
        want = ((self.input_ids, torch.int64, B), (self.slots, torch.int64, B), (self.positions, torch.int32, 3 * B),
                (self.context_lens, torch.int32, B), (self.temperatures, torch.float32, B), (self.block_tables, torch.int32, B * W))
        if any(t.dtype != d or t.numel() != n or t.device.type != "cpu" for t, d, n in want):
            return 0
        n64 = 4 + 2 * B
        total = n64 * 8 + 4 * (5 * B + B * W)
        if total > len(area):
            return 0
        a64 = np.ndarray((n64,), dtype=np.int64, buffer=area)
        a64[0], a64[1], a64[2], a64[3] = B, W, 0, 0
        a64[4:4 + B] = self.input_ids.numpy()
        a64[4 + B:] = self.slots.numpy()
        a32 = np.ndarray((5 * B + B * W,), dtype=np.int32, buffer=area, offset=n64 * 8)
        a32[:3 * B] = self.positions.contiguous().numpy().reshape(-1)
        a32[3 * B:4 * B] = self.context_lens.numpy()
        a32[4 * B:5 * B] = self.temperatures.numpy().view(np.int32)
        a32[5 * B:] = self.block_tables.contiguous().numpy().reshape(-1)
        return total

    @classmethod
    def unpack_decode(cls, area: memoryview) -> "StepInputs":
        head = np.ndarray((4,), dtype=np.int64, buffer=area)
        B, W = int(head[0]), int(head[1])
        n64 = 4 + 2 * B
        a64 = np.array(np.ndarray((n64,), dtype=np.int64, buffer=area))  # copies: the area is reused
        a32 = np.array(np.ndarray((5 * B + B * W,), dtype=np.int32, buffer=area, offset=n64 * 8))
        return cls(kind="decode", input_ids=torch.from_numpy(a64[4:4 + B]), positions=torch.from_numpy(a32[:3 * B].reshape(3, B)),
                   slots=torch.from_numpy(a64[4 + B:]), block_tables=torch.from_numpy(a32[5 * B:].reshape(B, W)),
                   temperatures=torch.from_numpy(a32[4 * B:5 * B].view(np.float32)), context_lens=torch.from_numpy(a32[3 * B:4 * B]))

    @property
    def num_tokens(self) -> int:
        return int(self.input_ids.shape[0])

    @property
    def num_seqs(self) -> int:
        return int(self.block_tables.shape[0])


class ModelInputPreparer:
    def __init__(self, page: int, max_blocks: int) -> None:
        self.page = page
        self.max_blocks = max_blocks

    def _block_table(self, seqs: tuple[Sequence, ...]) -> torch.Tensor:
        width = max(1, max(len(s.block_table) for s in seqs))
        bt = np.full((len(seqs), width), -1, dtype=np.int32)
        for i, s in enumerate(seqs):
            table = s.block_table
            if table:
                bt[i, : len(table)] = table
        return torch.from_numpy(bt)

    def prepare(self, plan: BatchPlan, have_visual: set[int] | None = None) -> StepInputs:
        if plan.phase is Phase.PREFILL:
            return self.prepare_prefill(plan, have_visual or set())
        return self.prepare_decode(plan)

    def prepare_prefill(self, plan: BatchPlan, have_visual: set[int]) -> StepInputs:
        """Flattened ids, M-RoPE positions, flat KV slots and the visual-row index of every token,
        built per sequence with array arithmetic (a 1600-token prompt costs about 0.1 ms here; a
        Python loop over its tokens cost 1.2 ms of the time to first token)."""
        ids_parts: list[np.ndarray] = []
        pos_parts: list[torch.Tensor] = []
        slot_parts: list[np.ndarray] = []
        vis_parts: list[np.ndarray] = []
        cu = [0]
        kv_lens: list[int] = []
        sample_rows: list[int] = []
        sample_seq: list[int] = []
        vision_jobs: list[VisionJob] = []
        vision_rows: list[tuple[int, int, int]] = []
        release: list[int] = []
        vis_cursor = 0
        any_visual = False
        for i, (seq, sl) in enumerate(zip(plan.seqs, plan.slices)):
            start, end = sl.start, sl.end
            toks = np.asarray(seq.token_ids[start:end], dtype=np.int64)
            ids_parts.append(toks)
            pos_parts.append(seq.positions_for(start, end))
            bs = seq.block_size
            phys = np.arange(start - seq.dropped_tokens, end - seq.dropped_tokens, dtype=np.int64)
            table = np.asarray(seq.block_table, dtype=np.int64)
            slot_parts.append(table[phys // bs] * bs + phys % bs)
            cu.append(cu[-1] + sl.length)
            kv_lens.append(seq.physical_len(end))
            if end == len(seq):
                sample_rows.append(cu[-1] - 1)
                sample_seq.append(i)
            lo, hi = seq.visual_index_range(start, end) if seq.is_multimodal else (0, 0)
            vis = np.full(sl.length, -1, dtype=np.int32)
            if hi > lo:
                any_visual = True
                if seq.seq_id not in have_visual and seq.pixel_values is not None:
                    grids = list(seq.image_grid_thw) + list(seq.video_grid_thw)
                    vision_jobs.append(VisionJob(seq.seq_id, seq.pixel_values, grids, seq.visual_embedding_cache_key))
                vision_rows.append((seq.seq_id, lo, hi - lo))
                is_visual = (toks == seq.image_token_id) | (toks == seq.video_token_id)
                count = int(is_visual.sum())
                vis[is_visual] = np.arange(vis_cursor, vis_cursor + count, dtype=np.int32)
                vis_cursor += count
            vis_parts.append(vis)
            if seq.is_multimodal and end >= seq.multimodal_prefix_boundary:
                release.append(seq.seq_id)
        temps = torch.tensor([plan.seqs[i].temperature for i in sample_seq], dtype=torch.float32)
        cat = lambda parts: torch.from_numpy(parts[0] if len(parts) == 1 else np.concatenate(parts))  # noqa: E731
        return StepInputs(
            kind="prefill",
            input_ids=cat(ids_parts),
            positions=torch.cat(pos_parts, dim=1).to(torch.int32).contiguous(),
            slots=cat(slot_parts),
            block_tables=self._block_table(plan.seqs),
            temperatures=temps,
            cu_seqlens_q=torch.tensor(cu, dtype=torch.int32),
            kv_lens=torch.tensor(kv_lens, dtype=torch.int32),
            max_q_len=max(s.length for s in plan.slices),
            sample_rows=torch.tensor(sample_rows, dtype=torch.int64),
            sample_seq=sample_seq,
            vis_index=cat(vis_parts) if any_visual else None,
            vision_jobs=vision_jobs,
            vision_rows=vision_rows,
            release_visual=release,
        )

    def prepare_decode(self, plan: BatchPlan) -> StepInputs:
        """One pass over the sequences into numpy rows (a decode step of 128 sequences is host-bound
        work of a few hundred microseconds; per-element ``torch.tensor`` calls would double it)."""
        seqs = plan.seqs
        n = len(seqs)
        ids = np.empty(n, dtype=np.int64)
        pos = np.empty(n, dtype=np.int32)
        slots = np.empty(n, dtype=np.int64)
        ctx = np.empty(n, dtype=np.int32)
        temps = np.empty(n, dtype=np.float32)
        for i, s in enumerate(seqs):
            toks = s.token_ids
            length = len(toks)
            phys = length - 1 - s.dropped_tokens
            bs = s.block_size
            ids[i] = toks[-1]
            pos[i] = length - 1 + s.rope_delta
            slots[i] = s.block_table[phys // bs] * bs + phys % bs
            ctx[i] = phys + 1
            temps[i] = s.temperature
        return StepInputs(
            kind="decode",
            input_ids=torch.from_numpy(ids),
            positions=torch.from_numpy(np.ascontiguousarray(np.broadcast_to(pos, (3, n)))),
            slots=torch.from_numpy(slots),
            block_tables=self._block_table(seqs),
            temperatures=torch.from_numpy(temps),
            context_lens=torch.from_numpy(ctx),
        )
