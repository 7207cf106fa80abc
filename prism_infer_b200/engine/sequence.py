"""Mutable per-request state (reference ``prism_infer/engine/sequence.py:19-567``).

Holds the tokens, the GPU / CPU page tables, chunked-prefill progress, the multimodal
payload (patch pixels and grids), the three-axis position ids and ``rope_delta``, cache
keys and, after compaction, the logical-to-physical KV layout.
"""

from __future__ import annotations

from typing import Any, Sequence as Seq

import torch

from ..sampling_params import SamplingParams
from .kv_layout import KVLayout
from .request import RequestLifecycle, RequestState
from .visual_pruning import VisualSpan, find_visual_spans


class Sequence:
    block_size = 256

    def __init__(
        self,
        seq_id: int,
        token_ids: Seq[int],
        sampling_params: SamplingParams | None = None,
        *,
        image_token_id: int = -1,
        video_token_id: int = -1,
        pixel_values: torch.Tensor | None = None,
        image_grid_thw: Seq[Seq[int]] | None = None,
        video_grid_thw: Seq[Seq[int]] | None = None,
        position_ids: torch.Tensor | None = None,
        rope_delta: int = 0,
        merge_size: int = 2,
    ) -> None:
        sp = sampling_params or SamplingParams()
        self.seq_id = seq_id
        self.token_ids = [int(t) for t in token_ids]
        if not self.token_ids:
            raise ValueError("a sequence needs at least one prompt token")
        self.num_prompt_tokens = len(self.token_ids)
        self.temperature = float(sp.temperature)
        self.max_tokens = int(sp.max_tokens)
        self.ignore_eos = bool(sp.ignore_eos)
        self.lifecycle = RequestLifecycle(seq_id)
        self.block_table: list[int] = []
        self.cpu_block_table: list[int] = []
        self.block_table_version = 0
        self.num_computed_tokens = 0      # logical tokens whose KV exists
        self.num_cached_tokens = 0        # logical tokens served from a cache at admission
        self.kv_layout: KVLayout | None = None
        # (page index, chain hash, token ids) of own full prompt pages whose content hash may be
        # published to the prefix index once the prefill chunk that fills the page has run
        self.unpublished_hashes: list[tuple[int, int, tuple[int, ...]]] = []
        self.image_token_id, self.video_token_id = image_token_id, video_token_id
        self.merge_size = merge_size
        self.pixel_values = pixel_values
        self.image_grid_thw = [tuple(int(x) for x in r) for r in image_grid_thw] if image_grid_thw is not None else []
        self.video_grid_thw = [tuple(int(x) for x in r) for r in video_grid_thw] if video_grid_thw is not None else []
        self.position_ids = position_ids  # [3, S] int64 CPU, prompt only
        self.rope_delta = int(rope_delta)
        self.multimodal_prefix_cache_key: str | None = None
        self.visual_embedding_cache_key: str | None = None
        self.visual_embeds: Any = None     # (main, [deepstack...]) once computed / cached
        self.arrival_ns: int | None = None
        self.deadline_ns: int | None = None
        self.pruning_record: dict | None = None
        self._spans: tuple[VisualSpan, ...] | None = None

    # ---------------------------------------------------------------- basic views
    def __len__(self) -> int:
        return len(self.token_ids)

    @property
    def state(self) -> RequestState:
        return self.lifecycle.state

    @property
    def is_finished(self) -> bool:
        return self.lifecycle.state.terminal

    @property
    def num_completion_tokens(self) -> int:
        return len(self.token_ids) - self.num_prompt_tokens

    @property
    def completion_token_ids(self) -> list[int]:
        return self.token_ids[self.num_prompt_tokens:]

    @property
    def last_token(self) -> int:
        return self.token_ids[-1]

    @property
    def is_multimodal(self) -> bool:
        return self.pixel_values is not None or bool(self.image_grid_thw) or bool(self.video_grid_thw)

    def append_token(self, token: int) -> None:
        self.token_ids.append(int(token))

    # ------------------------------------------------------------ physical KV geometry
    @property
    def dropped_tokens(self) -> int:
        return self.kv_layout.dropped if self.kv_layout is not None else 0

    def physical_len(self, logical_len: int | None = None) -> int:
        n = len(self.token_ids) if logical_len is None else logical_len
        return n - self.dropped_tokens

    @property
    def physical_computed(self) -> int:
        return self.num_computed_tokens - self.dropped_tokens if self.num_computed_tokens else 0

    def blocks_needed(self, logical_len: int | None = None) -> int:
        return -(-self.physical_len(logical_len) // self.block_size)

    def slot_of(self, logical_index: int) -> int:
        """Flat slot of a token at or beyond any compacted prefix."""
        phys = logical_index - self.dropped_tokens
        return self.block_table[phys // self.block_size] * self.block_size + phys % self.block_size

    # ------------------------------------------------------------------- multimodal
    @property
    def visual_spans(self) -> tuple[VisualSpan, ...]:
        if self._spans is None:
            self._spans = find_visual_spans(self.token_ids[: self.num_prompt_tokens], self.image_token_id, self.video_token_id)
        return self._spans

    @property
    def num_visual_tokens(self) -> int:
        return sum(s.count for s in self.visual_spans)

    @property
    def multimodal_prefix_boundary(self) -> int:
        """Prompt index right after the last visual placeholder (0 when there is none):
        everything before it is question-independent for a media-first prompt."""
        spans = self.visual_spans
        return spans[-1].end if spans else 0

    def vision_patch_count(self, start: int = 0, end: int | None = None) -> int:
        """Vision patches whose placeholder tokens fall in ``[start, end)``."""
        end = self.num_prompt_tokens if end is None else end
        unit = self.merge_size * self.merge_size
        return sum(max(0, min(s.end, end) - max(s.start, start)) for s in self.visual_spans) * unit

    def visual_index_range(self, start: int, end: int) -> tuple[int, int]:
        """Rows of the visual-embedding matrix consumed by prompt tokens ``[start, end)``."""
        before = sum(max(0, min(s.end, start) - s.start) for s in self.visual_spans if s.start < start)
        inside = sum(max(0, min(s.end, end) - max(s.start, start)) for s in self.visual_spans)
        return before, before + inside

    def positions_for(self, start: int, end: int) -> torch.Tensor:
        """``[3, end - start]`` int64 M-RoPE positions for logical tokens ``[start, end)``."""
        n_prompt = self.num_prompt_tokens
        parts = []
        if start < n_prompt:
            hi = min(end, n_prompt)
            if self.position_ids is not None:
                parts.append(self.position_ids[:, start:hi])
            else:
                parts.append(torch.arange(start, hi, dtype=torch.int64).expand(3, -1))
        if end > n_prompt:
            lo = max(start, n_prompt)
            parts.append((torch.arange(lo, end, dtype=torch.int64) + self.rope_delta).expand(3, -1))
        return parts[0] if len(parts) == 1 else torch.cat(parts, dim=1)

    # ---------------------------------------------------------------------- pickling
    def __getstate__(self) -> dict:
        """Compact wire form: decode steps ship only the last token, never pixels."""
        st = dict(self.__dict__)
        st["_spans"] = None
        st["visual_embeds"] = None
        if self.lifecycle.state is RequestState.DECODING:
            st["token_ids"] = None
            st["_wire_len"] = len(self.token_ids)
            st["_wire_last"] = self.token_ids[-1]
            st["pixel_values"] = None
            st["position_ids"] = None
        return st

    def __setstate__(self, st: dict) -> None:
        self.__dict__.update(st)
        if st.get("token_ids") is None:
            n, last = st["_wire_len"], st["_wire_last"]
            self.token_ids = [0] * (n - 1) + [last]
