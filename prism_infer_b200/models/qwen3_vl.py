"""Qwen3-VL as the engine runs it: packed, tensor-parallel weights and a forward built
only from ``prism_infer_b200.ops``.

Storage: per decoder layer one packed ``qkv`` matrix ``[(Hq + 2 Hkv) D / tp, H]`` (rank-local
heads), ``o`` ``[H, Hq D / tp]``, one packed ``gate_up`` ``[2 I / tp, H]`` (gate rows then up
rows, consumed by the dual-accumulator GEMM) and ``down`` ``[H, I / tp]``; embedding and LM
head are vocabulary-sharded.  Checkpoints keep their Hugging Face names; ``load`` routes
``q_proj / k_proj / v_proj`` and ``gate_proj / up_proj`` into the packed tensors (reference
``prism_infer/models/qwen3_vl.py:184-250,1572-1601`` and ``prism_infer/layers/linear.py:47-190``).

Forward (reference hot loop ``prism_infer/models/qwen3_vl.py:925-1022``): every layer is
add+RMSNorm -> QKV GEMM -> QK-norm + M-RoPE + KV store -> paged attention -> o_proj ->
add+RMSNorm -> dual GEMM with SwiGLU -> down_proj, with the residual carried separately and
DeepStack features added after layers 0..k-1.  Row-parallel projections produce fp32
partial slabs (split-K and, under tensor parallelism, one group per rank) that the next
add+RMSNorm sums in a fixed order.
"""

from __future__ import annotations

import math

from dataclasses import dataclass, field
from typing import Iterable, Iterator, Optional, Sequence

import torch

from .. import ops
from .architecture import Qwen3VLArch
from .position import vision_patch_coords, vision_pos_embed_plan, vision_segments
from .weights import LM, VIS

# at or below this many tokens the GEMMs are weight-streaming: split-K + fp32 partials
SMALL_T = 128


@dataclass
class AttnMeta:
    """Device-side attention metadata of one step."""

    is_prefill: bool
    block_tables: torch.Tensor                     # [S, max_blocks] int32
    slots: torch.Tensor                            # [T] int64 flat KV slots of the new tokens
    # prefill
    cu_seqlens_q: Optional[torch.Tensor] = None    # [S+1] int32
    kv_lens: Optional[torch.Tensor] = None         # [S] int32 keys visible (history + chunk)
    cu_seqlens_kv: Optional[torch.Tensor] = None   # [S+1] int32 running sum of kv_lens (None: the page-reading kernel)
    total_kv: int = 0                              # sum and maximum of kv_lens, known on the host
    max_kv_len: int = 0
    max_q_len: int = 0
    last_rows: Optional[torch.Tensor] = None       # [S] int64 row of each sequence's last token
    no_history: bool = False                       # every sequence attends only to this chunk's own keys
    # decode
    context_lens: Optional[torch.Tensor] = None    # [B] int32 (including the new token)
    nsplit: int = 0
    workspace: Optional[tuple[torch.Tensor, torch.Tensor]] = None
    # prefill with the attention pruning strategy: collects last-query attention over visual tokens
    scorer: Optional[object] = None


@dataclass
class VisionTowerState:
    """A vision-tower pass between blocks (``Qwen3VLModel.begin_vision / advance_vision / finish_vision``)."""

    x: torch.Tensor                  # [patches, vision hidden] after ``next_block`` blocks
    coords: torch.Tensor
    cu: torch.Tensor
    max_len: int
    comm: object = None              # tensor-parallel ranks: the communicator whose all-gather the mergers feed
    token_base: int = 0
    next_block: int = 0
    deep: list = field(default_factory=list)


@dataclass
class LayerWeights:
    input_norm: torch.Tensor
    qkv: torch.Tensor
    q_norm: torch.Tensor
    k_norm: torch.Tensor
    o: torch.Tensor
    post_norm: torch.Tensor
    gate_up: torch.Tensor
    down: torch.Tensor


@dataclass
class VisionBlockWeights:
    norm1_w: torch.Tensor
    norm1_b: torch.Tensor
    qkv_w: torch.Tensor
    qkv_b: torch.Tensor
    proj_w: torch.Tensor
    proj_b: torch.Tensor
    norm2_w: torch.Tensor
    norm2_b: torch.Tensor
    fc1_w: torch.Tensor
    fc1_b: torch.Tensor
    fc2_w: torch.Tensor
    fc2_b: torch.Tensor


@dataclass
class MergerWeights:
    norm_w: torch.Tensor
    norm_b: torch.Tensor
    fc1_w: torch.Tensor
    fc1_b: torch.Tensor
    fc2_w: torch.Tensor
    fc2_b: torch.Tensor
    post_norm: bool = False


@dataclass
class LayerwiseState:
    """What the layer loop carries from one layer to the next: the pending output of the last row-parallel projection
    (dense rows, split-K slabs or an exchange ticket), the residual, and the step's inputs."""

    positions: torch.Tensor
    meta: "AttnMeta"
    cache: "ops.KVCache"
    vis_index: Optional[torch.Tensor]
    deepstack: Optional[Sequence[torch.Tensor]]
    tokens: int
    small: bool
    scoring: bool
    dense: Optional[torch.Tensor] = None
    partials: Optional[torch.Tensor] = None
    ticket: object = None
    residual: Optional[torch.Tensor] = None
    next_layer: int = 0


class TPComm:
    """Collective hooks of a tensor-parallel rank; the single-rank default does nothing."""

    rank = 0
    size = 1

    def reduce_partials(self, partials: torch.Tensor) -> torch.Tensor:
        """fp32 ``[S, T, H]`` rank-local partial slabs -> slabs whose sum is the full result."""
        return partials

    def reduce_dense(self, x: torch.Tensor) -> torch.Tensor:
        """bf16 ``[T, H]`` rank-local partial result -> summed over ranks."""
        return x

    def greedy_merge(self, local_val: torch.Tensor, local_id: torch.Tensor) -> torch.Tensor:
        return local_id

    def gather_logits(self, logits: torch.Tensor) -> torch.Tensor:
        return logits

    def all_gather_rows(self, x: torch.Tensor) -> torch.Tensor:
        return x

    def begin_step(self) -> None:
        return None

    def row_parallel(self, x: torch.Tensor, w: torch.Tensor, stages: int = 0):
        """Row-parallel projection -> ``(dense, partials, ticket)``; exactly one is set.
        ``stages`` caps the operand ring of a decode-sized launch (0 = as deep as fits)."""
        T = x.shape[0]
        # short prefills (up to 511 tokens) split K too: o_proj and down_proj have 32 weight tiles at 8B widths,
        # one CTA each would leave 116 SMs idle
        if T <= SMALL_T or (x.is_cuda and T <= ops.SPLIT_K_MAX_TOKENS):
            splits = ops.choose_splits(w.shape[0], w.shape[1], T) if x.is_cuda else 1
            if splits > 1 or T <= SMALL_T:
                return None, ops.linear_partial(x, w, splits, stages=stages), None
        return ops.linear(x, w), None, None

    def add_rmsnorm(self, weight, eps, dense, partials, ticket, residual, extra=None, extra_index=None):
        """``(normed, new_residual)`` from whatever ``row_parallel`` returned."""
        return ops.add_rmsnorm(weight, eps, x=dense, partials=partials, residual=residual, extra=extra,
                               extra_index=extra_index)


class Qwen3VLModel:
    def __init__(self, arch: Qwen3VLArch, *, device, dtype: torch.dtype, comm: TPComm | None = None,
                 load_vision: bool = True) -> None:
        self.arch = arch
        self.device = torch.device(device)
        self.dtype = dtype
        self.comm = comm or TPComm()
        self.tp, self.rank = self.comm.size, self.comm.rank
        t = arch.text
        self.Hq, self.Hkv = t.num_heads // self.tp, t.num_kv_heads // self.tp
        self.D, self.H, self.I = t.head_dim, t.hidden_size, t.intermediate_size // self.tp
        self.V = t.vocab_size // self.tp
        self.vocab_start = self.rank * self.V
        self.load_vision = load_vision
        self._alloc()

    # ------------------------------------------------------------------- storage
    def _e(self, *shape: int) -> torch.Tensor:
        return torch.empty(shape, dtype=self.dtype, device=self.device)

    def _alloc(self) -> None:
        a, t, v = self.arch, self.arch.text, self.arch.vision
        qkv_rows = (self.Hq + 2 * self.Hkv) * self.D
        # the embedding table is replicated on every rank (1.2 GB at 8B widths): a lookup needs no exchange, where
        # the reference all-reduces vocabulary-sharded rows (prism_infer/layers/embed_head.py:49-74); the LM head
        # stays sharded by vocabulary rows
        self.embed = self._e(t.vocab_size, self.H)
        self.lm_head = self.embed[self.vocab_start:self.vocab_start + self.V] if t.tie_word_embeddings else self._e(self.V, self.H)
        self.final_norm = self._e(self.H)
        self.layers = [
            LayerWeights(self._e(self.H), self._e(qkv_rows, self.H), self._e(self.D), self._e(self.D),
                         self._e(self.H, self.Hq * self.D), self._e(self.H), self._e(2 * self.I, self.H),
                         self._e(self.H, self.I))
            for _ in range(t.num_layers)
        ]
        self.vision_blocks: list[VisionBlockWeights] = []
        self.mergers: dict[str, MergerWeights] = {}
        if self.load_vision:
            vh, vi = v.hidden_size, v.intermediate_size
            self.patch_w, self.patch_b = self._e(vh, v.patch_input_dim), self._e(vh)
            self.pos_embed = self._e(v.num_position_embeddings, vh)
            self.vision_blocks = [
                VisionBlockWeights(self._e(vh), self._e(vh), self._e(3 * vh, vh), self._e(3 * vh), self._e(vh, vh),
                                   self._e(vh), self._e(vh), self._e(vh), self._e(vi, vh), self._e(vi),
                                   self._e(vh, vi), self._e(vh))
                for _ in range(v.depth)
            ]
            md = v.merged_dim

            def merger(norm_dim: int, post: bool) -> MergerWeights:
                return MergerWeights(self._e(norm_dim), self._e(norm_dim), self._e(md, md), self._e(md),
                                     self._e(v.out_hidden_size, md), self._e(v.out_hidden_size), post)

            self.mergers["main"] = merger(vh, False)
            for k in range(len(v.deepstack_visual_indexes)):
                self.mergers[f"deepstack.{k}"] = merger(md, True)
            hd = v.head_dim
            self.vit_inv_freq = (1.0 / (v.rope_theta ** (torch.arange(0, hd // 2, 2, dtype=torch.float32) / (hd // 2)))).to(self.device)

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for t in self._all_tensors():
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        return total

    def _all_tensors(self) -> Iterator[torch.Tensor]:
        yield self.embed
        yield self.lm_head
        yield self.final_norm
        for l in self.layers:
            yield from (l.input_norm, l.qkv, l.q_norm, l.k_norm, l.o, l.post_norm, l.gate_up, l.down)
        if self.load_vision:
            yield from (self.patch_w, self.patch_b, self.pos_embed)
            for b in self.vision_blocks:
                yield from b.__dict__.values()
            for m in self.mergers.values():
                yield from (m.norm_w, m.norm_b, m.fc1_w, m.fc1_b, m.fc2_w, m.fc2_b)

    # ------------------------------------------------------------------- loading
    def _route(self, name: str) -> tuple[torch.Tensor, Optional[tuple[int, int, int]]] | None:
        """HF name -> (destination view, (dim, start, length) slice of the checkpoint tensor)."""
        r, D = self.rank, self.D
        if name.startswith(f"{LM}.layers."):
            rest = name[len(f"{LM}.layers."):]
            idx, sub = rest.split(".", 1)
            l = self.layers[int(idx)]
            q_rows, kv_rows = self.Hq * D, self.Hkv * D
            table = {
                "input_layernorm.weight": (l.input_norm, None),
                "post_attention_layernorm.weight": (l.post_norm, None),
                "self_attn.q_norm.weight": (l.q_norm, None),
                "self_attn.k_norm.weight": (l.k_norm, None),
                "self_attn.q_proj.weight": (l.qkv[:q_rows], (0, r * q_rows, q_rows)),
                "self_attn.k_proj.weight": (l.qkv[q_rows:q_rows + kv_rows], (0, r * kv_rows, kv_rows)),
                "self_attn.v_proj.weight": (l.qkv[q_rows + kv_rows:], (0, r * kv_rows, kv_rows)),
                "self_attn.o_proj.weight": (l.o, (1, r * q_rows, q_rows)),
                "mlp.gate_proj.weight": (l.gate_up[: self.I], (0, r * self.I, self.I)),
                "mlp.up_proj.weight": (l.gate_up[self.I:], (0, r * self.I, self.I)),
                "mlp.down_proj.weight": (l.down, (1, r * self.I, self.I)),
            }
            return table.get(sub)
        if name == f"{LM}.embed_tokens.weight":
            return self.embed, None
        if name == "lm_head.weight":
            return (None if self.arch.text.tie_word_embeddings else (self.lm_head, (0, r * self.V, self.V)))
        if name == f"{LM}.norm.weight":
            return self.final_norm, None
        if not self.load_vision or not name.startswith(VIS):
            return None
        if name == f"{VIS}.patch_embed.proj.weight":
            return self.patch_w, None
        if name == f"{VIS}.patch_embed.proj.bias":
            return self.patch_b, None
        if name == f"{VIS}.pos_embed.weight":
            return self.pos_embed, None
        if name.startswith(f"{VIS}.blocks."):
            rest = name[len(f"{VIS}.blocks."):]
            idx, sub = rest.split(".", 1)
            b = self.vision_blocks[int(idx)]
            table = {
                "norm1.weight": b.norm1_w, "norm1.bias": b.norm1_b, "norm2.weight": b.norm2_w, "norm2.bias": b.norm2_b,
                "attn.qkv.weight": b.qkv_w, "attn.qkv.bias": b.qkv_b, "attn.proj.weight": b.proj_w,
                "attn.proj.bias": b.proj_b, "mlp.linear_fc1.weight": b.fc1_w, "mlp.linear_fc1.bias": b.fc1_b,
                "mlp.linear_fc2.weight": b.fc2_w, "mlp.linear_fc2.bias": b.fc2_b,
            }
            dst = table.get(sub)
            return None if dst is None else (dst, None)
        for key, prefix in [("main", f"{VIS}.merger.")] + [
            (f"deepstack.{k}", f"{VIS}.deepstack_merger_list.{k}.") for k in range(len(self.arch.vision.deepstack_visual_indexes))
        ]:
            if name.startswith(prefix):
                m = self.mergers[key]
                table = {"norm.weight": m.norm_w, "norm.bias": m.norm_b, "linear_fc1.weight": m.fc1_w,
                         "linear_fc1.bias": m.fc1_b, "linear_fc2.weight": m.fc2_w, "linear_fc2.bias": m.fc2_b}
                dst = table.get(name[len(prefix):])
                return None if dst is None else (dst, None)
        return None

    def load(self, tensors: Iterable[tuple[str, torch.Tensor]], *, strict: bool = True) -> None:
        """Copy (and shard) checkpoint tensors into the packed storage."""
        from .weights import weight_shapes

        expected = set(weight_shapes(self.arch))
        if not self.load_vision:
            expected = {n for n in expected if not n.startswith(VIS)}
        seen: set[str] = set()
        for name, tensor in tensors:
            routed = self._route(name)
            if routed is None:
                if name in expected and not (name == "lm_head.weight" and self.arch.text.tie_word_embeddings):
                    if self.load_vision or not name.startswith(VIS):
                        raise KeyError(f"no destination for checkpoint tensor {name}")
                continue
            dst, sl = routed
            src = tensor
            if sl is not None:
                src = src.narrow(sl[0], sl[1], sl[2])
            src = src.reshape(dst.shape) if src.numel() == dst.numel() else src
            if src.shape != dst.shape:
                raise ValueError(f"{name}: checkpoint shape {tuple(tensor.shape)} does not fit {tuple(dst.shape)}")
            dst.copy_(src.to(device=self.device, dtype=self.dtype, non_blocking=True))
            seen.add(name)
        if strict:
            missing = expected - seen
            if self.arch.text.tie_word_embeddings:
                missing.discard("lm_head.weight")
            if missing:
                raise KeyError(f"checkpoint is missing {len(missing)} tensors, e.g. {sorted(missing)[:3]}")

    # -------------------------------------------------------------------- vision
    @torch.no_grad()
    def vision_shard_rows(self, grid_thw: Sequence[Sequence[int]]) -> Optional[tuple[int, int]]:
        """``(first patch row, patch rows)`` this rank runs the vision blocks on when the tower is split over the
        ranks, or ``None`` when every rank runs all of it.  A caller that holds the patches on the host can then
        upload its own rows only and pass them to ``encode_vision(..., local_rows=...)``."""
        grid = [tuple(int(x) for x in g) for g in grid_thw]
        total_tokens = sum(t * h * w for t, h, w in grid) // self.arch.vision.merge_unit
        if not (self.tp > 1 and hasattr(self.comm, "vision_begin") and self.device.type == "cuda" and total_tokens <= self.comm.vision_capacity()):
            return None
        start, rows, _ = self._vision_shards(grid)[self.rank]
        return start, rows

    def encode_vision(self, pixel_values: torch.Tensor, grid_thw: Sequence[Sequence[int]], *,
                      local_rows: Optional[tuple[int, int]] = None) -> tuple[torch.Tensor, list[torch.Tensor]]:
        """``pixel_values [N, C*Tp*P*P]`` -> merged visual tokens ``[N/4, H]`` and one
        DeepStack feature tensor per tap, identical on every rank.

        Tensor-parallel ranks with the fused communicator split the work by attention
        segment (one image or one temporal group each): every rank runs the blocks on its
        own segments only and the merger's last GEMM writes its rows into every rank's
        gathered output from its epilogue (fused merger GEMM -> all-gather).  The reference
        replicates the whole tower on every rank (``docs/ARCHITECTURE.md:83``).
        """
        grid = [tuple(int(x) for x in g) for g in grid_thw]
        unit = self.arch.vision.merge_unit
        total_tokens = sum(t * h * w for t, h, w in grid) // unit
        comm = self.comm
        if self.tp > 1 and pixel_values.device.type != "meta" and hasattr(comm, "vision_begin") and self.device.type == "cuda" \
                and comm.vision_begin(total_tokens):
            return self._encode_vision_sharded(pixel_values, grid, total_tokens, local_rows)
        if local_rows is not None:
            raise ValueError("local_rows is only meaningful when the tower is split over the ranks (see vision_shard_rows)")
        main, deep = self._vision_tower(pixel_values, grid, None, 0)
        return main, deep

    def _vision_shards(self, grid: list[tuple[int, int, int]]) -> list[tuple[int, int, list[tuple[int, int, int]]]]:
        """Contiguous, patch-balanced assignment of (item, temporal group) segments to ranks:
        per rank ``(first patch row, patch rows, sub-grid)``."""
        segs = [(h * w, (1, h, w)) for t, h, w in grid for _ in range(t)]
        total = sum(n for n, _ in segs)
        out = []
        i, start = 0, 0
        for r in range(self.tp):
            want_end = total * (r + 1) / self.tp
            rows, sub = 0, []
            while i < len(segs) and (start + rows + segs[i][0] / 2 <= want_end or (r == self.tp - 1)):
                rows += segs[i][0]
                g = segs[i][1]
                if sub and sub[-1][1:] == g[1:]:
                    sub[-1] = (sub[-1][0] + 1, g[1], g[2])  # consecutive frames of one clip
                else:
                    sub.append(g)
                i += 1
            out.append((start, rows, sub))
            start += rows
        return out

    def _encode_vision_sharded(self, pixel_values: torch.Tensor, grid, total_tokens: int, local_rows=None):
        comm = self.comm
        unit = self.arch.vision.merge_unit
        start, rows, sub = self._vision_shards(grid)[self.rank]
        n_out = 1 + len(self.arch.vision.deepstack_visual_indexes)
        if local_rows is not None:  # the caller uploaded this rank's rows only
            if tuple(local_rows) != (start, rows) or int(pixel_values.shape[0]) != rows:
                raise ValueError(f"local_rows {local_rows} with {int(pixel_values.shape[0])} rows does not match this rank's shard {(start, rows)}")
            mine = pixel_values
        else:
            mine = pixel_values[start:start + rows]
        if rows > 0:
            self._vision_tower(mine, sub, comm, start // unit)
        outs = comm.vision_finish(n_out, total_tokens)
        return outs[0], outs[1:]

    def _vision_geometry(self, grid):
        """Device tensors that depend only on the (t, h, w) grids of a call: position-embedding
        interpolation plan, rotary patch coordinates, attention segment offsets.  Serving
        repeats a handful of image shapes, so the last few results are kept."""
        key = tuple(tuple(int(v) for v in g) for g in grid)
        cache = self.__dict__.setdefault("_geometry_cache", {})
        hit = cache.get(key)
        if hit is not None:
            cache[key] = cache.pop(key)  # most recently used last
            return hit
        v, dev = self.arch.vision, self.device
        idx, wt = vision_pos_embed_plan(grid, v.grid_per_side, v.spatial_merge_size)
        coords = vision_patch_coords(grid, v.spatial_merge_size).to(torch.int32)
        segs = vision_segments(grid)
        cu = torch.tensor([0] + list(torch.tensor(segs).cumsum(0).tolist()), dtype=torch.int32)
        out = (idx.to(dev), wt.to(dev), coords.to(dev), cu.to(dev), max(segs))
        cache[key] = out
        while len(cache) > 32:
            cache.pop(next(iter(cache)))
        return out

    def _vision_tower(self, pixel_values: torch.Tensor, grid, comm, token_base: int):
        st = self._vision_begin(pixel_values, grid, comm, token_base)
        self.advance_vision(st, len(self.vision_blocks))
        return self.finish_vision(st)

    def _vision_begin(self, pixel_values: torch.Tensor, grid, comm, token_base: int) -> "VisionTowerState":
        dev = self.device
        x = ops.linear(pixel_values.to(device=dev, dtype=self.dtype, non_blocking=True), self.patch_w, bias=self.patch_b)
        idx, wt, coords, cu, max_len = self._vision_geometry(grid)
        ops.pos_embed_add(x, self.pos_embed, idx, wt)
        return VisionTowerState(x=x, coords=coords, cu=cu, max_len=max_len, comm=comm, token_base=token_base)

    def begin_vision(self, pixel_values: torch.Tensor, grid_thw: Sequence[Sequence[int]]) -> "VisionTowerState":
        """Patch embedding and position embedding of a vision-tower pass whose blocks ``advance_vision`` runs a few at a
        time (one rank; cooperative prefill lets decode steps of running sequences go in between; reference
        ``engine/model_runner.py:1346-1650`` vision-block quanta).  ``finish_vision`` gives what ``encode_vision`` returns."""
        if self.tp > 1:
            raise ValueError("the resumable vision tower runs on one rank")
        return self._vision_begin(pixel_values, [tuple(int(v) for v in g) for g in grid_thw], None, 0)

    def advance_vision(self, st: "VisionTowerState", max_blocks: int) -> bool:
        """Up to ``max_blocks`` more blocks (DeepStack taps are merged as their block completes); True when all have run."""
        v = self.arch.vision
        x = st.x
        N, vh, heads, hd = x.shape[0], v.hidden_size, v.num_heads, v.head_dim
        end = min(len(self.vision_blocks), st.next_block + max(0, int(max_blocks)))
        for i in range(st.next_block, end):
            b = self.vision_blocks[i]
            h = ops.layernorm(x, b.norm1_w, b.norm1_b, v.layer_norm_eps)
            qkv = ops.linear(h, b.qkv_w, bias=b.qkv_b)
            ops.vit_rope(qkv, st.coords, self.vit_inv_freq, heads, hd)
            q = qkv[:, :vh].view(N, heads, hd)
            k = qkv[:, vh:2 * vh].view(N, heads, hd)
            val = qkv[:, 2 * vh:].view(N, heads, hd)
            a = ops.varlen_attention(q, k, val, st.cu, st.max_len, causal=False)
            x = ops.linear(a.view(N, vh), b.proj_w, bias=b.proj_b, residual=x, out=x if x.is_cuda else None)
            h = ops.layernorm(x, b.norm2_w, b.norm2_b, v.layer_norm_eps)
            h = ops.linear(h, b.fc1_w, bias=b.fc1_b, act="gelu_tanh")
            x = ops.linear(h, b.fc2_w, bias=b.fc2_b, residual=x, out=x if x.is_cuda else None)
            if i in v.deepstack_visual_indexes:
                k_idx = v.deepstack_visual_indexes.index(i)
                st.deep.append(self._merge(x, self.mergers[f"deepstack.{k_idx}"], st.comm, 1 + k_idx, st.token_base))
        st.x, st.next_block = x, end
        return end == len(self.vision_blocks)

    def finish_vision(self, st: "VisionTowerState"):
        """Remaining blocks, then the main merger: merged visual tokens and the DeepStack features."""
        if st.next_block < len(self.vision_blocks):
            self.advance_vision(st, len(self.vision_blocks))
        return self._merge(st.x, self.mergers["main"], st.comm, 0, st.token_base), st.deep

    def _merge(self, x: torch.Tensor, m: MergerWeights, comm=None, output: int = 0, token_base: int = 0):
        v = self.arch.vision
        if m.post_norm:
            h = ops.layernorm(x.view(-1, v.merged_dim), m.norm_w, m.norm_b, v.layer_norm_eps)
        else:
            h = ops.layernorm(x, m.norm_w, m.norm_b, v.layer_norm_eps).view(-1, v.merged_dim)
        h = ops.linear(h, m.fc1_w, bias=m.fc1_b, act="gelu")
        if comm is not None:
            comm.allgather_linear(h, m.fc2_w, m.fc2_b, output, token_base)
            return None
        return ops.linear(h, m.fc2_w, bias=m.fc2_b)

    # ---------------------------------------------------------------------- text
    @torch.no_grad()
    def forward(
        self,
        input_ids: torch.Tensor,
        positions: torch.Tensor,
        meta: AttnMeta,
        cache: ops.KVCache,
        *,
        visual: Optional[torch.Tensor] = None,
        vis_index: Optional[torch.Tensor] = None,
        deepstack: Optional[Sequence[torch.Tensor]] = None,
    ) -> torch.Tensor:
        """Hidden states ``[T, H]`` after the final norm.

        ``input_ids [T]`` int64, ``positions [3, T]`` int32, ``vis_index [T]`` int32 maps
        visual placeholder rows to rows of ``visual`` / ``deepstack[k]`` (-1 elsewhere).
        """
        t = self.arch.text
        T = input_ids.shape[0]
        scoring = meta.scorer is not None and meta.is_prefill
        small = T <= SMALL_T and not scoring  # the scorer reads K rows of the dense projection
        comm = self.comm
        comm.begin_step()
        x = ops.embed(input_ids, self.embed, visual=visual, vis_index=vis_index)
        plan = self._decode_plan(cache, T) if (x.is_cuda and not meta.is_prefill and deepstack is None and visual is None) else None
        if plan is not None:
            # opt-in: decode steps of at most 4 tokens on one GPU, every layer in one persistent launch
            pre = plan.run(x, positions, meta.slots, meta.block_tables, meta.context_lens)
            h, _ = ops.add_rmsnorm(self.final_norm, t.rms_norm_eps, x=pre, residual=None)
            return h
        if (self.tp > 1 and x.is_cuda and meta.is_prefill and hasattr(comm, "prefill_fused") and comm.prefill_fused(T)
                and ops.TP_PREFILL_FUSED and not scoring):
            return self._forward_prefill_fused(x, positions, meta, cache, deepstack, vis_index)
        state = LayerwiseState(positions, meta, cache, vis_index, deepstack, T, small, scoring, dense=x)
        self.advance_layers(state, len(self.layers))
        return self.finish_layers(state)

    # ---- resumable form of the layer loop (cooperative prefill runs it a few layers at a time) ----------
    @torch.no_grad()
    def begin_layers(self, input_ids: torch.Tensor, positions: torch.Tensor, meta: AttnMeta, cache: ops.KVCache, *,
                     visual: Optional[torch.Tensor] = None, vis_index: Optional[torch.Tensor] = None,
                     deepstack: Optional[Sequence[torch.Tensor]] = None) -> "LayerwiseState":
        """Embedding of a step whose layers will be run by ``advance_layers`` in pieces (one rank; the reference's
        resumable layer-quantum forward is ``prism_infer/models/qwen3_vl.py:1024-1146``)."""
        if self.tp != 1:
            raise ValueError("the layer-by-layer form runs on one rank")
        T = input_ids.shape[0]
        scoring = meta.scorer is not None and meta.is_prefill
        self.comm.begin_step()
        x = ops.embed(input_ids, self.embed, visual=visual, vis_index=vis_index)
        return LayerwiseState(positions, meta, cache, vis_index, deepstack, T, T <= SMALL_T and not scoring, scoring, dense=x)

    @torch.no_grad()
    def advance_layers(self, st: "LayerwiseState", max_layers: int) -> bool:
        """Run up to ``max_layers`` more decoder layers; True once all layers have run."""
        t, comm = self.arch.text, self.comm
        positions, meta, cache, vis_index, deepstack, T = st.positions, st.meta, st.cache, st.vis_index, st.deepstack, st.tokens
        small, scoring = st.small, st.scoring
        n_deep = len(deepstack) if deepstack is not None else 0
        dense, partials, ticket, residual = st.dense, st.partials, st.ticket, st.residual
        stop = min(len(self.layers), st.next_layer + max(0, int(max_layers)))
        for i in range(st.next_layer, stop):
            l = self.layers[i]
            extra = deepstack[i - 1] if 0 < i <= n_deep else None
            h, residual = comm.add_rmsnorm(l.input_norm, t.rms_norm_eps, dense, partials, ticket, residual,
                                           extra, vis_index if extra is not None else None)
            direct = False
            if small and h.is_cuda:
                qkv_p = ops.linear_partial(h, l.qkv, ops.choose_splits(l.qkv.shape[0], self.H, T))
                q = ops.qk_norm_rope_store(qkv=None, partials=qkv_p, positions=positions, q_weight=l.q_norm, k_weight=l.k_norm,
                                           num_heads=self.Hq, num_kv_heads=self.Hkv, head_dim=self.D, theta=t.rope_theta,
                                           section=t.mrope_section, eps=t.rms_norm_eps, slots=meta.slots, cache=cache, layer=i)
            else:
                qkv = ops.linear(h, l.qkv)
                # no history: attend over the fresh bf16 K/V rows of the projection itself (as the
                # reference does, prism_infer/layers/attention.py:180-193) instead of re-reading
                # and dequantising the pages just written
                direct = meta.is_prefill and meta.no_history and qkv.is_cuda
                q = ops.qk_norm_rope_store(qkv=qkv, partials=None, positions=positions, q_weight=l.q_norm, k_weight=l.k_norm,
                                           num_heads=self.Hq, num_kv_heads=self.Hkv, head_dim=self.D, theta=t.rope_theta,
                                           section=t.mrope_section, eps=t.rms_norm_eps, slots=meta.slots, cache=cache, layer=i,
                                           k_writeback=direct or scoring)
                if scoring:  # K rows after QK-norm and rotary now sit in the projection buffer
                    meta.scorer.observe(i, q, qkv.view(T, self.Hq + 2 * self.Hkv, self.D)[:, self.Hq:self.Hq + self.Hkv],
                                        1.0 / math.sqrt(self.D))
            if direct:
                heads = qkv.view(T, self.Hq + 2 * self.Hkv, self.D)
                a = ops.varlen_attention(q, heads[:, self.Hq:self.Hq + self.Hkv], heads[:, self.Hq + self.Hkv:],
                                         meta.cu_seqlens_q, meta.max_q_len, causal=True)
            elif meta.is_prefill:
                a = ops.paged_prefill_attention(q, cache, i, meta.cu_seqlens_q, meta.kv_lens, meta.block_tables, meta.max_q_len,
                                                cu_seqlens_kv=meta.cu_seqlens_kv, total_kv=meta.total_kv, max_kv_len=meta.max_kv_len)
            else:
                a = ops.paged_decode_attention(q, cache, i, meta.block_tables, meta.context_lens, nsplit=meta.nsplit,
                                               workspace=meta.workspace)
            dense, partials, ticket = comm.row_parallel(a.view(T, self.Hq * self.D), l.o, stages=ops.O_PROJ_STAGES if small else 0)
            h, residual = comm.add_rmsnorm(l.post_norm, t.rms_norm_eps, dense, partials, ticket, residual)
            if small and h.is_cuda and self.I // 128 < 96:
                # too few 128-row tiles for the dual-accumulator kernel to keep enough SMs
                # streaming weights: split-K over the packed matrix, SwiGLU on the partial sums
                gu = ops.linear_partial(h, l.gate_up, ops.choose_splits(2 * self.I, self.H, T))
                act = ops.swiglu(partials=gu)
            else:
                act = ops.gate_up_swiglu(h, l.gate_up)
            dense, partials, ticket = comm.row_parallel(act, l.down)
        st.dense, st.partials, st.ticket, st.residual, st.next_layer = dense, partials, ticket, residual, stop
        return stop == len(self.layers)

    @torch.no_grad()
    def finish_layers(self, st: "LayerwiseState") -> torch.Tensor:
        """Final norm (with the last DeepStack tap when every layer has one); hidden states ``[T, H]``."""
        if st.next_layer != len(self.layers):
            raise RuntimeError(f"finish_layers after {st.next_layer} of {len(self.layers)} layers")
        t = self.arch.text
        n_deep = len(st.deepstack) if st.deepstack is not None else 0
        extra = st.deepstack[n_deep - 1] if n_deep == len(self.layers) else None
        h, _ = self.comm.add_rmsnorm(self.final_norm, t.rms_norm_eps, st.dense, st.partials, st.ticket, st.residual,
                                     extra, st.vis_index if extra is not None else None)
        return h

    def _decode_plan(self, cache: ops.KVCache, tokens: int):
        """The persistent decode kernel's plan for this cache, or ``None`` where it does not apply
        (switched off, which is the default; more than 4 tokens; unsupported head shapes; tensor
        parallelism)."""
        from ..ops import decode_layers as dl

        if not dl.ENABLED or tokens > dl.MAX_TOKENS or self.tp > 1:
            return None
        plans = self.__dict__.setdefault("_decode_plans", {})
        key = cache.payload.data_ptr()
        if key not in plans:
            t = self.arch.text
            plan = None
            if dl.supported(hidden=self.H, heads=self.Hq, kv_heads=self.Hkv, head_dim=self.D, intermediate=self.I):
                inv_freq, axis = ops._rope_tables(self.D, t.rope_theta, t.mrope_section, self.device)
                plan = dl.DecodeLayersPlan(self.layers, cache, hidden=self.H, heads=self.Hq, kv_heads=self.Hkv, head_dim=self.D,
                                           intermediate=self.I, eps=t.rms_norm_eps, inv_freq=inv_freq, axis=axis)
            plans[key] = plan
        plan = plans[key]
        return plan if plan is not None and tokens <= plan.max_tokens else None

    def _forward_prefill_fused(self, x, positions, meta, cache, deepstack, vis_index):
        """Tensor-parallel prefill with the exchanges fused into the kernels around them: each
        row-parallel projection (o_proj, down_proj) scatters its bf16 partial rows to the ranks
        that own them from the GEMM epilogue, and one kernel per exchange sums the owned rows, adds
        the residual shard (kept sharded by token row between layers), normalises and stores the
        rows into every rank's activation buffer, which the next column-parallel GEMM reads.  The
        reference runs an NCCL all-reduce after every row-parallel GEMM
        (``prism_infer/layers/linear.py:186-190``)."""
        t, comm = self.arch.text, self.comm
        T = x.shape[0]
        n_deep = len(deepstack) if deepstack is not None else 0
        layers = self.layers
        h, residual = comm.add_rmsnorm(layers[0].input_norm, t.rms_norm_eps, x, None, None, None)
        shard = False  # residual is the full [T, H] tensor until the first exchange
        for i, l in enumerate(layers):
            qkv = ops.linear(h, l.qkv)
            direct = meta.no_history
            q = ops.qk_norm_rope_store(qkv=qkv, partials=None, positions=positions, q_weight=l.q_norm, k_weight=l.k_norm,
                                       num_heads=self.Hq, num_kv_heads=self.Hkv, head_dim=self.D, theta=t.rope_theta,
                                       section=t.mrope_section, eps=t.rms_norm_eps, slots=meta.slots, cache=cache, layer=i,
                                       k_writeback=direct)
            if direct:
                heads = qkv.view(T, self.Hq + 2 * self.Hkv, self.D)
                a = ops.varlen_attention(q, heads[:, self.Hq:self.Hq + self.Hkv], heads[:, self.Hq + self.Hkv:],
                                         meta.cu_seqlens_q, meta.max_q_len, causal=True)
            else:
                a = ops.paged_prefill_attention(q, cache, i, meta.cu_seqlens_q, meta.kv_lens, meta.block_tables, meta.max_q_len,
                                                cu_seqlens_kv=meta.cu_seqlens_kv, total_kv=meta.total_kv, max_kv_len=meta.max_kv_len)
            ticket = comm.scatter_linear(a.view(T, self.Hq * self.D), l.o)
            h, residual = comm.reduce_norm_allgather(ticket, l.post_norm, t.rms_norm_eps, residual, residual_is_shard=shard)
            shard = True
            act = ops.gate_up_swiglu(h, l.gate_up)
            ticket = comm.scatter_linear(act, l.down)
            last = i + 1 == len(layers)
            norm_w = self.final_norm if last else layers[i + 1].input_norm
            # the DeepStack features of layer i + 1 are added where its input is formed
            extra = deepstack[i] if i < n_deep else None
            h, residual = comm.reduce_norm_allgather(ticket, norm_w, t.rms_norm_eps, residual, residual_is_shard=True, extra=extra,
                                                     extra_index=vis_index if extra is not None else None)
        return h

    @torch.no_grad()
    def enable_fp8_candidate_head(self) -> None:
        """``logits_precision="selective_fp32"``: keep a row-scaled E4M3 copy of the LM head for greedy decode steps
        of one row (reference ``prism_infer/models/qwen3_vl.py:1659-1753``); one rank, CUDA."""
        if self.tp == 1 and self.lm_head.is_cuda and self.lm_head.dtype == torch.bfloat16 and self.H % 16 == 0:
            self.lm_head_fp8 = ops.quantize_lm_head_fp8(self.lm_head)

    @torch.no_grad()
    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        """fp32 rank-local logits ``[B, V / tp]`` for the given hidden rows."""
        if hidden.is_cuda:
            return ops.linear_partial(hidden, self.lm_head, 1)[0]
        return ops.linear(hidden, self.lm_head).float()

    @torch.no_grad()
    def sample(self, hidden: torch.Tensor, temperature: Optional[torch.Tensor], *, seed: int = 0,
               step: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Next token per row: LM head, then arg-max / exponential-race sampling; under tensor
        parallelism ranks exchange their shard winners so every rank returns the same ids."""
        fp8_head = self.__dict__.get("lm_head_fp8")
        if (fp8_head is not None and temperature is None and self.tp == 1 and hidden.is_cuda
                and hidden.shape[0] <= ops.LM_HEAD_FP8_BATCH and not self.__dict__.get("keep_logits")):
            # greedy rows: candidates from the E4M3 copy of the head (half the bytes), exact rerank with the bf16 rows
            return ops.lm_head_fp8_greedy(hidden, fp8_head[0], fp8_head[1], self.lm_head, out=out)
        logits = self.logits(hidden)
        if self.__dict__.get("keep_logits"):
            # debugging aid (eager execution): full-vocabulary fp32 logits of the last sampled rows
            self.last_logits = (logits if self.tp == 1 else self.comm.gather_logits(logits)).float().clone()
        if self.tp == 1:
            return ops.sample(logits, temperature, seed=seed, step=step, out=out)
        if temperature is None or logits.is_cuda:
            # arg-max and the exponential race are both "largest perturbed logit wins", and the perturbation is keyed
            # by the global token id: every rank finds the winner of its vocabulary shard and the ranks exchange
            # (value, id) pairs; the full logits never travel
            val = torch.empty(logits.shape[0], dtype=torch.float32, device=logits.device)
            ids = ops.sample(logits, temperature, seed=seed, step=step, vocab_offset=self.vocab_start, out_val=val)
            tok = self.comm.greedy_merge(val, ids)
        else:  # the CPU sampler draws its noise per logits row, not per token id
            tok = ops.sample(self.comm.gather_logits(logits), temperature, seed=seed, step=step)
        if out is not None:
            out.copy_(tok)
            return out
        return tok
