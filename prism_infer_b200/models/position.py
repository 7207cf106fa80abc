"""3-axis (T, H, W) position ids for Qwen3-VL prompts and the M-RoPE tables.

``rope_index`` has the semantics of Hugging Face ``get_rope_index`` for Qwen3-VL
(reference ``prism_infer/models/qwen3_vl_position.py:108-483``): text runs advance all
three axes together; a visual span that starts at position ``p`` receives
``(p, p + h, p + w)`` over its merged grid and the next text token continues at
``max + 1``; a video contributes one span per temporal group (T = 1 each, because
timestamp text separates the groups).

``mrope_axis_table`` / ``mrope_cos_sin`` implement interleaved M-RoPE (reference
``prism_infer/vision/mrope.py:82-150``): frequency slot ``i`` uses the H position when
``i % 3 == 1 and i < 3 * section[1]``, the W position when ``i % 3 == 2 and
i < 3 * section[2]``, and the T position otherwise.
"""

from __future__ import annotations

from typing import Sequence

import numpy as np
import torch


def rope_index(
    input_ids: Sequence[int] | torch.Tensor,
    *,
    image_grid_thw: torch.Tensor | Sequence[Sequence[int]] | None = None,
    video_grid_thw: torch.Tensor | Sequence[Sequence[int]] | None = None,
    image_token_id: int,
    video_token_id: int,
    spatial_merge_size: int,
) -> tuple[torch.Tensor, int]:
    """Return ``position_ids [3, 1, S]`` (int64, CPU) and the scalar ``rope_delta``.

    ``rope_delta = max(position) + 1 - S``; a decode step at sequence length ``n``
    uses position ``n - 1 + rope_delta`` on all three axes.
    """
    ids = np.asarray(input_ids.tolist() if isinstance(input_ids, torch.Tensor) else input_ids, dtype=np.int64).reshape(-1)
    n = int(ids.shape[0])

    def _rows(grid) -> list[tuple[int, int, int]]:
        if grid is None:
            return []
        rows = grid.tolist() if isinstance(grid, torch.Tensor) else list(grid)
        return [(int(t), int(h), int(w)) for t, h, w in rows]

    image_rows = _rows(image_grid_thw)
    # A video of T temporal groups is T consecutive single-frame spans.
    video_rows = [(1, h, w) for (t, h, w) in _rows(video_grid_thw) for _ in range(t)]

    pos = np.empty((3, n), dtype=np.int64)
    if not image_rows and not video_rows:
        pos[:] = np.arange(n, dtype=np.int64)
        return torch.from_numpy(pos).view(3, 1, n), 0

    # maximal runs of equal "kind" (0 text, 1 image placeholder, 2 video placeholder); a placeholder
    # run may hold several grids back to back, so it is consumed grid by grid below
    kind = np.where(ids == image_token_id, 1, np.where(ids == video_token_id, 2, 0))
    starts = np.flatnonzero(np.diff(kind, prepend=-1)).tolist() if n else []
    ends = starts[1:] + [n]
    cursor = 0  # next position value
    img_i = vid_i = 0
    m = spatial_merge_size
    for lo, hi in zip(starts, ends):
        k = int(kind[lo])
        if k == 0:
            pos[:, lo:hi] = np.arange(cursor, cursor + hi - lo, dtype=np.int64)
            cursor += hi - lo
            continue
        i = lo
        while i < hi:
            if k == 1:
                if img_i >= len(image_rows):
                    raise ValueError("more image placeholder runs than image_grid_thw rows")
                t, h, w = image_rows[img_i]
                img_i += 1
            else:
                if vid_i >= len(video_rows):
                    raise ValueError("more video placeholder runs than video frames")
                t, h, w = video_rows[vid_i]
                vid_i += 1
            gh, gw = h // m, w // m
            span = t * gh * gw
            if i + span > hi:
                raise ValueError(f"placeholder run at {i} is shorter than its grid ({t}x{gh}x{gw} = {span})")
            grid = np.indices((t, gh, gw), dtype=np.int64).reshape(3, span)
            pos[:, i:i + span] = grid + cursor
            cursor += max(t, gh, gw)
            i += span
    if img_i != len(image_rows) or vid_i != len(video_rows):
        raise ValueError("fewer placeholder runs than grid rows")
    delta = int(pos.max()) + 1 - n
    return torch.from_numpy(pos).view(3, 1, n), delta


def mrope_axis_table(section: Sequence[int], half_dim: int) -> torch.Tensor:
    """``axis[i]`` in {0 (T), 1 (H), 2 (W)} for every rotary frequency slot ``i``."""
    axis = torch.zeros(half_dim, dtype=torch.int32)
    for i in range(half_dim):
        if i % 3 == 1 and i < 3 * section[1]:
            axis[i] = 1
        elif i % 3 == 2 and i < 3 * section[2]:
            axis[i] = 2
    return axis


def mrope_inv_freq(head_dim: int, theta: float) -> torch.Tensor:
    return 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))


def mrope_cos_sin(
    positions: torch.Tensor, head_dim: int, theta: float, section: Sequence[int]
) -> tuple[torch.Tensor, torch.Tensor]:
    """``positions [3, T]`` -> fp32 ``cos, sin [T, head_dim]`` (rotate-half layout)."""
    half = head_dim // 2
    inv = mrope_inv_freq(head_dim, theta).to(positions.device)
    axis = mrope_axis_table(section, half).to(positions.device).long()
    p = positions.to(torch.float32)[axis, :]  # [half, T]
    ang = (p * inv[:, None]).transpose(0, 1)  # [T, half]
    ang = torch.cat((ang, ang), dim=-1)
    return ang.cos(), ang.sin()


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def vision_patch_coords(grid_thw: Sequence[Sequence[int]], merge: int) -> torch.Tensor:
    """``[N, 2]`` (row, col) of each patch in merge-window-major order.

    Order inside an item is ``(t, h_block, w_block, h_in, w_in)``, the order in which
    the processor emits patches, so ``view(-1, merge*merge*C)`` merges 2x2 windows.
    """
    out = []
    for t, h, w in grid_thw:
        t, h, w = int(t), int(h), int(w)
        rows = torch.arange(h).view(h // merge, 1, merge, 1).expand(h // merge, w // merge, merge, merge)
        cols = torch.arange(w).view(1, w // merge, 1, merge).expand(h // merge, w // merge, merge, merge)
        rc = torch.stack((rows.reshape(-1), cols.reshape(-1)), dim=-1)
        out.append(rc.repeat(t, 1))
    return torch.cat(out, dim=0)


def vision_pos_embed_plan(
    grid_thw: Sequence[Sequence[int]], grid_per_side: int, merge: int
) -> tuple[torch.Tensor, torch.Tensor]:
    """Bilinear interpolation plan of the learned ``grid_per_side^2`` position table.

    Returns ``idx [4, N]`` (int64 rows of the table) and ``weight [4, N]`` (fp32), in
    the same merge-window-major patch order as ``vision_patch_coords`` (reference
    ``prism_infer/vision/vision_encoder.py:593-653``).
    """
    idx_parts, w_parts = [], []
    g = grid_per_side
    for t, h, w in grid_thw:
        t, h, w = int(t), int(h), int(w)
        hg = torch.linspace(0, g - 1, h)
        wg = torch.linspace(0, g - 1, w)
        hf, wf = hg.int(), wg.int()
        hc, wc = (hf + 1).clamp(max=g - 1), (wf + 1).clamp(max=g - 1)
        dh, dw = hg - hf, wg - wf
        idx = torch.stack(
            [
                (hf[:, None] * g + wf[None, :]).flatten(),
                (hf[:, None] * g + wc[None, :]).flatten(),
                (hc[:, None] * g + wf[None, :]).flatten(),
                (hc[:, None] * g + wc[None, :]).flatten(),
            ]
        ).long()
        wt = torch.stack(
            [
                ((1 - dh)[:, None] * (1 - dw)[None, :]).flatten(),
                ((1 - dh)[:, None] * dw[None, :]).flatten(),
                (dh[:, None] * (1 - dw)[None, :]).flatten(),
                (dh[:, None] * dw[None, :]).flatten(),
            ]
        )
        rc = vision_patch_coords([(1, h, w)], merge)
        order = (rc[:, 0] * w + rc[:, 1]).repeat(t)
        idx_parts.append(idx[:, order])
        w_parts.append(wt[:, order])
    return torch.cat(idx_parts, dim=1), torch.cat(w_parts, dim=1)


def vision_segments(grid_thw: Sequence[Sequence[int]]) -> list[int]:
    """Attention segment lengths: one segment of ``H*W`` patches per temporal index."""
    out: list[int] = []
    for t, h, w in grid_thw:
        out.extend([int(h) * int(w)] * int(t))
    return out
