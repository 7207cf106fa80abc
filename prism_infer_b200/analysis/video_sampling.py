"""Frame selection for video benchmarks.

``uniform_segment_center_indices`` reproduces the segment-centre rule of the reference
(``prism_infer/analysis/video_sampling.py:50-102``): the clip ``[start, end]`` is cut into
``frames`` equal segments and the frame at ``start + seg/2 + round(seg * i)`` is taken from
each.  ``sample_frame_sequence`` applies it to frames already in memory,
``sample_frame_manifest`` (:283-341) to a directory of numbered frame files (1-based,
contiguous), ``sample_video_file`` (:188-281) to a container file through OpenCV when it is
installed.  Every sampler returns the frames and a provenance record with the indices and a
SHA-256 over the sampled RGB bytes.
"""

from __future__ import annotations

import hashlib
import math
from collections.abc import Mapping, Sequence
from pathlib import Path
from typing import Any

import numpy as np

from .identity import canonical_json_sha256


def _as_int(name: str, v: object) -> int:
    if isinstance(v, bool) or not isinstance(v, int):
        raise ValueError(f"{name} must be an integer")
    return v


def _as_float(name: str, v: object) -> float:
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(float(v)):
        raise ValueError(f"{name} must be a finite number")
    return float(v)


def uniform_segment_center_indices(*, first_index: int, max_index: int, frames: int, fps: float,
                                   temporal_bound: Mapping[str, Any] | None = None) -> list[int]:
    first_index, max_index, frames = _as_int("first_index", first_index), _as_int("max_index", max_index), _as_int("frames", frames)
    if first_index < 0 or max_index < first_index or frames <= 0:
        raise ValueError("need 0 <= first_index <= max_index and frames > 0")
    fps = _as_float("fps", fps)
    if fps <= 0:
        raise ValueError("fps must be positive")
    lo, hi = first_index, max_index
    if temporal_bound is not None:
        start, end = _as_float("temporal_bound.start", temporal_bound.get("start")), _as_float("temporal_bound.end", temporal_bound.get("end"))
        if start < 0 or end <= start:
            raise ValueError("temporal bound needs 0 <= start < end")
        lo, hi = max(first_index, round(start * fps)), min(max_index, round(end * fps))
        if hi < lo:
            raise ValueError(f"temporal bound [{start}, {end}] s lies outside the available frames")
    seg = (hi - lo) / frames
    return [int(lo + seg / 2.0 + round(seg * i)) for i in range(frames)]


def _to_rgb_array(frame: Any) -> np.ndarray:
    if hasattr(frame, "convert"):  # PIL image
        frame = np.asarray(frame.convert("RGB"))
    arr = np.asarray(frame)
    if arr.ndim != 3 or arr.shape[2] != 3 or arr.dtype != np.uint8:
        raise ValueError(f"frame must be uint8 [H, W, 3], got {arr.dtype} {arr.shape}")
    return np.ascontiguousarray(arr)


def rgb_identity(frames: Sequence[np.ndarray], indices: Sequence[int]) -> str:
    rows = [{"index": int(i), "height": int(f.shape[0]), "width": int(f.shape[1]),
             "sha256": hashlib.sha256(f.tobytes()).hexdigest()} for f, i in zip(frames, indices)]
    return canonical_json_sha256(rows)


def sample_frame_sequence(all_frames: Sequence[Any], *, frames: int, fps: float,
                          temporal_bound: Mapping[str, Any] | None = None) -> tuple[list[np.ndarray], dict[str, Any]]:
    if len(all_frames) == 0:
        raise ValueError("no frames")
    idx = uniform_segment_center_indices(first_index=0, max_index=len(all_frames) - 1, frames=frames, fps=fps, temporal_bound=temporal_bound)
    picked = [_to_rgb_array(all_frames[i]) for i in idx]
    return picked, {"source_kind": "frame_sequence", "decoder": "none", "fps": float(fps), "source_frame_count": len(all_frames),
                    "sampled_indices": idx, "sampled_rgb_identity_sha256": rgb_identity(picked, idx)}


def sample_frame_manifest(frame_records: Sequence[Mapping[str, Any]], *, materialized_root: str | Path, frames: int, fps: float,
                          temporal_bound: Mapping[str, Any] | None = None) -> tuple[list[np.ndarray], dict[str, Any]]:
    """Records carry ``archive_member_path`` (``.../00012.jpg``, numbering starts at 1 and must
    be contiguous) and ``materialized_path`` relative to ``materialized_root``."""
    from PIL import Image

    if not frame_records:
        raise ValueError("frame manifest is empty")
    by_index: dict[int, Mapping[str, Any]] = {}
    for rec in frame_records:
        member = rec.get("archive_member_path")
        if not isinstance(member, str) or not Path(member).stem.isdigit():
            raise ValueError(f"frame file name is not numeric: {member!r}")
        i = int(Path(member).stem)
        if i in by_index:
            raise ValueError(f"duplicate frame index {i}")
        by_index[i] = rec
    top = max(by_index)
    missing = sorted(set(range(1, top + 1)) - set(by_index))
    if missing or 0 in by_index:
        raise ValueError(f"frame numbering must be 1..{top} without gaps; missing={missing[:8]}")
    idx = uniform_segment_center_indices(first_index=1, max_index=top, frames=frames, fps=fps, temporal_bound=temporal_bound)
    root = Path(materialized_root).resolve()
    picked = []
    for i in idx:
        path = (root / str(by_index[i]["materialized_path"])).resolve()
        if root not in path.parents:
            raise ValueError(f"materialized path escapes the root: {by_index[i]['materialized_path']!r}")
        with Image.open(path) as im:
            picked.append(_to_rgb_array(im))
    return picked, {"source_kind": "frame_directory", "decoder": "Pillow", "fps": float(fps), "source_frame_count": top,
                    "frame_access": {"method": "frame_manifest", "reported_frame_count": top, "fallback_trigger": None},
                    "sampled_indices": idx, "sampled_rgb_identity_sha256": rgb_identity(picked, idx)}


def sample_video_file(path: str | Path, *, frames: int, temporal_bound: Mapping[str, Any] | None = None) -> tuple[list[np.ndarray], dict[str, Any]]:
    """Decode with OpenCV: seek to each index; if a seek fails, count and decode sequentially."""
    try:
        import cv2  # type: ignore
    except ImportError as exc:
        raise RuntimeError("sampling a video container needs the optional dependency cv2 (opencv-python-headless)") from exc
    cap = cv2.VideoCapture(str(path))
    if not cap.isOpened():
        raise OSError(f"cannot open video: {path}")
    try:
        reported, fps = int(cap.get(cv2.CAP_PROP_FRAME_COUNT)), float(cap.get(cv2.CAP_PROP_FPS))
        if reported <= 0:
            raise ValueError(f"video reports no frames: {path}")
        idx = uniform_segment_center_indices(first_index=0, max_index=reported - 1, frames=frames, fps=fps, temporal_bound=temporal_bound)
        picked, method, trigger = [], "random_seek", None
        for i in idx:
            cap.set(cv2.CAP_PROP_POS_FRAMES, i)
            ok, bgr = cap.read()
            if not ok:
                method, trigger = "sequential", f"seek to frame {i} failed"
                break
            picked.append(np.ascontiguousarray(bgr[:, :, ::-1]))
        count = reported
        if method == "sequential":
            cap.release()
            cap = cv2.VideoCapture(str(path))
            decoded, n = {}, 0
            want = None
            while True:  # first pass decides the true frame count, so decode everything once
                ok, bgr = cap.read()
                if not ok:
                    break
                decoded[n] = bgr
                n += 1
                if len(decoded) > 4096:
                    raise ValueError("sequential fallback is limited to 4096 frames")
            count = n
            idx = uniform_segment_center_indices(first_index=0, max_index=count - 1, frames=frames, fps=fps, temporal_bound=temporal_bound)
            picked = [np.ascontiguousarray(decoded[i][:, :, ::-1]) for i in idx]
            del want
        return picked, {"source_kind": "video_file", "decoder": f"opencv {cv2.__version__}", "fps": fps, "source_frame_count": count,
                        "frame_access": {"method": method, "reported_frame_count": reported, "fallback_trigger": trigger},
                        "sampled_indices": idx, "sampled_rgb_identity_sha256": rgb_identity(picked, idx)}
    finally:
        cap.release()
