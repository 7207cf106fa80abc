"""Multimodal request preparation on the CPU (reference ``prism_infer/engine/vl_inputs.py``).

``PatchProcessor`` is the built-in image / video preprocessor with the output contract of
the Hugging Face Qwen3-VL processor: ``pixel_values [N, C * Tp * P * P]`` in
merge-window-major patch order ``(t, h_block, w_block, h_in, w_in)``, ``grid_thw`` rows
``(T, H, W)`` in patches, still images duplicated to fill the temporal patch, sizes snapped
to multiples of ``patch * merge`` inside the pixel budget, and one placeholder token per
merged 2x2 window.  Chat-template prompts and the optional Hugging Face processor live in
``chat_prompt.py``; the validators below are shared.
"""

from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import Any, Sequence

import numpy as np
import torch
import torch.nn.functional as F

IMAGE_MEAN = (0.5, 0.5, 0.5)
IMAGE_STD = (0.5, 0.5, 0.5)


@dataclass
class ImageInputs:
    input_ids: list[int]
    pixel_values: torch.Tensor
    image_grid_thw: list[tuple[int, int, int]]

    def validate(self, arch) -> None:
        _validate(self.input_ids, self.pixel_values, self.image_grid_thw, arch.image_token_id, arch)


@dataclass
class VideoInputs:
    input_ids: list[int]
    pixel_values: torch.Tensor
    video_grid_thw: list[tuple[int, int, int]]

    def validate(self, arch) -> None:
        _validate(self.input_ids, self.pixel_values, self.video_grid_thw, arch.video_token_id, arch)


def _validate(ids: Sequence[int], pixels: torch.Tensor, grid: Sequence[Sequence[int]], token_id: int, arch) -> None:
    v = arch.vision
    if pixels.dim() != 2 or pixels.shape[1] != v.patch_input_dim:
        raise ValueError(f"pixel_values must be [N, {v.patch_input_dim}], got {list(pixels.shape)}")
    patches = sum(int(t) * int(h) * int(w) for t, h, w in grid)
    if patches != pixels.shape[0]:
        raise ValueError(f"grid_thw describes {patches} patches but pixel_values has {pixels.shape[0]}")
    for t, h, w in grid:
        if h % v.spatial_merge_size or w % v.spatial_merge_size:
            raise ValueError(f"grid {t, h, w} is not a multiple of the spatial merge size")
    expected = patches // v.merge_unit
    found = sum(1 for t in ids if t == token_id)
    if found != expected:
        raise ValueError(f"prompt has {found} placeholder tokens, the grids need {expected}")


def to_uint8_hwc(image: Any) -> np.ndarray:
    """PIL image, numpy array, torch tensor or the path of an image file -> ``uint8 [H, W, 3]``."""
    if isinstance(image, (str, os.PathLike)):
        from PIL import Image

        with Image.open(os.fspath(image)) as im:
            return np.asarray(im.convert("RGB"))
    if isinstance(image, torch.Tensor):
        arr = image.detach().cpu().numpy()
    elif isinstance(image, np.ndarray):
        arr = image
    else:  # PIL
        arr = np.asarray(image.convert("RGB"))
    if arr.ndim == 3 and arr.shape[0] == 3 and arr.shape[-1] != 3:
        arr = np.transpose(arr, (1, 2, 0))
    if arr.ndim != 3 or arr.shape[-1] != 3:
        raise ValueError(f"image must be HxWx3, got shape {arr.shape}")
    if arr.dtype != np.uint8:
        arr = np.clip(arr * (255.0 if arr.max() <= 1.0 else 1.0), 0, 255).astype(np.uint8)
    return arr


def smart_resize(h: int, w: int, factor: int, min_pixels: int, max_pixels: int) -> tuple[int, int]:
    hb = max(factor, round(h / factor) * factor)
    wb = max(factor, round(w / factor) * factor)
    if hb * wb > max_pixels:
        beta = math.sqrt(h * w / max_pixels)
        hb = max(factor, math.floor(h / beta / factor) * factor)
        wb = max(factor, math.floor(w / beta / factor) * factor)
    elif hb * wb < min_pixels:
        beta = math.sqrt(min_pixels / (h * w))
        hb = math.ceil(h * beta / factor) * factor
        wb = math.ceil(w * beta / factor) * factor
    return hb, wb


VIDEO_SAMPLE_FPS, VIDEO_MIN_FRAMES, VIDEO_MAX_FRAMES = 2.0, 4, 768


def smart_resize_video(num_frames: int, h: int, w: int, temporal_factor: int, factor: int, min_pixels: int, max_pixels: int) -> tuple[int, int]:
    """Frame size of a clip under a budget on its whole volume (frames x height x width, frames rounded up to the
    temporal patch), the rule of the Hugging Face Qwen3-VL video processor: sides rounded to ``factor``, shrunk when the
    volume exceeds ``max_pixels``, enlarged when it is below ``min_pixels``."""
    if h < factor or w < factor:
        raise ValueError(f"height {h} or width {w} is smaller than the resize factor {factor}")
    if max(h, w) / min(h, w) > 200:
        raise ValueError(f"aspect ratio {max(h, w) / min(h, w):.1f} exceeds 200")
    hb, wb = round(h / factor) * factor, round(w / factor) * factor
    tb = math.ceil(num_frames / temporal_factor) * temporal_factor
    if tb * hb * wb > max_pixels:
        beta = math.sqrt(num_frames * h * w / max_pixels)
        hb = max(factor, math.floor(h / beta / factor) * factor)
        wb = max(factor, math.floor(w / beta / factor) * factor)
    elif tb * hb * wb < min_pixels:
        beta = math.sqrt(min_pixels / (num_frames * h * w))
        hb = math.ceil(h * beta / factor) * factor
        wb = math.ceil(w * beta / factor) * factor
    return hb, wb


def resize_bicubic(arr: np.ndarray, height: int, width: int) -> np.ndarray:
    """``uint8 [H, W, 3]`` -> ``uint8 [height, width, 3]`` with the antialiased bicubic filter of Pillow, which is what
    the Hugging Face image processor applies (within one grey level of it on random images; an interpolation without
    antialiasing differs by tens of levels when an image is shrunk).  Without Pillow: torch's antialiased bicubic."""
    try:
        from PIL import Image
    except ImportError:
        t = torch.from_numpy(arr).permute(2, 0, 1).unsqueeze(0).float()
        t = F.interpolate(t, size=(height, width), mode="bicubic", align_corners=False, antialias=True).clamp(0, 255)
        return t.squeeze(0).permute(1, 2, 0).round().to(torch.uint8).numpy()
    return np.asarray(Image.fromarray(arr).resize((width, height), resample=Image.BICUBIC))


def checkpoint_pixel_budgets(model_dir: str) -> dict[str, int]:
    """Pixel budgets a checkpoint directory records for its processor: ``min_pixels`` / ``max_pixels`` from
    ``preprocessor_config.json`` (``size.shortest_edge`` / ``size.longest_edge``, or the older ``min_pixels`` /
    ``max_pixels`` keys) and ``video_min_pixels`` / ``video_max_pixels`` (budgets on frames x height x width) from
    ``video_preprocessor_config.json``.  Missing files or keys are
    simply absent from the result; an image smaller than the checkpoint's minimum is then enlarged exactly as the
    checkpoint's own processor would."""
    import json
    import os

    def read(name: str) -> dict:
        path = os.path.join(model_dir, name)
        if not os.path.isfile(path):
            return {}
        with open(path, encoding="utf-8") as fh:
            value = json.load(fh)
        return value if isinstance(value, dict) else {}

    def budget(cfg: dict, size_key: str, flat_key: str):
        size = cfg.get("size")
        v = size.get(size_key) if isinstance(size, dict) else None
        v = cfg.get(flat_key) if v is None else v
        return int(v) if isinstance(v, (int, float)) and not isinstance(v, bool) and v > 0 else None

    out: dict[str, int] = {}
    image, video = read("preprocessor_config.json"), read("video_preprocessor_config.json")
    for key, cfg, size_key, flat in (("min_pixels", image, "shortest_edge", "min_pixels"), ("max_pixels", image, "longest_edge", "max_pixels"),
                                     ("video_min_pixels", video, "shortest_edge", "min_pixels"),
                                     ("video_max_pixels", video, "longest_edge", "max_pixels")):
        v = budget(cfg, size_key, flat)
        if v is not None:
            out[key] = v
    for key in ("fps", "min_frames", "max_frames"):  # how the checkpoint's video processor samples a file
        v = video.get(key)
        if isinstance(v, (int, float)) and not isinstance(v, bool) and v > 0:
            out[f"video_{key}"] = v if key == "fps" else int(v)
    return out


class PatchProcessor:
    """Images: per-image pixel budget (``min_pixels`` .. ``max_pixels``).  Clips: budget on the volume frames x height x
    width (``video_min_pixels`` .. ``video_max_pixels``), as the checkpoint's video processor counts it."""

    def __init__(self, arch, *, min_pixels: int | None = None, max_pixels: int | None = None,
                 video_max_pixels: int | None = None, video_min_pixels: int | None = None, video_fps: float | None = None,
                 video_min_frames: int | None = None, video_max_frames: int | None = None) -> None:
        self.arch = arch
        v = arch.vision
        self.factor = v.patch_size * v.spatial_merge_size
        self.min_pixels = min_pixels or 4 * self.factor * self.factor
        self.max_pixels = max_pixels or 16384 * self.factor * self.factor
        self.video_max_pixels = video_max_pixels or 24 * self.max_pixels // 16   # 25.2 M: the 8B checkpoint's recorded volume budget
        self.video_min_pixels = video_min_pixels or self.factor * self.factor * 4
        # sampling of a video file (frames per second of source time and the bounds on their number)
        self.video_fps = float(video_fps or VIDEO_SAMPLE_FPS)
        self.video_min_frames = int(video_min_frames or VIDEO_MIN_FRAMES)
        self.video_max_frames = int(video_max_frames or VIDEO_MAX_FRAMES)

    def _frames_to_patches(self, frames: np.ndarray) -> tuple[torch.Tensor, tuple[int, int, int]]:
        """``uint8 [F, H, W, 3]`` (F a multiple of the temporal patch) -> patches, grid."""
        v = self.arch.vision
        f, h, w, _ = frames.shape
        x = torch.from_numpy(frames).permute(0, 3, 1, 2).float() / 255.0
        mean = torch.tensor(IMAGE_MEAN).view(1, 3, 1, 1)
        std = torch.tensor(IMAGE_STD).view(1, 3, 1, 1)
        x = (x - mean) / std
        tp, p, m = v.temporal_patch_size, v.patch_size, v.spatial_merge_size
        gt, gh, gw = f // tp, h // p, w // p
        x = x.view(gt, tp, 3, gh // m, m, p, gw // m, m, p)
        # -> (t, h_block, w_block, h_in, w_in, C, Tp, P, P)
        x = x.permute(0, 3, 6, 4, 7, 2, 1, 5, 8).contiguous()
        return x.view(gt * gh * gw, 3 * tp * p * p), (gt, gh, gw)

    def process_image(self, image: Any) -> tuple[torch.Tensor, tuple[int, int, int]]:
        arr = to_uint8_hwc(image)
        h, w = arr.shape[:2]
        nh, nw = smart_resize(h, w, self.factor, self.min_pixels, self.max_pixels)
        if (nh, nw) != (h, w):
            arr = resize_bicubic(arr, nh, nw)
        tp = self.arch.vision.temporal_patch_size
        return self._frames_to_patches(np.repeat(arr[None], tp, axis=0))

    def process_video(self, frames: Sequence[Any]) -> tuple[torch.Tensor, tuple[int, int, int]]:
        arrs = [to_uint8_hwc(f) for f in frames]
        tp = self.arch.vision.temporal_patch_size
        while len(arrs) % tp:
            arrs.append(arrs[-1])
        h, w = arrs[0].shape[:2]
        nh, nw = smart_resize_video(len(arrs), h, w, tp, self.factor, self.video_min_pixels, self.video_max_pixels)
        stack = np.stack(arrs)
        if (nh, nw) != (h, w):
            stack = np.stack([resize_bicubic(f, nh, nw) for f in stack])
        return self._frames_to_patches(stack)

    def tokens_for(self, grid: tuple[int, int, int]) -> int:
        return grid[0] * grid[1] * grid[2] // self.arch.vision.merge_unit


def video_sample_indices(total_frames: int, source_fps: float | None, *, fps: float = VIDEO_SAMPLE_FPS, min_frames: int = VIDEO_MIN_FRAMES,
                         max_frames: int = VIDEO_MAX_FRAMES, num_frames: int | None = None) -> list[int]:
    """Which frames of a clip are read: ``fps`` frames per second of source time, at least ``min_frames`` and at most
    ``max_frames`` (and never more than the clip has), evenly spaced from the first to the last frame - the rule of the
    Hugging Face Qwen3-VL video processor.  A clip without a known frame rate counts as 24 frames per second."""
    if total_frames <= 0:
        raise ValueError("the clip has no frames")
    if num_frames is None:
        n = int(total_frames / float(source_fps or 24.0) * fps)
        num_frames = min(max(n, min_frames), max_frames, total_frames)
    if num_frames <= 0:
        raise ValueError("num_frames must be positive")
    return [int(i) for i in np.linspace(0, total_frames - 1, num_frames).round().astype(int)]


def load_video_file(path: str, *, fps: float = VIDEO_SAMPLE_FPS, min_frames: int = VIDEO_MIN_FRAMES, max_frames: int = VIDEO_MAX_FRAMES,
                    num_frames: int | None = None):
    """Decode the sampled frames of a video file with OpenCV -> ``(list of uint8 [H, W, 3] RGB frames, VideoTiming)``.
    Frames are read in one sequential pass (seeking is unreliable for many containers); the timing carries the source
    indices and frame rate, from which the prompt's time stamps follow."""
    try:
        import cv2  # type: ignore
    except ImportError as exc:
        raise RuntimeError("reading a video file needs the optional dependency cv2 (opencv-python-headless); "
                           "pass a list of frames instead") from exc
    from .chat_prompt import VideoTiming

    cap = cv2.VideoCapture(str(path))
    if not cap.isOpened():
        raise OSError(f"cannot open video: {path}")
    try:
        total, source_fps = int(cap.get(cv2.CAP_PROP_FRAME_COUNT)), float(cap.get(cv2.CAP_PROP_FPS)) or None
        if total <= 0:
            raise ValueError(f"video reports no frames: {path}")
        wanted = video_sample_indices(total, source_fps, fps=fps, min_frames=min_frames, max_frames=max_frames, num_frames=num_frames)
        need, frames, i = {}, [], 0
        for w in wanted:
            need[w] = need.get(w, 0) + 1
        last = max(wanted)
        while i <= last:
            ok, bgr = cap.read()
            if not ok:
                break
            for _ in range(need.get(i, 0)):
                frames.append(np.ascontiguousarray(bgr[:, :, ::-1]))
            i += 1
        if len(frames) != len(wanted):
            raise OSError(f"{path}: the container reports {total} frames but decoding stopped at frame {i}")
    finally:
        cap.release()
    return frames, VideoTiming(tuple(wanted), float(source_fps or 24.0))


def image_block(arch, n_tokens: int) -> list[int]:
    return [arch.vision_start_token_id] + [arch.image_token_id] * n_tokens + [arch.vision_end_token_id]


def video_blocks(arch, grid: tuple[int, int, int], merge_unit: int) -> list[int]:
    """One placeholder run per temporal group (timestamps would sit between them)."""
    per = grid[1] * grid[2] // merge_unit
    out: list[int] = []
    for _ in range(grid[0]):
        out += [arch.vision_start_token_id] + [arch.video_token_id] * per + [arch.vision_end_token_id]
    return out


def prepare_image_inputs(processor: PatchProcessor, tokenizer, prompt: str | Sequence[int], images: Sequence[Any], *,
                         chat=None) -> ImageInputs:
    """All images first, then the question (media-first layout).  With ``chat`` (a
    ``chat_prompt.ChatPrompt``) a string prompt is wrapped in the checkpoint's chat turns, as the
    reference does through the Hugging Face processor (``engine/vl_inputs.py:216-243``); token-id
    prompts and ``chat=None`` keep the bare layout."""
    arch = processor.arch
    ids: list[int] = []
    pixels, grids = [], []
    for img in images:
        pv, grid = processor.process_image(img)
        pixels.append(pv)
        grids.append(grid)
        ids += image_block(arch, processor.tokens_for(grid))
    if chat is not None and isinstance(prompt, str):
        from .chat_prompt import encode_with_media

        ids = encode_with_media(tokenizer, chat.image_prompt(prompt, len(grids)), arch,
                                image_tokens=[processor.tokens_for(g) for g in grids])
    else:
        ids += list(prompt) if not isinstance(prompt, str) else tokenizer.encode(prompt)
    out = ImageInputs(ids, torch.cat(pixels), grids)
    out.validate(arch)
    return out


def prepare_interleaved_image_inputs(processor: PatchProcessor, tokenizer, prompt: str, images: Sequence[Any],
                                     image_marker: str = "<image>", *, chat=None) -> ImageInputs:
    """The prompt names where each image goes with ``image_marker``."""
    arch = processor.arch
    parts = prompt.split(image_marker)
    if len(parts) - 1 != len(images):
        raise ValueError(f"prompt has {len(parts) - 1} {image_marker!r} markers for {len(images)} images")
    if chat is not None:
        from .chat_prompt import encode_with_media

        done = [processor.process_image(img) for img in images]
        grids = [g for _, g in done]
        ids = encode_with_media(tokenizer, chat.interleaved_image_prompt(prompt, len(images), image_marker=image_marker), arch,
                                image_tokens=[processor.tokens_for(g) for g in grids])
        out = ImageInputs(ids, torch.cat([pv for pv, _ in done]), grids)
        out.validate(arch)
        return out
    ids: list[int] = []
    pixels, grids = [], []
    for i, text in enumerate(parts):
        if text.strip():
            ids += tokenizer.encode(text)
        if i < len(images):
            pv, grid = processor.process_image(images[i])
            pixels.append(pv)
            grids.append(grid)
            ids += image_block(arch, processor.tokens_for(grid))
    out = ImageInputs(ids, torch.cat(pixels), grids)
    out.validate(arch)
    return out


def prepare_video_inputs(processor: PatchProcessor, tokenizer, prompt: str | Sequence[int], frames: Sequence[Any], *,
                         chat=None, timing=None) -> VideoInputs:
    """One clip, then the question.  With ``chat`` a string prompt gets the checkpoint's chat turns
    and each temporal group is preceded by its time stamp (``timing``: a ``chat_prompt.VideoTiming``
    with the source frame indices and frame rate; consecutive frames at 24 fps when absent, which
    is what the Hugging Face processor assumes for pre-sampled frames)."""
    arch = processor.arch
    pv, grid = processor.process_video(frames)
    if chat is not None and isinstance(prompt, str):
        from .chat_prompt import VideoTiming, encode_with_media

        timing = timing or VideoTiming(tuple(range(len(frames))))
        times = timing.group_times(arch.vision.temporal_patch_size)
        if len(times) != grid[0]:
            raise ValueError(f"timing describes {len(times)} temporal groups, the clip has {grid[0]}")
        ids = encode_with_media(tokenizer, chat.video_prompt(prompt), arch,
                                video_groups=[(grid[1] * grid[2] // arch.vision.merge_unit, times)])
    else:
        ids = video_blocks(arch, grid, arch.vision.merge_unit)
        ids += list(prompt) if not isinstance(prompt, str) else tokenizer.encode(prompt)
    out = VideoInputs(ids, pv, [grid])
    out.validate(arch)
    return out
