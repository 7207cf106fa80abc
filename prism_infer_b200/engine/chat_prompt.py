"""Chat-template prompts for instruction-tuned checkpoints (reference
``prism_infer/engine/vl_inputs.py:216-306`` builds them through the Hugging Face processor's
``apply_chat_template``; ``:438-509`` and the processor add one time stamp per temporal group of
a video).

A real Qwen3-VL-Instruct checkpoint expects ChatML turns with one media marker per image or
video; feeding it bare placeholder runs gives the same API and different tokens.  This module
renders the turns and expands the markers without needing the Hugging Face *processor* (pixels
go through ``PatchProcessor``):

* ``ChatPrompt.render`` uses the tokenizer's own chat template when it has one
  (``tokenizer.apply_chat_template``), otherwise the built-in ChatML layout Qwen3-VL ships.
* ``encode_with_media`` tokenises the rendered text and replaces every image marker by
  ``<|vision_start|> <|image_pad|> x n <|vision_end|>`` with ``n`` from the image's grid, and every
  video marker by one such block per temporal group, each preceded by the text
  ``<t seconds>`` where ``t`` is the mean time of the frames merged into the group.

When the checkpoint directory ships processor files and ``transformers`` can load them,
``HFProcessorAdapter`` runs the Hugging Face processor instead and converts its output to the
engine's ``ImageInputs`` / ``VideoInputs``.
"""

from __future__ import annotations

import os
import re
from dataclasses import dataclass
from typing import Any, Sequence

import torch

IMAGE_MARKER = "<|vision_start|><|image_pad|><|vision_end|>"
VIDEO_MARKER = "<|vision_start|><|video_pad|><|vision_end|>"
DEFAULT_VIDEO_FPS = 24.0  # what the Hugging Face processor assumes for pre-sampled frames without metadata
# a template may put white space between the three tokens of a marker
_MARKER = re.compile(r"<\|vision_start\|>\s*<\|(image|video)_pad\|>\s*<\|vision_end\|>")


@dataclass(frozen=True)
class VideoTiming:
    """Source frame indices of the sampled frames and the source frame rate."""

    frame_indices: tuple[int, ...]
    fps: float = DEFAULT_VIDEO_FPS

    def group_times(self, temporal_patch: int) -> list[float]:
        """Seconds shown before each temporal group: the mean of its first and last frame time
        (the last frame repeats when the count is not a multiple of the temporal patch)."""
        idx = list(self.frame_indices)
        while len(idx) % temporal_patch:
            idx.append(idx[-1])
        t = [i / float(self.fps) for i in idx]
        return [(t[i] + t[i + temporal_patch - 1]) / 2 for i in range(0, len(t), temporal_patch)]


def _content_text(content: Any) -> str:
    """ChatML body of one message: strings pass through; lists interleave text and media markers."""
    if isinstance(content, str):
        return content
    out = []
    for item in content:
        kind = item.get("type")
        if kind == "image":
            out.append(IMAGE_MARKER)
        elif kind == "video":
            out.append(VIDEO_MARKER)
        elif kind == "text":
            out.append(str(item.get("text", "")))
        else:
            raise ValueError(f"unsupported chat content type {kind!r}")
    return "".join(out)


class ChatPrompt:
    """Renders chat turns for a tokenizer (its own template if it has one, ChatML otherwise)."""

    def __init__(self, tokenizer: Any = None) -> None:
        self.tokenizer = tokenizer
        self.has_template = bool(getattr(tokenizer, "chat_template", None)) and hasattr(tokenizer, "apply_chat_template")

    def render(self, messages: Sequence[dict], *, add_generation_prompt: bool = True) -> str:
        if self.has_template:
            return self.tokenizer.apply_chat_template(list(messages), tokenize=False, add_generation_prompt=add_generation_prompt)
        text = "".join(f"<|im_start|>{m['role']}\n{_content_text(m['content'])}<|im_end|>\n" for m in messages)
        return text + ("<|im_start|>assistant\n" if add_generation_prompt else "")

    # ---- the three layouts of the public API ----------------------------------------------------
    def image_prompt(self, prompt: str, n_images: int, **kw) -> str:
        """All images first, then the question (media-first layout)."""
        if n_images < 1:
            raise ValueError("an image prompt needs at least one image")
        content = [{"type": "image"} for _ in range(n_images)] + [{"type": "text", "text": prompt}]
        return self.render([{"role": "user", "content": content}], **kw)

    def interleaved_image_prompt(self, prompt: str, n_images: int, *, image_marker: str = "<image>", **kw) -> str:
        """Images sit where ``image_marker`` appears in the prompt (questions that name their images)."""
        if not isinstance(prompt, str) or not prompt:
            raise ValueError("interleaved image prompt must be a non-empty string")
        if not isinstance(image_marker, str) or not image_marker:
            raise ValueError("image_marker must be a non-empty string")
        parts = prompt.split(image_marker)
        if len(parts) - 1 != n_images:
            raise ValueError(f"interleaved image marker count must equal image count: markers={len(parts) - 1}, images={n_images}")
        content: list[dict] = []
        for i, text in enumerate(parts):
            if text:
                content.append({"type": "text", "text": text})
            if i < n_images:
                content.append({"type": "image"})
        return self.render([{"role": "user", "content": content}], **kw)

    def video_prompt(self, prompt: str, **kw) -> str:
        return self.render([{"role": "user", "content": [{"type": "video"}, {"type": "text", "text": prompt}]}], **kw)


def encode_with_media(tokenizer: Any, text: str, arch, *, image_tokens: Sequence[int] = (),
                      video_groups: Sequence[tuple[int, Sequence[float]]] = ()) -> list[int]:
    """Token ids of ``text`` with its media markers expanded.

    ``image_tokens[i]`` is the placeholder count of the i-th image marker; ``video_groups[j]`` is
    ``(placeholders per temporal group, [seconds of each group])`` of the j-th video marker.  The
    text between markers is tokenised piecewise, so a tokenizer without the special tokens in its
    vocabulary (the offline ``IdTokenizer``) works as well as a Hugging Face one.
    """
    images, videos = list(image_tokens), list(video_groups)
    out: list[int] = []
    pos = 0

    def emit_text(chunk: str) -> None:
        if chunk:
            out.extend(int(t) for t in tokenizer.encode(chunk, add_special_tokens=False))

    for match in _MARKER.finditer(text):
        emit_text(text[pos:match.start()])
        pos = match.end()
        if match.group(1) == "image":
            if not images:
                raise ValueError("more image markers in the prompt than images")
            out += [arch.vision_start_token_id] + [arch.image_token_id] * int(images.pop(0)) + [arch.vision_end_token_id]
        else:
            if not videos:
                raise ValueError("more video markers in the prompt than videos")
            per_group, times = videos.pop(0)
            for t in times:
                emit_text(f"<{t:.1f} seconds>")
                out += [arch.vision_start_token_id] + [arch.video_token_id] * int(per_group) + [arch.vision_end_token_id]
    emit_text(text[pos:])
    if images or videos:
        raise ValueError("fewer media markers in the prompt than media")
    return out


# ---- optional Hugging Face processor ------------------------------------------------------------------
PROCESSOR_FILES = ("preprocessor_config.json", "processor_config.json")


def has_processor_files(model: str) -> bool:
    return os.path.isdir(model) and any(os.path.exists(os.path.join(model, f)) for f in PROCESSOR_FILES)


class HFProcessorAdapter:
    """The checkpoint's own Hugging Face processor behind the engine's input types (reference
    ``prism_infer/engine/vl_inputs.py:95-130``: ``AutoProcessor.from_pretrained`` with local files
    only and the pixel budgets written into ``size.longest_edge``)."""

    def __init__(self, model: str, *, image_max_pixels: int | None = None, video_max_pixels: int | None = None) -> None:
        from transformers import AutoProcessor

        self.processor = AutoProcessor.from_pretrained(model, local_files_only=True)
        for value, name in ((image_max_pixels, "image_processor"), (video_max_pixels, "video_processor")):
            if value is None:
                continue
            if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
                raise ValueError(f"{name} pixel budget must be a positive integer or None")
            size = getattr(getattr(self.processor, name, None), "size", None)
            if size is None:
                raise ValueError(f"processor.{name}.size has no longest_edge budget")
            if isinstance(size, dict):
                size["longest_edge"] = value
            else:
                size.longest_edge = value
        self.chat = ChatPrompt(self.processor if hasattr(self.processor, "apply_chat_template") else self.processor.tokenizer)

    def image_inputs(self, prompt_text: str, images: Sequence[Any]):
        from .vl_inputs import ImageInputs

        batch = self.processor(text=prompt_text, images=list(images), return_tensors="pt")
        for key in ("input_ids", "pixel_values", "image_grid_thw"):
            if key not in batch:
                raise ValueError(f"processor output missing required key {key!r}")
        return ImageInputs(batch["input_ids"][0].tolist(), batch["pixel_values"].contiguous().to(torch.float32),
                           [tuple(int(v) for v in row) for row in batch["image_grid_thw"].tolist()])

    def video_inputs(self, prompt_text: str, frames: Sequence[Any], timing: VideoTiming | None = None):
        from .vl_inputs import VideoInputs

        kwargs: dict[str, Any] = {"do_sample_frames": False}  # a list of frames is already the caller's sample
        if timing is not None:
            kwargs["video_metadata"] = [{"total_num_frames": len(timing.frame_indices), "fps": float(timing.fps),
                                         "frames_indices": list(timing.frame_indices)}]
        batch = self.processor(text=prompt_text, videos=[list(frames)], return_tensors="pt", videos_kwargs=kwargs)
        for key in ("input_ids", "pixel_values_videos", "video_grid_thw"):
            if key not in batch:
                raise ValueError(f"processor output missing required video key {key!r}")
        return VideoInputs(batch["input_ids"][0].tolist(), batch["pixel_values_videos"].contiguous().to(torch.float32),
                           [tuple(int(v) for v in row) for row in batch["video_grid_thw"].tolist()])
