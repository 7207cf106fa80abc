"""Chat-template prompts: the built-in ChatML layout, a tokenizer's own template, marker expansion
(image placeholder runs, per-group video time stamps) and, where the reference package is
installed next to the repository, string equality with its prompt builders on a synthetic
checkpoint directory."""

import os
import sys

import numpy as np
import pytest
import torch

from prism_infer_b200.engine.chat_prompt import ChatPrompt, VideoTiming, encode_with_media
from prism_infer_b200.engine.vl_inputs import (PatchProcessor, prepare_image_inputs, prepare_interleaved_image_inputs,
                                               prepare_video_inputs)
from prism_infer_b200.models.architecture import Qwen3VLArch
from prism_infer_b200.utils.tokenizer import IdTokenizer

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _img(seed, size=64):
    return np.random.default_rng(seed).integers(0, 256, (size, size, 3), dtype=np.uint8)


def test_builtin_chatml_layouts():
    chat = ChatPrompt(None)
    assert not chat.has_template
    assert chat.image_prompt("what is this?", 2) == (
        "<|im_start|>user\n<|vision_start|><|image_pad|><|vision_end|><|vision_start|><|image_pad|><|vision_end|>"
        "what is this?<|im_end|>\n<|im_start|>assistant\n")
    assert chat.interleaved_image_prompt("A <image> or B <image>?", 2) == (
        "<|im_start|>user\nA <|vision_start|><|image_pad|><|vision_end|> or B <|vision_start|><|image_pad|><|vision_end|>?"
        "<|im_end|>\n<|im_start|>assistant\n")
    assert chat.video_prompt("describe", add_generation_prompt=False) == (
        "<|im_start|>user\n<|vision_start|><|video_pad|><|vision_end|>describe<|im_end|>\n")
    with pytest.raises(ValueError, match="marker count"):
        chat.interleaved_image_prompt("only <image> one", 2)


def test_video_group_times_follow_the_frame_indices():
    assert VideoTiming((0, 12, 24, 36), fps=24.0).group_times(2) == [0.25, 1.25]
    assert VideoTiming((0, 10, 20), fps=10.0).group_times(2) == [0.5, 2.0]  # the last frame repeats


def test_marker_expansion_with_the_offline_tokenizer():
    arch = Qwen3VLArch.tiny()
    tok = IdTokenizer(arch.text.vocab_size, (arch.image_token_id, arch.video_token_id, arch.vision_start_token_id,
                                             arch.vision_end_token_id, arch.eos_token_id))
    proc, chat = PatchProcessor(arch), ChatPrompt(None)
    plain = prepare_image_inputs(proc, tok, "7 8 9", [_img(0), _img(1)])
    wrapped = prepare_image_inputs(proc, tok, "7 8 9", [_img(0), _img(1)], chat=chat)
    n_img = sum(t == arch.image_token_id for t in plain.input_ids)
    assert n_img == sum(t == arch.image_token_id for t in wrapped.input_ids) == 2 * 4
    assert torch.equal(plain.pixel_values, wrapped.pixel_values) and plain.image_grid_thw == wrapped.image_grid_thw
    last = len(wrapped.input_ids) - 1 - wrapped.input_ids[::-1].index(arch.vision_end_token_id)
    assert wrapped.input_ids[last + 1:last + 3] == [7, 8]  # the question follows the media (the offline tokenizer splits on blanks)
    assert len(wrapped.input_ids) > len(plain.input_ids)  # the turns' own tokens
    # token-id prompts are never wrapped
    assert prepare_image_inputs(proc, tok, [7, 8, 9], [_img(0)], chat=chat).input_ids[-3:] == [7, 8, 9]
    inter = prepare_interleaved_image_inputs(proc, tok, "1 <image> 2 <image> 3 4", [_img(2), _img(3)], chat=chat)
    ids = inter.input_ids
    first, second = ids.index(arch.vision_start_token_id), len(ids) - 1 - ids[::-1].index(arch.vision_start_token_id)
    assert 1 in ids[:first] and 2 in ids[first:second] and 3 in ids[second:]
    # video: one time stamp and one placeholder block per temporal group
    frames = [_img(s) for s in range(4)]
    vid = prepare_video_inputs(proc, tok, "5 6", frames, chat=chat, timing=VideoTiming((0, 12, 24, 36), 24.0))
    assert vid.video_grid_thw[0][0] == 2 and sum(t == arch.vision_start_token_id for t in vid.input_ids) == 2
    stamp = tok.encode("<0.2 seconds>")  # 0.25 formats as 0.2 (round half to even), as in the reference processor
    at = vid.input_ids.index(arch.vision_start_token_id)
    assert vid.input_ids[at - len(stamp):at] == stamp
    with pytest.raises(ValueError, match="temporal groups"):
        prepare_video_inputs(proc, tok, "5 6", frames, chat=chat, timing=VideoTiming((0, 1), 24.0))
    with pytest.raises(ValueError, match="fewer media markers"):
        encode_with_media(tok, "no marker here", arch, image_tokens=[4])


@pytest.fixture(scope="module")
def synthetic_checkpoint(tmp_path_factory):
    """Config, word-level tokenizer with a chat template and processor configs, no weights."""
    pytest.importorskip("tokenizers")
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_arm

    path = str(tmp_path_factory.mktemp("ckpt"))
    arch = Qwen3VLArch.qwen3_vl_8b()
    reference_arm.write_checkpoint(path, arch, with_weights=False)
    return path, arch


def test_tokenizer_template_is_used_and_expanded(synthetic_checkpoint):
    from transformers import AutoTokenizer

    path, arch = synthetic_checkpoint
    tok = AutoTokenizer.from_pretrained(path)
    chat = ChatPrompt(tok)
    assert chat.has_template
    text = chat.image_prompt("t5 t6", 2)
    assert text == tok.apply_chat_template([{"role": "user", "content": [{"type": "image"}, {"type": "image"},
                                                                         {"type": "text", "text": "t5 t6"}]}],
                                           tokenize=False, add_generation_prompt=True)
    ids = encode_with_media(tok, text, arch, image_tokens=[3, 2])
    assert ids.count(arch.image_token_id) == 5 and ids.count(arch.vision_start_token_id) == 2
    # the same ids as tokenising the text with its pads repeated, which is what the Hugging Face processor does
    expanded = text.replace("<|image_pad|>", " ".join(["<|image_pad|>"] * 3), 1)
    head, tail = expanded.rsplit("<|image_pad|>", 1)
    expanded = head + " ".join(["<|image_pad|>"] * 2) + tail
    assert ids == tok.encode(expanded, add_special_tokens=False)


def test_prompts_equal_the_reference_builders(synthetic_checkpoint):
    """Same strings as the reference's ``build_*_prompt`` (Hugging Face processor with the same template)."""
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "prism_infer")):
        pytest.skip("the reference package is not installed under baseline/_ref")
    from transformers import AutoTokenizer

    path, _ = synthetic_checkpoint
    tok = AutoTokenizer.from_pretrained(path)
    with open(os.path.join(path, "chat_template.jinja"), "w") as fh:  # the processor reads its template from a file
        fh.write(tok.chat_template)
    sys.path.insert(0, ref_root)
    try:
        from prism_infer.engine.vl_inputs import (build_image_prompt, build_interleaved_image_prompt, build_video_prompt,
                                                  load_vl_processor)

        proc = load_vl_processor(path)
    except Exception as exc:  # the reference needs more of the Hugging Face stack than this image has
        pytest.skip(f"reference processor unavailable: {exc}")
    finally:
        sys.path.remove(ref_root)
    chat, img = ChatPrompt(tok), _img(0)
    assert chat.image_prompt("t5 t6", 2) == build_image_prompt(proc, "t5 t6", [img, img])
    assert chat.interleaved_image_prompt("t1 <image> t2 <image>", 2) == build_interleaved_image_prompt(proc, "t1 <image> t2 <image>", [img, img])
    assert chat.video_prompt("t9") == build_video_prompt(proc, "t9", [img, img])


def test_native_input_preparation_equals_the_checkpoint_processor(synthetic_checkpoint):
    """``HFProcessorAdapter`` (the checkpoint's own Hugging Face processor) and the built-in preparation give the same
    token ids, grids and (within the resize tolerance) patches for images, and the same ids and grid for a clip with
    time stamps."""
    from transformers import AutoTokenizer

    from prism_infer_b200.engine.chat_prompt import HFProcessorAdapter, has_processor_files

    path, arch = synthetic_checkpoint
    tok = AutoTokenizer.from_pretrained(path)
    if not os.path.exists(os.path.join(path, "chat_template.jinja")):
        with open(os.path.join(path, "chat_template.jinja"), "w") as fh:
            fh.write(tok.chat_template)
    assert has_processor_files(path)
    adapter = HFProcessorAdapter(path)
    chat = ChatPrompt(tok)
    from prism_infer_b200.engine.vl_inputs import checkpoint_pixel_budgets

    budgets = checkpoint_pixel_budgets(path)
    assert {k: budgets[k] for k in ("min_pixels", "max_pixels", "video_min_pixels", "video_max_pixels")} == \
        {"min_pixels": 65536, "max_pixels": 16777216, "video_min_pixels": 4096, "video_max_pixels": 25165824}
    assert set(budgets) <= {"min_pixels", "max_pixels", "video_min_pixels", "video_max_pixels", "video_fps", "video_min_frames", "video_max_frames"}
    native = PatchProcessor(arch, **budgets)  # what the engine does for a checkpoint directory
    images = [_img(0, 64), np.random.default_rng(5).integers(0, 256, (100, 130, 3), dtype=np.uint8)]  # both below the minimum: enlarged
    mine = prepare_image_inputs(native, tok, "t5 t6 t7", images, chat=chat)
    theirs = adapter.image_inputs(adapter.chat.image_prompt("t5 t6 t7", 2), images)
    assert mine.input_ids == theirs.input_ids and [tuple(g) for g in mine.image_grid_thw] == [tuple(g) for g in theirs.image_grid_thw]
    assert mine.pixel_values.shape == theirs.pixel_values.shape
    assert float((mine.pixel_values - theirs.pixel_values).abs().max()) < 2.1 / 127.5
    frames = [_img(s, 64) for s in range(4)]
    timing = VideoTiming((0, 12, 24, 36), 24.0)
    mine_v = prepare_video_inputs(native, tok, "t5 t6", frames, chat=chat, timing=timing)
    theirs_v = adapter.video_inputs(adapter.chat.video_prompt("t5 t6"), frames, timing)
    assert [tuple(g) for g in mine_v.video_grid_thw] == [tuple(g) for g in theirs_v.video_grid_thw]
    assert float((mine_v.pixel_values - theirs_v.pixel_values).abs().max()) < 1e-5
    # the token ids of the clip cannot be compared on this synthetic checkpoint: its whitespace-split word-level vocabulary
    # needs blanks between the special tokens of the template, and the upstream processor looks for the unbroken run
    # "<|vision_start|><|video_pad|><|vision_end|>" when it inserts the per-group time stamps
    # a clip whose volume exceeds the budget is shrunk the way the upstream video processor shrinks it
    from transformers.models.qwen3_vl.video_processing_qwen3_vl import smart_resize as upstream_resize

    from prism_infer_b200.engine.vl_inputs import smart_resize_video

    for n, h, w, lo, hi in ((16, 448, 448, 4096, 25165824), (64, 720, 1280, 4096, 25165824), (3, 40, 64, 65536, 10 ** 7), (7, 333, 517, 4096, 2 * 10 ** 5)):
        assert smart_resize_video(n, h, w, 2, 32, lo, hi) == upstream_resize(n, h, w, 2, 32, lo, hi)
