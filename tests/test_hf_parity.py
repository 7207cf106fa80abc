"""Parity with the Hugging Face implementation of Qwen3-VL (``transformers.models.qwen3_vl``) on a tiny random-weight
model, CPU, fp32: checkpoint tensor names and shapes, 3-axis rope indices, the vision tower with its DeepStack taps,
last-token logits for image and video prompts, and greedy tokens of the engine.  The plain-PyTorch oracle of this
package is what every kernel and engine test compares against; these tests tie the oracle to the upstream model code."""

import numpy as np
import pytest
import torch

from prism_infer_b200 import LLM, SamplingParams
from prism_infer_b200.engine.vl_inputs import PatchProcessor, prepare_image_inputs, prepare_video_inputs
from prism_infer_b200.models.architecture import Qwen3VLArch
from prism_infer_b200.models.position import rope_index
from prism_infer_b200.models.reference_model import ReferenceQwen3VL
from prism_infer_b200.models.weights import random_weights
from prism_infer_b200.utils.tokenizer import load_tokenizer

hf_qwen3_vl = pytest.importorskip("transformers.models.qwen3_vl")


def _production_shaped_arch() -> Qwen3VLArch:
    """Small, but with the 8B model's structural numbers: 128-wide text heads with rotary sections 24 / 20 / 20, 72-wide
    vision heads, three DeepStack taps, a 48 x 48 learned position grid, grouped-query attention 4 : 1."""
    from prism_infer_b200.models.architecture import TextArch, VisionArch

    return Qwen3VLArch(
        text=TextArch(vocab_size=2048, hidden_size=512, num_layers=3, num_heads=4, num_kv_heads=1, head_dim=128, intermediate_size=768,
                      mrope_section=(24, 20, 20), max_position_embeddings=4096),
        vision=VisionArch(hidden_size=144, depth=4, num_heads=2, intermediate_size=288, num_position_embeddings=2304, out_hidden_size=512,
                          deepstack_visual_indexes=(0, 1, 3)),
        image_token_id=2001, video_token_id=2002, vision_start_token_id=2003, vision_end_token_id=2004, eos_token_id=2005)


@pytest.fixture(scope="module", params=["tiny", "production_shaped"])
def pair(request):
    arch = Qwen3VLArch.tiny() if request.param == "tiny" else _production_shaped_arch()
    cfg = hf_qwen3_vl.Qwen3VLConfig(**arch.to_hf_config())
    torch.manual_seed(0)
    hf = hf_qwen3_vl.Qwen3VLForConditionalGeneration(cfg).eval().float()
    g = torch.Generator().manual_seed(1)
    weights = {}
    for k, v in hf.state_dict().items():  # nothing left at its initial value: norm weights and biases are random too
        base = 1.0 if ("norm" in k and k.endswith("weight")) else 0.0
        weights[k] = torch.randn(v.shape, generator=g) * (0.05 if v.ndim > 1 else 0.2) + base
    hf.load_state_dict(weights)
    return arch, hf, weights, ReferenceQwen3VL(arch, weights)


def _types(arch, ids):
    mm = torch.zeros_like(ids, dtype=torch.int32)
    mm[ids == arch.image_token_id] = 1
    mm[ids == arch.video_token_id] = 2
    return mm


def _image(seed, h=224, w=224):
    return np.random.default_rng(seed).integers(0, 256, (h, w, 3), dtype=np.uint8)


def _hf_logits(arch, hf, inputs, extra_ids=()):
    ids = torch.tensor([list(inputs.input_ids) + list(extra_ids)])
    kw = {}
    if hasattr(inputs, "image_grid_thw"):
        kw.update(pixel_values=inputs.pixel_values.float(), image_grid_thw=torch.tensor(inputs.image_grid_thw))
    else:
        kw.update(pixel_values_videos=inputs.pixel_values.float(), video_grid_thw=torch.tensor(inputs.video_grid_thw))
    with torch.no_grad():
        out = hf(input_ids=ids, attention_mask=torch.ones_like(ids), mm_token_type_ids=_types(arch, ids), **kw)
    return out.logits[0, -1]


def test_checkpoint_tensor_names_and_shapes_are_the_upstream_ones(pair):
    arch, hf, _, _ = pair
    ours = random_weights(arch, dtype=torch.float32, seed=0)
    theirs = hf.state_dict()
    assert set(ours) == set(theirs)
    assert all(tuple(ours[k].shape) == tuple(theirs[k].shape) for k in ours)


@pytest.mark.parametrize("kind", ["images", "video", "text"])
def test_rope_index_equals_upstream(pair, kind):
    arch, hf, _, _ = pair
    tok, proc = load_tokenizer("random:tiny", arch), PatchProcessor(arch)
    kw = dict(image_grid_thw=None, video_grid_thw=None)
    if kind == "images":
        inp = prepare_image_inputs(proc, tok, [5, 6, 7], [_image(0), _image(1, 64, 96)])
        ids, kw["image_grid_thw"] = inp.input_ids, inp.image_grid_thw
    elif kind == "video":
        inp = prepare_video_inputs(proc, tok, [5, 6, 7], [_image(s, 64, 64) for s in range(6)])
        ids, kw["video_grid_thw"] = inp.input_ids, inp.video_grid_thw
    else:
        ids = list(range(10, 30))
    pos, delta = rope_index(ids, image_token_id=arch.image_token_id, video_token_id=arch.video_token_id,
                            spatial_merge_size=arch.vision.spatial_merge_size, **kw)
    t = torch.tensor([ids])
    hf_kw = {k: torch.tensor(v) for k, v in kw.items() if v is not None}
    hpos, hdelta = hf.model.get_rope_index(t, _types(arch, t), attention_mask=torch.ones_like(t), **hf_kw)
    assert torch.equal(pos[:, 0, :].long(), hpos[:, 0, :].long()) and int(delta) == int(hdelta)


def test_vision_tower_and_deepstack_taps_equal_upstream(pair):
    arch, hf, _, oracle = pair
    inp = prepare_image_inputs(PatchProcessor(arch), load_tokenizer("random:tiny", arch), [1], [_image(2), _image(3, 96, 64)])
    with torch.no_grad():
        out = hf.model.visual(inp.pixel_values.float(), grid_thw=torch.tensor(inp.image_grid_thw))
    main, deep = oracle.vision(inp.pixel_values.float(), inp.image_grid_thw)
    assert float((main - out.pooler_output).abs().max()) < 1e-4
    assert len(deep) == len(out.deepstack_features) == len(arch.vision.deepstack_visual_indexes)
    for a, b in zip(deep, out.deepstack_features):
        assert float((a - b).abs().max()) < 1e-4


@pytest.mark.parametrize("kind", ["images", "video"])
def test_last_token_logits_equal_upstream(pair, kind):
    arch, hf, _, oracle = pair
    tok, proc = load_tokenizer("random:tiny", arch), PatchProcessor(arch)
    if kind == "images":
        inp = prepare_image_inputs(proc, tok, [5, 6, 7, 8, 9], [_image(4), _image(5, 64, 96)])
        kw = dict(pixel_values=inp.pixel_values, image_grid_thw=inp.image_grid_thw)
    else:
        inp = prepare_video_inputs(proc, tok, [5, 6, 7, 8, 9], [_image(s, 64, 64) for s in range(4)])
        kw = dict(pixel_values=inp.pixel_values, video_grid_thw=inp.video_grid_thw)
    _, logits = oracle.generate_greedy(inp.input_ids, 1, return_logits=True, **kw)
    want = _hf_logits(arch, hf, inp)
    assert float((logits[0] - want).abs().max()) < 1e-4 * max(1.0, float(want.abs().max()))


def test_engine_greedy_tokens_equal_upstream_greedy_tokens(pair):
    """The engine on CPU (paged KV, the 56-token prompt prefilled in two chunks) against token-by-token arg-max of the upstream model."""
    arch, hf, weights, _ = pair
    inp = prepare_image_inputs(PatchProcessor(arch), load_tokenizer("random:tiny", arch), [5, 6, 7, 8, 9], [_image(6)])
    want, extra = [], []
    for _ in range(6):
        nxt = int(torch.argmax(_hf_logits(arch, hf, inp, extra)))
        want.append(nxt)
        extra.append(nxt)
    llm = LLM("random:tiny", arch=arch, weights=weights, device="cpu", max_model_len=256, kvcache_block_size=16, num_kvcache_blocks=32,
              enforce_eager=True, max_num_batched_tokens=256, max_chunk_size=52)
    got = llm.generate_prepared_image_inputs(inp, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))["token_ids"]
    llm.exit()
    assert got == want


def test_patch_processor_equals_the_upstream_image_processor():
    """Same grid, same patch layout (temporal pair, merge-block order, channel / time / row / column inside a patch), same
    normalisation; pixels within two grey levels where the image had to be resized (the upstream resize runs in torchvision)."""
    transformers = pytest.importorskip("transformers")
    from PIL import Image

    from prism_infer_b200.engine.vl_inputs import IMAGE_MEAN, IMAGE_STD

    arch = Qwen3VLArch.tiny()
    ours = PatchProcessor(arch)
    v = arch.vision
    theirs = transformers.Qwen2VLImageProcessor(patch_size=v.patch_size, temporal_patch_size=v.temporal_patch_size, merge_size=v.spatial_merge_size,
                                                image_mean=list(IMAGE_MEAN), image_std=list(IMAGE_STD),
                                                size={"shortest_edge": ours.min_pixels, "longest_edge": ours.max_pixels})
    for shape, exact in (((224, 224), True), ((64, 96), True), ((100, 130), False), ((37, 500), False), ((1000, 700), False)):
        arr = _image(sum(shape), *shape)
        mine, grid = ours.process_image(arr)
        out = theirs(images=[Image.fromarray(arr)], return_tensors="pt")
        assert list(grid) == out["image_grid_thw"][0].tolist()
        diff = float((mine - out["pixel_values"]).abs().max())
        assert diff < (1e-6 if exact else 2.1 / 127.5), (shape, diff)


def test_a_checkpoint_saved_by_the_upstream_model_loads_and_generates_the_same_tokens(pair, tmp_path):
    """``save_pretrained`` of the upstream model (config.json + safetensors) -> ``LLM(directory)``: the configuration
    parser and the safetensors routing see exactly what a real checkpoint directory holds."""
    arch, hf, _, _ = pair
    hf.save_pretrained(tmp_path / "ckpt", safe_serialization=True, max_shard_size="400KB")  # several shards and an index file
    assert len(list((tmp_path / "ckpt").glob("*.safetensors"))) > 3 and (tmp_path / "ckpt" / "model.safetensors.index.json").is_file()
    assert Qwen3VLArch.from_pretrained(str(tmp_path / "ckpt")) == arch
    inp = prepare_image_inputs(PatchProcessor(arch), load_tokenizer("random:tiny", arch), [9, 8, 7], [_image(7, 64, 96)])
    want, extra = [], []
    for _ in range(5):
        nxt = int(torch.argmax(_hf_logits(arch, hf, inp, extra)))
        want.append(nxt)
        extra.append(nxt)
    llm = LLM(str(tmp_path / "ckpt"), device="cpu", max_model_len=256, kvcache_block_size=16, num_kvcache_blocks=32,
              enforce_eager=True, max_num_batched_tokens=256, max_chunk_size=256)
    got = llm.generate_prepared_image_inputs(inp, SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))["token_ids"]
    llm.exit()
    assert got == want


def test_video_file_sampling_rule_equals_upstream_and_a_file_request_runs(pair, tmp_path):
    """Frame indices as the upstream video processor picks them for a range of clip lengths and frame rates; a video
    file goes through ``LLM.generate_video`` with the time stamps of its sampled frames and gives the oracle's tokens."""
    cv2 = pytest.importorskip("cv2")
    from transformers.models.qwen3_vl.video_processing_qwen3_vl import Qwen3VLVideoProcessor
    from transformers.video_utils import VideoMetadata

    from prism_infer_b200.engine.vl_inputs import load_video_file, video_sample_indices

    upstream = Qwen3VLVideoProcessor()
    for total, fps in ((40, 10.0), (7, 30.0), (3000, 25.0), (100000, 24.0), (5, None), (900, 29.97)):
        meta = VideoMetadata(total_num_frames=total, fps=fps)
        assert video_sample_indices(total, fps) == [int(i) for i in upstream.sample_frames(meta)], (total, fps)
    arch, _, weights, oracle = pair
    clip = tmp_path / "clip.avi"
    w = cv2.VideoWriter(str(clip), cv2.VideoWriter_fourcc(*"MJPG"), 10.0, (64, 64))
    rng = np.random.default_rng(0)
    for _ in range(40):
        w.write(rng.integers(0, 256, (64, 64, 3), dtype=np.uint8))
    w.release()
    frames, timing = load_video_file(str(clip))
    assert len(frames) == 8 and timing.fps == 10.0 and list(timing.frame_indices) == [int(i) for i in np.linspace(0, 39, 8).round()]
    llm = LLM("random:tiny", arch=arch, weights=weights, device="cpu", max_model_len=512, kvcache_block_size=16, num_kvcache_blocks=64,
              enforce_eager=True, max_num_batched_tokens=512, max_chunk_size=512)
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    from_file = llm.generate_video([5, 6, 7], str(clip), sp)
    inputs = llm.prepare_video([5, 6, 7], frames, timing=timing)
    assert from_file["token_ids"] == llm.generate_prepared_video_inputs(inputs, sp)["token_ids"]
    assert from_file["token_ids"] == oracle.generate_greedy(inputs.input_ids, 4, pixel_values=inputs.pixel_values, video_grid_thw=inputs.video_grid_thw)
    llm.exit()


def test_tied_embedding_checkpoint_loads_without_an_lm_head_tensor(tmp_path):
    """Smaller Qwen3-VL checkpoints tie the LM head to the embedding: the saved file has no ``lm_head.weight``."""
    import dataclasses

    from safetensors import safe_open

    arch = Qwen3VLArch.tiny()
    arch = dataclasses.replace(arch, text=dataclasses.replace(arch.text, tie_word_embeddings=True))
    torch.manual_seed(0)
    hf = hf_qwen3_vl.Qwen3VLForConditionalGeneration(hf_qwen3_vl.Qwen3VLConfig(**arch.to_hf_config())).eval().float()
    g = torch.Generator().manual_seed(5)
    with torch.no_grad():
        for name, p in hf.named_parameters():
            p.copy_(torch.randn(p.shape, generator=g) * (0.05 if p.ndim > 1 else 0.2) + (1.0 if ("norm" in name and name.endswith("weight")) else 0.0))
    assert hf.lm_head.weight.data_ptr() == hf.model.language_model.embed_tokens.weight.data_ptr()
    hf.save_pretrained(tmp_path / "ckpt", safe_serialization=True)
    with safe_open(str(tmp_path / "ckpt" / "model.safetensors"), "pt") as fh:
        assert "lm_head.weight" not in list(fh.keys())
    assert Qwen3VLArch.from_pretrained(str(tmp_path / "ckpt")).text.tie_word_embeddings
    ids, want = [5, 6, 7, 8, 9, 10], []
    for _ in range(5):
        t = torch.tensor([ids + want])
        with torch.no_grad():
            want.append(int(hf(input_ids=t, attention_mask=torch.ones_like(t)).logits[0, -1].argmax()))
    llm = LLM(str(tmp_path / "ckpt"), device="cpu", max_model_len=128, kvcache_block_size=16, num_kvcache_blocks=16, enforce_eager=True)
    got = llm.generate([ids], SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))[0]["token_ids"]
    llm.exit()
    assert got == want and len(set(want)) > 1
