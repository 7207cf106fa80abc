"""Reference arm of ``bench.py``: the unmodified reference engine, installed under
``baseline/_ref`` with ``pip install --no-deps --target``, driven through its own public API
(``LLM``, ``SamplingParams``, ``generate_prepared_image_inputs``) on the headline workload.

The reference needs a checkpoint directory, so this script writes one under the system
temp directory: ``config.json`` of the Qwen3-VL-8B architecture, random-init bf16 safetensors
shards with Hugging Face tensor names, and a synthetic word-level ``tokenizer.json`` plus
processor configs so that ``AutoTokenizer`` / ``AutoProcessor`` load offline.  Inputs are the
same synthetic patches and token ids the main arm uses, wrapped in the reference's
``ImageInputs``.  TPOT is ``(t(N tokens) - t(1 token)) / (N - 1)`` over two calls, timed with
CUDA events and the host clock.  Any failure is reported as an ``unavailable`` line.

The engine is built in the reference's own best documented mode for this workload first
(``benchmarks/bench_system.py:149-314``: the ``scaled_fp8_kv_compile_graph`` and
``scaled_fp8_kv_tuned_*_graph`` modes: 256-wide paged decode blocks, selective fp32 logits, fused
QK / add RMSNorm, fused M-RoPE, packed KV projection, compiled decode regions); a mode that does
not start on this image falls through to the next one and finally to the package defaults.  The
mode that ran is printed as ``config.reference_mode``; ``PRISM_REFERENCE_MODE`` pins one.
"""

from __future__ import annotations

import json
import os
import sys
import tempfile
import time
import traceback

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
SPECIAL = {151643: "<|endoftext|>", 151644: "<|im_start|>", 151645: "<|im_end|>", 151652: "<|vision_start|>",
           151653: "<|vision_end|>", 151654: "<|vision_pad|>", 151655: "<|image_pad|>", 151656: "<|video_pad|>"}


_TUNED = dict(logits_precision="selective_fp32", paged_decode_block_n=256)
_FUSED = dict(enable_fused_qk_rmsnorm=True, enable_fused_qk_mrope=True, enable_fused_add_rmsnorm=True,
              enable_packed_kv_projection=True)
# (name, extra LLM keyword arguments), fastest documented mode first
REFERENCE_MODES: list[tuple[str, dict]] = [
    ("scaled_fp8_kv_compile_graph", dict(execution_backend="compile_graph", decode_compile_region="stateless",
                                         decode_compile_mode="default", decode_compile_emulate_precision_casts=True,
                                         decode_compile_force_same_precision=True, allow_unsafe_decode_compile=True,
                                         **_TUNED, **_FUSED)),
    ("scaled_fp8_kv_tuned_kvproj_graph", dict(execution_backend="cuda_graph", **_TUNED, **_FUSED)),
    ("scaled_fp8_kv_tuned_graph", dict(execution_backend="cuda_graph", **_TUNED)),
    ("scaled_fp8_kv_graph (package defaults)", {}),
]


# Under tensor parallelism the reference requires ``logits_precision="model"`` (``config.py``: "tensor parallel
# execution requires logits_precision='model'") and its own tensor-parallel modes compile the attention region only
# (``benchmarks/bench_system.py:217-243``, ``tp2_tuned_graph`` / ``tp2_compile_graph``); KV stays scaled FP8, the
# configuration of this benchmark.
_TUNED_TP = dict(logits_precision="model", paged_decode_block_n=256)
REFERENCE_MODES_TP: list[tuple[str, dict]] = [
    ("scaled_fp8_kv_tp_compile_graph", dict(execution_backend="compile_graph", decode_compile_region="attention", **_TUNED_TP, **_FUSED)),
    ("scaled_fp8_kv_tp_tuned_graph", dict(execution_backend="cuda_graph", **_TUNED_TP, **_FUSED)),
    ("scaled_fp8_kv_tp_bn256_graph", dict(execution_backend="cuda_graph", **_TUNED_TP)),
    ("scaled_fp8_kv_graph (package defaults)", {}),
]


def reference_modes(world: int = 1) -> list[tuple[str, dict]]:
    modes = REFERENCE_MODES if world <= 1 else REFERENCE_MODES_TP
    pinned = os.environ.get("PRISM_REFERENCE_MODE")
    if pinned:
        chosen = [m for m in modes if m[0].split(" ")[0] == pinned]
        if not chosen:
            raise ValueError(f"PRISM_REFERENCE_MODE={pinned!r} is none of {[m[0].split(' ')[0] for m in modes]}")
        return chosen
    return list(modes)


def unavailable(why: str) -> None:
    print(json.dumps({"impl": "reference", "unavailable": " ".join(str(why).split())[:400]}), flush=True)


def write_checkpoint(path: str, arch, *, with_weights: bool = True) -> None:
    """Config, synthetic tokenizer / processor files and random-init weights."""
    import torch
    from tokenizers import Tokenizer, models, pre_tokenizers

    from prism_infer_b200.models.weights import iter_random_weights, save_checkpoint

    os.makedirs(path, exist_ok=True)
    marker = os.path.join(path, ".complete")
    if os.path.exists(marker):
        return
    vocab = {(SPECIAL.get(i) or f"t{i}"): i for i in range(arch.text.vocab_size)}
    tok = Tokenizer(models.WordLevel(vocab=vocab, unk_token="t0"))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    tok.save(os.path.join(path, "tokenizer.json"))
    template = ("{% for m in messages %}<|im_start|> {{ m['role'] }} {% if m['content'] is string %}{{ m['content'] }}"
                "{% else %}{% for c in m['content'] %}{% if c['type']=='image' %}<|vision_start|> <|image_pad|> <|vision_end|> "
                "{% elif c['type']=='video' %}<|vision_start|> <|video_pad|> <|vision_end|> {% else %}{{ c['text'] }}{% endif %}"
                "{% endfor %}{% endif %} <|im_end|> {% endfor %}{% if add_generation_prompt %}<|im_start|> assistant {% endif %}")
    with open(os.path.join(path, "tokenizer_config.json"), "w") as fh:
        json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "eos_token": "<|im_end|>", "pad_token": "<|endoftext|>",
                   "additional_special_tokens": list(SPECIAL.values()), "chat_template": template}, fh)
    common = {"processor_class": "Qwen3VLProcessor", "patch_size": 16, "temporal_patch_size": 2, "merge_size": 2,
              "image_mean": [0.5, 0.5, 0.5], "image_std": [0.5, 0.5, 0.5]}
    with open(os.path.join(path, "preprocessor_config.json"), "w") as fh:
        json.dump({**common, "image_processor_type": "Qwen2VLImageProcessorFast",
                   "size": {"shortest_edge": 65536, "longest_edge": 16777216}, "do_resize": True, "do_rescale": True,
                   "do_normalize": True, "do_convert_rgb": True}, fh)
    with open(os.path.join(path, "video_preprocessor_config.json"), "w") as fh:
        json.dump({**common, "video_processor_type": "Qwen3VLVideoProcessor",
                   "size": {"shortest_edge": 4096, "longest_edge": 25165824}, "do_sample_frames": False}, fh)
    if with_weights:
        dev = "cuda" if torch.cuda.is_available() else "cpu"
        save_checkpoint(path, arch, iter_random_weights(arch, dtype=torch.bfloat16, device=dev, seed=0), shard_bytes=2 << 30)
    else:
        with open(os.path.join(path, "config.json"), "w") as fh:
            json.dump(arch.to_hf_config(), fh)
    open(marker, "w").close()


def main(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return  # the reference starts its own worker ranks from one process
    if not os.path.isdir(os.path.join(REF, "prism_infer")):
        unavailable("reference is not installed under baseline/_ref (pip install --no-deps --target baseline/_ref <reference checkout>)")
        return
    try:
        import numpy as np
        import torch

        if not torch.cuda.is_available():
            unavailable("no CUDA device: the reference refuses to start without one")
            return
        sys.path.insert(0, ROOT)
        from prism_infer_b200.engine.vl_inputs import PatchProcessor, prepare_image_inputs
        from prism_infer_b200.models.architecture import Qwen3VLArch
        from prism_infer_b200.utils.tokenizer import IdTokenizer

        arch = Qwen3VLArch.qwen3_vl_8b()
        ckpt = os.path.join(tempfile.gettempdir(), "prism_ref_qwen3vl8b_random")
        write_checkpoint(ckpt, arch)
        # The reference starts its own worker ranks with its own tcp:// rendezvous.  Under torchrun the
        # elastic agent's variables must go, above all TORCHELASTIC_USE_AGENT_STORE: with it set,
        # init_process_group treats even rank 0 as a client of the agent's store and waits for a server
        # that does not exist on the reference's port.
        for k in list(os.environ):
            if k.startswith("TORCHELASTIC_") or k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "LOCAL_WORLD_SIZE", "GROUP_RANK",
                                                       "GROUP_WORLD_SIZE", "ROLE_RANK", "ROLE_WORLD_SIZE", "ROLE_NAME",
                                                       "MASTER_ADDR", "MASTER_PORT", "TORCH_NCCL_ASYNC_ERROR_HANDLING"):
                os.environ.pop(k, None)
        sys.path.insert(0, REF)
        from prism_infer import LLM, SamplingParams  # the unmodified reference
        from prism_infer.engine.vl_inputs import ImageInputs

        W, K = max(3, args.warmup), args.steps
        base = dict(tensor_parallel_size=args.gpus, max_model_len=4096, kvcache_block_size=256,
                    num_kvcache_blocks=max(16, args.batch * 12), compression_mode="scaled_fp8_kv",
                    max_num_seqs=max(args.batch, 1), max_num_batched_tokens=16384, max_chunk_size=8192,
                    cpu_kv_cache_ratio=0.0, enable_prefix_caching=False)
        rng = np.random.default_rng(0)
        proc = PatchProcessor(arch)
        tok = IdTokenizer(arch.text.vocab_size)

        prompt_tokens = [0]

        def make_inputs():
            images = [rng.integers(0, 256, (448, 448, 3), dtype=np.uint8) for _ in range(args.images)]
            mine = prepare_image_inputs(proc, tok, rng.integers(0, 150000, 32).tolist(), images)
            ids = torch.tensor([mine.input_ids], dtype=torch.long)
            prompt_tokens[0] = int(ids.shape[1])
            n_img = int((ids == arch.image_token_id).sum())
            return ImageInputs(input_ids=ids, attention_mask=torch.ones_like(ids), pixel_values=mine.pixel_values.to(torch.bfloat16),
                               image_grid_thw=torch.tensor(mine.image_grid_thw, dtype=torch.long),
                               image_token_id=arch.image_token_id, image_token_count=n_img, expected_image_tokens=n_img,
                               prompt_text="")

        def timed(max_tokens: int) -> tuple[float, float]:
            inputs = make_inputs()
            sp = SamplingParams(temperature=0.0, max_tokens=max_tokens, ignore_eos=True)
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            s.record()
            out = llm.generate_prepared_image_inputs(inputs, sp, use_tqdm=False)
            e.record()
            torch.cuda.synchronize()
            assert len(out["token_ids"]) == max_tokens, len(out["token_ids"])
            return s.elapsed_time(e), (time.perf_counter() - t0) * 1e3

        llm, mode_name, skipped = None, "", []
        for mode_name, extra in reference_modes(args.gpus):
            try:
                llm = LLM(ckpt, **base, **extra)
                timed(W + 1)  # warm-up: kernel JIT / compilation, graph replay paths
                break
            except Exception as exc:  # noqa: BLE001 - this mode does not start here: try the next one
                skipped.append(f"{mode_name}: {type(exc).__name__}: {' '.join(str(exc).split())[:160]}")
                if llm is not None:
                    try:
                        llm.exit()
                    except Exception:
                        pass
                llm = None
                import gc

                gc.collect()
                torch.cuda.empty_cache()
        if llm is None:
            unavailable("no reference mode started: " + " | ".join(skipped))
            return
        ttft_dev, ttft_wall = timed(1)
        full_dev, full_wall = timed(K + 1)
        tpot_dev = (full_dev - ttft_dev) / K
        tpot_wall = (full_wall - ttft_wall) / K
        print(json.dumps({
            "impl": "reference", "metric": "qwen3_vl_8b_decode_tpot_ms", "value": round(tpot_dev, 4), "unit": "ms/token",
            "n_gpus": args.gpus, "steps": K, "warmup": W, "ms_per_step": round(tpot_dev, 4), "higher_is_better": False,
            "scaling": "strong", "dtype": "bf16", "data": "synthetic (uniform-random images and token ids, random-init weights)",
            "config": {"model": "Qwen3-VL-8B (random init)", "global_batch": args.batch, "seq_len": prompt_tokens[0],
                       "images": f"{args.images}x448x448", "output_tokens": K + 1,
                       "kv": "scaled_fp8_kv", "parallelism": f"tp{args.gpus}", "decode": mode_name.split(" ")[0],
                       "reference_mode": mode_name, "reference_modes_skipped": skipped,
                       "timing": "(t(K+1 tokens) - t(1 token)) / K through generate_prepared_image_inputs"},
            "ttft_ms": round(ttft_wall, 2), "e2e": {"value": round(tpot_wall, 4), "unit": "ms/token"},
            "output_tok_per_s": round(args.batch * 1e3 / tpot_dev, 2),
        }), flush=True)
        try:
            llm.exit()
        except Exception:
            pass
    except BaseException as exc:  # noqa: BLE001 - every failure becomes an 'unavailable' line
        tb = traceback.format_exc().strip().splitlines()
        where = next((l.strip() for l in reversed(tb) if l.strip().startswith("File")), "")
        unavailable(f"{type(exc).__name__}: {exc} [{where}]")
