"""The engine on a B200: tiny model against the fp32 oracle, graph decode == eager decode."""

import numpy as np
import pytest
import torch

from prism_infer_b200 import LLM, SamplingParams
from prism_infer_b200.engine.vl_inputs import PatchProcessor, prepare_image_inputs
from prism_infer_b200.models.architecture import Qwen3VLArch
from prism_infer_b200.models.reference_model import ReferenceQwen3VL
from prism_infer_b200.models.weights import random_weights
from prism_infer_b200.ops import native
from prism_infer_b200.utils.tokenizer import load_tokenizer

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tiny(cuda_device):
    arch = Qwen3VLArch.tiny()
    # bf16-representable weights so the oracle (fp32) and the engine (bf16) hold the same values
    weights = {k: v.to(torch.bfloat16).float() for k, v in random_weights(arch, dtype=torch.float32, seed=0).items()}
    return arch, weights, ReferenceQwen3VL(arch, weights)


def _inputs(arch, n_text=24, seed=0):
    image = np.random.default_rng(seed).integers(0, 256, (224, 224, 3), dtype=np.uint8)
    g = torch.Generator().manual_seed(seed)
    text = torch.randint(0, 1000, (n_text,), generator=g).tolist()
    return prepare_image_inputs(PatchProcessor(arch), load_tokenizer("random:tiny", arch), text, [image])


def _agree(got, want_tokens, want_logits, margin=0.05):
    """Token-exact wherever the oracle's top-2 margin is not within bf16 noise."""
    for i, (g, w) in enumerate(zip(got, want_tokens)):
        if g != w:
            top2 = want_logits[i].topk(2).values
            assert float(top2[0] - top2[1]) < margin, f"step {i}: got {g}, oracle {w} with margin {float(top2[0] - top2[1])}"
            return  # later steps follow a different history
    assert len(got) == len(want_tokens)


@pytest.mark.parametrize("backend", ["eager", "cuda_graph"])
@pytest.mark.parametrize("mode", ["off", "scaled_fp8_kv"])
def test_tiny_image_prompt_on_gpu(tiny, backend, mode):
    arch, weights, oracle = tiny
    inputs = _inputs(arch)
    want, logits = oracle.generate_greedy(inputs.input_ids, 16, pixel_values=inputs.pixel_values,
                                          image_grid_thw=inputs.image_grid_thw, return_logits=True)
    llm = LLM("random:tiny", weights=weights, max_model_len=512, kvcache_block_size=256, num_kvcache_blocks=8,
              execution_backend=backend, compression_mode=mode, max_num_seqs=4, cpu_kv_cache_ratio=0.0)
    got = llm.generate_prepared_image_inputs(inputs, SamplingParams(temperature=0.0, max_tokens=16, ignore_eos=True))
    torch.cuda.synchronize()
    native.check_status()
    _agree(got["token_ids"], want, logits, margin=0.05 if mode == "off" else 0.3)
    llm.exit()


@pytest.fixture(scope="module")
def wide(cuda_device):
    """Production widths (hidden 4096, 32 / 8 heads of 128, M-RoPE 24/20/20, MLP 12288, vocabulary
    151936, vision hidden 1152 with 72-wide heads), two decoder and two vision layers."""
    arch = Qwen3VLArch.qwen3_vl_8b_2layer()
    # drawn on the device (1.8 G values take minutes on the host), bf16-representable, kept on the host
    weights = {k: v.to(torch.bfloat16).float().cpu() for k, v in random_weights(arch, dtype=torch.float32, device="cuda", seed=0).items()}
    return arch, weights, ReferenceQwen3VL(arch, weights)


@pytest.mark.parametrize("logits_precision", ["model", "selective_fp32"])
@pytest.mark.parametrize("backend", ["eager", "cuda_graph"])
def test_production_width_image_prompt_on_gpu(wide, backend, logits_precision):
    """The whole chain at the shapes the 8B model runs (split-K slabs, 256-token scaled-FP8 pages,
    GQA-4 decode, the 151936-row LM head; with ``selective_fp32`` the E4M3 candidate head and its exact
    rerank) against the fp32 oracle."""
    arch, weights, oracle = wide
    image = np.random.default_rng(5).integers(0, 256, (224, 224, 3), dtype=np.uint8)
    text = torch.randint(0, 150000, (24,), generator=torch.Generator().manual_seed(5)).tolist()
    inputs = prepare_image_inputs(PatchProcessor(arch), load_tokenizer("random:qwen3-vl-8b-2layer", arch), text, [image])
    want, logits = oracle.generate_greedy(inputs.input_ids, 16, pixel_values=inputs.pixel_values,
                                          image_grid_thw=inputs.image_grid_thw, return_logits=True)
    llm = LLM("random:qwen3-vl-8b-2layer", weights=weights, max_model_len=1024, kvcache_block_size=256, num_kvcache_blocks=6,
              execution_backend=backend, compression_mode="scaled_fp8_kv", max_num_seqs=2, cpu_kv_cache_ratio=0.0,
              logits_precision=logits_precision)
    assert (getattr(llm.runners.runner.model, "lm_head_fp8", None) is not None) == (logits_precision == "selective_fp32")
    got = llm.generate_prepared_image_inputs(inputs, SamplingParams(temperature=0.0, max_tokens=16, ignore_eos=True))
    torch.cuda.synchronize()
    native.check_status()
    _agree(got["token_ids"], want, logits, margin=0.3)
    llm.exit()


def test_production_width_chunked_prefill_and_prefix_hit_on_gpu(wide):
    """Later chunks of a chunked prefill and a request admitted on a prefix-cache hit attend over the paged cache: at
    head dimension 128 the keys are gathered from their scaled-FP8 pages and the tcgen05 kernel runs over them.
    Tokens against the fp32 oracle for both requests."""
    arch, weights, oracle = wide
    g = torch.Generator().manual_seed(9)
    prompt = torch.randint(0, 150000, (300,), generator=g).tolist()
    longer = prompt + torch.randint(0, 150000, (12,), generator=g).tolist()
    sp = SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)
    llm = LLM("random:qwen3-vl-8b-2layer", weights=weights, max_model_len=1024, kvcache_block_size=256, num_kvcache_blocks=8,
              execution_backend="cuda_graph", compression_mode="scaled_fp8_kv", max_num_seqs=2, cpu_kv_cache_ratio=0.0,
              max_num_batched_tokens=128, max_chunk_size=128)
    from prism_infer_b200 import ops

    calls = {"tc": 0}
    plain = ops.native.call

    def counting(name, *a):
        if name == "prism_paged_prefill_tc":
            calls["tc"] += 1
        return plain(name, *a)

    ops.native.call = counting
    try:
        for p in (prompt, longer):
            want, logits = oracle.generate_greedy(p, 5, return_logits=True)
            got = llm.generate([p], sp)[0]["token_ids"]
            torch.cuda.synchronize()
            native.check_status()
            _agree(got, want, logits, margin=0.3)
    finally:
        ops.native.call = plain
    # first request: chunks two and three of three, two layers each; second request: one prefill over the cached page
    assert calls["tc"] == 2 * 2 + 2, calls
    assert llm.metrics_snapshot()["engine"]["requests"][1]["cached_tokens"] == 256
    llm.exit()


def test_graph_decode_equals_eager_decode(tiny):
    arch, weights, _ = tiny
    prompts = [torch.randint(0, 1000, (n,), generator=torch.Generator().manual_seed(n)).tolist() for n in (9, 33, 70)]
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    outs = {}
    for backend in ("eager", "cuda_graph"):
        llm = LLM("random:tiny", weights=weights, max_model_len=512, kvcache_block_size=16, num_kvcache_blocks=64,
                  execution_backend=backend, compression_mode="scaled_fp8_kv", max_num_seqs=8, cpu_kv_cache_ratio=0.0)
        outs[backend] = [o["token_ids"] for o in llm.generate(prompts, sp)]
        llm.exit()
    assert outs["eager"] == outs["cuda_graph"]
    native.check_status()


def test_cooperative_layer_quanta_interleave_with_graph_decode(tiny):
    """A prompt arriving while another sequence decodes: its prefill runs one layer per quantum between graph decode
    steps; the tokens equal those of the engine without cooperative prefill."""
    arch, weights, _ = tiny
    first = torch.randint(0, 1000, (12,), generator=torch.Generator().manual_seed(1)).tolist()
    late = torch.randint(0, 1000, (150,), generator=torch.Generator().manual_seed(2)).tolist()
    outs = {}
    for cooperative in (False, True):
        llm = LLM("random:tiny", weights=weights, max_model_len=512, kvcache_block_size=16, num_kvcache_blocks=64,
                  execution_backend="cuda_graph", compression_mode="scaled_fp8_kv", max_num_seqs=8, cpu_kv_cache_ratio=0.0,
                  enable_cooperative_prefill=cooperative, cooperative_prefill_layer_quantum=1)
        a = llm.add_request(first, SamplingParams(temperature=0.0, max_tokens=16, ignore_eos=True))
        while llm.scheduler.num_decoding == 0:
            llm.step_result()
        b = llm.add_request(late, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
        done = {}
        while not llm.is_finished():
            for o in llm.step_result().outputs:
                if o.finished:
                    done[o.request_id] = list(o.token_ids)
        torch.cuda.synchronize()
        native.check_status()
        outs[cooperative] = (done[a], done[b])
        if cooperative:
            c = llm.cooperative_counters
            assert c["layer_quantum_prefills"] == 1 and c["layer_quanta"] == arch.text.num_layers and c["decode_steps_between_quanta"] >= 2
        llm.exit()
    assert outs[True] == outs[False]


def test_decode_run_ahead_gives_the_same_tokens(tiny):
    """Greedy decode with the next graph launched before this step's tokens are read: same tokens as without, most
    steps taken over from the launch that ran ahead (page boundaries, the first step and the batch changes are not),
    sampled rows never run ahead."""
    arch, weights, _ = tiny
    prompts = [torch.randint(0, 1000, (n,), generator=torch.Generator().manual_seed(n)).tolist() for n in (9, 33)]
    outs, meta = {}, {}
    for ahead in (False, True):
        llm = LLM("random:tiny", weights=weights, max_model_len=512, kvcache_block_size=16, num_kvcache_blocks=64,
                  execution_backend="cuda_graph", compression_mode="scaled_fp8_kv", max_num_seqs=8, cpu_kv_cache_ratio=0.0,
                  enable_decode_run_ahead=ahead)
        # 41 tokens: the last decode step's rows sit at offsets 0 and 8 of their 16-token pages, so a launch runs ahead
        # of it and is left unobserved when the sequences finish
        outs[ahead] = [o["token_ids"] for o in llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=41, ignore_eos=True))]
        sampled = llm.generate([prompts[0]], SamplingParams(temperature=0.8, max_tokens=8, ignore_eos=True))
        assert len(sampled[0]["token_ids"]) == 8
        meta[ahead] = llm.graph_metadata()["decode_run_ahead"]
        torch.cuda.synchronize()
        native.check_status()
        llm.exit()
    assert outs[True] == outs[False]
    assert meta[False] == {"taken": 0, "discarded": 0}
    assert meta[True]["taken"] >= 25 and meta[True]["discarded"] >= 1


def test_prefix_hit_and_compaction_on_gpu(tiny):
    arch, weights, _ = tiny
    llm = LLM("random:tiny", weights=weights, max_model_len=512, kvcache_block_size=16, num_kvcache_blocks=64,
              compression_mode="visual_compact_scaled_fp8", visual_pruning_keep_ratio=0.5, visual_pruning_min_keep_tokens=8,
              max_num_seqs=4, cpu_kv_cache_ratio=0.0)
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    a, b = _inputs(arch, 5, seed=7), _inputs(arch, 9, seed=7)
    b.input_ids[-9:] = [5, 6, 7, 8, 9, 10, 11, 12, 13]
    r1 = llm.generate_prepared_image_inputs(a, sp)
    llm.generate_prepared_image_inputs(b, sp)
    r3 = llm.generate_prepared_image_inputs(a, sp)
    meta = llm.multimodal_prefix_cache_metadata()
    assert meta["hits"] == 2 and meta["stores"] == 1
    assert r1["token_ids"] == r3["token_ids"]
    native.check_status()
    llm.exit()


def test_kv_arena_is_sized_from_a_measured_prefill(tiny):
    """Without an explicit page count the runner measures the activation peak of a full prefill step
    and gives the rest of the memory budget to the KV arena."""
    arch, weights, _ = tiny
    llm = LLM("random:tiny", weights=weights, max_model_len=512, kvcache_block_size=64, max_num_batched_tokens=512,
              gpu_memory_utilization=0.05, max_num_seqs=2, cpu_kv_cache_ratio=0.0)
    meta = llm.graph_metadata()
    sizing = meta["kv_sizing"]
    assert sizing is not None and sizing["warmup_tokens"] == 512 and sizing["activation_peak_bytes"] > 0
    assert meta["kv_pages"] >= 1 and meta["kv_pages"] == max(1, sizing["budget_bytes"] // meta["kv_bytes_per_page"])
    out = llm.generate([[1, 2, 3, 4]], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    assert len(out[0]["token_ids"]) == 4
    native.check_status()
    llm.exit()


def test_temperature_sampling_runs_in_graph(tiny):
    arch, weights, _ = tiny
    llm = LLM("random:tiny", weights=weights, max_model_len=256, kvcache_block_size=16, num_kvcache_blocks=32,
              max_num_seqs=4, cpu_kv_cache_ratio=0.0)
    outs = llm.generate([[1, 2, 3], [4, 5, 6, 7]], [SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True),
                                                    SamplingParams(temperature=1.5, max_tokens=5, ignore_eos=True)])
    assert all(len(o["token_ids"]) == 5 for o in outs)
    llm.exit()


def test_smoke_entry(cuda_device):
    import __graft_entry__

    __graft_entry__.smoke()


def test_attention_strategy_compaction_on_gpu(tiny, monkeypatch):
    """The attention pruning strategy on the device: K rows written back by the fused QK-norm /
    rotary kernel feed the scorer, the highest-scored visual tokens keep their rows, the question's
    rows move down in the same compaction, and decoding agrees with the oracle that masks the
    dropped keys for generated tokens."""
    from prism_infer_b200.models import reference_model

    arch, weights, oracle = tiny
    inp = _inputs(arch, 7, seed=11)
    L = len(inp.input_ids)
    llm = LLM("random:tiny", weights=weights, max_model_len=512, kvcache_block_size=16, num_kvcache_blocks=64,
              compression_mode="visual_compact", visual_pruning_strategy="attention", visual_pruning_keep_ratio=0.5,
              visual_pruning_min_keep_tokens=4, visual_pruning_attention_last_n_layers=2, max_num_seqs=4, cpu_kv_cache_ratio=0.0)
    layouts, seen = [], []
    commit = llm.executor.bm.commit_compaction
    monkeypatch.setattr(llm.executor.bm, "commit_compaction", lambda seq, plan: (layouts.append(plan.layout), commit(seq, plan))[1])
    take = llm.runners.runner.take_visual_scores
    llm.runners.runner.take_visual_scores = lambda: (lambda s: (seen.append(s), s)[1])(take())
    got = llm.generate_prepared_image_inputs(inp, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))["token_ids"]
    torch.cuda.synchronize()
    native.check_status()
    assert llm.executor.attention_counters == {"scored": 1, "uniform_fallback": 0}
    llm.exit()
    (layout,) = layouts
    visual = [i for i, t in enumerate(inp.input_ids) if t == arch.image_token_id]
    kept = [p for p in layout.retained_positions if p in set(visual)]
    (scores,) = [s for s in seen if s][0].values()
    keep = -(-len(visual) // 2)
    assert len(kept) == keep and kept == sorted(sorted(visual, key=lambda i: (-scores[i], i))[:keep])
    assert all(0.0 <= v <= 1.0 for v in scores.values())

    dropped = torch.tensor(sorted(set(visual) - set(kept)))
    real_sdpa = reference_model.F.scaled_dot_product_attention

    def masked_sdpa(q, k, v, attn_mask=None, is_causal=False, **kw):
        if not is_causal:
            return real_sdpa(q, k, v, attn_mask=attn_mask, **kw)
        S = q.shape[-2]
        allowed = torch.ones(S, S, dtype=torch.bool, device=q.device).tril()
        if S > L:
            allowed[L:, dropped.to(q.device)] = False
        return real_sdpa(q, k, v, attn_mask=allowed)

    monkeypatch.setattr(reference_model.F, "scaled_dot_product_attention", masked_sdpa)
    want, logits = oracle.generate_greedy(inp.input_ids, 8, pixel_values=inp.pixel_values, image_grid_thw=inp.image_grid_thw,
                                          return_logits=True)
    monkeypatch.setattr(reference_model.F, "scaled_dot_product_attention", real_sdpa)
    _agree(got, want, logits, margin=0.05)


def test_vision_tower_graph_replay_equals_eager(tiny):
    """``enable_vision_tensor_cudagraph``: the tower is captured per grid shape and replayed for
    later media of that shape; tokens are those of the eager tower, bit for bit (same kernels)."""
    arch, weights, _ = tiny
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    reqs = [_inputs(arch, 5, seed=21), _inputs(arch, 6, seed=22), _inputs(arch, 4, seed=23)]
    outs = {}
    for graphs in (False, True):
        llm = LLM("random:tiny", weights=weights, max_model_len=512, kvcache_block_size=16, num_kvcache_blocks=64,
                  max_num_seqs=4, cpu_kv_cache_ratio=0.0, enable_prefix_caching=False, enable_vision_tensor_cudagraph=graphs)
        outs[graphs] = [llm.generate_prepared_image_inputs(r, sp)["token_ids"] for r in reqs]
        meta = llm.graph_metadata()["vision_graphs"]
        assert meta == ({"entries": 1, "captures": 1, "replays": 2} if graphs else {"entries": 0, "captures": 0, "replays": 0})
        torch.cuda.synchronize()
        native.check_status()
        llm.exit()
    assert outs[True] == outs[False]

