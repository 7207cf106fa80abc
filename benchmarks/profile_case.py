"""Run one small, fixed kernel case a few times, for Nsight Compute captures.

The inputs are larger than the 126 MB L2 where bandwidth matters but only a few hundred MB
in total, and only a handful of launches run, so a ``--set full`` capture of one kernel ends
by itself in about a minute.

    python benchmarks/profile_case.py gemm_decode      # qkv-shaped weight-streaming GEMM, 1 token, split-K
    python benchmarks/profile_case.py gemm_prefill     # 2048 x 4096 x 6144 bf16 GEMM
    python benchmarks/profile_case.py gemm_dual        # dual-accumulator gate/up GEMM + SwiGLU, 2048 tokens
    python benchmarks/profile_case.py decode_attention # scaled-FP8 paged decode, batch 32, ctx 2048
    python benchmarks/profile_case.py prefill_attention
    python benchmarks/profile_case.py add_rmsnorm
    python benchmarks/profile_case.py decode_step 128  # ONE engine decode step at that batch inside cudaProfilerStart/Stop
                                                       # (launch list with --profile-from-start off; full-size model)
"""

from __future__ import annotations

import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from prism_infer_b200 import ops  # noqa: E402


def decode_step(batch: int) -> None:
    """``batch`` one-image requests on the 8B model, stepped until all of them decode; one further
    step runs between ``cudaProfilerStart`` and ``cudaProfilerStop``."""
    import numpy as np

    from prism_infer_b200 import LLM, SamplingParams
    from prism_infer_b200.engine.vl_inputs import PatchProcessor, prepare_image_inputs

    llm = LLM("random:qwen3-vl-8b", max_model_len=4096, kvcache_block_size=256, num_kvcache_blocks=max(64, batch * 4),
              compression_mode="scaled_fp8_kv", max_num_seqs=batch, max_num_batched_tokens=16384, max_chunk_size=2048,
              cpu_kv_cache_ratio=0.0, enable_prefix_caching=False)
    rng = np.random.default_rng(0)
    proc = PatchProcessor(llm.arch)
    sp = SamplingParams(temperature=0.0, max_tokens=64, ignore_eos=True)
    for _ in range(batch):
        inp = prepare_image_inputs(proc, llm.tokenizer, rng.integers(0, 150000, 32).tolist(),
                                   [rng.integers(0, 256, (448, 448, 3), dtype=np.uint8)])
        llm.add_prepared_image_request(inp, sp)
    while llm.scheduler.num_decoding < batch:
        llm.step_result()
    for _ in range(4):
        llm.step_result()
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    llm.step_result()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    print("done decode_step", batch)
    llm.exit()


def main() -> None:
    case = sys.argv[1] if len(sys.argv) > 1 else "gemm_decode"
    reps = int(sys.argv[2]) if len(sys.argv) > 2 else 4
    if case == "decode_step":
        decode_step(reps if len(sys.argv) > 2 else 128)
        return
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(0)

    def rnd(*shape, scale=1.0):
        return (torch.randn(*shape, generator=g, device=dev) * scale).to(torch.bfloat16)

    if case == "gemm_decode":
        ws = [rnd(6144, 4096, scale=0.02) for _ in range(4)]  # 4 x 50 MB: every launch misses L2
        x = rnd(1, 4096)
        for i in range(reps):
            ops.linear_partial(x, ws[i % 4], 3)
    elif case == "gemm_prefill":
        w, x = rnd(6144, 4096, scale=0.02), rnd(2048, 4096)
        for _ in range(reps):
            ops.linear(x, w)
    elif case in ("gemm_vit_fc1", "gemm_vit_fc1_tiled"):
        # vision-tower MLP up-projection: 6272 patches, 1152 -> 4304, bias + GELU(tanh); the
        # "_tiled" form forces the one-tile-per-CTA kernel (bn=256)
        w, x, b = rnd(4304, 1152, scale=0.03), rnd(6272, 1152), rnd(4304)
        for _ in range(reps):
            ops.linear(x, w, bias=b, act="gelu_tanh", bn=256 if case.endswith("tiled") else 0)
    elif case == "gemm_vit_proj":
        # vision-tower attention output projection with bias and in-place residual add
        w, x, b, res = rnd(1152, 1152, scale=0.03), rnd(6272, 1152), rnd(1152), rnd(6272, 1152)
        for _ in range(reps):
            ops.linear(x, w, bias=b, residual=res, out=res)
    elif case == "gemm_dual":
        w, x = rnd(24576, 4096, scale=0.02), rnd(2048, 4096)
        for _ in range(reps):
            ops.gate_up_swiglu(x, w)
    elif case == "decode_attention":
        B, ctx, page = 32, 2048, 256
        cache = ops.KVCache(1, B * ctx // page, 8, page, 128, ops.KV_FP8_SCALED, dev)
        cache.payload.view(torch.uint8).random_(0, 120)
        cache.scales.uniform_(0.005, 0.02)
        bt = torch.arange(B * ctx // page, dtype=torch.int32, device=dev).view(B, -1)
        cl = torch.full((B,), ctx, dtype=torch.int32, device=dev)
        q = rnd(B, 32, 128)
        for _ in range(reps):
            ops.paged_decode_attention(q, cache, 0, bt, cl)
    elif case == "prefill_attention":
        T, page = 2048, 256
        cache = ops.KVCache(1, T // page, 8, page, 128, ops.KV_FP8_SCALED, dev)
        cache.payload.view(torch.uint8).random_(0, 120)
        cache.scales.uniform_(0.005, 0.02)
        bt = torch.arange(T // page, dtype=torch.int32, device=dev).view(1, -1)
        q = rnd(T, 32, 128)
        cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
        kv = torch.tensor([T], dtype=torch.int32, device=dev)
        for _ in range(reps):
            ops.paged_prefill_attention(q, cache, 0, cu, kv, bt, T)
    elif case == "attention_tc":
        # causal prefill attention over fresh bf16 K/V rows (views of a packed projection), tcgen05 kernel
        T, Hq, Hkv, D = 2048, 32, 8, 128
        qkv = rnd(T, (Hq + 2 * Hkv) * D)
        heads = qkv.view(T, Hq + 2 * Hkv, D)
        q = heads[:, :Hq].contiguous()
        cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
        for _ in range(reps):
            ops.varlen_attention(q, heads[:, Hq:Hq + Hkv], heads[:, Hq + Hkv:], cu, T, causal=True)
    elif case == "add_rmsnorm":
        parts = torch.randn(4, 8, 4096, device=dev)
        res, w = rnd(8, 4096), rnd(4096)
        for _ in range(reps):
            ops.add_rmsnorm(w, 1e-6, partials=parts, residual=res)
    else:
        raise SystemExit(f"unknown case {case}")
    torch.cuda.synchronize()
    print("done", case)


if __name__ == "__main__":
    main()
