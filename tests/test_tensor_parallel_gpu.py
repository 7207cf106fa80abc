"""Tensor parallelism on real GPUs (needs at least two): TP2 against TP1 token for token,
fused-exchange path against the NCCL baseline path."""

import os

import pytest
import torch

from prism_infer_b200 import LLM, SamplingParams
from prism_infer_b200.models.architecture import Qwen3VLArch
from prism_infer_b200.models.weights import random_weights

pytestmark = [pytest.mark.gpu, pytest.mark.distributed]


def _run(tp, comm, weights, prompts, sp, backend="cuda_graph"):
    os.environ["PRISM_TP_COMM"] = comm
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    llm = LLM("random:tiny", weights=weights, tensor_parallel_size=tp, max_model_len=512, kvcache_block_size=16,
              num_kvcache_blocks=64, execution_backend=backend, compression_mode="scaled_fp8_kv", max_num_seqs=4,
              cpu_kv_cache_ratio=0.0, tensor_parallel_timeout_seconds=60)
    try:
        return [o["token_ids"] for o in llm.generate(prompts, sp)]
    finally:
        llm.exit()


@pytest.mark.timeout(600)
def test_tp2_matches_tp1_on_gpu(cuda_device):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    arch = Qwen3VLArch.tiny()
    weights = {k: v.to(torch.bfloat16).float() for k, v in random_weights(arch, dtype=torch.float32, seed=0).items()}
    prompts = [list(range(10, 19)), list(range(200, 240))]
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    base = _run(1, "nccl", weights, prompts, sp)
    nccl = _run(2, "nccl", weights, prompts, sp)
    fused = _run(2, "fused", weights, prompts, sp)
    assert nccl == fused, "fused exchange and NCCL all-reduce disagree"
    # TP changes the summation order of row-parallel GEMMs, so allow a late divergence only
    for b, f in zip(base, fused):
        assert b[:3] == f[:3]


@pytest.mark.timeout(600)
def test_tp2_fused_prefill_matches_nccl_prefill(cuda_device):
    """Prompts longer than the decode-sized threshold: the prefill runs through the fused GEMM ->
    reduce-scatter / reduce + norm -> all-gather kernels and must produce the tokens of the NCCL
    all-reduce arm (first tokens exactly; later ones may differ by summation order)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    arch = Qwen3VLArch.tiny()
    weights = {k: v.to(torch.bfloat16).float() for k, v in random_weights(arch, dtype=torch.float32, seed=0).items()}
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(5, 900, (n,), generator=g).tolist() for n in (300, 150, 421)]
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)

    def run(fused_prefill: bool):
        os.environ["PRISM_TP_PREFILL_FUSED"] = "1" if fused_prefill else "0"
        import prism_infer_b200.ops as ops_mod

        ops_mod.TP_PREFILL_FUSED = fused_prefill  # the driver rank imported ops already; workers read the variable
        return _run(2, "fused", weights, prompts, sp)

    try:
        plain = run(False)
        fused = run(True)
    finally:
        os.environ.pop("PRISM_TP_PREFILL_FUSED", None)
    for p, f in zip(plain, fused):
        assert p[:2] == f[:2], (p, f)
