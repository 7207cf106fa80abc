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
