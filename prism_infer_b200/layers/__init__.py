"""Module-level building blocks (reference ``prism_infer/layers/``): normalisation, activation,
rotary tables, tensor-parallel linear layers, vocabulary-parallel embedding and head, the
attention router and the sampler, each a thin ``nn.Module`` over the kernels in ``ops``."""

from .attention_router import Attention
from .basic import RMSNorm, RotaryEmbedding, SiluAndMul, apply_rotary_emb, get_rope
from .parallel_linear import (ColumnParallelLinear, LinearBase, MergedColumnParallelLinear, QKVParallelLinear,
                              ReplicatedLinear, RowParallelLinear, divide)
from .sampling import Sampler
from .vocab import ParallelLMHead, VocabParallelEmbedding

__all__ = [
    "Attention", "RMSNorm", "RotaryEmbedding", "SiluAndMul", "apply_rotary_emb", "get_rope", "ColumnParallelLinear",
    "LinearBase", "MergedColumnParallelLinear", "QKVParallelLinear", "ReplicatedLinear", "RowParallelLinear", "divide",
    "Sampler", "ParallelLMHead", "VocabParallelEmbedding",
]
