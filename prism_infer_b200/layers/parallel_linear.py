"""Tensor-parallel linear modules (reference ``prism_infer/layers/linear.py:9-190``).

Every class stores its rank-local weight ``[out_local, in_local]`` and a ``weight_loader`` that
cuts this rank's part out of a full checkpoint tensor, so the generic safetensors loader can
fill a model built from these modules.  The rank and world size come from the ``comm`` object
handed to the constructor (the engine's collective hooks; the default is the single-rank
no-op), not from a process-global group, so several differently sharded modules can live in one
process - which is how the CPU tests build all ranks side by side.

``forward`` accepts any number of leading dimensions and runs ``ops.linear`` - the tcgen05 GEMM
on a CUDA tensor, ``F.linear`` on a CPU tensor.  ``RowParallelLinear`` sums its partial results
over the ranks with ``comm.reduce_dense`` (NCCL all-reduce, or the one-shot exchange of the
fused communicator); the bias is added by rank 0 only so the sum counts it once.
"""

from __future__ import annotations

from typing import Sequence

import torch
from torch import nn

from .. import ops
from ..models.qwen3_vl import TPComm


def divide(numerator: int, denominator: int) -> int:
    """Exact quotient of a tensor-parallel dimension; anything else is a configuration error."""
    for name, v, low in (("numerator", numerator, 0), ("denominator", denominator, 1)):
        if isinstance(v, bool) or not isinstance(v, int) or v < low:
            kind = "a non-negative" if low == 0 else "a positive"
            raise ValueError(f"{name} must be {kind} integer, got {v!r}")
    if numerator % denominator:
        raise ValueError(f"tensor-parallel dimension {numerator} is not divisible by {denominator}")
    return numerator // denominator


class LinearBase(nn.Module):
    """Parameter storage; ``tp_dim`` is the weight dimension that is sharded (0 = output rows,
    1 = input columns, ``None`` = replicated)."""

    def __init__(self, in_local: int, out_local: int, bias: bool, tp_dim: int | None, comm: TPComm | None) -> None:
        super().__init__()
        self.comm = comm if comm is not None else TPComm()
        self.tp_rank, self.tp_size, self.tp_dim = self.comm.rank, self.comm.size, tp_dim
        self.weight = nn.Parameter(torch.empty(out_local, in_local), requires_grad=False)
        self.weight.weight_loader = self.weight_loader
        if bias:
            self.bias = nn.Parameter(torch.empty(out_local), requires_grad=False)
            self.bias.weight_loader = self.weight_loader
        else:
            self.register_parameter("bias", None)

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor, *shard) -> None:
        raise NotImplementedError

    def _rank_slice(self, full: torch.Tensor, dim: int) -> torch.Tensor:
        """This rank's equal share of ``full`` along ``dim`` (a bias has only dimension 0)."""
        dim = min(dim, full.dim() - 1)
        n = divide(full.shape[dim], self.tp_size)
        return full.narrow(dim, self.tp_rank * n, n)

    def _project(self, x: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor:
        lead = x.shape[:-1]
        y = ops.linear(x.reshape(-1, x.shape[-1]), self.weight, bias=bias)
        return y.view(*lead, self.weight.shape[0])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self._project(x, self.bias)


class ReplicatedLinear(LinearBase):
    """The same full projection on every rank."""

    def __init__(self, input_size: int, output_size: int, bias: bool = False, *, comm: TPComm | None = None) -> None:
        super().__init__(input_size, output_size, bias, None, comm)

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor) -> None:
        param.data.copy_(loaded_weight)


class ColumnParallelLinear(LinearBase):
    """Output features split over the ranks; the result stays sharded."""

    def __init__(self, input_size: int, output_size: int, bias: bool = False, *, comm: TPComm | None = None) -> None:
        size = (comm or TPComm()).size
        super().__init__(input_size, divide(output_size, size), bias, 0, comm)

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor) -> None:
        param.data.copy_(self._rank_slice(loaded_weight, 0))


class MergedColumnParallelLinear(ColumnParallelLinear):
    """Several column-parallel projections of one input stored as one weight (gate and up):
    rank-local layout ``[part0/tp | part1/tp | ...]``, each part loaded by its index."""

    def __init__(self, input_size: int, output_sizes: Sequence[int], bias: bool = False, *, comm: TPComm | None = None) -> None:
        self.output_sizes = tuple(output_sizes)
        if not self.output_sizes:
            raise ValueError("MergedColumnParallelLinear requires at least one output shard")
        size = (comm or TPComm()).size
        for part in self.output_sizes:
            divide(part, size)
        super().__init__(input_size, sum(self.output_sizes), bias, comm=comm)

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor, loaded_shard_id: int) -> None:
        i = loaded_shard_id
        if isinstance(i, bool) or not isinstance(i, int) or not 0 <= i < len(self.output_sizes):
            raise ValueError(f"invalid merged projection shard id: {i!r}")
        begin = sum(self.output_sizes[:i]) // self.tp_size
        rows = self.output_sizes[i] // self.tp_size
        param.data.narrow(0, begin, rows).copy_(self._rank_slice(loaded_weight, 0))


class QKVParallelLinear(ColumnParallelLinear):
    """Packed grouped-query attention projection: rank-local rows are this rank's query heads,
    then its key heads, then its value heads."""

    def __init__(self, hidden_size: int, head_size: int, total_num_heads: int, total_num_kv_heads: int | None = None,
                 bias: bool = False, *, comm: TPComm | None = None) -> None:
        size = (comm or TPComm()).size
        total_num_kv_heads = total_num_kv_heads or total_num_heads
        self.head_size = head_size
        self.num_heads = divide(total_num_heads, size)
        self.num_kv_heads = divide(total_num_kv_heads, size)
        super().__init__(hidden_size, (total_num_heads + 2 * total_num_kv_heads) * head_size, bias, comm=comm)

    def shard_rows(self, shard: str) -> tuple[int, int]:
        """``(first row, row count)`` of ``"q"``, ``"k"`` or ``"v"`` in the rank-local weight."""
        q, kv = self.num_heads * self.head_size, self.num_kv_heads * self.head_size
        try:
            return {"q": (0, q), "k": (q, kv), "v": (q + kv, kv)}[shard]
        except (KeyError, TypeError):
            raise ValueError(f"invalid QKV projection shard id: {shard!r}") from None

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor, loaded_shard_id: str) -> None:
        begin, rows = self.shard_rows(loaded_shard_id)
        param.data.narrow(0, begin, rows).copy_(self._rank_slice(loaded_weight, 0))


class RowParallelLinear(LinearBase):
    """Input features split over the ranks; partial results are summed across them."""

    def __init__(self, input_size: int, output_size: int, bias: bool = False, *, comm: TPComm | None = None) -> None:
        size = (comm or TPComm()).size
        super().__init__(divide(input_size, size), output_size, bias, 1, comm)

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor) -> None:
        if loaded_weight.dim() == 1:  # the bias is not sharded
            param.data.copy_(loaded_weight)
        else:
            param.data.copy_(self._rank_slice(loaded_weight, 1))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self._project(x, self.bias if self.tp_rank == 0 else None)
        if self.tp_size > 1:
            lead = y.shape
            y = self.comm.reduce_dense(y.reshape(-1, lead[-1])).view(lead)
        return y
