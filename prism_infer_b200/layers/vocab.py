"""Vocabulary-parallel embedding and output head modules (reference
``prism_infer/layers/embed_head.py:11-125``).

The vocabulary is cut into equal contiguous ranges, one per rank.  The embedding looks up the
ids that fall in its own range (``ops.embed`` writes zeros for the others in the same kernel)
and the ranks' results are summed; the head multiplies by its range of the output matrix and
either gathers the logits on every rank's behalf (``forward`` returns them on rank 0, ``None``
elsewhere) or, for greedy decoding, exchanges one ``(value, id)`` pair per row and picks the
global arg-max (``compute_greedy_tokens``; ties go to the lowest id, so the result equals the
arg-max over the gathered logits).
"""

from __future__ import annotations

import torch
from torch import nn

from .. import ops
from ..models.qwen3_vl import TPComm
from .parallel_linear import divide


class VocabParallelEmbedding(nn.Module):
    def __init__(self, num_embeddings: int, embedding_dim: int, *, comm: TPComm | None = None) -> None:
        super().__init__()
        for name, v in (("num_embeddings", num_embeddings), ("embedding_dim", embedding_dim)):
            if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
                raise ValueError(f"{name} must be a positive integer, got {v!r}")
        self.comm = comm if comm is not None else TPComm()
        self.tp_rank, self.tp_size = self.comm.rank, self.comm.size
        self.num_embeddings = num_embeddings
        self.num_embeddings_per_partition = divide(num_embeddings, self.tp_size)
        self.vocab_start_idx = self.tp_rank * self.num_embeddings_per_partition
        self.vocab_end_idx = self.vocab_start_idx + self.num_embeddings_per_partition
        self.weight = nn.Parameter(torch.empty(self.num_embeddings_per_partition, embedding_dim), requires_grad=False)
        self.weight.weight_loader = self.weight_loader

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor) -> None:
        param.data.copy_(loaded_weight.narrow(0, self.vocab_start_idx, param.shape[0]))

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        flat = ids.reshape(-1).to(torch.int64)
        y = ops.embed(flat, self.weight, vocab_start=self.vocab_start_idx)
        if self.tp_size > 1:
            y = self.comm.reduce_dense(y)
        return y.view(*ids.shape, self.weight.shape[1])


class ParallelLMHead(VocabParallelEmbedding):
    """``select_prefill_tokens``: when ``forward`` is given ``last_rows`` (the row of each
    sequence's last prompt token in a flattened prefill batch) only those rows are projected."""

    def __init__(self, num_embeddings: int, embedding_dim: int, bias: bool = False, select_prefill_tokens: bool = True, *,
                 comm: TPComm | None = None) -> None:
        if bias:
            raise ValueError("ParallelLMHead does not support bias")
        if not isinstance(select_prefill_tokens, bool):
            raise TypeError("select_prefill_tokens must be a boolean")
        super().__init__(num_embeddings, embedding_dim, comm=comm)
        self.select_prefill_tokens = select_prefill_tokens

    def _rows(self, x: torch.Tensor, last_rows: torch.Tensor | None) -> torch.Tensor:
        if last_rows is not None and self.select_prefill_tokens:
            x = x.index_select(0, last_rows.to(torch.int64))
        return x.contiguous()

    def _local_logits(self, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(x, self.weight).float()

    def forward(self, x: torch.Tensor, last_rows: torch.Tensor | None = None) -> torch.Tensor | None:
        logits = self._local_logits(self._rows(x, last_rows))
        if self.tp_size == 1:
            return logits
        full = self.comm.gather_logits(logits)
        return full if self.tp_rank == 0 else None

    def compute_greedy_tokens(self, x: torch.Tensor, last_rows: torch.Tensor | None = None) -> torch.Tensor:
        logits = self._local_logits(self._rows(x, last_rows))
        best = torch.empty(logits.shape[0], dtype=torch.float32, device=logits.device)
        ids = ops.sample(logits, None, vocab_offset=self.vocab_start_idx, out_val=best)
        return self.comm.greedy_merge(best, ids) if self.tp_size > 1 else ids
