"""Tensor-parallel collectives behind the model's ``TPComm`` hooks.

* ``NcclComm``: the baseline arm, what the reference does (``dist.all_reduce`` after every
  row-parallel GEMM, ``prism_infer/layers/linear.py:186-190``; vocabulary-parallel embedding
  all-reduce and distributed greedy arg-max, ``prism_infer/layers/embed_head.py:49-125``).
* ``FusedComm``: the product path for decode-sized steps (at most 128 tokens).  The
  row-parallel GEMM writes its fp32 partial tiles straight into every rank's slab buffer
  over NVLink from its epilogue, each element as one 8-byte word {value, sequence number}
  (``prism_gemm_wx_push``); the following add+RMSNorm kernel polls the words until they
  carry this exchange's sequence number, sums the ``tp * splits`` slabs in rank order
  (bitwise identical on every rank) and normalises (``prism_add_rmsnorm_packed``).  No NCCL
  call, no separate all-reduce kernel, no fence or flag round trip; two exchange slots are
  used alternately (a rank can only reach the next use of a slot after every peer has
  consumed the previous one, because the exchange in between needs all peers' data).  The
  greedy token is agreed on by a one-kernel (value, id) exchange.  Prefill-sized steps fall
  back to the NCCL path.
"""

from __future__ import annotations


import torch
import torch.distributed as dist

from .. import ops
from ..models.qwen3_vl import SMALL_T, TPComm
from ..ops import native
from . import symm


class NcclComm(TPComm):
    def __init__(self, rank: int, size: int, group=None) -> None:
        self.rank, self.size, self.group = rank, size, group

    def begin_step(self) -> None:
        return None

    def reduce_partials(self, partials: torch.Tensor) -> torch.Tensor:
        total = partials.sum(0, keepdim=True) if partials.shape[0] > 1 else partials
        dist.all_reduce(total, group=self.group)
        return total

    def reduce_dense(self, x: torch.Tensor) -> torch.Tensor:
        dist.all_reduce(x, group=self.group)
        return x

    def greedy_merge(self, local_val: torch.Tensor, local_id: torch.Tensor) -> torch.Tensor:
        packed = torch.stack((local_val.double(), local_id.double()))  # ids < 2**53 are exact
        gathered = [torch.empty_like(packed) for _ in range(self.size)]
        dist.all_gather(gathered, packed, group=self.group)
        allv = torch.stack([g[0] for g in gathered])  # [tp, B]
        alli = torch.stack([g[1] for g in gathered])
        best = allv.max(0).values
        cand = torch.where(allv == best[None], alli, torch.full_like(alli, float("inf")))
        return cand.min(0).values.long()

    def gather_logits(self, logits: torch.Tensor) -> torch.Tensor:
        parts = [torch.empty_like(logits) for _ in range(self.size)]
        dist.all_gather(parts, logits.contiguous(), group=self.group)
        return torch.cat(parts, dim=-1)

    def all_gather_rows(self, x: torch.Tensor) -> torch.Tensor:
        parts = [torch.empty_like(x) for _ in range(self.size)]
        dist.all_gather(parts, x.contiguous(), group=self.group)
        return torch.cat(parts, dim=0)

    def row_parallel(self, x: torch.Tensor, w: torch.Tensor, stages: int = 0):
        T = x.shape[0]
        if T <= SMALL_T and x.is_cuda:
            parts = ops.linear_partial(x, w, ops.choose_splits(w.shape[0], w.shape[1], T), stages=stages)
            return None, self.reduce_partials(parts), None
        y = ops.linear(x, w)
        return self.reduce_dense(y), None, None

    def add_rmsnorm(self, weight, eps, dense, partials, ticket, residual, extra=None, extra_index=None):
        return ops.add_rmsnorm(weight, eps, x=dense, partials=partials, residual=residual, extra=extra,
                               extra_index=extra_index)


class FusedComm(NcclComm):
    """One-shot fused exchange over peer memory for decode-sized steps."""

    def __init__(self, rank: int, size: int, hidden: int, group=None, region: symm.SymmetricRegion | None = None) -> None:
        super().__init__(rank, size, group)
        self.region = region or symm.SymmetricRegion.create(rank, size, hidden, group)
        self.hidden = hidden
        self.point = 0
        r = self.region
        self._slab_ptrs = [r.ptr_array(symm.OFF_SLABS + s * r.slab_bytes) for s in (0, 1)]
        self._flag_ptrs = [r.ptr_array(symm.OFF_FLAGS[s]) for s in (0, 1)]
        self._argmax_val = r.ptr_array(symm.OFF_ARGMAX_VAL)
        self._argmax_id = r.ptr_array(symm.OFF_ARGMAX_ID)
        self._argmax_flag = r.ptr_array(symm.OFF_ARGMAX_FLAGS)

    def begin_step(self) -> None:
        """Advance the step epoch (a kernel, so it is captured into decode graphs)."""
        self.point = 0
        native.call("prism_epoch_advance", self.region.local(symm.OFF_EPOCH), symm.POINTS_PER_STEP,
                    torch.cuda.current_stream().cuda_stream, 0)

    def row_parallel(self, x: torch.Tensor, w: torch.Tensor, stages: int = 0):
        T, K = x.shape
        M = w.shape[0]
        # every rank sends tp * splits * T rows of 8-byte words, so the one-shot exchange only wins
        # while T * tp is small (measured: TP8 ties with NCCL at 32 tokens, TP2 wins up to 128)
        if T > SMALL_T or M != self.hidden or self.point >= symm.ARGMAX_POINT or not x.is_cuda:
            return super().row_parallel(x, w, stages)
        if T * self.size > 192:
            # too many rows for the one-shot exchange: split-K partials stay local, one kernel sums them and sends
            # each row as bf16 to the rank that owns it; add_rmsnorm finishes the all-reduce (reduce + norm + all-gather)
            parts = ops.linear_partial(x, w, ops.choose_splits(M, K, T), stages=stages)
            return None, None, self.scatter_partials(parts)
        point, slot = self.point, self.point % 2
        r = self.region
        splits = min(symm.S_MAX, ops.choose_splits(M, K, T))
        eff = ops.effective_splits(K, splits)
        self.point += 1
        native.call(
            "prism_gemm_wx_push", w.data_ptr(), x.data_ptr(), M, T, K,
            w.stride(0), x.stride(0), M, M, eff, T * M, self._slab_ptrs[slot], self._flag_ptrs[slot], self.size,
            self.rank, point, r.local(symm.OFF_COUNTER[slot]), r.local(symm.OFF_EPOCH), 0, stages,
            torch.cuda.current_stream().cuda_stream, 1 if ops.pdl_enabled() else 0,
        )
        return None, None, (slot, point, self.size * eff, T)

    def add_rmsnorm(self, weight, eps, dense, partials, ticket, residual, extra=None, extra_index=None):
        if ticket is None:
            return super().add_rmsnorm(weight, eps, dense, partials, None, residual, extra, extra_index)
        if ticket[0] == "scatter":
            # the residual stays sharded by token row between exchanges: a full [T, H] tensor only comes from the
            # first (local) norm of the step
            return self.reduce_norm_allgather(ticket, weight, eps, residual,
                                              residual_is_shard=residual is not None and residual.shape[0] != ticket[3],
                                              extra=extra, extra_index=extra_index)
        slot, point, P, T = ticket
        H = self.hidden
        r = self.region
        out = torch.empty((T, H), dtype=torch.bfloat16, device=weight.device)
        new_res = residual if residual is not None else torch.empty((T, H), dtype=torch.bfloat16, device=weight.device)
        native.call(
            "prism_add_rmsnorm_packed", r.local(symm.OFF_SLABS + slot * r.slab_bytes), T * H, P,
            None if residual is None else residual.data_ptr(), new_res.data_ptr(),
            None if extra is None else extra.data_ptr(), None if extra is None else extra_index.data_ptr(),
            weight.data_ptr(), out.data_ptr(), T, H, float(eps), r.local(symm.OFF_EPOCH), point,
            torch.cuda.current_stream().cuda_stream, 1 if ops.pdl_enabled() else 0,
        )
        return out, new_res

    def greedy_merge(self, local_val: torch.Tensor, local_id: torch.Tensor) -> torch.Tensor:
        B = local_val.shape[0]
        if B > symm.B_MAX:
            return super().greedy_merge(local_val, local_id)
        out = torch.empty(B, dtype=torch.int64, device=local_val.device)
        r = self.region
        native.call(
            "prism_argmax_exchange", local_val.data_ptr(), local_id.data_ptr(), self._argmax_val, self._argmax_id,
            self._argmax_flag, r.local(symm.OFF_ARGMAX_FLAGS), r.local(symm.OFF_EPOCH), out.data_ptr(), self.size,
            self.rank, symm.ARGMAX_POINT, B, symm.B_MAX, torch.cuda.current_stream().cuda_stream,
            1 if ops.pdl_enabled() else 0,
        )
        return out

    # ---- prefill: row-parallel GEMM -> reduce-scatter, then reduce + norm -> all-gather -----------
    def prefill_fused(self, tokens: int) -> bool:
        return SMALL_T < tokens <= symm.PRE_T_MAX and self.hidden % 16 == 0

    def _exchange_point(self) -> tuple[int, int]:
        """(slot, point) of the next scatter / all-gather exchange.  Flags carry ``epoch + point``: the epoch
        is advanced by a kernel at the start of every step, so a replayed graph waits for fresh numbers."""
        self.point += 1
        point = self.point  # from 1: a flag that was never written (0) is below every number waited for
        if point >= symm.ARGMAX_POINT:
            raise RuntimeError("more exchanges in one step than the step epoch has points")
        return point % 2, point

    def scatter_linear(self, x: torch.Tensor, w: torch.Tensor):
        """Row-parallel projection whose epilogue writes each token row, as bf16, into the rank that
        owns it (``ceil(T / tp)`` consecutive rows per rank).  Returns the ticket for
        ``reduce_norm_allgather``."""
        T, K = x.shape
        rpo = -(-T // self.size)
        slot, point = self._exchange_point()
        r = self.region
        native.call("prism_gemm_wx_scatter", w.data_ptr(), x.data_ptr(), w.shape[0], T, K, w.stride(0), x.stride(0), rpo,
                    r.ptr_array(r.pre_offsets(slot)[0]), r.ptr_array(symm.OFF_PRE_RS_FLAGS[slot]), self.size, self.rank, point,
                    r.local(symm.OFF_EPOCH), r.local(symm.OFF_PRE_COUNTER[0]), torch.cuda.current_stream().cuda_stream,
                    1 if ops.pdl_enabled() else 0)
        return "scatter", slot, point, T, rpo

    def scatter_partials(self, partials: torch.Tensor):
        """Split-K partial rows ``[P, T, H]`` fp32 of a row-parallel projection: sum the slabs and send each
        row, as bf16, to the rank that owns it.  Returns the ticket for ``reduce_norm_allgather``."""
        P, T, H = partials.shape
        rpo = -(-T // self.size)
        slot, point = self._exchange_point()
        r = self.region
        native.call("prism_scatter_rows", partials.data_ptr(), partials.stride(0), P, T, H, rpo,
                    r.ptr_array(r.pre_offsets(slot)[0]), r.ptr_array(symm.OFF_PRE_RS_FLAGS[slot]), self.size, self.rank, point,
                    r.local(symm.OFF_EPOCH), r.local(symm.OFF_PRE_COUNTER[0]), torch.cuda.current_stream().cuda_stream,
                    1 if ops.pdl_enabled() else 0)
        return "scatter", slot, point, T, rpo

    def reduce_norm_allgather(self, ticket, weight: torch.Tensor, eps: float, residual: torch.Tensor | None, *,
                              residual_is_shard: bool, extra: torch.Tensor | None = None,
                              extra_index: torch.Tensor | None = None, wait: bool = True):
        """Sum the tp partial rows this rank owns, add the residual (a full ``[T, H]`` tensor or this
        rank's shard), RMSNorm, and store the normalised rows into every rank's activation buffer.
        Returns ``(h [T, H] view of the gathered rows, residual shard [rows_per_owner, H])``."""
        _, slot, point, T, rpo = ticket
        r, H = self.region, self.hidden
        row0 = self.rank * rpo
        rows = max(0, min(T, row0 + rpo) - row0)
        shard = residual if (residual is not None and residual_is_shard) else torch.empty((rpo, H), dtype=torch.bfloat16, device=weight.device)
        res_ptr = None
        if residual is not None and rows > 0:
            res_ptr = residual.data_ptr() if residual_is_shard else residual[row0:].data_ptr()
        stream = torch.cuda.current_stream().cuda_stream
        native.call("prism_reduce_norm_allgather", r.local(r.pre_offsets(slot)[0]), r.local(symm.OFF_PRE_RS_FLAGS[slot]), point,
                    self.size, self.rank, rpo, rows, row0, H, res_ptr, H, shard.data_ptr(),
                    None if extra is None else extra.data_ptr(), None if extra is None else extra_index.data_ptr(),
                    weight.data_ptr(), float(eps), r.ptr_array(r.pre_offsets(slot)[1]), r.ptr_array(symm.OFF_PRE_AG_FLAGS[slot]),
                    point, r.local(symm.OFF_EPOCH), r.local(symm.OFF_PRE_COUNTER[1]), stream, 1 if ops.pdl_enabled() else 0)
        if wait:
            self.wait_allgather(ticket)
        return r.pre_rows(slot, T), shard

    def wait_allgather(self, ticket) -> None:
        """Bounded wait until every rank's rows of this exchange are in the local activation buffer."""
        _, slot, point, _, _ = ticket
        native.call("prism_wait_flags", self.region.local(symm.OFF_PRE_AG_FLAGS[slot]), self.size, point,
                    self.region.local(symm.OFF_EPOCH), torch.cuda.current_stream().cuda_stream)

    # ---- sharded vision tower: merger GEMM -> all-gather ------------------------------------
    def vision_capacity(self) -> int:
        """Merged visual tokens one sharded vision-tower call can gather."""
        return symm.VIS_T_MAX

    def vision_begin(self, total_tokens: int) -> bool:
        """Start a sharded vision-tower call; False when the gathered outputs would not fit."""
        if total_tokens > symm.VIS_T_MAX:
            return False
        self.vision_seq = getattr(self, "vision_seq", 0) + 1
        self._vis_set = self.vision_seq % 2
        self._vis_pushed: set[int] = set()
        return True

    def allgather_linear(self, x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor, output: int, row_base: int) -> None:
        """``x @ w.T + bias`` written as bf16 rows ``[row_base, row_base + T)`` of gathered
        output ``output`` on every rank, straight from the GEMM epilogue."""
        r = self.region
        T, K = x.shape
        flags = r.ptr_array(symm.OFF_VIS_FLAGS + (self._vis_set * symm.VIS_OUTPUTS + output) * 64)
        bufs = r.ptr_array(r.vis_offset(self._vis_set, output))
        native.call(
            "prism_gemm_wx_allgather", w.data_ptr(), x.data_ptr(), w.shape[0], T, K, w.stride(0), x.stride(0),
            self.hidden, row_base, bias.data_ptr(), 0, bufs, flags, self.size, self.rank, self.vision_seq,
            r.local(symm.OFF_VIS_COUNTER), None, torch.cuda.current_stream().cuda_stream, 0,
        )
        self._vis_pushed.add(output)

    def vision_finish(self, n_outputs: int, total_tokens: int) -> list[torch.Tensor]:
        """Signal for outputs this rank had no rows for, wait for every rank, return copies."""
        r = self.region
        stream = torch.cuda.current_stream().cuda_stream
        outs = []
        for k in range(n_outputs):
            off = symm.OFF_VIS_FLAGS + (self._vis_set * symm.VIS_OUTPUTS + k) * 64
            if k not in self._vis_pushed:
                native.call("prism_signal_peers", r.ptr_array(off), self.size, self.rank, self.vision_seq, stream)
            native.call("prism_wait_flags", r.local(off), self.size, self.vision_seq, None, stream)
            outs.append(r.vis_rows(self._vis_set, k, total_tokens).clone())
        return outs

    def close(self) -> None:
        self.region.close()
