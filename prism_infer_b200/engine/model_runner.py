"""Per-rank owner of the model weights, the KV arena and the decode CUDA graphs
(reference ``prism_infer/engine/model_runner.py``: KV sizing ``:795-815``, allocation
``:817-890``, page copies ``:908-1031``, graph capture ``:1131-1158,2082-2127``, replay
with packed staging ``:1219-1313``).

B200-specific choices:

* One KV allocation ``[2, L, pages, Hkv/tp, page, D]`` (+ fp32 scales), sized from free HBM,
  head-major inside a page so each (page, head) is one contiguous 32 KB run of E4M3 bytes.
* Decode runs as one CUDA graph per batch bucket (1, 2, 4, 8, 16, 32, ...).  A single packed
  pinned host buffer is copied to the device by a memcpy node *inside* the graph, and the
  sampled tokens are copied back to pinned memory by another node, so a step is: fill the
  pinned buffer, replay, wait on the stream, read the tokens.  One graph per bucket serves
  greedy and temperature sampling (temperature is an input) and every context length (the
  attention loop bound is read from device memory).
* Kernels are launched with programmatic stream serialization so a GEMM prefetches its
  weight tiles while the previous kernel drains.
"""

from __future__ import annotations

from typing import Optional, Sequence as Seq

import torch

from .. import ops
from ..config import Config
from ..models.qwen3_vl import AttnMeta, Qwen3VLModel, TPComm
from ..models.weights import open_weight_source
from ..observability import profile_region
from .contracts import KVTransferPlan
from .input_preparation import StepInputs
from .kv_layout import CompactionPlan


def decode_buckets(max_num_seqs: int) -> list[int]:
    out = [b for b in (1, 2, 4, 8) if b <= max_num_seqs]
    b = 16
    while b < max_num_seqs:
        out.append(b)
        b *= 2
    if not out or out[-1] < max_num_seqs:
        out.append(max_num_seqs)
    return sorted(set(out))


class _DecodeGraph:
    """Static buffers + captured graph of one batch bucket."""

    def __init__(self, runner: "ModelRunner", bucket: int, greedy_only: bool = False) -> None:
        self.bucket = bucket
        self.greedy_only = greedy_only
        dev = runner.device
        mb = runner.max_blocks
        # byte layout of the packed staging buffer (all offsets 16-byte aligned)
        def al(x: int) -> int:
            return (x + 15) // 16 * 16
        self.off_ids = 0
        self.off_slots = al(self.off_ids + bucket * 8)
        self.off_pos = al(self.off_slots + bucket * 8)
        self.off_ctx = al(self.off_pos + 3 * bucket * 4)
        self.off_temp = al(self.off_ctx + bucket * 4)
        self.off_bt = al(self.off_temp + bucket * 4)
        self.nbytes = al(self.off_bt + bucket * mb * 4)
        pin = runner.on_cuda
        # Two pinned staging buffers and two token read-back buffers, used alternately: the host may stage step n + 1
        # while the copies of step n are still pending (one step runs ahead at most).  The copies run outside the
        # captured graph, which therefore reads and writes fixed device buffers only.
        self.hosts = [torch.zeros(self.nbytes, dtype=torch.uint8, pin_memory=pin) for _ in range(2)]
        self.dev = torch.zeros(self.nbytes, dtype=torch.uint8, device=dev)
        self.d_ids, self.d_slots, self.d_pos, self.d_ctx, self.d_temp, self.d_bt = self._views(self.dev, bucket, mb)
        self.tokens = torch.zeros(bucket, dtype=torch.int64, device=dev)
        self.tokens_hosts = [torch.zeros(bucket, dtype=torch.int64, pin_memory=pin) for _ in range(2)]
        self.done = [torch.cuda.Event() for _ in range(2)] if pin else [None, None]
        self.flip = 0
        self.step = torch.zeros(1, dtype=torch.int64, device=dev)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self._nps = [tuple(t.numpy() for t in self._views(h, bucket, mb)) for h in self.hosts]
        self._rows = [0, 0]  # rows of each staging buffer that hold real sequences
        for k in (0, 1):
            self.reset_rows(k, 0)

    @property
    def host(self) -> torch.Tensor:
        return self.hosts[self.flip]

    @property
    def tokens_host(self) -> torch.Tensor:
        return self.tokens_hosts[self.flip]

    def _views(self, buf: torch.Tensor, b: int, mb: int):
        ids = buf[self.off_ids:self.off_ids + b * 8].view(torch.int64)
        slots = buf[self.off_slots:self.off_slots + b * 8].view(torch.int64)
        pos = buf[self.off_pos:self.off_pos + 3 * b * 4].view(torch.int32).view(3, b)
        ctx = buf[self.off_ctx:self.off_ctx + b * 4].view(torch.int32)
        temp = buf[self.off_temp:self.off_temp + b * 4].view(torch.float32)
        bt = buf[self.off_bt:self.off_bt + b * mb * 4].view(torch.int32).view(b, mb)
        return ids, slots, pos, ctx, temp, bt

    def reset_rows(self, k: int, start: int) -> None:
        """Padding rows of staging buffer ``k``: token 0, no slot, empty context, no pages."""
        n = self._nps[k]
        n[0][start:] = 0
        n[1][start:] = -1
        n[2][:, start:] = 0
        n[3][start:] = 0
        n[4][start:] = 0
        n[5][start:] = -1

    def fill(self, inp: StepInputs, *, ahead: int = 0) -> int:
        """Stage one step's inputs in the next pinned buffer.  Writes go through numpy views of the
        pinned memory (a tenth of the cost of tensor slice assignment, and this runs on the critical
        path of every decode step); padding rows are rewritten only when the batch shrank.
        ``ahead = 1`` stages the step AFTER ``inp`` instead (same sequences one token later; the ids are
        taken from the device)."""
        self.flip ^= 1
        k = self.flip
        n = inp.num_seqs
        ids, slots, pos, ctx, temp, bt = self._nps[k]
        ids[:n] = inp.input_ids.numpy()
        slots[:n] = inp.slots.numpy() + ahead
        pos[:, :n] = inp.positions.numpy() + ahead
        ctx[:n] = inp.context_lens.numpy() + ahead
        temp[:n] = inp.temperatures.numpy()
        w = inp.block_tables.shape[1]
        bt[:n, :w] = inp.block_tables.numpy()
        bt[:n, w:] = -1
        if n < self._rows[k]:
            self.reset_rows(k, n)
        self._rows[k] = n
        return k

    def launch(self, k: int, n: int, *, ids_from_device: bool = False) -> None:
        """Copy staging buffer ``k`` to the device, replay the graph, read the tokens back into read-back buffer
        ``k``, record its event.  ``ids_from_device``: the input ids are the tokens the previous launch sampled
        (still in flight; stream order makes them ready)."""
        self.dev.copy_(self.hosts[k], non_blocking=True)
        if ids_from_device:
            self.d_ids[:n].copy_(self.tokens[:n], non_blocking=True)
        self.graph.replay()
        self.tokens_hosts[k].copy_(self.tokens, non_blocking=True)
        self.done[k].record()

    def wait(self, k: int, n: int) -> list[int]:
        self.done[k].synchronize()
        return self.tokens_hosts[k][:n].tolist()


class ModelRunner:
    def __init__(self, config: Config, *, rank: int = 0, comm: TPComm | None = None, device: str | None = None,
                 weights: dict[str, torch.Tensor] | None = None) -> None:
        self.config = config
        self.rank = rank
        self.comm = comm or TPComm()
        self.on_cuda = torch.cuda.is_available() if device is None else str(device).startswith("cuda")
        self.device = torch.device(device if device is not None else (f"cuda:{torch.cuda.current_device()}" if self.on_cuda else "cpu"))
        self.dtype = torch.bfloat16 if self.on_cuda else torch.float32
        arch = config.arch
        if self.on_cuda:
            from ..ops import native

            native.lib()  # fail loudly when the kernel library is missing
            ops.set_pdl(config.programmatic_dependent_launch)
            ops.apply_tuning()
        with profile_region("runner.load_weights"):
            self.model = Qwen3VLModel(arch, device=self.device, dtype=self.dtype, comm=self.comm)
            source = weights.items() if weights is not None else open_weight_source(
                config.model, arch, dtype=self.dtype, device=self.device, seed=config.seed)()
            self.model.load(source)
            if config.logits_precision == "selective_fp32" and self.on_cuda:
                self.model.enable_fp8_candidate_head()
        self.page = config.kvcache_block_size
        self.max_blocks = -(-config.max_model_len // self.page)
        self.kv_mode = config.kv_mode
        self._allocate_kv()
        self._visual: dict[int, tuple[torch.Tensor, list[torch.Tensor]]] = {}
        self._visual_cache: dict[str, tuple[torch.Tensor, list[torch.Tensor]]] = {}
        self._visual_cache_bytes = 0
        self.visual_cache_counters = {"hits": 0, "misses": 0, "evictions": 0}
        self._visual_scores: dict[int, dict[int, float]] = {}
        self._vision_graphs: dict[tuple, tuple] = {}
        self.vision_graph_counters = {"captures": 0, "replays": 0}
        self.graphs: dict[int, _DecodeGraph] = {}
        self.greedy_graphs: dict[int, _DecodeGraph] = {}
        self.run_ahead_counters = {"taken": 0, "discarded": 0}
        self.decode_counters: dict[str, dict[int, int]] = {"graph_batch_sizes": {}, "eager_batch_sizes": {}}
        self.buckets = decode_buckets(min(config.max_num_seqs, 512))
        self.sample_seed = config.seed
        self.steps_run = 0
        if self.on_cuda and config.prism.execution.uses_graphs:
            self.capture_graphs()

    # ------------------------------------------------------------------ KV arena
    def _allocate_kv(self) -> None:
        cfg, t = self.config, self.config.arch.text
        hkv = t.num_kv_heads // self.comm.size
        per_page = cfg.kv_bytes_per_page()
        blocks = cfg.num_kvcache_blocks
        if blocks <= 0:
            if self.on_cuda:
                blocks = self._measured_kv_blocks(per_page)
            else:
                blocks = max(8, 4 * self.max_blocks)
        cpu_blocks = cfg.num_cpu_blocks
        if cpu_blocks <= 0:
            want = int(blocks * cfg.cpu_kv_cache_ratio)
            cap = (4 << 30) // per_page if self.on_cuda else 64
            cpu_blocks = min(want, cap)
        self.kv = ops.KVCache(t.num_layers, blocks, hkv, self.page, t.head_dim, self.kv_mode, self.device, dtype=self.dtype)
        self.cpu_kv = ops.KVCache(t.num_layers, max(1, cpu_blocks), hkv, self.page, t.head_dim, self.kv_mode, "cpu",
                                  dtype=self.dtype, pin_memory=self.on_cuda) if cpu_blocks > 0 else None
        cfg.with_cache_capacity(blocks, cpu_blocks)

    GRAPH_POOL_RESERVE = 1 << 30  # decode-graph pools, vision-tower activations and allocator slack

    def _measured_kv_blocks(self, per_page: int) -> int:
        """Pages that fit after the weights and the activations of the largest prefill step.

        The activation peak is measured, not assumed (reference ``prism_infer/engine/model_runner.py:733-756,
        795-815``): a prefill of ``max_num_batched_tokens`` placeholder tokens runs once against a scratch
        cache, and the KV arena gets ``total * gpu_memory_utilization`` minus what is allocated now, minus
        the measured peak above that, minus a fixed reserve for graph pools.  Every tensor-parallel rank
        runs the same warm-up (its collectives pair up)."""
        cfg, t = self.config, self.config.arch.text
        dev = self.device
        tokens = max(1, min(int(cfg.max_num_batched_tokens), int(cfg.max_model_len)))
        hkv = t.num_kv_heads // self.comm.size
        torch.cuda.synchronize(dev)
        base = torch.cuda.memory_allocated(dev)
        torch.cuda.reset_peak_memory_stats(dev)
        scratch_pages = -(-tokens // self.page) + 1
        scratch = ops.KVCache(t.num_layers, scratch_pages, hkv, self.page, t.head_dim, self.kv_mode, dev, dtype=self.dtype)
        ids = torch.zeros(tokens, dtype=torch.int64, device=dev)
        pos = torch.arange(tokens, dtype=torch.int32, device=dev).repeat(3, 1).contiguous()
        slots = torch.arange(tokens, dtype=torch.int64, device=dev)
        bt = torch.arange(scratch_pages, dtype=torch.int32, device=dev).view(1, -1)
        meta = AttnMeta(is_prefill=True, block_tables=bt, slots=slots,
                        cu_seqlens_q=torch.tensor([0, tokens], dtype=torch.int32, device=dev),
                        kv_lens=torch.tensor([tokens], dtype=torch.int32, device=dev), max_q_len=tokens, no_history=True)
        hidden = self.model.forward(ids, pos, meta, scratch)
        self.model.sample(hidden[-1:], None)
        torch.cuda.synchronize(dev)
        peak = torch.cuda.max_memory_allocated(dev) - base - scratch.payload.numel() * scratch.payload.element_size()
        del scratch, hidden, ids, pos, slots, bt, meta
        torch.cuda.empty_cache()
        free, total = torch.cuda.mem_get_info(dev)
        used = total - free  # weights, this process's context, other processes on the device
        budget = int(total * cfg.gpu_memory_utilization) - used - max(0, peak) - self.GRAPH_POOL_RESERVE
        self.kv_sizing = {"warmup_tokens": tokens, "activation_peak_bytes": int(max(0, peak)), "used_bytes": int(used),
                          "budget_bytes": int(budget)}
        return max(1, budget // per_page)

    # --------------------------------------------------------------- page traffic
    def apply_kv_transfers(self, tr: KVTransferPlan) -> None:
        """Order matters: prefix-row copies, copy-on-write, swap-out, swap-in."""
        if tr.copy_prefix:
            with profile_region("engine.kv.copy_prefix"):
                ops.kv_page_copy(self.kv, self.kv, [s for s, _, _ in tr.copy_prefix], [d for _, d, _ in tr.copy_prefix],
                                 [r for _, _, r in tr.copy_prefix])
        if tr.copy_on_write:
            with profile_region("engine.kv.copy_on_write"):
                ops.kv_page_copy(self.kv, self.kv, [s for s, _ in tr.copy_on_write], [d for _, d in tr.copy_on_write])
        if tr.swap_out:
            with profile_region("engine.kv.swap_out"):
                ops.kv_page_copy(self.kv, self.cpu_kv, [g for g, _ in tr.swap_out], [c for _, c in tr.swap_out])
                if self.on_cuda:
                    torch.cuda.current_stream().synchronize()
        if tr.swap_in:
            with profile_region("engine.kv.swap_in"):
                ops.kv_page_copy(self.cpu_kv, self.kv, [c for c, _ in tr.swap_in], [g for _, g in tr.swap_in])

    def compact_kv(self, plans: Seq[CompactionPlan]) -> None:
        with profile_region("engine.kv.visual_compact"):
            for plan in plans:
                src = torch.tensor(plan.src_slots, dtype=torch.int64, device=self.device)
                dst = torch.tensor(plan.dst_slots, dtype=torch.int64, device=self.device)
                ops.kv_compact(self.kv, src, dst)

    # ------------------------------------------------------------------- vision
    def _encode(self, job) -> tuple[torch.Tensor, list[torch.Tensor]]:
        key = job.cache_key if self.config.enable_visual_embedding_cache else None
        if key is not None and key in self._visual_cache:
            self.visual_cache_counters["hits"] += 1
            val = self._visual_cache.pop(key)
            self._visual_cache[key] = val  # LRU refresh
            return val
        with profile_region("model.vision.encoder"):
            main, deep = self._tower(job.pixel_values, job.grid_thw)
        if key is not None:
            self.visual_cache_counters["misses"] += 1
            self._cache_visual(key, (main, deep))
        return main, deep

    VISION_GRAPH_MAX_PATCHES = 4096   # larger inputs are compute-bound: a graph would only hold memory
    VISION_GRAPH_ENTRIES = 8

    def _tower(self, pixel_values: torch.Tensor, grid_thw) -> tuple[torch.Tensor, list[torch.Tensor]]:
        """The vision tower, replayed from a CUDA graph per grid shape when
        ``enable_vision_tensor_cudagraph`` is set (reference ``MultimodalConfig``, ``config.py:279-322``):
        a single 448 x 448 image is about 300 launches for half a millisecond of device work, and
        serving repeats a handful of image shapes.  One rank, CUDA, at most
        ``VISION_GRAPH_MAX_PATCHES`` patches; the least recently used of ``VISION_GRAPH_ENTRIES``
        graphs is dropped.  Results are copied out of the graph's buffers."""
        n = int(pixel_values.shape[0])
        if not (self.on_cuda and self.comm.size == 1 and self.config.enable_vision_tensor_cudagraph and n <= self.VISION_GRAPH_MAX_PATCHES):
            return self.model.encode_vision(pixel_values, grid_thw)
        key = tuple(tuple(int(v) for v in g) for g in grid_thw)
        entry = self._vision_graphs.pop(key, None)
        if entry is None:
            self.vision_graph_counters["captures"] += 1
            static_in = torch.empty((n, pixel_values.shape[1]), dtype=self.dtype, device=self.device)
            stream = torch.cuda.Stream(device=self.device)
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                static_in.copy_(pixel_values, non_blocking=True)
                self.model.encode_vision(static_in, grid_thw)      # warm-up outside capture: geometry tensors, kernel attributes
                stream.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    main, deep = self.model.encode_vision(static_in, grid_thw)
            torch.cuda.current_stream().wait_stream(stream)
            entry = (graph, static_in, main, deep)
            while len(self._vision_graphs) >= self.VISION_GRAPH_ENTRIES:
                self._vision_graphs.pop(next(iter(self._vision_graphs)))
        else:
            self.vision_graph_counters["replays"] += 1
        self._vision_graphs[key] = entry  # most recently used last
        graph, static_in, main, deep = entry
        static_in.copy_(pixel_values, non_blocking=True)
        graph.replay()
        return main.clone(), [d.clone() for d in deep]

    def _cache_visual(self, key: str, value: tuple[torch.Tensor, list[torch.Tensor]]) -> None:
        """LRU insertion under the byte budget; an entry larger than the budget is not kept."""
        if key in self._visual_cache:
            return
        main, deep = value
        size = (1 + len(deep)) * main.numel() * main.element_size()
        budget = self.config.visual_embedding_cache_bytes
        while self._visual_cache and self._visual_cache_bytes + size > budget:
            _, (m, d) = next(iter(self._visual_cache.items()))
            self._visual_cache_bytes -= (1 + len(d)) * m.numel() * m.element_size()
            self._visual_cache.pop(next(iter(self._visual_cache)))
            self.visual_cache_counters["evictions"] += 1
        if size <= budget:
            self._visual_cache[key] = value
            self._visual_cache_bytes += size

    def _encode_jobs(self, jobs) -> None:
        """Vision tower for the sequences of one prefill step.  Jobs that miss the embedding cache
        are pushed through the tower together, up to ``vision_encoder_microbatch_patches`` patches
        per pass (reference ``models/qwen3_vl.py:1233-1281`` microbatches on frame boundaries): a
        pass over one 448 x 448 image is launch-bound, so a prefill batch of many single-image
        requests would otherwise pay the tower's ~300 launches once per request.  A single job is
        never split.  Attention is per image segment and every other op is per patch, so each
        job's rows are what a pass of its own would produce."""
        use_cache = self.config.enable_visual_embedding_cache
        pending = []
        for job in jobs:
            if use_cache and job.cache_key is not None and job.cache_key in self._visual_cache:
                self._visual[job.seq_id] = self._encode(job)  # cache hit: no tower work
            else:
                pending.append(job)
        budget = self.config.vision_encoder_microbatch_patches
        group: list = []
        patches = 0
        for job in pending:
            n = int(job.pixel_values.shape[0])
            if group and patches + n > budget:
                self._encode_group(group)
                group, patches = [], 0
            group.append(job)
            patches += n
        if group:
            self._encode_group(group)

    def _encode_group(self, group) -> None:
        if len(group) == 1:
            self._visual[group[0].seq_id] = self._encode(group[0])
            return
        unit = self.config.arch.vision.merge_unit
        grids = [g for j in group for g in j.grid_thw]
        shard = self.model.vision_shard_rows(grids) if (self.on_cuda and self.comm.size > 1) else None
        if shard is not None:
            # tensor-parallel ranks run the blocks on their own segments: upload those rows only, job by job, instead of
            # concatenating every job's patches on the host (nine processes doing that at once starve one another)
            lo, n = shard
            pieces, row = [], 0
            for j in group:
                rows_j = int(j.pixel_values.shape[0])
                a, b = max(lo, row), min(lo + n, row + rows_j)
                if a < b:
                    pieces.append(j.pixel_values[a - row:b - row].to(device=self.device, dtype=self.dtype, non_blocking=True))
                row += rows_j
            pixels = (pieces[0] if len(pieces) == 1 else torch.cat(pieces)) if pieces else \
                torch.empty((0, group[0].pixel_values.shape[1]), dtype=self.dtype, device=self.device)
            with profile_region("model.vision.encoder", metadata={"jobs": len(group)}):
                main, deep = self.model.encode_vision(pixels, grids, local_rows=shard)
        else:
            if self.on_cuda:  # each job's pinned patches travel as their own asynchronous copy
                pixels = torch.cat([j.pixel_values.to(device=self.device, dtype=self.dtype, non_blocking=True) for j in group])
            else:
                pixels = torch.cat([j.pixel_values for j in group])
            with profile_region("model.vision.encoder", metadata={"jobs": len(group)}):
                main, deep = self._tower(pixels, grids)
        row = 0
        for job in group:
            n = sum(int(t) * int(h) * int(w) for t, h, w in job.grid_thw) // unit
            result = (main[row:row + n].clone(), [d[row:row + n].clone() for d in deep])  # own storage: the batch can be freed
            row += n
            self._visual[job.seq_id] = result
            if self.config.enable_visual_embedding_cache and job.cache_key is not None:
                self.visual_cache_counters["misses"] += 1
                self._cache_visual(job.cache_key, result)

    def encode_for_sequence(self, job) -> None:
        """Vision tower for one sequence, kept until its prefill consumes it."""
        self._visual[job.seq_id] = self._encode(job)

    # ---- vision tower in block quanta (cooperative prefill on one rank; eager launches, no tower graph) ----
    def begin_encode(self, job) -> int | None:
        """Start the vision tower for one sequence; its blocks follow through ``advance_encode``.  Returns a handle,
        or None when the visual-embedding cache already holds the result (it is attached at once)."""
        if self.comm.size != 1:
            raise ValueError("the vision tower runs in block quanta on one rank only")
        key = job.cache_key if self.config.enable_visual_embedding_cache else None
        if key is not None and key in self._visual_cache:
            self._visual[job.seq_id] = self._encode(job)
            return None
        with profile_region("model.vision.encoder", metadata={"quantum": "begin"}):
            state = self.model.begin_vision(job.pixel_values, job.grid_thw)
        handle = self.__dict__.setdefault("_encode_handles", 0) + 1
        self._encode_handles = handle
        self.__dict__.setdefault("_pending_encodes", {})[handle] = (job, key, state)
        return handle

    def advance_encode(self, handle: int, max_blocks: int) -> bool:
        """Up to ``max_blocks`` more vision blocks; when the last has run the mergers follow and the result is attached
        to the sequence (and cached).  True when done."""
        job, key, state = self._pending_encodes[handle]
        with profile_region("model.vision.encoder", metadata={"quantum": max_blocks}):
            if not self.model.advance_vision(state, max_blocks):
                return False
            main, deep = self.model.finish_vision(state)
        del self._pending_encodes[handle]
        self._visual[job.seq_id] = (main, deep)
        if key is not None:
            self.visual_cache_counters["misses"] += 1
            self._cache_visual(key, (main, deep))
        return True

    def hydrate_visual_embedding(self, job) -> None:
        """Run the vision tower ahead of scheduling.  The result stays attached to the sequence
        until its prefill has consumed it (reference ``engine/model_runner.py:522-596``) - the
        LRU cache alone would lose it when a burst of submissions exceeds the cache budget, and
        the prefill would encode the media a second time - and in the cache for later requests
        with the same media."""
        self._visual[job.seq_id] = self._encode(job)

    def take_visual_scores(self) -> dict[int, dict[int, float]]:
        """Attention-strategy scores of the sequences scored since the last call (identical on
        every rank after the reduction)."""
        out, self._visual_scores = self._visual_scores, {}
        return out

    def release_visual(self, seq_id: int) -> None:
        """Drop the vision result of a sequence that will not be prefilled (cancelled, rejected)."""
        self._visual.pop(seq_id, None)

    def visual_embedding_cache_metadata(self) -> dict[str, object]:
        return {"enabled": self.config.enable_visual_embedding_cache, "entries": len(self._visual_cache),
                "bytes": self._visual_cache_bytes, **self.visual_cache_counters}

    # ------------------------------------------------------------------ execution
    def execute(self, inp: StepInputs) -> list[int]:
        """Run one step; returns the sampled token of every sampling row."""
        self.steps_run += 1
        if inp.kind != "prefill":  # which path each decode step took (benchmark records carry this as evidence)
            graph = bool(self.graphs) and inp.num_seqs <= self.buckets[-1]
            table = self.decode_counters["graph_batch_sizes" if graph else "eager_batch_sizes"]
            table[inp.num_seqs] = table.get(inp.num_seqs, 0) + 1
        if self.graphs and inp.kind != "prefill" and inp.num_seqs <= self.buckets[-1]:
            return self._run_decode_graph(inp)
        if getattr(self, "_ahead", None) is not None:  # a launch that ran ahead is not taken over across other kinds of steps
            self._ahead = None
            self.run_ahead_counters["discarded"] += 1
        if inp.kind == "prefill":
            return self._run_prefill(inp)
        return self._run_decode_eager(inp)

    def _to_dev(self, t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        if t is None or not self.on_cuda:
            return t
        return t.pin_memory().to(self.device, non_blocking=True)

    def _prefill_inputs(self, inp: StepInputs):
        """Vision tower for the step's jobs and the device-side inputs of its language prefill."""
        with profile_region("runner.prepare_inputs"):
            self._encode_jobs(inp.vision_jobs)
            visual = deep = None
            if inp.vision_rows:
                mains, deeps = [], None
                for seq_id, lo, n in inp.vision_rows:
                    m, d = self._visual[seq_id]
                    mains.append(m[lo:lo + n])
                    if deeps is None:
                        deeps = [[] for _ in d]
                    for k, dk in enumerate(d):
                        deeps[k].append(dk[lo:lo + n])
                visual = mains[0] if len(mains) == 1 else torch.cat(mains)
                deep = [dk[0] if len(dk) == 1 else torch.cat(dk) for dk in (deeps or [])]
            meta = AttnMeta(
                is_prefill=True, block_tables=self._to_dev(inp.block_tables), slots=self._to_dev(inp.slots),
                cu_seqlens_q=self._to_dev(inp.cu_seqlens_q), kv_lens=self._to_dev(inp.kv_lens), max_q_len=inp.max_q_len,
                no_history=bool(torch.equal(inp.kv_lens, inp.cu_seqlens_q[1:] - inp.cu_seqlens_q[:-1])))
            if not meta.no_history:  # key ranges for the gather + tensor-core attention over the paged cache
                cu_kv = torch.zeros(inp.kv_lens.shape[0] + 1, dtype=torch.int32)
                cu_kv[1:] = torch.cumsum(inp.kv_lens, 0)
                meta.cu_seqlens_kv, meta.total_kv, meta.max_kv_len = self._to_dev(cu_kv), int(cu_kv[-1]), int(inp.kv_lens.max())
            ids, pos, vis_index = self._to_dev(inp.input_ids), self._to_dev(inp.positions), self._to_dev(inp.vis_index)
            if inp.score_rows:
                from .visual_pruning import RuntimeVisualTokenScorer

                meta.scorer = RuntimeVisualTokenScorer(inp.score_rows, inp.score_layers)
        return ids, pos, meta, visual, vis_index, deep

    def _prefill_outputs(self, inp: StepInputs, meta: AttnMeta, hidden: torch.Tensor) -> list[int]:
        """After the layers: visual-token scores, release of consumed visual embeddings, first tokens."""
        if meta.scorer is not None:
            self._visual_scores.update(meta.scorer.finalize(world_size=self.comm.size, reduce_sum=self.comm.reduce_dense))
        for seq_id in inp.release_visual:
            self._visual.pop(seq_id, None)
        if inp.sample_rows is None or inp.sample_rows.numel() == 0:
            if self.on_cuda:
                torch.cuda.current_stream().synchronize()
            return []
        with profile_region("runner.sampler"):
            rows = hidden[self._to_dev(inp.sample_rows)]
            temps = self._to_dev(inp.temperatures) if bool((inp.temperatures > 0).any()) else None
            step = torch.tensor([self.steps_run], dtype=torch.int64, device=self.device)
            tok = self.model.sample(rows, temps, seed=self.sample_seed, step=step)
        return tok.tolist()

    def _run_prefill(self, inp: StepInputs) -> list[int]:
        ids, pos, meta, visual, vis_index, deep = self._prefill_inputs(inp)
        with profile_region("runner.run_model"):
            hidden = self.model.forward(ids, pos, meta, self.kv, visual=visual, vis_index=vis_index, deepstack=deep)
        return self._prefill_outputs(inp, meta, hidden)

    # ---- cooperative prefill: the same step, a few decoder layers at a time (reference
    # ``engine/model_runner.py:1346-1650``; one rank) -----------------------------------------------
    def begin_prefill(self, inp: StepInputs) -> int:
        """Vision tower, embedding and device inputs of a prefill step whose layers ``advance_prefill`` runs in
        quanta, so that decode steps of running sequences can go in between.  Returns a handle."""
        if self.comm.size != 1:
            raise ValueError("cooperative prefill runs on one rank")
        self.steps_run += 1
        self._ahead = None
        ids, pos, meta, visual, vis_index, deep = self._prefill_inputs(inp)
        state = self.model.begin_layers(ids, pos, meta, self.kv, visual=visual, vis_index=vis_index, deepstack=deep)
        handle = self.__dict__.setdefault("_prefill_handles", 0) + 1
        self._prefill_handles = handle
        self.__dict__.setdefault("_pending_prefills", {})[handle] = (inp, state)
        return handle

    def advance_prefill(self, handle: int, max_layers: int) -> bool:
        """Up to ``max_layers`` more decoder layers of a begun prefill; True when all have run."""
        _, state = self._pending_prefills[handle]
        with profile_region("runner.run_model", metadata={"layers": max_layers}):
            return self.model.advance_layers(state, max_layers)

    def finish_prefill(self, handle: int) -> list[int]:
        """Remaining layers, final norm, sampling; returns the first token of every sampling row."""
        inp, state = self._pending_prefills.pop(handle)
        with profile_region("runner.run_model"):
            self.model.advance_layers(state, len(self.model.layers))
            hidden = self.model.finish_layers(state)
        return self._prefill_outputs(inp, state.meta, hidden)

    def _run_decode_eager(self, inp: StepInputs) -> list[int]:
        meta = AttnMeta(is_prefill=False, block_tables=self._to_dev(inp.block_tables), slots=self._to_dev(inp.slots),
                        context_lens=self._to_dev(inp.context_lens))
        hidden = self.model.forward(self._to_dev(inp.input_ids), self._to_dev(inp.positions), meta, self.kv)
        temps = self._to_dev(inp.temperatures) if bool((inp.temperatures > 0).any()) else None
        step = torch.tensor([self.steps_run], dtype=torch.int64, device=self.device)
        return self.model.sample(hidden, temps, seed=self.sample_seed, step=step).tolist()

    # ---------------------------------------------------------------- CUDA graphs
    def _decode_body(self, g: _DecodeGraph) -> None:
        meta = AttnMeta(is_prefill=False, block_tables=g.d_bt, slots=g.d_slots, context_lens=g.d_ctx,
                        nsplit=ops.decode_splits(g.bucket, self.kv.num_kv_heads))
        hidden = self.model.forward(g.d_ids, g.d_pos, meta, self.kv)
        self.model.sample(hidden, None if g.greedy_only else g.d_temp, seed=self.sample_seed, step=g.step, out=g.tokens)

    def capture_graphs(self) -> None:
        """Capture one graph per bucket, largest first so smaller ones reuse its pool."""
        pool = None
        stream = torch.cuda.Stream(device=self.device)
        # the capture stream does not order itself after the stream that initialised the weights, the KV arena
        # and the exchange buffers: without this wait the warm-up launches below could overtake that work
        stream.wait_stream(torch.cuda.current_stream(self.device))
        # one graph per bucket takes the temperature as an input; tensor-parallel ranks add a
        # greedy-only graph whose sampler is the one-kernel (value, id) exchange
        # ... and so does a rank with the FP8 candidate head, which serves greedy rows only
        greedy_variants = self.comm.size > 1 or getattr(self.model, "lm_head_fp8", None) is not None
        variants = [(b, False) for b in self.buckets] + ([(b, True) for b in self.buckets] if greedy_variants else [])
        for bucket, greedy_only in sorted(variants, reverse=True):
            from ..ops import native as _native

            with torch.cuda.stream(stream):
                g = _DecodeGraph(self, bucket, greedy_only)  # its zero-filled buffers belong to the capture stream
                for _ in range(2):  # warm-up outside capture (lazy kernel attributes, tensor maps)
                    g.dev.copy_(g.host, non_blocking=True)
                    self._decode_body(g)
                stream.synchronize()
                graph = torch.cuda.CUDAGraph()
                before = _native.launch_count()
                with torch.cuda.graph(graph, pool=pool, stream=stream):
                    self._decode_body(g)  # the staging copy and the token read-back run outside the graph (see launch)
                    g.step.add_(1)
            g.graph = graph
            g.launches = _native.launch_count() - before
            pool = graph.pool() if pool is None else pool
            (self.greedy_graphs if greedy_only else self.graphs)[bucket] = g
        torch.cuda.current_stream(self.device).wait_stream(stream)
        torch.cuda.synchronize(self.device)

    def _run_decode_graph(self, inp: StepInputs) -> list[int]:
        """One decode step from the bucket's graph.  With ``decode_run_ahead`` the step after this one is launched
        before the host waits for this one's tokens, whenever it can be predicted: greedy rows only, the same
        sequences one position later, nobody's next slot in a new page.  Its input ids are the tokens this step
        samples, copied on the device.  The next call takes the launch over if its inputs are the predicted ones
        (the ids must be the tokens this step returned); otherwise the launch is left to finish unobserved: it wrote
        one K / V row per sequence at a position past that sequence's end, which nothing reads before it is written
        again, and every later kernel is ordered after it on the stream."""
        n = inp.num_seqs
        bucket = next(b for b in self.buckets if b >= n)
        greedy = bucket in self.greedy_graphs and not bool((inp.temperatures > 0).any())
        g = (self.greedy_graphs if greedy else self.graphs)[bucket]
        self._last_bucket, self._last_greedy = bucket, greedy
        ahead, self._ahead = getattr(self, "_ahead", None), None
        if ahead is not None and ahead["graph"] is g and self._is_predicted(ahead, inp):
            k = ahead["k"]
            self.run_ahead_counters["taken"] += 1
        else:
            if ahead is not None:
                self.run_ahead_counters["discarded"] += 1
            with profile_region("runner.cudagraph.copy_inputs"):
                k = g.fill(inp)
            with profile_region("runner.cudagraph.replay"):
                g.launch(k, n)
        all_greedy = not bool((inp.temperatures > 0).any())
        # one rank only: with it on, the two-GPU test-suite did not finish within its time limit (the headline
        # benchmark at two ranks did); until that is understood tensor-parallel ranks wait for every step
        if self.config.decode_run_ahead and self.comm.size == 1 and all_greedy and self._next_is_predictable(inp):
            with profile_region("runner.cudagraph.run_ahead"):
                k_next = g.fill(inp, ahead=1)
                g.launch(k_next, n, ids_from_device=True)
            self._ahead = {"graph": g, "k": k_next, "n": n, "slots": inp.slots + 1, "positions": inp.positions + 1,
                           "context_lens": inp.context_lens + 1, "block_tables": inp.block_tables}
        with profile_region("runner.cudagraph.wait"):
            tokens = g.wait(k, n)
        if self._ahead is not None:
            self._ahead["ids"] = tokens
        return tokens

    def _next_is_predictable(self, inp: StepInputs) -> bool:
        # the next token of a row goes to slot + 1 unless that is the first slot of a page the scheduler has yet to pick
        return bool(((inp.slots + 1) % self.page != 0).all()) and bool((inp.slots >= 0).all())

    @staticmethod
    def _is_predicted(ahead: dict, inp: StepInputs) -> bool:
        if inp.num_seqs != ahead["n"] or bool((inp.temperatures > 0).any()):
            return False
        if inp.input_ids.tolist() != ahead["ids"]:
            return False
        if not (torch.equal(inp.slots, ahead["slots"]) and torch.equal(inp.positions, ahead["positions"])
                and torch.equal(inp.context_lens, ahead["context_lens"])):
            return False
        a, b = inp.block_tables, ahead["block_tables"]
        w = min(a.shape[1], b.shape[1])
        return bool(torch.equal(a[:, :w], b[:, :w]) and (a[:, w:] < 0).all() and (b[:, w:] < 0).all())

    def time_decode_graph(self, steps: int) -> float:
        """Device milliseconds per decode step: CUDA events around ``steps`` back-to-back
        launches of the most recently used bucket graph (inputs stay as last filled)."""
        table = self.greedy_graphs if getattr(self, "_last_greedy", False) else self.graphs
        g = table[getattr(self, "_last_bucket", self.buckets[0])]
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(self.device)
        start.record()
        for _ in range(steps):
            g.dev.copy_(g.host, non_blocking=True)  # the step's staging copy and token read-back, as in launch()
            g.graph.replay()
            g.tokens_host.copy_(g.tokens, non_blocking=True)
        end.record()
        torch.cuda.synchronize(self.device)
        return start.elapsed_time(end) / steps

    def graph_metadata(self) -> dict[str, object]:
        return {"buckets": list(self.graphs), "pdl": ops.pdl_enabled(), "kv_pages": self.kv.num_blocks,
                "vision_graphs": {"entries": len(self._vision_graphs), **self.vision_graph_counters},
                "kv_bytes_per_page": self.config.kv_bytes_per_page(), "kv_mode": self.kv_mode,
                "launches_per_decode_graph": {str(b): getattr(g, "launches", 0) for b, g in self.graphs.items()},
                "staging_bytes": {str(b): g.nbytes for b, g in self.graphs.items()},
                "weight_bytes": self.model.weight_bytes(), "kv_sizing": getattr(self, "kv_sizing", None),
                "decode_run_ahead": dict(self.run_ahead_counters),
                "decode_steps": {k: {str(n): c for n, c in sorted(v.items())} for k, v in self.decode_counters.items()}}

    def barrier(self) -> None:
        if self.on_cuda:
            torch.cuda.synchronize(self.device)

    def keep_logits(self, on: bool) -> None:
        """Debugging aid for eager execution: keep the full-vocabulary fp32 logits of the rows sampled
        last (tensor-parallel ranks gather them), readable with ``last_logits``."""
        self.model.keep_logits = bool(on)
        self.model.last_logits = None

    def last_logits(self):
        """``[rows, vocab]`` fp32 on the CPU (rank 0 only; other ranks answer ``None``)."""
        t = getattr(self.model, "last_logits", None)
        if t is None or self.rank != 0:
            return None
        return t.cpu()

    def status(self) -> dict:
        """Device status words (bounded waits that ran out, bounds checks) of this rank."""
        if not self.on_cuda:
            return {}
        from ..ops import native

        return native.read_status(reset=True)

    def capacity(self) -> tuple[int, int]:
        return self.config.num_kvcache_blocks, self.config.num_cpu_blocks

    def exit(self) -> None:
        self.graphs.clear()
        self.greedy_graphs.clear()
        self._vision_graphs.clear()
        self._visual.clear()
        self._visual_cache.clear()
