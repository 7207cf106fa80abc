"""Engine orchestrator behind the public ``LLM`` class (reference
``prism_infer/engine/llm_engine.py:146-1538``).

Builds the configuration, starts the tensor-parallel ranks, owns tokenizer, processor,
scheduler and executor, and exposes request submission (``add_*_request``), the step loop
(``step_result`` / ``step`` / ``is_finished``), cancellation, metrics and the synchronous
``generate*`` helpers.  Generation results are dictionaries with ``text``, ``raw_text`` and
``token_ids``.
"""

from __future__ import annotations

import atexit
import hashlib
import os
import time
from typing import Any, Sequence as Seq

import torch

from ..config import Config
from ..models.position import rope_index
from ..observability import profile_region, profile_step_metadata
from ..sampling_params import SamplingParams
from ..utils.tokenizer import load_tokenizer
from .contracts import Phase, StepResult
from .executor import LocalRunnerGroup, ModelExecutor
from .input_preparation import VisionJob
from .metrics import EngineMetrics
from .progress import GenerationProgress
from .request import RequestIdAllocator, RequestState
from .scheduler import Scheduler
from .sequence import Sequence
from .vl_inputs import (ImageInputs, PatchProcessor, VideoInputs, checkpoint_pixel_budgets, load_video_file, prepare_image_inputs,
                        prepare_interleaved_image_inputs, prepare_video_inputs)


_HASH_CHUNKS = 8
_HASH_PARALLEL_MIN_BYTES = 4 << 20
_hash_pool = None


def _update_with_buffer(h, view: memoryview) -> None:
    """Feed ``view`` to ``h``.  A large buffer (the pixel tensor of several images is tens of
    megabytes, ~30 ms of SHA-256 on one core) is cut into fixed chunks that are hashed on a small
    thread pool (``hashlib`` releases the interpreter lock) and ``h`` absorbs the chunk digests in
    order: the key stays a pure function of the content and the host time drops by the number
    of cores used."""
    n = len(view)
    if n < _HASH_PARALLEL_MIN_BYTES:
        h.update(view)
        return
    global _hash_pool
    if _hash_pool is None:
        from concurrent.futures import ThreadPoolExecutor

        _hash_pool = ThreadPoolExecutor(_HASH_CHUNKS, thread_name_prefix="content-key")
    step = -(-n // _HASH_CHUNKS)
    step += -step % 64
    h.update(f"chunked:{step}:".encode())
    for d in _hash_pool.map(lambda off: hashlib.sha256(view[off:off + step]).digest(), range(0, n, step)):
        h.update(d)


def content_key(*parts: Any) -> str:
    """Content-addressed key over tensors / arrays / bytes / strings."""
    h = hashlib.sha256()
    for p in parts:
        if isinstance(p, torch.Tensor):
            h.update(str(tuple(p.shape)).encode())
            flat = p.detach().cpu().contiguous().view(torch.uint8).reshape(-1)
            _update_with_buffer(h, memoryview(flat.numpy()))
        elif isinstance(p, (bytes, bytearray)):
            _update_with_buffer(h, memoryview(p))
        else:
            h.update(repr(p).encode())
    return h.hexdigest()


class LLMEngine:
    def __init__(self, model: str, *, runner_group=None, weights: dict[str, torch.Tensor] | None = None,
                 device: str | None = None, **kwargs: Any) -> None:
        self.config = Config(model, **kwargs)
        cfg = self.config
        self.arch = cfg.arch
        if runner_group is None:
            self._validate_environment(device)
        self.tokenizer = load_tokenizer(cfg.model, self.arch)
        # options given by the caller win; otherwise the budgets the checkpoint's own processor files record
        recorded = checkpoint_pixel_budgets(cfg.model) if os.path.isdir(str(cfg.model)) else {}
        self.processor = PatchProcessor(self.arch, min_pixels=cfg.image_min_pixels or recorded.get("min_pixels"),
                                        max_pixels=cfg.image_max_pixels or recorded.get("max_pixels"),
                                        video_max_pixels=cfg.video_max_pixels or recorded.get("video_max_pixels"),
                                        video_min_pixels=recorded.get("video_min_pixels"), video_fps=recorded.get("video_fps"),
                                        video_min_frames=recorded.get("video_min_frames"), video_max_frames=recorded.get("video_max_frames"))
        from .chat_prompt import ChatPrompt, HFProcessorAdapter

        mode = cfg.chat_template
        chat = ChatPrompt(self.tokenizer)
        self.chat = chat if (mode == "always" or (mode == "auto" and chat.has_template)) else None
        self.hf_processor = None
        if cfg.hf_processor == "always":
            self.hf_processor = HFProcessorAdapter(cfg.model, image_max_pixels=cfg.image_max_pixels,
                                                   video_max_pixels=cfg.video_max_pixels)
        self._ids = RequestIdAllocator()
        self.metrics = EngineMetrics()
        # CUDA engines keep a request's patches as pinned bf16 (the model's dtype): the copy to the
        # device is then one asynchronous DMA of half the bytes instead of a staged pageable fp32
        # copy plus a cast, and tensor-parallel workers receive half the bytes as well
        self._stage_pixels = torch.cuda.is_available() and (device is None or str(device).startswith("cuda"))
        self._closed = False
        if runner_group is not None:
            self.runners = runner_group
        elif cfg.tp > 1:
            from ..parallel.tp_group import TensorParallelGroup

            self.runners = TensorParallelGroup(cfg, weights=weights)
            if self.runners.is_driver:
                cfg.with_cache_capacity(*self.runners.call("capacity"))
        else:
            from .model_runner import ModelRunner

            self.runners = LocalRunnerGroup(ModelRunner(cfg, device=device, weights=weights))
        # the runner resolved the KV capacity into the config
        self.scheduler = Scheduler(cfg, metrics=self.metrics)
        self.executor = ModelExecutor(cfg, self.runners, self.scheduler.block_manager)
        self._sequences: dict[int, Sequence] = {}
        self._cooperative_pending = False
        self._pending_prefill = None          # executor handle of a prefill whose layers run in quanta
        self._deferred: list[StepResult] = []  # results produced outside step_result (a pending prefill drained by a cancel)
        self._decode_after_interrupt = False
        self._pending_vision: dict | None = None
        self.cooperative_counters = {"vision_quanta": 0, "vision_block_quanta": 0, "layer_quantum_prefills": 0, "layer_quanta": 0, "decode_steps_between_quanta": 0,
                                     "slo_prefill_interruptions": 0, "slo_pending_deadline_finishes": 0, "slo_deadline_atomic_prefills": 0,
                                     "slo_light_atomic_prefills": 0, "coalesce_deferred_decode_steps": 0, "coalesce_deadline_releases": 0,
                                     "coalesced_atomic_prefills": 0, "underfilled_atomic_prefills": 0}
        self._fine_grain_latched = False
        self._steps_since_status = 0
        atexit.register(self.exit)

    def _validate_environment(self, device: str | None) -> None:
        """Fail before tokenizer, worker processes or weights exist (reference
        ``prism_infer/engine/llm_engine.py:151-167``).  A CPU engine (``device="cpu"``, the oracle
        and test path) needs neither a GPU nor the kernel library."""
        from ..parallel.tp_group import rank_info
        from ..runtime_capabilities import validate_runtime_capabilities, validate_tensor_parallel_environment

        cfg = self.config
        on_cuda = torch.cuda.is_available() if device is None else str(device).startswith("cuda")
        if on_cuda:
            validate_runtime_capabilities(True, execution_backend=cfg.prism.execution.backend,
                                          compression_mode=cfg.compression_mode)
        if cfg.tp > 1:
            devices = torch.cuda.device_count() if on_cuda else cfg.tp  # CPU ranks (gloo) need no devices
            validate_tensor_parallel_environment(self.arch, cfg.tp, devices, world_size=rank_info()[1])

    # ------------------------------------------------------------------- lifecycle
    def exit(self) -> None:
        if self._closed:
            return
        self._closed = True
        try:
            self.runners.close()
        except Exception:  # pragma: no cover - shutdown must not raise
            pass

    # ------------------------------------------------------------------ submission
    def _sampling(self, sp: SamplingParams | None) -> SamplingParams:
        return sp if sp is not None else SamplingParams()

    def _submit(self, seq: Sequence, *, raise_on_reject: bool = True) -> int:
        cfg = self.config
        seq.arrival_ns = seq.arrival_ns or time.perf_counter_ns()
        self.metrics.on_request_submitted(seq)
        self._sequences[seq.seq_id] = seq
        hit = None
        if seq.is_multimodal and seq.multimodal_prefix_cache_key:
            hit = self.scheduler.block_manager.probe_multimodal_prefix(seq)
        if (cfg.enable_visual_embedding_cache and cfg.tp == 1 and seq.is_multimodal and hit is None
                and seq.pixel_values is not None and seq.visual_embedding_cache_key):
            grids = list(seq.image_grid_thw) + list(seq.video_grid_thw)
            self.runners.call("hydrate_visual_embedding", VisionJob(seq.seq_id, seq.pixel_values, grids,
                                                                    seq.visual_embedding_cache_key))
            self.executor.mark_visual_ready(seq.seq_id)
        if not self.scheduler.add(seq):
            self.executor.drop_visual(seq.seq_id)
            self.metrics.on_request_finished(seq)
            if raise_on_reject:
                raise ValueError(f"request rejected: {seq.lifecycle.finish_reason}")
        return seq.seq_id

    def add_request(self, prompt: str | Seq[int], sampling_params: SamplingParams | None = None, *,
                    raise_on_reject: bool = True) -> int:
        ids = self.tokenizer.encode(prompt) if isinstance(prompt, str) else [int(t) for t in prompt]
        seq = Sequence(self._ids(), ids, self._sampling(sampling_params), image_token_id=self.arch.image_token_id,
                       video_token_id=self.arch.video_token_id)
        return self._submit(seq, raise_on_reject=raise_on_reject)

    def stage_pixels(self, pixels: torch.Tensor | None) -> torch.Tensor | None:
        """Patches in the form the runner copies from (pinned bf16 on CUDA engines, unchanged
        elsewhere).  Callers that preprocess ahead of submission (the online session's background
        thread) can call this themselves; an already staged tensor passes through."""
        if not self._stage_pixels or pixels is None or (pixels.dtype == torch.bfloat16 and pixels.is_pinned()):
            return pixels
        staged = torch.empty(pixels.shape, dtype=torch.bfloat16, pin_memory=True)
        staged.copy_(pixels)
        return staged

    def _multimodal_sequence(self, inputs: ImageInputs | VideoInputs, sp: SamplingParams | None,
                             media_key: str | None = None) -> Sequence:
        arch = self.arch
        image_grid = getattr(inputs, "image_grid_thw", None)
        video_grid = getattr(inputs, "video_grid_thw", None)
        inputs.validate(arch)
        pixels = self.stage_pixels(inputs.pixel_values)
        pos, delta = rope_index(inputs.input_ids, image_grid_thw=image_grid, video_grid_thw=video_grid,
                                image_token_id=arch.image_token_id, video_token_id=arch.video_token_id,
                                spatial_merge_size=arch.vision.spatial_merge_size)
        seq = Sequence(self._ids(), inputs.input_ids, self._sampling(sp), image_token_id=arch.image_token_id,
                       video_token_id=arch.video_token_id, pixel_values=pixels,
                       image_grid_thw=image_grid, video_grid_thw=video_grid, position_ids=pos[:, 0, :],
                       rope_delta=delta, merge_size=arch.vision.spatial_merge_size)
        if self.config.enable_prefix_caching or self.config.enable_visual_embedding_cache:
            key = media_key or content_key(pixels, image_grid, video_grid)
            seq.visual_embedding_cache_key = key
            if self.config.enable_prefix_caching:
                seq.multimodal_prefix_cache_key = key
        return seq

    def add_prepared_image_request(self, inputs: ImageInputs, sampling_params: SamplingParams | None = None, *,
                                   media_key: str | None = None, raise_on_reject: bool = True) -> int:
        return self._submit(self._multimodal_sequence(inputs, sampling_params, media_key), raise_on_reject=raise_on_reject)

    def add_prepared_video_request(self, inputs: VideoInputs, sampling_params: SamplingParams | None = None, *,
                                   media_key: str | None = None, raise_on_reject: bool = True) -> int:
        return self._submit(self._multimodal_sequence(inputs, sampling_params, media_key), raise_on_reject=raise_on_reject)

    def prepare_images(self, prompt: str | Seq[int], images: Seq[Any], *, image_marker: str | None = None) -> ImageInputs:
        """Prompt + images -> ``ImageInputs`` the way this engine was configured: chat turns around a
        string prompt when the checkpoint has a chat template, the checkpoint's Hugging Face processor
        when ``hf_processor="always"``, the built-in patch processor otherwise.  ``image_marker``
        selects the interleaved layout (images where the marker appears in the prompt)."""
        images = list(images)
        if self.hf_processor is not None and isinstance(prompt, str):
            chat = self.hf_processor.chat
            text = (chat.interleaved_image_prompt(prompt, len(images), image_marker=image_marker) if image_marker
                    else chat.image_prompt(prompt, len(images)))
            return self.hf_processor.image_inputs(text, images)
        if image_marker:
            return prepare_interleaved_image_inputs(self.processor, self.tokenizer, prompt, images, image_marker, chat=self.chat)
        return prepare_image_inputs(self.processor, self.tokenizer, prompt, images, chat=self.chat)

    def prepare_video(self, prompt: str | Seq[int], frames: Seq[Any] | str, *, timing=None) -> VideoInputs:
        """Prompt + sampled frames (+ ``chat_prompt.VideoTiming``) -> ``VideoInputs``; see ``prepare_images``.
        ``frames`` may also be the path of a video file: its frames are sampled at two per second of source time
        (4 to 768 of them, evenly spaced) and their source times go into the prompt's time stamps."""
        if isinstance(frames, (str, os.PathLike)):
            p = self.processor
            frames, file_timing = load_video_file(os.fspath(frames), fps=p.video_fps, min_frames=p.video_min_frames, max_frames=p.video_max_frames)
            timing = timing or file_timing
        frames = list(frames)
        if self.hf_processor is not None and isinstance(prompt, str):
            return self.hf_processor.video_inputs(self.hf_processor.chat.video_prompt(prompt), frames, timing)
        return prepare_video_inputs(self.processor, self.tokenizer, prompt, frames, chat=self.chat, timing=timing)

    def add_vl_request(self, prompt: str | Seq[int], image: Any, sampling_params: SamplingParams | None = None, **kw) -> int:
        with profile_region("preprocess.image", cuda=False):
            inputs = self.prepare_images(prompt, [image])
        return self.add_prepared_image_request(inputs, sampling_params, **kw)

    def add_images_request(self, prompt: str | Seq[int], images: Seq[Any], sampling_params: SamplingParams | None = None, **kw) -> int:
        with profile_region("preprocess.images", cuda=False):
            inputs = self.prepare_images(prompt, images)
        return self.add_prepared_image_request(inputs, sampling_params, **kw)

    def add_interleaved_images_request(self, prompt: str, images: Seq[Any], sampling_params: SamplingParams | None = None,
                                       *, image_marker: str = "<image>", **kw) -> int:
        with profile_region("preprocess.interleaved_images", cuda=False):
            inputs = self.prepare_images(prompt, images, image_marker=image_marker)
        return self.add_prepared_image_request(inputs, sampling_params, **kw)

    def add_video_request(self, prompt: str | Seq[int], frames: Seq[Any], sampling_params: SamplingParams | None = None, *,
                          timing=None, **kw) -> int:
        with profile_region("preprocess.video", cuda=False):
            inputs = self.prepare_video(prompt, frames, timing=timing)
        return self.add_prepared_video_request(inputs, sampling_params, **kw)

    # ------------------------------------------------------------------------ step
    def step_result(self) -> StepResult:
        with profile_region("engine.step", cuda=False):
            if self._deferred:
                return self._deferred.pop(0)
            if self._pending_vision is not None:
                return self._continue_pending_vision()
            if self._pending_prefill is not None:
                return self._continue_pending_prefill()
            if self._should_coalesce_prefill():
                with profile_region("engine.scheduler.schedule", cuda=False):
                    held = self.scheduler.schedule_decode(count=True)
                if held is not None:  # the waiting requests stay queued; the running ones take their step
                    self.cooperative_counters["coalesce_deferred_decode_steps"] += 1
                    return self._run_plan(held)
            policy = self.scheduler.policy
            heavy_gap = getattr(policy, "decode_batches_since_heavy", None)
            with profile_region("engine.scheduler.schedule", cuda=False):
                plan = self.scheduler.schedule()
            if plan.is_idle and plan.kv_transfers.empty:
                return StepResult(Phase.IDLE)
            cooperative = self.config.cooperative_prefill and plan.phase is Phase.PREFILL and self.scheduler.num_decoding > 0
            if cooperative and plan.num_vision_patches > 0 and not self._cooperative_pending:
                # vision quantum now, language prefill on a later step.  The plan's page transfers
                # ran with the quantum; the scheduler lists a transfer only in the plan that admits
                # its sequence (or grows its table), so the re-planned prefill carries none of
                # them again and every transfer it does carry belongs to a new admission
                if self.config.cooperative_prefill_vision_block_quantum < self.arch.vision.depth:
                    # the tower a few blocks at a time, a decode step of the running sequences after every quantum
                    self._pending_vision = self.executor.begin_hydrate(plan)
                    if self._pending_vision is not None:
                        self._pending_vision["heavy_gap"] = heavy_gap
                        return self._continue_pending_vision()
                    self._cooperative_pending = False
                else:
                    self._cooperative_pending = self.executor.hydrate_vision(plan) > 0
                if self._cooperative_pending:
                    self.cooperative_counters["vision_quanta"] += 1
                    if heavy_gap is not None:
                        # the quantum is not the heavy prefill itself: the decode batches counted so far still stand,
                        # or the language prefill would wait a whole spacing interval behind its own vision tower
                        policy.decode_batches_since_heavy = heavy_gap
                    self.scheduler.consecutive_prefill_batches = self.scheduler.policy.max_consecutive_prefill
                    return StepResult(Phase.IDLE)
            self._cooperative_pending = False
            if cooperative and not self.executor.attention_strategy:
                cooperative = self._cooperative_is_useful(plan)
            if cooperative and not self.executor.attention_strategy:
                # layer quanta: the prefill's embedding now, its decoder layers a few at a time with a decode step
                # of the running sequences after every quantum (reference engine/llm_engine.py:1040-1103)
                profile_step_metadata({"phase": "prefill_begin", "batch_size": plan.batch_size, "tokens": plan.num_tokens,
                                       "vision_patches": plan.num_vision_patches})
                self._pending_prefill = self.executor.begin_prefill(plan)
                self.cooperative_counters["layer_quantum_prefills"] += 1
                return self._decode_between_quanta()
            return self._run_plan(plan)

    def _run_plan(self, plan) -> StepResult:
        profile_step_metadata({"phase": plan.phase.value, "batch_size": plan.batch_size, "tokens": plan.num_tokens,
                               "vision_patches": plan.num_vision_patches})
        result = self.executor.execute(plan)
        return self._commit(plan, result)

    def _commit(self, plan, result) -> StepResult:
        self._steps_since_status += 1
        if 0 < self.config.device_status_check_interval <= self._steps_since_status:
            self.check_device_status()
        if plan.is_idle:
            return StepResult(Phase.IDLE)
        with profile_region("engine.scheduler.postprocess", cuda=False):
            outputs = self.scheduler.postprocess(plan, result.tokens)
        self.metrics.on_batch_completed(plan, result.duration_ms, result.compactions)
        for o in outputs:
            if o.finished:
                self._sequences.pop(o.request_id, None)
        return StepResult(plan.phase, tuple(outputs), plan.num_tokens)

    # ---- cooperative prefill by layer quanta ------------------------------------------------------
    def _decode_between_quanta(self) -> StepResult:
        """One decode step of the running sequences while a prefill is pending; the scheduler's decode plan only
        touches decoding sequences (victims of a preemption included), never the ones whose prefill is under way."""
        with profile_region("engine.scheduler.schedule", cuda=False):
            plan = self.scheduler.schedule_decode(count=True)
        if plan is None:
            return StepResult(Phase.IDLE)
        self.cooperative_counters["decode_steps_between_quanta"] += 1
        return self._run_plan(plan)

    def _continue_pending_vision(self, *, drain: bool = False) -> StepResult:
        """One quantum of the pending vision-tower work, then (next call) a decode step; when the tower is done the
        language prefill is planned again by the following step."""
        handle = self._pending_vision
        if handle.pop("decode_next", False) and not drain and self.scheduler.num_decoding > 0:
            return self._decode_between_quanta()
        blocks = self.arch.vision.depth if (drain or self.scheduler.num_decoding == 0) else self.config.cooperative_prefill_vision_block_quantum
        done = self.executor.advance_hydrate(handle, blocks)
        self.cooperative_counters["vision_block_quanta"] += 1
        if not done:
            handle["decode_next"] = True
            return StepResult(Phase.IDLE)
        self._pending_vision = None
        self.cooperative_counters["vision_quanta"] += 1
        self._cooperative_pending = True
        policy = self.scheduler.policy
        if handle.get("heavy_gap") is not None:
            policy.decode_batches_since_heavy = max(handle["heavy_gap"], getattr(policy, "decode_batches_since_heavy", 0))
        self.scheduler.consecutive_prefill_batches = policy.max_consecutive_prefill
        return StepResult(Phase.IDLE)

    def _finish_pending_prefill(self) -> StepResult:
        handle, self._pending_prefill = self._pending_prefill, None
        result = self.executor.finish_prefill(handle)
        self.cooperative_counters["layer_quanta"] += handle["quanta"]
        return self._commit(handle["plan"], result)

    # ---- service-level side (SLO-aware policy; reference engine/llm_engine.py:870-912, 1040-1077) --------------
    def _release_ns(self, seq) -> int | None:
        """When a request's prefill has to run without further delay: its time-to-first-token deadline minus the
        reserve of its cost tier.  None without a deadline or without the SLO-aware policy."""
        policy = self.scheduler.policy
        if seq.deadline_ns is None or not hasattr(policy, "reserve_ns"):
            return None
        return seq.deadline_ns - policy.reserve_ns(seq)

    def _slo_due(self, seqs) -> bool:
        now = self.scheduler.clock_ns()
        return any(r is not None and now >= r for r in map(self._release_ns, seqs))

    def _cooperative_is_useful(self, plan) -> bool:
        """Whether a prefill that meets running decodes yields to them in layer quanta, or runs in one piece
        (reference engine/llm_engine.py:913-966)."""
        c = self.cooperative_counters
        policy = self.scheduler.policy
        if hasattr(policy, "cost_tier") and any(s.deadline_ns is not None for s in plan.seqs) \
                and all(policy.cost_tier(s) < 2 for s in plan.seqs):
            c["slo_light_atomic_prefills"] += 1  # cheap prompts with a deadline: quanta would only delay their first token
            return False
        if self._slo_due(plan.seqs):
            # a request of the plan has used up its time-to-first-token slack: no yielding to decode steps
            c["slo_deadline_atomic_prefills"] += 1
            return False
        if self.config.cooperative_prefill_coalesce_ms <= 0:
            return True
        if plan.batch_size >= self.config.cooperative_prefill_coalesce_min_seqs:
            c["coalesced_atomic_prefills"] += 1  # one pass over the weights serves many requests: worth stalling decode once
            return False
        if self.scheduler.num_decoding >= max(1, (self.config.max_num_seqs + 3) // 4):
            self._fine_grain_latched = True      # stays on: the engine has been under load
        heavy = plan.num_vision_patches >= self.config.heavy_prefill_vision_patch_threshold
        if heavy or self._fine_grain_latched:
            return True
        c["underfilled_atomic_prefills"] += 1
        return False

    def _should_coalesce_prefill(self) -> bool:
        """Hold a few waiting requests back while sequences decode, so that one prefill can serve more of them: until
        the oldest has waited ``cooperative_prefill_coalesce_ms``, or a waiting request reaches its release time,
        or enough of them have gathered (reference engine/llm_engine.py:986-1017)."""
        cfg = self.config
        if not cfg.cooperative_prefill or cfg.cooperative_prefill_coalesce_ms <= 0 or self.scheduler.num_decoding == 0:
            return False
        waiting = list(self.scheduler.waiting)
        if not waiting or len(waiting) >= cfg.cooperative_prefill_coalesce_min_seqs:
            return False
        if any(s.state is RequestState.PREFILLING for s in self.scheduler.running):
            return False  # a chunked prefill under way is not held up
        arrivals = [s.arrival_ns for s in waiting if s.arrival_ns is not None]
        if not arrivals:
            return False
        fixed = min(arrivals) + int(cfg.cooperative_prefill_coalesce_ms * 1e6)
        release = min([fixed] + [r for r in map(self._release_ns, waiting) if r is not None])
        wait = self.scheduler.clock_ns() < release
        if not wait and release < fixed:
            self.cooperative_counters["coalesce_deadline_releases"] += 1
        return wait

    def _slo_interrupt_tier(self) -> int | None:
        """The cost tier an interrupting prefill may admit up to, when a waiting request that is cheaper than
        everything in the pending prefill has reached its release time."""
        policy = self.scheduler.policy
        if not hasattr(policy, "cost_tier"):
            return None
        pending_tier = min(policy.cost_tier(s) for s in self._pending_prefill["plan"].seqs)
        if pending_tier <= 0:
            return None
        now = self.scheduler.clock_ns()
        for seq in self.scheduler.waiting:
            release = self._release_ns(seq)
            if policy.cost_tier(seq) < pending_tier and release is not None and now >= release:
                return pending_tier - 1
        return None

    def _continue_pending_prefill(self) -> StepResult:
        if self._decode_after_interrupt:  # the running sequences get their step before the next decision
            self._decode_after_interrupt = False
            if self.scheduler.num_decoding > 0:
                return self._decode_between_quanta()
        tier = self._slo_interrupt_tier()
        if tier is not None:
            with profile_region("engine.scheduler.schedule", cuda=False):
                plan = self.scheduler.schedule_prefill(max_cost_tier=tier)
            if plan is not None:
                self.cooperative_counters["slo_prefill_interruptions"] += 1
                self._decode_after_interrupt = True
                return self._run_plan(plan)
        if self._slo_due(self._pending_prefill["plan"].seqs):
            self.cooperative_counters["slo_pending_deadline_finishes"] += 1
            return self._finish_pending_prefill()
        if self.scheduler.num_decoding == 0:  # nothing left to protect: run the rest in one piece
            return self._finish_pending_prefill()
        done = self.executor.advance_prefill(self._pending_prefill, self.config.cooperative_prefill_layer_quantum)
        if done:
            return self._finish_pending_prefill()
        return self._decode_between_quanta()

    def step(self) -> tuple[list[tuple[int, list[int]]], int]:
        """Compatibility form: ``([(request_id, completion_token_ids), ...], signed token count)``
        where the count is positive for prefill and negative for decode."""
        res = self.step_result()
        done = [(o.request_id, list(o.token_ids)) for o in res.finished]
        return done, (res.num_tokens if res.phase is Phase.PREFILL else -res.num_tokens)

    def is_finished(self) -> bool:
        return self.scheduler.is_finished() and not self._deferred

    def check_device_status(self) -> None:
        """Read every rank's kernel status words (bounded waits that ran out, failed bounds checks;
        kernels never trap, they record and carry on) and raise when one is set.  The step loop
        calls this every ``device_status_check_interval`` steps, so a missing peer or a corrupt page
        table surfaces as an engine failure - an ``ERROR`` event and an unhealthy ``/health`` under
        ``prism-serve`` - instead of silently wrong tokens."""
        self._steps_since_status = 0
        answer = self.runners.call("status")
        per_rank = answer if isinstance(answer, list) else [answer]
        bad = {(rank, unit): words for rank, st in enumerate(per_rank) if st for unit, words in st.items() if words[0] != 0}
        if bad:
            raise RuntimeError(f"device status reports failures (rank, unit) -> (code, detail, block, count): {bad}")

    def cancel_request(self, request_id: int) -> bool:
        vision = self._pending_vision
        if vision is not None and any(job.seq_id == request_id for job in vision["jobs"]):
            # the runner holds a half-run tower pass for this plan: let it finish, then drop the result with the request
            while self._pending_vision is not None:
                self._continue_pending_vision(drain=True)
        pending = self._pending_prefill
        if pending is not None and any(seq.seq_id == request_id for seq in pending["plan"].seqs):
            # its pages must stay allocated until the layers that still write them have run: finish the prefill
            # first (the other sequences' first tokens are delivered by the next step_result), then cancel
            self._deferred.append(self._finish_pending_prefill())
        ok = self.scheduler.cancel(request_id)
        self.executor.drop_visual(request_id)
        self._sequences.pop(request_id, None)
        return ok

    def set_first_token_deadline(self, request_id: int, ttft_slo_ms: float) -> bool:
        """Give an open request a time-to-first-token target, counted from its arrival.  The SLO-aware scheduler policy
        orders the waiting queue by these deadlines and the cooperative prefill yields to them; under the other policies
        the value is recorded and changes nothing.  Call it right after the request was added, before the next step.
        False when the request is unknown."""
        if not (float(ttft_slo_ms) > 0.0) or float(ttft_slo_ms) == float("inf"):
            raise ValueError("ttft_slo_ms must be a finite positive number")
        seq = self._sequences.get(request_id) or self.scheduler.find(request_id)
        if seq is None:
            return False
        seq.deadline_ns = int(seq.arrival_ns or time.perf_counter_ns()) + int(float(ttft_slo_ms) * 1e6)
        return True

    def prompt_token_count(self, request_id: int) -> int | None:
        """Length of an open request's prompt as the model sees it (media placeholders expanded); ``None`` once the
        request is gone."""
        seq = self._sequences.get(request_id) or self.scheduler.find(request_id)
        return int(seq.num_prompt_tokens) if seq is not None else None

    def request_state(self, request_id: int) -> RequestState | None:
        seq = self._sequences.get(request_id) or self.scheduler.find(request_id)
        return seq.state if seq is not None else None

    # --------------------------------------------------------------------- metrics
    def metrics_snapshot(self) -> dict[str, object]:
        return {"engine": self.metrics.snapshot(), "scheduler": self.scheduler.metrics_snapshot()}

    def reset_metrics(self) -> None:
        self.metrics.reset()

    def serving_stats(self) -> dict[str, float]:
        """Flat ``name -> number`` view of the host-side counters, for a metrics endpoint: scheduler queues and counters,
        KV pages, the multimodal prefix cache, the cooperative-prefill counters and latency summaries of the finished
        newest 2048 finished requests.  No command goes to the worker ranks and no device work is issued, so the
        owner thread can call it between steps at any cadence."""
        from ..analysis.online_serving import percentile

        out: dict[str, float] = {}
        for k, v in self.scheduler.metrics_snapshot().items():
            out[f"scheduler_{k}"] = float(v)
        pool = self.scheduler.block_manager.gpu
        out["kv_pages_total"] = float(pool.num_blocks)
        out["kv_pages_used"] = float(pool.num_blocks - pool.num_free)
        out["kv_bytes_per_page"] = float(self.config.kv_bytes_per_page())
        for k, v in self.scheduler.block_manager.prefix_cache_metadata().items():
            if isinstance(v, (int, float)) and not isinstance(v, bool) and k not in ("free_pages", "total_pages"):
                out[f"prefix_cache_{k}"] = float(v)
        for k, v in self.cooperative_counters.items():
            if isinstance(v, (int, float)) and not isinstance(v, bool):
                out[f"cooperative_{k}"] = float(v)
        done = self.metrics.recent_finished(2048)
        out["latency_window_requests"] = float(len(done))
        for key in ("ttft_ms", "tpot_ms", "queue_ms", "latency_ms"):
            xs = sorted(float(r[key]) for r in done if r.get(key) is not None)
            if xs:
                out[f"{key}_p50"], out[f"{key}_p99"] = percentile(xs, 0.5), percentile(xs, 0.99)
        return out

    def multimodal_prefix_cache_metadata(self) -> dict[str, object]:
        meta = self.scheduler.block_manager.prefix_cache_metadata()
        per_page = self.config.kv_bytes_per_page()
        meta["resident_bytes"] = int(meta["resident_pages"]) * per_page
        meta["bytes_per_page"] = per_page
        return meta

    def visual_embedding_cache_metadata(self) -> dict[str, object]:
        return self.runners.call("visual_embedding_cache_metadata")

    def visual_pruning_decisions(self, *, clear: bool = False) -> list[dict[str, object]]:
        """What was kept of every recent prompt's visual tokens: applied selections of the compacting modes, and with
        ``enable_visual_pruning_shadow`` the selections a compacting mode would have made (``applied`` false)."""
        out = [dict(r) for r in self.executor.pruning_decisions]
        if clear:
            self.executor.pruning_decisions.clear()
        return out

    def graph_metadata(self) -> dict[str, object]:
        return self.runners.call("graph_metadata")

    def cooperative_prefill_policy_metadata(self) -> dict[str, object]:
        return {"enabled": self.config.cooperative_prefill, **self.cooperative_counters}

    def barrier(self) -> None:
        """Wait until every rank's device has finished the work issued so far."""
        self.runners.call("barrier")

    def keep_logits(self, on: bool = True) -> None:
        """Debugging aid (eager execution only): keep the full fp32 logits of the last sampled rows."""
        self.runners.call("keep_logits", bool(on))

    def last_logits(self):
        """``[rows, vocab]`` fp32 CPU tensor of the rows sampled in the last step, or ``None``."""
        return self.runners.call("last_logits")

    def time_decode_graph(self, steps: int) -> float:
        """Device ms per decode step from back-to-back graph launches (max over ranks)."""
        res = self.runners.call("time_decode_graph", steps)
        return max(res) if isinstance(res, (list, tuple)) else float(res)

    @property
    def is_driver(self) -> bool:
        return getattr(self.runners, "is_driver", True)

    def serve_forever(self) -> None:
        """Tensor-parallel worker ranks (torchrun launch) execute rank 0's commands here."""
        self.runners.serve_forever()

    # -------------------------------------------------------------------- generate
    def _format(self, token_ids: list[int]) -> dict[str, Any]:
        raw = self.tokenizer.decode(token_ids, skip_special_tokens=False)
        text = self.tokenizer.decode(token_ids, skip_special_tokens=True)
        return {"text": text, "raw_text": raw, "token_ids": list(token_ids)}

    def _run_until_done(self, ids: list[int], use_tqdm: bool | None = None) -> dict[int, list[int]]:
        want = set(ids)
        out: dict[int, list[int]] = {}
        with GenerationProgress(len(want), enabled=use_tqdm) as progress:
            while want - set(out):
                t0 = time.perf_counter()
                res = self.step_result()
                progress.observe_step(res.phase, res.num_tokens, time.perf_counter() - t0)
                for o in res.finished:
                    out[o.request_id] = list(o.token_ids)
                    if o.request_id in want:
                        progress.complete_request()
                if res.phase is Phase.IDLE and self.is_finished():
                    break
        for rid in want - set(out):  # rejected or cancelled
            out[rid] = []
        return out

    def _broadcast_sp(self, n: int, sp) -> list[SamplingParams | None]:
        if isinstance(sp, (list, tuple)):
            if len(sp) != n:
                raise ValueError("one SamplingParams per prompt is required")
            return list(sp)
        return [sp] * n

    def generate(self, prompts: Seq[str] | Seq[Seq[int]], sampling_params=None, use_tqdm: bool | None = None) -> list[dict[str, Any]]:
        sps = self._broadcast_sp(len(prompts), sampling_params)
        ids = [self.add_request(p, sp) for p, sp in zip(prompts, sps)]
        done = self._run_until_done(ids, use_tqdm)
        return [self._format(done[i]) for i in ids]

    def generate_vl(self, prompt, image, sampling_params=None, use_tqdm: bool | None = None) -> dict[str, Any]:
        rid = self.add_vl_request(prompt, image, sampling_params)
        return self._format(self._run_until_done([rid], use_tqdm)[rid])

    def generate_images(self, prompt, images, sampling_params=None, use_tqdm: bool | None = None) -> dict[str, Any]:
        rid = self.add_images_request(prompt, images, sampling_params)
        return self._format(self._run_until_done([rid], use_tqdm)[rid])

    def generate_interleaved_images(self, prompt, images, sampling_params=None, use_tqdm: bool | None = None, *,
                                    image_marker: str = "<image>") -> dict[str, Any]:
        rid = self.add_interleaved_images_request(prompt, images, sampling_params, image_marker=image_marker)
        return self._format(self._run_until_done([rid], use_tqdm)[rid])

    def generate_video(self, prompt, frames, sampling_params=None, use_tqdm: bool | None = None) -> dict[str, Any]:
        rid = self.add_video_request(prompt, frames, sampling_params)
        return self._format(self._run_until_done([rid], use_tqdm)[rid])

    def generate_prepared_image_inputs(self, inputs: ImageInputs, sampling_params=None, use_tqdm: bool | None = None) -> dict[str, Any]:
        rid = self.add_prepared_image_request(inputs, sampling_params)
        return self._format(self._run_until_done([rid], use_tqdm)[rid])

    def generate_prepared_video_inputs(self, inputs: VideoInputs, sampling_params=None, use_tqdm: bool | None = None) -> dict[str, Any]:
        rid = self.add_prepared_video_request(inputs, sampling_params)
        return self._format(self._run_until_done([rid], use_tqdm)[rid])

    def generate_mixed(self, requests: Seq[dict[str, Any]], sampling_params=None, use_tqdm: bool | None = None) -> list[dict[str, Any]]:
        """Batch of heterogeneous requests: each dict has ``type`` in ``text | image | images |
        interleaved_images | video`` plus ``prompt`` and the matching media field."""
        sps = self._broadcast_sp(len(requests), sampling_params)
        ids = []
        for req, sp in zip(requests, sps):
            kind = req.get("type", "text")
            sp = req.get("sampling_params", sp)
            if kind == "text":
                ids.append(self.add_request(req["prompt"], sp))
            elif kind == "image":
                ids.append(self.add_vl_request(req["prompt"], req["image"], sp))
            elif kind == "images":
                ids.append(self.add_images_request(req["prompt"], req["images"], sp))
            elif kind == "interleaved_images":
                ids.append(self.add_interleaved_images_request(req["prompt"], req["images"], sp,
                                                               image_marker=req.get("image_marker", "<image>")))
            elif kind == "video":
                ids.append(self.add_video_request(req["prompt"], req.get("frames", req.get("video")), sp))
            else:
                raise ValueError(f"unknown request type {kind!r}")
        done = self._run_until_done(ids, use_tqdm)
        return [self._format(done[i]) for i in ids]
