"""Tensor-parallel rank group: process start-up, rendezvous and lock-step dispatch.

One process per GPU.  Rank 0 (the driver) owns the scheduler and sends every device action
(``execute``, KV page transfers, compaction, metadata queries) through the shared-memory
control plane; each rank, the driver included, applies it to its own ``ModelRunner``.
Ranks are either started by ``torch.distributed.run`` (every process builds ``LLM``; ranks
above 0 end up in ``serve_forever``) or spawned here from a single user process, as the
reference does (``prism_infer/engine/llm_engine.py:176-204``,
``prism_infer/engine/model_runner.py:229-245,424-476``).  ``torch.distributed`` is used for
rendezvous, IPC-handle exchange and the baseline / prefill collectives; the decode exchange
runs in the fused kernels over peer memory (``parallel/comm.py``).
"""

from __future__ import annotations

import os
import socket
import time
from typing import Any

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from .control import ControlDriver, ControlSegment, ControlWorker, TPMethod


def rank_info() -> tuple[int, int]:
    """``(rank, world size)`` of a process started by ``torch.distributed.run``; ``(0, 1)`` otherwise."""
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _init_process_group(rank: int, world: int, init_method: str, use_cuda: bool, timeout_s: int, store=None) -> None:
    """``init_method`` is ``tcp://host:port`` (external launch) or ``store://host:port`` for groups
    spawned here: the driver then already owns a ``TCPStore`` it bound to port 0 (passed as
    ``store``), so there is no window in which another process can take a probed "free" port."""
    import datetime

    if dist.is_initialized():
        return
    timeout = datetime.timedelta(seconds=timeout_s)
    kwargs: dict[str, Any] = dict(backend="nccl" if use_cuda else "gloo", rank=rank, world_size=world, timeout=timeout)
    if init_method.startswith("store://"):
        if store is None:
            host, port = init_method[len("store://"):].rsplit(":", 1)
            store = dist.TCPStore(host, int(port), world, False, timeout=timeout)
        kwargs["store"] = store
    else:
        kwargs["init_method"] = init_method
    if use_cuda:
        kwargs["device_id"] = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group(**kwargs)


def _make_comm(rank: int, world: int, hidden: int, use_cuda: bool):
    from .comm import FusedComm, NcclComm

    mode = os.environ.get("PRISM_TP_COMM", "fused" if use_cuda else "nccl")
    if use_cuda and mode == "fused":
        return FusedComm(rank, world, hidden)
    return NcclComm(rank, world)


def _build_runner(config, rank: int, world: int, use_cuda: bool, weights):
    from ..engine.model_runner import ModelRunner

    comm = _make_comm(rank, world, config.arch.text.hidden_size, use_cuda)
    device = f"cuda:{torch.cuda.current_device()}" if use_cuda else "cpu"
    return ModelRunner(config, rank=rank, comm=comm, device=device, weights=weights)


def _share_host_threads(world: int) -> None:
    """Every rank is a process with its own intra-op thread pool; sized for the whole machine each, the pools
    of eight ranks fight over the cores whenever the ranks do the same host work at the same time."""
    cores = os.cpu_count() or 1
    torch.set_num_threads(max(1, min(torch.get_num_threads(), cores // max(1, world))))


def _worker_entry(rank: int, world: int, init_method: str, seg_name: str, model: str, flat_options: dict, weights,
                  use_cuda: bool) -> None:
    """Process target of a spawned worker rank."""
    from ..config import Config

    if use_cuda:
        torch.cuda.set_device(rank)
        _share_host_threads(world)
    config = Config(model, **flat_options)
    _init_process_group(rank, world, init_method, use_cuda, config.tensor_parallel_timeout_seconds)
    seg = ControlSegment(seg_name, world - 1, create=False)
    worker = ControlWorker(seg, rank - 1, rank)
    try:
        runner = _build_runner(config, rank, world, use_cuda, weights)
        dist.barrier()
        worker.serve(runner)
        runner.exit()
    finally:
        seg.close()
        if dist.is_initialized():
            dist.destroy_process_group()


class TensorParallelGroup:
    def __init__(self, config, *, weights=None, use_cuda: bool | None = None) -> None:
        self.config = config
        world = config.tp
        self.world = world
        self.use_cuda = torch.cuda.is_available() if use_cuda is None else use_cuda
        env_rank, env_world = rank_info()
        self.external = env_world > 1
        self.procs: list[mp.Process] = []
        self.seg: ControlSegment | None = None
        self.driver: ControlDriver | None = None
        self.worker: ControlWorker | None = None
        timeout = config.tensor_parallel_timeout_seconds
        if self.external:
            if env_world != world:
                raise ValueError(f"tensor_parallel_size {world} does not match WORLD_SIZE {env_world}")
            self.rank = env_rank
            if self.use_cuda:
                torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", env_rank)))
            addr, port = os.environ.get("MASTER_ADDR", "127.0.0.1"), os.environ.get("MASTER_PORT", "29500")
            _init_process_group(self.rank, world, f"tcp://{addr}:{port}", self.use_cuda, timeout)
            name = [None]
            if self.rank == 0:
                self.seg = ControlSegment(None, world - 1, create=True)
                name[0] = self.seg.name
            dist.broadcast_object_list(name, src=0)
            if self.rank != 0:
                self.seg = ControlSegment(name[0], world - 1, create=False)
        else:
            self.rank = 0
            if self.use_cuda:
                if torch.cuda.device_count() < world:
                    raise ValueError(f"tensor_parallel_size {world} needs {world} GPUs, found {torch.cuda.device_count()}")
                torch.cuda.set_device(0)
                _share_host_threads(world)
            import datetime

            master = dist.TCPStore("127.0.0.1", 0, world, True, timeout=datetime.timedelta(seconds=timeout), wait_for_workers=False)
            init_method = f"store://127.0.0.1:{master.port}"
            self.seg = ControlSegment(None, world - 1, create=True)
            ctx = mp.get_context("spawn")
            flat = dict(getattr(config, "_flat_options", {}))
            for r in range(1, world):
                p = ctx.Process(target=_worker_entry, args=(r, world, init_method, self.seg.name, config.model, flat,
                                                            weights, self.use_cuda), daemon=True)
                p.start()
                self.procs.append(p)
            try:
                _init_process_group(0, world, init_method, self.use_cuda, timeout, store=master)
            except Exception:
                self._terminate_workers()
                raise
        if self.rank == 0:
            self.driver = ControlDriver(self.seg, timeout_s=float(timeout),
                                        exit_codes=(lambda: [p.exitcode for p in self.procs]) if self.procs else None)
        else:
            self.worker = ControlWorker(self.seg, self.rank - 1, self.rank)
        try:
            self.runner = _build_runner(config, self.rank, world, self.use_cuda, weights)
            dist.barrier()
        except Exception:
            self._terminate_workers()
            raise

    # ------------------------------------------------------------------------------
    @property
    def is_driver(self) -> bool:
        return self.rank == 0

    def call(self, method: str, *args):
        """Run ``method`` on every rank; returns rank 0's value (all ranks' for timings)."""
        if not self.is_driver:
            raise RuntimeError("only the driver rank issues commands")
        assert self.driver is not None
        rid = self.driver.post(method, args)
        local_error: BaseException | None = None
        value = None
        try:
            value = getattr(self.runner, method)(*args)
        except BaseException as exc:  # noqa: BLE001 - re-raised after the workers were heard
            local_error = exc
        try:
            others = self.driver.collect(method, rid)
        except Exception as exc:
            if local_error is not None:
                raise exc from local_error
            raise
        if local_error is not None:
            raise local_error
        if method in (TPMethod.TIME_DECODE_GRAPH.value, TPMethod.STATUS.value):
            return [value, *others]  # per-rank answers
        return value

    def barrier(self) -> None:
        self.call("barrier")

    def serve_forever(self) -> None:
        assert self.worker is not None
        try:
            self.worker.serve(self.runner)
        finally:
            self.runner.exit()
            self._teardown()

    def _terminate_workers(self) -> None:
        for p in self.procs:
            if p.is_alive():
                p.terminate()
        for p in self.procs:
            p.join(timeout=5)
            if p.is_alive():
                p.kill()

    def _teardown(self) -> None:
        comm = getattr(self.runner, "comm", None)
        if hasattr(comm, "close"):
            try:
                if self.use_cuda:
                    torch.cuda.synchronize()
                comm.close()
            except Exception:
                pass
        if self.seg is not None:
            self.seg.close()
            self.seg = None
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:
                pass

    def close(self) -> None:
        """Shut the group down: ask workers to exit, then escalate join -> terminate -> kill."""
        if self.is_driver and self.driver is not None and self.seg is not None:
            try:
                rid = self.driver.post(TPMethod.EXIT, ())
                self.driver.collect("exit", rid, timeout_s=10.0)
            except Exception:
                pass
            self.driver.shutdown()
        deadline = time.monotonic() + 10.0
        for p in self.procs:
            p.join(timeout=max(0.1, deadline - time.monotonic()))
        self._terminate_workers()
        self.runner.exit()
        self._teardown()
