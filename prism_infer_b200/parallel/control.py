"""Host control plane between the driver rank and the tensor-parallel workers.

A typed request / acknowledge RPC like the reference's pipe-based plane
(``prism_infer/engine/tp_control.py:14-366``: whitelisted methods, monotonically increasing
request ids, a deadline per command that names the ranks still pending, worker tracebacks
forwarded to the driver), but carried by one shared-memory segment instead of pickled
pipes: the driver writes the command once, every worker polls a sequence word, executes,
and writes its acknowledgement into its own slot.  There is no per-step system call on the
decode path, which matters when a tensor-parallel decode step takes a few hundred
microseconds.

Segment layout (little-endian 64-bit words unless noted)::

    [0]   command sequence number (written last by the driver)
    [1]   payload length in bytes
    [2]   shutdown flag
    [3]   payload capacity in bytes        [4]   reply capacity per worker in bytes
    [8 + 8*r ...]  per-worker slot r: ack sequence, status (0 ok, 1 error), reply length
    [HEADER ...]                       command payload (see below)
    [HEADER + payload_cap + r*reply_cap ...]   reply area of worker r (pickle)

Command payload: ``u64 n_buffers, u64 pickle_length, u64 size[n_buffers]``, the pickle
(protocol 5), then every out-of-band buffer at a 64-byte boundary.  Arrays of 64 KiB and more
(pixel patches of a prefill) travel out of band: the driver copies them into the segment once
and the workers unpickle zero-copy views of the segment, valid until they acknowledge.
"""

from __future__ import annotations

import enum
import pickle
import time
import traceback
from multiprocessing import shared_memory
from typing import Any, Callable

import numpy as np

HEADER_WORDS = 8 + 8 * 64
HEADER_BYTES = HEADER_WORDS * 8
DEFAULT_PAYLOAD_CAP = 96 << 20
DEFAULT_REPLY_CAP = 1 << 20


class TPMethod(enum.Enum):
    """Whitelist of runner methods a command may name."""

    EXECUTE = "execute"
    APPLY_KV_TRANSFERS = "apply_kv_transfers"
    COMPACT_KV = "compact_kv"
    HYDRATE_VISUAL_EMBEDDING = "hydrate_visual_embedding"
    ENCODE_FOR_SEQUENCE = "encode_for_sequence"
    RELEASE_VISUAL = "release_visual"
    TAKE_VISUAL_SCORES = "take_visual_scores"
    VISUAL_EMBEDDING_CACHE_METADATA = "visual_embedding_cache_metadata"
    GRAPH_METADATA = "graph_metadata"
    TIME_DECODE_GRAPH = "time_decode_graph"
    CAPACITY = "capacity"
    BARRIER = "barrier"
    KEEP_LOGITS = "keep_logits"
    LAST_LOGITS = "last_logits"
    STATUS = "status"
    EXIT = "exit"


class TPControlError(RuntimeError):
    pass


class TPTimeout(TPControlError):
    def __init__(self, method: str, request_id: int, pending: list[int], deadline_s: float) -> None:
        super().__init__(f"tensor-parallel command {method!r} (request {request_id}) timed out after "
                         f"{deadline_s:.1f}s; pending ranks: {pending}")
        self.pending = pending


class TPWorkerExited(TPControlError):
    """A worker process ended while its acknowledgement was awaited (seen through the process handle, without
    waiting for the deadline)."""

    def __init__(self, method: str, request_id: int, exited: dict[int, int | None]) -> None:
        super().__init__(f"tensor-parallel command {method!r} (request {request_id}): worker process ended before it "
                         f"acknowledged; rank -> exit code: {exited}")
        self.exited = exited


class TPWorkerError(TPControlError):
    def __init__(self, rank: int, exc_type: str, message: str, tb: str) -> None:
        super().__init__(f"rank {rank} failed with {exc_type}: {message}\n--- worker traceback ---\n{tb}")
        self.rank, self.exc_type, self.worker_traceback = rank, exc_type, tb


class ControlSegment:
    """Shared-memory segment plus typed views; created by the driver, attached by workers."""

    def __init__(self, name: str | None, n_workers: int, *, create: bool, payload_cap: int = DEFAULT_PAYLOAD_CAP,
                 reply_cap: int = DEFAULT_REPLY_CAP) -> None:
        self.n_workers = n_workers
        size = HEADER_BYTES + payload_cap + n_workers * reply_cap
        if create:
            self.shm = shared_memory.SharedMemory(name=name, create=True, size=size)
            self.shm.buf[:HEADER_BYTES] = bytes(HEADER_BYTES)
        else:
            self.shm = shared_memory.SharedMemory(name=name, create=False)
        self.owner = create
        self.words = np.ndarray((HEADER_WORDS,), dtype=np.int64, buffer=self.shm.buf)
        self.buf = self.shm.buf
        if create:
            self.words[3], self.words[4] = payload_cap, reply_cap
        # the geometry travels in the header so attaching processes never guess it
        self.payload_cap, self.reply_cap = int(self.words[3]), int(self.words[4])

    @property
    def name(self) -> str:
        return self.shm.name

    def payload(self, n: int) -> memoryview:
        return self.buf[HEADER_BYTES:HEADER_BYTES + n]

    def reply(self, worker: int, n: int) -> memoryview:
        off = HEADER_BYTES + self.payload_cap + worker * self.reply_cap
        return self.buf[off:off + n]

    def close(self) -> None:
        self.words = None  # release the exported buffer before closing
        self.buf = None
        try:
            self.shm.close()
            if self.owner:
                self.shm.unlink()
        except (FileNotFoundError, BufferError):
            pass


OUT_OF_BAND_MIN_BYTES = 64 << 10
PAYLOAD_KIND_WORD = 5   # header word: how the command area is encoded
PAYLOAD_PICKLE, PAYLOAD_DECODE = 0, 1


def write_payload(seg: ControlSegment, obj: Any) -> int:
    """Serialise ``obj`` into the command area; returns the number of bytes used."""
    buffers: list[pickle.PickleBuffer] = []

    def keep_in_band(buf: pickle.PickleBuffer) -> bool:
        if buf.raw().nbytes < OUT_OF_BAND_MIN_BYTES:
            return True
        buffers.append(buf)
        return False

    blob = pickle.dumps(obj, protocol=5, buffer_callback=keep_in_band)
    head = 16 + 8 * len(buffers)
    offsets, cursor = [], (head + len(blob) + 63) // 64 * 64
    for b in buffers:
        offsets.append(cursor)
        cursor = (cursor + b.raw().nbytes + 63) // 64 * 64
    if cursor > seg.payload_cap:
        raise TPControlError(f"command payload of {cursor} bytes exceeds the channel capacity")
    area = seg.payload(cursor)
    words = np.ndarray((2 + len(buffers),), dtype=np.int64, buffer=area)
    words[0], words[1] = len(buffers), len(blob)
    for i, b in enumerate(buffers):
        words[2 + i] = b.raw().nbytes
    area[head:head + len(blob)] = blob
    for off, b in zip(offsets, buffers):
        raw = b.raw()
        area[off:off + raw.nbytes] = raw
    return cursor


def read_payload(seg: ControlSegment, total: int) -> Any:
    area = seg.payload(total)
    n_buf, blob_len = (int(v) for v in np.ndarray((2,), dtype=np.int64, buffer=area))
    sizes = [int(v) for v in np.ndarray((n_buf,), dtype=np.int64, buffer=area, offset=16)]
    head = 16 + 8 * n_buf
    views, cursor = [], (head + blob_len + 63) // 64 * 64
    for size in sizes:
        views.append(area[cursor:cursor + size])
        cursor = (cursor + size + 63) // 64 * 64
    return pickle.loads(bytes(area[head:head + blob_len]), buffers=views)


class ControlDriver:
    """Driver side: broadcast a command, run the local copy, collect acknowledgements."""

    def __init__(self, segment: ControlSegment, *, timeout_s: float = 120.0, worker_ranks: list[int] | None = None,
                 exit_codes: Callable[[], list[int | None]] | None = None, liveness_period_s: float = 0.05) -> None:
        """``exit_codes()`` (optional; the group that spawned the workers reads their process handles) gives per worker
        ``None`` while its process runs and its exit code afterwards; it is asked every ``liveness_period_s`` while
        acknowledgements are pending, so a worker that died is reported at once instead of at the deadline."""
        self.seg = segment
        self.timeout_s = timeout_s
        self.exit_codes = exit_codes
        self.liveness_period_s = liveness_period_s
        self.request_id = 0
        self.worker_ranks = worker_ranks or list(range(1, segment.n_workers + 1))

    def post(self, method: TPMethod | str, args: tuple) -> int:
        m = TPMethod(method) if not isinstance(method, TPMethod) else method
        total = 0
        if m is TPMethod.EXECUTE and len(args) == 1 and hasattr(args[0], "pack_decode"):
            total = args[0].pack_decode(self.seg.payload(self.seg.payload_cap))  # fixed binary form of a decode step
        self.seg.words[PAYLOAD_KIND_WORD] = PAYLOAD_DECODE if total else PAYLOAD_PICKLE
        if not total:
            total = write_payload(self.seg, (m.value, args))
        self.seg.words[1] = total
        self.request_id += 1
        self.seg.words[0] = self.request_id  # publish last
        return self.request_id

    def collect(self, method: str, request_id: int, timeout_s: float | None = None) -> list[Any]:
        deadline_s = self.timeout_s if timeout_s is None else timeout_s
        deadline = time.monotonic() + deadline_s
        n = self.seg.n_workers
        done = [False] * n
        results: list[Any] = [None] * n
        spins = 0
        next_liveness = time.monotonic() + self.liveness_period_s
        while not all(done):
            for w in range(n):
                if done[w]:
                    continue
                base = 8 + 8 * w
                ack = int(self.seg.words[base])
                if ack > request_id:
                    raise TPControlError(f"rank {self.worker_ranks[w]} acknowledged request {ack}, expected {request_id}")
                if ack == request_id:
                    status, length = int(self.seg.words[base + 1]), int(self.seg.words[base + 2])
                    value = pickle.loads(bytes(self.seg.reply(w, length))) if length else None
                    if status != 0:
                        raise TPWorkerError(self.worker_ranks[w], *value)
                    results[w] = value
                    done[w] = True
            if all(done):
                break
            spins += 1
            if spins > 2000:
                time.sleep(0.0002)
            now = time.monotonic()
            if self.exit_codes is not None and now >= next_liveness:
                next_liveness = now + self.liveness_period_s
                codes = self.exit_codes()
                # a worker that acknowledged and then ended (the answer to EXIT) is read on the next pass, not reported
                gone = [w for w in range(n) if not done[w] and codes[w] is not None and int(self.seg.words[8 + 8 * w]) != request_id]
                if gone:
                    raise TPWorkerExited(method, request_id, {self.worker_ranks[w]: codes[w] for w in gone})
            if now > deadline:
                pending = [self.worker_ranks[w] for w in range(n) if not done[w]]
                raise TPTimeout(method, request_id, pending, deadline_s)
        return results

    def shutdown(self) -> None:
        if self.seg.words is not None:
            self.seg.words[2] = 1


class ControlWorker:
    """Worker side: poll for the next command, execute it on the runner, acknowledge."""

    def __init__(self, segment: ControlSegment, worker_index: int, rank: int) -> None:
        self.seg = segment
        self.w = worker_index
        self.rank = rank
        self.last = 0

    def wait_command(self, poll_sleep_after: int = 20000) -> tuple[int, str, tuple] | None:
        spins = 0
        while True:
            seq = int(self.seg.words[0])
            if seq > self.last:
                n = int(self.seg.words[1])
                if int(self.seg.words[PAYLOAD_KIND_WORD]) == PAYLOAD_DECODE:
                    from ..engine.input_preparation import StepInputs

                    return seq, TPMethod.EXECUTE.value, (StepInputs.unpack_decode(self.seg.payload(n)),)
                method, args = read_payload(self.seg, n)
                return seq, method, args
            if int(self.seg.words[2]):
                return None
            spins += 1
            if spins > poll_sleep_after:
                time.sleep(0.0005)

    def acknowledge(self, seq: int, value: Any = None, error: BaseException | None = None) -> None:
        base = 8 + 8 * self.w
        if error is not None:
            payload = (type(error).__name__, str(error), "".join(traceback.format_exception(error)))
            status = 1
        else:
            payload, status = value, 0
        blob = pickle.dumps(payload, protocol=pickle.HIGHEST_PROTOCOL) if payload is not None else b""
        if len(blob) > self.seg.reply_cap:
            blob = pickle.dumps(("ReplyTooLarge", f"{len(blob)} bytes", ""), protocol=pickle.HIGHEST_PROTOCOL)
            status = 1
        if blob:
            self.seg.reply(self.w, len(blob))[:] = blob
        self.seg.words[base + 1] = status
        self.seg.words[base + 2] = len(blob)
        self.last = seq
        self.seg.words[base] = seq  # publish last

    def serve(self, runner: Any, *, drop_ack: Any = None) -> None:
        """Run commands until ``exit`` or shutdown.  A worker that hits an exception forwards
        it and then stops, like the reference's worker loop (``model_runner.py:424-445``)."""
        while True:
            cmd = self.wait_command()
            if cmd is None:
                return
            seq, method, args = cmd
            try:
                if method == TPMethod.EXIT.value:
                    self.acknowledge(seq)
                    return
                TPMethod(method)  # whitelist check
                value = getattr(runner, method)(*args)
                if method == TPMethod.EXECUTE.value:
                    value = None  # every rank samples the same tokens; the driver keeps its own copy
            except BaseException as exc:  # noqa: BLE001 - forwarded to the driver
                self.acknowledge(seq, error=exc)
                return
            if drop_ack is not None and drop_ack(seq, method):
                self.last = seq
                continue
            self.acknowledge(seq, value)
