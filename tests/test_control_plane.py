"""Tensor-parallel control plane under failure, with every fault made on the host: a
worker that raises, a worker that never acknowledges, a worker that dies, a wrong method
name.  Workers are real processes talking through the shared-memory segment."""

import multiprocessing as mp
import os
import time

import pytest

from prism_infer_b200.parallel.control import (ControlDriver, ControlSegment, ControlWorker, TPControlError, TPMethod,
                                               TPTimeout, TPWorkerError, TPWorkerExited)


class EchoRunner:
    def __init__(self, rank):
        self.rank = rank
        self.calls = 0

    def execute(self, x):
        self.calls += 1
        if x == "raise":
            raise ValueError(f"bad input on rank {self.rank}")
        return (self.rank, x, self.calls)

    def capacity(self):
        return (10 + self.rank, 0)

    def barrier(self):
        return None


def _worker(name, n_workers, index, mode):
    seg = ControlSegment(name, n_workers, create=False)
    worker = ControlWorker(seg, index, index + 1)
    runner = EchoRunner(index + 1)
    if mode == "drop_second_ack":
        worker.serve(runner, drop_ack=lambda seq, method: seq == 2)
    elif mode == "die_on_second":
        cmd = worker.wait_command()
        worker.acknowledge(cmd[0], getattr(runner, cmd[1])(*cmd[2]))
        worker.wait_command()
        os._exit(17)
    else:
        worker.serve(runner)
    seg.close()


def _start(n_workers, modes):
    seg = ControlSegment(None, n_workers, create=True, payload_cap=1 << 20, reply_cap=1 << 16)
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(seg.name, n_workers, i, modes[i]), daemon=True) for i in range(n_workers)]
    for p in procs:
        p.start()
    return seg, procs


def _stop(seg, procs, driver):
    driver.shutdown()
    for p in procs:
        p.join(timeout=10)
        if p.is_alive():
            p.kill()
    seg.close()


@pytest.mark.timeout(120)
def test_rpc_round_trip_and_worker_exception_is_forwarded():
    seg, procs = _start(2, ["ok", "ok"])
    driver = ControlDriver(seg, timeout_s=30.0)
    try:
        rid = driver.post(TPMethod.EXECUTE, ("hello",))
        assert driver.collect("execute", rid) == [None, None]   # step results are not sent back: the driver holds its own
        rid = driver.post("capacity", ())
        assert driver.collect("capacity", rid) == [(11, 0), (12, 0)]
        with pytest.raises(ValueError):
            driver.post("not_a_method", ())
        rid = driver.post("execute", ("raise",))
        with pytest.raises(TPWorkerError) as err:
            driver.collect("execute", rid)
        assert err.value.exc_type == "ValueError" and "bad input" in str(err.value) and "Traceback" in err.value.worker_traceback
    finally:
        _stop(seg, procs, driver)


@pytest.mark.timeout(120)
def test_dropped_ack_times_out_and_names_the_pending_rank():
    seg, procs = _start(2, ["ok", "drop_second_ack"])
    driver = ControlDriver(seg, timeout_s=30.0)
    try:
        rid = driver.post("execute", (1,))
        driver.collect("execute", rid)
        rid = driver.post("execute", (2,))
        t0 = time.monotonic()
        with pytest.raises(TPTimeout) as err:
            driver.collect("execute", rid, timeout_s=0.3)
        assert err.value.pending == [2] and time.monotonic() - t0 < 5.0
        assert "pending ranks: [2]" in str(err.value)
    finally:
        _stop(seg, procs, driver)


@pytest.mark.timeout(120)
def test_dead_worker_is_detected_by_the_deadline():
    seg, procs = _start(1, ["die_on_second"])
    driver = ControlDriver(seg, timeout_s=30.0)
    try:
        rid = driver.post("execute", ("a",))
        assert driver.collect("execute", rid) == [(1, "a", 1)]
        rid = driver.post("execute", ("b",))
        with pytest.raises(TPTimeout):
            driver.collect("execute", rid, timeout_s=0.5)
        procs[0].join(timeout=10)
        assert procs[0].exitcode == 17
    finally:
        _stop(seg, procs, driver)


@pytest.mark.timeout(120)
def test_dead_worker_is_reported_at_once_through_its_process_handle():
    """With the workers' exit codes at hand the driver does not wait for the deadline: the rank that ended is named with
    its exit code while the healthy rank's answer is still accepted, and a worker that acknowledges EXIT and then ends
    is not mistaken for a dead one."""
    seg, procs = _start(2, ["echo", "die_on_second"])
    driver = ControlDriver(seg, timeout_s=60.0, exit_codes=lambda: [p.exitcode for p in procs], liveness_period_s=0.02)
    try:
        rid = driver.post("execute", ("a",))
        assert driver.collect("execute", rid) == [None, (2, "a", 1)]  # a serving worker keeps execute's value to itself
        rid = driver.post("execute", ("b",))
        t0 = time.monotonic()
        with pytest.raises(TPWorkerExited) as info:
            driver.collect("execute", rid)
        assert time.monotonic() - t0 < 20.0 and info.value.exited == {2: 17} and isinstance(info.value, TPControlError)
    finally:
        _stop(seg, procs, driver)
    seg, procs = _start(1, ["echo"])
    driver = ControlDriver(seg, timeout_s=60.0, exit_codes=lambda: [p.exitcode for p in procs], liveness_period_s=0.0)
    try:
        rid = driver.post(TPMethod.EXIT, ())
        assert driver.collect("exit", rid) == [None]
    finally:
        _stop(seg, procs, driver)


def test_oversized_payload_is_refused():
    seg = ControlSegment(None, 1, create=True, payload_cap=1024, reply_cap=1024)
    driver = ControlDriver(seg)
    try:
        with pytest.raises(TPControlError):
            driver.post("execute", (b"x" * 4096,))
    finally:
        seg.close()


def test_large_arrays_travel_out_of_band_and_small_ones_in_band():
    import numpy as np
    import torch

    from prism_infer_b200.engine.input_preparation import StepInputs, VisionJob
    from prism_infer_b200.parallel import control

    seg = control.ControlSegment(None, 1, create=True, payload_cap=8 << 20, reply_cap=1 << 16)
    try:
        big = torch.randn(300, 1536).to(torch.bfloat16)           # 900 KiB -> out of band
        inp = StepInputs(kind="prefill", input_ids=torch.arange(7), positions=torch.zeros(3, 7, dtype=torch.int32),
                         slots=torch.arange(7), block_tables=torch.zeros(1, 4, dtype=torch.int32), temperatures=torch.zeros(1),
                         vision_jobs=[VisionJob(5, big, [(1, 10, 30)], "k")])
        n = control.write_payload(seg, ("execute", (inp,)))
        assert n > big.numel() * 2
        header = np.ndarray((3,), dtype=np.int64, buffer=seg.payload(n))
        assert header[0] == 1 and header[2] == big.numel() * 2   # exactly one out-of-band buffer: the patches
        method, (got,) = control.read_payload(seg, n)
        assert method == "execute" and torch.equal(got.input_ids, inp.input_ids) and got.kv_lens is None
        job = got.vision_jobs[0]
        assert job.pixel_values.dtype == torch.bfloat16 and torch.equal(job.pixel_values, big) and job.grid_thw == [(1, 10, 30)]
        del got, job, header
        with pytest.raises(control.TPControlError):
            control.write_payload(seg, torch.zeros(16 << 20, dtype=torch.uint8).numpy())
    finally:
        seg.close()


def test_decode_step_travels_in_the_fixed_binary_form():
    """A decode ``StepInputs`` is sent without pickle; every field arrives bit-identical, the
    worker's copy does not alias the command area, and anything else still goes through pickle."""
    import numpy as np
    import torch

    from prism_infer_b200.engine.input_preparation import StepInputs
    from prism_infer_b200.parallel import control
    from prism_infer_b200.parallel.control import ControlDriver, ControlSegment, ControlWorker, TPMethod

    seg = ControlSegment(None, 1, create=True, payload_cap=1 << 16)
    try:
        driver, worker = ControlDriver(seg), ControlWorker(seg, 0, 1)
        g = torch.Generator().manual_seed(0)
        B, W = 5, 7
        inp = StepInputs(kind="decode", input_ids=torch.randint(0, 150000, (B,), generator=g), positions=torch.randint(0, 4000, (3, B), generator=g, dtype=torch.int32),
                         slots=torch.randint(0, 1 << 40, (B,), generator=g), block_tables=torch.randint(-1, 900, (B, W), generator=g, dtype=torch.int32),
                         temperatures=torch.tensor([0.0, 0.7, 1.0, 0.0, 1.3]), context_lens=torch.randint(1, 4000, (B,), generator=g, dtype=torch.int32))
        driver.post(TPMethod.EXECUTE, (inp,))
        assert int(seg.words[control.PAYLOAD_KIND_WORD]) == control.PAYLOAD_DECODE
        seq, method, (got,) = worker.wait_command()
        assert method == "execute" and got.kind == "decode" and got.num_seqs == B
        for name in ("input_ids", "positions", "slots", "block_tables", "temperatures", "context_lens"):
            a, b = getattr(inp, name), getattr(got, name)
            assert a.dtype == b.dtype and a.shape == b.shape and torch.equal(a, b), name
        worker.acknowledge(seq, [1, 2, 3])
        assert driver.collect("execute", seq) == [[1, 2, 3]]
        seg.payload(64)[:] = bytes(64)                      # the next command overwrites the area
        assert torch.equal(got.input_ids, inp.input_ids)
        # a prefill step and a non-StepInputs argument use the pickle form
        pre = StepInputs(kind="prefill", input_ids=torch.arange(4), positions=torch.zeros(3, 4, dtype=torch.int32), slots=torch.arange(4),
                         block_tables=torch.zeros(1, 2, dtype=torch.int32), temperatures=torch.zeros(1), cu_seqlens_q=torch.tensor([0, 4], dtype=torch.int32),
                         kv_lens=torch.tensor([4], dtype=torch.int32), max_q_len=4)
        driver.post(TPMethod.EXECUTE, (pre,))
        assert int(seg.words[control.PAYLOAD_KIND_WORD]) == control.PAYLOAD_PICKLE
        seq, method, (got,) = worker.wait_command()
        assert got.kind == "prefill" and torch.equal(got.cu_seqlens_q, pre.cu_seqlens_q)
        worker.acknowledge(seq)
        driver.collect("execute", seq)
        # unexpected dtype: falls back rather than reinterpreting bytes
        odd = StepInputs(kind="decode", input_ids=inp.input_ids.to(torch.int32), positions=inp.positions, slots=inp.slots, block_tables=inp.block_tables,
                         temperatures=inp.temperatures, context_lens=inp.context_lens)
        assert odd.pack_decode(seg.payload(1 << 16)) == 0 and inp.pack_decode(seg.payload(32)) == 0
    finally:
        seg.close()
