"""Tensor-parallel control plane under failure, with every fault made on the host: a
worker that raises, a worker that never acknowledges, a worker that dies, a wrong method
name.  Workers are real processes talking through the shared-memory segment."""

import multiprocessing as mp
import os
import time

import pytest

from prism_infer_b200.parallel.control import (ControlDriver, ControlSegment, ControlWorker, TPControlError, TPMethod,
                                               TPTimeout, TPWorkerError)


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
        assert driver.collect("execute", rid) == [(1, "hello", 1), (2, "hello", 1)]
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
