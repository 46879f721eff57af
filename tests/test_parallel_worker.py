"""ParallelWorker on CPU ranks (gloo): calls, async calls, failure detection, restart."""
import time

import pytest
import torch

from telefuser_b200.testing.stages import AllReduceStage, cpu_runtime_config
from telefuser_b200.worker.parallel_worker import ParallelWorker, WorkerFailedError


def test_two_ranks_allreduce_and_async():
    w = ParallelWorker(AllReduceStage(cpu_runtime_config(2, sp_ulysses_degree=2)))
    try:
        out = w.process(torch.ones(4))
        assert torch.equal(out, torch.full((4,), 3.0))
        wait = w.call("process", torch.ones(2) * 2, async_call=True)
        assert torch.equal(wait(), torch.full((2,), 6.0))
        info = w.info()
        assert info["rank"] == 0 and info["parallel_called"] is True
    finally:
        w.close()
    w.close()  # idempotent
    with pytest.raises(WorkerFailedError):
        w.process(torch.ones(1))


def test_single_rank_runs_without_process_group():
    w = ParallelWorker(AllReduceStage(cpu_runtime_config(1)))
    try:
        assert torch.equal(w.process(torch.ones(3)), torch.ones(3))
        assert w.info()["parallel_called"] is False
    finally:
        w.close()


def test_rank_exception_marks_worker_failed_and_restart_recovers():
    w = ParallelWorker(AllReduceStage(cpu_runtime_config(2, sp_ulysses_degree=2)))
    try:
        with pytest.raises(WorkerFailedError, match="injected failure on rank 1"):
            w.fail_on_rank(1)
        assert w.failed and "ValueError" in w.failure_reason
        with pytest.raises(WorkerFailedError):
            w.process(torch.ones(1))
        w.restart()
        assert not w.failed
        assert torch.equal(w.process(torch.ones(2)), torch.full((2,), 3.0))
    finally:
        w.close()


def test_timeout_and_dead_rank_are_detected():
    w = ParallelWorker(AllReduceStage(cpu_runtime_config(2, timeout=3, sp_ulysses_degree=2)))
    try:
        t0 = time.monotonic()
        with pytest.raises(WorkerFailedError, match="within 3 s|exited"):
            w.sleep(30.0)
        assert time.monotonic() - t0 < 15
        assert w.failed and all(not p.is_alive() for p in w.processes)
    finally:
        w.close()
    w2 = ParallelWorker(AllReduceStage(cpu_runtime_config(2, timeout=20, sp_ulysses_degree=2)))
    try:
        with pytest.raises(WorkerFailedError):
            w2.exit_on_rank(0)
        assert w2.failed
    finally:
        w2.close()
