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


@pytest.mark.gpu
def test_results_stay_on_the_device_when_asked():
    """One rank on cuda:0 with `results_on_device`: the parent receives CUDA tensors (an IPC handle, no host copy) and
    the values survive the next call of the worker."""
    from telefuser_b200.core.config import ModelRuntimeConfig, ParallelConfig

    cfg = ModelRuntimeConfig(device_type="cuda", device_id=0, torch_dtype=torch.float32,
                             parallel_config=ParallelConfig(timeout=120, results_on_device=True))  # fmt: skip
    stage = AllReduceStage(cfg)
    stage.device_type = "cuda"
    w = ParallelWorker(stage)
    try:
        a = w.process(torch.arange(8.0))
        assert a.is_cuda and torch.equal(a.cpu(), torch.arange(8.0))
        b = w.process(torch.ones(8, device="cuda"))  # a CUDA argument crosses the same way
        assert b.is_cuda and torch.equal(b.cpu(), torch.ones(8))
        kept = a.clone()
        del a
        c = w.process(torch.full((8,), 5.0))
        assert torch.equal(kept.cpu(), torch.arange(8.0)) and torch.equal(c.cpu(), torch.full((8,), 5.0))
    finally:
        w.close()
