"""ParallelWorker: runs a stage as `world_size` SPMD processes, one per GPU.

The parent spawns the ranks (spawn context), gives each its own request queue
and shares one response queue. A call ``worker.method(*args)`` is broadcast to
every rank; rank 0 returns the result. Each rank, when ``world_size > 1``,
initialises ``torch.distributed`` over ``env://`` on 127.0.0.1 (NCCL on CUDA,
gloo on CPU), re-binds the stage to its device and calls
``stage.parallel_models()`` before serving requests.

Failure handling: a rank that raises reports a picklable error and leaves its
loop (its peers may be blocked in a collective, so the whole group is treated
as failed); the parent bounds every wait by ``ParallelConfig.timeout`` and on
expiry, queue failure or a reported error marks the worker failed and kills all
ranks. Later calls raise ``WorkerFailedError``. ``restart()`` re-spawns the
group from the pristine stage (an addition over the reference, which has no
recovery). Role parity: telefuser/worker/parallel_worker.py:32-383.
"""

from __future__ import annotations

import os
import queue as pyqueue
import time
import traceback
from typing import Any, Callable

import torch
import torch.multiprocessing as mp

from telefuser_b200.utils.system import PortAllocator

_EXIT = "__exit__"


class WorkerFailedError(RuntimeError):
    pass


class RemoteError:
    """Picklable carrier of an exception raised inside a rank."""

    def __init__(self, rank: int, exc: BaseException):
        self.rank = rank
        self.type_name = type(exc).__name__
        self.message = str(exc)
        self.traceback = traceback.format_exc()

    def __str__(self) -> str:
        return f"rank {self.rank}: {self.type_name}: {self.message}\n{self.traceback}"


def to_device(obj: Any, device) -> Any:
    """Moves every tensor in a nested list/tuple/dict structure to `device`."""
    if isinstance(obj, torch.Tensor):
        return obj.to(device)
    if isinstance(obj, (list, tuple)):
        return type(obj)(to_device(o, device) for o in obj)
    if isinstance(obj, dict):
        return {k: to_device(v, device) for k, v in obj.items()}
    return obj


def _rank_device(device_type: str, device_ids, rank: int):
    if device_type == "cpu":
        return torch.device("cpu")
    return torch.device(device_type, device_ids[rank])


def _worker_loop(rank: int, stage, world_size: int, port: int, device_type: str, device_ids, timeout_s: int,
                 intra_op_threads: int, queues_in, queue_out, empty_cache_each_call: bool,
                 results_on_device: bool = False) -> None:  # fmt: skip
    import torch.distributed as dist

    initialised = False
    held = None  # the last device-resident result stays referenced here until the next call replaces it
    device = _rank_device(device_type, device_ids, rank)
    try:
        if world_size > 1:
            torch.set_num_threads(max(1, intra_op_threads))
            os.environ.update(RANK=str(rank), WORLD_SIZE=str(world_size), MASTER_ADDR="127.0.0.1",
                              MASTER_PORT=str(port), LOCAL_RANK=str(rank))  # fmt: skip
            os.environ.setdefault("TORCH_NCCL_AVOID_RECORD_STREAMS", "1")
            backend = "gloo" if device.type == "cpu" else "nccl"
            if device.type == "cuda":
                torch.cuda.set_device(device)
            import datetime

            kw = {"device_id": device} if device.type == "cuda" else {}
            dist.init_process_group(backend=backend, init_method="env://", world_size=world_size, rank=rank,
                                    timeout=datetime.timedelta(seconds=timeout_s), **kw)  # fmt: skip
            initialised = True
        elif device.type == "cuda":
            torch.cuda.set_device(device)
        from telefuser_b200.utils import profiler

        profiler.mark_as_worker_process()
        stage.device = device
        if getattr(stage, "onload_models_flag", False) and device.type == "cuda" and hasattr(stage, "onload_models"):
            # The parent marked the models as resident, but they arrive where the parent held them (every rank
            # unpickles the same device index): bring them to this rank's own GPU before anything runs.
            stage.onload_models()
        if hasattr(stage, "configure_device_waits"):
            stage.configure_device_waits()
        if world_size > 1:
            stage.parallel_models()
        queue_out.put(("ready", rank, None))
        while True:
            name, args, kwargs = queues_in[rank].get()
            if name == _EXIT:
                break
            args, kwargs = to_device(args, device), to_device(kwargs, device)
            with torch.no_grad():
                result = getattr(stage, name)(*args, **kwargs)
            if hasattr(stage, "check_device_waits"):
                stage.check_device_waits(final=True)  # an expired wait on a peer fails the call on this rank
            if empty_cache_each_call and device.type == "cuda":
                torch.cuda.empty_cache()
            # every rank acknowledges every call, so a failure on any rank is seen by the parent
            if rank != 0:
                queue_out.put(("ok", rank, None))
            elif results_on_device and device.type == "cuda":
                # The result crosses to the parent as a CUDA IPC handle (no host copy): the consumer has no stream
                # order with this process, so the producing work is finished first, and the memory stays referenced
                # here until the next call.
                held = to_device(result, device)
                torch.cuda.synchronize(device)
                queue_out.put(("ok", rank, held))
            else:
                queue_out.put(("ok", rank, to_device(result, "cpu")))
    except BaseException as e:  # noqa: BLE001 - reported to the parent, then the rank exits
        try:
            queue_out.put(("error", rank, RemoteError(rank, e)))
        except Exception:  # noqa: BLE001
            pass
    finally:
        try:
            if device.type == "cuda":
                torch.cuda.synchronize()
                torch.cuda.empty_cache()
                torch.cuda.ipc_collect()
            if initialised:
                dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


class ParallelWorker:
    def __init__(self, stage, start: bool = True, empty_cache_each_call: bool = False) -> None:
        self.stage = stage
        self.parallel_config = stage.model_runtime_config.parallel_config
        self.parallel_config.validate()
        self.device_ids = self.parallel_config.device_ids or [stage.model_runtime_config.device_id]
        self.world_size = len(self.device_ids)
        self.device_type = getattr(stage, "device_type", "cuda" if torch.cuda.is_available() else "cpu")
        self.timeout = self.parallel_config.timeout
        self.empty_cache_each_call = empty_cache_each_call
        self.failed = False
        self.closed = False
        self.failure_reason: str | None = None
        self.processes = []
        self.queues_in = []
        self.queue_out = None
        self.port = None
        if start:
            self._spawn()

    # ---- lifecycle -------------------------------------------------------------
    def _spawn(self) -> None:
        ctx = mp.get_context("spawn")
        self.port = PortAllocator.allocate()
        self.queues_in = [ctx.Queue() for _ in range(self.world_size)]
        self.queue_out = ctx.Queue()
        self.processes = []
        for rank in range(self.world_size):
            p = ctx.Process(
                target=_worker_loop,
                args=(rank, self.stage, self.world_size, self.port, self.device_type, self.device_ids, self.timeout,
                      self.parallel_config.worker_intra_op_threads, self.queues_in, self.queue_out,
                      self.empty_cache_each_call, bool(getattr(self.parallel_config, "results_on_device", False))),  # fmt: skip
                daemon=True,
            )
            p.start()
            self.processes.append(p)
        # start-up (process spawn, imports, rendezvous) gets its own, longer allowance
        ready, deadline = 0, time.monotonic() + max(self.timeout, 180)
        while ready < self.world_size:
            kind, rank, payload = self._get(deadline)
            if kind == "ready":
                ready += 1
            elif kind == "error":
                self._mark_failed(f"worker start-up failed: {payload}")
                raise WorkerFailedError(self.failure_reason)

    def restart(self) -> None:
        """Kills whatever is left of the group and spawns a fresh one from the same stage object."""
        self._terminate()
        self.failed, self.closed, self.failure_reason = False, False, None
        self._spawn()

    def _terminate(self) -> None:
        for p in self.processes:
            if p.is_alive():
                p.kill()
        for p in self.processes:
            p.join(timeout=5)
        for q in [*self.queues_in, self.queue_out]:
            if q is not None:
                try:
                    q.close()
                    q.cancel_join_thread()
                except Exception:  # noqa: BLE001
                    pass
        if self.port is not None:
            PortAllocator.release(self.port)
        self.processes, self.queues_in, self.queue_out, self.port = [], [], None, None

    def _mark_failed(self, reason: str) -> None:
        if not self.failed:
            self.failed = True
            self.failure_reason = reason
        self._terminate()

    def _ensure_usable(self) -> None:
        if self.closed:
            raise WorkerFailedError("ParallelWorker is closed")
        if self.failed:
            raise WorkerFailedError(f"ParallelWorker failed earlier: {self.failure_reason}")

    def close(self) -> None:
        if self.closed:
            return
        self.closed = True
        if not self.failed:
            for q in self.queues_in:
                try:
                    q.put((_EXIT, None, None))
                except Exception:  # noqa: BLE001
                    pass
            for p in self.processes:
                p.join(timeout=10)
        self._terminate()

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass

    # ---- calls ----------------------------------------------------------------------
    def _get(self, deadline: float):
        while True:
            remaining = deadline - time.monotonic()
            if remaining <= 0:
                self._mark_failed(f"no answer from the worker group within {self.timeout} s")
                raise WorkerFailedError(self.failure_reason)
            try:
                return self.queue_out.get(timeout=min(remaining, 1.0))
            except pyqueue.Empty:
                dead = [i for i, p in enumerate(self.processes) if not p.is_alive()]
                if dead:
                    # drain one last time: the rank may have reported before exiting
                    try:
                        return self.queue_out.get(timeout=0.2)
                    except pyqueue.Empty:
                        self._mark_failed(f"rank(s) {dead} exited unexpectedly")
                        raise WorkerFailedError(self.failure_reason) from None
            except (OSError, EOFError, ValueError) as e:
                self._mark_failed(f"result queue failed: {e}")
                raise WorkerFailedError(self.failure_reason) from e

    def put_data(self, name: str, args, kwargs) -> None:
        share_cpu = self.parallel_config.queue_with_cpu
        for rank in range(self.world_size):
            if share_cpu or self.device_type == "cpu":
                payload = (name, to_device(args, "cpu"), to_device(kwargs, "cpu"))
            else:
                dev = _rank_device(self.device_type, self.device_ids, rank)
                payload = (name, to_device(args, dev), to_device(kwargs, dev))
            self.queues_in[rank].put(payload)

    def _wait_result(self):
        deadline = time.monotonic() + self.timeout
        result, acks = None, 0
        while acks < self.world_size:
            kind, rank, payload = self._get(deadline)
            if kind == "error":
                self._mark_failed(str(payload))
                raise WorkerFailedError(self.failure_reason)
            acks += 1
            if rank == 0:
                result = payload
        return result

    def call(self, name: str, *args, async_call: bool = False, **kwargs):
        self._ensure_usable()
        self.put_data(name, args, kwargs)
        if async_call:
            return self._wait_result
        return self._wait_result()

    def __call__(self, *args, **kwargs):
        return self.call("process", *args, **kwargs)

    def __getattr__(self, name: str) -> Callable:
        if name.startswith("_") or name in ("stage",):
            raise AttributeError(name)

        def method(*args, **kwargs):
            return self.call(name, *args, **kwargs)

        method._parallel_worker = self  # lets auto_async_call issue the call asynchronously
        method._method_name = name
        return method
