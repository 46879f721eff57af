"""`auto_async_call`: one calling convention for in-process stages and `ParallelWorker`s.

Returns a `wait()` closure either way, so a pipeline can start several stages and collect
the results later (reference: telefuser/utils/func.py:17).
"""

from __future__ import annotations

from typing import Any, Callable


def auto_async_call(method: Callable, *args, **kwargs) -> Callable[[], Any]:
    owner = getattr(method, "__self__", None)
    from telefuser_b200.worker.parallel_worker import ParallelWorker

    if isinstance(owner, ParallelWorker):  # bound `worker.call`-style partials are not used; go by name
        return owner.call(method.__name__, *args, async_call=True, **kwargs)
    worker = getattr(method, "_parallel_worker", None)
    if worker is not None:
        return worker.call(method._method_name, *args, async_call=True, **kwargs)
    result = method(*args, **kwargs)
    if callable(result) and getattr(result, "__name__", "") == "_wait_result":
        return result
    return lambda: result
