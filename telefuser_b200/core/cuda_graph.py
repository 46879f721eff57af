"""CUDA-graph replay of a model forward (what `CompileConfig.enabled` switches on: there is no tracing compiler
on the hot path, the launch-bound part of a step is captured once and replayed).

`GraphRunner(fn)` keeps one captured graph per call signature (tensor shapes / dtypes / devices and the values of
all non-tensor arguments). The first call with a signature runs `fn` eagerly `warmup` times on a side stream (lazy
initialisation such as fused-weight views, tensor-map caches and kernel attributes happens there), then captures
one run into a `torch.cuda.CUDAGraph` with static input buffers. Later calls copy the arguments into the static
buffers, replay, and return clones of the outputs (the static outputs are overwritten by the next replay, and a
guidance step holds the conditional output while the unconditional one is computed).

What must hold for a captured function: no host synchronisation, no data-dependent control flow on device values,
the same kernels and buffer sizes for a given signature. The native kernels launch on the current stream and take
their pointers from torch tensors, so they are captured like any torch op; tensors allocated during capture come
from the graph's private pool and stay valid across replays.
"""

from __future__ import annotations

from typing import Any, Callable

import torch


def _signature(x: Any):
    if isinstance(x, torch.Tensor):
        return ("T", tuple(x.shape), x.dtype, x.device.type, x.device.index)
    if isinstance(x, (list, tuple)):
        return (type(x).__name__, tuple(_signature(v) for v in x))
    if isinstance(x, dict):
        return ("dict", tuple((k, _signature(v)) for k, v in sorted(x.items())))
    if isinstance(x, (int, float, bool, str)) or x is None:
        return x
    return ("obj", id(x))


def _map_tensors(x: Any, fn: Callable):
    if isinstance(x, torch.Tensor):
        return fn(x)
    if isinstance(x, (list, tuple)):
        return type(x)(_map_tensors(v, fn) for v in x)
    if isinstance(x, dict):
        return {k: _map_tensors(v, fn) for k, v in x.items()}
    return x


def _flatten(x: Any, out: list) -> list:
    if isinstance(x, torch.Tensor):
        out.append(x)
    elif isinstance(x, (list, tuple)):
        for v in x:
            _flatten(v, out)
    elif isinstance(x, dict):
        for v in x.values():
            _flatten(v, out)
    return out


class _Captured:
    def __init__(self, graph, static_args, static_kwargs, static_out) -> None:
        self.graph, self.static_args, self.static_kwargs, self.static_out = graph, static_args, static_kwargs, static_out
        self.static_inputs = _flatten((static_args, static_kwargs), [])
        self.replays = 0


class GraphRunner:
    def __init__(self, fn: Callable, warmup: int = 2, max_graphs: int = 8) -> None:
        self.fn, self.warmup, self.max_graphs = fn, warmup, max_graphs
        self.graphs: dict = {}
        self.eager_calls = 0

    def __call__(self, *args, **kwargs):
        tensors = _flatten((args, kwargs), [])
        if not tensors or not all(t.is_cuda for t in tensors) or torch.cuda.is_current_stream_capturing():
            self.eager_calls += 1
            return self.fn(*args, **kwargs)
        key = _signature((args, kwargs))
        cap = self.graphs.get(key)
        if cap is None:
            if len(self.graphs) >= self.max_graphs:  # too many shapes (a growing window, say): stop capturing
                self.eager_calls += 1
                return self.fn(*args, **kwargs)
            cap = self.graphs[key] = self._capture(args, kwargs)
        for dst, src in zip(cap.static_inputs, tensors):
            if dst.data_ptr() != src.data_ptr():
                dst.copy_(src)
        cap.graph.replay()
        cap.replays += 1
        return _map_tensors(cap.static_out, lambda t: t.clone())

    def _capture(self, args, kwargs) -> _Captured:
        static_args = _map_tensors(args, lambda t: t.clone())
        static_kwargs = _map_tensors(kwargs, lambda t: t.clone())
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(self.warmup):
                self.fn(*static_args, **static_kwargs)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = self.fn(*static_args, **static_kwargs)
        return _Captured(graph, static_args, static_kwargs, out)

    def reset(self) -> None:
        self.graphs.clear()

    def stats(self) -> dict:
        return {"graphs": len(self.graphs), "replays": sum(c.replays for c in self.graphs.values()),
                "eager_calls": self.eager_calls}  # fmt: skip
