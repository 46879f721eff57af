"""Base class of every model: parallel / offload / quantisation / capture hooks.

Mirrors the hook surface of the reference's ``telefuser/core/base_model.py:18-262``
(`enable_usp`, `enable_pp`, `enable_quant`, `enable_async_offload`,
`set_attention_config`, `compile`, FSDP / TP plan getters, state-dict converter)
so stages can drive any model the same way.
"""

from __future__ import annotations

from typing import Any

import torch
import torch.nn as nn

from .config import AttentionConfig, CompileConfig, OffloadConfig, QuantConfig


class BaseModel(nn.Module):
    def __init__(self) -> None:
        super().__init__()
        self.usp_flag = False
        self.pp_flag = False
        self.fsdp_flag = False
        self.async_offload_flag = False
        self.graph_capture = False
        self.device_mesh = None
        self.attention_config = AttentionConfig.dense_attention()
        self.quant_config: QuantConfig | None = None
        self._feature_cache = None
        self.layer_name_list: list[str] = ["blocks"]

    # ---- feature cache ---------------------------------------------------
    @property
    def feature_cache(self):
        if self._feature_cache is None:
            from telefuser_b200.feature_cache.base import NoOpCache

            self._feature_cache = NoOpCache()
        return self._feature_cache

    def set_feature_cache(self, cache) -> None:
        self._feature_cache = cache

    def set_ada_taylor_cache(self, cache) -> None:
        self._feature_cache = cache

    # ---- devices -----------------------------------------------------------
    def onload_device(self, device) -> None:
        self.to(device)

    def offload_device(self, pin: bool = True) -> None:
        self.to("cpu")
        if pin and torch.cuda.is_available():
            for p in self.parameters():
                if not p.data.is_pinned():
                    p.data = p.data.pin_memory()

    # ---- parallel hooks ------------------------------------------------------
    def enable_usp(self) -> None:
        self.usp_flag = True

    def enable_pp(self, *args, **kwargs) -> None:
        raise NotImplementedError(f"{type(self).__name__} has no pipeline-parallel path")

    def get_fsdp_module_names(self) -> list[str]:
        return list(self.layer_name_list)

    def get_tp_plan(self) -> dict[str, Any]:
        return {}

    # ---- runtime features ------------------------------------------------------
    def set_attention_config(self, config: AttentionConfig) -> None:
        self.attention_config = config
        for m in self.modules():
            if m is not self and hasattr(m, "attention_config"):
                m.attention_config = config

    def enable_quant(self, quant: QuantConfig | torch.dtype | str | None = None) -> int:
        """Quantises the linears of the model's block lists (`get_fsdp_module_names()`) in the requested format (FP8 by
        default; "int8", "mxfp8", "nvfp4", "nf4" or the matching `QuantType`); embeddings, heads, norms and modulation
        tables outside the blocks stay as they are. Models override this to name what must be skipped inside a block.
        Returns the number of layers converted."""
        from telefuser_b200.ops.quant import quantize_model_

        try:
            lists = list(self.get_fsdp_module_names())
        except NotImplementedError:
            lists = []
        if not lists:
            raise NotImplementedError(f"{type(self).__name__} names no block list to quantise")
        return quantize_model_(self, quant, tuple(f"{name}.*" for name in lists), ("modulation", "adaLN", "router", "gate."))

    def enable_async_offload(self, device: torch.device, offload_config: OffloadConfig) -> None:
        from telefuser_b200.offload.async_offload import AsyncOffloadManager

        blocks = getattr(self, self.layer_name_list[0])
        self.async_offload_manager = AsyncOffloadManager(
            blocks,
            enabled=True,
            offload_ratio=offload_config.offload_ratio,
            prefetch_size=offload_config.prefetch_size,
            device=device,
            pin_cpu_memory=offload_config.pin_cpu_memory,
        )
        self.async_offload_flag = True

    def enable_sequential_cpu_offload(self, device, **kwargs) -> None:
        from telefuser_b200.offload.sequential_offload import enable_sequential_cpu_offload

        enable_sequential_cpu_offload(self, device, **kwargs)

    def compile(self, config: CompileConfig | None = None, **kwargs):  # noqa: A003 - mirrors nn.Module.compile
        """Switches the forward to CUDA-graph replay (there is no tracing compiler here): from the next call on,
        `__call__` goes through a `GraphRunner` whenever `graph_capturable()` says the call can be captured."""
        if config is None or config.enabled:
            from .cuda_graph import GraphRunner

            self.graph_capture = True
            self._graph_runner = GraphRunner(lambda *a, **k: nn.Module.__call__(self, *a, **k),
                                             warmup=int(kwargs.get("warmup", 2)))  # fmt: skip
        else:
            self.graph_capture, self._graph_runner = False, None
        return self

    def graph_capturable(self) -> bool:
        """A forward can be replayed from a graph when nothing in it depends on the host between calls: no
        layer-wise offload (host-driven copies), no pipeline-parallel send / receive, no sequence-parallel exchange
        (peer barriers pair up with other ranks' launches) and no feature cache (it decides per step on the host)."""
        from telefuser_b200.feature_cache.base import NoOpCache

        return not (self.async_offload_flag or self.pp_flag or self.usp_flag or self.fsdp_flag
                    or not isinstance(self.feature_cache, NoOpCache))  # fmt: skip

    def __call__(self, *args, **kwargs):
        runner = getattr(self, "_graph_runner", None)
        if runner is not None and self.graph_capture and self.graph_capturable():
            return runner(*args, **kwargs)
        return super().__call__(*args, **kwargs)

    def mark_compile_static(self, *args, **kwargs) -> None:
        return None

    @staticmethod
    def state_dict_converter():
        return None
