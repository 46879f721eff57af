"""BasePipeline: shared behaviour of every generation pipeline.

Subclasses get their `init` and `__call__` wrapped automatically (`__init_subclass__`):
`init` logs the configuration once, `__call__` resets the timing registry, times the call and
releases cached GPU memory afterwards. Also here: metrics switches, image / video tensor
conversion, size checks, seeded noise, configuration dump.
Role parity: telefuser/core/base_pipeline.py:27-423.
"""

from __future__ import annotations

import functools
import gc
import json
import time
from typing import Any

import numpy as np
import torch

from telefuser_b200.core.config_serializer import to_jsonable
from telefuser_b200.utils.logging import logger
from telefuser_b200.utils.profiler import GlobalTimingRegistry


class BasePipeline:
    def __init_subclass__(cls, **kwargs):
        super().__init_subclass__(**kwargs)
        if "init" in cls.__dict__:
            orig_init = cls.__dict__["init"]

            @functools.wraps(orig_init)
            def init(self, *a, **k):
                out = orig_init(self, *a, **k)
                cfg = getattr(self, "config", None)
                if cfg is not None:
                    logger.info(f"{cls.__name__} initialised: {json.dumps(to_jsonable(cfg), default=str)[:2000]}")
                return out

            cls.init = init
        if "__call__" in cls.__dict__:
            orig_call = cls.__dict__["__call__"]

            @functools.wraps(orig_call)
            def call(self, *a, **k):
                GlobalTimingRegistry.instance().reset()
                t0 = time.perf_counter()
                try:
                    return orig_call(self, *a, **k)
                finally:
                    self.last_call_seconds = time.perf_counter() - t0
                    logger.info(f"{cls.__name__} call finished in {self.last_call_seconds:.2f} s")
                    gc.collect()
                    if torch.cuda.is_available():
                        torch.cuda.empty_cache()

            cls.__call__ = call

    def __init__(self, device: str | torch.device = "cuda", torch_dtype: torch.dtype = torch.bfloat16) -> None:
        self.device = torch.device(device) if not isinstance(device, torch.device) else device
        self.torch_dtype = torch_dtype
        self.height_division_factor = 16
        self.width_division_factor = 16
        self.metrics_enabled = False
        self.last_call_seconds: float | None = None
        self._model_info: list[dict] = []

    # ---- metrics -------------------------------------------------------------
    def _get_stages(self) -> list:
        return []

    def close(self) -> None:
        """Ends the worker processes of every stage that runs as SPMD ranks (idempotent). Pipelines that hold other
        resources override it and call this."""
        seen = set()
        for st in list(self._get_stages()) + [v for v in vars(self).values() if hasattr(v, "processes")]:
            if id(st) in seen or not hasattr(st, "processes") or not callable(getattr(st, "close", None)):
                continue
            seen.add(id(st))
            st.close()

    def enable_metrics(self, registry: Any | None = None) -> None:
        self.metrics_enabled = True
        for st in self._get_stages():
            if hasattr(st, "enable_metrics"):
                st.enable_metrics(registry)

    def disable_metrics(self) -> None:
        self.metrics_enabled = False
        for st in self._get_stages():
            if hasattr(st, "disable_metrics"):
                st.disable_metrics()

    def get_prometheus_metrics(self) -> str:
        from telefuser_b200.metrics import get_metrics_registry

        return get_metrics_registry().to_prometheus()

    def export_metrics(self, path: str) -> str:
        from telefuser_b200.metrics import get_metrics_registry

        with open(path, "w") as f:
            json.dump(get_metrics_registry().to_dict(), f, indent=2)
        return path

    # ---- sizes / tensors ----------------------------------------------------------
    def check_resize_height_width(self, height: int, width: int) -> tuple[int, int]:
        hf, wf = self.height_division_factor, self.width_division_factor
        if height % hf:
            height = (height + hf - 1) // hf * hf
            logger.warning(f"height is rounded up to {height} (multiple of {hf})")
        if width % wf:
            width = (width + wf - 1) // wf * wf
            logger.warning(f"width is rounded up to {width} (multiple of {wf})")
        return height, width

    def preprocess_image(self, image, height: int | None = None, width: int | None = None) -> torch.Tensor:
        """PIL image -> [1, 3, H, W] in [-1, 1]."""
        from PIL import Image

        if height is not None and width is not None:
            image = image.resize((width, height), Image.LANCZOS)
        arr = np.asarray(image.convert("RGB"), dtype=np.float32)
        return torch.from_numpy(arr).permute(2, 0, 1).unsqueeze(0) / 127.5 - 1.0

    @staticmethod
    def tensor2video(frames: torch.Tensor) -> list:
        """[3, T, H, W] in [-1, 1] -> list of PIL images."""
        from PIL import Image

        from telefuser_b200.ops import functional as TF

        arr = TF.frames_to_uint8(frames).cpu().numpy()
        return [Image.fromarray(a) for a in arr]

    @staticmethod
    def generate_noise(shape, seed: int | None = None, device="cpu", dtype=torch.float32) -> torch.Tensor:
        gen = None if seed is None else torch.Generator(device=device).manual_seed(seed)
        return torch.randn(shape, generator=gen, device=device, dtype=dtype)

    def dump_config(self, path: str | None = None) -> dict:
        data = {"pipeline": type(self).__name__, "device": str(self.device), "dtype": str(self.torch_dtype),
                "config": to_jsonable(getattr(self, "config", None)), "models": self._model_info}  # fmt: skip
        if path is not None:
            with open(path, "w") as f:
                json.dump(data, f, indent=2, default=str)
        return data
