"""Frame-rate conversion stage shared by the video pipelines (RIFE).
Role parity: telefuser/pipelines/common/rift_vfi.py:11-54."""

from __future__ import annotations

from typing import Any

import numpy as np
import torch

from telefuser_b200.core.base_stage import BaseStage, with_model_offload
from telefuser_b200.core.config import ModelRuntimeConfig


def images_to_tensor(images: list) -> torch.Tensor:
    """list of PIL images -> [N, H, W, 3] float in [0, 1]."""
    return torch.from_numpy(np.stack([np.asarray(im.convert("RGB"), dtype=np.float32) for im in images])) / 255.0


def tensor_to_images(frames: torch.Tensor) -> list:
    from PIL import Image

    arr = (frames.float() * 255).clamp(0, 255).cpu().numpy().astype(np.uint8)
    return [Image.fromarray(a) for a in arr]


class RiftVFIStage(BaseStage):
    def __init__(self, name: str, module_manager: Any, model_runtime_config: ModelRuntimeConfig, model=None) -> None:
        super().__init__(name, model_runtime_config)
        self.vfi_model = model if model is not None else module_manager.fetch_module("vfi_model")
        self.model_names = ["vfi_model"]

    @with_model_offload(["vfi_model"])
    @torch.no_grad()
    def process(self, input_video: list, base_fps: int, target_fps: int) -> list:
        out = self.vfi_model.interpolate_frames(images_to_tensor(input_video), base_fps, target_fps, device=self.device)
        return tensor_to_images(out)
