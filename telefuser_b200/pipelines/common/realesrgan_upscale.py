"""Image / frame upscaling stage shared by the pipelines (Real-ESRGAN).
Role parity: telefuser/pipelines/common/realesrgan_upscale.py:11-92."""

from __future__ import annotations

from typing import Any

import torch

from telefuser_b200.core.base_stage import BaseStage, with_model_offload
from telefuser_b200.core.config import ModelRuntimeConfig

from .vfi import images_to_tensor, tensor_to_images


class RealESRGANStage(BaseStage):
    def __init__(self, name: str, module_manager: Any, model_runtime_config: ModelRuntimeConfig, model=None) -> None:
        super().__init__(name, model_runtime_config)
        self.upscaler_model = model if model is not None else module_manager.fetch_module("upscaler_model")
        self.model_names = ["upscaler_model"]

    @with_model_offload(["upscaler_model"])
    @torch.no_grad()
    def process(self, input_images: list) -> list:
        if not input_images:
            return input_images
        return tensor_to_images(self.upscaler_model.upscale_frames(images_to_tensor(input_images), device=self.device))

    @with_model_offload(["upscaler_model"])
    @torch.no_grad()
    def process_tensor(self, input_tensor: torch.Tensor) -> torch.Tensor:
        """[N, H, W, 3] in [0, 1] -> [N, H*s, W*s, 3]."""
        if input_tensor.numel() == 0:
            return input_tensor
        return self.upscaler_model.upscale_frames(input_tensor, device=self.device)
