"""LTX-2 pipeline stages around the denoiser: prompt encoding, image conditioning / video decoding, latent upsampling.

Role parity: telefuser/pipelines/ltx_video/{gemma_text_encoding,vae,upsampler}.py.
"""

from __future__ import annotations

import math
import os
from typing import Any

import numpy as np
import torch
import torch.nn.functional as F

from telefuser_b200.core.base_stage import BaseStage, with_model_offload
from telefuser_b200.core.config import ModelRuntimeConfig
from telefuser_b200.models.ltx_upsampler import upsample_video
from telefuser_b200.models.ltx_video_vae import VIDEO_SCALE_FACTORS

DEFAULT_TILE_SIZE, DEFAULT_TILE_STRIDE = (64, 512), (40, 448)


def image_to_array(image) -> np.ndarray:
    """PIL image, path, bytes, array or tensor -> uint8-range float array [H, W, 3]."""
    from PIL import Image

    if isinstance(image, torch.Tensor):
        image = image.detach().cpu().numpy()
    if isinstance(image, np.ndarray):
        arr = image
        if arr.ndim == 3 and arr.shape[0] in (1, 3) and arr.shape[-1] not in (1, 3):
            arr = arr.transpose(1, 2, 0)
        return arr.astype(np.float32)
    if isinstance(image, (bytes, bytearray)):
        import io

        image = Image.open(io.BytesIO(image))
    elif isinstance(image, (str, os.PathLike)):
        image = Image.open(image)
    return np.asarray(image.convert("RGB"), dtype=np.float32)


def resize_and_center_crop(frame: torch.Tensor, height: int, width: int) -> torch.Tensor:
    """[H, W, 3] -> [1, 3, 1, height, width]: scale so the target is covered, then crop the centre."""
    x = frame.permute(2, 0, 1)[None]
    h, w = x.shape[-2:]
    scale = max(height / h, width / w)
    nh, nw = math.ceil(h * scale), math.ceil(w * scale)
    x = F.interpolate(x, size=(nh, nw), mode="bilinear", align_corners=False)
    top, left = (nh - height) // 2, (nw - width) // 2
    return x[:, :, top : top + height, left : left + width].unsqueeze(2)


class GemmaTextEncodingStage(BaseStage):
    """`process(prompts)` -> one (video_encoding, audio_encoding, attention_mask) per prompt."""

    def __init__(self, name: str, module_manager: Any, config: ModelRuntimeConfig, max_txt_length: int = 1024, text_encoder=None,
                 embeddings_processor=None, tokenizer=None) -> None:  # fmt: skip
        super().__init__(name, config)
        paths = None
        if text_encoder is None:
            text_encoder, paths = module_manager.fetch_module("gemma_text_encoder", require_model_path=True)
        self.text_encoder = text_encoder
        self.embeddings_processor = embeddings_processor if embeddings_processor is not None else module_manager.fetch_module("ltx_embeddings_processor")
        if tokenizer is None and paths:
            from telefuser_b200.models.umt5 import HuggingfaceTokenizer

            first = paths[0] if isinstance(paths, (list, tuple)) else paths
            tokenizer = HuggingfaceTokenizer(os.path.dirname(first), max_txt_length, None)
        self.tokenizer = tokenizer
        self.model_names = ["text_encoder", "embeddings_processor"]

    @staticmethod
    def pad_inputs_for_attention_alignment(inputs: dict, pad_token_id: int = 0, alignment: int = 8) -> dict:
        """Right-pad ids (with `pad_token_id`) and masks (with 0) to a multiple of `alignment` tokens."""
        n = inputs["input_ids"].shape[1]
        extra = -n % alignment
        if extra:
            for key, value in (("input_ids", pad_token_id), ("attention_mask", 0), ("token_type_ids", 0)):
                if inputs.get(key) is not None:
                    inputs[key] = F.pad(inputs[key], (0, extra), value=value)
        return inputs

    def encode_prompt(self, prompt: str):
        ids, mask = self.tokenizer(prompt, return_mask=True, add_special_tokens=True)
        ids, mask = ids.to(self.device), mask.to(self.device)
        hidden = self.text_encoder(input_ids=ids, attention_mask=mask, output_hidden_states=True)
        dtype = next(self.embeddings_processor.parameters()).dtype
        return self.embeddings_processor.process_hidden_states(tuple(h.to(dtype) for h in hidden), mask)

    @with_model_offload(["text_encoder", "embeddings_processor"])
    @torch.no_grad()
    def process(self, prompt_list: list) -> list:
        return [self.encode_prompt(p) for p in prompt_list]


class VAEStage(BaseStage):
    def __init__(self, name: str, module_manager: Any, config: ModelRuntimeConfig, vae=None) -> None:
        super().__init__(name, config)
        self.vae = vae if vae is not None else module_manager.fetch_module("ltx_video_vae")
        self.model_names = ["vae"]

    def _encode_image_latent(self, image, height: int, width: int) -> torch.Tensor:
        frame = torch.tensor(image_to_array(image), dtype=torch.float32, device=self.device)
        x = resize_and_center_crop(frame, height, width)
        return self.vae.encode((x / 127.5 - 1.0).to(self.device, self.torch_dtype), tiled=False)

    def encode_image(self, image, height: int, width: int, frame_idx: int = 0, strength: float = 1.0):
        """-> [1, 1 + C, latent_idx + 1, h, w]: channel 0 is the denoise mask (1 = free), the rest the clean latents,
        with the image in the latent frame that holds pixel frame `frame_idx`; None when there is nothing to apply."""
        strength = max(0.0, min(1.0, float(strength)))
        if image is None or strength <= 0.0:
            return None
        if frame_idx < 0:
            raise ValueError(f"frame_idx must be non-negative, got {frame_idx}")
        idx = frame_idx // VIDEO_SCALE_FACTORS.time
        enc = self._encode_image_latent(image, height, width)
        if enc.shape[0] != 1 or enc.shape[2] != 1:
            raise ValueError(f"expected an image latent [1, C, 1, h, w], got {tuple(enc.shape)}")
        b, c, _, h, w = enc.shape
        latents = torch.zeros((b, c, idx + 1, h, w), device=enc.device, dtype=enc.dtype)
        latents[:, :, idx : idx + 1] = enc
        mask = torch.ones((b, 1, idx + 1, h, w), device=enc.device, dtype=enc.dtype)
        mask[:, :, idx : idx + 1] = 1.0 - strength
        return torch.cat([mask, latents], dim=1)

    def decode_video(self, latents, generator=None, tiled: bool = True, tile_size=DEFAULT_TILE_SIZE, tile_stride=DEFAULT_TILE_STRIDE):
        chunks = list(self.vae.decode(latents.to(self.device, self.torch_dtype), tiled=tiled, tile_size=tile_size, tile_stride=tile_stride,
                                      generator=generator))  # fmt: skip
        return torch.cat(chunks, dim=2)

    def parallel_models(self) -> None:
        self.vae.set_parallelism(self.model_runtime_config.parallel_config.world_size)

    @with_model_offload(["vae"])
    @torch.no_grad()
    def process(self, method: str, *args: Any, **kwargs: Any) -> Any:
        if method not in ("encode_image", "decode_video"):
            raise NotImplementedError(f"{method} is not supported by the LTX VAE stage")
        return getattr(self, method)(*args, **kwargs)


class UpsamplerStage(BaseStage):
    def __init__(self, name: str, module_manager: Any, config: ModelRuntimeConfig, spatial_upsampler=None, vae=None) -> None:
        super().__init__(name, config)
        self.spatial_upsampler = spatial_upsampler if spatial_upsampler is not None else module_manager.fetch_module("ltx_spatial_upsampler")
        self.vae = vae if vae is not None else module_manager.fetch_module("ltx_video_vae")
        self.model_names = ["spatial_upsampler", "vae"]

    @with_model_offload(["spatial_upsampler", "vae"])
    @torch.no_grad()
    def process(self, latent: torch.Tensor) -> torch.Tensor:
        return upsample_video(latent.to(self.device, self.torch_dtype), self.vae.encoder, self.spatial_upsampler)
