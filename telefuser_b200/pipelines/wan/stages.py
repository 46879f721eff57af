"""Text-encoding, CLIP-encoding and VAE stages of the Wan pipelines.

Role parity: telefuser/pipelines/wan_video/text_encoding.py:16-58, clip_encoding.py and
vae.py:17-260 (`encode_image` I2V mask-concat / TI2V single frame, `encode_video`,
`decode_video`, cached streaming decode, `process(method, ...)` dispatch).
"""

from __future__ import annotations

import os
from typing import Any

import torch

from telefuser_b200.core.base_stage import BaseStage, with_model_offload
from telefuser_b200.core.config import ModelRuntimeConfig
from telefuser_b200.metrics import with_metrics
from telefuser_b200.utils.profiler import ProfilingContext4Debug


class TextEncodingStage(BaseStage):
    def __init__(self, name: str, module_manager: Any, model_runtime_config: ModelRuntimeConfig,
                 max_txt_length: int = 512, text_encoder=None, tokenizer=None) -> None:  # fmt: skip
        super().__init__(name, model_runtime_config)
        if text_encoder is not None:
            self.text_encoder, path = text_encoder, None
        else:
            self.text_encoder, path = module_manager.fetch_module("wan_video_text_encoder", require_model_path=True)
        self.tokenizer = tokenizer
        if self.tokenizer is None and path is not None:
            from telefuser_b200.models.umt5 import HuggingfaceTokenizer

            first = path[0] if isinstance(path, (list, tuple)) else path
            self.tokenizer = HuggingfaceTokenizer(os.path.join(os.path.dirname(first), "google/umt5-xxl"),
                                                  max_txt_length, "whitespace")  # fmt: skip
        self.max_txt_length = max_txt_length
        self.model_names = ["text_encoder"]

    def encode_prompt(self, prompt: str) -> torch.Tensor:
        ids, mask = self.tokenizer(prompt, return_mask=True, add_special_tokens=True)
        ids, mask = ids.to(self.device), mask.to(self.device)
        emb = self.text_encoder(ids, mask)
        lens = mask.gt(0).sum(dim=1)
        for i, n in enumerate(lens.tolist()):
            emb[i, n:] = 0
        return emb

    @with_model_offload(["text_encoder"])
    @ProfilingContext4Debug("text_encoding")
    @torch.no_grad()
    @with_metrics
    def process(self, prompt_list: list[str]) -> list[torch.Tensor]:
        return [self.encode_prompt(p).to(self.torch_dtype) for p in prompt_list]


class ClipEncodingStage(BaseStage):
    """Image encoder for I2V conditioning (open-CLIP ViT-H/14 visual features, 257 tokens x 1280)."""

    def __init__(self, name: str, module_manager: Any, model_runtime_config: ModelRuntimeConfig, image_encoder=None):
        super().__init__(name, model_runtime_config)
        self.image_encoder = image_encoder or module_manager.fetch_module("wan_video_image_encoder")
        self.model_names = ["image_encoder"]

    @with_model_offload(["image_encoder"])
    @torch.no_grad()
    @with_metrics
    def process(self, image: torch.Tensor, end_image: torch.Tensor | None = None) -> torch.Tensor:
        feats = self.image_encoder.encode_image([image.to(self.device)])
        if end_image is not None:
            feats = torch.cat([feats, self.image_encoder.encode_image([end_image.to(self.device)])], dim=1)
        return feats.to(self.torch_dtype)


class VAEStage(BaseStage):
    def __init__(self, name: str, module_manager: Any, model_runtime_config: ModelRuntimeConfig, vae=None) -> None:
        super().__init__(name, model_runtime_config)
        self.vae = vae if vae is not None else module_manager.fetch_module("wan_video_vae")
        self.model_names = ["vae"]
        self._streams: dict = {}

    def parallel_models(self) -> None:
        self.vae.parallelism = self.model_runtime_config.parallel_config.world_size

    # ---- I2V conditioning -------------------------------------------------------
    def encode_image(self, image, end_image, num_frames, tiled=False, tile_size=(34, 34), tile_stride=(18, 16),
                     concat_mask=True):  # fmt: skip
        """Wan2.1 I2V (`concat_mask`): encode [image, zeros..., (end_image)] and prepend a 4-channel frame mask.
        Wan2.2 TI2V: encode only the given frame(s)."""
        h, w = image.shape[2], image.shape[3]
        image = image.to(self.device).squeeze(0)
        kw = dict(device=self.device, tiled=tiled, tile_size=tile_size, tile_stride=tile_stride)
        if not concat_mask:
            start = self.vae.encode(image.unsqueeze(1).unsqueeze(0), **kw)[0]
            if end_image is None:
                return start, num_frames
            end = self.vae.encode(end_image.to(self.device).squeeze(0).unsqueeze(1).unsqueeze(0), **kw)[0]
            return (start, end), num_frames
        parts = [image.unsqueeze(1)]
        if end_image is not None:
            parts += [torch.zeros(3, num_frames - 2, h, w, device=self.device),
                      end_image.to(self.device).squeeze(0).unsqueeze(1)]  # fmt: skip
        else:
            parts += [torch.zeros(3, num_frames - 1, h, w, device=self.device)]
        y = self.vae.encode(torch.cat(parts, dim=1).unsqueeze(0), **kw)[0]
        msk = torch.zeros(4, *y.shape[1:], device=self.device, dtype=y.dtype)
        msk[:, 0] = 1
        if end_image is not None:
            msk[:, -1] = 1
        return torch.cat([msk, y]).unsqueeze(0)

    @ProfilingContext4Debug("vae encode video")
    def encode_video(self, video, tiled=False, tile_size=(34, 34), tile_stride=(18, 16)):
        return self.vae.encode(video, device=self.device, tiled=tiled, tile_size=tile_size, tile_stride=tile_stride)

    @ProfilingContext4Debug("vae decode video")
    def decode_video(self, latents, tiled=False, tile_size=(34, 34), tile_stride=(18, 16)):
        return self.vae.decode(latents, device=self.device, tiled=tiled, tile_size=tile_size, tile_stride=tile_stride)

    # ---- streaming --------------------------------------------------------------------
    def decode_video_cached(self, latents, handle: str = "default"):
        st = self._streams.get(("decode", handle))
        if st is None:
            st = self._streams[("decode", handle)] = self.vae.new_stream("decode")
        return self.vae.cached_decode(latents.to(self.device), st)

    def encode_video_cached(self, frames, handle: str = "default"):
        st = self._streams.get(("encode", handle))
        if st is None:
            st = self._streams[("encode", handle)] = self.vae.new_stream("encode")
        return self.vae.cached_encode(frames.to(self.device), st)

    def release_stream(self, handle: str = "default") -> None:
        self._streams.pop(("decode", handle), None)
        self._streams.pop(("encode", handle), None)

    @with_model_offload(["vae"])
    @torch.no_grad()
    @with_metrics
    def process(self, method: str, *args, **kwargs):
        if method not in ("encode_image", "encode_video", "decode_video", "decode_video_cached",
                          "encode_video_cached", "release_stream"):  # fmt: skip
            raise ValueError(f"unknown VAE method {method}")
        return getattr(self, method)(*args, **kwargs)
