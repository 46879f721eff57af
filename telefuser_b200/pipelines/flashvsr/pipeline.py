"""FlashVSR streaming video super-resolution pipeline.

The low-quality clip is bicubically upscaled to the target size (padded to a multiple of 128) and consumed in
chunks: the first chunk takes 25 frames (6 latent frames), every later chunk 8 frames (2 latent frames). Per
chunk: project the LQ frames to conditioning tokens (`Causal_LQ4x_Proj`, cache carried between clips), one DiT
evaluation on fresh noise (single step: latents = noise - prediction) with the sparse-attention KV cache
carried between chunks, then the tiny conditional decoder on (latents, LQ frames). Calls can be chained for an
endless stream: the pipeline keeps the last frames of the previous call.
Role parity: telefuser/pipelines/flashvsr/{flashvsr_stream,dit_denoising,vae}.py.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import numpy as np
import torch
import torch.nn.functional as F

from telefuser_b200.core.base_pipeline import BasePipeline
from telefuser_b200.core.base_stage import BaseStage, with_model_offload
from telefuser_b200.core.config import ModelRuntimeConfig
from telefuser_b200.parallel import mesh as pmesh
from telefuser_b200.utils.func import auto_async_call


def compute_scaled_and_target_dims(w0: int, h0: int, scale: float = 4.0, multiple: int = 128):
    if w0 <= 0 or h0 <= 0 or scale <= 0:
        raise ValueError("invalid size or scale")
    sW, sH = int(round(w0 * scale)), int(round(h0 * scale))
    tW, tH = int(round(sW / multiple)) * multiple, int(round(sH / multiple)) * multiple
    if tW == 0 or tH == 0:
        raise ValueError(f"scaled size {sW}x{sH} is too small for a multiple of {multiple}")
    return sW, sH, tW, tH


def prepare_input_tensor(video: list, scale: float = 4, dtype=torch.bfloat16, device="cpu"):
    """PIL frames -> ([1, 3, F, tH, tW] in [-1, 1], tH, tW, sH, sW): bicubic upscale, zero pad / crop to the target."""
    if not video:
        raise RuntimeError("input video is empty")
    w0, h0 = video[0].size
    sW, sH, tW, tH = compute_scaled_and_target_dims(w0, h0, scale, 128)
    arr = torch.from_numpy(np.stack([np.asarray(im.convert("RGB"), np.uint8) for im in video])).permute(0, 3, 1, 2).float()
    up = F.interpolate(arr, size=(sH, sW), mode="bicubic", align_corners=False, antialias=True)
    up = F.pad(up, [0, max(tW - sW, 0), 0, max(tH - sH, 0)])[:, :, :tH, :tW]
    vid = (up / 255 * 2.0 - 1.0).permute(1, 0, 2, 3).unsqueeze(0)
    return vid.to(dtype=dtype, device=device), tH, tW, min(sH, tH), min(sW, tW)


@dataclass
class FlashVSRPipelineConfig:
    vae_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    dit_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    enable_denoising_parallel: bool = False
    max_chunk_num: int = 128
    enable_metrics: bool = False


class FlashVSRVAEStage(BaseStage):
    def __init__(self, name: str, module_manager: Any, config: ModelRuntimeConfig, vae=None) -> None:
        super().__init__(name, config)
        self.vae = vae if vae is not None else module_manager.fetch_module("wan_video_decoder")
        self.model_names = ["vae"]

    def decode_video(self, latents: torch.Tensor, cond_video: torch.Tensor) -> torch.Tensor:
        """latents [1, C, T, h, w], cond_video [1, 3, 4T(-3), 8h, 8w] -> frames [1, 3, T', 8h, 8w] in [-1, 1]."""
        p = next(self.vae.parameters())
        out = self.vae.decode(latents.transpose(1, 2).to(self.device, p.dtype), cond=cond_video.to(self.device, p.dtype))
        return out.transpose(1, 2).mul(2).sub(1)

    def clean_cache(self) -> None:
        self.vae.clean_mem()

    @with_model_offload(["vae"])
    @torch.no_grad()
    def process(self, method: str, *args, **kwargs):
        if method not in ("decode_video", "clean_cache"):
            raise NotImplementedError(f"{method} is not a FlashVSR decoder operation")
        return getattr(self, method)(*args, **kwargs)


class FlashVSRDenoisingStage(BaseStage):
    def __init__(self, name: str, module_manager: Any, config: ModelRuntimeConfig, dit=None) -> None:
        super().__init__(name, config)
        self.dit = dit if dit is not None else module_manager.fetch_module("flashvsr_dit")
        self.model_names = ["dit"]
        self.cur_process_idx = 0
        self.pre_LQ_video_cache = None
        self.proj_tile, self.proj_tile_size, self.proj_tile_stride = False, (512, 1024), (384, 896)

    def parallel_models(self) -> None:
        cfg = self.model_runtime_config.parallel_config
        self.dit.device_mesh = pmesh.create_device_mesh_from_config(cfg)
        self.dit.LQ_proj_in.set_parallelism(cfg.world_size)
        if cfg.sp_degree > 1:
            self.dit.enable_usp()

    @staticmethod
    def _compute_topk_ratio(sparse_ratio: float, height: int, width: int) -> float:
        return sparse_ratio * 768 * 1280 / (height * width)

    def _project(self, video, start_frame: int, num_clips: int, clip_length: int = 4, overlap: int = 3):
        outs = []
        for i in range(num_clips):
            s = start_frame + max(0, i * clip_length - overlap)
            e = start_frame + (i + 1) * clip_length - overlap
            if e > video.shape[2]:
                break
            cur = self.dit.proj_LQ_video_clip(video[:, :, s:e].to(self.device), tile=self.proj_tile,
                                              tile_size=self.proj_tile_size, tile_stride=self.proj_tile_stride)  # fmt: skip
            if cur is not None:
                outs.append(cur[0])
        return torch.cat(outs, dim=1)

    def _one_step(self, noise, lq_tokens, topk_ratio, kv_ratio, local_range):
        x = noise.to(self.device, self.torch_dtype)
        pred = self.dit(x, LQ_latents=[lq_tokens], is_stream=True, topk_ratio=topk_ratio, kv_ratio=kv_ratio,
                        cur_process_idx=self.cur_process_idx, local_range=local_range)  # fmt: skip
        self.cur_process_idx += 1
        return x - pred

    @with_model_offload(["dit"])
    @torch.no_grad()
    def denoise(self, LQ_video, seed, rand_device, height, width, sparse_ratio: float = 2.0, local_range: int = 9,
                proj_tile: bool = False, proj_tile_size=(512, 1024), proj_tile_stride=(384, 896), kv_ratio: int = 3):  # fmt: skip
        self.proj_tile, self.proj_tile_size, self.proj_tile_stride = proj_tile, proj_tile_size, proj_tile_stride
        topk_ratio = self._compute_topk_ratio(sparse_ratio, height, width)
        lat_shape = (LQ_video.shape[-2] // 8, LQ_video.shape[-1] // 8)
        gen = None if seed is None else torch.Generator(rand_device).manual_seed(seed)
        latents_total, ref_total = [], []
        if self.cur_process_idx == 0:
            if LQ_video.shape[2] < 25:
                raise RuntimeError(f"the first chunk needs at least 25 frames, got {LQ_video.shape[2]}")
            noise = torch.randn((1, 16, 6, *lat_shape), generator=gen, device=rand_device, dtype=torch.float32)
            self.pre_LQ_video_cache = LQ_video[:, :, 21:25]
            tokens = self._project(LQ_video, 0, 7, 4, 3)
            latents_total.append(self._one_step(noise, tokens, topk_ratio, kv_ratio, local_range))
            ref_total.append(LQ_video[:, :, :21].to(self.device))
            LQ_video = LQ_video[:, :, 25:]
        loops = LQ_video.shape[2] // 8
        if loops > 0:
            noise = torch.randn((1, 16, loops * 2, *lat_shape), generator=gen, device=rand_device, dtype=torch.float32)
            combined = torch.cat([self.pre_LQ_video_cache.to(LQ_video), LQ_video], dim=2)
            for c in range(loops):
                tokens = self._project(combined, 4 + c * 8, 2, 4, 0)
                latents_total.append(self._one_step(noise[:, :, 2 * c : 2 * c + 2], tokens, topk_ratio, kv_ratio, local_range))
                ref_total.append(combined[:, :, c * 8 : (c + 1) * 8].to(self.device))
            self.pre_LQ_video_cache = combined[:, :, -4:]
        if not latents_total:
            return torch.empty(0), torch.empty(0)
        return torch.cat(latents_total, dim=2), torch.cat(ref_total, dim=2)

    def clean_cache(self) -> None:
        self.dit.clean_LQ_proj_in_cache()
        self.dit.clear_kv_cache()
        self.cur_process_idx = 0
        self.pre_LQ_video_cache = None

    def process(self, method: str, *args, **kwargs):
        if method not in ("denoise", "clean_cache"):
            raise NotImplementedError(f"{method} is not a FlashVSR DiT operation")
        return getattr(self, method)(*args, **kwargs)


class FlashVSRStreamPipeline(BasePipeline):
    def __init__(self, device="cuda", torch_dtype=torch.bfloat16) -> None:
        super().__init__(device=device, torch_dtype=torch_dtype)
        self.pre_frames_cache = None
        self.process_chunk_idx = 0

    def _get_stages(self) -> list:
        return [self.vae_stage, self.denoise_stage]

    def init(self, module_manager, config: FlashVSRPipelineConfig):
        from telefuser_b200.worker.parallel_worker import ParallelWorker

        self.config = config
        self.vae_stage = FlashVSRVAEStage("vae", module_manager, config.vae_config)
        self.denoise_stage = FlashVSRDenoisingStage("denoise", module_manager, config.dit_config)
        self.vae_stage.onload_models_flag = self.denoise_stage.onload_models_flag = True
        if config.enable_denoising_parallel:
            self.denoise_stage = ParallelWorker(self.denoise_stage)

    @torch.no_grad()
    def __call__(self, seed: int | None = None, LQ_video: list | None = None, sparse_ratio: float = 2.0, kv_ratio: int = 3,
                 local_range: int = 9, scale: float = 4, rand_device: str = "cpu", proj_tile: bool = False,
                 output_type: str = "pil"):  # fmt: skip
        num_frames = len(LQ_video)
        video, height, width, real_h, real_w = prepare_input_tensor(LQ_video, scale=scale, dtype=self.torch_dtype, device="cpu")
        continuing = self.pre_frames_cache is not None and self.process_chunk_idx < self.config.max_chunk_num
        if continuing:
            video = torch.cat([self.pre_frames_cache, video], dim=2)
        else:
            self.clean_cache()
        latents, ref = auto_async_call(self.denoise_stage.process, "denoise", proj_tile=proj_tile, LQ_video=video,
                                       seed=seed, rand_device=rand_device, sparse_ratio=sparse_ratio, local_range=local_range,
                                       kv_ratio=kv_ratio, height=height, width=width)()  # fmt: skip
        frames = auto_async_call(self.vae_stage.process, "decode_video", latents, ref)()
        out = frames[0][:, -(num_frames - 4) :, :real_h, :real_w] if continuing else frames[0][:, :, :real_h, :real_w]
        self.pre_frames_cache = torch.cat([video[:, :, -8:-7], video[:, :, -8:]], dim=2)
        self.process_chunk_idx += num_frames // 8
        return out if output_type == "pt" else self.tensor2video(out)

    def clean_cache(self) -> None:
        auto_async_call(self.denoise_stage.process, "clean_cache")()
        self.vae_stage.clean_cache()
        self.pre_frames_cache = None
        self.process_chunk_idx = 0
