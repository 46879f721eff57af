"""LongCat-Video pipeline: text-to-video, image-to-video, video continuation and a sparse refinement pass.

Conditioning frames (an image, or the tail of a video) are encoded and placed in front of the noise latents;
they keep timestep 0 and are never updated, or (`use_kv_cache`) their keys / values are cached once and only the
new frames run through the DiT. Guidance is classifier-free with the optional "zero-star" rescaling of the
negative branch; `use_distill` picks the few-step sigma ladder of the distilled LoRA, `enhance_hf` replaces the
tail of the schedule by uniform low-noise steps. Refinement: the low-resolution latents are resized to the target
grid, mixed with noise at `t_thresh` and denoised for a few steps with the 3-D block-sparse attention.
Role parity: telefuser/pipelines/longcat_video/{longcat_video,dit_denoising,refine_denoise,text_encoding}.py.
"""

from __future__ import annotations

import html
import re
from dataclasses import dataclass, field
from typing import Any

import numpy as np
import torch
import torch.nn.functional as F

from telefuser_b200.core.base_pipeline import BasePipeline
from telefuser_b200.core.base_stage import BaseStage, with_model_offload
from telefuser_b200.core.config import ModelRuntimeConfig
from telefuser_b200.parallel import mesh as pmesh
from telefuser_b200.parallel import shard as pshard
from telefuser_b200.schedulers.flow_match_discrete import constant_shift
from telefuser_b200.utils.func import auto_async_call

REFINE_LORA_KEY = "refinement_lora"
DISTILL_LORA_KEY = "cfg_step_lora"

# 720p-class buckets whose sides are multiples of 64 (VAE 8 x patch 2 x sparse chunk 4), keyed by height / width.
_BUCKETS_960_F64 = {0.25: (448, 1792), 0.33: (512, 1536), 0.42: (576, 1408), 0.5: (640, 1280), 0.57: (704, 1216),
                    0.67: (768, 1152), 0.78: (832, 1088), 0.88: (896, 1024), 1.0: (960, 960), 1.14: (1024, 896),
                    1.31: (1088, 832), 1.5: (1152, 768), 1.73: (1216, 704), 2.0: (1280, 640), 2.44: (1408, 576),
                    3.0: (1536, 512), 4.0: (1792, 448)}  # fmt: skip


def bsa_align_resolution(height: int, width: int) -> tuple[int, int]:
    ratio = height / width
    return _BUCKETS_960_F64[min(_BUCKETS_960_F64, key=lambda r: abs(r - ratio))]


def prompt_clean(text: str) -> str:
    text = html.unescape(html.unescape(text)).strip()
    return re.sub(r"\s+", " ", text).strip()


def cfg_zero_star(pos: torch.Tensor, neg: torch.Tensor, scale: float) -> torch.Tensor:
    """neg * a + scale * (pos - neg * a) with a = <pos, neg> / |neg|^2 (per sample)."""
    p, n = pos.flatten(1).float(), neg.flatten(1).float()
    a = ((p * n).sum(1, keepdim=True) / ((n * n).sum(1, keepdim=True) + 1e-8)).view(-1, *([1] * (pos.dim() - 1))).to(pos.dtype)
    return neg * a + scale * (pos - neg * a)


class SigmaLadder:
    """Euler stepping over an explicit sigma ladder (shifted by s*t / (1 + (s-1)*t), terminal 0 appended)."""

    def __init__(self, num_train_timesteps: int = 1000, shift: float = 1.0) -> None:
        self.num_train_timesteps, self.shift = num_train_timesteps, shift
        self.sigmas = self.timesteps = None

    def set_timesteps(self, sigmas: torch.Tensor, device=None) -> None:
        s = constant_shift(sigmas.float(), self.shift) if self.shift != 1.0 else sigmas.float()
        self.set_raw(s * self.num_train_timesteps, device)

    def set_raw(self, timesteps: torch.Tensor, device=None) -> None:
        self.timesteps = timesteps.float().to(device)
        self.sigmas = torch.cat([self.timesteps / self.num_train_timesteps, self.timesteps.new_zeros(1)])

    def step(self, model_output, index: int, sample):
        return (sample.float() + model_output.float() * float(self.sigmas[index + 1] - self.sigmas[index])).to(sample.dtype)


@dataclass
class LongCatVideoPipelineConfig:
    vae_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    dit_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    text_encoding_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    enable_denoising_parallel: bool = False
    enable_refine: bool = False
    refine_height: int = 720
    refine_width: int = 1280
    refine_num_steps: int = 50
    refine_t_thresh: float = 0.5
    enable_refine_bsa: bool = True
    num_ref_video_frames: int = 13


class LongCatTextEncodingStage(BaseStage):
    def __init__(self, name: str, module_manager: Any, config: ModelRuntimeConfig, text_encoder=None, tokenizer=None,
                 max_sequence_length: int = 512) -> None:  # fmt: skip
        super().__init__(name, config)
        self.text_encoder = text_encoder if text_encoder is not None else module_manager.fetch_module("wan_video_text_encoder")
        self.tokenizer = tokenizer if tokenizer is not None else module_manager.fetch_module("tokenizer")
        self.max_sequence_length = max_sequence_length
        self.model_names = ["text_encoder"]

    @with_model_offload(["text_encoder"])
    @torch.no_grad()
    def process(self, prompt_list: list[str]) -> list[tuple[torch.Tensor, torch.Tensor]]:
        """-> per prompt (embeddings [1, 1, L, C], mask [1, L])."""
        out = []
        for p in prompt_list:
            ids, mask = self.tokenizer(prompt_clean(p), return_mask=True, add_special_tokens=True)
            emb = self.text_encoder(ids.to(self.device), mask.to(self.device)).to(self.torch_dtype)
            out.append((emb.unsqueeze(1), mask.to(self.device)))
        return out


class LongCatDitDenoisingStage(BaseStage):
    def __init__(self, name: str, module_manager: Any, config: ModelRuntimeConfig, dit=None) -> None:
        super().__init__(name, config)
        self.dit = dit if dit is not None else module_manager.fetch_module("longcat_video_dit")
        self.model_names = ["dit"]
        self.num_timesteps, self.num_distill_sample_steps = 1000, 50
        self.scheduler = SigmaLadder()
        self.mesh = pmesh.get_mesh()

    def parallel_models(self) -> None:
        cfg = self.model_runtime_config.parallel_config
        self.mesh = pmesh.create_device_mesh_from_config(cfg)
        self.dit.device_mesh = self.mesh
        if cfg.sp_degree > 1:
            self.dit.enable_usp()
        if cfg.enable_fsdp:
            from telefuser_b200.parallel.fsdp import shard_model

            shard_model(self.dit, self.device, wrap_module_names=self.dit.get_fsdp_module_names())

    def get_timesteps_sigmas(self, sampling_steps: int, use_distill: bool = False) -> torch.Tensor:
        if not use_distill:
            return torch.linspace(1, 0.001, sampling_steps)
        n = self.num_distill_sample_steps
        ladder = (torch.arange(1, n + 1, dtype=torch.float32) * (self.num_timesteps // n)).round().long().flip(0)
        pick = np.floor(np.linspace(0, n, num=sampling_steps, endpoint=False)).astype(np.int64)
        return ladder[pick].float() / self.num_timesteps

    def predict_noise_with_cfg(self, latents, timestep, pos, pos_mask, neg, neg_mask, cfg_scale: float = 1.0,
                               use_cfg_zero_star: bool = False, num_cond_latents: int = 0):  # fmt: skip
        run = lambda e, m: self.dit(latents, timestep, e, m, num_cond_latents=num_cond_latents)  # noqa: E731
        if cfg_scale == 1.0 or neg is None:
            return run(pos, pos_mask)
        if self.mesh.size("cfg") == 2:
            is_pos = self.mesh.coord("cfg") == 0
            p, n = pshard.cfg_parallel_unshard(run(pos, pos_mask) if is_pos else run(neg, neg_mask), self.mesh)
        else:
            p, n = run(pos, pos_mask), run(neg, neg_mask)
        return cfg_zero_star(p, n, cfg_scale) if use_cfg_zero_star else n + cfg_scale * (p - n)

    @with_model_offload(["dit"])
    @torch.no_grad()
    def process(self, latents, num_inference_steps, num_cond_latents, prompt_embeds, prompt_attention_mask,
                negative_prompt_embeds=None, negative_prompt_attention_mask=None, cfg_scale: float = 4.0,
                sigma_shift: float = 12.0, use_kv_cache: bool = False, use_cfg_zero_star: bool = True,
                use_distill: bool = False, enhance_hf: bool = False):  # fmt: skip
        self.scheduler.shift = sigma_shift
        self.scheduler.set_timesteps(self.get_timesteps_sigmas(num_inference_steps, use_distill), self.device)
        if enhance_hf:  # keep the steps above t = 500, then ten uniform steps down to 0
            ts = self.scheduler.timesteps
            tail = torch.linspace(500, 0, 11, device=ts.device)[:-1]
            self.scheduler.set_raw(torch.cat([ts[ts > 500], tail]), self.device)
        latents = latents.to(self.device, self.torch_dtype)
        if use_kv_cache and num_cond_latents > 0:
            self.dit.cache_clean_latents(latents[:, :, :num_cond_latents])
            latents = latents[:, :, num_cond_latents:]
        for i, t in enumerate(self.scheduler.timesteps):
            ts = t.reshape(1, 1).expand(latents.shape[0], latents.shape[2]).clone()
            if not use_kv_cache:
                ts[:, :num_cond_latents] = 0
            pred = -self.predict_noise_with_cfg(latents, ts, prompt_embeds, prompt_attention_mask, negative_prompt_embeds,
                                                negative_prompt_attention_mask, cfg_scale, use_cfg_zero_star,
                                                num_cond_latents).to(latents.device)  # fmt: skip
            if use_kv_cache or num_cond_latents == 0:
                latents = self.scheduler.step(pred, i, latents)
            else:
                latents[:, :, num_cond_latents:] = self.scheduler.step(pred[:, :, num_cond_latents:], i,
                                                                        latents[:, :, num_cond_latents:])  # fmt: skip
        self.dit.clear_cache()
        return latents


class LongCatRefineDenoisingStage(BaseStage):
    """Few-step refinement of upsampled latents; shares the DiT with the base stage."""

    def __init__(self, name: str, module_manager: Any, config: ModelRuntimeConfig, dit=None) -> None:
        super().__init__(name, config)
        self.dit = dit if dit is not None else module_manager.fetch_module("longcat_video_dit")
        self.model_names = ["dit"]
        self.num_timesteps = 1000
        self.scheduler = SigmaLadder()

    @with_model_offload(["dit"])
    @torch.no_grad()
    def process(self, lq_latents, num_refine_steps: int, num_cond_latents: int, prompt_embeds, prompt_attention_mask,
                t_thresh: float = 0.5, seed: int | None = None, enable_bsa: bool = False):  # fmt: skip
        loras = getattr(self.dit, "lora_dict", {})
        if REFINE_LORA_KEY in loras:
            self.dit.enable_loras([REFINE_LORA_KEY])
        if enable_bsa:
            self.dit.enable_bsa()
        try:
            return self._denoise(lq_latents, num_refine_steps, num_cond_latents, prompt_embeds, prompt_attention_mask, t_thresh, seed)
        finally:
            if REFINE_LORA_KEY in loras:
                self.dit.disable_all_loras()
            if enable_bsa:
                self.dit.disable_bsa()
            self.dit.clear_cache()

    def _denoise(self, lq, steps, num_cond_latents, emb, mask, t_thresh, seed):
        lq = lq.to(self.device)
        gen = torch.Generator(device=lq.device)
        if seed is not None:
            gen.manual_seed(seed)
        noise = torch.randn(lq.shape, generator=gen, device=lq.device, dtype=torch.float32).to(lq.dtype)
        latents = ((1.0 - t_thresh) * lq + t_thresh * noise).to(self.torch_dtype)
        ts = torch.linspace(1, 0.001, steps) * self.num_timesteps
        t0 = torch.tensor([t_thresh * self.num_timesteps])
        self.scheduler.set_raw(torch.cat([t0, ts[ts < t0]]), self.device)
        for i, t in enumerate(self.scheduler.timesteps):
            tt = t.reshape(1, 1).expand(latents.shape[0], latents.shape[2]).clone()
            tt[:, :num_cond_latents] = 0
            pred = -self.dit(latents, tt, emb, mask, num_cond_latents=num_cond_latents).to(latents.device)
            if num_cond_latents > 0:
                latents[:, :, num_cond_latents:] = self.scheduler.step(pred[:, :, num_cond_latents:], i,
                                                                        latents[:, :, num_cond_latents:])  # fmt: skip
            else:
                latents = self.scheduler.step(pred, i, latents)
        return latents


class LongCatVideoPipeline(BasePipeline):
    def __init__(self, device="cuda", torch_dtype=torch.bfloat16) -> None:
        super().__init__(device=device, torch_dtype=torch_dtype)
        self.height_division_factor = self.width_division_factor = 16
        self.base_fps = 15
        self.vae_stage = self.text_encoding_stage = self.refine_stage = None

    def _get_stages(self) -> list:
        return [s for s in (self.vae_stage, self.denoise_stage, self.text_encoding_stage, self.refine_stage) if s is not None]

    def init(self, module_manager, config: LongCatVideoPipelineConfig, text_stage=None, vae_stage=None):
        from telefuser_b200.worker.parallel_worker import ParallelWorker

        self.config = config
        self.num_ref_video_frames = config.num_ref_video_frames
        self.denoise_stage = LongCatDitDenoisingStage("denoise", module_manager, config.dit_config)
        self.denoise_stage.onload_models_flag = True
        if config.enable_refine:
            self.refine_stage = LongCatRefineDenoisingStage("refine", module_manager, config.dit_config, dit=self.denoise_stage.dit)
            self.refine_stage.onload_models_flag = True
        self.text_encoding_stage = text_stage
        if text_stage is None and module_manager.fetch_module("wan_video_text_encoder") is not None:
            self.text_encoding_stage = LongCatTextEncodingStage("text_encoding", module_manager, config.text_encoding_config)
        self.vae_stage = vae_stage
        if vae_stage is None and module_manager.fetch_module("wan_video_vae") is not None:
            from telefuser_b200.pipelines.wan.stages import VAEStage

            self.vae_stage = VAEStage("vae", module_manager, config.vae_config)
        if config.enable_denoising_parallel:
            self.denoise_stage = ParallelWorker(self.denoise_stage)

    def _encode(self, frames: torch.Tensor, tiler: dict) -> torch.Tensor:
        return auto_async_call(self.vae_stage.process, "encode_video", frames, **tiler)().to(self.device, self.torch_dtype)

    @torch.no_grad()
    def __call__(self, prompt: str = "", negative_prompt: str = "", input_image=None, input_video=None, seed=None,
                 rand_device=None, height: int = 480, width: int = 832, num_frames: int = 81, cfg_scale: float = 4.0,
                 num_inference_steps: int = 50, tiled: bool = True, tile_size=(30, 52), tile_stride=(15, 26),
                 sigma_shift: float = 12.0, use_kv_cache: bool = False, use_cfg_zero_star: bool = True,
                 return_latents: bool = False, need_encode: bool = True, use_distill: bool = False, enhance_hf: bool = False,
                 enable_refine: bool = False, refine_height=None, refine_width=None, refine_num_steps=None,
                 refine_t_thresh=None, enable_refine_bsa=None, prompt_embeds=None, negative_prompt_embeds=None):  # fmt: skip
        """prompt_embeds / negative_prompt_embeds: optional (embeddings [1, 1, L, C], mask [1, L]) pairs."""
        if input_image is None and input_video is None:
            use_kv_cache = False
        height, width = self.check_resize_height_width(height, width)
        if num_frames % 4 != 1:
            num_frames = (num_frames + 2) // 4 * 4 + 1
        tiler = {"tiled": tiled, "tile_size": tile_size, "tile_stride": tile_stride}
        latents = self.generate_noise((1, 16, (num_frames - 1) // 4 + 1, height // 8, width // 8), seed=seed,
                                      device=rand_device or "cpu", dtype=torch.float32).to(self.device, self.torch_dtype)  # fmt: skip
        if prompt_embeds is None:
            embs = self.text_encoding_stage.process([prompt] + ([negative_prompt] if cfg_scale > 1 else []))
            prompt_embeds, negative_prompt_embeds = embs[0], (embs[1] if cfg_scale > 1 else None)
        pos, pos_mask = prompt_embeds
        neg, neg_mask = negative_prompt_embeds if (negative_prompt_embeds is not None and cfg_scale > 1) else (None, None)
        num_cond = 0
        ref = None
        if input_video is not None:
            if need_encode:  # [1, 3, F, H, W] frames in [-1, 1]: the last `num_ref_video_frames` condition the clip
                ref = self._encode(input_video[:, :, -self.num_ref_video_frames :], tiler)
            else:  # latents of the previous clip
                ref = input_video[:, :, -((self.num_ref_video_frames - 1) // 4) :].to(self.device, self.torch_dtype)
        elif input_image is not None:
            img = input_image if isinstance(input_image, torch.Tensor) else self.preprocess_image(input_image, height, width)
            ref = self._encode(img.unsqueeze(2), tiler)
        if ref is not None:
            num_cond = ref.shape[2]
            latents[:, :, :num_cond] = ref
        out = auto_async_call(self.denoise_stage.process, latents, num_inference_steps, num_cond, pos, pos_mask, neg, neg_mask,
                              cfg_scale, sigma_shift, use_kv_cache, use_cfg_zero_star, use_distill, enhance_hf)()  # fmt: skip
        if use_kv_cache and ref is not None:
            out = torch.cat([ref.to(out), out], dim=2)
        if enable_refine and self.refine_stage is not None:
            c = self.config
            rh, rw = refine_height or c.refine_height, refine_width or c.refine_width
            bsa = c.enable_refine_bsa if enable_refine_bsa is None else enable_refine_bsa
            if bsa:
                rh, rw = bsa_align_resolution(rh, rw)
            up = F.interpolate(out.float(), size=(out.shape[2], rh // 8, rw // 8), mode="trilinear", align_corners=False)
            out = self.refine_stage.process(up.to(self.torch_dtype), refine_num_steps or c.refine_num_steps, num_cond, pos,
                                            pos_mask, refine_t_thresh or c.refine_t_thresh, seed, bsa)  # fmt: skip
        if return_latents or self.vae_stage is None:
            return out
        frames = auto_async_call(self.vae_stage.process, "decode_video", out, **tiler)()
        return self.tensor2video(frames[0])
