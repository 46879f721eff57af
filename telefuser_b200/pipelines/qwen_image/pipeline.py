"""Qwen-Image text-to-image and image-edit pipeline.

Stages: prompt encoding (an injected callable returning `(embeddings [1, L, 3584], mask)`; embeddings
may also be passed directly), denoising (`QwenImageDenoisingStage`: flow matching with the resolution
dependent exponential shift, norm-preserving classifier-free guidance, optional CFG-parallel pair and
Ulysses sequence parallelism), image VAE (any object with `encode` / `decode`; latents are returned
when none is configured). Edit mode appends the encoded reference image(s) as extra image streams.
Role parity: telefuser/pipelines/qwen_image/{qwen_image,qwen_image_edit,dit_denoising}.py.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch

from telefuser_b200.core.base_pipeline import BasePipeline
from telefuser_b200.core.base_stage import BaseStage, with_model_offload
from telefuser_b200.core.config import ModelRuntimeConfig
from telefuser_b200.parallel import mesh as pmesh
from telefuser_b200.parallel import shard as pshard
from telefuser_b200.schedulers.flow_match import FlowMatchScheduler


@dataclass
class QwenImagePipelineConfig:
    dit_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    text_encoding_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    vae_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    enable_denoising_parallel: bool = False


def norm_preserving_cfg(cond: torch.Tensor, uncond: torch.Tensor, scale: float) -> torch.Tensor:
    """u + s (c - u), rescaled so that every row keeps the norm of the conditional prediction."""
    comb = uncond + scale * (cond - uncond)
    cn = torch.norm(cond.float(), dim=-1, keepdim=True)
    nn_ = torch.norm(comb.float(), dim=-1, keepdim=True)
    return (comb.float() * (cn / nn_)).to(cond.dtype)


class QwenImageDenoisingStage(BaseStage):
    def __init__(self, name: str, module_manager: Any, config: ModelRuntimeConfig, dit=None) -> None:
        super().__init__(name, config)
        self.dit = dit if dit is not None else module_manager.fetch_module("qwen_image_dit")
        self.model_names = ["dit"]
        self.scheduler = FlowMatchScheduler("Qwen-Image")
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

    def predict_noise_with_cfg(self, latents, timestep, pos, neg, pos_mask, neg_mask, edit_latents, cfg_scale: float):
        x = latents.to(self.torch_dtype)
        kw = dict(edit_latents=edit_latents)
        if cfg_scale == 1.0 or neg is None:
            return self.dit(x, timestep, pos, pos_mask, cond_flag=True, **kw)
        if self.mesh.size("cfg") == 2:
            is_pos = self.mesh.coord("cfg") == 0
            mine = self.dit(x, timestep, pos if is_pos else neg, pos_mask if is_pos else neg_mask, cond_flag=is_pos, **kw)
            cond, uncond = pshard.cfg_parallel_unshard(mine, self.mesh)
        else:
            cond = self.dit(x, timestep, pos, pos_mask, cond_flag=True, **kw)
            uncond = self.dit(x, timestep, neg, neg_mask, cond_flag=False, **kw)
        return norm_preserving_cfg(cond, uncond, cfg_scale)

    @with_model_offload(["dit"])
    @torch.no_grad()
    def process(self, latents, pos, neg, pos_mask, neg_mask, cfg_scale: float, num_inference_steps: int,
                edit_latents=None, denoising_strength: float = 1.0, exponential_shift_mu: float | None = None,
                shift_terminal: float | None = 0.02):  # fmt: skip
        latents = latents.to(self.device, torch.float32)
        # the shift is derived from latents.shape[1] as the public pipeline does (its dynamic_shift_len argument)
        self.scheduler.set_timesteps(num_inference_steps, denoising_strength=denoising_strength,
                                     dynamic_shift_len=latents.shape[1], exponential_shift_mu=exponential_shift_mu,
                                     shift_terminal=shift_terminal)  # fmt: skip
        self.setup_feature_cache(self.dit, self.model_runtime_config.feature_cache_config, num_inference_steps)
        self.dit.feature_cache.reset()
        if edit_latents is not None:
            edits = edit_latents if isinstance(edit_latents, (list, tuple)) else [edit_latents]
            edit_latents = [e.to(self.device, self.torch_dtype) for e in edits]
        for t in self.scheduler.timesteps:
            ts = t.reshape(1).to(self.device, torch.float32).expand(latents.shape[0])
            pred = self.predict_noise_with_cfg(latents, ts, pos, neg, pos_mask, neg_mask, edit_latents, cfg_scale)
            latents = self.scheduler.step(pred.float(), t, latents)
        return latents


class QwenImagePipeline(BasePipeline):
    def __init__(self, device="cuda", torch_dtype=torch.bfloat16) -> None:
        super().__init__(device=device, torch_dtype=torch_dtype)
        self.text_stage: Callable | None = None
        self.vae = None

    def _get_stages(self) -> list:
        return [self.denoising_stage]

    def init(self, module_manager, config: QwenImagePipelineConfig, text_stage: Callable | None = None, vae=None):
        from telefuser_b200.worker.parallel_worker import ParallelWorker

        self.config = config
        self.text_stage, self.vae = text_stage, vae
        self.denoising_stage = QwenImageDenoisingStage("denoise", module_manager, config.dit_config)
        self.denoising_stage.onload_models_flag = True
        if config.enable_denoising_parallel:
            self.denoising_stage = ParallelWorker(self.denoising_stage)

    @staticmethod
    def check_resize_height_width(height: int, width: int) -> tuple[int, int]:
        return (height + 15) // 16 * 16, (width + 15) // 16 * 16

    def _encode(self, prompt: str, images=None):
        if self.text_stage is None:
            raise RuntimeError("no text stage configured: pass prompt embeddings")
        out = self.text_stage(prompt, images) if images is not None else self.text_stage(prompt)
        return out if isinstance(out, tuple) else (out, None)

    @torch.no_grad()
    def __call__(self, prompt: str = "", negative_prompt: str = "", cfg_scale: float = 4.0, num_inference_steps: int = 40,
                 seed: int | None = None, height: int = 1328, width: int = 1328, prompt_emb=None, prompt_emb_mask=None,
                 negative_prompt_emb=None, negative_prompt_emb_mask=None, edit_image_latents=None,
                 exponential_shift_mu: float | None = None, input_latents=None, denoising_strength: float = 1.0,
                 decode: bool = True):  # fmt: skip
        height, width = self.check_resize_height_width(height, width)
        pos, pmask = (prompt_emb, prompt_emb_mask) if prompt_emb is not None else self._encode(prompt)
        neg = nmask = None
        if cfg_scale != 1.0:
            if negative_prompt_emb is not None:
                neg, nmask = negative_prompt_emb, negative_prompt_emb_mask
            else:
                neg, nmask = self._encode(negative_prompt)
        dev, dt = self.device, self.torch_dtype
        noise = self.generate_noise((1, 16, height // 8, width // 8), seed=seed, device="cpu").to(dev)
        latents = noise
        if input_latents is not None and denoising_strength < 1.0:
            s0 = denoising_strength
            latents = (1 - s0) * input_latents.to(dev, torch.float32) + s0 * noise

        def mask_of(e, m):
            return torch.ones(e.shape[:2], dtype=torch.long, device=dev) if m is None else m.to(dev)

        args = (latents, pos.to(dev, dt), None if neg is None else neg.to(dev, dt), mask_of(pos, pmask),
                None if neg is None else mask_of(neg, nmask), cfg_scale, num_inference_steps, edit_image_latents,
                denoising_strength, exponential_shift_mu)  # fmt: skip
        out = self.denoising_stage.process(*args)
        out = out() if callable(out) else out
        if decode and self.vae is not None:
            return self.vae.decode(out.to(dt))
        return out
