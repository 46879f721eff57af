"""Z-Image text-to-image pipeline.

Stages: text encoding (causal LM, second-to-last hidden state, chat template with thinking enabled, padding
rows dropped so each prompt keeps its own length), denoising (`ZImageDenoisingStage`: discrete flow-matching
Euler steps with a token-count dependent exponential shift; the model sees t' = (1000 - t) / 1000 and predicts
the negative velocity; guidance pos + s (pos - neg) with optional truncation late in the trajectory and norm
capping), VAE decode (2-D KL autoencoder, latents / scaling_factor + shift_factor).
Role parity: telefuser/pipelines/z_image/{z_image,dit_denoising,text_encoding,vae}.py.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch

from telefuser_b200.core.base_pipeline import BasePipeline
from telefuser_b200.core.base_stage import BaseStage, with_model_offload
from telefuser_b200.core.config import ModelRuntimeConfig
from telefuser_b200.parallel import mesh as pmesh
from telefuser_b200.parallel import shard as pshard
from telefuser_b200.schedulers.flow_match_discrete import FlowMatchDiscreteScheduler, linear_mu


@dataclass
class ZImagePipelineConfig:
    vae_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    dit_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    text_encoding_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    enable_denoising_parallel: bool = False


def guided_prediction(pos, neg, scale: float, normalization: float = 0.0):
    """pos + scale (pos - neg); with `normalization` > 0 the result's norm is capped at normalization * |pos|."""
    comb = pos + scale * (pos - neg)
    if normalization and normalization > 0:
        cond_norm, new_norm = torch.linalg.vector_norm(pos.float()), torch.linalg.vector_norm(comb.float())
        new_norm = torch.where(new_norm < 1e-6, torch.ones_like(new_norm), new_norm)
        comb = comb * torch.clamp(cond_norm * normalization / new_norm, max=1.0).to(comb.dtype)
    return comb


class ZImageTextEncodingStage(BaseStage):
    def __init__(self, name: str, module_manager: Any, config: ModelRuntimeConfig, encoder=None, tokenizer=None) -> None:
        super().__init__(name, config)
        self.text_encoder = encoder if encoder is not None else module_manager.fetch_module("text_encoder")
        self.tokenizer = tokenizer if tokenizer is not None else module_manager.fetch_module("tokenizer")
        self.model_names = ["text_encoder"]

    def encode(self, prompts: list[str], max_sequence_length: int = 512) -> list[torch.Tensor]:
        texts = [self.tokenizer.apply_chat_template([{"role": "user", "content": p}], tokenize=False,
                                                    add_generation_prompt=True, enable_thinking=True) for p in prompts]  # fmt: skip
        enc = self.tokenizer(texts, padding="max_length", max_length=max_sequence_length, truncation=True, return_tensors="pt")
        mask = enc.attention_mask.to(self.device).bool()
        out = self.text_encoder(input_ids=enc.input_ids.to(self.device), attention_mask=mask, output_hidden_states=True)
        hidden = out.hidden_states[-2] if hasattr(out, "hidden_states") else out[-2]
        return [hidden[i][mask[i]] for i in range(len(prompts))]

    @with_model_offload(["text_encoder"])
    @torch.no_grad()
    def process(self, prompt, negative_prompt=None, max_sequence_length: int = 512, num_images_per_prompt: int = 1):
        prompts = [prompt] if isinstance(prompt, str) else list(prompt)
        pos = self.encode(prompts, max_sequence_length)
        neg = []
        if negative_prompt is not None:
            negs = [negative_prompt] * len(prompts) if isinstance(negative_prompt, str) else list(negative_prompt)
            if len(negs) != len(prompts):
                raise ValueError("one negative prompt per prompt")
            neg = self.encode(negs, max_sequence_length)
        rep = num_images_per_prompt
        return [e for e in pos for _ in range(rep)], [e for e in neg for _ in range(rep)]


class ZImageVAEStage(BaseStage):
    def __init__(self, name: str, module_manager: Any, config: ModelRuntimeConfig, vae=None) -> None:
        super().__init__(name, config)
        self.vae = vae if vae is not None else module_manager.fetch_module("z_image_vae")
        self.model_names = ["vae"]

    def decode(self, latents: torch.Tensor, tiled: bool = False) -> torch.Tensor:
        c = self.vae.config
        z = latents.to(self.device, self.torch_dtype) / c.scaling_factor + (c.shift_factor or 0.0)
        if not tiled:
            return self.vae.decode(z)
        return tiled_decode(self.vae, z)

    @with_model_offload(["vae"])
    @torch.no_grad()
    def process(self, method: str, *args, **kwargs):
        if method != "decode":
            raise NotImplementedError(f"{method} is not a Z-Image VAE operation")
        return self.decode(*args, **kwargs)


def tiled_decode(vae, z: torch.Tensor, tile: int = 64, overlap: int = 16) -> torch.Tensor:
    """Decodes overlapping latent tiles and cross-fades them linearly over the overlap."""
    f = vae.spatial_factor
    B, _, H, W = z.shape
    out = z.new_zeros(B, vae.config.out_channels, H * f, W * f, dtype=torch.float32)
    weight = torch.zeros(1, 1, H * f, W * f, device=z.device)
    stride = tile - overlap
    for y in range(0, max(H - overlap, 1), stride):
        for x in range(0, max(W - overlap, 1), stride):
            y1, x1 = min(y + tile, H), min(x + tile, W)
            img = vae.decode(z[:, :, y:y1, x:x1]).float()
            h, w = img.shape[-2:]
            ramp = lambda n, lo, hi: torch.minimum(  # noqa: E731
                torch.ones(n, device=z.device) if lo else (torch.arange(n, device=z.device) + 1).clamp(max=overlap * f) / (overlap * f),
                torch.ones(n, device=z.device) if hi else (n - torch.arange(n, device=z.device)).clamp(max=overlap * f) / (overlap * f))
            wy, wx = ramp(h, y == 0, y1 == H), ramp(w, x == 0, x1 == W)
            m = (wy[:, None] * wx[None, :])[None, None]
            out[:, :, y * f : y * f + h, x * f : x * f + w] += img * m
            weight[:, :, y * f : y * f + h, x * f : x * f + w] += m
    return (out / weight).to(z.dtype)


class ZImageDenoisingStage(BaseStage):
    def __init__(self, name: str, module_manager: Any, config: ModelRuntimeConfig, scheduler=None, dit=None) -> None:
        super().__init__(name, config)
        self.dit = dit if dit is not None else module_manager.fetch_module("zimage_dit")
        self.model_names = ["dit"]
        self.scheduler = scheduler or FlowMatchDiscreteScheduler()
        self.batch_cfg = False
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

    def predict_noise(self, latents, t, prompt_emb: list, cond_flag: bool = True):
        xs = list(latents.to(self.torch_dtype).unsqueeze(2).unbind(0))
        return torch.stack(self.dit(xs, t, prompt_emb, cond_flag=cond_flag)).squeeze(2)  # [B, C, H, W]

    def predict_noise_with_cfg(self, latents, timestep, pos: list, neg, cfg_scale: float = 5.0, cfg_truncation: float = 1.0,
                               cfg_normalization: float = 0.0):  # fmt: skip
        t = (1000 - timestep.expand(latents.shape[0]).float()) / 1000
        scale = cfg_scale
        if cfg_truncation <= 1.0 and float(t[0]) > cfg_truncation:
            scale = 0.0
        if not (scale > 0 and neg):
            return -self.predict_noise(latents, t, pos, True)
        if self.mesh.size("cfg") == 2:
            is_pos = self.mesh.coord("cfg") == 0
            mine = self.predict_noise(latents, t, pos if is_pos else neg, is_pos)
            p, n = pshard.cfg_parallel_unshard(mine, self.mesh)
        elif self.batch_cfg:
            both = self.predict_noise(torch.cat([latents, latents]), torch.cat([t, t]), list(pos) + list(neg))
            p, n = both.chunk(2)
        else:
            p, n = self.predict_noise(latents, t, pos, True), self.predict_noise(latents, t, neg, False)
        return -guided_prediction(p, n, scale, float(cfg_normalization or 0.0))

    @with_model_offload(["dit"])
    @torch.no_grad()
    def process(self, latents, prompt_embeds: list, cfg_scale: float, num_inference_steps: int, negative_prompt_embeds=None,
                cfg_normalization: float = 0.0, cfg_truncation: float = 1.0):  # fmt: skip
        dev = self.device
        seq = (latents.shape[2] // 2) * (latents.shape[3] // 2)
        self.scheduler.sigma_min = 0.0
        self.scheduler.set_timesteps_mu(num_inference_steps, linear_mu(seq, 256, 0.5, 4096, 1.15), device=dev)
        self.setup_feature_cache(self.dit, self.model_runtime_config.feature_cache_config, num_inference_steps)
        self.dit.feature_cache.reset()
        latents = latents.to(dev, torch.float32)
        pos = [e.to(dev, self.torch_dtype) for e in prompt_embeds]
        neg = [e.to(dev, self.torch_dtype) for e in (negative_prompt_embeds or [])]
        for t in self.scheduler.timesteps:
            pred = self.predict_noise_with_cfg(latents, t.reshape(1).to(dev), pos, neg, cfg_scale, cfg_truncation, cfg_normalization)
            latents = self.scheduler.step(pred.float(), t, latents, return_dict=False)[0]
        return latents


class ZImagePipeline(BasePipeline):
    def __init__(self, device="cuda", torch_dtype=torch.bfloat16) -> None:
        super().__init__(device=device, torch_dtype=torch_dtype)
        self.vae_stage = self.text_encoding_stage = None

    def _get_stages(self) -> list:
        return [s for s in (self.vae_stage, self.denoise_stage, self.text_encoding_stage) if s is not None]

    def init(self, module_manager, config: ZImagePipelineConfig):
        from telefuser_b200.worker.parallel_worker import ParallelWorker

        self.config = config
        self.scheduler = module_manager.fetch_module("scheduler") or FlowMatchDiscreteScheduler()
        self.denoise_stage = ZImageDenoisingStage("denoise", module_manager, config.dit_config, self.scheduler)
        self.denoise_stage.onload_models_flag = True
        if module_manager.fetch_module("z_image_vae") is not None:
            self.vae_stage = ZImageVAEStage("vae", module_manager, config.vae_config)
        if module_manager.fetch_module("text_encoder") is not None:
            self.text_encoding_stage = ZImageTextEncodingStage("text_encoding", module_manager, config.text_encoding_config)
        if config.enable_denoising_parallel:
            self.denoise_stage = ParallelWorker(self.denoise_stage)

    @staticmethod
    def check_resize_height_width(height: int, width: int) -> tuple[int, int]:
        return (height + 15) // 16 * 16, (width + 15) // 16 * 16

    @torch.no_grad()
    def __call__(self, prompt="", negative_prompt: str | None = "", seed: int | None = None, height: int = 1328,
                 width: int = 1328, cfg_scale: float = 5.0, cfg_normalization: float = 0.0, cfg_truncation: float = 1.0,
                 num_inference_steps: int = 30, num_images_per_prompt: int = 1, tiled: bool = False, prompt_embeds=None,
                 negative_prompt_embeds=None, output_type: str = "pil"):  # fmt: skip
        from telefuser_b200.pipelines.flux2_klein.pipeline import Flux2KleinPipeline

        height, width = self.check_resize_height_width(height, width)
        if cfg_scale <= 1:
            negative_prompt, negative_prompt_embeds = None, None
        if prompt_embeds is not None:
            pos, neg = list(prompt_embeds), list(negative_prompt_embeds or [])
        else:
            if self.text_encoding_stage is None:
                raise RuntimeError("no text encoder loaded: pass prompt_embeds")
            pos, neg = self.text_encoding_stage.process(prompt, negative_prompt, num_images_per_prompt=num_images_per_prompt)
        noise = self.generate_noise((len(pos), 16, height // 8, width // 8), seed=seed, device="cpu")
        out = self.denoise_stage.process(noise, pos, cfg_scale, num_inference_steps, neg, cfg_normalization, cfg_truncation)
        out = out() if callable(out) else out
        if output_type == "latent" or self.vae_stage is None:
            return out
        image = self.vae_stage.process("decode", out, tiled=tiled)
        return image if output_type == "pt" else Flux2KleinPipeline.vae_output_to_images(image)
