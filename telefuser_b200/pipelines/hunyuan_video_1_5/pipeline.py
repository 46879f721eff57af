"""HunyuanVideo-1.5 text / image-to-video pipeline with the optional super-resolution pass.

Base stage: the DiT input is [noisy latents, conditioning latents, mask] on the channel axis (image-to-video puts
the encoded image in the first latent frame and marks it in the mask; text-to-video passes zeros); discrete
flow-matching Euler steps, classifier-free guidance, guidance-embedding and mean-flow (second timestep) variants.
SR stage: the low-resolution latents, resized to the target grid and re-noised to `lq_noise_strength`, are
appended as a second condition; once the trajectory drops below that noise level the condition is zeroed.
Text (LLM + glyph ByT5), vision (image encoder) and VAE components are injected as callables / modules.
Role parity: telefuser/pipelines/hunyuan_video_1_5/{pipeline,dit_denoising,sr_dit_denoising}.py.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch
import torch.nn.functional as F

from telefuser_b200.core.base_pipeline import BasePipeline
from telefuser_b200.core.base_stage import BaseStage, with_model_offload
from telefuser_b200.core.config import ModelRuntimeConfig
from telefuser_b200.parallel import mesh as pmesh
from telefuser_b200.parallel import shard as pshard
from telefuser_b200.schedulers.flow_match_discrete import FlowMatchDiscreteScheduler


@dataclass
class HunyuanVideo15PipelineConfig:
    dit_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    sr_dit_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    vae_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    text_encoding_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    sigma_shift: float = 7.0
    sr_sigma_shift: float = 2.0
    lq_noise_strength: float = 0.7
    use_meanflow: bool = False
    enable_denoising_parallel: bool = False


def image_condition(image_latents, latents):
    """Encoded first frame [B, C, 1, h, w] -> [B, C + 1, T, h, w]: the image in frame 0, zeros elsewhere, plus the mask."""
    cond = image_latents.repeat(1, 1, latents.shape[2], 1, 1)
    cond[:, :, 1:] = 0.0
    mask = torch.zeros_like(latents[:, :1])
    mask[:, :, 0] = 1.0
    return torch.cat([cond, mask], dim=1)


def empty_condition(latents):
    return torch.cat([torch.zeros_like(latents), torch.zeros_like(latents[:, :1])], dim=1)


class HunyuanVideoDenoisingStage(BaseStage):
    def __init__(self, name: str, module_manager: Any, config: ModelRuntimeConfig, scheduler=None, dit=None,
                 use_meanflow: bool = False, module_name: str = "hunyuan_video_dit") -> None:  # fmt: skip
        super().__init__(name, config)
        self.dit = dit if dit is not None else module_manager.fetch_module(module_name)
        self.model_names = ["dit"]
        self.scheduler = scheduler or FlowMatchDiscreteScheduler(shift=7.0)
        self.use_meanflow = use_meanflow
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

    def _guided(self, x, t, pos, neg, cfg_scale, common: dict):
        """pos / neg: dicts with text_states, encoder_attention_mask, byt5_text_states, byt5_text_mask."""
        if not (cfg_scale > 1.0 and neg is not None):
            return self.dit(x, t, cond_flag=True, **pos, **common)
        if self.mesh.size("cfg") == 2:
            is_pos = self.mesh.coord("cfg") == 0
            c, u = pshard.cfg_parallel_unshard(self.dit(x, t, cond_flag=is_pos, **(pos if is_pos else neg), **common), self.mesh)
        else:
            c, u = self.dit(x, t, cond_flag=True, **pos, **common), self.dit(x, t, cond_flag=False, **neg, **common)
        return u + cfg_scale * (c - u)

    def _loop(self, latents, condition_at, pos, neg, cfg_scale, common, scheduler, num_inference_steps):
        scheduler.set_timesteps(num_inference_steps, device=self.device)
        self.setup_feature_cache(self.dit, self.model_runtime_config.feature_cache_config, num_inference_steps)
        self.dit.feature_cache.reset()
        ts = scheduler.timesteps
        for i, t in enumerate(ts):
            tb = t.reshape(1).to(self.device, torch.float32)
            if self.use_meanflow:
                common["timestep_r"] = (ts[i + 1].reshape(1) if i + 1 < len(ts) else torch.zeros(1)).to(self.device, torch.float32)
            x = torch.cat([latents, condition_at(t)], dim=1).to(self.torch_dtype)
            pred = self._guided(x, tb, pos, neg, cfg_scale, common)
            latents = scheduler.step(pred.float(), t, latents, return_dict=False)[0]
        return latents

    @with_model_offload(["dit"])
    @torch.no_grad()
    def process(self, latents, num_inference_steps, prompt_emb_posi, prompt_emb_nega=None, text_states_2=None,
                cfg_scale: float = 1.0, image_latents=None, vision_states=None, attention_mask=None, nega_attention_mask=None,
                task_type: str = "t2v", byt5_text_states=None, byt5_text_mask=None, byt5_text_states_nega=None,
                byt5_text_mask_nega=None):  # fmt: skip
        latents = latents.to(self.device, torch.float32)
        common = dict(text_states_2=text_states_2, vision_states=vision_states, mask_type=task_type)
        if getattr(self.dit, "guidance_embed", False):
            common["guidance"] = torch.full((latents.shape[0],), float(cfg_scale), device=self.device)
        if image_latents is not None and task_type == "i2v":
            cond = image_condition(image_latents.to(latents), latents)
        else:
            cond = empty_condition(latents)
        pos = dict(text_states=prompt_emb_posi, encoder_attention_mask=attention_mask, byt5_text_states=byt5_text_states,
                   byt5_text_mask=byt5_text_mask)  # fmt: skip
        neg = None if prompt_emb_nega is None else dict(text_states=prompt_emb_nega, encoder_attention_mask=nega_attention_mask,
                                                        byt5_text_states=byt5_text_states_nega, byt5_text_mask=byt5_text_mask_nega)  # fmt: skip
        return self._loop(latents, lambda t: cond, pos, neg, cfg_scale, common, self.scheduler, num_inference_steps)


class HunyuanVideoSRDenoisingStage(HunyuanVideoDenoisingStage):
    def __init__(self, name: str, module_manager: Any, config: ModelRuntimeConfig, dit=None, sigma_shift: float = 2.0,
                 lq_noise_strength: float = 0.7) -> None:  # fmt: skip
        super().__init__(name, module_manager, config, FlowMatchDiscreteScheduler(shift=sigma_shift), dit, False,
                         "hunyuan_video_sr_dit")  # fmt: skip
        self.lq_noise_strength = lq_noise_strength

    @with_model_offload(["dit"])
    @torch.no_grad()
    def process(self, latents, lq_latents, num_inference_steps, prompt_emb_posi, prompt_emb_nega=None, cfg_scale: float = 1.0,
                image_cond=None, vision_states=None, attention_mask=None, nega_attention_mask=None, task_type: str = "t2v",
                byt5_text_states=None, byt5_text_mask=None, byt5_text_states_nega=None, byt5_text_mask_nega=None, seed=None):  # fmt: skip
        latents = latents.to(self.device, torch.float32)
        lq = lq_latents.to(self.device, torch.float32)
        if lq.shape[2:] != latents.shape[2:]:
            lq = F.interpolate(lq, size=latents.shape[2:], mode="trilinear", align_corners=False)
        gen = None if seed is None else torch.Generator(device=lq.device).manual_seed(seed)
        s = self.lq_noise_strength
        lq = (1 - s) * lq + s * torch.randn(lq.shape, generator=gen, device=lq.device)
        task = image_condition(image_cond.to(latents), latents) if (image_cond is not None and task_type == "i2v") \
            else empty_condition(latents)  # fmt: skip
        full = torch.cat([task, lq, torch.ones_like(lq[:, :1])], dim=1)
        zeroed = torch.cat([task, torch.zeros_like(lq), torch.zeros_like(lq[:, :1])], dim=1)
        common = dict(text_states_2=None, vision_states=vision_states, mask_type=task_type)
        pos = dict(text_states=prompt_emb_posi, encoder_attention_mask=attention_mask, byt5_text_states=byt5_text_states,
                   byt5_text_mask=byt5_text_mask)  # fmt: skip
        neg = None if prompt_emb_nega is None else dict(text_states=prompt_emb_nega, encoder_attention_mask=nega_attention_mask,
                                                        byt5_text_states=byt5_text_states_nega, byt5_text_mask=byt5_text_mask_nega)  # fmt: skip
        return self._loop(latents, lambda t: zeroed if float(t) < 1000 * s else full, pos, neg, cfg_scale, common,
                          self.scheduler, num_inference_steps)  # fmt: skip


class HunyuanVideo15Pipeline(BasePipeline):
    """`text_stage(prompts) -> list of dicts (text_states, mask, byt5_text_states, byt5_text_mask)`;
    `vision_stage(image) -> vision tokens`; `vae` has encode / decode (latents are returned without one)."""

    def __init__(self, device="cuda", torch_dtype=torch.bfloat16) -> None:
        super().__init__(device=device, torch_dtype=torch_dtype)
        self.height_division_factor = self.width_division_factor = 16
        self.text_stage = self.vision_stage = self.vae = self.sr_stage = self.upsampler = None

    def _get_stages(self) -> list:
        return [s for s in (self.denoise_stage, self.sr_stage) if s is not None]

    def init(self, module_manager, config: HunyuanVideo15PipelineConfig, text_stage=None, vision_stage=None, vae=None, upsampler=None):
        from telefuser_b200.worker.parallel_worker import ParallelWorker

        self.config = config
        self.text_stage, self.vision_stage, self.vae = text_stage, vision_stage, vae
        self.upsampler = upsampler if upsampler is not None else module_manager.fetch_module("upsampler")
        self.denoise_stage = HunyuanVideoDenoisingStage("denoise", module_manager, config.dit_config,
                                                        FlowMatchDiscreteScheduler(shift=config.sigma_shift),
                                                        use_meanflow=config.use_meanflow)  # fmt: skip
        self.denoise_stage.onload_models_flag = True
        if module_manager.fetch_module("hunyuan_video_sr_dit") is not None:
            self.sr_stage = HunyuanVideoSRDenoisingStage("sr_denoise", module_manager, config.sr_dit_config,
                                                         sigma_shift=config.sr_sigma_shift,
                                                         lq_noise_strength=config.lq_noise_strength)  # fmt: skip
            self.sr_stage.onload_models_flag = True
        if config.enable_denoising_parallel:
            self.denoise_stage = ParallelWorker(self.denoise_stage)

    @torch.no_grad()
    def __call__(self, prompt: str = "", negative_prompt: str = "", input_image=None, seed=None, height: int = 480,
                 width: int = 848, num_frames: int = 121, cfg_scale: float = 6.0, num_inference_steps: int = 50,
                 enable_sr: bool = False, sr_height=None, sr_width=None, sr_num_inference_steps: int = 6, text=None,
                 negative_text=None, vision_states=None, image_latents=None, latent_channels: int = 32,
                 spatial_factor: int = 16, return_latents: bool = False):  # fmt: skip
        height, width = self.check_resize_height_width(height, width)
        if text is None:
            enc = self.text_stage([prompt] + ([negative_prompt] if cfg_scale > 1 else []))
            text, negative_text = enc[0], (enc[1] if cfg_scale > 1 else None)
        task = "i2v" if (input_image is not None or image_latents is not None) else "t2v"
        if input_image is not None and image_latents is None:
            img = input_image if isinstance(input_image, torch.Tensor) else self.preprocess_image(input_image, height, width)
            frame = img.unsqueeze(2).to(self.device, self.torch_dtype)
            image_latents = self.vae.encode_latents(frame) if hasattr(self.vae, "encode_latents") else self.vae.encode(frame)
            if vision_states is None and self.vision_stage is not None:
                vision_states = self.vision_stage(img)
        shape = (1, latent_channels, (num_frames - 1) // 4 + 1, height // spatial_factor, width // spatial_factor)
        noise = self.generate_noise(shape, seed=seed, device="cpu").to(self.device)
        kw = dict(prompt_emb_posi=text["text_states"], attention_mask=text.get("mask"), byt5_text_states=text.get("byt5_text_states"),
                  byt5_text_mask=text.get("byt5_text_mask"), vision_states=vision_states, task_type=task)  # fmt: skip
        if negative_text is not None:
            kw.update(prompt_emb_nega=negative_text["text_states"], nega_attention_mask=negative_text.get("mask"),
                      byt5_text_states_nega=negative_text.get("byt5_text_states"), byt5_text_mask_nega=negative_text.get("byt5_text_mask"))  # fmt: skip
        out = self.denoise_stage.process(noise, num_inference_steps, cfg_scale=cfg_scale, image_latents=image_latents, **kw)
        out = out() if callable(out) else out
        if enable_sr and self.sr_stage is not None:
            sh, sw = self.check_resize_height_width(sr_height or height * 2, sr_width or width * 2)
            hi = self.generate_noise((1, latent_channels, shape[2], sh // spatial_factor, sw // spatial_factor),
                                     seed=None if seed is None else seed + 1, device="cpu").to(self.device)  # fmt: skip
            cond = None if image_latents is None else F.interpolate(image_latents.float(), size=(1, *hi.shape[3:]), mode="trilinear")
            if self.upsampler is not None:  # learned refinement of the bilinearly resized low-resolution latents
                from telefuser_b200.models.hunyuan_video_vae import resize_latents

                up_dtype = next(self.upsampler.parameters()).dtype
                out = self.upsampler(resize_latents(out.to(up_dtype), tuple(hi.shape[3:]))).to(out.dtype)
            out = self.sr_stage.process(hi, out, sr_num_inference_steps, cfg_scale=1.0, image_cond=cond, seed=seed, **kw)
        if return_latents or self.vae is None:
            return out
        if hasattr(self.vae, "decode_latents"):
            return self.tensor2video(self.vae.decode_latents(out.to(self.torch_dtype))[0])
        return self.tensor2video(self.vae.decode(out.to(self.torch_dtype))[0])


class HunyuanTextEncodingStage:
    """Prompt list -> list of dicts (text_states, mask, byt5_text_states, byt5_text_mask) from the LLM and glyph encoders."""

    def __init__(self, text_encoder, byt5_encoder=None, data_type: str = "video") -> None:
        self.text_encoder, self.byt5_encoder, self.data_type = text_encoder, byt5_encoder, data_type

    @torch.no_grad()
    def __call__(self, prompts: list) -> list:
        out = []
        for p in prompts:
            enc = self.text_encoder(p, data_type=self.data_type)
            item = {"text_states": enc.hidden_state, "mask": enc.attention_mask}
            if self.byt5_encoder is not None:
                item.update(self.byt5_encoder(p))
            out.append(item)
        return out
