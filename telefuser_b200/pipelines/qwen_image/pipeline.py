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

    @classmethod
    def from_pretrained(cls, model_id_or_path: str, device="cuda", torch_dtype=torch.bfloat16, cache_dir=None,
                        attention_config=None, parallel_devices=None, cfg_degree=None, sp_ulysses_degree=None,
                        quant_config=None, **kwargs):  # fmt: skip
        """Qwen-Image from a diffusers-layout folder or hub id: `transformer/` (sharded DiT), `vae/`,
        `text_encoder/` (Qwen2.5-VL) and `tokenizer/` (+ `processor/` for the edit models). The text stage and the
        image VAE are built here, so the returned pipeline takes plain prompts.
        Loader of telefuser/pipelines/qwen_image/qwen_image.py:194."""
        from telefuser_b200.core.module_manager import ModuleManager
        from telefuser_b200.models.hf_text_encoders import QwenImageTextEncoder
        from telefuser_b200.models.qwen_image_dit import QwenImageDiT
        from telefuser_b200.models.qwen_image_vae import QwenImageVAE
        from telefuser_b200.utils.hf import resolve_hf_path
        from telefuser_b200.utils.hf_model_analyzer import HFModelAnalyzer

        from .text_encoding import QwenImageTextEncodingStage

        root = resolve_hf_path(model_id_or_path, cache_dir)
        found = HFModelAnalyzer(root)
        need = {"transformer": found.get_transformer_path(), "vae": found.get_vae_path(),
                "text_encoder": found.get_text_encoder_path(), "tokenizer": found.get_tokenizer_path()}  # fmt: skip
        missing = [k for k, v in need.items() if not v]
        if missing:
            raise FileNotFoundError(f"{root} lacks {', '.join(missing)}; found {sorted(found.analyze())}")
        mm = ModuleManager(torch_dtype=torch_dtype, device=str(device))
        mm.load_model(need["transformer"], model_class=QwenImageDiT, name="qwen_image_dit", model_resource="diffusers",
                      quant_config=quant_config)  # fmt: skip
        mm.load_model(need["vae"], model_class=QwenImageVAE, name="qwen_image_vae", model_resource="diffusers")
        mm.load_model(need["text_encoder"], model_class=QwenImageTextEncoder, name="qwen_image_text_encoder",
                      model_resource="diffusers")  # fmt: skip
        from transformers import AutoProcessor, AutoTokenizer

        tokenizer = AutoTokenizer.from_pretrained(need["tokenizer"])
        proc_dir = found.component_folder("processor") or (root + "/processor")
        import os

        processor = AutoProcessor.from_pretrained(proc_dir) if os.path.isdir(proc_dir) else None
        config = QwenImagePipelineConfig()
        for c in (config.dit_config, config.text_encoding_config, config.vae_config):
            c.torch_dtype, c.device_type = torch_dtype, torch.device(device).type
            c.device_id = torch.device(device).index or 0
        if attention_config is not None:
            config.dit_config.attention_config = attention_config
        if parallel_devices and len(parallel_devices) > 1:
            n = len(parallel_devices)
            pc = config.dit_config.parallel_config
            pc.device_ids = list(parallel_devices)
            pc.cfg_degree = cfg_degree or (2 if n % 2 == 0 else 1)
            pc.sp_ulysses_degree = sp_ulysses_degree or n // pc.cfg_degree
            config.enable_denoising_parallel = True
        for k, v in kwargs.items():
            if hasattr(config, k):
                setattr(config, k, v)
        text_stage = QwenImageTextEncodingStage(mm.fetch_module("qwen_image_text_encoder"), tokenizer, processor, device,
                                                torch_dtype)  # fmt: skip
        pipe = cls(device=device, torch_dtype=torch_dtype)
        pipe.init(mm, config, text_stage=lambda prompt, images=None: (
            text_stage.encode_prompt(prompt) if images is None else text_stage.encode_prompt_with_image(prompt, images)),
            vae=mm.fetch_module("qwen_image_vae"))  # fmt: skip
        return pipe

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
