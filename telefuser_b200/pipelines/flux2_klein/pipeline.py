"""FLUX.2-klein text-to-image / reference-image editing pipeline.

Stages: text encoding (a causal LM whose hidden states at three depths are concatenated channel-wise into
the joint embedding, chat-templated prompt padded to a fixed length), denoising (flow matching with the
empirical resolution/step dependent shift, optional classifier-free guidance run sequentially or as a
CFG-parallel pair, reference-image tokens appended with their own time coordinate), VAE (2x2 patchified
latent normalised by the autoencoder's BatchNorm statistics). Latent tokens carry 4-axis ids (T, H, W, L).
Role parity: telefuser/pipelines/flux2_klein/{pipeline,dit_denoising,text_encoding,vae}.py.
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
from telefuser_b200.schedulers.flow_match import FlowMatchScheduler, flux2_empirical_mu


@dataclass
class Flux2KleinPipelineConfig:
    dit_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    text_encoding_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    vae_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    sample_solver: str = "euler"
    enable_denoising_parallel: bool = False


def latent_ids(height: int, width: int, t: int = 0) -> torch.Tensor:
    """[height*width, 4] integer (T, H, W, L) coordinates in row-major token order."""
    return torch.cartesian_prod(torch.tensor([t]), torch.arange(height), torch.arange(width), torch.arange(1))


def text_ids(length: int) -> torch.Tensor:
    z = torch.zeros(length, dtype=torch.long)
    return torch.stack([z, z, z, torch.arange(length)], dim=1)


def reference_image_ids(shapes, scale: int = 10) -> torch.Tensor:
    """Reference image i (latent height, width) sits at time coordinate scale * (i + 1)."""
    return torch.cat([latent_ids(h, w, scale * (i + 1)) for i, (h, w) in enumerate(shapes)], dim=0)


def patchify_latents(z: torch.Tensor) -> torch.Tensor:
    B, C, H, W = z.shape
    return z.view(B, C, H // 2, 2, W // 2, 2).permute(0, 1, 3, 5, 2, 4).reshape(B, C * 4, H // 2, W // 2)


def unpatchify_latents(z: torch.Tensor) -> torch.Tensor:
    B, C, H, W = z.shape
    return z.reshape(B, C // 4, 2, 2, H, W).permute(0, 1, 4, 2, 5, 3).reshape(B, C // 4, H * 2, W * 2)


def pack_latents(z: torch.Tensor) -> torch.Tensor:
    return z.flatten(2).transpose(1, 2)


def unpack_latents_with_ids(tokens: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """tokens [B, S, C] placed at their (H, W) coordinates -> [B, C, H, W]."""
    ids = ids[0] if ids.ndim == 3 else ids
    h_ids, w_ids = ids[:, 1].long(), ids[:, 2].long()
    H, W = int(h_ids.max()) + 1, int(w_ids.max()) + 1
    out = tokens.new_zeros(tokens.shape[0], H * W, tokens.shape[2])
    out[:, (h_ids * W + w_ids).to(tokens.device)] = tokens
    return out.view(tokens.shape[0], H, W, -1).permute(0, 3, 1, 2)


class Flux2TextEncodingStage(BaseStage):
    """prompt -> ([B, L, n_layers * hidden], ids). `encoder` is a causal LM returning `hidden_states`."""

    def __init__(self, name: str, module_manager: Any, config: ModelRuntimeConfig, encoder=None, tokenizer=None) -> None:
        super().__init__(name, config)
        self.text_encoder = encoder if encoder is not None else module_manager.fetch_module("text_encoder")
        self.tokenizer = tokenizer if tokenizer is not None else module_manager.fetch_module("tokenizer")
        self.model_names = ["text_encoder"]

    def embed(self, prompts: list[str], max_sequence_length: int, layers) -> torch.Tensor:
        ids, masks = [], []
        for p in prompts:
            text = self.tokenizer.apply_chat_template([{"role": "user", "content": p}], tokenize=False,
                                                      add_generation_prompt=True, enable_thinking=False)  # fmt: skip
            enc = self.tokenizer(text, return_tensors="pt", padding="max_length", truncation=True, max_length=max_sequence_length)
            ids.append(enc["input_ids"])
            masks.append(enc["attention_mask"])
        out = self.text_encoder(input_ids=torch.cat(ids).to(self.device), attention_mask=torch.cat(masks).to(self.device),
                                output_hidden_states=True, use_cache=False)  # fmt: skip
        return torch.cat([out.hidden_states[k] for k in layers], dim=-1).to(self.device, self.torch_dtype)

    @with_model_offload(["text_encoder"])
    @torch.no_grad()
    def process(self, prompt, negative_prompt=None, num_images_per_prompt: int = 1, max_sequence_length: int = 512,
                hidden_states_layers=(9, 18, 27)):  # fmt: skip
        prompts = [prompt] if isinstance(prompt, str) else list(prompt)
        pos = self.embed(prompts, max_sequence_length, hidden_states_layers).repeat_interleave(num_images_per_prompt, 0)
        neg = None
        if negative_prompt is not None:
            negs = [negative_prompt] * len(prompts) if isinstance(negative_prompt, str) else list(negative_prompt)
            if len(negs) == 1:
                negs = negs * len(prompts)
            neg = self.embed(negs, max_sequence_length, hidden_states_layers).repeat_interleave(num_images_per_prompt, 0)
        return pos, text_ids(pos.shape[1]), neg, None if neg is None else text_ids(neg.shape[1])


class Flux2VAEStage(BaseStage):
    def __init__(self, name: str, module_manager: Any, config: ModelRuntimeConfig, vae=None) -> None:
        super().__init__(name, config)
        self.vae = vae if vae is not None else module_manager.fetch_module("vae")
        self.model_names = ["vae"]

    @staticmethod
    def preprocess_image(image) -> torch.Tensor:
        import numpy as np

        arr = np.asarray(image.convert("RGB"), dtype=np.float32)
        return torch.from_numpy(arr / 255 * 2 - 1).permute(2, 0, 1).unsqueeze(0)

    def encode_image(self, image: torch.Tensor) -> torch.Tensor:
        z = patchify_latents(self.vae.encode(image.to(self.device, self.torch_dtype)).mode())
        mean, std = self.vae.latent_stats(self.device, z.dtype)
        return pack_latents((z - mean) / std)

    def decode_latents(self, latents: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        z = unpack_latents_with_ids(latents.to(self.device, self.torch_dtype), ids)
        mean, std = self.vae.latent_stats(self.device, z.dtype)
        return self.vae.decode(unpatchify_latents(z * std + mean))

    @with_model_offload(["vae"])
    @torch.no_grad()
    def process(self, method: str, *args, **kwargs):
        if method not in ("encode_image", "decode_latents"):
            raise NotImplementedError(f"{method} is not a FLUX.2 VAE operation")
        return getattr(self, method)(*args, **kwargs)


class Flux2DenoisingStage(BaseStage):
    def __init__(self, name: str, module_manager: Any, config: ModelRuntimeConfig, scheduler=None, dit=None) -> None:
        super().__init__(name, config)
        self.transformer = dit if dit is not None else module_manager.fetch_module("flux2_dit")
        self.model_names = ["transformer"]
        self.scheduler = scheduler or FlowMatchScheduler("FLUX.2")
        self.mesh = pmesh.get_mesh()

    def parallel_models(self) -> None:
        cfg = self.model_runtime_config.parallel_config
        self.mesh = pmesh.create_device_mesh_from_config(cfg)
        self.transformer.device_mesh = self.mesh
        if cfg.sp_degree > 1:
            self.transformer.enable_usp()
        if cfg.enable_fsdp:
            from telefuser_b200.parallel.fsdp import shard_model

            shard_model(self.transformer, self.device, wrap_module_names=self.transformer.get_fsdp_module_names())

    def predict_noise_with_cfg(self, latents, timestep, pos, pos_ids, lat_ids, cfg_scale, neg=None, neg_ids=None,
                               image_latents=None, image_ids=None):  # fmt: skip
        x, ids = latents, lat_ids
        if image_latents is not None:
            x = torch.cat([latents, image_latents], dim=1)
            ids = torch.cat([lat_ids, image_ids], dim=0)
        n = latents.shape[1]

        def run(emb, tids, flag):
            return self.transformer(x.to(self.torch_dtype), emb, timestep / 1000, ids, tids, cond_flag=flag)[:, :n]

        if not (cfg_scale > 1.0 and neg is not None):
            return run(pos, pos_ids, True)
        if self.mesh.size("cfg") == 2:
            is_pos = self.mesh.coord("cfg") == 0
            mine = run(pos if is_pos else neg, pos_ids if is_pos else neg_ids, is_pos)
            cond, uncond = pshard.cfg_parallel_unshard(mine, self.mesh)
        else:
            cond, uncond = run(pos, pos_ids, True), run(neg, neg_ids, False)
        return uncond + cfg_scale * (cond - uncond)

    @with_model_offload(["transformer"])
    @torch.no_grad()
    def process(self, latents, prompt_embeds, text_ids, cfg_scale: float, num_inference_steps: int, latent_ids,
                negative_prompt_embeds=None, negative_text_ids=None, image_latents=None, image_latent_ids=None,
                sigmas=None):  # fmt: skip
        dev, dt = self.device, self.torch_dtype
        mu = flux2_empirical_mu(latents.shape[1], num_inference_steps)
        if sigmas is None:
            sigmas = torch.linspace(1.0, 1 / num_inference_steps, num_inference_steps).tolist()
        self.scheduler.set_timesteps_with_mu(sigmas=sigmas, mu=mu)
        self.setup_feature_cache(self.transformer, self.model_runtime_config.feature_cache_config, num_inference_steps)
        self.transformer.feature_cache.reset()
        latents = latents.to(dev, torch.float32)
        pos = prompt_embeds.to(dev, dt)
        neg = None if negative_prompt_embeds is None else negative_prompt_embeds.to(dev, dt)
        image_latents = None if image_latents is None else image_latents.to(dev, dt)
        for t in self.scheduler.timesteps:
            ts = t.reshape(1).to(dev, torch.float32).expand(latents.shape[0])
            pred = self.predict_noise_with_cfg(latents, ts, pos, text_ids, latent_ids, cfg_scale, neg, negative_text_ids,
                                               image_latents, image_latent_ids)  # fmt: skip
            latents = self.scheduler.step(pred.float(), t, latents)
        return latents


class Flux2KleinPipeline(BasePipeline):
    def __init__(self, device="cuda", torch_dtype=torch.bfloat16) -> None:
        super().__init__(device=device, torch_dtype=torch_dtype)
        self.text_encoding_stage = None
        self.vae_stage = None

    def _get_stages(self) -> list:
        return [s for s in (self.vae_stage, self.denoise_stage, self.text_encoding_stage) if s is not None]

    def init(self, module_manager, config: Flux2KleinPipelineConfig):
        from telefuser_b200.worker.parallel_worker import ParallelWorker

        if config.sample_solver != "euler":
            raise NotImplementedError(f"solver {config.sample_solver} is not supported")
        self.config = config
        self.scheduler = FlowMatchScheduler("FLUX.2")
        self.denoise_stage = Flux2DenoisingStage("denoise", module_manager, config.dit_config, self.scheduler)
        self.denoise_stage.onload_models_flag = True
        if module_manager.fetch_module("vae") is not None:
            self.vae_stage = Flux2VAEStage("vae", module_manager, config.vae_config)
        if module_manager.fetch_module("text_encoder") is not None:
            self.text_encoding_stage = Flux2TextEncodingStage("text_encoding", module_manager, config.text_encoding_config)
        if config.enable_denoising_parallel:
            self.denoise_stage = ParallelWorker(self.denoise_stage)

    @classmethod
    def from_pretrained(cls, model_id_or_path: str, device="cuda", torch_dtype=torch.bfloat16, cache_dir=None,
                        attention_config=None, parallel_devices=None, cfg_degree=None, sp_ulysses_degree=None,
                        quant_config=None, **kwargs):  # fmt: skip
        """FLUX.2 [klein] from a diffusers-layout folder or hub id: `transformer/`, `vae/` (2-D KL autoencoder),
        `text_encoder/` (a Qwen3 causal LM, loaded through transformers) and `tokenizer/`.
        Loader of telefuser/pipelines/flux2_klein/pipeline.py:286."""
        from telefuser_b200.core.module_manager import ModuleManager
        from telefuser_b200.models.autoencoder_kl import AutoencoderKL
        from telefuser_b200.models.flux2_dit import Flux2DiT
        from telefuser_b200.utils.hf import resolve_hf_path
        from telefuser_b200.utils.hf_model_analyzer import HFModelAnalyzer

        root = resolve_hf_path(model_id_or_path, cache_dir)
        found = HFModelAnalyzer(root)
        dit_path, vae_path = found.get_transformer_path(), found.get_vae_path()
        if not dit_path:
            raise FileNotFoundError(f"{root} has no transformer weights; found {sorted(found.analyze())}")
        mm = ModuleManager(torch_dtype=torch_dtype, device=str(device))
        mm.load_model(dit_path, model_class=Flux2DiT, name="flux2_dit", model_resource="diffusers", quant_config=quant_config)
        if vae_path:
            mm.load_model(vae_path, model_class=AutoencoderKL, name="vae", model_resource="diffusers")
        enc_dir, tok_dir = found.component_folder("text_encoder"), found.get_tokenizer_path()
        if enc_dir and tok_dir:
            from transformers import AutoModelForCausalLM, AutoTokenizer

            mm.load_from_huggingface(enc_dir, "text_encoder", AutoModelForCausalLM, torch_dtype=torch_dtype, device=device)
            mm.add_module(AutoTokenizer.from_pretrained(tok_dir), "tokenizer", path=tok_dir)
        config = Flux2KleinPipelineConfig()
        for c in (config.dit_config, config.text_encoding_config, config.vae_config):
            c.torch_dtype, c.device_type = torch_dtype, torch.device(device).type
            c.device_id = torch.device(device).index or 0
        if attention_config is not None:
            config.dit_config.attention_config = attention_config
        if parallel_devices and len(parallel_devices) > 1:
            n = len(parallel_devices)
            pc = config.dit_config.parallel_config
            pc.device_ids = list(parallel_devices)
            pc.cfg_degree = cfg_degree or 1
            pc.sp_ulysses_degree = sp_ulysses_degree or n // pc.cfg_degree
            config.enable_denoising_parallel = True
        for k, v in kwargs.items():
            if hasattr(config, k):
                setattr(config, k, v)
        pipe = cls(device=device, torch_dtype=torch_dtype)
        pipe.init(mm, config)
        return pipe

    @staticmethod
    def check_resize_height_width(height: int, width: int) -> tuple[int, int]:
        return (height + 15) // 16 * 16, (width + 15) // 16 * 16

    @staticmethod
    def vae_output_to_images(x: torch.Tensor) -> list:
        from PIL import Image

        arr = ((x.float().cpu() / 2 + 0.5).clamp(0, 1) * 255).permute(0, 2, 3, 1).numpy().astype("uint8")
        return [Image.fromarray(a) for a in arr]

    @torch.no_grad()
    def __call__(self, prompt="", negative_prompt: str | None = "", seed: int | None = None, height: int = 1024,
                 width: int = 1024, cfg_scale: float = 4.0, num_inference_steps: int = 50, num_images_per_prompt: int = 1,
                 max_sequence_length: int = 512, hidden_states_layers=(9, 18, 27), reference_images=None,
                 prompt_embeds=None, negative_prompt_embeds=None, output_type: str = "pil"):  # fmt: skip
        height, width = self.check_resize_height_width(height, width)
        lh, lw = height // 16, width // 16
        if cfg_scale <= 1:
            negative_prompt, negative_prompt_embeds = None, None
        if prompt_embeds is not None:
            pos, pos_ids = prompt_embeds, text_ids(prompt_embeds.shape[1])
            neg = negative_prompt_embeds
            neg_ids = None if neg is None else text_ids(neg.shape[1])
        else:
            if self.text_encoding_stage is None:
                raise RuntimeError("no text encoder loaded: pass prompt_embeds")
            pos, pos_ids, neg, neg_ids = self.text_encoding_stage.process(
                prompt, negative_prompt, num_images_per_prompt, max_sequence_length, hidden_states_layers)  # fmt: skip
        batch = pos.shape[0]
        noise = self.generate_noise((batch, 128, lh, lw), seed=seed, device="cpu")
        ids = latent_ids(lh, lw)
        image_latents = image_ids = None
        if reference_images:
            if self.vae_stage is None:
                raise RuntimeError("reference images need a VAE")
            refs = [r if isinstance(r, torch.Tensor) else Flux2VAEStage.preprocess_image(r) for r in reference_images]
            toks = [self.vae_stage.process("encode_image", r) for r in refs]
            image_latents = torch.cat(toks, dim=1).repeat(batch, 1, 1)
            image_ids = reference_image_ids([(r.shape[-2] // 16, r.shape[-1] // 16) for r in refs])
        out = self.denoise_stage.process(pack_latents(noise), pos, pos_ids, cfg_scale, num_inference_steps, ids, neg, neg_ids,
                                         image_latents, image_ids)  # fmt: skip
        out = out() if callable(out) else out
        if output_type == "latent" or self.vae_stage is None:
            return out
        image = self.vae_stage.process("decode_latents", out, ids)
        return image if output_type == "pt" else self.vae_output_to_images(image)
