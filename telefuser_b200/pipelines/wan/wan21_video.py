"""Wan2.1 video pipeline (T2V / I2V / FLF2V).

    pipe = Wan21VideoPipeline.from_pretrained(model_id_or_path=..., device="cuda", torch_dtype=torch.bfloat16)
    frames = pipe(prompt, num_frames=81, height=480, width=832)

Stages: text encoding (UMT5) -> [CLIP + VAE image conditioning] -> denoising loop -> VAE decode.
The denoising and VAE stages can each run as a `ParallelWorker` rank group
(`enable_denoising_parallel`, `enable_vae_parallel`). `from_random_init` builds the same
pipeline with random weights of a named architecture for benchmarks and tests without
checkpoints. Role parity: telefuser/pipelines/wan_video/wan21_video.py:27-353.
"""

from __future__ import annotations

import glob
import os
from dataclasses import dataclass, field

import torch

from telefuser_b200.core.base_pipeline import BasePipeline
from telefuser_b200.core.config import (AttentionConfig, AttnImplType, ModelRuntimeConfig, OffloadConfig, ParallelConfig,
                                        WeightOffloadType)  # fmt: skip
from telefuser_b200.core.module_manager import ModuleManager
from telefuser_b200.schedulers.flow_match import FlowMatchScheduler
from telefuser_b200.utils.func import auto_async_call
from telefuser_b200.utils.logging import logger
from telefuser_b200.worker.parallel_worker import ParallelWorker

from .denoising import WanDenoisingStage
from .stages import ClipEncodingStage, TextEncodingStage, VAEStage


@dataclass
class Wan21VideoPipelineConfig:
    vae_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    dit_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    clip_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    text_encoding_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    vfi_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    sample_solver: str = "euler"
    enable_clip_stage: bool = False
    enable_denoising_parallel: bool = False
    enable_vae_parallel: bool = False
    enable_vfi: bool = False
    enable_metrics: bool = False


def discover_wan_components(root: str) -> dict[str, str | list[str]]:
    """Finds the component files of a Wan checkpoint folder (official or diffusers layout)."""
    found: dict[str, str | list[str]] = {}

    def first(*patterns):
        for p in patterns:
            hits = sorted(glob.glob(os.path.join(root, p), recursive=True))
            if hits:
                return hits
        return []

    dit = first("diffusion_pytorch_model*.safetensors", "transformer/diffusion_pytorch_model*.safetensors",
                "*dit*.safetensors", "*.safetensors")  # fmt: skip
    if dit:
        found["dit"] = dit if len(dit) > 1 else dit[0]
    t5 = first("models_t5_umt5-xxl-enc-bf16.pth", "*t5*.pth", "*umt5*.safetensors", "text_encoder/*.safetensors")
    if t5:
        found["text_encoder"] = t5[0]
    vae = first("Wan2.1_VAE.pth", "*VAE*.pth", "*vae*.safetensors", "vae/*.safetensors")
    if vae:
        found["vae"] = vae[0]
    clip = first("models_clip_open-clip-xlm-roberta-large-vit-huge-14.pth", "*clip*.pth", "image_encoder/*.safetensors")
    if clip:
        found["clip"] = clip[0]
    return found


class Wan21VideoPipeline(BasePipeline):
    def __init__(self, device: str | torch.device = "cuda", torch_dtype: torch.dtype = torch.bfloat16) -> None:
        super().__init__(device=device, torch_dtype=torch_dtype)
        self.height_division_factor = 16
        self.width_division_factor = 16
        self.base_fps = 16

    def _get_stages(self) -> list:
        stages = [self.vae_stage, self.denoise_stage, self.text_encoding_stage]
        if hasattr(self, "clip_stage"):
            stages.append(self.clip_stage)
        return stages

    def init(self, module_manager: ModuleManager, config: Wan21VideoPipelineConfig, text_stage=None):
        self._model_info = module_manager.get_model_info()
        self.config = config
        self.vae_stage = VAEStage("vae", module_manager, config.vae_config)
        if config.enable_clip_stage:
            self.clip_stage = ClipEncodingStage("clip", module_manager, config.clip_config)
        if config.sample_solver == "euler":
            self.scheduler = FlowMatchScheduler(template="Wan")
        elif config.sample_solver == "unipc":
            from telefuser_b200.schedulers.unipc import FlowUniPCMultistepScheduler

            self.scheduler = FlowUniPCMultistepScheduler(num_train_timesteps=1000, shift=1, use_dynamic_shifting=False)
        else:
            raise NotImplementedError(f"solver {config.sample_solver} is not supported")
        self.denoise_stage = WanDenoisingStage("denoise", module_manager, config.dit_config, self.scheduler)
        self.text_encoding_stage = text_stage or TextEncodingStage("text_encoding", module_manager,
                                                                   config.text_encoding_config)  # fmt: skip
        if config.enable_denoising_parallel:
            self.denoise_stage = ParallelWorker(self.denoise_stage)
        if config.enable_vae_parallel:
            self.vae_stage = ParallelWorker(self.vae_stage)
        if config.enable_metrics:
            self.enable_metrics()

    # ---- public pieces (also used by benchmarks) -----------------------------------
    def encode_prompts(self, prompt: str, negative_prompt: str, cfg_scale: float):
        prompts = [prompt] + ([negative_prompt] if cfg_scale != 1.0 else [])
        embs = auto_async_call(self.text_encoding_stage.process, prompts)()
        return embs[0], (embs[1] if cfg_scale != 1.0 else None)

    def denoise(self, latents, num_inference_steps, prompt_emb_posi, prompt_emb_nega, cfg_scale=5.0, sigma_shift=5.0,
                ref_latent=None, clip_context=None):  # fmt: skip
        return auto_async_call(self.denoise_stage.process, latents, num_inference_steps, ref_latent, prompt_emb_posi,
                               prompt_emb_nega, clip_context, cfg_scale, sigma_shift)()  # fmt: skip

    def decode(self, latents, **tiler_kwargs):
        return auto_async_call(self.vae_stage.process, "decode_video", latents, **tiler_kwargs)()

    @torch.no_grad()
    def __call__(self, prompt, negative_prompt="", input_image=None, end_image=None, seed=None, rand_device=None,
                 height=480, width=832, num_frames=81, cfg_scale=5.0, num_inference_steps=50, sigma_shift=5.0,
                 tiled=False, tile_size=(30, 52), tile_stride=(15, 26), target_fps=None, output_type="pil"):  # fmt: skip
        height, width = self.check_resize_height_width(height, width)
        if num_frames % 4 != 1:
            num_frames = (num_frames + 2) // 4 * 4 + 1
            logger.warning(f"num_frames must be 4n+1; rounded to {num_frames}")
        tiler = {"tiled": tiled, "tile_size": tile_size, "tile_stride": tile_stride}
        noise = self.generate_noise((1, 16, (num_frames - 1) // 4 + 1, height // 8, width // 8), seed=seed,
                                    device=rand_device or "cpu", dtype=torch.float32)  # fmt: skip
        posi, nega = self.encode_prompts(prompt, negative_prompt, cfg_scale)
        ref_latent = clip_context = None
        if input_image is not None:
            img = self.preprocess_image(input_image, height, width)
            end = self.preprocess_image(end_image, height, width) if end_image is not None else None
            ref_wait = auto_async_call(self.vae_stage.process, "encode_image", img, end, num_frames, **tiler)
            if hasattr(self, "clip_stage"):
                clip_context = auto_async_call(self.clip_stage.process, img, end)()
            ref_latent = ref_wait()
        latents = self.denoise(noise.to(self.device), num_inference_steps, posi, nega, cfg_scale, sigma_shift,
                               ref_latent, clip_context)  # fmt: skip
        frames = self.decode(latents, **tiler)
        if output_type == "pt":
            return frames
        return self.tensor2video(frames[0])

    def close(self) -> None:
        for st in (getattr(self, "denoise_stage", None), getattr(self, "vae_stage", None)):
            if isinstance(st, ParallelWorker):
                st.close()

    # ---- constructors ------------------------------------------------------------------
    @staticmethod
    def _runtime_configs(device, torch_dtype, parallel_devices, attn_impl, offload_type, sp_ulysses_degree=None,
                         cfg_degree=1):  # fmt: skip
        dev = torch.device(device)
        base = dict(device_type=dev.type, device_id=dev.index or 0, torch_dtype=torch_dtype)
        off = OffloadConfig(offload_type=offload_type or WeightOffloadType.NO_CPU_OFFLOAD)
        pc = ParallelConfig()
        if parallel_devices:
            n = len(parallel_devices)
            u = sp_ulysses_degree or max(1, n // cfg_degree)
            pc = ParallelConfig(device_ids=list(parallel_devices), cfg_degree=cfg_degree, sp_ulysses_degree=u)
        attn = AttentionConfig.dense_attention(attn_impl or AttnImplType.TCGEN05)
        dit = ModelRuntimeConfig(offload_config=off, attention_config=attn, parallel_config=pc, **base)
        other = lambda: ModelRuntimeConfig(offload_config=off, **base)  # noqa: E731
        return Wan21VideoPipelineConfig(vae_config=other(), dit_config=dit, clip_config=other(),
                                        text_encoding_config=other(), enable_denoising_parallel=bool(parallel_devices))  # fmt: skip

    @classmethod
    def from_pretrained(cls, model_id_or_path: str, device="cuda", torch_dtype=torch.bfloat16, parallel_devices=None,
                        attn_impl=None, offload_type=None, sample_solver="euler", **kwargs):  # fmt: skip
        from telefuser_b200.utils.hf import resolve_hf_path

        root = resolve_hf_path(model_id_or_path)
        comps = discover_wan_components(root)
        if "dit" not in comps or "vae" not in comps or "text_encoder" not in comps:
            raise FileNotFoundError(f"{root} lacks a Wan component (found {sorted(comps)})")
        load_dev = "cpu" if offload_type not in (None, WeightOffloadType.NO_CPU_OFFLOAD) else str(device)
        mm = ModuleManager(torch_dtype=torch_dtype, device=load_dev)
        from telefuser_b200.models.umt5 import WanTextEncoder
        from telefuser_b200.models.wan_dit import WanModel
        from telefuser_b200.models.wan_vae import WanVideoVAE

        mm.load_model(comps["dit"], model_class=WanModel, name="wan_video_dit",
                      model_resource="diffusers" if "transformer" in str(comps["dit"]) else "official")  # fmt: skip
        mm.load_model(comps["vae"], model_class=WanVideoVAE, name="wan_video_vae")
        mm.load_model(comps["text_encoder"], model_class=WanTextEncoder, name="wan_video_text_encoder")
        config = cls._runtime_configs(device, torch_dtype, parallel_devices, attn_impl, offload_type,
                                      kwargs.get("sp_ulysses_degree"), kwargs.get("cfg_degree", 1))  # fmt: skip
        config.sample_solver = sample_solver
        if "clip" in comps and mm.fetch_module("wan_video_dit").has_image_input:
            from telefuser_b200.models.wan_image_encoder import WanImageEncoder

            mm.load_model(comps["clip"], model_class=WanImageEncoder, name="wan_video_image_encoder")
            config.enable_clip_stage = True
        pipe = cls(device=device, torch_dtype=torch_dtype)
        pipe.init(mm, config)
        return pipe

    @classmethod
    def from_random_init(cls, preset="wan2.1-t2v-1.3b", device="cuda", torch_dtype=torch.bfloat16, parallel_devices=None,
                         text_encoder_layers: int = 2, seed: int = 0, vae_dim: int | None = None, **kwargs):  # fmt: skip
        """Random weights of the named DiT architecture, the real VAE architecture (`vae_dim`: a narrower one for CPU
        tests) and a short UMT5 stack."""
        from telefuser_b200.models.umt5 import WanTextEncoder
        from telefuser_b200.models.wan_dit import WanModel, WanModelConfig
        from telefuser_b200.models.wan_vae import WanVideoVAE
        from telefuser_b200.testing.synthetic import HashTokenizer, random_init_

        torch.manual_seed(seed)
        cfgm = WanModelConfig.preset(preset) if isinstance(preset, str) else preset
        with torch.device("meta"):
            dit = WanModel.from_config(cfgm)
            te = WanTextEncoder(vocab=4096, dim=cfgm.text_dim, dim_attn=cfgm.text_dim, dim_ffn=cfgm.text_dim * 2,
                                num_heads=max(1, cfgm.text_dim // 64), num_layers=text_encoder_layers)  # fmt: skip
        dit = random_init_(dit.to_empty(device=device).to(torch_dtype), seed)
        te = random_init_(te.to_empty(device=device).to(torch_dtype), seed + 1)
        vae = random_init_((WanVideoVAE() if vae_dim is None else WanVideoVAE(dim=vae_dim)).to(device=device, dtype=torch_dtype),
                           seed + 2, std=0.03)  # fmt: skip
        mm = ModuleManager(torch_dtype=torch_dtype, device=str(device))
        mm.add_module(dit.eval(), "wan_video_dit")
        mm.add_module(vae.eval(), "wan_video_vae")
        mm.add_module(te.eval(), "wan_video_text_encoder")
        config = cls._runtime_configs(device, torch_dtype, parallel_devices, None, None,
                                      kwargs.get("sp_ulysses_degree"), kwargs.get("cfg_degree", 1))  # fmt: skip
        pipe = cls(device=device, torch_dtype=torch_dtype)
        text_stage = TextEncodingStage("text_encoding", mm, config.text_encoding_config, text_encoder=te,
                                       tokenizer=HashTokenizer(4096, 512))  # fmt: skip
        pipe.init(mm, config, text_stage=text_stage)
        return pipe
