"""Wan2.2 pipelines: the A14B text/image-to-video pipeline with two expert DiTs and the 5B TI2V pipeline.

`Wan22VideoPipeline`: UMT5 text encoding -> [VAE image conditioning, mask-concatenated as in Wan2.1 I2V] ->
`MoeDitDenoisingStage` (high-noise / low-noise expert, own guidance scales, optional latent-cache hand-off)
-> 16-channel VAE decode. Solvers: euler, unipc, mix-euler (separate step counts and shifts per expert).
`Wan22TI2VPipeline`: one 5B DiT on the 48-channel VAE (stride 4 x 16 x 16); a reference image replaces the
first latent frame and is marked clean with per-token timesteps (`TI2VDenoisingStage`).
Role parity: telefuser/pipelines/wan_video/{wan22_video,wan22_ti2v}.py.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from telefuser_b200.core.base_pipeline import BasePipeline
from telefuser_b200.core.config import ModelRuntimeConfig
from telefuser_b200.core.module_manager import ModuleManager
from telefuser_b200.schedulers.flow_match import FlowMatchScheduler
from telefuser_b200.utils.func import auto_async_call
from telefuser_b200.utils.logging import logger
from telefuser_b200.worker.parallel_worker import ParallelWorker

from .moe_dit_denoising import MoeDitDenoisingStage
from .stages import TextEncodingStage, VAEStage
from .ti2v_denoising import TI2VDenoisingStage


def _scheduler(solver: str):
    if solver == "euler":
        return FlowMatchScheduler(template="Wan")
    if solver == "mix-euler":
        return FlowMatchScheduler(template="Wan-Mix")
    if solver == "unipc":
        from telefuser_b200.schedulers.unipc import FlowUniPCMultistepScheduler

        return FlowUniPCMultistepScheduler(num_train_timesteps=1000, shift=1, use_dynamic_shifting=False)
    raise NotImplementedError(f"solver {solver} is not supported")


def _round_frames(num_frames: int) -> int:
    if num_frames % 4 != 1:
        num_frames = (num_frames + 2) // 4 * 4 + 1
        logger.warning(f"num_frames must be 4n+1; rounded to {num_frames}")
    return num_frames


def _load_wan_components(model_id_or_path, torch_dtype, offload, *, experts: int, vae_class, vae_name: str, cache_dir=None):
    """Resolves a Wan2.2 model folder (official or diffusers layout) and loads its DiT(s), VAE and UMT5 encoder
    into a ModuleManager. Returns (module manager, tokenizer folder or None)."""
    from telefuser_b200.models.umt5 import WanTextEncoder
    from telefuser_b200.models.wan_dit import WanModel
    from telefuser_b200.utils.hf import resolve_hf_path
    from telefuser_b200.utils.hf_model_analyzer import HFModelAnalyzer

    root = resolve_hf_path(model_id_or_path, cache_dir)
    found = HFModelAnalyzer(root)
    comps = found.analyze()
    dits = [found.get_transformer_path()] + ([found.get_transformer_2_path()] if experts == 2 else [])
    missing = [n for n, v in (("a DiT", dits[0]), ("the second (low-noise) DiT", dits[-1]), ("a VAE", found.get_vae_path()),
                              ("a text encoder", found.get_text_encoder_path())) if not v]  # fmt: skip
    if missing:
        raise FileNotFoundError(f"{root} lacks {', '.join(missing)}; found {sorted(comps)}")
    mm = ModuleManager(torch_dtype=torch_dtype, device="cpu" if offload else None)
    for role, path in zip(("transformer", "transformer_2"), dits):  # high-noise expert first
        diffusers = (comps[role].class_name or "").endswith("Transformer3DModel")
        mm.load_model(path, model_class=WanModel, name="wan_video_dit", model_resource="diffusers" if diffusers else "official")
    mm.load_model(found.get_vae_path(), model_class=vae_class, name=vae_name)
    mm.load_model(found.get_text_encoder_path(), model_class=WanTextEncoder, name="wan_video_text_encoder")
    logger.info(f"loaded {root}:\n{found.describe()}")
    return mm, found.get_tokenizer_path()


def _text_stage(mm, config, tokenizer_dir):
    """A diffusers folder keeps the tokenizer in its own sub-folder; the official layout keeps it beside the
    encoder file (`google/umt5-xxl`), which the stage finds by itself."""
    if tokenizer_dir is None:
        return None
    from telefuser_b200.models.umt5 import HuggingfaceTokenizer

    return TextEncodingStage("text_encoding", mm, config, tokenizer=HuggingfaceTokenizer(tokenizer_dir, 512, "whitespace"))


def _apply_parallel(configs, parallel_devices, sp_ulysses_degree, cfg_degree) -> bool:
    if not parallel_devices or len(parallel_devices) < 2:
        return False
    n = len(parallel_devices)
    cfg_degree = cfg_degree or (2 if n % 2 == 0 and n >= 4 else 1)
    for c in configs:
        c.parallel_config.device_ids = list(parallel_devices)
        c.parallel_config.cfg_degree = cfg_degree
        c.parallel_config.sp_ulysses_degree = sp_ulysses_degree or n // cfg_degree
    return True


@dataclass
class Wan22VideoPipelineConfig:
    vae_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    dit_high_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    dit_low_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    text_encoding_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    vfi_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    sample_solver: str = "euler"
    enable_denoising_parallel: bool = False
    enable_vae_parallel: bool = False
    enable_vfi: bool = False
    enable_metrics: bool = False


class Wan22VideoPipeline(BasePipeline):
    def __init__(self, device="cuda", torch_dtype=torch.bfloat16) -> None:
        super().__init__(device=device, torch_dtype=torch_dtype)
        self.height_division_factor = self.width_division_factor = 16
        self.base_fps = 16

    def _get_stages(self) -> list:
        return [self.vae_stage, self.denoise_stage, self.text_encoding_stage]

    def init(self, module_manager: ModuleManager, config: Wan22VideoPipelineConfig, text_stage=None):
        self._model_info = module_manager.get_model_info()
        self.config = config
        self.vae_stage = VAEStage("vae", module_manager, config.vae_config)
        self.scheduler = _scheduler(config.sample_solver)
        self.denoise_stage = MoeDitDenoisingStage("denoise", module_manager, config.dit_high_config, config.dit_low_config,
                                                  self.scheduler)  # fmt: skip
        self.text_encoding_stage = text_stage or TextEncodingStage("text_encoding", module_manager, config.text_encoding_config)
        if config.enable_vfi:
            from telefuser_b200.pipelines.common.vfi import RiftVFIStage

            self.vfi_stage = RiftVFIStage("vfi", module_manager, config.vfi_config)
        if config.enable_vae_parallel:
            self.vae_stage = ParallelWorker(self.vae_stage)
        if config.enable_denoising_parallel:
            self.denoise_stage = ParallelWorker(self.denoise_stage)
        if config.enable_metrics:
            self.enable_metrics()

    @torch.no_grad()
    def __call__(self, prompt, negative_prompt="", input_image=None, end_image=None, seed=None, rand_device=None, height=480,
                 width=832, num_frames=81, num_inference_steps=50, sigma_shift=5.0, tiled=False, tile_size=(30, 52),
                 tile_stride=(15, 26), cfg_scale_high=5.0, cfg_scale_low=5.0, boundary=0.875, target_fps=None,
                 latent_data: dict | None = None, output_type="pil"):  # fmt: skip
        height, width = self.check_resize_height_width(height, width)
        num_frames = _round_frames(num_frames)
        tiler = {"tiled": tiled, "tile_size": tile_size, "tile_stride": tile_stride}
        noise = self.generate_noise((1, 16, (num_frames - 1) // 4 + 1, height // 8, width // 8), seed=seed,
                                    device=rand_device or "cpu", dtype=torch.float32)  # fmt: skip
        prompts = [prompt] + ([negative_prompt] if cfg_scale_high != 1.0 else [])
        embs_wait = auto_async_call(self.text_encoding_stage.process, prompts)
        ref_latent = None
        if input_image is not None:
            img = self.preprocess_image(input_image, height, width)
            end = self.preprocess_image(end_image, height, width) if end_image is not None else None
            ref_latent = auto_async_call(self.vae_stage.process, "encode_image", img, end, num_frames, **tiler)()
        embs = embs_wait()
        posi, nega = embs[0], (embs[1] if cfg_scale_high != 1.0 else None)
        result = auto_async_call(self.denoise_stage.process, noise.to(self.device), num_inference_steps, ref_latent, posi, nega,
                                 cfg_scale_high, cfg_scale_low, sigma_shift, boundary, latent_data=latent_data)()  # fmt: skip
        latents, payload = result if isinstance(result, tuple) else (result, None)
        frames = auto_async_call(self.vae_stage.process, "decode_video", latents, **tiler)()
        out = frames if output_type == "pt" else self.tensor2video(frames[0])
        if getattr(self, "vfi_stage", None) is not None and target_fps is not None and output_type != "pt":
            out = auto_async_call(self.vfi_stage.process, out, self.base_fps, target_fps)()
        if payload is not None:
            payload["num_frames"] = num_frames
            return out, payload
        return out

    @classmethod
    def from_pretrained(cls, model_id_or_path: str, device="cuda", torch_dtype=torch.bfloat16, cache_dir=None,
                        attention_config=None, parallel_devices=None, sample_solver="euler", offload_type=None,
                        enable_metrics=False, sp_ulysses_degree=None, cfg_degree=None, **kwargs):  # fmt: skip
        """Wan2.2 A14B from a model folder or hub id: `high_noise_model/` + `low_noise_model/` (official) or
        `transformer/` + `transformer_2/` (diffusers), the 16-channel VAE and the UMT5 encoder. Keyword arguments
        that name a field of `Wan22VideoPipelineConfig` set it. Loader of telefuser/pipelines/wan_video/wan22_video.py:220."""
        from telefuser_b200.core.config import WeightOffloadType
        from telefuser_b200.models.wan_vae import WanVideoVAE

        offload = offload_type not in (None, WeightOffloadType.NO_CPU_OFFLOAD)
        mm, tokenizer_dir = _load_wan_components(model_id_or_path, torch_dtype, offload, experts=2, vae_class=WanVideoVAE,
                                                 vae_name="wan_video_vae", cache_dir=cache_dir)  # fmt: skip
        config = Wan22VideoPipelineConfig(sample_solver=sample_solver, enable_metrics=enable_metrics)
        runtime = (config.vae_config, config.dit_high_config, config.dit_low_config, config.text_encoding_config)
        for c in runtime:
            c.torch_dtype, c.device_type = torch_dtype, torch.device(device).type
            c.device_id = torch.device(device).index or 0
            if offload:
                c.offload_config.offload_type = offload_type
        if attention_config is not None:
            config.dit_high_config.attention_config = config.dit_low_config.attention_config = attention_config
        config.enable_denoising_parallel = _apply_parallel((config.dit_high_config, config.dit_low_config), parallel_devices,
                                                           sp_ulysses_degree, cfg_degree)  # fmt: skip
        for k, v in kwargs.items():
            if hasattr(config, k):
                setattr(config, k, v)
        pipe = cls(device=device, torch_dtype=torch_dtype)
        pipe.init(mm, config, text_stage=_text_stage(mm, config.text_encoding_config, tokenizer_dir))
        return pipe

    def close(self) -> None:
        for st in (getattr(self, "denoise_stage", None), getattr(self, "vae_stage", None)):
            if isinstance(st, ParallelWorker):
                st.close()


@dataclass
class Wan22TI2VPipelineConfig:
    vae_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    dit_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    text_encoding_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    sample_solver: str = "euler"
    enable_denoising_parallel: bool = False
    enable_vae_parallel: bool = False
    enable_metrics: bool = False


class Wan22TI2VPipeline(BasePipeline):
    def __init__(self, device="cuda", torch_dtype=torch.bfloat16) -> None:
        super().__init__(device=device, torch_dtype=torch_dtype)
        self.height_division_factor = self.width_division_factor = 32
        self.base_fps = 24
        self.z_dim = 48

    def _get_stages(self) -> list:
        return [self.vae_stage, self.denoise_stage, self.text_encoding_stage]

    def init(self, module_manager: ModuleManager, config: Wan22TI2VPipelineConfig, text_stage=None):
        self._model_info = module_manager.get_model_info()
        self.config = config
        vae = module_manager.fetch_module("wan22_video_vae") or module_manager.fetch_module("wan_video_vae")
        self.vae_stage = VAEStage("vae", module_manager, config.vae_config, vae=vae)
        self.z_dim = vae.z_dim
        self.scheduler = _scheduler(config.sample_solver)
        self.denoise_stage = TI2VDenoisingStage("denoise", module_manager, config.dit_config, self.scheduler)
        self.text_encoding_stage = text_stage or TextEncodingStage("text_encoding", module_manager, config.text_encoding_config)
        if config.enable_vae_parallel:
            self.vae_stage = ParallelWorker(self.vae_stage)
        if config.enable_denoising_parallel:
            self.denoise_stage = ParallelWorker(self.denoise_stage)
        if config.enable_metrics:
            self.enable_metrics()

    @torch.no_grad()
    def __call__(self, prompt, negative_prompt="", input_image=None, end_image=None, seed=None, rand_device=None, height=704,
                 width=1280, num_frames=121, cfg_scale=5.0, num_inference_steps=50, sigma_shift=5.0, tiled=False,
                 tile_size=(30, 52), tile_stride=(15, 26), output_type="pil"):  # fmt: skip
        height, width = self.check_resize_height_width(height, width)
        num_frames = _round_frames(num_frames)
        tiler = {"tiled": tiled, "tile_size": tile_size, "tile_stride": tile_stride}
        f = self.vae_stage.vae.upsampling_factor if hasattr(self.vae_stage, "vae") else 16
        noise = self.generate_noise((1, self.z_dim, (num_frames - 1) // 4 + 1, height // f, width // f), seed=seed,
                                    device=rand_device or "cpu", dtype=torch.float32)  # fmt: skip
        prompts = [prompt] + ([negative_prompt] if cfg_scale != 1.0 else [])
        embs_wait = auto_async_call(self.text_encoding_stage.process, prompts)
        ref_latent = ref_mask = None
        if input_image is not None:
            img = self.preprocess_image(input_image, height, width)
            end = self.preprocess_image(end_image, height, width) if end_image is not None else None
            ref_latent, ref_mask = auto_async_call(self.vae_stage.process, "encode_image", img, end, num_frames,
                                                   concat_mask=False, **tiler)()  # fmt: skip
        embs = embs_wait()
        posi, nega = embs[0], (embs[1] if cfg_scale != 1.0 else None)
        latents = auto_async_call(self.denoise_stage.process, noise.to(self.device), num_inference_steps, ref_latent, ref_mask,
                                  posi, nega, cfg_scale, sigma_shift)()  # fmt: skip
        frames = auto_async_call(self.vae_stage.process, "decode_video", latents, **tiler)()
        return frames if output_type == "pt" else self.tensor2video(frames[0])

    @classmethod
    def from_pretrained(cls, model_id_or_path: str, device="cuda", torch_dtype=torch.bfloat16, cache_dir=None,
                        attention_config=None, parallel_devices=None, sample_solver="euler", offload_type=None,
                        enable_metrics=False, sp_ulysses_degree=None, cfg_degree=None, **kwargs):  # fmt: skip
        """Wan2.2 TI2V 5B from a model folder or hub id: one DiT, the 48-channel VAE (`Wan2.2_VAE.pth` or `vae/`)
        and the UMT5 encoder. Loader of telefuser/pipelines/wan_video/wan22_ti2v.py:276."""
        from telefuser_b200.core.config import WeightOffloadType
        from telefuser_b200.models.wan22_vae import Wan22VideoVAE

        offload = offload_type not in (None, WeightOffloadType.NO_CPU_OFFLOAD)
        mm, tokenizer_dir = _load_wan_components(model_id_or_path, torch_dtype, offload, experts=1, vae_class=Wan22VideoVAE,
                                                 vae_name="wan22_video_vae", cache_dir=cache_dir)  # fmt: skip
        config = Wan22TI2VPipelineConfig(sample_solver=sample_solver, enable_metrics=enable_metrics)
        for c in (config.vae_config, config.dit_config, config.text_encoding_config):
            c.torch_dtype, c.device_type = torch_dtype, torch.device(device).type
            c.device_id = torch.device(device).index or 0
            if offload:
                c.offload_config.offload_type = offload_type
        if attention_config is not None:
            config.dit_config.attention_config = attention_config
        config.enable_denoising_parallel = _apply_parallel((config.dit_config,), parallel_devices, sp_ulysses_degree, cfg_degree)
        for k, v in kwargs.items():
            if hasattr(config, k):
                setattr(config, k, v)
        pipe = cls(device=device, torch_dtype=torch_dtype)
        pipe.init(mm, config, text_stage=_text_stage(mm, config.text_encoding_config, tokenizer_dir))
        return pipe

    def close(self) -> None:
        for st in (getattr(self, "denoise_stage", None), getattr(self, "vae_stage", None)):
            if isinstance(st, ParallelWorker):
                st.close()
