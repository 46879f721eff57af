"""LingBot-Video generation: text (+ first frame) -> video with the dense or MoE transformer, and the
low-noise refiner pass.

Stages: text encoding (an injected callable / stage returning `(embeddings [1, L, 2560], mask)`; prompt
embeddings can also be passed in directly), denoising (`LingBotVideoDenoisingStage`: flow-matching Euler
steps with classifier-free guidance evaluated sequentially, batched in one forward, or split over a
CFG-parallel pair; first-frame conditioning is re-injected before every step), Wan VAE encode / decode.
The denoising stage wires Ulysses sequence parallelism and expert parallelism from the mesh.
`refine()` re-noises an up-sampled video to `t_thresh` and denoises the low-noise tail only.
Role parity: telefuser/pipelines/lingbot_video/{pipeline,denoising,refiner,data}.py.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import numpy as np
import torch

from telefuser_b200.core.base_pipeline import BasePipeline
from telefuser_b200.core.base_stage import BaseStage, with_model_offload
from telefuser_b200.core.config import ModelRuntimeConfig
from telefuser_b200.ops import functional as TF
from telefuser_b200.parallel import mesh as pmesh
from telefuser_b200.parallel import shard as pshard
from telefuser_b200.schedulers.flow_match import FlowMatchScheduler

from .data import DEFAULT_NEGATIVE_PROMPT, default_negative_caption  # noqa: F401 (re-exported)


@dataclass
class LingBotVideoPipelineConfig:
    text_encoding_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    dit_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    vae_config: ModelRuntimeConfig = field(default_factory=ModelRuntimeConfig)
    guidance_scale: float = 3.0
    num_inference_steps: int = 50
    shift: float = 3.0
    batch_cfg: bool = False
    enable_denoising_parallel: bool = False
    enable_expert_parallel: bool = False

    def __post_init__(self) -> None:
        if self.guidance_scale < 0 or self.num_inference_steps <= 0 or self.shift <= 0:
            raise ValueError("guidance_scale must be non-negative; steps and shift must be positive")


@dataclass
class LingBotVideoRequest:
    caption: str = ""
    num_frames: int = 81
    height: int = 480
    width: int = 832
    image: torch.Tensor | None = None  # [1, 3, H, W] (or [1, 3, T, H, W]) in [-1, 1] for TI2V
    seed: int = 0


@dataclass
class LingBotVideoGeneration:
    output: torch.Tensor
    prompt_conditions: dict


def validate_frame_count(num_frames: int) -> int:
    if num_frames != 1 and (num_frames - 1) % 4:
        raise ValueError(f"num_frames must be 1 or 4n+1, got {num_frames}")
    return num_frames


def latent_shape(num_frames: int, height: int, width: int) -> tuple[int, int, int]:
    validate_frame_count(num_frames)
    if height % 16 or width % 16:
        raise ValueError("height and width must be multiples of 16")
    return (num_frames - 1) // 4 + 1, height // 8, width // 8


def reinject_ti2v_condition(latent, condition, mask):
    """Replaces the conditioned temporal prefix (mask over frames) with the clean condition latent."""
    if condition.shape[2] > latent.shape[2] or latent.shape[:2] != condition.shape[:2]:
        raise ValueError("condition must match the latent's batch / channels and be no longer in time")
    if condition.shape != latent.shape:
        n = condition.shape[2]
        if mask.ndim != 1 or not bool(mask[:n].all()) or bool(mask[n:].any()):
            raise ValueError("a prefix condition needs a prefix-only temporal mask")
        out = latent.clone()
        out[:, :, :n] = condition.to(latent.dtype)
        return out
    m = mask.to(device=latent.device, dtype=torch.bool)
    if m.ndim == 1:
        m = m.reshape(1, 1, -1, 1, 1)
    return torch.where(m, condition.to(latent.dtype), latent)


def transformer_timestep(timestep: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """sigma is rounded to the transformer dtype before the time embedding, as the public sampler does."""
    sigma = timestep.float() / 1000.0
    if dtype in (torch.bfloat16, torch.float16):
        sigma = sigma.to(dtype)
    return (sigma * 1000.0).float()


def compute_refiner_sigmas(sigma_max: float, sigma_min: float, num_inference_steps: int, shift: float,
                           t_thresh: float | None, tail_steps: int = 0):  # fmt: skip
    """Descending sigmas of the low-noise refiner pass: the shifted `num_inference_steps`-step schedule restricted to
    sigma <= `t_thresh` (with `t_thresh` itself put in front when the schedule does not hit it), followed by `tail_steps`
    extra, evenly spaced sigmas between the last one and `sigma_min`. None when no threshold is given (full schedule)."""
    if t_thresh is None:
        return None
    if not (0 < t_thresh <= 1 and num_inference_steps >= 1 and tail_steps >= 0):
        raise ValueError(f"refiner schedule: t_thresh in (0, 1], steps >= 1, tail_steps >= 0; got {t_thresh}, "
                         f"{num_inference_steps}, {tail_steps}")  # fmt: skip
    grid = np.linspace(sigma_max, sigma_min, num_inference_steps + 1)[:-1]
    grid = shift * grid / (1.0 + (shift - 1.0) * grid)
    kept = grid[grid <= t_thresh + 1e-6]
    if kept.size == 0 or abs(float(kept[0]) - t_thresh) > 1e-6:
        kept = np.concatenate([[t_thresh], kept])
    if tail_steps:
        last = float(kept[-1])
        kept = np.concatenate([kept, np.linspace(last, min(sigma_min, last), tail_steps + 2)[1:-1]])
    ok = np.all(np.isfinite(kept)) and kept.min() >= 0 and kept.max() <= 1 and np.all(np.diff(kept) < 0)
    if not ok:
        raise ValueError(f"refiner schedule is not a finite, strictly descending sequence in [0, 1]: {kept.tolist()}")
    return kept.astype(np.float32)


def prepare_refiner_latent(x_up, noise, t_thresh):
    th = torch.as_tensor(t_thresh, device=x_up.device, dtype=x_up.dtype)
    while th.ndim < x_up.ndim:
        th = th.unsqueeze(-1)
    return (1.0 - th) * x_up + th * noise


def batch_cfg_prompt_inputs(pos, neg, pos_mask, neg_mask):
    """Pads the two prompts to one length and stacks them for a single batched forward."""
    def pad(e, m, n):
        if m is None:
            m = torch.ones(e.shape[:2], dtype=torch.bool, device=e.device)
        p = n - e.shape[1]
        if p:
            e, m = torch.nn.functional.pad(e, (0, 0, 0, p)), torch.nn.functional.pad(m, (0, p), value=False)
        return e, m

    n = max(pos.shape[1], neg.shape[1])
    (pe, pm), (ne, nm) = pad(pos, pos_mask, n), pad(neg, neg_mask, n)
    return torch.cat((pe, ne)), torch.cat((pm, nm))


class LingBotVideoDenoisingStage(BaseStage):
    def __init__(self, name: str, module_manager: Any, config: ModelRuntimeConfig, dit=None, batch_cfg: bool = False,
                 expert_parallel: bool = False) -> None:  # fmt: skip
        super().__init__(name, config)
        self.dit = dit
        if dit is None:
            self.dit = (module_manager.fetch_module("lingbot_video_moe_transformer")
                        or module_manager.fetch_module("lingbot_video_transformer"))  # fmt: skip
        self.model_names = ["dit"]
        self.batch_cfg, self.expert_parallel = batch_cfg, expert_parallel
        self.mesh = pmesh.get_mesh()
        self.scheduler = FlowMatchScheduler("Wan")

    def parallel_models(self) -> None:
        cfg = self.model_runtime_config.parallel_config
        self.mesh = pmesh.create_device_mesh_from_config(cfg)
        self.dit.device_mesh = self.mesh
        if cfg.sp_ulysses_degree > 1:
            self.dit.set_ulysses_group(self.mesh.group("ulysses"))
        if self.expert_parallel or cfg.ep_degree > 1:
            self.dit.enable_expert_parallel(self.mesh.group("ep") or self.mesh.group("ulysses"))
        if cfg.enable_fsdp:
            from telefuser_b200.parallel.fsdp import shard_model

            shard_model(self.dit, self.device, wrap_module_names=self.dit.get_fsdp_module_names())

    def predict_noise_with_cfg(self, latent, timestep, pos, neg, pos_mask, neg_mask, guidance_scale: float):
        """Returns (cond, uncond); uncond is None without guidance."""
        x = latent.to(self.torch_dtype)
        t = transformer_timestep(timestep, self.torch_dtype)
        use_cfg = guidance_scale > 1.0 and neg is not None
        if use_cfg and self.mesh.size("cfg") == 2:
            mine = (pos, pos_mask) if self.mesh.coord("cfg") == 0 else (neg, neg_mask)
            return pshard.cfg_parallel_unshard(self.dit(x, t, *mine), self.mesh)
        if use_cfg and self.batch_cfg:
            emb, mask = batch_cfg_prompt_inputs(pos, neg, pos_mask, neg_mask)
            both = self.dit(x.repeat(2, 1, 1, 1, 1), t.repeat(2), emb, mask)
            return both[:1], both[1:]
        cond = self.dit(x, t, pos, pos_mask)
        return cond, (self.dit(x, t, neg, neg_mask) if use_cfg else None)

    @with_model_offload(["dit"])
    @torch.no_grad()
    def denoise(self, latent, pos, neg, pos_mask, neg_mask, guidance_scale: float, num_inference_steps: int,
                shift: float, condition=None, condition_mask=None, sigmas=None):  # fmt: skip
        """latent fp32 [1, C, F, H, W] -> denoised latent. `sigmas`: explicit descending schedule (refiner)."""
        latent = latent.to(self.device, torch.float32)
        if sigmas is None:
            self.scheduler.set_timesteps(num_inference_steps, shift=shift)
            sig = self.scheduler.sigmas.tolist()
        else:
            sig = [float(s) for s in sigmas]
        sig = sig + [0.0] if len(sig) == num_inference_steps or sigmas is not None else sig
        for i in range(len(sig) - 1):
            if condition is not None:
                latent = reinject_ti2v_condition(latent, condition.to(latent), condition_mask)
            t = torch.full((latent.shape[0],), sig[i] * 1000.0, device=self.device)
            cond, uncond = self.predict_noise_with_cfg(latent, t, pos, neg, pos_mask, neg_mask, guidance_scale)
            latent = TF.cfg_euler_step(latent, cond, uncond, guidance_scale, sig[i + 1] - sig[i])
        if condition is not None:
            latent = reinject_ti2v_condition(latent, condition.to(latent), condition_mask)
        return latent


class LingBotVideoPipeline(BasePipeline):
    def __init__(self, device="cuda", torch_dtype=torch.bfloat16) -> None:
        super().__init__(device=device, torch_dtype=torch_dtype)
        self.text_stage: Callable | None = None

    def _get_stages(self) -> list:
        return [s for s in (self.denoising_stage, getattr(self, "vae_stage", None)) if s is not None]

    def init(self, module_manager, config: LingBotVideoPipelineConfig, text_stage: Callable | None = None):
        from telefuser_b200.worker.parallel_worker import ParallelWorker

        self.config = config
        self.text_stage = text_stage
        self.denoising_stage = LingBotVideoDenoisingStage("denoise", module_manager, config.dit_config,
                                                          batch_cfg=config.batch_cfg,
                                                          expert_parallel=config.enable_expert_parallel)  # fmt: skip
        self.denoising_stage.onload_models_flag = True
        self.in_channels = self.denoising_stage.dit.config.in_channels
        if config.enable_denoising_parallel:
            self.denoising_stage = ParallelWorker(self.denoising_stage)
        self.vae_stage = None
        if module_manager.fetch_module("wan_video_vae") is not None:
            from telefuser_b200.pipelines.wan.stages import VAEStage

            self.vae_stage = VAEStage("vae", module_manager, config.vae_config)
            self.vae_stage.onload_models_flag = True

    @classmethod
    def from_pretrained(cls, model_id_or_path: str, device="cuda", torch_dtype=torch.bfloat16, cache_dir=None,
                        parallel_devices=None, cfg_degree=None, sp_ulysses_degree=None, expert_parallel: bool = False,
                        quant_config=None, **kwargs):  # fmt: skip
        """LingBot-Video (dense or MoE, told apart by the checkpoint keys) from a model folder or hub id:
        `transformer/`, `vae/` (Wan 16-channel VAE) and `text_encoder/` + `processor/` (Qwen3-VL, loaded through
        transformers). Keyword arguments that name a field of `LingBotVideoPipelineConfig` set it."""
        import os

        from telefuser_b200.core.module_manager import ModuleManager
        from telefuser_b200.models.wan_vae import WanVideoVAE
        from telefuser_b200.utils.hf import resolve_hf_path
        from telefuser_b200.utils.hf_model_analyzer import HFModelAnalyzer

        from .text_encoding import LingBotVideoTextEncodingStage

        root = resolve_hf_path(model_id_or_path, cache_dir)
        found = HFModelAnalyzer(root)
        dit_path = found.get_transformer_path()
        if not dit_path:
            raise FileNotFoundError(f"{root} has no transformer weights; found {sorted(found.analyze())}")
        mm = ModuleManager(torch_dtype=torch_dtype, device=str(device))
        if not mm.load_model(dit_path, quant_config=quant_config):  # the registry tells dense from MoE by the keys
            raise ValueError(f"{dit_path}: not a LingBot-Video transformer checkpoint")
        if found.get_vae_path():
            mm.load_model(found.get_vae_path(), model_class=WanVideoVAE, name="wan_video_vae")
        config = LingBotVideoPipelineConfig(**{k: v for k, v in kwargs.items() if k in LingBotVideoPipelineConfig.__dataclass_fields__})
        for c in (config.dit_config, config.vae_config):
            c.torch_dtype, c.device_type = torch_dtype, torch.device(device).type
            c.device_id = torch.device(device).index or 0
        if parallel_devices and len(parallel_devices) > 1:
            n = len(parallel_devices)
            pc = config.dit_config.parallel_config
            pc.device_ids = list(parallel_devices)
            pc.cfg_degree = cfg_degree or (2 if n % 2 == 0 else 1)
            pc.sp_ulysses_degree = sp_ulysses_degree or n // pc.cfg_degree
            if expert_parallel:
                pc.ep_degree = n
            config.enable_denoising_parallel = True
            config.enable_expert_parallel = expert_parallel
        text_stage = None
        enc_dir = found.component_folder("text_encoder")
        proc_dir = found.component_folder("processor") or os.path.join(root, "processor")
        if enc_dir and os.path.isdir(proc_dir):
            from transformers import AutoModelForImageTextToText, AutoProcessor

            mm.load_from_huggingface(enc_dir, "text_encoder", AutoModelForImageTextToText, torch_dtype=torch_dtype, device=device)
            mm.add_module(AutoProcessor.from_pretrained(proc_dir), "processor", path=proc_dir)
            text_stage = LingBotVideoTextEncodingStage("text_encoding", mm, config.dit_config)
        pipe = cls(device=device, torch_dtype=torch_dtype)
        pipe.init(mm, config, text_stage=text_stage)
        return pipe

    def _encode_text(self, caption: str):
        if self.text_stage is None:
            raise RuntimeError("no text stage configured: pass prompt embeddings to generate()")
        out = self.text_stage(caption)
        return out if isinstance(out, tuple) else (out, None)

    @torch.no_grad()
    def generate(self, request: LingBotVideoRequest, negative_caption: str | None = None, prompt_embeds=None,
                 negative_prompt_embeds=None, prompt_mask=None, negative_prompt_mask=None, decode: bool = True):  # fmt: skip
        cfg = self.config
        frames, lh, lw = latent_shape(request.num_frames, request.height, request.width)
        if request.image is not None and request.num_frames == 1:
            raise ValueError("image conditioning continues a video from its first frame; a one-frame request has nothing to generate")
        pos, pos_mask = (prompt_embeds, prompt_mask) if prompt_embeds is not None else self._encode_text(request.caption)
        neg = neg_mask = None
        if cfg.guidance_scale > 1.0:
            if negative_prompt_embeds is not None:
                neg, neg_mask = negative_prompt_embeds, negative_prompt_mask
            else:
                neg, neg_mask = self._encode_text(negative_caption or default_negative_caption(request.num_frames))
        condition = mask = None
        if request.image is not None:
            if self.vae_stage is None:
                raise ValueError("image conditioning needs a VAE")
            img = request.image if request.image.ndim == 5 else request.image.unsqueeze(2)
            condition = self.vae_stage.process("encode_video", img[:, :, :1].to(self.device)).float()
            mask = torch.zeros(frames, dtype=torch.bool, device=self.device)
            mask[: condition.shape[2]] = True
        gen = torch.Generator(device="cpu").manual_seed(request.seed)
        latent = torch.randn(1, self.in_channels, frames, lh, lw, generator=gen).to(self.device)
        dev = self.device
        args = (latent, pos.to(dev, self.torch_dtype), None if neg is None else neg.to(dev, self.torch_dtype),
                None if pos_mask is None else pos_mask.to(dev), None if neg_mask is None else neg_mask.to(dev),
                cfg.guidance_scale, cfg.num_inference_steps, cfg.shift, condition, mask)  # fmt: skip
        out = self.denoising_stage.denoise(*args)
        out = out() if callable(out) else out
        cond = {"positive_prompt_embeds": pos, "negative_prompt_embeds": neg, "has_visual_condition": condition is not None}
        if not decode:
            return LingBotVideoGeneration(out, cond)
        if self.vae_stage is None:
            raise RuntimeError("decode=True needs a VAE")
        return LingBotVideoGeneration(self.vae_stage.process("decode_video", out.to(self.torch_dtype)), cond)

    __call__ = generate

    @torch.no_grad()
    def refine(self, video_latent_up, prompt_embeds, negative_prompt_embeds=None, t_thresh: float = 0.3,
               num_inference_steps: int = 50, shift: float | None = None, tail_steps: int = 0, seed: int = 0,
               guidance_scale: float | None = None):  # fmt: skip
        """Refiner pass on an up-sampled latent: noise to `t_thresh`, denoise only the sigmas below it."""
        cfg = self.config
        sig = compute_refiner_sigmas(1.0, 0.0, num_inference_steps, shift or cfg.shift, t_thresh, tail_steps)
        gen = torch.Generator(device="cpu").manual_seed(seed)
        x = video_latent_up.to(self.device, torch.float32)
        noise = torch.randn(x.shape, generator=gen).to(self.device)
        latent = prepare_refiner_latent(x, noise, float(sig[0]))
        g = cfg.guidance_scale if guidance_scale is None else guidance_scale
        dev = self.device
        neg = None if negative_prompt_embeds is None else negative_prompt_embeds.to(dev, self.torch_dtype)
        out = self.denoising_stage.denoise(latent, prompt_embeds.to(dev, self.torch_dtype), neg, None, None, g, len(sig),
                                           cfg.shift, None, None, sig)  # fmt: skip
        return out() if callable(out) else out
