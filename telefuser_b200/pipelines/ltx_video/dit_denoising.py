"""LTX-2 joint audio-video denoising: token layouts, conditioning, multi-modal guidance, the denoising loop.

Video latents [B, 128, F, H, W] become one token per latent voxel whose rotary position is the pixel-space box
it covers (time in seconds, first frame causal); audio latents [B, 8, T, 16] become one token per latent frame
positioned by the seconds it spans. A `LatentState` carries tokens, the per-token denoise mask (1 = free, 0 =
clamped to the clean latent), positions and an optional token-to-token attention mask for appended keyframes.
Each step runs the x0 model up to four times (prompt, negative prompt, self-attention skipped in chosen blocks,
audio<->video attention skipped) and combines the results per modality; the Euler update then works on x0.
Role parity: telefuser/pipelines/ltx_video/dit_denoising.py:25-1010.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field, replace
from typing import Any, NamedTuple

import torch

from telefuser_b200.core.base_stage import BaseStage, with_model_offload
from telefuser_b200.core.config import ModelRuntimeConfig
from telefuser_b200.models.ltx_dit import (
    BatchedPerturbationConfig,
    Modality,
    Perturbation,
    PerturbationConfig,
    PerturbationType,
)
from telefuser_b200.models.ltx_video_vae import (
    VIDEO_LATENT_CHANNELS,
    VIDEO_SCALE_FACTORS,
    SpatioTemporalScaleFactors,
    VideoLatentShape,
)
from telefuser_b200.schedulers.flow_match import FlowMatchScheduler

STAGE_2_DISTILLED_SIGMA_VALUES = [0.909375, 0.725, 0.421875, 0.0]


class AudioLatentShape(NamedTuple):
    batch: int
    channels: int
    frames: int
    mel_bins: int

    def to_torch_shape(self) -> torch.Size:
        return torch.Size(self)

    def token_count(self) -> int:
        return self.frames

    def mask_shape(self) -> "AudioLatentShape":
        return AudioLatentShape(self.batch, 1, self.frames, 1)

    @staticmethod
    def from_duration(batch: int, duration: float, channels: int = 8, mel_bins: int = 16, sample_rate: int = 16000,
                      hop_length: int = 160, audio_latent_downsample_factor: int = 4) -> "AudioLatentShape":  # fmt: skip
        per_second = float(sample_rate) / float(hop_length) / float(audio_latent_downsample_factor)
        return AudioLatentShape(batch, channels, round(duration * per_second), mel_bins)


@dataclass(frozen=True)
class LatentState:
    latent: torch.Tensor
    denoise_mask: torch.Tensor
    positions: torch.Tensor
    clean_latent: torch.Tensor
    attention_mask: torch.Tensor | None = None

    def clone(self) -> "LatentState":
        return LatentState(self.latent.clone(), self.denoise_mask.clone(), self.positions.clone(), self.clean_latent.clone(),
                           None if self.attention_mask is None else self.attention_mask.clone())  # fmt: skip


class VideoLatentPatchifier:
    def __init__(self, patch_size: int = 1) -> None:
        self.patch_size = (1, patch_size, patch_size)

    def get_token_count(self, shape: VideoLatentShape) -> int:
        return shape.frames * shape.height * shape.width // math.prod(self.patch_size)

    def patchify(self, x: torch.Tensor) -> torch.Tensor:
        B, C, F_, H, W = x.shape
        _, p, q = self.patch_size
        x = x.reshape(B, C, F_, H // p, p, W // q, q).permute(0, 2, 3, 5, 1, 4, 6)
        return x.reshape(B, F_ * (H // p) * (W // q), C * p * q)

    def unpatchify(self, tokens: torch.Tensor, shape: VideoLatentShape) -> torch.Tensor:
        _, p, q = self.patch_size
        B, f, h, w = tokens.shape[0], shape.frames, shape.height // p, shape.width // q
        x = tokens.reshape(B, f, h, w, -1, p, q).permute(0, 4, 1, 2, 5, 3, 6)
        return x.reshape(B, -1, f, h * p, w * q)

    def get_patch_grid_bounds(self, shape: VideoLatentShape, device=None) -> torch.Tensor:
        """-> [B, 3, tokens, 2]: start / end of every patch on the latent (frame, row, column) axes."""
        axes = [torch.arange(0, n, s, device=device) for n, s in zip((shape.frames, shape.height, shape.width), self.patch_size)]
        starts = torch.stack(torch.meshgrid(*axes, indexing="ij"), dim=0)
        ends = starts + torch.tensor(self.patch_size, device=device).view(3, 1, 1, 1)
        return torch.stack((starts, ends), dim=-1).flatten(1, 3)[None].repeat(shape.batch, 1, 1, 1)


class AudioPatchifier:
    """One token per `patch_size` latent frames; positions are the seconds covered (causal first frame)."""

    def __init__(self, patch_size: int = 1, sample_rate: int = 16000, hop_length: int = 160, downsample: int = 4,
                 is_causal: bool = True, shift: int = 0) -> None:  # fmt: skip
        self.patch_size = (patch_size, 1, 1)
        self.sample_rate, self.hop_length, self.audio_latent_downsample_factor = sample_rate, hop_length, downsample
        self.is_causal, self.shift = is_causal, shift

    def get_token_count(self, shape: AudioLatentShape) -> int:
        return shape.frames // self.patch_size[0]

    def patchify(self, x: torch.Tensor) -> torch.Tensor:
        B, C, T, M = x.shape
        p = self.patch_size[0]
        return x.reshape(B, C, T // p, p, M).permute(0, 2, 1, 3, 4).reshape(B, T // p, C * p * M)

    def unpatchify(self, tokens: torch.Tensor, shape: AudioLatentShape) -> torch.Tensor:
        B, T, p = tokens.shape[0], tokens.shape[1], self.patch_size[0]
        return tokens.reshape(B, T, shape.channels, p, shape.mel_bins).permute(0, 2, 1, 3, 4).reshape(B, shape.channels, T * p,
                                                                                                       shape.mel_bins)  # fmt: skip

    def get_patch_grid_bounds(self, shape: AudioLatentShape, device=None) -> torch.Tensor:
        idx = torch.arange(self.shift, shape.frames + self.shift, dtype=torch.float32, device=device or "cpu")
        d = float(self.audio_latent_downsample_factor)
        mel = torch.stack([idx * d, (idx + 1) * d], dim=-1)
        if self.is_causal:
            mel = (mel + 1.0 - d).clamp_min(0.0)
        seconds = mel * float(self.hop_length) / float(self.sample_rate)
        return seconds[None, None].expand(shape.batch, 1, -1, 2).contiguous()


def get_pixel_coords(latent_coords: torch.Tensor, scale: SpatioTemporalScaleFactors, causal_fix: bool = False) -> torch.Tensor:
    px = latent_coords.clone()
    for axis, s in enumerate(scale):
        px[:, axis] *= s
    if causal_fix:
        px[:, 0] = (px[:, 0] - (scale.time - 1)).clamp_min(0)
    return px


@dataclass(frozen=True)
class LatentTools:
    patchifier: Any
    target_shape: Any

    def patchify(self, s: LatentState) -> LatentState:
        p = self.patchifier.patchify
        return replace(s.clone(), latent=p(s.latent), denoise_mask=p(s.denoise_mask), clean_latent=p(s.clean_latent))

    def unpatchify(self, s: LatentState) -> LatentState:
        u = self.patchifier.unpatchify
        return replace(s.clone(), latent=u(s.latent, self.target_shape), denoise_mask=u(s.denoise_mask, self.target_shape.mask_shape()),
                       clean_latent=u(s.clean_latent, self.target_shape))  # fmt: skip

    def clear_conditioning(self, s: LatentState) -> LatentState:
        """Drop appended conditioning tokens and open every mask."""
        n = self.patchifier.get_token_count(self.target_shape)
        return LatentState(s.latent[:, :n], torch.ones_like(s.denoise_mask)[:, :n], s.positions[:, :, :n], s.clean_latent[:, :n], None)

    def _positions(self, device) -> torch.Tensor:
        raise NotImplementedError

    def create_initial_state(self, device, dtype, initial_latent: torch.Tensor | None = None) -> LatentState:
        shape = self.target_shape.to_torch_shape()
        latent = torch.zeros(*shape, device=device, dtype=dtype) if initial_latent is None else initial_latent.to(device, dtype)
        mask = torch.ones(*self.target_shape.mask_shape().to_torch_shape(), device=device, dtype=torch.float32)
        return self.patchify(LatentState(latent, mask, self._positions(device).to(dtype), latent.clone()))


@dataclass(frozen=True)
class VideoLatentTools(LatentTools):
    fps: float = 24.0
    scale_factors: SpatioTemporalScaleFactors = VIDEO_SCALE_FACTORS
    causal_fix: bool = True

    def _positions(self, device) -> torch.Tensor:
        pos = get_pixel_coords(self.patchifier.get_patch_grid_bounds(self.target_shape, device), self.scale_factors, self.causal_fix).float()
        pos[:, 0] /= self.fps
        return pos


@dataclass(frozen=True)
class AudioLatentTools(LatentTools):
    def _positions(self, device) -> torch.Tensor:
        return self.patchifier.get_patch_grid_bounds(self.target_shape, device)


# ---- conditioning --------------------------------------------------------------------------
class ConditioningError(RuntimeError):
    pass


def resolve_cross_mask(attention_mask, num_new_tokens: int, batch_size: int, device, dtype) -> torch.Tensor:
    if isinstance(attention_mask, (int, float)):
        return torch.full((batch_size, num_new_tokens), float(attention_mask), device=device, dtype=dtype)
    if attention_mask.ndim == 1:
        return attention_mask[None].expand(batch_size, -1).to(device=device, dtype=dtype)
    if attention_mask.ndim == 2:
        return attention_mask.to(device=device, dtype=dtype)
    raise ValueError(f"unsupported attention mask shape {tuple(attention_mask.shape)}")


def build_attention_mask(existing_mask, num_noisy_tokens: int, num_new_tokens: int, num_existing_tokens: int, cross_mask, device,
                         dtype) -> torch.Tensor:  # fmt: skip
    """[B, total, total] weights in [0, 1]: old block kept, new tokens see each other, new <-> noisy by `cross_mask`;
    earlier conditioning tokens and the new ones do not see each other."""
    total = num_existing_tokens + num_new_tokens
    m = torch.zeros((cross_mask.shape[0], total, total), device=device, dtype=dtype)
    m[:, :num_existing_tokens, :num_existing_tokens] = 1.0 if existing_mask is None else existing_mask
    m[:, num_existing_tokens:, num_existing_tokens:] = 1.0
    m[:, :num_noisy_tokens, num_existing_tokens:] = cross_mask.unsqueeze(1)
    m[:, num_existing_tokens:, :num_noisy_tokens] = cross_mask.unsqueeze(2)
    return m


def update_attention_mask(latent_state: LatentState, attention_mask, num_noisy_tokens: int, num_new_tokens: int, batch_size: int,
                          device, dtype):  # fmt: skip
    if attention_mask is None:
        if latent_state.attention_mask is None:
            return None
        cross = torch.ones(batch_size, num_new_tokens, device=device, dtype=dtype)
    else:
        cross = resolve_cross_mask(attention_mask, num_new_tokens, batch_size, device, dtype)
    return build_attention_mask(latent_state.attention_mask, num_noisy_tokens, num_new_tokens, latent_state.latent.shape[1], cross,
                                device, dtype)  # fmt: skip


class VideoConditionByLatentIndex:
    """Overwrite the tokens of latent frame `latent_idx` onward with an encoded clip; strength 1 freezes them."""

    def __init__(self, latent: torch.Tensor, strength: float, latent_idx: int) -> None:
        self.latent, self.strength, self.latent_idx = latent, strength, latent_idx

    def apply_to(self, latent_state: LatentState, latent_tools: LatentTools) -> LatentState:
        tgt = latent_tools.target_shape
        b, c, _, h, w = self.latent.shape
        if (b, c, h, w) != (tgt.batch, tgt.channels, tgt.height, tgt.width):
            raise ConditioningError(f"conditioning latent {tuple(self.latent.shape)} does not fit the target {tuple(tgt)}")
        tokens = latent_tools.patchifier.patchify(self.latent)
        start = latent_tools.patchifier.get_token_count(tgt._replace(frames=self.latent_idx))
        s = latent_state.clone()
        s.latent[:, start : start + tokens.shape[1]] = tokens
        s.clean_latent[:, start : start + tokens.shape[1]] = tokens
        s.denoise_mask[:, start : start + tokens.shape[1]] = 1.0 - self.strength
        return s


class VideoConditionByKeyframeIndex:
    """Append encoded keyframes as extra tokens positioned at pixel frame `frame_idx`."""

    def __init__(self, keyframes: torch.Tensor, frame_idx: int, strength: float) -> None:
        self.keyframes, self.frame_idx, self.strength = keyframes, frame_idx, strength

    def apply_to(self, latent_state: LatentState, latent_tools: VideoLatentTools) -> LatentState:
        k = self.keyframes
        tokens = latent_tools.patchifier.patchify(k)
        bounds = latent_tools.patchifier.get_patch_grid_bounds(VideoLatentShape.from_torch_shape(k.shape), k.device)
        pos = get_pixel_coords(bounds, latent_tools.scale_factors, latent_tools.causal_fix if self.frame_idx == 0 else False).float()
        pos[:, 0] = (pos[:, 0] + self.frame_idx) / latent_tools.fps
        mask = torch.full((*tokens.shape[:2], 1), 1.0 - self.strength, device=k.device, dtype=k.dtype)
        return LatentState(
            latent=torch.cat([latent_state.latent, tokens], dim=1),
            denoise_mask=torch.cat([latent_state.denoise_mask, mask.to(latent_state.denoise_mask.dtype)], dim=1),
            positions=torch.cat([latent_state.positions, pos.to(latent_state.positions.dtype)], dim=2),
            clean_latent=torch.cat([latent_state.clean_latent, tokens], dim=1),
            attention_mask=update_attention_mask(latent_state, None, latent_tools.target_shape.token_count(), tokens.shape[1],
                                                 tokens.shape[0], k.device, k.dtype))  # fmt: skip


class ConditioningItemAttentionStrengthWrapper:
    """Weights how strongly the tokens appended by `conditioning` and the noisy tokens attend to each other."""

    def __init__(self, conditioning, attention_mask) -> None:
        self.conditioning, self.attention_mask = conditioning, attention_mask

    def apply_to(self, latent_state: LatentState, latent_tools: LatentTools) -> LatentState:
        new = self.conditioning.apply_to(latent_state, latent_tools)
        added = new.latent.shape[1] - latent_state.latent.shape[1]
        if added == 0:
            return new
        return replace(new, attention_mask=update_attention_mask(latent_state, self.attention_mask, latent_tools.target_shape.token_count(),
                                                                 added, new.latent.shape[0], new.latent.device, new.latent.dtype))  # fmt: skip


# ---- guidance --------------------------------------------------------------------------------
@dataclass(frozen=True)
class MultiModalGuiderParams:
    cfg_scale: float = 1.0
    stg_scale: float = 0.0
    stg_blocks: list | None = field(default_factory=list)
    rescale_scale: float = 0.0
    modality_scale: float = 1.0
    skip_step: int = 0


@dataclass(frozen=True)
class MultiModalGuider:
    params: MultiModalGuiderParams
    negative_context: torch.Tensor | None = None

    def calculate(self, cond, uncond_text, uncond_perturbed, uncond_modality):
        p = self.params
        pred = (cond + (p.cfg_scale - 1) * (cond - uncond_text) + p.stg_scale * (cond - uncond_perturbed)
                + (p.modality_scale - 1) * (cond - uncond_modality))  # fmt: skip
        if p.rescale_scale != 0:
            pred = pred * (p.rescale_scale * (cond.std() / pred.std()) + (1 - p.rescale_scale))
        return pred

    def do_unconditional_generation(self) -> bool:
        return not math.isclose(self.params.cfg_scale, 1.0)

    def do_perturbed_generation(self) -> bool:
        return not math.isclose(self.params.stg_scale, 0.0)

    def do_isolated_modality_generation(self) -> bool:
        return not math.isclose(self.params.modality_scale, 1.0)

    def should_skip_step(self, step_index: int) -> bool:
        return self.params.skip_step != 0 and step_index % (self.params.skip_step + 1) != 0


class GaussianNoiser:
    def __init__(self, noise: torch.Tensor) -> None:
        self.noise = noise

    def __call__(self, s: LatentState, noise_scale: float = 1.0) -> LatentState:
        noise = self.noise.to(device=s.latent.device, dtype=s.latent.dtype)
        if noise.shape != s.latent.shape:
            raise ValueError(f"noise shape {tuple(noise.shape)} does not match latent shape {tuple(s.latent.shape)}")
        m = s.denoise_mask.to(s.latent.dtype) * noise_scale
        return replace(s, latent=noise * m + s.latent * (1 - m))


def resolve_context(context) -> tuple[torch.Tensor, torch.Tensor]:
    """(video encoding, audio encoding) from a dict, an object with those attributes, or a sequence."""
    if isinstance(context, dict):
        v, a = context.get("video_encoding"), context.get("audio_encoding")
    elif hasattr(context, "video_encoding") and hasattr(context, "audio_encoding"):
        v, a = context.video_encoding, context.audio_encoding
    elif isinstance(context, (list, tuple)) and len(context) >= 2:
        v, a = context[0], context[1]
    else:
        raise TypeError(f"unsupported context {type(context)!r}")
    if not isinstance(v, torch.Tensor) or not isinstance(a, torch.Tensor):
        raise TypeError("video_encoding and audio_encoding must be tensors")
    return v, a


def _skip(kind: PerturbationType, blocks) -> Perturbation:
    return Perturbation(kind, blocks)


class DitDenoisingStage(BaseStage):
    def __init__(self, name: str, module_manager: Any, config: ModelRuntimeConfig, model_name: str = "ltx_dit", scheduler=None,
                 dit=None, batched_guidance: bool = False) -> None:  # fmt: skip
        super().__init__(name, config)
        self.dit = dit if dit is not None else module_manager.fetch_module(model_name)
        self.model_names = ["dit"]
        self.scheduler = scheduler or FlowMatchScheduler(template="LTX.2")
        self.flow_match_scheduler = FlowMatchScheduler(template="LTX.2")
        self.video_patchifier, self.audio_patchifier = VideoLatentPatchifier(1), AudioPatchifier(1)
        self.forward_calls = 0
        self._lora_applied = False
        # run the guidance passes of a step (prompt, negative prompt, perturbed, modality-isolated) as one batch of up to four
        self.batched_guidance = batched_guidance

    def _maybe_apply_loras(self) -> None:
        """Merges the stage's configured LoRA files into the velocity model once (stage 2 usually carries the distilled LoRA)."""
        if self._lora_applied:
            return
        self._lora_applied = True
        configs = getattr(self.model_runtime_config, "lora_configs", None) or []
        if not configs:
            return
        from telefuser_b200.utils.lora import LoRALoader

        target, loader = getattr(self.dit, "velocity_model", self.dit), LoRALoader()
        for cfg in configs:
            loader.apply_lora(target, cfg.path, strength=cfg.strength)

    def _x0(self, video: Modality, audio: Modality, perturbations=None):
        self.forward_calls += 1
        return self.dit(video, audio, perturbations, x0=True)

    def _prepare_schedule(self, num_inference_steps: int, sigmas, initial_video_latent):
        if sigmas is None:
            self.flow_match_scheduler.set_timesteps(num_inference_steps=num_inference_steps, latent=initial_video_latent)
            sigmas = self.flow_match_scheduler.sigmas
        sigmas = torch.as_tensor(sigmas).to(dtype=torch.float32, device=self.device)
        timesteps = (sigmas[:-1] * self.scheduler.num_train_timesteps).to(dtype=torch.float32, device="cpu")
        self.scheduler.sigmas, self.scheduler.timesteps = sigmas.cpu(), timesteps
        return sigmas, timesteps

    @staticmethod
    def _modality(state: LatentState, context: torch.Tensor, sigma: torch.Tensor, enabled: bool = True) -> Modality:
        return Modality(latent=state.latent, sigma=sigma.reshape(1).expand(state.latent.shape[0]), timesteps=state.denoise_mask * sigma,
                        positions=state.positions, context=context, enabled=enabled, context_mask=None,
                        attention_mask=state.attention_mask)  # fmt: skip

    @staticmethod
    def _stack(m: Modality, contexts: list) -> Modality:
        """One sample -> a batch with one entry per context (same latents, positions and timesteps)."""
        n = len(contexts)
        rep = lambda t: None if t is None else t.repeat(n, *([1] * (t.dim() - 1)))  # noqa: E731
        return Modality(latent=rep(m.latent), sigma=m.sigma.reshape(-1)[:1].expand(n), timesteps=rep(m.timesteps), positions=rep(m.positions),
                        context=torch.cat(contexts, dim=0), enabled=m.enabled, context_mask=None, attention_mask=rep(m.attention_mask))  # fmt: skip

    def _build_denoise_fn(self, positive_context, negative_context, video_params: MultiModalGuiderParams,
                          audio_params: MultiModalGuiderParams, simple_denoise: bool):  # fmt: skip
        pos_v, pos_a = resolve_context(positive_context)
        neg_v, neg_a = resolve_context(negative_context) if negative_context is not None else (None, None)
        if simple_denoise:
            return lambda vs, as_, sigmas, i: self._x0(self._modality(vs, pos_v, sigmas[i]), self._modality(as_, pos_a, sigmas[i]))
        vg, ag = MultiModalGuider(video_params, neg_v), MultiModalGuider(audio_params, neg_a)
        last: list = [None, None]
        P = PerturbationType

        def step(vs: LatentState, as_: LatentState, sigmas: torch.Tensor, i: int):
            skip_v, skip_a = vg.should_skip_step(i), ag.should_skip_step(i)
            if skip_v and skip_a:
                return last[0], last[1]
            sigma = sigmas[i]
            video, audio = self._modality(vs, pos_v, sigma, not skip_v), self._modality(as_, pos_a, sigma, not skip_a)
            if self.batched_guidance and vs.latent.shape[0] == 1 and not (skip_v or skip_a):
                passes = [("cond", pos_v, pos_a, PerturbationConfig.empty())]
                if vg.do_unconditional_generation() or ag.do_unconditional_generation():
                    passes.append(("neg", pos_v if neg_v is None else neg_v, pos_a if neg_a is None else neg_a, PerturbationConfig.empty()))
                if vg.do_perturbed_generation() or ag.do_perturbed_generation():
                    items = ([_skip(P.SKIP_VIDEO_SELF_ATTN, video_params.stg_blocks)] if vg.do_perturbed_generation() else []) + (
                        [_skip(P.SKIP_AUDIO_SELF_ATTN, audio_params.stg_blocks)] if ag.do_perturbed_generation() else [])  # fmt: skip
                    passes.append(("ptb", pos_v, pos_a, PerturbationConfig(items)))
                if vg.do_isolated_modality_generation() or ag.do_isolated_modality_generation():
                    passes.append(("mod", pos_v, pos_a, PerturbationConfig([_skip(P.SKIP_A2V_CROSS_ATTN, None), _skip(P.SKIP_V2A_CROSS_ATTN, None)])))
                out_v, out_a = self._x0(self._stack(video, [p[1] for p in passes]), self._stack(audio, [p[2] for p in passes]),
                                        BatchedPerturbationConfig([p[3] for p in passes]))  # fmt: skip
                got = {p[0]: (out_v[i : i + 1], out_a[i : i + 1]) for i, p in enumerate(passes)}
                zero = (0.0, 0.0)
                last[0] = vg.calculate(got["cond"][0], got.get("neg", zero)[0], got.get("ptb", zero)[0], got.get("mod", zero)[0])
                last[1] = ag.calculate(got["cond"][1], got.get("neg", zero)[1], got.get("ptb", zero)[1], got.get("mod", zero)[1])
                return last[0], last[1]
            cond_v, cond_a = self._x0(video, audio)
            neg = ptb = mod = (0.0, 0.0)
            if vg.do_unconditional_generation() or ag.do_unconditional_generation():
                neg = self._x0(self._modality(vs, pos_v if neg_v is None else neg_v, sigma),
                               self._modality(as_, pos_a if neg_a is None else neg_a, sigma))  # fmt: skip
            if vg.do_perturbed_generation() or ag.do_perturbed_generation():
                items = ([_skip(P.SKIP_VIDEO_SELF_ATTN, video_params.stg_blocks)] if vg.do_perturbed_generation() else []) + (
                    [_skip(P.SKIP_AUDIO_SELF_ATTN, audio_params.stg_blocks)] if ag.do_perturbed_generation() else [])  # fmt: skip
                ptb = self._x0(video, audio, BatchedPerturbationConfig([PerturbationConfig(items)] * vs.latent.shape[0]))
            if vg.do_isolated_modality_generation() or ag.do_isolated_modality_generation():
                items = [_skip(P.SKIP_A2V_CROSS_ATTN, None), _skip(P.SKIP_V2A_CROSS_ATTN, None)]
                mod = self._x0(video, audio, BatchedPerturbationConfig([PerturbationConfig(items)] * vs.latent.shape[0]))
            last[0] = last[0] if skip_v else vg.calculate(cond_v, neg[0], ptb[0], mod[0])
            last[1] = last[1] if skip_a else ag.calculate(cond_a, neg[1], ptb[1], mod[1])
            return last[0], last[1]

        return step

    def _apply_conditioning_latents(self, s: LatentState, tools: VideoLatentTools, cond: torch.Tensor) -> LatentState:
        """`cond` [B, 1 + C, F_cond, H, W]: a per-voxel denoise mask then clean latents; voxels with mask < 1 are applied."""
        if cond.ndim != 5 or cond.shape[1] != 1 + VIDEO_LATENT_CHANNELS:
            raise ValueError(f"expected conditioning [B, {1 + VIDEO_LATENT_CHANNELS}, F, H, W], got {tuple(cond.shape)}")
        cond = cond.to(device=self.device, dtype=self.torch_dtype)
        tgt = tools.target_shape
        if cond.shape[0] != s.latent.shape[0] or tuple(cond.shape[3:]) != (tgt.height, tgt.width) or cond.shape[2] > tgt.frames:
            raise ValueError(f"conditioning {tuple(cond.shape)} does not fit the target latent {tuple(tgt)}")
        if cond.shape[2] == 0:
            return s
        mask = tools.patchifier.patchify(cond[:, :1]).float()
        tokens = tools.patchifier.patchify(cond[:, 1:])
        n = tokens.shape[1]
        update = mask < 1.0
        if not bool(update.any()):
            return s
        s = s.clone()
        s.latent[:, :n] = torch.where(update, tokens, s.latent[:, :n])
        s.clean_latent[:, :n] = torch.where(update, tokens, s.clean_latent[:, :n])
        s.denoise_mask[:, :n] = torch.where(update, mask.to(s.denoise_mask.dtype), s.denoise_mask[:, :n])
        return s

    def _create_initial_states(self, height, width, num_frames, frame_rate, conditionings, video_noiser, audio_noiser, noise_scale,
                               initial_video_latent, initial_audio_latent, batch: int = 1):  # fmt: skip
        vtools = VideoLatentTools(self.video_patchifier, VideoLatentShape.from_pixels(batch, num_frames, height, width), fps=frame_rate)
        vs = vtools.create_initial_state(self.device, self.torch_dtype, initial_video_latent)
        if isinstance(conditionings, torch.Tensor):
            vs = self._apply_conditioning_latents(vs, vtools, conditionings)
        else:
            for item in conditionings or []:
                vs = item.apply_to(latent_state=vs, latent_tools=vtools)
        vs = video_noiser(vs, noise_scale)
        atools = AudioLatentTools(self.audio_patchifier, AudioLatentShape.from_duration(batch, float(num_frames) / float(frame_rate)))
        as_ = audio_noiser(atools.create_initial_state(self.device, self.torch_dtype, initial_audio_latent), noise_scale)
        return vs, as_, vtools, atools

    def _denoise(self, vs: LatentState, as_: LatentState, sigmas, timesteps, denoise_fn):
        for i, t in enumerate(timesteps):
            den_v, den_a = denoise_fn(vs, as_, sigmas, i)
            den_v = (den_v * vs.denoise_mask + vs.clean_latent.float() * (1 - vs.denoise_mask)).to(den_v.dtype)
            den_a = (den_a * as_.denoise_mask + as_.clean_latent.float() * (1 - as_.denoise_mask)).to(den_a.dtype)
            final = i + 1 >= len(timesteps)
            if hasattr(self.scheduler, "template"):
                nv = self.scheduler.step(den_v, t, vs.latent, to_final=final)
                na = self.scheduler.step(den_a, t, as_.latent, to_final=final)
            else:  # multistep solvers predicting x0
                nv, na = (self.scheduler.step(d, t, s.latent, return_dict=False) for d, s in ((den_v, vs), (den_a, as_)))
                nv, na = (x[0] if isinstance(x, tuple) else x for x in (nv, na))
            vs, as_ = replace(vs, latent=nv), replace(as_, latent=na)
        return vs, as_

    @with_model_offload(["dit"])
    @torch.no_grad()
    def process(self, height: int, width: int, num_frames: int, frame_rate: float, conditionings, positive_context, negative_context,
                num_inference_steps: int, video_guider_params: MultiModalGuiderParams, audio_guider_params: MultiModalGuiderParams,
                video_noise: torch.Tensor, audio_noise: torch.Tensor, initial_video_latent=None, initial_audio_latent=None, sigmas=None,
                noise_scale: float = 1.0, simple_denoise: bool = False):  # fmt: skip
        """-> (video LatentState [B, 128, F, H, W], audio LatentState [B, 8, T, 16]) after the last step."""
        self._maybe_apply_loras()
        sigmas, timesteps = self._prepare_schedule(num_inference_steps, sigmas, initial_video_latent)
        fn = self._build_denoise_fn(positive_context, negative_context, video_guider_params, audio_guider_params, simple_denoise)
        vs, as_, vtools, atools = self._create_initial_states(height, width, num_frames, frame_rate, conditionings,
                                                              GaussianNoiser(video_noise), GaussianNoiser(audio_noise), noise_scale,
                                                              initial_video_latent, initial_audio_latent)  # fmt: skip
        vs, as_ = self._denoise(vs, as_, sigmas, timesteps, fn)
        return vtools.unpatchify(vtools.clear_conditioning(vs)), atools.unpatchify(atools.clear_conditioning(as_))

    @staticmethod
    def stage2_sigmas(device) -> torch.Tensor:
        return torch.tensor(STAGE_2_DISTILLED_SIGMA_VALUES, device=device, dtype=torch.float32)
