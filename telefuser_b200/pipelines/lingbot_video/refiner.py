"""LingBot-Video refiner hand-off: a finished low-resolution video goes through a second, low-noise denoising pass at
a higher resolution.

    video (base model, e.g. 480p)  ->  frame selection at the training frame rate  ->  bicubic resize to the refiner size
    ->  VAE encode  ->  mix with noise at the threshold sigma  ->  denoise only the sigmas below the threshold
    ->  VAE decode

Videos are [B, 3, F, H, W] in [-1, 1] throughout (what the pipelines produce and the VAE stage takes).
Role parity: telefuser/pipelines/lingbot_video/refiner.py:61-316 (frame budget, aligned indices, video preparation,
first-frame geometry, `LingBotVideoRefinerStage`); the sigma tail and the latent mix live in `pipeline.py`.
"""

from __future__ import annotations

import math

import numpy as np
import torch

from .pipeline import compute_refiner_sigmas, prepare_refiner_latent


def compute_training_frame_budget(num_source_frames: int, source_fps: float, sample_fps: int = 24, vae_tc: int = 4):
    """(frames to sample, frame rate they represent, latent frames) for a clip of `num_source_frames` at `source_fps`.
    Clips faster than the training rate are thinned to it; the count is then cut to 4n + 1 for the VAE."""
    if num_source_frames <= 0:
        return 1, 0.0, 1
    if min(source_fps, sample_fps, vae_tc) <= 0:
        raise ValueError("frame rates and the VAE's temporal factor must be positive")
    wanted = int(num_source_frames / source_fps * sample_fps) if source_fps > sample_fps else num_source_frames
    frames = max((wanted - 1) // vae_tc * vae_tc + 1, 1)
    return frames, frames / num_source_frames * source_fps, (frames - 1) // vae_tc + 1


def compute_training_aligned_indices(num_source_frames: int, sample_frames: int) -> torch.Tensor:
    """Which source frames make up the sample: evenly spaced (first and last included) when there are enough, else all
    of them followed by repeats of the last one."""
    if sample_frames <= 0:
        return torch.empty(0, dtype=torch.long)
    if num_source_frames <= 0:
        return torch.zeros(sample_frames, dtype=torch.long)
    if num_source_frames >= sample_frames:
        return torch.from_numpy(np.linspace(0, num_source_frames - 1, sample_frames, dtype=int)).long()
    pad = torch.full((sample_frames - num_source_frames,), num_source_frames - 1)
    return torch.cat([torch.arange(num_source_frames), pad])


def prepare_refiner_video(video: torch.Tensor, source_fps: float, height: int, width: int, sample_fps: int = 24,
                          vae_tc: int = 4, max_frames: int | None = None):  # fmt: skip
    """Frame selection + bicubic resize of a video in [-1, 1]. Returns (video [B, 3, F', height, width], facts)."""
    if video.ndim != 5 or video.shape[1] != 3:
        raise ValueError(f"a video is [B, 3, F, H, W], got {tuple(video.shape)}")
    if height <= 0 or width <= 0 or (max_frames is not None and max_frames < 1):
        raise ValueError("the target size and max_frames must be positive")
    total = video.shape[2]
    frames, vae_fps, latents = compute_training_frame_budget(total, source_fps, sample_fps, vae_tc)
    uncapped = frames
    capped = max_frames is not None and frames > max_frames
    if capped:
        frames = int(max_frames)
        vae_fps, latents = frames / total * source_fps, (frames - 1) // vae_tc + 1
    picked = video.index_select(2, compute_training_aligned_indices(total, frames).to(video.device))
    B, C, F, H, W = picked.shape
    flat = picked.transpose(1, 2).reshape(B * F, C, H, W).float()
    if (H, W) != (height, width):
        flat = torch.nn.functional.interpolate(flat, size=(height, width), mode="bicubic", align_corners=False).clamp(-1.0, 1.0)
    out = flat.reshape(B, F, C, height, width).transpose(1, 2).contiguous()
    return out, {"src_fps": float(source_fps), "num_source_frames": int(total), "sample_frame": int(frames),
                 "sample_frame_uncapped": int(uncapped), "max_frames": max_frames, "truncated_by_max_frames": bool(capped),
                 "vae_fps": float(vae_fps), "t_vae": int(latents)}  # fmt: skip


def first_frame_for_refiner(image, target_height: int, target_width: int, geometry_height: int, geometry_width: int) -> torch.Tensor:
    """The clean first frame of an image-conditioned video at the refiner's size: the image is centre-cropped to the
    aspect ratio of the LOW-resolution run (`geometry_*`, so that it shows what the base model saw) and resized
    bicubically. `image`: a PIL image or a path. Returns [1, 3, 1, target_height, target_width] in [-1, 1]."""
    from PIL import Image

    img = (image if isinstance(image, Image.Image) else Image.open(image)).convert("RGB")
    w, h = img.size
    want = geometry_width / geometry_height
    if w / h > want:
        ch, cw = h, max(1, int(round(h * want)))
    else:
        cw, ch = w, max(1, int(round(w / want)))
    left, top = int(round((w - cw) / 2.0)), int(round((h - ch) / 2.0))
    img = img.crop((left, top, left + cw, top + ch)).resize((target_width, target_height), resample=Image.BICUBIC)
    px = torch.from_numpy(np.asarray(img, dtype=np.float32) / 127.5 - 1.0)
    return px.permute(2, 0, 1)[None, :, None].contiguous()


class LingBotVideoRefinerStage:
    """The refiner as a stage of its own: it owns a denoising stage (the refiner transformer, possibly behind a worker
    group) and uses a VAE stage for the way in and out. `refine()` returns the refined video in [-1, 1]."""

    def __init__(self, denoising_stage, vae_stage, device="cuda", torch_dtype=torch.bfloat16) -> None:
        self.denoising_stage, self.vae_stage = denoising_stage, vae_stage
        self.device, self.torch_dtype = device, torch_dtype

    @staticmethod
    def _value(result):
        return result() if callable(result) else result

    def close(self) -> None:
        close = getattr(self.denoising_stage, "close", None)
        if callable(close):
            close()

    def _encode(self, video: torch.Tensor) -> torch.Tensor:
        return self._value(self.vae_stage.process("encode_video", video.to(self.device))).float()

    @torch.no_grad()
    def refine(self, lowres_video: torch.Tensor, positive_prompt_embeds, negative_prompt_embeds=None, positive_attention_mask=None,
               negative_attention_mask=None, num_inference_steps: int = 8, guidance_scale: float = 3.0, shift: float = 3.0,
               t_thresh: float = 0.85, tail_steps: int = 2, clean_first_frame: torch.Tensor | None = None, seed: int = 0,
               noise: torch.Tensor | None = None, before_decode=None, decode: bool = True) -> torch.Tensor:  # fmt: skip
        """`lowres_video`: the base model's output already resampled to the refiner's size (`prepare_refiner_video`).
        `clean_first_frame` ([B, 3, H, W] or [B, 3, 1, H, W]): for image-conditioned videos, frame 0 is replaced by its
        clean latent before every step and at the end. `before_decode`: called after denoising (e.g. to release the
        refiner's weights before the high-resolution VAE decode)."""
        x_up = self._encode(lowres_video)
        condition = mask = None
        if clean_first_frame is not None:
            first = clean_first_frame if clean_first_frame.ndim == 5 else clean_first_frame.unsqueeze(2)
            condition = self._encode(first)[:, :, :1].contiguous()
            x_up = x_up.clone()
            x_up[:, :, :1] = condition
            mask = torch.zeros(x_up.shape[2], dtype=torch.bool, device=x_up.device)
            mask[0] = True
        if noise is None:
            noise = torch.randn(x_up.shape, generator=torch.Generator(device="cpu").manual_seed(seed)).to(x_up)
        elif noise.shape != x_up.shape:
            raise ValueError(f"injected noise {tuple(noise.shape)} does not match the encoded video {tuple(x_up.shape)}")
        sig = compute_refiner_sigmas(1.0, 0.0, num_inference_steps, shift, t_thresh, tail_steps)
        latent = prepare_refiner_latent(x_up, noise.to(x_up), float(sig[0]))
        dev, dt = self.device, self.torch_dtype
        neg = None if negative_prompt_embeds is None else negative_prompt_embeds.to(dev, dt)
        latent = self._value(self.denoising_stage.denoise(latent, positive_prompt_embeds.to(dev, dt), neg, positive_attention_mask,
                                                          negative_attention_mask, guidance_scale, len(sig), shift, condition,
                                                          mask, sig))  # fmt: skip
        if before_decode is not None:
            before_decode()
        if not decode:
            return latent
        return self._value(self.vae_stage.process("decode_video", latent.to(dt)))


def refiner_size(height: int, width: int, scale: float = 2.25, multiple: int = 16) -> tuple[int, int]:
    """Refiner resolution for a base run of height x width: scaled and rounded UP to the patch grid (480 x 832 at the
    default 2.25 gives 1088 x 1872; the published recipe uses 1088 x 1920 for 16:9 inputs)."""
    return math.ceil(height * scale / multiple) * multiple, math.ceil(width * scale / multiple) * multiple


__all__ = ["compute_training_frame_budget", "compute_training_aligned_indices", "prepare_refiner_video", "first_frame_for_refiner",
           "LingBotVideoRefinerStage", "refiner_size"]  # fmt: skip
