"""LTX-2 latent upsampler: residual conv stacks around a learned pixel-shuffle (x2 space, x2 time, or a rational scale).

The two-stage pipeline denoises at half resolution, upsamples the (de-normalised) latents here and refines them
at full resolution. Convolutions and GroupNorm run through cuDNN in channels-last layout; this model is a few
milliseconds per call and has no custom kernel.
Role parity: telefuser/models/ltx_upsampler.py:26-399.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn

from telefuser_b200.core.base_model import BaseModel

LTX23_SPATIAL_UPSAMPLER_CONFIG = dict(in_channels=128, mid_channels=1024, num_blocks_per_stage=4, dims=3, spatial_upsample=True,
                                      temporal_upsample=False)  # fmt: skip


def _frames_to_batch(x):
    b, c, f, h, w = x.shape
    return x.permute(0, 2, 1, 3, 4).reshape(b * f, c, h, w)


def _batch_to_frames(x, b: int):
    bf, c, h, w = x.shape
    return x.reshape(b, bf // b, c, h, w).permute(0, 2, 1, 3, 4)


class BlurDownsample(nn.Module):
    """Anti-aliased stride-`stride` downsampling on (H, W) with a fixed separable binomial kernel."""

    def __init__(self, dims: int, stride: int, kernel_size: int = 5) -> None:
        super().__init__()
        if dims not in (2, 3) or stride < 1 or kernel_size < 3 or kernel_size % 2 == 0:
            raise ValueError("BlurDownsample needs dims 2 or 3, stride >= 1 and an odd kernel >= 3")
        self.dims, self.stride, self.kernel_size = dims, stride, kernel_size
        k = torch.tensor([math.comb(kernel_size - 1, i) for i in range(kernel_size)], dtype=torch.float32)
        k2 = torch.outer(k, k)
        self.register_buffer("kernel", (k2 / k2.sum())[None, None])

    def _apply_2d(self, x):
        c = x.shape[1]
        return F.conv2d(x, self.kernel.to(x.dtype).expand(c, 1, -1, -1), stride=self.stride, padding=self.kernel_size // 2, groups=c)

    def forward(self, x):
        if self.stride == 1:
            return x
        if self.dims == 2:
            return self._apply_2d(x)
        return _batch_to_frames(self._apply_2d(_frames_to_batch(x)), x.shape[0])


class PixelShuffleND(nn.Module):
    """Moves channel factors into time (dims 1), space (dims 2) or both (dims 3)."""

    def __init__(self, dims: int, upscale_factors=(2, 2, 2)) -> None:
        super().__init__()
        if dims not in (1, 2, 3):
            raise ValueError("dims must be 1, 2 or 3")
        self.dims, self.upscale_factors = dims, tuple(upscale_factors)

    def forward(self, x):
        p = self.upscale_factors
        if self.dims == 2:
            return F.pixel_shuffle(x, p[0]) if p[0] == p[1] else self._shuffle2(x, p[0], p[1])
        b, c, d, h, w = x.shape
        if self.dims == 1:
            return x.reshape(b, c // p[0], p[0], d, h, w).permute(0, 1, 3, 2, 4, 5).reshape(b, c // p[0], d * p[0], h, w)
        n = c // (p[0] * p[1] * p[2])
        x = x.reshape(b, n, p[0], p[1], p[2], d, h, w).permute(0, 1, 5, 2, 6, 3, 7, 4)
        return x.reshape(b, n, d * p[0], h * p[1], w * p[2])

    @staticmethod
    def _shuffle2(x, p1: int, p2: int):
        b, c, h, w = x.shape
        n = c // (p1 * p2)
        return x.reshape(b, n, p1, p2, h, w).permute(0, 1, 4, 2, 5, 3).reshape(b, n, h * p1, w * p2)


class ResBlock(nn.Module):
    def __init__(self, channels: int, mid_channels: int | None = None, dims: int = 3) -> None:
        super().__init__()
        mid_channels = mid_channels or channels
        conv = nn.Conv2d if dims == 2 else nn.Conv3d
        self.conv1, self.norm1 = conv(channels, mid_channels, 3, padding=1), nn.GroupNorm(32, mid_channels)
        self.conv2, self.norm2 = conv(mid_channels, channels, 3, padding=1), nn.GroupNorm(32, channels)
        self.activation = nn.SiLU()

    def forward(self, x):
        y = self.activation(self.norm1(self.conv1(x)))
        return self.activation(self.norm2(self.conv2(y)) + x)


def _rational_for_scale(scale: float) -> tuple[int, int]:
    table = {0.75: (3, 4), 1.5: (3, 2), 2.0: (2, 1), 4.0: (4, 1)}
    if float(scale) not in table:
        raise ValueError(f"unsupported spatial scale {scale}; choose from {sorted(table)}")
    return table[float(scale)]


class SpatialRationalResampler(nn.Module):
    """Scale by num / den: learned x num pixel-shuffle then anti-aliased / den downsampling, frame by frame."""

    def __init__(self, mid_channels: int, scale: float) -> None:
        super().__init__()
        self.scale = float(scale)
        self.num, self.den = _rational_for_scale(self.scale)
        self.conv = nn.Conv2d(mid_channels, self.num**2 * mid_channels, 3, padding=1)
        self.pixel_shuffle = PixelShuffleND(2, (self.num, self.num))
        self.blur_down = BlurDownsample(2, self.den)

    def forward(self, x):
        return _batch_to_frames(self.blur_down(self.pixel_shuffle(self.conv(_frames_to_batch(x)))), x.shape[0])


class LatentUpsampler(BaseModel):
    def __init__(self, in_channels: int = 128, mid_channels: int = 512, num_blocks_per_stage: int = 4, dims: int = 3,
                 spatial_upsample: bool = True, temporal_upsample: bool = False, spatial_scale: float = 2.0,
                 rational_resampler: bool = False) -> None:  # fmt: skip
        super().__init__()
        self.in_channels, self.mid_channels, self.num_blocks_per_stage, self.dims = in_channels, mid_channels, num_blocks_per_stage, dims
        self.spatial_upsample, self.temporal_upsample = spatial_upsample, temporal_upsample
        self.spatial_scale, self.rational_resampler = float(spatial_scale), rational_resampler
        conv = nn.Conv2d if dims == 2 else nn.Conv3d
        self.initial_conv = conv(in_channels, mid_channels, 3, padding=1)
        self.initial_norm = nn.GroupNorm(32, mid_channels)
        self.initial_activation = nn.SiLU()
        self.res_blocks = nn.ModuleList([ResBlock(mid_channels, dims=dims) for _ in range(num_blocks_per_stage)])
        if spatial_upsample and temporal_upsample:
            self.upsampler = nn.Sequential(nn.Conv3d(mid_channels, 8 * mid_channels, 3, padding=1), PixelShuffleND(3))
        elif spatial_upsample and rational_resampler:
            self.upsampler = SpatialRationalResampler(mid_channels, self.spatial_scale)
        elif spatial_upsample:
            self.upsampler = nn.Sequential(nn.Conv2d(mid_channels, 4 * mid_channels, 3, padding=1), PixelShuffleND(2))
        elif temporal_upsample:
            self.upsampler = nn.Sequential(nn.Conv3d(mid_channels, 2 * mid_channels, 3, padding=1), PixelShuffleND(1))
        else:
            raise ValueError("either spatial_upsample or temporal_upsample must be set")
        self.post_upsample_res_blocks = nn.ModuleList([ResBlock(mid_channels, dims=dims) for _ in range(num_blocks_per_stage)])
        self.final_conv = conv(mid_channels, in_channels, 3, padding=1)

    def _upsample(self, x, b: int):
        if self.dims == 2 and not isinstance(self.upsampler, SpatialRationalResampler) and not self.temporal_upsample:
            return self.upsampler(x)
        if self.temporal_upsample:
            return self.upsampler(x)[:, :, 1:]  # the first latent frame stands for a single pixel frame
        if isinstance(self.upsampler, SpatialRationalResampler):
            return self.upsampler(x)
        return _batch_to_frames(self.upsampler(_frames_to_batch(x)), b)

    def forward(self, latent):
        b = latent.shape[0]
        x = _frames_to_batch(latent) if self.dims == 2 else latent
        x = self.initial_activation(self.initial_norm(self.initial_conv(x)))
        for blk in self.res_blocks:
            x = blk(x)
        x = self._upsample(x, b)
        for blk in self.post_upsample_res_blocks:
            x = blk(x)
        x = self.final_conv(x)
        return _batch_to_frames(x, b) if self.dims == 2 else x


def upsample_video(latent, video_encoder, upsampler: LatentUpsampler):
    """De-normalise with the VAE's per-channel statistics, upsample, normalise again."""
    stats = video_encoder.per_channel_statistics
    return stats.normalize(upsampler(stats.un_normalize(latent)))


class LatentUpsamplerConfigurator:
    @classmethod
    def from_config(cls, config: dict) -> LatentUpsampler:
        keys = ("in_channels", "mid_channels", "num_blocks_per_stage", "dims", "spatial_upsample", "temporal_upsample", "spatial_scale",
                "rational_resampler")  # fmt: skip
        return LatentUpsampler(**{k: config[k] for k in keys if k in config})


class LTXSpatialUpsampler(LatentUpsampler):
    def __init__(self, **overrides) -> None:
        super().__init__(**{**LTX23_SPATIAL_UPSAMPLER_CONFIG, **overrides})

    @staticmethod
    def state_dict_converter():
        return LTXSpatialUpsamplerStateDictConverter()


class LTXSpatialUpsamplerStateDictConverter:
    def from_official(self, state_dict: dict):
        return dict(state_dict), {}

    from_diffusers = from_official
