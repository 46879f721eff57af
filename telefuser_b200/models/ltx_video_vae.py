"""LTX-2 video VAE: 3 x (1 + 8k) x H x W pixels <-> 128 x (1 + k) x H/32 x W/32 latents, with tiled encode / decode.

Encoder: 4 x 4 space-to-depth, causal 3-D convs (the first frame is replicated in front so a latent frame
never sees later pixels), residual stacks with per-pixel RMS norm, space-to-depth downsamplers with an averaged
skip path, a uniform log-variance channel that is dropped, and per-channel latent normalisation. Decoder: the
mirror image with depth-to-space upsamplers, optional noise injection and optional timestep conditioning.
Tiled paths cut overlapping windows (temporal windows start one latent frame early because that frame decodes
to a single pixel frame), blend them with trapezoidal ramps and stream the decoded video chunk by chunk.
Convolutions run through cuDNN; the norms and rearrangements are PyTorch.
Role parity: telefuser/models/ltx_video_vae.py:35-2660.
"""

from __future__ import annotations

import itertools
import math
from dataclasses import dataclass
from enum import Enum
from typing import Iterator, NamedTuple

import torch
from torch import nn

from telefuser_b200.core.base_model import BaseModel
from telefuser_b200.models.ltx_dit import PixArtAlphaCombinedTimestepSizeEmbeddings

DEFAULT_LTX23_ENCODER_BLOCKS = (
    ("res_x", {"num_layers": 4}), ("compress_space_res", {"multiplier": 2}), ("res_x", {"num_layers": 6}),
    ("compress_time_res", {"multiplier": 2}), ("res_x", {"num_layers": 4}), ("compress_all_res", {"multiplier": 2}),
    ("res_x", {"num_layers": 2}), ("compress_all_res", {"multiplier": 1}), ("res_x", {"num_layers": 2}))  # fmt: skip
DEFAULT_LTX23_DECODER_BLOCKS = (
    ("res_x", {"num_layers": 4}), ("compress_space", {"multiplier": 2}), ("res_x", {"num_layers": 6}),
    ("compress_time", {"multiplier": 2}), ("res_x", {"num_layers": 4}), ("compress_all", {"multiplier": 1}),
    ("res_x", {"num_layers": 2}), ("compress_all", {"multiplier": 2}), ("res_x", {"num_layers": 2}))  # fmt: skip


class NormLayerType(Enum):
    GROUP_NORM = "group_norm"
    PIXEL_NORM = "pixel_norm"


class LogVarianceType(Enum):
    PER_CHANNEL = "per_channel"
    UNIFORM = "uniform"
    CONSTANT = "constant"
    NONE = "none"


class PaddingModeType(Enum):
    ZEROS = "zeros"
    REFLECT = "reflect"
    REPLICATE = "replicate"
    CIRCULAR = "circular"


class SpatioTemporalScaleFactors(NamedTuple):
    time: int = 8
    height: int = 32
    width: int = 32

    @classmethod
    def default(cls) -> "SpatioTemporalScaleFactors":
        return cls()


VIDEO_SCALE_FACTORS = SpatioTemporalScaleFactors.default()
VIDEO_LATENT_CHANNELS = 128


class VideoPixelShape(NamedTuple):
    batch: int
    frames: int
    width: int
    height: int
    fps: float = 1.0

    def to_torch_shape(self, channels: int = 3) -> torch.Size:
        return torch.Size([self.batch, channels, self.frames, self.height, self.width])


class VideoLatentShape(NamedTuple):
    batch: int
    channels: int
    frames: int
    height: int
    width: int

    def to_torch_shape(self) -> torch.Size:
        return torch.Size(self)

    @staticmethod
    def from_torch_shape(shape) -> "VideoLatentShape":
        return VideoLatentShape(*shape)

    @staticmethod
    def from_pixels(batch: int, num_frames: int, height: int, width: int, channels: int = VIDEO_LATENT_CHANNELS,
                    scale: SpatioTemporalScaleFactors = VIDEO_SCALE_FACTORS) -> "VideoLatentShape":  # fmt: skip
        return VideoLatentShape(batch, channels, (num_frames - 1) // scale.time + 1, height // scale.height, width // scale.width)

    def token_count(self) -> int:
        return self.frames * self.height * self.width

    def mask_shape(self) -> "VideoLatentShape":
        return self._replace(channels=1)

    def upscale(self, scale: SpatioTemporalScaleFactors = VIDEO_SCALE_FACTORS) -> VideoPixelShape:
        return VideoPixelShape(self.batch, (self.frames - 1) * scale.time + 1, self.width * scale.width, self.height * scale.height)


# ---- layers --------------------------------------------------------------------------------
class PixelNorm(nn.Module):
    """x / sqrt(mean(x^2 over `dim`) + eps): an RMS norm over channels at every voxel, no weights."""

    def __init__(self, dim: int = 1, eps: float = 1e-8) -> None:
        super().__init__()
        self.dim, self.eps = dim, eps

    def forward(self, x):
        return x * torch.rsqrt(x.float().pow(2).mean(dim=self.dim, keepdim=True) + self.eps).to(x.dtype)


def _norm(kind: NormLayerType, channels: int, groups: int, eps: float = 1e-6) -> nn.Module:
    return nn.GroupNorm(groups, channels, eps=eps, affine=True) if kind == NormLayerType.GROUP_NORM else PixelNorm()


class CausalConv3d(nn.Module):
    """Time padding by replicating the first frame (causal) or both end frames; spatial padding inside the conv."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size: int = 3, stride=1, dilation: int = 1, groups: int = 1,
                 bias: bool = True, spatial_padding_mode: PaddingModeType = PaddingModeType.ZEROS) -> None:  # fmt: skip
        super().__init__()
        self.in_channels, self.out_channels, self.time_kernel_size = in_channels, out_channels, kernel_size
        self.conv = nn.Conv3d(in_channels, out_channels, (kernel_size,) * 3, stride=stride, dilation=(dilation, 1, 1),
                              padding=(0, kernel_size // 2, kernel_size // 2), padding_mode=spatial_padding_mode.value, groups=groups,
                              bias=bias)  # fmt: skip

    def forward(self, x, causal: bool = True):
        k = self.time_kernel_size - 1
        if causal:
            x = torch.cat([x[:, :, :1].expand(-1, -1, k, -1, -1), x], dim=2)
        else:
            x = torch.cat([x[:, :, :1].expand(-1, -1, k // 2, -1, -1), x, x[:, :, -1:].expand(-1, -1, k // 2, -1, -1)], dim=2)
        return self.conv(x)

    @property
    def weight(self):
        return self.conv.weight


def _conv(dims, cin: int, cout: int, stride=1, pad: PaddingModeType = PaddingModeType.ZEROS) -> CausalConv3d:
    if dims != 3:
        raise ValueError("only 3-D convolutions are built (the released LTX-2 VAEs use dims = 3)")
    return CausalConv3d(cin, cout, 3, stride=stride, spatial_padding_mode=pad)


def _space_to_depth(x, p):
    """b c (d p1) (h p2) (w p3) -> b (c p1 p2 p3) d h w"""
    b, c, d, h, w = x.shape
    x = x.reshape(b, c, d // p[0], p[0], h // p[1], p[1], w // p[2], p[2]).permute(0, 1, 3, 5, 7, 2, 4, 6)
    return x.reshape(b, c * p[0] * p[1] * p[2], d // p[0], h // p[1], w // p[2])


def _depth_to_space(x, p):
    """b (c p1 p2 p3) d h w -> b c (d p1) (h p2) (w p3)"""
    b, c, d, h, w = x.shape
    n = c // (p[0] * p[1] * p[2])
    x = x.reshape(b, n, p[0], p[1], p[2], d, h, w).permute(0, 1, 5, 2, 6, 3, 7, 4)
    return x.reshape(b, n, d * p[0], h * p[1], w * p[2])


def patchify(x, patch_size_hw: int, patch_size_t: int = 1):
    """[B, C, F, H, W] -> [B, C * pt * p * p, F / pt, H / p, W / p] with channel order (c, pt, column, row)."""
    if patch_size_hw == 1 and patch_size_t == 1:
        return x
    if x.dim() == 4:
        return patchify(x.unsqueeze(2), patch_size_hw, 1).squeeze(2)
    b, c, f, h, w = x.shape
    p, q = patch_size_t, patch_size_hw
    x = x.reshape(b, c, f // p, p, h // q, q, w // q, q).permute(0, 1, 3, 7, 5, 2, 4, 6)
    return x.reshape(b, c * p * q * q, f // p, h // q, w // q)


def unpatchify(x, patch_size_hw: int, patch_size_t: int = 1):
    if patch_size_hw == 1 and patch_size_t == 1:
        return x
    if x.dim() == 4:
        return unpatchify(x.unsqueeze(2), patch_size_hw, 1).squeeze(2)
    b, c, f, h, w = x.shape
    p, q = patch_size_t, patch_size_hw
    n = c // (p * q * q)
    x = x.reshape(b, n, p, q, q, f, h, w).permute(0, 1, 5, 2, 6, 4, 7, 3)  # (c, pt, r, q) -> (f pt) (h q) (w r)
    return x.reshape(b, n, f * p, h * q, w * q)


class PerChannelStatistics(nn.Module):
    def __init__(self, latent_channels: int = 128) -> None:
        super().__init__()
        self.register_buffer("std-of-means", torch.ones(latent_channels))
        self.register_buffer("mean-of-means", torch.zeros(latent_channels))

    def _stats(self, x):
        return self.get_buffer("mean-of-means").view(1, -1, 1, 1, 1).to(x), self.get_buffer("std-of-means").view(1, -1, 1, 1, 1).to(x)

    def un_normalize(self, x):
        mean, std = self._stats(x)
        return x * std + mean

    def normalize(self, x):
        mean, std = self._stats(x)
        return (x - mean) / std


class SpaceToDepthDownsample(nn.Module):
    def __init__(self, dims, in_channels: int, out_channels: int, stride, spatial_padding_mode=PaddingModeType.ZEROS) -> None:
        super().__init__()
        self.stride = tuple(stride)
        self.group_size = in_channels * math.prod(stride) // out_channels
        self.conv = _conv(dims, in_channels, out_channels // math.prod(stride), pad=spatial_padding_mode)

    def forward(self, x, causal: bool = True):
        if self.stride[0] == 2:
            x = torch.cat([x[:, :, :1], x], dim=2)
        skip = _space_to_depth(x, self.stride)
        skip = skip.unflatten(1, (-1, self.group_size)).mean(dim=2)
        return _space_to_depth(self.conv(x, causal=causal), self.stride) + skip


class DepthToSpaceUpsample(nn.Module):
    def __init__(self, dims, in_channels: int, stride, residual: bool = False, out_channels_reduction_factor: int = 1,
                 spatial_padding_mode=PaddingModeType.ZEROS) -> None:  # fmt: skip
        super().__init__()
        self.stride, self.residual, self.out_channels_reduction_factor = tuple(stride), residual, out_channels_reduction_factor
        self.out_channels = math.prod(stride) * in_channels // out_channels_reduction_factor
        self.conv = _conv(dims, in_channels, self.out_channels, pad=spatial_padding_mode)

    def forward(self, x, causal: bool = True):
        skip = None
        if self.residual:
            skip = _depth_to_space(x, self.stride).repeat(1, math.prod(self.stride) // self.out_channels_reduction_factor, 1, 1, 1)
        x = _depth_to_space(self.conv(x, causal=causal), self.stride)
        if self.stride[0] == 2:
            x = x[:, :, 1:]
            skip = None if skip is None else skip[:, :, 1:]
        return x if skip is None else x + skip


class ResnetBlock3D(nn.Module):
    def __init__(self, dims, in_channels: int, out_channels: int | None = None, dropout: float = 0.0, groups: int = 32, eps: float = 1e-6,
                 norm_layer: NormLayerType = NormLayerType.PIXEL_NORM, inject_noise: bool = False, timestep_conditioning: bool = False,
                 spatial_padding_mode=PaddingModeType.ZEROS) -> None:  # fmt: skip
        super().__init__()
        out_channels = out_channels or in_channels
        self.in_channels, self.out_channels, self.inject_noise = in_channels, out_channels, inject_noise
        self.timestep_conditioning = timestep_conditioning
        self.norm1 = _norm(norm_layer, in_channels, groups, eps)
        self.non_linearity = nn.SiLU()
        self.conv1 = _conv(dims, in_channels, out_channels, pad=spatial_padding_mode)
        self.norm2 = _norm(norm_layer, out_channels, groups, eps)
        self.conv2 = _conv(dims, out_channels, out_channels, pad=spatial_padding_mode)
        if inject_noise:
            self.per_channel_scale1 = nn.Parameter(torch.zeros(in_channels, 1, 1))
            self.per_channel_scale2 = nn.Parameter(torch.zeros(in_channels, 1, 1))
        same = in_channels == out_channels
        self.conv_shortcut = nn.Identity() if same else nn.Conv3d(in_channels, out_channels, 1)
        self.norm3 = nn.Identity() if same else nn.GroupNorm(1, in_channels, eps=eps, affine=True)
        if timestep_conditioning:
            self.scale_shift_table = nn.Parameter(torch.zeros(4, in_channels))

    @staticmethod
    def _noise(h, scale, generator):
        n = torch.randn(h.shape[-2:], device=h.device, dtype=h.dtype, generator=generator)[None]
        return h + (n * scale.to(h))[None, :, None]

    def forward(self, x, causal: bool = True, timestep=None, generator=None):
        h = self.norm1(x)
        if self.timestep_conditioning:
            if timestep is None:
                raise ValueError("timestep conditioning needs a timestep")
            ada = self.scale_shift_table[None, ..., None, None, None].to(h) + timestep.reshape(x.shape[0], 4, -1, 1, 1, 1).to(h)
            shift1, scale1, shift2, scale2 = ada.unbind(dim=1)
            h = h * (1 + scale1) + shift1
        h = self.conv1(self.non_linearity(h), causal=causal)
        if self.inject_noise:
            h = self._noise(h, self.per_channel_scale1, generator)
        h = self.norm2(h)
        if self.timestep_conditioning:
            h = h * (1 + scale2) + shift2
        h = self.conv2(self.non_linearity(h), causal=causal)
        if self.inject_noise:
            h = self._noise(h, self.per_channel_scale2, generator)
        return self.conv_shortcut(self.norm3(x)) + h


class UNetMidBlock3D(nn.Module):
    def __init__(self, dims, in_channels: int, dropout: float = 0.0, num_layers: int = 1, resnet_eps: float = 1e-6, resnet_groups: int = 32,
                 norm_layer: NormLayerType = NormLayerType.GROUP_NORM, inject_noise: bool = False, timestep_conditioning: bool = False,
                 spatial_padding_mode=PaddingModeType.ZEROS) -> None:  # fmt: skip
        super().__init__()
        self.timestep_conditioning = timestep_conditioning
        if timestep_conditioning:
            self.time_embedder = PixArtAlphaCombinedTimestepSizeEmbeddings(in_channels * 4, 0)
        self.res_blocks = nn.ModuleList([
            ResnetBlock3D(dims, in_channels, in_channels, dropout, resnet_groups or min(in_channels // 4, 32), resnet_eps, norm_layer,
                          inject_noise, timestep_conditioning, spatial_padding_mode) for _ in range(num_layers)])  # fmt: skip

    def forward(self, x, causal: bool = True, timestep=None, generator=None):
        emb = None
        if self.timestep_conditioning:
            if timestep is None:
                raise ValueError("timestep conditioning needs a timestep")
            emb = self.time_embedder(timestep.flatten().float()).view(x.shape[0], -1, 1, 1, 1)
        for blk in self.res_blocks:
            x = blk(x, causal=causal, timestep=emb, generator=generator)
        return x


_DOWN_STRIDES = {"compress_time": (2, 1, 1), "compress_space": (1, 2, 2), "compress_all": (2, 2, 2)}


def _make_encoder_block(name: str, cfg: dict, cin: int, dims, norm_layer, groups: int, pad):
    if name == "res_x":
        return UNetMidBlock3D(dims, cin, num_layers=cfg["num_layers"], resnet_groups=groups, norm_layer=norm_layer, spatial_padding_mode=pad), cin
    if name == "res_x_y":
        cout = cin * cfg.get("multiplier", 2)
        return ResnetBlock3D(dims, cin, cout, groups=groups, norm_layer=norm_layer, spatial_padding_mode=pad), cout
    if name in _DOWN_STRIDES:
        return _conv(dims, cin, cin, stride=_DOWN_STRIDES[name], pad=pad), cin
    if name == "compress_all_x_y":
        cout = cin * cfg.get("multiplier", 2)
        return _conv(dims, cin, cout, stride=(2, 2, 2), pad=pad), cout
    if name.endswith("_res") and name[:-4] in _DOWN_STRIDES:
        cout = cin * cfg.get("multiplier", 2)
        return SpaceToDepthDownsample(dims, cin, cout, _DOWN_STRIDES[name[:-4]], pad), cout
    raise ValueError(f"unknown encoder block {name}")


def _make_decoder_block(name: str, cfg: dict, cin: int, dims, norm_layer, timestep_conditioning: bool, groups: int, pad):
    if name == "res_x":
        return UNetMidBlock3D(dims, cin, num_layers=cfg["num_layers"], resnet_groups=groups, norm_layer=norm_layer,
                              inject_noise=cfg.get("inject_noise", False), timestep_conditioning=timestep_conditioning,
                              spatial_padding_mode=pad), cin  # fmt: skip
    if name == "res_x_y":
        cout = cin // cfg.get("multiplier", 2)
        return ResnetBlock3D(dims, cin, cout, groups=groups, norm_layer=norm_layer, inject_noise=cfg.get("inject_noise", False),
                             spatial_padding_mode=pad), cout  # fmt: skip
    if name in _DOWN_STRIDES:
        m = cfg.get("multiplier", 1)
        return DepthToSpaceUpsample(dims, cin, _DOWN_STRIDES[name], residual=cfg.get("residual", False) and name == "compress_all",
                                    out_channels_reduction_factor=m, spatial_padding_mode=pad), cin // m  # fmt: skip
    raise ValueError(f"unknown decoder block {name}")


# ---- tiling ----------------------------------------------------------------------------------
def compute_trapezoidal_mask_1d(length: int, ramp_left: int, ramp_right: int, left_starts_from_0: bool = False) -> torch.Tensor:
    if length <= 0:
        raise ValueError("mask length must be positive")
    ramp_left, ramp_right = max(0, min(ramp_left, length)), max(0, min(ramp_right, length))
    mask = torch.ones(length)
    if ramp_left > 0:
        fade = torch.linspace(0.0, 1.0, ramp_left + (1 if left_starts_from_0 else 2))[:-1]
        mask[:ramp_left] *= fade if left_starts_from_0 else fade[1:]
    if ramp_right > 0:
        mask[-ramp_right:] *= torch.linspace(1.0, 0.0, ramp_right + 2)[1:-1]
    return mask.clamp_(0, 1)


def compute_rectangular_mask_1d(length: int, left_ramp: int, right_ramp: int) -> torch.Tensor:
    if length <= 0:
        raise ValueError("mask length must be positive")
    mask = torch.ones(length)
    mask[: max(left_ramp, 0)] = 0
    if right_ramp > 0:
        mask[-right_ramp:] = 0
    return mask


@dataclass(frozen=True)
class DimensionIntervals:
    starts: list
    ends: list
    left_ramps: list
    right_ramps: list


def _whole(length: int) -> DimensionIntervals:
    return DimensionIntervals([0], [length], [0], [0])


def split_with_symmetric_overlaps(size: int, overlap: int):
    def split(length: int) -> DimensionIntervals:
        if length <= size:
            return _whole(length)
        n = (length + size - 2 * overlap - 1) // (size - overlap)
        starts = [i * (size - overlap) for i in range(n)]
        ends = [s + size for s in starts]
        ends[-1] = length
        return DimensionIntervals(starts, ends, [0] + [overlap] * (n - 1), [overlap] * (n - 1) + [0])

    return split


def split_temporal_latents(size: int, overlap: int):
    """Latent windows after the first start one frame early: that frame decodes to one pixel frame and is blended away."""
    base = split_with_symmetric_overlaps(size, overlap)

    def split(length: int) -> DimensionIntervals:
        if length <= size:
            return _whole(length)
        iv = base(length)
        return DimensionIntervals([iv.starts[0]] + [s - 1 for s in iv.starts[1:]], iv.ends, [iv.left_ramps[0]] + [r + 1 for r in iv.left_ramps[1:]],
                                  iv.right_ramps)  # fmt: skip

    return split


def split_temporal_frames(size: int, overlap: int):
    """Pixel-frame windows for encoding: each but the last takes one extra frame (1 + 8k) and has no right ramp."""
    base = split_with_symmetric_overlaps(size, overlap)

    def split(length: int) -> DimensionIntervals:
        if length <= size:
            return _whole(length)
        iv = base(length)
        return DimensionIntervals(iv.starts, [e + 1 for e in iv.ends[:-1]] + [iv.ends[-1]], iv.left_ramps, [0] * len(iv.right_ramps))

    return split


def map_temporal_interval_to_frame(begin, end, left_ramp, right_ramp, scale):
    start, stop = begin * scale, 1 + (end - 1) * scale
    left = 0 if left_ramp == 0 else 1 + (left_ramp - 1) * scale
    return slice(start, stop), compute_trapezoidal_mask_1d(stop - start, left, right_ramp * scale, True)


def map_temporal_interval_to_latent(begin, end, left_ramp, right_ramp=0, scale=1):
    start, stop = begin // scale, (end - 1) // scale + 1
    if right_ramp // scale != 0:
        raise ValueError("temporal encode tiles must not have a right ramp")
    return slice(start, stop), compute_rectangular_mask_1d(stop - start, 0 if left_ramp == 0 else 1 + (left_ramp - 1) // scale, 0)


def map_spatial_interval_to_pixel(begin, end, left_ramp, right_ramp, scale):
    return slice(begin * scale, end * scale), compute_trapezoidal_mask_1d((end - begin) * scale, left_ramp * scale, right_ramp * scale, False)


def map_spatial_interval_to_latent(begin, end, left_ramp, right_ramp, scale):
    start, stop = begin // scale, end // scale
    return slice(start, stop), compute_rectangular_mask_1d(stop - start, max(0, left_ramp // scale - 1), 0 if right_ramp == 0 else 1)


class Tile(NamedTuple):
    in_coords: tuple
    out_coords: tuple
    masks_1d: tuple

    @property
    def blend_mask(self) -> torch.Tensor:
        n = len(self.out_coords)
        out = torch.ones([1] * n)
        for axis, m in enumerate(self.masks_1d):
            if m is not None:
                shape = [1] * n
                shape[axis] = m.shape[0]
                out = out * m.view(shape)
        return out


def create_tiles(shape, splitters: list, mappers: list) -> list:
    """`splitters[axis]`: length -> DimensionIntervals or None (whole axis); `mappers[axis]`: (map function, scale) or None."""
    if len(splitters) != len(shape) or len(mappers) != len(shape):
        raise ValueError("one splitter and one mapper per axis are needed")
    per_axis = []
    for length, split, mapper in zip(shape, splitters, mappers):
        iv = _whole(length) if split is None else split(length)
        entries = []
        for b, e, lr, rr in zip(iv.starts, iv.ends, iv.left_ramps, iv.right_ramps):
            dst, mask = (slice(0, None), None) if mapper is None else mapper[0](b, e, lr, rr, mapper[1])
            entries.append((slice(b, e), dst, mask))
        per_axis.append(entries)
    return [Tile(tuple(c[0] for c in combo), tuple(c[1] for c in combo), tuple(c[2] for c in combo))
            for combo in itertools.product(*per_axis)]  # fmt: skip


def _validate_tiling(size: int, overlap: int, minimum: int, multiple: int, what: str) -> None:
    if size < minimum or size % multiple or overlap % multiple or overlap >= size:
        raise ValueError(f"{what} tile size {size} / overlap {overlap}: size >= {minimum}, both multiples of {multiple}, overlap < size")


def prepare_tiles_for_encoding(video, spatial_tile_size_in_pixels=None, spatial_tile_overlap_in_pixels: int = 0,
                               temporal_tile_size_in_frames=None, temporal_tile_overlap_in_frames: int = 0) -> list:  # fmt: skip
    splitters, mappers = [None] * 5, [None] * 5
    if spatial_tile_size_in_pixels is not None:
        _validate_tiling(spatial_tile_size_in_pixels, spatial_tile_overlap_in_pixels, 64, 32, "spatial")
        overlap = max(spatial_tile_overlap_in_pixels, 64)
        for axis, scale in ((3, VIDEO_SCALE_FACTORS.height), (4, VIDEO_SCALE_FACTORS.width)):
            splitters[axis] = split_with_symmetric_overlaps(spatial_tile_size_in_pixels, overlap)
            mappers[axis] = (map_spatial_interval_to_latent, scale)
    if temporal_tile_size_in_frames is not None:
        _validate_tiling(temporal_tile_size_in_frames, temporal_tile_overlap_in_frames, 16, 8, "temporal")
        splitters[2] = split_temporal_frames(temporal_tile_size_in_frames, max(temporal_tile_overlap_in_frames, 16))
        mappers[2] = (map_temporal_interval_to_latent, VIDEO_SCALE_FACTORS.time)
    return create_tiles(video.shape, splitters, mappers)


# ---- encoder / decoder -------------------------------------------------------------------------
class VideoEncoder(nn.Module):
    def __init__(self, convolution_dimensions=3, in_channels: int = 3, out_channels: int = 128, encoder_blocks=(), patch_size: int = 4,
                 norm_layer: NormLayerType = NormLayerType.PIXEL_NORM, latent_log_var: LogVarianceType = LogVarianceType.UNIFORM,
                 encoder_spatial_padding_mode: PaddingModeType = PaddingModeType.ZEROS) -> None:  # fmt: skip
        super().__init__()
        self.patch_size, self.norm_layer, self.latent_channels, self.latent_log_var = patch_size, norm_layer, out_channels, latent_log_var
        self.per_channel_statistics = PerChannelStatistics(out_channels)
        pad, ch = encoder_spatial_padding_mode, out_channels
        self.conv_in = _conv(convolution_dimensions, in_channels * patch_size**2, ch, pad=pad)
        self.down_blocks = nn.ModuleList()
        for name, params in encoder_blocks:
            blk, ch = _make_encoder_block(name, {"num_layers": params} if isinstance(params, int) else params, ch,
                                          convolution_dimensions, norm_layer, 32, pad)  # fmt: skip
            self.down_blocks.append(blk)
        self.conv_norm_out = _norm(norm_layer, ch, 32)
        self.conv_act = nn.SiLU()
        extra = {LogVarianceType.PER_CHANNEL: out_channels, LogVarianceType.UNIFORM: 1, LogVarianceType.CONSTANT: 1, LogVarianceType.NONE: 0}
        self.conv_out = _conv(convolution_dimensions, ch, out_channels + extra[latent_log_var], pad=pad)

    def forward(self, sample):
        """[B, 3, 1 + 8k, H, W] in [-1, 1] -> normalised latent means [B, 128, 1 + k, H / 32, W / 32]."""
        crop = (sample.shape[2] - 1) % 8
        if crop:
            sample = sample[:, :, :-crop]
        x = self.conv_in(patchify(sample, self.patch_size, 1))
        for blk in self.down_blocks:
            x = blk(x)
        x = self.conv_out(self.conv_act(self.conv_norm_out(x)))
        if self.latent_log_var == LogVarianceType.UNIFORM and x.shape[1] < 2:
            raise ValueError("uniform log-variance needs at least two output channels")
        return self.per_channel_statistics.normalize(x[:, : self.latent_channels])

    def tiled_encode(self, video, tile_size=(64, 512), tile_stride=(40, 448)):
        p = next(self.parameters())
        crop = (video.shape[2] - 1) % VIDEO_SCALE_FACTORS.time
        if crop:
            video = video[:, :, :-crop]
        b, _, f, h, w = video.shape
        shape = VideoLatentShape.from_pixels(b, f, h, w, self.latent_channels)
        tiles = prepare_tiles_for_encoding(video, tile_size[1], tile_size[1] - tile_stride[1], tile_size[0], tile_size[0] - tile_stride[0])
        out = torch.zeros(shape.to_torch_shape(), device=p.device, dtype=p.dtype)
        weight = torch.zeros_like(out)
        for t in tiles:
            mask = t.blend_mask.to(out)
            out[t.out_coords] += self.forward(video[t.in_coords].to(out)) * mask
            weight[t.out_coords] += mask
        return out / weight.clamp(min=1e-8)


class VideoDecoder(nn.Module):
    def __init__(self, convolution_dimensions=3, in_channels: int = 128, out_channels: int = 3, decoder_blocks=(), patch_size: int = 4,
                 norm_layer: NormLayerType = NormLayerType.PIXEL_NORM, causal: bool = False, timestep_conditioning: bool = False,
                 decoder_spatial_padding_mode: PaddingModeType = PaddingModeType.REFLECT, base_channels: int = 128) -> None:  # fmt: skip
        super().__init__()
        self.video_downscale_factors = VIDEO_SCALE_FACTORS
        self.patch_size, self.causal, self.timestep_conditioning = patch_size, causal, timestep_conditioning
        self.per_channel_statistics = PerChannelStatistics(in_channels)
        self.decode_noise_scale, self.decode_timestep = 0.025, 0.05
        pad, ch = decoder_spatial_padding_mode, base_channels * 8
        self.conv_in = _conv(convolution_dimensions, in_channels, ch, pad=pad)
        self.up_blocks = nn.ModuleList()
        for name, params in reversed(list(decoder_blocks)):
            blk, ch = _make_decoder_block(name, {"num_layers": params} if isinstance(params, int) else params, ch,
                                          convolution_dimensions, norm_layer, timestep_conditioning, 32, pad)  # fmt: skip
            self.up_blocks.append(blk)
        self.conv_norm_out = _norm(norm_layer, ch, 32)
        self.conv_act = nn.SiLU()
        self.conv_out = _conv(convolution_dimensions, ch, out_channels * patch_size**2, pad=pad)
        if timestep_conditioning:
            self.timestep_scale_multiplier = nn.Parameter(torch.tensor(1000.0))
            self.last_time_embedder = PixArtAlphaCombinedTimestepSizeEmbeddings(ch * 2, 0)
            self.last_scale_shift_table = nn.Parameter(torch.zeros(2, ch))

    def forward(self, sample, timestep=None, generator=None):
        """Normalised latents [B, 128, 1 + k, h, w] -> pixels [B, 3, 1 + 8k, 32h, 32w]."""
        B = sample.shape[0]
        scaled_t = None
        if self.timestep_conditioning:
            noise = torch.randn(sample.size(), generator=generator, dtype=sample.dtype, device=sample.device) * self.decode_noise_scale
            sample = noise + (1.0 - self.decode_noise_scale) * sample
        x = self.per_channel_statistics.un_normalize(sample)
        if self.timestep_conditioning:
            if timestep is None:
                timestep = torch.full((B,), self.decode_timestep, device=x.device, dtype=x.dtype)
            scaled_t = timestep * self.timestep_scale_multiplier.to(x)
        x = self.conv_in(x, causal=self.causal)
        for blk in self.up_blocks:
            if isinstance(blk, UNetMidBlock3D):
                x = blk(x, causal=self.causal, timestep=scaled_t, generator=generator)
            elif isinstance(blk, ResnetBlock3D):
                x = blk(x, causal=self.causal, generator=generator)
            else:
                x = blk(x, causal=self.causal)
        x = self.conv_norm_out(x)
        if self.timestep_conditioning:
            emb = self.last_time_embedder(scaled_t.flatten().float()).view(B, 2, -1, 1, 1, 1).to(x)
            shift, scale = (self.last_scale_shift_table[None, ..., None, None, None].to(x) + emb).unbind(dim=1)
            x = x * (1 + scale) + shift
        return unpatchify(self.conv_out(self.conv_act(x), causal=self.causal), self.patch_size, 1)

    def _prepare_tiles(self, latent, tile_size=(64, 512), tile_stride=(40, 448)) -> list:
        splitters, mappers = [None] * 5, [None] * 5
        t_size, s_size = tile_size
        s_overlap, t_overlap = s_size - tile_stride[1], t_size - tile_stride[0]
        _validate_tiling(s_size, s_overlap, 64, 32, "spatial")
        _validate_tiling(t_size, t_overlap, 16, 8, "temporal")
        long_side = max(latent.shape[3], latent.shape[4])
        for axis, factor in ((3, self.video_downscale_factors.height), (4, self.video_downscale_factors.width)):
            overlap = s_overlap // factor
            size = max(max(2, overlap + 1), round((s_size // factor) * latent.shape[axis] / long_side))
            splitters[axis], mappers[axis] = split_with_symmetric_overlaps(size, overlap), (map_spatial_interval_to_pixel, factor)
        t = self.video_downscale_factors.time
        splitters[2], mappers[2] = split_temporal_latents(t_size // t, t_overlap // t), (map_temporal_interval_to_frame, t)
        return create_tiles(latent.shape, splitters, mappers)

    def _decode_group(self, tiles: list, buffer, latent, timestep, generator):
        """Decode the tiles of one temporal window into `buffer`; returns the accumulated blend weights."""
        t0 = tiles[0].out_coords[2].start
        weights = torch.zeros_like(buffer)
        for tile in tiles:
            dec = self.forward(latent[tile.in_coords], timestep, generator)
            mask = tile.blend_mask.to(buffer)
            off = tile.out_coords[2].start - t0
            n = min(tile.out_coords[2].stop - tile.out_coords[2].start, dec.shape[2], buffer.shape[2] - off)
            where = (slice(None), slice(None), slice(off, off + n), tile.out_coords[3], tile.out_coords[4])
            m = mask[:, :, :n] if mask.shape[2] > 1 else mask
            buffer[where] += dec[:, :, :n] * m
            weights[where] += m
        return weights

    def tiled_decode(self, latent, tile_size=(64, 512), tile_stride=(40, 448), timestep=None, generator=None) -> Iterator[torch.Tensor]:
        """Yields consecutive pixel chunks; a chunk is released once the next window has been blended into its tail."""
        full = VideoLatentShape.from_torch_shape(latent.shape).upscale(self.video_downscale_factors)
        groups: list = []
        for tile in self._prepare_tiles(latent, tile_size, tile_stride):
            if groups and groups[-1][0].out_coords[2] == tile.out_coords[2]:
                groups[-1].append(tile)
            else:
                groups.append([tile])
        prev = prev_w = prev_slice = None
        for group in groups:
            cur = group[0].out_coords[2]
            buf = torch.zeros(full._replace(frames=cur.stop - cur.start).to_torch_shape(), device=latent.device, dtype=latent.dtype)
            w = self._decode_group(group, buf, latent, timestep, generator)
            if prev is not None:
                if prev_slice.stop > cur.start:
                    n = prev_slice.stop - cur.start
                    tail = slice(cur.start - prev_slice.start, None)
                    prev[:, :, tail] += buf[:, :, :n]
                    prev_w[:, :, tail] += w[:, :, :n]
                    buf[:, :, :n] = prev[:, :, tail]
                    w[:, :, :n] = prev_w[:, :, tail]
                yield (prev / prev_w.clamp(min=1e-8))[:, :, : cur.start - prev_slice.start]
            prev, prev_w, prev_slice = buf, w, cur
        if prev is not None:
            yield prev / prev_w.clamp(min=1e-8)


def decode_video(latent, video_decoder: VideoDecoder, tiled: bool = False, tile_size=(64, 512), tile_stride=(40, 448), generator=None):
    if tiled:
        yield from video_decoder.tiled_decode(latent, tile_size=tile_size, tile_stride=tile_stride, generator=generator)
    else:
        yield video_decoder(latent, generator=generator)


def get_video_chunks_number(num_frames: int, tiled: bool = False, tile_size=(64, 512), tile_stride=(40, 448)) -> int:
    return (num_frames - 1 + tile_stride[0] - 1) // tile_stride[0] if tiled else 1


def _vae_kwargs(config: dict) -> dict:
    c = config.get("vae", config)
    return dict(convolution_dimensions=c.get("dims", 3), in_channels=c.get("in_channels", 3), out_channels=c.get("out_channels", 3),
                latent_channels=c.get("latent_channels", 128), encoder_blocks=tuple(c.get("encoder_blocks", DEFAULT_LTX23_ENCODER_BLOCKS)),
                decoder_blocks=tuple(c.get("decoder_blocks", DEFAULT_LTX23_DECODER_BLOCKS)), patch_size=c.get("patch_size", 4),
                norm_layer=NormLayerType(c.get("norm_layer", "pixel_norm")), latent_log_var=LogVarianceType(c.get("latent_log_var", "uniform")),
                causal_decoder=c.get("causal_decoder", False), timestep_conditioning=c.get("timestep_conditioning", False),
                spatial_padding_mode=PaddingModeType(c.get("spatial_padding_mode", "zeros")),
                decoder_base_channels=c.get("decoder_base_channels", 128))  # fmt: skip


class VideoEncoderConfigurator:
    @classmethod
    def from_config(cls, config: dict) -> VideoEncoder:
        k = _vae_kwargs(config)
        return VideoEncoder(k["convolution_dimensions"], k["in_channels"], k["latent_channels"], config.get("vae", config).get("encoder_blocks", []),
                            k["patch_size"], k["norm_layer"], k["latent_log_var"], k["spatial_padding_mode"])  # fmt: skip


class VideoDecoderConfigurator:
    @classmethod
    def from_config(cls, config: dict) -> VideoDecoder:
        k = _vae_kwargs(config)
        return VideoDecoder(k["convolution_dimensions"], k["latent_channels"], k["out_channels"], config.get("vae", config).get("decoder_blocks", []),
                            k["patch_size"], k["norm_layer"], k["causal_decoder"], k["timestep_conditioning"], k["spatial_padding_mode"],
                            k["decoder_base_channels"])  # fmt: skip


class LTXVideoVAE(BaseModel):
    def __init__(self, convolution_dimensions=3, in_channels: int = 3, out_channels: int = 3, latent_channels: int = 128,
                 encoder_blocks=DEFAULT_LTX23_ENCODER_BLOCKS, decoder_blocks=DEFAULT_LTX23_DECODER_BLOCKS, patch_size: int = 4,
                 norm_layer: NormLayerType = NormLayerType.PIXEL_NORM, latent_log_var: LogVarianceType = LogVarianceType.UNIFORM,
                 causal_decoder: bool = False, timestep_conditioning: bool = False,
                 spatial_padding_mode: PaddingModeType = PaddingModeType.ZEROS, decoder_base_channels: int = 128) -> None:  # fmt: skip
        super().__init__()
        self.encoder = VideoEncoder(convolution_dimensions, in_channels, latent_channels, list(encoder_blocks), patch_size, norm_layer,
                                    latent_log_var, spatial_padding_mode)  # fmt: skip
        self.decoder = VideoDecoder(convolution_dimensions, latent_channels, out_channels, list(decoder_blocks), patch_size, norm_layer,
                                    causal_decoder, timestep_conditioning, spatial_padding_mode, decoder_base_channels)  # fmt: skip
        self.parallelism = 1

    @classmethod
    def from_config(cls, config: dict) -> "LTXVideoVAE":
        return cls(**_vae_kwargs(config))

    @property
    def per_channel_statistics(self) -> nn.Module:
        return self.encoder.per_channel_statistics

    def set_parallelism(self, parallelism: int) -> None:
        self.parallelism = parallelism

    def encode(self, video, tiled: bool = False, tile_size=(64, 512), tile_stride=(40, 448)):
        return self.encoder.tiled_encode(video, tile_size, tile_stride) if tiled else self.encoder(video)

    def decode(self, latent, tiled: bool = False, tile_size=(64, 512), tile_stride=(40, 448), timestep=None, generator=None):
        if tiled:
            yield from self.decoder.tiled_decode(latent, tile_size, tile_stride, timestep, generator)
        else:
            yield self.decoder(latent, timestep=timestep, generator=generator)

    @staticmethod
    def state_dict_converter():
        return LTXVideoVAEStateDictConverter()


class LTXVideoVAEStateDictConverter:
    """The shared checkpoint keeps `vae.encoder.*`, `vae.decoder.*` and one `vae.per_channel_statistics.*` for both halves."""

    def from_official(self, sd: dict):
        out = {}
        for k, v in sd.items():
            if k.startswith("vae.encoder.") or k.startswith("vae.decoder."):
                out[k[len("vae."):]] = v
            elif k.startswith("vae.per_channel_statistics."):
                suffix = k[len("vae.per_channel_statistics."):]
                if suffix in ("std-of-means", "mean-of-means"):
                    out["encoder.per_channel_statistics." + suffix] = v
                    out["decoder.per_channel_statistics." + suffix] = v
        return (out or dict(sd)), {}

    from_diffusers = from_official


LTXVideoDecoder = VideoDecoder
LTXVideoEncoder = VideoEncoder
