"""HunyuanVideo-1.5 causal 3-D VAE (32 latent channels at 16 x 16 x 4 in the released config) and its latent
super-resolution upsamplers.

Every conv is causal in time (replicate padding, all temporal padding in front). Down / up-samplers are
space-to-depth / depth-to-space rearrangements around a conv, with an averaged (down) or repeated (up) shortcut;
where time is resampled the first frame is handled on its own so that 1 + 4k frames map to 1 + k latents. The
middle block attends frame-causally over all positions. Encoder and decoder add a channel-folded shortcut around
their last / first conv. Spatial tiling blends overlapping tiles linearly; `use_slicing` runs samples one by one.
Convolutions run through cuDNN; norms, rearrangements and blending are PyTorch.
Role parity: telefuser/models/hunyuan_video_vae.py:39-850, telefuser/models/hunyuan_video_upsampler.py:20-320.
"""

from __future__ import annotations

import json
import math
import os
from contextlib import contextmanager
from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from telefuser_b200.core.base_model import BaseModel
from telefuser_b200.ops import functional as TF


class RMSNorm(nn.Module):
    def __init__(self, dim: int, channel_first: bool = True, images: bool = True, bias: bool = False) -> None:
        super().__init__()
        shape = (dim, *((1, 1) if images else (1, 1, 1))) if channel_first else (dim,)
        self.channel_first, self.scale = channel_first, dim**0.5
        self.gamma = nn.Parameter(torch.ones(shape))
        self.bias = nn.Parameter(torch.zeros(shape)) if bias else None

    def forward(self, x):
        y = F.normalize(x, dim=1 if self.channel_first else -1) * self.scale * self.gamma
        return y if self.bias is None else y + self.bias


class CausalConv3d(nn.Module):
    def __init__(self, chan_in: int, chan_out: int, kernel_size: int, stride: int = 1, dilation: int = 1, pad_mode: str = "replicate",
                 disable_causal: bool = False, **kwargs) -> None:  # fmt: skip
        super().__init__()
        k = kernel_size // 2
        self.pad_mode = pad_mode
        self.time_causal_padding = (k,) * 6 if disable_causal else (k, k, k, k, kernel_size - 1, 0)
        self.conv = nn.Conv3d(chan_in, chan_out, kernel_size, stride=stride, dilation=dilation, **kwargs)

    def forward(self, x):
        return self.conv(F.pad(x, self.time_causal_padding, mode=self.pad_mode))


def frame_causal_mask(n_frame: int, n_hw: int, device) -> torch.Tensor:
    """bool [S, S]: a position sees every position of its own and earlier frames."""
    frame = torch.arange(n_frame * n_hw, device=device) // n_hw
    return frame[:, None] >= frame[None, :]


class AttnBlock(nn.Module):
    def __init__(self, in_channels: int) -> None:
        super().__init__()
        self.in_channels = in_channels
        self.norm = RMSNorm(in_channels, images=False)
        self.q, self.k, self.v, self.proj_out = (nn.Conv3d(in_channels, in_channels, 1) for _ in range(4))

    def forward(self, x):
        h = self.norm(x)
        b, c, f, hh, ww = h.shape
        q, k, v = (m(h).flatten(2).transpose(1, 2).unsqueeze(2) for m in (self.q, self.k, self.v))
        mask = None if f == 1 else frame_causal_mask(f, hh * ww, h.device)
        o = TF.attention(q, k, v, mask=mask)
        return x + self.proj_out(o.squeeze(2).transpose(1, 2).reshape(b, c, f, hh, ww))


class ResnetBlock(nn.Module):
    def __init__(self, in_channels: int, out_channels: int | None = None) -> None:
        super().__init__()
        out_channels = out_channels or in_channels
        self.in_channels, self.out_channels = in_channels, out_channels
        self.norm1, self.conv1 = RMSNorm(in_channels, images=False), CausalConv3d(in_channels, out_channels, 3)
        self.norm2, self.conv2 = RMSNorm(out_channels, images=False), CausalConv3d(out_channels, out_channels, 3)
        if in_channels != out_channels:
            self.nin_shortcut = nn.Conv3d(in_channels, out_channels, 1)

    def forward(self, x):
        h = self.conv2(F.silu(self.norm2(self.conv1(F.silu(self.norm1(x))))))
        return (self.nin_shortcut(x) if self.in_channels != self.out_channels else x) + h


def _fold(x, r1: int):
    """b c (f r1) (h 2) (w 2) -> b (r1 2 2 c) f h w"""
    b, c, f, h, w = x.shape
    x = x.reshape(b, c, f // r1, r1, h // 2, 2, w // 2, 2).permute(0, 3, 5, 7, 1, 2, 4, 6)
    return x.reshape(b, r1 * 4 * c, f // r1, h // 2, w // 2)


def _unfold(x, r1: int):
    """b (r1 2 2 c) f h w -> b c (f r1) (h 2) (w 2)"""
    b, c, f, h, w = x.shape
    n = c // (r1 * 4)
    x = x.reshape(b, r1, 2, 2, n, f, h, w).permute(0, 4, 5, 1, 6, 2, 7, 3)
    return x.reshape(b, n, f * r1, h * 2, w * 2)


class Downsample(nn.Module):
    def __init__(self, in_channels: int, out_channels: int, add_temporal_downsample: bool = True) -> None:
        super().__init__()
        factor = 8 if add_temporal_downsample else 4
        if out_channels % factor:
            raise ValueError("downsample output channels must be a multiple of the folding factor")
        self.conv = CausalConv3d(in_channels, out_channels // factor, 3)
        self.add_temporal_downsample, self.group_size = add_temporal_downsample, factor * in_channels // out_channels

    def _avg(self, x, channels: int, group: int):
        return x.unflatten(1, (channels, group)).mean(dim=2)

    def forward(self, x):
        h = self.conv(x)
        if not self.add_temporal_downsample:
            h = _fold(h, 1)
            return h + self._avg(_fold(x, 1), h.shape[1], self.group_size)
        h_first = _fold(h[:, :, :1], 1)
        h = torch.cat([torch.cat([h_first, h_first], dim=1), _fold(h[:, :, 1:], 2)], dim=2)
        c = h.shape[1]
        skip = torch.cat([self._avg(_fold(x[:, :, :1], 1), c, self.group_size // 2), self._avg(_fold(x[:, :, 1:], 2), c, self.group_size)], dim=2)
        return h + skip


class Upsample(nn.Module):
    def __init__(self, in_channels: int, out_channels: int, add_temporal_upsample: bool = True) -> None:
        super().__init__()
        factor = 8 if add_temporal_upsample else 4
        self.conv = CausalConv3d(in_channels, out_channels * factor, 3)
        self.add_temporal_upsample, self.repeats = add_temporal_upsample, factor * out_channels // in_channels

    def forward(self, x):
        h = self.conv(x)
        if not self.add_temporal_upsample:
            return _unfold(h, 1) + _unfold(x.repeat_interleave(self.repeats, dim=1), 1)
        h_first = _unfold(h[:, :, :1], 1)
        h = torch.cat([h_first[:, : h_first.shape[1] // 2], _unfold(h[:, :, 1:], 2)], dim=2)
        skip = torch.cat([_unfold(x[:, :, :1], 1).repeat_interleave(self.repeats // 2, dim=1),
                          _unfold(x[:, :, 1:], 2).repeat_interleave(self.repeats, dim=1)], dim=2)  # fmt: skip
        return h + skip


class _Level(nn.Module):
    def __init__(self) -> None:
        super().__init__()
        self.block = nn.ModuleList()


class _Mid(nn.Module):
    def __init__(self, channels: int) -> None:
        super().__init__()
        self.block_1, self.attn_1, self.block_2 = ResnetBlock(channels, channels), AttnBlock(channels), ResnetBlock(channels, channels)

    def forward(self, x):
        return self.block_2(self.attn_1(self.block_1(x)))


class Encoder(nn.Module):
    def __init__(self, in_channels: int, z_channels: int, block_out_channels, num_res_blocks: int, ffactor_spatial: int, ffactor_temporal: int,
                 downsample_match_channel: bool = True) -> None:  # fmt: skip
        super().__init__()
        if block_out_channels[-1] % (2 * z_channels):
            raise ValueError("the last encoder width must be a multiple of 2 * z_channels")
        self.z_channels, self.block_out_channels, self.num_res_blocks = z_channels, tuple(block_out_channels), num_res_blocks
        self.conv_in = CausalConv3d(in_channels, block_out_channels[0], 3)
        self.down = nn.ModuleList()
        cin = block_out_channels[0]
        for i, ch in enumerate(block_out_channels):
            level = _Level()
            for _ in range(num_res_blocks):
                level.block.append(ResnetBlock(cin, ch))
                cin = ch
            spatial = i < math.log2(ffactor_spatial)
            temporal = spatial and i >= math.log2(ffactor_spatial / ffactor_temporal)
            if spatial or temporal:
                cout = block_out_channels[i + 1] if downsample_match_channel else cin
                level.downsample = Downsample(cin, cout, temporal)
                cin = cout
            self.down.append(level)
        self.mid = _Mid(cin)
        self.norm_out = RMSNorm(cin, images=False)
        self.conv_out = CausalConv3d(cin, 2 * z_channels, 3)

    def forward(self, x):
        h = self.conv_in(x)
        for level in self.down:
            for blk in level.block:
                h = blk(h)
            if hasattr(level, "downsample"):
                h = level.downsample(h)
        h = self.mid(h)
        skip = h.unflatten(1, (2 * self.z_channels, -1)).mean(dim=2)
        return self.conv_out(F.silu(self.norm_out(h))) + skip


class Decoder(nn.Module):
    def __init__(self, z_channels: int, out_channels: int, block_out_channels, num_res_blocks: int, ffactor_spatial: int, ffactor_temporal: int,
                 upsample_match_channel: bool = True) -> None:  # fmt: skip
        super().__init__()
        if block_out_channels[0] % z_channels:
            raise ValueError("the first decoder width must be a multiple of z_channels")
        self.z_channels, self.block_out_channels, self.num_res_blocks = z_channels, tuple(block_out_channels), num_res_blocks
        cin = block_out_channels[0]
        self.conv_in = CausalConv3d(z_channels, cin, 3)
        self.mid = _Mid(cin)
        self.up = nn.ModuleList()
        for i, ch in enumerate(block_out_channels):
            level = _Level()
            for _ in range(num_res_blocks + 1):
                level.block.append(ResnetBlock(cin, ch))
                cin = ch
            spatial, temporal = i < math.log2(ffactor_spatial), i < math.log2(ffactor_temporal)
            if spatial or temporal:
                cout = block_out_channels[i + 1] if upsample_match_channel else cin
                level.upsample = Upsample(cin, cout, temporal)
                cin = cout
            self.up.append(level)
        self.norm_out = RMSNorm(cin, images=False)
        self.conv_out = CausalConv3d(cin, out_channels, 3)

    def forward(self, z):
        h = self.conv_in(z) + z.repeat_interleave(self.block_out_channels[0] // self.z_channels, dim=1)
        h = self.mid(h)
        for level in self.up:
            for blk in level.block:
                h = blk(h)
            if hasattr(level, "upsample"):
                h = level.upsample(h)
        return self.conv_out(F.silu(self.norm_out(h)))


class DiagonalGaussianDistribution:
    def __init__(self, parameters: torch.Tensor, deterministic: bool = False) -> None:
        self.parameters = parameters
        self.mean, logvar = parameters.chunk(2, dim=1)
        self.logvar = logvar.clamp(-30.0, 20.0)
        self.deterministic = deterministic
        self.std, self.var = torch.exp(0.5 * self.logvar), torch.exp(self.logvar)
        if deterministic:
            self.std = self.var = torch.zeros_like(self.mean)

    def sample(self, generator=None):
        noise = torch.randn(self.mean.shape, generator=generator, device=self.parameters.device if generator is None else generator.device,
                            dtype=self.parameters.dtype)  # fmt: skip
        return self.mean + self.std * noise.to(self.parameters.device)

    def kl(self, other=None):
        if self.deterministic:
            return torch.zeros(1, device=self.mean.device)
        dims = list(range(1, self.mean.dim()))
        if other is None:
            return 0.5 * torch.sum(self.mean.pow(2) + self.var - 1.0 - self.logvar, dim=dims)
        return 0.5 * torch.sum((self.mean - other.mean).pow(2) / other.var + self.var / other.var - 1.0 - self.logvar + other.logvar, dim=dims)

    def mode(self):
        return self.mean


@dataclass
class AutoencoderKLOutput:
    latent_dist: DiagonalGaussianDistribution


@dataclass
class DecoderOutput:
    sample: torch.Tensor
    posterior: DiagonalGaussianDistribution | None = None


def _blend(prev, cur, extent: int, dim: int):
    """Linear cross-fade of the first `extent` entries of `cur` along `dim` with the last `extent` of `prev`."""
    extent = min(prev.shape[dim], cur.shape[dim], extent)
    if extent <= 0:
        return cur
    shape = [1] * cur.dim()
    shape[dim] = extent
    w = (torch.arange(extent, device=cur.device, dtype=cur.dtype) / extent).view(shape)
    head = prev.narrow(dim, prev.shape[dim] - extent, extent) * (1 - w) + cur.narrow(dim, 0, extent) * w
    return torch.cat([head, cur.narrow(dim, extent, cur.shape[dim] - extent)], dim=dim)


class HunyuanVideoVAE(BaseModel):
    def __init__(self, in_channels: int = 3, out_channels: int = 3, latent_channels: int = 16, block_out_channels=(128, 256, 512, 512),
                 layers_per_block: int = 2, ffactor_spatial: int = 8, ffactor_temporal: int = 4, scaling_factor: float = 0.476986,
                 shift_factor: float | None = None, sample_size: int = 256, sample_tsize: int = 64) -> None:  # fmt: skip
        super().__init__()
        self.ffactor_spatial, self.ffactor_temporal = ffactor_spatial, ffactor_temporal
        self.scaling_factor, self.shift_factor = scaling_factor, shift_factor
        self.encoder = Encoder(in_channels, latent_channels, tuple(block_out_channels), layers_per_block, ffactor_spatial, ffactor_temporal)
        self.decoder = Decoder(latent_channels, out_channels, tuple(reversed(block_out_channels)), layers_per_block, ffactor_spatial, ffactor_temporal)
        self.use_slicing = self.use_spatial_tiling = False
        self.tile_sample_min_size, self.tile_latent_min_size = sample_size, sample_size // ffactor_spatial
        self.tile_sample_min_tsize, self.tile_latent_min_tsize = sample_tsize, sample_tsize // ffactor_temporal
        self.tile_overlap_factor = 0.25

    @classmethod
    def from_pretrained(cls, path: str, torch_dtype: torch.dtype = torch.float32, **kwargs) -> "HunyuanVideoVAE":
        from telefuser_b200.utils.model_weight import load_state_dict

        with open(os.path.join(path, "config.json")) as f:
            cfg = json.load(f)
        keys = ("in_channels", "out_channels", "latent_channels", "block_out_channels", "layers_per_block", "ffactor_spatial", "ffactor_temporal",
                "scaling_factor", "shift_factor", "sample_size", "sample_tsize")  # fmt: skip
        model = cls(**{k: cfg[k] for k in keys if k in cfg})
        for name in ("diffusion_pytorch_model.safetensors", "diffusion_pytorch_model.bin"):
            if os.path.isfile(os.path.join(path, name)):
                model.load_state_dict(load_state_dict(os.path.join(path, name)), strict=False)
                return model.to(torch_dtype)
        raise FileNotFoundError(f"no VAE weights under {path}")

    # ---- tiling / slicing switches -------------------------------------------------------------
    def set_tile_sample_min_size(self, sample_size: int, tile_overlap_factor: float = 0.2) -> None:
        self.tile_sample_min_size, self.tile_latent_min_size = sample_size, sample_size // self.ffactor_spatial
        self.tile_overlap_factor = tile_overlap_factor

    def enable_spatial_tiling(self, use_tiling: bool = True) -> None:
        self.use_spatial_tiling = use_tiling

    def disable_spatial_tiling(self) -> None:
        self.use_spatial_tiling = False

    enable_tiling, disable_tiling = enable_spatial_tiling, disable_spatial_tiling

    def enable_slicing(self) -> None:
        self.use_slicing = True

    def disable_slicing(self) -> None:
        self.use_slicing = False

    @contextmanager
    def memory_efficient_context(self):
        saved = (self.use_slicing, self.use_spatial_tiling)
        self.use_slicing = self.use_spatial_tiling = True
        try:
            yield
        finally:
            self.use_slicing, self.use_spatial_tiling = saved

    def _tiled(self, x, net: nn.Module, tile_in: int, tile_out: int):
        """Run `net` on overlapping square tiles of side `tile_in`; cross-fade and crop in the output domain."""
        stride = int(tile_in * (1 - self.tile_overlap_factor))
        extent = int(tile_out * self.tile_overlap_factor)
        keep = tile_out - extent
        rows = [[net(x[..., i : i + tile_in, j : j + tile_in]) for j in range(0, x.shape[-1], stride)] for i in range(0, x.shape[-2], stride)]
        out_rows = []
        for i, row in enumerate(rows):
            out = []
            for j, tile in enumerate(row):
                if i > 0:
                    tile = _blend(rows[i - 1][j], tile, extent, -2)
                if j > 0:
                    tile = _blend(row[j - 1], tile, extent, -1)
                row[j] = tile  # the neighbours below / to the right fade against the blended tile
                out.append(tile[..., :keep, :keep])
            out_rows.append(torch.cat(out, dim=-1))
        return torch.cat(out_rows, dim=-2)

    def spatial_tiled_encode(self, x):
        return self._tiled(x, self.encoder, self.tile_sample_min_size, self.tile_latent_min_size)

    def spatial_tiled_decode(self, z):
        return self._tiled(z, self.decoder, self.tile_latent_min_size, self.tile_sample_min_size)

    def _run(self, x, plain: nn.Module, tiled, limit: int):
        def one(t):
            return tiled(t) if self.use_spatial_tiling and max(t.shape[-2:]) > limit else plain(t)

        return torch.cat([one(s) for s in x.split(1)]) if self.use_slicing and x.shape[0] > 1 else one(x)

    def encode(self, x, return_dict: bool = True):
        """Video [B, 3, 1 + 4k, H, W] -> posterior over latents [B, C, 1 + k, H / s, W / s] (unscaled)."""
        if x.dim() != 5:
            raise ValueError("expected [B, C, T, H, W]")
        posterior = DiagonalGaussianDistribution(self._run(x, self.encoder, self.spatial_tiled_encode, self.tile_sample_min_size))
        return AutoencoderKLOutput(posterior) if return_dict else (posterior,)

    def decode(self, z, return_dict: bool = True, generator=None):
        dec = self._run(z, self.decoder, self.spatial_tiled_decode, self.tile_latent_min_size)
        return DecoderOutput(dec) if return_dict else (dec,)

    def forward(self, sample, sample_posterior: bool = False, return_posterior: bool = True, return_dict: bool = True):
        posterior = self.encode(sample).latent_dist
        dec = self.decode(posterior.sample() if sample_posterior else posterior.mode()).sample
        if not return_dict:
            return (dec, posterior) if return_posterior else (dec,)
        return DecoderOutput(dec, posterior if return_posterior else None)

    # ---- scaled-latent helpers used by the pipeline ----------------------------------------------
    def encode_latents(self, x, sample: bool = False, generator=None):
        dist = self.encode(x).latent_dist
        return (dist.sample(generator) if sample else dist.mode()) * self.scaling_factor

    def decode_latents(self, z, memory_efficient: bool = True):
        if not memory_efficient:
            return self.decode(z / self.scaling_factor).sample
        with self.memory_efficient_context():
            return self.decode(z / self.scaling_factor).sample

    def get_latent_size(self, video_size):
        t, h, w = video_size
        return t // self.ffactor_temporal, h // self.ffactor_spatial, w // self.ffactor_spatial

    def get_video_size(self, latent_size):
        t, h, w = latent_size
        return t * self.ffactor_temporal, h * self.ffactor_spatial, w * self.ffactor_spatial

    @staticmethod
    def state_dict_converter():
        return HunyuanVideoVAEStateDictConverter()


class HunyuanVideoVAEStateDictConverter:
    def from_official(self, sd: dict):
        out = {(k[4:] if k.startswith("vae.") else k): v for k, v in sd.items()}
        width = out["encoder.conv_in.conv.weight"].shape[0] if "encoder.conv_in.conv.weight" in out else 128
        z = out["decoder.conv_in.conv.weight"].shape[1] if "decoder.conv_in.conv.weight" in out else 16
        widths, i = [width], 0
        while f"encoder.down.{i}.downsample.conv.conv.weight" in out:
            i += 1
            widths.append(out[f"encoder.down.{i}.block.0.conv1.conv.weight"].shape[1])
        while f"encoder.down.{len(widths)}.block.0.conv1.conv.weight" in out:
            widths.append(out[f"encoder.down.{len(widths)}.block.0.conv1.conv.weight"].shape[0])
        return out, {"latent_channels": z, "block_out_channels": widths}

    from_diffusers = from_official


# ---- latent super-resolution ---------------------------------------------------------------------
class SRResidualCausalBlock3D(nn.Module):
    def __init__(self, channels: int) -> None:
        super().__init__()
        self.block = nn.Sequential(CausalConv3d(channels, channels, 3), nn.SiLU(), CausalConv3d(channels, channels, 3), nn.SiLU(),
                                   CausalConv3d(channels, channels, 3))  # fmt: skip

    def forward(self, x):
        return x + self.block(x)


def resize_latents(z, target_hw):
    """Bilinear resize of every latent frame to `target_hw`."""
    if target_hw is None or tuple(z.shape[-2:]) == tuple(target_hw):
        return z
    b, c, f, h, w = z.shape
    y = F.interpolate(z.transpose(1, 2).reshape(b * f, c, h, w), size=tuple(target_hw), mode="bilinear", align_corners=False)
    return y.reshape(b, f, c, *target_hw).transpose(1, 2)


class SRTo720pUpsampler(nn.Module):
    """Refines bilinearly resized 480p latents: conv, residual causal blocks, conv (optionally plus the input)."""

    def __init__(self, in_channels: int = 32, out_channels: int = 32, hidden_channels: int | None = None, num_blocks: int = 6,
                 global_residual: bool = False) -> None:  # fmt: skip
        super().__init__()
        hidden_channels = hidden_channels or 64
        self.in_conv = CausalConv3d(in_channels, hidden_channels, 3)
        self.blocks = nn.ModuleList([SRResidualCausalBlock3D(hidden_channels) for _ in range(num_blocks)])
        self.out_conv = CausalConv3d(hidden_channels, out_channels, 3)
        self.global_residual = bool(global_residual)
        self.config = dict(in_channels=in_channels, out_channels=out_channels, hidden_channels=hidden_channels, num_blocks=num_blocks,
                           global_residual=global_residual)  # fmt: skip

    def forward(self, x):
        y = self.in_conv(x)
        for blk in self.blocks:
            y = blk(y)
        y = self.out_conv(y)
        return y + x if self.global_residual and y.shape == x.shape else y

    @classmethod
    def from_pretrained(cls, path: str, torch_dtype: torch.dtype = torch.float32, **kwargs):
        return _load_upsampler(cls, path, torch_dtype, ("in_channels", "out_channels", "hidden_channels", "num_blocks", "global_residual"))


class SRTo1080pUpsampler(nn.Module):
    """720p -> 1080p: resize, then a decoder-style residual stack with a channel-repeated input shortcut."""

    def __init__(self, z_channels: int = 32, out_channels: int = 32, block_out_channels=(128, 256), num_res_blocks: int = 2,
                 is_residual: bool = False) -> None:  # fmt: skip
        super().__init__()
        self.num_res_blocks, self.block_out_channels, self.z_channels, self.is_residual = num_res_blocks, tuple(block_out_channels), z_channels, is_residual
        cin = block_out_channels[0]
        self.conv_in = CausalConv3d(z_channels, cin, 3)
        self.up = nn.ModuleList()
        for ch in block_out_channels:
            level = _Level()
            for _ in range(num_res_blocks + 1):
                level.block.append(ResnetBlock(cin, ch))
                cin = ch
            self.up.append(level)
        self.norm_out = RMSNorm(cin, images=False)
        self.conv_out = CausalConv3d(cin, out_channels, 3)
        self.config = dict(z_channels=z_channels, out_channels=out_channels, block_out_channels=tuple(block_out_channels),
                           num_res_blocks=num_res_blocks, is_residual=is_residual)  # fmt: skip

    def forward(self, z, target_shape=None):
        z = resize_latents(z, target_shape)
        h = self.conv_in(z) + z.repeat_interleave(self.block_out_channels[0] // self.z_channels, dim=1)
        for level in self.up:
            for blk in level.block:
                h = blk(h)
        return self.conv_out(F.silu(self.norm_out(h)))

    @classmethod
    def from_pretrained(cls, path: str, torch_dtype: torch.dtype = torch.float32, **kwargs):
        return _load_upsampler(cls, path, torch_dtype, ("z_channels", "out_channels", "block_out_channels", "num_res_blocks", "is_residual"))


def _load_upsampler(cls, path: str, torch_dtype, keys):
    from telefuser_b200.utils.model_weight import load_state_dict

    cfg = {}
    if os.path.isfile(os.path.join(path, "config.json")):
        with open(os.path.join(path, "config.json")) as f:
            cfg = json.load(f)
    model = cls(**{k: cfg[k] for k in keys if k in cfg})
    for name in ("diffusion_pytorch_model.safetensors", "diffusion_pytorch_model.bin", "model.safetensors"):
        if os.path.isfile(os.path.join(path, name)):
            model.load_state_dict(load_state_dict(os.path.join(path, name)), strict=False)
            return model.to(torch_dtype)
    raise FileNotFoundError(f"no upsampler weights under {path}")
