"""Wan2.2 causal video VAE (48 latent channels, stride 4 x 16 x 16).

Pixels are 2x2 pixel-unshuffled to 12 channels, then a causal 3-D pyramid (widths dim*[1,2,4,4], encoder
dim 160, decoder dim 256) compresses 4 x 8 x 8. Each pyramid level is a residual group whose shortcut is
parameter free: group-averaged space/time-to-channel on the way down (`AvgDown3D`), channel-duplicating
channel-to-space/time on the way up (`DupUp3D`, dropping the duplicated first frame of a stream). The causal
convolution state, chunked encode / decode, tiling, 2-D spatial parallel decode and streaming are those of
the 16-channel VAE (`wan_vae`), whose building blocks are reused.
Role parity: telefuser/models/wan22_video_vae.py:24-1548.
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from telefuser_b200.models.wan_vae import (AttentionBlock, CausalConv3d, CausalState, Resample, ResidualBlock, RMS_norm,
                                           VideoVAE, WanVideoVAE, WanVideoVAEStateDictConverter, _run, causal_step,
                                           count_causal_slots)  # fmt: skip

WAN22_VAE_MEAN = [-0.2289, -0.0052, -0.1323, -0.2339, -0.2799, 0.0174, 0.1838, 0.1557, -0.1382, 0.0542, 0.2813, 0.0891,
                  0.1570, -0.0098, 0.0375, -0.1825, -0.2246, -0.1207, -0.0698, 0.5109, 0.2665, -0.2108, -0.2158, 0.2502,
                  -0.2055, -0.0322, 0.1109, 0.1567, -0.0729, 0.0899, -0.2799, -0.1230, -0.0313, -0.1649, 0.0117, 0.0723,
                  -0.2839, -0.2083, -0.0520, 0.3748, 0.0152, 0.1957, 0.1433, -0.2944, 0.3573, -0.0548, -0.1681, -0.0667]  # fmt: skip
WAN22_VAE_STD = [0.4765, 1.0364, 0.4514, 1.1677, 0.5313, 0.4990, 0.4818, 0.5013, 0.8158, 1.0344, 0.5894, 1.0901,
                 0.6885, 0.6165, 0.8454, 0.4978, 0.5759, 0.3523, 0.7135, 0.6804, 0.5833, 1.4146, 0.8986, 0.5659,
                 0.7069, 0.5338, 0.4889, 0.4917, 0.4069, 0.4999, 0.6866, 0.4093, 0.5709, 0.6065, 0.6415, 0.4944,
                 0.5726, 1.2042, 0.5458, 1.6887, 0.3971, 1.0600, 0.3943, 0.5537, 0.5444, 0.4089, 0.7468, 0.7744]  # fmt: skip


def patchify(x: torch.Tensor, p: int = 2) -> torch.Tensor:
    """[B, C, T, H, W] -> [B, C*p*p, T, H/p, W/p]; channel order (c, column offset, row offset)."""
    if p == 1:
        return x
    B, C, T, H, W = x.shape
    x = x.view(B, C, T, H // p, p, W // p, p)  # b c f h q w r
    return x.permute(0, 1, 6, 4, 2, 3, 5).reshape(B, C * p * p, T, H // p, W // p)


def unpatchify(x: torch.Tensor, p: int = 2) -> torch.Tensor:
    if p == 1:
        return x
    B, C, T, H, W = x.shape
    x = x.view(B, C // (p * p), p, p, T, H, W)  # b c r q f h w
    return x.permute(0, 1, 4, 5, 3, 6, 2).reshape(B, C // (p * p), T, H * p, W * p)


class AvgDown3D(nn.Module):
    """Space/time-to-channel followed by a mean over groups of channels (no parameters)."""

    def __init__(self, in_channels: int, out_channels: int, factor_t: int, factor_s: int = 1) -> None:
        super().__init__()
        self.out_channels, self.factor_t, self.factor_s = out_channels, factor_t, factor_s
        self.factor = factor_t * factor_s * factor_s
        if in_channels * self.factor % out_channels:
            raise ValueError("channel counts do not divide")
        self.group_size = in_channels * self.factor // out_channels

    def forward(self, x):
        ft, fs = self.factor_t, self.factor_s
        x = F.pad(x, (0, 0, 0, 0, (ft - x.shape[2] % ft) % ft, 0))
        B, C, T, H, W = x.shape
        x = x.view(B, C, T // ft, ft, H // fs, fs, W // fs, fs).permute(0, 1, 3, 5, 7, 2, 4, 6)
        x = x.reshape(B, self.out_channels, self.group_size, T // ft, H // fs, W // fs)
        return x.mean(dim=2)


class DupUp3D(nn.Module):
    """Channel duplication followed by channel-to-space/time (no parameters)."""

    def __init__(self, in_channels: int, out_channels: int, factor_t: int, factor_s: int = 1) -> None:
        super().__init__()
        self.out_channels, self.factor_t, self.factor_s = out_channels, factor_t, factor_s
        self.factor = factor_t * factor_s * factor_s
        if out_channels * self.factor % in_channels:
            raise ValueError("channel counts do not divide")
        self.repeats = out_channels * self.factor // in_channels

    def forward(self, x, first_chunk: bool = False):
        ft, fs = self.factor_t, self.factor_s
        B, _, T, H, W = x.shape
        x = x.repeat_interleave(self.repeats, dim=1).view(B, self.out_channels, ft, fs, fs, T, H, W)
        x = x.permute(0, 1, 5, 2, 6, 3, 7, 4).reshape(B, self.out_channels, T * ft, H * fs, W * fs)
        return x[:, :, ft - 1 :] if first_chunk else x


class Down_ResidualBlock(nn.Module):
    def __init__(self, in_dim: int, out_dim: int, dropout: float, mult: int, temperal_downsample: bool = False,
                 down_flag: bool = False) -> None:  # fmt: skip
        super().__init__()
        self.avg_shortcut = AvgDown3D(in_dim, out_dim, 2 if temperal_downsample else 1, 2 if down_flag else 1)
        layers = []
        for _ in range(mult):
            layers.append(ResidualBlock(in_dim, out_dim, dropout))
            in_dim = out_dim
        if down_flag:
            layers.append(Resample(out_dim, "downsample3d" if temperal_downsample else "downsample2d"))
        self.downsamples = nn.Sequential(*layers)

    def forward(self, x, state: CausalState | None = None):
        return _run(self.downsamples, x, state) + self.avg_shortcut(x)


class Up_ResidualBlock(nn.Module):
    def __init__(self, in_dim: int, out_dim: int, dropout: float, mult: int, temperal_upsample: bool = False,
                 up_flag: bool = False) -> None:  # fmt: skip
        super().__init__()
        self.avg_shortcut = DupUp3D(in_dim, out_dim, 2 if temperal_upsample else 1, 2) if up_flag else None
        layers = []
        for _ in range(mult):
            layers.append(ResidualBlock(in_dim, out_dim, dropout))
            in_dim = out_dim
        if up_flag:
            layers.append(Resample(out_dim, "upsample3d" if temperal_upsample else "upsample2d", keep_width=True))
        self.upsamples = nn.Sequential(*layers)

    def forward(self, x, state: CausalState | None = None, first_chunk: bool = False):
        y = _run(self.upsamples, x, state)
        return y if self.avg_shortcut is None else y + self.avg_shortcut(x, first_chunk)


class Encoder3d(nn.Module):
    def __init__(self, dim=160, z_dim=96, dim_mult=(1, 2, 4, 4), num_res_blocks=2, temperal_downsample=(False, True, True),
                 dropout=0.0) -> None:  # fmt: skip
        super().__init__()
        dims = [dim * u for u in [1, *dim_mult]]
        self.conv1 = CausalConv3d(12, dims[0], 3, padding=1)
        self.downsamples = nn.Sequential(*[
            Down_ResidualBlock(i_d, o_d, dropout, num_res_blocks, temperal_downsample[i] if i < len(temperal_downsample) else False,
                               i != len(dim_mult) - 1)
            for i, (i_d, o_d) in enumerate(zip(dims[:-1], dims[1:]))])  # fmt: skip
        out_dim = dims[-1]
        self.middle = nn.Sequential(ResidualBlock(out_dim, out_dim, dropout), AttentionBlock(out_dim),
                                    ResidualBlock(out_dim, out_dim, dropout))  # fmt: skip
        self.head = nn.Sequential(RMS_norm(out_dim, images=False), nn.SiLU(), CausalConv3d(out_dim, z_dim, 3, padding=1))

    def forward(self, x, state: CausalState | None = None):
        x = causal_step(self.conv1, x, state)
        for blk in self.downsamples:
            x = blk(x, state)
        return _run(self.head, _run(self.middle, x, state), state)


class Decoder3d(nn.Module):
    def __init__(self, dim=256, z_dim=48, dim_mult=(1, 2, 4, 4), num_res_blocks=2, temperal_upsample=(True, True, False),
                 dropout=0.0) -> None:  # fmt: skip
        super().__init__()
        dims = [dim * u for u in [dim_mult[-1], *dim_mult[::-1]]]
        self.conv1 = CausalConv3d(z_dim, dims[0], 3, padding=1)
        self.middle = nn.Sequential(ResidualBlock(dims[0], dims[0], dropout), AttentionBlock(dims[0]),
                                    ResidualBlock(dims[0], dims[0], dropout))  # fmt: skip
        self.upsamples = nn.Sequential(*[
            Up_ResidualBlock(i_d, o_d, dropout, num_res_blocks + 1, temperal_upsample[i] if i < len(temperal_upsample) else False,
                             i != len(dim_mult) - 1)
            for i, (i_d, o_d) in enumerate(zip(dims[:-1], dims[1:]))])  # fmt: skip
        self.head = nn.Sequential(RMS_norm(dims[-1], images=False), nn.SiLU(), CausalConv3d(dims[-1], 12, 3, padding=1))

    def forward(self, x, state: CausalState | None = None):
        first = state.first_chunk if state is not None else False
        x = _run(self.middle, causal_step(self.conv1, x, state), state)
        for blk in self.upsamples:
            x = blk(x, state, first)
        return _run(self.head, x, state)


class VideoVAE22(VideoVAE):
    """Same chunked encode / decode drivers as the 16-channel model around the patchified pyramid."""

    def __init__(self, dim=160, dec_dim=256, z_dim=48, dim_mult=(1, 2, 4, 4), num_res_blocks=2,
                 temperal_downsample=(False, True, True), dropout=0.0) -> None:  # fmt: skip
        nn.Module.__init__(self)
        self.dim, self.z_dim = dim, z_dim
        self.temperal_downsample = tuple(temperal_downsample)
        self.encoder = Encoder3d(dim, z_dim * 2, dim_mult, num_res_blocks, self.temperal_downsample, dropout)
        self.conv1 = CausalConv3d(z_dim * 2, z_dim * 2, 1)
        self.conv2 = CausalConv3d(z_dim, z_dim, 1)
        self.decoder = Decoder3d(dec_dim, z_dim, dim_mult, num_res_blocks, self.temperal_downsample[::-1], dropout)

    def encode_chunk(self, frames, state: CausalState, scale):
        return super().encode_chunk(patchify(frames), state, scale)

    def encode(self, x, scale):
        return super().encode(patchify(x), scale)

    def decode_chunk(self, z, state: CausalState, scale):
        x = self.conv2(self._denormalise(z, scale))
        outs = []
        for i in range(x.shape[2]):
            state.rewind()
            outs.append(self.decoder(x[:, :, i : i + 1], state))
            state.first_chunk = False
        return unpatchify(torch.cat(outs, dim=2))


class Wan22VideoVAE(WanVideoVAE):
    def __init__(self, z_dim: int = 48, parallelism: int = 1, dim: int = 160, dec_dim: int = 256) -> None:
        super().__init__(z_dim=16, parallelism=parallelism, dim=8)  # placeholder model replaced below
        self.z_dim = z_dim
        self.mean = torch.tensor(WAN22_VAE_MEAN[:z_dim] if z_dim <= 48 else [0.0] * z_dim)
        self.std = torch.tensor(WAN22_VAE_STD[:z_dim] if z_dim <= 48 else [1.0] * z_dim)
        self.scale = [self.mean, 1.0 / self.std]
        self.model = VideoVAE22(dim=dim, dec_dim=dec_dim, z_dim=z_dim).eval().requires_grad_(False)
        self.upsampling_factor = 16

    @staticmethod
    def state_dict_converter():
        return WanVideoVAEStateDictConverter()


def _register() -> None:
    from telefuser_b200.core.model_registry import register_architecture

    register_architecture("wan22_video_vae", Wan22VideoVAE, lambda: VideoVAE22(), keys_only=False)


_register()

__all__ = ["AvgDown3D", "DupUp3D", "VideoVAE22", "Wan22VideoVAE", "count_causal_slots", "patchify", "unpatchify"]
