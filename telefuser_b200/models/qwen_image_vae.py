"""Qwen-Image VAE (16 latent channels, 8 x 8 spatial) for single images.

The checkpoint is a causal video VAE (3-D convs, temporal resamplers). An image is one frame, and with one
frame a causal 3-D conv whose time padding is all zeros in front reduces to a 2-D conv with the last temporal tap
of its kernel; the temporal resamplers are skipped. So the weights keep the checkpoint's 5-D layout (strict
loading), while the forward pass runs 2-D channels-last convs on that tap: a third of the FLOPs and no 5-D
tensors. Norms are L2-normalise * sqrt(C) * gamma over channels; the middle block has single-head attention.
Role parity: telefuser/models/qwen_image_vae.py:11-643.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from telefuser_b200.core.base_model import BaseModel
from telefuser_b200.ops import functional as TF

LATENT_MEAN = [-0.7571, -0.7089, -0.9113, 0.1075, -0.1745, 0.9653, -0.1517, 1.5508, 0.4134, -0.0715, 0.5517, -0.3632, -0.1922, -0.9497,
               0.2503, -0.2921]  # fmt: skip
LATENT_STD = [2.8184, 1.4541, 2.3275, 2.6558, 1.2196, 1.7708, 2.6052, 2.0743, 3.2687, 2.1526, 2.8652, 1.5579, 1.6382, 1.1253, 2.8251,
              1.9160]  # fmt: skip


class QwenImageCausalConv3d(nn.Conv3d):
    """Holds a [O, I, kt, kh, kw] kernel; `forward` takes one frame [B, C, H, W] and applies the last temporal tap."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride=1, padding=0) -> None:
        super().__init__(in_channels, out_channels, kernel_size, stride=stride, padding=padding)
        self._spatial_padding = (self.padding[1], self.padding[2])
        self.padding = (0, 0, 0)

    def forward(self, x):
        return F.conv2d(x, self.weight[:, :, -1], self.bias, stride=self.stride[1:], padding=self._spatial_padding)


class QwenImageRMS_norm(nn.Module):  # noqa: N801
    def __init__(self, dim: int, channel_first: bool = True, images: bool = True, bias: bool = False) -> None:
        super().__init__()
        tail = (1, 1) if images else (1, 1, 1)
        shape = (dim, *tail) if channel_first else (dim,)
        self.channel_first, self.scale = channel_first, dim**0.5
        self.gamma = nn.Parameter(torch.ones(shape))
        self.bias = nn.Parameter(torch.zeros(shape)) if bias else None

    def forward(self, x):
        """x: one frame [B, C, H, W] (channel_first) or [..., C]."""
        if self.channel_first:
            g = self.gamma.reshape(1, -1, 1, 1)
            y = F.normalize(x, dim=1) * self.scale * g
            return y if self.bias is None else y + self.bias.reshape(1, -1, 1, 1)
        y = F.normalize(x, dim=-1) * self.scale * self.gamma
        return y if self.bias is None else y + self.bias


class QwenImageResidualBlock(nn.Module):
    def __init__(self, in_dim: int, out_dim: int, dropout: float = 0.0, non_linearity: str = "silu") -> None:
        super().__init__()
        self.in_dim, self.out_dim = in_dim, out_dim
        self.norm1 = QwenImageRMS_norm(in_dim, images=False)
        self.conv1 = QwenImageCausalConv3d(in_dim, out_dim, 3, padding=1)
        self.norm2 = QwenImageRMS_norm(out_dim, images=False)
        self.conv2 = QwenImageCausalConv3d(out_dim, out_dim, 3, padding=1)
        self.conv_shortcut = QwenImageCausalConv3d(in_dim, out_dim, 1) if in_dim != out_dim else nn.Identity()

    def forward(self, x):
        h = self.conv1(F.silu(self.norm1(x)))
        return self.conv2(F.silu(self.norm2(h))) + self.conv_shortcut(x)


class QwenImageAttentionBlock(nn.Module):
    def __init__(self, dim: int) -> None:
        super().__init__()
        self.dim = dim
        self.norm = QwenImageRMS_norm(dim)
        self.to_qkv = nn.Conv2d(dim, dim * 3, 1)
        self.proj = nn.Conv2d(dim, dim, 1)

    def forward(self, x):
        b, c, h, w = x.shape
        q, k, v = self.to_qkv(self.norm(x)).reshape(b, 1, 3 * c, h * w).permute(0, 3, 1, 2).chunk(3, dim=-1)
        o = TF.attention(q, k, v)  # [b, h w, 1, c]: one head of width c
        return x + self.proj(o.squeeze(2).transpose(1, 2).reshape(b, c, h, w))


class QwenImageResample(nn.Module):
    def __init__(self, dim: int, mode: str) -> None:
        super().__init__()
        self.dim, self.mode = dim, mode
        if mode in ("upsample2d", "upsample3d"):
            self.resample = nn.Sequential(nn.Upsample(scale_factor=(2.0, 2.0), mode="nearest-exact"), nn.Conv2d(dim, dim // 2, 3, padding=1))
            if mode == "upsample3d":
                self.time_conv = QwenImageCausalConv3d(dim, dim * 2, (3, 1, 1), padding=(1, 0, 0))
        elif mode in ("downsample2d", "downsample3d"):
            self.resample = nn.Sequential(nn.ZeroPad2d((0, 1, 0, 1)), nn.Conv2d(dim, dim, 3, stride=(2, 2)))
            if mode == "downsample3d":
                self.time_conv = QwenImageCausalConv3d(dim, dim, (3, 1, 1), stride=(2, 1, 1), padding=(0, 0, 0))
        else:
            self.resample = nn.Identity()

    def forward(self, x):
        if self.mode.startswith("upsample"):
            return self.resample[1](self.resample[0](x.float()).type_as(x))
        return self.resample(x)  # the temporal convs only act from the second frame of a video on


class QwenImageMidBlock(nn.Module):
    def __init__(self, dim: int, dropout: float = 0.0, non_linearity: str = "silu", num_layers: int = 1) -> None:
        super().__init__()
        self.dim = dim
        self.resnets = nn.ModuleList([QwenImageResidualBlock(dim, dim, dropout) for _ in range(num_layers + 1)])
        self.attentions = nn.ModuleList([QwenImageAttentionBlock(dim) for _ in range(num_layers)])

    def forward(self, x):
        x = self.resnets[0](x)
        for attn, res in zip(self.attentions, self.resnets[1:]):
            x = res(attn(x))
        return x


class QwenImageEncoder3d(nn.Module):
    def __init__(self, dim: int = 128, z_dim: int = 4, dim_mult=(1, 2, 4, 4), num_res_blocks: int = 2, attn_scales=(),
                 temperal_downsample=(True, True, False), dropout: float = 0.0, non_linearity: str = "silu") -> None:  # fmt: skip
        super().__init__()
        dims = [dim * u for u in [1, *dim_mult]]
        scale = 1.0
        self.conv_in = QwenImageCausalConv3d(3, dims[0], 3, padding=1)
        self.down_blocks = nn.ModuleList()
        for i, (cin, cout) in enumerate(zip(dims[:-1], dims[1:])):
            for _ in range(num_res_blocks):
                self.down_blocks.append(QwenImageResidualBlock(cin, cout, dropout))
                if scale in attn_scales:
                    self.down_blocks.append(QwenImageAttentionBlock(cout))
                cin = cout
            if i != len(dim_mult) - 1:
                self.down_blocks.append(QwenImageResample(cout, "downsample3d" if temperal_downsample[i] else "downsample2d"))
                scale /= 2.0
        self.mid_block = QwenImageMidBlock(cout, dropout, non_linearity, 1)
        self.norm_out = QwenImageRMS_norm(cout, images=False)
        self.conv_out = QwenImageCausalConv3d(cout, z_dim, 3, padding=1)

    def forward(self, x):
        x = self.conv_in(x)
        for layer in self.down_blocks:
            x = layer(x)
        return self.conv_out(F.silu(self.norm_out(self.mid_block(x))))


class QwenImageUpBlock(nn.Module):
    def __init__(self, in_dim: int, out_dim: int, num_res_blocks: int, dropout: float = 0.0, upsample_mode: str | None = None,
                 non_linearity: str = "silu") -> None:  # fmt: skip
        super().__init__()
        self.in_dim, self.out_dim = in_dim, out_dim
        self.resnets = nn.ModuleList([QwenImageResidualBlock(in_dim if i == 0 else out_dim, out_dim, dropout) for i in range(num_res_blocks + 1)])
        self.upsamplers = nn.ModuleList([QwenImageResample(out_dim, upsample_mode)]) if upsample_mode is not None else None

    def forward(self, x):
        for res in self.resnets:
            x = res(x)
        return x if self.upsamplers is None else self.upsamplers[0](x)


class QwenImageDecoder3d(nn.Module):
    def __init__(self, dim: int = 128, z_dim: int = 4, dim_mult=(1, 2, 4, 4), num_res_blocks: int = 2, attn_scales=(),
                 temperal_upsample=(False, True, True), dropout: float = 0.0, non_linearity: str = "silu") -> None:  # fmt: skip
        super().__init__()
        dims = [dim * u for u in [dim_mult[-1], *dim_mult[::-1]]]
        self.conv_in = QwenImageCausalConv3d(z_dim, dims[0], 3, padding=1)
        self.mid_block = QwenImageMidBlock(dims[0], dropout, non_linearity, 1)
        self.up_blocks = nn.ModuleList()
        for i, (cin, cout) in enumerate(zip(dims[:-1], dims[1:])):
            mode = None if i == len(dim_mult) - 1 else ("upsample3d" if temperal_upsample[i] else "upsample2d")
            self.up_blocks.append(QwenImageUpBlock(cin // 2 if i > 0 else cin, cout, num_res_blocks, dropout, mode, non_linearity))
        self.norm_out = QwenImageRMS_norm(cout, images=False)
        self.conv_out = QwenImageCausalConv3d(cout, 3, 3, padding=1)

    def forward(self, x):
        x = self.mid_block(self.conv_in(x))
        for blk in self.up_blocks:
            x = blk(x)
        return self.conv_out(F.silu(self.norm_out(x)))


class QwenImageVAE(BaseModel):
    def __init__(self, base_dim: int = 96, z_dim: int = 16, dim_mult=(1, 2, 4, 4), num_res_blocks: int = 2, attn_scales=(),
                 temperal_downsample=(False, True, True), dropout: float = 0.0) -> None:  # fmt: skip
        super().__init__()
        self.z_dim, self.temperal_downsample, self.temperal_upsample = z_dim, list(temperal_downsample), list(temperal_downsample)[::-1]
        self.encoder = QwenImageEncoder3d(base_dim, z_dim * 2, list(dim_mult), num_res_blocks, list(attn_scales), self.temperal_downsample, dropout)
        self.quant_conv = QwenImageCausalConv3d(z_dim * 2, z_dim * 2, 1)
        self.post_quant_conv = QwenImageCausalConv3d(z_dim, z_dim, 1)
        self.decoder = QwenImageDecoder3d(base_dim, z_dim, list(dim_mult), num_res_blocks, list(attn_scales), self.temperal_upsample, dropout)
        self.mean = torch.tensor(LATENT_MEAN[:z_dim] if z_dim <= 16 else LATENT_MEAN).view(1, -1, 1, 1)
        self.std = 1.0 / torch.tensor(LATENT_STD[:z_dim] if z_dim <= 16 else LATENT_STD).view(1, -1, 1, 1)

    def _stats(self, x):
        return self.mean.to(x), self.std.to(x)

    def encode(self, x, **kwargs):
        """Image [B, 3, H, W] in [-1, 1] -> normalised latent mean [B, 16, H / 8, W / 8]."""
        x = x.contiguous(memory_format=torch.channels_last)
        z = self.quant_conv(self.encoder(x))[:, : self.z_dim]
        mean, inv_std = self._stats(z)
        return (z - mean) * inv_std

    def decode(self, z, **kwargs):
        mean, inv_std = self._stats(z)
        z = (z / inv_std + mean).contiguous(memory_format=torch.channels_last)
        return self.decoder(self.post_quant_conv(z))

    @staticmethod
    def state_dict_converter():
        return QwenImageVAEStateDictConverter()


class QwenImageVAEStateDictConverter:
    def from_diffusers(self, sd: dict):
        return dict(sd), {}

    from_official = from_diffusers


def _register() -> None:
    from telefuser_b200.core.model_registry import register_architecture

    register_architecture("qwen_image_vae", QwenImageVAE, lambda: QwenImageVAE(), resource="diffusers")


_register()
