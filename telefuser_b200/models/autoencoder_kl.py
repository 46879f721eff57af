"""2-D KL image autoencoder in the diffusers parameter layout (FLUX.1 / FLUX.2 / Z-Image VAEs).

Encoder: conv_in, `len(block_out_channels)` down blocks (ResNet pairs, stride-2 conv with (0,1,0,1) padding
between levels), mid block (ResNet, single-head attention, ResNet), GroupNorm+SiLU+conv_out to 2x latent
channels (mean, log-variance). Decoder mirrors it with nearest-neighbour 2x upsampling and one more ResNet
per level. The FLUX.2 variant adds a parameter-free BatchNorm over the 2x2-patchified latent whose running
statistics normalise what the transformer sees. The reference takes these classes from the diffusers package
(telefuser/pipelines/flux2_klein/pipeline.py:17, telefuser/pipelines/z_image/pipeline.py); here they are part
of the framework so that no external model code is needed.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.nn.functional as F
from torch import nn

from telefuser_b200.ops import functional as TF


@dataclass
class AutoencoderKLConfig:
    in_channels: int = 3
    out_channels: int = 3
    latent_channels: int = 16
    block_out_channels: tuple = (128, 256, 512, 512)
    layers_per_block: int = 2
    norm_num_groups: int = 32
    use_quant_conv: bool = False
    use_post_quant_conv: bool = False
    mid_block_add_attention: bool = True
    scaling_factor: float = 0.3611
    shift_factor: float | None = 0.1159
    batch_norm: bool = False  # FLUX.2: statistics over the patchified latent (4 x latent_channels)
    batch_norm_eps: float = 1e-4
    patch_size: tuple = field(default_factory=lambda: (2, 2))

    @classmethod
    def flux2(cls) -> "AutoencoderKLConfig":
        return cls(latent_channels=32, use_quant_conv=True, use_post_quant_conv=True, batch_norm=True,
                   scaling_factor=1.0, shift_factor=None)  # fmt: skip


class ResnetBlock2D(nn.Module):
    def __init__(self, cin: int, cout: int, groups: int) -> None:
        super().__init__()
        self.norm1 = nn.GroupNorm(groups, cin, eps=1e-6)
        self.conv1 = nn.Conv2d(cin, cout, 3, padding=1)
        self.norm2 = nn.GroupNorm(groups, cout, eps=1e-6)
        self.conv2 = nn.Conv2d(cout, cout, 3, padding=1)
        self.conv_shortcut = nn.Conv2d(cin, cout, 1) if cin != cout else None

    def forward(self, x):
        h = self.conv1(F.silu(self.norm1(x)))
        h = self.conv2(F.silu(self.norm2(h)))
        return h + (x if self.conv_shortcut is None else self.conv_shortcut(x))


class SpatialAttention(nn.Module):
    """Single-head self attention over the H*W positions of the bottleneck."""

    def __init__(self, ch: int, groups: int) -> None:
        super().__init__()
        self.group_norm = nn.GroupNorm(groups, ch, eps=1e-6)
        self.to_q, self.to_k, self.to_v = (nn.Linear(ch, ch) for _ in range(3))
        self.to_out = nn.ModuleList([nn.Linear(ch, ch)])

    def forward(self, x):
        B, C, H, W = x.shape
        h = self.group_norm(x).flatten(2).transpose(1, 2)  # [B, HW, C]
        q, k, v = (lin(h).unsqueeze(2) for lin in (self.to_q, self.to_k, self.to_v))
        o = TF.attention(q, k, v).squeeze(2)
        return x + self.to_out[0](o).transpose(1, 2).reshape(B, C, H, W)


class _Sampler(nn.Module):
    def __init__(self, ch: int, down: bool) -> None:
        super().__init__()
        self.down = down
        self.conv = nn.Conv2d(ch, ch, 3, stride=2 if down else 1, padding=0 if down else 1)

    def forward(self, x):
        if self.down:
            return self.conv(F.pad(x, (0, 1, 0, 1)))
        return self.conv(F.interpolate(x, scale_factor=2.0, mode="nearest"))


class _Level(nn.Module):
    def __init__(self, cin: int, cout: int, n: int, groups: int, sampler: str | None) -> None:
        super().__init__()
        self.resnets = nn.ModuleList([ResnetBlock2D(cin if i == 0 else cout, cout, groups) for i in range(n)])
        if sampler == "down":
            self.downsamplers = nn.ModuleList([_Sampler(cout, True)])
        elif sampler == "up":
            self.upsamplers = nn.ModuleList([_Sampler(cout, False)])

    def forward(self, x):
        for r in self.resnets:
            x = r(x)
        for s in getattr(self, "downsamplers", getattr(self, "upsamplers", ())):
            x = s(x)
        return x


class _Mid(nn.Module):
    def __init__(self, ch: int, groups: int, attention: bool) -> None:
        super().__init__()
        self.attentions = nn.ModuleList([SpatialAttention(ch, groups)] if attention else [])
        self.resnets = nn.ModuleList([ResnetBlock2D(ch, ch, groups) for _ in range(2)])

    def forward(self, x):
        x = self.resnets[0](x)
        for a in self.attentions:
            x = a(x)
        return self.resnets[1](x)


class Encoder2D(nn.Module):
    def __init__(self, c: AutoencoderKLConfig) -> None:
        super().__init__()
        ch = c.block_out_channels
        self.conv_in = nn.Conv2d(c.in_channels, ch[0], 3, padding=1)
        self.down_blocks = nn.ModuleList(
            [_Level(ch[max(i - 1, 0)], ch[i], c.layers_per_block, c.norm_num_groups, "down" if i < len(ch) - 1 else None)
             for i in range(len(ch))])  # fmt: skip
        self.mid_block = _Mid(ch[-1], c.norm_num_groups, c.mid_block_add_attention)
        self.conv_norm_out = nn.GroupNorm(c.norm_num_groups, ch[-1], eps=1e-6)
        self.conv_out = nn.Conv2d(ch[-1], 2 * c.latent_channels, 3, padding=1)

    def forward(self, x):
        x = self.conv_in(x)
        for b in self.down_blocks:
            x = b(x)
        return self.conv_out(F.silu(self.conv_norm_out(self.mid_block(x))))


class Decoder2D(nn.Module):
    def __init__(self, c: AutoencoderKLConfig) -> None:
        super().__init__()
        ch = tuple(reversed(c.block_out_channels))
        self.conv_in = nn.Conv2d(c.latent_channels, ch[0], 3, padding=1)
        self.mid_block = _Mid(ch[0], c.norm_num_groups, c.mid_block_add_attention)
        self.up_blocks = nn.ModuleList(
            [_Level(ch[max(i - 1, 0)], ch[i], c.layers_per_block + 1, c.norm_num_groups, "up" if i < len(ch) - 1 else None)
             for i in range(len(ch))])  # fmt: skip
        self.conv_norm_out = nn.GroupNorm(c.norm_num_groups, ch[-1], eps=1e-6)
        self.conv_out = nn.Conv2d(ch[-1], c.out_channels, 3, padding=1)

    def forward(self, z):
        x = self.mid_block(self.conv_in(z))
        for b in self.up_blocks:
            x = b(x)
        return self.conv_out(F.silu(self.conv_norm_out(x)))


class DiagonalGaussian:
    def __init__(self, moments: torch.Tensor) -> None:
        self.mean, logvar = moments.chunk(2, dim=1)
        self.logvar = logvar.clamp(-30.0, 20.0)

    def mode(self) -> torch.Tensor:
        return self.mean

    def sample(self, generator=None) -> torch.Tensor:
        noise = torch.randn(self.mean.shape, generator=generator, device=self.mean.device, dtype=self.mean.dtype)
        return self.mean + torch.exp(0.5 * self.logvar) * noise


class AutoencoderKL(nn.Module):
    def __init__(self, config: AutoencoderKLConfig | None = None) -> None:
        super().__init__()
        c = self.config = config or AutoencoderKLConfig()
        self.encoder, self.decoder = Encoder2D(c), Decoder2D(c)
        self.quant_conv = nn.Conv2d(2 * c.latent_channels, 2 * c.latent_channels, 1) if c.use_quant_conv else None
        self.post_quant_conv = nn.Conv2d(c.latent_channels, c.latent_channels, 1) if c.use_post_quant_conv else None
        if c.batch_norm:
            n = c.latent_channels * c.patch_size[0] * c.patch_size[1]
            self.bn = nn.BatchNorm2d(n, eps=c.batch_norm_eps, affine=False, track_running_stats=True)

    @property
    def spatial_factor(self) -> int:
        return 2 ** (len(self.config.block_out_channels) - 1)

    def encode(self, x: torch.Tensor) -> DiagonalGaussian:
        m = self.encoder(x)
        return DiagonalGaussian(m if self.quant_conv is None else self.quant_conv(m))

    def decode(self, z: torch.Tensor) -> torch.Tensor:
        return self.decoder(z if self.post_quant_conv is None else self.post_quant_conv(z))

    def latent_stats(self, device, dtype) -> tuple[torch.Tensor, torch.Tensor]:
        """(mean, std) [1, C, 1, 1] of the patchified latent from the BatchNorm running statistics."""
        mean = self.bn.running_mean.view(1, -1, 1, 1).to(device, dtype)
        std = torch.sqrt(self.bn.running_var.view(1, -1, 1, 1).to(device, dtype) + self.config.batch_norm_eps)
        return mean, std


def _register() -> None:
    from telefuser_b200.core.model_registry import register_architecture

    register_architecture("flux2_vae", AutoencoderKL, lambda: AutoencoderKL(AutoencoderKLConfig.flux2()), resource="diffusers")
    register_architecture("flux_vae", AutoencoderKL, lambda: AutoencoderKL(), resource="diffusers")


_register()
