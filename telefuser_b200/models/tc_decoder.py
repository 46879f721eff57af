"""Tiny conditional video decoder (TAEHV layout) used by FlashVSR instead of the full VAE decoder.

A purely 2-D conv stack applied per frame, made temporal by `MemBlock`s (each sees the previous frame's input
next to the current one) and `TGrow` layers (1x1 convs that emit 2 frames per frame). The low-quality clip is
pixel-unshuffled (4 x 8 x 8) and concatenated to the latent as conditioning. Streaming: instead of walking a
per-frame work queue, a whole chunk runs as one batch and every MemBlock carries the last frame of the previous
chunk, which yields the same frames with T-times larger convolutions.
Role parity: telefuser/models/TCDecoder.py:18-352.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from telefuser_b200.utils.model_weight import hash_state_dict_keys


class IdentityConv2d(nn.Conv2d):
    def __init__(self, C: int, kernel_size: int = 3, bias: bool = False) -> None:
        super().__init__(C, C, kernel_size, padding=kernel_size // 2, bias=bias)
        with torch.no_grad():
            nn.init.dirac_(self.weight)
            if self.bias is not None:
                self.bias.zero_()


def conv(n_in: int, n_out: int, **kw):
    return nn.Conv2d(n_in, n_out, 3, padding=1, **kw)


class Clamp(nn.Module):
    def forward(self, x):
        return torch.tanh(x / 3) * 3


class MemBlock(nn.Module):
    def __init__(self, n_in: int, n_out: int) -> None:
        super().__init__()
        self.conv = nn.Sequential(conv(n_in * 2, n_out), nn.ReLU(inplace=True), conv(n_out, n_out), nn.ReLU(inplace=True),
                                  conv(n_out, n_out))  # fmt: skip
        self.skip = nn.Conv2d(n_in, n_out, 1, bias=False) if n_in != n_out else nn.Identity()
        self.act = nn.ReLU(inplace=True)

    def forward(self, x, past):
        return self.act(self.conv(torch.cat([x, past], 1)) + self.skip(x))


class TPool(nn.Module):
    def __init__(self, n_f: int, stride: int) -> None:
        super().__init__()
        self.stride = stride
        self.conv = nn.Conv2d(n_f * stride, n_f, 1, bias=False)

    def forward(self, x):
        _, C, H, W = x.shape
        return self.conv(x.reshape(-1, self.stride * C, H, W))


class TGrow(nn.Module):
    def __init__(self, n_f: int, stride: int) -> None:
        super().__init__()
        self.stride = stride
        self.conv = nn.Conv2d(n_f, n_f * stride, 1, bias=False)

    def forward(self, x):
        _, C, H, W = x.shape
        return self.conv(x).reshape(-1, C, H, W)


def pixel_unshuffle_3d(x: torch.Tensor, ff: int, hh: int, ww: int) -> torch.Tensor:
    """[B, C, F, H, W] -> [B, F/ff, C*ff*hh*ww, H/hh, W/ww]; a short clip is front-padded with its first frame."""
    B, C, F, H, W = x.shape
    if F % ff:
        x = torch.cat([x[:, :, :1].repeat(1, 1, ff - F % ff, 1, 1), x], dim=2)
        F = x.shape[2]
    x = x.view(B, C, F // ff, ff, H // hh, hh, W // ww, ww).permute(0, 1, 3, 5, 7, 2, 4, 6)
    return x.reshape(B, C * ff * hh * ww, F // ff, H // hh, W // ww).transpose(1, 2)


class TAEHV(nn.Module):
    image_channels = 3

    def __init__(self, decoder_time_upscale=(True, True), decoder_space_upscale=(True, True, True),
                 channels=(512, 256, 128, 128), latent_channels: int = 16) -> None:  # fmt: skip
        super().__init__()
        self.latent_channels = latent_channels
        n = list(channels)
        self.frames_to_trim = 2 ** sum(decoder_time_upscale) - 1
        up = lambda on: nn.Upsample(scale_factor=2 if on else 1)  # noqa: E731
        base = [Clamp(), conv(latent_channels, n[0]), nn.ReLU(inplace=True),
                MemBlock(n[0], n[0]), MemBlock(n[0], n[0]), MemBlock(n[0], n[0]), up(decoder_space_upscale[0]),
                TGrow(n[0], 1), conv(n[0], n[1], bias=False),
                MemBlock(n[1], n[1]), MemBlock(n[1], n[1]), MemBlock(n[1], n[1]), up(decoder_space_upscale[1]),
                TGrow(n[1], 2 if decoder_time_upscale[0] else 1), conv(n[1], n[2], bias=False),
                MemBlock(n[2], n[2]), MemBlock(n[2], n[2]), MemBlock(n[2], n[2]), up(decoder_space_upscale[2]),
                TGrow(n[2], 2 if decoder_time_upscale[1] else 1), conv(n[2], n[3], bias=False), nn.ReLU(inplace=True),
                conv(n[3], self.image_channels)]  # fmt: skip
        self.decoder = self._deepen(base)
        self.mem: list = [None] * len(self.decoder)
        self._started = False

    @staticmethod
    def _deepen(layers: list, k: int = 3) -> nn.Sequential:
        """After every ReLU that follows a conv (or a MemBlock) insert an identity-initialised conv + ReLU."""
        out: list = []
        for b in layers:
            out.append(b)
            if isinstance(b, nn.ReLU) and len(out) >= 2:
                prev = out[-2]
                C = prev.out_channels if isinstance(prev, nn.Conv2d) else (prev.conv[-1].out_channels if isinstance(prev, MemBlock) else None)
                if C is not None:
                    out += [IdentityConv2d(C, k, bias=False), nn.ReLU(inplace=True)]
        return nn.Sequential(*out)

    def patch_tgrow_layers(self, sd: dict) -> dict:
        own = self.state_dict()
        for i, layer in enumerate(self.decoder):
            key = f"decoder.{i}.conv.weight"
            if isinstance(layer, TGrow) and key in sd and sd[key].shape[0] > own[key].shape[0]:
                sd[key] = sd[key][-own[key].shape[0] :]
        return sd

    def clean_mem(self) -> None:
        self.mem = [None] * len(self.decoder)
        self._started = False

    @torch.no_grad()
    def decode(self, x: torch.Tensor, cond: torch.Tensor | None = None, **_unused) -> torch.Tensor:
        """x: [N, T, C, H, W] latents (NTCHW); cond: [N, 3, 4T, 8H, 8W] low-quality frames -> [N, T', 3, 8H, 8W].
        Memory persists across calls (streaming); the first call drops the `frames_to_trim` warm-up frames."""
        first = not self._started
        if cond is not None:
            x = torch.cat([pixel_unshuffle_3d(cond, 4, 8, 8).to(x), x], dim=2)
        N, T = x.shape[:2]
        h = x.reshape(N * T, *x.shape[2:])
        for i, b in enumerate(self.decoder):
            if isinstance(b, MemBlock):
                cur = h.view(N, -1, *h.shape[1:])
                head = torch.zeros_like(cur[:, :1]) if self.mem[i] is None else self.mem[i].to(cur).unsqueeze(1)
                past = torch.cat([head, cur[:, :-1]], dim=1)
                self.mem[i] = cur[:, -1].clone()
                h = b(h, past.reshape(h.shape))
            else:
                h = b(h)
        self._started = True
        out = h.view(N, -1, *h.shape[1:])
        return out[:, self.frames_to_trim :] if first else out

    def forward(self, *a, **k):
        raise NotImplementedError("decoder-only model: call decode()")

    @staticmethod
    def state_dict_converter():
        return TAEHVStateDictConverter()


class TAEHVStateDictConverter:
    def from_official(self, sd: dict):
        if hash_state_dict_keys(sd) == "4c3523c69fb7b24cf2db147a715b277f":
            return sd, dict(latent_channels=16 + 768)
        return sd, {}
