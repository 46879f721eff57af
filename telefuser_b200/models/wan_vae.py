"""Wan causal video VAE (16 latent channels, stride 4 x 8 x 8).

Architecture and state-dict keys follow the published checkpoint (and the
reference's ``telefuser/models/wan_video_vae.py:92-716``): causal 3-D convolutions,
L2-normalising RMS norm, residual blocks, single-head per-frame attention,
2x spatial resampling with optional temporal resampling. What differs is how
causality across chunks is carried: every causal convolution owns a slot in a
`CausalState` that keeps the last two input frames, so whole-video decode,
chunked decode and session streaming are the same code path and the state can be
kept per streaming session. Convolutions run channels-last-3d.

Parallel decode: `decode_dist_2d` splits the latent on a 2-D grid with a halo, each
rank decodes its tile and the tiles are all-gathered and stitched; `tiled_decode`
/ `tiled_encode` blend overlapping tiles and, across ranks, sum values and weights.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from telefuser_b200.core.base_model import BaseModel
from telefuser_b200.ops import functional as TF

CACHE_T = 2

WAN21_LATENT_MEAN = [-0.7571, -0.7089, -0.9113, 0.1075, -0.1745, 0.9653, -0.1517, 1.5508,
                     0.4134, -0.0715, 0.5517, -0.3632, -0.1922, -0.9497, 0.2503, -0.2921]  # fmt: skip
WAN21_LATENT_STD = [2.8184, 1.4541, 2.3275, 2.6558, 1.2196, 1.7708, 2.6052, 2.0743,
                    3.2687, 2.1526, 2.8652, 1.5579, 1.6382, 1.1253, 2.8251, 1.9160]  # fmt: skip


class CausalState:
    """Per-convolution tails of the input seen so far (one slot per causal conv, in call order)."""

    def __init__(self, num_slots: int):
        self.slots: list = [None] * num_slots
        self.cursor = 0
        self.first_chunk = True

    def rewind(self) -> None:
        self.cursor = 0

    def next_slot(self) -> int:
        i = self.cursor
        self.cursor += 1
        return i


class CausalConv3d(nn.Conv3d):
    """Conv3d that pads time on the left only; the pad can be supplied from the previous chunk."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self._pad_t = 2 * self.padding[0]
        self._pad_hw = (self.padding[2], self.padding[2], self.padding[1], self.padding[1])
        self.padding = (0, 0, 0)

    def _native_ok(self, x) -> bool:
        """The tensor-core kernel covers stride-1, undilated, ungrouped convolutions with "same" spatial padding."""
        kt, kh, kw = self.kernel_size
        return (x.is_cuda and x.dtype == torch.bfloat16 and self.weight.dtype == torch.bfloat16
                and self.stride == (1, 1, 1) and self.dilation == (1, 1, 1) and self.groups == 1
                and self._pad_hw == ((kw - 1) // 2, (kw - 1) // 2, (kh - 1) // 2, (kh - 1) // 2)
                and self._pad_t == kt - 1 and self.in_channels % 8 == 0
                and (self.out_channels % 8 == 0 or self.out_channels <= 32) and TF.use_native_kernels(x))  # fmt: skip

    def _taps(self):
        w = self.weight
        key = (w.data_ptr(), w._version, w.device)
        if getattr(self, "_taps_key", None) != key:
            self._taps_cache, self._taps_key = TF.conv_weight_taps(w), key
        return self._taps_cache

    def forward(self, x, prev=None, residual=None):
        if self._native_ok(x):
            # implicit GEMM on the tensor cores: padding (and `prev`) are read in place, nothing is copied or padded
            return TF.conv3d_causal(x, self.weight, self.bias, prev, residual, self._pad_t, self._taps())
        y = self._forward_library(x, prev)
        return y if residual is None else y + residual

    def _forward_library(self, x, prev=None):
        pad_t = self._pad_t
        if prev is not None and pad_t > 0:
            prev = prev.to(x.device)
            x = torch.cat([prev, x], dim=2)
            pad_t -= prev.shape[2]
        x = F.pad(x, (*self._pad_hw, max(pad_t, 0), 0))
        if x.is_cuda:
            x = x.contiguous(memory_format=torch.channels_last_3d)
        return super().forward(x)


def _fast(x) -> bool:
    """CUDA bf16 activations take the native path: channels-last throughout, norm + SiLU in one pass, convolutions as
    implicit GEMMs on the tensor cores with the residual added in their epilogue."""
    return x.is_cuda and x.dtype == torch.bfloat16 and TF.use_native_kernels(x)


def causal_step(conv: CausalConv3d, x, state: CausalState | None, residual=None):
    """Runs `conv` on a chunk, feeding it the stored tail and storing the new tail."""
    if state is None:
        return conv(x, None, residual)
    i = state.next_slot()
    old = state.slots[i]
    tail = x[:, :, -CACHE_T:].clone()
    if tail.shape[2] < CACHE_T and old is not None:
        tail = torch.cat([old[:, :, -1:].to(tail.device), tail], dim=2)
    y = conv(x, old, residual)
    state.slots[i] = tail
    return y


class RMS_norm(nn.Module):
    def __init__(self, dim: int, channel_first: bool = True, images: bool = True, bias: bool = False):
        super().__init__()
        bdims = (1, 1, 1) if not images else (1, 1)
        shape = (dim, *bdims) if channel_first else (dim,)
        self.channel_first = channel_first
        self.scale = dim**0.5
        self.gamma = nn.Parameter(torch.ones(shape))
        self.bias = nn.Parameter(torch.zeros(shape)) if bias else 0.0

    def forward(self, x):
        return F.normalize(x, dim=(1 if self.channel_first else -1)) * self.scale * self.gamma + self.bias


class Upsample(nn.Upsample):
    def forward(self, x):
        return super().forward(x.float()).type_as(x)


class Resample(nn.Module):
    def __init__(self, dim: int, mode: str, keep_width: bool = False):
        assert mode in ("none", "upsample2d", "upsample3d", "downsample2d", "downsample3d")
        super().__init__()
        self.dim, self.mode = dim, mode
        if mode in ("upsample2d", "upsample3d"):
            # the 16-channel VAE halves the width in the upsampling conv, the 48-channel one keeps it
            self.resample = nn.Sequential(Upsample(scale_factor=(2.0, 2.0), mode="nearest-exact"),
                                          nn.Conv2d(dim, dim if keep_width else dim // 2, 3, padding=1))  # fmt: skip
            if mode == "upsample3d":
                self.time_conv = CausalConv3d(dim, dim * 2, (3, 1, 1), padding=(1, 0, 0))
        elif mode in ("downsample2d", "downsample3d"):
            self.resample = nn.Sequential(nn.ZeroPad2d((0, 1, 0, 1)), nn.Conv2d(dim, dim, 3, stride=(2, 2)))
            if mode == "downsample3d":
                self.time_conv = CausalConv3d(dim, dim, (3, 1, 1), stride=(2, 1, 1), padding=(0, 0, 0))
        else:
            self.resample = nn.Identity()

    def _spatial(self, x):
        b, c, t, h, w = x.shape
        if self.mode in ("upsample2d", "upsample3d") and _fast(x) and c % 8 == 0:
            # frames as a batch of channels-last images: 2x nearest upsample, then the 3x3 convolution as an implicit
            # GEMM (a 3-D convolution with one tap in time over the frame axis)
            conv = self.resample[1]
            img = x.permute(0, 2, 1, 3, 4).reshape(b * t, c, h, w)
            up = TF.upsample2x_nearest(img)  # [b*t, c, 2h, 2w] channels-last
            vol = up.permute(1, 0, 2, 3).unsqueeze(0)  # [1, c, b*t, 2h, 2w], channels-last-3d strides, no copy
            key = (conv.weight.data_ptr(), conv.weight._version)
            if getattr(self, "_taps_key", None) != key:
                self._taps_cache, self._taps_key = TF.conv_weight_taps(conv.weight.unsqueeze(2)), key
            y = TF.conv3d_causal(vol, conv.weight.unsqueeze(2), conv.bias, pad_t=0, weight_taps=self._taps_cache)
            return y.reshape(1, -1, b, t, 2 * h, 2 * w).squeeze(0).permute(1, 0, 2, 3, 4) if b > 1 else y
        y = self.resample(x.permute(0, 2, 1, 3, 4).reshape(b * t, c, h, w))
        return y.reshape(b, t, *y.shape[1:]).permute(0, 2, 1, 3, 4)

    def forward(self, x, state: CausalState | None = None):
        b, c, t, h, w = x.shape
        if self.mode == "upsample3d" and state is not None:
            i = state.next_slot()
            if state.slots[i] is None:
                state.slots[i] = "first"  # the first latent frame is not doubled in time
            else:
                old = state.slots[i]
                tail = x[:, :, -CACHE_T:].clone()
                if tail.shape[2] < CACHE_T:
                    head = torch.zeros_like(tail) if isinstance(old, str) else old[:, :, -1:].to(tail.device)
                    tail = torch.cat([head, tail], dim=2)
                y = self.time_conv(x) if isinstance(old, str) else self.time_conv(x, old)
                state.slots[i] = tail
                if _fast(y) and y.permute(0, 2, 3, 4, 1).is_contiguous():
                    # channels-last: frame 2t + k takes channels [k*c, (k+1)*c) of frame t; one copy, layout kept
                    yl = y.permute(0, 2, 3, 4, 1).reshape(b, t, h, w, 2, c).permute(0, 1, 4, 2, 3, 5)
                    x = yl.reshape(b, 2 * t, h, w, c).permute(0, 4, 1, 2, 3)
                else:
                    y = y.reshape(b, 2, c, t, h, w)
                    x = torch.stack((y[:, 0], y[:, 1]), dim=3).reshape(b, c, t * 2, h, w)
        x = self._spatial(x)
        if self.mode == "downsample3d" and state is not None:
            i = state.next_slot()
            if state.slots[i] is None:
                state.slots[i] = x.clone()
            else:
                last = x[:, :, -1:].clone()
                x = self.time_conv(torch.cat([state.slots[i][:, :, -1:], x], dim=2))
                state.slots[i] = last
        return x


class ResidualBlock(nn.Module):
    def __init__(self, in_dim: int, out_dim: int, dropout: float = 0.0):
        super().__init__()
        self.in_dim, self.out_dim = in_dim, out_dim
        self.residual = nn.Sequential(
            RMS_norm(in_dim, images=False), nn.SiLU(), CausalConv3d(in_dim, out_dim, 3, padding=1),
            RMS_norm(out_dim, images=False), nn.SiLU(), nn.Dropout(dropout),
            CausalConv3d(out_dim, out_dim, 3, padding=1))  # fmt: skip
        self.shortcut = CausalConv3d(in_dim, out_dim, 1) if in_dim != out_dim else nn.Identity()

    def forward(self, x, state: CausalState | None = None):
        h = self.shortcut(x)
        n1, _, c1, n2, _, _, c2 = self.residual
        if _fast(x) and not torch.is_tensor(n1.bias) and not torch.is_tensor(n2.bias):
            y = causal_step(c1, TF.pixel_norm_act(x, n1.gamma), state)
            return causal_step(c2, TF.pixel_norm_act(y, n2.gamma), state, residual=h)  # + h in the conv's epilogue
        for layer in self.residual:
            x = causal_step(layer, x, state) if isinstance(layer, CausalConv3d) else layer(x)
        return x + h


class AttentionBlock(nn.Module):
    """Single-head self-attention over the pixels of each frame."""

    def __init__(self, dim: int):
        super().__init__()
        self.dim = dim
        self.norm = RMS_norm(dim)
        self.to_qkv = nn.Conv2d(dim, dim * 3, 1)
        self.proj = nn.Conv2d(dim, dim, 1)
        nn.init.zeros_(self.proj.weight)

    def forward(self, x, state=None):
        b, c, t, h, w = x.shape
        y = self.norm(x.permute(0, 2, 1, 3, 4).reshape(b * t, c, h, w))
        q, k, v = self.to_qkv(y).reshape(b * t, 1, c * 3, h * w).permute(0, 3, 1, 2).contiguous().chunk(3, dim=-1)
        y = TF.attention(q, k, v)  # [b t, h w, 1, c]: one head of width c
        y = self.proj(y.squeeze(2).permute(0, 2, 1).reshape(b * t, c, h, w))
        return y.reshape(b, t, c, h, w).permute(0, 2, 1, 3, 4) + x


def _run(layers, x, state):
    layers = list(layers)
    if (len(layers) == 3 and isinstance(layers[0], RMS_norm) and isinstance(layers[1], nn.SiLU) and _fast(x)
            and not torch.is_tensor(layers[0].bias)):  # the norm -> SiLU -> conv head
        return causal_step(layers[2], TF.pixel_norm_act(x, layers[0].gamma), state)
    for layer in layers:
        if isinstance(layer, (ResidualBlock, Resample, AttentionBlock)):
            x = layer(x, state)
        elif isinstance(layer, CausalConv3d):
            x = causal_step(layer, x, state)
        else:
            x = layer(x)
    return x


def count_causal_slots(module: nn.Module) -> int:
    n = sum(1 for m in module.modules() if isinstance(m, CausalConv3d))
    # a downsample3d also keeps the spatially-resampled tail; shortcuts (1x1x1) take no slot
    n -= sum(1 for m in module.modules() if isinstance(m, ResidualBlock) and isinstance(m.shortcut, CausalConv3d))
    return n


class Encoder3d(nn.Module):
    def __init__(self, dim=128, z_dim=4, dim_mult=(1, 2, 4, 4), num_res_blocks=2, attn_scales=(),
                 temperal_downsample=(True, True, False), dropout=0.0):  # fmt: skip
        super().__init__()
        dims = [dim * u for u in [1, *dim_mult]]
        scale = 1.0
        self.conv1 = CausalConv3d(3, dims[0], 3, padding=1)
        downs = []
        for i, (in_dim, out_dim) in enumerate(zip(dims[:-1], dims[1:])):
            for _ in range(num_res_blocks):
                downs.append(ResidualBlock(in_dim, out_dim, dropout))
                if scale in attn_scales:
                    downs.append(AttentionBlock(out_dim))
                in_dim = out_dim
            if i != len(dim_mult) - 1:
                downs.append(Resample(out_dim, "downsample3d" if temperal_downsample[i] else "downsample2d"))
                scale /= 2.0
        self.downsamples = nn.Sequential(*downs)
        self.middle = nn.Sequential(ResidualBlock(out_dim, out_dim, dropout), AttentionBlock(out_dim),
                                    ResidualBlock(out_dim, out_dim, dropout))  # fmt: skip
        self.head = nn.Sequential(RMS_norm(out_dim, images=False), nn.SiLU(), CausalConv3d(out_dim, z_dim, 3, padding=1))

    def forward(self, x, state: CausalState | None = None):
        x = causal_step(self.conv1, x, state)
        x = _run(self.downsamples, x, state)
        x = _run(self.middle, x, state)
        return _run(self.head, x, state)


class Decoder3d(nn.Module):
    def __init__(self, dim=128, z_dim=4, dim_mult=(1, 2, 4, 4), num_res_blocks=2, attn_scales=(),
                 temperal_upsample=(False, True, True), dropout=0.0):  # fmt: skip
        super().__init__()
        dims = [dim * u for u in [dim_mult[-1], *dim_mult[::-1]]]
        scale = 1.0 / 2 ** (len(dim_mult) - 2)
        self.conv1 = CausalConv3d(z_dim, dims[0], 3, padding=1)
        self.middle = nn.Sequential(ResidualBlock(dims[0], dims[0], dropout), AttentionBlock(dims[0]),
                                    ResidualBlock(dims[0], dims[0], dropout))  # fmt: skip
        ups = []
        for i, (in_dim, out_dim) in enumerate(zip(dims[:-1], dims[1:])):
            if i in (1, 2, 3):
                in_dim = in_dim // 2
            for _ in range(num_res_blocks + 1):
                ups.append(ResidualBlock(in_dim, out_dim, dropout))
                if scale in attn_scales:
                    ups.append(AttentionBlock(out_dim))
                in_dim = out_dim
            if i != len(dim_mult) - 1:
                ups.append(Resample(out_dim, "upsample3d" if temperal_upsample[i] else "upsample2d"))
                scale *= 2.0
        self.upsamples = nn.Sequential(*ups)
        self.head = nn.Sequential(RMS_norm(out_dim, images=False), nn.SiLU(), CausalConv3d(out_dim, 3, 3, padding=1))

    def forward(self, x, state: CausalState | None = None):
        x = causal_step(self.conv1, x, state)
        x = _run(self.middle, x, state)
        x = _run(self.upsamples, x, state)
        return _run(self.head, x, state)


class VideoVAE(nn.Module):
    def __init__(self, dim=96, z_dim=16, dim_mult=(1, 2, 4, 4), num_res_blocks=2, attn_scales=(),
                 temperal_downsample=(False, True, True), dropout=0.0):  # fmt: skip
        super().__init__()
        self.dim, self.z_dim = dim, z_dim
        self.temperal_downsample = tuple(temperal_downsample)
        self.encoder = Encoder3d(dim, z_dim * 2, dim_mult, num_res_blocks, attn_scales, self.temperal_downsample, dropout)
        self.conv1 = CausalConv3d(z_dim * 2, z_dim * 2, 1)
        self.conv2 = CausalConv3d(z_dim, z_dim, 1)
        self.decoder = Decoder3d(dim, z_dim, dim_mult, num_res_blocks, attn_scales, self.temperal_downsample[::-1], dropout)

    def new_encoder_state(self) -> CausalState:
        return CausalState(count_causal_slots(self.encoder))

    def new_decoder_state(self) -> CausalState:
        return CausalState(count_causal_slots(self.decoder))

    @staticmethod
    def _normalise(mu, scale):
        mean, inv_std = (s.to(dtype=mu.dtype, device=mu.device).view(1, -1, 1, 1, 1) for s in scale)
        return (mu - mean) * inv_std

    @staticmethod
    def _denormalise(z, scale):
        mean, inv_std = (s.to(dtype=z.dtype, device=z.device).view(1, -1, 1, 1, 1) for s in scale)
        return z / inv_std + mean

    def encode_chunk(self, frames, state: CausalState, scale):
        """Encodes the next frames of a stream (1 frame first, then multiples of 4)."""
        state.rewind()
        out = self.encoder(frames, state)
        mu, _ = self.conv1(out).chunk(2, dim=1)
        return self._normalise(mu, scale)

    def encode(self, x, scale):
        """x: [B, 3, T, H, W] with T = 4n+1 -> latent mean [B, z, n+1, H/8, W/8]."""
        state = self.new_encoder_state()
        t = x.shape[2]
        outs = []
        for i in range(1 + (t - 1) // 4):
            state.rewind()
            chunk = x[:, :, :1] if i == 0 else x[:, :, 1 + 4 * (i - 1) : 1 + 4 * i]
            outs.append(self.encoder(chunk, state))
        mu, _ = self.conv1(torch.cat(outs, dim=2)).chunk(2, dim=1)
        return self._normalise(mu, scale)

    def decode_chunk(self, z, state: CausalState, scale):
        """Decodes the next latent frames of a stream, one latent frame at a time."""
        x = self.conv2(self._denormalise(z, scale))
        outs = []
        for i in range(x.shape[2]):
            state.rewind()
            outs.append(self.decoder(x[:, :, i : i + 1], state))
        return torch.cat(outs, dim=2)

    def decode(self, z, scale):
        return self.decode_chunk(z, self.new_decoder_state(), scale)


class VAEStreamState:
    """Session-owned state of a streaming encode or decode (kept by the stage, not by the model)."""

    def __init__(self, vae: "WanVideoVAE", kind: str):
        self.kind = kind
        self.state = vae.model.new_encoder_state() if kind == "encode" else vae.model.new_decoder_state()
        self.frames_seen = 0


GRID_FOR_RANKS = {1: (1, 1), 2: (1, 2), 4: (2, 2), 8: (2, 4)}


def calculate_2d_grid(h: int, w: int, ranks: int) -> tuple[int, int]:
    """(rows, cols) of the tile grid: the longer side gets more tiles."""
    r, c = GRID_FOR_RANKS.get(ranks, (1, ranks))
    return (c, r) if h > w and r != c else (r, c)


def blend_mask(h: int, w: int, border: int, edges: tuple[bool, bool, bool, bool], device, dtype):
    """Linear ramps of width `border` on the sides that touch a neighbouring tile (top, bottom, left, right)."""
    ramp_h = torch.ones(h, device=device, dtype=dtype)
    ramp_w = torch.ones(w, device=device, dtype=dtype)
    if border > 0:
        r = (torch.arange(border, device=device, dtype=dtype) + 1) / border
        if edges[0]:
            ramp_h[:border] = r
        if edges[1]:
            ramp_h[-border:] = torch.minimum(ramp_h[-border:], r.flip(0))
        if edges[2]:
            ramp_w[:border] = r
        if edges[3]:
            ramp_w[-border:] = torch.minimum(ramp_w[-border:], r.flip(0))
    return ramp_h[:, None] * ramp_w[None, :]


class WanVideoVAE(BaseModel):
    """Wrapper with latent normalisation, tiling, 2-D spatial parallel decode and streaming."""

    def __init__(self, z_dim: int = 16, parallelism: int = 1, dim: int = 96):
        super().__init__()
        self.z_dim = z_dim
        self.mean = torch.tensor(WAN21_LATENT_MEAN[:z_dim] if z_dim <= 16 else [0.0] * z_dim)
        self.std = torch.tensor(WAN21_LATENT_STD[:z_dim] if z_dim <= 16 else [1.0] * z_dim)
        self.scale = [self.mean, 1.0 / self.std]
        self.model = VideoVAE(dim=dim, z_dim=z_dim).eval().requires_grad_(False)
        self.upsampling_factor = 8
        self.parallelism = parallelism
        self.layer_name_list = []

    # ---- whole-video API ---------------------------------------------------------
    @torch.no_grad()
    def encode(self, videos, device=None, tiled=False, tile_size=(34, 34), tile_stride=(18, 16)):
        """videos: [B, 3, T, H, W] in [-1, 1] -> [B, z, (T-1)/4+1, H/8, W/8]."""
        p = next(self.model.parameters())
        videos = videos.to(device=device or p.device, dtype=p.dtype)
        if tiled:
            return self.tiled_encode(videos, tile_size, tile_stride)
        return self.model.encode(videos, self.scale)

    @torch.no_grad()
    def decode(self, latents, device=None, tiled=False, tile_size=(34, 34), tile_stride=(18, 16)):
        p = next(self.model.parameters())
        latents = latents.to(device=device or p.device, dtype=p.dtype)
        if self.parallelism > 1:
            return self.decode_dist_2d(latents)
        if tiled:
            return self.tiled_decode(latents, tile_size, tile_stride)
        return self.model.decode(latents, self.scale).clamp_(-1, 1)

    # ---- tiling -----------------------------------------------------------------------
    @staticmethod
    def _tile_starts(size: int, tile: int, stride: int) -> list[int]:
        if size <= tile:
            return [0]
        starts = list(range(0, size - tile, stride)) + [size - tile]
        return sorted(set(starts))

    def _tiled(self, x, tile_size, tile_stride, fn, out_scale: float, out_channels: int, t_out: int):
        import torch.distributed as dist

        B, _, _, H, W = x.shape
        th, tw = tile_size
        sh, sw = tile_stride
        rows, cols = self._tile_starts(H, th, sh), self._tile_starts(W, tw, sw)
        Ho, Wo = int(H * out_scale), int(W * out_scale)
        values = torch.zeros(B, out_channels, t_out, Ho, Wo, device=x.device, dtype=torch.float32)
        weight = torch.zeros(1, 1, 1, Ho, Wo, device=x.device, dtype=torch.float32)
        rank, world = (dist.get_rank(), dist.get_world_size()) if (self.parallelism > 1 and dist.is_initialized()) else (0, 1)
        tiles = [(r, c) for r in rows for c in cols]
        for n, (r, c) in enumerate(tiles):
            if n % world != rank:
                continue
            part = fn(x[:, :, :, r : r + th, c : c + tw]).float()
            ph, pw = part.shape[-2:]
            border = int(min(th - sh, tw - sw) * out_scale)
            edges = (r > 0, r + th < H, c > 0, c + tw < W)
            m = blend_mask(ph, pw, border, edges, x.device, torch.float32)
            ro, co = int(r * out_scale), int(c * out_scale)
            values[:, :, :, ro : ro + ph, co : co + pw] += part * m
            weight[:, :, :, ro : ro + ph, co : co + pw] += m
        if world > 1:
            dist.all_reduce(values)
            dist.all_reduce(weight)
        return values / weight.clamp_min(1e-6)

    def tiled_decode(self, latents, tile_size=(34, 34), tile_stride=(18, 16)):
        t_out = (latents.shape[2] - 1) * 4 + 1
        f = float(self.upsampling_factor)
        out = self._tiled(latents, tile_size, tile_stride, lambda z: self.model.decode(z, self.scale), f, 3, t_out)
        return out.clamp_(-1, 1).to(latents.dtype)

    def tiled_encode(self, videos, tile_size=(34, 34), tile_stride=(18, 16)):
        f = self.upsampling_factor
        ts = (tile_size[0] * f, tile_size[1] * f)
        st = (tile_stride[0] * f, tile_stride[1] * f)
        t_out = (videos.shape[2] - 1) // 4 + 1
        out = self._tiled(videos, ts, st, lambda v: self.model.encode(v, self.scale), 1.0 / f, self.z_dim, t_out)
        return out.to(videos.dtype)

    # ---- 2-D domain decomposition -----------------------------------------------------
    def decode_dist_2d(self, latents, halo: int = 2):
        """Each rank decodes one tile of a rows x cols grid (plus a latent halo); tiles are all-gathered."""
        import torch.distributed as dist

        world = dist.get_world_size() if dist.is_initialized() else 1
        rank = dist.get_rank() if dist.is_initialized() else 0
        B, C, T, H, W = latents.shape
        rows, cols = calculate_2d_grid(H, W, world)
        hs, ws = math.ceil(H / rows), math.ceil(W / cols)
        r, c = divmod(rank, cols)
        h0, w0 = r * hs, c * ws
        h1, w1 = min(H, h0 + hs), min(W, w0 + ws)
        a0, b0 = max(0, h0 - halo), max(0, w0 - halo)
        a1, b1 = min(H, h1 + halo), min(W, w1 + halo)
        f = self.upsampling_factor
        tile = self.model.decode(latents[:, :, :, a0:a1, b0:b1], self.scale)
        tile = tile[:, :, :, (h0 - a0) * f : (h0 - a0) * f + (h1 - h0) * f, (w0 - b0) * f : (w0 - b0) * f + (w1 - w0) * f]
        if world == 1:
            return tile.clamp_(-1, 1)
        padded = torch.zeros(B, 3, tile.shape[2], hs * f, ws * f, device=tile.device, dtype=tile.dtype)
        padded[:, :, :, : tile.shape[3], : tile.shape[4]] = tile
        parts = [torch.empty_like(padded) for _ in range(world)]
        dist.all_gather(parts, padded.contiguous())
        out = torch.zeros(B, 3, tile.shape[2], rows * hs * f, cols * ws * f, device=tile.device, dtype=tile.dtype)
        for k, part in enumerate(parts):
            rr, cc = divmod(k, cols)
            out[:, :, :, rr * hs * f : (rr + 1) * hs * f, cc * ws * f : (cc + 1) * ws * f] = part
        return out[:, :, :, : H * f, : W * f].clamp_(-1, 1)

    # ---- streaming --------------------------------------------------------------------
    def new_stream(self, kind: str) -> VAEStreamState:
        return VAEStreamState(self, kind)

    @torch.no_grad()
    def cached_encode(self, frames, stream: VAEStreamState):
        """Encodes the next frames of a session (first call: 1 + 4k frames, later: 4k frames)."""
        p = next(self.model.parameters())
        frames = frames.to(device=p.device, dtype=p.dtype)
        outs, t, i = [], frames.shape[2], 0
        if stream.frames_seen == 0:
            outs.append(self.model.encode_chunk(frames[:, :, :1], stream.state, self.scale))
            i = 1
        while i < t:
            outs.append(self.model.encode_chunk(frames[:, :, i : i + 4], stream.state, self.scale))
            i += 4
        stream.frames_seen += t
        return torch.cat(outs, dim=2)

    @torch.no_grad()
    def cached_decode(self, latents, stream: VAEStreamState):
        p = next(self.model.parameters())
        latents = latents.to(device=p.device, dtype=p.dtype)
        stream.frames_seen += latents.shape[2]
        return self.model.decode_chunk(latents, stream.state, self.scale).clamp_(-1, 1)

    @staticmethod
    def state_dict_converter():
        return WanVideoVAEStateDictConverter()


class WanVideoVAEStateDictConverter:
    """The published VAE file stores the `VideoVAE` keys bare or under `model_state`; prefix them with `model.`."""

    def from_official(self, state_dict: dict):
        if "model_state" in state_dict:
            state_dict = state_dict["model_state"]
        sd = dict(state_dict) if any(k.startswith("model.") for k in state_dict) else {"model." + k: v for k, v in state_dict.items()}
        # width and latent channels follow from the decoder's ends (96 / 16 in the published file; narrower in test models)
        ctor = {}
        head, entry = sd.get("model.decoder.head.2.weight"), sd.get("model.conv2.weight")
        if head is not None and head.shape[1] != 96:
            ctor["dim"] = int(head.shape[1])
        if entry is not None and entry.shape[0] != 16:
            ctor["z_dim"] = int(entry.shape[0])
        return sd, ctor

    from_civitai = from_official
    from_diffusers = from_official


def _register() -> None:
    from telefuser_b200.core.model_registry import register_architecture

    register_architecture("wan_video_vae", WanVideoVAE, lambda: VideoVAE(), keys_only=False)


_register()
