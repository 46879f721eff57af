"""LTX-2 audio path: latent -> stereo log-mel decoder, mel -> waveform vocoder, optional bandwidth extension.

AudioDecoder: latents [B, 8, T, 16] are de-normalised per (channel, mel-bin), then a 2-D conv decoder that is causal
along time (all padding in front; nearest x2 upsampling drops the first row) produces [B, 2, 4T - 3, mel bins].
Vocoder: a HiFi-GAN / BigVGAN-style stack of transposed 1-D convs and residual blocks; the AMP variant wraps every
activation (Snake / SnakeBeta) in x2 Kaiser-sinc upsampling and low-pass downsampling to avoid aliasing.
VocoderWithBWE: runs the vocoder, recomputes a log-mel of its output with a conv STFT, predicts a high-band
residual with a second generator and adds it to a Hann-windowed-sinc resampling of the low-rate waveform.
All ops are convolutions through cuDNN plus elementwise PyTorch; audio is a negligible share of a generation.
Role parity: telefuser/models/ltx_audio_vae.py:25-1183.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from enum import Enum
from typing import Any

import torch
import torch.nn.functional as F
from torch import nn

from telefuser_b200.ops import functional as TF

LRELU_SLOPE = 0.1


class NormType(Enum):
    GROUP = "group"
    PIXEL = "pixel"


class CausalityAxis(Enum):
    NONE = None
    WIDTH = "width"
    HEIGHT = "height"
    WIDTH_COMPATIBILITY = "width-compatibility"


class AttentionType(Enum):
    VANILLA = "vanilla"
    LINEAR = "linear"
    NONE = "none"


class PixelNorm(nn.Module):
    def __init__(self, dim: int = 1, eps: float = 1e-8) -> None:
        super().__init__()
        self.dim, self.eps = dim, eps

    def forward(self, x):
        return x * torch.rsqrt(x.float().pow(2).mean(dim=self.dim, keepdim=True) + self.eps).to(x.dtype)


def build_normalization_layer(in_channels: int, *, num_groups: int = 32, normtype: NormType = NormType.GROUP) -> nn.Module:
    if normtype == NormType.GROUP:
        return nn.GroupNorm(num_groups, in_channels, eps=1e-6, affine=True)
    return PixelNorm(1, 1e-6)


class CausalConv2d(nn.Module):
    """Conv2d whose whole padding along the causal axis (height = time here) sits in front."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride: int = 1, dilation=1, groups: int = 1, bias: bool = True,
                 causality_axis: CausalityAxis = CausalityAxis.HEIGHT) -> None:  # fmt: skip
        super().__init__()
        self.causality_axis = causality_axis
        kh, kw = (kernel_size, kernel_size) if isinstance(kernel_size, int) else kernel_size
        dh, dw = (dilation, dilation) if isinstance(dilation, int) else dilation
        ph, pw = (kh - 1) * dh, (kw - 1) * dw
        if causality_axis == CausalityAxis.NONE:
            self.padding = (pw // 2, pw - pw // 2, ph // 2, ph - ph // 2)
        elif causality_axis in (CausalityAxis.WIDTH, CausalityAxis.WIDTH_COMPATIBILITY):
            self.padding = (pw, 0, ph // 2, ph - ph // 2)
        else:
            self.padding = (pw // 2, pw - pw // 2, ph, 0)
        self.conv = nn.Conv2d(in_channels, out_channels, (kh, kw), stride=stride, padding=0, dilation=(dh, dw), groups=groups, bias=bias)

    def forward(self, x):
        return self.conv(F.pad(x, self.padding))


def make_conv2d(in_channels: int, out_channels: int, kernel_size, stride: int = 1, padding=None, dilation: int = 1, groups: int = 1,
                bias: bool = True, causality_axis: CausalityAxis | None = None) -> nn.Module:  # fmt: skip
    if causality_axis is not None:
        return CausalConv2d(in_channels, out_channels, kernel_size, stride, dilation, groups, bias, causality_axis)
    if padding is None:
        padding = kernel_size // 2 if isinstance(kernel_size, int) else tuple(k // 2 for k in kernel_size)
    return nn.Conv2d(in_channels, out_channels, kernel_size, stride, padding, dilation, groups, bias)


class AttnBlock(nn.Module):
    """Single-head attention over all (time, mel) positions with 1x1-conv projections."""

    def __init__(self, in_channels: int, norm_type: NormType = NormType.GROUP) -> None:
        super().__init__()
        self.in_channels = in_channels
        self.norm = build_normalization_layer(in_channels, normtype=norm_type)
        self.q, self.k, self.v, self.proj_out = (nn.Conv2d(in_channels, in_channels, 1) for _ in range(4))

    def forward(self, x):
        h = self.norm(x)
        b, c, hh, ww = h.shape
        q, k, v = (m(h).reshape(b, c, hh * ww).transpose(1, 2).unsqueeze(2) for m in (self.q, self.k, self.v))
        o = TF.attention(q, k, v, scale=float(c) ** -0.5).squeeze(2)
        return x + self.proj_out(o.transpose(1, 2).reshape(b, c, hh, ww))


def make_attn(in_channels: int, attn_type: AttentionType = AttentionType.VANILLA, norm_type: NormType = NormType.GROUP) -> nn.Module:
    if attn_type == AttentionType.VANILLA:
        return AttnBlock(in_channels, norm_type)
    if attn_type == AttentionType.NONE:
        return nn.Identity()
    raise NotImplementedError(f"attention type {attn_type.value} is not built")


class ResnetBlock(nn.Module):
    def __init__(self, *, in_channels: int, out_channels: int | None = None, conv_shortcut: bool = False, dropout: float = 0.0,
                 temb_channels: int = 512, norm_type: NormType = NormType.GROUP,
                 causality_axis: CausalityAxis = CausalityAxis.HEIGHT) -> None:  # fmt: skip
        super().__init__()
        if causality_axis != CausalityAxis.NONE and norm_type == NormType.GROUP:
            raise ValueError("a causal block cannot use GroupNorm (it mixes statistics across time)")
        out_channels = out_channels or in_channels
        self.in_channels, self.out_channels, self.use_conv_shortcut, self.causality_axis = in_channels, out_channels, conv_shortcut, causality_axis
        self.norm1 = build_normalization_layer(in_channels, normtype=norm_type)
        self.non_linearity = nn.SiLU()
        self.conv1 = make_conv2d(in_channels, out_channels, 3, causality_axis=causality_axis)
        if temb_channels > 0:
            self.temb_proj = nn.Linear(temb_channels, out_channels)
        self.norm2 = build_normalization_layer(out_channels, normtype=norm_type)
        self.conv2 = make_conv2d(out_channels, out_channels, 3, causality_axis=causality_axis)
        if in_channels != out_channels:
            if conv_shortcut:
                self.conv_shortcut = make_conv2d(in_channels, out_channels, 3, causality_axis=causality_axis)
            else:
                self.nin_shortcut = make_conv2d(in_channels, out_channels, 1, causality_axis=causality_axis)

    def forward(self, x, temb=None):
        h = self.conv1(self.non_linearity(self.norm1(x)))
        if temb is not None:
            h = h + self.temb_proj(self.non_linearity(temb))[:, :, None, None]
        h = self.conv2(self.non_linearity(self.norm2(h)))
        if self.in_channels != self.out_channels:
            x = self.conv_shortcut(x) if self.use_conv_shortcut else self.nin_shortcut(x)
        return x + h


class Upsample(nn.Module):
    def __init__(self, in_channels: int, with_conv: bool, causality_axis: CausalityAxis = CausalityAxis.HEIGHT) -> None:
        super().__init__()
        self.with_conv, self.causality_axis = with_conv, causality_axis
        if with_conv:
            self.conv = make_conv2d(in_channels, in_channels, 3, causality_axis=causality_axis)

    def forward(self, x):
        x = F.interpolate(x, scale_factor=2.0, mode="nearest")
        if self.with_conv:
            x = self.conv(x)
            if self.causality_axis == CausalityAxis.HEIGHT:
                x = x[:, :, 1:]
            elif self.causality_axis == CausalityAxis.WIDTH:
                x = x[:, :, :, 1:]
        return x


class AudioPatchifier:
    def __init__(self, patch_size: int = 1) -> None:
        self.patch_size = (patch_size, 1, 1)

    def patchify(self, x):
        b, c, t, m = x.shape
        p = self.patch_size[0]
        return x.reshape(b, c, t // p, p, m).permute(0, 2, 1, 3, 4).reshape(b, t // p, c * p * m)

    def unpatchify(self, tokens, shape: "AudioLatentShape"):
        b, t, p = tokens.shape[0], tokens.shape[1], self.patch_size[0]
        return tokens.reshape(b, t, shape.channels, p, shape.mel_bins).permute(0, 2, 1, 3, 4).reshape(b, shape.channels, t * p, shape.mel_bins)


@dataclass(frozen=True)
class AudioLatentShape:
    batch: int
    channels: int
    frames: int
    mel_bins: int


class PerChannelStatistics(nn.Module):
    def __init__(self, latent_channels: int = 128) -> None:
        super().__init__()
        self.register_buffer("std-of-means", torch.ones(latent_channels))
        self.register_buffer("mean-of-means", torch.zeros(latent_channels))

    def un_normalize(self, x):
        return x * self.get_buffer("std-of-means").to(x) + self.get_buffer("mean-of-means").to(x)


class _Stage(nn.Module):
    def __init__(self) -> None:
        super().__init__()
        self.block, self.attn = nn.ModuleList(), nn.ModuleList()


class _Mid(nn.Module):
    def __init__(self, channels: int, temb: int, dropout: float, norm_type, axis, attn_type, add_attention: bool) -> None:
        super().__init__()
        kw = dict(in_channels=channels, out_channels=channels, temb_channels=temb, dropout=dropout, norm_type=norm_type, causality_axis=axis)
        self.block_1 = ResnetBlock(**kw)
        self.attn_1 = make_attn(channels, attn_type, norm_type) if add_attention else nn.Identity()
        self.block_2 = ResnetBlock(**kw)

    def forward(self, x):
        return self.block_2(self.attn_1(self.block_1(x)))


class AudioDecoder(nn.Module):
    def __init__(self, *, ch: int, out_ch: int, ch_mult=(1, 2, 4, 8), num_res_blocks: int = 2, attn_resolutions=None, dropout: float = 0.0,
                 in_channels: int = 2, resolution: int = 256, z_channels: int = 8, double_z: bool = True,
                 attn_type: AttentionType = AttentionType.VANILLA, mid_block_add_attention: bool = True, norm_type: NormType = NormType.PIXEL,
                 causality_axis: CausalityAxis = CausalityAxis.HEIGHT, sample_rate: int = 16000, mel_hop_length: int = 160,
                 is_causal: bool = True, mel_bins: int | None = None, **_ignored: Any) -> None:  # fmt: skip
        super().__init__()
        attn_resolutions = {8, 16, 32} if attn_resolutions is None else set(attn_resolutions)
        self.per_channel_statistics = PerChannelStatistics(ch)
        self.sample_rate, self.mel_hop_length, self.is_causal, self.mel_bins = sample_rate, mel_hop_length, is_causal, mel_bins
        self.patchifier = AudioPatchifier(1)
        self.ch, self.out_ch, self.num_resolutions, self.num_res_blocks, self.resolution = ch, out_ch, len(ch_mult), num_res_blocks, resolution
        self.z_channels, self.causality_axis, self.norm_type = z_channels, causality_axis, norm_type
        block_in = ch * ch_mult[-1]
        self.conv_in = make_conv2d(z_channels, block_in, 3, causality_axis=causality_axis)
        self.non_linearity = nn.SiLU()
        self.mid = _Mid(block_in, 0, dropout, norm_type, causality_axis, attn_type, mid_block_add_attention)
        res = resolution // 2 ** (self.num_resolutions - 1)
        stages = []
        for level in reversed(range(self.num_resolutions)):
            stage, block_out = _Stage(), ch * ch_mult[level]
            for _ in range(num_res_blocks + 1):
                stage.block.append(ResnetBlock(in_channels=block_in, out_channels=block_out, temb_channels=0, dropout=dropout,
                                               norm_type=norm_type, causality_axis=causality_axis))  # fmt: skip
                block_in = block_out
                if res in attn_resolutions:
                    stage.attn.append(make_attn(block_in, attn_type, norm_type))
            if level != 0:
                stage.upsample = Upsample(block_in, True, causality_axis)
                res *= 2
            stages.insert(0, stage)
        self.up = nn.ModuleList(stages)
        self.norm_out = build_normalization_layer(block_in, normtype=norm_type)
        self.conv_out = make_conv2d(block_in, out_ch, 3, causality_axis=causality_axis)

    def forward(self, sample):
        b, c, t, m = sample.shape
        shape = AudioLatentShape(b, c, t, m)
        x = self.patchifier.unpatchify(self.per_channel_statistics.un_normalize(self.patchifier.patchify(sample)), shape)
        frames = t * 4 if self.causality_axis == CausalityAxis.NONE else max(t * 4 - 3, 1)
        bins = self.mel_bins if self.mel_bins is not None else m
        h = self.mid(self.conv_in(x))
        for level in reversed(range(self.num_resolutions)):
            stage = self.up[level]
            for i, blk in enumerate(stage.block):
                h = blk(h)
                if len(stage.attn):
                    h = stage.attn[i](h)
            if level != 0:
                h = stage.upsample(h)
        h = self.conv_out(self.non_linearity(self.norm_out(h)))
        h = h[:, : self.out_ch, :frames, :bins]
        if h.shape[2] < frames or h.shape[3] < bins:
            h = F.pad(h, (0, bins - h.shape[3], 0, frames - h.shape[2]))
        return h


# ---- vocoder --------------------------------------------------------------------------------
def get_padding(kernel_size: int, dilation: int = 1) -> int:
    return int((kernel_size * dilation - dilation) / 2)


def kaiser_sinc_filter1d(cutoff: float, half_width: float, kernel_size: int) -> torch.Tensor:
    """Windowed-sinc low-pass with a Kaiser window chosen from the transition width; [1, 1, kernel_size]."""
    half = kernel_size // 2
    amplitude = 2.285 * (half - 1) * math.pi * 4 * half_width + 7.95
    if amplitude > 50.0:
        beta = 0.1102 * (amplitude - 8.7)
    elif amplitude >= 21.0:
        beta = 0.5842 * (amplitude - 21) ** 0.4 + 0.07886 * (amplitude - 21.0)
    else:
        beta = 0.0
    window = torch.kaiser_window(kernel_size, beta=beta, periodic=False)
    t = torch.arange(-half, half) + 0.5 if kernel_size % 2 == 0 else torch.arange(kernel_size) - half
    if cutoff == 0:
        return torch.zeros(1, 1, kernel_size)
    f = 2 * cutoff * window * torch.sinc(2 * cutoff * t)
    return (f / f.sum()).view(1, 1, kernel_size)


class LowPassFilter1d(nn.Module):
    def __init__(self, cutoff: float = 0.5, half_width: float = 0.6, stride: int = 1, padding: bool = True,
                 padding_mode: str = "replicate", kernel_size: int = 12) -> None:  # fmt: skip
        super().__init__()
        if not 0.0 <= cutoff <= 0.5:
            raise ValueError("cutoff must lie in [0, 0.5]")
        self.kernel_size, self.stride, self.padding, self.padding_mode = kernel_size, stride, padding, padding_mode
        self.pad_left, self.pad_right = kernel_size // 2 - int(kernel_size % 2 == 0), kernel_size // 2
        self.register_buffer("filter", kaiser_sinc_filter1d(cutoff, half_width, kernel_size))

    def forward(self, x):
        c = x.shape[1]
        if self.padding:
            x = F.pad(x, (self.pad_left, self.pad_right), mode=self.padding_mode)
        return F.conv1d(x, self.filter.to(x).expand(c, -1, -1), stride=self.stride, groups=c)


class UpSample1d(nn.Module):
    def __init__(self, ratio: int = 2, kernel_size: int | None = None, persistent: bool = True, window_type: str = "kaiser") -> None:
        super().__init__()
        self.ratio = self.stride = ratio
        if window_type == "hann":
            rolloff, lp_width = 0.99, 6
            width = math.ceil(lp_width / rolloff)
            self.kernel_size, self.pad = 2 * width * ratio + 1, width
            self.pad_left, self.pad_right = 2 * width * ratio, 2 * width * ratio + 1 - ratio
            t = (torch.arange(self.kernel_size) / ratio - width) * rolloff
            window = torch.cos(t.clamp(-lp_width, lp_width) * math.pi / lp_width / 2) ** 2
            filt = (torch.sinc(t) * window * rolloff / ratio).view(1, 1, -1)
        else:
            self.kernel_size = int(6 * ratio // 2) * 2 if kernel_size is None else kernel_size
            self.pad = self.kernel_size // ratio - 1
            self.pad_left = self.pad * ratio + (self.kernel_size - ratio) // 2
            self.pad_right = self.pad * ratio + (self.kernel_size - ratio + 1) // 2
            filt = kaiser_sinc_filter1d(0.5 / ratio, 0.6 / ratio, self.kernel_size)
        self.register_buffer("filter", filt, persistent=persistent)

    def forward(self, x):
        c = x.shape[1]
        x = F.pad(x, (self.pad, self.pad), mode="replicate")
        x = self.ratio * F.conv_transpose1d(x, self.filter.to(x).expand(c, -1, -1), stride=self.stride, groups=c)
        return x[..., self.pad_left : -self.pad_right]


class DownSample1d(nn.Module):
    def __init__(self, ratio: int = 2, kernel_size: int | None = None) -> None:
        super().__init__()
        self.ratio = ratio
        self.kernel_size = int(6 * ratio // 2) * 2 if kernel_size is None else kernel_size
        self.lowpass = LowPassFilter1d(0.5 / ratio, 0.6 / ratio, stride=ratio, kernel_size=self.kernel_size)

    def forward(self, x):
        return self.lowpass(x)


class Snake(nn.Module):
    """x + sin^2(alpha x) / alpha, per channel (alpha stored as its log)."""

    def __init__(self, in_features: int, alpha: float = 1.0, alpha_trainable: bool = True, alpha_logscale: bool = True) -> None:
        super().__init__()
        self.alpha_logscale, self.eps = alpha_logscale, 1e-9
        self.alpha = nn.Parameter(torch.zeros(in_features) if alpha_logscale else torch.ones(in_features) * alpha, requires_grad=alpha_trainable)

    def _scales(self):
        a = self.alpha[None, :, None]
        a = a.exp() if self.alpha_logscale else a
        return a, a

    def forward(self, x):
        a, b = self._scales()
        return x + torch.sin(x * a).pow(2) / (b + self.eps)


class SnakeBeta(Snake):
    """Snake with a separate magnitude parameter: x + sin^2(alpha x) / beta."""

    def __init__(self, in_features: int, alpha: float = 1.0, alpha_trainable: bool = True, alpha_logscale: bool = True) -> None:
        super().__init__(in_features, alpha, alpha_trainable, alpha_logscale)
        self.beta = nn.Parameter(torch.zeros(in_features) if alpha_logscale else torch.ones(in_features) * alpha, requires_grad=alpha_trainable)

    def _scales(self):
        a, b = self.alpha[None, :, None], self.beta[None, :, None]
        return (a.exp(), b.exp()) if self.alpha_logscale else (a, b)


class Activation1d(nn.Module):
    def __init__(self, activation: nn.Module, up_ratio: int = 2, down_ratio: int = 2, up_kernel_size: int = 12, down_kernel_size: int = 12) -> None:
        super().__init__()
        self.act, self.upsample, self.downsample = activation, UpSample1d(up_ratio, up_kernel_size), DownSample1d(down_ratio, down_kernel_size)

    def forward(self, x):
        return self.downsample(self.act(self.upsample(x)))


class ResBlock1(nn.Module):
    def __init__(self, channels: int, kernel_size: int = 3, dilation=(1, 3, 5)) -> None:
        super().__init__()
        self.convs1 = nn.ModuleList([nn.Conv1d(channels, channels, kernel_size, 1, dilation=d, padding="same") for d in dilation])
        self.convs2 = nn.ModuleList([nn.Conv1d(channels, channels, kernel_size, 1, dilation=1, padding="same") for _ in dilation])

    def forward(self, x):
        for c1, c2 in zip(self.convs1, self.convs2):
            x = c2(F.leaky_relu(c1(F.leaky_relu(x, LRELU_SLOPE)), LRELU_SLOPE)) + x
        return x


class AMPBlock1(nn.Module):
    def __init__(self, channels: int, kernel_size: int = 3, dilation=(1, 3, 5), activation: str = "snake") -> None:
        super().__init__()
        act = SnakeBeta if activation == "snakebeta" else Snake
        self.convs1 = nn.ModuleList([nn.Conv1d(channels, channels, kernel_size, 1, dilation=d, padding=get_padding(kernel_size, d)) for d in dilation])
        self.convs2 = nn.ModuleList([nn.Conv1d(channels, channels, kernel_size, 1, padding=get_padding(kernel_size, 1)) for _ in dilation])
        self.acts1 = nn.ModuleList([Activation1d(act(channels)) for _ in dilation])
        self.acts2 = nn.ModuleList([Activation1d(act(channels)) for _ in dilation])

    def forward(self, x):
        for c1, c2, a1, a2 in zip(self.convs1, self.convs2, self.acts1, self.acts2):
            x = x + c2(a2(c1(a1(x))))
        return x


class Vocoder(nn.Module):
    """Stereo log-mel [B, 2, T, 64] -> waveform [B, 2, T * prod(upsample_rates)]."""

    def __init__(self, resblock_kernel_sizes=None, upsample_rates=None, upsample_kernel_sizes=None, resblock_dilation_sizes=None,
                 upsample_initial_channel: int = 1024, resblock: str = "1", output_sampling_rate: int = 24000, activation: str = "snake",
                 use_tanh_at_final: bool = True, apply_final_activation: bool = True, use_bias_at_final: bool = True,
                 in_channels: int = 128) -> None:  # fmt: skip
        super().__init__()
        resblock_kernel_sizes = resblock_kernel_sizes or [3, 7, 11]
        upsample_rates = upsample_rates or [6, 5, 2, 2, 2]
        upsample_kernel_sizes = upsample_kernel_sizes or [16, 15, 8, 4, 4]
        resblock_dilation_sizes = resblock_dilation_sizes or [[1, 3, 5]] * 3
        self.output_sampling_rate, self.num_kernels, self.num_upsamples = output_sampling_rate, len(resblock_kernel_sizes), len(upsample_rates)
        self.use_tanh_at_final, self.apply_final_activation, self.is_amp = use_tanh_at_final, apply_final_activation, resblock == "AMP1"
        c0 = upsample_initial_channel
        self.conv_pre = nn.Conv1d(in_channels, c0, 7, 1, padding=3)
        self.ups = nn.ModuleList(nn.ConvTranspose1d(c0 // 2**i, c0 // 2 ** (i + 1), k, s, padding=(k - s) // 2)
                                 for i, (s, k) in enumerate(zip(upsample_rates, upsample_kernel_sizes)))  # fmt: skip
        self.resblocks = nn.ModuleList()
        for i in range(len(upsample_rates)):
            for k, d in zip(resblock_kernel_sizes, resblock_dilation_sizes):
                ch = c0 // 2 ** (i + 1)
                self.resblocks.append(AMPBlock1(ch, k, tuple(d), activation) if self.is_amp else ResBlock1(ch, k, tuple(d)))
        final = c0 // 2 ** len(upsample_rates)
        self.act_post = Activation1d(SnakeBeta(final)) if self.is_amp else nn.LeakyReLU()
        self.conv_post = nn.Conv1d(final, 2, 7, 1, padding=3, bias=use_bias_at_final)

    def forward(self, x):
        x = x.transpose(2, 3)
        if x.dim() == 4:
            if x.shape[1] != 2:
                raise ValueError("the vocoder expects stereo mel input")
            x = x.flatten(1, 2)
        x = self.conv_pre(x)
        for i, up in enumerate(self.ups):
            x = up(x if self.is_amp else F.leaky_relu(x, LRELU_SLOPE))
            acc = self.resblocks[i * self.num_kernels](x)
            for j in range(1, self.num_kernels):
                acc = acc + self.resblocks[i * self.num_kernels + j](x)
            x = acc / self.num_kernels
        x = self.conv_post(self.act_post(x))
        if self.apply_final_activation:
            x = torch.tanh(x) if self.use_tanh_at_final else x.clamp(-1, 1)
        return x


class _STFTFn(nn.Module):
    """STFT as a strided conv with stored real / imaginary bases (causal: all padding in front)."""

    def __init__(self, filter_length: int, hop_length: int, win_length: int) -> None:
        super().__init__()
        self.hop_length, self.win_length = hop_length, win_length
        n = filter_length // 2 + 1
        self.register_buffer("forward_basis", torch.zeros(n * 2, 1, filter_length))
        self.register_buffer("inverse_basis", torch.zeros(n * 2, 1, filter_length))

    def forward(self, y):
        y = y.unsqueeze(1) if y.dim() == 2 else y
        spec = F.conv1d(F.pad(y, (max(0, self.win_length - self.hop_length), 0)), self.forward_basis, stride=self.hop_length)
        n = spec.shape[1] // 2
        real, imag = spec[:, :n], spec[:, n:]
        return torch.sqrt(real**2 + imag**2), torch.atan2(imag.float(), real.float()).to(real.dtype)


class MelSTFT(nn.Module):
    def __init__(self, filter_length: int, hop_length: int, win_length: int, n_mel_channels: int) -> None:
        super().__init__()
        self.stft_fn = _STFTFn(filter_length, hop_length, win_length)
        self.register_buffer("mel_basis", torch.zeros(n_mel_channels, filter_length // 2 + 1))

    def mel_spectrogram(self, y):
        magnitude, phase = self.stft_fn(y)
        mel = torch.matmul(self.mel_basis.to(magnitude.dtype), magnitude)
        return torch.log(mel.clamp(min=1e-5)), magnitude, phase, torch.norm(magnitude, dim=1)


class VocoderWithBWE(nn.Module):
    def __init__(self, vocoder: Vocoder, bwe_generator: Vocoder, mel_stft: MelSTFT, input_sampling_rate: int, output_sampling_rate: int,
                 hop_length: int) -> None:  # fmt: skip
        super().__init__()
        self.vocoder, self.bwe_generator, self.mel_stft = vocoder, bwe_generator, mel_stft
        self.input_sampling_rate, self.output_sampling_rate, self.hop_length = input_sampling_rate, output_sampling_rate, hop_length
        self.resampler = UpSample1d(output_sampling_rate // input_sampling_rate, persistent=False, window_type="hann")

    @property
    def conv_pre(self):
        return self.vocoder.conv_pre

    @property
    def conv_post(self):
        return self.vocoder.conv_post

    def forward(self, x):
        low = self.vocoder(x)
        n = low.shape[-1]
        out_len = n * self.output_sampling_rate // self.input_sampling_rate
        if n % self.hop_length:
            low = F.pad(low, (0, self.hop_length - n % self.hop_length))
        b, c, _ = low.shape
        mel = self.mel_stft.mel_spectrogram(low.reshape(b * c, -1))[0]
        residual = self.bwe_generator(mel.reshape(b, c, mel.shape[1], mel.shape[2]).transpose(2, 3))
        skip = self.resampler(low)
        if residual.shape != skip.shape:
            raise ValueError(f"bandwidth-extension residual {tuple(residual.shape)} does not match the resampled signal {tuple(skip.shape)}")
        return (residual + skip).clamp(-1, 1)[..., :out_len]


class AudioDecoderConfigurator:
    @classmethod
    def from_config(cls, config: dict) -> AudioDecoder:
        a = config.get("audio_vae", {})
        params = a.get("model", {}).get("params", {})
        dd = params.get("ddconfig", {})
        pre = a.get("preprocessing", {})
        bins = dd.get("mel_bins") or pre.get("mel", {}).get("n_mel_channels") or a.get("variables", {}).get("mel_bins")
        return AudioDecoder(ch=int(dd.get("ch", 128)), out_ch=int(dd.get("out_ch", 2)), ch_mult=tuple(dd.get("ch_mult", (1, 2, 4))),
                            num_res_blocks=int(dd.get("num_res_blocks", 2)), attn_resolutions=set(dd.get("attn_resolutions", {8, 16, 32})),
                            resolution=int(dd.get("resolution", 256)), z_channels=int(dd.get("z_channels", 8)),
                            norm_type=NormType(dd.get("norm_type", "pixel")), causality_axis=CausalityAxis(dd.get("causality_axis", "height")),
                            dropout=float(dd.get("dropout", 0.0)), mid_block_add_attention=bool(dd.get("mid_block_add_attention", True)),
                            sample_rate=int(params.get("sampling_rate", 16000)), mel_hop_length=int(pre.get("stft", {}).get("hop_length", 160)),
                            is_causal=bool(pre.get("stft", {}).get("causal", True)), mel_bins=None if bins is None else int(bins))  # fmt: skip


def _vocoder_from(c: dict, resblock: str, activation: str, rate: int, final_activation: bool) -> Vocoder:
    return Vocoder(c.get("resblock_kernel_sizes", [3, 7, 11]), c.get("upsample_rates", [6, 5, 2, 2, 2]),
                   c.get("upsample_kernel_sizes", [16, 15, 8, 4, 4]), c.get("resblock_dilation_sizes", [[1, 3, 5]] * 3),
                   int(c.get("upsample_initial_channel", 1024)), str(c.get("resblock", resblock)), rate, str(c.get("activation", activation)),
                   bool(c.get("use_tanh_at_final", True)), final_activation, bool(c.get("use_bias_at_final", True)))  # fmt: skip


class VocoderConfigurator:
    @classmethod
    def from_config(cls, config: dict):
        cfg = config.get("vocoder", {})
        if "bwe" not in cfg:
            return _vocoder_from(cfg, "1", "snake", int(cfg.get("output_sampling_rate", 24000)), True)
        bwe = cfg["bwe"]
        rate_in, rate_out = int(bwe.get("input_sampling_rate", 24000)), int(bwe.get("output_sampling_rate", 48000))
        n_fft, hop = int(bwe.get("n_fft", 1024)), int(bwe.get("hop_length", 256))
        return VocoderWithBWE(_vocoder_from(cfg.get("vocoder", {}), "AMP1", "snakebeta", rate_in, True),
                              _vocoder_from(bwe, "AMP1", "snakebeta", rate_out, False),
                              MelSTFT(n_fft, hop, n_fft, int(bwe.get("num_mels", 64))), rate_in, rate_out, hop)  # fmt: skip


def split_audio_state_dicts(state_dict: dict) -> tuple[dict, dict]:
    """Shared LTX checkpoint -> (audio decoder weights, vocoder weights) with their prefixes removed."""
    dec, voc = {}, {}
    for k, v in state_dict.items():
        if k.startswith("audio_vae.decoder."):
            dec[k[len("audio_vae.decoder."):]] = v
        elif k.startswith("audio_vae.per_channel_statistics."):
            dec["per_channel_statistics." + k[len("audio_vae.per_channel_statistics."):]] = v
        elif k.startswith("vocoder."):
            voc[k[len("vocoder."):]] = v
    return dec, voc
