"""LTX-2 audio-video transformer (video-only, audio-only or joint), velocity and x0 forms.

Two token streams, video (inner width heads x 128) and audio (heads x 64), run through the same block: RMSNorm +
AdaLN-single modulation, self-attention (full-width q/k RMSNorm, rotary embedding over the whole inner width from
fractional positions, optional per-head sigmoid output gates), text cross-attention (optionally with its own AdaLN
on queries and on the prompt), bidirectional audio<->video cross-attention with rotary embeddings on the shared
time axis and timestep-driven scale / shift / gate tables, and a GELU-tanh MLP. Guidance perturbations can skip
a block's self- or cross-modal attention per sample (a skipped self-attention passes the value projection).
The modulated norms, the MLP (activation and gate * y + residual in the GEMM epilogues) and attention run on the
native kernels; the full-width rotary embedding and the masked forms use PyTorch.
Role parity: telefuser/models/ltx_dit.py:84-2227.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, replace
from enum import Enum

import numpy as np
import torch
import torch.nn.functional as F
from torch import nn

from telefuser_b200.core.base_model import BaseModel
from telefuser_b200.ops import functional as TF

ADALN_NUM_BASE_PARAMS, ADALN_NUM_CROSS_ATTN_PARAMS = 6, 3


class LTXRopeType(Enum):
    INTERLEAVED = "interleaved"
    SPLIT = "split"


class LTXModelType(Enum):
    AudioVideo = "ltx av model"
    VideoOnly = "ltx video only model"
    AudioOnly = "ltx audio only model"

    def is_video_enabled(self) -> bool:
        return self in (LTXModelType.AudioVideo, LTXModelType.VideoOnly)

    def is_audio_enabled(self) -> bool:
        return self in (LTXModelType.AudioVideo, LTXModelType.AudioOnly)


class PerturbationType(Enum):
    SKIP_A2V_CROSS_ATTN = "skip_a2v_cross_attn"
    SKIP_V2A_CROSS_ATTN = "skip_v2a_cross_attn"
    SKIP_VIDEO_SELF_ATTN = "skip_video_self_attn"
    SKIP_AUDIO_SELF_ATTN = "skip_audio_self_attn"


@dataclass(frozen=True)
class Perturbation:
    type: PerturbationType
    blocks: list | None  # None: every block

    def is_perturbed(self, kind: PerturbationType, block: int) -> bool:
        return self.type == kind and (self.blocks is None or block in self.blocks)


@dataclass(frozen=True)
class PerturbationConfig:
    perturbations: list | None

    def is_perturbed(self, kind: PerturbationType, block: int) -> bool:
        return bool(self.perturbations) and any(p.is_perturbed(kind, block) for p in self.perturbations)

    @staticmethod
    def empty() -> "PerturbationConfig":
        return PerturbationConfig([])


@dataclass(frozen=True)
class BatchedPerturbationConfig:
    perturbations: list

    def mask_like(self, kind: PerturbationType, block: int, values: torch.Tensor) -> torch.Tensor:
        m = torch.tensor([0.0 if p.is_perturbed(kind, block) else 1.0 for p in self.perturbations], device=values.device,
                         dtype=values.dtype)  # fmt: skip
        return m.view(-1, *([1] * (values.dim() - 1)))

    def any_in_batch(self, kind: PerturbationType, block: int) -> bool:
        return any(p.is_perturbed(kind, block) for p in self.perturbations)

    def all_in_batch(self, kind: PerturbationType, block: int) -> bool:
        return all(p.is_perturbed(kind, block) for p in self.perturbations)

    @staticmethod
    def empty(batch_size: int) -> "BatchedPerturbationConfig":
        return BatchedPerturbationConfig([PerturbationConfig.empty() for _ in range(batch_size)])


def to_velocity(sample, sigma, denoised_sample, calc_dtype=torch.float32):
    sigma = float(sigma) if not isinstance(sigma, torch.Tensor) or sigma.numel() == 1 else sigma.to(calc_dtype)
    return ((sample.to(calc_dtype) - denoised_sample.to(calc_dtype)) / sigma).to(sample.dtype)


def to_denoised(sample, velocity, sigma, calc_dtype=torch.float32):
    sigma = sigma.to(calc_dtype) if isinstance(sigma, torch.Tensor) else sigma
    return (sample.to(calc_dtype) - velocity.to(calc_dtype) * sigma).to(sample.dtype)


# ---- rotary embedding from fractional positions ----------------------------------------------
def _freq_grid(theta: float, n_pos_dims: int, inner_dim: int, double: bool) -> torch.Tensor:
    n = inner_dim // (2 * n_pos_dims)
    if double:
        return torch.tensor(np.power(theta, np.linspace(0.0, 1.0, n, dtype=np.float64)) * math.pi / 2, dtype=torch.float32)
    return (theta ** torch.linspace(math.log(1, theta), math.log(theta, theta), n, dtype=torch.float32)) * math.pi / 2


def precompute_freqs_cis(indices_grid, dim: int, out_dtype, theta: float = 10000.0, max_pos=None, use_middle_indices_grid=False,
                         num_attention_heads: int = 32, rope_type: LTXRopeType = LTXRopeType.INTERLEAVED,
                         double_precision: bool = False):  # fmt: skip
    """indices_grid [B, n_dims, T(, bounds)] -> (cos, sin): [B, T, dim] (interleaved) or [B, heads, T, dim/heads/2] (split)."""
    max_pos = max_pos or [20, 2048, 2048]
    freqs = _freq_grid(theta, indices_grid.shape[1], dim, double_precision)
    if use_middle_indices_grid:
        if indices_grid.dim() != 4:
            raise ValueError("middle-of-bounds positions need a [B, D, T, bounds] grid")
        indices_grid = indices_grid.mean(dim=-1) if indices_grid.shape[-1] == 2 else indices_grid[..., 0]
    elif indices_grid.dim() == 4:
        indices_grid = indices_grid[..., 0]
    frac = torch.stack([indices_grid[:, i] / max_pos[i] for i in range(indices_grid.shape[1])], dim=-1)  # [B, T, n]
    ang = (freqs.to(frac.device) * (frac.unsqueeze(-1) * 2 - 1)).transpose(-1, -2).flatten(2)  # [B, T, n_freq * n]
    if rope_type == LTXRopeType.SPLIT:
        pad = dim // 2 - ang.shape[-1]
        cos, sin = ang.cos(), ang.sin()
        if pad:
            cos = torch.cat([torch.ones_like(cos[..., :pad]), cos], dim=-1)
            sin = torch.cat([torch.zeros_like(sin[..., :pad]), sin], dim=-1)
        B, T = cos.shape[:2]
        return (cos.reshape(B, T, num_attention_heads, -1).transpose(1, 2).to(out_dtype),
                sin.reshape(B, T, num_attention_heads, -1).transpose(1, 2).to(out_dtype))  # fmt: skip
    cos, sin = ang.cos().repeat_interleave(2, dim=-1), ang.sin().repeat_interleave(2, dim=-1)
    pad = dim % (2 * indices_grid.shape[1])
    if pad:
        cos = torch.cat([torch.ones_like(cos[..., :pad]), cos], dim=-1)
        sin = torch.cat([torch.zeros_like(sin[..., :pad]), sin], dim=-1)
    return cos.to(out_dtype), sin.to(out_dtype)


def apply_rotary_emb(x, freqs_cis, rope_type: LTXRopeType = LTXRopeType.INTERLEAVED):
    cos, sin = freqs_cis
    if rope_type == LTXRopeType.INTERLEAVED:
        a, b = x.unflatten(-1, (-1, 2)).unbind(-1)
        rot = torch.stack((-b, a), dim=-1).flatten(-2)
        return x * cos + rot * sin
    (_, H, T, _), B = cos.shape, x.shape[0]  # split halves per head: x [B, T, H*D]; tables may have batch 1
    xh = x.reshape(B, T, H, -1).transpose(1, 2)
    first, second = xh.unflatten(-1, (2, -1)).unbind(-2)
    out = torch.stack([first * cos - second * sin, second * cos + first * sin], dim=-2).flatten(-2)
    return out.transpose(1, 2).reshape(B, T, -1)


# ---- embeddings ---------------------------------------------------------------------------
def get_timestep_embedding(t, dim: int, flip_sin_to_cos=False, downscale_freq_shift: float = 1, scale: float = 1, max_period=10000):
    half = dim // 2
    exponent = -math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.device) / (half - downscale_freq_shift)
    emb = scale * t[:, None].float() * torch.exp(exponent)[None, :]
    emb = torch.cat([emb.sin(), emb.cos()], dim=-1)
    return torch.cat([emb[:, half:], emb[:, :half]], dim=-1) if flip_sin_to_cos else emb


class TimestepEmbedding(nn.Module):
    def __init__(self, in_channels: int, time_embed_dim: int) -> None:
        super().__init__()
        self.linear_1, self.linear_2 = nn.Linear(in_channels, time_embed_dim), nn.Linear(time_embed_dim, time_embed_dim)

    def forward(self, x):
        l1, l2 = self.linear_1, self.linear_2
        return F.linear(F.silu(F.linear(x, l1.weight.float(), l1.bias.float())), l2.weight.float(), l2.bias.float())


class PixArtAlphaCombinedTimestepSizeEmbeddings(nn.Module):
    def __init__(self, embedding_dim: int, size_emb_dim: int = 0) -> None:
        super().__init__()
        self.timestep_embedder = TimestepEmbedding(256, embedding_dim)

    def forward(self, timestep):
        return self.timestep_embedder(get_timestep_embedding(timestep, 256, flip_sin_to_cos=True, downscale_freq_shift=0))


class AdaLayerNormSingle(nn.Module):
    def __init__(self, embedding_dim: int, embedding_coefficient: int = 6) -> None:
        super().__init__()
        self.emb = PixArtAlphaCombinedTimestepSizeEmbeddings(embedding_dim, embedding_dim // 3)
        self.linear = nn.Linear(embedding_dim, embedding_coefficient * embedding_dim)

    def forward(self, timestep):
        """-> fp32 (coefficients [N, k * dim], embedded timestep [N, dim])."""
        e = self.emb(timestep)
        return F.linear(F.silu(e), self.linear.weight.float(), self.linear.bias.float()), e


class PixArtAlphaTextProjection(nn.Module):
    def __init__(self, in_features: int, hidden_size: int, out_features: int | None = None) -> None:
        super().__init__()
        self.linear_1 = nn.Linear(in_features, hidden_size)
        self.linear_2 = nn.Linear(hidden_size, out_features or hidden_size)

    def forward(self, caption):
        return TF.linear(TF.linear(caption, self.linear_1.weight, self.linear_1.bias, act="gelu_tanh"), self.linear_2.weight,
                         self.linear_2.bias)  # fmt: skip


# ---- attention / MLP ------------------------------------------------------------------------
class _Weight(nn.Module):
    def __init__(self, dim: int) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))


def _masked_attention(q, k, v, mask):
    s = (q.float().permute(0, 2, 1, 3) @ k.float().permute(0, 2, 3, 1)) / math.sqrt(q.shape[-1]) + mask.float()
    return (torch.softmax(s, dim=-1) @ v.float().permute(0, 2, 1, 3)).permute(0, 2, 1, 3).to(q.dtype)


class Attention(nn.Module):
    def __init__(self, query_dim: int, context_dim: int | None = None, heads: int = 8, dim_head: int = 64, norm_eps: float = 1e-6,
                 rope_type: LTXRopeType = LTXRopeType.INTERLEAVED, apply_gated_attention: bool = False) -> None:  # fmt: skip
        super().__init__()
        inner = heads * dim_head
        context_dim = context_dim or query_dim
        self.heads, self.dim_head, self.rope_type, self.eps = heads, dim_head, rope_type, norm_eps
        self.q_norm, self.k_norm = _Weight(inner), _Weight(inner)
        self.to_q, self.to_k, self.to_v = nn.Linear(query_dim, inner), nn.Linear(context_dim, inner), nn.Linear(context_dim, inner)
        self.to_gate_logits = nn.Linear(query_dim, heads) if apply_gated_attention else None
        self.to_out = nn.Sequential(nn.Linear(inner, query_dim), nn.Identity())

    def forward(self, x, context=None, mask=None, pe=None, k_pe=None, perturbation_mask=None, all_perturbed: bool = False):
        """-> attention output before the out projection is added to anything (the projection is applied here)."""
        context = x if context is None else context
        H, D = self.heads, self.dim_head
        v = TF.linear(context, self.to_v.weight, self.to_v.bias)
        if all_perturbed:
            out = v
        else:
            q = TF.linear(x, self.to_q.weight, self.to_q.bias)
            k = TF.linear(context, self.to_k.weight, self.to_k.bias)
            TF.rmsnorm_rope_(q, self.q_norm.weight, 1, eps=self.eps)
            TF.rmsnorm_rope_(k, self.k_norm.weight, 1, eps=self.eps)
            if pe is not None:
                q = apply_rotary_emb(q.float(), pe, self.rope_type).to(v.dtype)
                k = apply_rotary_emb(k.float(), pe if k_pe is None else k_pe, self.rope_type).to(v.dtype)
            q4, k4, v4 = q.unflatten(-1, (H, D)), k.unflatten(-1, (H, D)), v.unflatten(-1, (H, D))
            if mask is None:
                out = TF.attention(q4.contiguous(), k4.contiguous(), v4)
            else:
                out = _masked_attention(q4, k4, v4, mask)
            out = out.flatten(-2)
            if perturbation_mask is not None:
                out = out * perturbation_mask + v * (1 - perturbation_mask)
        if self.to_gate_logits is not None:
            gates = 2.0 * torch.sigmoid(TF.linear(x, self.to_gate_logits.weight, self.to_gate_logits.bias).float())
            out = (out.unflatten(-1, (H, D)).float() * gates.unsqueeze(-1)).flatten(-2).to(x.dtype)
        return TF.linear(out, self.to_out[0].weight, self.to_out[0].bias)


class GELUApprox(nn.Module):
    def __init__(self, dim_in: int, dim_out: int) -> None:
        super().__init__()
        self.proj = nn.Linear(dim_in, dim_out)


class FeedForward(nn.Module):
    def __init__(self, dim: int, dim_out: int, mult: int = 4) -> None:
        super().__init__()
        self.net = nn.Sequential(GELUApprox(dim, int(dim * mult)), nn.Identity(), nn.Linear(int(dim * mult), dim_out))

    def forward(self, x, residual=None, gate=None):
        h = TF.linear(x, self.net[0].proj.weight, self.net[0].proj.bias, act="gelu_tanh")
        return TF.linear(h, self.net[2].weight, self.net[2].bias, residual=residual, gate=gate)


@dataclass
class TransformerConfig:
    dim: int
    heads: int
    d_head: int
    context_dim: int
    apply_gated_attention: bool = False
    cross_attention_adaln: bool = False


@dataclass
class Modality:
    latent: torch.Tensor  # [B, T, D]
    sigma: torch.Tensor  # [B]
    timesteps: torch.Tensor  # [B, T] or [B, 1]
    positions: torch.Tensor  # [B, n_dims, T(, bounds)]
    context: torch.Tensor
    enabled: bool = True
    context_mask: torch.Tensor | None = None
    attention_mask: torch.Tensor | None = None


@dataclass(frozen=True)
class TransformerArgs:
    x: torch.Tensor
    context: torch.Tensor
    context_mask: torch.Tensor | None
    timesteps: torch.Tensor
    embedded_timestep: torch.Tensor
    positional_embeddings: tuple
    cross_positional_embeddings: tuple | None
    cross_scale_shift_timestep: torch.Tensor | None
    cross_gate_timestep: torch.Tensor | None
    enabled: bool
    prompt_timestep: torch.Tensor | None = None
    self_attention_mask: torch.Tensor | None = None


def _ada(table: torch.Tensor, timestep: torch.Tensor, indices: slice):
    """table [k, C] + timestep coefficients [B, T|1, k*C] -> tuple of fp32 [B, T|1, C] for the rows in `indices`."""
    k = table.shape[0]
    vals = table[indices].float()[None, None] + timestep.reshape(timestep.shape[0], timestep.shape[1], k, -1)[:, :, indices]
    return vals.unbind(dim=2)


class BasicAVTransformerBlock(nn.Module):
    def __init__(self, idx: int, video: TransformerConfig | None = None, audio: TransformerConfig | None = None,
                 rope_type: LTXRopeType = LTXRopeType.INTERLEAVED, norm_eps: float = 1e-6) -> None:  # fmt: skip
        super().__init__()
        self.idx, self.norm_eps = idx, norm_eps
        def att(c: TransformerConfig, context_dim: int | None = None) -> Attention:
            return Attention(c.dim, context_dim, c.heads, c.d_head, norm_eps, rope_type, c.apply_gated_attention)

        if video is not None:
            self.attn1 = att(video)
            self.attn2 = att(video, video.context_dim)
            self.ff = FeedForward(video.dim, video.dim)
            self.scale_shift_table = nn.Parameter(torch.zeros(ADALN_NUM_BASE_PARAMS + (3 if video.cross_attention_adaln else 0), video.dim))
        if audio is not None:
            self.audio_attn1 = att(audio)
            self.audio_attn2 = att(audio, audio.context_dim)
            self.audio_ff = FeedForward(audio.dim, audio.dim)
            self.audio_scale_shift_table = nn.Parameter(torch.zeros(ADALN_NUM_BASE_PARAMS + (3 if audio.cross_attention_adaln else 0), audio.dim))
        if audio is not None and video is not None:
            self.audio_to_video_attn = Attention(video.dim, audio.dim, audio.heads, audio.d_head, norm_eps, rope_type, video.apply_gated_attention)
            self.video_to_audio_attn = Attention(audio.dim, video.dim, audio.heads, audio.d_head, norm_eps, rope_type, audio.apply_gated_attention)
            self.scale_shift_table_a2v_ca_audio = nn.Parameter(torch.zeros(5, audio.dim))
            self.scale_shift_table_a2v_ca_video = nn.Parameter(torch.zeros(5, video.dim))
        self.cross_attention_adaln = bool((video and video.cross_attention_adaln) or (audio and audio.cross_attention_adaln))
        if self.cross_attention_adaln and video is not None:
            self.prompt_scale_shift_table = nn.Parameter(torch.zeros(2, video.dim))
        if self.cross_attention_adaln and audio is not None:
            self.audio_prompt_scale_shift_table = nn.Parameter(torch.zeros(2, audio.dim))

    def _norm_mod(self, x, scale, shift):
        return TF.rmsnorm_modulate(x, None, shift, scale, self.norm_eps)

    def _text_cross(self, x, args: TransformerArgs, attn: Attention, table, prompt_table):
        if not self.cross_attention_adaln:
            return attn(TF.rmsnorm_modulate(x, None, None, None, self.norm_eps), context=args.context, mask=args.context_mask)
        shift_q, scale_q, gate = _ada(table, args.timesteps, slice(6, 9))
        pt = args.prompt_timestep
        shift_kv, scale_kv = (prompt_table.float()[None, None] + pt.reshape(x.shape[0], pt.shape[1], 2, -1)).unbind(dim=2)
        ctx = (args.context.float() * (1 + scale_kv) + shift_kv).to(x.dtype)
        return (attn(self._norm_mod(x, scale_q, shift_q), context=ctx, mask=args.context_mask).float() * gate).to(x.dtype)

    def _self_branch(self, x, args, attn1, attn2, table, prompt_table, kind, perturbations):
        shift, scale, gate = _ada(table, args.timesteps, slice(0, 3))
        skip_all = perturbations.all_in_batch(kind, self.idx)
        pmask = perturbations.mask_like(kind, self.idx, x) if (not skip_all and perturbations.any_in_batch(kind, self.idx)) else None
        a = attn1(self._norm_mod(x, scale, shift), pe=args.positional_embeddings, mask=args.self_attention_mask,
                  perturbation_mask=pmask, all_perturbed=skip_all)  # fmt: skip
        x = TF.gated_residual(x, a, gate)
        return x + self._text_cross(x, args, attn2, table, prompt_table)

    def _av_tables(self, table, args, indices):
        scale, shift = _ada(table[:4], args.cross_scale_shift_timestep, indices)
        (gate,) = _ada(table[4:], args.cross_gate_timestep, slice(None))
        return scale, shift, gate

    def forward(self, video: TransformerArgs | None, audio: TransformerArgs | None, perturbations: BatchedPerturbationConfig | None = None):
        if video is None and audio is None:
            raise ValueError("at least one of video or audio must be given")
        P = PerturbationType
        perturbations = perturbations or BatchedPerturbationConfig.empty((video or audio).x.shape[0])
        vx = video.x if video is not None else None
        ax = audio.x if audio is not None else None
        run_vx = video is not None and video.enabled and vx.numel() > 0
        run_ax = audio is not None and audio.enabled and ax.numel() > 0
        run_a2v = run_vx and audio is not None and ax.numel() > 0
        run_v2a = run_ax and video is not None and vx.numel() > 0
        if run_vx:
            vx = self._self_branch(vx, video, self.attn1, self.attn2, self.scale_shift_table,
                                   getattr(self, "prompt_scale_shift_table", None), P.SKIP_VIDEO_SELF_ATTN, perturbations)  # fmt: skip
        if run_ax:
            ax = self._self_branch(ax, audio, self.audio_attn1, self.audio_attn2, self.audio_scale_shift_table,
                                   getattr(self, "audio_prompt_scale_shift_table", None), P.SKIP_AUDIO_SELF_ATTN, perturbations)  # fmt: skip
        if run_a2v or run_v2a:
            tv, ta = self.scale_shift_table_a2v_ca_video, self.scale_shift_table_a2v_ca_audio
            if run_a2v and not perturbations.all_in_batch(P.SKIP_A2V_CROSS_ATTN, self.idx):
                sv, hv, gate = self._av_tables(tv, video, slice(0, 2))
                sa, ha, _ = self._av_tables(ta, audio, slice(0, 2))
                out = self.audio_to_video_attn(self._norm_mod(vx, sv, hv), context=self._norm_mod(ax, sa, ha),
                                               pe=video.cross_positional_embeddings, k_pe=audio.cross_positional_embeddings)  # fmt: skip
                a2v_in = (out.float() * gate * perturbations.mask_like(P.SKIP_A2V_CROSS_ATTN, self.idx, vx).float()).to(vx.dtype)
            else:
                a2v_in = None
            if run_v2a and not perturbations.all_in_batch(P.SKIP_V2A_CROSS_ATTN, self.idx):
                sa, ha, gate = self._av_tables(ta, audio, slice(2, 4))
                sv, hv, _ = self._av_tables(tv, video, slice(2, 4))
                # both directions read the streams as they were before either update, so the a2v result is added last
                out = self.video_to_audio_attn(self._norm_mod(ax, sa, ha), context=self._norm_mod(vx, sv, hv),
                                               pe=audio.cross_positional_embeddings, k_pe=video.cross_positional_embeddings)  # fmt: skip
                ax = ax + (out.float() * gate * perturbations.mask_like(P.SKIP_V2A_CROSS_ATTN, self.idx, ax).float()).to(ax.dtype)
            if a2v_in is not None:
                vx = vx + a2v_in
        if run_vx:
            shift, scale, gate = _ada(self.scale_shift_table, video.timesteps, slice(3, 6))
            vx = self.ff(self._norm_mod(vx, scale, shift), residual=vx, gate=gate)
        if run_ax:
            shift, scale, gate = _ada(self.audio_scale_shift_table, audio.timesteps, slice(3, 6))
            ax = self.audio_ff(self._norm_mod(ax, scale, shift), residual=ax, gate=gate)
        return (replace(video, x=vx) if video is not None else None, replace(audio, x=ax) if audio is not None else None)


class LTXModel(nn.Module):
    def __init__(self, *, model_type: LTXModelType = LTXModelType.AudioVideo, num_attention_heads: int = 32,
                 attention_head_dim: int = 128, in_channels: int = 128, out_channels: int = 128, num_layers: int = 48,
                 cross_attention_dim: int = 4096, norm_eps: float = 1e-6, positional_embedding_theta: float = 10000.0,
                 positional_embedding_max_pos=None, timestep_scale_multiplier: int = 1000, use_middle_indices_grid: bool = True,
                 audio_num_attention_heads: int = 32, audio_attention_head_dim: int = 64, audio_in_channels: int = 128,
                 audio_out_channels: int = 128, audio_cross_attention_dim: int = 2048, audio_positional_embedding_max_pos=None,
                 av_ca_timestep_scale_multiplier: int = 1, rope_type: LTXRopeType = LTXRopeType.INTERLEAVED,
                 double_precision_rope: bool = False, apply_gated_attention: bool = False, caption_projection=None,
                 audio_caption_projection=None, cross_attention_adaln: bool = False) -> None:  # fmt: skip
        super().__init__()
        self.model_type, self.cross_attention_adaln, self.rope_type = model_type, cross_attention_adaln, rope_type
        self.use_middle_indices_grid, self.double_precision_rope = use_middle_indices_grid, double_precision_rope
        self.timestep_scale_multiplier, self.positional_embedding_theta = timestep_scale_multiplier, positional_embedding_theta
        self.norm_eps = norm_eps
        k = ADALN_NUM_BASE_PARAMS + (ADALN_NUM_CROSS_ATTN_PARAMS if cross_attention_adaln else 0)
        vcfg = acfg = None
        if model_type.is_video_enabled():
            self.positional_embedding_max_pos = positional_embedding_max_pos or [20, 2048, 2048]
            self.num_attention_heads, self.inner_dim = num_attention_heads, num_attention_heads * attention_head_dim
            self.patchify_proj = nn.Linear(in_channels, self.inner_dim)
            if caption_projection is not None:
                self.caption_projection = caption_projection
            self.adaln_single = AdaLayerNormSingle(self.inner_dim, k)
            self.prompt_adaln_single = AdaLayerNormSingle(self.inner_dim, 2) if cross_attention_adaln else None
            self.scale_shift_table = nn.Parameter(torch.zeros(2, self.inner_dim))
            self.proj_out = nn.Linear(self.inner_dim, out_channels)
            vcfg = TransformerConfig(self.inner_dim, num_attention_heads, attention_head_dim, cross_attention_dim,
                                     apply_gated_attention, cross_attention_adaln)  # fmt: skip
        if model_type.is_audio_enabled():
            self.audio_positional_embedding_max_pos = audio_positional_embedding_max_pos or [20]
            self.audio_num_attention_heads = audio_num_attention_heads
            self.audio_inner_dim = audio_num_attention_heads * audio_attention_head_dim
            self.audio_patchify_proj = nn.Linear(audio_in_channels, self.audio_inner_dim)
            if audio_caption_projection is not None:
                self.audio_caption_projection = audio_caption_projection
            self.audio_adaln_single = AdaLayerNormSingle(self.audio_inner_dim, k)
            self.audio_prompt_adaln_single = AdaLayerNormSingle(self.audio_inner_dim, 2) if cross_attention_adaln else None
            self.audio_scale_shift_table = nn.Parameter(torch.zeros(2, self.audio_inner_dim))
            self.audio_proj_out = nn.Linear(self.audio_inner_dim, audio_out_channels)
            acfg = TransformerConfig(self.audio_inner_dim, audio_num_attention_heads, audio_attention_head_dim,
                                     audio_cross_attention_dim, apply_gated_attention, cross_attention_adaln)  # fmt: skip
        self.cross_pe_max_pos = None
        if vcfg is not None and acfg is not None:
            self.cross_pe_max_pos = max(self.positional_embedding_max_pos[0], self.audio_positional_embedding_max_pos[0])
            self.av_ca_timestep_scale_multiplier, self.audio_cross_attention_dim = av_ca_timestep_scale_multiplier, audio_cross_attention_dim
            self.av_ca_video_scale_shift_adaln_single = AdaLayerNormSingle(self.inner_dim, 4)
            self.av_ca_audio_scale_shift_adaln_single = AdaLayerNormSingle(self.audio_inner_dim, 4)
            self.av_ca_a2v_gate_adaln_single = AdaLayerNormSingle(self.inner_dim, 1)
            self.av_ca_v2a_gate_adaln_single = AdaLayerNormSingle(self.audio_inner_dim, 1)
        self.transformer_blocks = nn.ModuleList([BasicAVTransformerBlock(i, vcfg, acfg, rope_type, norm_eps) for i in range(num_layers)])

    # ---- argument preparation ---------------------------------------------------------------
    def _timestep(self, t, adaln: AdaLayerNormSingle, batch: int):
        coef, emb = adaln((t * self.timestep_scale_multiplier).flatten().float())
        return coef.view(batch, -1, coef.shape[-1]), emb.view(batch, -1, emb.shape[-1])

    def _pe(self, positions, dim: int, max_pos, heads: int, middle: bool):
        return precompute_freqs_cis(positions, dim, torch.float32, self.positional_embedding_theta, max_pos, middle, heads,
                                    self.rope_type, self.double_precision_rope)  # fmt: skip

    def _prepare(self, m: Modality, other: Modality | None, audio: bool) -> TransformerArgs:
        pre = "audio_" if audio else ""
        proj = getattr(self, pre + "patchify_proj")
        inner = self.audio_inner_dim if audio else self.inner_dim
        heads = self.audio_num_attention_heads if audio else self.num_attention_heads
        max_pos = self.audio_positional_embedding_max_pos if audio else self.positional_embedding_max_pos
        dt = proj.weight.dtype
        x = TF.linear(m.latent.to(dt), proj.weight, proj.bias)
        B = x.shape[0]
        timestep, embedded = self._timestep(m.timesteps, getattr(self, pre + "adaln_single"), B)
        prompt_adaln = getattr(self, pre + "prompt_adaln_single", None)
        prompt_t = self._timestep(m.sigma, prompt_adaln, B)[0] if prompt_adaln is not None else None
        cap = getattr(self, pre + "caption_projection", None)
        ctx = m.context.to(dt)
        ctx = cap(ctx) if cap is not None else ctx
        ctx = ctx.view(B, -1, ctx.shape[-1])
        cmask = m.context_mask
        if cmask is not None and not torch.is_floating_point(cmask):
            cmask = (cmask - 1).to(torch.float32).reshape(cmask.shape[0], 1, -1, cmask.shape[-1]) * torch.finfo(torch.float32).max
        smask = None
        if m.attention_mask is not None:
            am = m.attention_mask.float()
            smask = torch.where(am > 0, torch.log(am.clamp_min(torch.finfo(torch.float32).tiny)),
                                torch.full_like(am, torch.finfo(torch.float32).min)).unsqueeze(1)  # fmt: skip
        args = TransformerArgs(x=x, context=ctx, context_mask=cmask, timesteps=timestep, embedded_timestep=embedded,
                               positional_embeddings=self._pe(m.positions, inner, max_pos, heads, self.use_middle_indices_grid),
                               cross_positional_embeddings=None, cross_scale_shift_timestep=None, cross_gate_timestep=None,
                               enabled=m.enabled, prompt_timestep=prompt_t, self_attention_mask=smask)  # fmt: skip
        if other is None or self.cross_pe_max_pos is None:
            return args
        cross_t = other.sigma.view(m.timesteps.shape[0], 1, *[1] * (m.timesteps.dim() - 2)) * self.timestep_scale_multiplier
        factor = self.av_ca_timestep_scale_multiplier / self.timestep_scale_multiplier
        ss_adaln = self.av_ca_audio_scale_shift_adaln_single if audio else self.av_ca_video_scale_shift_adaln_single
        gate_adaln = self.av_ca_v2a_gate_adaln_single if audio else self.av_ca_a2v_gate_adaln_single
        ss = ss_adaln(cross_t.flatten().float())[0].view(B, -1, 4 * inner)
        gate = gate_adaln(cross_t.flatten().float() * factor)[0].view(B, -1, inner)
        cross_pe = self._pe(m.positions[:, 0:1], self.audio_cross_attention_dim, [self.cross_pe_max_pos], heads, True)
        return replace(args, cross_positional_embeddings=cross_pe, cross_scale_shift_timestep=ss, cross_gate_timestep=gate)

    def _output(self, table, proj_out, x, embedded):
        vals = table.float()[None, None] + embedded[:, :, None]
        return TF.linear(TF.layernorm_modulate(x, vals[:, :, 0], vals[:, :, 1], eps=self.norm_eps), proj_out.weight, proj_out.bias)

    @torch.no_grad()
    def forward(self, video: Modality | None, audio: Modality | None, perturbations: BatchedPerturbationConfig | None = None):
        if video is not None and not self.model_type.is_video_enabled():
            raise ValueError("video is not enabled for this model")
        if audio is not None and not self.model_type.is_audio_enabled():
            raise ValueError("audio is not enabled for this model")
        va = self._prepare(video, audio, False) if video is not None else None
        aa = self._prepare(audio, video, True) if audio is not None else None
        for blk in self.transformer_blocks:
            va, aa = blk(va, aa, perturbations)
        vx = self._output(self.scale_shift_table, self.proj_out, va.x, va.embedded_timestep) if va is not None else None
        ax = self._output(self.audio_scale_shift_table, self.audio_proj_out, aa.x, aa.embedded_timestep) if aa is not None else None
        return vx, ax


class X0Model(nn.Module):
    """Wraps the velocity model so that it returns denoised samples."""

    def __init__(self, velocity_model: LTXModel) -> None:
        super().__init__()
        self.velocity_model = velocity_model

    def forward(self, video, audio, perturbations=None):
        vx, ax = self.velocity_model(video, audio, perturbations)
        dv = to_denoised(video.latent, vx, video.timesteps.unsqueeze(-1) if video.timesteps.dim() == 2 else video.timesteps) if vx is not None else None
        da = to_denoised(audio.latent, ax, audio.timesteps.unsqueeze(-1) if audio.timesteps.dim() == 2 else audio.timesteps) if ax is not None else None
        return dv, da


LTX23_DEV_TRANSFORMER_CONFIG = {"transformer": dict(
    num_attention_heads=32, attention_head_dim=128, in_channels=128, out_channels=128, num_layers=48, cross_attention_dim=4096,
    norm_eps=1e-6, positional_embedding_theta=10000.0, positional_embedding_max_pos=[20, 2048, 2048], timestep_scale_multiplier=1000,
    use_middle_indices_grid=True, audio_num_attention_heads=32, audio_attention_head_dim=64, audio_in_channels=128,
    audio_out_channels=128, audio_cross_attention_dim=2048, audio_positional_embedding_max_pos=[20],
    av_ca_timestep_scale_multiplier=1000, rope_type="split", frequencies_precision="float64", apply_gated_attention=True,
    cross_attention_adaln=True, caption_channels=3840, caption_proj_before_connector=True)}  # fmt: skip


def build_ltx_model_from_config(config: dict, model_type: LTXModelType = LTXModelType.AudioVideo) -> LTXModel:
    c = dict(config.get("transformer", {}))
    cap = acap = None
    if not c.get("caption_proj_before_connector", False) and "caption_channels" in c:
        cap = PixArtAlphaTextProjection(c["caption_channels"], c.get("num_attention_heads", 32) * c.get("attention_head_dim", 128))
        if model_type.is_audio_enabled():
            acap = PixArtAlphaTextProjection(c["caption_channels"], c.get("audio_num_attention_heads", 32) * c.get("audio_attention_head_dim", 64))
    keys = ("num_attention_heads", "attention_head_dim", "in_channels", "out_channels", "num_layers", "cross_attention_dim", "norm_eps",
            "positional_embedding_theta", "positional_embedding_max_pos", "timestep_scale_multiplier", "use_middle_indices_grid",
            "audio_num_attention_heads", "audio_attention_head_dim", "audio_in_channels", "audio_out_channels",
            "audio_cross_attention_dim", "audio_positional_embedding_max_pos", "av_ca_timestep_scale_multiplier",
            "apply_gated_attention", "cross_attention_adaln")  # fmt: skip
    kw = {k: c[k] for k in keys if k in c}
    return LTXModel(model_type=model_type, rope_type=LTXRopeType(c.get("rope_type", "interleaved")),
                    double_precision_rope=c.get("frequencies_precision", False) == "float64", caption_projection=cap,
                    audio_caption_projection=acap, **kw)  # fmt: skip


class LTXVideoTransformer(BaseModel):
    def __init__(self, config: dict | None = None, model_type: LTXModelType = LTXModelType.AudioVideo) -> None:
        super().__init__()
        self.velocity_model = build_ltx_model_from_config(config or LTX23_DEV_TRANSFORMER_CONFIG, model_type)
        self.layer_name_list = ["velocity_model.transformer_blocks"]
        self.dtype = torch.bfloat16

    def get_fsdp_module_names(self) -> list[str]:
        return ["velocity_model.transformer_blocks"]

    def enable_quant(self, quant=None) -> int:
        """`quant`: a QuantConfig, a QuantType or a name. NF4 packs the block linears to 4.5 bits per weight (the 22B
        model then fits one GPU several times over); "fp8" (the default), "int8", "mxfp8" and "nvfp4" select the other
        stored formats. The per-head gate projections stay in bf16."""
        from telefuser_b200.ops.quant import quantize_model_

        self.quant_type = getattr(quant, "quant_type", quant)
        return quantize_model_(self, quant, ("velocity_model.transformer_blocks.*",), ("to_gate_logits",))

    def forward(self, video: Modality | None, audio: Modality | None = None, perturbations=None, x0: bool = False):
        if x0:
            return X0Model(self.velocity_model)(video, audio, perturbations)
        return self.velocity_model(video, audio, perturbations)

    @staticmethod
    def state_dict_converter():
        return LTXVideoTransformerStateDictConverter()


class LTXVideoTransformerStateDictConverter:
    """Checkpoints store the transformer under `model.diffusion_model.`; other entries (VAEs, vocoder) are dropped."""

    def from_official(self, sd: dict):
        prefix = "model.diffusion_model."
        out = {"velocity_model." + k[len(prefix):]: v for k, v in sd.items() if k.startswith(prefix)}
        return (out or dict(sd)), {}

    from_diffusers = from_official
