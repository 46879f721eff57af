"""Z-Image single-stream DiT.

Tokens: image patches (2x2, frame patch 1) and caption features, each padded to a multiple of 32 with a
learned pad token. Two modulated "noise refiner" blocks run on the image tokens, two unmodulated "context
refiner" blocks on the caption tokens, then `n_layers` modulated blocks on [image; caption]. A block is a
sandwich-norm transformer layer: RMSNorm * (1 + scale) -> attention (per-head RMSNorm, 3-axis interleaved
RoPE, theta 256) -> RMSNorm -> tanh-gated residual, then the same around a SwiGLU MLP. The modulation comes
from a 256-wide timestep embedding through one Linear per block. Samples are lists (variable sizes); samples
of equal token counts run as one batch, others one by one, which equals the masked batched evaluation because
padding beyond a sample's own length is never attended.
Role parity: telefuser/models/z_image_dit.py:20-695.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn

from telefuser_b200.core.base_model import BaseModel
from telefuser_b200.models.qwen_image_dit import _WeightOnly
from telefuser_b200.ops import functional as TF

ADALN_EMBED_DIM = 256
SEQ_MULTI_OF = 32


def timestep_embedding(t: torch.Tensor, dim: int = 256, max_period: float = 10000.0) -> torch.Tensor:
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    args = t[:, None].float() * freqs[None]
    return torch.cat([args.cos(), args.sin()], dim=-1)


class TimestepEmbedder(nn.Module):
    def __init__(self, out_size: int, mid_size: int) -> None:
        super().__init__()
        self.mlp = nn.Sequential(nn.Linear(256, mid_size), nn.SiLU(), nn.Linear(mid_size, out_size))

    def forward(self, t):
        h = F.silu(F.linear(timestep_embedding(t), self.mlp[0].weight.float(), self.mlp[0].bias.float()))
        return F.linear(h, self.mlp[2].weight.float(), self.mlp[2].bias.float())  # fp32 [B, out]


def rope_tables(ids: torch.Tensor, axes_dims, theta: float) -> tuple[torch.Tensor, torch.Tensor]:
    """ids [S, 3] -> fp32 (cos, sin) [S, head_dim / 2]; angles rounded to fp32 before cos / sin."""
    parts = []
    for i, d in enumerate(axes_dims):
        inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float64, device=ids.device) / d))
        parts.append(torch.outer(ids[:, i].to(torch.float64), inv).float())
    ang = torch.cat(parts, dim=-1)
    return ang.cos().contiguous(), ang.sin().contiguous()


class FeedForward(nn.Module):
    def __init__(self, dim: int, hidden: int) -> None:
        super().__init__()
        self.w1 = nn.Linear(dim, hidden, bias=False)
        self.w2 = nn.Linear(hidden, dim, bias=False)
        self.w3 = nn.Linear(dim, hidden, bias=False)
        self._w13 = None

    def forward(self, x):
        from telefuser_b200.models.wan_dit import _fuse_linear_weights

        w = self.w1.weight
        if self._w13 is None or self._w13[0].data_ptr() != w.data_ptr() or self._w13[0].dtype != w.dtype:
            self._w13 = _fuse_linear_weights([self.w1, self.w3])
        return TF.linear(TF.silu_and_mul(TF.linear(x, self._w13[0])), self.w2.weight)


class ZImageAttention(nn.Module):
    def __init__(self, dim: int, n_heads: int, n_kv_heads: int, qk_norm: bool, eps: float) -> None:
        super().__init__()
        self.n_heads, self.n_kv_heads, self.head_dim, self.eps = n_heads, n_kv_heads, dim // n_heads, eps
        self.to_q = nn.Linear(dim, n_heads * self.head_dim, bias=False)
        self.to_k = nn.Linear(dim, n_kv_heads * self.head_dim, bias=False)
        self.to_v = nn.Linear(dim, n_kv_heads * self.head_dim, bias=False)
        self.to_out = nn.ModuleList([nn.Linear(n_heads * self.head_dim, dim, bias=False)])
        self.norm_q = _WeightOnly(self.head_dim) if qk_norm else None
        self.norm_k = _WeightOnly(self.head_dim) if qk_norm else None
        self._qkv = None
        self.usp = False

    def forward(self, x, rope):
        from telefuser_b200.models.wan_dit import _fuse_linear_weights

        B, S, _ = x.shape
        H, Hk, D = self.n_heads, self.n_kv_heads, self.head_dim
        w = self.to_q.weight
        if self._qkv is None or self._qkv[0].data_ptr() != w.data_ptr() or self._qkv[0].dtype != w.dtype:
            self._qkv = _fuse_linear_weights([self.to_q, self.to_k, self.to_v])
        fused = TF.linear(x, self._qkv[0])
        q = fused[..., : H * D].unflatten(-1, (H, D))
        k = fused[..., H * D : (H + Hk) * D].unflatten(-1, (Hk, D))
        v = fused[..., (H + Hk) * D :].unflatten(-1, (Hk, D))
        cos, sin = rope if B == 1 else tuple(t.repeat(B, 1) for t in rope)
        if self.norm_q is not None:
            if H == Hk:
                TF.headnorm_rope_(q, self.norm_q.weight, cos, sin, self.eps, k=k, weight_k=self.norm_k.weight)
            else:
                TF.headnorm_rope_(q, self.norm_q.weight, cos, sin, self.eps)
                TF.headnorm_rope_(k, self.norm_k.weight, cos, sin, self.eps)
        else:
            q = TF.rope_reference(q.reshape(1, B * S, H, D), cos, sin).reshape(B, S, H, D).to(x.dtype)
            k = TF.rope_reference(k.reshape(1, B * S, Hk, D), cos, sin).reshape(B, S, Hk, D).to(x.dtype)
        if Hk != H:
            k, v = (t.repeat_interleave(H // Hk, dim=2) for t in (k, v))
        if self.usp:
            from telefuser_b200.parallel.ring import long_context_attention

            o = long_context_attention(q, k, v)
        else:
            o = TF.attention(q, k, v)
        return TF.linear(o.reshape(B, S, H * D), self.to_out[0].weight)


class ZImageTransformerBlock(nn.Module):
    def __init__(self, dim: int, n_heads: int, n_kv_heads: int, norm_eps: float, qk_norm: bool, modulation: bool = True):
        super().__init__()
        self.eps, self.modulation = norm_eps, modulation
        self.attention = ZImageAttention(dim, n_heads, n_kv_heads, qk_norm, norm_eps)
        self.feed_forward = FeedForward(dim, int(dim / 3 * 8))
        self.attention_norm1, self.ffn_norm1 = _WeightOnly(dim), _WeightOnly(dim)
        self.attention_norm2, self.ffn_norm2 = _WeightOnly(dim), _WeightOnly(dim)
        if modulation:
            self.adaLN_modulation = nn.ModuleList([nn.Linear(min(dim, ADALN_EMBED_DIM), 4 * dim)])

    def forward(self, x, rope, adaln_input=None):
        if self.modulation:
            lin = self.adaLN_modulation[0]
            m = F.linear(adaln_input, lin.weight.float(), lin.bias.float()).unsqueeze(1)  # fp32 [B, 1, 4C]
            scale_msa, gate_msa, scale_mlp, gate_mlp = m.chunk(4, dim=2)
        else:
            scale_msa = gate_msa = scale_mlp = gate_mlp = None
        tanh = self.modulation
        a = self.attention(TF.rmsnorm_modulate(x, self.attention_norm1.weight, None, scale_msa, self.eps), rope)
        x = TF.rmsnorm_gate_residual(x, a, self.attention_norm2.weight, gate_msa, self.eps, tanh_gate=tanh)
        f = self.feed_forward(TF.rmsnorm_modulate(x, self.ffn_norm1.weight, None, scale_mlp, self.eps))
        return TF.rmsnorm_gate_residual(x, f, self.ffn_norm2.weight, gate_mlp, self.eps, tanh_gate=tanh)


class FinalLayer(nn.Module):
    def __init__(self, hidden: int, out_channels: int) -> None:
        super().__init__()
        self.linear = nn.Linear(hidden, out_channels)
        self.adaLN_modulation = nn.Sequential(nn.SiLU(), nn.Linear(min(hidden, ADALN_EMBED_DIM), hidden))

    def forward(self, x, c):
        lin = self.adaLN_modulation[1]
        scale = F.linear(F.silu(c), lin.weight.float(), lin.bias.float()).unsqueeze(1)
        return TF.linear(TF.layernorm_modulate(x, None, scale, eps=1e-6), self.linear.weight, self.linear.bias)


def _pad_to_multiple(tokens: torch.Tensor) -> tuple[torch.Tensor, int]:
    pad = (-tokens.shape[0]) % SEQ_MULTI_OF
    if pad:
        tokens = torch.cat([tokens, tokens[-1:].expand(pad, -1)], dim=0)
    return tokens, pad


def _grid(size, start, device):
    axes = [torch.arange(s0, s0 + n, dtype=torch.int32, device=device) for s0, n in zip(start, size)]
    return torch.stack(torch.meshgrid(axes, indexing="ij"), dim=-1).flatten(0, 2)


class ZImageTransformer2DModel(BaseModel):
    def __init__(self, all_patch_size=(2,), all_f_patch_size=(1,), in_channels: int = 16, dim: int = 3840, n_layers: int = 30,
                 n_refiner_layers: int = 2, n_heads: int = 30, n_kv_heads: int = 30, norm_eps: float = 1e-5,
                 qk_norm: bool = True, cap_feat_dim: int = 2560, rope_theta: float = 256.0, t_scale: float = 1000.0,
                 axes_dims=(32, 48, 48), axes_lens=(1536, 512, 512)) -> None:  # fmt: skip
        super().__init__()
        if dim // n_heads != sum(axes_dims):
            raise ValueError("RoPE axes must add up to the head dimension")
        self.in_channels = self.out_channels = in_channels
        self.all_patch_size, self.all_f_patch_size = tuple(all_patch_size), tuple(all_f_patch_size)
        self.dim, self.n_heads, self.n_layers = dim, n_heads, n_layers
        self.rope_theta, self.t_scale, self.axes_dims, self.axes_lens = rope_theta, t_scale, tuple(axes_dims), tuple(axes_lens)
        self.layer_name_list = ["layers"]
        self.all_x_embedder = nn.ModuleDict()
        self.all_final_layer = nn.ModuleDict()
        for p, fp in zip(self.all_patch_size, self.all_f_patch_size):
            self.all_x_embedder[f"{p}-{fp}"] = nn.Linear(fp * p * p * in_channels, dim)
            self.all_final_layer[f"{p}-{fp}"] = FinalLayer(dim, p * p * fp * in_channels)
        blk = (dim, n_heads, n_kv_heads, norm_eps, qk_norm)
        self.noise_refiner = nn.ModuleList([ZImageTransformerBlock(*blk, modulation=True) for _ in range(n_refiner_layers)])
        self.context_refiner = nn.ModuleList([ZImageTransformerBlock(*blk, modulation=False) for _ in range(n_refiner_layers)])
        self.t_embedder = TimestepEmbedder(min(dim, ADALN_EMBED_DIM), 1024)
        self.cap_embedder = nn.Sequential(_WeightOnly(cap_feat_dim), nn.Linear(cap_feat_dim, dim))
        self.norm_eps = norm_eps
        self.x_pad_token = nn.Parameter(torch.zeros(1, dim))
        self.cap_pad_token = nn.Parameter(torch.zeros(1, dim))
        self.layers = nn.ModuleList([ZImageTransformerBlock(*blk) for _ in range(n_layers)])
        self.dtype = torch.bfloat16

    def enable_usp(self) -> None:
        super().enable_usp()
        for b in self.layers:
            b.attention.usp = True

    def get_fsdp_module_names(self) -> list[str]:
        return ["layers"]

    def enable_quant(self, quant=None) -> int:
        from telefuser_b200.ops.quant import quantize_model_

        return quantize_model_(self, quant, ("layers.*",), ("adaLN_modulation",))

    def enable_async_offload(self, device, offload_config) -> None:
        from telefuser_b200.offload.async_offload import AsyncOffloadManager

        self.async_offload_manager = AsyncOffloadManager(
            list(self.layers), enabled=True, offload_ratio=offload_config.offload_ratio,
            prefetch_size=offload_config.prefetch_size, device=device, pin_cpu_memory=offload_config.pin_cpu_memory)  # fmt: skip
        self.async_offload_flag = True

    def forward_blocks(self, unified, rope, adaln_input):
        offload = getattr(self, "async_offload_manager", None) if self.async_offload_flag else None
        for i, layer in enumerate(self.layers):
            if offload is not None:
                offload.before_layer(i)
            unified = layer(unified, rope, adaln_input)
            if offload is not None:
                offload.after_layer(i)
        return unified

    def _embed_sample(self, image, cap, p: int, fp: int):
        """One sample -> (image tokens, caption tokens, image rope, caption rope, (F, H, W), n image tokens)."""
        dev = image.device
        dt = self.all_x_embedder[f"{p}-{fp}"].weight.dtype
        cap, cap_pad = _pad_to_multiple(cap.to(dt))
        cap_len = cap.shape[0]
        cap_ids = _grid((cap_len, 1, 1), (1, 0, 0), dev)
        C, Fr, H, W = image.shape
        ft, ht, wt = Fr // fp, H // p, W // p
        tok = image.to(dt).view(C, ft, fp, ht, p, wt, p).permute(1, 3, 5, 2, 4, 6, 0).reshape(ft * ht * wt, fp * p * p * C)
        n_img = tok.shape[0]
        tok, img_pad = _pad_to_multiple(tok)
        img_ids = _grid((ft, ht, wt), (cap_len + 1, 0, 0), dev)
        if img_pad:
            img_ids = torch.cat([img_ids, img_ids.new_zeros(img_pad, 3)], dim=0)
        emb = self.all_x_embedder[f"{p}-{fp}"]
        x = TF.linear(tok, emb.weight, emb.bias)
        if img_pad:
            x[n_img:] = self.x_pad_token.to(dt)
        c = TF.rmsnorm_modulate(cap, self.cap_embedder[0].weight, None, None, self.norm_eps)
        c = TF.linear(c, self.cap_embedder[1].weight, self.cap_embedder[1].bias)
        if cap_pad:
            c[cap_len - cap_pad :] = self.cap_pad_token.to(dt)
        return (x, c, rope_tables(img_ids, self.axes_dims, self.rope_theta),
                rope_tables(cap_ids, self.axes_dims, self.rope_theta), (Fr, H, W), n_img)  # fmt: skip

    def _run_group(self, xs, cs, img_rope, cap_rope, adaln, final, cond_flag: bool):
        """Samples of identical token counts and positions as one batch: [B, S, C] each."""
        x, c = torch.stack(xs), torch.stack(cs)
        for layer in self.noise_refiner:
            x = layer(x, img_rope, adaln)
        for layer in self.context_refiner:
            c = layer(c, cap_rope)
        unified = torch.cat([x, c], dim=1)
        rope = tuple(torch.cat([a, b], dim=0) for a, b in zip(img_rope, cap_rope))
        ori = unified
        cache = self.feature_cache
        if cache.should_compute(cond_flag):
            unified = self.forward_blocks(unified, rope, adaln)
            cache.update(unified, ori, cond_flag)
        else:
            unified = cache.approximate(unified, cond_flag)
        return final(unified, adaln)

    @torch.no_grad()
    def forward(self, x: list, t: torch.Tensor, cap_feats: list, patch_size: int = 2, f_patch_size: int = 1, cond_flag: bool = True):
        """x: list of [C, F, H, W] latents; t [B] in [0, 1]; cap_feats: list of [L_i, cap_feat_dim] -> list of [C, F, H, W]."""
        if patch_size not in self.all_patch_size or f_patch_size not in self.all_f_patch_size:
            raise ValueError("unsupported patch size")
        p, fp = patch_size, f_patch_size
        adaln = self.t_embedder(t.to(x[0].device).float() * self.t_scale)
        samples = [self._embed_sample(img, cap, p, fp) for img, cap in zip(x, cap_feats)]
        final = self.all_final_layer[f"{p}-{fp}"]
        same = all(s[0].shape == samples[0][0].shape and s[1].shape == samples[0][1].shape and s[4] == samples[0][4]
                   for s in samples)  # fmt: skip
        if same:
            s0 = samples[0]
            out = self._run_group([s[0] for s in samples], [s[1] for s in samples], s0[2], s0[3], adaln, final, cond_flag)
            outs = list(out.unbind(0))
        else:
            outs = [self._run_group([s[0]], [s[1]], s[2], s[3], adaln[i : i + 1], final, cond_flag)[0]
                    for i, s in enumerate(samples)]  # fmt: skip
        res = []
        for o, s in zip(outs, samples):
            Fr, H, W = s[4]
            o = o[: s[5]].view(Fr // fp, H // p, W // p, fp, p, p, self.out_channels)
            res.append(o.permute(6, 0, 3, 1, 4, 2, 5).reshape(self.out_channels, Fr, H, W))
        return res

    @staticmethod
    def state_dict_converter():
        return ZImageDitStateDictConverter()


class ZImageDitStateDictConverter:
    def from_diffusers(self, sd: dict):
        return sd, {}

    def from_official(self, sd: dict):
        return sd, {}


def _register() -> None:
    from telefuser_b200.core.model_registry import register_architecture

    register_architecture("zimage_dit", ZImageTransformer2DModel, lambda: ZImageTransformer2DModel(), resource="diffusers")


_register()
