"""Qwen-Image MM-DiT: dual-stream (image / text) blocks with joint attention.

60 blocks, width 3072, 24 heads x 128, text width 3584, 2x2 latent patches (64 channels in / out).
Every block: per-stream AdaLN (LayerNorm + shift/scale/gate from the timestep embedding), per-stream
fused QKV GEMM, per-head RMSNorm + centred 3-axis RoPE (axes 16/56/56, text positions placed after the
largest image coordinate), ONE attention over [text; image], per-stream output projection and GELU-tanh
MLP with the gate and the residual folded into the GEMM epilogues. Edit latents are extra image streams
appended to the image tokens with their own frame index. Parameter names follow the public checkpoint.
Role parity: telefuser/models/qwen_image_dit.py:32-814.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn

from telefuser_b200.core.base_model import BaseModel
from telefuser_b200.ops import functional as TF
from telefuser_b200.parallel import shard as pshard


def timestep_embedding(t: torch.Tensor, dim: int = 256, scale: float = 1000.0, max_period: float = 10000.0):
    """cos-first sinusoidal embedding (flip_sin_to_cos, downscale_freq_shift 0)."""
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    ang = scale * t.float()[:, None] * freqs[None, :]
    return torch.cat([ang.cos(), ang.sin()], dim=-1)


class _WeightOnly(nn.Module):
    def __init__(self, dim: int) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))


class _TimestepEmbedder(nn.Module):
    def __init__(self, in_dim: int, dim: int) -> None:
        super().__init__()
        self.linear_1 = nn.Linear(in_dim, dim)
        self.linear_2 = nn.Linear(dim, dim)


class _TimeTextEmbed(nn.Module):
    def __init__(self, dim: int) -> None:
        super().__init__()
        self.timestep_embedder = _TimestepEmbedder(256, dim)

    def forward(self, timestep):
        e = self.timestep_embedder
        h = F.silu(F.linear(timestep_embedding(timestep), e.linear_1.weight.float(), e.linear_1.bias.float()))
        return F.linear(h, e.linear_2.weight.float(), e.linear_2.bias.float())  # fp32 [B, dim]


class _GeluProj(nn.Module):
    def __init__(self, dim: int, inner: int) -> None:
        super().__init__()
        self.proj = nn.Linear(dim, inner)


class FeedForward(nn.Module):
    """`net.0.proj` (GELU-tanh) -> `net.2`."""

    def __init__(self, dim: int, mult: int = 4) -> None:
        super().__init__()
        self.net = nn.ModuleList([_GeluProj(dim, dim * mult), nn.Identity(), nn.Linear(dim * mult, dim)])

    def forward(self, x, residual=None, gate=None):
        h = TF.linear(x, self.net[0].proj.weight, self.net[0].proj.bias, act="gelu_tanh")
        return TF.linear(h, self.net[2].weight, self.net[2].bias, residual=residual, gate=gate)


class QwenEmbedRope:
    def __init__(self, theta: float, axes_dim, scale_rope: bool = True) -> None:
        self.theta, self.axes_dim, self.scale_rope = theta, tuple(axes_dim), scale_rope

    def _angles(self, pos: torch.Tensor) -> torch.Tensor:
        """pos: float [S, 3] -> angles [S, sum(axes)/2]."""
        out = []
        for a, d in enumerate(self.axes_dim):
            inv = 1.0 / torch.pow(self.theta, torch.arange(0, d, 2, dtype=torch.float32) / d)
            out.append(pos[:, a : a + 1] * inv[None])
        return torch.cat(out, dim=-1)

    def __call__(self, img_shapes, txt_len: int, device):
        """Returns ((cos, sin) for the image tokens, (cos, sin) for the text tokens), fp32 [S, D/2]."""
        pos, max_idx = [], 0
        for idx, (f, h, w) in enumerate(img_shapes):
            if self.scale_rope:
                hh = torch.cat([torch.arange(-(h - h // 2), 0), torch.arange(0, h // 2)]).float()
                ww = torch.cat([torch.arange(-(w - w // 2), 0), torch.arange(0, w // 2)]).float()
                max_idx = max(max_idx, h // 2, w // 2)
            else:
                hh, ww = torch.arange(h).float(), torch.arange(w).float()
                max_idx = max(max_idx, h, w)
            ff = torch.arange(idx, idx + f).float()
            grid = torch.stack(torch.meshgrid(ff, hh, ww, indexing="ij"), dim=-1).reshape(-1, 3)
            pos.append(grid)
        ia = self._angles(torch.cat(pos))
        tp = torch.arange(max_idx, max_idx + txt_len).float()
        ta = self._angles(tp[:, None].expand(-1, 3))
        return (ia.cos().to(device), ia.sin().to(device)), (ta.cos().to(device), ta.sin().to(device))


class QwenDoubleStreamAttention(nn.Module):
    def __init__(self, dim: int, num_heads: int, head_dim: int) -> None:
        super().__init__()
        self.num_heads, self.head_dim = num_heads, head_dim
        self.to_q, self.to_k, self.to_v = (nn.Linear(dim, dim) for _ in range(3))
        self.norm_q, self.norm_k = _WeightOnly(head_dim), _WeightOnly(head_dim)
        self.add_q_proj, self.add_k_proj, self.add_v_proj = (nn.Linear(dim, dim) for _ in range(3))
        self.norm_added_q, self.norm_added_k = _WeightOnly(head_dim), _WeightOnly(head_dim)
        self.to_out = nn.Sequential(nn.Linear(dim, dim))
        self.to_add_out = nn.Linear(dim, dim)
        self._img = self._txt = None
        self.usp = False

    def fused_img(self):
        from telefuser_b200.models.wan_dit import _fuse_linear_weights

        w = self.to_q.weight
        if self._img is None or self._img[0].data_ptr() != w.data_ptr() or self._img[0].dtype != w.dtype:
            self._img = _fuse_linear_weights([self.to_q, self.to_k, self.to_v])
        return self._img

    def fused_txt(self):
        from telefuser_b200.models.wan_dit import _fuse_linear_weights

        w = self.add_q_proj.weight
        if self._txt is None or self._txt[0].data_ptr() != w.data_ptr() or self._txt[0].dtype != w.dtype:
            self._txt = _fuse_linear_weights([self.add_q_proj, self.add_k_proj, self.add_v_proj])
        return self._txt

    def forward(self, image, text, img_rope, txt_rope):
        """image [B, Si, C], text [B, St, C] (already modulated) -> attention outputs before the out projections."""
        B, Si, C = image.shape
        St = text.shape[1]
        H, D = self.num_heads, self.head_dim
        Wt, bt = self.fused_txt()
        Wi, bi = self.fused_img()
        if B == 1:  # both projections write straight into the joint buffer
            joint = torch.empty(B, St + Si, 3 * C, device=image.device, dtype=image.dtype)
            TF.linear(text, Wt, bt, out=joint[:, :St])
            TF.linear(image, Wi, bi, out=joint[:, St:])
        else:
            joint = torch.cat([TF.linear(text, Wt, bt), TF.linear(image, Wi, bi)], dim=1)
            txt_rope = tuple(t.repeat(B, 1) for t in txt_rope)
            img_rope = tuple(t.repeat(B, 1) for t in img_rope)
        q, k, v = (joint[..., i * C : (i + 1) * C].unflatten(-1, (H, D)) for i in range(3))
        TF.headnorm_rope_(q[:, :St], self.norm_added_q.weight, txt_rope[0], txt_rope[1], 1e-6, k=k[:, :St],
                          weight_k=self.norm_added_k.weight)  # fmt: skip
        TF.headnorm_rope_(q[:, St:], self.norm_q.weight, img_rope[0], img_rope[1], 1e-6, k=k[:, St:],
                          weight_k=self.norm_k.weight)  # fmt: skip
        if self.usp:
            from telefuser_b200.parallel.ring import long_context_attention

            o = long_context_attention(q, k, v)
        else:
            o = TF.attention(q, k, v)
        o = o.reshape(B, St + Si, C)
        return o[:, St:], o[:, :St]


class QwenImageTransformerBlock(nn.Module):
    def __init__(self, dim: int, num_heads: int, head_dim: int, eps: float = 1e-6) -> None:
        super().__init__()
        self.dim, self.eps = dim, eps
        self.img_mod = nn.Sequential(nn.SiLU(), nn.Linear(dim, 6 * dim))
        self.attn = QwenDoubleStreamAttention(dim, num_heads, head_dim)
        self.img_mlp = FeedForward(dim)
        self.txt_mod = nn.Sequential(nn.SiLU(), nn.Linear(dim, 6 * dim))
        self.txt_mlp = FeedForward(dim)

    def _mods(self, mod: nn.Sequential, silu_temb):
        m = F.linear(silu_temb, mod[1].weight.float(), mod[1].bias.float())  # fp32 [B, 6C]
        return [c.unsqueeze(1) for c in m.chunk(6, dim=-1)]  # shift1, scale1, gate1, shift2, scale2, gate2

    def forward(self, image, text, silu_temb, img_rope, txt_rope):
        si1, ci1, gi1, si2, ci2, gi2 = self._mods(self.img_mod, silu_temb)
        st1, ct1, gt1, st2, ct2, gt2 = self._mods(self.txt_mod, silu_temb)
        a = self.attn
        io, to = a(TF.layernorm_modulate(image, si1, ci1, eps=self.eps), TF.layernorm_modulate(text, st1, ct1, eps=self.eps),
                   img_rope, txt_rope)  # fmt: skip
        image = TF.linear(io, a.to_out[0].weight, a.to_out[0].bias, residual=image, gate=gi1)
        text = TF.linear(to, a.to_add_out.weight, a.to_add_out.bias, residual=text, gate=gt1)
        image = self.img_mlp(TF.layernorm_modulate(image, si2, ci2, eps=self.eps), residual=image, gate=gi2)
        text = self.txt_mlp(TF.layernorm_modulate(text, st2, ct2, eps=self.eps), residual=text, gate=gt2)
        return text, image


class _AdaNormOut(nn.Module):
    def __init__(self, dim: int) -> None:
        super().__init__()
        self.linear = nn.Linear(dim, 2 * dim)


class QwenImageDiT(BaseModel):
    def __init__(self, num_layers: int = 60, dim: int = 3072, num_heads: int = 24, head_dim: int = 128,
                 text_dim: int = 3584, in_channels: int = 64, axes_dim=(16, 56, 56)) -> None:  # fmt: skip
        super().__init__()
        if sum(axes_dim) != head_dim:
            raise ValueError("RoPE axes must add up to the head dimension")
        self.dim, self.num_layers = dim, num_layers
        self.pos_embed = QwenEmbedRope(10000.0, axes_dim, scale_rope=True)
        self.time_text_embed = _TimeTextEmbed(dim)
        self.txt_norm = _WeightOnly(text_dim)
        self.img_in = nn.Linear(in_channels, dim)
        self.txt_in = nn.Linear(text_dim, dim)
        self.transformer_blocks = nn.ModuleList([QwenImageTransformerBlock(dim, num_heads, head_dim)
                                                 for _ in range(num_layers)])  # fmt: skip
        self.norm_out = _AdaNormOut(dim)
        self.proj_out = nn.Linear(dim, in_channels)
        self.layer_name_list = ["transformer_blocks"]
        self.dtype = torch.bfloat16

    def enable_usp(self) -> None:
        super().enable_usp()
        for b in self.transformer_blocks:
            b.attn.usp = True

    def get_fsdp_module_names(self) -> list[str]:
        return ["transformer_blocks"]

    def enable_quant(self, quant=None) -> int:
        from telefuser_b200.ops.quant import quantize_model_

        return quantize_model_(self, quant, ("transformer_blocks.*",), ("img_mod", "txt_mod"))

    @staticmethod
    def _patchify(x):
        B, C, H, W = x.shape
        return x.reshape(B, C, H // 2, 2, W // 2, 2).permute(0, 2, 4, 1, 3, 5).reshape(B, (H // 2) * (W // 2), C * 4)

    def forward_blocks(self, image, text, silu_temb, img_rope, txt_rope):
        offload = getattr(self, "async_offload_manager", None) if self.async_offload_flag else None
        for i, blk in enumerate(self.transformer_blocks):
            if offload is not None:
                offload.before_layer(i)
            text, image = blk(image, text, silu_temb, img_rope, txt_rope)
            if offload is not None:
                offload.after_layer(i)
        return image

    @torch.no_grad()
    def forward(self, latents, timestep, prompt_emb, prompt_emb_mask=None, edit_latents=None, cond_flag: bool = True):
        """latents [B, 16, H, W]; timestep [B] in [0, 1000]; prompt_emb [B, L, text_dim] -> [B, 16, H, W]."""
        B, C, H, W = latents.shape
        L = prompt_emb.shape[1] if prompt_emb_mask is None else int(prompt_emb_mask[0].sum())
        prompt_emb = prompt_emb[:, :L]
        shapes = [(1, H // 2, W // 2)]
        dt = self.img_in.weight.dtype
        image = self._patchify(latents.to(dt))
        n_img = image.shape[1]
        if edit_latents is not None:
            edits = edit_latents if isinstance(edit_latents, (list, tuple)) else [edit_latents]
            shapes += [(1, e.shape[2] // 2, e.shape[3] // 2) for e in edits]
            image = torch.cat([image] + [self._patchify(e.to(dt)) for e in edits], dim=1)
        image = TF.linear(image, self.img_in.weight, self.img_in.bias)
        temb = self.time_text_embed(timestep.to(latents.device) / 1000.0)
        silu_temb = F.silu(temb)
        text = TF.rmsnorm_modulate(prompt_emb.to(dt), self.txt_norm.weight, None, None, 1e-6)
        text = TF.linear(text, self.txt_in.weight, self.txt_in.bias)
        img_rope, txt_rope = self.pos_embed(shapes, L, latents.device)
        if self.usp_flag:
            image, text, ic, isn, tc, ts = pshard.sequence_parallel_shard(
                [image, text, img_rope[0], img_rope[1], txt_rope[0], txt_rope[1]], [1, 1, 0, 0, 0, 0])  # fmt: skip
            img_rope, txt_rope = (ic, isn), (tc, ts)
        img_rope = tuple(t.contiguous() for t in img_rope)
        txt_rope = tuple(t.contiguous() for t in txt_rope)
        ori = image
        cache = self.feature_cache
        if cache.should_compute(cond_flag):
            image = self.forward_blocks(image, text, silu_temb, img_rope, txt_rope)
            cache.update(image, ori, cond_flag)
        else:
            image = cache.approximate(image, cond_flag)
        emb = F.linear(silu_temb, self.norm_out.linear.weight.float(), self.norm_out.linear.bias.float())
        scale, shift = emb.chunk(2, dim=-1)
        image = TF.layernorm_modulate(image, shift.unsqueeze(1), scale.unsqueeze(1), eps=1e-6)
        image = TF.linear(image, self.proj_out.weight, self.proj_out.bias)
        if self.usp_flag:
            total = sum(f * h * w for f, h, w in shapes)
            (image,) = pshard.sequence_parallel_unshard([image], [1], [total])
        image = image[:, :n_img]
        out = image.reshape(B, H // 2, W // 2, C, 2, 2).permute(0, 3, 1, 4, 2, 5)
        return out.reshape(B, C, H, W)

    @staticmethod
    def state_dict_converter():
        return QwenImageDitStateDictConverter()


class QwenImageDitStateDictConverter:
    def from_diffusers(self, sd: dict):
        return sd, {}

    def from_official(self, sd: dict):
        return sd, {}


def _register() -> None:
    from telefuser_b200.core.model_registry import register_architecture

    register_architecture("qwen_image_dit", QwenImageDiT, lambda: QwenImageDiT())


_register()
