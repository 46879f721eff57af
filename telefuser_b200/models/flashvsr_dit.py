"""FlashVSR: one-step streaming video super-resolution DiT (Wan 1.3B backbone).

Differences to the Wan DiT: self-attention is windowed top-k block-sparse with a per-layer cache of the last
temporal window groups (`ops.local_sparse_attention`), so the model runs clip by clip (6 latent frames first, 2
afterwards) with rotary frame positions that keep counting; cross-attention keys / values come from one learned
context and are computed once; the timestep is fixed (1000) so the modulation tables are constants; the
low-quality video enters as per-layer additive conditioning from `Causal_LQ4x_Proj`. Under sequence parallelism
the heads are scattered (Ulysses) around the sparse attention, whose cache then holds this rank's heads.
Role parity: telefuser/models/flashvsr_dit.py:33-608.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn

from telefuser_b200.core.base_model import BaseModel
from telefuser_b200.models.video_projector import Causal_LQ4x_Proj
from telefuser_b200.models.wan_dit import (AffineLayerNorm, WanHead, WanSelfAttention, _fuse_linear_weights, RMSNormWeight,
                                           rope_angles_1d, sinusoidal_embedding_1d)  # fmt: skip
from telefuser_b200.ops import functional as TF
from telefuser_b200.ops.local_sparse_attention import local_sparse_attention
from telefuser_b200.parallel import shard as pshard


class SparseSelfAttention(WanSelfAttention):
    usp = False

    def forward(self, x, cos, sin, grid, topk: int, kv_len: int, cache, local_range: int = 9, win=(2, 8, 8)):
        """-> (attention output before the out projection, new (cache_k, cache_v))."""
        B, S, C = x.shape
        H = self.num_heads
        f, h, w = grid
        W, b = self.fused_qkv()
        qkv = TF.linear(x, W, b)
        q, k, v = qkv[..., :C], qkv[..., C : 2 * C], qkv[..., 2 * C :]
        TF.rmsnorm_rope_(q, self.norm_q.weight, H, cos, sin, self.norm_q.eps, x2=k, weight2=self.norm_k.weight)
        heads, width = H, C
        if self.usp:
            from telefuser_b200.parallel import ulysses

            group = pshard._sp(None)[3]
            q, k, v = (ulysses.scatter_heads(t.unflatten(-1, (H, -1)).contiguous(), group).flatten(-2) for t in (q, k, v))
            heads, width = q.shape[-1] // self.head_dim, q.shape[-1]
        pk, pv = cache if cache is not None else (None, None)
        o, ck, cv = local_sparse_attention(q.contiguous(), k.contiguous(), v.contiguous(), B, f, h, w, width, topk, local_range,
                                           heads, kv_len, pk, pv, win)  # fmt: skip
        if self.usp:
            o = ulysses.gather_heads(o.unflatten(-1, (heads, -1)), group).flatten(-2)
        return o, (ck, cv)


class CachedCrossAttention(nn.Module):
    def __init__(self, dim: int, num_heads: int, eps: float = 1e-6) -> None:
        super().__init__()
        self.num_heads, self.head_dim = num_heads, dim // num_heads
        self.q, self.k, self.v, self.o = (nn.Linear(dim, dim) for _ in range(4))
        self.norm_q, self.norm_k = RMSNormWeight(dim, eps), RMSNormWeight(dim, eps)
        self.cache_k = self.cache_v = None

    @torch.no_grad()
    def init_cache(self, ctx):
        k = TF.linear(ctx, self.k.weight, self.k.bias)
        TF.rmsnorm_rope_(k, self.norm_k.weight, self.num_heads, eps=self.norm_k.eps)
        self.cache_k, self.cache_v = k, TF.linear(ctx, self.v.weight, self.v.bias)

    def clear_cache(self) -> None:
        self.cache_k = self.cache_v = None

    def forward(self, x):
        H, D = self.num_heads, self.head_dim
        q = TF.linear(x, self.q.weight, self.q.bias)
        TF.rmsnorm_rope_(q, self.norm_q.weight, H, eps=self.norm_q.eps)
        k, v = self.cache_k.to(q.device), self.cache_v.to(q.device)
        if k.shape[0] != q.shape[0]:
            k, v = k.expand(q.shape[0], -1, -1), v.expand(q.shape[0], -1, -1)
        o = TF.attention(q.unflatten(-1, (H, D)), k.unflatten(-1, (H, D)), v.unflatten(-1, (H, D)))
        return o.flatten(-2)


class DiTBlock(nn.Module):
    def __init__(self, dim: int, num_heads: int, ffn_dim: int, eps: float = 1e-6) -> None:
        super().__init__()
        self.self_attn = SparseSelfAttention(dim, num_heads, eps)
        self.cross_attn = CachedCrossAttention(dim, num_heads, eps)
        self.norm1 = AffineLayerNorm(dim, eps, elementwise_affine=False)
        self.norm2 = AffineLayerNorm(dim, eps, elementwise_affine=False)
        self.norm3 = AffineLayerNorm(dim, eps)
        self.ffn = nn.Sequential(nn.Linear(dim, ffn_dim), nn.GELU(approximate="tanh"), nn.Linear(ffn_dim, dim))
        self.modulation = nn.Parameter(torch.randn(1, 6, dim) / dim**0.5)

    def forward(self, x, t_mod, cos, sin, grid, topk, kv_len, cache, local_range, win):
        """t_mod: fp32 [B, 6, C]."""
        mod = self.modulation.float() + t_mod
        shift_msa, scale_msa, gate_msa, shift_mlp, scale_mlp, gate_mlp = (mod[:, i : i + 1] for i in range(6))
        a, cache = self.self_attn(self.norm1(x, shift_msa, scale_msa), cos, sin, grid, topk, kv_len, cache, local_range, win)
        x = TF.linear(a, self.self_attn.o.weight, self.self_attn.o.bias, residual=x, gate=gate_msa)
        c = self.cross_attn(self.norm3(x))
        x = TF.linear(c, self.cross_attn.o.weight, self.cross_attn.o.bias, residual=x)
        h = TF.linear(self.norm2(x, shift_mlp, scale_mlp), self.ffn[0].weight, self.ffn[0].bias, act="gelu_tanh")
        return TF.linear(h, self.ffn[2].weight, self.ffn[2].bias, residual=x, gate=gate_mlp), cache


class FlashVSRModel(BaseModel):
    def __init__(self, dim=1536, in_dim=16, ffn_dim=8960, out_dim=16, text_dim=4096, freq_dim=256, eps=1e-6,
                 patch_size=(1, 2, 2), num_heads=12, num_layers=30, lq_layers: int = 1, ctx_len: int = 512) -> None:  # fmt: skip
        super().__init__()
        self.dim, self.num_layers, self.freq_dim, self.patch_size = dim, num_layers, freq_dim, tuple(patch_size)
        self.num_heads, self.head_dim = num_heads, dim // num_heads
        self.patch_embedding = nn.Conv3d(in_dim, dim, kernel_size=self.patch_size, stride=self.patch_size)
        self.text_embedding = nn.Sequential(nn.Linear(text_dim, dim), nn.GELU(approximate="tanh"), nn.Linear(dim, dim))
        self.time_embedding = nn.Sequential(nn.Linear(freq_dim, dim), nn.SiLU(), nn.Linear(dim, dim))
        self.time_projection = nn.Sequential(nn.SiLU(), nn.Linear(dim, dim * 6))
        self.blocks = nn.ModuleList([DiTBlock(dim, num_heads, ffn_dim, eps) for _ in range(num_layers)])
        self.head = WanHead(dim, out_dim, self.patch_size, eps)
        self.LQ_proj_in = Causal_LQ4x_Proj(in_dim=3, out_dim=dim, layer_num=lq_layers)
        self.ctx = nn.Parameter(torch.zeros(1, ctx_len, text_dim, dtype=torch.bfloat16))
        self.layer_name_list = ["blocks"]
        self.dtype = torch.bfloat16
        self._cross_kv_initialized = False
        self.kv_cache: list = [None] * num_layers

    # ---- caches ---------------------------------------------------------------------
    def clear_cross_kv(self) -> None:
        for blk in self.blocks:
            blk.cross_attn.clear_cache()
        self._cross_kv_initialized = False

    def clear_kv_cache(self) -> None:
        self.kv_cache = [None] * self.num_layers

    def clean_LQ_proj_in_cache(self) -> None:
        self.LQ_proj_in.clear_cache()

    @torch.no_grad()
    def init_ctx_and_time_embedding(self) -> None:
        dt = self.patch_embedding.weight.dtype
        ctx = self.ctx.to(dt)
        te = self.text_embedding
        ctx = TF.linear(TF.linear(ctx, te[0].weight, te[0].bias, act="gelu_tanh"), te[2].weight, te[2].bias)
        for blk in self.blocks:
            blk.cross_attn.init_cache(ctx)
        emb = sinusoidal_embedding_1d(self.freq_dim, torch.tensor([1000.0], device=self.ctx.device))
        lin1, lin2, proj = self.time_embedding[0], self.time_embedding[2], self.time_projection[1]
        t = torch.nn.functional.linear(torch.nn.functional.silu(torch.nn.functional.linear(emb, lin1.weight.float(), lin1.bias.float())),
                                       lin2.weight.float(), lin2.bias.float())  # fmt: skip
        self.t = t  # fp32 [1, C]
        self.t_mod = torch.nn.functional.linear(torch.nn.functional.silu(t), proj.weight.float(), proj.bias.float()).unflatten(1, (6, self.dim))
        self._cross_kv_initialized = True

    def proj_LQ_video_clip(self, video_clip, tile: bool = False, tile_size=(512, 512), tile_stride=(256, 256)):
        if tile:
            return self.LQ_proj_in.tile_stream_forward(video_clip, tile_size, tile_stride)
        return self.LQ_proj_in.stream_forward(video_clip)

    def enable_usp(self) -> None:
        super().enable_usp()
        for blk in self.blocks:
            blk.self_attn.usp = True

    def rope(self, grid, frame_start: int, device):
        f, h, w = grid
        d_hw = self.head_dim // 3
        a_f = rope_angles_1d(self.head_dim - 2 * d_hw)[frame_start : frame_start + f]
        a_h, a_w = rope_angles_1d(d_hw)[:h], rope_angles_1d(d_hw)[:w]
        ang = torch.cat([a_f.view(f, 1, 1, -1).expand(f, h, w, -1), a_h.view(1, h, 1, -1).expand(f, h, w, -1),
                         a_w.view(1, 1, w, -1).expand(f, h, w, -1)], dim=-1).reshape(f * h * w, -1)  # fmt: skip
        return ang.cos().float().to(device).contiguous(), ang.sin().float().to(device).contiguous()

    @torch.no_grad()
    def forward(self, x, LQ_latents=None, is_stream: bool = False, topk_ratio: float = 2.0, kv_ratio: float = 3.0,
                cur_process_idx: int = 0, local_range: int = 9, win_size=(2, 8, 8), offload_kvcache: bool = False):  # fmt: skip
        """x: [B, 16, f, H, W] noisy latents of one clip -> [B, 16, f, H, W]."""
        if not self._cross_kv_initialized:
            self.init_ctx_and_time_embedding()
        dt = self.patch_embedding.weight.dtype
        x = self.patch_embedding(x.to(dt))
        f, h, w = x.shape[2:]
        x = x.flatten(2).transpose(1, 2).contiguous()
        windows = h * w // math.prod(win_size[1:])
        topk = int(windows * windows * topk_ratio) - 1
        kv_len = int(kv_ratio)
        cos, sin = self.rope((f, h, w), 0 if cur_process_idx == 0 else 4 + cur_process_idx * 2, x.device)
        for i, blk in enumerate(self.blocks):
            if LQ_latents is not None and i < len(LQ_latents):
                x = x + LQ_latents[i].to(x)
            cache = self.kv_cache[i]
            if cache is not None and offload_kvcache:
                cache = tuple(c.to(x.device, non_blocking=True) for c in cache)
            x, new = blk(x, self.t_mod.to(x.device), cos, sin, (f, h, w), topk, kv_len, cache, local_range, win_size)
            self.kv_cache[i] = tuple(c.cpu() for c in new) if offload_kvcache else new
        x = self.head(x, self.t.to(x.device).unsqueeze(1))
        p = self.patch_size
        x = x.view(x.shape[0], f, h, w, p[0], p[1], p[2], -1).permute(0, 7, 1, 4, 2, 5, 3, 6)
        return x.reshape(x.shape[0], -1, f * p[0], h * p[1], w * p[2])

    @staticmethod
    def state_dict_converter():
        return FlashVSRStateDictConverter()


class FlashVSRStateDictConverter:
    def from_official(self, sd: dict):
        from telefuser_b200.utils.model_weight import hash_state_dict_keys

        if hash_state_dict_keys(sd) == "0f889085aa6209c79f284d963d6cbe95":
            return sd, dict(patch_size=[1, 2, 2], in_dim=16, dim=1536, ffn_dim=8960, freq_dim=256, text_dim=4096, out_dim=16,
                            num_heads=12, num_layers=30, eps=1e-6)  # fmt: skip
        return sd, {}


__all__ = ["FlashVSRModel", "DiTBlock", "SparseSelfAttention", "CachedCrossAttention", "_fuse_linear_weights"]
