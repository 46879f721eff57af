"""LongCat-Video DiT: single-stream blocks with per-frame modulation, cross-attention and SwiGLU MLP.

Every latent frame carries its own timestep, so the AdaLN tables are per frame ([B, T, C]) and clean conditioning
frames (timestep 0) can sit in front of the noisy ones: they attend only among themselves while the noisy
frames attend to everything, or their keys / values are computed once and kept as a per-block KV cache for
video continuation. Self-attention has a fused QKV projection, per-head RMSNorm and 3-axis interleaved RoPE
(axes split d - 4*(d//6), 2*(d//6), 2*(d//6)); the refinement stage can switch it to 3-D chunked top-k block
sparse attention. The cache holds rotated keys (positions of the conditioning frames never change).
Role parity: telefuser/models/longcat_video_dit.py:34-1214.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn

from telefuser_b200.core.base_model import BaseModel
from telefuser_b200.models.qwen_image_dit import _WeightOnly
from telefuser_b200.models.wan_dit import AffineLayerNorm, _fuse_linear_weights
from telefuser_b200.ops import functional as TF
from telefuser_b200.parallel import shard as pshard


def rope_tables_3d(head_dim: int, grid, base: float = 10000.0):
    """fp32 (cos, sin) [T*H*W, head_dim/2] for interleaved pairs."""
    T, H, W = grid
    d_h = d_w = 2 * (head_dim // 6)
    d_t = head_dim - 4 * (head_dim // 6)

    def ang(n, d):
        inv = 1.0 / (base ** (torch.arange(0, d, 2)[: d // 2].float() / d))
        return torch.arange(n, dtype=torch.float32)[:, None] * inv[None, :]

    a = torch.cat([ang(T, d_t)[:, None, None, :].expand(T, H, W, -1), ang(H, d_h)[None, :, None, :].expand(T, H, W, -1),
                   ang(W, d_w)[None, None, :, :].expand(T, H, W, -1)], dim=-1).reshape(T * H * W, -1)  # fmt: skip
    return a.cos().contiguous(), a.sin().contiguous()


def _rows(table: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """Per-frame table [B, T, C] for tokens x [B, N, C]: the fused kernels take it as is (N/T rows per table row),
    the fp32 fallbacks need one row per token."""
    if x.is_cuda and x.dtype == torch.bfloat16:
        return table
    return table.repeat_interleave(x.shape[1] // table.shape[1], dim=1)


class Attention(nn.Module):
    def __init__(self, dim: int, num_heads: int, enable_bsa: bool = False, bsa_params: dict | None = None) -> None:
        super().__init__()
        self.dim, self.num_heads, self.head_dim = dim, num_heads, dim // num_heads
        self.enable_bsa, self.bsa_params = enable_bsa, bsa_params or {}
        self.qkv = nn.Linear(dim, dim * 3)
        self.q_norm, self.k_norm = _WeightOnly(self.head_dim), _WeightOnly(self.head_dim)
        self.proj = nn.Linear(dim, dim)

    def forward(self, x, rope, shape=None, num_cond_latents: int = 0, return_kv: bool = False, kv_cache=None, usp: bool = False):
        """x [B, N, C]; rope = (cos, sin) rows for exactly these N tokens -> attention output before `proj`."""
        B, N, C = x.shape
        H, D = self.num_heads, self.head_dim
        qkv = TF.linear(x, self.qkv.weight, self.qkv.bias)
        q, k, v = (qkv[..., i * C : (i + 1) * C].unflatten(-1, (H, D)) for i in range(3))
        cos, sin = rope if B == 1 else tuple(t.repeat(B, 1) for t in rope)
        TF.headnorm_rope_(q, self.q_norm.weight, cos, sin, 1e-6, k=k, weight_k=self.k_norm.weight)
        group = None
        if usp:
            from telefuser_b200.parallel import ulysses

            group = pshard._sp(None)[3]
            q, k, v = (ulysses.scatter_heads(t.contiguous(), group) for t in (q, k, v))
        new_cache = (k.clone(), v.clone()) if return_kv else None
        if kv_cache is not None:
            ck, cv = (c.to(k.device) for c in kv_cache)
            if ck.shape[0] == 1 and B > 1:
                ck, cv = ck.expand(B, -1, -1, -1), cv.expand(B, -1, -1, -1)
            o = TF.attention(q, torch.cat([ck, k], dim=1), torch.cat([cv, v], dim=1))
        elif num_cond_latents and num_cond_latents > 0:
            n_cond = num_cond_latents * (q.shape[1] // shape[0])
            o = torch.cat([TF.attention(q[:, :n_cond], k[:, :n_cond], v[:, :n_cond]), TF.attention(q[:, n_cond:], k, v)], dim=1)
        elif self.enable_bsa and shape is not None and not usp:
            from telefuser_b200.ops.sparse_attention import bsa_3d_attention

            o = bsa_3d_attention(q.contiguous(), k.contiguous(), v.contiguous(), shape, shape, **self.bsa_params)
        else:
            o = TF.attention(q, k, v)
        if usp:
            o = ulysses.gather_heads(o, group)
        return o.reshape(B, -1, C), new_cache


class MultiHeadCrossAttention(nn.Module):
    def __init__(self, dim: int, num_heads: int) -> None:
        super().__init__()
        self.dim, self.num_heads, self.head_dim = dim, num_heads, dim // num_heads
        self.q_linear = nn.Linear(dim, dim)
        self.kv_linear = nn.Linear(dim, dim * 2)
        self.proj = nn.Linear(dim, dim)
        self.q_norm, self.k_norm = _WeightOnly(self.head_dim), _WeightOnly(self.head_dim)

    def forward(self, x, cond, kv_seqlen: list[int]):
        """x [B, N, C]; cond [1, sum(kv_seqlen), C] (valid text tokens of all samples in a row)."""
        B, N, C = x.shape
        H, D = self.num_heads, self.head_dim
        q = TF.linear(x, self.q_linear.weight, self.q_linear.bias).unflatten(-1, (H, D))
        kv = TF.linear(cond, self.kv_linear.weight, self.kv_linear.bias)
        k, v = kv[..., :C].unflatten(-1, (H, D)), kv[..., C:].unflatten(-1, (H, D))
        TF.headnorm_rope_(q, self.q_norm.weight, None, None, 1e-6)
        TF.headnorm_rope_(k, self.k_norm.weight, None, None, 1e-6)
        outs, off = [], 0
        for b in range(B):  # every sample sees only its own text tokens
            n = int(kv_seqlen[b])
            outs.append(TF.attention(q[b : b + 1], k[:, off : off + n], v[:, off : off + n]))
            off += n
        return torch.cat(outs).reshape(B, N, C)


class FeedForwardSwiGLU(nn.Module):
    def __init__(self, dim: int, hidden_dim: int, multiple_of: int = 256) -> None:
        super().__init__()
        hidden_dim = multiple_of * ((int(2 * hidden_dim / 3) + multiple_of - 1) // multiple_of)
        self.w1 = nn.Linear(dim, hidden_dim, bias=False)
        self.w2 = nn.Linear(hidden_dim, dim, bias=False)
        self.w3 = nn.Linear(dim, hidden_dim, bias=False)
        self._w13 = None

    def forward(self, x, residual=None, gate=None):
        w = self.w1.weight
        if self._w13 is None or self._w13[0].data_ptr() != w.data_ptr() or self._w13[0].dtype != w.dtype:
            self._w13 = _fuse_linear_weights([self.w1, self.w3])
        return TF.linear(TF.silu_and_mul(TF.linear(x, self._w13[0])), self.w2.weight, residual=residual, gate=gate)


class TimestepEmbedder(nn.Module):
    def __init__(self, t_embed_dim: int, frequency_embedding_size: int = 256) -> None:
        super().__init__()
        self.frequency_embedding_size = frequency_embedding_size
        self.mlp = nn.Sequential(nn.Linear(frequency_embedding_size, t_embed_dim), nn.SiLU(), nn.Linear(t_embed_dim, t_embed_dim))

    def forward(self, t):
        half = self.frequency_embedding_size // 2
        freqs = torch.exp(-math.log(10000) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
        args = t[:, None].float() * freqs[None]
        emb = torch.cat([args.cos(), args.sin()], dim=-1)
        h = F.silu(F.linear(emb, self.mlp[0].weight.float(), self.mlp[0].bias.float()))
        return F.linear(h, self.mlp[2].weight.float(), self.mlp[2].bias.float())


class CaptionEmbedder(nn.Module):
    def __init__(self, in_channels: int, hidden_size: int) -> None:
        super().__init__()
        self.y_proj = nn.Sequential(nn.Linear(in_channels, hidden_size), nn.GELU(approximate="tanh"),
                                    nn.Linear(hidden_size, hidden_size))  # fmt: skip

    def forward(self, caption):
        p = self.y_proj
        return TF.linear(TF.linear(caption, p[0].weight, p[0].bias, act="gelu_tanh"), p[2].weight, p[2].bias)


class PatchEmbed3D(nn.Module):
    def __init__(self, patch_size=(1, 2, 2), in_chans: int = 16, embed_dim: int = 96) -> None:
        super().__init__()
        self.patch_size = tuple(patch_size)
        self.proj = nn.Conv3d(in_chans, embed_dim, kernel_size=self.patch_size, stride=self.patch_size)

    def forward(self, x):
        p = self.patch_size
        pads = [(-x.shape[4]) % p[2], (-x.shape[3]) % p[1], (-x.shape[2]) % p[0]]
        if any(pads):
            x = F.pad(x, (0, pads[0], 0, pads[1], 0, pads[2]))
        return self.proj(x).flatten(2).transpose(1, 2)


class FinalLayer_FP32(nn.Module):
    def __init__(self, hidden_size: int, num_patch: int, out_channels: int, adaln_tembed_dim: int) -> None:
        super().__init__()
        self.linear = nn.Linear(hidden_size, num_patch * out_channels)
        self.adaLN_modulation = nn.Sequential(nn.SiLU(), nn.Linear(adaln_tembed_dim, 2 * hidden_size))

    def forward(self, x, t):
        lin = self.adaLN_modulation[1]
        shift, scale = F.linear(F.silu(t), lin.weight.float(), lin.bias.float()).chunk(2, dim=-1)  # [B, T, C]
        h = TF.layernorm_modulate(x, _rows(shift, x), _rows(scale, x), eps=1e-6)
        return TF.linear(h, self.linear.weight, self.linear.bias)


class LongCatSingleStreamBlock(nn.Module):
    def __init__(self, hidden_size: int, num_heads: int, mlp_ratio: int, adaln_tembed_dim: int, enable_bsa: bool = False,
                 bsa_params: dict | None = None) -> None:  # fmt: skip
        super().__init__()
        self.adaLN_modulation = nn.Sequential(nn.SiLU(), nn.Linear(adaln_tembed_dim, 6 * hidden_size))
        self.pre_crs_attn_norm = AffineLayerNorm(hidden_size, 1e-6, elementwise_affine=True)
        self.attn = Attention(hidden_size, num_heads, enable_bsa, bsa_params)
        self.cross_attn = MultiHeadCrossAttention(hidden_size, num_heads)
        self.ffn = FeedForwardSwiGLU(hidden_size, int(hidden_size * mlp_ratio))

    def forward(self, x, y, t, y_seqlen, latent_shape, rope, num_cond_latents: int = 0, return_kv: bool = False, kv_cache=None,
                skip_crs_attn: bool = False, usp: bool = False):  # fmt: skip
        lin = self.adaLN_modulation[1]
        mods = F.linear(F.silu(t), lin.weight.float(), lin.bias.float()).chunk(6, dim=-1)  # fp32 [B, T, C] each
        shift_msa, scale_msa, gate_msa, shift_mlp, scale_mlp, gate_mlp = (_rows(m, x) for m in mods)
        a, cache = self.attn(TF.layernorm_modulate(x, shift_msa, scale_msa, eps=1e-6), rope, latent_shape, num_cond_latents,
                             return_kv, kv_cache, usp)  # fmt: skip
        x = TF.linear(a, self.attn.proj.weight, self.attn.proj.bias, residual=x, gate=gate_msa)
        if not skip_crs_attn:
            n0 = 0 if kv_cache is not None else num_cond_latents * (x.shape[1] // latent_shape[0]) if num_cond_latents else 0
            xn = x[:, n0:]
            c = self.cross_attn(self.pre_crs_attn_norm(xn), y, y_seqlen)
            c = TF.linear(c, self.cross_attn.proj.weight, self.cross_attn.proj.bias, residual=xn)
            x = c if n0 == 0 else torch.cat([x[:, :n0], c], dim=1)
        x = self.ffn(TF.layernorm_modulate(x, shift_mlp, scale_mlp, eps=1e-6), residual=x, gate=gate_mlp)
        return x, cache


class LongCatVideoTransformer3DModel(BaseModel):
    def __init__(self, in_channels: int = 16, out_channels: int = 16, hidden_size: int = 4096, depth: int = 48,
                 num_heads: int = 32, caption_channels: int = 4096, mlp_ratio: int = 4, adaln_tembed_dim: int = 512,
                 frequency_embedding_size: int = 256, patch_size=(1, 2, 2), enable_bsa: bool = False,
                 bsa_params: dict | None = None, cp_split_hw=None, text_tokens_zero_pad: bool = True) -> None:  # fmt: skip
        super().__init__()
        bsa_params = bsa_params or {"sparsity": 0.9375, "chunk_3d_shape_q": [4, 4, 4], "chunk_3d_shape_k": [4, 4, 4]}
        self.patch_size, self.in_channels, self.out_channels = tuple(patch_size), in_channels, out_channels
        if self.patch_size[0] != 1:
            raise ValueError("the patch embedding must not compress time")
        self.head_dim = hidden_size // num_heads
        self.x_embedder = PatchEmbed3D(self.patch_size, in_channels, hidden_size)
        self.t_embedder = TimestepEmbedder(adaln_tembed_dim, frequency_embedding_size)
        self.y_embedder = CaptionEmbedder(caption_channels, hidden_size)
        self.blocks = nn.ModuleList([LongCatSingleStreamBlock(hidden_size, num_heads, mlp_ratio, adaln_tembed_dim, enable_bsa,
                                                              bsa_params) for _ in range(depth)])  # fmt: skip
        self.final_layer = FinalLayer_FP32(hidden_size, math.prod(self.patch_size), out_channels, adaln_tembed_dim)
        self.text_tokens_zero_pad = text_tokens_zero_pad
        self.caption_channels = caption_channels
        self.layer_name_list = ["blocks"]
        self.kv_cache_dict: dict = {}
        self.dtype = torch.bfloat16

    # ---- switches -------------------------------------------------------------------
    def enable_bsa(self) -> None:
        for b in self.blocks:
            b.attn.enable_bsa = True

    def disable_bsa(self) -> None:
        for b in self.blocks:
            b.attn.enable_bsa = False

    def get_fsdp_module_names(self) -> list[str]:
        return ["blocks"]

    # LoRAs are registered by key and merged into the weights while enabled; disabling subtracts the same delta.
    def load_lora(self, lora, lora_key: str, strength: float = 1.0) -> None:
        if not hasattr(self, "lora_dict"):
            self.lora_dict, self.active_loras = {}, []
        if isinstance(lora, (str, bytes)) or hasattr(lora, "__fspath__"):
            from telefuser_b200.utils.model_weight import load_state_dict

            lora = load_state_dict(str(lora))
        self.lora_dict[lora_key] = (lora, strength)

    def _merge(self, key: str, sign: float) -> None:
        from telefuser_b200.utils.lora import LoRALoader

        lora, strength = self.lora_dict[key]
        LoRALoader().apply_lora(self, lora, strength=sign * strength)
        for b in self.blocks:
            b.ffn._w13 = None  # fused views are rebuilt from the updated weights

    def enable_loras(self, lora_key_list: list[str] | None = None) -> None:
        self.disable_all_loras()
        for key in lora_key_list or []:
            if key in getattr(self, "lora_dict", {}):
                self._merge(key, 1.0)
                self.active_loras.append(key)

    def disable_all_loras(self) -> None:
        for key in getattr(self, "active_loras", []):
            self._merge(key, -1.0)
        self.active_loras = []

    def clear_cache(self) -> None:
        self.kv_cache_dict = {}

    @torch.no_grad()
    def cache_clean_latents(self, cond_latents: torch.Tensor, offload_kv_cache: bool = False, model_max_length: int = 512):
        """Runs the clean conditioning frames alone (timestep 0, no text) and keeps every block's keys / values."""
        B, _, T = cond_latents.shape[:3]
        dt = self.x_embedder.proj.weight.dtype
        empty = torch.zeros(B, 1, model_max_length, self.caption_channels, device=cond_latents.device, dtype=dt)
        _, cache = self.forward(cond_latents.to(dt), torch.zeros(B, T, device=cond_latents.device), empty, return_kv=True,
                                skip_crs_attn=True, offload_kv_cache=offload_kv_cache)  # fmt: skip
        self.kv_cache_dict = cache

    # ---- forward --------------------------------------------------------------------
    def forward_blocks(self, x, y, t, y_seqlens, latent_shape, rope, num_cond_latents=0, return_kv=False, skip_crs_attn=False,
                       offload_kv_cache=False):  # fmt: skip
        N = x.shape[1]
        usp = self.usp_flag
        if usp:
            P = pshard._sp(None)[1]
            if N % P or num_cond_latents:
                raise ValueError("sequence parallel LongCat needs a token count divisible by the group size and takes "
                                 "conditioning frames through the KV cache only")
            x, rc, rs = pshard.sequence_parallel_shard([x, rope[0], rope[1]], [1, 0, 0])
            # per-token modulation rows for this shard (a shard may cut through frames)
            t = t.repeat_interleave(N // latent_shape[0], dim=1)
            (t,) = pshard.sequence_parallel_shard([t], [1])
            rope, latent_shape = (rc.contiguous(), rs.contiguous()), (x.shape[1], 1, 1)
        offload = getattr(self, "async_offload_manager", None) if self.async_offload_flag else None
        caches = {}
        for i, blk in enumerate(self.blocks):
            if offload is not None:
                offload.before_layer(i)
            x, cache = blk(x, y, t, y_seqlens, latent_shape, rope, num_cond_latents, return_kv, self.kv_cache_dict.get(i),
                           skip_crs_attn, usp)  # fmt: skip
            if offload is not None:
                offload.after_layer(i)
            if return_kv:
                caches[i] = tuple(c.cpu() for c in cache) if offload_kv_cache else tuple(c.contiguous() for c in cache)
        if usp:
            (x,) = pshard.sequence_parallel_unshard([x], [1], [N])
        return (x, caches) if return_kv else x

    @torch.no_grad()
    def forward(self, hidden_states, timestep, encoder_hidden_states, encoder_attention_mask=None, num_cond_latents: int = 0,
                return_kv: bool = False, skip_crs_attn: bool = False, offload_kv_cache: bool = False, **_unused):  # fmt: skip
        """hidden_states [B, C, T, H, W]; timestep [B] or [B, T]; encoder_hidden_states [B, 1, L, caption_channels];
        encoder_attention_mask [B, 1, 1, L] or [B, L] -> fp32 [B, C_out, T, H, W] (and the KV caches when asked)."""
        B, _, T, H, W = hidden_states.shape
        p = self.patch_size
        grid = (T // p[0], -(-H // p[1]), -(-W // p[2]))
        dev = hidden_states.device
        per_frame = grid[1] * grid[2]
        cos, sin = rope_tables_3d(self.head_dim, (grid[0] + (num_cond_latents if self.kv_cache_dict else 0), grid[1], grid[2]))
        skip = num_cond_latents * per_frame if self.kv_cache_dict else 0
        rope = (cos[skip:].to(dev).contiguous(), sin[skip:].to(dev).contiguous())
        if timestep.dim() == 1:
            timestep = timestep.unsqueeze(1).expand(-1, grid[0])
        dt = self.x_embedder.proj.weight.dtype
        x = self.x_embedder(hidden_states.to(dt))
        t = self.t_embedder(timestep.to(dev).float().flatten()).reshape(B, grid[0], -1)  # fp32 [B, T, C_t]
        y = self.y_embedder(encoder_hidden_states.to(dt))  # [B, 1, L, C]
        if encoder_attention_mask is not None:
            mask = encoder_attention_mask.reshape(B, -1).to(dev)
            if self.text_tokens_zero_pad:
                y = y * mask[:, None, :, None].to(y.dtype)
                mask = torch.ones_like(mask)
            y_seqlens = mask.sum(dim=1).tolist()
            y = y.squeeze(1)[mask != 0].view(1, -1, x.shape[-1])
        else:
            y_seqlens = [y.shape[2]] * B
            y = y.squeeze(1).reshape(1, -1, x.shape[-1])
        out = self.forward_blocks(x, y, t, y_seqlens, grid, rope, num_cond_latents, return_kv, skip_crs_attn, offload_kv_cache)
        x, caches = out if return_kv else (out, None)
        x = self.final_layer(x, t)
        x = x.view(B, grid[0], grid[1], grid[2], p[0], p[1], p[2], self.out_channels).permute(0, 7, 1, 4, 2, 5, 3, 6)
        x = x.reshape(B, self.out_channels, grid[0] * p[0], grid[1] * p[1], grid[2] * p[2]).float()
        return (x, caches) if return_kv else x

    @staticmethod
    def state_dict_converter():
        return LongCatVideoTransformer3DModelDictConverter()


class LongCatVideoTransformer3DModelDictConverter:
    def from_diffusers(self, sd: dict):
        return sd, {}

    def from_official(self, sd: dict):
        return sd, {}


def _register() -> None:
    from telefuser_b200.core.model_registry import register_architecture

    register_architecture("longcat_video_dit", LongCatVideoTransformer3DModel,
                          lambda: LongCatVideoTransformer3DModel(depth=1), resource="diffusers", keys_only=True)  # fmt: skip


_register()
