"""FLUX.2 transformer (klein and dev sizes): double-stream blocks followed by single-stream blocks.

All linears are bias free. One timestep(+guidance) embedding drives three shared modulation tables
(image double-stream, text double-stream, single-stream) that every block of a kind reuses.
Double block: per-stream LayerNorm+modulate, per-stream fused QKV GEMM written into one joint
[text; image] buffer, per-head RMSNorm + 4-axis interleaved RoPE in place, one joint attention,
per-stream out projection and SwiGLU MLP with gate and residual in the GEMM epilogue.
Single block: one GEMM produces Q, K, V and the SwiGLU input; Q / K / V are consumed as strided views;
the output projection runs as two K-slices of one weight (attention part, MLP part) so that the
[attention, mlp] concatenation is never materialised.
Parameter names follow the public (diffusers layout) checkpoint.
Role parity: telefuser/models/flux2_dit.py:30-1126.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from telefuser_b200.core.base_model import BaseModel
from telefuser_b200.models.qwen_image_dit import _WeightOnly, timestep_embedding
from telefuser_b200.ops import functional as TF
from telefuser_b200.parallel import shard as pshard


@dataclass
class Flux2DiTConfig:
    patch_size: int = 1
    in_channels: int = 128
    out_channels: int | None = None
    num_layers: int = 8
    num_single_layers: int = 24
    attention_head_dim: int = 128
    num_attention_heads: int = 32
    joint_attention_dim: int = 12288
    timestep_guidance_channels: int = 256
    mlp_ratio: float = 3.0
    axes_dims_rope: tuple = (32, 32, 32, 32)
    rope_theta: float = 2000.0
    eps: float = 1e-6
    guidance_embeds: bool = False

    @classmethod
    def klein_4b(cls) -> "Flux2DiTConfig":
        return cls(num_layers=5, num_single_layers=20, num_attention_heads=24, joint_attention_dim=7680)

    @classmethod
    def klein_9b(cls) -> "Flux2DiTConfig":
        return cls()

    @classmethod
    def dev(cls) -> "Flux2DiTConfig":
        return cls(num_single_layers=48, num_attention_heads=48, joint_attention_dim=15360, guidance_embeds=True)


def rope_tables(ids: torch.Tensor, axes_dim, theta: float) -> tuple[torch.Tensor, torch.Tensor]:
    """ids [S, n_axes] -> fp32 (cos, sin) [S, sum(axes)/2]; one angle per interleaved (even, odd) pair."""
    ids = ids[0] if ids.ndim == 3 else ids
    pos = ids.to(torch.float64)
    out = []
    for i, d in enumerate(axes_dim):
        inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float64, device=ids.device) / d))
        out.append(torch.outer(pos[:, i].float().double(), inv))
    ang = torch.cat(out, dim=-1)
    return ang.cos().float().contiguous(), ang.sin().float().contiguous()


class _TimestepMLP(nn.Module):
    def __init__(self, in_dim: int, dim: int) -> None:
        super().__init__()
        self.linear_1 = nn.Linear(in_dim, dim, bias=False)
        self.linear_2 = nn.Linear(dim, dim, bias=False)

    def forward(self, proj):
        return F.linear(F.silu(F.linear(proj, self.linear_1.weight.float())), self.linear_2.weight.float())


class Flux2TimestepGuidanceEmbeddings(nn.Module):
    def __init__(self, in_channels: int, dim: int, guidance_embeds: bool) -> None:
        super().__init__()
        self.in_channels = in_channels
        self.timestep_embedder = _TimestepMLP(in_channels, dim)
        self.guidance_embedder = _TimestepMLP(in_channels, dim) if guidance_embeds else None

    def forward(self, timestep, guidance=None):
        """timestep / guidance already multiplied by 1000 -> fp32 [B, dim]."""
        emb = self.timestep_embedder(timestep_embedding(timestep, self.in_channels, scale=1.0))
        if guidance is not None and self.guidance_embedder is not None:
            emb = emb + self.guidance_embedder(timestep_embedding(guidance, self.in_channels, scale=1.0))
        return emb


class Flux2Modulation(nn.Module):
    def __init__(self, dim: int, mod_param_sets: int) -> None:
        super().__init__()
        self.mod_param_sets = mod_param_sets
        self.linear = nn.Linear(dim, dim * 3 * mod_param_sets, bias=False)

    def forward(self, silu_temb):
        """-> list of fp32 [B, 1, dim] chunks ordered (shift, scale, gate) per set."""
        m = F.linear(silu_temb, self.linear.weight.float())
        return [c.unsqueeze(1) for c in m.chunk(3 * self.mod_param_sets, dim=-1)]


class Flux2FeedForward(nn.Module):
    def __init__(self, dim: int, mult: float) -> None:
        super().__init__()
        inner = int(dim * mult)
        self.linear_in = nn.Linear(dim, inner * 2, bias=False)
        self.linear_out = nn.Linear(inner, dim, bias=False)

    def forward(self, x, residual=None, gate=None):
        h = TF.silu_and_mul(TF.linear(x, self.linear_in.weight))
        return TF.linear(h, self.linear_out.weight, residual=residual, gate=gate)


def _joint_attention(q, k, v, usp: bool):
    if usp:
        from telefuser_b200.parallel.ring import long_context_attention

        return long_context_attention(q, k, v)
    return TF.attention(q, k, v)


def _per_batch(rope, B: int):
    return rope if B == 1 else tuple(t.repeat(B, 1) for t in rope)


class Flux2Attention(nn.Module):
    """Joint attention of a double-stream block; returns the two streams before their out projections."""

    def __init__(self, dim: int, heads: int, head_dim: int, eps: float) -> None:
        super().__init__()
        self.heads, self.head_dim, self.eps = heads, head_dim, eps
        inner = heads * head_dim
        self.to_q, self.to_k, self.to_v = (nn.Linear(dim, inner, bias=False) for _ in range(3))
        self.norm_q, self.norm_k = _WeightOnly(head_dim), _WeightOnly(head_dim)
        self.add_q_proj, self.add_k_proj, self.add_v_proj = (nn.Linear(dim, inner, bias=False) for _ in range(3))
        self.norm_added_q, self.norm_added_k = _WeightOnly(head_dim), _WeightOnly(head_dim)
        self.to_add_out = nn.Linear(inner, dim, bias=False)
        self.to_out = nn.Sequential(nn.Linear(inner, dim, bias=False))
        self._img = self._txt = None
        self.usp = False

    def _fused(self, slot: str, linears):
        from telefuser_b200.models.wan_dit import _fuse_linear_weights

        cur = getattr(self, slot)
        w = linears[0].weight
        if cur is None or cur[0].data_ptr() != w.data_ptr() or cur[0].dtype != w.dtype:
            cur = _fuse_linear_weights(linears)
            setattr(self, slot, cur)
        return cur[0]

    def forward(self, image, text, img_rope, txt_rope):
        B, Si, _ = image.shape
        St = text.shape[1]
        H, D = self.heads, self.head_dim
        C = H * D
        Wi = self._fused("_img", [self.to_q, self.to_k, self.to_v])
        Wt = self._fused("_txt", [self.add_q_proj, self.add_k_proj, self.add_v_proj])
        if B == 1:
            joint = torch.empty(B, St + Si, 3 * C, device=image.device, dtype=image.dtype)
            TF.linear(text, Wt, out=joint[:, :St])
            TF.linear(image, Wi, out=joint[:, St:])
        else:
            joint = torch.cat([TF.linear(text, Wt), TF.linear(image, Wi)], dim=1)
        q, k, v = (joint[..., i * C : (i + 1) * C].unflatten(-1, (H, D)) for i in range(3))
        tr, ir = _per_batch(txt_rope, B), _per_batch(img_rope, B)
        TF.headnorm_rope_(q[:, :St], self.norm_added_q.weight, tr[0], tr[1], self.eps, k=k[:, :St],
                          weight_k=self.norm_added_k.weight)  # fmt: skip
        TF.headnorm_rope_(q[:, St:], self.norm_q.weight, ir[0], ir[1], self.eps, k=k[:, St:], weight_k=self.norm_k.weight)
        o = _joint_attention(q, k, v, self.usp).reshape(B, St + Si, C)
        return o[:, St:], o[:, :St]


class Flux2TransformerBlock(nn.Module):
    def __init__(self, dim: int, heads: int, head_dim: int, mlp_ratio: float, eps: float) -> None:
        super().__init__()
        self.eps = eps
        self.attn = Flux2Attention(dim, heads, head_dim, eps)
        self.ff = Flux2FeedForward(dim, mlp_ratio)
        self.ff_context = Flux2FeedForward(dim, mlp_ratio)

    def forward(self, image, text, mod_img, mod_txt, img_rope, txt_rope):
        si1, ci1, gi1, si2, ci2, gi2 = mod_img
        st1, ct1, gt1, st2, ct2, gt2 = mod_txt
        a = self.attn
        io, to = a(TF.layernorm_modulate(image, si1, ci1, eps=self.eps), TF.layernorm_modulate(text, st1, ct1, eps=self.eps),
                   img_rope, txt_rope)  # fmt: skip
        image = TF.linear(io, a.to_out[0].weight, residual=image, gate=gi1)
        image = self.ff(TF.layernorm_modulate(image, si2, ci2, eps=self.eps), residual=image, gate=gi2)
        text = TF.linear(to, a.to_add_out.weight, residual=text, gate=gt1)
        text = self.ff_context(TF.layernorm_modulate(text, st2, ct2, eps=self.eps), residual=text, gate=gt2)
        return text, image


class Flux2ParallelSelfAttention(nn.Module):
    """Attention and SwiGLU MLP of a single-stream block sharing one input and one output projection."""

    def __init__(self, dim: int, heads: int, head_dim: int, mlp_ratio: float, eps: float) -> None:
        super().__init__()
        self.heads, self.head_dim, self.eps = heads, head_dim, eps
        self.inner = heads * head_dim
        self.mlp_hidden = int(dim * mlp_ratio)
        self.to_qkv_mlp_proj = nn.Linear(dim, 3 * self.inner + 2 * self.mlp_hidden, bias=False)
        self.norm_q, self.norm_k = _WeightOnly(head_dim), _WeightOnly(head_dim)
        self.to_out = nn.Linear(self.inner + self.mlp_hidden, dim, bias=False)
        self.usp = False

    def forward(self, x, rope, residual, gate):
        B, S, _ = x.shape
        H, D, C = self.heads, self.head_dim, self.inner
        fused = TF.linear(x, self.to_qkv_mlp_proj.weight)
        q, k, v = (fused[..., i * C : (i + 1) * C].unflatten(-1, (H, D)) for i in range(3))
        r = _per_batch(rope, B)
        TF.headnorm_rope_(q, self.norm_q.weight, r[0], r[1], self.eps, k=k, weight_k=self.norm_k.weight)
        o = _joint_attention(q, k, v, self.usp).reshape(B, S, C)
        m = TF.silu_and_mul(fused[..., 3 * C :])
        W = self.to_out.weight
        if TF.is_quantized_weight(W):  # quantised weights carry scales per output row or per K block: no K-slicing
            return TF.linear(torch.cat([o, m], dim=-1), W, residual=residual, gate=gate)
        h = TF.linear(o, W[:, :C], residual=residual, gate=gate)
        return TF.linear(m, W[:, C:], residual=h, gate=gate)


class Flux2SingleTransformerBlock(nn.Module):
    def __init__(self, dim: int, heads: int, head_dim: int, mlp_ratio: float, eps: float) -> None:
        super().__init__()
        self.eps = eps
        self.attn = Flux2ParallelSelfAttention(dim, heads, head_dim, mlp_ratio, eps)

    def forward(self, x, mod, rope):
        shift, scale, gate = mod
        return self.attn(TF.layernorm_modulate(x, shift, scale, eps=self.eps), rope, x, gate)


class _AdaNormOut(nn.Module):
    def __init__(self, dim: int) -> None:
        super().__init__()
        self.linear = nn.Linear(dim, 2 * dim, bias=False)


class Flux2DiT(BaseModel):
    def __init__(self, config: Flux2DiTConfig | None = None) -> None:
        super().__init__()
        c = self.config = config or Flux2DiTConfig()
        if sum(c.axes_dims_rope) != c.attention_head_dim:
            raise ValueError("RoPE axes must add up to the head dimension")
        self.out_channels = c.out_channels or c.in_channels
        dim = self.inner_dim = c.num_attention_heads * c.attention_head_dim
        self.time_guidance_embed = Flux2TimestepGuidanceEmbeddings(c.timestep_guidance_channels, dim, c.guidance_embeds)
        self.double_stream_modulation_img = Flux2Modulation(dim, 2)
        self.double_stream_modulation_txt = Flux2Modulation(dim, 2)
        self.single_stream_modulation = Flux2Modulation(dim, 1)
        self.x_embedder = nn.Linear(c.in_channels, dim, bias=False)
        self.context_embedder = nn.Linear(c.joint_attention_dim, dim, bias=False)
        blk = (dim, c.num_attention_heads, c.attention_head_dim, c.mlp_ratio, c.eps)
        self.transformer_blocks = nn.ModuleList([Flux2TransformerBlock(*blk) for _ in range(c.num_layers)])
        self.single_transformer_blocks = nn.ModuleList([Flux2SingleTransformerBlock(*blk) for _ in range(c.num_single_layers)])
        self.norm_out = _AdaNormOut(dim)
        self.proj_out = nn.Linear(dim, c.patch_size * c.patch_size * self.out_channels, bias=False)
        self.layer_name_list = ["transformer_blocks", "single_transformer_blocks"]
        self.dtype = torch.bfloat16

    def enable_usp(self) -> None:
        super().enable_usp()
        for b in list(self.transformer_blocks) + list(self.single_transformer_blocks):
            b.attn.usp = True

    def get_fsdp_module_names(self) -> list[str]:
        return ["transformer_blocks", "single_transformer_blocks"]

    def enable_quant(self, quant=None) -> int:
        from telefuser_b200.ops.quant import quantize_model_

        return quantize_model_(self, quant, ("transformer_blocks.*", "single_transformer_blocks.*"))

    def _offload(self):
        return getattr(self, "async_offload_manager", None) if self.async_offload_flag else None

    def forward_double_blocks(self, image, text, mod_img, mod_txt, img_rope, txt_rope):
        offload = self._offload()
        for i, blk in enumerate(self.transformer_blocks):
            if offload is not None:
                offload.before_layer(i)
            text, image = blk(image, text, mod_img, mod_txt, img_rope, txt_rope)
            if offload is not None:
                offload.after_layer(i)
        return text, image

    def forward_single_blocks(self, x, mod, rope):
        offload = self._offload()
        base = len(self.transformer_blocks)
        for i, blk in enumerate(self.single_transformer_blocks):
            if offload is not None:
                offload.before_layer(base + i)
            x = blk(x, mod, rope)
            if offload is not None:
                offload.after_layer(base + i)
        return x

    def enable_async_offload(self, device, offload_config) -> None:
        from telefuser_b200.offload.async_offload import AsyncOffloadManager

        blocks = list(self.transformer_blocks) + list(self.single_transformer_blocks)
        self.async_offload_manager = AsyncOffloadManager(
            blocks, enabled=True, offload_ratio=offload_config.offload_ratio, prefetch_size=offload_config.prefetch_size,
            device=device, pin_cpu_memory=offload_config.pin_cpu_memory)  # fmt: skip
        self.async_offload_flag = True

    @torch.no_grad()
    def forward(self, hidden_states, encoder_hidden_states, timestep, img_ids, txt_ids, guidance=None, cond_flag: bool = True):
        """hidden_states [B, Si, in_channels] packed latent tokens; encoder_hidden_states [B, St, joint_attention_dim];
        timestep [B] in [0, 1]; img_ids [Si, 4], txt_ids [St, 4] (T, H, W, L coordinates) -> [B, Si, out_channels]."""
        c = self.config
        dt = self.x_embedder.weight.dtype
        dev = hidden_states.device
        temb = self.time_guidance_embed(timestep.to(dev).float() * 1000,
                                        None if guidance is None else guidance.to(dev).float() * 1000)  # fmt: skip
        silu_temb = F.silu(temb)
        mod_img = self.double_stream_modulation_img(silu_temb)
        mod_txt = self.double_stream_modulation_txt(silu_temb)
        mod_single = self.single_stream_modulation(silu_temb)
        image = TF.linear(hidden_states.to(dt), self.x_embedder.weight)
        text = TF.linear(encoder_hidden_states.to(dt), self.context_embedder.weight)
        img_rope = rope_tables(img_ids.to(dev), c.axes_dims_rope, c.rope_theta)
        txt_rope = rope_tables(txt_ids.to(dev), c.axes_dims_rope, c.rope_theta)
        n_img = image.shape[1]
        if self.usp_flag:
            P = pshard._sp(None)[1]
            if image.shape[1] % P or text.shape[1] % P:
                raise ValueError("sequence parallel FLUX.2 needs image and text lengths divisible by the group size")
            image, text, ic, isn, tc, ts = pshard.sequence_parallel_shard(
                [image, text, img_rope[0], img_rope[1], txt_rope[0], txt_rope[1]], [1, 1, 0, 0, 0, 0])  # fmt: skip
            img_rope, txt_rope = (ic.contiguous(), isn.contiguous()), (tc.contiguous(), ts.contiguous())
        ori = image
        cache = self.feature_cache
        if cache.should_compute(cond_flag):
            text, image = self.forward_double_blocks(image, text, mod_img, mod_txt, img_rope, txt_rope)
            St = text.shape[1]
            rope = tuple(torch.cat([t, i], dim=0) for t, i in zip(txt_rope, img_rope))
            image = self.forward_single_blocks(torch.cat([text, image], dim=1), mod_single, rope)[:, St:]
            cache.update(image, ori, cond_flag)
        else:
            image = cache.approximate(image, cond_flag)
        emb = F.linear(silu_temb, self.norm_out.linear.weight.float())
        scale, shift = emb.chunk(2, dim=-1)
        image = TF.layernorm_modulate(image, shift.unsqueeze(1), scale.unsqueeze(1), eps=c.eps)
        out = TF.linear(image, self.proj_out.weight)
        if self.usp_flag:
            (out,) = pshard.sequence_parallel_unshard([out], [1], [n_img])
        return out

    @staticmethod
    def state_dict_converter():
        return Flux2DiTStateDictConverter()


class Flux2DiTStateDictConverter:
    """The diffusers layout is native; the official single-file layout only renames prefixes."""

    _PREFIXES = (("img_in.weight", "x_embedder.weight"), ("txt_in.weight", "context_embedder.weight"),
                 ("time_in.", "time_guidance_embed."), ("vector_in.", "double_stream_modulation_img.linear."),
                 ("guidance_in.", "time_guidance_embed.guidance_embedder."), ("double_blocks.", "transformer_blocks."),
                 ("single_blocks.", "single_transformer_blocks."), ("final_layer.", "norm_out."))  # fmt: skip

    def from_diffusers(self, sd: dict):
        return sd, {}

    def from_official(self, sd: dict):
        out = {}
        for key, value in sd.items():
            for old, new in self._PREFIXES:
                if key.startswith(old):
                    key = new + key[len(old):]
                    break
            out[key] = value
        return out, {}


def _register() -> None:
    from telefuser_b200.core.model_registry import register_architecture

    register_architecture("flux2_dit", Flux2DiT, lambda: Flux2DiT())


_register()
