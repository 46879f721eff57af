"""HunyuanVideo-1.5 MM-DiT (double-stream blocks, optional single-stream blocks; also the super-resolution DiT).

Streams: video tokens (patchified latents concatenated with the conditioning latents and a mask channel) and a
text stream assembled from the LLM text tokens refined by a two-block token refiner, glyph (ByT5) tokens and
vision (image encoder) tokens, each tagged with a learned condition-type embedding. One vector (timestep, plus
optional pooled text / guidance / second timestep embeddings) modulates every block. A double block is the usual
dual-stream layer with per-stream fused QKV GEMMs written into one joint [video; text] buffer, per-head RMSNorm,
3-axis interleaved RoPE (16/56/56, theta 256) on the video part only, one joint attention and per-stream
GELU-tanh MLPs with gate and residual in the GEMM epilogues.
Role parity: telefuser/models/hunyuan_video_dit.py:333-2124.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn

from telefuser_b200.core.base_model import BaseModel
from telefuser_b200.models.qwen_image_dit import _WeightOnly
from telefuser_b200.models.wan_dit import _fuse_linear_weights
from telefuser_b200.ops import functional as TF
from telefuser_b200.parallel import shard as pshard


def timestep_embedding(t: torch.Tensor, dim: int = 256, max_period: float = 10000.0) -> torch.Tensor:
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    args = t[:, None].float() * freqs[None]
    return torch.cat([args.cos(), args.sin()], dim=-1)


def rope_tables(rope_dim_list, sizes, theta: float, device):
    """fp32 (cos, sin) [T*H*W, head_dim/2], one angle per interleaved pair, axes in (t, h, w) order."""
    grids = torch.meshgrid(*[torch.arange(n, dtype=torch.float32) for n in sizes], indexing="ij")
    parts = []
    for d, g in zip(rope_dim_list, grids):
        inv = 1.0 / (theta ** (torch.arange(0, d, 2)[: d // 2].float() / d))
        parts.append(torch.outer(g.reshape(-1), inv))
    ang = torch.cat(parts, dim=1)
    return ang.cos().to(device).contiguous(), ang.sin().to(device).contiguous()


def _f32(lin: nn.Linear, x: torch.Tensor) -> torch.Tensor:
    return F.linear(x, lin.weight.float(), None if lin.bias is None else lin.bias.float())


class TimestepEmbedder(nn.Module):
    def __init__(self, hidden_size: int, frequency_embedding_size: int = 256) -> None:
        super().__init__()
        self.frequency_embedding_size = frequency_embedding_size
        self.mlp = nn.Sequential(nn.Linear(frequency_embedding_size, hidden_size), nn.SiLU(), nn.Linear(hidden_size, hidden_size))

    def forward(self, t):
        return _f32(self.mlp[2], F.silu(_f32(self.mlp[0], timestep_embedding(t, self.frequency_embedding_size))))


class ModulateDiT(nn.Module):
    def __init__(self, hidden_size: int, factor: int) -> None:
        super().__init__()
        self.linear = nn.Linear(hidden_size, factor * hidden_size)

    def forward(self, vec):
        """fp32 vec [B, C] -> list of fp32 [B, 1, C]."""
        return [c.unsqueeze(1) for c in _f32(self.linear, F.silu(vec)).chunk(self.linear.out_features // vec.shape[-1], dim=-1)]


class PatchEmbed(nn.Module):
    def __init__(self, patch_size, in_chans: int, embed_dim: int, is_reshape_temporal_channels=False, concat_condition=True):
        super().__init__()
        self.patch_size = tuple(patch_size)
        if concat_condition:
            in_chans = in_chans + in_chans // 2 + 1 if is_reshape_temporal_channels else in_chans * 2 + 1
        self.proj = nn.Conv3d(in_chans, embed_dim, kernel_size=self.patch_size, stride=self.patch_size)

    def forward(self, x):
        return self.proj(x).flatten(2).transpose(1, 2)


class TextProjection(nn.Module):
    def __init__(self, in_channels: int, hidden_size: int) -> None:
        super().__init__()
        self.linear_1, self.linear_2 = nn.Linear(in_channels, hidden_size), nn.Linear(hidden_size, hidden_size)

    def forward(self, x):
        return self.linear_2(F.silu(self.linear_1(x)))


class VisionProjection(nn.Module):
    def __init__(self, input_dim: int, output_dim: int) -> None:
        super().__init__()
        self.proj = nn.Sequential(nn.LayerNorm(input_dim), nn.Linear(input_dim, input_dim), nn.GELU(),
                                  nn.Linear(input_dim, output_dim), nn.LayerNorm(output_dim))  # fmt: skip

    def forward(self, x):
        return self.proj(x)


class ByT5Mapper(nn.Module):
    def __init__(self, in_dim=1472, out_dim=3072, hidden_dim=12288, out_dim1=3072, use_residual=False) -> None:
        super().__init__()
        self.layernorm = nn.LayerNorm(in_dim)
        self.fc1, self.fc2, self.fc3 = nn.Linear(in_dim, hidden_dim), nn.Linear(hidden_dim, out_dim), nn.Linear(out_dim, out_dim1)
        self.use_residual = use_residual

    def forward(self, x):
        y = self.fc3(F.gelu(self.fc2(F.gelu(self.fc1(self.layernorm(x))))))
        return y + x if self.use_residual else y


class MLP(nn.Module):
    def __init__(self, in_channels: int, hidden_channels: int, act: str = "gelu_tanh") -> None:
        super().__init__()
        self.fc1, self.fc2, self.act = nn.Linear(in_channels, hidden_channels), nn.Linear(hidden_channels, in_channels), act

    def forward(self, x, residual=None, gate=None):
        if self.act == "gelu_tanh":
            h = TF.linear(x, self.fc1.weight, self.fc1.bias, act="gelu_tanh")
        else:
            h = F.silu(TF.linear(x, self.fc1.weight, self.fc1.bias))
        return TF.linear(h, self.fc2.weight, self.fc2.bias, residual=residual, gate=gate)


class MLPEmbedder(nn.Module):
    def __init__(self, in_dim: int, hidden_dim: int) -> None:
        super().__init__()
        self.in_layer, self.out_layer = nn.Linear(in_dim, hidden_dim), nn.Linear(hidden_dim, hidden_dim)

    def forward(self, x):
        return _f32(self.out_layer, F.silu(_f32(self.in_layer, x.float())))


class FinalLayer(nn.Module):
    def __init__(self, hidden_size: int, patch_size, out_channels: int) -> None:
        super().__init__()
        self.linear = nn.Linear(hidden_size, math.prod(patch_size) * out_channels)
        self.adaLN_modulation = nn.Sequential(nn.SiLU(), nn.Linear(hidden_size, 2 * hidden_size))

    def forward(self, x, vec):
        shift, scale = _f32(self.adaLN_modulation[1], F.silu(vec)).chunk(2, dim=1)
        return TF.linear(TF.layernorm_modulate(x, shift.unsqueeze(1), scale.unsqueeze(1), eps=1e-6), self.linear.weight, self.linear.bias)


class IndividualTokenRefinerBlock(nn.Module):
    def __init__(self, hidden_size: int, heads_num: int, mlp_width_ratio: float = 4.0) -> None:
        super().__init__()
        self.heads_num = heads_num
        self.norm1 = nn.LayerNorm(hidden_size, eps=1e-6)
        self.self_attn_qkv = nn.Linear(hidden_size, hidden_size * 3)
        self.self_attn_proj = nn.Linear(hidden_size, hidden_size)
        self.norm2 = nn.LayerNorm(hidden_size, eps=1e-6)
        self.mlp = MLP(hidden_size, int(hidden_size * mlp_width_ratio), act="silu")
        self.adaLN_modulation = nn.Sequential(nn.SiLU(), nn.Linear(hidden_size, 2 * hidden_size))

    def forward(self, x, c):
        gate_msa, gate_mlp = (g.unsqueeze(1) for g in _f32(self.adaLN_modulation[1], F.silu(c)).chunk(2, dim=1))
        B, L, C = x.shape
        n1 = TF.layernorm_modulate(x, None, None, self.norm1.weight, self.norm1.bias, 1e-6)
        qkv = TF.linear(n1, self.self_attn_qkv.weight, self.self_attn_qkv.bias).view(B, L, 3, self.heads_num, -1)
        a = TF.attention(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]).reshape(B, L, C)
        x = TF.linear(a, self.self_attn_proj.weight, self.self_attn_proj.bias, residual=x, gate=gate_msa)
        n2 = TF.layernorm_modulate(x, None, None, self.norm2.weight, self.norm2.bias, 1e-6)
        return self.mlp(n2, residual=x, gate=gate_mlp)


class IndividualTokenRefiner(nn.Module):
    def __init__(self, hidden_size: int, heads_num: int, depth: int) -> None:
        super().__init__()
        self.blocks = nn.ModuleList([IndividualTokenRefinerBlock(hidden_size, heads_num) for _ in range(depth)])

    def forward(self, x, c):
        for b in self.blocks:
            x = b(x, c)
        return x


class SingleTokenRefiner(nn.Module):
    def __init__(self, in_channels: int, hidden_size: int, heads_num: int, depth: int) -> None:
        super().__init__()
        self.input_embedder = nn.Linear(in_channels, hidden_size)
        self.t_embedder = TimestepEmbedder(hidden_size)
        self.c_embedder = TextProjection(in_channels, hidden_size)
        self.individual_token_refiner = IndividualTokenRefiner(hidden_size, heads_num, depth)

    def forward(self, x, t):
        ce = self.c_embedder
        c = self.t_embedder(t) + _f32(ce.linear_2, F.silu(_f32(ce.linear_1, x.float().mean(dim=1))))
        return self.individual_token_refiner(TF.linear(x, self.input_embedder.weight, self.input_embedder.bias), c)


def _joint_attention(q, k, v, usp: bool):
    if usp:
        from telefuser_b200.parallel.ring import long_context_attention

        return long_context_attention(q, k, v)
    return TF.attention(q, k, v)


class MMDoubleStreamBlock(nn.Module):
    def __init__(self, hidden_size: int, heads_num: int, mlp_width_ratio: float = 4.0, mlp_act_type: str = "gelu_tanh",
                 qk_norm: bool = True, qkv_bias: bool = False) -> None:  # fmt: skip
        super().__init__()
        self.heads_num, self.head_dim = heads_num, hidden_size // heads_num
        hid = int(hidden_size * mlp_width_ratio)
        lin = lambda: nn.Linear(hidden_size, hidden_size, bias=qkv_bias)  # noqa: E731
        norm = lambda: _WeightOnly(self.head_dim) if qk_norm else None  # noqa: E731
        self.img_mod = ModulateDiT(hidden_size, 6)
        self.img_attn_q, self.img_attn_k, self.img_attn_v, self.img_attn_proj = lin(), lin(), lin(), lin()
        self.img_attn_q_norm, self.img_attn_k_norm = norm(), norm()
        self.img_mlp = MLP(hidden_size, hid, mlp_act_type)
        self.txt_mod = ModulateDiT(hidden_size, 6)
        self.txt_attn_q, self.txt_attn_k, self.txt_attn_v, self.txt_attn_proj = lin(), lin(), lin(), lin()
        self.txt_attn_q_norm, self.txt_attn_k_norm = norm(), norm()
        self.txt_mlp = MLP(hidden_size, hid, mlp_act_type)
        self._img = self._txt = None
        self.usp = False

    def _fused(self, slot: str, linears):
        cur = getattr(self, slot)
        w = linears[0].weight
        if cur is None or cur[0].data_ptr() != w.data_ptr() or cur[0].dtype != w.dtype:
            cur = _fuse_linear_weights(linears)
            setattr(self, slot, cur)
        return cur

    def forward(self, img, txt, vec, rope):
        si1, ci1, gi1, si2, ci2, gi2 = self.img_mod(vec)
        st1, ct1, gt1, st2, ct2, gt2 = self.txt_mod(vec)
        B, Si, C = img.shape
        St = txt.shape[1]
        H, D = self.heads_num, self.head_dim
        Wi, bi = self._fused("_img", [self.img_attn_q, self.img_attn_k, self.img_attn_v])
        Wt, bt = self._fused("_txt", [self.txt_attn_q, self.txt_attn_k, self.txt_attn_v])
        im, tm = TF.layernorm_modulate(img, si1, ci1, eps=1e-6), TF.layernorm_modulate(txt, st1, ct1, eps=1e-6)
        if B == 1:
            joint = torch.empty(B, Si + St, 3 * C, device=img.device, dtype=img.dtype)
            TF.linear(im, Wi, bi, out=joint[:, :Si])
            TF.linear(tm, Wt, bt, out=joint[:, Si:])
        else:
            joint = torch.cat([TF.linear(im, Wi, bi), TF.linear(tm, Wt, bt)], dim=1)
        q, k, v = (joint[..., i * C : (i + 1) * C].unflatten(-1, (H, D)) for i in range(3))
        if self.img_attn_q_norm is not None:
            cos, sin = (None, None) if rope is None else (rope if B == 1 else tuple(t.repeat(B, 1) for t in rope))
            TF.headnorm_rope_(q[:, :Si], self.img_attn_q_norm.weight, cos, sin, 1e-6, k=k[:, :Si], weight_k=self.img_attn_k_norm.weight)
            TF.headnorm_rope_(q[:, Si:], self.txt_attn_q_norm.weight, None, None, 1e-6, k=k[:, Si:], weight_k=self.txt_attn_k_norm.weight)
        o = _joint_attention(q, k, v, self.usp).reshape(B, Si + St, C)
        img = TF.linear(o[:, :Si], self.img_attn_proj.weight, self.img_attn_proj.bias, residual=img, gate=gi1)
        img = self.img_mlp(TF.layernorm_modulate(img, si2, ci2, eps=1e-6), residual=img, gate=gi2)
        txt = TF.linear(o[:, Si:], self.txt_attn_proj.weight, self.txt_attn_proj.bias, residual=txt, gate=gt1)
        txt = self.txt_mlp(TF.layernorm_modulate(txt, st2, ct2, eps=1e-6), residual=txt, gate=gt2)
        return img, txt


class LinearWarpforSingle(nn.Module):
    def __init__(self, in_dim: int, out_dim: int, bias: bool = True) -> None:
        super().__init__()
        self.fc = nn.Linear(in_dim, out_dim, bias=bias)


class MMSingleStreamBlock(nn.Module):
    def __init__(self, hidden_size: int, heads_num: int, mlp_width_ratio: float = 4.0, qk_norm: bool = True) -> None:
        super().__init__()
        self.heads_num, self.head_dim, self.hidden_size = heads_num, hidden_size // heads_num, hidden_size
        self.mlp_hidden_dim = int(hidden_size * mlp_width_ratio)
        self.linear1_q, self.linear1_k, self.linear1_v = (nn.Linear(hidden_size, hidden_size) for _ in range(3))
        self.linear1_mlp = nn.Linear(hidden_size, self.mlp_hidden_dim)
        self.linear2 = LinearWarpforSingle(hidden_size + self.mlp_hidden_dim, hidden_size, bias=True)
        self.q_norm = _WeightOnly(self.head_dim) if qk_norm else None
        self.k_norm = _WeightOnly(self.head_dim) if qk_norm else None
        self.modulation = ModulateDiT(hidden_size, 3)
        self._fused = None
        self.usp = False

    def forward(self, x, vec, txt_len: int, rope):
        shift, scale, gate = self.modulation(vec)
        B, S, C = x.shape
        H, D = self.heads_num, self.head_dim
        w = self.linear1_q.weight
        if self._fused is None or self._fused[0].data_ptr() != w.data_ptr() or self._fused[0].dtype != w.dtype:
            self._fused = _fuse_linear_weights([self.linear1_q, self.linear1_k, self.linear1_v, self.linear1_mlp])
        fused = TF.linear(TF.layernorm_modulate(x, shift, scale, eps=1e-6), self._fused[0], self._fused[1])
        q, k, v = (fused[..., i * C : (i + 1) * C].unflatten(-1, (H, D)) for i in range(3))
        Si = S - txt_len
        if self.q_norm is not None:
            cos, sin = rope if B == 1 else tuple(t.repeat(B, 1) for t in rope)
            TF.headnorm_rope_(q[:, :Si], self.q_norm.weight, cos, sin, 1e-6, k=k[:, :Si], weight_k=self.k_norm.weight)
            TF.headnorm_rope_(q[:, Si:], self.q_norm.weight, None, None, 1e-6, k=k[:, Si:], weight_k=self.k_norm.weight)
        o = _joint_attention(q, k, v, self.usp).reshape(B, S, C)
        m = F.gelu(fused[..., 3 * C :], approximate="tanh")
        W = self.linear2.fc.weight
        if TF.is_quantized_weight(W):  # scales per output row or per K block: one GEMM over the joined input
            return TF.linear(torch.cat([o, m], dim=-1), W, self.linear2.fc.bias, residual=x, gate=gate)
        h = TF.linear(o, W[:, :C], self.linear2.fc.bias, residual=x, gate=gate)  # the output projection in two K-slices
        return TF.linear(m, W[:, C:], residual=h, gate=gate)


class HunyuanVideoDiT(BaseModel):
    def __init__(self, patch_size=(1, 1, 1), in_channels: int = 32, concat_condition: bool = True, out_channels=None,
                 hidden_size: int = 2048, heads_num: int = 16, mlp_width_ratio: float = 4.0, mlp_act_type: str = "gelu_tanh",
                 mm_double_blocks_depth: int = 54, mm_single_blocks_depth: int = 0, rope_dim_list=(16, 56, 56),
                 qkv_bias: bool = True, qk_norm: bool = True, qk_norm_type: str = "rms", guidance_embed: bool = False,
                 use_meanflow: bool = False, text_projection: str = "single_refiner", use_attention_mask: bool = True,
                 text_states_dim: int = 3584, text_states_dim_2=None, text_pool_type=None, rope_theta: float = 256,
                 glyph_byT5_v2: bool = True, vision_projection: str = "linear", vision_states_dim: int = 1152,
                 is_reshape_temporal_channels: bool = False, use_cond_type_embedding: bool = True, **_unused) -> None:  # fmt: skip
        super().__init__()
        if hidden_size % heads_num or sum(rope_dim_list) != hidden_size // heads_num:
            raise ValueError("the RoPE axes must add up to the head dimension")
        self.patch_size, self.in_channels = tuple(patch_size), in_channels
        self.out_channels = in_channels if out_channels is None else out_channels
        self.hidden_size, self.heads_num = hidden_size, heads_num
        self.rope_dim_list, self.rope_theta = tuple(rope_dim_list), rope_theta
        self.guidance_embed, self.text_projection = guidance_embed, text_projection
        self.byt5_in = ByT5Mapper(1472, hidden_size, hidden_size, hidden_size, False) if glyph_byT5_v2 else None
        self.img_in = PatchEmbed(self.patch_size, in_channels, hidden_size, is_reshape_temporal_channels, concat_condition)
        self.vision_in = VisionProjection(vision_states_dim, hidden_size) if vision_projection == "linear" else None
        if text_projection == "linear":
            self.txt_in = TextProjection(text_states_dim, hidden_size)
        elif text_projection == "single_refiner":
            self.txt_in = SingleTokenRefiner(text_states_dim, hidden_size, heads_num, depth=2)
        else:
            raise NotImplementedError(f"unsupported text_projection {text_projection}")
        self.time_in = TimestepEmbedder(hidden_size)
        self.vector_in = MLPEmbedder(text_states_dim_2, hidden_size) if text_pool_type is not None else None
        self.guidance_in = TimestepEmbedder(hidden_size) if guidance_embed else None
        self.time_r_in = TimestepEmbedder(hidden_size) if use_meanflow else None
        self.double_blocks = nn.ModuleList([MMDoubleStreamBlock(hidden_size, heads_num, mlp_width_ratio, mlp_act_type, qk_norm,
                                                                qkv_bias) for _ in range(mm_double_blocks_depth)])  # fmt: skip
        self.single_blocks = nn.ModuleList([MMSingleStreamBlock(hidden_size, heads_num, mlp_width_ratio, qk_norm)
                                            for _ in range(mm_single_blocks_depth)])  # fmt: skip
        self.final_layer = FinalLayer(hidden_size, self.patch_size, self.out_channels)
        self.cond_type_embedding = nn.Embedding(3, hidden_size) if use_cond_type_embedding else None
        self.dtype = torch.bfloat16
        self.layer_name_list = ["double_blocks", "single_blocks"]

    def enable_usp(self) -> None:
        super().enable_usp()
        for b in list(self.double_blocks) + list(self.single_blocks):
            b.usp = True

    def get_fsdp_module_names(self) -> list[str]:
        return ["double_blocks", "single_blocks"]

    def enable_quant(self, quant=None) -> int:
        """Attention and MLP projections of both block lists in the requested stored format; the modulation linears
        (`img_mod`, `txt_mod`, `modulation`) are evaluated in fp32 from the time embedding and stay as they are."""
        from telefuser_b200.ops.quant import quantize_model_

        return quantize_model_(self, quant, ("double_blocks.*", "single_blocks.*"), ("_mod.", "modulation"))

    def get_rotary_pos_embed(self, rope_sizes, device="cpu"):
        return rope_tables(self.rope_dim_list, rope_sizes, self.rope_theta, device)

    def _tagged(self, tokens, kind: int):
        return tokens if self.cond_type_embedding is None else tokens + self.cond_type_embedding.weight[kind].to(tokens.dtype)

    @torch.no_grad()
    def forward(self, hidden_states, timestep, text_states, text_states_2=None, encoder_attention_mask=None, timestep_r=None,
                vision_states=None, freqs_cos=None, freqs_sin=None, return_dict: bool = False, guidance=None,
                mask_type: str = "t2v", byt5_text_states=None, byt5_text_mask=None, cond_flag: bool = True):  # fmt: skip
        """hidden_states [B, C_in, T, H, W] (latents + conditioning + mask); timestep [B]; text_states [B, L, text_dim]
        with `encoder_attention_mask` [B, L] -> [B, C_out, T, H, W]."""
        dt = self.img_in.proj.weight.dtype
        dev = hidden_states.device
        valid = lambda e, m: e if m is None else e[:, m[0].nonzero(as_tuple=True)[0]]  # noqa: E731
        txt = valid(text_states, encoder_attention_mask).to(dt)
        B, _, ot, oh, ow = hidden_states.shape
        p = self.patch_size
        grid = (ot // p[0], oh // p[1], ow // p[2])
        rope = (freqs_cos.to(dev), freqs_sin.to(dev)) if freqs_cos is not None else self.get_rotary_pos_embed(grid, dev)
        if rope[0].shape[-1] == self.hidden_size // self.heads_num:  # tables with one entry per element -> per pair
            rope = (rope[0][:, ::2].contiguous(), rope[1][:, ::2].contiguous())
        img = self.img_in(hidden_states.to(dt))
        t = timestep.to(dev)
        vec = self.time_in(t)
        if text_states_2 is not None and self.vector_in is not None:
            vec = vec + self.vector_in(text_states_2)
        if self.guidance_embed:
            g = guidance if guidance is not None else torch.tensor([6016.0], device=dev)
            vec = vec + self.guidance_in(g.to(dev))
        if timestep_r is not None and self.time_r_in is not None:
            vec = vec + self.time_r_in(timestep_r.to(dev))
        txt = self.txt_in(txt, t) if self.text_projection == "single_refiner" else self.txt_in(txt)
        txt = self._tagged(txt, 0)

        def match_batch(x):
            if x.shape[0] == 1 and txt.shape[0] > 1:
                return x.expand(txt.shape[0], -1, -1)
            return x[:1] if x.shape[0] > 1 and txt.shape[0] == 1 else x

        if self.byt5_in is not None and byt5_text_states is not None:
            glyph = self._tagged(self.byt5_in(valid(byt5_text_states, byt5_text_mask).to(dt)), 1)
            txt = torch.cat([match_batch(glyph), txt], dim=1)
        if self.vision_in is not None and vision_states is not None:
            # text-to-video passes all-zero vision states: no vision tokens join the text stream then
            if not (mask_type == "t2v" and torch.all(vision_states == 0)):
                vis = self._tagged(self.vision_in(vision_states.to(dt)), 2)
                txt = torch.cat([match_batch(vis), txt], dim=1)
        n_img = img.shape[1]
        if self.usp_flag:
            P = pshard._sp(None)[1]
            if n_img % P or txt.shape[1] % P:
                raise ValueError("sequence parallel HunyuanVideo needs video and text lengths divisible by the group size")
            img, txt, rc, rs = pshard.sequence_parallel_shard([img, txt, rope[0], rope[1]], [1, 1, 0, 0])
            rope = (rc.contiguous(), rs.contiguous())
        ori = img
        cache = self.feature_cache
        if cache.should_compute(cond_flag):
            offload = getattr(self, "async_offload_manager", None) if self.async_offload_flag else None
            for i, blk in enumerate(self.double_blocks):
                if offload is not None:
                    offload.before_layer(i)
                img, txt = blk(img, txt, vec, rope)
                if offload is not None:
                    offload.after_layer(i)
            if len(self.single_blocks) > 0:
                x = torch.cat([img, txt], dim=1)
                for blk in self.single_blocks:
                    x = blk(x, vec, txt.shape[1], rope)
                img = x[:, : img.shape[1]]
            cache.update(img, ori, cond_flag)
        else:
            img = cache.approximate(img, cond_flag)
        out = self.final_layer(img, vec)
        if self.usp_flag:
            (out,) = pshard.sequence_parallel_unshard([out], [1], [n_img])
        c = self.out_channels
        out = out.view(B, grid[0], grid[1], grid[2], c, p[0], p[1], p[2]).permute(0, 4, 1, 5, 2, 6, 3, 7)
        return out.reshape(B, c, grid[0] * p[0], grid[1] * p[1], grid[2] * p[2])

    @staticmethod
    def state_dict_converter():
        return HunyuanVideoStateDictConverter()


class HunyuanVideoStateDictConverter:
    def from_official(self, sd: dict):
        return sd, {}

    def from_diffusers(self, sd: dict):
        return sd, {}
