"""LingBot-Video transformers: dense (1.3B) and mixture-of-experts (128 experts, top-8, 30B-A3B).

Joint [video; text] token stream, sandwich RMSNorm around attention and FFN with tanh gates, per-head
q/k RMSNorm + three-axis RoPE (theta 256, axes 32/48/48, text positions on the time axis), SwiGLU FFN
or group-limited sigmoid-routed experts plus one shared expert. Parameter names follow the public
checkpoints, so their state dicts load unchanged.

Execution here: one fused-QKV GEMM, `headnorm_rope_` (per-head norm + RoPE on q and k in one launch),
the tcgen05 attention kernel (head_dim 128), `rmsnorm_modulate` / `rmsnorm_gate_residual` row kernels
for the sandwich glue, fused gate|up GEMM + SiLU-mul, and for sparse layers the route -> plan ->
permute -> grouped GEMM -> combine kernel chain of `ops.moe` (optionally expert-parallel). Samples of a
batch run one after another, each with its text cut to its valid length, which equals the reference's
packed-sequence form without building masks.
Role parity: telefuser/models/lingbot_video_dit.py:23-560, lingbot_video_moe.py:22-349.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn

from telefuser_b200.core.base_model import BaseModel
from telefuser_b200.ops import functional as TF
from telefuser_b200.ops import moe as MOE
from telefuser_b200.parallel import ulysses


@dataclass
class LingBotVideoConfig:
    patch_size: tuple = (1, 2, 2)
    in_channels: int = 16
    out_channels: int = 16
    hidden_size: int = 2048
    num_attention_heads: int = 16
    depth: int = 24
    intermediate_size: int = 6144
    text_dim: int = 2560
    freq_dim: int = 256
    norm_eps: float = 1e-6
    rope_theta: float = 256.0
    axes_dims: tuple = (32, 48, 48)
    qkv_bias: bool = False
    out_bias: bool = True
    patch_embed_bias: bool = True
    timestep_mlp_bias: bool = True
    # mixture of experts (num_experts == 0: dense model)
    num_experts: int = 0
    num_experts_per_tok: int = 8
    moe_intermediate_size: int = 768
    decoder_sparse_step: int = 1
    mlp_only_layers: tuple = field(default_factory=tuple)
    n_group: int = 4
    topk_group: int = 2
    routed_scaling_factor: float = 2.5
    n_shared_experts: int = 1

    @classmethod
    def preset(cls, name: str) -> "LingBotVideoConfig":
        table = {
            "dense-1.3b": dict(),
            "moe-30b-a3b": dict(depth=48, num_experts=128),
            "tiny": dict(hidden_size=128, num_attention_heads=2, depth=2, intermediate_size=256, text_dim=32,
                         axes_dims=(16, 24, 24)),
            "tiny-moe": dict(hidden_size=128, num_attention_heads=2, depth=2, intermediate_size=256, text_dim=32,
                             axes_dims=(16, 24, 24), num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64,
                             n_group=2, topk_group=1),
        }  # fmt: skip
        return cls(**table[name])


class RMSNormWeight(nn.Module):
    def __init__(self, dim: int, eps: float) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.variance_epsilon = eps


def _fuse_rows(mods: list[nn.Linear]):
    from telefuser_b200.models.wan_dit import _fuse_linear_weights

    return _fuse_linear_weights(mods)


class LingBotVideoMLP(nn.Module):
    def __init__(self, hidden: int, inter: int) -> None:
        super().__init__()
        self.gate_proj = nn.Linear(hidden, inter, bias=False)
        self.up_proj = nn.Linear(hidden, inter, bias=False)
        self.down_proj = nn.Linear(inter, hidden, bias=False)
        self._gu = None

    def fused_gate_up(self):
        w = self.gate_proj.weight
        if self._gu is None or self._gu.data_ptr() != w.data_ptr() or self._gu.dtype != w.dtype or self._gu.device != w.device:
            self._gu = _fuse_rows([self.gate_proj, self.up_proj])[0]
        return self._gu

    def forward(self, x):
        return TF.linear(TF.act_mul(TF.linear(x, self.fused_gate_up()), "silu"), self.down_proj.weight)


class LingBotVideoRouter(nn.Module):
    def __init__(self, hidden: int, num_experts: int, top_k: int, n_group: int, topk_group: int, route_scale: float):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(num_experts, hidden))
        self.register_buffer("e_score_correction_bias", torch.zeros(num_experts), persistent=True)
        self.num_experts, self.top_k, self.n_group, self.topk_group = num_experts, top_k, n_group, topk_group
        self.route_scale = route_scale

    def forward(self, tokens):
        logits = F.linear(tokens.float(), self.weight.float())  # fp32 logits: routing is sensitive to rounding
        return MOE.route_topk(logits, self.n_group, self.topk_group, self.top_k, self.e_score_correction_bias,
                              self.route_scale, return_counts=True)  # fmt: skip


class LingBotVideoGroupedExperts(nn.Module):
    def __init__(self, num_experts: int, hidden: int, inter: int) -> None:
        super().__init__()
        self.w1 = nn.Parameter(torch.empty(num_experts, inter, hidden))
        self.w2 = nn.Parameter(torch.empty(num_experts, hidden, inter))
        self.w3 = nn.Parameter(torch.empty(num_experts, inter, hidden))
        # per-output-channel scales of e4m3 expert weights; None until `quantize_fp8_`
        self.register_buffer("w1_scale", None, persistent=True)
        self.register_buffer("w2_scale", None, persistent=True)
        self.register_buffer("w3_scale", None, persistent=True)
        self._w13 = None
        self._w13_scale = None
        self.ep = None  # expert-parallel state set by `enable_expert_parallel`

    def quantize_fp8_(self) -> None:
        """In place: the three stacked expert weights become e4m3 with one scale per output channel of each expert
        (W8A8 at run time: tokens are quantised per row in front of each GEMM). Role parity:
        telefuser/models/lingbot_video_moe.py:76-87."""
        if self.w1.dtype == torch.float8_e4m3fn:
            return
        if self.ep is not None:
            raise RuntimeError("quantise the experts before `enable_expert_parallel`; the sharded exchange path is bf16")
        for name in ("w1", "w2", "w3"):
            q, scale = MOE.quantize_expert_weight_fp8(getattr(self, name).detach())
            setattr(self, name, nn.Parameter(q, requires_grad=False))
            setattr(self, name + "_scale", scale)
        self._w13 = self._w13_scale = None

    def fused_w13_scale(self):
        """[E, 2I] fp32: gate-row scales then up-row scales, matching `fused_w13`."""
        s = self._w13_scale
        if s is None or s.device != self.w1.device:
            s = self._w13_scale = torch.cat([self.w1_scale, self.w3_scale], dim=1).to(self.w1.device).contiguous()
        return s

    def fused_w13(self):
        """[E, 2I, C]: gate rows then up rows of every expert; w1 / w3 become views of it."""
        w = self.w1
        if self._w13 is None or self._w13.device != w.device or self._w13.dtype != w.dtype or \
                self._w13.data_ptr() != w.data_ptr():  # fmt: skip
            E, inter, C = w.shape
            buf = torch.empty(E, 2 * inter, C, dtype=w.dtype, device=w.device)
            buf[:, :inter].copy_(self.w1.data)
            buf[:, inter:].copy_(self.w3.data)
            self.w1.data, self.w3.data = buf[:, :inter], buf[:, inter:]
            self._w13 = buf
        return self._w13

    def forward(self, tokens, indices, weights, counts=None):
        if self.w2.dtype == torch.float8_e4m3fn:
            if self.ep is not None:
                raise RuntimeError("expert parallelism exchanges bf16 expert inputs; e4m3 experts run unsharded")
            return MOE.experts_forward_fp8(tokens, indices, weights, self.fused_w13(), self.fused_w13_scale(), self.w2.data,
                                           self.w2_scale, counts=counts)  # fmt: skip
        if self.ep is not None:
            from telefuser_b200.parallel.expert import experts_forward_ep

            return experts_forward_ep(tokens, indices, weights, self.fused_w13(), self.w2.data, self.ep)
        return MOE.experts_forward(tokens, indices, weights, self.fused_w13(), self.w2.data, counts=counts)


class LingBotVideoSparseMoeBlock(nn.Module):
    def __init__(self, cfg: LingBotVideoConfig) -> None:
        super().__init__()
        self.router = LingBotVideoRouter(cfg.hidden_size, cfg.num_experts, cfg.num_experts_per_tok, cfg.n_group,
                                         cfg.topk_group, cfg.routed_scaling_factor)  # fmt: skip
        self.experts = LingBotVideoGroupedExperts(cfg.num_experts, cfg.hidden_size, cfg.moe_intermediate_size)
        self.shared_experts = (LingBotVideoMLP(cfg.hidden_size, cfg.moe_intermediate_size * cfg.n_shared_experts)
                               if cfg.n_shared_experts > 0 else None)  # fmt: skip

    def forward(self, x, valid: int | None = None):
        B, S, C = x.shape
        tokens = x.reshape(-1, C)
        ids, w, counts = self.router(tokens)
        if valid is not None and valid < B * S:  # padded tail rows carry no weight
            w = w.clone()
            w[valid:] = 0
        out = self.experts(tokens, ids, w.to(torch.float32), counts).reshape(B, S, C)
        if self.shared_experts is not None:
            out = out + self.shared_experts(x)
        return out


class LingBotVideoAttention(nn.Module):
    def __init__(self, hidden: int, heads: int, eps: float, qkv_bias: bool, out_bias: bool) -> None:
        super().__init__()
        self.num_heads, self.head_dim = heads, hidden // heads
        self.to_q = nn.Linear(hidden, hidden, bias=qkv_bias)
        self.to_k = nn.Linear(hidden, hidden, bias=qkv_bias)
        self.to_v = nn.Linear(hidden, hidden, bias=qkv_bias)
        self.norm_q = RMSNormWeight(self.head_dim, eps)
        self.norm_k = RMSNormWeight(self.head_dim, eps)
        self.to_out = nn.Linear(hidden, hidden, bias=out_bias)
        self.ulysses_group = None
        self._qkv = None

    def fused_qkv(self):
        w = self.to_q.weight
        if self._qkv is None or self._qkv[0].device != w.device or self._qkv[0].dtype != w.dtype or \
                self._qkv[0].data_ptr() != w.data_ptr():  # fmt: skip
            self._qkv = _fuse_rows([self.to_q, self.to_k, self.to_v])
        return self._qkv

    def forward(self, x, cos, sin, kv_len: int | None = None):
        """x: [1, S_local, C]; cos/sin: fp32 [S_local, D/2]; kv_len: valid keys of the whole sequence."""
        B, S, C = x.shape
        H, D = self.num_heads, self.head_dim
        W, b = self.fused_qkv()
        qkv = TF.linear(x, W, b)
        q, k, v = (qkv[..., i * C : (i + 1) * C].unflatten(-1, (H, D)) for i in range(3))
        eps = self.norm_q.variance_epsilon
        TF.headnorm_rope_(q, self.norm_q.weight, cos, sin, eps, k=k, weight_k=self.norm_k.weight)
        g = self.ulysses_group
        if g is not None and dist.is_initialized() and dist.get_world_size(g) > 1:
            hq, hk, hv = (ulysses.scatter_heads(t.contiguous(), g) for t in (q, k, v))
            n = hk.shape[1] if kv_len is None else kv_len
            o = ulysses.gather_heads(TF.attention(hq, hk[:, :n], hv[:, :n]), g)
        else:
            n = S if kv_len is None else kv_len
            o = TF.attention(q, k[:, :n], v[:, :n])
        return TF.linear(o.reshape(B, S, C), self.to_out.weight, self.to_out.bias)


class LingBotVideoBlock(nn.Module):
    def __init__(self, cfg: LingBotVideoConfig, layer_index: int) -> None:
        super().__init__()
        C, eps = cfg.hidden_size, cfg.norm_eps
        self.scale_shift_table = nn.Parameter(torch.zeros(1, 6 * C))
        self.norm1 = RMSNormWeight(C, eps)
        self.attn = LingBotVideoAttention(C, cfg.num_attention_heads, eps, cfg.qkv_bias, cfg.out_bias)
        self.norm_post_attn = RMSNormWeight(C, eps)
        self.norm2 = RMSNormWeight(C, eps)
        sparse = (cfg.num_experts > 0 and layer_index not in cfg.mlp_only_layers
                  and (layer_index + 1) % cfg.decoder_sparse_step == 0)  # fmt: skip
        self.ffn = LingBotVideoSparseMoeBlock(cfg) if sparse else LingBotVideoMLP(C, cfg.intermediate_size)
        self.norm_post_ffn = RMSNormWeight(C, eps)
        self.eps = eps

    def forward(self, x, temb6, cos, sin, kv_len=None, valid=None):
        """x: [1, S, C]; temb6: fp32 [1, 6C] time modulation of this sample."""
        C = x.shape[-1]
        mod = (temb6.float() + self.scale_shift_table.float()).view(1, 6, C)
        shift_msa, scale_msa, gate_msa, shift_mlp, scale_mlp, gate_mlp = (mod[:, i : i + 1] for i in range(6))
        h = TF.rmsnorm_modulate(x, self.norm1.weight, shift_msa, scale_msa, self.eps)
        a = self.attn(h, cos, sin, kv_len)
        x = TF.rmsnorm_gate_residual(x, a, self.norm_post_attn.weight, gate_msa, self.eps)
        h = TF.rmsnorm_modulate(x, self.norm2.weight, shift_mlp, scale_mlp, self.eps)
        m = self.ffn(h, valid) if isinstance(self.ffn, LingBotVideoSparseMoeBlock) else self.ffn(h)
        return TF.rmsnorm_gate_residual(x, m, self.norm_post_ffn.weight, gate_mlp, self.eps)


def joint_position_ids(text_len: int, grid_t: int, grid_h: int, grid_w: int, device) -> torch.Tensor:
    """[video; text] positions on (time, height, width): video frames start after the text on the time axis."""
    t = torch.arange(grid_t, device=device, dtype=torch.int32) + text_len + 1
    hh = torch.arange(grid_h, device=device, dtype=torch.int32)
    ww = torch.arange(grid_w, device=device, dtype=torch.int32)
    video = torch.stack(torch.meshgrid(t, hh, ww, indexing="ij"), dim=-1).flatten(0, 2)
    tt = torch.arange(text_len, device=device, dtype=torch.int32) + 1
    text = torch.stack((tt, torch.zeros_like(tt), torch.zeros_like(tt)), dim=-1)
    return torch.cat((video, text), dim=0)


def rope_tables(position_ids: torch.Tensor, axes_dims, theta: float):
    """fp32 cos / sin [S, D/2]; frequencies in float64 as the public implementation does."""
    pos = position_ids.detach().to("cpu", torch.float64)
    ang = []
    for axis, d in enumerate(axes_dims):
        inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float64) / d))
        ang.append((pos[:, axis : axis + 1] * inv[None]).float())
    a = torch.cat(ang, dim=-1).to(position_ids.device)
    return a.cos().contiguous(), a.sin().contiguous()


class LingBotVideoTimeEmbedder(nn.Module):
    def __init__(self, freq_dim: int, hidden: int, bias: bool = True) -> None:
        super().__init__()
        self.frequency_dim = freq_dim
        self.linear_1 = nn.Linear(freq_dim, hidden, bias=bias)
        self.linear_2 = nn.Linear(hidden, hidden, bias=bias)

    def forward(self, timesteps):
        half = self.frequency_dim // 2
        expo = -math.log(10000.0) * torch.arange(half, device=timesteps.device, dtype=torch.float32) / half
        ang = timesteps.float().reshape(-1, 1) * expo.exp().reshape(1, -1)
        emb = torch.cat((ang.cos(), ang.sin()), dim=-1)
        if self.frequency_dim % 2:
            emb = F.pad(emb, (0, 1))
        w1, w2 = self.linear_1, self.linear_2
        h = F.silu(F.linear(emb, w1.weight.float(), None if w1.bias is None else w1.bias.float()))
        return F.linear(h, w2.weight.float(), None if w2.bias is None else w2.bias.float())  # fp32 [B, C]


class LingBotVideoTextEmbedder(nn.Module):
    def __init__(self, text_dim: int, hidden: int) -> None:
        super().__init__()
        self.norm = RMSNormWeight(text_dim, 1e-6)
        self.linear_1 = nn.Linear(text_dim, hidden)
        self.linear_2 = nn.Linear(hidden, hidden)

    def forward(self, x):
        h = TF.rmsnorm_modulate(x, self.norm.weight, None, None, self.norm.variance_epsilon)
        h = F.silu(TF.linear(h.to(self.linear_1.weight.dtype), self.linear_1.weight, self.linear_1.bias))
        return TF.linear(h, self.linear_2.weight, self.linear_2.bias)


class LingBotVideoTransformer3DModel(BaseModel):
    def __init__(self, config: LingBotVideoConfig | None = None, **kw) -> None:
        super().__init__()
        cfg = config or LingBotVideoConfig(**kw)
        if cfg.hidden_size // cfg.num_attention_heads != sum(cfg.axes_dims):
            raise ValueError("head dimension must equal sum(axes_dims)")
        self.config = cfg
        self.patch_size, self.out_channels = tuple(cfg.patch_size), cfg.out_channels
        self.num_layers = cfg.depth
        C = cfg.hidden_size
        self.patch_embedder = nn.Linear(cfg.in_channels * math.prod(cfg.patch_size), C, bias=cfg.patch_embed_bias)
        self.time_embedder = LingBotVideoTimeEmbedder(cfg.freq_dim, C, cfg.timestep_mlp_bias)
        self.time_modulation = nn.Sequential(nn.SiLU(), nn.Linear(C, 6 * C))
        self.text_embedder = LingBotVideoTextEmbedder(cfg.text_dim, C)
        self.blocks = nn.ModuleList([LingBotVideoBlock(cfg, i) for i in range(cfg.depth)])
        self.norm_out = nn.LayerNorm(C, elementwise_affine=False, eps=cfg.norm_eps)
        self.norm_out_modulation = nn.Sequential(nn.SiLU(), nn.Linear(C, 2 * C))
        self.proj_out = nn.Linear(C, math.prod(cfg.patch_size) * cfg.out_channels)
        self.ulysses_group = None
        self.dtype = torch.bfloat16

    # ---- runtime wiring ---------------------------------------------------------
    def set_ulysses_group(self, group) -> None:
        self.ulysses_group = group
        for b in self.blocks:
            b.attn.ulysses_group = group

    def enable_usp(self) -> None:
        super().enable_usp()
        if self.device_mesh is not None and self.device_mesh.size("ulysses") > 1:
            self.set_ulysses_group(self.device_mesh.group("ulysses"))

    def enable_expert_parallel(self, group) -> None:
        from telefuser_b200.parallel.expert import ExpertParallelState

        for b in self.blocks:
            if isinstance(b.ffn, LingBotVideoSparseMoeBlock):
                b.ffn.experts.ep = ExpertParallelState.shard_(b.ffn.experts, group)

    def get_fsdp_module_names(self) -> list[str]:
        return ["blocks"]

    def quantize_experts_fp8_(self) -> int:
        """Routed expert weights of every sparse block to e4m3 (the shared experts and attention projections are
        `nn.Linear` layers and follow `enable_quant`); returns the number of expert banks converted."""
        n = 0
        for b in self.blocks:
            if isinstance(b.ffn, LingBotVideoSparseMoeBlock):
                b.ffn.experts.quantize_fp8_()
                n += 1
        return n

    def enable_quant(self, quant=None) -> int:
        """The block linears in the requested format (routers and gates stay as they are); for FP8 the stacked routed
        experts are quantised too, since they hold most of a MoE checkpoint's bytes."""
        from telefuser_b200.ops.quant import resolve_quant_kind

        n = super().enable_quant(quant)
        if resolve_quant_kind(quant) == "fp8":
            n += self.quantize_experts_fp8_()
        return n

    def promote_stability_layers_to_fp32(self) -> None:
        """Norm weights, modulation tables, time MLPs and routers stay fp32 (the kernels read them as fp32)."""
        keep = {"time_embedder", "time_modulation", "norm", "norm1", "norm2", "norm_q", "norm_k", "norm_post_attn",
                "norm_post_ffn", "norm_out_modulation", "router"}  # fmt: skip
        for name, p in self.named_parameters():
            if any(part in keep for part in name.split(".")) or name.endswith("scale_shift_table"):
                p.data = p.data.float()
        for name, b in self.named_buffers():
            if "router" in name:
                b.data = b.data.float()

    # ---- forward ----------------------------------------------------------------------
    def _patchify(self, x):
        B, Cc, Fr, Hh, Ww = x.shape
        pt, ph, pw = self.patch_size
        g = (Fr // pt, Hh // ph, Ww // pw)
        x = x.reshape(B, Cc, g[0], pt, g[1], ph, g[2], pw).permute(0, 2, 4, 6, 3, 5, 7, 1)
        return x.reshape(B, g[0] * g[1] * g[2], -1), g

    def _forward_one(self, video, grid, temb, text):
        """video: [1, Nv, C]; temb: fp32 [1, C]; text: [1, L, text_dim] (valid tokens only)."""
        Nv, L = video.shape[1], text.shape[1]
        joint = torch.cat((video, self.text_embedder(text).to(video.dtype)), dim=1)
        cos, sin = rope_tables(joint_position_ids(L, *grid, video.device), self.config.axes_dims, self.config.rope_theta)
        S = Nv + L
        P, r, pad = 1, 0, 0
        g = self.ulysses_group
        if g is not None and dist.is_initialized() and dist.get_world_size(g) > 1:
            P, r = dist.get_world_size(g), dist.get_rank(g)
            pad = (-S) % P
            if pad:
                joint = F.pad(joint, (0, 0, 0, pad))
                cos, sin = F.pad(cos, (0, 0, 0, pad), value=1.0), F.pad(sin, (0, 0, 0, pad))
            n = (S + pad) // P
            joint, cos, sin = joint[:, r * n : (r + 1) * n], cos[r * n : (r + 1) * n], sin[r * n : (r + 1) * n]
        local = joint.shape[1]
        valid = max(0, min(local, S - r * local)) if pad else None
        silu_t = F.silu(temb)
        tm, om = self.time_modulation[1], self.norm_out_modulation[1]
        temb6 = F.linear(silu_t, tm.weight.float(), tm.bias.float())
        joint = joint.contiguous()
        cos, sin = cos.contiguous(), sin.contiguous()
        for blk in self.blocks:
            joint = blk(joint, temb6, cos, sin, S if P > 1 or pad else None, valid)
        fm = F.linear(silu_t, om.weight.float(), om.bias.float()).view(1, 2, -1)
        h = TF.layernorm_modulate(joint, fm[:, 0:1], fm[:, 1:2], eps=self.config.norm_eps)
        out = TF.linear(h, self.proj_out.weight, self.proj_out.bias)
        if P > 1:
            parts = [torch.empty_like(out) for _ in range(P)]
            dist.all_gather(parts, out.contiguous(), group=g)
            out = torch.cat(parts, dim=1)
        return out[:, :Nv]

    @torch.no_grad()
    def forward(self, hidden_states, timestep, encoder_hidden_states, encoder_attention_mask=None, **_unused):
        """hidden_states: [B, C, F, H, W]; timestep: [B]; encoder_hidden_states: [B, L, text_dim] -> [B, C, F, H, W]."""
        B, _, Fr, Hh, Ww = hidden_states.shape
        patches, grid = self._patchify(hidden_states.to(self.patch_embedder.weight.dtype))
        video = TF.linear(patches, self.patch_embedder.weight, self.patch_embedder.bias)
        temb = self.time_embedder(timestep.to(hidden_states.device).reshape(-1).expand(B) if timestep.numel() == 1
                                  else timestep.to(hidden_states.device))  # fmt: skip
        if encoder_attention_mask is None:
            lens = [encoder_hidden_states.shape[1]] * B
        else:
            lens = [int(v) for v in encoder_attention_mask.bool().sum(-1).tolist()]
        outs = []
        for i in range(B):
            text = encoder_hidden_states[i : i + 1, : lens[i]].to(video.dtype)
            outs.append(self._forward_one(video[i : i + 1], grid, temb[i : i + 1], text))
        out = torch.cat(outs, dim=0)
        pt, ph, pw = self.patch_size
        out = out.reshape(B, *grid, pt, ph, pw, self.out_channels).permute(0, 7, 1, 4, 2, 5, 3, 6)
        return out.reshape(B, self.out_channels, Fr, Hh, Ww)

    @staticmethod
    def state_dict_converter():
        return LingBotVideoStateDictConverter()


class LingBotVideoMoeTransformer3DModel(LingBotVideoTransformer3DModel):
    """Same class with `num_experts > 0`; kept as a separate name for checkpoint detection."""


def infer_lingbot_video_config(sd: dict) -> dict:
    C = sd["patch_embedder.weight"].shape[0]
    depth = 1 + max(int(k.split(".")[1]) for k in sd if k.startswith("blocks."))
    head_dim = sd["blocks.0.attn.norm_q.weight"].shape[0]
    cfg = dict(hidden_size=C, num_attention_heads=C // head_dim, depth=depth, text_dim=sd["text_embedder.linear_1.weight"].shape[1],
               freq_dim=sd["time_embedder.linear_1.weight"].shape[1], qkv_bias="blocks.0.attn.to_q.bias" in sd,
               out_bias="blocks.0.attn.to_out.bias" in sd, patch_embed_bias="patch_embedder.bias" in sd,
               timestep_mlp_bias="time_embedder.linear_1.bias" in sd)  # fmt: skip
    dense = [k for k in sd if k.endswith("ffn.gate_proj.weight")]
    if dense:
        cfg["intermediate_size"] = sd[dense[0]].shape[0]
    routers = [k for k in sd if k.endswith("ffn.router.weight")]
    if routers:
        first = routers[0].rsplit(".router.weight", 1)[0]
        cfg.update(num_experts=sd[routers[0]].shape[0], moe_intermediate_size=sd[first + ".experts.w1"].shape[1],
                   n_shared_experts=(sd[first + ".shared_experts.gate_proj.weight"].shape[0] // sd[first + ".experts.w1"].shape[1]
                                     if first + ".shared_experts.gate_proj.weight" in sd else 0))  # fmt: skip
        sparse_layers = sorted(int(k.split(".")[1]) for k in routers)
        cfg["mlp_only_layers"] = tuple(i for i in range(depth) if i not in sparse_layers)
    return cfg


class LingBotVideoStateDictConverter:
    def from_diffusers(self, sd: dict):
        return sd, infer_lingbot_video_config(sd)

    from_official = from_diffusers


def _register() -> None:
    from telefuser_b200.core.model_registry import register_architecture

    register_architecture("lingbot_video_transformer", LingBotVideoTransformer3DModel,
                          lambda: LingBotVideoTransformer3DModel(LingBotVideoConfig.preset("dense-1.3b")))  # fmt: skip
    register_architecture("lingbot_video_moe_transformer", LingBotVideoMoeTransformer3DModel,
                          lambda: LingBotVideoMoeTransformer3DModel(LingBotVideoConfig.preset("moe-30b-a3b")))  # fmt: skip


_register()
