"""Wan2.1 / Wan2.2 video DiT (T2V, I2V, TI2V, FLF2V; 1.3B / 5B / 14B).

Same architecture and state-dict key layout as the reference's ``WanModel``
(``telefuser/models/wan_video_dit.py:351-453,456-1219``) so the published
safetensors checkpoints load unchanged, but the forward is laid out for the
sm_100a kernel set:

* one fused QKV GEMM (q/k/v weights are views of one [3*dim, dim] buffer),
* RMSNorm(q), RMSNorm(k) and 3-D RoPE in a single in-place pass over the fused buffer,
* tcgen05 flash attention reading q/k/v straight from that buffer,
* output / FFN-down projections with ``x + gate * y`` folded into the GEMM epilogue,
* LayerNorm + AdaLN modulation in one pass, fp32 modulation tables computed once
  per forward for all blocks.

On CPU tensors every op falls back to its fp32 PyTorch reference, which is what
the gloo sequence-parallel tests run.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn

from telefuser_b200.core.base_model import BaseModel
from telefuser_b200.ops import functional as TF
from telefuser_b200.parallel import mesh as pmesh
from telefuser_b200.parallel import shard as pshard


@dataclass
class WanModelConfig:
    dim: int = 1536
    in_dim: int = 16
    ffn_dim: int = 8960
    out_dim: int = 16
    text_dim: int = 4096
    freq_dim: int = 256
    eps: float = 1e-6
    patch_size: tuple[int, int, int] = (1, 2, 2)
    num_heads: int = 12
    num_layers: int = 30
    has_image_input: bool = False
    has_image_pos_emb: bool = False

    @classmethod
    def preset(cls, name: str) -> "WanModelConfig":
        presets = {
            "wan2.1-t2v-1.3b": dict(dim=1536, ffn_dim=8960, num_heads=12, num_layers=30),
            "wan2.1-t2v-14b": dict(dim=5120, ffn_dim=13824, num_heads=40, num_layers=40),
            "wan2.1-i2v-14b": dict(dim=5120, ffn_dim=13824, num_heads=40, num_layers=40, in_dim=36,
                                   has_image_input=True),  # fmt: skip
            "wan2.2-ti2v-5b": dict(dim=3072, ffn_dim=14336, num_heads=24, num_layers=30, in_dim=48, out_dim=48),
            "tiny": dict(dim=128, ffn_dim=512, num_heads=4, num_layers=2, text_dim=256),
        }
        return cls(**presets[name.lower()])


def sinusoidal_embedding_1d(dim: int, position: torch.Tensor) -> torch.Tensor:
    half = dim // 2
    freqs = torch.pow(10000.0, -torch.arange(half, dtype=torch.float64, device=position.device) / half)
    ang = torch.outer(position.to(torch.float64), freqs)
    return torch.cat([ang.cos(), ang.sin()], dim=1).float()


def rope_angles_1d(dim: int, end: int = 1024, theta: float = 10000.0) -> torch.Tensor:
    """Angles [end, dim/2] (float64) of the 1-D rotary table."""
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2)[: dim // 2].double() / dim))
    return torch.outer(torch.arange(end, dtype=torch.float64), inv)


def rope_tables_3d(head_dim: int, grid: tuple[int, int, int], device, frame_start: int = 0, frame_step: int = 1):
    """cos/sin [F*H*W, head_dim/2] fp32 for a (frames, height, width) token grid.

    The head dim is split as ``d - 2*(d//3)`` (frames), ``d//3`` (height),
    ``d//3`` (width), as in the reference (wan_video_dit.py:60-97, 1176-1190).
    """
    f, h, w = grid
    d_hw = head_dim // 3
    d_f = head_dim - 2 * d_hw
    a_f = rope_angles_1d(d_f)[frame_start : frame_start + frame_step * f : frame_step]
    a_h = rope_angles_1d(d_hw)[:h]
    a_w = rope_angles_1d(d_hw)[:w]
    ang = torch.cat(
        [
            a_f.view(f, 1, 1, -1).expand(f, h, w, -1),
            a_h.view(1, h, 1, -1).expand(f, h, w, -1),
            a_w.view(1, 1, w, -1).expand(f, h, w, -1),
        ],
        dim=-1,
    ).reshape(f * h * w, -1)
    return ang.cos().float().to(device).contiguous(), ang.sin().float().to(device).contiguous()


class RMSNormWeight(nn.Module):
    """Holds the RMSNorm scale; the normalisation itself runs inside fused kernels."""

    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x):
        return TF.rmsnorm_reference(x, self.weight, self.eps)


class AffineLayerNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6, elementwise_affine: bool = True):
        super().__init__()
        self.eps = eps
        if elementwise_affine:
            self.weight = nn.Parameter(torch.ones(dim))
            self.bias = nn.Parameter(torch.zeros(dim))
        else:
            self.register_parameter("weight", None)
            self.register_parameter("bias", None)

    def forward(self, x, shift=None, scale=None):
        return TF.layernorm_modulate(x, shift, scale, self.weight, self.bias, self.eps)


def _rows_adjacent(ts: list[torch.Tensor]) -> bool:
    """True if the contiguous tensors `ts` follow one another in one storage without gaps."""
    base = ts[0].untyped_storage().data_ptr()
    nxt = ts[0].data_ptr()
    for t in ts:
        if not t.is_contiguous() or t.untyped_storage().data_ptr() != base or t.data_ptr() != nxt:
            return False
        nxt += t.numel() * t.element_size()
    return True


def _fuse_linear_weights(linears: list[nn.Linear]):
    """Re-homes the weights/biases of `linears` as row slices of one buffer; returns (W, b)."""
    w0 = linears[0].weight
    n = [lin.weight.shape[0] for lin in linears]
    if _rows_adjacent([lin.weight.data for lin in linears]) and (
            linears[0].bias is None or _rows_adjacent([lin.bias.data for lin in linears])):  # fmt: skip
        # Already row slices of one buffer (e.g. re-homed by the weight-sharding wrapper): view, no copy.
        W = torch.as_strided(w0.data, (sum(n), w0.shape[1]), (w0.shape[1], 1))
        b = torch.as_strided(linears[0].bias.data, (sum(n),), (1,)) if linears[0].bias is not None else None
        return _with_fused_scale(W, linears), b
    W = torch.empty(sum(n), w0.shape[1], dtype=w0.dtype, device=w0.device)
    b = None
    if linears[0].bias is not None:
        b = torch.empty(sum(n), dtype=linears[0].bias.dtype, device=w0.device)
    o = 0
    for lin, k in zip(linears, n):
        W[o : o + k].copy_(lin.weight.data)
        lin.weight.data = W[o : o + k]
        if b is not None:
            b[o : o + k].copy_(lin.bias.data)
            lin.bias.data = b[o : o + k]
        o += k
    return _with_fused_scale(W, linears), b


def _with_fused_scale(W: torch.Tensor, linears: list[nn.Linear]) -> torch.Tensor:
    """Quantised parts carry their scales as tags on the weight (`tfb_scale` per output channel for e4m3 / int8, tiled
    block scales for MXFP8 / NVFP4, block maxima for NF4); the fused view gets the matching concatenation."""
    mx = [getattr(lin.weight, "tfb_mx_sf", None) for lin in linears]
    if all(s is not None for s in mx):
        # block-scaled weights: the scale tiles cover 128 output rows each, so they concatenate tile-wise when
        # every part is a whole number of tiles, and through the row-major form otherwise
        mx = [s.to(W.device) for s in mx]
        if all(lin.weight.shape[0] % 128 == 0 for lin in linears):
            W.tfb_mx_sf = torch.cat(mx, dim=0).contiguous()
        else:
            rows = [TF.mx_untile_scales(s, lin.weight.shape[0]) for s, lin in zip(mx, linears)]
            W.tfb_mx_sf = TF.mx_tile_scales(torch.cat(rows, dim=0))
        return W
    f4 = [getattr(lin.weight, "tfb_nvfp4_sf", None) for lin in linears]
    if all(s is not None for s in f4):
        # NVFP4 parts keep their own tensor scale: the fused view carries one global scale per output row
        W.tfb_nvfp4_sf = torch.cat([s.to(W.device) for s in f4], dim=0).contiguous()
        W.tfb_nvfp4_global = torch.cat([lin.weight.tfb_nvfp4_global.to(W.device).reshape(1).expand(lin.weight.shape[0])
                                        for lin in linears]).contiguous()  # fmt: skip
        return W
    nf4 = [getattr(lin.weight, "tfb_nf4_absmax", None) for lin in linears]
    if all(s is not None for s in nf4):
        # NF4 blocks run over the flattened weight: parts that are whole numbers of blocks concatenate as they are
        block = getattr(linears[0].weight, "tfb_nf4_block", 64)
        if any((lin.weight.numel() * 2) % block for lin in linears):
            raise ValueError(f"NF4 weights of {[tuple(lin.weight.shape) for lin in linears]} packed bytes do not end on "
                             f"a {block}-value block: they cannot share one fused matrix")
        W.tfb_nf4_absmax, W.tfb_nf4_block = torch.cat([s.to(W.device) for s in nf4]).contiguous(), block
        return W
    scales = [TF.fp8_weight_scale(lin.weight) for lin in linears]
    if all(s is not None for s in scales):
        W.tfb_scale = torch.cat([s.reshape(-1) for s in scales]).contiguous()
    return W


class WanSelfAttention(nn.Module):
    def __init__(self, dim: int, num_heads: int, eps: float = 1e-6):
        super().__init__()
        self.dim, self.num_heads, self.head_dim = dim, num_heads, dim // num_heads
        self.q = nn.Linear(dim, dim)
        self.k = nn.Linear(dim, dim)
        self.v = nn.Linear(dim, dim)
        self.o = nn.Linear(dim, dim)
        self.norm_q = RMSNormWeight(dim, eps)
        self.norm_k = RMSNormWeight(dim, eps)
        self._qkv = None
        self.attention_config = None  # set through the model's `set_attention_config`
        self.sparse_ctx = None  # (RadialMaskMap, decay factor, dense?) set by the model for every forward

    def fused_qkv(self):
        w = self.q.weight
        if self._qkv is None or self._qkv[0].device != w.device or self._qkv[0].dtype != w.dtype or \
                self._qkv[0].data_ptr() != w.data_ptr():  # fmt: skip
            self._qkv = _fuse_linear_weights([self.q, self.k, self.v])
        return self._qkv

    def forward(self, x, cos, sin, usp: bool = False):
        B, S, C = x.shape
        H, D = self.num_heads, self.head_dim
        W, b = self.fused_qkv()
        qkv = TF.linear(x, W, b)  # [B, S, 3C]
        q, k, v = qkv[..., :C], qkv[..., C : 2 * C], qkv[..., 2 * C :]
        TF.rmsnorm_rope_(q, self.norm_q.weight, H, cos, sin, self.norm_q.eps, x2=k, weight2=self.norm_k.weight)
        q, k, v = (t.unflatten(-1, (H, D)) for t in (q, k, v))
        if usp:
            from telefuser_b200.parallel.ring import long_context_attention

            o = long_context_attention(q, k, v)  # Ulysses, ring or both, by the mesh's SP degrees
        elif self.sparse_ctx is not None and not self.sparse_ctx[2]:
            from telefuser_b200.ops.sparse_attention import radial_attention

            o = radial_attention(q, k, v, self.sparse_ctx[0], self.sparse_ctx[1])
        else:
            cfg = self.attention_config
            o = TF.attention(q, k, v, quant="int8" if cfg is not None and cfg.attn_impl.quantized() else None)
        return o.reshape(B, S, C)


class WanCrossAttention(nn.Module):
    def __init__(self, dim: int, num_heads: int, eps: float = 1e-6, has_image_input: bool = False):
        super().__init__()
        self.dim, self.num_heads, self.head_dim = dim, num_heads, dim // num_heads
        self.q = nn.Linear(dim, dim)
        self.k = nn.Linear(dim, dim)
        self.v = nn.Linear(dim, dim)
        self.o = nn.Linear(dim, dim)
        self.norm_q = RMSNormWeight(dim, eps)
        self.norm_k = RMSNormWeight(dim, eps)
        self.has_image_input = has_image_input
        if has_image_input:
            self.k_img = nn.Linear(dim, dim)
            self.v_img = nn.Linear(dim, dim)
            self.norm_k_img = RMSNormWeight(dim, eps)
        self._kv = None

    def fused_kv(self):
        w = self.k.weight
        if self._kv is None or self._kv[0].device != w.device or self._kv[0].dtype != w.dtype or \
                self._kv[0].data_ptr() != w.data_ptr():  # fmt: skip
            self._kv = _fuse_linear_weights([self.k, self.v])
        return self._kv

    def forward(self, x, context):
        B, S, C = x.shape
        H, D = self.num_heads, self.head_dim
        if self.has_image_input:
            img, ctx = context[:, :257], context[:, 257:]
        else:
            img, ctx = None, context
        q = TF.linear(x, self.q.weight, self.q.bias)
        TF.rmsnorm_rope_(q, self.norm_q.weight, H, eps=self.norm_q.eps)
        Wkv, bkv = self.fused_kv()
        kv = TF.linear(ctx, Wkv, bkv)
        k, v = kv[..., :C], kv[..., C:]
        TF.rmsnorm_rope_(k, self.norm_k.weight, H, eps=self.norm_k.eps)
        qh = q.unflatten(-1, (H, D))
        o = TF.attention(qh, k.unflatten(-1, (H, D)), v.unflatten(-1, (H, D)))
        if img is not None:
            ki = TF.linear(img, self.k_img.weight, self.k_img.bias)
            TF.rmsnorm_rope_(ki, self.norm_k_img.weight, H, eps=self.norm_k_img.eps)
            vi = TF.linear(img, self.v_img.weight, self.v_img.bias)
            o = o + TF.attention(qh, ki.unflatten(-1, (H, D)), vi.unflatten(-1, (H, D)))
        return o.reshape(B, S, C)


class WanBlock(nn.Module):
    def __init__(self, has_image_input: bool, dim: int, num_heads: int, ffn_dim: int, eps: float = 1e-6):
        super().__init__()
        self.dim, self.num_heads, self.ffn_dim = dim, num_heads, ffn_dim
        self.self_attn = WanSelfAttention(dim, num_heads, eps)
        self.cross_attn = WanCrossAttention(dim, num_heads, eps, has_image_input)
        self.norm1 = AffineLayerNorm(dim, eps, elementwise_affine=False)
        self.norm2 = AffineLayerNorm(dim, eps, elementwise_affine=False)
        self.norm3 = AffineLayerNorm(dim, eps)
        self.ffn = nn.Sequential(nn.Linear(dim, ffn_dim), nn.GELU(approximate="tanh"), nn.Linear(ffn_dim, dim))
        self.modulation = nn.Parameter(torch.randn(1, 6, dim) / dim**0.5)

    def forward(self, x, context, mod, cos, sin, usp: bool = False):
        """x: [B, S, C]; mod: fp32 [B, S|1, 6, C] = block modulation + time projection."""
        shift_msa, scale_msa, gate_msa, shift_mlp, scale_mlp, gate_mlp = (mod[:, :, i] for i in range(6))
        h = self.norm1(x, shift_msa, scale_msa)
        a = self.self_attn(h, cos, sin, usp)
        x = TF.linear(a, self.self_attn.o.weight, self.self_attn.o.bias, residual=x, gate=gate_msa)
        h = self.norm3(x)
        c = self.cross_attn(h, context)
        x = TF.linear(c, self.cross_attn.o.weight, self.cross_attn.o.bias, residual=x)
        h = self.norm2(x, shift_mlp, scale_mlp)
        h = TF.linear(h, self.ffn[0].weight, self.ffn[0].bias, act="gelu_tanh")
        if getattr(self, "tp_size", 1) > 1:  # FFN split over TP ranks: partial sums meet before the gate
            from telefuser_b200.parallel import mesh as pmesh
            from telefuser_b200.parallel.tp import all_reduce_sum

            B, S, C = x.shape
            if pmesh.get_mesh().fused and x.is_cuda and B == 1 and S % self.tp_size == 0:
                # row-parallel GEMM whose epilogue scatters the partial tiles to the row owners over NVLink
                from telefuser_b200.parallel.symm import get_workspace
                from telefuser_b200.parallel.tp_fused import gemm_all_reduce

                ws = get_workspace(self.tp_group, 2 * S * C * 2 + (1 << 20), tag="tp")
                y = gemm_all_reduce(h.reshape(S, -1), self.ffn[2].weight, self.ffn[2].bias, residual=x.reshape(S, C),
                                    gate=gate_mlp.reshape(-1, C), group=self.tp_group, ws=ws)  # fmt: skip
                return y.view(B, S, C)
            y = all_reduce_sum(TF.linear(h, self.ffn[2].weight, self.ffn[2].bias), self.tp_group)
            return TF.gated_residual(x, y, gate_mlp)
        x = TF.linear(h, self.ffn[2].weight, self.ffn[2].bias, residual=x, gate=gate_mlp)
        return x


class WanImageMLP(nn.Module):
    def __init__(self, in_dim: int, out_dim: int, has_pos_emb: bool = False):
        super().__init__()
        self.proj = nn.Sequential(nn.LayerNorm(in_dim), nn.Linear(in_dim, in_dim), nn.GELU(),
                                  nn.Linear(in_dim, out_dim), nn.LayerNorm(out_dim))  # fmt: skip
        self.has_pos_emb = has_pos_emb
        if has_pos_emb:
            self.emb_pos = nn.Parameter(torch.zeros(1, 514, 1280))

    def forward(self, x):
        if self.has_pos_emb:
            x = x + self.emb_pos.to(dtype=x.dtype, device=x.device)
        return self.proj(x)


class WanHead(nn.Module):
    def __init__(self, dim: int, out_dim: int, patch_size, eps: float):
        super().__init__()
        self.norm = AffineLayerNorm(dim, eps, elementwise_affine=False)
        self.head = nn.Linear(dim, out_dim * math.prod(patch_size))
        self.modulation = nn.Parameter(torch.randn(1, 2, dim) / dim**0.5)

    def forward(self, x, t):
        """t: fp32 [B, S|1, C]."""
        mod = self.modulation.float().unsqueeze(0) + t.unsqueeze(2)  # [B, S|1, 2, C]
        h = self.norm(x, mod[:, :, 0], mod[:, :, 1])
        return TF.linear(h, self.head.weight, self.head.bias)


class WanModel(BaseModel):
    def __init__(self, dim=1536, in_dim=16, ffn_dim=8960, out_dim=16, text_dim=4096, freq_dim=256, eps=1e-6,
                 patch_size=(1, 2, 2), num_heads=12, num_layers=30, has_image_input=False,
                 has_image_pos_emb=False):  # fmt: skip
        super().__init__()
        self.dim, self.freq_dim, self.num_heads, self.num_layers = dim, freq_dim, num_heads, num_layers
        self.in_dim, self.out_dim = in_dim, out_dim
        self.head_dim = dim // num_heads
        self.patch_size = tuple(patch_size)
        self.has_image_input = has_image_input
        self.has_image_pos_emb = has_image_pos_emb
        self.patch_embedding = nn.Conv3d(in_dim, dim, kernel_size=self.patch_size, stride=self.patch_size)
        self.text_embedding = nn.Sequential(nn.Linear(text_dim, dim), nn.GELU(approximate="tanh"), nn.Linear(dim, dim))
        self.time_embedding = nn.Sequential(nn.Linear(freq_dim, dim), nn.SiLU(), nn.Linear(dim, dim))
        self.time_projection = nn.Sequential(nn.SiLU(), nn.Linear(dim, dim * 6))
        self.blocks = nn.ModuleList(
            [WanBlock(has_image_input, dim, num_heads, ffn_dim, eps) for _ in range(num_layers)]
        )
        self.head = WanHead(dim, out_dim, self.patch_size, eps)
        if has_image_input:
            self.img_emb = WanImageMLP(1280, dim, has_pos_emb=has_image_pos_emb)
        self.dtype = torch.bfloat16
        self.pp_start_idx, self.pp_end_idx = 0, num_layers
        self._rope_cache: dict = {}
        self._mod_stack = None

    @classmethod
    def from_config(cls, cfg: WanModelConfig) -> "WanModel":
        return cls(**cfg.__dict__)

    # ---- pieces ------------------------------------------------------------
    def rope(self, grid, device, frame_start=0, frame_step=1):
        key = (tuple(grid), str(device), frame_start, frame_step)
        if key not in self._rope_cache:
            if len(self._rope_cache) > 8:
                self._rope_cache.clear()
            self._rope_cache[key] = rope_tables_3d(self.head_dim, grid, device, frame_start, frame_step)
        return self._rope_cache[key]

    def patchify(self, x):
        B, C, F, H, W = x.shape
        pt, ph, pw = self.patch_size
        f, h, w = F // pt, H // ph, W // pw
        tokens = x.reshape(B, C, f, pt, h, ph, w, pw).permute(0, 2, 4, 6, 1, 3, 5, 7).reshape(B, f * h * w, -1)
        wgt = self.patch_embedding.weight.reshape(self.dim, -1)
        return TF.linear(tokens.to(wgt.dtype), wgt, self.patch_embedding.bias), (f, h, w)

    def unpatchify(self, x, grid):
        f, h, w = grid
        pt, ph, pw = self.patch_size
        B = x.shape[0]
        x = x.reshape(B, f, h, w, pt, ph, pw, self.out_dim).permute(0, 7, 1, 4, 2, 5, 3, 6)
        return x.reshape(B, self.out_dim, f * pt, h * ph, w * pw)

    def time_embed(self, timestep, seq_len):
        """Returns (t [B, S|1, C] fp32, t_mod [B, S|1, 6, C] fp32)."""
        B = timestep.shape[0]
        flat = timestep.flatten()
        e = sinusoidal_embedding_1d(self.freq_dim, flat)
        w0, w2 = self.time_embedding[0], self.time_embedding[2]
        e = torch.nn.functional.silu(torch.nn.functional.linear(e, w0.weight.float(), w0.bias.float()))
        e = torch.nn.functional.linear(e, w2.weight.float(), w2.bias.float())
        wp = self.time_projection[1]
        tm = torch.nn.functional.linear(torch.nn.functional.silu(e), wp.weight.float(), wp.bias.float())
        if timestep.dim() == 1:
            return e.view(B, 1, self.dim), tm.view(B, 1, 6, self.dim)
        return e.view(B, seq_len, self.dim), tm.view(B, seq_len, 6, self.dim)

    def block_modulations(self, t_mod):
        """fp32 [L, B, S|1, 6, C]: every block's modulation table plus the time projection."""
        if self._mod_stack is None or self._mod_stack.device != t_mod.device:
            self._mod_stack = torch.stack([b.modulation.detach().float() for b in self.blocks]).to(t_mod.device)
        if t_mod.shape[1] > 1:  # per-token modulation is large: add per block instead
            return None
        return self._mod_stack.unsqueeze(1) + t_mod.unsqueeze(0)  # [L,1,1,6,C] + [1,B,1,6,C]

    def embed_text(self, context):
        te = self.text_embedding
        h = TF.linear(context.to(self.dtype), te[0].weight, te[0].bias, act="gelu_tanh")
        return TF.linear(h, te[2].weight, te[2].bias)

    def enable_pp(self, start: int | None = None, end: int | None = None, pp_group=None) -> None:
        from telefuser_b200.parallel.pp import PipelineP2PComm

        if pp_group is None and self.device_mesh is not None and self.device_mesh.size("pp") > 1:
            pp_group = self.device_mesh.group("pp")
        self.pp_comm = PipelineP2PComm(pp_group)
        if start is None or end is None:
            start, end = self.pp_comm.get_stage_indices(self.num_layers)
        self.pp_flag = True
        self.pp_start_idx, self.pp_end_idx = start, end

    def forward_blocks(self, x, context, t_mod, cos, sin, start=None, end=None):
        mods = self.block_modulations(t_mod)
        start = self.pp_start_idx if start is None else start
        end = self.pp_end_idx if end is None else end
        offload = getattr(self, "async_offload_manager", None) if self.async_offload_flag else None
        for i in range(start, end):
            blk = self.blocks[i]
            mod = mods[i] if mods is not None else blk.modulation.float().unsqueeze(0) + t_mod
            if offload is not None:
                offload.before_layer(i)
            x = blk(x, context, mod, cos, sin, self.usp_flag)
            if offload is not None:
                offload.after_layer(i)
        return x

    # ---- forward -------------------------------------------------------------
    @torch.no_grad()
    def enable_radial_attention(self, dense_layers: int = 0, dense_timesteps: int = 40, decay_factor: float = 1.0):
        """Radial block-sparse self-attention outside the dense warm-up layers / steps
        (telefuser/models/wan_video_dit.py:975-1010)."""
        from telefuser_b200.core.config import AttentionConfig

        self.set_attention_config(AttentionConfig.radial_attention(dense_timesteps, dense_layers, decay_factor))

    def _set_sparse_context(self, grid, numeral_timestep: int) -> None:
        sc = getattr(self.attention_config, "sparse_config", None) if self.attention_config is not None else None
        if sc is None or sc.sparse_impl != "radial" or self.usp_flag:
            for blk in self.blocks:
                blk.self_attn.sparse_ctx = None
            return
        from telefuser_b200.ops.sparse_attention import RadialMaskMap

        f, h, w = grid
        key = (f, h * w)
        if getattr(self, "_radial_key", None) != key:
            self._radial_map, self._radial_key = RadialMaskMap(f * h * w, f, "wan"), key
        for i, blk in enumerate(self.blocks):
            blk.self_attn.sparse_ctx = (self._radial_map, sc.decay_factor, sc.should_use_dense(numeral_timestep, i))

    def forward(self, x, timestep, context, clip_feature=None, cond_flag=True, add_condition=None,
                freq_start_idx=0, freq_interval=1, numeral_timestep: int = 0, **_unused):  # fmt: skip
        """x: [B, C, F, H, W] latents; timestep: [B] or [B, S]; context: [B, L, text_dim]."""
        t, t_mod = self.time_embed(timestep.to(x.device), None if timestep.dim() == 1 else timestep.shape[1])
        context = self.embed_text(context)
        if self.has_image_input and clip_feature is not None:
            context = torch.cat([self.img_emb(clip_feature.to(self.dtype)), context], dim=1)
        x, grid = self.patchify(x)
        self._set_sparse_context(grid, numeral_timestep)
        if add_condition is not None:
            x = x + add_condition
        seq_len = x.shape[1]
        cos, sin = self.rope(grid, x.device, freq_start_idx, freq_interval)
        if self.usp_flag:
            x, t_mod, t, cos, sin = pshard.sequence_parallel_shard([x, t_mod, t, cos, sin], [1, 1, 1, 0, 0])
        ori_x = x
        if self.pp_flag and self.pp_comm.world_size > 1:
            # Each stage embeds for itself; only the token stream crosses the stage boundary.
            if not self.pp_comm.is_first:
                x = self.pp_comm.recv_latent(tuple(x.shape), x.dtype, x.device)
            x = self.forward_blocks(x, context, t_mod, cos, sin)
            if not self.pp_comm.is_last:
                self.pp_comm.send_latent(x)
                return None
        else:
            cache = self.feature_cache
            if cache.should_compute(cond_flag):
                x = self.forward_blocks(x, context, t_mod, cos, sin)
                cache.update(x, ori_x, cond_flag)
            else:
                x = cache.approximate(x, cond_flag)
        x = self.head(x, t)
        if self.usp_flag:
            (x,) = pshard.sequence_parallel_unshard([x], [1], [seq_len])
        return self.unpatchify(x, grid)

    def enable_quant(self, quant=None) -> int:
        """Quantised block projections (attention q/k/v/o and both FFN layers): per-token x per-channel FP8 by default,
        block-scaled MXFP8 for `QuantType.MXFP8` ("mxfp8"), integer W8A8 for `QuantType.INT8` ("int8"), NVFP4 or NF4
        weight storage for "nvfp4" / "nf4"; embeddings, the head and all norms / modulation tables stay in bf16 /
        fp32. A `QuantConfig` adds its `skip_modules` to that list. Returns the number of layers converted."""
        from telefuser_b200.ops.quant import quantize_model_

        return quantize_model_(self, quant, ("blocks.*",), ("head", "time_embedding", "time_projection", "patch_embedding",
                                                            "text_embedding", "img_emb"))  # fmt: skip

    # ---- parallel plans --------------------------------------------------------
    def get_fsdp_module_names(self) -> list[str]:
        return ["blocks"]

    def get_tp_plan(self) -> dict[str, str]:
        """FFN column / row split (the FFN holds 2/3 of a block's weights). The attention projections
        stay replicated: q/k RMSNorm runs over the full hidden width, which a head split would cut.
        The reference plan (telefuser/models/wan_video_dit.py:1228-1304) lists the attention
        projections as well but is not wired to any pipeline."""
        return {"blocks.*.ffn.0": "colwise", "blocks.*.ffn.2": "rowwise", "blocks.*": "group"}

    @staticmethod
    def state_dict_converter():
        from telefuser_b200.models.wan_dit_convert import WanModelStateDictConverter

        return WanModelStateDictConverter()


def _register() -> None:
    from telefuser_b200.core.model_registry import register_architecture

    for preset in ("wan2.1-t2v-1.3b", "wan2.1-t2v-14b", "wan2.1-i2v-14b", "wan2.2-ti2v-5b"):
        register_architecture("wan_video_dit", WanModel, lambda p=preset: WanModel.from_config(WanModelConfig.preset(p)))


_register()
