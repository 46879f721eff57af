"""LiveAct speech-to-video DiT: Wan-14B I2V blocks + per-frame audio cross-attention + compressed KV memory.

The model generates latent frames chunk by chunk. Self-attention reads a per-layer, per-timestep KV memory of six
frame slots: two anchor frames, two slots that each hold five older frames compressed into one (a depth-wise
temporal convolution, or a plain mean), and the two most recent frames; keys are stored unrotated and rotated
by their slot position each time. Every latent frame cross-attends to its own 32 audio context tokens
(`SingleStreamAttention`, batched over frames) produced by `AudioProjModel` from windows of speech features, and
to text plus 257 CLIP image tokens as in Wan I2V.
Role parity: telefuser/models/liveact_dit.py:35-1213.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn

from telefuser_b200.core.base_model import BaseModel
from telefuser_b200.models.wan_dit import (AffineLayerNorm, RMSNormWeight, WanCrossAttention, WanHead, WanImageMLP,
                                           _fuse_linear_weights, rope_angles_1d, sinusoidal_embedding_1d)  # fmt: skip
from telefuser_b200.ops import functional as TF
from telefuser_b200.parallel import shard as pshard


def rope_tables(head_dim: int, f: int, h: int, w: int, start_frame: int, device):
    """fp32 (cos, sin) [f*h*w, head_dim/2]; the pair axes split d - 4*(d//6), 2*(d//6), 2*(d//6) over (t, h, w)."""
    d_hw = 2 * (head_dim // 6)
    a_t = rope_angles_1d(head_dim - 2 * d_hw)[start_frame : start_frame + f]
    a_h, a_w = rope_angles_1d(d_hw)[:h], rope_angles_1d(d_hw)[:w]
    ang = torch.cat([a_t.view(f, 1, 1, -1).expand(f, h, w, -1), a_h.view(1, h, 1, -1).expand(f, h, w, -1),
                     a_w.view(1, 1, w, -1).expand(f, h, w, -1)], dim=-1).reshape(f * h * w, -1)  # fmt: skip
    return ang.cos().float().to(device), ang.sin().float().to(device)


class SingleStreamAttention(nn.Module):
    """Every latent frame attends to its own audio tokens (frames form the batch dimension)."""

    def __init__(self, dim: int, encoder_hidden_states_dim: int, num_heads: int, qkv_bias: bool = True) -> None:
        super().__init__()
        self.dim, self.num_heads, self.head_dim = dim, num_heads, dim // num_heads
        self.q_linear = nn.Linear(dim, dim, bias=qkv_bias)
        self.kv_linear = nn.Linear(encoder_hidden_states_dim, dim * 2, bias=qkv_bias)
        self.proj = nn.Linear(dim, dim)
        self.sp_flag, self.sp_rank, self.sp_size = False, 0, 1

    def forward(self, x, encoder_hidden_states, shape, start_f: int = 0):
        """x [B, n_t*S, C]; encoder_hidden_states [1, frames, tokens, C_a] -> [B, n_t*S, C] (before the residual)."""
        enc = encoder_hidden_states.squeeze(0)
        _, n_h, n_w = shape
        S = n_h * n_w
        B0, N, C = x.shape
        n_t = N // S
        xf = x.reshape(B0 * n_t, S, C)
        H, D = self.num_heads, self.head_dim
        q = TF.linear(xf, self.q_linear.weight, self.q_linear.bias).unflatten(-1, (H, D))
        first = start_f + (self.sp_rank * n_t if self.sp_flag else 0)
        kv = TF.linear(enc[first : first + n_t].to(xf.dtype), self.kv_linear.weight, self.kv_linear.bias)
        k, v = kv[..., :C].unflatten(-1, (H, D)), kv[..., C:].unflatten(-1, (H, D))
        o = TF.attention(q, k, v).reshape(B0 * n_t, S, C)
        return TF.linear(o, self.proj.weight, self.proj.bias).reshape(B0, N, C)


class MemorySelfAttention(nn.Module):
    def __init__(self, dim: int, num_heads: int, eps: float = 1e-6, mean_memory: bool = False) -> None:
        super().__init__()
        self.dim, self.num_heads, self.head_dim, self.mean_memory = dim, num_heads, dim // num_heads, mean_memory
        self.q, self.k, self.v, self.o = (nn.Linear(dim, dim) for _ in range(4))
        self.norm_q, self.norm_k = RMSNormWeight(dim, eps), RMSNormWeight(dim, eps)
        self.memory_proj_k = nn.Conv1d(dim, dim, kernel_size=5, stride=5, groups=dim, bias=False)
        self.memory_proj_v = nn.Conv1d(dim, dim, kernel_size=5, stride=5, groups=dim, bias=False)
        self._qkv = None
        self.sp_flag = False

    def post_init(self, device=None) -> None:
        """The memory convolutions start as a plain mean over five frames."""
        nn.init.constant_(self.memory_proj_k.weight, 0.2)
        nn.init.constant_(self.memory_proj_v.weight, 0.2)

    def _compress(self, t: torch.Tensor, tokens_per_frame: int, conv: nn.Conv1d) -> torch.Tensor:
        """[B, 5*tpf, H, D]: five frames -> one frame; token (frame j, position p) sits at j*tpf + p."""
        B, N, H, D = t.shape
        if self.mean_memory:
            return t.view(B, N // 5, 5, H, D).mean(dim=2)
        # Depth-wise stride-5 convolution along the flattened token axis (output token q mixes tokens 5q .. 5q+4),
        # written as a weighted sum; under head-sharded sequence parallelism only this rank's channels take part.
        w = conv.weight.view(self.num_heads, D, 5)
        if H != self.num_heads:
            r = pshard._sp(None)[2]
            w = w[r * H : (r + 1) * H]
        return (t.view(B, N // 5, 5, H, D).permute(0, 1, 3, 4, 2) * w.to(t.dtype).view(1, 1, H, D, 5)).sum(-1)

    def compress_cache(self, k_full, v_full, k_cache, v_cache, tpf: int) -> None:
        k_cache[:, 2 * tpf : 3 * tpf] = self._compress(k_full[:, 2 * tpf : 7 * tpf], tpf, self.memory_proj_k)
        v_cache[:, 2 * tpf : 3 * tpf] = self._compress(v_full[:, 2 * tpf : 7 * tpf], tpf, self.memory_proj_v)
        k_cache[:, 3 * tpf : 4 * tpf] = self._compress(k_full[:, 7 * tpf : 12 * tpf], tpf, self.memory_proj_k)
        v_cache[:, 3 * tpf : 4 * tpf] = self._compress(v_full[:, 7 * tpf : 12 * tpf], tpf, self.memory_proj_v)
        k_cache[:, 4 * tpf : 6 * tpf] = k_full[:, 12 * tpf : 14 * tpf]
        v_cache[:, 4 * tpf : 6 * tpf] = v_full[:, 12 * tpf : 14 * tpf]

    def forward(self, x, h: int, w: int, kv_cache, start_idx: int, end_idx: int | None, tokens_per_frame: int):
        B, S, C = x.shape
        H, D = self.num_heads, self.head_dim
        wq = self.q.weight
        if self._qkv is None or self._qkv[0].data_ptr() != wq.data_ptr() or self._qkv[0].dtype != wq.dtype:
            self._qkv = _fuse_linear_weights([self.q, self.k, self.v])
        qkv = TF.linear(x, self._qkv[0], self._qkv[1])
        q, k, v = qkv[..., :C], qkv[..., C : 2 * C], qkv[..., 2 * C :]
        TF.rmsnorm_rope_(q, self.norm_q.weight, H, eps=self.norm_q.eps, x2=k, weight2=self.norm_k.weight)
        q, k, v = (t.unflatten(-1, (H, D)) for t in (q, k, v))
        group = None
        if self.sp_flag:
            from telefuser_b200.parallel import ulysses

            group = pshard._sp(None)[3]
            q, k, v = (ulysses.scatter_heads(t.contiguous(), group) for t in (q, k, v))
        k_cache, v_cache = kv_cache.load(x.device, x.dtype)
        tpf = tokens_per_frame
        if start_idx != 0:
            k_full, v_full = torch.cat([k_cache, k], dim=1), torch.cat([v_cache, v], dim=1)
        else:
            k_cache[:, : 6 * tpf], v_cache[:, : 6 * tpf] = k, v
            k_full, v_full = k_cache, v_cache
        qc, qs = rope_tables(D, q.shape[1] // tpf, h, w, start_idx // tpf, x.device)
        kc, ks = rope_tables(D, k_full.shape[1] // tpf, h, w, 0, x.device)
        rq = TF.rope_reference(q, qc, qs)
        rk = TF.rope_reference(k_full, kc, ks)
        o = TF.attention(rq, rk[:, :end_idx].contiguous(), v_full[:, :end_idx].contiguous())
        if start_idx != 0:
            self.compress_cache(k_full, v_full, k_cache, v_cache, tpf)
        kv_cache.store(k_cache, v_cache)
        if self.sp_flag:
            o = ulysses.gather_heads(o, group)
        return o.reshape(B, -1, C)


class LiveActBlock(nn.Module):
    def __init__(self, dim: int, ffn_dim: int, num_heads: int, cross_attn_norm: bool = False, eps: float = 1e-6,
                 output_dim: int = 768, norm_input_visual: bool = True, mean_memory: bool = False) -> None:  # fmt: skip
        super().__init__()
        self.norm1 = AffineLayerNorm(dim, eps, elementwise_affine=False)
        self.self_attn = MemorySelfAttention(dim, num_heads, eps, mean_memory)
        self.norm3 = AffineLayerNorm(dim, eps, elementwise_affine=True) if cross_attn_norm else None
        self.cross_attn = WanCrossAttention(dim, num_heads, eps, has_image_input=True)
        self.norm2 = AffineLayerNorm(dim, eps, elementwise_affine=False)
        self.ffn = nn.Sequential(nn.Linear(dim, ffn_dim), nn.GELU(approximate="tanh"), nn.Linear(ffn_dim, dim))
        self.modulation = nn.Parameter(torch.randn(1, 6, dim) / dim**0.5)
        self.audio_cross_attn = SingleStreamAttention(dim, output_dim, num_heads, qkv_bias=True)
        self.norm_x = AffineLayerNorm(dim, eps, elementwise_affine=True) if norm_input_visual else None

    def forward(self, x, e, f, h, w, context, kv_cache, start_idx, end_idx, audio_embedding=None, skip_audio=False,
                tokens_per_frame=None):  # fmt: skip
        """e: fp32 [B, 6, C]."""
        mod = self.modulation.float() + e
        sh1, sc1, g1, sh2, sc2, g2 = (mod[:, i : i + 1] for i in range(6))
        tpf = tokens_per_frame or h * w
        a = self.self_attn(self.norm1(x, sh1, sc1), h, w, kv_cache, start_idx, end_idx, tpf)
        x = TF.linear(a, self.self_attn.o.weight, self.self_attn.o.bias, residual=x, gate=g1)
        c = self.cross_attn(x if self.norm3 is None else self.norm3(x), context)
        x = TF.linear(c, self.cross_attn.o.weight, self.cross_attn.o.bias, residual=x)
        if not skip_audio:
            start_f = start_idx // tpf
            xa = self.audio_cross_attn(x if self.norm_x is None else self.norm_x(x), audio_embedding, (f, h, w), start_f)
            if start_f == 0 and (not self.audio_cross_attn.sp_flag or self.audio_cross_attn.sp_rank == 0):
                xa[:, :tpf] = 0  # the reference frame is not driven by audio
            x = x + xa
        hdn = TF.linear(self.norm2(x, sh2, sc2), self.ffn[0].weight, self.ffn[0].bias, act="gelu_tanh")
        return TF.linear(hdn, self.ffn[2].weight, self.ffn[2].bias, residual=x, gate=g2)


class AudioProjModel(nn.Module):
    def __init__(self, seq_len: int = 5, seq_len_vf: int = 12, blocks: int = 12, channels: int = 768,
                 intermediate_dim: int = 512, output_dim: int = 768, context_tokens: int = 32,
                 norm_output_audio: bool = False) -> None:  # fmt: skip
        super().__init__()
        self.context_tokens, self.output_dim = context_tokens, output_dim
        self.proj1 = nn.Linear(seq_len * blocks * channels, intermediate_dim)
        self.proj1_vf = nn.Linear(seq_len_vf * blocks * channels, intermediate_dim)
        self.proj2 = nn.Linear(intermediate_dim, intermediate_dim)
        self.proj3 = nn.Linear(intermediate_dim, context_tokens * output_dim)
        self.norm = nn.LayerNorm(output_dim) if norm_output_audio else nn.Identity()

    def forward(self, audio_embeds, audio_embeds_vf):
        """[B, 1, w, blocks, C] (first frame) and [B, n_t, w', blocks, C] -> [B, 1 + n_t, context_tokens, output_dim]."""
        B = audio_embeds.shape[0]
        a = torch.relu(self.proj1(audio_embeds.flatten(2)))
        b = torch.relu(self.proj1_vf(audio_embeds_vf.flatten(2)))
        c = torch.relu(self.proj2(torch.cat([a, b], dim=1)))
        tokens = self.proj3(c).reshape(B, -1, self.context_tokens, self.output_dim)
        return self.norm(tokens)


class LiveActDiT(BaseModel):
    def __init__(self, model_type: str = "i2v", patch_size=(1, 2, 2), text_len: int = 512, in_dim: int = 36, dim: int = 5120,
                 ffn_dim: int = 13824, freq_dim: int = 256, text_dim: int = 4096, out_dim: int = 16, num_heads: int = 40,
                 num_layers: int = 40, window_size=(-1, -1), qk_norm: bool = True, cross_attn_norm: bool = True,
                 eps: float = 1e-6, audio_window: int = 5, intermediate_dim: int = 512, output_dim: int = 768,
                 context_tokens: int = 32, vae_scale: int = 4, norm_input_visual: bool = True,
                 norm_output_audio: bool = True, weight_init: bool = True, mean_memory: bool = False,
                 clip_dim: int = 1280) -> None:  # fmt: skip
        super().__init__()
        if model_type != "i2v":
            raise ValueError("LiveAct is an image-to-video model")
        self.patch_size, self.text_len, self.dim, self.freq_dim = tuple(patch_size), text_len, dim, freq_dim
        self.out_dim, self.num_heads, self.num_layers, self.head_dim = out_dim, num_heads, num_layers, dim // num_heads
        self.audio_window, self.vae_scale, self.mean_memory = audio_window, vae_scale, mean_memory
        self.layer_name_list = ["blocks"]
        self.patch_embedding = nn.Conv3d(in_dim, dim, kernel_size=self.patch_size, stride=self.patch_size)
        self.text_embedding = nn.Sequential(nn.Linear(text_dim, dim), nn.GELU(approximate="tanh"), nn.Linear(dim, dim))
        self.time_embedding = nn.Sequential(nn.Linear(freq_dim, dim), nn.SiLU(), nn.Linear(dim, dim))
        self.time_projection = nn.Sequential(nn.SiLU(), nn.Linear(dim, dim * 6))
        self.blocks = nn.ModuleList([LiveActBlock(dim, ffn_dim, num_heads, cross_attn_norm, eps, output_dim, norm_input_visual,
                                                  mean_memory) for _ in range(num_layers)])  # fmt: skip
        self.head = WanHead(dim, out_dim, self.patch_size, eps)
        self.img_emb = WanImageMLP(clip_dim, dim)
        self.audio_proj = AudioProjModel(audio_window, audio_window + vae_scale - 1, intermediate_dim=intermediate_dim,
                                         output_dim=output_dim, context_tokens=context_tokens,
                                         norm_output_audio=norm_output_audio)  # fmt: skip
        self.dtype = torch.bfloat16
        if weight_init:
            for blk in self.blocks:
                blk.self_attn.post_init()

    # ---- switches -------------------------------------------------------------------
    def enable_usp(self) -> None:
        super().enable_usp()
        _, P, r, _ = pshard._sp(None)
        for blk in self.blocks:
            blk.self_attn.sp_flag = True
            blk.audio_cross_attn.sp_flag, blk.audio_cross_attn.sp_rank, blk.audio_cross_attn.sp_size = True, r, P

    def get_fsdp_module_names(self) -> list[str]:
        return ["blocks"]

    def set_mean_memory(self, mean_memory: bool) -> None:
        self.mean_memory = mean_memory
        for blk in self.blocks:
            blk.self_attn.mean_memory = mean_memory

    def time_embed(self, t: torch.Tensor):
        """-> (e [B, C], e0 [B, 6, C]) in fp32."""
        emb = sinusoidal_embedding_1d(self.freq_dim, t.float())
        l1, l2, pr = self.time_embedding[0], self.time_embedding[2], self.time_projection[1]
        e = F.linear(F.silu(F.linear(emb, l1.weight.float(), l1.bias.float())), l2.weight.float(), l2.bias.float())
        return e, F.linear(F.silu(e), pr.weight.float(), pr.bias.float()).unflatten(1, (6, self.dim))

    def audio_context(self, audio: torch.Tensor) -> torch.Tensor:
        """audio [B, 1 + 4*n_t, window, blocks, C] speech features per video frame -> [1, 1 + n_t, B*tokens, C_out]:
        the first frame keeps its own window; every later latent frame gathers the windows of its 4 video frames
        (left half of the first, centres of the middle ones, right half of the last)."""
        first, later = audio[:, :1], audio[:, 1:]
        B, n = later.shape[0], later.shape[1] // self.vae_scale
        later = later.reshape(B, n, self.vae_scale, *later.shape[2:])
        mid = self.audio_window // 2
        parts = [later[:, :, :1, : mid + 1].flatten(2, 3), later[:, :, 1:-1, mid : mid + 1].flatten(2, 3),
                 later[:, :, -1:, mid:].flatten(2, 3)]  # fmt: skip
        tokens = self.audio_proj(first, torch.cat(parts, dim=2))
        return torch.cat(tokens.split(1), dim=2)

    @torch.no_grad()
    def forward(self, x: list, t: torch.Tensor, context: list, clip_fea=None, y: list | None = None, audio=None, e0=None,
                kv_cache: list | None = None, start_idx: int = 0, end_idx: int | None = None, skip_audio: bool = False):  # fmt: skip
        """x, y: lists of [C, f, H, W] (noisy latents, conditioning); context: list of [L, text_dim];
        kv_cache: one `KVCache` per block -> [B, out_dim, f, H, W]."""
        dt = self.patch_embedding.weight.dtype
        lat = torch.stack([torch.cat([u, v], dim=0) for u, v in zip(x, y)]).to(dt)
        h5 = self.patch_embedding(lat)
        f, h, w = h5.shape[2:]
        tok = h5.flatten(2).transpose(1, 2).contiguous()
        e, e0_new = self.time_embed(t.to(tok.device))
        e0 = e0_new if e0 is None else e0.float()
        ctx = torch.stack([torch.cat([u, u.new_zeros(self.text_len - u.shape[0], u.shape[1])]) for u in context]).to(dt)
        te = self.text_embedding
        ctx = TF.linear(TF.linear(ctx, te[0].weight, te[0].bias, act="gelu_tanh"), te[2].weight, te[2].bias)
        ctx = torch.cat([self.img_emb(clip_fea.to(dt)), ctx], dim=1)
        audio_embedding = None if audio is None else self.audio_context(audio.to(tok.device, dt)).to(dt)
        seq_len = tok.shape[1]
        if self.usp_flag:
            (tok,) = pshard.sequence_parallel_shard([tok], [1])
        for i, blk in enumerate(self.blocks):
            tok = blk(tok, e0, f, h, w, ctx, kv_cache[i], start_idx, end_idx, audio_embedding, skip_audio, h * w)
        out = self.head(tok, e.unsqueeze(1))
        if self.usp_flag:
            (out,) = pshard.sequence_parallel_unshard([out], [1], [seq_len])
        p = self.patch_size
        out = out[:, : f * h * w].view(-1, f, h, w, p[0], p[1], p[2], self.out_dim).permute(0, 7, 1, 4, 2, 5, 3, 6)
        return out.reshape(-1, self.out_dim, f * p[0], h * p[1], w * p[2])

    @staticmethod
    def state_dict_converter():
        return LiveActDiTStateDictConverter()


class LiveActDiTStateDictConverter:
    def from_official(self, sd: dict):
        return sd, {}

    def from_diffusers(self, sd: dict):
        return sd, {}


__all__ = ["LiveActDiT", "AudioProjModel", "MemorySelfAttention", "SingleStreamAttention", "math"]
