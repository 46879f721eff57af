"""LingBot-World-Fast causal DiT: chunk-autoregressive Wan-14B derivative with camera / action control.

Per chunk the model sees only the new latent frames; self-attention keys/values of past chunks
live in a per-layer `RollingKVCache` (bounded window + pinned sink frames) and text K/V are
computed once per session. Same state-dict layout as the reference
(telefuser/models/lingbot_world_fast_dit.py:41-679). Kernel layout matches the Wan DiT: fused QKV
GEMM, one RMSNorm+RoPE pass (RoPE phase offset by the chunk's first frame), tcgen05 attention over
the cache window, gate/residual folded into GEMM epilogues; the camera injection's scale and shift
projections run as one GEMM.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from telefuser_b200.cache.rolling_kv import RollingKVCache
from telefuser_b200.core.base_model import BaseModel
from telefuser_b200.models.wan_dit import (AffineLayerNorm, RMSNormWeight, WanHead, _fuse_linear_weights,
                                           rope_tables_3d, sinusoidal_embedding_1d)  # fmt: skip
from telefuser_b200.ops import functional as TF
from telefuser_b200.parallel import shard as pshard
from telefuser_b200.parallel.mesh import get_mesh
from telefuser_b200.parallel import ulysses


class CrossAttnCache:
    def __init__(self):
        self.k = self.v = None

    @property
    def is_init(self) -> bool:
        return self.k is not None


class LingBotCacheState:
    """All per-session model state: one rolling KV cache and one text K/V cache per block."""

    def __init__(self, model: "LingBotWorldFastDiT", batch: int, kv_size: int, device, dtype, heads_local: int,
                 frame_tokens: int):  # fmt: skip
        rolling = model.local_attn_size != -1
        self.kv = [RollingKVCache(batch, kv_size, heads_local, model.head_dim, device, dtype,
                                  sink_tokens=model.sink_size * frame_tokens, rolling=rolling)
                   for _ in range(model.num_layers)]  # fmt: skip
        self.cross = [CrossAttnCache() for _ in range(model.num_layers)]
        self.frame_tokens = frame_tokens

    def reset(self) -> None:
        for c in self.kv:
            c.reset()
        for c in self.cross:
            c.k = c.v = None

    def nbytes(self) -> int:
        return sum(c.nbytes() for c in self.kv)

    def snapshot(self, to_cpu: bool = True) -> dict:
        """Everything a later `restore` needs to continue the session: the filled part of every rolling K/V buffer
        with its cursors. The text K/V caches are derived from the prompt embedding on the next call, so they are
        not stored."""
        def keep(t):
            return t.detach().to("cpu", copy=True) if to_cpu else t.detach().clone()

        return {"frame_tokens": self.frame_tokens,
                "kv": [{"k": keep(c.k[:, : c.local_end]), "v": keep(c.v[:, : c.local_end]), "global_end": c.global_end,
                        "local_end": c.local_end} for c in self.kv]}  # fmt: skip

    def restore(self, snap: dict) -> None:
        if len(snap["kv"]) != len(self.kv) or snap["frame_tokens"] != self.frame_tokens:
            raise ValueError("the snapshot was taken from a session of another model or resolution")
        for c, s in zip(self.kv, snap["kv"]):
            n = s["local_end"]
            if n > c.kv_size or s["k"].shape[2:] != c.k.shape[2:]:
                raise ValueError("the snapshot does not fit this session's K/V buffers")
            c.k[:, :n].copy_(s["k"])
            c.v[:, :n].copy_(s["v"])
            c.global_end, c.local_end = s["global_end"], n
        for c in self.cross:
            c.k = c.v = None


class CausalSelfAttention(nn.Module):
    def __init__(self, dim, num_heads, local_attn_size=-1, sink_size=0, qk_norm=True, eps=1e-6):
        super().__init__()
        self.dim, self.num_heads, self.head_dim = dim, num_heads, dim // num_heads
        self.local_attn_size, self.sink_size = local_attn_size, sink_size
        self.q = nn.Linear(dim, dim)
        self.k = nn.Linear(dim, dim)
        self.v = nn.Linear(dim, dim)
        self.o = nn.Linear(dim, dim)
        self.norm_q = RMSNormWeight(dim, eps) if qk_norm else None
        self.norm_k = RMSNormWeight(dim, eps) if qk_norm else None
        self._qkv = None

    def fused_qkv(self):
        w = self.q.weight
        if self._qkv is None or self._qkv[0].data_ptr() != w.data_ptr() or self._qkv[0].dtype != w.dtype:
            self._qkv = _fuse_linear_weights([self.q, self.k, self.v])
        return self._qkv

    def forward(self, x, cos, sin, cache: RollingKVCache, current_start: int, max_attention_size: int,
                valid_seq_len: int, usp: bool):  # fmt: skip
        B, S, C = x.shape
        H, D = self.num_heads, self.head_dim
        W, b = self.fused_qkv()
        qkv = TF.linear(x, W, b)
        q, k, v = qkv[..., :C], qkv[..., C : 2 * C], qkv[..., 2 * C :]
        if self.norm_q is not None:
            TF.rmsnorm_rope_(q, self.norm_q.weight, H, cos, sin, self.norm_q.eps, x2=k, weight2=self.norm_k.weight)
        else:
            q.copy_(TF.rope_reference(q.unflatten(-1, (H, D)), cos, sin).flatten(-2))
            k.copy_(TF.rope_reference(k.unflatten(-1, (H, D)), cos, sin).flatten(-2))
        q, k, v = (t.unflatten(-1, (H, D)) for t in (q, k, v))
        if usp:
            hq = ulysses.scatter_heads(q, async_op=True)
            hk = ulysses.scatter_heads(k, async_op=True)
            hv = ulysses.scatter_heads(v, async_op=True)
            q, k, v = (h.wait()[:, :valid_seq_len] for h in (hq, hk, hv))
        cache.append(k, v, current_start)
        kw, vw = cache.window(max_attention_size)
        o = TF.attention(q, kw, vw)
        if usp:
            # the sharded sequence was zero-padded to a multiple of the Ulysses degree: restore that length
            padded = S * get_mesh().size("ulysses")
            if padded > o.shape[1]:
                o = F.pad(o, (0, 0, 0, 0, 0, padded - o.shape[1]))
            o = ulysses.gather_heads(o)
        return o.reshape(B, S, C)


class CachedCrossAttention(nn.Module):
    def __init__(self, dim, num_heads, eps=1e-6):
        super().__init__()
        self.dim, self.num_heads, self.head_dim = dim, num_heads, dim // num_heads
        self.q = nn.Linear(dim, dim)
        self.k = nn.Linear(dim, dim)
        self.v = nn.Linear(dim, dim)
        self.o = nn.Linear(dim, dim)
        self.norm_q = RMSNormWeight(dim, eps)
        self.norm_k = RMSNormWeight(dim, eps)

    def forward(self, x, context, cache: CrossAttnCache | None):
        B, S, C = x.shape
        H, D = self.num_heads, self.head_dim
        q = TF.linear(x, self.q.weight, self.q.bias)
        TF.rmsnorm_rope_(q, self.norm_q.weight, H, eps=self.norm_q.eps)
        if cache is not None and cache.is_init:
            k, v = cache.k, cache.v
        else:
            k = TF.linear(context, self.k.weight, self.k.bias)
            TF.rmsnorm_rope_(k, self.norm_k.weight, H, eps=self.norm_k.eps)
            v = TF.linear(context, self.v.weight, self.v.bias)
            k, v = k.unflatten(-1, (H, D)), v.unflatten(-1, (H, D))
            if cache is not None:
                cache.k, cache.v = k, v
        return TF.attention(q.unflatten(-1, (H, D)), k, v).reshape(B, S, C)


class LingBotWorldFastBlock(nn.Module):
    def __init__(self, dim, ffn_dim, num_heads, local_attn_size=-1, sink_size=0, qk_norm=True, cross_attn_norm=True,
                 eps=1e-6):  # fmt: skip
        super().__init__()
        self.self_attn = CausalSelfAttention(dim, num_heads, local_attn_size, sink_size, qk_norm, eps)
        self.cross_attn = CachedCrossAttention(dim, num_heads, eps)
        self.norm1 = AffineLayerNorm(dim, eps, elementwise_affine=False)
        self.norm2 = AffineLayerNorm(dim, eps, elementwise_affine=False)
        self.norm3 = AffineLayerNorm(dim, eps) if cross_attn_norm else None
        self.ffn = nn.Sequential(nn.Linear(dim, ffn_dim), nn.GELU(approximate="tanh"), nn.Linear(ffn_dim, dim))
        self.modulation = nn.Parameter(torch.randn(1, 6, dim) / dim**0.5)
        self.cam_injector_layer1 = nn.Linear(dim, dim)
        self.cam_injector_layer2 = nn.Linear(dim, dim)
        self.cam_scale_layer = nn.Linear(dim, dim)
        self.cam_shift_layer = nn.Linear(dim, dim)
        self._cam = None

    def fused_cam_scale_shift(self):
        w = self.cam_scale_layer.weight
        if self._cam is None or self._cam[0].data_ptr() != w.data_ptr() or self._cam[0].dtype != w.dtype:
            self._cam = _fuse_linear_weights([self.cam_scale_layer, self.cam_shift_layer])
        return self._cam

    def inject_control(self, x, control_tokens):
        h = F.silu(TF.linear(control_tokens, self.cam_injector_layer1.weight, self.cam_injector_layer1.bias))
        h = TF.linear(h, self.cam_injector_layer2.weight, self.cam_injector_layer2.bias, residual=control_tokens)
        W, b = self.fused_cam_scale_shift()
        ss = TF.linear(h, W, b)
        C = x.shape[-1]
        return torch.addcmul(ss[..., C:], x, 1.0 + ss[..., :C])

    def forward(self, x, mod, context, cos, sin, kv: RollingKVCache, cross: CrossAttnCache, current_start,
                max_attention_size, valid_seq_len, control_tokens=None, usp=False):  # fmt: skip
        shift_msa, scale_msa, gate_msa, shift_mlp, scale_mlp, gate_mlp = (mod[:, :, i] for i in range(6))
        a = self.self_attn(self.norm1(x, shift_msa, scale_msa), cos, sin, kv, current_start, max_attention_size,
                           valid_seq_len, usp)  # fmt: skip
        x = TF.linear(a, self.self_attn.o.weight, self.self_attn.o.bias, residual=x, gate=gate_msa)
        if control_tokens is not None:
            x = self.inject_control(x, control_tokens)
        h = self.norm3(x) if self.norm3 is not None else x
        c = self.cross_attn(h, context, cross)
        x = TF.linear(c, self.cross_attn.o.weight, self.cross_attn.o.bias, residual=x)
        h = TF.linear(self.norm2(x, shift_mlp, scale_mlp), self.ffn[0].weight, self.ffn[0].bias, act="gelu_tanh")
        return TF.linear(h, self.ffn[2].weight, self.ffn[2].bias, residual=x, gate=gate_mlp)


class LingBotWorldFastDiT(BaseModel):
    def __init__(self, patch_size=(1, 2, 2), text_len=512, in_dim=32, dim=5120, ffn_dim=13824, freq_dim=256,
                 text_dim=4096, out_dim=16, num_heads=40, num_layers=40, local_attn_size=-1, sink_size=0, qk_norm=True,
                 cross_attn_norm=True, eps=1e-6, control_type="cam"):  # fmt: skip
        super().__init__()
        self.patch_size = tuple(patch_size)
        self.text_len, self.in_dim, self.dim, self.ffn_dim, self.freq_dim = text_len, in_dim, dim, ffn_dim, freq_dim
        self.text_dim, self.out_dim, self.num_heads, self.num_layers = text_dim, out_dim, num_heads, num_layers
        self.head_dim = dim // num_heads
        self.local_attn_size, self.sink_size, self.control_type = local_attn_size, sink_size, control_type
        control_dim = 6 if control_type == "cam" else 7
        self.control_dim = control_dim
        self.patch_embedding = nn.Conv3d(in_dim, dim, kernel_size=self.patch_size, stride=self.patch_size)
        self.patch_embedding_wancamctrl = nn.Linear(control_dim * 64 * math.prod(self.patch_size), dim)
        self.c2ws_hidden_states_layer1 = nn.Linear(dim, dim)
        self.c2ws_hidden_states_layer2 = nn.Linear(dim, dim)
        self.text_embedding = nn.Sequential(nn.Linear(text_dim, dim), nn.GELU(approximate="tanh"), nn.Linear(dim, dim))
        self.time_embedding = nn.Sequential(nn.Linear(freq_dim, dim), nn.SiLU(), nn.Linear(dim, dim))
        self.time_projection = nn.Sequential(nn.SiLU(), nn.Linear(dim, dim * 6))
        self.blocks = nn.ModuleList([
            LingBotWorldFastBlock(dim, ffn_dim, num_heads, local_attn_size, sink_size, qk_norm, cross_attn_norm, eps)
            for _ in range(num_layers)])  # fmt: skip
        self.head = WanHead(dim, out_dim, self.patch_size, eps)
        self.dtype = torch.bfloat16
        self._mod_stack = None
        self._rope_cache: dict = {}

    # ---- session state -------------------------------------------------------------
    def new_cache_state(self, batch: int, kv_size: int, frame_tokens: int, device=None, dtype=None,
                        ulysses_degree: int = 1) -> LingBotCacheState:  # fmt: skip
        p = next(self.parameters())
        return LingBotCacheState(self, batch, kv_size, device or p.device, dtype or p.dtype,
                                 self.num_heads // ulysses_degree, frame_tokens)  # fmt: skip

    # ---- pieces -------------------------------------------------------------------------
    def time_embed(self, t, seq_len):
        B = t.shape[0]
        e = sinusoidal_embedding_1d(self.freq_dim, t.flatten())
        w0, w2, wp = self.time_embedding[0], self.time_embedding[2], self.time_projection[1]
        e = F.linear(F.silu(F.linear(e, w0.weight.float(), w0.bias.float())), w2.weight.float(), w2.bias.float())
        tm = F.linear(F.silu(e), wp.weight.float(), wp.bias.float())
        if t.dim() == 1:
            return e.view(B, 1, self.dim), tm.view(B, 1, 6, self.dim)
        return e.view(B, seq_len, self.dim), tm.view(B, seq_len, 6, self.dim)

    def prepare_control_tokens(self, control):
        if control is None:
            return None
        pt, ph, pw = self.patch_size
        B, C, F_, H, W = control.shape
        f, h, w = F_ // pt, H // ph, W // pw
        tok = control.reshape(B, C, f, pt, h, ph, w, pw).permute(0, 2, 4, 6, 1, 3, 5, 7).reshape(B, f * h * w, -1)
        tok = tok.to(self.dtype)
        tok = TF.linear(tok, self.patch_embedding_wancamctrl.weight, self.patch_embedding_wancamctrl.bias)
        hid = F.silu(TF.linear(tok, self.c2ws_hidden_states_layer1.weight, self.c2ws_hidden_states_layer1.bias))
        return TF.linear(hid, self.c2ws_hidden_states_layer2.weight, self.c2ws_hidden_states_layer2.bias, residual=tok)

    def patchify(self, x):
        B, C, F_, H, W = x.shape
        pt, ph, pw = self.patch_size
        f, h, w = F_ // pt, H // ph, W // pw
        tok = x.reshape(B, C, f, pt, h, ph, w, pw).permute(0, 2, 4, 6, 1, 3, 5, 7).reshape(B, f * h * w, -1)
        wgt = self.patch_embedding.weight.reshape(self.dim, -1)
        return TF.linear(tok.to(wgt.dtype), wgt, self.patch_embedding.bias), (f, h, w)

    def unpatchify(self, x, grid):
        f, h, w = grid
        pt, ph, pw = self.patch_size
        B = x.shape[0]
        x = x.reshape(B, f, h, w, pt, ph, pw, self.out_dim).permute(0, 7, 1, 4, 2, 5, 3, 6)
        return x.reshape(B, self.out_dim, f * pt, h * ph, w * pw)

    @torch.no_grad()
    def forward(self, x, timestep, context, y=None, control_tensor=None, cache: LingBotCacheState | None = None,
                current_start: int = 0, max_attention_size: int = 1_000_000):  # fmt: skip
        if cache is None:
            raise ValueError("LingBotWorldFastDiT needs a cache state (see new_cache_state)")
        if y is not None:
            x = torch.cat([x, y.to(device=x.device, dtype=x.dtype)], dim=1)
        x, grid = self.patchify(x)
        seq_len = x.shape[1]
        t_head, t_mod = self.time_embed(timestep.to(x.device), seq_len)
        te = self.text_embedding
        context = TF.linear(TF.linear(context.to(self.dtype), te[0].weight, te[0].bias, act="gelu_tanh"),
                            te[2].weight, te[2].bias)  # fmt: skip
        control_tokens = self.prepare_control_tokens(control_tensor)
        frame_tokens = grid[1] * grid[2]
        key = (grid, current_start // frame_tokens, str(x.device))
        if key not in self._rope_cache:
            if len(self._rope_cache) > 16:
                self._rope_cache.clear()
            self._rope_cache[key] = rope_tables_3d(self.head_dim, grid, x.device, frame_start=key[1])
        cos, sin = self._rope_cache[key]
        if self.usp_flag:
            tensors, dims = [x, cos, sin], [1, 0, 0]
            if t_mod.shape[1] == seq_len:
                tensors += [t_mod, t_head]
                dims += [1, 1]
            if control_tokens is not None:
                tensors.append(control_tokens)
                dims.append(1)
            out = pshard.sequence_parallel_shard(tensors, dims)
            x, cos, sin = out[:3]
            rest = out[3:]
            if t_mod.shape[1] == seq_len:
                t_mod, t_head = rest[0], rest[1]
                rest = rest[2:]
            if control_tokens is not None:
                control_tokens = rest[0]
        if self._mod_stack is None or self._mod_stack.device != t_mod.device:
            self._mod_stack = torch.stack([b.modulation.detach().float() for b in self.blocks]).to(t_mod.device)
        for i, blk in enumerate(self.blocks):
            mod = self._mod_stack[i].unsqueeze(0) + t_mod
            x = blk(x, mod, context, cos, sin, cache.kv[i], cache.cross[i], current_start, max_attention_size,
                    seq_len, control_tokens, self.usp_flag)  # fmt: skip
        x = self.head(x, t_head)
        if self.usp_flag:
            (x,) = pshard.sequence_parallel_unshard([x], [1], [seq_len])
        return self.unpatchify(x, grid).float()

    def get_fsdp_module_names(self):
        return ["blocks"]

    @staticmethod
    def state_dict_converter():
        return LingBotWorldFastDiTConverter()


class LingBotWorldFastDiTConverter:
    """Infers the architecture from tensor shapes (the checkpoint has no config file)."""

    def __init__(self, **overrides):
        self.overrides = overrides

    def from_official(self, sd: dict):
        sd = {k.removeprefix("model."): v for k, v in sd.items()}
        pe = sd["patch_embedding.weight"]
        dim = pe.shape[0]
        layers = 1 + max(int(k.split(".")[1]) for k in sd if k.startswith("blocks."))
        ctrl = sd["patch_embedding_wancamctrl.weight"].shape[1] // (64 * math.prod(pe.shape[2:]))
        cfg = dict(patch_size=tuple(pe.shape[2:]), in_dim=pe.shape[1], dim=dim,
                   ffn_dim=sd["blocks.0.ffn.0.weight"].shape[0], freq_dim=sd["time_embedding.0.weight"].shape[1],
                   text_dim=sd["text_embedding.0.weight"].shape[1],
                   out_dim=sd["head.head.weight"].shape[0] // math.prod(pe.shape[2:]), num_heads=dim // 128,
                   num_layers=layers, qk_norm="blocks.0.self_attn.norm_q.weight" in sd,
                   cross_attn_norm="blocks.0.norm3.weight" in sd, control_type="cam" if ctrl == 6 else "act")  # fmt: skip
        cfg.update(self.overrides)
        return sd, cfg

    from_diffusers = from_official
    from_civitai = from_official
