"""UMT5-XXL text encoder used by the Wan pipelines (24 layers, dim 4096, 64 heads, gated-GELU FFN,
per-layer relative position bias, no attention scaling).

State-dict keys match the encoder checkpoint published with Wan
(`token_embedding`, `blocks.N.{norm1,attn.{q,k,v,o},norm2,ffn.{gate.0,fc1,fc2},pos_embedding.embedding}`,
`norm`), i.e. the layout of the reference's ``telefuser/models/wan_video_text_encoder.py:34-317``.
Projections run through the tcgen05 GEMM; the gate and up projections are one GEMM followed by
the fused `gelu_tanh(a) * b` kernel. Attention is 512 tokens with an additive bias, so it uses
PyTorch SDPA (cold path).
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from telefuser_b200.core.base_model import BaseModel
from telefuser_b200.ops import functional as TF


class T5LayerNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x):
        return TF.rmsnorm_reference(x, self.weight, self.eps)


class T5RelativeEmbedding(nn.Module):
    def __init__(self, num_buckets: int, num_heads: int, bidirectional: bool = True, max_dist: int = 128):
        super().__init__()
        self.num_buckets, self.num_heads, self.bidirectional, self.max_dist = num_buckets, num_heads, bidirectional, max_dist
        self.embedding = nn.Embedding(num_buckets, num_heads)

    def bucket(self, rel_pos):
        if self.bidirectional:
            nb = self.num_buckets // 2
            base = (rel_pos > 0).long() * nb
            rel_pos = rel_pos.abs()
        else:
            nb = self.num_buckets
            base = torch.zeros_like(rel_pos)
            rel_pos = -torch.min(rel_pos, torch.zeros_like(rel_pos))
        exact = nb // 2
        large = exact + (torch.log(rel_pos.float() / exact) / math.log(self.max_dist / exact) * (nb - exact)).long()
        large = torch.min(large, torch.full_like(large, nb - 1))
        return base + torch.where(rel_pos < exact, rel_pos, large)

    def forward(self, lq: int, lk: int):
        dev = self.embedding.weight.device
        rel = torch.arange(lk, device=dev).unsqueeze(0) - torch.arange(lq, device=dev).unsqueeze(1)
        return self.embedding(self.bucket(rel)).permute(2, 0, 1).unsqueeze(0).contiguous()  # [1, H, Lq, Lk]


class T5Attention(nn.Module):
    def __init__(self, dim: int, dim_attn: int, num_heads: int):
        super().__init__()
        self.num_heads, self.head_dim = num_heads, dim_attn // num_heads
        self.q = nn.Linear(dim, dim_attn, bias=False)
        self.k = nn.Linear(dim, dim_attn, bias=False)
        self.v = nn.Linear(dim, dim_attn, bias=False)
        self.o = nn.Linear(dim_attn, dim, bias=False)

    def forward(self, x, mask=None, pos_bias=None):
        B, L, _ = x.shape
        H, D = self.num_heads, self.head_dim
        q = TF.linear(x, self.q.weight).view(B, L, H, D)
        k = TF.linear(x, self.k.weight).view(B, L, H, D)
        v = TF.linear(x, self.v.weight).view(B, L, H, D)
        if pos_bias is not None and pos_bias.shape[1] != H:  # heads split over TP ranks
            pos_bias = pos_bias[:, getattr(self, "head_start", 0) :][:, :H]
        bias = pos_bias.to(q.dtype) if pos_bias is not None else torch.zeros(1, H, L, L, device=x.device, dtype=q.dtype)
        if mask is not None:
            m = mask.view(B, 1, 1, -1) if mask.dim() == 2 else mask.unsqueeze(1)
            bias = bias.expand(B, -1, -1, -1).masked_fill(m == 0, torch.finfo(q.dtype).min)
        o = TF.attention(q, k, v, scale=1.0, bias=bias)  # T5: no 1/sqrt(d); relative-position bias on the scores
        return TF.linear(o.reshape(B, L, H * D), self.o.weight)


class T5FeedForward(nn.Module):
    def __init__(self, dim: int, dim_ffn: int):
        super().__init__()
        self.dim, self.dim_ffn = dim, dim_ffn
        self.gate = nn.Sequential(nn.Linear(dim, dim_ffn, bias=False), nn.GELU(approximate="tanh"))
        self.fc1 = nn.Linear(dim, dim_ffn, bias=False)
        self.fc2 = nn.Linear(dim_ffn, dim, bias=False)
        self._fused = None

    def fused_gate_up(self):
        w = self.gate[0].weight
        if self._fused is None or self._fused.data_ptr() != w.data_ptr() or self._fused.dtype != w.dtype:
            W = torch.cat([self.gate[0].weight.data, self.fc1.weight.data], dim=0)
            n = W.shape[0] // 2  # local width: the weights may be TP shards
            self.gate[0].weight.data = W[:n]
            self.fc1.weight.data = W[n:]
            self._fused = W
        return self._fused

    def forward(self, x):
        h = TF.act_mul(TF.linear(x, self.fused_gate_up()), "gelu_tanh")
        return TF.linear(h, self.fc2.weight)


class T5Block(nn.Module):
    def __init__(self, dim, dim_attn, dim_ffn, num_heads, num_buckets, shared_pos):
        super().__init__()
        self.shared_pos = shared_pos
        self.norm1 = T5LayerNorm(dim)
        self.attn = T5Attention(dim, dim_attn, num_heads)
        self.norm2 = T5LayerNorm(dim)
        self.ffn = T5FeedForward(dim, dim_ffn)
        self.pos_embedding = None if shared_pos else T5RelativeEmbedding(num_buckets, num_heads, True)

    def forward(self, x, mask=None, pos_bias=None):
        e = pos_bias if self.shared_pos else self.pos_embedding(x.size(1), x.size(1))
        x = x + self.attn(self.norm1(x), mask, e)
        return x + self.ffn(self.norm2(x))


class WanTextEncoder(BaseModel):
    def __init__(self, vocab=256384, dim=4096, dim_attn=4096, dim_ffn=10240, num_heads=64, num_layers=24,
                 num_buckets=32, shared_pos=False, dropout=0.1):  # fmt: skip
        super().__init__()
        self.dim, self.num_layers = dim, num_layers
        self.token_embedding = nn.Embedding(vocab, dim)
        self.pos_embedding = T5RelativeEmbedding(num_buckets, num_heads, True) if shared_pos else None
        self.blocks = nn.ModuleList([T5Block(dim, dim_attn, dim_ffn, num_heads, num_buckets, shared_pos)
                                     for _ in range(num_layers)])  # fmt: skip
        self.norm = T5LayerNorm(dim)

    @torch.no_grad()
    def forward(self, ids, mask=None):
        x = self.token_embedding(ids)
        e = self.pos_embedding(x.size(1), x.size(1)) if self.pos_embedding is not None else None
        for blk in self.blocks:
            x = blk(x, mask, e)
        return self.norm(x)

    def get_tp_plan(self) -> dict:
        """Megatron split: q/k/v and gate/fc1 by output features (heads), o and fc2 by input features
        with one all-reduce after each attention and FFN."""
        return {"blocks.*.attn.q": "colwise", "blocks.*.attn.k": "colwise", "blocks.*.attn.v": "colwise",
                "blocks.*.attn.o": "rowwise", "blocks.*.attn": ["heads", "allreduce"],
                "blocks.*.ffn.gate.0": "colwise", "blocks.*.ffn.fc1": "colwise", "blocks.*.ffn.fc2": "rowwise",
                "blocks.*.ffn": "allreduce"}  # fmt: skip

    @staticmethod
    def state_dict_converter():
        return WanTextEncoderStateDictConverter()


class WanTextEncoderStateDictConverter:
    """Keys are used as published; sizes that differ from UMT5-XXL (smaller encoders, test models) are read off the tensors."""

    def from_official(self, state_dict):
        sd, ctor = dict(state_dict), {}
        emb, q, fc1 = sd.get("token_embedding.weight"), sd.get("blocks.0.attn.q.weight"), sd.get("blocks.0.ffn.fc1.weight")
        pos = sd.get("blocks.0.pos_embedding.embedding.weight")
        if emb is not None and q is not None and fc1 is not None and tuple(emb.shape) != (256384, 4096):
            layers = 1 + max(int(k.split(".")[1]) for k in sd if k.startswith("blocks."))
            ctor = dict(vocab=int(emb.shape[0]), dim=int(emb.shape[1]), dim_attn=int(q.shape[0]), dim_ffn=int(fc1.shape[0]), num_layers=layers)
            shared = sd.get("pos_embedding.embedding.weight")
            if pos is not None:
                ctor.update(num_buckets=int(pos.shape[0]), num_heads=int(pos.shape[1]))
            elif shared is not None:
                ctor.update(num_buckets=int(shared.shape[0]), num_heads=int(shared.shape[1]), shared_pos=True)
        return sd, ctor

    from_civitai = from_official
    from_diffusers = from_official


class HuggingfaceTokenizer:
    """Tokenizer wrapper: optional whitespace cleaning, fixed-length padding, returns (ids, mask)."""

    def __init__(self, name: str, seq_len: int | None = None, clean: str | None = None, **kwargs):
        from transformers import AutoTokenizer

        self.name, self.seq_len, self.clean = name, seq_len, clean
        self.tokenizer = AutoTokenizer.from_pretrained(name, **kwargs)
        self.vocab_size = self.tokenizer.vocab_size

    @staticmethod
    def _clean(text: str, mode: str | None) -> str:
        import html
        import re

        if mode is None:
            return text
        text = html.unescape(html.unescape(text)).strip()
        text = re.sub(r"\s+", " ", text).strip()
        return text.lower() if mode == "lower" else text

    def __call__(self, sequence, return_mask: bool = False, **kwargs):
        if isinstance(sequence, str):
            sequence = [sequence]
        sequence = [self._clean(s, self.clean) for s in sequence]
        kw = dict(return_tensors="pt")
        if self.seq_len is not None:
            kw.update(padding="max_length", truncation=True, max_length=self.seq_len)
        kw.update(kwargs)
        enc = self.tokenizer(sequence, **kw)
        return (enc.input_ids, enc.attention_mask) if return_mask else enc.input_ids


def _register() -> None:
    from telefuser_b200.core.model_registry import register_architecture

    register_architecture("wan_video_text_encoder", WanTextEncoder, WanTextEncoder)


_register()
