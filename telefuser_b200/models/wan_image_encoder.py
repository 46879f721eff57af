"""CLIP image tower used by Wan image-to-video: ViT-H/14 (open-clip XLM-Roberta-large / ViT-huge-14).

Only the visual tower is needed: 224x224 input, 14x14 patches, class token + 256 patch tokens,
width 1280, 32 pre-norm blocks (16 heads, GELU MLP x4); the pipeline consumes the hidden states after
the first 31 blocks, `[B, 257, 1280]`. Parameter names follow the public checkpoint
(`model.visual.*`), its textual tower and logit scale are dropped on load.
Role parity: telefuser/models/wan_video_image_encoder.py:62-304 (VisionTransformer),
:479-534 (WanImageEncoder, converter).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from telefuser_b200.core.base_model import BaseModel
from telefuser_b200.ops import functional as TF

CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


class _Attention(nn.Module):
    def __init__(self, dim: int, num_heads: int) -> None:
        super().__init__()
        self.num_heads, self.head_dim = num_heads, dim // num_heads
        self.to_qkv = nn.Linear(dim, dim * 3)
        self.proj = nn.Linear(dim, dim)

    def forward(self, x):
        B, S, C = x.shape
        q, k, v = TF.linear(x, self.to_qkv.weight, self.to_qkv.bias).view(B, S, 3, self.num_heads, self.head_dim).unbind(2)
        o = TF.attention(q, k, v)
        return TF.linear(o.reshape(B, S, C), self.proj.weight, self.proj.bias)


class _Block(nn.Module):
    def __init__(self, dim: int, mlp_ratio: float, num_heads: int, activation: str, eps: float) -> None:
        super().__init__()
        self.norm1 = nn.LayerNorm(dim, eps=eps)
        self.attn = _Attention(dim, num_heads)
        self.norm2 = nn.LayerNorm(dim, eps=eps)
        self.activation = activation
        self.mlp = nn.Sequential(nn.Linear(dim, int(dim * mlp_ratio)), nn.GELU(), nn.Linear(int(dim * mlp_ratio), dim))

    def _mlp(self, x):
        h = TF.linear(x, self.mlp[0].weight, self.mlp[0].bias)
        h = h * torch.sigmoid(1.702 * h) if self.activation == "quick_gelu" else F.gelu(h)
        return TF.linear(h, self.mlp[2].weight, self.mlp[2].bias)

    def forward(self, x):
        x = x + self.attn(F.layer_norm(x.float(), x.shape[-1:], self.norm1.weight.float(), self.norm1.bias.float(),
                                       self.norm1.eps).to(x.dtype))  # fmt: skip
        return x + self._mlp(F.layer_norm(x.float(), x.shape[-1:], self.norm2.weight.float(), self.norm2.bias.float(),
                                          self.norm2.eps).to(x.dtype))  # fmt: skip


class VisionTransformer(nn.Module):
    def __init__(self, image_size=224, patch_size=14, dim=1280, mlp_ratio=4, out_dim=1024, num_heads=16, num_layers=32,
                 activation="gelu", pre_norm=True, eps=1e-5) -> None:  # fmt: skip
        super().__init__()
        self.image_size, self.patch_size, self.dim = image_size, patch_size, dim
        n = (image_size // patch_size) ** 2
        self.patch_embedding = nn.Conv2d(3, dim, kernel_size=patch_size, stride=patch_size, bias=not pre_norm)
        self.cls_embedding = nn.Parameter(torch.randn(1, 1, dim) / dim**0.5)
        self.pos_embedding = nn.Parameter(torch.randn(1, n + 1, dim) / dim**0.5)
        self.pre_norm = nn.LayerNorm(dim, eps=eps) if pre_norm else None
        self.transformer = nn.Sequential(*[_Block(dim, mlp_ratio, num_heads, activation, eps) for _ in range(num_layers)])
        self.post_norm = nn.LayerNorm(dim, eps=eps)
        self.head = nn.Parameter(torch.randn(dim, out_dim) / dim**0.5)

    def forward(self, x, use_31_block: bool = False):
        B = x.shape[0]
        p = self.patch_size
        # stride == kernel: the patch convolution is a GEMM over unfolded patches
        patches = x.unfold(2, p, p).unfold(3, p, p).permute(0, 2, 3, 1, 4, 5).reshape(B, -1, 3 * p * p)
        w = self.patch_embedding.weight.reshape(self.dim, -1)
        x = TF.linear(patches.to(w.dtype), w, self.patch_embedding.bias)
        x = torch.cat([self.cls_embedding.expand(B, -1, -1).to(x.dtype), x], dim=1) + self.pos_embedding.to(x.dtype)
        if self.pre_norm is not None:
            x = self.pre_norm(x.float()).to(x.dtype) if x.dtype != torch.float32 else self.pre_norm(x)
        blocks = self.transformer[:-1] if use_31_block else self.transformer
        for blk in blocks:
            x = blk(x)
        return x


class _Clip(nn.Module):
    def __init__(self, **vision_kw) -> None:
        super().__init__()
        self.visual = VisionTransformer(**vision_kw)
        self.image_size = self.visual.image_size


class WanImageEncoder(BaseModel):
    def __init__(self, **vision_kw) -> None:
        super().__init__()
        self.model = _Clip(**vision_kw)
        self.layer_name_list = []

    @torch.no_grad()
    def encode_image(self, images: list[torch.Tensor]) -> torch.Tensor:
        """images: list of `[1, 3, H, W]` in [-1, 1] -> `[N, 257, 1280]` penultimate hidden states."""
        size = (self.model.image_size,) * 2
        x = torch.cat([F.interpolate(u.float(), size=size, mode="bicubic", align_corners=False) for u in images])
        x = x * 0.5 + 0.5
        mean = torch.tensor(CLIP_MEAN, device=x.device).view(1, 3, 1, 1)
        std = torch.tensor(CLIP_STD, device=x.device).view(1, 3, 1, 1)
        x = ((x - mean) / std).to(self.model.visual.pos_embedding.dtype)
        return self.model.visual(x, use_31_block=True)

    forward = encode_image

    @staticmethod
    def state_dict_converter():
        return WanImageEncoderStateDictConverter()


class WanImageEncoderStateDictConverter:
    def from_diffusers(self, state_dict: dict):
        return state_dict, {}

    def from_official(self, state_dict: dict):
        out = {}
        for name, p in state_dict.items():
            if name.startswith("textual.") or name == "log_scale":
                continue
            out["model." + name] = p
        return out, {}


def _register() -> None:
    from telefuser_b200.core.model_registry import register_model_config

    # Fingerprint (MD5 of the sorted key list) of the public open-clip-xlm-roberta-large-vit-huge-14
    # checkpoint, textual tower included; same value as telefuser/models/wan_video_image_encoder.py:531.
    register_model_config(None, "5941c53e207d62f20f9025686193c40b", ["wan_video_image_encoder"], [WanImageEncoder],
                          "official")  # fmt: skip


_register()
