"""Causal projector of the low-quality input video into per-layer DiT conditioning (FlashVSR).

Frames are pixel-unshuffled 16 x 16 (3 -> 768 channels), two causal convolutions (kernel 4 in time, stride 2,
replicate padding in space and time, the last two input frames cached between clips) reduce time 4x, then one
Linear per conditioned DiT layer maps the 3072 channels to the model width. `forward` handles a whole video,
`stream_forward` one clip at a time with the cache carried in the module (first clip: warm-up only, returns
None), `tile_stream_forward` the same per spatial tile with linear blending (tiles spread over ranks).
Role parity: telefuser/models/video_projector.py:14-457.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from telefuser_b200.models.wan_vae import RMS_norm, blend_mask

CACHE_T = 2


class ReplicateCausalConv3d(nn.Conv3d):
    """Causal in time (left padding only, optionally supplied by the previous clip); replicate padding."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self._pad = (self.padding[2], self.padding[2], self.padding[1], self.padding[1], 2 * self.padding[0], 0)
        self.padding = (0, 0, 0)

    def forward(self, x, cache_x=None):
        pad = list(self._pad)
        if cache_x is not None and pad[4] > 0:
            x = torch.cat([cache_x.to(x.device), x], dim=2)
            pad[4] -= cache_x.shape[2]
        return super().forward(F.pad(x, pad, mode="replicate"))


def pixel_unshuffle_space(x: torch.Tensor, hh: int = 16, ww: int = 16) -> torch.Tensor:
    B, C, T, H, W = x.shape
    x = x.view(B, C, T, H // hh, hh, W // ww, ww).permute(0, 1, 4, 6, 2, 3, 5)
    return x.reshape(B, C * hh * ww, T, H // hh, W // ww)


class Causal_LQ4x_Proj(nn.Module):
    def __init__(self, in_dim: int = 3, out_dim: int = 1536, layer_num: int = 30, parallelism: int = 1,
                 hidden_dim1: int = 2048, hidden_dim2: int = 3072) -> None:  # fmt: skip
        super().__init__()
        self.layer_num, self.out_dim, self.parallelism = layer_num, out_dim, parallelism
        self.conv1 = ReplicateCausalConv3d(in_dim * 256, hidden_dim1, (4, 3, 3), stride=(2, 1, 1), padding=(1, 1, 1))
        self.norm1 = RMS_norm(hidden_dim1, images=False)
        self.conv2 = ReplicateCausalConv3d(hidden_dim1, hidden_dim2, (4, 3, 3), stride=(2, 1, 1), padding=(1, 1, 1))
        self.norm2 = RMS_norm(hidden_dim2, images=False)
        self.linear_layers = nn.ModuleList([nn.Linear(hidden_dim2, out_dim) for _ in range(layer_num)])
        self.clear_cache()

    def clear_cache(self) -> None:
        self.cache: dict = {"conv1": None, "conv2": None}
        self.clip_idx = 0

    def set_parallelism(self, parallelism: int) -> None:
        self.parallelism = parallelism

    def _step(self, clip, key1: str, key2: str, emit: bool):
        """One 4-frame clip through both convolutions; returns the conv2 features (or None on the warm-up clip)."""
        x = pixel_unshuffle_space(clip)
        tail1 = x[:, :, -CACHE_T:].clone()
        x = F.silu(self.norm1(self.conv1(x, self.cache.get(key1))))
        self.cache[key1] = tail1
        tail2 = x[:, :, -CACHE_T:].clone()
        if not emit:
            self.cache[key2] = tail2
            return None
        y = F.silu(self.norm2(self.conv2(x, self.cache.get(key2))))
        self.cache[key2] = tail2
        return y

    def _project(self, feats: torch.Tensor) -> list[torch.Tensor]:
        tokens = feats.flatten(2).transpose(1, 2)  # [B, f*h*w, C]
        return [lin(tokens) for lin in self.linear_layers]

    def forward(self, video: torch.Tensor) -> list[torch.Tensor]:
        """video [B, 3, T, H, W] with T = 4n+1 -> layer_num tensors [B, n*(H/16)*(W/16), out_dim]."""
        self.clear_cache()
        video = torch.cat([video[:, :, :1].repeat(1, 1, 3, 1, 1), video], dim=2)
        outs = []
        for i in range(video.shape[2] // 4):
            y = self._step(video[:, :, 4 * i : 4 * i + 4], "conv1", "conv2", emit=i > 0)
            if y is not None:
                outs.append(y)
        return self._project(torch.cat(outs, dim=2))

    def stream_forward(self, video_clip: torch.Tensor):
        first = self.clip_idx == 0
        if first:
            video_clip = torch.cat([video_clip[:, :, :1].repeat(1, 1, 3, 1, 1), video_clip], dim=2)
        y = self._step(video_clip, "conv1", "conv2", emit=not first)
        self.clip_idx += 1
        return None if y is None else self._project(y)

    def tile_stream_forward(self, video_clip, tile_size=(512, 512), tile_stride=(256, 256), device=None):
        device = device or video_clip.device
        (sh, sw), (th, tw) = tile_stride, tile_size
        _, _, T, H, W = video_clip.shape
        tasks = [(h, min(h + th, H), w, min(w + tw, W))
                 for h in range(0, H, sh) if not (h - sh >= 0 and h - sh + th >= H)
                 for w in range(0, W, sw) if not (w - sw >= 0 and w - sw + tw >= W)]  # fmt: skip
        first = self.clip_idx == 0
        oT, oH, oW = (T + 3) // 4, H // 16, W // 16
        values = [torch.zeros(1, oT, oH, oW, self.out_dim, dtype=video_clip.dtype, device=device) for _ in range(self.layer_num)]
        weight = torch.zeros(1, oT, oH, oW, dtype=video_clip.dtype, device=device)
        world, rank = (dist.get_world_size(), dist.get_rank()) if self.parallelism > 1 and dist.is_initialized() else (1, 0)
        for i, (h0, h1, w0, w1) in enumerate(tasks):
            if i % world != rank:
                continue
            clip = video_clip[:, :, :, h0:h1, w0:w1]
            if first:
                clip = torch.cat([clip[:, :, :1].repeat(1, 1, 3, 1, 1), clip], dim=2)
            y = self._step(clip, f"conv1-{h0}-{w0}", f"conv2-{h0}-{w0}", emit=not first)
            if y is None:
                continue
            ph, pw = (h1 - h0) // 16, (w1 - w0) // 16
            m = blend_mask(ph, pw, min((th - sh) // 16, (tw - sw) // 16), (h0 > 0, h1 < H, w0 > 0, w1 < W), device, y.dtype)
            for li, lin in enumerate(self.linear_layers):
                o = lin(y.flatten(2).transpose(1, 2)).view(1, oT, ph, pw, -1)
                values[li][:, :, h0 // 16 : h0 // 16 + ph, w0 // 16 : w0 // 16 + pw] += o * m[None, None, :, :, None]
            weight[:, :, h0 // 16 : h0 // 16 + ph, w0 // 16 : w0 // 16 + pw] += m
        self.clip_idx += 1
        if first:
            return None
        if world > 1:
            for v in values:
                dist.all_reduce(v)
            dist.all_reduce(weight)
        weight = weight.masked_fill(weight == 0, 1)
        return [(v / weight.unsqueeze(-1)).view(1, -1, self.out_dim) for v in values]
